"""The Redodra decoder restated plainly: float64 torch on the CPU, whole sequences at once, one function per
mechanism, no cache, no batching, no code shared with the library.  The tests compare the engine with this.

Notation: T tokens, D the stream's width; W["name"] the tensors under the names of the weight file
(matrices [out, in]); positions count from 0; t is the query's position and s a key's.
"""
import math

import torch


# ---- small pieces ---------------------------------------------------------------------------------------
def squash_norm(x, W, name):
    """tanh(alpha x) * w + b, elementwise: no statistics of the row."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.logaddexp(x, torch.zeros_like(x))


def short_conv(x, taps, bias=None):
    """x [T, C], taps [C, K]: y_t = sum_k taps[:, K - 1 - k] * x_(t - k), nothing before the sequence's start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x], dim=0)
    y = torch.zeros_like(x)
    for k in range(K):
        y = y + padded[K - 1 - k:K - 1 - k + T] * taps[:, K - 1 - k]
    return y if bias is None else y + bias


def rotate_adjacent(x, base, dims):
    """x [T, heads, d]: channels (2i, 2i + 1) of the first `dims` turn by t * base^(-2i / dims); the rest pass."""
    T = x.shape[0]
    i = torch.arange(dims // 2, dtype=torch.float64)
    a = torch.arange(T, dtype=torch.float64)[:, None] * torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def capped(scores, cap):
    return cap * torch.tanh(scores / cap)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z / 2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z / 2."""
    ap, an = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(torch.clamp(z, max=0.0)) - z) + 0.5 * z)


# ---- mixers ---------------------------------------------------------------------------------------------
def gated_attention_keys(h, W, p, m):
    """The rotated keys and the values of a layer with projections of its own: ([T, G, d], [T, G, dv])."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = rotate_adjacent((h @ W[p + "k"].T).view(T, G, d), m["rot"]["base"], m["rot"]["dims"])
    return k, (h @ W[p + "v"].T).view(T, G, dv)


def gated_attention(h, W, p, m, kv):
    """Causal attention with rotary queries and keys, capped scores, a sink in the denominator of the softmax
    and a gate per head on the result; `kv` are the keys and values (this layer's or another's)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate_adjacent((h @ W[p + "q"].T).view(T, H, d), m["rot"]["base"], m["rot"]["dims"])
    k, v = kv
    rep = H // G
    scores = capped(torch.einsum("thd,shd->hts", q, k.repeat_interleave(rep, dim=1)) * m["scale"], m["softcap"])
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    scores = scores.masked_fill(~visible[None], float("-inf"))
    sink = W[p + "sink"].view(H, 1, 1)
    top = torch.maximum(scores.amax(-1, keepdim=True), sink)
    e = torch.exp(scores - top)
    weights = e / (e.sum(-1, keepdim=True) + torch.exp(sink - top))
    o = torch.einsum("hts,shd->thd", weights, v.repeat_interleave(rep, dim=1))
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def windowed_attention(h, W, p, m):
    """Attention without rotation: biased projections, capped scores minus r1 ln(1 + r2 (t - s)), keys limited to
    the last `size` positions plus the first `keep_first` of the sequence, plain softmax."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, d)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, dv)
    rep = H // G
    scores = capped(torch.einsum("thd,shd->hts", q, k.repeat_interleave(rep, dim=1)) * m["scale"], m["softcap"])
    t = torch.arange(T)
    dist = (t[:, None] - t[None, :]).double().clamp(min=0.0)
    scores = scores - W[p + "r1"].view(H, 1, 1) * torch.log1p(W[p + "r2"].view(H, 1, 1) * dist[None])
    visible = (t[None, :] <= t[:, None]) & ((t[:, None] - t[None, :] < m["mask"]["size"]) | (t[None, :] < m["mask"]["keep_first"]))
    scores = scores.masked_fill(~visible[None], float("-inf"))
    o = torch.einsum("hts,shd->thd", torch.softmax(scores, dim=-1), v.repeat_interleave(rep, dim=1))
    return o.reshape(T, H * dv) @ W[p + "o"].T + W[p + "o.b"]


def state_space(h, W, p, m, eps):
    """A selective state space with a scalar decay per head: per head a state S [N, dv],
    S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T,  y_t = S_t^T C_t + D x_t;
    x, B, C come from one projection through a short convolution and silu; the gated y is normed in groups."""
    T = h.shape[0]
    H, dv, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * dv
    zxbcdt = h @ W[p + "in"].T
    z, xbc, dt = zxbcdt[:, :inner], zxbcdt[:, inner:2 * inner + 2 * G * N], zxbcdt[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, dim=1)
    dt = softplus(dt + W[p + "dt_bias"])
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * dt)                     # [T, H]
    S = torch.zeros(H, N, dv, dtype=torch.float64)
    y = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnd,hn->hd", S, C[t]) + W[p + "D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    y = rms_norm(y.view(T, ng, inner // ng), W[p + "norm"].view(ng, inner // ng), eps).reshape(T, inner)
    return y @ W[p + "o"].T


def delta_rule(h, W, p, m, eps):
    """The gated delta rule: per head a state S [d, dv];  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;
    o = S^T q.  q, k, v pass short convolutions and silu; q and k are unit vectors, q also times d^(-1/2)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(H // G, dim=1), k.repeat_interleave(H // G, dim=1)
    beta = torch.sigmoid(h @ W[p + "b"].T)                                               # [T, H]
    g = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    S = torch.zeros(H, d, dv, dtype=torch.float64)
    o = torch.zeros(T, H, dv, dtype=torch.float64)
    for t in range(T):
        S = g[t][:, None, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hkd,hk->hd", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkd,hk->hd", S, q[t])
    o = rms_norm(o, W[p + "norm"], eps) * silu(h @ W[p + "g"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def side_by_side(h, W, p, m, eps):
    """Half the sum of the two members' results, each RMS-normed over the width first."""
    left = windowed_attention(h, W, p + "left.", m["left"])
    right = state_space(h, W, p + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, W[p + "left.out"], eps) + rms_norm(right, W[p + "right.out"], eps))


def feed_forward(h, W, p):
    return xielu(h @ W[p + "up"].T, W[p + "act"][0], W[p + "act"][1]) @ W[p + "down"].T


# ---- the model ----------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, streams=None, results=None):
    """float64 logits [T, vocab] of a whole sequence; `streams` (a list) receives what every layer hands on (after
    the weighted sum over depth), `results` every layer's own result before that sum."""
    W = {k: v.double() for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)]
    history = [x]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = squash_norm(x, W, p + "norm1")
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept[i] = gated_attention_keys(h, W, p + "mix.", m)
            mixed = gated_attention(h, W, p + "mix.", m, kept[i if src is None else src])
        elif layer["type"] == "delta":
            mixed = delta_rule(h, W, p + "mix.", m, eps)
        elif layer["type"] == "parallel":
            mixed = side_by_side(h, W, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + squash_norm(mixed, W, p + "norm1b")
        if layer.get("mlp") is not None:
            x = x + squash_norm(feed_forward(squash_norm(x, W, p + "norm2"), W, p + "mlp."), W, p + "norm2b")
        history.append(x)
        if results is not None:
            results.append(x.clone())
        x = sum(W[p + "dwa"][j] * history[j] for j in range(i + 2))
        if streams is not None:
            streams.append(x.clone())
    return squash_norm(x, W, "final.norm") @ W["head"].T


def greedy(cfg, weights, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


# ---- tensors ------------------------------------------------------------------------------------------------
def _norm_shapes(shapes, name, D):
    shapes[name] = (D,)
    shapes[name + ".b"] = (D,)
    shapes[name + ".alpha"] = ()


def tensor_shapes(cfg):
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "head": (cfg["vocab"], D)}
    _norm_shapes(shapes, "final.norm", D)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if layer.get("mlp") is not None else ()):
            _norm_shapes(shapes, p + n, D)
        x = p + "mix."
        if layer["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes[x + "q"] = (H * d, D)
            if m.get("kv_from") is None:
                shapes[x + "k"], shapes[x + "v"] = (G * d, D), (G * dv, D)
            shapes.update({x + "sink": (H,), x + "g": (H, D), x + "o": (D, H * dv)})
        elif layer["type"] == "delta":
            H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            shapes.update({x + "q": (G * d, D), x + "k": (G * d, D), x + "v": (H * dv, D),
                           x + "q.conv": (G * d, K), x + "k.conv": (G * d, K), x + "v.conv": (H * dv, K),
                           x + "b": (H, D), x + "a": (H, D), x + "dt_bias": (H,), x + "A_log": (H,),
                           x + "g": (H * dv, D), x + "norm": (dv,), x + "o": (D, H * dv)})
        else:
            a, s = m["left"], m["right"]
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            L = x + "left."
            shapes.update({L + "q": (H * d, D), L + "q.b": (H * d,), L + "k": (G * d, D), L + "k.b": (G * d,),
                           L + "v": (G * dv, D), L + "v.b": (G * dv,), L + "r1": (H,), L + "r2": (H,),
                           L + "o": (D, H * dv), L + "o.b": (D,), L + "out": (D,)})
            inner, gn = s["heads"] * s["vdim"], s["groups"] * s["state"]
            R = x + "right."
            shapes.update({R + "in": (2 * inner + 2 * gn + s["heads"], D), R + "conv": (inner + 2 * gn, s["conv"]),
                           R + "conv.b": (inner + 2 * gn,), R + "dt_bias": (s["heads"],), R + "A_log": (s["heads"],),
                           R + "D": (s["heads"],), R + "norm": (inner,), R + "o": (D, inner), R + "out": (D,)})
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            shapes.update({p + "mlp.up": (F, D), p + "mlp.down": (D, F), p + "mlp.act": (2,)})
        shapes[p + "dwa"] = (i + 2,)
    return shapes


def random_weights(cfg, seed, hot=1.0):
    """bfloat16 tensors.  Matrices N(0, hot^2 / in); norm weights 1 + N(0, 0.2) with small offsets b and alpha
    near 1; short convolutions of unit size; decays between 0.7 and 1 per step; sinks, distance factors and
    activation parameters of order 1; the weights over depth favour the newest result and sum to about 1."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *shape: torch.randn(*shape, generator=g)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            t = 0.8 + 0.4 * torch.rand((), generator=g)
        elif name.endswith(".b") and len(shape) == 1 and ("norm" in name):
            t = 0.1 * rn(*shape)
        elif last in ("norm", "norm1", "norm2", "norm1b", "norm2b", "out"):
            t = 1.0 + 0.2 * rn(*shape)
        elif last == "conv":
            t = rn(*shape) / math.sqrt(shape[1])
        elif name.endswith("conv.b") or (name.endswith(".b") and len(shape) == 1):
            t = 0.3 * rn(*shape)
        elif last == "A_log":
            t = torch.log(0.5 + 1.5 * torch.rand(shape, generator=g))
        elif last == "dt_bias":
            t = -2.0 + 1.5 * torch.rand(shape, generator=g)
        elif last == "D":
            t = 1.0 + 0.3 * rn(*shape)
        elif last == "sink":
            t = rn(*shape)
        elif last == "r1":
            t = 0.2 + 0.6 * torch.rand(shape, generator=g)
        elif last == "r2":
            t = 0.1 + 0.9 * torch.rand(shape, generator=g)
        elif last == "act":
            t = 0.5 * rn(*shape)
        elif last == "dwa":
            t = 0.15 * rn(*shape)
            t[-1] += 1.0
        elif name == "embed":
            t = rn(*shape)
        else:
            t = rn(*shape) * (hot / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out
