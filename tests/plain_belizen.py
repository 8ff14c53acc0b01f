"""A plain, slow restatement of the Belizen decoder, one function per mechanism, written from its equations and
sharing nothing with the library: whole sequences at once, no cache, no batching, float64 unless told otherwise.
Tests compare the engine with it.

Notation: x_t is the stream at token t (width D), m the residual factor.  A layer is
    x <- x + m * mixer(n1(x));  x <- x + m * ff(n2(x))        n(x) = x / sqrt(mean(x^2) + eps) * w
The mixer is softmax attention over a sliding window that keeps the first positions (queries and keys normalised per
head, rotated with interpolated frequencies, capped scores, an elementwise sigmoid gate on the result) or gated linear
attention with a decay per key channel.  The feed-forward is a gated dense layer or a mixture of bounded gated experts
with experts that hand their input through, and an always-on shared expert.  A run of layers may be passed several
times.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def interpolated_frequencies(dims, base, scaling, dtype=torch.float64):
    """Frequencies f_i = base^(-2i/dims), i < dims/2, and the factor on cos and sin.  With `scaling` (factor, original,
    fast, slow): channels whose wavelength is long against the original context are slowed by `factor`, fast ones are
    left alone, and a linear ramp over the channel index joins the two; cos and sin grow by 0.1 ln(factor) + 1."""
    half = dims // 2
    i = torch.arange(half, dtype=dtype)
    f = torch.pow(torch.tensor(float(base), dtype=dtype), -2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def channel_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(channel_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(channel_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_first_channels(x, positions, freq, mag, dims):
    """x [T, heads, dim]: channel i < dims/2 is paired with channel i + dims/2; the pair (u, v) at position p becomes
    (u c - v s, v c + u s) with c = mag cos(p f_i), s = mag sin(p f_i); channels from `dims` on pass."""
    half = dims // 2
    ang = positions.to(x.dtype)[:, None] * freq.to(x.dtype)[None, :]
    c, s = (mag * torch.cos(ang))[:, None, :], (mag * torch.sin(ang))[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def window_visible(n, size, keep_first):
    """vis[i, j]: j <= i and (i - j < size or j < keep_first).  size None: causal."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    vis = j <= i
    if size is not None:
        vis = vis & ((i - j < size) | (j < keep_first))
    return vis


def attention_mixer(h, w, pre, a, eps):
    """The attention mixer of one layer on the normalised input h [T, D]; `a` is the layer's "mixer" entry."""
    n = h.shape[0]
    H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(n, H, d)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(n, G, d)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(n, G, dv)
    q = rms_norm(q, w[pre + "q.norm"], eps)
    k = rms_norm(k, w[pre + "k.norm"], eps)
    rot = a.get("rot")
    if rot:
        freq, mag = interpolated_frequencies(rot["dims"], rot["base"], rot.get("scaling"), h.dtype)
        pos = torch.arange(n)
        q = rotate_first_channels(q, pos, freq, mag, rot["dims"])
        k = rotate_first_channels(k, pos, freq, mag, rot["dims"])
    mask = a.get("mask") or {}
    vis = window_visible(n, mask.get("size"), mask.get("keep_first", 0))
    cap = a.get("softcap")
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * a["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~vis, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    out = out.reshape(n, H * dv) * torch.sigmoid(h @ w[pre + "g"].T)
    return out @ w[pre + "o"].T


def linear_attention_mixer(h, w, pre, a, eps, state=None, return_state=False):
    """Gated linear attention: per head a state S [dim, vdim], S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, with
    alpha = sigmoid(W_a2 W_a1 h + b)^(1/tau); o RMS-normed per head, gated by silu(W_g h), projected."""
    n = h.shape[0]
    H, d, dv = a["heads"], a["dim"], a["vdim"]
    q = (h @ w[pre + "q"].T).view(n, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].T).view(n, H, d)
    v = (h @ w[pre + "v"].T).view(n, H, dv)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / a["tau"]).view(n, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(n, H, dv, dtype=h.dtype)
    for t in range(n):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, w[pre + "norm"], eps).reshape(n, H * dv)
    out = (o * torch.nn.functional.silu(h @ w[pre + "g"].T)) @ w[pre + "o"].T
    return (out, S) if return_state else out


def dense_ff(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def bounded_expert(h, w, pre, limit):
    """W_down (g sigmoid(1.702 g) (u + 1)), g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit)."""
    g = torch.clamp(h @ w[pre + "gate"].T, max=limit)
    u = torch.clamp(h @ w[pre + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[pre + "down"].T


def route(h, router, correction, top):
    """Softmax scores over all router outputs; the `top` largest of score + correction are chosen (ties to the lower
    index); the weights are the chosen plain scores.  Returns ids [T, top] and weights [T, top]."""
    s = torch.softmax((h.to(torch.float64) @ router.to(torch.float64).T), dim=-1)
    choice = s + correction.to(torch.float64)
    ids = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    return ids, torch.gather(s, 1, ids).to(h.dtype)


def experts_ff(h, w, pre, mlp):
    """The mixture: real experts 0 .. experts-1, then `identity` experts whose output is their input."""
    r = mlp["router"]
    real, ident, top = r["experts"], r.get("identity", 0), r["top"]
    ids, weights = route(h, w[pre + "router"], w[pre + "correction"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(ids[t, c])
            y = bounded_expert(h[t:t + 1], w, f"{pre}e{e}.", mlp["expert"]["limit"])[0] if e < real else h[t]
            out[t] += weights[t, c] * y
    if mlp.get("shared"):
        out = out + bounded_expert(h, w, pre + "shared.", mlp["shared"]["limit"])
    assert ident + real == w[pre + "router"].shape[0]
    return out


def run_order(cfg):
    """[(layer, pass number or None at the first layer of a pass)]: layers start .. stop-1 are passed `times` times."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  layers_out: a list that receives the stream after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps, m = cfg["norm"]["eps"], cfg["residual_mult"]
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x = x0.clone()
    for i, entering in run_order(cfg):
        if entering is not None:
            if entering > 0:
                x = x + x0
            x = x + w["loop.step"][entering]
        L, pre = cfg["layers"][i], f"l{i}."
        h = rms_norm(x, w[pre + "norm1"], eps)
        if L["type"] == "attention":
            x = x + m * attention_mixer(h, w, pre + "mix.", L["mixer"], eps)
        else:
            x = x + m * linear_attention_mixer(h, w, pre + "mix.", L["mixer"], eps)
        if L.get("mlp"):
            h = rms_norm(x, w[pre + "norm2"], eps)
            if L["mlp"]["kind"] == "dense":
                x = x + m * dense_ff(h, w, pre + "mlp.")
            else:
                x = x + m * experts_ff(h, w, pre + "mlp.", L["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def greedy(cfg, w, prompt, n_new):
    """The n_new tokens with the largest logit, one after another, the whole sequence recomputed for each."""
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(torch.argmax(forward(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]


def tensor_shapes(cfg):
    """Name -> shape of every tensor a model of this configuration has."""
    D = cfg["width"]
    out = {"embed": (cfg["vocab"], D), "final.norm": (D,)}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], D)
    for i, L in enumerate(cfg["layers"]):
        p, a = f"l{i}.", L["mixer"]
        out[p + "norm1"] = (D,)
        if L["type"] == "attention":
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            out.update({p + "mix.q": (H * d, D), p + "mix.q.b": (H * d,), p + "mix.k": (G * d, D), p + "mix.k.b": (G * d,),
                        p + "mix.v": (G * dv, D), p + "mix.v.b": (G * dv,), p + "mix.q.norm": (d,), p + "mix.k.norm": (d,),
                        p + "mix.g": (H * dv, D), p + "mix.o": (D, H * dv)})
        else:
            H, d, dv, r = a["heads"], a["dim"], a["vdim"], a["rank"]
            out.update({p + "mix.q": (H * d, D), p + "mix.k": (H * d, D), p + "mix.v": (H * dv, D), p + "mix.g": (H * dv, D),
                        p + "mix.o": (D, H * dv), p + "mix.norm": (dv,), p + "mix.a1": (r, D), p + "mix.a2": (H * d, r),
                        p + "mix.a2.b": (H * d,)})
        mlp = L.get("mlp")
        if not mlp:
            continue
        out[p + "norm2"] = (D,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], D), p + "mlp.up": (mlp["ff"], D), p + "mlp.down": (D, mlp["ff"])})
            continue
        r, f = mlp["router"], mlp["expert"]["ff"]
        for e in range(r["experts"]):
            out.update({f"{p}mlp.e{e}.gate": (f, D), f"{p}mlp.e{e}.up": (f, D), f"{p}mlp.e{e}.down": (D, f)})
        n = r["experts"] + r.get("identity", 0)
        out.update({p + "mlp.router": (n, D), p + "mlp.correction": (n,)})
        if mlp.get("shared"):
            s = mlp["shared"]["ff"]
            out.update({p + "mlp.shared.gate": (s, D), p + "mlp.shared.up": (s, D), p + "mlp.shared.down": (D, s)})
    return out
