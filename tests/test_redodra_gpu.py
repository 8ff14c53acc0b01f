"""The Redodra decoder in the engine against the plain restatement (`plain_redodra`): each mechanism's kernels
alone, then whole models: prompts whole, token by token, in portions down to two tokens, unequal batches, slots
and pages used again, keys at the edges of windows, of the kept first positions and of pages, far keys, the first
tokens of a sequence, long decoding, and greedy generation through `Model.generate`."""
import math

import pytest
import torch

import plain_redodra
import redodra_models
from conftest import random_tokens, rel_err

# Worst row's max |a - b| / max |b| against the plain model in float64.  float32 runs: a kernel fault shows far
# above 1e-4.  bfloat16 runs keep bfloat16 activations between the kernels of a sublayer (the stream, the states,
# the norms and the scores stay float32): rounding alone reaches a few 1e-2 on single rows of a model five or six
# layers deep; a key too many or too few, a lost state or a missing sink costs 0.2 and more.
TOL = {"float32": 1e-4, "bfloat16": 6e-2}
PART_TOL = {torch.float32: 3e-5, torch.bfloat16: 3e-2}

pytestmark = pytest.mark.gpu

DEV = "cuda"
F32 = torch.float32


def d(t, dtype=None):
    return t.to(device=DEV, dtype=dtype or t.dtype).contiguous()


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device=DEV)


def make_ctx(cache, slots, starts, counts, dtype, ws):
    """A step context for a part tested outside an engine: sequences in the given slots, continued from `starts`
    by `counts` tokens each."""
    from rust_inference_b200.engine.context import StepContext, pack_step
    tokens = [[0] * c for c in counts]
    meta, layout, sc = pack_step(starts, tokens, [[] for _ in tokens])
    o, c = layout["seq_slot"]
    meta[o:o + c] = slots
    cache.reserve([(s, st + n) for s, st, n in zip(slots, starts, counts)])
    dev = torch.from_numpy(meta).to(DEV)
    v = lambda name: dev[layout[name][0]:layout[name][0] + layout[name][1]]
    return StepContext(
        n_tokens=sc["n_tokens"], n_seqs=sc["n_seqs"], token_ids=v("token_ids"), token_pos=v("token_pos"),
        token_seq=v("token_seq"), seq_slot=v("seq_slot"), seq_start=v("seq_start"), seq_len=v("seq_len"),
        cu_seqlens=v("cu_seqlens"), logit_rows=v("logit_rows"), n_logit_rows=sc["n_logit_rows"],
        max_new=sc["max_new"], max_len=sc["max_len"], all_single=sc["all_single"], page_table=cache.page_table,
        page_size=cache.page_size, dtype=dtype, device=torch.device(DEV), workspace=ws)


# ---------------------------------------------------------------------------------------------------
# elementwise work on the stream
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(1, 72), (5, 130), (300, 256), (7, 4100)])
def test_squash_norm_kernel(dtype, rows, width):
    """tanh(alpha x) w + b on all rows and on picked rows; inputs large enough to saturate."""
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(rows + width)
    x = torch.randn(rows, width, generator=g) * 2.5
    W = {"n": 1 + 0.3 * torch.randn(width, generator=g), "n.b": 0.2 * torch.randn(width, generator=g), "n.alpha": torch.tensor(0.7)}
    want = plain_redodra.squash_norm(x.double(), {k: v.double() for k, v in W.items()}, "n")
    out = torch.empty(rows, width, dtype=dtype, device=DEV)
    ops.dyt_norm(d(x), d(W["n"]), d(W["n.b"]), d(W["n.alpha"].reshape(1)), out)
    tol = 2e-6 if dtype == F32 else 6e-3
    assert rel_err(out, want) < tol
    pick = [rows - 1, 0]
    out2 = torch.empty(2, width, dtype=dtype, device=DEV)
    ops.dyt_norm(d(x), d(W["n"]), d(W["n.b"]), d(W["n.alpha"].reshape(1)), out2, i32(pick))
    assert rel_err(out2, want[pick]) < tol


@pytest.mark.parametrize("rows,width,index,entries", [(3, 72, 0, 2), (40, 130, 2, 6), (9, 256, 4, 6), (1, 96, 1, 3)])
def test_stream_update_in_one_pass(rows, width, index, entries):
    """The end of a sublayer as one kernel: the branch is normed and joins the stream, the result enters the history,
    the stream becomes the weighted sum over depth, and the next norm of it is written; the branch is left zeroed.
    `entries` = index + 2 is the last layer, which stores nothing."""
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(index + width)
    rn = lambda *s: torch.randn(*s, generator=g)
    stream, branch, bias = rn(rows, width), rn(rows, width) * 2, rn(width)
    hist = rn(entries, rows, width)
    pw, pb, pa = 1 + 0.2 * rn(width), 0.1 * rn(width), torch.tensor([0.9])
    nw, nb, na = 1 + 0.2 * rn(width), 0.1 * rn(width), torch.tensor([1.2])
    dw = rn(index + 2)
    f = lambda t: t.double()
    joined = f(stream) + torch.tanh(0.9 * (f(branch) + f(bias))) * f(pw) + f(pb)
    past = f(hist).clone()
    past[index + 1] = joined
    mixed = sum(f(dw)[j] * past[j] for j in range(index + 2))
    nxt = torch.tanh(1.2 * mixed) * f(nw) + f(nb)
    store = index + 2 < entries
    for out_dtype in (torch.float32, torch.bfloat16):
        s, b, h = d(stream), d(branch), d(hist)
        out = torch.empty(rows, width, dtype=out_dtype, device=DEV)
        ops.stream_update(s, branch=b, branch_bias=d(bias), post=(d(pw), d(pb), d(pa)), history=h, depth_w=d(dw),
                          depth_index=index, store_result=store, next_norm=(d(nw), d(nb), d(na)), next_out=out)
        assert rel_err(s, mixed) < 2e-6
        assert rel_err(out, nxt) < (2e-6 if out_dtype == F32 else 6e-3)
        assert float(b.abs().max()) == 0.0
        if store:
            assert rel_err(h[index + 1], joined) < 2e-6
        keep = [j for j in range(entries) if j != index + 1 or not store]
        assert torch.equal(h[keep].cpu(), hist[keep])
    # nothing but the join
    s, b = d(stream), d(branch)
    ops.stream_update(s, branch=b)
    assert rel_err(s, f(stream) + f(branch)) < 1e-6 and float(b.abs().max()) == 0.0


@pytest.mark.parametrize("rows,width,members", [(3, 72, 2), (50, 320, 2), (7, 1000, 4), (2, 96, 1)])
def test_normed_sum_of_members(rows, width, members):
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(rows)
    rn = lambda *s: torch.randn(*s, generator=g)
    xs = [rn(rows, width) * (10.0 ** m) for m in range(members)]
    bs = [rn(width) if m % 2 == 0 else None for m in range(members)]
    ws = [1 + 0.3 * rn(width) for _ in range(members)]
    sc = [0.5, 0.25, 2.0, 1.0][:members]
    base = rn(rows, width)
    want = base.double()
    for x, b, w, s in zip(xs, bs, ws, sc):
        y = x.double() + (b.double() if b is not None else 0.0)
        want = want + s * plain_redodra.rms_norm(y, w.double(), 1e-5)
    out = d(base)
    dev = [d(x) for x in xs]
    ops.normed_sum([(x, d(b) if b is not None else None, d(w), s) for x, b, w, s in zip(dev, bs, ws, sc)], out, 1e-5, accumulate=True)
    assert rel_err(out, want) < 3e-6
    assert all(float(x.abs().max()) == 0.0 for x in dev)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_learned_activation_kernel(dtype):
    """Both branches, the joint at zero, large arguments on either side (e^z - 1 for small z without cancellation)."""
    from rust_inference_b200.kernels import ops
    z = torch.cat([torch.linspace(-30, 30, 4001), torch.tensor([0.0, -1e-6, 1e-6, -1e-3, 1e-3])]).to(dtype)
    pq = torch.tensor([0.3, -0.4])
    want = plain_redodra.xielu(z.double(), pq[0].double(), pq[1].double())
    out = torch.empty_like(z, device=DEV)
    ops.xielu(d(z), out, d(pq))
    got = out.double().cpu()
    err = (got - want).abs() / (want.abs() + z.double().abs() + 1e-30)      # the function crosses zero left of the origin
    assert float(err.max()) < (3e-6 if dtype == F32 else 5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,ff", [(1, 72, 40), (5, 128, 200), (130, 128, 264), (600, 256, 520), (2100, 512, 1024), (9, 100, 36)])
def test_activation_in_the_product_s_epilogue(dtype, n, width, ff):
    """act(x W^T) as one kernel: few and many tokens (every form of the tensor-core kernel), sizes it refuses."""
    from rust_inference_b200.kernels import linear
    g = torch.Generator().manual_seed(n + ff)
    x = torch.randn(n, width, generator=g).to(dtype)
    w = (torch.randn(ff, width, generator=g) * (2.0 / math.sqrt(width))).to(dtype)
    pq = torch.tensor([0.4, -0.3])
    want = plain_redodra.xielu(x.double() @ w.double().T, pq[0].double(), pq[1].double())
    out = torch.empty(n, ff, dtype=dtype, device=DEV)
    linear.activated(d(x), linear.Weight(d(w)), out, None, d(pq))
    assert rel_err(out, want) < (1e-5 if dtype == F32 else 1e-2)


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("groups,size,w_len,gate_first", [(4, 24, 24, False), (1, 72, 72, False), (2, 64, 128, True),
                                                         (3, 40, 120, True), (8, 8, 8, False), (1, 130, 130, True), (2, 640, 640, True),
                                                         (1, 1030, 1030, False)])
def test_gated_group_norm_kernel(out_dtype, groups, size, w_len, gate_first):
    """RMS norm over groups of channels with a silu gate before or after it; one weight for all groups or one per channel."""
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(groups * size)
    n, col = 9, 5
    x = torch.randn(n, groups * size, generator=g) * 3
    gate = torch.randn(n, col + groups * size + 3, generator=g)
    w = 1 + 0.3 * torch.randn(w_len, generator=g)
    gt = plain_redodra.silu(gate[:, col:col + groups * size].double())
    xd = x.double() * (gt if gate_first else 1.0)
    wd = w.double().repeat(groups * size // w_len).view(groups, size)
    want = plain_redodra.rms_norm(xd.view(n, groups, size), wd, 1e-5).reshape(n, -1) * (1.0 if gate_first else gt) * 0.5
    out = torch.empty(n, groups * size, dtype=out_dtype, device=DEV)
    ops.gated_group_norm(d(x), d(gate), col, d(w), out, groups=groups, group_size=size, gate_first=gate_first, eps=1e-5, out_scale=0.5)
    assert rel_err(out, want) < (3e-6 if out_dtype == F32 else 6e-3)


# ---------------------------------------------------------------------------------------------------
# mixers alone, outside an engine
# ---------------------------------------------------------------------------------------------------
GATED_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink", "gate": "g"}
WINDOW_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
                "r1": "r1", "r2": "r2"}
DELTA_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b", "a": "a",
               "dt_bias": "dt_bias", "A_log": "A_log", "gate": "g", "norm": "norm", "o": "o"}
SSM_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D", "norm": "norm", "o": "o"}


def _weights(kind, m, width, seed, hot=1.0, edit=None, eps=1e-5):
    """Random tensors of a one-layer model around the mixer, for the plain functions: (tensors, prefix)."""
    dummy_left = redodra_models.window(heads=1, kv=1, dim=8, vdim=8, scale=1.0, cap=1.0, size=1, keep=0)
    dummy_right = redodra_models.ssm(heads=1, vdim=8, state=1, groups=1, conv=1, norm_groups=1)
    layer = {"delta": {"type": "delta", "mixer": m}, "gated": {"type": "attention", "mixer": m},
             "ssm": {"type": "parallel", "mixer": {"left": dummy_left, "right": m}},
             "window": {"type": "parallel", "mixer": {"left": m, "right": dummy_right}}}[kind]
    cfg = {"width": width, "vocab": 10, "norm": {"eps": eps}, "layers": [dict(layer, mlp=None)]}
    W = {k: v.float() for k, v in plain_redodra.random_weights(cfg, seed, hot=hot).items()}
    prefix = "l0.mix." + {"ssm": "right.", "window": "left."}.get(kind, "")
    if edit is not None:
        edit(W, prefix)
    return W, prefix


def _mixer(kind, m, dtype, width, seed, hot=1.0, edit=None, eps=1e-5):
    """One mixer of the library holding the tensors of `_weights`; the same tensors in float64 for the plain functions."""
    from rust_inference_b200.parts.registry import lookup
    from rust_inference_b200.parts.spec import PartSpec
    common = dict(hidden_size=width, dtype=dtype, device=DEV)
    if kind == "delta":
        part = lookup("mixer", "gated_delta_rule")(n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                                   conv=m["conv"], eps=eps, names=DELTA_NAMES, **common)
    elif kind == "ssm":
        part = lookup("mixer", "selective_state_space")(n_heads=m["heads"], v_head_dim=m["vdim"], state=m["state"], groups=m["groups"],
                                                        conv=m["conv"], norm_groups=m["norm_groups"], eps=eps, conv_bias=True,
                                                        names=SSM_NAMES, **common)
    else:
        if kind == "gated":
            pos = PartSpec("rope", {"head_dim": m["dim"], "base": m["rot"]["base"], "style": "interleaved", "rot_dims": m["rot"]["dims"],
                                    "exact_angles": True})
            extra = dict(qkv_bias=False, sink=True, head_gate=True, names=GATED_NAMES)
        else:
            pos = PartSpec("unrotated", {})
            extra = dict(qkv_bias=True, o_bias=True, distance_bias=True, window=m["mask"]["size"], keep_first=m["mask"]["keep_first"],
                         names=WINDOW_NAMES)
        part = lookup("mixer", "gqa_attention")(n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                                position=pos, scale=m["scale"], softcap=m["softcap"], **extra, **common)
    W, prefix = _weights(kind, m, width, seed, hot, edit, eps)
    tensors = {local: d(W[prefix + local], F32 if ts.role == "vector" else dtype) for local, ts in part.tensor_specs().items()}
    part.set_tensors(tensors)
    part.prepare(2048)
    return part, {k: v.double() for k, v in W.items()}, prefix


def _drive(part, cache, x, portions, dtype, ws, slot=None, free=True):
    """The part over one sequence cut into portions (the last size repeats); what it adds to a zeroed float32 stream."""
    n, width = x.shape
    slot = cache.alloc_slot() if slot is None else slot
    got = torch.zeros(n, width, device=DEV)
    at, i = 0, 0
    while at < n:
        take = min(portions[min(i, len(portions) - 1)], n - at)
        ctx = make_ctx(cache, [slot], [at], [take], dtype, ws)
        part.forward(d(x[at:at + take]), got[at:at + take], ctx, cache.layer(0), True)
        at += take
        i += 1
        cache.commit(slot, at)
    if free:
        cache.free_slot(slot)
    return got


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,conv", [(4, 2, 16, 24, 3), (1, 1, 40, 72, 1), (6, 2, 8, 8, 5), (4, 4, 64, 128, 4),
                                                    (2, 1, 128, 64, 2), (3, 3, 20, 130, 4), (2, 2, 256, 32, 4)])
def test_delta_rule_alone(dtype, heads, kv, dim, vdim, conv):
    """The gated delta rule as a whole prompt, in portions down to one token and in a slot that another sequence has
    used: state and the convolutions' last inputs are carried, and start at zero."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n = 96, 150
    m = redodra_models.delta(heads=heads, kv=kv, dim=dim, vdim=vdim, conv=conv)
    part, W, p = _mixer("delta", m, dtype, width, seed=dim + vdim, hot=1.5)
    g = torch.Generator().manual_seed(conv)
    x = torch.randn(n, width, generator=g).to(dtype)
    want = plain_redodra.delta_rule(x.double(), W, p, m, 1e-5)
    cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
    ws = Workspace(DEV)
    for portions in ([n], [1], [2], [70, 1, 1, 3, 33, 2], [3, 1]):
        assert rel_err(_drive(part, cache, x, portions, dtype, ws), want) < PART_TOL[dtype], portions


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,state,groups,conv,ng", [(3, 16, 8, 1, 4, 1), (1, 40, 1, 1, 1, 1), (4, 8, 24, 2, 2, 4), (8, 32, 64, 2, 4, 2),
                                                             (2, 64, 128, 1, 4, 4), (6, 12, 20, 3, 3, 9), (2, 130, 256, 2, 5, 1)])
def test_state_space_alone(dtype, heads, vdim, state, groups, conv, ng):
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n = 80, 150
    m = redodra_models.ssm(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=ng)
    part, W, p = _mixer("ssm", m, dtype, width, seed=state + vdim, hot=1.5)
    g = torch.Generator().manual_seed(conv)
    x = torch.randn(n, width, generator=g).to(dtype)
    want = plain_redodra.state_space(x.double(), W, p, m, 1e-5)
    cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
    ws = Workspace(DEV)
    for portions in ([n], [1], [2], [70, 1, 1, 3, 33, 2], [3, 1]):
        assert rel_err(_drive(part, cache, x, portions, dtype, ws), want) < PART_TOL[dtype], portions


@pytest.mark.parametrize("kind", ["delta", "ssm"])
def test_a_state_remembers_a_far_token(kind):
    """With decays of almost 1 one large early input stays in the state: 300 tokens later the output still differs by
    far more than rounding from the same sequence without it, the library agrees with the plain result on both, also
    when the later tokens come one by one, and a batch of the two sequences equals each alone."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n = 64, 330

    def slow_decay(W, p):
        W[p + "A_log"].fill_(-9.0)
        W[p + "dt_bias"].fill_(-1.0)
    if kind == "delta":
        m = redodra_models.delta(heads=2, kv=1, dim=32, vdim=16, conv=2)
        plain = plain_redodra.delta_rule
    else:
        m = redodra_models.ssm(heads=2, vdim=16, state=32, groups=1, conv=2, norm_groups=2)
        plain = plain_redodra.state_space
    part, W, p = _mixer(kind, m, F32, width, seed=5, edit=slow_decay)
    g = torch.Generator().manual_seed(9)
    a = torch.randn(n, width, generator=g) * 0.5
    b = a.clone()
    b[4] = b[4] * 8.0
    wa, wb = plain(a.double(), W, p, m, 1e-5), plain(b.double(), W, p, m, 1e-5)
    assert float((wa[-1] - wb[-1]).abs().max()) > 1e-2 * float(wa[-1].abs().max())
    cache = SequenceCache([part.cache_request()], max_tokens=2048, max_seq_len=512, dtype=F32, device=DEV, n_slots=3)
    ws = Workspace(DEV)
    for x, want in ((a, wa), (b, wb)):
        assert rel_err(_drive(part, cache, x, [n], F32, ws), want) < 1e-4
        assert rel_err(_drive(part, cache, x, [40, 1], F32, ws), want) < 1e-4
    # the two as one batch of unequal portions, then one token each per step
    slots = [cache.alloc_slot(), cache.alloc_slot()]
    got = [torch.zeros(n, width, device=DEV), torch.zeros(n, width, device=DEV)]
    first = [37, 5]
    ctx = make_ctx(cache, slots, [0, 0], first, F32, ws)
    out = torch.zeros(sum(first), width, device=DEV)
    part.forward(d(torch.cat([a[:first[0]], b[:first[1]]])), out, ctx, cache.layer(0), True)
    got[0][:first[0]], got[1][:first[1]] = out[:first[0]], out[first[0]:]
    at = list(first)
    for s, k in zip(slots, at):
        cache.commit(s, k)
    while min(at) < n:
        live = [i for i in (0, 1) if at[i] < n]
        ctx = make_ctx(cache, [slots[i] for i in live], [at[i] for i in live], [1] * len(live), F32, ws)
        out = torch.zeros(len(live), width, device=DEV)
        part.forward(d(torch.stack([(a, b)[i][at[i]] for i in live])), out, ctx, cache.layer(0), True)
        for r, i in enumerate(live):
            got[i][at[i]] = out[r]
            at[i] += 1
            cache.commit(slots[i], at[i])
    assert rel_err(got[0], wa) < 1e-4 and rel_err(got[1], wb) < 1e-4


def _blind_channel(W, p):
    """Channel 0 of the input reaches the values only: queries, keys and gates do not read it.  A large number there
    makes a position's value dwarf the others while its score stays ordinary, so whoever sees the position shows it."""
    for name in ("q", "k", "g"):
        if p + name in W:
            W[p + name][:, 0] = 0.0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,size,keep", [(4, 2, 16, 24, 20, 3), (2, 2, 8, 8, 150, 70), (1, 1, 24, 24, 1, 1), (3, 1, 8, 16, 33, 0),
                                                         (4, 2, 64, 64, 70, 10), (2, 1, 128, 128, 129, 64), (6, 2, 64, 32, 64, 65)])
def test_window_and_kept_edges_with_a_value_that_dwarfs_the_rest(dtype, heads, kv, dim, vdim, size, keep):
    """Unrotated attention over a window that keeps the sequence's first positions, with capped scores and the bias by
    distance.  One position's value is made huge: the results differ by orders of magnitude between the last query that
    sees it and the first that does not.  The position lies at the window's edge on both sides of a page border, and is
    the last kept position (seen for ever) or the first one not kept (lost when the window has passed).  As one prompt,
    and with the later tokens one by one."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n, cut = 128, 330, 150
    m = redodra_models.window(heads=heads, kv=kv, dim=dim, vdim=vdim, scale=0.6 / math.sqrt(dim), cap=7.0, size=size, keep=keep)
    part, W, p = _mixer("window", m, dtype, width, seed=dim + size, hot=1.5, edit=_blind_channel)
    cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
    ws = Workspace(DEV)
    places = sorted({63, 64, 130, max(keep - 1, 0), keep})
    for big in places:
        g = torch.Generator().manual_seed(big)
        x = (torch.randn(n, width, generator=g) * 0.3).to(dtype)
        x[big, 0] = 3e4
        want = plain_redodra.windowed_attention(x.double(), W, p, m)
        lost = big + size                                         # the first query that no longer sees `big` through the window
        if big >= keep and lost < n:
            assert float(want[lost - 1].abs().max()) > 20 * float(want[lost].abs().max())
        if big < keep:
            quiet = x.clone()
            quiet[big, 0] = 0.0
            assert float(want[n - 1].abs().max()) > 20 * float(plain_redodra.windowed_attention(quiet.double(), W, p, m)[n - 1].abs().max())
        tol = 3e-5 if dtype == F32 else 3e-2
        assert rel_err(_drive(part, cache, x, [n], dtype, ws), want) < tol, big
        assert rel_err(_drive(part, cache, x, [cut, 1], dtype, ws), want) < tol, big
    # portions whose borders fall inside the window and inside the kept positions
    assert rel_err(_drive(part, cache, x, [2, 1, 61, 3, 64, 7], dtype, ws), want) < tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot", [(4, 1, 32, 16, 8), (3, 3, 8, 8, 8), (4, 2, 64, 64, 32), (8, 2, 64, 64, 64), (2, 1, 128, 128, 2),
                                                   (2, 2, 40, 72, 10)])
def test_causal_attention_with_sink_and_gate_sees_a_far_value(dtype, heads, kv, dim, vdim, rot):
    """Causal attention with rotation of the first channels in adjacent pairs, capped scores, a sink in the denominator
    and a gate per head.  A huge value at position 2 must reach queries hundreds of positions and several pages later,
    in a prompt and decoding.  One head's sink is large (it takes almost all the weight), one is very negative (no
    effect), so a sink left out or counted wrongly changes the result by orders of magnitude."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n = 128, 330
    m = redodra_models.attn(heads=heads, kv=kv, dim=dim, vdim=vdim, scale=0.8 / math.sqrt(dim), cap=9.0, base=3000.0, rot=rot)

    def edit(W, p):
        _blind_channel(W, p)
        W[p + "sink"][0] = 9.0
        W[p + "sink"][-1] = -30.0
    part, W, p = _mixer("gated", m, dtype, width, seed=dim + rot, hot=1.5, edit=edit)
    cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
    ws = Workspace(DEV)
    g = torch.Generator().manual_seed(rot)
    x = (torch.randn(n, width, generator=g) * 0.3).to(dtype)
    x[2, 0] = 3e4
    h = x.double()
    want = plain_redodra.gated_attention(h, W, p, m, plain_redodra.gated_attention_keys(h, W, p, m))
    quiet = h.clone()
    quiet[2, 0] = 0.0
    small = plain_redodra.gated_attention(quiet, W, p, m, plain_redodra.gated_attention_keys(quiet, W, p, m))
    assert float(want[n - 1].abs().max()) > 20 * float(small[n - 1].abs().max())
    tol = 3e-5 if dtype == F32 else 3e-2
    assert rel_err(_drive(part, cache, x, [n], dtype, ws), want) < tol
    assert rel_err(_drive(part, cache, x, [200, 1], dtype, ws), want) < tol
    assert rel_err(_drive(part, cache, x, [1, 2, 60, 1, 64, 5], dtype, ws), want) < tol
    # the first tokens of a sequence alone: one key and the sink
    assert rel_err(_drive(part, cache, x[:1], [1], dtype, ws), want[:1]) < tol
    assert rel_err(_drive(part, cache, x[:3], [1], dtype, ws), want[:3]) < tol


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    made = {}

    def get(name, seed=0):
        if (name, seed) not in made:
            made[(name, seed)] = redodra_models.make(tmp_path_factory.mktemp("redodra"), name, seed=seed)
        return made[(name, seed)]
    return get


def _engine(model, dtype, **kw):
    from rust_inference_b200.engine.engine import Engine
    return Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=kw.pop("max_tokens", 2048), n_slots=kw.pop("n_slots", 6), **kw)


def _run(eng, slot, tokens, portions):
    """Feed `tokens` to `slot` cut as `portions` says (a list of sizes, the last repeated); logits of every token."""
    rows, at, i = [], 0, 0
    while at < len(tokens):
        k = portions[min(i, len(portions) - 1)]
        rows.append(eng.step([slot], [tokens[at:at + k]], "all").cpu())
        at += k
        i += 1
    return torch.cat(rows)


class Streams:
    rows = []

    def __init__(self):
        self.seen = []

    def record(self, label, hidden, picked=False):
        if not picked:
            self.seen.append(hidden.float().cpu().clone())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_layers_and_decoding(dtype, name, models):
    """A whole prompt (what every layer hands on too), the same with its last tokens one by one (across the edges of
    windows, kept positions and pages), and a slot used again: its state must start at zero, its pages hold old rows."""
    model = models(name)
    eng = _engine(model, dtype)
    reqs = eng.model.cache_requests()
    for i, L in enumerate(model.cfg["layers"]):
        if L["type"] == "attention" and L["mixer"].get("kv_from") is not None:
            assert i >= len(reqs) or reqs[i] is None                   # a reader keeps nothing of its own
    tokens = random_tokens(230, model.cfg["vocab"], 1)
    streams = []
    want = model.plain_logits(tokens, streams=streams)
    tol = TOL[dtype]
    probe = Streams()
    s = eng.alloc_slot()
    got = eng.step([s], [tokens], "all", probe=probe)
    assert rel_err(got, want) < tol
    assert len(probe.seen) == len(streams)
    for a, b in zip(probe.seen, streams):
        assert rel_err(a, b) < tol
    eng.free_slot(s)
    s2 = eng.alloc_slot()
    assert s2 == s
    got = _run(eng, s2, tokens, [60, 1])
    assert rel_err(got, want) < tol
    eng.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_portions_of_several_sizes(dtype, name, models):
    model = models(name)
    eng = _engine(model, dtype)
    tokens = random_tokens(197, model.cfg["vocab"], 2)
    want = model.plain_logits(tokens)
    for portions in ([2], [1, 2, 3, 5, 7, 20, 19, 64, 2], [63, 1, 1, 66, 66], [64, 64, 69], [150, 47], [1]):
        s = eng.alloc_slot()
        assert rel_err(_run(eng, s, tokens, portions), want) < TOL[dtype], portions
        eng.free_slot(s)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batch_against_each_alone(dtype, name, models):
    """Prompts of 1, 2, 70 and 160 tokens as one batch, then decoded together while the short ones leave;
    then a request in a freed slot (a state that must start at zero) while the others still decode."""
    model = models(name)
    eng = _engine(model, dtype)
    vocab = model.cfg["vocab"]
    lens, extra = [1, 2, 70, 160], [3, 9, 30, 12]
    seqs = [random_tokens(n + e, vocab, 10 + i) for i, (n, e) in enumerate(zip(lens, extra))]
    want = [model.plain_logits(t) for t in seqs]
    slots = [eng.alloc_slot() for _ in seqs]
    got = [[] for _ in seqs]
    out = eng.step(slots, [t[:n] for t, n in zip(seqs, lens)], "all").cpu()
    o = 0
    for b, n in enumerate(lens):
        got[b].append(out[o:o + n])
        o += n
    at = list(lens)
    second = None
    while any(a < len(t) for a, t in zip(at, seqs)):
        live = [b for b in range(len(seqs)) if at[b] < len(seqs[b])]
        out = eng.step([slots[b] for b in live], [[seqs[b][at[b]]] for b in live], "last").cpu()
        for i, b in enumerate(live):
            got[b].append(out[i:i + 1])
            at[b] += 1
            if at[b] == len(seqs[b]):
                eng.free_slot(slots[b])
        if second is None and len(live) < len(seqs):
            t2 = random_tokens(77, vocab, 99)
            s = eng.alloc_slot()
            second = (rel_err(eng.step([s], [t2], "all"), model.plain_logits(t2)), s)
            eng.free_slot(s)
    for b in range(len(seqs)):
        assert rel_err(torch.cat(got[b]), want[b]) < TOL[dtype], b
    assert second is not None and second[0] < TOL[dtype]
    eng.check_device_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_through_captured_steps(dtype, name, models):
    """Three tokens of prompt, then 260 decode steps of a batch of two (captured steps), across four pages and past
    every window and every kept position: logits of every step against the plain model."""
    model = models(name)
    eng = _engine(model, dtype)
    vocab = model.cfg["vocab"]
    seqs = [random_tokens(263, vocab, 21), random_tokens(263, vocab, 22)]
    want = [model.plain_logits(t) for t in seqs]
    slots = [eng.alloc_slot(), eng.alloc_slot()]
    eng.step(slots, [t[:3] for t in seqs], "none")
    rows = [[], []]
    for p in range(3, 263):
        out = eng.step(slots, [[t[p]] for t in seqs], "last").cpu()
        rows[0].append(out[0:1])
        rows[1].append(out[1:2])
    assert eng.decode_graph(2) is not None and eng.decode_graph(2).graph is not None
    for b in range(2):
        assert rel_err(torch.cat(rows[b]), want[b][3:]) < TOL[dtype]
    eng.check_device_status()


def test_what_carries_a_far_token(tmp_path):
    """The first token lies outside the window of a late position and is not kept: in a model of windowed layers
    whose other member forgets quickly the late logits do not depend on it; with a causal layer, a delta layer or a
    slowly forgetting state they do.  The engine agrees with the plain model in every case, decoding the last tokens."""
    R = redodra_models
    par = R.layer("parallel", R.side(R.window(heads=2, kv=1, dim=16, vdim=16, scale=0.25, cap=20.0, size=9, keep=0),
                                     R.ssm(heads=2, vdim=8, state=8, groups=1, conv=2, norm_groups=1)), 40)
    kept = R.layer("parallel", R.side(R.window(heads=2, kv=1, dim=16, vdim=16, scale=0.25, cap=20.0, size=9, keep=1),
                                      R.ssm(heads=2, vdim=8, state=8, groups=1, conv=2, norm_groups=1)), 40)
    causal = R.layer("attention", R.attn(heads=2, kv=1, dim=16, vdim=16, scale=0.2, cap=20.0, base=1000.0, rot=8), 40)
    delta = R.layer("delta", R.delta(heads=2, kv=1, dim=16, vdim=8, conv=2), 40)
    base = {"architecture": "Redodra", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}}

    def forget(fast):
        def edit(W):
            for k in W:
                if k.endswith("right.A_log") or k.endswith("mix.A_log"):
                    W[k].fill_(2.0 if fast else -6.0)
                if k.endswith("dt_bias"):
                    W[k].fill_(3.0 if fast else -1.0)
        return edit
    cases = (("windows", [par, par, par], True, False), ("slow_state", [par, par, par], False, True),
             ("kept", [par, kept, par], True, True), ("causal", [par, causal, par], True, True), ("delta", [par, delta, par], False, True))
    for name, layers, fast, reaches in cases:
        model = R.make(tmp_path, name, cfg={**base, "layers": layers}, edit=forget(fast))
        eng = _engine(model, "float32")
        a = random_tokens(230, 97, 5)
        b = [(a[0] + 1) % 97] + a[1:]
        out = []
        for t in (a, b):
            s = eng.alloc_slot()
            got = _run(eng, s, t, [228, 1])
            eng.free_slot(s)
            assert rel_err(got, model.plain_logits(t)) < TOL["float32"], name
            out.append(got[-1])
        differs = float((out[0] - out[1]).abs().max()) > 1e-4
        assert differs == reaches, name


def test_greedy_generation_through_the_api(models):
    """`Model.generate` (admission, prefill, captured decode steps, sampling on the device) against the plain
    model's greedy continuation, for prompts of unequal length; what a position costs in the cache and what a
    sequence costs in state."""
    from rust_inference_b200 import Model, SamplerConfig
    model = models("A")
    prompts = [random_tokens(5, model.cfg["vocab"], 31), random_tokens(40, model.cfg["vocab"], 32), [7]]
    n_new = 12
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=1024)
    got = m.generate(prompts, n_new, SamplerConfig.plain(temperature=0.0), stop_ids=())
    for p, g in zip(prompts, got):
        assert list(g.tokens) == plain_redodra.greedy(model.cfg, model.weights, p, n_new)
    per_position = 0
    for L in model.cfg["layers"]:
        mx = L["mixer"]
        if L["type"] == "attention" and mx.get("kv_from") is None:
            per_position += mx["kv_heads"] * (mx["dim"] + mx["vdim"]) * 4
        elif L["type"] == "parallel":
            per_position += mx["left"]["kv_heads"] * (mx["left"]["dim"] + mx["left"]["vdim"]) * 4
    assert m.memory()["cache_bytes_per_position"] == per_position


def test_state_dict_round_trip(models):
    """The tensors come back apart under the file's names."""
    from rust_inference_b200 import Model
    model = models("B")
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=512)
    sd = m.state_dict()
    assert set(sd) == set(model.weights)
    for k, v in model.weights.items():
        assert torch.equal(sd[k].float().cpu().reshape(v.shape), v), k


def test_trace_replay_picks_the_model_by_its_config(models, tmp_path):
    """`bin/trace_run` on a Redodra folder: two requests start together, go on by one token and end at different
    steps; then a third request takes a slot given back."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    model = models("A")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a, b, c = (random_tokens(n, model.cfg["vocab"], 40 + n) for n in (70, 9, 30))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[66]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[67]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[68]], "want": []}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": [a[69]], "want": [0]}], "end": ["a"]},
             {"step": 5, "entries": [{"id": "c", "tokens": c, "want": [0, 29]}], "end": ["c"]}]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / ("out_" + dtype)
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model.folder, "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(6)]
        wa, wb, wc = (model.plain_logits(t) for t in (a, b, c))
        read = lambda i, rows: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(rows, -1))
        assert not (out / "3.f32").exists()
        tol = TOL[dtype]
        assert rel_err(read(0, 3), torch.stack([wa[0], wa[65], wb[6]])) < tol
        assert rel_err(read(1, 1), wa[66:67]) < tol
        assert rel_err(read(2, 2), torch.stack([wa[67], wb[8]])) < tol
        assert rel_err(read(4, 1), wa[69:70]) < tol
        assert rel_err(read(5, 2), wc[[0, 29]]) < tol


def test_the_command_line_on_a_redodra_folder(models, tmp_path):
    """`bin/gguf-infer` as a process: greedy ids from a model folder equal the plain model's, and the random-weights
    mode runs from a config.json alone."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli = os.path.join(root, "bin", "gguf-infer")
    model = models("B")
    prompts = [random_tokens(n, model.cfg["vocab"], 70 + n) for n in (9, 1)]
    args = [sys.executable, cli, "--model", model.folder, "--temperature", "0", "--repetition-penalty", "1", "--max-tokens", "6",
            "--dtype", "float32", "--max-seq-len", "256", "--stop-ids", ""]
    for p in prompts:
        args += ["--prompt", ",".join(str(t) for t in p)]
    p = subprocess.run(args, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert [[int(t) for t in l.split()] for l in lines] == [plain_redodra.greedy(model.cfg, model.weights, q, 6) for q in prompts]
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(redodra_models.CONFIGS["A"]))
    p = subprocess.run([sys.executable, cli, "--random-config", str(cfg_file), "--weights-seed", "3", "--random-prompts", "2:4:20",
                        "-n", "5", "--max-seq-len", "128"], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len([l for l in p.stdout.splitlines() if l.strip()]) == 2


@pytest.mark.parametrize("kind,dim", [("gated", 64), ("gated", 128), ("window", 64), ("window", 128)])
def test_tensor_core_kernel_takes_the_forms_of_the_score(kind, dim, monkeypatch):
    """bfloat16 heads of 64 and 128 channels with a cap, a bias, kept positions, a sink or a gate run on the tensor-core
    kernel, prompts and single tokens alike: the generic kernel is not called."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    from rust_inference_b200.kernels import ops

    def refuse(*a, **k):
        raise AssertionError("the generic attention kernel was called")
    width, n, dtype = 128, 200, torch.bfloat16
    if kind == "gated":
        m = redodra_models.attn(heads=4, kv=2, dim=dim, vdim=dim, scale=0.8 / math.sqrt(dim), cap=9.0, base=3000.0, rot=16)
    else:
        m = redodra_models.window(heads=4, kv=1, dim=dim, vdim=dim, scale=0.6 / math.sqrt(dim), cap=7.0, size=70, keep=5)
    part, W, p = _mixer(kind, m, dtype, width, seed=dim, hot=1.5)
    cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
    x = (torch.randn(n, width, generator=torch.Generator().manual_seed(3)) * 0.3).to(dtype)
    h = x.double()
    want = (plain_redodra.gated_attention(h, W, p, m, plain_redodra.gated_attention_keys(h, W, p, m)) if kind == "gated"
            else plain_redodra.windowed_attention(h, W, p, m))
    monkeypatch.setattr(ops, "attention_generic", refuse)
    ws = Workspace(DEV)
    assert rel_err(_drive(part, cache, x, [150, 1], dtype, ws), want) < 3e-2


@pytest.mark.parametrize("kind,dim,heads,kv", [("gated", 64, 8, 2), ("gated", 128, 4, 4), ("window", 64, 6, 2), ("window", 128, 16, 1)])
@pytest.mark.parametrize("splits", [None, "1", "3"])
def test_single_tokens_with_forms_of_the_score_in_runs_of_pages(kind, dim, heads, kv, splits, monkeypatch):
    """Steps of one token per sequence with a cap, a bias, kept positions, a sink or a gate: the heads of a kv head are
    one CTA's rows and the pages are cut into runs (one run, a few, as many as the GPU holds: some stay empty).  Kept
    positions fill more than one page and lie pages before the window; a query whose key is the far one stands out."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    from rust_inference_b200.kernels import ops, attention as attn_kernels

    def refuse(*a, **k):
        raise AssertionError("another attention kernel was called for a step of single tokens")
    width, n, first, dtype = 128, 460, 430, torch.bfloat16
    if kind == "gated":
        m = redodra_models.attn(heads=heads, kv=kv, dim=dim, vdim=dim, scale=0.9 / math.sqrt(dim), cap=11.0, base=5000.0, rot=32)
    else:
        m = redodra_models.window(heads=heads, kv=kv, dim=dim, vdim=dim, scale=0.7 / math.sqrt(dim), cap=6.0, size=150, keep=70)
    part, W, p = _mixer(kind, m, dtype, width, seed=dim + heads, hot=1.5)
    cache = SequenceCache([part.cache_request()], max_tokens=2048, max_seq_len=1024, dtype=dtype, device=DEV, n_slots=2)
    x = (torch.randn(n, width, generator=torch.Generator().manual_seed(heads)) * 0.3).to(dtype)
    x[n - 7] = x[3] * 4                    # a late query that resembles an early key (a kept position, far before the window)
    h = x.double()
    want = (plain_redodra.gated_attention(h, W, p, m, plain_redodra.gated_attention_keys(h, W, p, m)) if kind == "gated"
            else plain_redodra.windowed_attention(h, W, p, m))
    if splits is not None:
        monkeypatch.setenv("RI_B200_DECODE_SPLITS", splits)
    ws = Workspace(DEV)
    whole = _drive(part, cache, x, [n], dtype, ws)
    monkeypatch.setattr(ops, "attention_generic", refuse)
    prefill = ops.attention_prefill_forms
    calls = []

    def prompts_only(q, *a, **k):
        assert q.shape[0] > 1, "the prompts' kernel was called for a step of single tokens"
        return prefill(q, *a, **k)
    decode = ops.attention_decode_forms

    def counted(*a, **k):
        calls.append(k["n_splits"])
        return decode(*a, **k)
    monkeypatch.setattr(ops, "attention_prefill_forms", prompts_only)
    monkeypatch.setattr(ops, "attention_decode_forms", counted)
    got = _drive(part, cache, x, [first, 1], dtype, ws)
    assert len(calls) == n - first and (splits is None or set(calls) == {int(splits)})
    assert rel_err(got, want) < 3e-2 and rel_err(whole, want) < 3e-2
    assert rel_err(got[first:], want[first:]) < 3e-2
    assert rel_err(got[first:], whole[first:]) < 2e-2
