"""The Belizen decoder in the engine against the plain restatement (`plain_belizen`): each mechanism's kernels alone,
then whole models: prompts whole, token by token, in portions down to two tokens, unequal batches, slots and pages used
again, keys at the edges of windows, of the kept first positions and of pages, far keys, the first tokens of a
sequence, long decoding, and greedy generation through `Model.generate`."""
import math

import pytest
import torch

import belizen_models as bm
import plain_belizen
from conftest import random_tokens, rel_err
from test_redodra_gpu import _drive, d, make_ctx

# Worst row's max |a - b| / max |b| against the plain model in float64.  float32 runs: a kernel fault shows far above
# 1e-4.  bfloat16 runs keep bfloat16 activations between the kernels of a sublayer (the stream, the states, the norms,
# the router and the scores stay float32): rounding alone reaches a few 1e-2 on single rows of a model whose layers
# run up to ten times (observed: float32 2e-5, bfloat16 1e-2); a key too many or too few, a lost state or a wrong expert
# costs 0.2 and more.
TOL = {"float32": 1e-4, "bfloat16": 3e-2}

pytestmark = pytest.mark.gpu

DEV = "cuda"
F32, BF16 = torch.float32, torch.bfloat16


# ---------------------------------------------------------------------------------------------------
# the gate of the dense feed-forward in the products' epilogue
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("n,width,ff", [(1, 72, 40), (5, 128, 200), (130, 128, 264), (600, 256, 520), (9, 100, 36)])
def test_tanh_gelu_gate_with_a_factor_in_the_product_s_epilogue(dtype, n, width, ff):
    """act(W_gate x) * (W_up x) * factor with the tanh form of GELU, in every form of the contraction (FFMA, tcgen05
    with few tokens, with more than 128 and with 512 or more); pre-activations from -6 to 6."""
    from rust_inference_b200.kernels import linear, ops
    g = torch.Generator().manual_seed(n + ff)
    x = (torch.randn(n, width, generator=g) * 2.0).to(dtype)
    wg = (torch.randn(ff, width, generator=g) / math.sqrt(width)).to(dtype)
    wu = (torch.randn(ff, width, generator=g) / math.sqrt(width)).to(dtype)
    want = plain_belizen.gelu_tanh(x.double() @ wg.double().T) * (x.double() @ wu.double().T) * 0.65
    form = ops.gate_form(alpha=ops.GELU_TANH_ALPHA, cubic=ops.GELU_TANH_CUBIC, mult=0.65, device=DEV)
    out = torch.empty(n, ff, dtype=dtype, device=DEV)
    linear.gated(d(x), linear.Weight(d(wg)), linear.Weight(d(wu)), out, None, form=form)
    assert rel_err(out, want) < (2e-5 if dtype == F32 else 1.2e-2)


def test_interpolated_rotation_tables():
    """cos and sin of the library's tables against the plain frequencies: slowed channels, untouched ones, the ramp
    between them and the magnitude; also limits that leave the ramp empty on one side."""
    from rust_inference_b200.parts.rope import rope_tables
    for dims, base, scaling in ((32, 20000.0, (6.0, 512, 24.0, 1.5)), (8, 5000.0, (3.0, 64, 8.0, 0.5)), (2, 100.0, (2.0, 16, 1.0, 1.0)),
                                (64, 500000.0, (8.0, 4096, 4.0, 2.0)), (16, 50.0, (1.5, 100000, 64.0, 32.0))):
        sc = dict(zip(("factor", "original", "fast", "slow"), scaling))
        cos, sin = rope_tables(dims, base, 300, exact_angles=True, interpolation=sc)
        f, mag = plain_belizen.interpolated_frequencies(dims, base, sc)
        ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
        assert torch.allclose(torch.from_numpy(cos).double(), mag * torch.cos(ang), atol=2e-7)
        assert torch.allclose(torch.from_numpy(sin).double(), mag * torch.sin(ang), atol=2e-7)


# ---------------------------------------------------------------------------------------------------
# parts alone, outside an engine
# ---------------------------------------------------------------------------------------------------
def _part(role, layer, dtype, width, seed, eps=1e-5, mult=1.0, edit=None, pin=True):
    """One part of the library as the model's builder makes it for a one-layer model, holding random tensors; the same
    tensors in float64 for the plain functions, and the tensors' prefix."""
    from rust_inference_b200.config.belizen_config import BelizenConfig
    from rust_inference_b200.models.belizen import build_spec
    from rust_inference_b200.parts.registry import lookup
    cfg = bm.model(vocab=10, width=width, eps=eps, scale=1.0, mult=mult, layers=[layer])
    W = {k: v.float() for k, v in bm.random_weights(cfg, seed, pin_routing=pin).items()}
    prefix = "l0.mix." if role == "mixer" else "l0.mlp."
    if edit is not None:
        edit(W, prefix)
    ps = build_spec(BelizenConfig.from_dict(cfg)).layers[0].parts[role]
    part = lookup("mixer" if role == "mixer" else "feed_forward", ps.kind)(hidden_size=width, dtype=dtype, device=DEV, **ps.params)
    part.set_tensors({local: d(W[prefix + local], F32 if ts.role == "vector" else dtype) for local, ts in part.tensor_specs().items()})
    part.prepare(2048)
    return part, {k: v.double() for k, v in W.items()}, prefix


class _Scratch:
    """What a feed-forward needs of a step's context: its buffers."""

    def __init__(self, ws, dtype):
        self.ws, self.dtype = ws, dtype

    def buffer(self, name, shape, dtype):
        return self.ws.get(name, shape, dtype)

    def zeroed_buffer(self, name, shape, dtype):
        return self.ws.get_zeroed(name, shape, dtype)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("experts,identity,top,ff,shared", [(3, 5, 3, 24, 40), (5, 0, 1, 16, None), (8, 3, 5, 64, 96), (2, 6, 2, 8, None),
                                                            (1, 1, 2, 40, 24), (12, 3, 6, 20, 12)])
def test_softmax_router_with_pass_through_experts(dtype, experts, identity, top, ff, shared):
    """The mixture as a part against the plain one, for 1, 7, 300 and 1,100 tokens (the experts' products on the FFMA
    pipe and on the tensor cores, the gather inside the arranging kernel and in a kernel of its own): softmax scores
    over all router outputs, the correction on the choice only, weights not normalised, chosen experts that hand
    their input through, a factor on the whole.  bfloat16 runs pin the choice by the corrections, float32 runs route
    freely; with 2 experts of 8 and the choice pinned to the others no pair reaches an expert with tensors."""
    from rust_inference_b200.engine.context import Workspace
    width = 72 if ff == 16 else 128
    mlp = bm.moe(experts=experts, top=top, ff=ff, limit=0.9, identity=identity, shared=None if shared is None else (shared, 1.3))
    layer = bm.layer("gla", bm.gla(heads=1, dim=8, vdim=8, tau=2.0, rank=2), mlp)

    def only_pass_through(W, p):
        if experts == 2:
            W[p + "correction"][:2] = -50.0
    part, W, p = _part("feed_forward", layer, dtype, width, seed=experts + top, mult=0.6, edit=only_pass_through, pin=dtype == BF16)
    ws = Workspace(DEV)
    for n in (1, 7, 300, 1100):
        g = torch.Generator().manual_seed(n)
        x = torch.randn(n, width, generator=g).to(dtype)
        want = 0.6 * plain_belizen.experts_ff(x.double(), W, p, mlp)
        got = torch.zeros(n, width, device=DEV)
        part.forward(d(x), got, _Scratch(ws, dtype))
        assert rel_err(got, want) < (3e-5 if dtype == F32 else 2e-2), n


def test_router_choice_and_weights():
    """The routing kernel against the plain router: ids in the order of the choice, weights the plain scores."""
    from rust_inference_b200.kernels import ops
    for n, width, outputs, top in ((1, 72, 5, 1), (9, 128, 12, 4), (40, 256, 70, 8), (700, 100, 33, 6), (3000, 64, 3, 3)):
        g = torch.Generator().manual_seed(n)
        x = torch.randn(n, width, generator=g)
        router = torch.randn(outputs, width, generator=g) / math.sqrt(width) * 2
        corr = 0.1 * torch.randn(outputs, generator=g)
        ids, weights = plain_belizen.route(x.double(), router.double(), corr.double(), top)
        sums = torch.empty(n, outputs + 1, dtype=torch.float32, device=DEV)
        count = torch.zeros(n, dtype=torch.int32, device=DEV)
        for split in ((1, 2, 5, 16) if n < 296 else (1,)):          # the router's rows over so many blocks per token
            got_ids = torch.empty(n, top, dtype=torch.int32, device=DEV)
            got_w = torch.empty(n, top, dtype=torch.float32, device=DEV)
            ops.moe_route(d(x), d(router), d(corr), got_ids, got_w, top=top, softmax=True, normalise=False, split=split,
                          split_sums=sums, split_count=count)
            assert torch.equal(got_ids.cpu().long(), ids), split
            assert torch.allclose(got_w.cpu().double(), weights, rtol=2e-5, atol=1e-7), split
            assert int(count.abs().sum()) == 0                       # the counters are zero again


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("heads,dim,vdim,tau,rank", [(3, 24, 40, 8.0, 5), (1, 72, 33, 1.0, 1), (2, 8, 16, 20.0, 12), (4, 64, 64, 12.0, 24),
                                                      (2, 130, 100, 4.0, 7), (5, 6, 9, 2.5, 3)])
def test_linear_attention_alone(dtype, heads, dim, vdim, tau, rank):
    """The mixer over one sequence whole (long runs are scanned in pieces side by side), in portions of 1, 2, 5, 64 and
    140 tokens, token by token, and in a slot that was used before: the state must start at zero and move on."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n = 96, 300
    m = bm.gla(heads=heads, dim=dim, vdim=vdim, tau=tau, rank=rank)
    part, W, p = _part("mixer", bm.layer("gla", m), dtype, width, seed=dim + rank, mult=0.8)
    g = torch.Generator().manual_seed(rank)
    x = (torch.randn(n, width, generator=g) * 0.7).to(dtype)
    want = 0.8 * plain_belizen.linear_attention_mixer(x.double(), W, p, m, 1e-5)
    cache = SequenceCache([part.cache_request()], max_tokens=2048, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
    ws = Workspace(DEV)
    tol = 3e-5 if dtype == F32 else 3e-2
    for portions in ([n], [140, 64, 5, 2, 1], [2], [129, 1]):
        assert rel_err(_drive(part, cache, x, portions, dtype, ws), want) < tol, portions


def test_linear_attention_remembers_a_far_token():
    """With slow decays one early token changes the result hundreds of positions later by far more than rounding; the
    library agrees with the plain result with and without it, also token by token, and two sequences as one batch
    equal each alone."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n = 64, 330
    m = bm.gla(heads=2, dim=32, vdim=16, tau=64.0, rank=4)

    def slow(W, p):
        W[p + "a2.b"].fill_(6.0)
    part, W, p = _part("mixer", bm.layer("gla", m), F32, width, seed=5, edit=slow)
    g = torch.Generator().manual_seed(9)
    a = torch.randn(n, width, generator=g) * 0.5
    b = a.clone()
    b[4] = b[4] * 8.0
    wa = plain_belizen.linear_attention_mixer(a.double(), W, p, m, 1e-5)
    wb = plain_belizen.linear_attention_mixer(b.double(), W, p, m, 1e-5)
    assert float((wa[-1] - wb[-1]).abs().max()) > 1e-2 * float(wa[-1].abs().max())
    cache = SequenceCache([part.cache_request()], max_tokens=2048, max_seq_len=512, dtype=F32, device=DEV, n_slots=3)
    ws = Workspace(DEV)
    for x, want in ((a, wa), (b, wb)):
        assert rel_err(_drive(part, cache, x, [n], F32, ws), want) < 1e-4
        assert rel_err(_drive(part, cache, x, [40, 1], F32, ws), want) < 1e-4
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
        W[p + name][:, 0] = 0.0


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("heads,kv,dim,vdim,size,keep,rot", [(4, 2, 16, 24, 20, 3, 8), (2, 2, 8, 8, 150, 70, 8), (1, 1, 24, 24, 1, 1, None),
                                                             (3, 1, 8, 16, 33, 0, 2), (4, 2, 64, 64, 70, 10, 32), (2, 1, 128, 128, 129, 64, 128),
                                                             (6, 2, 64, 32, 64, 65, 16)])
def test_window_and_kept_edges_with_a_value_that_dwarfs_the_rest(dtype, heads, kv, dim, vdim, size, keep, rot):
    """The attention mixer (biases, normed and rotated heads, capped scores, the window with kept first positions, the
    gate on the result).  One position's value is made huge: the results differ by orders of magnitude between the
    last query that sees it and the first that does not.  The position lies at the window's edge on both sides of a
    page border, and is the last kept position (seen for ever) or the first one not kept (lost when the window has
    passed).  As one prompt, with the later tokens one by one, and in portions whose borders fall inside the window."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n, cut = 128, 330, 150
    m = bm.attn(heads=heads, kv=kv, dim=dim, vdim=vdim, scale=0.6 / math.sqrt(dim), cap=7.0, size=size, keep=keep,
                base=None if rot is None else 3000.0, rot=rot, scaling=None if rot in (None, 2) else (4.0, 128, 16.0, 1.0))
    part, W, p = _part("mixer", bm.layer("attention", m), dtype, width, seed=dim + size, mult=0.9, edit=_blind_channel)
    cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
    ws = Workspace(DEV)
    tol = 3e-5 if dtype == F32 else 3e-2
    for big in sorted({63, 64, 130, max(keep - 1, 0), keep}):
        g = torch.Generator().manual_seed(big)
        x = (torch.randn(n, width, generator=g) * 0.3).to(dtype)
        x[big, 0] = 3e4
        want = 0.9 * plain_belizen.attention_mixer(x.double(), W, p, m, 1e-5)
        lost = big + size                                         # the first query that no longer sees `big` through the window
        if big >= keep and lost < n:
            assert float(want[lost - 1].abs().max()) > 20 * float(want[lost].abs().max())
        if big < keep:
            quiet = x.clone()
            quiet[big, 0] = 0.0
            assert float(want[n - 1].abs().max()) > 20 * float(plain_belizen.attention_mixer(quiet.double(), W, p, m, 1e-5)[n - 1].abs().max())
        assert rel_err(_drive(part, cache, x, [n], dtype, ws), want) < tol, big
        assert rel_err(_drive(part, cache, x, [cut, 1], dtype, ws), want) < tol, big
    assert rel_err(_drive(part, cache, x, [2, 1, 61, 3, 64, 7], dtype, ws), want) < tol
    # the first tokens of a sequence alone
    assert rel_err(_drive(part, cache, x[:1], [1], dtype, ws), want[:1]) < tol
    assert rel_err(_drive(part, cache, x[:3], [1], dtype, ws), want[:3]) < tol


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("heads,kv,dim,vdim,rot", [(4, 1, 32, 16, 8), (4, 2, 64, 64, 32), (2, 1, 128, 128, 2), (2, 2, 40, 72, 10)])
def test_causal_attention_sees_a_far_value(dtype, heads, kv, dim, vdim, rot):
    """Without a window a huge value at position 2 reaches queries hundreds of positions and several pages later, in a
    prompt and decoding; scores are not capped here."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n = 128, 330
    m = bm.attn(heads=heads, kv=kv, dim=dim, vdim=vdim, scale=0.8 / math.sqrt(dim), base=3000.0, rot=rot, scaling=(2.0, 256, 8.0, 2.0))
    part, W, p = _part("mixer", bm.layer("attention", m), dtype, width, seed=dim + rot, edit=_blind_channel)
    cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=dtype, device=DEV, n_slots=2)
    ws = Workspace(DEV)
    g = torch.Generator().manual_seed(rot)
    x = (torch.randn(n, width, generator=g) * 0.3).to(dtype)
    x[2, 0] = 3e4
    want = plain_belizen.attention_mixer(x.double(), W, p, m, 1e-5)
    quiet = x.clone()
    quiet[2, 0] = 0.0
    assert float(want[n - 1].abs().max()) > 10 * float(plain_belizen.attention_mixer(quiet.double(), W, p, m, 1e-5)[n - 1].abs().max())
    tol = 3e-5 if dtype == F32 else 3e-2
    assert rel_err(_drive(part, cache, x, [n], dtype, ws), want) < tol
    assert rel_err(_drive(part, cache, x, [200, 1], dtype, ws), want) < tol
    assert rel_err(_drive(part, cache, x, [1, 2, 60, 1, 64, 5], dtype, ws), want) < tol


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    made = {}

    def get(name, dtype="bfloat16", seed=0):
        pin = dtype == "bfloat16"                 # float32 runs route freely
        if (name, pin, seed) not in made:
            made[(name, pin, seed)] = bm.make(tmp_path_factory.mktemp("belizen"), name, seed=seed, pin_routing=pin)
        return made[(name, pin, seed)]
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
    """A whole prompt (the stream after every layer run too: a looped layer counts each time), the same with its last
    tokens one by one (across the edges of windows, kept positions and pages), and a slot used again: its states must
    start at zero, its pages hold old rows."""
    model = models(name, dtype)
    eng = _engine(model, dtype)
    tokens = random_tokens(230, model.cfg["vocab"], 1)
    streams = []
    want = model.plain_logits(tokens, layers_out=streams)
    assert len(streams) == len(plain_belizen.run_order(model.cfg))
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
    model = models(name, dtype)
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
    """Prompts of 1, 2, 70 and 160 tokens as one batch, then decoded together while the short ones leave; then a
    request in a freed slot (states that must start at zero) while the others still decode."""
    model = models(name, dtype)
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
    model = models(name, dtype)
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
    """The first token lies outside the window of a late position and is not kept: in a model of windowed layers the
    late logits do not depend on it; with a kept first position, a layer without a window or a gla layer they do.  The
    engine agrees with the plain model in every case, decoding the last tokens."""
    win = bm.layer("attention", bm.attn(heads=2, kv=1, dim=16, vdim=16, scale=0.25, cap=20.0, size=9, keep=0, base=1000.0, rot=8), bm.dense(40))
    kept = bm.layer("attention", bm.attn(heads=2, kv=1, dim=16, vdim=16, scale=0.25, cap=20.0, size=9, keep=1, base=1000.0, rot=8), bm.dense(40))
    causal = bm.layer("attention", bm.attn(heads=2, kv=1, dim=16, vdim=16, scale=0.2, cap=20.0, base=1000.0, rot=8), bm.dense(40))
    state = bm.layer("gla", bm.gla(heads=2, dim=16, vdim=8, tau=32.0, rank=3), bm.dense(40))

    def slow(W):
        for k in W:
            if k.endswith("a2.b"):
                W[k].fill_(5.0)
    cases = (("windows", [win, win, win], None, False), ("kept", [win, kept, win], None, True), ("causal", [win, causal, win], None, True),
             ("state", [win, state, win], None, True), ("looped", [win, win], (0, 2, 3), False), ("looped_state", [win, state], (1, 2, 2), True))
    for name, layers, loop, reaches in cases:
        cfg = bm.model(vocab=97, width=64, eps=1e-6, scale=2.0, mult=0.9, cap=10.0, layers=layers, loop=loop)
        model = bm.make(tmp_path, name, cfg=cfg, edit=slow, pin_routing=False)
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


def test_rank_from_the_tensor_s_shape(models, tmp_path):
    """config.json without the decays' rank: the weight file's shapes give it."""
    model = bm.make(tmp_path, "A", seed=3, drop_rank=True, pin_routing=False)
    eng = _engine(model, "float32")
    tokens = random_tokens(50, model.cfg["vocab"], 3)
    s = eng.alloc_slot()
    assert rel_err(eng.step([s], [tokens], "all"), model.plain_logits(tokens)) < TOL["float32"]


def test_greedy_generation_through_the_api(models):
    """`Model.generate` (admission, prefill, captured decode steps, sampling on the device) against the plain model's
    greedy continuation, for prompts of unequal length; what a position costs in the cache."""
    from rust_inference_b200 import Model, SamplerConfig
    model = models("A", "float32")
    prompts = [random_tokens(5, model.cfg["vocab"], 31), random_tokens(40, model.cfg["vocab"], 32), [7]]
    n_new = 12
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=1024)
    got = m.generate(prompts, n_new, SamplerConfig.plain(temperature=0.0), stop_ids=())
    for p, g in zip(prompts, got):
        assert list(g.tokens) == plain_belizen.greedy(model.cfg, model.weights, p, n_new)
    per_position = 0
    for i, _ in plain_belizen.run_order(model.cfg):
        L = model.cfg["layers"][i]
        if L["type"] == "attention":
            per_position += L["mixer"]["kv_heads"] * (L["mixer"]["dim"] + L["mixer"]["vdim"]) * 4
    assert m.memory()["cache_bytes_per_position"] == per_position


def test_state_dict_round_trip(models):
    """The tensors come back apart under the file's names."""
    from rust_inference_b200 import Model
    model = models("B", "float32")
    m = Model.load(model.folder, dtype="float32", max_tokens_in_cache=512)
    sd = m.state_dict()
    assert set(sd) == set(model.weights)
    for k, v in model.weights.items():
        assert torch.equal(sd[k].float().cpu().reshape(v.shape), v), k


def test_trace_replay_picks_the_model_by_its_config(models, tmp_path):
    """`bin/trace_run` on a Belizen folder: two requests start together, go on by one token and end at different
    steps; then a third request takes a slot given back."""
    import json
    import os
    import subprocess
    import sys
    import numpy as np
    model = models("A", "float32")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    a, b, c = (random_tokens(n, model.cfg["vocab"], 40 + n) for n in (70, 9, 30))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[66]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[67]], "want": [0]}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": [a[68]], "want": []}], "end": []},
             {"step": 4, "entries": [{"id": "a", "tokens": [a[69]], "want": [0]}], "end": ["a"]},
             {"step": 5, "entries": [{"id": "c", "tokens": c, "want": [0, 29]}], "end": ["c"]}]
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model.folder, "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "256"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(6)]
    wa, wb, wc = (model.plain_logits(t) for t in (a, b, c))
    V = model.cfg["vocab"]
    read = lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V))
    assert rel_err(read(0), torch.stack([wa[0], wa[65], wb[6]])) < 1e-4
    assert rel_err(read(1), wa[66:67]) < 1e-4
    assert rel_err(read(2), torch.stack([wa[67], wb[8]])) < 1e-4
    assert not (out / "3.f32").exists()
    assert rel_err(read(4), wa[69:70]) < 1e-4
    assert rel_err(read(5), torch.stack([wc[0], wc[29]])) < 1e-4


def test_the_command_line_on_a_belizen_folder(models, tmp_path):
    """`bin/gguf-infer` as a process: greedy ids from a model folder equal the plain model's, and the random-weights
    mode runs from a config.json alone (which must then give the decays' rank)."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli = os.path.join(root, "bin", "gguf-infer")
    model = models("B", "float32")
    prompts = [random_tokens(n, model.cfg["vocab"], 70 + n) for n in (9, 1)]
    args = [sys.executable, cli, "--model", model.folder, "--temperature", "0", "--repetition-penalty", "1", "--max-tokens", "6",
            "--dtype", "float32", "--max-seq-len", "256", "--stop-ids", ""]
    for p in prompts:
        args += ["--prompt", ",".join(str(t) for t in p)]
    p = subprocess.run(args, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert [[int(t) for t in l.split()] for l in lines] == [plain_belizen.greedy(model.cfg, model.weights, q, 6) for q in prompts]
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(bm.CONFIGS["A"]))
    p = subprocess.run([sys.executable, cli, "--random-config", str(cfg_file), "--weights-seed", "3", "--random-prompts", "2:4:20",
                        "-n", "5", "--max-seq-len", "128"], capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len([l for l in p.stdout.splitlines() if l.strip()]) == 2


# ---------------------------------------------------------------------------------------------------
# small kernels alone
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("rows,width,ld,col", [(1, 72, 200, 100), (7, 128, 512, 384), (300, 264, 1000, 8), (5, 33, 90, 41), (2100, 1024, 3080, 2048)])
def test_sigmoid_gate_in_place(dtype, rows, width, ld, col):
    """x *= sigmoid(gate columns) * factor: rows that move 16 bytes at a time (widths and offsets that are multiples
    of 8) and rows that cannot."""
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(rows + width)
    x = torch.randn(rows, width, generator=g).to(dtype)
    wide = (torch.randn(rows, ld, generator=g) * 3.0).to(dtype)
    want = x.double() * torch.sigmoid(wide.double()[:, col:col + width]) * 0.45
    got = ops.sigmoid_gate_(d(x), d(wide), col, 0.45)
    assert rel_err(got, want) < (1e-6 if dtype == F32 else 6e-3)


def test_logit_cap_and_stream_add():
    from rust_inference_b200.kernels import ops
    g = torch.Generator().manual_seed(4)
    x = torch.randn(37, 301, generator=g) * 40.0
    got = ops.softcap_(d(x), 17.0)
    assert torch.allclose(got.cpu().double(), 17.0 * torch.tanh(x.double() / 17.0), atol=2e-5)
    s, other, row = torch.randn(9, 100, generator=g), torch.randn(9, 100, generator=g), torch.randn(100, generator=g)
    for o, r in ((other, row), (None, row), (other, None)):
        want = s.clone() + (o if o is not None else 0) + (r if r is not None else 0)
        got = ops.stream_add(d(s.clone()), None if o is None else d(o), None if r is None else d(r))
        assert torch.allclose(got.cpu(), want, atol=1e-6)


def test_pass_entry_alone():
    """What joins the stream at a pass: the pass's vector always, the kept embedding output from the second pass on."""
    from rust_inference_b200.engine.context import Workspace
    from rust_inference_b200.parts.registry import lookup
    width, n = 72, 11
    part = lookup("stream", "pass_entry")(passes=3, readd_input=True, weight_name="step", hidden_size=width, dtype=BF16, device=DEV)
    assert {k: tuple(v.shape) for k, v in part.tensor_specs().items()} == {"step": (3, width)}
    g = torch.Generator().manual_seed(1)
    step, first = torch.randn(3, width, generator=g), torch.randn(n, width, generator=g)
    part.set_tensors({"step": d(step)})
    ctx = _Scratch(Workspace(DEV), BF16)
    stream = d(first.clone())
    part.begin(stream, ctx)
    want = first.clone()
    for t in range(3):
        stream += 1.0                                 # a layer's work between the passes
        want = want + 1.0 + (first if t > 0 else 0) + step[t]
        part.forward(stream, ctx, t)
        assert torch.allclose(stream.cpu(), want, atol=1e-5), t
    with pytest.raises(ValueError):
        part.forward(stream, ctx, 3)


@pytest.mark.parametrize("heads,kv,dim,cap,size,keep", [(20, 1, 64, None, 100, 5), (4, 1, 128, None, 64, 64), (8, 2, 64, 9.0, None, None),
                                                        (40, 2, 64, 9.0, 70, 0), (2, 2, 128, 30.0, 200, 129)])
def test_tensor_core_sizes_with_each_form_alone(heads, kv, dim, cap, size, keep):
    """bfloat16 heads of 64 and 128: kept first positions without a cap, a cap without a window, a window and a cap
    without kept positions, more than 16 query heads to a kv head (whose single tokens take the prompts' kernel), kept
    positions beyond two pages; a prompt of five pages, then single tokens, then portions."""
    from rust_inference_b200.cache.sequence_cache import SequenceCache
    from rust_inference_b200.engine.context import Workspace
    width, n = 128, 330
    m = bm.attn(heads=heads, kv=kv, dim=dim, vdim=dim, scale=0.7 / math.sqrt(dim), cap=cap, size=size, keep=keep, base=2000.0, rot=dim // 2,
                scaling=(3.0, 96, 8.0, 1.0))
    part, W, p = _part("mixer", bm.layer("attention", m), BF16, width, seed=heads + dim)
    cache = SequenceCache([part.cache_request()], max_tokens=1024, max_seq_len=512, dtype=BF16, device=DEV, n_slots=2)
    ws = Workspace(DEV)
    g = torch.Generator().manual_seed(dim)
    x = (torch.randn(n, width, generator=g) * 0.5).to(BF16)
    want = plain_belizen.attention_mixer(x.double(), W, p, m, 1e-5)
    for portions in ([n], [300, 1], [1, 2, 60, 1, 64, 5, 130, 67]):
        assert rel_err(_drive(part, cache, x, portions, BF16, ws), want) < 3e-2, portions
