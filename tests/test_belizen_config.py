"""Belizen without a GPU: the configuration reader and its errors, the tensors the model declares against the plain
list, the schedule of a run of layers that is passed several times and its cache requests, the rank that a tensor's
shape gives, and the plain restatement's mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import belizen_models as bm
import plain_belizen
from rust_inference_b200.config.model_config import ConfigError
from rust_inference_b200.config.registry import config_from_dict, get_architecture, load_spec, registered_architectures
from rust_inference_b200.engine.model import DecoderModel, declared_tensors


def _spec(cfg, shapes=None):
    arch = get_architecture("Belizen")
    return arch.build_spec(arch.parse_config(cfg, shapes=shapes))


def test_registered_and_round_trip():
    assert "Belizen" in registered_architectures()
    for cfg in bm.CONFIGS.values():
        parsed = config_from_dict(cfg)
        again = config_from_dict(parsed.to_dict())
        assert again.to_dict() == parsed.to_dict()
        assert again.layers == parsed.layers and again.loop == parsed.loop


@pytest.mark.parametrize("name", list(bm.CONFIGS))
def test_declared_tensors_equal_the_plain_list(name):
    cfg = bm.CONFIGS[name]
    got = {k: tuple(v.shape) for k, v in declared_tensors(_spec(cfg)).items()}
    assert got == plain_belizen.tensor_shapes(cfg)


def test_schedule_of_passes_and_cache_requests():
    from rust_inference_b200.cache.sequence_cache import KVRequest, StateRequest
    spec = _spec(bm.CONFIGS["A"])                  # layers 1 and 2 three times
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (1, 3), (2, 4), (1, 5), (2, 6), (3, 7)]
    assert [e.before for e in spec.schedule] == [None, (0, 0), None, (0, 1), None, (0, 2), None, None]
    assert [(layer, entering) for layer, entering in plain_belizen.run_order(bm.CONFIGS["A"])] == \
        [(e.layer, None if e.before is None else e.before[1]) for e in spec.schedule]
    model = DecoderModel(spec, dtype=torch.float32, device="cpu")
    assert all(w for _, _, w in model.schedule)    # every pass has caches of its own
    reqs = model.cache_requests()
    assert reqs[0] == KVRequest(2, 16, 20, 24)
    assert reqs[1] == reqs[3] == reqs[5] == StateRequest((3, 24, 40), torch.float32)
    assert reqs[2] == reqs[4] == reqs[6] == KVRequest(2, 8, 150, None)
    assert "loop.step" in model.declared_tensors() and tuple(model.declared_tensors()["loop.step"].shape) == (3, 96)
    # the whole model as the loop; no loop at all
    specB = _spec(bm.CONFIGS["B"])
    assert [(e.layer, e.cache, e.before) for e in specB.schedule] == [(0, 0, (0, 0)), (1, 1, None), (2, 2, None),
                                                                      (0, 3, (0, 1)), (1, 4, None), (2, 5, None)]
    specC = _spec(bm.CONFIGS["C"])
    assert [(e.layer, e.cache, e.before) for e in specC.schedule] == [(i, i, None) for i in range(4)]
    assert "loop.step" not in declared_tensors(specC)


def test_rank_from_shapes():
    cfg = copy.deepcopy(bm.CONFIGS["A"])
    del cfg["layers"][1]["mixer"]["rank"], cfg["layers"][3]["mixer"]["rank"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.rank"):
        config_from_dict(cfg)
    spec = _spec(cfg, shapes={"l1.mix.a1": (5, 96), "l3.mix.a1": (1, 96)})
    assert {k: tuple(v.shape) for k, v in declared_tensors(spec).items()} == plain_belizen.tensor_shapes(bm.CONFIGS["A"])


def test_load_spec_reads_the_rank_from_the_folder(tmp_path):
    torch.manual_seed(0)
    try:
        model = bm.make(tmp_path, "A", drop_rank=True)
    except (OSError, RuntimeError) as e:          # the weight file's writer is native code that may not be built here
        pytest.skip(str(e))
    _, spec = load_spec(model.folder)
    assert {k: tuple(v.shape) for k, v in declared_tensors(spec).items()} == plain_belizen.tensor_shapes(bm.CONFIGS["A"])


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.pop("residual_mult"), "residual_mult"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), r"layers\[0\]\.mixer lacks 'scale'"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=64), "exceeds dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "not a feed-forward"),
    (lambda c: c["layers"][1]["mixer"].update(tau=0.0), "tau"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "cannot be chosen"),
    (lambda c: c["layers"][1]["mlp"]["expert"].update(limit=-1.0), "limit"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["loop"].update(times=0), "times"),
    (lambda c: c.update(logit_softcap=-3.0), "logit_softcap"),
])
def test_configuration_errors_name_the_key(edit, message):
    cfg = copy.deepcopy(bm.CONFIGS["A"])
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(cfg)


def test_optional_things_may_be_absent():
    cfg = copy.deepcopy(bm.CONFIGS["A"])
    m = cfg["layers"][0]["mixer"]
    del m["mask"], m["rot"], m["softcap"], cfg["loop"], cfg["logit_softcap"]
    cfg["layers"][1]["mlp"]["router"].pop("identity")
    cfg["layers"][1]["mlp"].pop("shared")
    parsed = config_from_dict(cfg)
    a = parsed.layers[0].mixer
    assert a.window is None and a.keep_first == 0 and a.rot is None and a.softcap == 0.0
    assert parsed.loop is None and parsed.logit_softcap == 0.0
    assert parsed.layers[1].mlp.identity == 0 and parsed.layers[1].mlp.shared_ff is None
    spec = _spec(cfg)
    assert spec.stream_parts == () and spec.layers[0].parts["mixer"].params["position"].kind == "unrotated"


# ---- the plain mechanisms against closed forms -------------------------------------------------------------------
def test_plain_window_mask():
    vis = plain_belizen.window_visible(10, 3, 2)
    assert vis[9].tolist() == [True, True, False, False, False, False, False, True, True, True]
    assert vis[2].tolist() == [True, True, True] + [False] * 7
    assert plain_belizen.window_visible(4, None, 0).tolist() == torch.tril(torch.ones(4, 4)).bool().tolist()


def test_plain_frequencies():
    f, mag = plain_belizen.interpolated_frequencies(8, 100.0, None)
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75], dtype=torch.float64)) and mag == 1.0
    # every channel beyond the slow limit is divided by the factor, every one before the fast limit is left alone
    sc = {"factor": 8.0, "original": 2048, "fast": 16.0, "slow": 2.0}
    f0, _ = plain_belizen.interpolated_frequencies(64, 50000.0, None)
    f1, mag = plain_belizen.interpolated_frequencies(64, 50000.0, sc)
    assert math.isclose(mag, 0.1 * math.log(8.0) + 1.0)
    turns = 2048 * f0 / (2 * math.pi)
    assert torch.allclose(f1[turns > 24], f0[turns > 24]) and torch.allclose(f1[turns < 1.4], f0[turns < 1.4] / 8.0)
    mid = (turns < 12) & (turns > 2.8)
    assert mid.any() and bool(((f1[mid] < f0[mid]) & (f1[mid] > f0[mid] / 8.0)).all())


def test_plain_linear_attention_closed_form():
    """With constant decay a and one key channel the state is a geometric sum."""
    D = 4
    a = {"heads": 1, "dim": 1, "vdim": 2, "tau": 2.0, "rank": 1}
    w = {"q": torch.ones(1, D), "k": torch.ones(1, D), "v": torch.tensor([[1.0, 0, 0, 0], [0, 1.0, 0, 0]]), "g": torch.zeros(2, D),
         "o": torch.eye(D)[:, :2], "norm": torch.ones(2), "a1": torch.zeros(1, D), "a2": torch.zeros(1, 1), "a2.b": torch.zeros(1)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.tensor([[1.0, 2.0, 0, 0], [3.0, -1.0, 0, 0], [0.5, 0.5, 0, 0]], dtype=torch.float64)
    _, S = plain_belizen.linear_attention_mixer(h, w, "", a, 1e-6, return_state=True)
    alpha = 0.5 ** 0.5                       # sigmoid(0)^(1/2)
    ks = h.sum(dim=1)
    want = sum(alpha ** (2 - t) * ks[t] * h[t, :2] for t in range(3))
    assert torch.allclose(S[0, 0], want)
    # silu(0) = 0 closes the gate
    assert float(plain_belizen.linear_attention_mixer(h, w, "", a, 1e-6).abs().max()) == 0.0


def test_plain_router_and_pass_through():
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=torch.float64)
    router = torch.tensor([[1.0, 0.0], [0.0, 1.0], [0.0, 0.0]], dtype=torch.float64)
    ids, wts = plain_belizen.route(h, router, torch.tensor([0.0, 0.0, 10.0], dtype=torch.float64), 2)
    s = torch.softmax(h @ router.T, dim=-1)
    assert ids.tolist() == [[2, 0], [2, 1]]                      # the correction decides, the weights ignore it
    assert torch.allclose(wts, torch.stack([s[0, [2, 0]], s[1, [2, 1]]]))
    mlp = {"router": {"experts": 0, "identity": 3, "top": 1}, "expert": {"ff": 1, "limit": 1.0}}
    out = plain_belizen.experts_ff(h, {"router": router, "correction": torch.tensor([0.0, 0.0, 10.0])}, "", mlp)
    assert torch.allclose(out, h * s[:, 2:3])
