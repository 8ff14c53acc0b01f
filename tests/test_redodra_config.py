"""Redodra without a GPU: the configuration reader and its errors, the tensors the model declares against the plain
list, the schedule and cache requests (layers that read another layer's keys, mixers that keep a matrix state and a
convolution's last inputs), and the plain restatement's mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import plain_redodra
import redodra_models
from rust_inference_b200.config.model_config import ConfigError
from rust_inference_b200.config.registry import config_from_dict, get_architecture, registered_architectures
from rust_inference_b200.engine.model import DecoderModel, declared_tensors


def _spec(cfg):
    arch = get_architecture("Redodra")
    return arch.build_spec(arch.parse_config(cfg))


def test_registered_and_round_trip():
    assert "Redodra" in registered_architectures()
    for cfg in redodra_models.CONFIGS.values():
        parsed = config_from_dict(cfg)
        assert parsed.to_dict() == cfg


@pytest.mark.parametrize("name", list(redodra_models.CONFIGS))
def test_declared_tensors_equal_the_plain_list(name):
    cfg = redodra_models.CONFIGS[name]
    got = {k: tuple(v.shape) for k, v in declared_tensors(_spec(cfg)).items()}
    assert got == plain_redodra.tensor_shapes(cfg)


def test_schedule_and_cache_requests():
    from rust_inference_b200.cache.sequence_cache import KVRequest, StateRequest
    spec = _spec(redodra_models.CONFIGS["A"])
    assert [(e.layer, e.cache) for e in spec.schedule] == [(0, 0), (1, 1), (2, 2), (3, 1), (4, 4), (5, 1)]
    model = DecoderModel(spec, dtype=torch.float32, device="cpu")
    assert [w for _, _, w in model.schedule] == [True, True, True, False, True, False]
    reqs = model.cache_requests()
    assert len(reqs) == 5 and reqs[3] is None
    assert reqs[1] == KVRequest(1, 32, None, 16)
    # a parallel layer: keys and values of the window attention, then the state space's matrix and carried inputs
    assert reqs[0] == (KVRequest(2, 16, 20, 24), (StateRequest((3, 8, 16)), StateRequest((3, 3 * 16 + 2 * 8))))
    assert reqs[2] == (StateRequest((4, 16, 24)), StateRequest((2, 2 * 2 * 16 + 4 * 24)))
    # a convolution of one tap carries nothing
    specB = _spec(redodra_models.CONFIGS["B"])
    assert DecoderModel(specB, dtype=torch.float32, device="cpu").cache_requests()[0][1] == StateRequest((0, 2 * 40 + 72))


def test_nested_requests_get_storage_of_their_own():
    """The cache answers a nested request with nested layers; equal requests share a group, slots start zeroed."""
    from rust_inference_b200.cache.sequence_cache import CompositeLayer, KVLayer, SequenceCache, StateLayer
    model = DecoderModel(_spec(redodra_models.CONFIGS["A"]), dtype=torch.float32, device="cpu")
    cache = SequenceCache(model.cache_requests(), max_tokens=256, max_seq_len=128, dtype=torch.float32, device="cpu", n_slots=3)
    top = cache.layer(0)
    assert isinstance(top, CompositeLayer) and isinstance(top.parts[0], KVLayer) and isinstance(top.parts[1], CompositeLayer)
    matrix, carried = top.parts[1].parts
    assert isinstance(matrix, StateLayer) and tuple(matrix.state.shape) == (3, 3, 8, 16)
    assert tuple(carried.state.shape) == (3, 3, 64)
    assert cache.layer(3) is None
    matrix.state.fill_(7.0)
    carried.state.fill_(7.0)
    slot = cache.alloc_slot()
    assert float(matrix.state[slot].abs().max()) == 0.0 and float(carried.state[slot].abs().max()) == 0.0


def _broken(path, value=None, drop=False):
    cfg = copy.deepcopy(redodra_models.CONFIGS["A"])
    at = cfg
    for k in path[:-1]:
        at = at[k]
    if drop:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return cfg


@pytest.mark.parametrize("path,value,drop,word", [
    (("width",), None, True, "width"),
    (("norm", "eps"), 0.0, False, "eps"),
    (("layers", 0, "type"), "conv", False, "conv"),
    (("layers", 1, "mixer", "kv_heads"), 3, False, "multiple"),
    (("layers", 1, "mixer", "rot", "dims"), 7, False, "even"),
    (("layers", 1, "mixer", "rot", "dims"), 34, False, "exceeds"),
    (("layers", 1, "mixer", "scale"), None, True, "scale"),
    (("layers", 1, "mixer", "softcap"), -2.0, False, "softcap"),
    (("layers", 3, "mixer", "kv_from"), 3, False, "earlier"),
    (("layers", 3, "mixer", "kv_from"), 2, False, "keys and values of its own"),
    (("layers", 3, "mixer", "dim"), 16, False, "equal"),
    (("layers", 5, "mixer", "kv_from"), 3, False, "keys and values of its own"),
    (("layers", 2, "mixer", "conv"), 0, False, "conv"),
    (("layers", 2, "mixer", "kv_heads"), 3, False, "multiple"),
    (("layers", 0, "mixer", "right"), None, True, "right"),
    (("layers", 0, "mixer", "right", "groups"), 2, False, "groups"),
    (("layers", 0, "mixer", "right", "norm_groups"), 5, False, "equal parts"),
    (("layers", 0, "mixer", "left", "mask", "size"), 0, False, "size"),
    (("layers", 0, "mlp", "kind"), "moe", False, "moe"),
])
def test_configuration_errors_name_the_key(path, value, drop, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_broken(path, value, drop))
    assert word in str(e.value)


def test_plain_mechanisms_against_closed_forms():
    f64 = torch.float64
    # the activation is continuous at 0 with slope 1/2, quadratic to the right, and tends to a line to the left
    p, q = torch.tensor(0.3, dtype=f64), torch.tensor(-0.2, dtype=f64)
    ap, an = math.log1p(math.exp(0.3)), 0.5 + math.log1p(math.exp(-0.2))
    z = torch.tensor([-30.0, -1e-9, 0.0, 1e-9, 2.0], dtype=f64)
    y = plain_redodra.xielu(z, p, q)
    assert math.isclose(float(y[4]), ap * 4.0 + 1.0, rel_tol=1e-12)
    assert math.isclose(float(y[0]), an * (-1.0 + 30.0) - 15.0, rel_tol=1e-9)
    assert abs(float(y[1]) + 0.5e-9) < 1e-15 and float(y[2]) == 0.0 and abs(float(y[3]) - 0.5e-9) < 1e-15
    # a short convolution whose only non-zero tap is the last one is the identity; the one before it a shift
    x = torch.randn(6, 3, dtype=f64)
    taps = torch.zeros(3, 4, dtype=f64)
    taps[:, 3] = 1.0
    assert torch.equal(plain_redodra.short_conv(x, taps), x)
    taps = torch.zeros(3, 4, dtype=f64)
    taps[:, 2] = 2.0
    assert torch.equal(plain_redodra.short_conv(x, taps)[1:], 2.0 * x[:-1]) and float(plain_redodra.short_conv(x, taps)[0].abs().max()) == 0.0
    # adjacent pairs: identity at position 0, lengths kept, channels beyond `dims` untouched
    h = torch.randn(4, 2, 10, dtype=f64)
    r = plain_redodra.rotate_adjacent(h, 100.0, 6)
    assert torch.equal(r[0], h[0]) and torch.equal(r[..., 6:], h[..., 6:])
    assert torch.allclose(r[..., 0:6:2] ** 2 + r[..., 1:6:2] ** 2, h[..., 0:6:2] ** 2 + h[..., 1:6:2] ** 2)
    assert math.isclose(float(r[3, 0, 2]), float(h[3, 0, 2] * math.cos(3 * 100.0 ** (-2 / 6)) - h[3, 0, 3] * math.sin(3 * 100.0 ** (-2 / 6))), rel_tol=1e-12)


def test_plain_delta_rule_writes_what_it_is_told():
    """With beta = 1 and no decay, reading with the key just written returns the value just written (times the
    query's factor): the rule replaces what the state held along that key."""
    D, d, dv = 8, 4, 3
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": dv, "conv": 1}
    g = torch.Generator().manual_seed(1)
    W = {k: torch.randn(*s, generator=g, dtype=torch.float64) if s else torch.tensor(1.0, dtype=torch.float64)
         for k, s in {"q": (d, D), "k": (d, D), "v": (dv, D), "b": (1, D), "a": (1, D), "g": (dv, D), "o": (D, dv)}.items()}
    W["k"] = W["q"].clone()                                           # the query is the key
    W.update({"q.conv": torch.ones(d, 1, dtype=torch.float64), "k.conv": torch.ones(d, 1, dtype=torch.float64),
              "v.conv": torch.ones(dv, 1, dtype=torch.float64), "dt_bias": torch.tensor([-200.0], dtype=torch.float64),
              "A_log": torch.tensor([0.0], dtype=torch.float64), "norm": torch.ones(dv, dtype=torch.float64)})
    W["b"] = torch.zeros(1, D, dtype=torch.float64)
    h = torch.randn(5, D, generator=g, dtype=torch.float64)
    # beta = sigmoid(0) = 1/2: the read-out is v / 2 along the unit key after the first token
    W["a"] = torch.zeros(1, D, dtype=torch.float64)
    out = plain_redodra.delta_rule(h[:1], {("x." + k): v for k, v in W.items()}, "x.", m, 0.0)
    v = plain_redodra.silu(h[:1] @ W["v"].T)
    k = plain_redodra.silu(h[:1] @ W["k"].T)
    kk = float((k * k).sum() / ((k * k).sum() + 1e-6))
    o = 0.5 * v * kk * d ** -0.5
    want = (o / torch.sqrt((o * o).mean(-1, keepdim=True)) * plain_redodra.silu(h[:1] @ W["g"].T)) @ W["o"].T
    assert torch.allclose(out, want, rtol=1e-9, atol=1e-12)


def test_plain_state_space_with_constant_inputs_is_a_geometric_sum():
    """One head, one state row, a one-tap convolution: y_t = C B dt x sum_s a^s + D x for constant inputs."""
    m = {"heads": 1, "vdim": 1, "state": 1, "groups": 1, "conv": 1, "norm_groups": 1}
    f64 = torch.float64
    W = {"x.in": torch.tensor([[0.0], [1.0], [1.0], [1.0], [0.0]], dtype=f64), "x.conv": torch.ones(3, 1, dtype=f64),
         "x.conv.b": torch.zeros(3, dtype=f64), "x.dt_bias": torch.tensor([0.3], dtype=f64), "x.A_log": torch.tensor([-0.5], dtype=f64),
         "x.D": torch.tensor([0.7], dtype=f64), "x.norm": torch.ones(1, dtype=f64), "x.o": torch.ones(1, 1, dtype=f64)}
    h = torch.full((6, 1), 0.9, dtype=f64)
    # z = 0: the gate silu(0) closes everything; move the gate off zero through the first row of the projection
    W["x.in"][0, 0] = 2.0
    out = plain_redodra.state_space(h, W, "x.", m, 0.0)
    s = float(plain_redodra.silu(torch.tensor(0.9, dtype=f64)))
    dt = math.log1p(math.exp(0.3))
    a = math.exp(-math.exp(-0.5) * dt)
    for t in range(6):
        y = s * s * dt * s * sum(a ** k for k in range(t + 1)) + 0.7 * s
        gated = y * float(plain_redodra.silu(torch.tensor(1.8, dtype=f64)))
        assert math.isclose(float(out[t]), gated / math.sqrt(gated * gated), rel_tol=1e-9)        # a norm over one channel: the sign
        assert y > 0
