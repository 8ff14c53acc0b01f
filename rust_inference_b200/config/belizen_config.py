"""Typed configuration of the Belizen decoder, read from config.json.

config.json gives every size and every constant that can differ between models of the design:

    {"architecture": "Belizen", "vocab": V, "width": D, "norm": {"eps": e}, "embedding": {"scale": s},
     "residual_mult": m, "logit_softcap": c (optional), "loop": {"start", "stop", "times"} (optional),
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap" (optional),
                           "mask": {"size", "keep_first"} (optional),
                           "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"} (optional)} (optional)},
                 "mlp": null | {"kind": "dense", "ff"}
                            | {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "identity" (optional)},
                               "shared": {"ff", "limit"} (optional)}},
                {"type": "gla", "mixer": {"heads", "dim", "vdim", "tau", "rank" (optional)}, "mlp": ...},
                ...]}

Sizes and constants have no defaults: a missing key is an error that names it.  Optional are only the things a model or
a layer may lack.  The rank of a gla layer's decay map is the one size config.json may leave to the weights: without
`rank` it is the number of rows of the tensor `l<i>.mix.a1`, which the caller hands over as `shapes`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .lulisun_config import _float, _get, _int
from .model_config import ConfigError

ARCHITECTURE = "Belizen"


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int                     # rotated channels: the first ones of every head
    scaling: tuple | None         # (factor, original, fast, slow) of the interpolated frequencies, or None


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                # 0: scores are not capped
    window: int | None            # a query sees itself and the window - 1 positions before it (None: all)
    keep_first: int               # and the first so many positions of the sequence, whatever the window
    rot: RotaryConfig | None


@dataclass(frozen=True)
class LinearAttentionConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class ExpertsConfig:
    experts: int                  # experts with tensors
    identity: int                 # router outputs after theirs whose expert hands its input through
    top: int
    ff: int
    limit: float
    shared_ff: int | None
    shared_limit: float | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class BelizenLayerConfig:
    kind: str                     # "attention" | "gla"
    mixer: Any
    mlp: Any                      # DenseMlpConfig | ExpertsConfig | None


def _positive(x: float, what: str) -> float:
    if not x > 0:
        raise ConfigError(f"config.json: {what} must be positive, found {x}")
    return x


def _attention(m: Mapping, w: str) -> AttentionConfig:
    rot = None
    if m.get("rot") is not None:
        r, rw = m["rot"], w + ".rot"
        dims = _int(r, "dims", rw, minimum=2)
        if dims % 2:
            raise ConfigError(f"config.json: {rw}.dims {dims} must be even")
        scaling = None
        if r.get("scaling") is not None:
            sc, sw = r["scaling"], rw + ".scaling"
            scaling = tuple(_positive(_float(sc, k, sw), f"{sw}.{k}") for k in ("factor", "original", "fast", "slow"))
        base = _positive(_float(r, "base", rw), rw + ".base")
        if scaling is not None and not base > 1:
            raise ConfigError(f"config.json: {rw}.base must exceed 1 where frequencies are interpolated, found {base}")
        rot = RotaryConfig(base=base, dims=dims, scaling=scaling)
    mask = m.get("mask")
    window = None if mask is None else _int(mask, "size", w + ".mask")
    keep = 0 if mask is None or mask.get("keep_first") is None else _int(mask, "keep_first", w + ".mask", minimum=0)
    cap = 0.0 if m.get("softcap") is None else _positive(_float(m, "softcap", w), w + ".softcap")
    a = AttentionConfig(heads=_int(m, "heads", w), kv_heads=_int(m, "kv_heads", w), dim=_int(m, "dim", w),
                        vdim=_int(m, "vdim", w), scale=_float(m, "scale", w), softcap=cap, window=window, keep_first=keep,
                        rot=rot)
    if a.heads % a.kv_heads:
        raise ConfigError(f"config.json: {w}: {a.heads} heads are not a multiple of {a.kv_heads} kv heads")
    if rot is not None and rot.dims > a.dim:
        raise ConfigError(f"config.json: {w}.rot.dims {rot.dims} exceeds dim {a.dim}")
    return a


def _mlp(mlp: Mapping, w: str):
    kind = _get(mlp, "kind", w)
    if kind == "dense":
        return DenseMlpConfig(ff=_int(mlp, "ff", w))
    if kind != "moe":
        raise ConfigError(f"config.json: {w}.kind {kind!r} is not a feed-forward of this design (have: 'dense', 'moe')")
    expert, router = _get(mlp, "expert", w), _get(mlp, "router", w)
    shared = mlp.get("shared")
    e = ExpertsConfig(
        experts=_int(router, "experts", w + ".router"),
        identity=0 if router.get("identity") is None else _int(router, "identity", w + ".router", minimum=0),
        top=_int(router, "top", w + ".router"), ff=_int(expert, "ff", w + ".expert"),
        limit=_positive(_float(expert, "limit", w + ".expert"), w + ".expert.limit"),
        shared_ff=None if shared is None else _int(shared, "ff", w + ".shared"),
        shared_limit=None if shared is None else _positive(_float(shared, "limit", w + ".shared"), w + ".shared.limit"))
    if e.top > e.experts + e.identity:
        raise ConfigError(f"config.json: {w}.router: {e.top} of {e.experts + e.identity} experts cannot be chosen")
    return e


@dataclass(frozen=True)
class BelizenConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    logit_softcap: float          # 0: logits are not capped
    loop: LoopConfig | None
    layers: tuple
    raw: Any = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], shapes: Mapping[str, tuple] | None = None) -> "BelizenConfig":
        entries = _get(d, "layers", "the model")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            m, mw = _get(entry, "mixer", where), where + ".mixer"
            if kind == "attention":
                mixer = _attention(m, mw)
            elif kind == "gla":
                if m.get("rank") is not None:
                    rank = _int(m, "rank", mw)
                elif shapes is not None and f"l{i}.mix.a1" in shapes and len(shapes[f"l{i}.mix.a1"]) == 2:
                    rank = int(shapes[f"l{i}.mix.a1"][0])
                else:
                    raise ConfigError(f"config.json: {mw}.rank is missing, and so is the tensor l{i}.mix.a1 whose rows give it")
                mixer = LinearAttentionConfig(heads=_int(m, "heads", mw), dim=_int(m, "dim", mw), vdim=_int(m, "vdim", mw),
                                              tau=_positive(_float(m, "tau", mw), mw + ".tau"), rank=rank)
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design (have: 'attention', 'gla')")
            mlp = entry.get("mlp")
            layers.append(BelizenLayerConfig(kind, mixer, None if mlp is None else _mlp(mlp, where + ".mlp")))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = LoopConfig(start=_int(lp, "start", "loop", minimum=0), stop=_int(lp, "stop", "loop"),
                              times=_int(lp, "times", "loop"))
            if not loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: loop: layers {loop.start} .. {loop.stop - 1} are no run of the {len(layers)} layers")
        eps = _positive(_float(_get(d, "norm", "the model"), "eps", "norm"), "norm.eps")
        cap = 0.0 if d.get("logit_softcap") is None else _positive(_float(d, "logit_softcap", "the model"), "logit_softcap")
        return cls(architecture=ARCHITECTURE, vocab_size=_int(d, "vocab", "the model"),
                   hidden_size=_int(d, "width", "the model"), norm_eps=eps,
                   embedding_scale=_float(_get(d, "embedding", "the model"), "scale", "embedding"),
                   residual_mult=_float(d, "residual_mult", "the model"), logit_softcap=cap, loop=loop,
                   layers=tuple(layers), raw=dict(d))

    def to_dict(self) -> dict:
        """The config.json form (a gla layer's rank is written out)."""
        layers = []
        for L in self.layers:
            a = L.mixer
            if L.kind == "attention":
                mixer = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
                if a.softcap:
                    mixer["softcap"] = a.softcap
                if a.window is not None:
                    mixer["mask"] = {"size": a.window, "keep_first": a.keep_first}
                if a.rot is not None:
                    mixer["rot"] = {"base": a.rot.base, "dims": a.rot.dims}
                    if a.rot.scaling is not None:
                        mixer["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), a.rot.scaling))
            else:
                mixer = {"heads": a.heads, "dim": a.dim, "vdim": a.vdim, "tau": a.tau, "rank": a.rank}
            f = L.mlp
            if f is None:
                mlp = None
            elif isinstance(f, DenseMlpConfig):
                mlp = {"kind": "dense", "ff": f.ff}
            else:
                mlp = {"kind": "moe", "expert": {"ff": f.ff, "limit": f.limit},
                       "router": {"experts": f.experts, "identity": f.identity, "top": f.top}}
                if f.shared_ff is not None:
                    mlp["shared"] = {"ff": f.shared_ff, "limit": f.shared_limit}
            layers.append({"type": L.kind, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
               "residual_mult": self.residual_mult, "layers": layers}
        if self.logit_softcap:
            out["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out
