"""Typed configuration of the Redodra decoder, read from config.json.

config.json gives every size and every constant that can differ between models of the design:

    {"architecture": "Redodra", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot": {"base", "dims"},
                           "kv_from": j (optional: the layer reads layer j's cached keys and values)},
                 "mlp": null | {"kind": "dense", "ff"}},
                {"type": "delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ...},
                {"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "mask": {"size", "keep_first"}},
                           "right": {"heads", "vdim", "state", "groups", "conv", "norm_groups"}},
                 "mlp": ...},
                ...]}

Sizes and constants have no defaults: a missing key is an error that names it.  Optional are only the things a layer
may lack: `softcap` (scores are not capped), `mask` (every earlier position is visible) and its `keep_first` (none
kept), `rot` (nothing is rotated), `kv_from`, `mlp`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .lulisun_config import _float, _get, _int
from .model_config import ConfigError

ARCHITECTURE = "Redodra"


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int                # rotated channels: the first ones of every head, adjacent pairs


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int                 # size of a query / key head
    vdim: int                # size of a value head
    scale: float
    softcap: float           # 0: scores are not capped
    rot: RotaryConfig | None = None
    window: int | None = None        # a query sees itself and the window - 1 positions before it (None: all)
    keep_first: int = 0              # the first so many positions stay visible beyond the window
    kv_from: int | None = None       # the layer whose cached keys and values this one reads (None: its own)


@dataclass(frozen=True)
class DeltaRuleConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                # taps of the short convolutions


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class ParallelConfig:
    left: AttentionConfig
    right: StateSpaceConfig


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int


@dataclass(frozen=True)
class RedodraLayerConfig:
    kind: str                # "attention" | "delta" | "parallel"
    mixer: Any
    mlp: DenseMlpConfig | None
    raw: Any = None


def _attention(m: Mapping, w: str, *, rotary: bool, layer: int, layers: list) -> AttentionConfig:
    rot = None
    if rotary and m.get("rot") is not None:
        r = m["rot"]
        rot = RotaryConfig(base=_float(r, "base", w + ".rot"), dims=_int(r, "dims", w + ".rot", minimum=2))
        if rot.dims % 2:
            raise ConfigError(f"config.json: {w}.rot.dims {rot.dims} must be even")
        if rot.base <= 0:
            raise ConfigError(f"config.json: {w}.rot.base must be positive")
    mask = m.get("mask")
    window, keep = None, 0
    if mask is not None:
        window = _int(mask, "size", w + ".mask")
        keep = _int(mask, "keep_first", w + ".mask", minimum=0) if mask.get("keep_first") is not None else 0
    cap = _float(m, "softcap", w) if m.get("softcap") is not None else 0.0
    a = AttentionConfig(heads=_int(m, "heads", w), kv_heads=_int(m, "kv_heads", w), dim=_int(m, "dim", w),
                        vdim=_int(m, "vdim", w), scale=_float(m, "scale", w), softcap=cap, rot=rot, window=window,
                        keep_first=keep, kv_from=m.get("kv_from"))
    if a.heads % a.kv_heads:
        raise ConfigError(f"config.json: {w}: {a.heads} heads are not a multiple of {a.kv_heads} kv heads")
    if cap < 0:
        raise ConfigError(f"config.json: {w}.softcap must not be negative, found {cap}")
    if rot is not None and rot.dims > a.dim:
        raise ConfigError(f"config.json: {w}.rot.dims {rot.dims} exceeds dim {a.dim}")
    src = a.kv_from
    if src is not None:
        if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < layer:
            raise ConfigError(f"config.json: {w}.kv_from {src!r} must name an earlier layer")
        owner = layers[src]
        o = owner.mixer
        if owner.kind != "attention" or o.kv_from is not None:
            raise ConfigError(f"config.json: {w}.kv_from {src}: that layer keeps no keys and values of its own")
        if (o.kv_heads, o.dim, o.vdim, o.rot) != (a.kv_heads, a.dim, a.vdim, a.rot):
            raise ConfigError(f"config.json: {w}.kv_from {src}: kv_heads, dim, vdim and rot must equal that layer's")
    return a


@dataclass(frozen=True)
class RedodraConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple
    raw: Any = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RedodraConfig":
        entries = _get(d, "layers", "the model")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers: list = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            m = _get(entry, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                mixer = _attention(m, mw, rotary=True, layer=i, layers=layers)
            elif kind == "delta":
                mixer = DeltaRuleConfig(heads=_int(m, "heads", mw), kv_heads=_int(m, "kv_heads", mw), dim=_int(m, "dim", mw),
                                        vdim=_int(m, "vdim", mw), conv=_int(m, "conv", mw))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: {mw}: {mixer.heads} heads are not a multiple of {mixer.kv_heads} kv heads")
            elif kind == "parallel":
                left = _attention(_get(m, "left", mw), mw + ".left", rotary=False, layer=i, layers=layers)
                if left.kv_from is not None:
                    raise ConfigError(f"config.json: {mw}.left.kv_from: a member of a parallel mixer keeps its own keys")
                r, rw = _get(m, "right", mw), mw + ".right"
                right = StateSpaceConfig(heads=_int(r, "heads", rw), vdim=_int(r, "vdim", rw), state=_int(r, "state", rw),
                                         groups=_int(r, "groups", rw), conv=_int(r, "conv", rw),
                                         norm_groups=_int(r, "norm_groups", rw))
                if right.heads % right.groups:
                    raise ConfigError(f"config.json: {rw}: {right.heads} heads are not a multiple of {right.groups} groups")
                if (right.heads * right.vdim) % right.norm_groups:
                    raise ConfigError(f"config.json: {rw}: {right.heads * right.vdim} channels do not split into "
                                      f"{right.norm_groups} equal parts")
                mixer = ParallelConfig(left, right)
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  "(have: 'attention', 'delta', 'parallel')")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                fw = where + ".mlp"
                if _get(mlp, "kind", fw) != "dense":
                    raise ConfigError(f"config.json: {fw}.kind {mlp['kind']!r} is not a feed-forward of this design (have: 'dense')")
                ff = DenseMlpConfig(ff=_int(mlp, "ff", fw))
            layers.append(RedodraLayerConfig(kind, mixer, ff, raw=entry))
        eps = _float(_get(d, "norm", "the model"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cls(architecture=ARCHITECTURE, vocab_size=_int(d, "vocab", "the model"),
                   hidden_size=_int(d, "width", "the model"), norm_eps=eps, layers=tuple(layers), raw=dict(d))

    def to_dict(self) -> dict:
        """The config.json form."""
        def attention(a: AttentionConfig) -> dict:
            out = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale}
            if a.softcap:
                out["softcap"] = a.softcap
            if a.rot is not None:
                out["rot"] = {"base": a.rot.base, "dims": a.rot.dims}
            if a.window is not None:
                out["mask"] = {"size": a.window, "keep_first": a.keep_first}
            if a.kv_from is not None:
                out["kv_from"] = a.kv_from
            return out

        layers = []
        for L in self.layers:
            m = L.mixer
            if L.kind == "attention":
                mixer = attention(m)
            elif L.kind == "delta":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            else:
                r = m.right
                mixer = {"left": attention(m.left),
                         "right": {"heads": r.heads, "vdim": r.vdim, "state": r.state, "groups": r.groups, "conv": r.conv,
                                   "norm_groups": r.norm_groups}}
            layers.append({"type": L.kind, "mixer": mixer, "mlp": None if L.mlp is None else {"kind": "dense", "ff": L.mlp.ff}})
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps}, "layers": layers}
