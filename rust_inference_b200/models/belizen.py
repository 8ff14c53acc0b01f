"""The Belizen decoder as a `ModelSpec`.

Every layer is pre-norm with a factor m on both branches (`pre_norm_optional_ff`; the parts' `out_scale`):
x <- x + m mixer(n1(x)), then x <- x + m ff(n2(x)), RMS norms with plain weights.  The mixer is one of

* `attention`: grouped-query attention with projection biases, queries and keys RMS-normed per head and rotated in the
  halves layout on their first channels with interpolated frequencies, capped scores, a sliding window that keeps the
  sequence's first positions visible, and the concatenated heads times sigmoid(W_g h) element by element
  (`gqa_attention` with `qk_norm_eps`, `softcap`, `window`, `keep_first`, `out_gate`; `rope` with `interpolation`);
* `gla`: gated linear attention with a decay per key channel from a low-rank map (`gated_linear_attention`).

The feed-forward is a gated dense layer with the tanh form of GELU (`gated_dense`), a mixture of bounded gated experts
chosen by a softmax router with a correction on the choice, experts that hand their input through and an always-on
shared expert (`routed_experts`), or absent.  A run of layers may be passed several times with the same weights, every
pass with caches of its own: that is the schedule, and what joins the stream where a pass begins is the stream part
`pass_entry`.  The embedding is scaled and tied to the head, whose logits are capped.

Tensor names: `embed`, `final.norm`, `loop.step`, `l<i>.norm{1,2}`, `l<i>.mix.{q,k,v,g,o}`, `l<i>.mix.{q,k,v}.b`,
`l<i>.mix.{q,k}.norm`, `l<i>.mix.{norm,a1,a2,a2.b}`, `l<i>.mlp.{gate,up,down}`, `l<i>.mlp.{router,correction}`,
`l<i>.mlp.e<j>.{gate,up,down}`, `l<i>.mlp.shared.{gate,up,down}`.
"""
from __future__ import annotations

from ..config.belizen_config import ARCHITECTURE, BelizenConfig, DenseMlpConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# the configuration gives no context length: positions are bounded by the cache a run is given
MAX_POSITIONS = 1 << 17

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                    "q_norm": "q.norm", "k_norm": "k.norm", "out_gate": "g"}
_GLA_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm", "decay_in": "a1", "decay_out": "a2",
              "decay_bias": "a2.b"}
_DENSE_NAMES = {"gate": "gate", "up": "up", "down": "down"}
_EXPERT_NAMES = {"router": "router", "correction": "correction", "gate": "e{e}.gate", "up": "e{e}.up", "down": "e{e}.down",
                 "shared_gate": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down"}


def _norm(prefix: str, eps: float) -> PartSpec:
    return PartSpec("rmsnorm", {"eps": eps, "weight_name": ""}, prefix=prefix)


def run_order(n_layers: int, loop) -> list:
    """[(layer, run, pass that begins here or None)]: layers start .. stop - 1 are passed `times` times in a row."""
    if loop is None:
        return [(i, i, None) for i in range(n_layers)]
    order = [(i, None) for i in range(loop.start)]
    for t in range(loop.times):
        order += [(i, t if i == loop.start else None) for i in range(loop.start, loop.stop)]
    order += [(i, None) for i in range(loop.stop, n_layers)]
    return [(layer, run, entering) for run, (layer, entering) in enumerate(order)]


def build_spec(cfg: BelizenConfig) -> ModelSpec:
    m, eps = cfg.residual_mult, cfg.norm_eps
    layers = []
    for i, L in enumerate(cfg.layers):
        a = L.mixer
        if L.kind == "attention":
            if a.rot is not None:
                interpolation = None
                if a.rot.scaling is not None:
                    interpolation = dict(zip(("factor", "original", "fast", "slow"), a.rot.scaling))
                position = PartSpec("rope", {"head_dim": a.dim, "base": a.rot.base, "style": "half", "rot_dims": a.rot.dims,
                                             "exact_angles": True, "interpolation": interpolation})
            else:
                position = PartSpec("unrotated", {})
            mixer = PartSpec("gqa_attention", {
                "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim, "qkv_bias": True,
                "position": position, "scale": a.scale, "softcap": a.softcap, "window": a.window,
                "keep_first": a.keep_first if a.window is not None else 0, "qk_norm_eps": eps, "out_gate": True,
                "out_scale": m, "names": _ATTENTION_NAMES}, prefix="mix.")
        else:
            mixer = PartSpec("gated_linear_attention", {
                "n_heads": a.heads, "head_dim": a.dim, "v_head_dim": a.vdim, "rank": a.rank, "tau": a.tau, "eps": eps,
                "out_scale": m, "names": _GLA_NAMES}, prefix="mix.")
        parts = {"mixer": mixer, "mixer_norm": _norm("norm1", eps)}
        f = L.mlp
        if f is not None:
            if isinstance(f, DenseMlpConfig):
                ff = PartSpec("gated_dense", {"intermediate_size": f.ff, "activation": "gelu_tanh", "out_scale": m,
                                              "names": _DENSE_NAMES}, prefix="mlp.")
            else:
                ff = PartSpec("routed_experts", {
                    "n_experts": f.experts, "identity": f.identity, "top": f.top, "expert_size": f.ff,
                    "router_kind": "softmax", "normalise": False, "expert_form": {"limit": f.limit},
                    "shared_size": f.shared_ff, "shared_form": None if f.shared_ff is None else {"limit": f.shared_limit},
                    "shared_gate": False, "out_scale": m, "names": _EXPERT_NAMES}, prefix="mlp.")
            parts["feed_forward"], parts["feed_forward_norm"] = ff, _norm("norm2", eps)
        layers.append(LayerSpec(prefix=f"l{i}.", arrangement="pre_norm_optional_ff", parts=parts))
    stream_parts = ()
    if cfg.loop is not None:
        stream_parts = (PartSpec("pass_entry", {"passes": cfg.loop.times, "readd_input": True, "weight_name": "step"},
                                 prefix="loop."),)
    schedule = tuple(ScheduleEntry(layer=layer, cache=run, before=None if entering is None else (0, entering))
                     for layer, run, entering in run_order(len(cfg.layers), cfg.loop))
    embedding = PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "weight_name": "", "scale": cfg.embedding_scale},
                         prefix="embed")
    head = PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "norm": _norm("final.norm", eps), "tied": True,
                                    "weight_prefix": None, "softcap": cfg.logit_softcap})
    return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=MAX_POSITIONS,
                     layers=tuple(layers), schedule=schedule, embedding=embedding, head=head, stream_parts=stream_parts)


register_architecture(ARCHITECTURE, BelizenConfig.from_dict, build_spec, replace=True, reads_shapes=True)
