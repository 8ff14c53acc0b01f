"""The Redodra decoder as a `ModelSpec`.

Every layer normalises each sublayer going in and coming out (`pre_post_norm`):
x <- x + n1b(mixer(n1(x))), then x <- x + n2b(ff(n2(x))), all four norms of the form tanh(alpha x) w + b
(`dynamic_tanh`).  What a layer hands on is a learned weighted sum of the embedding's output and of all layers'
results so far (`weighted_depth_sum`).  The mixer is one of

* `attention`: grouped-query causal attention with adjacent-pair rotary positions on the first channels of a head,
  capped scores, a learned sink in the softmax's denominator and a sigmoid gate per head on the result
  (`gqa_attention` with `softcap`, `sink`, `head_gate`); a layer may attend over the keys and values another layer
  cached, with its own queries: that is the schedule;
* `delta`: the gated delta rule behind short convolutions (`gated_delta_rule`);
* `parallel`: attention without rotation over a sliding window that keeps the sequence's first positions visible, with
  projection biases and a logarithmic distance bias on the scores (`gqa_attention` with `unrotated` positions, `window`,
  `keep_first`, `distance_bias`), beside a selective state space (`selective_state_space`); each result is RMS-normed
  over the width and the two are averaged (`parallel_mixers` with `member_norm`).

The feed-forward is W_down act(W_up x) with the learned activation xIELU (`dense_act`) or absent.  The head has the
model's norm and a matrix of its own.

Tensor names: `embed`, `head`, `final.norm{,.b,.alpha}`, `l<i>.norm{1,1b,2,2b}{,.b,.alpha}`, `l<i>.dwa`,
`l<i>.mlp.{up,down,act}`, `l<i>.mix.{q,k,v,sink,g,o}`, `l<i>.mix.{q,k,v}{,.conv}`, `l<i>.mix.{b,a,dt_bias,A_log,g,norm,o}`,
`l<i>.mix.left.{q,k,v,o}{,.b}`, `l<i>.mix.left.{r1,r2,out}`, `l<i>.mix.right.{in,conv,conv.b,dt_bias,A_log,D,norm,o,out}`.
"""
from __future__ import annotations

from ..config.redodra_config import ARCHITECTURE, RedodraConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# the configuration gives no context length: positions are bounded by the cache a run is given
MAX_POSITIONS = 1 << 17

_GATED_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink", "gate": "g"}
_WINDOW_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b",
                 "r1": "r1", "r2": "r2"}
_DELTA_NAMES = {"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv", "beta": "b",
                "a": "a", "dt_bias": "dt_bias", "A_log": "A_log", "gate": "g", "norm": "norm", "o": "o"}
_SSM_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "A_log": "A_log", "D": "D",
              "norm": "norm", "o": "o"}
_MLP_NAMES = {"up": "up", "down": "down", "act": "act"}


def _norm(prefix: str) -> PartSpec:
    return PartSpec("dynamic_tanh", {"weight_name": "", "bias_name": ".b", "alpha_name": ".alpha"}, prefix=prefix)


def _attention_params(a, names: dict) -> dict:
    if a.rot is not None:
        position = PartSpec("rope", {"head_dim": a.dim, "base": a.rot.base, "style": "interleaved", "rot_dims": a.rot.dims,
                                     "exact_angles": True})
    else:
        position = PartSpec("unrotated", {})
    return {"n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim, "position": position,
            "scale": a.scale, "softcap": a.softcap, "window": a.window, "keep_first": a.keep_first, "names": names}


def build_spec(cfg: RedodraConfig) -> ModelSpec:
    layers, schedule = [], []
    runs = len(cfg.layers)
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        cache = i
        if L.kind == "attention":
            mixer = PartSpec("gqa_attention", dict(_attention_params(m, _GATED_NAMES), qkv_bias=False, sink=True,
                                                   head_gate=True, own_kv=m.kv_from is None), prefix="mix.")
            if m.kv_from is not None:
                cache = m.kv_from
        elif L.kind == "delta":
            mixer = PartSpec("gated_delta_rule", {"n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
                                                  "v_head_dim": m.vdim, "conv": m.conv, "eps": cfg.norm_eps,
                                                  "names": _DELTA_NAMES}, prefix="mix.")
        else:
            left = PartSpec("gqa_attention", dict(_attention_params(m.left, _WINDOW_NAMES), qkv_bias=True, o_bias=True,
                                                  distance_bias=True), prefix="left.")
            r = m.right
            right = PartSpec("selective_state_space", {"n_heads": r.heads, "v_head_dim": r.vdim, "state": r.state,
                                                       "groups": r.groups, "conv": r.conv, "norm_groups": r.norm_groups,
                                                       "eps": cfg.norm_eps, "conv_bias": True, "names": _SSM_NAMES},
                             prefix="right.")
            mixer = PartSpec("parallel_mixers", {"members": ((left, 0.5), (right, 0.5)),
                                                 "member_norm": {"eps": cfg.norm_eps, "weight_name": "out"}}, prefix="mix.")
        parts = {"mixer": mixer, "mixer_norm": _norm("norm1"), "mixer_post_norm": _norm("norm1b"),
                 "depth": PartSpec("weighted_depth_sum", {"index": i, "entries": runs + 1, "weight_name": ""}, prefix="dwa")}
        if L.mlp is not None:
            parts["feed_forward"] = PartSpec("dense_act", {"intermediate_size": L.mlp.ff, "activation": "xielu",
                                                           "names": _MLP_NAMES}, prefix="mlp.")
            parts["feed_forward_norm"], parts["feed_forward_post_norm"] = _norm("norm2"), _norm("norm2b")
        layers.append(LayerSpec(prefix=f"l{i}.", arrangement="pre_post_norm", parts=parts))
        schedule.append(ScheduleEntry(layer=i, cache=cache))
    head = PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "norm": _norm("final.norm"), "tied": False,
                                    "weight_prefix": "head", "weight_name": ""})
    embedding = PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "weight_name": ""}, prefix="embed")
    return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=MAX_POSITIONS,
                     layers=tuple(layers), schedule=tuple(schedule), embedding=embedding, head=head)


register_architecture(ARCHITECTURE, RedodraConfig.from_dict, build_spec, replace=True)
