"""Prefill and decode throughput of a Redodra-style model beside the two closest models of equal size (a Lulisun-style
model: attention beside a recurrence with a matrix state; a dense decoder: plain attention and a gated feed-forward), and
the time of each of its kernels against its roofline (`python bench.py --arch redodra`).

All models get random bf16 weights and the same width, depth, heads and head size.  The Redodra model has four layers:
window attention beside a state space, causal attention with a sink and a gate, the gated delta rule, and causal
attention over the second layer's keys.  A kernel's roofline time is the slowest of its multiply-adds at the measured
bf16 throughput, its bytes at the measured copy bandwidth and, for the recurrences, its float32 multiply-adds at the
FFMA pipe's nominal rate; `x_roofline` is measured time over that.  Timed with CUDA events after warm-up, a 256 MiB
write between iterations (flushes L2).
"""
from __future__ import annotations

import json
import math
import sys
import time

import torch

from . import arch_bench
from .arch_bench import Timer, _roofline_ms, _step_context, ffma_peak_tflops, throughput
from .vadodra_bench import dense_norm_and_rope

SIZES = {
    # width; attention heads / kv heads / head size; window and kept first positions; rotated channels; heads and state
    # rows of the state space (its value heads are as wide as the attention's), its groups; heads of the delta rule;
    # feed-forward width, vocabulary.  `chunk`, `rheads` and the experts are the Lulisun model's of equal size.
    "1k": dict(width=1024, layers=4, heads=8, kv=2, hd=128, window=512, keep=64, rot=64, sheads=16, svdim=64, state=128, groups=2,
               dheads=8, ff=4096, vocab=32000, chunk=512, rheads=4, experts=16, top=2, eff=512, egroups=4, ekeep=2, shared=1024),
    "2k": dict(width=2048, layers=4, heads=16, kv=4, hd=128, window=1024, keep=64, rot=64, sheads=32, svdim=64, state=128, groups=4,
               dheads=16, ff=8192, vocab=32000, chunk=1024, rheads=8, experts=32, top=4, eff=512, egroups=8, ekeep=4, shared=2048),
    "4k": dict(width=4096, layers=4, heads=32, kv=8, hd=128, window=1024, keep=128, rot=128, sheads=64, svdim=64, state=128, groups=8,
               dheads=32, ff=14336, vocab=32000, chunk=2048, rheads=16, experts=64, top=6, eff=1024, egroups=8, ekeep=4, shared=4096),
}


def redodra_config(s: dict) -> dict:
    scale = 1.0 / math.sqrt(s["hd"])
    mlp = {"kind": "dense", "ff": s["ff"]}
    attn = {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["hd"], "vdim": s["hd"], "scale": scale, "softcap": 50.0,
            "rot": {"base": 10000.0, "dims": s["rot"]}}
    side = {"left": {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["hd"], "vdim": s["hd"], "scale": scale, "softcap": 50.0,
                     "mask": {"size": s["window"], "keep_first": s["keep"]}},
            "right": {"heads": s["sheads"], "vdim": s["svdim"], "state": s["state"], "groups": s["groups"], "conv": 4,
                      "norm_groups": s["groups"]}}
    delta = {"heads": s["dheads"], "kv_heads": s["dheads"], "dim": s["hd"], "vdim": s["hd"], "conv": 4}
    return {"architecture": "Redodra", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "layers": [
        {"type": "parallel", "mixer": side, "mlp": mlp}, {"type": "attention", "mixer": attn, "mlp": mlp},
        {"type": "delta", "mixer": delta, "mlp": mlp}, {"type": "attention", "mixer": dict(attn, kv_from=1), "mlp": mlp}]}


def _lulisun_sizes(s: dict) -> dict:
    return dict(s, ff=s["eff"], groups=s["egroups"], keep=s["ekeep"])


def dense_config(s: dict, max_positions: int) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "hidden_size": s["width"], "num_hidden_layers": s["layers"],
            "num_attention_heads": s["heads"], "num_key_value_heads": s["kv"], "head_dim": s["hd"],
            "intermediate_size": s["ff"], "vocab_size": s["vocab"], "rope_theta": 10000.0, "rms_norm_eps": 1e-5,
            "attention_bias": False, "tie_word_embeddings": False, "max_position_embeddings": max_positions}


def time_parts(engine, s: dict, lens_before: list, new_tokens: int, peaks: dict, timer: Timer) -> dict:
    """Milliseconds of the Redodra model's mixers and feed-forward and of their kernels alone, for a step of `new_tokens`
    tokens per sequence on top of `lens_before` cached positions, with each kernel's roofline."""
    from . import attention as attn_kernels, linear, ops
    slots, ctx = _step_context(engine, lens_before, new_tokens, s["vocab"], 5)
    dev, bf, f32 = engine.device, torch.bfloat16, torch.float32
    n, width, B = ctx.n_tokens, s["width"], len(lens_before)
    residual = torch.zeros(n, width, dtype=f32, device=dev)
    x = (torch.randn(n, width, device=dev) * 0.5).to(bf)
    out = {}

    def row(name, ms, flops, bytes_, fp32_flops=0.0):
        ideal = _roofline_ms(flops, bytes_, peaks, fp32_flops)
        times = {"tensor": flops / (peaks["bf16_tflops"] * 1e12), "hbm": bytes_ / (peaks["hbm_gbs"] * 1e9),
                 "ffma": fp32_flops / (peaks["fp32_ffma_tflops_nominal"] * 1e12)}
        out[name] = {"ms": round(ms, 4), "roofline_ms": round(ideal, 6), "x_roofline": round(ms / ideal, 2),
                     "bound": max(times, key=times.get)}

    blocks = [layer.block for layer in engine.model.layers]
    # ---- the norm and the end of a sublayer ---------------------------------------------------------------------
    normed = torch.empty(n, width, dtype=bf, device=dev)
    stream = torch.randn(n, width, device=dev)
    row("squash_norm", timer(lambda: blocks[0].mixer_norm.forward(stream, normed)), 0.0, n * width * 6 + width * 8)
    branch = torch.randn(n, width, device=dev)
    depth = blocks[1].depth
    kw = depth.fused(ctx, stream)
    ms = timer(lambda: ops.stream_update(stream, branch=branch, post=blocks[1].feed_forward_post_norm.fused(),
                                         next_norm=blocks[2].mixer_norm.fused(), next_out=normed, **kw))
    # stream and branch read and written, the layer's result stored, the earlier results read, the next norm written
    row("join_depth_sum_norm", ms, 0.0, n * width * (16 + 4 + 4 * (depth.index + 1) + 2))

    # ---- window attention beside a state space (layer 0) ------------------------------------------------------------
    par, cache0 = blocks[0].mixer, engine.cache.layer(0)
    (_, left), (_, right) = par.members
    kv_layer, state_layers = cache0.parts
    out["parallel_mixer_ms"] = round(timer(lambda: par.forward(x, residual, ctx, cache0, True)), 4)
    hd, heads, kv, window, keep = s["hd"], s["heads"], s["kv"], s["window"], s["keep"]
    vis, kv_bytes = 0, 0
    for before in lens_before:
        for p in range(before, before + new_tokens):
            first = max(0, p - window + 1)
            vis += p + 1 - first + min(keep, first)
        first = max(0, before - window + 1)
        kv_bytes += (before + new_tokens - first + min(keep, first)) * kv * 2 * hd * 2
    qkv = (torch.randn(n, left.q_dim + left.kv_dim + left.v_dim, device=dev) * 0.5).to(bf)
    mixed = torch.empty(n, left.o_dim, dtype=bf, device=dev)
    ms = timer(lambda: attn_kernels.attention(qkv, kv_layer, mixed, ctx, n_heads=heads, n_kv_heads=kv, head_dim=hd, scale=left.scale,
                                              window=window, softcap=left.softcap, keep_first=keep, dist=left.dist))
    row("window_attention", ms, 4.0 * hd * vis * heads, kv_bytes + n * heads * hd * 2 * 2)
    joined = [(torch.randn(n, width, device=dev), None, w, 0.5) for w in par.norm_weights]
    row("normed_sum", timer(lambda: ops.normed_sum(joined, residual, 1e-5, accumulate=True)), 0.0, n * width * (2 * 8 + 8))

    def scan_rows(tag, part, matrix, carried, dim, vdim, H, groups, delta, prepare_kw, scan_kw, norm_kw):
        z = torch.randn(n, part.width, device=dev) * 0.5
        u = torch.empty(n, part.conv_ch + 2 * H, dtype=f32, device=dev)
        ms = timer(lambda: ops.scan_prepare(z, conv_ch=part.conv_ch, taps=part.w_conv, conv_state=carried.state, heads=H, a_log=part.a_log,
                                            dt_bias=part.dt_bias, out=u, cu_seqlens=ctx.cu_seqlens, token_seq=ctx.token_seq,
                                            seq_slot=ctx.seq_slot, n_seqs=ctx.n_seqs, **prepare_kw))
        row(tag + "_prepare", ms, 0.0, n * (part.conv_ch * 8 + 4 * H * 4) + 2 * B * carried.state[0].numel() * 4)
        o = torch.empty(n, H * vdim, dtype=f32, device=dev)
        piece, max_pieces = (0, 1) if delta else ops.scan_pieces(ctx.max_new, ctx.n_seqs * H * -(-vdim // 16))     # as the part calls it
        if piece:
            scan_kw = dict(scan_kw, piece=piece, max_pieces=max_pieces,
                           piece_state=torch.empty(ctx.n_seqs, max_pieces, H, dim, vdim, dtype=f32, device=dev),
                           piece_decay=torch.empty(ctx.n_seqs, max_pieces, H, dtype=f32, device=dev))
        ms = timer(lambda: ops.state_scan(u, matrix.state, o, ctx.cu_seqlens, ctx.seq_slot, n_seqs=ctx.n_seqs, heads=H, groups=groups,
                                          dim=dim, vdim=vdim, delta=delta, longest_run=ctx.max_new, **scan_kw))
        # the prepared rows read (keys and queries once per head that shares them), the result written, every state read
        # and written; per token, head and state element three (state space) or four (delta rule) float32 multiply-adds
        scan_bytes = n * (H * (2 * dim + vdim + 2) + H * vdim) * 4 + 2 * B * H * dim * vdim * 4
        row(tag + "_scan", ms, 0.0, scan_bytes, fp32_flops=(8.0 if delta else 6.0) * n * H * dim * vdim)
        normed_o = torch.empty(n, H * vdim, dtype=bf, device=dev)
        ms = timer(lambda: ops.gated_group_norm(o, z, norm_kw["gate_col"], part.norm, normed_o, **norm_kw["args"]))
        row(tag + "_gated_norm", ms, 0.0, n * H * vdim * (4 + 4 + 2))

    matrix, carried = state_layers.parts
    H, gn = right.n_heads, right.groups * right.state
    scan_rows("state_space", right, matrix, carried, right.state, right.v_head_dim, H, right.groups, False,
              dict(conv_col=right.inner, conv_bias=right.b_conv, unit_heads=0, unit_dim=0, scaled_heads=0, unit_scale=1.0,
                   decay_col=2 * right.inner + 2 * gn, step_col=-1),
              dict(q_col=right.inner + gn, k_col=right.inner, v_col=0, decay_col=right.conv_ch, step_col=right.conv_ch + H, skip=right.skip),
              dict(gate_col=0, args=dict(groups=right.norm_groups, group_size=right.inner // right.norm_groups, gate_first=True, eps=1e-5)))

    # ---- causal attention with a sink and a gate (layer 1) -----------------------------------------------------------
    gat, cache1 = blocks[1].mixer, engine.cache.layer(1)
    out["gated_attention_mixer_ms"] = round(timer(lambda: gat.forward(x, residual, ctx, cache1, True)), 4)
    causal = sum(p + 1 for before in lens_before for p in range(before, before + new_tokens))
    all_kv = sum(before + new_tokens for before in lens_before) * kv * 2 * hd * 2
    gate_col = gat.q_dim + gat.kv_dim + gat.v_dim
    qkvg = (torch.randn(n, gat.w_qkv.n, device=dev) * 0.5).to(bf)
    gate = qkvg[:, gate_col:gate_col + heads]
    ms = timer(lambda: attn_kernels.attention(qkvg, cache1, mixed, ctx, n_heads=heads, n_kv_heads=kv, head_dim=hd, scale=gat.scale,
                                              softcap=gat.softcap, sink=gat.sinks, gate=gate))
    row("gated_attention", ms, 4.0 * hd * causal * heads, all_kv + n * heads * hd * 2 * 2)
    ms = timer(lambda: gat.position.apply_and_store(qkvg, ctx, cache1, n_heads=heads, n_kv_heads=kv, head_dim=hd, write_kv=True))
    row("rotate_store", ms, 0.0, n * (2 * heads + 4 * kv) * hd * 2)

    # ---- the gated delta rule (layer 2) -----------------------------------------------------------------------------
    dl, cache2 = blocks[2].mixer, engine.cache.layer(2)
    out["delta_mixer_ms"] = round(timer(lambda: dl.forward(x, residual, ctx, cache2, True)), 4)
    matrix, carried = cache2.parts
    H, G = dl.n_heads, dl.n_kv_heads
    scan_rows("delta_rule", dl, matrix, carried, dl.head_dim, dl.v_head_dim, H, G, True,
              dict(conv_col=0, conv_bias=None, unit_heads=2 * G, unit_dim=dl.head_dim, scaled_heads=G, unit_scale=dl.head_dim ** -0.5,
                   decay_col=dl.a_col, step_col=dl.beta_col),
              dict(q_col=0, k_col=dl.qk_dim, v_col=2 * dl.qk_dim, decay_col=dl.conv_ch, step_col=dl.conv_ch + H),
              dict(gate_col=dl.gate_col, args=dict(groups=H, group_size=dl.v_head_dim, gate_first=False, eps=1e-5)))

    # ---- feed-forward --------------------------------------------------------------------------------------------
    ff = blocks[0].feed_forward
    out["feed_forward_ms"] = round(timer(lambda: ff.forward(x, residual, ctx)), 4)
    inter = ff.intermediate_size
    act = torch.empty(n, inter, dtype=bf, device=dev)
    row("up_activation", timer(lambda: linear.activated(x, ff.w_up, act, ctx, ff.act)), 2.0 * n * inter * width,
        inter * width * 2 + n * (width + inter) * 2)
    row("down", timer(lambda: linear.into_residual(act, ff.w_down, residual, ctx)), 2.0 * n * inter * width,
        inter * width * 2 + n * (inter * 2 + width * 8))
    engine.workspace.rezero()
    for slot in slots:
        engine.free_slot(slot)
    return out


def main(sizes: str, peaks: dict, peak_source: str, *, prefill_tokens: int = 2048, batch: int = 8, context: int | None = None,
         steps: int = 64) -> int:
    from ..config.registry import config_from_dict
    from ..engine.engine import Engine
    s = SIZES[sizes]
    if context is None:
        context = s["window"] + s["window"] // 4        # the window layers see a full window and the kept positions
    torch.cuda.set_device(0)
    timer = Timer("cuda:0")
    peaks = dict(peaks, fp32_ffma_tflops_nominal=round(ffma_peak_tflops(), 1))
    cache_tokens = batch * (context + steps + 128) + prefill_tokens + 4096
    result = {"arch": "redodra", "sizes": sizes, "config": s, "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
              "peaks": dict(peaks, source=peak_source), "l2": "256 MiB written between timed iterations"}
    ls = _lulisun_sizes(s)
    models = (("redodra", redodra_config(s)), ("lulisun", arch_bench.lulisun_config(ls)), ("dense", dense_config(s, cache_tokens)))
    for kind, cfg in models:
        t0 = time.time()
        engine = Engine.from_random(config_from_dict(cfg), seed=0, std=0.02, dtype="bfloat16", device="cuda:0",
                                    max_tokens=cache_tokens, n_slots=batch + 2)
        print(f"[bench] {kind} ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        r = throughput(engine, s, prefill_tokens=prefill_tokens, batch=batch, context=context, steps=steps, timer=timer)
        for phase, before, new in (("prefill_parts", [0], prefill_tokens), ("decode_parts", [context] * batch, 1)):
            if kind == "redodra":
                r[phase] = time_parts(engine, s, before, new, peaks, timer)
            elif kind == "lulisun":
                r[phase] = arch_bench.time_parts(engine, "lulisun", ls, before, new, peaks, timer)
            else:
                r[phase] = arch_bench.time_parts(engine, "dense", s, before, new, peaks, timer)
                r[phase].update(dense_norm_and_rope(engine, s, before, new, peaks, timer))
        engine.check_device_status()
        result[kind] = r
        del engine
        torch.cuda.empty_cache()
    # how far each kernel of the new design is from its roofline, over the like kernel of the closest model
    like = {"window_attention": ("lulisun", "attention"), "gated_attention": ("dense", "attention"),
            "state_space_scan": ("lulisun", "recurrence"), "delta_rule_scan": ("lulisun", "recurrence"),
            "up_activation": ("dense", "gate_up"), "down": ("dense", "down"), "squash_norm": ("dense", "rms_norm"),
            "join_depth_sum_norm": ("dense", "rms_norm"), "normed_sum": ("dense", "rms_norm"), "rotate_store": ("dense", "rotate_store"),
            "state_space_prepare": ("dense", "rotate_store"), "delta_rule_prepare": ("dense", "rotate_store"),
            "state_space_gated_norm": ("dense", "rms_norm"), "delta_rule_gated_norm": ("dense", "rms_norm")}
    ratios = {}
    for phase in ("prefill_parts", "decode_parts"):
        for name, (model, other) in like.items():
            ratios[f"{phase[:-6]}.{name} (over {model} {other})"] = round(
                result["redodra"][phase][name]["x_roofline"] / result[model][phase][other]["x_roofline"], 2)
    result["x_roofline_over_like"] = ratios
    print(json.dumps(result))
    return 0
