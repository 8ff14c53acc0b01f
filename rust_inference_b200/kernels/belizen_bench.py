"""Prefill and decode throughput of a Belizen-style model beside the two closest models of equal size (a Lulisun-style
model: attention beside a gated linear recurrence, routed experts with a shared one; a dense decoder: plain attention and
a gated feed-forward), and the time of each of its kernels against its roofline (`python bench.py --arch belizen`).

All models get random bf16 weights and the same width, depth, heads and head size.  The Belizen model has four layers:
window attention with kept first positions and a dense gated feed-forward, two layers of gated linear attention with
routed experts, and window attention with routed experts; its dense feed-forward is as wide as the experts a token uses
plus the shared expert.  A kernel's roofline time is the slowest of its multiply-adds at the measured bf16 throughput,
its bytes at the measured copy bandwidth and, for the recurrence and the router, its float32 multiply-adds at the FFMA
pipe's nominal rate; `x_roofline` is measured time over that.  Timed with CUDA events after warm-up, a 256 MiB write
between iterations (flushes L2).
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
    # width; attention heads / kv heads / head size; window and kept first positions; rotated channels; heads of the gated
    # linear attention (as wide as the attention's) and the rank of its decay; experts with tensors / pass-through ones /
    # chosen / expert width / shared width; vocabulary.  `chunk`, `groups` and `keep` are the Lulisun model's.
    "1k": dict(width=1024, layers=4, heads=8, kv=2, hd=128, window=512, kept=64, rot=64, rheads=4, rank=32, experts=16, identity=4,
               top=2, ff=512, shared=1024, vocab=32000, chunk=512, groups=4, keep=2),
    "2k": dict(width=2048, layers=4, heads=16, kv=4, hd=128, window=1024, kept=64, rot=64, rheads=8, rank=64, experts=32, identity=8,
               top=4, ff=512, shared=2048, vocab=32000, chunk=1024, groups=8, keep=4),
    "4k": dict(width=4096, layers=4, heads=32, kv=8, hd=128, window=1024, kept=128, rot=128, rheads=16, rank=64, experts=64,
               identity=16, top=6, ff=1024, shared=4096, vocab=32000, chunk=2048, groups=8, keep=4),
}


def belizen_config(s: dict) -> dict:
    attn = {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["hd"], "vdim": s["hd"], "scale": 1.0 / math.sqrt(s["hd"]),
            "softcap": 30.0, "mask": {"size": s["window"], "keep_first": s["kept"]},
            "rot": {"base": 10000.0, "dims": s["rot"], "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    gla = {"heads": s["rheads"], "dim": s["hd"], "vdim": s["hd"], "tau": 16.0, "rank": s["rank"]}
    moe = {"kind": "moe", "expert": {"ff": s["ff"], "limit": 7.0},
           "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"]}, "shared": {"ff": s["shared"], "limit": 7.0}}
    dense = {"kind": "dense", "ff": s["top"] * s["ff"] + s["shared"]}
    return {"architecture": "Belizen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "residual_mult": 0.5, "logit_softcap": 30.0, "loop": {"start": 1, "stop": 3, "times": 1}, "layers": [
                {"type": "attention", "mixer": attn, "mlp": dense}, {"type": "gla", "mixer": gla, "mlp": moe},
                {"type": "gla", "mixer": gla, "mlp": moe}, {"type": "attention", "mixer": attn, "mlp": moe}]}


def time_parts(engine, s: dict, lens_before: list, new_tokens: int, peaks: dict, timer: Timer) -> dict:
    """Milliseconds of the Belizen model's mixers and feed-forwards and of their kernels alone, for a step of `new_tokens`
    tokens per sequence on top of `lens_before` cached positions, with each kernel's roofline."""
    from . import attention as attn_kernels, linear, ops, tcgen05
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
    normed = torch.empty(n, width, dtype=bf, device=dev)
    stream = torch.randn(n, width, device=dev)
    row("rms_norm", timer(lambda: blocks[0].mixer_norm.forward(stream, normed)), 0.0, n * width * 6 + width * 4)
    entry = engine.model.stream_parts[0]
    row("pass_entry", timer(lambda: ops.stream_add(stream, None, entry.step[0])), 0.0, n * width * 8 + width * 4)

    # ---- window attention (layer 0) ------------------------------------------------------------------------------------
    att, cache0 = blocks[0].mixer, engine.cache.layer(0)
    out["attention_mixer_ms"] = round(timer(lambda: att.forward(x, residual, ctx, cache0, True)), 4)
    hd, heads, kv, window, kept = s["hd"], s["heads"], s["kv"], s["window"], s["kept"]
    vis, kv_bytes = 0, 0
    for before in lens_before:
        for p in range(before, before + new_tokens):
            first = max(0, p - window + 1)
            vis += p + 1 - first + min(kept, first)
        first = max(0, before - window + 1)
        kv_bytes += (before + new_tokens - first + min(kept, first)) * kv * 2 * hd * 2
    qkv = (torch.randn(n, att.w_qkv.n, device=dev) * 0.5).to(bf)
    mixed = torch.empty(n, att.o_dim, dtype=bf, device=dev)
    ms = timer(lambda: attn_kernels.attention(qkv, cache0, mixed, ctx, n_heads=heads, n_kv_heads=kv, head_dim=hd, scale=att.scale,
                                              window=window, softcap=att.softcap, keep_first=kept))
    row("window_attention", ms, 4.0 * hd * vis * heads, kv_bytes + n * heads * hd * 2 * 2)
    ms = timer(lambda: att.position.apply_normed_and_store(qkv, ctx, cache0, n_heads=heads, n_kv_heads=kv, head_dim=hd, write_kv=True,
                                                           q_weight=att.q_norm, k_weight=att.k_norm, eps=1e-5))
    row("norm_rotate_store", ms, 0.0, n * (2 * heads + 4 * kv) * hd * 2)
    gate_col = att.q_dim + att.kv_dim + att.v_dim
    row("output_gate", timer(lambda: ops.sigmoid_gate_(mixed, qkv, gate_col, 0.5)), 0.0, n * att.o_dim * 2 * 3)
    row("qkv_gate_projection", timer(lambda: linear.project(x, att.w_qkv, qkv, ctx, bias=att.b_qkv)), 2.0 * n * att.w_qkv.n * width,
        att.w_qkv.n * width * 2 + n * (width + att.w_qkv.n) * 2)

    # ---- gated linear attention (layer 1) ------------------------------------------------------------------------------
    gla, cache1 = blocks[1].mixer, engine.cache.layer(1)
    out["linear_attention_mixer_ms"] = round(timer(lambda: gla.forward(x, residual, ctx, cache1, True)), 4)
    H, dim, vdim = gla.n_heads, gla.head_dim, gla.v_head_dim
    z = torch.randn(n, gla.width, device=dev) * 0.5
    row("linear_attention_projection", timer(lambda: linear.logits(x, gla.w_in, z, ctx)), 2.0 * n * gla.width * width,
        gla.width * width * 2 + n * (width * 2 + gla.width * 4))
    decay = torch.empty(n, gla.q_dim, dtype=f32, device=dev)
    o = torch.empty(n, gla.v_dim, dtype=bf, device=dev)
    o_raw = torch.empty(n, gla.v_dim, dtype=f32, device=dev)
    piece, most = ops.recurrence_pieces(ctx.max_new, ctx.n_seqs, H, dim, vdim)
    scratch = torch.empty(ctx.n_seqs * most * H * dim * (vdim + 1), dtype=f32, device=dev) if piece else None

    def recur():
        ops.gated_linear_attention(z, q_col=gla.q_col, k_col=gla.k_col, v_col=gla.v_col, g_col=gla.g_col, a_col=gla.a_col,
                                   rank=gla.rank, w2=gla.w2, bias=gla.decay_bias, tau=gla.tau, q_scale=1.0, decay=decay,
                                   norm_weight=gla.norm, state=cache1.state, cu_seqlens=ctx.cu_seqlens, seq_slot=ctx.seq_slot, out=o,
                                   n_seqs=ctx.n_seqs, heads=H, dim=dim, vdim=vdim, eps=1e-5, out_scale=0.5, o_raw=o_raw, piece=piece,
                                   max_pieces=most, scratch=scratch, longest_run=ctx.max_new)
    # z read once (q, k, v, the gates, the decay's input) and the decays written and read, o written, every sequence's state
    # read and written; per token, head and state element three float32 multiply-adds that no tensor core may take, and
    # per token and key channel `rank` more for the decay
    rec_bytes = n * (gla.width * 4 + gla.q_dim * 8 + gla.v_dim * 2) + 2 * B * H * dim * vdim * 4
    row("linear_attention_recurrence", timer(recur), 0.0, rec_bytes, fp32_flops=6.0 * n * H * dim * vdim + 2.0 * n * gla.q_dim * gla.rank)

    # ---- feed-forwards ---------------------------------------------------------------------------------------------------
    ff = blocks[0].feed_forward
    out["dense_feed_forward_ms"] = round(timer(lambda: ff.forward(x, residual, ctx)), 4)
    inter = ff.intermediate_size
    act = torch.empty(n, inter, dtype=bf, device=dev)
    row("gate_up", timer(lambda: linear.gated(x, ff.w_gate, ff.w_up, act, ctx, form=ff.form)), 2.0 * n * 2 * inter * width,
        2 * inter * width * 2 + n * (width + inter) * 2)
    row("down", timer(lambda: linear.into_residual(act, ff.w_down, residual, ctx)), 2.0 * n * inter * width,
        inter * width * 2 + n * (inter * 2 + width * 8))
    mx = blocks[1].feed_forward
    out["experts_feed_forward_ms"] = round(timer(lambda: mx.forward(x, residual, ctx)), 4)
    top, experts, f, outputs = s["top"], s["experts"], s["ff"], s["experts"] + s["identity"]
    pairs = n * top
    ids = torch.empty(n, top, dtype=torch.int32, device=dev)
    wts = torch.empty(n, top, dtype=f32, device=dev)
    route = lambda: ops.moe_route(x, mx.router, mx.correction, ids, wts, top=top, softmax=True, normalise=False, **mx.route_cut(n, ctx))
    row("router", timer(route), 0.0, outputs * width * 4 + n * width * 2, fp32_flops=2.0 * n * outputs * width)
    real = int((ids < experts).sum())
    used = int(torch.unique(ids[ids < experts]).numel())
    fast = mx._on_tensor_cores(x)
    rows = tcgen05.GROUPED_TILE_ROWS if fast else ops.moe_tile_rows()
    i32 = lambda k: torch.zeros(k, dtype=torch.int32, device=dev)
    offsets, order, tiles, n_tiles, place = i32(experts + 1), i32(pairs), i32(2 * (-(-pairs // rows) + experts)), i32(1), i32(pairs)
    arrange = lambda: ops.moe_arrange(ids, pairs, experts, rows, offsets, order, tiles, n_tiles, place)
    arrange()
    y = torch.empty(pairs, width, dtype=f32, device=dev)
    acts = torch.empty(pairs, f, dtype=bf, device=dev)
    if fast:
        xs = torch.zeros(pairs, width, dtype=bf, device=dev)
        gather = lambda: ops.moe_gather(x, xs, order, n_pairs=pairs, top=top, listed=offsets[experts:experts + 1])
        gather()
        ms_up = timer(lambda: tcgen05.grouped_gemm(xs, mx.w_gate, mx.w_up, acts, offsets, tiles, n_tiles, n_pairs=pairs,
                                                   gate_form=mx.expert_form))
        ms_down = timer(lambda: tcgen05.grouped_gemm(acts, mx.w_down, None, y, offsets, tiles, n_tiles, n_pairs=pairs))
        out["gather_ms"] = round(timer(gather), 4)
    else:
        ms_up = timer(lambda: ops.moe_grouped_simt(x, mx.w_gate, mx.w_up, acts, offsets, order, tiles, n_tiles, n_pairs=pairs, top=top,
                                                   gate_form=mx.expert_form))
        ms_down = timer(lambda: ops.moe_grouped_simt(acts, mx.w_down, None, y, offsets, order, tiles, n_tiles, n_pairs=pairs, top=top))
    out["arrange_ms"] = round(timer(arrange), 4)
    # the pairs that reach an expert with tensors do the work; the others are the input handed through
    row("experts_gate_up", ms_up, 2.0 * real * 2 * f * width, used * 2 * f * width * 2 + real * (width + f) * 2)
    row("experts_down", ms_down, 2.0 * real * f * width, used * f * width * 2 + real * (f * 2 + width * 4))
    shared_y = torch.randn(n, width, device=dev)
    ms = timer(lambda: ops.moe_combine(residual, y, wts, top=top, shared_y=shared_y, place=place if fast else None, ids=ids, x=x,
                                       n_real=experts, scale=0.5))
    row("combine", ms, 0.0, real * width * 4 + n * width * (4 + 8 + 2) + pairs * 12)
    out["pairs_with_tensors"], out["experts_used"], out["experts_kernel"] = real, used, "tcgen05" if fast else "ffma"
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
    result = {"arch": "belizen", "sizes": sizes, "config": s, "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
              "peaks": dict(peaks, source=peak_source), "l2": "256 MiB written between timed iterations"}
    models = (("belizen", belizen_config(s)), ("lulisun", arch_bench.lulisun_config(s)), ("dense", arch_bench.dense_config(s, cache_tokens)))
    for kind, cfg in models:
        t0 = time.time()
        engine = Engine.from_random(config_from_dict(cfg), seed=0, std=0.02, dtype="bfloat16", device="cuda:0",
                                    max_tokens=cache_tokens, n_slots=batch + 2)
        print(f"[bench] {kind} ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        r = throughput(engine, s, prefill_tokens=prefill_tokens, batch=batch, context=context, steps=steps, timer=timer)
        for phase, before, new in (("prefill_parts", [0], prefill_tokens), ("decode_parts", [context] * batch, 1)):
            if kind == "belizen":
                r[phase] = time_parts(engine, s, before, new, peaks, timer)
            else:
                r[phase] = arch_bench.time_parts(engine, kind, s, before, new, peaks, timer)
                if kind == "dense":
                    r[phase].update(dense_norm_and_rope(engine, s, before, new, peaks, timer))
        engine.check_device_status()
        result[kind] = r
        del engine
        torch.cuda.empty_cache()
    # how far each kernel of the new design is from its roofline, over the like kernel of the closest model
    like = {"window_attention": ("lulisun", "attention"), "linear_attention_recurrence": ("lulisun", "recurrence"),
            "experts_gate_up": ("lulisun", "experts_gate_up"), "experts_down": ("lulisun", "experts_down"),
            "gate_up": ("dense", "gate_up"), "down": ("dense", "down"), "rms_norm": ("dense", "rms_norm"),
            "norm_rotate_store": ("dense", "rotate_store"), "output_gate": ("dense", "rms_norm"), "pass_entry": ("dense", "rms_norm"),
            "combine": ("dense", "rms_norm"), "qkv_gate_projection": ("dense", "down"), "linear_attention_projection": ("dense", "down")}
    ratios = {}
    for phase in ("prefill_parts", "decode_parts"):
        for name, (model, other) in like.items():
            ratios[f"{phase[:-6]}.{name} (over {model} {other})"] = round(
                result["belizen"][phase][name]["x_roofline"] / result[model][phase][other]["x_roofline"], 2)
        ratios[f"{phase[:-6]}.router ms (over lulisun router ms)"] = round(
            result["belizen"][phase]["router"]["ms"] / max(result["lulisun"][phase]["route_ms"], 1e-6), 2)
    result["x_roofline_over_like"] = ratios
    print(json.dumps(result))
    return 0
