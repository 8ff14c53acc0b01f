"""Prefill and decode throughput of a Lulisun-style model beside a dense decoder of equal size, and
the time of each of their kernels against its roofline (`python bench.py --arch lulisun`).

Both models get random bf16 weights and the same width, depth, heads and head size; the dense
decoder's feed-forward is as wide as the experts a token uses plus the shared expert, so a token costs
both models the same multiply-adds.  A kernel's roofline time is the slower of its multiply-adds at the
measured bf16 throughput and its bytes at the measured copy bandwidth; `x_roofline` is measured time
over that.  Timed with CUDA events after warm-up, a 256 MiB write between iterations (flushes L2).
"""
from __future__ import annotations

import json
import math
import random
import sys
import time

import torch

SIZES = {
    # width, layers, attention heads / kv heads / head size, chunk, rotated channels, recurrent heads,
    # experts / chosen / expert width / groups / kept groups / shared width, vocabulary
    "1k": dict(width=1024, layers=4, heads=8, kv=2, hd=128, chunk=512, rot=64, rheads=4, experts=16, top=2, ff=512,
               groups=4, keep=2, shared=1024, vocab=32000),
    "2k": dict(width=2048, layers=4, heads=16, kv=4, hd=128, chunk=1024, rot=64, rheads=8, experts=32, top=4, ff=512,
               groups=8, keep=4, shared=2048, vocab=32000),
    "4k": dict(width=4096, layers=2, heads=32, kv=8, hd=128, chunk=2048, rot=128, rheads=16, experts=64, top=6, ff=1024,
               groups=8, keep=4, shared=4096, vocab=32000),
}


def lulisun_config(s: dict) -> dict:
    layer = {"type": "parallel", "mixer": {
        "left": {"heads": s["heads"], "kv_heads": s["kv"], "dim": s["hd"], "vdim": s["hd"], "scale": 1.0 / math.sqrt(s["hd"]),
                 "mask": {"size": s["chunk"]}, "rot": {"base": 10000.0, "dims": s["rot"]}},
        "right": {"heads": s["rheads"], "dim": s["hd"], "vdim": s["hd"]}, "left_scale": 0.7, "right_scale": 0.7},
        "mlp": {"kind": "moe", "expert": {"ff": s["ff"]},
                "router": {"experts": s["experts"], "top": s["top"], "groups": {"count": s["groups"], "keep": s["keep"]}},
                "shared": {"ff": s["shared"]}}}
    return {"architecture": "Lulisun", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
            "layers": [layer] * s["layers"]}


def dense_config(s: dict, max_positions: int) -> dict:
    return {"architectures": ["LlamaForCausalLM"], "hidden_size": s["width"], "num_hidden_layers": s["layers"],
            "num_attention_heads": s["heads"], "num_key_value_heads": s["kv"], "head_dim": s["hd"],
            "intermediate_size": s["top"] * s["ff"] + s["shared"], "vocab_size": s["vocab"], "rope_theta": 10000.0,
            "rms_norm_eps": 1e-5, "attention_bias": False, "tie_word_embeddings": False,
            "max_position_embeddings": max_positions}


class Timer:
    def __init__(self, device):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)

    def __call__(self, fn, warm: int = 3, iters: int = 7) -> float:
        """Median milliseconds of fn()."""
        times = []
        for i in range(warm + iters):
            self.flush.fill_(i & 1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= warm:
                times.append(e0.elapsed_time(e1))
        times.sort()
        return times[len(times) // 2]


def _roofline_ms(flops: float, bytes_: float, peaks: dict, fp32_flops: float = 0.0) -> float:
    return max(flops / (peaks["bf16_tflops"] * 1e12), bytes_ / (peaks["hbm_gbs"] * 1e9),
               fp32_flops / (peaks["fp32_ffma_tflops_nominal"] * 1e12)) * 1e3


def ffma_peak_tflops() -> float:
    """Nominal float32 throughput of the FFMA pipe: SMs x 128 lanes x 2 x the SM clock (not measured)."""
    p = torch.cuda.get_device_properties(torch.cuda.current_device())
    khz = getattr(p, "clock_rate", 0) or 1_965_000
    return p.multi_processor_count * 128 * 2 * khz * 1e3 / 1e12


def _step_context(engine, lens_before: list, new_tokens: int, vocab: int, seed: int):
    """Slots that hold `lens_before[b]` cached positions each, and the context of a step that brings
    `new_tokens` more tokens to every one of them."""
    rng = random.Random(seed)
    slots = [engine.alloc_slot() for _ in lens_before]
    for s, n in zip(slots, lens_before):
        if n:
            engine.step([s], [[rng.randrange(vocab) for _ in range(n)]], "none")
    tokens = [[rng.randrange(vocab) for _ in range(new_tokens)] for _ in slots]
    ctx = engine.make_context(slots, tokens, [[len(t) - 1] for t in tokens])
    return slots, ctx


def _parts_of(engine):
    block = engine.model.layers[0].block
    return block, engine.cache.layer(0)


def time_parts(engine, kind: str, s: dict, lens_before: list, new_tokens: int, peaks: dict, timer: Timer) -> dict:
    """Milliseconds of one layer's mixer and feed-forward and of their heavy kernels alone, for a step of
    `new_tokens` tokens per sequence on top of `lens_before` cached positions, with each kernel's roofline."""
    from . import attention as attn_kernels, linear, ops
    slots, ctx = _step_context(engine, lens_before, new_tokens, s["vocab"], 5)
    block, cache_layer = _parts_of(engine)
    n = ctx.n_tokens
    residual = torch.zeros(n, s["width"], dtype=torch.float32, device=engine.device)
    x = (torch.randn(n, s["width"], device=engine.device) * 0.5).to(torch.bfloat16)
    hd, heads, kv = s["hd"], s["heads"], s["kv"]
    out = {}
    # pairs of (query, visible key) over the step, for the attention's multiply-adds and bytes
    chunk = s["chunk"] if kind == "lulisun" else 0
    vis = 0
    for before in lens_before:
        for p in range(before, before + new_tokens):
            vis += (p % chunk if chunk else p) + 1
    attn_flops = 4.0 * hd * vis * heads
    kv_bytes = 0
    for before in lens_before:
        last = before + new_tokens - 1
        first = (before // chunk) * chunk if chunk else 0
        kv_bytes += (last + 1 - first) * kv * 2 * hd * 2
    qo_bytes = n * heads * hd * 2 * 2

    def row(name, ms, flops, bytes_, fp32_flops=0.0):
        ideal = _roofline_ms(flops, bytes_, peaks, fp32_flops)
        times = {"tensor": flops / (peaks["bf16_tflops"] * 1e12), "hbm": bytes_ / (peaks["hbm_gbs"] * 1e9),
                 "ffma": fp32_flops / (peaks["fp32_ffma_tflops_nominal"] * 1e12)}
        out[name] = {"ms": round(ms, 4), "roofline_ms": round(ideal, 4), "x_roofline": round(ms / ideal, 2),
                     "bound": max(times, key=times.get)}

    if kind == "lulisun":
        left, right = (m for _, m in block.mixer.members)
        kv_layer, state_layer = cache_layer.parts
        out["mixer_ms"] = round(timer(lambda: block.mixer.forward(x, residual, ctx, cache_layer, True)), 4)
        qkv = torch.randn(n, left.q_dim + left.kv_dim + left.v_dim, device=engine.device).to(torch.bfloat16)
        mixed = torch.empty(n, left.o_dim, dtype=torch.bfloat16, device=engine.device)
        ms = timer(lambda: attn_kernels.attention(qkv, kv_layer, mixed, ctx, n_heads=heads, n_kv_heads=kv, head_dim=hd,
                                                  scale=left.scale, chunk=left.chunk, v_head_dim=left.v_head_dim,
                                                  out_scale=left.out_scale))
        row("attention", ms, attn_flops, kv_bytes + qo_bytes)
        rh = s["rheads"]
        zw = 2 * rh * hd + rh * hd
        z = torch.randn(n, zw, device=engine.device)
        o = torch.empty(n, rh * hd, dtype=torch.bfloat16, device=engine.device)

        piece, most = ops.recurrence_pieces(ctx.max_new, ctx.n_seqs, rh, hd, hd)
        o_raw = torch.empty(n, rh * hd, dtype=torch.float32, device=engine.device)
        scratch = torch.empty(ctx.n_seqs * most * rh * hd * (hd + 1), dtype=torch.float32, device=engine.device) if piece else None

        def recur():
            ops.gated_recurrence(z, right.f_bias, right.lower, right.norm, state_layer.state, ctx.cu_seqlens, ctx.seq_slot, o,
                                 n_seqs=ctx.n_seqs, heads=rh, dim=hd, vdim=hd, eps=1e-5, out_scale=0.7, o_raw=o_raw,
                                 piece=piece, max_pieces=most, scratch=scratch, longest_run=ctx.max_new)
        ms = timer(recur)
        # z read and (its q, f and v columns) written once, o written, the state of every sequence read and written
        rec_bytes = n * zw * 4 * 2 + n * rh * hd * 2 + 2 * len(lens_before) * rh * hd * hd * 4
        # and, per token, head and state element, three float32 multiply-adds that no tensor core may take
        row("recurrence", ms, 0.0, rec_bytes, fp32_flops=6.0 * n * rh * hd * hd)
        ff = block.feed_forward
        out["feed_forward_ms"] = round(timer(lambda: ff.forward(x, residual, ctx)), 4)
        # the routed products alone: routing as the model does it on these activations
        pairs, top, experts, f = n * s["top"], s["top"], s["experts"], s["ff"]
        ids = torch.empty(n, top, dtype=torch.int32, device=engine.device)
        wts = torch.empty(n, top, dtype=torch.float32, device=engine.device)
        gate = torch.empty(n, dtype=torch.float32, device=engine.device)
        ops.moe_route(x, ff.router, ff.correction, ids, wts, top=top, groups=s["groups"], keep=s["keep"],
                      gate_weight=ff.shared_mix, gate_out=gate)
        used = int(torch.unique(ids).numel())
        fast = ff._on_tensor_cores(x)
        from . import tcgen05
        rows = tcgen05.GROUPED_TILE_ROWS if fast else ops.moe_tile_rows()
        i32 = lambda k: torch.zeros(k, dtype=torch.int32, device=engine.device)
        offsets, order, tiles, n_tiles, place = i32(experts + 1), i32(pairs), i32(2 * (-(-pairs // rows) + experts)), i32(1), i32(pairs)
        ops.moe_arrange(ids, pairs, experts, rows, offsets, order, tiles, n_tiles, place)
        act = torch.empty(pairs, f, dtype=torch.bfloat16, device=engine.device)
        y = torch.empty(pairs, s["width"], dtype=torch.float32, device=engine.device)
        if fast:
            xs = torch.empty(pairs, s["width"], dtype=torch.bfloat16, device=engine.device)
            ops.moe_gather(x, xs, order, n_pairs=pairs, top=top)
            ms_up = timer(lambda: tcgen05.grouped_gemm(xs, ff.w_gate, ff.w_up, act, offsets, tiles, n_tiles, n_pairs=pairs))
            ms_down = timer(lambda: tcgen05.grouped_gemm(act, ff.w_down, None, y, offsets, tiles, n_tiles, n_pairs=pairs))
        else:
            ms_up = timer(lambda: ops.moe_grouped_simt(x, ff.w_gate, ff.w_up, act, offsets, order, tiles, n_tiles,
                                                       n_pairs=pairs, top=top))
            ms_down = timer(lambda: ops.moe_grouped_simt(act, ff.w_down, None, y, offsets, order, tiles, n_tiles,
                                                         n_pairs=pairs, top=top))
        out["route_ms"] = round(timer(lambda: ops.moe_route(x, ff.router, ff.correction, ids, wts, top=top, groups=s["groups"],
                                                            keep=s["keep"], gate_weight=ff.shared_mix, gate_out=gate,
                                                            **ff.route_cut(n, ctx))), 4)
        out["arrange_ms"] = round(timer(lambda: ops.moe_arrange(ids, pairs, experts, rows, offsets, order, tiles, n_tiles, place)), 4)
        if fast:
            out["gather_ms"] = round(timer(lambda: ops.moe_gather(x, xs, order, n_pairs=pairs, top=top)), 4)
        out["combine_ms"] = round(timer(lambda: ops.moe_combine(residual, y, wts, top=top, place=place if fast else None)), 4)
        row("experts_gate_up", ms_up, 2.0 * pairs * 2 * f * s["width"],
            used * 2 * f * s["width"] * 2 + pairs * (s["width"] + f) * 2)
        row("experts_down", ms_down, 2.0 * pairs * f * s["width"], used * f * s["width"] * 2 + pairs * (f * 2 + s["width"] * 4))
        out["experts_used"] = used
        out["experts_kernel"] = "tcgen05" if fast else "ffma"
    else:
        mixer, ff = block.mixer, block.feed_forward
        out["mixer_ms"] = round(timer(lambda: mixer.forward(x, residual, ctx, cache_layer, True)), 4)
        qkv = torch.randn(n, mixer.q_dim + 2 * mixer.kv_dim, device=engine.device).to(torch.bfloat16)
        mixed = torch.empty(n, mixer.q_dim, dtype=torch.bfloat16, device=engine.device)
        ms = timer(lambda: attn_kernels.attention(qkv, cache_layer, mixed, ctx, n_heads=heads, n_kv_heads=kv, head_dim=hd,
                                                  scale=mixer.scale))
        row("attention", ms, attn_flops, kv_bytes + qo_bytes)
        out["feed_forward_ms"] = round(timer(lambda: ff.forward(x, residual, ctx)), 4)
        inter = ff.intermediate_size
        act = torch.empty(n, inter, dtype=torch.bfloat16, device=engine.device)
        ms_up = timer(lambda: linear.gated(x, ff.w_gate, ff.w_up, act, ctx))
        ms_down = timer(lambda: linear.into_residual(act, ff.w_down, residual, ctx))
        row("gate_up", ms_up, 2.0 * n * 2 * inter * s["width"], 2 * inter * s["width"] * 2 + n * (s["width"] + inter) * 2)
        row("down", ms_down, 2.0 * n * inter * s["width"], inter * s["width"] * 2 + n * (inter * 2 + s["width"] * 8))
    engine.workspace.rezero()
    for slot in slots:
        engine.free_slot(slot)
    return out


def throughput(engine, s: dict, *, prefill_tokens: int, batch: int, context: int, steps: int, timer: Timer) -> dict:
    from ..sampling.params import SamplerConfig
    rng = random.Random(1)
    prompt = [rng.randrange(s["vocab"]) for _ in range(prefill_tokens)]

    def prefill():
        slot = engine.alloc_slot()
        engine.step([slot], [prompt], "last")
        engine.free_slot(slot)
    pre_ms = timer(prefill, warm=2, iters=5)
    slots = [engine.alloc_slot() for _ in range(batch)]
    for sl in slots:
        engine.step([sl], [[rng.randrange(s["vocab"]) for _ in range(context)]], "none")
    greedy = SamplerConfig.plain(temperature=0.0)
    toks = engine.decode_steps(slots, [1] * batch, 16, greedy)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    toks = engine.decode_steps(slots, toks[-1].tolist(), steps, greedy, on_step=lambda i: e0.record() if i == 0 else None)
    e1.record()
    torch.cuda.synchronize()
    engine.check_device_status()
    ms = e0.elapsed_time(e1) / steps
    for sl in slots:
        engine.free_slot(sl)
    return {"prefill_tokens": prefill_tokens, "prefill_ms": round(pre_ms, 3), "prefill_tok_s": round(prefill_tokens / pre_ms * 1e3, 1),
            "decode_batch": batch, "decode_context": context, "decode_ms_per_step": round(ms, 4),
            "decode_tok_s": round(batch / ms * 1e3, 1)}


def main(sizes: str, peaks: dict, peak_source: str, *, prefill_tokens: int = 2048, batch: int = 8, context: int | None = None,
         steps: int = 64) -> int:
    from ..config.registry import config_from_dict
    from ..engine.engine import Engine
    s = SIZES[sizes]
    if context is None:
        context = s["chunk"] + s["chunk"] // 4        # a quarter into a chunk: the decode step sees that many keys
    torch.cuda.set_device(0)
    timer = Timer("cuda:0")
    peaks = dict(peaks, fp32_ffma_tflops_nominal=round(ffma_peak_tflops(), 1))
    cache_tokens = batch * (context + steps + 128) + prefill_tokens + 4096
    result = {"arch": "lulisun", "sizes": sizes, "config": s, "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
              "peaks": dict(peaks, source=peak_source), "l2": "256 MiB written between timed iterations"}
    for kind, cfg in (("lulisun", lulisun_config(s)), ("dense", dense_config(s, cache_tokens))):
        t0 = time.time()
        engine = Engine.from_random(config_from_dict(cfg), seed=0, std=0.02, dtype="bfloat16", device="cuda:0",
                                    max_tokens=cache_tokens, n_slots=batch + 2)
        print(f"[bench] {kind} ready in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        r = throughput(engine, s, prefill_tokens=prefill_tokens, batch=batch, context=context, steps=steps, timer=timer)
        r["prefill_parts"] = time_parts(engine, kind, s, [0], prefill_tokens, peaks, timer)
        r["decode_parts"] = time_parts(engine, kind, s, [context] * batch, 1, peaks, timer)
        engine.check_device_status()
        result[kind] = r
        del engine
        torch.cuda.empty_cache()
    # how far each kernel of the new design is from its roofline, over the like kernel of the dense decoder
    like = {"attention": "attention", "experts_gate_up": "gate_up", "experts_down": "down"}
    ratios = {}
    for phase in ("prefill_parts", "decode_parts"):
        for name, other in like.items():
            ratios[f"{phase[:-6]}.{name}"] = round(result["lulisun"][phase][name]["x_roofline"]
                                                   / result["dense"][phase][other]["x_roofline"], 2)
        ratios[f"{phase[:-6]}.recurrence (over dense attention)"] = round(
            result["lulisun"][phase]["recurrence"]["x_roofline"] / result["dense"][phase]["attention"]["x_roofline"], 2)
    result["x_roofline_over_dense"] = ratios
    print(json.dumps(result))
    return 0
