"""Attention over the paged cache: which kernel runs, by dtype, head size and step shape.

  bfloat16, head_dim 64 or 128   one token per sequence: split-K over runs of pages
                                 (`attention_mma`); otherwise the tcgen05 flash-style causal
                                 kernel (`attention_tcgen05`), with the mma.sync one behind it
  bfloat16, head_dim 64 or 128,  scores with a cap, a bias by distance, kept first positions, a sink or a
  further forms of the score     gate per head: the mma.sync kernel with those forms (`attention_prefill_forms`),
                                 for prompts and for single tokens
  anything else                  the generic kernel (`attention_generic`): any head size, any
                                 dtype, float32 arithmetic

Besides causality a mixer may limit a query's keys to the last `window` keys or to the query's own
chunk of positions.  The tensor-core kernels take either as one signed span (`csrc/common.cuh:
first_visible_key`); both at once, or values of another head size than the keys', go to the
generic kernel.
"""
from __future__ import annotations

import functools
import os

import torch

from . import ops


@functools.lru_cache(maxsize=None)
def _sm_count() -> int:
    """SMs of the current device (148 on a B200)."""
    return int(torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count)

# RI_B200_PREFILL_ATTENTION=mma keeps the mma.sync prefill kernel (for comparisons)
_PREFILL = os.environ.get("RI_B200_PREFILL_ATTENTION", "tcgen05")
# RI_B200_DECODE_ATTENTION=cluster / cp_async / tma forces one of the decode kernels (default: by batch size)
_DECODE = os.environ.get("RI_B200_DECODE_ATTENTION", "auto")
# RI_B200_SCORE_FORMS_ATTENTION=generic keeps the generic kernel for scores with a cap, a bias, a sink or a gate;
# =prefill keeps the prompts' kernel for steps of one token per sequence too; =mma_prefill keeps the mma.sync kernel for
# prompts whose only forms are a cap and kept first positions (which the tcgen05 kernel takes)
_FORMS = os.environ.get("RI_B200_SCORE_FORMS_ATTENTION", "mma")
CLUSTER_SPLITS = 8     # a thread-block cluster holds at most 8 CTAs portably


def decode_splits(n_seqs: int, n_kv_heads: int, max_seq_len: int, page_size: int, limit: int = 32) -> int:
    """Runs of pages per (sequence, kv head): as many CTAs as are resident at once (two per SM),
    never more, so the grid is one wave; never more runs than the longest sequence has pages.
    Depends on the batch size and the cache geometry only, so a captured step keeps its grid."""
    pairs = max(1, n_seqs * n_kv_heads)
    want = (2 * _sm_count()) // pairs
    if os.environ.get("RI_B200_DECODE_SPLITS"):
        want = int(os.environ["RI_B200_DECODE_SPLITS"])
    return max(1, min(want, limit, -(-max_seq_len // page_size)))


def decode_plan(n_seqs: int, n_kv_heads: int, max_seq_len: int, page_size: int, head_dim: int | None = None):
    """Which decode kernel a step of n_seqs sequences takes, and into how many runs of pages it
    cuts a sequence: ("cluster" | "tma" | "cp_async", splits).  Left to itself it answers "cluster"
    (the TMA-fed kernel with the 2..8 runs of a sequence as one thread-block cluster) while a step's
    sequences x kv heads leave SMs idle, and "tma" (the same kernel, one run per sequence) beyond;
    "cp_async" (pages by cp.async, runs merged through scratch by a second kernel) is only taken
    when RI_B200_DECODE_ATTENTION asks for it: it is the kernel of the allocation-free entry point
    and the comparison for the other two.

    Split runs are merged inside the kernel when the splits of a (sequence, kv head) fit a
    thread-block cluster: no scratch round trip and no second kernel.  With `head_dim` given the
    device is asked how many such clusters it holds at once, and the runs are made fewer until the
    whole step is resident together."""
    if _DECODE in ("auto", "cluster"):
        splits = decode_splits(n_seqs, n_kv_heads, max_seq_len, page_size, CLUSTER_SPLITS)
        if head_dim is not None:
            from . import attention_tc
            while splits >= 2 and attention_tc.decode_cluster_capacity(head_dim, splits) < n_seqs * n_kv_heads:
                splits -= 1
        if splits >= 2:
            return "cluster", splits
    # no clusters (one run per sequence is enough, or the device holds too few): the same kernel, its runs,
    # if any, merged through scratch by a second kernel
    splits = decode_splits(n_seqs, n_kv_heads, max_seq_len, page_size)
    return ("cp_async" if _DECODE == "cp_async" else "tma"), splits


def decode_kernel(name: str):
    if name == "cluster":
        from . import attention_tc
        return attention_tc.decode_cluster
    if name == "tma":
        from . import attention_tc
        return attention_tc.decode
    return ops.attention_decode


def attention(qkv, cache_layer, out, ctx, *, n_heads, n_kv_heads, head_dim, scale, window=0, chunk=0,
              v_head_dim=None, out_scale=1.0, softcap=0.0, keep_first=0, sink=None, dist=None, gate=None):
    """out[t] = softmax(q_t K^T * scale) V over the keys 0..pos(t) of t's slot.  q is the
    leading n_heads*head_dim columns of `qkv`, already rotated.  `window`: only the last so many
    keys; `chunk`: only the keys of the query's own block of that many positions (counted from the
    start of the sequence); `v_head_dim`: values of another head size than keys; `out_scale`: a
    factor on the result.  The tensor-core kernels take a window or a chunk (as one signed span) and
    equal head sizes; values of their own size, or both limits at once, are the generic kernel's.
    `softcap`, `keep_first`, `sink`, `dist`, `gate`: a cap on the scores, first positions that stay visible beyond
    the window, a term without key in the softmax's denominator, a bias by distance and a gate per head on the
    result (see `ops.attention_generic`)."""
    q_ld = qkv.shape[1]
    same_sizes = v_head_dim is None or v_head_dim == head_dim
    plain = not (softcap or keep_first or sink is not None or dist is not None or gate is not None)
    if qkv.dtype == torch.bfloat16 and same_sizes and not (window and chunk) and plain:
        span = window if window else -int(chunk or 0)
        decode = ctx.all_single
        if ops.attention_mma_supports(head_dim, ctx.page_size, n_heads, n_kv_heads, decode):
            if decode:
                max_len = ctx.page_table.shape[1] * ctx.page_size
                name, splits = decode_plan(ctx.n_seqs, n_kv_heads, max_len, ctx.page_size, head_dim)
                part_o = part_ml = None
                if splits > 1 and name != "cluster":
                    part_o = ctx.buffer("attn_part_o", (ctx.n_seqs * n_heads * splits * head_dim,), torch.float32)
                    part_ml = ctx.buffer("attn_part_ml", (ctx.n_seqs * n_heads * splits * 2,), torch.float32)
                decode_kernel(name)(
                    qkv, q_ld, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_len,
                    ctx.cu_seqlens, out, n_seqs=ctx.n_seqs, n_heads=n_heads, n_kv_heads=n_kv_heads,
                    head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=span, n_splits=splits,
                    part_o=part_o, part_ml=part_ml)
                if out_scale != 1.0:
                    ops.scale_(out, out_scale)         # a step's few rows: not worth a parameter of three merges
                return out
            from . import attention_tc
            if _PREFILL != "mma" and attention_tc.supports(head_dim, ctx.page_size, n_heads, n_kv_heads, q_ld,
                                                           out.shape[1]):
                return attention_tc.prefill(
                    qkv, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_start, ctx.cu_seqlens,
                    out, n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=n_heads, n_kv_heads=n_kv_heads,
                    head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=span, out_scale=out_scale)
            ops.attention_prefill(
                qkv, q_ld, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_start,
                ctx.cu_seqlens, out, n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=n_heads,
                n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=span)
            if out_scale != 1.0:
                ops.scale_(out, out_scale)
            return out
    if (qkv.dtype == torch.bfloat16 and same_sizes and not chunk and not plain and _FORMS != "generic"
            and ops.attention_mma_supports(head_dim, ctx.page_size, n_heads, n_kv_heads, False) and q_ld % 8 == 0
            and out.shape[1] % 2 == 0):
        # the forms of the score and the mask on the tensor cores
        if ctx.all_single and n_heads // n_kv_heads <= 16 and _FORMS != "prefill":
            # one token per sequence: the heads of a kv head are one CTA's rows, the sequence's pages cut into runs
            longest = ctx.page_table.shape[1] * ctx.page_size
            if window:
                longest = min(longest, window + keep_first + 2 * ctx.page_size)
            splits = decode_splits(ctx.n_seqs, n_kv_heads, longest, ctx.page_size)
            part_o = part_ml = None
            if splits > 1:
                part_o = ctx.buffer("attn_forms_part_o", (ctx.n_seqs * n_heads * splits * head_dim,), torch.float32)
                part_ml = ctx.buffer("attn_forms_part_ml", (ctx.n_seqs * n_heads * splits * 2,), torch.float32)
            return ops.attention_decode_forms(
                qkv, q_ld, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_len, ctx.cu_seqlens, out,
                n_seqs=ctx.n_seqs, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=ctx.page_size,
                scale=scale, window=window or 0, softcap=softcap, keep_first=keep_first, sink=sink, dist=dist, gate=gate,
                out_scale=out_scale, n_splits=splits, part_o=part_o, part_ml=part_ml)
        # prompts and continuations (and single tokens, if asked for): a cap and kept first positions alone are forms of
        # the tcgen05 kernel; a sink, a bias by distance or a gate per head stay with the mma.sync kernel
        from . import attention_tc
        if (sink is None and dist is None and gate is None and _FORMS != "mma_prefill" and _PREFILL != "mma"
                and not (ctx.all_single and _FORMS == "prefill")
                and attention_tc.supports(head_dim, ctx.page_size, n_heads, n_kv_heads, q_ld, out.shape[1])):
            return attention_tc.prefill(
                qkv, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_start, ctx.cu_seqlens, out,
                n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
                page_size=ctx.page_size, scale=scale, window=window or 0, out_scale=out_scale, softcap=softcap,
                keep_first=keep_first)
        return ops.attention_prefill_forms(
            qkv, q_ld, cache_layer.k, cache_layer.v, ctx.page_table, ctx.seq_slot, ctx.seq_start, ctx.cu_seqlens, out,
            n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
            page_size=ctx.page_size, scale=scale, window=window or 0, softcap=softcap, keep_first=keep_first, sink=sink,
            dist=dist, gate=gate, out_scale=out_scale)
    return ops.attention_generic(
        qkv, q_ld, cache_layer.k, cache_layer.v, ctx.page_table, ctx.token_pos, ctx.token_seq,
        ctx.seq_slot, out, n_tokens=qkv.shape[0], n_heads=n_heads, n_kv_heads=n_kv_heads,
        head_dim=head_dim, page_size=ctx.page_size, scale=scale, window=window, chunk=chunk or 0,
        v_head_dim=v_head_dim, out_scale=out_scale, softcap=softcap, keep_first=keep_first, sink=sink, dist=dist,
        gate=gate)


# RI_B200_LATENT_ATTENTION=generic keeps the generic kernel for attention over a shared latent (for comparisons)
_LATENT = os.environ.get("RI_B200_LATENT_ATTENTION", "mma")
LATENT_TILE_KEYS = 32


def latent_splits(n_ctas: int, longest: int, tile_rows: int) -> int:
    """Runs of keys per sequence for a step whose row tiles alone make n_ctas CTAs: as many as fill the SMs once
    (the kernel holds one CTA per SM, two of its smallest), never more than the longest sequence has key tiles."""
    per_sm, most = (2, 32) if tile_rows <= 16 else (1, 16)
    return max(1, min(most, per_sm * _sm_count() // max(1, n_ctas), -(-longest // LATENT_TILE_KEYS)))


def latent_attention(q_wide, cache_layer, out, ctx, *, n_heads, key_dim, rank, scale):
    """Attention of n_heads query heads over ONE kv head whose keys are the cached rows [key_dim] and whose
    values are the rows' first `rank` channels (no storage of their own); causal.  q_wide is
    [T, n_heads * key_dim]; out is head-major, [n_heads, T, rank].  bfloat16 with a latent the tensor-core kernel
    is built for: `latent_attention_mma` (steps of few rows cut the keys into runs); anything else: the generic
    kernel."""
    rd = key_dim - rank
    if q_wide.dtype == torch.bfloat16 and _LATENT != "generic" and ops.latent_attention_mma_supports(rank, rd, ctx.page_size):
        n = q_wide.shape[0]
        rows = ctx.max_new * n_heads
        tile_rows = ops.latent_attention_mma_tile_rows(rows, rank)
        tiles = -(-rows // tile_rows)
        # a decode step's grid may depend on the batch size and the cache geometry only (captured steps)
        longest = ctx.page_table.shape[1] * ctx.page_size if ctx.all_single else ctx.max_len
        splits = latent_splits(tiles * ctx.n_seqs, longest, tile_rows)
        part_o = part_ml = None
        if splits > 1:
            part_o = ctx.buffer("latent_part_o", (n * n_heads * splits * rank,), torch.float32)
            part_ml = ctx.buffer("latent_part_ml", (n * n_heads * splits * 2,), torch.float32)
        return ops.latent_attention_mma(q_wide, cache_layer.k, ctx.page_table, ctx.seq_slot, ctx.seq_start, ctx.cu_seqlens,
                                        out, n_seqs=ctx.n_seqs, max_new=ctx.max_new, n_heads=n_heads, rank=rank, rot_dim=rd,
                                        scale=scale, n_splits=splits, part_o=part_o, part_ml=part_ml)
    return ops.attention_generic(
        q_wide, q_wide.shape[1], cache_layer.k, cache_layer.k, ctx.page_table, ctx.token_pos, ctx.token_seq,
        ctx.seq_slot, out, n_tokens=q_wide.shape[0], n_heads=n_heads, n_kv_heads=1, head_dim=key_dim,
        page_size=ctx.page_size, scale=scale, v_head_dim=rank, values_in_keys=True, head_major=True)
