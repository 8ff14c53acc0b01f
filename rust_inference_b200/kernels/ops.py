"""Python faces of the CUDA kernels: they check the tensors they are given, pass raw
pointers and the current CUDA stream to the C ABI, and raise on any error.

There is no other implementation behind them.  A tensor that is not on a CUDA device,
a missing compiler or a library that does not load is an error, never a detour.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_float, c_void_p, c_longlong, c_ulonglong

import math

import torch

from .build import load

RI_F32, RI_BF16 = 0, 1
_DTYPE_CODE = {torch.float32: RI_F32, torch.bfloat16: RI_BF16}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def _p(t) -> c_void_p:
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel called with a tensor that is not on a CUDA device; "
                              "this library has no CPU path")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise KernelError(msg)


_launches = 0


def launch_count() -> int:
    """How many kernel entry points have been called (each launches one kernel)."""
    return _launches


_limits = None          # checked build: (vocabulary, slots, pages) for libraries still to be loaded
_limited: set = set()   # libraries that have them


def _call(module: str, fn: str, *args) -> None:
    global _launches
    lib = load(module)
    if _limits is not None and module not in _limited:
        _apply_limits(module, lib)
    rc = getattr(lib, fn)(*args)
    if rc != 0:
        raise KernelError(f"{fn}: {lib.ri_last_error().decode()}")
    _launches += 1


# ----------------------------------------------------------------------------
# The checked build (RI_B200_CHECK_BOUNDS=1)
# ----------------------------------------------------------------------------
BOUND_CHECKS = {1: "a token id outside the vocabulary", 2: "a cache slot that does not exist",
                3: "a position beyond a sequence's page table", 4: "a page that does not exist"}


def checked_build() -> bool:
    from . import build
    return build.CHECKED


def _apply_limits(module: str, lib) -> None:
    from . import build
    if build.MODULES[module].endswith(".cu"):
        if lib.ri_bounds_set_limits(c_int(_limits[0]), c_int(_limits[1]), c_int(_limits[2])) != 0:
            raise KernelError(f"{module}: {lib.ri_last_error().decode()}")
    _limited.add(module)


def bounds_set_limits(vocab: int, slots: int, pages: int) -> None:
    """Checked build only: the limits that kernels are not given as arguments (0: not checked), for
    every CUDA library loaded so far and, at its first call, every one loaded later."""
    global _limits
    from . import build
    _limits = (int(vocab), int(slots), int(pages))
    _limited.clear()
    for module in build.loaded_cuda_modules():
        _apply_limits(module, load(module))


def bounds_report() -> list:
    """Checked build only: what the kernels recorded since the last call, per library:
    (library, what was outside, the index, its limit, how many indices were outside).  Reads the
    records back (synchronises the device) and clears them."""
    from . import build
    out = []
    for module in build.loaded_cuda_modules():
        lib = load(module)
        rec = (c_int * 4)()
        if lib.ri_bounds_report(rec) != 0:
            raise KernelError(f"{module}: {lib.ri_last_error().decode()}")
        if rec[3]:
            out.append((module, BOUND_CHECKS.get(rec[0], f"check {rec[0]}"), rec[1], rec[2], rec[3]))
    return out


# ----------------------------------------------------------------------------
# The timeline build (RI_B200_TIMELINE=1)
# ----------------------------------------------------------------------------
TIMELINE_PHASES = 6


def timeline_build() -> bool:
    from . import build
    return build.TIMELINE


def timeline_read(strict: bool = True) -> list:
    """Timeline build only: one record per kernel launched since the last call, in the order the kernels
    came onto the device: {"module", "entry_ns", "entry_line", "wait_ns", "wait_line", "phases_ns"} with
    the device-wide timer's values (0: that mark was not passed) and the source lines of the kernel's
    `let_next_kernel_start()` and `wait_for_previous_kernels()`.  Synchronises the device and clears
    the records.  `strict`: raise when launches fell on the same record (thousands since the last read)."""
    import ctypes
    from . import build
    words = 5 + TIMELINE_PHASES
    cap = 4096
    out = []
    for module in build.loaded_cuda_modules():
        lib = load(module)
        buf = (ctypes.c_ulonglong * (cap * words))()
        n = lib.ri_timeline_read(buf, c_int(cap))
        if n < 0:
            raise KernelError(f"{module}: {lib.ri_last_error().decode()}")
        found = 0
        for i in range(cap):
            if buf[i * words]:
                r = buf[i * words:(i + 1) * words]
                out.append({"module": module, "entry_ns": r[0], "entry_line": r[1], "wait_ns": r[2], "wait_line": r[3],
                            "grid": r[4] - 1, "phases_ns": list(r[5:])})
                found += 1
        if strict and found != n:
            raise KernelError(f"{module}: {n} launches since the last read but {found} records: launches fell on "
                              f"the same record (the timeline keeps {cap})")
    out.sort(key=lambda r: r["entry_ns"])
    return out


# ----------------------------------------------------------------------------
def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """out[t, :] = table[ids[t], :] * scale, widened to float32 first.  ids: int32 [T]; out: float32 [T, H]."""
    _need_cuda(table, ids, out)
    n, hidden = out.shape
    _need(ids.dtype == torch.int32 and ids.numel() == n, "embed_gather: ids must be int32 [T]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
          and table.shape[1] == hidden, "embed_gather: bad out/table")
    _call("elementwise", "ri_embed_gather", _p(table), c_int(dtype_code(table.dtype)), _p(ids), _p(out),
          c_int(n), c_int(hidden), c_float(scale), _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, :] = rmsnorm(x[rows[r] or r, :]) * weight.  x, weight float32; out float32 or bfloat16."""
    _need_cuda(x, weight, out, rows)
    n_rows, n = out.shape
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32, "rmsnorm: x and weight must be float32")
    _need(x.is_contiguous() and out.is_contiguous() and x.shape[-1] == n and weight.numel() == n,
          "rmsnorm: bad shapes")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() == n_rows, "rmsnorm: rows must be int32 [R]")
    else:
        _need(x.shape[0] >= n_rows, "rmsnorm: x has fewer rows than out")
    _call("elementwise", "ri_rmsnorm", _p(x), _p(weight), _p(rows), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n_rows), c_int(n), c_float(eps), _stream())
    return out


def rmsnorm_pair(x: torch.Tensor, weight_a: torch.Tensor, weight_b: torch.Tensor, eps: float, out_a: torch.Tensor,
                 out_b: torch.Tensor) -> None:
    """out_a = rmsnorm(x) * weight_a and out_b = rmsnorm(x) * weight_b of the same rows with one pass over the
    statistics.  x and the weights float32; the outputs float32 or bfloat16, [R, n] each."""
    _need_cuda(x, weight_a, weight_b, out_a, out_b)
    n_rows, n = out_a.shape
    _need(x.dtype == torch.float32 and weight_a.dtype == torch.float32 and weight_b.dtype == torch.float32
          and x.is_contiguous() and x.shape[-1] == n and x.shape[0] >= n_rows and weight_a.numel() == n
          and weight_b.numel() == n, "rmsnorm_pair: x and the weights must be float32 [.., n]")
    _need(out_b.shape == out_a.shape and out_b.dtype == out_a.dtype and out_a.is_contiguous() and out_b.is_contiguous(),
          "rmsnorm_pair: two outputs of one shape and dtype")
    _call("elementwise", "ri_rmsnorm_pair", _p(x), _p(weight_a), _p(weight_b), _p(out_a), _p(out_b),
          c_int(dtype_code(out_a.dtype)), c_int(n_rows), c_int(n), c_float(eps), _stream())


def layernorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
              rows: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, :] = (x - mean) / sqrt(var + eps) * weight of the row x[rows[r] or r, :] (no bias; var: the mean of
    the squared deviations).  x, weight float32; out float32 or bfloat16."""
    _need_cuda(x, weight, out, rows)
    n_rows, n = out.shape
    _need(x.dtype == torch.float32 and weight.dtype == torch.float32, "layernorm: x and weight must be float32")
    _need(x.is_contiguous() and out.is_contiguous() and x.shape[-1] == n and weight.numel() == n,
          "layernorm: bad shapes")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() == n_rows, "layernorm: rows must be int32 [R]")
    else:
        _need(x.shape[0] >= n_rows, "layernorm: x has fewer rows than out")
    _call("elementwise", "ri_layernorm", _p(x), _p(weight), _p(rows), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n_rows), c_int(n), c_float(eps), _stream())
    return out


def rope_normed_cache_write(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, q_weight, k_weight, eps: float,
                            token_pos, token_seq, seq_slot, page_table: torch.Tensor, kcache, vcache, *, n_heads: int,
                            n_kv_heads: int, head_dim: int, page_size: int, style: int, write_kv: bool,
                            rot_dims: int | None = None, v_head_dim: int | None = None, values_from_keys: bool = False) -> None:
    """`rope_cache_write` for heads that are RMS-normalised before they are rotated: every q head times
    q_weight / rms (float32 [head_dim], shared by the heads; None: not normalised), every k head likewise
    with k_weight.  With values_from_keys qkv holds no values: the cache's values are the key heads as
    projected, before norm and rotation."""
    _need_cuda(qkv, cos, sin, q_weight, k_weight, token_pos, token_seq, seq_slot, page_table, kcache, vcache)
    n = qkv.shape[0]
    rot = head_dim if rot_dims is None else int(rot_dims)
    v_hd = head_dim if v_head_dim is None else int(v_head_dim)
    cols = (n_heads + n_kv_heads) * head_dim + (0 if values_from_keys else n_kv_heads * v_hd)
    _need(qkv.is_contiguous() and qkv.shape[1] >= cols, "rope_normed_cache_write: qkv holds too few columns")
    _need(0 <= rot <= head_dim and rot % 2 == 0, "rope_normed_cache_write: rotated channels must be even and at most head_dim")
    _need(not values_from_keys or v_hd == head_dim, "rope_normed_cache_write: values taken from the keys have their size")
    _need(rot == 0 or (cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[1] == rot // 2
                       and cos.is_contiguous() and sin.is_contiguous()),
          "rope_normed_cache_write: tables must be float32 [positions, rotated channels / 2]")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.is_contiguous() and w.numel() == head_dim),
              "rope_normed_cache_write: norm weights must be float32 [head_dim]")
    if write_kv:
        _need(kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous()
              and vcache.is_contiguous(), "rope_normed_cache_write: cache dtype/layout")
        _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim)
              and tuple(vcache.shape[1:]) == (n_kv_heads, page_size, v_hd), "rope_normed_cache_write: cache shape")
    _call("elementwise", "ri_rope_normed_cache_write", _p(qkv), c_int(dtype_code(qkv.dtype)), c_int(qkv.shape[1]),
          _p(cos), _p(sin), _p(q_weight), _p(k_weight), c_float(eps), _p(token_pos), _p(token_seq), _p(seq_slot),
          _p(page_table), c_int(page_table.shape[1]), _p(kcache), _p(vcache), c_int(n), c_int(n_heads), c_int(n_kv_heads),
          c_int(head_dim), c_int(page_size), c_int(style), c_int(1 if write_kv else 0), c_int(rot if rot else -1), c_int(v_hd),
          c_int(1 if values_from_keys else 0), _stream())


def rope_cache_write(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, token_pos, token_seq,
                     seq_slot, page_table: torch.Tensor, kcache, vcache, *, n_heads: int,
                     n_kv_heads: int, head_dim: int, page_size: int, style: int, write_kv: bool,
                     rot_dims: int | None = None, v_head_dim: int | None = None) -> None:
    """Rotate q (in place) and k by the table rows of each token's position; store rotated k and v
    at the token's cache position.  kcache: one layer, [pages, kv heads, page_size, head_dim]; vcache
    the same with v_head_dim (default: head_dim).  rot_dims: only the first so many channels of a
    head are rotated (default: all), the tables then having rot_dims/2 columns; 0: nothing is rotated (no
    tables), keys and values are only stored.  A row of qkv may hold more columns after these (they are left
    alone), and without write_kv only the query columns need to be there."""
    _need_cuda(qkv, cos, sin, token_pos, token_seq, seq_slot, page_table, kcache, vcache)
    n = qkv.shape[0]
    rot = head_dim if rot_dims is None else int(rot_dims)
    v_hd = head_dim if v_head_dim is None else int(v_head_dim)
    _need(qkv.is_contiguous() and qkv.shape[1] >= n_heads * head_dim + ((n_kv_heads * (head_dim + v_hd)) if write_kv else 0),
          "rope_cache_write: qkv must be [T, (heads + kv heads) * head_dim + kv heads * value head size (or more)]")
    _need(0 <= rot <= head_dim and rot % 2 == 0, "rope_cache_write: rotated channels must be even and at most head_dim")
    _need(rot == 0 or (cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[1] == rot // 2
                       and cos.is_contiguous() and sin.is_contiguous()),
          "rope_cache_write: tables must be float32 [positions, rotated channels / 2]")
    if write_kv:
        _need(kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype and kcache.is_contiguous()
              and vcache.is_contiguous(), "rope_cache_write: cache dtype/layout")
        _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim)
              and tuple(vcache.shape[1:]) == (n_kv_heads, page_size, v_hd), "rope_cache_write: cache shape")
    _call("elementwise", "ri_rope_cache_write", _p(qkv), c_int(dtype_code(qkv.dtype)), c_int(qkv.shape[1]),
          _p(cos), _p(sin), _p(token_pos), _p(token_seq), _p(seq_slot), _p(page_table),
          c_int(page_table.shape[1]), _p(kcache), _p(vcache), c_int(n), c_int(n_heads), c_int(n_kv_heads),
          c_int(head_dim), c_int(page_size), c_int(style), c_int(1 if write_kv else 0), c_int(rot), c_int(v_hd),
          _stream())


def rope_cache_write_acc(acc: torch.Tensor, bias, q_out: torch.Tensor, cos, sin, token_pos, token_seq, seq_slot,
                         page_table, kcache, vcache, *, n_heads: int, n_kv_heads: int, head_dim: int,
                         page_size: int, style: int, write_kv: bool) -> None:
    """The rotary + cache-write kernel fed from float32 accumulators acc[T, (heads + 2 kv heads) * head_dim]
    (+ bias): q goes to q_out[T, heads * head_dim], k and v to the cache, and `acc` is zeroed again."""
    _need_cuda(acc, bias, q_out, cos, sin, token_pos, token_seq, seq_slot, page_table, kcache, vcache)
    n = acc.shape[0]
    _need(acc.dtype == torch.float32 and acc.is_contiguous()
          and acc.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim, "rope_cache_write_acc: accumulator shape")
    _need(q_out.is_contiguous() and q_out.shape == (n, n_heads * head_dim), "rope_cache_write_acc: q_out shape")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == acc.shape[1]), "rope_cache_write_acc: bias")
    if write_kv:
        _need(kcache.dtype == q_out.dtype and vcache.dtype == q_out.dtype
              and tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim), "rope_cache_write_acc: cache")
    _call("elementwise", "ri_rope_cache_write_acc", _p(acc), c_int(acc.shape[1]), _p(bias), _p(q_out),
          c_int(dtype_code(q_out.dtype)), _p(cos), _p(sin), _p(token_pos), _p(token_seq), _p(seq_slot),
          _p(page_table), c_int(page_table.shape[1]), _p(kcache), _p(vcache), c_int(n), c_int(n_heads),
          c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_int(style), c_int(1 if write_kv else 0), _stream())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _need_cuda(gate_up, out)
    n, inter = out.shape
    _need(gate_up.shape == (n, 2 * inter) and gate_up.dtype == out.dtype and gate_up.is_contiguous()
          and out.is_contiguous(), "silu_mul: bad shapes")
    _call("elementwise", "ri_silu_mul", _p(gate_up), _p(out), c_int(dtype_code(out.dtype)), c_int(n),
          c_int(inter), _stream())
    return out


# epilogues of the contractions
EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL, EPI_SILU_MUL, EPI_ACT = 0, 1, 2, 3, 4


GELU_TANH_ALPHA = 2.0 * math.sqrt(2.0 / math.pi)      # 0.5 z (1 + tanh(y)) = z sigmoid(2 y)
GELU_TANH_CUBIC = 0.044715


def gate_form(*, alpha: float = 1.0, limit: float = float("inf"), shift: float = 0.0, cubic: float = 0.0,
              mult: float = 1.0, device="cuda") -> torch.Tensor:
    """The five constants of the gated epilogue on the device: the gate is
    mult * g' sigmoid(alpha g' (1 + cubic g'^2)) (u' + shift) with g' = min(g, limit), u' = clamp(u, -limit, limit).
    The defaults are SiLU(g) * u; GELU_TANH_ALPHA and GELU_TANH_CUBIC make the gate the tanh form of GELU."""
    return torch.tensor([alpha, limit, shift, cubic, mult], dtype=torch.float32, device=device)


def whole_gate_form(form: torch.Tensor) -> torch.Tensor:
    """A form given as its first three constants (alpha, limit, shift) gets cubic 0 and mult 1."""
    if form.numel() == 3:
        return torch.cat([form.reshape(-1), form.new_tensor([0.0, 1.0])])
    return form


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int, *,
              bias: torch.Tensor | None = None, w2: torch.Tensor | None = None,
              gate_form: torch.Tensor | None = None, act_form: torch.Tensor | None = None) -> torch.Tensor:
    """out = x @ w.T with the chosen epilogue, on the FFMA pipe (float32 accumulate).  gate_form (gated
    epilogue only): float32 [5] on the device (`gate_form`; the first three alone are accepted), {alpha, limit, shift, cubic, mult} of mult g' sigmoid(alpha g' (1 + cubic g'^2)) (u' + shift) with
    g' = min(g, limit), u' = clamp(u, -limit, limit); None: SiLU(g) * u.  act_form (EPI_ACT only): float32 [2] on the
    device, the two constants of the learned activation (`xielu`)."""
    _need_cuda(x, w, out, bias, w2)
    m, k = x.shape
    n = w.shape[0]
    _need(w.shape[1] == k and x.dtype == w.dtype and x.is_contiguous() and w.is_contiguous()
          and out.is_contiguous() and out.shape == (m, n), "gemm: bad shapes")
    want_out = torch.float32 if mode in (EPI_STORE_F32, EPI_RESIDUAL) else x.dtype
    _need(out.dtype == want_out, f"gemm: epilogue {mode} writes {want_out}, out is {out.dtype}")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == n, "gemm: bias must be float32 [N]")
    if w2 is not None:
        _need(w2.shape == w.shape and w2.dtype == w.dtype and w2.is_contiguous(), "gemm: second matrix")
    if gate_form is not None:
        gate_form = whole_gate_form(gate_form)
        _need(mode == EPI_SILU_MUL and bias is None and gate_form.is_cuda and gate_form.dtype == torch.float32
              and gate_form.numel() == 5, "gemm: a gate form is five float32 constants of the gated epilogue")
        bias = gate_form                      # the gated epilogue takes no bias: its constants travel in that argument
    _need((mode == EPI_ACT) == (act_form is not None), "gemm: the activation epilogue and its constants go together")
    if act_form is not None:
        _need(bias is None and act_form.is_cuda and act_form.dtype == torch.float32 and act_form.numel() == 2,
              "gemm: an activation's form is two float32 constants, and its epilogue takes no bias")
        bias = act_form
    _call("gemm_simt", "ri_gemm_simt", _p(x), _p(w), _p(w2), _p(bias), _p(out), c_int(dtype_code(x.dtype)),
          c_int(mode), c_int(m), c_int(n), c_int(k), _stream())
    return out


def attention_generic(q: torch.Tensor, q_ld: int, kcache, vcache, page_table, token_pos, token_seq,
                      seq_slot, out: torch.Tensor, *, n_tokens: int, n_heads: int, n_kv_heads: int,
                      head_dim: int, page_size: int, scale: float, window: int = 0, chunk: int = 0,
                      v_head_dim: int | None = None, out_scale: float = 1.0, values_in_keys: bool = False,
                      head_major: bool = False, softcap: float = 0.0, keep_first: int = 0, sink=None, dist=None,
                      gate=None) -> torch.Tensor:
    """Attention of every given token over its slot's cached keys 0..position (any sizes), limited to
    the last `window` keys and / or to the query's own block of `chunk` positions when those are not 0;
    values of head size v_head_dim (default: head_dim); the result times out_scale.  values_in_keys: the
    values are the first v_head_dim channels of the keys (vcache is not read).  head_major: out is
    [heads, tokens, v_head_dim] instead of [tokens, heads * v_head_dim].  softcap: scores become
    softcap * tanh(score / softcap); dist (float32 [2, heads]: r1, r2): r1 ln(1 + r2 (pos - key)) is taken off the
    score; keep_first: with a window, the first so many positions stay visible; sink (float32 [heads]): one more
    term exp(sink) in the softmax's denominator; gate ([tokens, >= heads] in q's dtype, a view is fine): the head's
    result times the sigmoid of its entry."""
    _need_cuda(q, kcache, vcache, page_table, token_pos, token_seq, seq_slot, out, sink, dist, gate)
    _need(sink is None or (sink.dtype == torch.float32 and sink.is_contiguous() and sink.numel() == n_heads),
          "attention: sink must be float32 [heads]")
    _need(dist is None or (dist.dtype == torch.float32 and dist.is_contiguous() and dist.numel() == 2 * n_heads),
          "attention: dist must be float32 [2, heads]")
    _need(gate is None or (gate.dtype == q.dtype and gate.stride(1) == 1 and gate.shape[0] == n_tokens
                           and gate.shape[1] >= n_heads), "attention: gate must be [tokens, heads] in q's dtype")
    _need(not keep_first or window > 0, "attention: kept first positions go with a window")
    v_hd = head_dim if v_head_dim is None else int(v_head_dim)
    if values_in_keys:
        _need(v_hd <= head_dim, "attention: values inside keys cannot be wider than the keys")
        vcache = kcache
    _need(q.dtype == kcache.dtype == vcache.dtype == out.dtype, "attention: dtypes differ")
    _need(out.is_contiguous() and out.numel() == n_tokens * n_heads * v_hd, "attention: out shape")
    _need(tuple(kcache.shape[1:]) == (n_kv_heads, page_size, head_dim)
          and (values_in_keys or tuple(vcache.shape[1:]) == (n_kv_heads, page_size, v_hd))
          and kcache.shape[0] == vcache.shape[0], "attention: cache shape")
    rows = kcache.shape[0] * kcache.shape[1] * kcache.shape[2]
    out_ld = v_hd if head_major else n_heads * v_hd
    out_hs = n_tokens * v_hd if head_major else v_hd
    _call("attention_generic", "ri_attention_generic", _p(q), c_int(q_ld), _p(kcache), _p(vcache),
          _p(page_table), c_int(page_table.shape[1]), _p(token_pos), _p(token_seq), _p(seq_slot), _p(out),
          c_int(out_ld), c_int(dtype_code(q.dtype)), c_int(n_tokens), c_int(n_heads),
          c_int(n_kv_heads), c_int(head_dim), c_int(v_hd), c_int(page_size), c_longlong(rows), c_float(scale),
          c_int(window), c_int(chunk), c_float(out_scale), c_int(head_dim if values_in_keys else v_hd),
          c_longlong(out_hs), c_float(softcap), c_int(keep_first), _p(sink), _p(dist), _p(gate),
          c_int(gate.stride(0) if gate is not None else 0), _stream())
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, *, temperature: float, top_k: int = 0, top_p: float = 1.0,
           penalty: float = 1.0, recent: torch.Tensor | None = None, recent_count: torch.Tensor | None = None,
           seed: int = 0, row_stream: torch.Tensor | None = None,
           row_counter: torch.Tensor | None = None, counter_offset: int = 0,
           mirror: torch.Tensor | None = None, newest: torch.Tensor | None = None,
           seed_dev: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V] (overwritten).  out: int32 [R].  `mirror`: a
    pinned int32 host tensor [R] that receives the tokens as well (the kernel writes it directly).
    `newest`: int32 [R] on the device, one more recent id per row for the repetition penalty.
    `seed_dev`: int64 [1] on the device, a seed that takes the place of `seed` (read when the kernel runs)."""
    _need(seed_dev is None or (seed_dev.is_cuda and seed_dev.dtype == torch.int64 and seed_dev.numel() >= 1),
          "sample: seed_dev must be int64 [1] on the device")
    _need_cuda(logits, out, recent, recent_count, row_stream, row_counter, newest)
    _need(newest is None or (newest.dtype == torch.int32 and newest.is_contiguous() and newest.numel() >= logits.shape[0]),
          "sample: newest must be int32 [R]")
    rows, vocab = logits.shape
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "sample: logits must be contiguous float32")
    _need(out.dtype == torch.int32 and out.numel() >= rows, "sample: out must be int32 [R]")
    for t in (recent, recent_count, row_stream, row_counter):
        _need(t is None or (t.dtype == torch.int32 and t.is_contiguous()), "sample: index tensors must be int32")
    _need((recent is None) == (recent_count is None), "sample: recent and recent_count go together")
    if mirror is not None:
        _need(mirror.device.type == "cpu" and mirror.is_pinned() and mirror.dtype == torch.int32
              and mirror.is_contiguous() and mirror.numel() >= rows, "sample: mirror must be pinned int32 [R]")
    _call("sampling", "ri_sample", _p(logits), c_int(rows), c_int(vocab), _p(out), c_float(temperature),
          c_int(top_k), c_float(top_p), c_float(penalty), _p(recent),
          c_int(recent.shape[1] if recent is not None else 0), _p(recent_count),
          c_ulonglong(seed & 0xFFFFFFFFFFFFFFFF), _p(row_stream), _p(row_counter), c_int(counter_offset),
          c_void_p(mirror.data_ptr() if mirror is not None else 0), _p(newest), _p(seed_dev), _stream())
    return out


def cast(src: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """src (float32 or bfloat16, contiguous, on the device) in the other of the two precisions."""
    _need_cuda(src)
    _need(src.is_contiguous(), "cast: contiguous tensors only")
    out = torch.empty(src.shape, dtype=dtype, device=src.device)
    _call("elementwise", "ri_cast", _p(src), c_int(dtype_code(src.dtype)), _p(out), c_int(dtype_code(dtype)),
          c_longlong(src.numel()), _stream())
    return out


def stream_add(x: torch.Tensor, other: torch.Tensor | None = None, row: torch.Tensor | None = None) -> torch.Tensor:
    """x += other + row in place: x float32 [T, width], other the same shape or None, row float32 [width] or None."""
    _need_cuda(x, other, row)
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "stream_add: x must be contiguous float32 [T, width]")
    _need(other is None or (other.dtype == torch.float32 and other.is_contiguous() and other.shape == x.shape),
          "stream_add: other must have x's shape")
    _need(row is None or (row.dtype == torch.float32 and row.is_contiguous() and row.numel() == x.shape[1]),
          "stream_add: row must be float32 [width]")
    _call("elementwise", "ri_stream_add", _p(x), _p(other), _p(row), c_int(x.shape[0]), c_int(x.shape[1]), _stream())
    return x


def sigmoid_gate_(x: torch.Tensor, gate: torch.Tensor, gate_col: int = 0, factor: float = 1.0) -> torch.Tensor:
    """x *= sigmoid(gate[:, gate_col : gate_col + width]) * factor in place (float32 arithmetic, one rounding); x
    contiguous [T, width], gate contiguous [T, >= gate_col + width] of the same dtype."""
    _need_cuda(x, gate)
    _need(x.is_contiguous() and gate.is_contiguous() and x.dim() == 2 and gate.dim() == 2 and gate.dtype == x.dtype
          and gate.shape[0] == x.shape[0] and gate.shape[1] >= gate_col + x.shape[1] and gate_col >= 0,
          "sigmoid_gate: x [T, width] and gate [T, >= gate_col + width] of one dtype")
    _call("elementwise", "ri_sigmoid_gate", _p(x), _p(gate), c_int(dtype_code(x.dtype)), c_int(gate.shape[1]), c_int(gate_col),
          c_int(x.shape[0]), c_int(x.shape[1]), c_float(factor), _stream())
    return x


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x = cap * tanh(x / cap) in place; x float32, contiguous."""
    _need_cuda(x)
    _need(x.dtype == torch.float32 and x.is_contiguous() and cap > 0, "softcap: contiguous float32 and a positive cap")
    _call("elementwise", "ri_softcap", _p(x), c_longlong(x.numel()), c_float(cap), _stream())
    return x


def scale_(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x *= factor in place (float32 arithmetic, one rounding); x float32 or bfloat16, contiguous, on the device."""
    _need_cuda(x)
    _need(x.is_contiguous(), "scale_: contiguous tensors only")
    _call("elementwise", "ri_scale", _p(x), c_int(dtype_code(x.dtype)), c_longlong(x.numel()), c_float(factor), _stream())
    return x


def fill_normal(out: torch.Tensor, key: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
    """out[i] = mean + std * z_i with z_i a standard normal number that depends on (key, i) only
    (`sampling.rng.normal` restates it on the host).  out: float32 or bfloat16, contiguous, on the device."""
    _need_cuda(out)
    _need(out.is_contiguous(), "fill_normal: contiguous tensors only")
    _call("elementwise", "ri_fill_normal", _p(out), c_int(dtype_code(out.dtype)), c_longlong(out.numel()),
          c_ulonglong(key & 0xFFFFFFFFFFFFFFFF), c_float(mean), c_float(std), _stream())
    return out


def advance_decode(token_pos: torch.Tensor, seq_start: torch.Tensor, seq_len: torch.Tensor, token_ids: torch.Tensor,
                   *, draw_counter: torch.Tensor | None = None, turn: torch.Tensor | None = None,
                   host_ring: torch.Tensor | None = None, log_ring: torch.Tensor | None = None) -> None:
    """The end of a decode step: positions, starts and lengths (int32 [n] each) grow by one in
    place.  Optionally the sampler's draw counters grow by one, and the step's tokens are copied
    into slot (turn % slots) of `host_ring` (pinned int32 [slots, n]) and of `log_ring` (device int32
    [slots, n]); `turn` (device int32 [1]) then grows by one."""
    n = token_pos.numel()
    _need_cuda(token_pos, seq_start, seq_len, token_ids, draw_counter, turn, log_ring)
    for t in (token_pos, seq_start, seq_len, token_ids, draw_counter, turn, log_ring):
        _need(t is None or (t.dtype == torch.int32 and t.is_contiguous()), "advance_decode: arrays must be int32")
    _need(seq_start.numel() == n and seq_len.numel() == n and token_ids.numel() >= n
          and (draw_counter is None or draw_counter.numel() >= n), "advance_decode: one entry per sequence")
    if host_ring is not None:
        _need(host_ring.device.type == "cpu" and host_ring.is_pinned() and host_ring.dtype == torch.int32
              and host_ring.is_contiguous() and host_ring.ndim == 2 and host_ring.shape[1] == n,
              "advance_decode: host_ring must be pinned int32 [slots, n]")
    if log_ring is not None:
        _need(log_ring.ndim == 2 and log_ring.shape[1] == n, "advance_decode: log_ring must be int32 [slots, n]")
    _need((host_ring is None and log_ring is None) or turn is not None, "advance_decode: rings need the turn counter")
    _call("elementwise", "ri_advance_decode", _p(token_pos), _p(seq_start), _p(seq_len), c_int(n), _p(token_ids),
          _p(draw_counter), _p(turn), c_void_p(host_ring.data_ptr() if host_ring is not None else 0),
          c_int(host_ring.shape[0] if host_ring is not None else 0), _p(log_ring),
          c_int(log_ring.shape[0] if log_ring is not None else 0), _stream())


def sample_cluster_min_vocab(vocab: int) -> None:
    """Rows of at least `vocab` entries are sampled by a cluster of thread blocks where the options
    allow it (0: never; the library's default is 32,768).  For comparisons and tests."""
    load("sampling").ri_sample_set_cluster_min_vocab(c_int(vocab))


def sample_cluster_any_rows(on: bool) -> None:
    """Whether such rows are sampled by clusters however many rows a call brings (the library's default:
    only while the clusters are few enough to run together; more rows take a block each).  For
    comparisons and tests."""
    load("sampling").ri_sample_set_cluster_any_rows(c_int(1 if on else 0))


def attention_mma_supports(head_dim: int, page_size: int, n_heads: int, n_kv_heads: int, decode: bool) -> bool:
    lib = load("attention_mma")
    return bool(lib.ri_attention_mma_supports(c_int(head_dim), c_int(page_size), c_int(n_heads),
                                              c_int(n_kv_heads), c_int(1 if decode else 0)))


def attention_decode(q: torch.Tensor, q_ld: int, kcache, vcache, page_table, seq_slot, seq_len, cu_seqlens,
                     out: torch.Tensor, *, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int,
                     page_size: int, scale: float, window: int, n_splits: int, part_o=None, part_ml=None):
    """bf16 attention of one new token per sequence over its slot's keys, split into runs of
    pages; partial results go through the float32 scratch part_o / part_ml when n_splits > 1."""
    _need_cuda(q, kcache, vcache, page_table, seq_slot, seq_len, cu_seqlens, out, part_o, part_ml)
    _need(q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_decode: bf16 only")
    if n_splits > 1:
        _need(part_o is not None and part_o.dtype == torch.float32
              and part_o.numel() >= n_seqs * n_heads * n_splits * head_dim
              and part_ml is not None and part_ml.numel() >= n_seqs * n_heads * n_splits * 2,
              "attention_decode: scratch too small")
    _call("attention_mma", "ri_attention_decode", _p(q), c_int(q_ld), _p(kcache), _p(vcache), _p(page_table),
          c_int(page_table.shape[1]), _p(seq_slot), _p(seq_len), _p(cu_seqlens), _p(out), c_int(out.shape[1]),
          c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_float(scale),
          c_int(window), c_int(n_splits), _p(part_o), _p(part_ml), _stream())
    return out


def attention_prefill(q: torch.Tensor, q_ld: int, kcache, vcache, page_table, seq_slot, seq_start, cu_seqlens,
                      out: torch.Tensor, *, n_seqs: int, max_new: int, n_heads: int, n_kv_heads: int,
                      head_dim: int, page_size: int, scale: float, window: int):
    """bf16 causal attention of every new token of every sequence over its slot's keys."""
    _need_cuda(q, kcache, vcache, page_table, seq_slot, seq_start, cu_seqlens, out)
    _need(q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_prefill: bf16 only")
    _call("attention_mma", "ri_attention_prefill", _p(q), c_int(q_ld), _p(kcache), _p(vcache), _p(page_table),
          c_int(page_table.shape[1]), _p(seq_slot), _p(seq_start), _p(cu_seqlens), _p(out), c_int(out.shape[1]),
          c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
          c_float(scale), c_int(window), _stream())
    return out


def attention_prefill_forms(q: torch.Tensor, q_ld: int, kcache, vcache, page_table, seq_slot, seq_start, cu_seqlens,
                            out: torch.Tensor, *, n_seqs: int, max_new: int, n_heads: int, n_kv_heads: int,
                            head_dim: int, page_size: int, scale: float, window: int = 0, softcap: float = 0.0,
                            keep_first: int = 0, sink=None, dist=None, gate=None, out_scale: float = 1.0):
    """bf16 causal attention of every new token of every sequence over its slot's keys on the tensor cores, with the
    score's cap, the bias by distance (dist float32 [2, heads]), kept first positions beyond the window, a sink
    (float32 [heads]) and a gate per head (bf16 [tokens, heads], any row stride), each off when zero or None."""
    _need_cuda(q, kcache, vcache, page_table, seq_slot, seq_start, cu_seqlens, out, sink, dist, gate)
    _need(q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_prefill_forms: bf16 only")
    if sink is not None:
        _f32_vec(sink, n_heads, "attention_prefill_forms: sink")
    if dist is not None:
        _f32_vec(dist, 2 * n_heads, "attention_prefill_forms: dist")
    gate_ld = 0
    if gate is not None:
        _need(gate.dtype == torch.bfloat16 and gate.dim() == 2 and gate.shape[1] == n_heads and gate.stride(1) == 1,
              "attention_prefill_forms: gate must be bf16 [tokens, heads]")
        gate_ld = gate.stride(0)
    _call("attention_mma", "ri_attention_prefill_forms", _p(q), c_int(q_ld), _p(kcache), _p(vcache), _p(page_table),
          c_int(page_table.shape[1]), _p(seq_slot), _p(seq_start), _p(cu_seqlens), _p(out), c_int(out.shape[1]),
          c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size),
          c_float(scale), c_int(window), c_float(softcap), c_int(keep_first), _p(sink), _p(dist), _p(gate), c_int(gate_ld),
          c_float(out_scale), _stream())
    return out


def attention_decode_forms(q: torch.Tensor, q_ld: int, kcache, vcache, page_table, seq_slot, seq_len, cu_seqlens,
                           out: torch.Tensor, *, n_seqs: int, n_heads: int, n_kv_heads: int, head_dim: int, page_size: int,
                           scale: float, window: int = 0, softcap: float = 0.0, keep_first: int = 0, sink=None, dist=None,
                           gate=None, out_scale: float = 1.0, n_splits: int = 1, part_o=None, part_ml=None):
    """The same forms for a step of one token per sequence: a CTA per (sequence, kv head, run of pages), the runs'
    partial results (float32 scratch part_o [seqs * heads * splits * head_dim], part_ml [seqs * heads * splits * 2])
    merged by a second kernel when n_splits > 1."""
    _need_cuda(q, kcache, vcache, page_table, seq_slot, seq_len, cu_seqlens, out, sink, dist, gate, part_o, part_ml)
    _need(q.dtype == torch.bfloat16 and kcache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16,
          "attention_decode_forms: bf16 only")
    if sink is not None:
        _f32_vec(sink, n_heads, "attention_decode_forms: sink")
    if dist is not None:
        _f32_vec(dist, 2 * n_heads, "attention_decode_forms: dist")
    gate_ld = 0
    if gate is not None:
        _need(gate.dtype == torch.bfloat16 and gate.dim() == 2 and gate.shape[1] == n_heads and gate.stride(1) == 1,
              "attention_decode_forms: gate must be bf16 [tokens, heads]")
        gate_ld = gate.stride(0)
    if n_splits > 1:
        _need(part_o is not None and part_ml is not None and part_o.dtype == torch.float32 and part_ml.dtype == torch.float32
              and part_o.numel() >= n_seqs * n_heads * n_splits * head_dim and part_ml.numel() >= n_seqs * n_heads * n_splits * 2,
              "attention_decode_forms: scratch for the runs' partial results")
    _call("attention_mma", "ri_attention_decode_forms", _p(q), c_int(q_ld), _p(kcache), _p(vcache), _p(page_table),
          c_int(page_table.shape[1]), _p(seq_slot), _p(seq_len), _p(cu_seqlens), _p(out), c_int(out.shape[1]),
          c_int(n_seqs), c_int(n_heads), c_int(n_kv_heads), c_int(head_dim), c_int(page_size), c_float(scale), c_int(window),
          c_float(softcap), c_int(keep_first), _p(sink), _p(dist), _p(gate), c_int(gate_ld), c_float(out_scale),
          c_int(n_splits), _p(part_o), _p(part_ml), _stream())
    return out


# ----------------------------------------------------------------------------
# A gated linear recurrence with a matrix state per head (csrc/recurrent.cu)
# ----------------------------------------------------------------------------
RECURRENCE_PIECE = 64           # tokens of a long run of new tokens that one block scans


def recurrence_pieces(max_new: int, n_seqs: int, heads: int, dim: int, vdim: int, limit_bytes: int = 1 << 30) -> tuple:
    """(piece, most pieces per sequence) for a step whose longest run of new tokens is max_new: (0, 1) for
    short runs (one pass per sequence); else pieces of RECURRENCE_PIECE tokens, longer ones while the
    scratch for their states would exceed limit_bytes."""
    if max_new <= 2 * RECURRENCE_PIECE:
        return 0, 1
    piece = RECURRENCE_PIECE
    while n_seqs * -(-max_new // piece) * heads * dim * (vdim + 1) * 4 > limit_bytes and piece < max_new:
        piece *= 2
    return piece, -(-max_new // piece)


def gated_recurrence(z: torch.Tensor, bias: torch.Tensor, lower: torch.Tensor, norm_weight: torch.Tensor,
                     state: torch.Tensor, cu_seqlens: torch.Tensor, seq_slot: torch.Tensor, out: torch.Tensor, *,
                     n_seqs: int, heads: int, dim: int, vdim: int, eps: float, out_scale: float = 1.0,
                     o_raw: torch.Tensor | None = None, piece: int = 0, max_pieces: int = 1,
                     scratch: torch.Tensor | None = None, longest_run: int = 0) -> torch.Tensor:
    """S <- diag(f) S + (1 - f) v^T, o = S^T q per head over every sequence's new tokens in order, then
    o / rms(o) * norm_weight * out_scale per head.  z: float32 [T, 2*heads*dim + heads*vdim] holding the
    projections [q | f | v] before their activations (q and f are overwritten); state: float32 [slots, heads,
    dim, vdim], read and left at the sequence's last token; out: [T, heads*vdim] in the run dtype; o_raw:
    float32 [T, heads*vdim] scratch.  piece > 0: every sequence's new tokens are cut into pieces of that many
    tokens (at most max_pieces per sequence) that are scanned side by side, their states in `scratch`
    (float32, n_seqs * max_pieces * heads * dim * (vdim + 1) values): `recurrence_pieces` chooses.
    longest_run: the most new tokens any sequence brings (0: unknown), which sizes the scan's shared memory."""
    _need_cuda(z, bias, lower, norm_weight, state, cu_seqlens, seq_slot, out, o_raw, scratch)
    n = z.shape[0]
    _need(z.dtype == torch.float32 and z.is_contiguous() and z.shape[1] == 2 * heads * dim + heads * vdim,
          "gated_recurrence: z must be float32 [T, 2*heads*dim + heads*vdim]")
    for t, size in ((bias, heads * dim), (lower, heads * dim), (norm_weight, vdim)):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == size, "gated_recurrence: float32 vectors")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
          "gated_recurrence: state must be float32 [slots, heads, dim, vdim]")
    _need(out.is_contiguous() and out.shape == (n, heads * vdim), "gated_recurrence: out shape")
    _need(cu_seqlens.dtype == torch.int32 and seq_slot.dtype == torch.int32 and cu_seqlens.numel() >= n_seqs + 1
          and seq_slot.numel() >= n_seqs, "gated_recurrence: the step's arrays must be int32")
    if o_raw is None:
        o_raw = torch.empty((n, heads * vdim), dtype=torch.float32, device=z.device)
    _need(o_raw.dtype == torch.float32 and o_raw.is_contiguous() and o_raw.numel() >= n * heads * vdim,
          "gated_recurrence: o_raw must be float32 [T, heads*vdim]")
    if piece > 0:
        need = n_seqs * max_pieces * heads * dim * (vdim + 1)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=z.device)
        _need(scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
              "gated_recurrence: scratch too small for the pieces")
    _call("recurrent", "ri_gated_recurrence", _p(z), c_int(z.shape[1]), _p(bias), _p(lower), _p(norm_weight), _p(state),
          _p(cu_seqlens), _p(seq_slot), _p(o_raw), _p(out), c_int(dtype_code(out.dtype)), c_int(n), c_int(n_seqs),
          c_int(heads), c_int(dim), c_int(vdim), c_float(eps), c_float(out_scale), c_int(piece), c_int(max_pieces),
          _p(scratch if piece > 0 else None), c_int(max(0, min(int(longest_run), n))), _stream())
    global _launches
    _launches += 4 if piece > 0 else 1                    # several kernels behind one entry point
    return out


def gated_linear_attention(z: torch.Tensor, *, q_col: int, k_col: int, v_col: int, g_col: int, a_col: int, rank: int,
                           w2: torch.Tensor, bias: torch.Tensor, tau: float, q_scale: float, decay: torch.Tensor,
                           norm_weight: torch.Tensor, state: torch.Tensor, cu_seqlens: torch.Tensor, seq_slot: torch.Tensor,
                           out: torch.Tensor, n_seqs: int, heads: int, dim: int, vdim: int, eps: float,
                           out_scale: float = 1.0, o_raw: torch.Tensor | None = None, piece: int = 0, max_pieces: int = 1,
                           scratch: torch.Tensor | None = None, longest_run: int = 0) -> torch.Tensor:
    """The recurrence with a key of its own: per head S <- diag(f) S + k v^T, o = S^T q over every sequence's new tokens
    in order, with f = sigmoid(w2 a + bias)^(1/tau) per key channel from the low-rank input a, q scaled by q_scale; then
    o / rms(o) * norm_weight * silu(gate) * out_scale per head.  z: float32 [T, ld] with the columns of q and k
    ([heads, dim] each), v and the gates ([heads, vdim] each) and a ([rank]) as projected (q is scaled in place); w2:
    float32 [heads*dim, rank]; decay: float32 [T, heads*dim] scratch; the rest as `gated_recurrence`."""
    _need_cuda(z, w2, bias, decay, norm_weight, state, cu_seqlens, seq_slot, out, o_raw, scratch)
    n = z.shape[0]
    qdim = heads * dim
    _need(z.dtype == torch.float32 and z.is_contiguous() and z.dim() == 2, "gated_linear_attention: z must be float32 [T, ld]")
    _need(w2.dtype == torch.float32 and w2.is_contiguous() and tuple(w2.shape) == (qdim, rank),
          "gated_linear_attention: w2 must be float32 [heads*dim, rank]")
    for t, size in ((bias, qdim), (norm_weight, vdim)):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == size, "gated_linear_attention: float32 vectors")
    _need(decay.dtype == torch.float32 and decay.is_contiguous() and decay.numel() >= n * qdim,
          "gated_linear_attention: decay must be float32 [T, heads*dim]")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
          "gated_linear_attention: state must be float32 [slots, heads, dim, vdim]")
    _need(out.is_contiguous() and out.shape == (n, heads * vdim), "gated_linear_attention: out shape")
    _need(cu_seqlens.dtype == torch.int32 and seq_slot.dtype == torch.int32 and cu_seqlens.numel() >= n_seqs + 1
          and seq_slot.numel() >= n_seqs, "gated_linear_attention: the step's arrays must be int32")
    if o_raw is None:
        o_raw = torch.empty((n, heads * vdim), dtype=torch.float32, device=z.device)
    _need(o_raw.dtype == torch.float32 and o_raw.is_contiguous() and o_raw.numel() >= n * heads * vdim,
          "gated_linear_attention: o_raw must be float32 [T, heads*vdim]")
    if piece > 0:
        need = n_seqs * max_pieces * heads * dim * (vdim + 1)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=z.device)
        _need(scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
              "gated_linear_attention: scratch too small for the pieces")
    _call("recurrent", "ri_gated_linear_attention", _p(z), c_int(z.shape[1]), c_int(q_col), c_int(k_col), c_int(v_col),
          c_int(g_col), c_int(a_col), c_int(rank), _p(w2), _p(bias), c_float(tau), c_float(q_scale), _p(decay),
          _p(norm_weight), _p(state), _p(cu_seqlens), _p(seq_slot), _p(o_raw), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n), c_int(n_seqs), c_int(heads), c_int(dim), c_int(vdim), c_float(eps), c_float(out_scale), c_int(piece),
          c_int(max_pieces), _p(scratch if piece > 0 else None), c_int(max(0, min(int(longest_run), n))), _stream())
    global _launches
    _launches += 5 if piece > 0 else 2
    return out


# ----------------------------------------------------------------------------
# Routed experts (csrc/moe.cu)
# ----------------------------------------------------------------------------
def moe_route(x: torch.Tensor, router: torch.Tensor, correction: torch.Tensor, ids: torch.Tensor,
              weights: torch.Tensor, *, top: int, groups: int = 1, keep: int = 1,
              gate_weight: torch.Tensor | None = None, gate_out: torch.Tensor | None = None,
              softmax: bool = False, normalise: bool = True, split: int = 1, split_sums: torch.Tensor | None = None,
              split_count: torch.Tensor | None = None) -> None:
    """Per token the `top` experts with the largest sigmoid(router x) + correction among the `keep` best of
    `groups` groups (a group's score: the sum of its two largest), ids int32 [T, top], and their weights
    float32 [T, top] (the plain sigmoid scores, normalised).  gate_weight float32 [width]: gate_out[t] =
    sigmoid(gate_weight . x_t) as well.  softmax: the scores are softmax(router x) over all experts instead of
    sigmoids; normalise False: the weights are the chosen scores as they are.  split > 1 (steps of fewer than 296
    tokens): the router's rows are cut over that many blocks per token, which leave their sums in split_sums (float32
    [T, experts + 1]) and count themselves in split_count (int32 [T], zero before the call and after it)."""
    _need_cuda(x, router, correction, ids, weights, gate_weight, gate_out)
    n, width = x.shape
    experts = router.shape[0]
    _need(x.is_contiguous() and router.dtype == torch.float32 and router.is_contiguous() and router.shape[1] == width
          and correction.dtype == torch.float32 and correction.numel() == experts, "moe_route: router and correction")
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and ids.numel() >= n * top and weights.dtype == torch.float32
          and weights.is_contiguous() and weights.numel() >= n * top, "moe_route: ids int32 and weights float32 [T, top]")
    _need((gate_weight is None) == (gate_out is None), "moe_route: gate weight and output go together")
    if gate_weight is not None:
        _need(gate_weight.dtype == torch.float32 and gate_weight.is_contiguous() and gate_weight.numel() == width
              and gate_out.dtype == torch.float32 and gate_out.numel() >= n, "moe_route: gate")
    if split > 1:
        _need_cuda(split_sums, split_count)
        _need(n < 296 and split_sums is not None and split_sums.dtype == torch.float32 and split_sums.is_contiguous()
              and split_sums.numel() >= n * (experts + 1) and split_count is not None and split_count.dtype == torch.int32
              and split_count.numel() >= n, "moe_route: rows cut over blocks need few tokens, float32 sums and int32 counters")
    _call("moe", "ri_moe_route", _p(x), c_int(dtype_code(x.dtype)), _p(router), _p(correction), _p(gate_weight), _p(ids),
          _p(weights), _p(gate_out), c_int(n), c_int(width), c_int(experts), c_int(top), c_int(groups), c_int(keep),
          c_int((1 if softmax else 0) | (0 if normalise else 2)), c_int(max(1, split)), _p(split_sums if split > 1 else None),
          _p(split_count if split > 1 else None), _stream())


def moe_tile_rows() -> int:
    return int(load("moe").ri_moe_tile_rows())


def moe_arrange(ids: torch.Tensor, n_pairs: int, experts: int, tile_rows: int, offsets: torch.Tensor,
                order: torch.Tensor, tiles: torch.Tensor, n_tiles: torch.Tensor, place: torch.Tensor | None = None,
                gather: tuple | None = None) -> None:
    """The (token, choice) pairs listed expert by expert (`offsets` int32 [experts + 1] into `order` int32
    [pairs]) and cut into tiles of at most tile_rows pairs of one expert (`tiles` int32 [2 * (pairs /
    tile_rows + experts)]: expert and first index; `n_tiles` int32 [1]).  `place` int32 [pairs]: where in
    `order` each pair stands.  `gather` = (x, xs, top): the kernel also copies the activations into the
    lists' order, xs[i] = x[order[i] // top] (as `moe_gather` does; for steps of few pairs)."""
    _need_cuda(ids, offsets, order, tiles, n_tiles, place)
    for t in (ids, offsets, order, tiles, n_tiles, place):
        _need(t is None or (t.dtype == torch.int32 and t.is_contiguous()), "moe_arrange: int32 arrays")
    _need(offsets.numel() >= experts + 1 and order.numel() >= n_pairs and (place is None or place.numel() >= n_pairs)
          and tiles.numel() >= 2 * (-(-n_pairs // tile_rows) + experts), "moe_arrange: arrays too small")
    x = xs = None
    top = width = 0
    if gather is not None:
        x, xs, top = gather
        _need_cuda(x, xs)
        width = x.shape[1]
        _need(x.dtype == torch.bfloat16 and xs.dtype == torch.bfloat16 and x.is_contiguous() and xs.is_contiguous()
              and xs.shape == (n_pairs, width) and x.shape[0] * top >= n_pairs and width % 8 == 0, "moe_arrange: gather shapes")
    _call("moe", "ri_moe_arrange", _p(ids), c_int(n_pairs), c_int(experts), c_int(tile_rows), _p(offsets), _p(order),
          _p(tiles), _p(n_tiles), _p(place), _p(x), _p(xs), c_int(top), c_int(width), _stream())


def moe_gather(x: torch.Tensor, xs: torch.Tensor, order: torch.Tensor, *, n_pairs: int, top: int,
               listed: torch.Tensor | None = None) -> torch.Tensor:
    """xs[i] = x[order[i] // top]: the activations in the order of the experts' lists (bfloat16 rows of a
    multiple of 8 values).  listed (int32 [1] on the device): how many pairs the lists hold, where some are in none."""
    _need_cuda(x, xs, order, listed)
    _need(listed is None or listed.dtype == torch.int32, "moe_gather: listed must be int32")
    _need(x.dtype == torch.bfloat16 and xs.dtype == torch.bfloat16 and x.is_contiguous() and xs.is_contiguous()
          and xs.shape == (n_pairs, x.shape[1]) and x.shape[0] * top >= n_pairs, "moe_gather: shapes")
    _call("moe", "ri_moe_gather", _p(x), _p(xs), _p(order), c_int(n_pairs), c_int(top), c_int(x.shape[1]), _p(listed),
          _stream())
    return xs


def moe_grouped_simt(x: torch.Tensor, w: torch.Tensor, w2: torch.Tensor | None, out: torch.Tensor, offsets, order,
                     tiles, n_tiles, *, n_pairs: int, top: int, gate_form: torch.Tensor | None = None) -> torch.Tensor:
    """The experts' contractions over the arranged pairs, on the FFMA pipe.  With w2: x [T, K], w and w2
    [experts, N, K], out[p] = silu(w[e] x[p // top]) * (w2[e] x[p // top]) in the run dtype; without:
    x [pairs, K], out[p] = w[e] x[p] in float32.  gate_form (`gate_form`, with w2): another gate than SiLU."""
    _need_cuda(x, w, w2, out, offsets, order, tiles, n_tiles, gate_form)
    experts, n, k = w.shape
    gate = w2 is not None
    _need(gate_form is None or (gate and gate_form.dtype == torch.float32 and gate_form.numel() == 5),
          "moe_grouped: a gate form is five float32 constants of the gated form")
    _need(x.dtype == w.dtype and x.is_contiguous() and w.is_contiguous() and x.shape[1] == k, "moe_grouped: x and w")
    _need(not gate or (w2.shape == w.shape and w2.dtype == w.dtype and w2.is_contiguous()), "moe_grouped: second matrix")
    _need(out.is_contiguous() and out.shape == (n_pairs, n) and out.dtype == (x.dtype if gate else torch.float32),
          "moe_grouped: out")
    _need(x.shape[0] * (top if gate else 1) >= n_pairs, "moe_grouped: fewer rows than pairs")
    _call("moe", "ri_moe_grouped_simt", _p(x), _p(w), _p(w2), _p(out), c_int(dtype_code(x.dtype)), c_int(1 if gate else 0),
          _p(offsets), _p(order), _p(tiles), _p(n_tiles), c_int(n_pairs), c_int(experts), c_int(top), c_int(n), c_int(k),
          _p(gate_form), _stream())
    return out


def moe_combine(residual: torch.Tensor, y: torch.Tensor, weights: torch.Tensor, *, top: int,
                shared_y: torch.Tensor | None = None, gate: torch.Tensor | None = None,
                place: torch.Tensor | None = None, ids: torch.Tensor | None = None, x: torch.Tensor | None = None,
                n_real: int = 0, scale: float = 1.0) -> None:
    """residual[t] += scale * (sum_c weights[t, c] * y[row of pair t * top + c] (+ gate[t] * shared_y[t], or + shared_y[t]
    without a gate)); sums in float32.  A pair's row of y is the pair's own number, or place[pair] when `place` is given.
    With ids (int32 [T, top]), x (the experts' input [T, width]) and n_real, a chosen id >= n_real is an expert that hands
    its input through: its row is x[t]."""
    _need_cuda(residual, y, weights, shared_y, gate, place, ids, x)
    n, width = residual.shape
    for t in (residual, y, weights, shared_y, gate):
        _need(t is None or (t.dtype == torch.float32 and t.is_contiguous()), "moe_combine: float32 tensors")
    _need(y.shape == (n * top, width) and weights.numel() >= n * top, "moe_combine: shapes")
    _need(place is None or (place.dtype == torch.int32 and place.numel() >= n * top), "moe_combine: place must be int32 [pairs]")
    _need(gate is None or shared_y is not None, "moe_combine: a gate goes with a shared result")
    _need(shared_y is None or (shared_y.shape == (n, width) and (gate is None or gate.numel() >= n)), "moe_combine: the shared result")
    _need((ids is None) == (x is None), "moe_combine: ids and the experts' input go together")
    if ids is not None:
        _need(ids.dtype == torch.int32 and ids.is_contiguous() and ids.numel() >= n * top and x.is_contiguous()
              and tuple(x.shape) == (n, width), "moe_combine: ids int32 [T, top] and x [T, width]")
    _call("moe", "ri_moe_combine", _p(residual), _p(y), _p(weights), _p(shared_y), _p(gate), _p(place), c_int(n),
          c_int(width), c_int(top), _p(ids), _p(x), c_int(dtype_code(x.dtype) if x is not None else RI_F32), c_int(n_real),
          c_float(scale), _stream())


# ---- attention over a shared low-rank latent (csrc/latent.cu) ------------------------------------------
def latent_prepare(proj: torch.Tensor, cos, sin, latent_weight, eps: float, token_pos, token_seq, seq_slot, page_table,
                   cache, q_nope: torch.Tensor, q_wide: torch.Tensor, offsets, order, tiles, n_tiles, *, n_heads: int,
                   head_dim: int, rot_dim: int, rank: int, rot_dims: int, style: int, page_size: int, write_kv: bool,
                   tile_rows: int) -> None:
    """From the projection [T, heads * (head_dim + rot_dim) (+ rank + rot_dim ...)]: the heads' unrotated query
    parts head by head into q_nope [heads, T, head_dim], their rotated parts into the last rot_dim channels of
    q_wide [T, heads, rank + rot_dim]; with write_kv the RMS-normalised latent (times latent_weight) and the rotated
    key part into the token's row of `cache` [pages, 1, page_size, rank + rot_dim]; and the lists of the per-head
    grouped products (head h owns rows h * T .. (h + 1) * T, in tiles of tile_rows)."""
    _need_cuda(proj, cos, sin, latent_weight, token_pos, token_seq, seq_slot, page_table, cache, q_nope, q_wide,
               offsets, order, tiles, n_tiles)
    n = proj.shape[0]
    wide = rank + rot_dim
    need_cols = n_heads * (head_dim + rot_dim) + (wide if write_kv else 0)
    _need(proj.is_contiguous() and proj.shape[1] >= need_cols, "latent_prepare: the projection holds too few columns")
    _need(q_nope.dtype == proj.dtype and q_wide.dtype == proj.dtype and q_nope.is_contiguous() and q_wide.is_contiguous()
          and q_nope.numel() == n * n_heads * head_dim and q_wide.numel() == n * n_heads * wide, "latent_prepare: query buffers")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape[1] == rot_dims // 2 and cos.is_contiguous()
          and sin.is_contiguous() and 0 < rot_dims <= rot_dim and rot_dims % 2 == 0, "latent_prepare: rotation tables")
    if write_kv:
        _need(latent_weight is not None and latent_weight.dtype == torch.float32 and latent_weight.numel() == rank,
              "latent_prepare: the latent's norm weight must be float32 [rank]")
        _need(cache.dtype == proj.dtype and cache.is_contiguous() and tuple(cache.shape[1:]) == (1, page_size, wide),
              "latent_prepare: cache shape")
    per_head = -(-n // tile_rows)
    for t in (offsets, order, tiles, n_tiles):
        _need(t.dtype == torch.int32 and t.is_contiguous(), "latent_prepare: int32 lists")
    _need(offsets.numel() >= n_heads + 1 and order.numel() >= n_heads * n and tiles.numel() >= 2 * n_heads * per_head,
          "latent_prepare: lists too small")
    _call("latent", "ri_latent_prepare", _p(proj), c_int(dtype_code(proj.dtype)), c_int(proj.shape[1]), _p(cos), _p(sin),
          _p(latent_weight), c_float(eps), _p(token_pos), _p(token_seq), _p(seq_slot), _p(page_table),
          c_int(page_table.shape[1]), _p(cache), _p(q_nope), _p(q_wide), _p(offsets), _p(order), _p(tiles), _p(n_tiles),
          c_int(n), c_int(n_heads), c_int(head_dim), c_int(rot_dim), c_int(rank), c_int(rot_dims), c_int(style),
          c_int(page_size), c_int(1 if write_kv else 0), c_int(tile_rows), _stream())


def latent_widen(q_lat: torch.Tensor, q_wide: torch.Tensor, *, n_tokens: int, n_heads: int, rank: int, rot_dim: int) -> None:
    """q_wide[t, h, :rank] = q_lat[h, t, :] (float32 [heads, T, rank] into the run dtype's wide query rows)."""
    _need_cuda(q_lat, q_wide)
    _need(q_lat.dtype == torch.float32 and q_lat.is_contiguous() and q_lat.numel() == n_tokens * n_heads * rank
          and q_wide.is_contiguous() and q_wide.numel() == n_tokens * n_heads * (rank + rot_dim), "latent_widen: shapes")
    _call("latent", "ri_latent_widen", _p(q_lat), _p(q_wide), c_int(dtype_code(q_wide.dtype)), c_int(n_tokens),
          c_int(n_heads), c_int(rank), c_int(rot_dim), _stream())


def latent_gate(v: torch.Tensor, gates: torch.Tensor | None, out: torch.Tensor, *, n_tokens: int, n_heads: int,
                v_head_dim: int) -> None:
    """out[t, h * v_head_dim + j] = v[h, t, j] * sigmoid(gates[t, h]) (v float32, head by head; gates a view of
    columns of the projection, row stride gates.stride(0); None: no gate)."""
    _need_cuda(v, gates, out)
    _need(v.dtype == torch.float32 and v.is_contiguous() and v.numel() == n_tokens * n_heads * v_head_dim
          and out.is_contiguous() and out.shape == (n_tokens, n_heads * v_head_dim), "latent_gate: shapes")
    ld = 0
    if gates is not None:
        _need(gates.dtype == out.dtype and gates.shape == (n_tokens, n_heads) and gates.stride(1) == 1, "latent_gate: gates")
        ld = gates.stride(0)
    _call("latent", "ri_latent_gate", _p(v), _p(gates), c_int(ld), _p(out), c_int(dtype_code(out.dtype)), c_int(n_tokens),
          c_int(n_heads), c_int(v_head_dim), _stream())


def latent_attention_mma_supports(rank: int, rot_dim: int, page_size: int) -> bool:
    return bool(load("latent_attention_mma").ri_latent_attention_mma_supports(c_int(rank), c_int(rot_dim), c_int(page_size)))


def latent_attention_mma_tile_rows(rows: int, rank: int) -> int:
    """Query rows a CTA of the kernel takes in a step whose longest run of new rows (tokens x heads) is `rows`."""
    return int(load("latent_attention_mma").ri_latent_attention_mma_tile_rows(c_longlong(rows), c_int(rank)))


def latent_attention_mma(q_wide: torch.Tensor, cache: torch.Tensor, page_table, seq_slot, seq_start, cu_seqlens,
                         out: torch.Tensor, *, n_seqs: int, max_new: int, n_heads: int, rank: int, rot_dim: int, scale: float,
                         n_splits: int = 1, part_o: torch.Tensor | None = None, part_ml: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of n_heads query heads over one cached row per position on the tensor cores (bfloat16):
    q_wide [T, n_heads * (rank + rot_dim)], cache [pages, 1, 64, rank + rot_dim] (keys: the rows; values: their
    first `rank` channels), out head-major [n_heads, T, rank].  n_splits > 1 cuts every sequence's keys into runs
    whose partial results (part_o float32 [T * n_heads * n_splits * rank], part_ml float32 [T * n_heads * n_splits
    * 2]) a second kernel merges."""
    _need_cuda(q_wide, cache, page_table, seq_slot, seq_start, cu_seqlens, out, part_o, part_ml)
    n = q_wide.shape[0]
    wide = rank + rot_dim
    _need(q_wide.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
          and q_wide.is_contiguous() and cache.is_contiguous() and out.is_contiguous(), "latent_attention: bfloat16, contiguous")
    _need(q_wide.shape[1] == n_heads * wide and tuple(cache.shape[1:]) == (1, 64, wide) and out.numel() == n * n_heads * rank,
          "latent_attention: shapes")
    if n_splits > 1:
        _need(part_o is not None and part_ml is not None and part_o.dtype == torch.float32 and part_ml.dtype == torch.float32
              and part_o.numel() >= n * n_heads * n_splits * rank and part_ml.numel() >= n * n_heads * n_splits * 2,
              "latent_attention: scratch for the runs' partial results")
    _call("latent_attention_mma", "ri_latent_attention_mma", _p(q_wide), _p(cache), _p(page_table), c_int(page_table.shape[1]),
          _p(seq_slot), _p(seq_start), _p(cu_seqlens), c_int(n_seqs), c_int(max_new), c_int(n_heads), c_int(n), c_int(rank),
          c_int(rot_dim), c_float(scale), c_int(n_splits), _p(part_o), _p(part_ml), _p(out), _stream())
    if n_splits > 1:
        global _launches
        _launches += 1                       # the merge is a kernel of its own
    return out


# ----------------------------------------------------------------------------
# The hidden stream: norms without statistics, sums over depth, sums of normalised branches
# ----------------------------------------------------------------------------
def _f32_vec(t, n, what):
    _need(t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n, f"{what} must be float32 [{n}]")


def dyt_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, alpha: torch.Tensor, out: torch.Tensor,
             rows: torch.Tensor | None = None) -> torch.Tensor:
    """out[r, :] = tanh(alpha * x[rows[r] or r, :]) * weight + bias.  x, weight, bias, alpha (one number) float32;
    out float32 or bfloat16."""
    _need_cuda(x, weight, bias, alpha, out, rows)
    n_rows, n = out.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape[-1] == n and out.is_contiguous(), "dyt_norm: bad shapes")
    _f32_vec(weight, n, "dyt_norm: weight"); _f32_vec(bias, n, "dyt_norm: bias"); _f32_vec(alpha, 1, "dyt_norm: alpha")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() == n_rows, "dyt_norm: rows must be int32 [R]")
    else:
        _need(x.shape[0] >= n_rows, "dyt_norm: x has fewer rows than out")
    _call("stream", "ri_dyt_norm", _p(x), _p(weight), _p(bias), _p(alpha), _p(rows), _p(out), c_int(dtype_code(out.dtype)),
          c_int(n_rows), c_int(n), _stream())
    return out


def stream_update(stream_x: torch.Tensor, *, branch=None, branch_bias=None, post=None, history=None, depth_w=None,
                  depth_index: int = 0, store_result: bool = True, next_norm=None, next_out=None) -> None:
    """One pass over the float32 stream [T, n]: stream += post(branch + branch_bias) (post = (weight, bias, alpha) of a
    tanh norm, None: the branch as it is; the branch buffer is left zeroed); with `history` (float32 [>= depth_index + 2,
    T, n]) the result is stored as entry depth_index + 1 (if store_result) and the stream becomes
    sum_j depth_w[j] * history[j] over j <= depth_index + 1; with next_norm = (weight, bias, alpha) next_out receives
    that norm of the new stream."""
    _need_cuda(stream_x, branch, branch_bias, history, depth_w, next_out)
    t, n = stream_x.shape
    _need(stream_x.dtype == torch.float32 and stream_x.is_contiguous(), "stream_update: the stream must be float32")
    if branch is not None:
        _need(branch.dtype == torch.float32 and branch.is_contiguous() and tuple(branch.shape) == (t, n), "stream_update: branch")
    if branch_bias is not None:
        _f32_vec(branch_bias, n, "stream_update: branch bias")
    pw = pb = pa = nw = nb = na = None
    if post is not None:
        pw, pb, pa = post
        _f32_vec(pw, n, "stream_update: norm weight"); _f32_vec(pb, n, "stream_update: norm bias"); _f32_vec(pa, 1, "stream_update: alpha")
    if history is not None:
        _need(history.dtype == torch.float32 and history.is_contiguous() and history.shape[0] >= depth_index + 2
              and tuple(history.shape[1:]) == (t, n), "stream_update: history must be float32 [entries, T, n]")
        _f32_vec(depth_w, depth_index + 2, "stream_update: depth weights")
    next_dtype = 0
    if next_norm is not None:
        nw, nb, na = next_norm
        _f32_vec(nw, n, "stream_update: next weight"); _f32_vec(nb, n, "stream_update: next bias"); _f32_vec(na, 1, "stream_update: next alpha")
        _need(next_out is not None and next_out.is_contiguous() and tuple(next_out.shape) == (t, n), "stream_update: next_out")
        next_dtype = dtype_code(next_out.dtype)
    _call("stream", "ri_stream_update", _p(stream_x), _p(branch), _p(branch_bias), _p(pw), _p(pb), _p(pa), _p(history),
          _p(depth_w), c_int(depth_index), c_int(1 if store_result else 0), _p(nw), _p(nb), _p(na),
          _p(next_out if next_norm is not None else None), c_int(next_dtype), c_int(t), c_int(n), _stream())


def normed_sum(members: list, out: torch.Tensor, eps: float, accumulate: bool = False) -> torch.Tensor:
    """out (+)= sum over members (x, bias or None, weight, scale) of scale * rmsnorm(x + bias) * weight, row by row; every x
    (float32 [T, n]) is left zeroed."""
    t, n = out.shape
    _need(1 <= len(members) <= 4, "normed_sum: one to four members")
    _need(out.dtype == torch.float32 and out.is_contiguous(), "normed_sum: out must be float32")
    xs, bs, ws, sc = (c_void_p * 4)(), (c_void_p * 4)(), (c_void_p * 4)(), (c_float * 4)()
    for m, (x, bias, w, scale) in enumerate(members):
        _need_cuda(x, bias, w)
        _need(x.dtype == torch.float32 and x.is_contiguous() and tuple(x.shape) == (t, n), "normed_sum: member shape")
        _f32_vec(w, n, "normed_sum: weight")
        if bias is not None:
            _f32_vec(bias, n, "normed_sum: bias")
        xs[m], bs[m], ws[m], sc[m] = x.data_ptr(), (bias.data_ptr() if bias is not None else None), w.data_ptr(), float(scale)
    _call("stream", "ri_normed_sum", xs, bs, ws, sc, c_int(len(members)), _p(out), c_int(t), c_int(n), c_float(eps),
          c_int(1 if accumulate else 0), _stream())
    return out


def xielu(x: torch.Tensor, out: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """out = a_p x^2 + x/2 for x > 0, a_n (e^x - 1 - x) + x/2 otherwise, with a_p = softplus(pq[0]) and
    a_n = 1/2 + softplus(pq[1]); float32 arithmetic; out may be x."""
    _need_cuda(x, out, pq)
    _need(x.dtype == out.dtype and x.is_contiguous() and out.is_contiguous() and x.numel() == out.numel(), "xielu: shapes")
    _f32_vec(pq, 2, "xielu: parameters")
    _call("stream", "ri_xielu", _p(x), _p(out), c_int(dtype_code(x.dtype)), _p(pq), c_longlong(x.numel()), _stream())
    return out


def add_row_bias(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x[t, :] += bias (float32)."""
    _need_cuda(x, bias)
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "add_row_bias: x must be float32 [T, n]")
    _f32_vec(bias, x.shape[1], "add_row_bias: bias")
    _call("stream", "ri_add_row_bias", _p(x), _p(bias), c_int(x.shape[0]), c_int(x.shape[1]), _stream())
    return x


# ----------------------------------------------------------------------------
# Recurrent mixers with one decay per head (state space, gated delta rule)
# ----------------------------------------------------------------------------
def scan_prepare(z: torch.Tensor, *, conv_col: int, conv_ch: int, taps: torch.Tensor, conv_bias, conv_state: torch.Tensor,
                 unit_heads: int, unit_dim: int, scaled_heads: int, unit_scale: float, heads: int, decay_col: int,
                 step_col: int, a_log: torch.Tensor, dt_bias: torch.Tensor, out: torch.Tensor, cu_seqlens, token_seq,
                 seq_slot, n_seqs: int) -> torch.Tensor:
    """Per token of z (float32 [T, ld]): the short causal convolution (taps float32 [conv_ch, K], last column the
    current token's; bias or None) and silu of the columns conv_col .. conv_col + conv_ch, reading the inputs before
    the step from conv_state (float32 [slots, K - 1, conv_ch]) and moving those on; the first unit_heads heads of
    unit_dim channels made unit vectors (the first scaled_heads of them times unit_scale); per head the decay
    exp(-exp(a_log) * softplus(z[decay_col + h] + dt_bias)) and the step (sigmoid(z[step_col + h]), or with
    step_col < 0 the softplus itself).  out: float32 [T, >= conv_ch + 2 heads] = [channels | decays | steps]."""
    _need_cuda(z, taps, conv_bias, conv_state, a_log, dt_bias, out, cu_seqlens, token_seq, seq_slot)
    t = z.shape[0]
    k = taps.shape[1]
    _need(z.dtype == torch.float32 and z.is_contiguous() and out.dtype == torch.float32 and out.is_contiguous()
          and out.shape[0] == t, "scan_prepare: z and out must be float32 [T, .]")
    _need(taps.dtype == torch.float32 and taps.is_contiguous() and taps.shape[0] == conv_ch, "scan_prepare: taps")
    _need(conv_bias is None or (conv_bias.dtype == torch.float32 and conv_bias.numel() == conv_ch), "scan_prepare: bias")
    _need(conv_state.dtype == torch.float32 and conv_state.is_contiguous()
          and tuple(conv_state.shape[1:]) == (max(k - 1, 0), conv_ch), "scan_prepare: carried inputs must be [slots, K - 1, channels]")
    _f32_vec(a_log, heads, "scan_prepare: A_log"); _f32_vec(dt_bias, heads, "scan_prepare: dt_bias")
    _call("state_scan", "ri_scan_prepare", _p(z), c_int(z.shape[1]), c_int(conv_col), c_int(conv_ch), _p(taps), _p(conv_bias),
          c_int(k), _p(conv_state), c_int(unit_heads), c_int(unit_dim), c_int(scaled_heads), c_float(unit_scale), c_int(heads),
          c_int(decay_col), c_int(step_col), _p(a_log), _p(dt_bias), _p(out), c_int(out.shape[1]), _p(cu_seqlens),
          _p(token_seq), _p(seq_slot), c_int(t), c_int(n_seqs), _stream())
    return out


def state_scan(u: torch.Tensor, state: torch.Tensor, o: torch.Tensor, cu_seqlens, seq_slot, *, n_seqs: int, heads: int,
               groups: int, dim: int, vdim: int, q_col: int, k_col: int, v_col: int, decay_col: int, step_col: int,
               delta: bool, skip=None, longest_run: int = 0, piece: int = 0, max_pieces: int = 1, piece_state=None,
               piece_decay=None) -> torch.Tensor:
    """The recurrence over every sequence's new tokens from its slot's state (float32 [slots, heads, dim, vdim]), which
    moves on.  u: float32 [T, ld] with the columns of queries and keys ([groups, dim] each), values ([heads, vdim]),
    decays and steps ([heads] each); o: float32 [T, heads * vdim].  delta: the gated delta rule
    (S <- a S; S += k (step (v - S^T k))^T); else S <- a S + k (step v)^T and o += skip * v.  piece > 0 (not the delta
    rule): long runs are scanned in pieces of that many tokens side by side, from zero, then again from start states that
    a carry over the pieces gives; float32 scratch piece_state [n_seqs, max_pieces, heads, dim, vdim] and piece_decay
    [n_seqs, max_pieces, heads], max_pieces * piece at least the longest run."""
    _need_cuda(u, state, o, cu_seqlens, seq_slot, skip, piece_state, piece_decay)
    if piece > 0:
        _need(not delta and piece_state is not None and piece_decay is not None and piece_state.dtype == torch.float32
              and piece_decay.dtype == torch.float32 and piece_state.is_contiguous() and piece_decay.is_contiguous()
              and piece_state.numel() >= n_seqs * max_pieces * heads * dim * vdim
              and piece_decay.numel() >= n_seqs * max_pieces * heads, "state_scan: scratch of the pieces")
    _need(u.dtype == torch.float32 and u.is_contiguous() and o.dtype == torch.float32 and o.is_contiguous()
          and tuple(o.shape) == (u.shape[0], heads * vdim), "state_scan: u and o must be float32")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
          "state_scan: state must be float32 [slots, heads, dim, vdim]")
    if skip is not None:
        _f32_vec(skip, heads, "state_scan: skip")
    _call("state_scan", "ri_state_scan", _p(u), c_int(u.shape[1]), c_int(q_col), c_int(k_col), c_int(v_col), c_int(decay_col),
          c_int(step_col), _p(skip), _p(state), _p(o), _p(cu_seqlens), _p(seq_slot), c_int(n_seqs), c_int(heads), c_int(groups),
          c_int(dim), c_int(vdim), c_int(1 if delta else 0), c_int(longest_run), c_int(piece), c_int(max_pieces),
          _p(piece_state), _p(piece_decay), _stream())
    return o


SCAN_PIECE = 64                 # tokens of a long run of new tokens that one block of the state space's scan takes


def scan_pieces(max_new: int, blocks: int) -> tuple:
    """(piece, most pieces per sequence) of the state space's scan for a step whose longest run of new tokens is
    max_new and whose one-pass grid has `blocks` blocks (sequences x heads x tiles of 16 value columns): (0, 1), one
    pass per sequence, for runs of up to two pieces and for grids that fill the SMs by themselves (the passes over
    pieces do the multiply-adds twice: measured, they halve the time at 64 blocks, change nothing at 128 and lose at 256)."""
    if max_new <= 2 * SCAN_PIECE or blocks > torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count:
        return 0, 1
    return SCAN_PIECE, -(-max_new // SCAN_PIECE)


def gated_group_norm(x: torch.Tensor, gate: torch.Tensor, gate_col: int, weight: torch.Tensor, out: torch.Tensor, *,
                     groups: int, group_size: int, gate_first: bool, eps: float, out_scale: float = 1.0) -> torch.Tensor:
    """Per token and group of group_size channels of x (float32 [T, groups * group_size]): RMS norm over the group times
    weight[channel % len(weight)], and a gate silu(gate[t, gate_col + channel]) applied before the norm (gate_first) or
    after it; the result times out_scale into out (float32 or bfloat16)."""
    _need_cuda(x, gate, weight, out)
    t = x.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.shape[1] == groups * group_size, "gated_group_norm: x")
    _need(gate.dtype == torch.float32 and gate.is_contiguous() and gate.shape[0] == t
          and gate.shape[1] >= gate_col + groups * group_size, "gated_group_norm: gate")
    _need(weight.dtype == torch.float32 and weight.is_contiguous(), "gated_group_norm: weight")
    _need(out.is_contiguous() and tuple(out.shape) == (t, groups * group_size), "gated_group_norm: out")
    _call("state_scan", "ri_gated_group_norm", _p(x), c_int(x.shape[1]), _p(gate), c_int(gate.shape[1]), c_int(gate_col), _p(weight),
          c_int(weight.numel()), _p(out), c_int(dtype_code(out.dtype)), c_int(t), c_int(groups), c_int(group_size),
          c_int(1 if gate_first else 0), c_float(eps), c_float(out_scale), _stream())
    return out
