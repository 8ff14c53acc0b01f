"""Grouped-query attention over the cache (attention.rs:54-124)."""
from __future__ import annotations

import math

import torch

from ..cache.sequence_cache import KVRequest
from ..kernels import linear, attention as attn_kernels
from .base import Mixer
from .registry import register, lookup
from .spec import TensorSpec, PartSpec


@register("mixer", "gqa_attention")
class GQAttention(Mixer):
    """q, k, v projections with optional biases (attention.rs:66-76), the position encoding
    on q and k fused with the cache write (:78-90), attention of every new token over the
    keys 0..position of its slot with scale 1/sqrt(head_dim) (:95-121), query head h reading
    kv head h / (heads / kv heads) (:37, :96), and the output projection without bias added
    onto the residual stream (:123, transformer.rs:38-39)."""

    # Beyond the dense decoder's form, as parameters: values of a head size of their own (`v_head_dim`),
    # a score scale other than 1/sqrt(head_dim) (`scale`), keys limited to the query's own block of
    # `chunk` positions counted from the start of the sequence, a factor on the mixer's result
    # (`out_scale`, applied to the attention's output in float32 before the output projection), and
    # the tensors' names below the part's prefix (`names`: q, k, v, o and, with biases, q_bias, ...).
    # `qk_norm_eps`: every q and k head is RMS-normalised before the rotation, with one weight of head_dim
    # values for the q heads and one for the k heads (`names`: q_norm, k_norm).  `values_from_keys`: there is
    # no value projection; a position's values are its keys as projected, before norm and rotation.
    # Forms of the score, the mask and the result (all off by default): `softcap` (scores become
    # softcap * tanh(score / softcap) after the scale); `distance_bias` (r1_h ln(1 + r2_h * distance) is taken off the
    # capped score, two learned numbers per head, `names`: r1, r2); `keep_first` (with a window: the first so many
    # positions of the sequence stay visible beyond it, at their true positions); `sink` (the softmax's denominator
    # also holds exp(sink_h), a learned number per head without key or value); `head_gate` (the head's result times
    # sigmoid(W_g x)_h, one more row per head in the projection, `names`: gate); `o_bias` (a bias on the output
    # projection, `names`: o_bias); `own_kv` False: the layer has no key and value projections and attends over the
    # cache of the layer the schedule gives it, with its own queries.  `out_gate`: the concatenated heads' result is
    # multiplied element by element with sigmoid(W_g x) before the output projection (one more row per value channel of
    # every head in the projection, `names`: out_gate).
    _NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
              "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias",
              "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "o_bias": "o_proj.bias", "sink": "sinks",
              "gate": "gate_proj.weight", "r1": "distance_r1", "r2": "distance_r2", "out_gate": "out_gate_proj.weight"}

    def __init__(self, *, n_heads: int, n_kv_heads: int, head_dim: int, qkv_bias: bool,
                 position: PartSpec, window: int | None = None, v_head_dim: int | None = None,
                 scale: float | None = None, chunk: int | None = None, out_scale: float = 1.0,
                 names: dict | None = None, qk_norm_eps: float | None = None, values_from_keys: bool = False,
                 softcap: float = 0.0, distance_bias: bool = False, keep_first: int = 0, sink: bool = False,
                 head_gate: bool = False, o_bias: bool = False, own_kv: bool = True, out_gate: bool = False,
                 hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} kv heads")
        if chunk is not None and chunk <= 0:
            raise ValueError(f"a chunk holds at least one position, found {chunk}")
        self.n_heads, self.n_kv_heads, self.head_dim = n_heads, n_kv_heads, head_dim
        self.v_head_dim = head_dim if v_head_dim is None else int(v_head_dim)
        self.values_from_keys = bool(values_from_keys)
        if self.values_from_keys and self.v_head_dim != head_dim:
            raise ValueError(f"values taken from keys of size {head_dim} cannot have the size {self.v_head_dim}")
        if window is not None and window <= 0:
            raise ValueError(f"a window holds at least one position, found {window}")
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.q_dim, self.kv_dim = n_heads * head_dim, n_kv_heads * head_dim
        self.v_dim, self.o_dim = n_kv_heads * self.v_head_dim, n_heads * self.v_head_dim
        self.qkv_bias = bool(qkv_bias)
        if self.values_from_keys and self.qkv_bias:
            raise ValueError("values taken from keys and projection biases are not combined")
        self.q_norm = self.k_norm = None
        self.softcap, self.keep_first = float(softcap), int(keep_first or 0)
        self.distance_bias, self.sink, self.head_gate = bool(distance_bias), bool(sink), bool(head_gate)
        self.o_bias, self.own_kv, self.out_gate = bool(o_bias), bool(own_kv), bool(out_gate)
        if self.out_gate and self.head_gate:
            raise ValueError("a gate per head and a gate per channel are not combined")
        if self.softcap < 0 or self.keep_first < 0:
            raise ValueError(f"a score cap and a number of kept positions are not negative, found {softcap}, {keep_first}")
        if self.keep_first and window is None:
            raise ValueError("kept first positions go with a window")
        if not self.own_kv and (self.values_from_keys or self.qk_norm_eps is not None):
            raise ValueError("a layer without keys of its own has no key norm and no values taken from keys")
        # what only the general path (one projection, then the position encoding, then attention with these forms) does
        self.extended = bool(self.softcap or self.distance_bias or self.keep_first or self.sink or self.head_gate
                             or self.out_gate or not self.own_kv)
        self.sinks = self.dist = self.b_o = None
        self.window = window
        self.chunk = chunk
        self.out_scale = float(out_scale)
        self.scale = 1.0 / math.sqrt(float(head_dim)) if scale is None else float(scale)
        self.names = dict(self._NAMES, **(names or {}))
        self.position = lookup("position", position.kind)(
            hidden_size=hidden_size, dtype=dtype, device=device, **position.params)
        self.w_qkv = self.b_qkv = self.w_o = None

    def tensor_specs(self):
        h, nm = self.hidden_size, self.names
        specs = {
            nm["q"]: TensorSpec((self.q_dim, h)),
            nm["k"]: TensorSpec((self.kv_dim, h)),
            nm["v"]: TensorSpec((self.v_dim, h)),
            nm["o"]: TensorSpec((h, self.o_dim)),
        }
        if self.values_from_keys:
            del specs[nm["v"]]
        if not self.own_kv:
            del specs[nm["k"]], specs[nm["v"]]
        if self.head_gate:
            specs[nm["gate"]] = TensorSpec((self.n_heads, h))
        if self.out_gate:
            specs[nm["out_gate"]] = TensorSpec((self.o_dim, h))
        if self.sink:
            specs[nm["sink"]] = TensorSpec((self.n_heads,), role="vector", init="zeros")
        if self.distance_bias:
            specs[nm["r1"]] = TensorSpec((self.n_heads,), role="vector", init="ones")
            specs[nm["r2"]] = TensorSpec((self.n_heads,), role="vector", init="ones")
        if self.o_bias:
            specs[nm["o_bias"]] = TensorSpec((h,), role="vector")
        if self.qk_norm_eps is not None:
            specs[nm["q_norm"]] = TensorSpec((self.head_dim,), role="vector", init="ones")
            specs[nm["k_norm"]] = TensorSpec((self.head_dim,), role="vector", init="ones")
        if self.qkv_bias:
            specs[nm["q_bias"]] = TensorSpec((self.q_dim,), role="vector")
            if self.own_kv:
                specs[nm["k_bias"]] = TensorSpec((self.kv_dim,), role="vector")
                specs[nm["v_bias"]] = TensorSpec((self.v_dim,), role="vector")
        return specs

    def set_tensors(self, tensors):
        nm = self.names
        # one matrix for the three projections: one pass over x
        mats = [tensors[nm["q"]]]
        if self.own_kv:
            mats += [tensors[nm["k"]]] + ([] if self.values_from_keys else [tensors[nm["v"]]])
        if self.head_gate or self.out_gate:
            # one more row per head (or per value channel of every head): the gates come out of the same product
            mats.append(tensors[nm["gate" if self.head_gate else "out_gate"]])
            rows = sum(m.shape[0] for m in mats)
            if rows % 8:                               # rows of zeros keep a token's row a multiple of 16 bytes, which the
                mats.append(torch.zeros(-rows % 8, mats[0].shape[1], dtype=mats[0].dtype, device=mats[0].device))   # tensor-core kernels want
        self.w_qkv = linear.Weight(torch.cat(mats, dim=0))
        if self.sink:
            self.sinks = tensors[nm["sink"]].contiguous()
        if self.distance_bias:
            self.dist = torch.stack([tensors[nm["r1"]], tensors[nm["r2"]]], dim=0).contiguous()
        if self.o_bias:
            self.b_o = tensors[nm["o_bias"]].contiguous()
            self.b_o_scaled = self.b_o if self.out_scale == 1.0 else self.b_o * self.out_scale
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors[nm["q_norm"]].contiguous(), tensors[nm["k_norm"]].contiguous()
        if self.qkv_bias:
            biases = [tensors[nm["q_bias"]]] + ([tensors[nm["k_bias"]], tensors[nm["v_bias"]]] if self.own_kv else [])
            self.b_qkv = torch.cat(biases, dim=0).contiguous()
            if self.b_qkv.numel() < self.w_qkv.n:      # the gates' rows, and the rows of zeros after them
                self.b_qkv = torch.cat([self.b_qkv, self.b_qkv.new_zeros(self.w_qkv.n - self.b_qkv.numel())]).contiguous()
        self.w_o = linear.Weight(tensors[nm["o"]])

    def get_tensors(self):
        q, kv, nm = self.q_dim, self.kv_dim, self.names
        w = self.w_qkv.t
        out = {nm["q"]: w[:q], nm["o"]: self.w_o.t}
        at = q
        if self.own_kv:
            out[nm["k"]] = w[q:q + kv]
            at = q + kv
            if not self.values_from_keys:
                out[nm["v"]] = w[at:at + self.v_dim]
                at += self.v_dim
        if self.head_gate:
            out[nm["gate"]] = w[at:at + self.n_heads]
        if self.out_gate:
            out[nm["out_gate"]] = w[at:at + self.o_dim]
        if self.sink:
            out[nm["sink"]] = self.sinks
        if self.distance_bias:
            out[nm["r1"]], out[nm["r2"]] = self.dist[0], self.dist[1]
        if self.o_bias:
            out[nm["o_bias"]] = self.b_o
        if self.qk_norm_eps is not None:
            out[nm["q_norm"]], out[nm["k_norm"]] = self.q_norm, self.k_norm
        if self.qkv_bias:
            b = self.b_qkv
            out[nm["q_bias"]] = b[:q]
            if self.own_kv:
                out.update({nm["k_bias"]: b[q:q + kv], nm["v_bias"]: b[q + kv:q + kv + self.v_dim]})
        return out

    def prepare(self, max_positions):
        self.position.prepare(max_positions)

    def cache_request(self):
        return KVRequest(self.n_kv_heads, self.head_dim, self.window,
                         None if self.v_head_dim == self.head_dim else self.v_head_dim)

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        n = x.shape[0]
        # a layer that has key and value projections but is scheduled to read another layer's cache leaves its own unused
        kv_width = (self.kv_dim + (0 if self.values_from_keys else self.v_dim)) if self.own_kv else 0
        gate_col = self.q_dim + kv_width
        width = self.w_qkv.n                           # with gates: one more column per head, padded to a multiple of 8
        special = self.values_from_keys or self.qk_norm_eps is not None
        usual = (self.v_head_dim == self.head_dim and not getattr(self.position, "partial", False) and not special
                 and not self.extended)
        from_acc = getattr(self.position, "apply_and_store_from_accumulators", None) if usual else None
        if from_acc is not None and linear.wants_split(x, self.w_qkv):
            # a small step: the projection is split over K into float32 accumulators, and the
            # position encoding adds the bias, rotates and stores from there
            acc = ctx.zeroed_buffer("qkv_acc", (n, width), torch.float32)
            linear.accumulate_split(x, self.w_qkv, acc, ctx)
            qkv = ctx.buffer("q_rot", (n, self.q_dim), self.dtype)
            from_acc(acc, self.b_qkv, qkv, ctx, cache_layer, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads,
                     head_dim=self.head_dim, write_kv=writes_cache)
        else:
            qkv = ctx.buffer("qkv", (n, width), self.dtype)
            linear.project(x, self.w_qkv, qkv, ctx, bias=self.b_qkv)
            extra = {} if usual else {"v_head_dim": self.v_head_dim}
            if special:
                # norm of the heads, rotation and cache write as one kernel (the position encoding's)
                self.position.apply_normed_and_store(
                    qkv, ctx, cache_layer, n_heads=self.n_heads, n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
                    write_kv=writes_cache, q_weight=self.q_norm, k_weight=self.k_norm,
                    eps=self.qk_norm_eps if self.qk_norm_eps is not None else 0.0,
                    values_from_keys=self.values_from_keys, **extra)
            else:
                self.position.apply_and_store(qkv, ctx, cache_layer, n_heads=self.n_heads,
                                              n_kv_heads=self.n_kv_heads, head_dim=self.head_dim,
                                              write_kv=writes_cache and self.own_kv, **extra)
        mixed = ctx.buffer("attn_out", (n, self.o_dim), self.dtype)
        attn_kernels.attention(qkv, cache_layer, mixed, ctx, n_heads=self.n_heads,
                               n_kv_heads=self.n_kv_heads, head_dim=self.head_dim, scale=self.scale,
                               window=self.window or 0, chunk=self.chunk or 0, v_head_dim=self.v_head_dim,
                               out_scale=1.0 if self.out_gate else self.out_scale, softcap=self.softcap,
                               keep_first=self.keep_first, sink=self.sinks, dist=self.dist,
                               gate=qkv[:, gate_col:gate_col + self.n_heads] if self.head_gate else None)
        from ..kernels import ops
        if self.out_gate:
            # the gates of the projection's last columns, the mixer's factor with them (float32, one rounding)
            ops.sigmoid_gate_(mixed, qkv, gate_col, self.out_scale)
        linear.into_residual(mixed, self.w_o, residual, ctx)
        if self.o_bias:
            ops.add_row_bias(residual, self.b_o_scaled)
