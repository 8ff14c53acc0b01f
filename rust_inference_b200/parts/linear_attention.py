"""Gated linear attention: a matrix state per head with a decay per key channel."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import StateRequest
from ..kernels import linear, ops
from .base import Mixer
from .registry import register
from .spec import TensorSpec


@register("mixer", "gated_linear_attention")
class GatedLinearAttention(Mixer):
    """Per head a state S [dim, vdim] in float32, zero at the start of a sequence and carried from token to token in
    the slot's state area:

        q = Wq x * dim^(-1/2)      k = Wk x      v = Wv x      f = sigmoid(W2 (W1 x) + b)^(1/tau)
        S <- diag(f) S + k v^T      o = S^T q

    The decay f acts on the rows of S that belong to key channels and comes from a low-rank map (`rank` is W1's number
    of rows).  Every head's o is RMS-normed over vdim with one weight shared by the heads, the heads are concatenated,
    multiplied by silu(Wg x) and projected by Wo onto the residual stream.  The five projections run as one product
    with float32 results; the decay (as exp(log_sigmoid(.) / tau)), the state, the norm and the gate are float32 in both
    precisions.  `out_scale` multiplies the mixer's result (applied with the gate, in float32).  `names` gives the
    tensors' names below the part's prefix.  The scan is the one of `gated_linear_recurrence`, with a key of its own in
    place of that form's 1 - f."""

    _NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight",
              "o": "o_proj.weight", "norm": "o_norm.weight", "decay_in": "a_proj.0.weight", "decay_out": "a_proj.1.weight",
              "decay_bias": "a_proj.1.bias"}

    def __init__(self, *, n_heads: int, head_dim: int, v_head_dim: int, rank: int, tau: float, eps: float,
                 out_scale: float = 1.0, names: dict | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if n_heads <= 0 or head_dim <= 0 or v_head_dim <= 0 or rank <= 0:
            raise ValueError(f"gated_linear_attention: sizes must be positive, found heads {n_heads}, dim {head_dim}, "
                             f"vdim {v_head_dim}, rank {rank}")
        if not tau > 0:
            raise ValueError(f"gated_linear_attention: tau must be positive, found {tau}")
        self.n_heads, self.head_dim, self.v_head_dim, self.rank = n_heads, head_dim, v_head_dim, int(rank)
        self.q_dim, self.v_dim = n_heads * head_dim, n_heads * v_head_dim
        self.tau, self.eps, self.out_scale = float(tau), float(eps), float(out_scale)
        self.names = dict(self._NAMES, **(names or {}))
        # columns of the one product: q | k | v | gate | decay input (| rows of zeros up to a multiple of 8)
        self.q_col, self.k_col = 0, self.q_dim
        self.v_col = 2 * self.q_dim
        self.g_col = self.v_col + self.v_dim
        self.a_col = self.g_col + self.v_dim
        self.width = -(-(self.a_col + self.rank) // 8) * 8
        self.w_in = self.w_o = self.w2 = self.decay_bias = self.norm = None

    def tensor_specs(self):
        h, nm = self.hidden_size, self.names
        return {
            nm["q"]: TensorSpec((self.q_dim, h)),
            nm["k"]: TensorSpec((self.q_dim, h)),
            nm["v"]: TensorSpec((self.v_dim, h)),
            nm["gate"]: TensorSpec((self.v_dim, h)),
            nm["o"]: TensorSpec((h, self.v_dim)),
            nm["norm"]: TensorSpec((self.v_head_dim,), role="vector", init="ones"),
            nm["decay_in"]: TensorSpec((self.rank, h)),
            nm["decay_out"]: TensorSpec((self.q_dim, self.rank), role="vector"),     # float32: the decay's own arithmetic
            nm["decay_bias"]: TensorSpec((self.q_dim,), role="vector"),
        }

    def set_tensors(self, tensors):
        nm = self.names
        mats = [tensors[nm[k]] for k in ("q", "k", "v", "gate", "decay_in")]
        rows = sum(m.shape[0] for m in mats)
        if rows < self.width:
            mats.append(torch.zeros(self.width - rows, self.hidden_size, dtype=mats[0].dtype, device=mats[0].device))
        self.w_in = linear.Weight(torch.cat(mats, dim=0))
        self.w_o = linear.Weight(tensors[nm["o"]])
        self.w2 = tensors[nm["decay_out"]].contiguous()
        self.decay_bias, self.norm = tensors[nm["decay_bias"]].contiguous(), tensors[nm["norm"]].contiguous()

    def get_tensors(self):
        nm, w = self.names, self.w_in.t
        return {nm["q"]: w[:self.k_col], nm["k"]: w[self.k_col:self.v_col], nm["v"]: w[self.v_col:self.g_col],
                nm["gate"]: w[self.g_col:self.a_col], nm["decay_in"]: w[self.a_col:self.a_col + self.rank],
                nm["o"]: self.w_o.t, nm["norm"]: self.norm, nm["decay_out"]: self.w2, nm["decay_bias"]: self.decay_bias}

    def cache_request(self):
        return StateRequest((self.n_heads, self.head_dim, self.v_head_dim), torch.float32)

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        if not writes_cache:
            raise ValueError("a recurrent state has one writer: a layer cannot read another layer's state")
        n = x.shape[0]
        z = ctx.buffer("gla_z", (n, self.width), torch.float32)
        linear.logits(x, self.w_in, z, ctx)                          # float32 results in both precisions
        decay = ctx.buffer("gla_decay", (n, self.q_dim), torch.float32)
        o = ctx.buffer("gla_o", (n, self.v_dim), self.dtype)
        o_raw = ctx.buffer("gla_o_raw", (n, self.v_dim), torch.float32)
        # long runs of new tokens are cut into pieces that are scanned side by side
        piece, most = ops.recurrence_pieces(ctx.max_new, ctx.n_seqs, self.n_heads, self.head_dim, self.v_head_dim)
        scratch = None
        if piece:
            scratch = ctx.buffer("gla_pieces", (ctx.n_seqs * most * self.n_heads * self.head_dim
                                                * (self.v_head_dim + 1),), torch.float32)
        ops.gated_linear_attention(
            z, q_col=self.q_col, k_col=self.k_col, v_col=self.v_col, g_col=self.g_col, a_col=self.a_col, rank=self.rank,
            w2=self.w2, bias=self.decay_bias, tau=self.tau, q_scale=self.head_dim ** -0.5, decay=decay,
            norm_weight=self.norm, state=cache_layer.state, cu_seqlens=ctx.cu_seqlens, seq_slot=ctx.seq_slot, out=o,
            n_seqs=ctx.n_seqs, heads=self.n_heads, dim=self.head_dim, vdim=self.v_head_dim, eps=self.eps,
            out_scale=self.out_scale, o_raw=o_raw, piece=piece, max_pieces=most, scratch=scratch, longest_run=ctx.max_new)
        linear.into_residual(o, self.w_o, residual, ctx)
