"""A selective state space with one scalar decay per head and token (the form whose authors call it state-space
duality): a matrix state per head, written by an outer product and read by a matrix-vector product."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import StateRequest
from ..kernels import linear, ops
from .base import Mixer
from .registry import register
from .spec import TensorSpec


@register("mixer", "selective_state_space")
class SelectiveStateSpace(Mixer):
    """One projection of the input gives, side by side, a gate z [inner], the values x [inner], the write vectors
    B [groups, state], the read vectors C [groups, state] and a raw step per head (inner = heads * v_head_dim).
    x, B and C pass a short causal convolution per channel (taps [channels, K], the last column the current
    token's, a bias if `conv_bias`) and silu.  With dt = softplus(raw + dt_bias) and a = exp(-exp(A_log) dt), per head
    (head h reads group h // (heads / groups)):

        S <- a S + B (dt x)^T          y = S^T C + D x                      S: [state, v_head_dim], float32

    y (heads side by side) is multiplied by silu(z), RMS-normed in `norm_groups` equal parts with one weight per
    channel, and projected back.  The state and the convolution's last K - 1 inputs live in the slot's state area (two
    requests: the cache answers with two state layers), start at zero and are carried from step to step, so a prompt
    may be cut anywhere.  Projection results, convolution, decay, state and norm are float32 in both precisions.
    `out_scale` multiplies the mixer's result (in the norm).  `names` gives the tensors' names below the prefix."""

    _NAMES = {"in": "in_proj.weight", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "dt_bias": "dt_bias",
              "A_log": "A_log", "D": "D", "norm": "norm.weight", "o": "out_proj.weight"}

    def __init__(self, *, n_heads: int, v_head_dim: int, state: int, groups: int, conv: int, norm_groups: int, eps: float,
                 conv_bias: bool = True, out_scale: float = 1.0, names: dict | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if groups <= 0 or n_heads % groups:
            raise ValueError(f"{n_heads} heads are not a multiple of {groups} groups")
        self.n_heads, self.v_head_dim, self.state, self.groups = int(n_heads), int(v_head_dim), int(state), int(groups)
        self.inner = self.n_heads * self.v_head_dim
        if norm_groups <= 0 or self.inner % norm_groups:
            raise ValueError(f"{self.inner} channels do not split into {norm_groups} equal parts for the norm")
        if conv < 1:
            raise ValueError(f"a convolution has at least one tap, found {conv}")
        self.taps, self.norm_groups = int(conv), int(norm_groups)
        self.eps, self.out_scale, self.conv_bias = float(eps), float(out_scale), bool(conv_bias)
        self.conv_ch = self.inner + 2 * self.groups * self.state
        self.width = 2 * self.inner + 2 * self.groups * self.state + self.n_heads
        self.names = dict(self._NAMES, **(names or {}))
        self.w_in = self.w_o = self.w_conv = self.b_conv = self.dt_bias = self.a_log = self.skip = self.norm = None

    def tensor_specs(self):
        h, nm = self.hidden_size, self.names
        specs = {
            nm["in"]: TensorSpec((self.width, h)),
            nm["conv"]: TensorSpec((self.conv_ch, self.taps), role="vector"),
            nm["dt_bias"]: TensorSpec((self.n_heads,), role="vector"),
            nm["A_log"]: TensorSpec((self.n_heads,), role="vector"),
            nm["D"]: TensorSpec((self.n_heads,), role="vector", init="ones"),
            nm["norm"]: TensorSpec((self.inner,), role="vector", init="ones"),
            nm["o"]: TensorSpec((h, self.inner)),
        }
        if self.conv_bias:
            specs[nm["conv_bias"]] = TensorSpec((self.conv_ch,), role="vector")
        return specs

    def set_tensors(self, tensors):
        nm = self.names
        self.w_in, self.w_o = linear.Weight(tensors[nm["in"]]), linear.Weight(tensors[nm["o"]])
        self.w_conv = tensors[nm["conv"]].contiguous()
        self.b_conv = tensors[nm["conv_bias"]].contiguous() if self.conv_bias else None
        self.dt_bias, self.a_log = tensors[nm["dt_bias"]].contiguous(), tensors[nm["A_log"]].contiguous()
        self.skip, self.norm = tensors[nm["D"]].contiguous(), tensors[nm["norm"]].contiguous()

    def get_tensors(self):
        nm = self.names
        out = {nm["in"]: self.w_in.t, nm["conv"]: self.w_conv, nm["dt_bias"]: self.dt_bias, nm["A_log"]: self.a_log,
               nm["D"]: self.skip, nm["norm"]: self.norm, nm["o"]: self.w_o.t}
        if self.conv_bias:
            out[nm["conv_bias"]] = self.b_conv
        return out

    def cache_request(self):
        return (StateRequest((self.n_heads, self.state, self.v_head_dim), torch.float32),
                StateRequest((self.taps - 1, self.conv_ch), torch.float32))

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        if not writes_cache:
            raise ValueError("a recurrent state has one writer: a layer cannot read another layer's state")
        matrix, carried = cache_layer.parts
        n, H, gn = x.shape[0], self.n_heads, self.groups * self.state
        z = ctx.buffer("scan_z", (n, self.width), torch.float32)
        linear.logits(x, self.w_in, z, ctx)                            # float32 results in both precisions
        u = ctx.buffer("scan_u", (n, self.conv_ch + 2 * H), torch.float32)
        ops.scan_prepare(z, conv_col=self.inner, conv_ch=self.conv_ch, taps=self.w_conv, conv_bias=self.b_conv,
                         conv_state=carried.state, unit_heads=0, unit_dim=0, scaled_heads=0, unit_scale=1.0, heads=H,
                         decay_col=2 * self.inner + 2 * gn, step_col=-1, a_log=self.a_log, dt_bias=self.dt_bias, out=u,
                         cu_seqlens=ctx.cu_seqlens, token_seq=ctx.token_seq, seq_slot=ctx.seq_slot, n_seqs=ctx.n_seqs)
        y = ctx.buffer("scan_o", (n, self.inner), torch.float32)
        piece, max_pieces = ops.scan_pieces(ctx.max_new, ctx.n_seqs * H * -(-self.v_head_dim // 16))
        pieces = {}
        if piece:                      # a long run of new tokens: its pieces side by side, from zero and again from their start states
            pieces = {"piece": piece, "max_pieces": max_pieces,
                      "piece_state": ctx.buffer("scan_piece_state", (ctx.n_seqs, max_pieces, H, self.state, self.v_head_dim), torch.float32),
                      "piece_decay": ctx.buffer("scan_piece_decay", (ctx.n_seqs, max_pieces, H), torch.float32)}
        ops.state_scan(u, matrix.state, y, ctx.cu_seqlens, ctx.seq_slot, n_seqs=ctx.n_seqs, heads=H, groups=self.groups,
                       dim=self.state, vdim=self.v_head_dim, q_col=self.inner + gn, k_col=self.inner, v_col=0,
                       decay_col=self.conv_ch, step_col=self.conv_ch + H, delta=False, skip=self.skip,
                       longest_run=ctx.max_new, **pieces)
        normed = ctx.buffer("scan_normed", (n, self.inner), self.dtype)
        ops.gated_group_norm(y, z, 0, self.norm, normed, groups=self.norm_groups, group_size=self.inner // self.norm_groups,
                             gate_first=True, eps=self.eps, out_scale=self.out_scale)
        linear.into_residual(normed, self.w_o, residual, ctx)
