"""The gated delta rule: a matrix state per head that is decayed, corrected towards the new value along the key, and
read by the query."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import StateRequest
from ..kernels import linear, ops
from .base import Mixer
from .registry import register
from .spec import TensorSpec


@register("mixer", "gated_delta_rule")
class GatedDeltaRule(Mixer):
    """q, k [n_kv_heads, head_dim] and v [n_heads, v_head_dim] are projections of the input that pass a short causal
    convolution per channel (taps [channels, K], the last column the current token's, no bias) and silu; q and k are
    then made unit vectors per head, x / sqrt(sum x^2 + 1e-6), q also times head_dim^(-1/2); head h reads the q/k head
    h // (n_heads / n_kv_heads).  With beta = sigmoid(W_b x) and g = exp(-exp(A_log) softplus(W_a x + dt_bias)), one of
    each per head:

        S <- g S;    u = beta (v - S^T k);    S <- S + k u^T;    o = S^T q            S: [head_dim, v_head_dim], float32

    so the read-out sees the token's own write.  Every head's o is RMS-normed over v_head_dim with one weight shared by
    the heads, multiplied by silu(W_g x) (heads side by side) and projected back.  State and the convolutions' last
    K - 1 inputs live in the slot's state area and are carried from step to step.  All projections run as one product
    with float32 results; everything up to the output projection is float32 in both precisions.  `out_scale`
    multiplies the mixer's result (in the norm).  `names` gives the tensors' names below the prefix."""

    _NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "q_conv": "q_conv1d.weight",
              "k_conv": "k_conv1d.weight", "v_conv": "v_conv1d.weight", "beta": "b_proj.weight", "a": "a_proj.weight",
              "dt_bias": "dt_bias", "A_log": "A_log", "gate": "g_proj.weight", "norm": "o_norm.weight", "o": "o_proj.weight"}

    def __init__(self, *, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, conv: int, eps: float,
                 out_scale: float = 1.0, names: dict | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} query/key heads")
        if conv < 1:
            raise ValueError(f"a convolution has at least one tap, found {conv}")
        self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim = int(n_heads), int(n_kv_heads), int(head_dim), int(v_head_dim)
        self.taps, self.eps, self.out_scale = int(conv), float(eps), float(out_scale)
        self.qk_dim, self.v_dim = self.n_kv_heads * self.head_dim, self.n_heads * self.v_head_dim
        self.conv_ch = 2 * self.qk_dim + self.v_dim
        # the projection's columns: q | k | v | gate | beta | a
        self.gate_col = self.conv_ch
        self.beta_col = self.gate_col + self.v_dim
        self.a_col = self.beta_col + self.n_heads
        self.width = self.a_col + self.n_heads
        self.names = dict(self._NAMES, **(names or {}))
        self.w_in = self.w_o = self.w_conv = self.dt_bias = self.a_log = self.norm = None

    def tensor_specs(self):
        h, nm, K = self.hidden_size, self.names, self.taps
        return {
            nm["q"]: TensorSpec((self.qk_dim, h)), nm["k"]: TensorSpec((self.qk_dim, h)), nm["v"]: TensorSpec((self.v_dim, h)),
            nm["q_conv"]: TensorSpec((self.qk_dim, K), role="vector"), nm["k_conv"]: TensorSpec((self.qk_dim, K), role="vector"),
            nm["v_conv"]: TensorSpec((self.v_dim, K), role="vector"),
            nm["beta"]: TensorSpec((self.n_heads, h)), nm["a"]: TensorSpec((self.n_heads, h)),
            nm["dt_bias"]: TensorSpec((self.n_heads,), role="vector"), nm["A_log"]: TensorSpec((self.n_heads,), role="vector"),
            nm["gate"]: TensorSpec((self.v_dim, h)), nm["norm"]: TensorSpec((self.v_head_dim,), role="vector", init="ones"),
            nm["o"]: TensorSpec((h, self.v_dim)),
        }

    def set_tensors(self, tensors):
        nm = self.names
        self.w_in = linear.Weight(torch.cat([tensors[nm[n]] for n in ("q", "k", "v", "gate", "beta", "a")], dim=0))
        self.w_conv = torch.cat([tensors[nm["q_conv"]], tensors[nm["k_conv"]], tensors[nm["v_conv"]]], dim=0).contiguous()
        self.dt_bias, self.a_log = tensors[nm["dt_bias"]].contiguous(), tensors[nm["A_log"]].contiguous()
        self.norm = tensors[nm["norm"]].contiguous()
        self.w_o = linear.Weight(tensors[nm["o"]])

    def get_tensors(self):
        nm, qk, w, c = self.names, self.qk_dim, self.w_in.t, self.w_conv
        return {nm["q"]: w[:qk], nm["k"]: w[qk:2 * qk], nm["v"]: w[2 * qk:self.conv_ch],
                nm["gate"]: w[self.gate_col:self.beta_col], nm["beta"]: w[self.beta_col:self.a_col], nm["a"]: w[self.a_col:],
                nm["q_conv"]: c[:qk], nm["k_conv"]: c[qk:2 * qk], nm["v_conv"]: c[2 * qk:],
                nm["dt_bias"]: self.dt_bias, nm["A_log"]: self.a_log, nm["norm"]: self.norm, nm["o"]: self.w_o.t}

    def cache_request(self):
        return (StateRequest((self.n_heads, self.head_dim, self.v_head_dim), torch.float32),
                StateRequest((self.taps - 1, self.conv_ch), torch.float32))

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        if not writes_cache:
            raise ValueError("a recurrent state has one writer: a layer cannot read another layer's state")
        matrix, carried = cache_layer.parts
        n, H, G = x.shape[0], self.n_heads, self.n_kv_heads
        z = ctx.buffer("scan_z", (n, self.width), torch.float32)
        linear.logits(x, self.w_in, z, ctx)                            # float32 results in both precisions
        u = ctx.buffer("scan_u", (n, self.conv_ch + 2 * H), torch.float32)
        ops.scan_prepare(z, conv_col=0, conv_ch=self.conv_ch, taps=self.w_conv, conv_bias=None, conv_state=carried.state,
                         unit_heads=2 * G, unit_dim=self.head_dim, scaled_heads=G, unit_scale=self.head_dim ** -0.5, heads=H,
                         decay_col=self.a_col, step_col=self.beta_col, a_log=self.a_log, dt_bias=self.dt_bias, out=u,
                         cu_seqlens=ctx.cu_seqlens, token_seq=ctx.token_seq, seq_slot=ctx.seq_slot, n_seqs=ctx.n_seqs)
        o = ctx.buffer("scan_o", (n, self.v_dim), torch.float32)
        ops.state_scan(u, matrix.state, o, ctx.cu_seqlens, ctx.seq_slot, n_seqs=ctx.n_seqs, heads=H, groups=G,
                       dim=self.head_dim, vdim=self.v_head_dim, q_col=0, k_col=self.qk_dim, v_col=2 * self.qk_dim,
                       decay_col=self.conv_ch, step_col=self.conv_ch + H, delta=True, longest_run=ctx.max_new)
        normed = ctx.buffer("scan_normed", (n, self.v_dim), self.dtype)
        ops.gated_group_norm(o, z, self.gate_col, self.norm, normed, groups=H, group_size=self.v_head_dim,
                             gate_first=False, eps=self.eps, out_scale=self.out_scale)
        linear.into_residual(normed, self.w_o, residual, ctx)
