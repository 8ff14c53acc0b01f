"""Rotary position encoding, with base and pairing as parameters (rope.rs:42-98)."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import PositionEncoding
from .registry import register

_STYLES = {"half": 0, "interleaved": 1}


def interpolated_frequencies(rot_dims: int, base: float, *, factor: float, original: float, fast: float, slow: float):
    """(frequencies float64 [rot_dims / 2], magnitude) of a rotation whose slow channels are interpolated (the YaRN form
    of context extension).  With f_i = base^(-2i/rot_dims) and c(t) = rot_dims ln(original / (2 pi t)) / (2 ln base) the
    channel whose wave turns t times over the original context: lo = max(floor(c(fast)), 0), hi = min(ceil(c(slow)),
    rot_dims - 1), ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); the frequency is f_i / factor * ramp_i +
    f_i (1 - ramp_i), and cos and sin are multiplied by 0.1 ln(factor) + 1."""
    half = rot_dims // 2
    i = np.arange(half, dtype=np.float64)
    f = np.power(np.float64(base), -2.0 * i / np.float64(rot_dims))

    def channel(turns):
        return rot_dims * np.log(np.float64(original) / (2.0 * np.pi * np.float64(turns))) / (2.0 * np.log(np.float64(base)))

    lo = max(int(np.floor(channel(fast))), 0)
    hi = min(int(np.ceil(channel(slow))), rot_dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / np.float64(factor) * ramp + f * (1.0 - ramp), 0.1 * float(np.log(np.float64(factor))) + 1.0


def rope_tables(head_dim: int, base: float, n_positions: int, exact_angles: bool = False, scaling_factor: float = 1.0,
                interpolation: dict | None = None):
    """cos, sin as float32 [n_positions, head_dim/2], built the way rope.rs:47-55 does:
    exponent = 2i/dim, theta = 1/base^exponent and angle = pos*theta are 32-bit numbers
    (the power is taken in float64 and rounded once); cos and sin are taken of the 32-bit
    angle in float64 and rounded once.  With exact_angles frequency and angle stay float64 and
    only cos and sin are rounded.  Every frequency is divided by scaling_factor (linear position scaling).
    `interpolation` (factor, original, fast, slow): the frequencies and the magnitude of `interpolated_frequencies`."""
    half = head_dim // 2
    if interpolation is not None:
        # frequencies of their own per channel and a magnitude on cos and sin; angles in float64, rounded once
        theta, magnitude = interpolated_frequencies(head_dim, base, **interpolation)
        angle = np.arange(n_positions, dtype=np.float64)[:, None] * (theta / np.float64(scaling_factor))[None, :]
        return (magnitude * np.cos(angle)).astype(np.float32), (magnitude * np.sin(angle)).astype(np.float32)
    if exact_angles:
        theta = np.power(np.float64(base), -2.0 * np.arange(half, dtype=np.float64) / np.float64(head_dim))
        theta = theta / np.float64(scaling_factor)
        angle = np.arange(n_positions, dtype=np.float64)[:, None] * theta[None, :]
        return np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    exponent = (2 * np.arange(half)).astype(np.float32) / np.float32(head_dim)
    theta = (1.0 / np.power(np.float64(np.float32(base)), exponent.astype(np.float64))).astype(np.float32)
    if scaling_factor != 1.0:
        theta = (theta / np.float32(scaling_factor)).astype(np.float32)
    pos = np.arange(n_positions, dtype=np.float32)
    angle = (pos[:, None] * theta[None, :]).astype(np.float32)
    cos = np.cos(angle.astype(np.float64)).astype(np.float32)
    sin = np.sin(angle.astype(np.float64)).astype(np.float32)
    return cos, sin


@register("position", "rope")
class RotaryEncoding(PositionEncoding):
    """Rotates every q head and every k head by the angles of the token's absolute
    position (attention.rs:78-87); v is not rotated.  style "interleaved" pairs (2i, 2i+1)
    as rope.rs:92-96 does; "half" pairs (i, i + dim/2).  `rot_dims` < head_dim rotates only
    the first rot_dims channels of every head (frequencies base^(-2i/rot_dims), pairs within
    them) and lets the rest pass.  `scaling_factor` divides every frequency (linear position scaling).
    `interpolation` (a dict factor, original, fast, slow): slow channels are interpolated and cos and sin get a
    magnitude (`interpolated_frequencies`); the tables hold it, the kernels are the same."""

    def __init__(self, *, head_dim: int, base: float, style: str = "half", rot_dims: int | None = None,
                 exact_angles: bool = False, scaling_factor: float = 1.0, interpolation: dict | None = None,
                 hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if style not in _STYLES:
            raise ValueError(f"rope style must be one of {sorted(_STYLES)}, found {style!r}")
        rot = head_dim if rot_dims is None else int(rot_dims)
        if rot % 2 or not 0 < rot <= head_dim:
            raise ValueError(f"rope rotates an even number of channels, at most head_dim {head_dim}; found {rot}")
        self.head_dim = head_dim
        self.rot_dims = rot
        self.base = float(base)
        self.style = _STYLES[style]
        self.exact_angles = bool(exact_angles)
        self.scaling_factor = float(scaling_factor)
        if not self.scaling_factor > 0:
            raise ValueError(f"a rope scaling factor is positive, found {scaling_factor}")
        self.interpolation = None
        if interpolation is not None:
            missing = [k for k in ("factor", "original", "fast", "slow") if k not in interpolation]
            if missing:
                raise ValueError(f"rope interpolation lacks {missing}")
            self.interpolation = {k: float(interpolation[k]) for k in ("factor", "original", "fast", "slow")}
            if not (self.interpolation["factor"] > 0 and self.interpolation["original"] > 0 and
                    self.interpolation["fast"] > 0 and self.interpolation["slow"] > 0 and self.base > 1):
                raise ValueError(f"rope interpolation needs positive constants and a base above 1, found {interpolation}")
        self.cos = self.sin = None

    @property
    def partial(self) -> bool:
        return self.rot_dims != self.head_dim

    def prepare(self, max_positions: int) -> None:
        if self.cos is None or self.cos.shape[0] < max_positions:
            cos, sin = rope_tables(self.rot_dims, self.base, max_positions, self.exact_angles, self.scaling_factor,
                                   self.interpolation)
            self.cos = torch.from_numpy(cos).contiguous().to(self.device)
            self.sin = torch.from_numpy(sin).contiguous().to(self.device)

    def apply_and_store(self, qkv, ctx, cache_layer, *, n_heads, n_kv_heads, head_dim, write_kv, v_head_dim=None):
        if self.cos is None or self.cos.shape[0] < ctx.max_len:
            raise RuntimeError("rope tables do not cover the step's positions; call prepare() first")
        ops.rope_cache_write(qkv, self.cos, self.sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot,
                             ctx.page_table, cache_layer.k, cache_layer.v, n_heads=n_heads,
                             n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=ctx.page_size,
                             style=self.style, write_kv=write_kv, rot_dims=self.rot_dims, v_head_dim=v_head_dim)

    def apply_normed_and_store(self, qkv, ctx, cache_layer, *, n_heads, n_kv_heads, head_dim, write_kv, q_weight,
                               k_weight, eps, values_from_keys=False, v_head_dim=None):
        """The same after an RMS norm of every q and k head (weights shared by the heads; None: no norm); with
        values_from_keys the cached values are the keys as projected, before norm and rotation."""
        if self.cos is None or self.cos.shape[0] < ctx.max_len:
            raise RuntimeError("rope tables do not cover the step's positions; call prepare() first")
        ops.rope_normed_cache_write(qkv, self.cos, self.sin, q_weight, k_weight, eps, ctx.token_pos, ctx.token_seq,
                                    ctx.seq_slot, ctx.page_table, cache_layer.k, cache_layer.v, n_heads=n_heads,
                                    n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=ctx.page_size, style=self.style,
                                    write_kv=write_kv, rot_dims=self.rot_dims, v_head_dim=v_head_dim,
                                    values_from_keys=values_from_keys)

    def apply_and_store_from_accumulators(self, acc, bias, q_out, ctx, cache_layer, *, n_heads, n_kv_heads,
                                          head_dim, write_kv):
        """The same from float32 accumulators of a K-split projection (bias not yet added): q goes
        to q_out, and `acc` is left zeroed."""
        if self.cos is None or self.cos.shape[0] < ctx.max_len:
            raise RuntimeError("rope tables do not cover the step's positions; call prepare() first")
        ops.rope_cache_write_acc(acc, bias, q_out, self.cos, self.sin, ctx.token_pos, ctx.token_seq, ctx.seq_slot,
                                 ctx.page_table, cache_layer.k, cache_layer.v, n_heads=n_heads,
                                 n_kv_heads=n_kv_heads, head_dim=head_dim, page_size=ctx.page_size,
                                 style=self.style, write_kv=write_kv)


@register("position", "unrotated")
class Unrotated(PositionEncoding):
    """No rotation: queries stay as projected, keys and values go into the cache as they are.  For mixers whose positions
    enter elsewhere (a bias on the scores that depends on the distance), or nowhere."""

    partial = True          # the usual fused paths rotate whole heads

    def apply_and_store(self, qkv, ctx, cache_layer, *, n_heads, n_kv_heads, head_dim, write_kv, v_head_dim=None):
        if not write_kv:
            return
        ops.rope_cache_write(qkv, None, None, ctx.token_pos, ctx.token_seq, ctx.seq_slot, ctx.page_table, cache_layer.k,
                             cache_layer.v, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
                             page_size=ctx.page_size, style=0, write_kv=True, rot_dims=0, v_head_dim=v_head_dim)

    def apply_normed_and_store(self, qkv, ctx, cache_layer, *, n_heads, n_kv_heads, head_dim, write_kv, q_weight,
                               k_weight, eps, values_from_keys=False, v_head_dim=None):
        """The RMS norm of every q and k head (weights shared by the heads; None: no norm) without any rotation; keys
        and values go into the cache."""
        ops.rope_normed_cache_write(qkv, None, None, q_weight, k_weight, eps, ctx.token_pos, ctx.token_seq, ctx.seq_slot,
                                    ctx.page_table, cache_layer.k, cache_layer.v, n_heads=n_heads, n_kv_heads=n_kv_heads,
                                    head_dim=head_dim, page_size=ctx.page_size, style=0, write_kv=write_kv, rot_dims=0,
                                    v_head_dim=v_head_dim, values_from_keys=values_from_keys)
