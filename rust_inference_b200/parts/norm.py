"""Norms of the hidden stream: RMSNorm with eps as a parameter (rmsnorm.rs:4-29, math.rs:237-256), a layer norm, and a
norm without statistics (a scaled tanh of every element)."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm
from .registry import register
from .spec import TensorSpec


@register("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x * (1 / sqrt(mean(x^2) + eps)) * weight; statistics in float32.  The weight
    multiplies directly, unless `unit_offset` says that the file holds weight - 1: then the
    factor is 1 + weight (formed once, in float32, when the weight arrives).  `weight_name` is
    the tensor's name below the part's prefix."""

    def __init__(self, *, eps: float, unit_offset: bool = False, weight_name: str = "weight", hidden_size: int,
                 dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.eps = float(eps)
        self.unit_offset = bool(unit_offset)
        self.weight_name = weight_name
        self.weight = self.factor = None

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.hidden_size,), role="vector",
                                             init="zeros" if self.unit_offset else "ones")}

    def set_tensors(self, tensors):
        self.weight = tensors[self.weight_name]
        self.factor = self.weight + 1.0 if self.unit_offset else self.weight

    def get_tensors(self):
        return {self.weight_name: self.weight}

    def forward(self, x, out, rows=None):
        return ops.rmsnorm(x, self.factor, self.eps, out, rows)

    # up to so many rows two norms of the same stream run as one kernel (a launch costs more than the rows)
    PAIR_MAX_ROWS = 128

    def forward_with(self, other, x, out, out_other) -> bool:
        """out = self(x) and out_other = other(x) in one kernel, if `other` is an RMS norm with the same eps
        and the step is small; False (nothing done) otherwise."""
        if not isinstance(other, RMSNorm) or other.eps != self.eps or out.shape[0] > self.PAIR_MAX_ROWS:
            return False
        ops.rmsnorm_pair(x, self.factor, other.factor, self.eps, out, out_other)
        return True


@register("norm", "layernorm")
class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * weight, var the mean of the squared deviations; no bias;
    statistics in float32.  `weight_name` is the tensor's name below the part's prefix."""

    def __init__(self, *, eps: float, weight_name: str = "weight", hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.eps = float(eps)
        self.weight_name = weight_name
        self.weight = None

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.hidden_size,), role="vector", init="ones")}

    def set_tensors(self, tensors):
        self.weight = tensors[self.weight_name]

    def get_tensors(self):
        return {self.weight_name: self.weight}

    def forward(self, x, out, rows=None):
        return ops.layernorm(x, self.weight, self.eps, out, rows)


@register("norm", "dynamic_tanh")
class DynamicTanh(Norm):
    """y = tanh(alpha * x) * weight + bias: no mean and no variance is computed, every element is squashed by itself
    (alpha is one learned number).  float32 arithmetic.  `weight_name`, `bias_name` and `alpha_name` are the tensors'
    names below the part's prefix.  Because no element needs its row, this norm joins the elementwise passes over the
    stream (`fused()` gives the three tensors such a pass needs)."""

    def __init__(self, *, weight_name: str = "weight", bias_name: str = "bias", alpha_name: str = "alpha",
                 hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.weight_name, self.bias_name, self.alpha_name = weight_name, bias_name, alpha_name
        self.weight = self.bias = self.alpha = None

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.hidden_size,), role="vector", init="ones"),
                self.bias_name: TensorSpec((self.hidden_size,), role="vector", init="zeros"),
                self.alpha_name: TensorSpec((), role="vector", init="ones")}

    def set_tensors(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()
        self.bias = tensors[self.bias_name].contiguous()
        self.alpha = tensors[self.alpha_name].reshape(1).contiguous()

    def get_tensors(self):
        return {self.weight_name: self.weight, self.bias_name: self.bias, self.alpha_name: self.alpha.reshape(())}

    def fused(self):
        return self.weight, self.bias, self.alpha

    def forward(self, x, out, rows=None):
        return ops.dyt_norm(x, self.weight, self.bias, self.alpha, out, rows)
