"""A weighted sum over depth: what a layer hands on is a learned combination of the embedding's output and of the
results of all layers up to and including itself."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import DepthMix
from .registry import register
from .spec import TensorSpec


@register("depth", "weighted_depth_sum")
class WeightedDepthSum(DepthMix):
    """With X_0 the embedding's output and X_(j+1) the result of the j-th layer run, the run `index` hands on
    sum over j = 0 .. index + 1 of w[j] * X_j, w being this layer's tensor of index + 2 numbers (`weight_name` below the
    part's prefix).  X_(index+1) is the layer's result computed from what the run before handed on.  The results of a
    step's tokens are kept in a float32 scratch [entries, tokens, hidden] (`entries` = layer runs + 1); the last run
    stores nothing, since nobody reads it."""

    def __init__(self, *, index: int, entries: int, weight_name: str = "weight", hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if not 0 <= index < entries - 1:
            raise ValueError(f"weighted_depth_sum: run {index} of {entries - 1}")
        self.index, self.entries = int(index), int(entries)
        self.weight_name = weight_name
        self.weight = None

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.index + 2,), role="vector", init="unit_last")}

    def set_tensors(self, tensors):
        self.weight = tensors[self.weight_name].contiguous()

    def get_tensors(self):
        return {self.weight_name: self.weight}

    def _history(self, ctx, stream):
        return ctx.buffer("depth_history", (self.entries, stream.shape[0], stream.shape[1]), torch.float32)

    def enter(self, stream, ctx):
        if self.index == 0:
            self._history(ctx, stream)[0].copy_(stream)

    def fused(self, ctx, stream):
        return {"history": self._history(ctx, stream), "depth_w": self.weight, "depth_index": self.index,
                "store_result": self.index + 2 < self.entries}

    def leave(self, stream, ctx):
        ops.stream_update(stream, **self.fused(ctx, stream))
