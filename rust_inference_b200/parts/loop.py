"""What happens to the stream where a pass over a run of layers begins."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import StreamStep
from .registry import register
from .spec import TensorSpec


@register("stream", "pass_entry")
class PassEntry(StreamStep):
    """A run of layers that is passed `passes` times in a row with the same weights: right before the first layer of
    pass t the stream gets, in this order, the embedding's output once more (the stream as it was before the model's
    first layer; passes t > 0 only, with `readd_input`) and the learned vector step[t] (tensor `weight_name` below the
    part's prefix, [passes, hidden]).  The embedding's output of the step's tokens is kept in a float32 scratch from
    `begin` on, where anything reads it again."""

    def __init__(self, *, passes: int, readd_input: bool = True, weight_name: str = "step", hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if passes <= 0:
            raise ValueError(f"a run of layers is passed at least once, found {passes}")
        self.passes, self.readd_input, self.weight_name = int(passes), bool(readd_input), weight_name
        self.step = None

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.passes, self.hidden_size), role="vector")}

    def set_tensors(self, tensors):
        self.step = tensors[self.weight_name].contiguous()

    def get_tensors(self):
        return {self.weight_name: self.step}

    def _kept(self, ctx, stream):
        return ctx.buffer("pass_entry_input", tuple(stream.shape), torch.float32)

    def begin(self, stream, ctx):
        if self.readd_input and self.passes > 1:
            self._kept(ctx, stream).copy_(stream)

    def forward(self, stream, ctx, arg):
        if not 0 <= arg < self.passes:
            raise ValueError(f"pass {arg} of {self.passes}")
        again = self._kept(ctx, stream) if (self.readd_input and arg > 0) else None
        ops.stream_add(stream, again, self.step[arg])
