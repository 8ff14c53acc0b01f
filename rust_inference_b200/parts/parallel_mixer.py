"""Several mixers on the same input, their results summed with fixed factors."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer
from .registry import lookup, register
from .spec import PartSpec, TensorSpec


@register("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    """residual += sum_m scale_m * mixer_m(x).  `members` lists (PartSpec, scale) pairs; a member's
    tensors sit below its spec's prefix, its factor is handed to it as `out_scale` (members apply it to
    their result in float32, before their output projection), and its cache is the member of the same
    place in the layer's composite cache request: an attention member keeps keys and values, a
    recurrent one a state, both in one cache layer.

    `member_norm` = {"eps": e, "weight_name": name}: every member's result is RMS-normed over the model width with a
    plain weight of its own (the tensor `name` below the member's prefix) before it is scaled and added:
    residual += sum_m scale_m * rmsnorm(mixer_m(x)) * w_m.  A member then writes into a zeroed float32 buffer of its
    own, and one kernel norms and adds all of them."""

    def __init__(self, *, members, member_norm: dict | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.members = []
        self.member_norm = dict(member_norm) if member_norm else None
        if self.member_norm is not None and len(members) > 4:
            raise ValueError("parallel_mixers: at most four members are normed and added together")
        self.scales, self.norm_weights = [], []
        for spec, scale in members:
            if not isinstance(spec, PartSpec):
                raise TypeError("parallel_mixers: a member is a (PartSpec, scale) pair")
            inner_scale = 1.0 if self.member_norm is not None else float(scale)     # a norm would undo a factor before it
            part = lookup("mixer", spec.kind)(hidden_size=hidden_size, dtype=dtype, device=device,
                                              **dict(spec.params, out_scale=inner_scale))
            self.members.append((spec.prefix, part))
            self.scales.append(float(scale))
        if not self.members:
            raise ValueError("parallel_mixers: no members")
        self.graph_safe = all(getattr(p, "graph_safe", True) for _, p in self.members)

    def tensor_specs(self):
        out = {}
        for prefix, part in self.members:
            for local, ts in part.tensor_specs().items():
                if prefix + local in out:
                    raise ValueError(f"parallel_mixers: two members declare {prefix + local!r}")
                out[prefix + local] = ts
            if self.member_norm is not None:
                name = prefix + self.member_norm["weight_name"]
                if name in out:
                    raise ValueError(f"parallel_mixers: the member's norm weight {name!r} is a tensor of the member")
                out[name] = TensorSpec((self.hidden_size,), role="vector", init="ones")
        return out

    def set_tensors(self, tensors):
        for prefix, part in self.members:
            part.set_tensors({local: tensors[prefix + local] for local in part.tensor_specs()})
        if self.member_norm is not None:
            self.norm_weights = [tensors[prefix + self.member_norm["weight_name"]].contiguous() for prefix, _ in self.members]

    def get_tensors(self):
        out = {prefix + local: t for prefix, part in self.members for local, t in part.get_tensors().items()}
        if self.member_norm is not None:
            for (prefix, _), w in zip(self.members, self.norm_weights):
                out[prefix + self.member_norm["weight_name"]] = w
        return out

    def prepare(self, max_positions):
        for _, part in self.members:
            part.prepare(max_positions)

    def cache_request(self):
        return tuple(part.cache_request() for _, part in self.members)

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        if self.member_norm is None:
            for (_, part), sub in zip(self.members, cache_layer.parts):
                part.forward(x, residual, ctx, sub, writes_cache)
            return
        joined = []
        for m, ((_, part), sub) in enumerate(zip(self.members, cache_layer.parts)):
            own = ctx.zeroed_buffer(f"member_result_{m}", tuple(residual.shape), torch.float32)
            part.forward(x, own, ctx, sub, writes_cache)
            joined.append((own, None, self.norm_weights[m], self.scales[m]))
        ops.normed_sum(joined, residual, self.member_norm["eps"], accumulate=True)
