"""Feed-forwards without biases: SwiGLU (mlp.rs:31-46), down( silu(gate x) * (up x) ), the same with another gate
activation and a factor on the result (`gated_dense`), the bounded gated
form down( g sigmoid(alpha g) (u + shift) ) with g = min(gate x, limit), u = clamp(up x, -limit, limit), and the
ungated form down( act(up x) ) with a learned activation."""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from .base import FeedForward
from .registry import register
from .spec import TensorSpec


@register("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, *, intermediate_size: int, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.intermediate_size = intermediate_size
        self.w_gate = self.w_up = self.w_down = None

    def tensor_specs(self):
        i, h = self.intermediate_size, self.hidden_size
        return {
            "gate_proj.weight": TensorSpec((i, h)),
            "up_proj.weight": TensorSpec((i, h)),
            "down_proj.weight": TensorSpec((h, i)),
        }

    def set_tensors(self, tensors):
        self.w_gate = linear.Weight(tensors["gate_proj.weight"])
        self.w_up = linear.Weight(tensors["up_proj.weight"])
        self.w_down = linear.Weight(tensors["down_proj.weight"])

    def get_tensors(self):
        return {"gate_proj.weight": self.w_gate.t, "up_proj.weight": self.w_up.t, "down_proj.weight": self.w_down.t}

    def forward(self, x, residual, ctx):
        act = ctx.buffer("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        # gate and up in one pass over x, SiLU-gate in the epilogue (mlp.rs:35-43)
        linear.gated(x, self.w_gate, self.w_up, act, ctx)
        # down projection added onto the residual stream (mlp.rs:45, transformer.rs:47)
        linear.into_residual(act, self.w_down, residual, ctx)


@register("feed_forward", "bounded_glu")
class BoundedGLU(FeedForward):
    """y = g * sigmoid(alpha * g) * (u + shift) with g = min(W_gate x, limit) and u = clamp(W_up x, -limit, limit);
    out = W_down y.  The activation is the gated epilogue of the gate / up contraction with these three
    constants (float32 arithmetic on the accumulators).  `names`: gate, up, down below the part's prefix."""

    _NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}

    def __init__(self, *, intermediate_size: int, limit: float, alpha: float = 1.702, shift: float = 1.0,
                 out_scale: float = 1.0, names: dict | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if not limit > 0:
            raise ValueError(f"the bound of a bounded gate is positive, found {limit}")
        self.intermediate_size = intermediate_size
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.out_scale = float(out_scale)           # a factor on the part's result, applied with the gate in float32
        self.names = dict(self._NAMES, **(names or {}))
        self.form = torch.tensor([self.alpha, self.limit, self.shift, 0.0, self.out_scale], dtype=torch.float32,
                                 device=self.device)
        self.w_gate = self.w_up = self.w_down = None

    def tensor_specs(self):
        i, h, nm = self.intermediate_size, self.hidden_size, self.names
        return {nm["gate"]: TensorSpec((i, h)), nm["up"]: TensorSpec((i, h)), nm["down"]: TensorSpec((h, i))}

    def set_tensors(self, tensors):
        nm = self.names
        self.w_gate = linear.Weight(tensors[nm["gate"]])
        self.w_up = linear.Weight(tensors[nm["up"]])
        self.w_down = linear.Weight(tensors[nm["down"]])

    def get_tensors(self):
        nm = self.names
        return {nm["gate"]: self.w_gate.t, nm["up"]: self.w_up.t, nm["down"]: self.w_down.t}

    def forward(self, x, residual, ctx):
        act = ctx.buffer("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        linear.gated(x, self.w_gate, self.w_up, act, ctx, form=self.form)
        linear.into_residual(act, self.w_down, residual, ctx)


@register("feed_forward", "gated_dense")
class GatedDense(FeedForward):
    """out = out_scale * W_down (act(W_gate x) * (W_up x)) with `activation` "silu" or "gelu_tanh"
    (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), computed as z sigmoid(2 sqrt(2/pi) z (1 + 0.044715 z^2))).
    The activation and the factor are the gated epilogue of the gate / up contraction (float32 arithmetic on the
    accumulators).  `names`: gate, up, down below the part's prefix."""

    _NAMES = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
    ACTIVATIONS = {"silu": (1.0, 0.0), "gelu_tanh": (ops.GELU_TANH_ALPHA, ops.GELU_TANH_CUBIC)}

    def __init__(self, *, intermediate_size: int, activation: str = "silu", out_scale: float = 1.0,
                 names: dict | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"gated_dense: unknown activation {activation!r}; known: {', '.join(self.ACTIVATIONS)}")
        self.intermediate_size, self.activation, self.out_scale = int(intermediate_size), activation, float(out_scale)
        self.names = dict(self._NAMES, **(names or {}))
        alpha, cubic = self.ACTIVATIONS[activation]
        self.form = torch.tensor([alpha, float("inf"), 0.0, cubic, self.out_scale], dtype=torch.float32, device=self.device)
        self.w_gate = self.w_up = self.w_down = None

    def tensor_specs(self):
        i, h, nm = self.intermediate_size, self.hidden_size, self.names
        return {nm["gate"]: TensorSpec((i, h)), nm["up"]: TensorSpec((i, h)), nm["down"]: TensorSpec((h, i))}

    def set_tensors(self, tensors):
        nm = self.names
        self.w_gate = linear.Weight(tensors[nm["gate"]])
        self.w_up = linear.Weight(tensors[nm["up"]])
        self.w_down = linear.Weight(tensors[nm["down"]])

    def get_tensors(self):
        nm = self.names
        return {nm["gate"]: self.w_gate.t, nm["up"]: self.w_up.t, nm["down"]: self.w_down.t}

    def forward(self, x, residual, ctx):
        act = ctx.buffer("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        linear.gated(x, self.w_gate, self.w_up, act, ctx, form=self.form)
        linear.into_residual(act, self.w_down, residual, ctx)


@register("feed_forward", "dense_act")
class DenseActivation(FeedForward):
    """out = W_down act(W_up x), no gate.  `activation` "xielu": with the two learned numbers p, q of the tensor `act`,
    act(z) = softplus(p) z^2 + z / 2 for z > 0 and (1/2 + softplus(q)) (e^z - 1 - z) + z / 2 otherwise, applied to
    the up projection's float32 accumulators in that product's epilogue; p and q are read on the device.  `names`: up, down, act below the prefix."""

    _NAMES = {"up": "up_proj.weight", "down": "down_proj.weight", "act": "act"}
    ACTIVATIONS = ("xielu",)

    def __init__(self, *, intermediate_size: int, activation: str = "xielu", names: dict | None = None,
                 hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"dense_act: unknown activation {activation!r}; known: {', '.join(self.ACTIVATIONS)}")
        self.intermediate_size, self.activation = int(intermediate_size), activation
        self.names = dict(self._NAMES, **(names or {}))
        self.w_up = self.w_down = self.act = None

    def tensor_specs(self):
        i, h, nm = self.intermediate_size, self.hidden_size, self.names
        return {nm["up"]: TensorSpec((i, h)), nm["down"]: TensorSpec((h, i)), nm["act"]: TensorSpec((2,), role="vector")}

    def set_tensors(self, tensors):
        nm = self.names
        self.w_up, self.w_down = linear.Weight(tensors[nm["up"]]), linear.Weight(tensors[nm["down"]])
        self.act = tensors[nm["act"]].contiguous()

    def get_tensors(self):
        nm = self.names
        return {nm["up"]: self.w_up.t, nm["down"]: self.w_down.t, nm["act"]: self.act}

    def forward(self, x, residual, ctx):
        act = ctx.buffer("ffn_act", (x.shape[0], self.intermediate_size), self.dtype)
        linear.activated(x, self.w_up, act, ctx, self.act)
        linear.into_residual(act, self.w_down, residual, ctx)
