"""A routed mixture of gated feed-forward experts, with an optional always-on shared expert."""
from __future__ import annotations

import torch

from ..kernels import linear, ops
from .base import FeedForward
from .registry import register
from .spec import TensorSpec


@register("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """`n_experts` experts of the form down(silu(gate x) * (up x)), of which every token uses `top`.

    Router: s = sigmoid(W_router x) in float32; c = s + correction ranks the experts.  Experts e with the same
    e // (n_experts / n_groups) form a group, ranked by its top-2 sum of c; only the `group_keep` highest groups
    remain candidates (the rest are removed from the ranking, whatever the sign of their c).  The `top`
    candidates with the highest c run, weighted by s / (sum of the chosen s + 1e-20).  A shared expert of
    width `shared_size` (None: none) runs for every token and is added times sigmoid(w_sg . x).

    Other forms, as parameters: `router_kind` "softmax" (s = softmax(W_router x) over all router outputs instead of
    sigmoids); `normalise` False (the weights are the chosen s as they are); `identity` (so many more router outputs
    after the experts', which stand for experts without tensors whose output is their input x itself, times the
    weight); `expert_form` / `shared_form` (a dict with limit and optionally alpha, shift: the bounded gate
    g' sigmoid(alpha g') (u' + shift) of `bounded_glu` instead of SiLU); `shared_gate` False (the shared expert has no
    learned gate and is added as it is); `out_scale` (a factor on the part's whole result, applied in float32 as it
    joins the stream).

    Everything from the router to the sum runs on the device (`csrc/moe.cu`), so decode steps stay
    inside captured graphs.  Experts are kept stacked: gate, up [experts, ff, hidden], down [experts,
    hidden, ff].  `names` gives the tensors' names below the part's prefix; "{e}" is the expert's number."""

    _NAMES = {"router": "router.weight", "correction": "router.correction", "gate": "experts.{e}.gate_proj.weight",
              "up": "experts.{e}.up_proj.weight", "down": "experts.{e}.down_proj.weight",
              "shared_gate": "shared.gate_proj.weight", "shared_up": "shared.up_proj.weight",
              "shared_down": "shared.down_proj.weight", "shared_mix": "shared.mix.weight"}

    ROUTERS = ("sigmoid", "softmax")

    def __init__(self, *, n_experts: int, top: int, expert_size: int, n_groups: int = 1, group_keep: int = 1,
                 shared_size: int | None = None, names: dict | None = None, router_kind: str = "sigmoid",
                 normalise: bool = True, identity: int = 0, expert_form: dict | None = None,
                 shared_form: dict | None = None, shared_gate: bool = True, out_scale: float = 1.0,
                 hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        if router_kind not in self.ROUTERS:
            raise ValueError(f"routed_experts: unknown router {router_kind!r}; known: {', '.join(self.ROUTERS)}")
        if identity < 0 or (identity and n_groups != 1):
            raise ValueError(f"{identity} experts without tensors (not negative; not combined with groups)")
        if not 0 < top <= n_experts + identity:
            raise ValueError(f"{top} of {n_experts + identity} experts cannot be chosen")
        self.router_kind, self.normalise, self.identity = router_kind, bool(normalise), int(identity)
        self.shared_gate, self.out_scale = bool(shared_gate), float(out_scale)
        self.expert_form = self._form(expert_form, device)
        self.shared_form = self._form(shared_form, device)
        if n_groups <= 0 or n_experts % n_groups or not 0 < group_keep <= n_groups:
            raise ValueError(f"{n_experts} experts do not form {n_groups} equal groups of which {group_keep} are kept")
        if group_keep * (n_experts // n_groups) + identity < top:
            raise ValueError(f"{group_keep} groups of {n_experts // n_groups} experts cannot give {top} choices")
        self.n_experts, self.top, self.expert_size = n_experts, top, expert_size
        self.n_groups, self.group_keep = n_groups, group_keep
        self.shared_size = shared_size
        self.names = dict(self._NAMES, **(names or {}))
        self.router = self.correction = self.w_gate = self.w_up = self.w_down = None
        self.shared = self.shared_mix = None

    @staticmethod
    def _form(form, device):
        """The bounded gate's constants on the device (None: SiLU)."""
        if form is None:
            return None
        limit = float(form["limit"])
        if not limit > 0:
            raise ValueError(f"the bound of a bounded gate is positive, found {limit}")
        return torch.tensor([float(form.get("alpha", 1.702)), limit, float(form.get("shift", 1.0)), 0.0, 1.0],
                            dtype=torch.float32, device=device)

    def tensor_specs(self):
        h, f, nm = self.hidden_size, self.expert_size, self.names
        outputs = self.n_experts + self.identity
        specs = {nm["router"]: TensorSpec((outputs, h), role="vector"),
                 nm["correction"]: TensorSpec((outputs,), role="vector", init="zeros")}
        for e in range(self.n_experts):
            specs[nm["gate"].format(e=e)] = TensorSpec((f, h))
            specs[nm["up"].format(e=e)] = TensorSpec((f, h))
            specs[nm["down"].format(e=e)] = TensorSpec((h, f))
        if self.shared_size is not None:
            s = self.shared_size
            specs[nm["shared_gate"]] = TensorSpec((s, h))
            specs[nm["shared_up"]] = TensorSpec((s, h))
            specs[nm["shared_down"]] = TensorSpec((h, s))
            if self.shared_gate:
                specs[nm["shared_mix"]] = TensorSpec((1, h), role="vector")
        return specs

    def set_tensors(self, tensors):
        nm, n = self.names, self.n_experts
        self.router = tensors[nm["router"]].contiguous()
        self.correction = tensors[nm["correction"]].contiguous()
        self.w_gate = torch.stack([tensors[nm["gate"].format(e=e)] for e in range(n)]).contiguous()
        self.w_up = torch.stack([tensors[nm["up"].format(e=e)] for e in range(n)]).contiguous()
        self.w_down = torch.stack([tensors[nm["down"].format(e=e)] for e in range(n)]).contiguous()
        if self.shared_size is not None:
            self.shared = tuple(linear.Weight(tensors[nm[k]]) for k in ("shared_gate", "shared_up", "shared_down"))
            if self.shared_gate:
                self.shared_mix = tensors[nm["shared_mix"]].reshape(-1).contiguous()

    def get_tensors(self):
        nm = self.names
        out = {nm["router"]: self.router, nm["correction"]: self.correction}
        for e in range(self.n_experts):
            out[nm["gate"].format(e=e)] = self.w_gate[e]
            out[nm["up"].format(e=e)] = self.w_up[e]
            out[nm["down"].format(e=e)] = self.w_down[e]
        if self.shared_size is not None:
            out[nm["shared_gate"]], out[nm["shared_up"]], out[nm["shared_down"]] = (w.t for w in self.shared)
            if self.shared_gate:
                out[nm["shared_mix"]] = self.shared_mix.view(1, -1)
        return out

    # steps of more tokens than this run the experts' products on the tensor cores (tiles of 128 rows of one
    # expert, their weights streamed by TMA) when the sizes allow; the FFMA form is the 32-bit path and
    # the fallback for other sizes
    TENSOR_CORE_MIN_TOKENS = 0
    GATHER_IN_ARRANGE_PAIRS = 256       # up to so many (token, choice) pairs the arranging block also gathers their rows
    ROUTE_SPLIT_TOKENS, ROUTE_SPLIT_BLOCKS, ROUTE_SPLIT_MOST = 64, 148, 16     # steps of up to 64 tokens: the router's rows
    #                                     over up to 16 blocks per token, about one block per SM in all

    def _on_tensor_cores(self, x) -> bool:
        if x.dtype != torch.bfloat16 or x.shape[0] <= self.TENSOR_CORE_MIN_TOKENS:
            return False
        from ..kernels import tcgen05
        return (tcgen05.grouped_supports(x.dtype, self.w_gate) and tcgen05.grouped_supports(x.dtype, self.w_down)
                and self.hidden_size % 8 == 0)

    def route_cut(self, n: int, ctx) -> dict:
        """Keyword arguments of `ops.moe_route` for a step of n tokens: a step of few tokens cuts the router's rows over
        several blocks per token, so that more SMs than tokens read them (scratch from the step's workspace)."""
        outputs = self.router.shape[0] + (1 if self.shared_mix is not None else 0)
        if n > self.ROUTE_SPLIT_TOKENS:
            return {}
        split = min(self.ROUTE_SPLIT_MOST, self.ROUTE_SPLIT_BLOCKS // n, outputs // 4)
        if split <= 1:
            return {}
        return dict(split=split, split_sums=ctx.buffer("moe_route_sums", (n, self.router.shape[0] + 1), torch.float32),
                    split_count=ctx.zeroed_buffer("moe_route_count", (n,), torch.int32))

    def forward(self, x, residual, ctx):
        n, h, top, experts = x.shape[0], self.hidden_size, self.top, self.n_experts
        pairs = n * top
        ids = ctx.buffer("moe_ids", (n, top), torch.int32)
        weights = ctx.buffer("moe_weights", (n, top), torch.float32)
        gate = ctx.buffer("moe_shared_gate", (n,), torch.float32) if self.shared_mix is not None else None
        cut = self.route_cut(n, ctx)
        ops.moe_route(x, self.router, self.correction, ids, weights, top=top, groups=self.n_groups,
                      keep=self.group_keep, gate_weight=self.shared_mix, gate_out=gate,
                      softmax=self.router_kind == "softmax", normalise=self.normalise, **cut)
        fast = self._on_tensor_cores(x)
        if fast:
            from ..kernels import tcgen05
            rows = tcgen05.GROUPED_TILE_ROWS
        else:
            rows = ops.moe_tile_rows()
        offsets = ctx.buffer("moe_offsets", (experts + 1,), torch.int32)
        order = ctx.buffer("moe_order", (pairs,), torch.int32)
        tiles = ctx.buffer("moe_tiles", (2 * (-(-pairs // rows) + experts),), torch.int32)
        n_tiles = ctx.buffer("moe_n_tiles", (1,), torch.int32)
        place = ctx.buffer("moe_place", (pairs,), torch.int32) if fast else None
        # an expert's rows consecutive: the activations are gathered into the lists' order (by the arranging
        # kernel itself when the pairs are few); act and y stay in that order
        xs = ctx.buffer("moe_x_sorted", (pairs, h), self.dtype) if fast else None
        small = fast and pairs <= self.GATHER_IN_ARRANGE_PAIRS
        ops.moe_arrange(ids, pairs, experts, rows, offsets, order, tiles, n_tiles, place,
                        gather=(x, xs, top) if small else None)
        act = ctx.buffer("moe_act", (pairs, self.expert_size), self.dtype)
        y = ctx.buffer("moe_y", (pairs, h), torch.float32)
        if fast:
            if not small:
                ops.moe_gather(x, xs, order, n_pairs=pairs, top=top,
                               listed=offsets[experts:experts + 1] if self.identity else None)
            tcgen05.grouped_gemm(xs, self.w_gate, self.w_up, act, offsets, tiles, n_tiles, n_pairs=pairs,
                                 gate_form=self.expert_form)
            tcgen05.grouped_gemm(act, self.w_down, None, y, offsets, tiles, n_tiles, n_pairs=pairs)
        else:
            ops.moe_grouped_simt(x, self.w_gate, self.w_up, act, offsets, order, tiles, n_tiles, n_pairs=pairs, top=top,
                                 gate_form=self.expert_form)
            ops.moe_grouped_simt(act, self.w_down, None, y, offsets, order, tiles, n_tiles, n_pairs=pairs, top=top)
        shared_y = None
        if self.shared is not None:
            w_gate, w_up, w_down = self.shared
            sact = ctx.buffer("moe_shared_act", (n, self.shared_size), self.dtype)
            linear.gated(x, w_gate, w_up, sact, ctx, form=self.shared_form)
            shared_y = ctx.buffer("moe_shared_y", (n, h), torch.float32)
            linear.logits(sact, w_down, shared_y, ctx)
        # ids at or beyond the experts with tensors were left out of the lists: their rows are the input itself
        through = dict(ids=ids, x=x, n_real=experts) if self.identity else {}
        ops.moe_combine(residual, y, weights, top=top, shared_y=shared_y, gate=gate, place=place, scale=self.out_scale,
                        **through)
