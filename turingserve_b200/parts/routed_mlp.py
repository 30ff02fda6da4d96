"""Routed feed-forward: every token goes through the ``top_k`` of ``num_experts`` small feed-forwards
down_e(act(up_e(.))) whose router scores are largest.

Router logits and scores are 32-bit.  The (token, choice) pairs are sorted by expert on the device and the
two products run over the sorted groups; the chosen score multiplies the expert's input (``weight_on``
"input", the product reads score * x rounded to the engine's type) or its output; a token's choices are
summed in 32-bit in the order of their rank.  No count comes back to the host, so the chain may sit in a
captured step.  The experts' weights are stacked [E, ff, hidden] and [E, hidden, ff] when they arrive.

Many rows (``LIBRARY_ROWS`` pairs or more, outside a capture): the group sizes are read back once, the input
rows are gathered in sorted order, and every expert's rows go through ``ops().linear`` as a product of their own,
i.e. to the many-row kernels and the vendor library that the dense products of such steps use.
"""

from __future__ import annotations

import torch

from turingserve_b200 import kernels
from turingserve_b200.parts.base import BuildContext, FeedForward, ParamSpec, register
from turingserve_b200.parts.mlp import ACTIVATIONS


class RoutedMLP(FeedForward):
    # from this many (token, choice) pairs in a step the experts' products are launched one by one (2,048 tokens of
    # width 3,584 through 8 experts of 7,104: 2.7 ms for the two grouped products, 0.5 ms this way)
    LIBRARY_ROWS = 1024

    def __init__(self, spec, ctx: BuildContext) -> None:
        self.hidden = ctx.hidden_size
        self.E, self.top, self.inter = int(spec.num_experts), int(spec.top_k), int(spec.intermediate_size)
        if not 1 <= self.top <= self.E:
            raise ValueError(f"routed_mlp: top {self.top} of {self.E} experts")
        if spec.activation not in ACTIVATIONS:
            raise ValueError(f"routed_mlp: activation {spec.activation!r} has no kernel")
        if spec.scoring not in ("sigmoid", "softmax") or spec.weight_on not in ("input", "output"):
            raise ValueError(f"routed_mlp: scoring {spec.scoring!r} / weight_on {spec.weight_on!r}")
        self.activation, self.softmax = spec.activation, spec.scoring == "softmax"
        self.renormalize, self.on_input = bool(spec.renormalize), spec.weight_on == "input"
        self.w_router = self.w_up = self.w_down = None

    def parameters(self) -> dict[str, ParamSpec]:
        p = {"router": ParamSpec((self.E, self.hidden), compute_dtype=False)}
        for e in range(self.E):
            p[f"e{e}.up"] = ParamSpec((self.inter, self.hidden))
            p[f"e{e}.down"] = ParamSpec((self.hidden, self.inter))
        return p

    def load(self, t: dict[str, torch.Tensor]) -> None:
        self.w_router = t["router"].float().contiguous()
        self.w_up = torch.stack([t[f"e{e}.up"] for e in range(self.E)]).contiguous()
        self.w_down = torch.stack([t[f"e{e}.down"] for e in range(self.E)]).contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops = kernels.ops()
        T, top = x.shape[0], self.top
        idx = torch.empty((T, top), dtype=torch.int32, device=x.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=x.device)
        ops.router_topk(idx, weights, x, self.w_router, self.softmax, self.renormalize)
        offsets, order, place, tiles = ops.moe_align(idx, self.E)
        a = torch.empty((T * top, self.inter), dtype=x.dtype, device=x.device)
        y = torch.empty((T * top, self.hidden), dtype=torch.float32, device=x.device)
        # the experts' input rows in sorted order, weighted and rounded once (the products then read plain rows)
        xs = torch.empty((T * top, self.hidden), dtype=x.dtype, device=x.device)
        ops.moe_gather(xs, x, order, weights if self.on_input else None, top)
        if T * top >= self.LIBRARY_ROWS and x.is_cuda and not torch.cuda.is_current_stream_capturing():
            bounds = offsets[: self.E + 1].tolist()                      # the one read-back of this path
            for e in range(self.E):
                lo, hi = bounds[e], bounds[e + 1]
                if hi > lo:
                    ops.linear(a[lo:hi], xs[lo:hi], self.w_up[e])
            ops.activation(a, a, self.activation)
            for e in range(self.E):
                lo, hi = bounds[e], bounds[e + 1]
                if hi > lo:
                    ops.linear(y[lo:hi], a[lo:hi], self.w_down[e])
        else:
            ops.grouped_linear(a, xs, self.w_up, None, None, offsets, tiles, 1, self.activation)
            ops.grouped_linear(y, a, self.w_down, None, None, offsets, tiles, 1)
        out = torch.empty((T, self.hidden), dtype=x.dtype, device=x.device)
        ops.moe_combine(out, y, place, None if self.on_input else weights, top)
        return out


register("feed_forward", "routed_mlp", RoutedMLP)
