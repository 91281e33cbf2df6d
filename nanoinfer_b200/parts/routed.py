"""A routed feed-forward (mixture of experts): every row goes through ``top`` of ``n_expert`` small
two-layer experts without biases, chosen by a router whose logits and softmax are 32-bit.

z = W_router h, s = softmax(z) over ALL experts, the ``top`` largest are chosen; their weights are the
scores s themselves (``renorm`` divides them by their sum);
out = sum_e s_e W_down[e] act(W_up[e] h), plus, with ``shared_inner`` > 0, one expert of the same form
that every row goes through unweighted.  Routing happens on the device (csrc/moe.cu): nothing of it is
read by the host, so a step's launches depend on its shape only.
"""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from .base import MATRIX, FeedForward, ParamSpec, StepContext, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, width: int, n_expert: int, top: int, inner: int, activation: str = "erf",
                 renorm: bool = False, shared_inner: int = 0, shared_activation: str = "erf"):
        if not 0 < top <= n_expert:
            raise ValueError(f"routed_experts: top {top} must be between 1 and the number of experts {n_expert}")
        for a in (activation, shared_activation):
            if a not in ("tanh", "erf"):
                raise ValueError(f"routed_experts: activation {a!r} is not one of 'tanh', 'erf'")
        self.width, self.n_expert, self.top, self.inner = int(width), int(n_expert), int(top), int(inner)
        self.activation, self.renorm = activation, bool(renorm)
        self.shared_inner, self.shared_activation = int(shared_inner), shared_activation

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec("router", (self.n_expert, self.width), MATRIX)]
        for e in range(self.n_expert):
            specs += [ParamSpec(f"expert{e}_up", (self.inner, self.width), MATRIX),
                      ParamSpec(f"expert{e}_down", (self.width, self.inner), MATRIX)]
        if self.shared_inner:
            specs += [ParamSpec("shared_up", (self.shared_inner, self.width), MATRIX),
                      ParamSpec("shared_down", (self.width, self.shared_inner), MATRIX)]
        return specs

    def matrix_flops_per_row(self) -> float:
        per_expert = 2.0 * 2 * self.inner * self.width
        return 2.0 * self.n_expert * self.width + self.top * per_expert + 2.0 * 2 * self.shared_inner * self.width

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p, E = self.params, self.n_expert
        # the experts' matrices stacked, [E, F, C] and [E, C, F]: a kernel finds expert e at a fixed stride, and
        # the first matrices of all experts are one matrix [E * F, C]; the parameters by name become views of
        # the stacks (no second copy stays behind)
        self.w_up = torch.stack([p[f"expert{e}_up"] for e in range(E)], 0).contiguous()
        self.w_down = torch.stack([p[f"expert{e}_down"] for e in range(E)], 0).contiguous()
        for e in range(E):
            p[f"expert{e}_up"], p[f"expert{e}_down"] = self.w_up[e], self.w_down[e]

    def reserve(self, workspace, limits) -> None:
        n = limits.max_rows
        workspace.reserve("moe.ids", n * self.top, torch.int32)
        workspace.reserve("moe.weights", n * self.top, torch.float32)
        workspace.reserve("moe.inner", n * self.top * self.inner, self.dtype)
        workspace.reserve("moe.parts", n * self.top * self.width, torch.float32)
        if self.n_expert <= ops.MOE_DENSE_MAX_RATIO * self.top:
            workspace.reserve("moe.inner_all", n * self.n_expert * self.inner, self.dtype)
        if self.shared_inner:
            workspace.reserve("moe.shared", n * self.shared_inner, self.dtype)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext) -> None:
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, p, ws, n = ctx.n_rows, self.params, ctx.workspace, ctx.max_rows
        ids = ws.get("moe.ids", (n, self.top), torch.int32)
        weights = ws.get("moe.weights", (n, self.top), torch.float32)
        ops.trace_scope(ctx.layer, "router")
        ops.moe_route(xn, p["router"], T, self.top, self.renorm, ids, weights)
        inner = ws.get("moe.inner", (n * self.top, self.inner), self.dtype)
        ops.trace_scope(ctx.layer, "experts")
        ops.moe_experts(xn, self.w_up, self.w_down, ids, weights, inner, x, T, self.top,
                        ops.ACT_CODES[self.activation], ws)
        if self.shared_inner:
            hs = ws.get("moe.shared", (n, self.shared_inner), self.dtype)
            ops.trace_scope(ctx.layer, "shared_fc")
            ops.linear(xn, p["shared_up"], None, hs, T, act=ops.ACT_CODES[self.shared_activation])
            ops.trace_scope(ctx.layer, "shared_proj")
            ops.linear(hs, p["shared_down"], None, x, T, residual=True)
