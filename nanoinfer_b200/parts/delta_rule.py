"""The generalised delta rule: a recurrent mixer with a matrix state per head.

r, k, v = W_r h, W_k h, W_v h (heads x dim each); decay per head and key channel
w = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 h) + w0)); removal rate a = sigmoid(W_a h + b_a); with the
head's unit key u = k / sqrt(sum(k^2) + 1e-6):
    S_t = diag(w) S_(t-1) - (a * u) (u^T S_(t-1)) + k v^T,    o_t = S_t^T r
(both terms read the old state).  Each head's o is divided by its root mean square, the heads are
concatenated, multiplied by a weight and by sigmoid(W_g h), and go through W_o.  The state starts at
zero, is 32-bit and lives in the request's state slot; everything that enters the recurrence is 32-bit
(the projections leave their product as 32-bit floats).  The work on the device is shaped by the step's
shape alone, so steps are captured in graphs like those of a mixer without state.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import (INIT_ONE_PLUS_NORMAL, MATRIX, VECTOR, KVCacheView, Mixer, ParamSpec, StateSpec, StepContext,
                   StepLimits, Workspace, register_mixer)


@register_mixer("general_delta")
class GeneralDeltaRule(Mixer):
    capture_safe = True

    def __init__(self, width: int, n_head: int, head_dim: int, decay_rank: int, eps: float):
        if min(width, n_head, head_dim, decay_rank) <= 0:
            raise ValueError("general_delta: sizes must be positive")
        if head_dim > 224:
            raise ValueError(f"general_delta: head_dim {head_dim} is not supported (at most 224: the state of a "
                             "head lives in one block's shared memory)")
        self.width, self.n_head, self.head_dim = int(width), int(n_head), int(head_dim)
        self.decay_rank, self.eps = int(decay_rank), float(eps)
        self.inner = self.n_head * self.head_dim

    def param_specs(self) -> List[ParamSpec]:
        n, c, r = self.inner, self.width, self.decay_rank
        return [ParamSpec("r_weight", (n, c), MATRIX), ParamSpec("k_weight", (n, c), MATRIX),
                ParamSpec("v_weight", (n, c), MATRIX), ParamSpec("g_weight", (n, c), MATRIX),
                ParamSpec("a_weight", (n, c), MATRIX), ParamSpec("a_bias", (n,), VECTOR),
                ParamSpec("w1_weight", (r, c), MATRIX), ParamSpec("w2_weight", (n, r), MATRIX),
                ParamSpec("w0", (n,), VECTOR), ParamSpec("out_norm", (n,), VECTOR, INIT_ONE_PLUS_NORMAL),
                ParamSpec("out_weight", (c, n), MATRIX)]

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.n_head, self.head_dim, self.head_dim), torch.float32)

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p = self.params
        # the six products that read the mixer's input are one
        self.w_in = torch.cat([p[k] for k in ("r_weight", "k_weight", "v_weight", "g_weight", "a_weight",
                                              "w1_weight")], 0).contiguous()

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        n = limits.max_rows
        workspace.reserve("delta.proj", n * (5 * self.inner + self.decay_rank), torch.float32)
        workspace.reserve("delta.lora", n * self.decay_rank, self.dtype)
        workspace.reserve("delta.decay", n * self.inner, torch.float32)
        workspace.reserve("delta.out", n * self.inner, self.dtype)
        workspace.reserve("delta.unit", n * self.inner, torch.float32)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if state is None:
            raise ValueError("general_delta needs a state slot tensor")
        T, p, ws, n, N = ctx.n_rows, self.params, ctx.workspace, ctx.max_rows, self.inner
        proj = ws.get("delta.proj", (n, 5 * N + self.decay_rank), torch.float32)
        ops.trace_scope(ctx.layer, "delta_in")
        ops.linear(xn, self.w_in, None, proj, T)
        lora = ws.get("delta.lora", (n, self.decay_rank), self.dtype)
        ops.unary(proj[:, 5 * N:], lora, T, ops.UNARY_TANH)
        wl = ws.get("delta.decay", (n, N), torch.float32)
        ops.trace_scope(ctx.layer, "decay_up")
        ops.linear(lora, p["w2_weight"], None, wl, T)
        o = ws.get("delta.out", (n, N), self.dtype)
        unit = ws.get("delta.unit", (n, N), torch.float32)
        ops.delta_rule(proj, (0, N, 2 * N, 3 * N, 4 * N), wl, p["w0"], p["a_bias"], p["out_norm"], state, ctx,
                       self.n_head, self.head_dim, self.eps, o, unit)
        ops.trace_scope(ctx.layer, "delta_proj")
        ops.linear(o, p["out_weight"], None, x, T, residual=True)
