"""The matrix memory of xLSTM (mLSTM): a recurrent mixer with a matrix state per head and exponential gates
that are kept from overflowing by a running maximum of their logarithms.

q = W_q h * dim^(-1/2), k = W_k h (heads x dim), v = W_v h (heads x v_dim); per head a log input gate
gi = cap * tanh((W_i h + b_i) / cap) and a log forget gate gf = logsigmoid(cap * tanh((W_f h + b_f) / cap)).
With S, n and the running maximum mx all starting at zero:
    mx' = max(gf + mx, gi);   S' = exp(gf + mx - mx') S + exp(gi - mx') k v^T;   n' likewise with k alone;
    o = S'^T q / (max(|n' . q|, exp(-mx')) + 1e-6).
Each head's o is divided by its root mean square, the heads are concatenated, multiplied by a weight and by
sigmoid(W_g h), and go through W_o.  State and everything that enters the recurrence are 32-bit (the projections
leave their product as 32-bit floats); the state lives in the request's state slot.  The work on the device is
shaped by the step's shape alone, so steps are captured in graphs like those of a mixer without state.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import (INIT_ONE_PLUS_NORMAL, MATRIX, VECTOR, KVCacheView, Mixer, ParamSpec, StateSpec, StepContext,
                   StepLimits, Workspace, register_mixer)


@register_mixer("mlstm")
class MatrixLSTM(Mixer):
    capture_safe = True

    def __init__(self, width: int, n_head: int, head_dim: int, v_dim: int, gate_cap: float, eps: float):
        if min(width, n_head, head_dim, v_dim) <= 0:
            raise ValueError("mlstm: sizes must be positive")
        if head_dim > 256:
            raise ValueError(f"mlstm: head_dim {head_dim} is not supported (at most 256: a column of the state lives "
                             "in the registers of four threads)")
        if not gate_cap > 0.0:
            raise ValueError(f"mlstm: gate_cap {gate_cap} must be positive")
        self.width, self.n_head, self.head_dim, self.v_dim = int(width), int(n_head), int(head_dim), int(v_dim)
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        self.n_qk, self.n_v = self.n_head * self.head_dim, self.n_head * self.v_dim
        #: columns of the fused projection's output: q | k | v | g | input gate | forget gate, a multiple of 8 wide
        self.offsets = (0, self.n_qk, 2 * self.n_qk, 2 * self.n_qk + self.n_v, 2 * self.n_qk + 2 * self.n_v,
                        2 * self.n_qk + 2 * self.n_v + self.n_head)
        self.n_proj = -(-(self.offsets[5] + self.n_head) // 8) * 8

    def param_specs(self) -> List[ParamSpec]:
        c = self.width
        return [ParamSpec("q_weight", (self.n_qk, c), MATRIX), ParamSpec("k_weight", (self.n_qk, c), MATRIX),
                ParamSpec("v_weight", (self.n_v, c), MATRIX), ParamSpec("g_weight", (self.n_v, c), MATRIX),
                ParamSpec("i_weight", (self.n_head, c), MATRIX), ParamSpec("i_bias", (self.n_head,), VECTOR),
                ParamSpec("f_weight", (self.n_head, c), MATRIX), ParamSpec("f_bias", (self.n_head,), VECTOR),
                ParamSpec("out_norm", (self.n_v,), VECTOR, INIT_ONE_PLUS_NORMAL),
                ParamSpec("out_weight", (c, self.n_v), MATRIX)]

    def state_spec(self) -> Optional[StateSpec]:
        return StateSpec((self.n_head * ops.mlstm_state_floats(self.head_dim, self.v_dim),), torch.float32)

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p = self.params
        # the six products that read the mixer's input are one; the parameters by name become views of it
        w = torch.zeros(self.n_proj, self.width, dtype=p["q_weight"].dtype, device=p["q_weight"].device)
        for key, at in zip(("q_weight", "k_weight", "v_weight", "g_weight", "i_weight", "f_weight"), self.offsets):
            n = p[key].shape[0]
            w[at:at + n] = p[key]
            p[key] = w[at:at + n]
        self.w_in = w

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        n = limits.max_rows
        workspace.reserve("mlstm.proj", n * self.n_proj, torch.float32)
        workspace.reserve("mlstm.gates", n * self.n_head * 4, torch.float32)
        workspace.reserve("mlstm.num", n * self.n_v, torch.float32)
        workspace.reserve("mlstm.den", n * self.n_head, torch.float32)
        workspace.reserve("mlstm.out", n * self.n_v, self.dtype)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if state is None:
            raise ValueError("mlstm needs a state slot tensor")
        if isinstance(xn, ops.NormInput):
            xn = xn.materialise(ctx.n_rows)
        T, p, ws, n = ctx.n_rows, self.params, ctx.workspace, ctx.max_rows
        proj = ws.get("mlstm.proj", (n, self.n_proj), torch.float32)
        ops.trace_scope(ctx.layer, "mlstm_in")
        ops.linear(xn, self.w_in, None, proj, T)
        o = ws.get("mlstm.out", (n, self.n_v), self.dtype)
        ops.mlstm(proj, self.offsets, p["i_bias"], p["f_bias"], self.gate_cap, p["out_norm"], state, ctx, self.n_head,
                  self.head_dim, self.v_dim, self.eps, o, ws)
        ops.trace_scope(ctx.layer, "mlstm_proj")
        ops.linear(o, p["out_weight"], None, x, T, residual=True)
