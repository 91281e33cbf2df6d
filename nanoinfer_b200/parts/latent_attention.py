"""Attention through a low-rank latent shared by all heads.

Queries go through a latent of their own: c_q = rmsnorm(W_dq h) * w, q = W_uq c_q, head by head
[nope_dim unrotated | rot_dim rotated].  Keys and values come from ONE latent per token:
W_dkv h = [c raw (kv_rank) | k_rot raw (rot_dim)], c = rmsnorm(c raw) * w, k_rot rotated by the token's
position and shared by all heads; a head's unrotated key is W_uk[h] c and its value W_uv[h] c.  The cache
holds c and k_rot only (one row of kv_rank + rot_dim per token, one plane, one head).

Scores never build the keys: (q_nope . W_uk[h] c) = (W_uk[h]^T q_nope) . c, so each head's query is
carried into the latent space, every head attends over the same cached rows, and W_uv[h] is applied to
the weighted sum of latents (csrc/latent_attention.cu, csrc/linear_heads.cu).  A layer built with
``own_kv=False`` has no W_dkv and reads the cache of the layer the schedule names, with its own W_uk,
W_uv, queries and window.  Rotation: interleaved pairs (2i, 2i+1) of the first ``rot_dims`` values of the
rotated part, angle = position * rot_base^(-2i / rot_dims).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kernels import ops
from .base import (INIT_ONE_PLUS_NORMAL, MATRIX, VECTOR, KVCacheSpec, KVCacheView, Mixer, ParamSpec, StepContext,
                   StepLimits, Workspace, register_mixer)


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, width: int, n_head: int, nope_dim: int, rot_dim: int, v_dim: int, q_rank: int,
                 kv_rank: int, scale: float, eps: float, window: int = 0, rot_base: float = 10000.0,
                 rot_dims: Optional[int] = None, own_kv: bool = True):
        rot_dims = rot_dim if rot_dims is None else rot_dims
        for name, v in (("width", width), ("n_head", n_head), ("v_dim", v_dim), ("q_rank", q_rank),
                        ("kv_rank", kv_rank)):
            if int(v) <= 0:
                raise ValueError(f"latent_attention: {name} must be positive, got {v}")
        if nope_dim < 0 or rot_dim < 0 or nope_dim + rot_dim == 0:
            raise ValueError("latent_attention: a head needs unrotated or rotated query dimensions")
        if rot_dims < 0 or rot_dims > rot_dim or rot_dims % 2:
            raise ValueError(f"latent_attention: rot_dims {rot_dims} must be even and at most rot_dim {rot_dim}")
        if kv_rank > 1024 or window < 0:
            raise ValueError("latent_attention: kv_rank at most 1024, window >= 0")
        self.width, self.n_head, self.nope_dim, self.rot_dim, self.v_dim = int(width), int(n_head), int(nope_dim), int(rot_dim), int(v_dim)
        self.q_rank, self.kv_rank, self.scale, self.eps = int(q_rank), int(kv_rank), float(scale), float(eps)
        self.window, self.rot_base, self.rot_dims, self.own_kv = int(window), float(rot_base), int(rot_dims), bool(own_kv)
        self.qk_dim = self.nope_dim + self.rot_dim
        self.latent_dim = self.kv_rank + self.rot_dim

    def param_specs(self) -> List[ParamSpec]:
        H = self.n_head
        specs = [ParamSpec("q_down", (self.q_rank, self.width), MATRIX),
                 ParamSpec("q_norm", (self.q_rank,), VECTOR, INIT_ONE_PLUS_NORMAL),
                 ParamSpec("q_up", (H * self.qk_dim, self.q_rank), MATRIX)]
        if self.own_kv:
            specs += [ParamSpec("kv_down", (self.latent_dim, self.width), MATRIX),
                      ParamSpec("kv_norm", (self.kv_rank,), VECTOR, INIT_ONE_PLUS_NORMAL)]
        specs += [ParamSpec("k_up", (H * self.nope_dim, self.kv_rank), MATRIX),
                  ParamSpec("v_up", (H * self.v_dim, self.kv_rank), MATRIX),
                  ParamSpec("out_weight", (self.width, H * self.v_dim), MATRIX)]
        return specs

    def kv_spec(self) -> Optional[KVCacheSpec]:
        return KVCacheSpec(1, self.latent_dim, self.window, planes=1)

    def flops_per_key(self) -> float:
        return 2.0 * self.n_head * (self.latent_dim + self.kv_rank)

    def prepare(self, dtype, device) -> None:
        super().prepare(dtype, device)
        p, H = self.params, self.n_head
        # the two down-projections read the same rows: one product
        self.down = torch.cat([p["q_down"], p["kv_down"]], 0).contiguous() if self.own_kv else p["q_down"]
        # W_uk per head, transposed: the map from a head's unrotated query into the latent space
        self.k_up_t = p["k_up"].view(H, self.nope_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.v_up = p["v_up"].view(H, self.v_dim, self.kv_rank)
        i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
        self.freqs = (self.rot_base ** (-2.0 * i / max(self.rot_dims, 1))).to(device)

    def reserve(self, workspace: Workspace, limits: StepLimits) -> None:
        n, H = limits.max_rows, self.n_head
        workspace.reserve("latent.proj", n * (self.q_rank + self.latent_dim), torch.float32)
        workspace.reserve("latent.cq", n * self.q_rank, self.dtype)
        workspace.reserve("latent.q", n * H * self.qk_dim, self.dtype)
        workspace.reserve("latent.q_full", n * H * self.latent_dim, torch.float32)
        workspace.reserve("latent.out", n * H * self.kv_rank, self.dtype)
        workspace.reserve("latent.att", n * H * self.v_dim, self.dtype)
        ops.latent_attention_reserve(workspace, H, self.kv_rank)

    def forward(self, xn: torch.Tensor, x: torch.Tensor, ctx: StepContext, cache: Optional[KVCacheView],
                state: Optional[torch.Tensor], writes_cache: bool = True) -> None:
        if cache is None:
            raise ValueError("latent_attention needs a paged latent cache")
        if writes_cache != self.own_kv:
            raise ValueError("latent_attention: a layer without W_dkv must read another layer's cache, and only it")
        T, p, H, ws, n = ctx.n_rows, self.params, self.n_head, ctx.workspace, ctx.max_rows
        D = self.latent_dim
        proj = ws.get("latent.proj", (n, self.down.shape[0]), torch.float32)
        ops.trace_scope(ctx.layer, "latent_down")
        ops.linear(xn, self.down, None, proj, T)
        cq = ws.get("latent.cq", (n, self.q_rank), self.dtype)
        ops.latent_prep(proj, self.q_rank, self.kv_rank, self.rot_dim, self.rot_dims, self.freqs, p["q_norm"],
                        p.get("kv_norm"), self.eps, cq, cache.layer if self.own_kv else None,
                        cache.block_table if self.own_kv else None, ctx.row_entry, ctx.positions, T, ctx.status)
        q = ws.get("latent.q", (n, H * self.qk_dim), self.dtype)
        ops.trace_scope(ctx.layer, "q_up")
        ops.linear(cq, p["q_up"], None, q, T)
        qf = ws.get("latent.q_full", (n, H, D), torch.float32)
        if self.nope_dim:
            ops.trace_scope(ctx.layer, "q_absorb")
            ops.linear_heads(q, self.qk_dim, self.k_up_t, qf.view(n, H * D), D, T)
        ops.rope_heads(q, self.nope_dim, self.rot_dim, self.rot_dims, self.freqs, ctx.positions, qf, self.kv_rank, H, T)
        lat = ws.get("latent.out", (n, H * self.kv_rank), self.dtype)
        ops.latent_attention(qf, cache.layer, lat, cache.block_table, ctx, H, self.kv_rank, self.scale, self.window)
        att = ws.get("latent.att", (n, H * self.v_dim), self.dtype)
        ops.trace_scope(ctx.layer, "v_up")
        ops.linear_heads(lat, self.kv_rank, self.v_up, att, self.v_dim, T)
        ops.trace_scope(ctx.layer, "attn_proj")
        ops.linear(att, p["out_weight"], None, x, T, residual=True)
