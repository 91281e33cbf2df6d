"""A plain, slow Vadonex for the tests: whole sequences, no cache, one function a mechanism.

It shares no code with ``nanoinfer_b200``: it reads the model folder with the ``safetensors`` package
and ``json`` and computes in float64 torch.  Linear weights are [out, in] and applied as W x.

Notation: h is a sublayer's input [n, width]; positions count from 0; rms(x) = x / sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- small pieces
def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension, the eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * weight


def softplus(v: float) -> float:
    return math.log1p(math.exp(v))


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    pos = softplus(p) * z * z + z / 2
    neg = (0.5 + softplus(q)) * (torch.expm1(z) - z) + z / 2
    return torch.where(z > 0, pos, neg)


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Rotary positions on the first ``dims`` values of the last dimension (the rest pass): values 2i and
    2i+1 are a pair (u, w) -> (u cos a - w sin a, w cos a + u sin a), a = position * base^(-2i / dims).
    v: [n, ..., d]; positions: [n]."""
    if dims == 0:
        return v
    out = v.clone()
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]      # [n, dims/2]
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [dims // 2]
    c, s = ang.cos().view(shape), ang.sin().view(shape)
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


def visible(n_q: int, n_k: int, q_pos0: int, window: int) -> torch.Tensor:
    """[n_q, n_k] mask: query at position q_pos0 + i sees key j with 0 <= pos - j (< window if window > 0)."""
    qi = torch.arange(q_pos0, q_pos0 + n_q)[:, None]
    kj = torch.arange(n_k)[None, :]
    ok = qi - kj >= 0
    if window > 0:
        ok &= qi - kj < window
    return ok


# --------------------------------------------------------------------------- mixers
def latent_kv(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float):
    """What a layer with a W_dkv leaves for attention: the normed latent c [n, kv_rank] and the rotated
    shared key part [n, rot_dim]."""
    n, kr = h.shape[0], m["kv_rank"]
    dkv = h @ W[p + "dkv"].T
    c = rms_norm(dkv[:, :kr], W[p + "dkv.norm"], eps)
    rot = m.get("rot") or {}
    k_rot = rotate_pairs(dkv[:, kr:], torch.arange(n), float(rot.get("base", 1.0)), int(rot.get("dims", 0)))
    return c, k_rot


def latent_attention(h, W, p: str, m: dict, eps: float, kv) -> torch.Tensor:
    """Queries through a latent of their own; per head the key is [W_uk c | shared rotated part], the value
    W_uv c; softmax over the visible keys; W_o on the concatenated heads.  ``kv``: (c, k_rot) of this layer
    or of the layer it reads."""
    n, H, d, r, vd = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, k_rot = kv
    cq = rms_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], eps)
    q = (cq @ W[p + "uq"].T).view(n, H, d + r)
    rot = m.get("rot") or {}
    q_rot = rotate_pairs(q[..., d:], torch.arange(n), float(rot.get("base", 1.0)), int(rot.get("dims", 0)))
    k_nope = (c @ W[p + "uk"].T).view(n, H, d)
    v = (c @ W[p + "uv"].T).view(n, H, vd)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], k_nope) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    s = s.masked_fill(~visible(n, n, 0, int((m.get("mask") or {}).get("size", 0))), float("-inf"))
    o = torch.einsum("hij,jhd->ihd", torch.softmax(s, dim=-1), v).reshape(n, H * vd)
    return o @ W[p + "o"].T


def general_delta(h, W, p: str, m: dict, eps: float) -> torch.Tensor:
    """S_t = diag(w) S_(t-1) - (a u)(u^T S_(t-1)) + k v^T, o_t = S_t^T r, per head, from a zero state."""
    n, H, d = h.shape[0], m["heads"], m["dim"]
    r = (h @ W[p + "r"].T).view(n, H, d)
    k = (h @ W[p + "k"].T).view(n, H, d)
    v = (h @ W[p + "v"].T).view(n, H, d)
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).view(n, H, d)
    a = torch.sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).view(n, H, d)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=h.dtype)
    o = torch.zeros(n, H, d, dtype=h.dtype)
    for t in range(n):
        uS = torch.einsum("hi,hij->hj", u[t], S)
        S = w[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hij,hi->hj", S, r[t])
    o = rms(o, eps).reshape(n, H * d) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


# --------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W, p: str) -> torch.Tensor:
    pp, qq = (float(t) for t in W[p + "act"])
    return xielu(h @ W[p + "up"].T, pp, qq) @ W[p + "down"].T


def routed_ff(h, W, p: str, mlp: dict, margins: Optional[torch.Tensor] = None) -> torch.Tensor:
    """softmax over all experts of the router's logits, the ``top`` largest chosen, weighted by their
    scores as they are; a shared expert, if any, is added for every row.  ``margins`` [n] (optional) is
    lowered to each row's relative gap between the last score chosen and the first one left out (where that
    last score weighs anything: a choice between two experts that both count for less than 0.002 is no
    call at all): a test of a reduced-precision engine leaves out rows whose choice is that close a call."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    s = torch.softmax(h @ W[p + "router"].T, dim=-1)
    score, chosen = torch.topk(s, top, dim=-1)
    if margins is not None and top < E:
        ranked = torch.sort(s, dim=-1, descending=True).values
        gap = (ranked[:, top - 1] - ranked[:, top]) / ranked[:, top - 1]
        torch.minimum(margins, torch.where(ranked[:, top - 1] < 2e-3, torch.ones_like(gap), gap), out=margins)
    out = torch.zeros_like(h)
    for e in range(E):
        hit = chosen == e
        rows = hit.any(-1)
        if rows.any():
            weight = (score * hit).sum(-1)[rows]
            out[rows] += weight[:, None] * (gelu_erf(h[rows] @ W[p + f"e{e}.up"].T) @ W[p + f"e{e}.down"].T)
    if mlp.get("shared") is not None:
        out = out + gelu_erf(h @ W[p + "shared.up"].T) @ W[p + "shared.down"].T
    return out


# --------------------------------------------------------------------------- the model
class PlainVadonex:
    def __init__(self, model_dir: str):
        from safetensors import safe_open

        with open(os.path.join(model_dir, "config.json")) as fh:
            self.cfg = json.load(fh)
        self.W: Dict[str, torch.Tensor] = {}
        with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
            for name in f.keys():
                self.W[name] = f.get_tensor(name).to(torch.float64)

    def forward(self, tokens: Sequence[int], keep_layers: bool = False):
        cfg, W = self.cfg, self.W
        eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
        x = W["embed"][torch.as_tensor(list(tokens), dtype=torch.long)]
        levels: List[torch.Tensor] = [x]
        #: per position, the closest call any router of the model made (1: none was close, or no router)
        self.router_margin = torch.ones(len(x), dtype=torch.float64)
        kept: Dict[int, tuple] = {}
        after = []
        for i, layer in enumerate(cfg["layers"]):
            m = layer["mixer"]
            if layer["type"] == "latent_attention":
                src = m.get("kv_from")
                if src is None:
                    kept[i] = latent_kv(x, W, f"l{i}.mix.", m, eps)
                mixed = latent_attention(x, W, f"l{i}.mix.", m, eps, kept[i if src is None else src])
            else:
                mixed = general_delta(x, W, f"l{i}.mix.", m, eps)
            x = rms_norm(alpha * x + mixed, W[f"l{i}.norm1"], eps)
            mlp = layer.get("mlp")
            if mlp is not None:
                f = dense_ff(x, W, f"l{i}.mlp.") if mlp["kind"] == "dense" else routed_ff(x, W, f"l{i}.mlp.", mlp, self.router_margin)
                x = rms_norm(alpha * x + f, W[f"l{i}.norm2"], eps)
            levels.append(x)
            d = W[f"l{i}.dwa"]
            x = sum(d[j] * levels[j] for j in range(i + 2))
            after.append(x)
        logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
        return (logits, after) if keep_layers else logits

    def logits(self, tokens: Sequence[int]) -> torch.Tensor:
        return self.forward(tokens)

    def greedy(self, prompt: Sequence[int], n_new: int) -> List[int]:
        toks = list(prompt)
        for _ in range(n_new):
            toks.append(int(self.forward(toks)[-1].argmax()))
        return toks[len(prompt):]
