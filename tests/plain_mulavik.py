"""A plain, slow Mulavik for the tests: whole sequences, no cache, one function a mechanism.

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
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * weight


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    return torch.clamp(z, min=0.0) ** 2


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_pairs(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """v [n, heads, d]: values 2i and 2i+1 (i < dims/2) of every head are a pair (u, w) that turns by
    a = position * base^(-2i/dims): (u cos a - w sin a, w cos a + u sin a); the other values pass."""
    if dims == 0:
        return v
    out = v.clone()
    i = torch.arange(dims // 2, dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * base ** (-2.0 * i / dims)[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, w = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - w * s
    out[..., 1:dims:2] = w * c + u * s
    return out


# --------------------------------------------------------------------------- mixers
def sink_attention(h, W: Dict[str, torch.Tensor], p: str, m: dict, pos0: int = 0) -> torch.Tensor:
    """Causal attention with grouped key/value heads, rotary positions on part of each head and a softmax
    whose denominator has one more term, exp(0): weights exp(s_j) / (1 + sum_j exp(s_j))."""
    n, H, G, d, dv = h.shape[0], m["heads"], m.get("kv_heads") or m["heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    pos = torch.arange(pos0, pos0 + n)
    q = rotate_pairs((h @ W[p + "q"].T).view(n, H, d), pos, float(rot.get("base", 1.0)), int(rot.get("dims", 0)))
    k = rotate_pairs((h @ W[p + "k"].T).view(n, G, d), pos, float(rot.get("base", 1.0)), int(rot.get("dims", 0)))
    v = (h @ W[p + "v"].T).view(n, G, dv)
    out = torch.zeros(n, H, dv, dtype=h.dtype)
    causal = torch.tril(torch.ones(n, n, dtype=torch.bool))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~causal, -math.inf)
        top = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        w = e / (torch.exp(-top) + e.sum(dim=-1, keepdim=True))
        out[:, a] = w @ v[:, g]
    return out.reshape(n, H * dv) @ W[p + "o"].T


def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def mlstm(h, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, state=None, return_state: bool = False):
    """The matrix memory, token by token.  Per head: log gates i = cap(W_i h + b_i) and
    f = logsigmoid(cap(W_f h + b_f)); with the running maximum mx (0 at the start)
        mx' = max(f + mx, i);  S' = e^(f + mx - mx') S + e^(i - mx') k v^T;  n' likewise with k alone;
        o = S'^T q / (max(|n' . q|, e^(-mx')) + 1e-6),   q scaled by dim^(-1/2).
    Then each head's o over its root mean square, times a weight over all heads, times sigmoid(W_g h), W_o."""
    n, H, d, dv, cap = h.shape[0], m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ W[p + "q"].T).view(n, H, d) * d ** -0.5
    k = (h @ W[p + "k"].T).view(n, H, d)
    v = (h @ W[p + "v"].T).view(n, H, dv)
    gi = capped(h @ W[p + "i"].T + W[p + "i.b"], cap)
    gf = torch.nn.functional.logsigmoid(capped(h @ W[p + "f"].T + W[p + "f.b"], cap))
    if state is None:
        S = torch.zeros(H, d, dv, dtype=h.dtype)
        nn = torch.zeros(H, d, dtype=h.dtype)
        mx = torch.zeros(H, dtype=h.dtype)
    else:
        S, nn, mx = (t.clone() for t in state)
    o = torch.zeros(n, H, dv, dtype=h.dtype)
    for t in range(n):
        new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - new), torch.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        nn = keep[:, None] * nn + take[:, None] * k[t]
        mx = new
        den = torch.maximum((nn * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    y = rms(o, eps).reshape(n, H * dv) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    out = y @ W[p + "o"].T
    return (out, (S, nn, mx)) if return_state else out


# --------------------------------------------------------------------------- feed-forwards
def dense_ff(h, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return relu_squared(h @ W[p + "up"].T) @ W[p + "down"].T


def gated_expert(h, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


#: a router's call is close where the last chosen logit leads the first unchosen one by less than this, over the
#: root mean square of the row's logits
CLOSE_CALL = 0.03


def routed_ff(h, W: Dict[str, torch.Tensor], p: str, mlp: dict, margins: Optional[list] = None,
              given: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Sigmoid scores, the ``top`` largest chosen, the score multiplies the expert's INPUT; a shared expert
    for every row, times sigmoid of one number per row.  ``given`` [n, top]: choices made elsewhere (in reduced
    precision); a row whose own call is close follows them, after a check that they differ from its own only by
    experts whose logits lie that close to the border."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ W[p + "router"].T
    s = torch.sigmoid(z)
    order = torch.sort(s, dim=-1, descending=True, stable=True)
    if margins is not None:
        # by how much the last chosen expert's logit leads the first unchosen one's, over the logits' root mean square
        if top < E:
            zs = torch.sort(z, dim=-1, descending=True).values
            margins.append((zs[:, top - 1] - zs[:, top]) / z.pow(2).mean(-1).sqrt().clamp_min(1e-30))
        else:
            margins.append(torch.full((h.shape[0],), math.inf, dtype=h.dtype))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        chosen = [int(e) for e in order.indices[t, :top]]
        if given is not None and top < E:
            zs = torch.sort(z[t], descending=True).values
            rms_z = float(z[t].pow(2).mean().sqrt())
            if float(zs[top - 1] - zs[top]) < CLOSE_CALL * rms_z:
                other = [int(e) for e in given[t]]
                border = float(zs[top - 1] + zs[top]) / 2
                for e in set(other) ^ set(chosen):
                    assert abs(float(z[t, e]) - border) <= CLOSE_CALL * rms_z, (t, e, chosen, other)
                assert len(set(other)) == top
                chosen = other
        for e in chosen:
            out[t] += gated_expert(s[t, e] * h[t:t + 1], W, f"{p}e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, W, p + "shared.") * torch.sigmoid(h @ W[p + "shared.sg"].T)
    return out


# --------------------------------------------------------------------------- the model
class PlainMulavik:
    def __init__(self, model_dir: str):
        from safetensors import safe_open

        with open(os.path.join(model_dir, "config.json")) as fh:
            self.cfg = json.load(fh)
        self.W: Dict[str, torch.Tensor] = {}
        with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
            for name in f.keys():
                self.W[name] = f.get_tensor(name).to(torch.float64)
        self.eps = float(self.cfg["norm"]["eps"])
        #: after ``logits``: per position, the smallest relative margin by which any router chose its last expert
        self.router_margin: Optional[torch.Tensor] = None
        #: after ``logits``: the residual stream behind every layer, [layers, n, width]
        self.streams: Optional[torch.Tensor] = None

    def layer(self, i: int, x: torch.Tensor, margins: list, given: Optional[torch.Tensor] = None) -> torch.Tensor:
        W, eps, layer, p = self.W, self.eps, self.cfg["layers"][i], f"l{i}."
        h = rms_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "attention":
            y = sink_attention(h, W, p + "mix.", layer["mixer"])
        elif layer["type"] == "mlstm":
            y = mlstm(h, W, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, W[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            y = dense_ff(h, W, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(h, W, p + "mlp.", mlp, margins, given)
            x = x + rms_norm(y, W[p + "norm2b"], eps)
        return x

    def logits(self, tokens: Sequence[int], choices: Optional[Dict[int, torch.Tensor]] = None) -> torch.Tensor:
        """``choices``: per routed layer, the experts [n, top] that a reduced-precision run chose; rows whose own
        call is close follow them (``routed_ff``)."""
        W = self.W
        x = W["embed"][torch.tensor(list(tokens), dtype=torch.long)] * float(self.cfg["embedding"]["scale"])
        margins: List[torch.Tensor] = []
        streams = []
        for i in range(len(self.cfg["layers"])):
            x = self.layer(i, x, margins, None if choices is None else choices.get(i))
            streams.append(x)
        self.streams = torch.stack(streams)
        self.router_margin = (torch.stack(margins).min(0).values if margins
                              else torch.full((len(tokens),), math.inf, dtype=torch.float64))
        return rms_norm(x, W["final.norm"], self.eps) @ W["head"].T

    def greedy(self, prompt: Sequence[int], n_new: int) -> List[int]:
        toks = list(prompt)
        for _ in range(n_new):
            toks.append(int(self.logits(toks)[-1].argmax()))
        return toks[len(prompt):]
