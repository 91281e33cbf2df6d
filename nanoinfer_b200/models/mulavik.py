"""Mulavik as a ModelSpec: a token embedding times a constant, without positions; layers that normalise a
sublayer's input AND its output before the sum (``sandwich_norm``), each with a mixer (causal attention with
grouped key/value heads, key and value heads of sizes of their own, rotary positions on part of each head and a
softmax sink; or the matrix memory of xLSTM) and an optional feed-forward (dense with the square of relu; or routed:
sigmoid scores, the chosen experts' scores multiplying what the experts read, gated SiLU experts, a shared expert
times a sigmoid of one number a row); a final RMS norm and an untied head.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``, ``final.norm``, ``head``;
attention ``l<i>.mix.{q, k, v, o}``; matrix memory ``l<i>.mix.{q, k, v, g, i, i.b, f, f.b, norm, o}``; dense
feed-forward ``l<i>.mlp.{up, down}``; routed ``l<i>.mlp.{router, e<k>.gate, e<k>.up, e<k>.down, shared.gate,
shared.up, shared.down, shared.sg}``.  Matrices are stored [out, in].
"""
from __future__ import annotations

from ..config.mulavik import MulavikConfig
from ..parts.base import TensorRef
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _refs(prefix: str, names: dict) -> dict:
    return {key: TensorRef(prefix + name) for key, name in names.items()}


def build_mulavik_spec(cfg: MulavikConfig) -> ModelSpec:
    c, eps = cfg.width, cfg.eps

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(width=c, eps=eps), {"weight": TensorRef(name)})

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        parts = {"norm_1": norm(p + "norm1"), "norm_1b": norm(p + "norm1b")}
        position = None
        if layer["type"] == "attention":
            rot = m.get("rot")
            if rot is not None and int(rot.get("dims", 0)) > 0:
                position = PartSpec("rotary_pairs", dict(base=float(rot["base"]), dims=int(rot["dims"])))
            parts["mixer"] = PartSpec("general_attention", dict(
                width=c, n_head=m["heads"], n_kv_head=m.get("kv_heads") or m["heads"], head_dim=m["dim"],
                v_dim=m["vdim"], scale=float(m["scale"]), window=0, sink=True),
                _refs(p, {"q_weight": "mix.q", "k_weight": "mix.k", "v_weight": "mix.v", "out_weight": "mix.o"}))
        else:
            parts["mixer"] = PartSpec("mlstm", dict(
                width=c, n_head=m["heads"], head_dim=m["dim"], v_dim=m["vdim"], gate_cap=float(m["gate_cap"]), eps=eps),
                _refs(p, {"q_weight": "mix.q", "k_weight": "mix.k", "v_weight": "mix.v", "g_weight": "mix.g",
                          "i_weight": "mix.i", "i_bias": "mix.i.b", "f_weight": "mix.f", "f_bias": "mix.f.b",
                          "out_norm": "mix.norm", "out_weight": "mix.o"}))
        mlp = layer.get("mlp")
        if mlp is not None:
            parts["norm_2"], parts["norm_2b"] = norm(p + "norm2"), norm(p + "norm2b")
            if mlp["kind"] == "dense":
                parts["feed_forward"] = PartSpec(
                    "dense_mlp", dict(width=c, inner=mlp["ff"], activation="relu2", bias=False),
                    _refs(p, {"fc_weight": "mlp.up", "proj_weight": "mlp.down"}))
            else:
                n_expert, shared = mlp["router"]["experts"], mlp.get("shared")
                names = {"router": "mlp.router"}
                for e in range(n_expert):
                    names[f"expert{e}_gate"] = f"mlp.e{e}.gate"
                    names[f"expert{e}_up"], names[f"expert{e}_down"] = f"mlp.e{e}.up", f"mlp.e{e}.down"
                if shared is not None:
                    names.update({"shared_gate": "mlp.shared.gate", "shared_up": "mlp.shared.up",
                                  "shared_down": "mlp.shared.down", "shared_row_gate": "mlp.shared.sg"})
                parts["feed_forward"] = PartSpec("routed_experts", dict(
                    width=c, n_expert=n_expert, top=mlp["router"]["top"], inner=mlp["expert"]["ff"],
                    activation="silu", renorm=False, shared_inner=shared["ff"] if shared is not None else 0,
                    shared_activation="silu", score="sigmoid", gated=True, weight_on="input",
                    shared_row_gate=shared is not None), _refs(p, names))
        layers.append(LayerSpec("sandwich_norm", parts, mixer_position=position))
        schedule.append(ScheduleEntry(i))
    return ModelSpec(
        width=c,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, width=c, scale=cfg.embedding_scale),
                           {"table": TensorRef("embed")}),
        position=None,
        layers=layers,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab, width=c), {"weight": TensorRef("head")}),
        max_positions=None,
    )
