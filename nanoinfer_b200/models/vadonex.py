"""Vadonex as a ModelSpec: token embedding without positions; layers that normalise after the sum with
the stream scaled by ``postln_alpha``, each a latent-attention or generalised-delta-rule mixer and an
optional dense (xIELU) or routed (erf-GELU experts, unrenormalised softmax scores, an optional shared
expert) feed-forward; after every layer a weighted average over the embedding's output and all layers'
results goes on; a final RMS norm and an untied head.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.dwa``, ``final.norm``, ``head``;
latent attention ``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, o}`` (no ``dkv*`` in a layer that
reads another's cache); delta rule ``l<i>.mix.{r, k, v, g, a, a.b, w1, w2, w0, norm, o}``; dense
feed-forward ``l<i>.mlp.{up, down, act}``; routed ``l<i>.mlp.{router, e<k>.up, e<k>.down, shared.up,
shared.down}``.  Matrices are stored [out, in].
"""
from __future__ import annotations

import math

from ..config.base import ConfigError
from ..config.vadonex import VadonexConfig
from ..parts.base import TensorRef
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _refs(prefix: str, names: dict) -> dict:
    return {key: TensorRef(prefix + name) for key, name in names.items()}


def build_vadonex_spec(cfg: VadonexConfig) -> ModelSpec:
    c, eps = cfg.width, cfg.eps
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        parts = {"norm_1": PartSpec("rmsnorm", dict(width=c, eps=eps), {"weight": TensorRef(p + "norm1")})}
        kv_from = None
        if layer["type"] == "latent_attention":
            kv_from = m.get("kv_from")
            rot = m.get("rot") or {}
            names = {"q_down": "mix.dq", "q_norm": "mix.dq.norm", "q_up": "mix.uq", "k_up": "mix.uk",
                     "v_up": "mix.uv", "out_weight": "mix.o"}
            if kv_from is None:
                names.update({"kv_down": "mix.dkv", "kv_norm": "mix.dkv.norm"})
            parts["mixer"] = PartSpec("latent_attention", dict(
                width=c, n_head=m["heads"], nope_dim=m["dim"], rot_dim=m["rot_dim"], v_dim=m["vdim"],
                q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=eps,
                window=int((m.get("mask") or {}).get("size", 0)), rot_base=float(rot.get("base", 10000.0)),
                rot_dims=int(rot.get("dims", 0)), own_kv=kv_from is None), _refs(p, names))
        else:
            if m.get("decay_rank") is None:
                raise ConfigError(f"config.json: layers[{i}].mixer.decay_rank is not given and no tensor "
                                  f"{p}mix.w1 was seen to take it from")
            names = {"r_weight": "mix.r", "k_weight": "mix.k", "v_weight": "mix.v", "g_weight": "mix.g",
                     "a_weight": "mix.a", "a_bias": "mix.a.b", "w1_weight": "mix.w1", "w2_weight": "mix.w2",
                     "w0": "mix.w0", "out_norm": "mix.norm", "out_weight": "mix.o"}
            parts["mixer"] = PartSpec("general_delta", dict(width=c, n_head=m["heads"], head_dim=m["dim"],
                                                            decay_rank=m["decay_rank"], eps=eps), _refs(p, names))
        mlp = layer.get("mlp")
        if mlp is not None:
            parts["norm_2"] = PartSpec("rmsnorm", dict(width=c, eps=eps), {"weight": TensorRef(p + "norm2")})
            if mlp["kind"] == "dense":
                parts["feed_forward"] = PartSpec(
                    "dense_mlp", dict(width=c, inner=mlp["ff"], activation="xielu", bias=False),
                    _refs(p, {"fc_weight": "mlp.up", "proj_weight": "mlp.down", "act_params": "mlp.act"}))
            else:
                n_expert, shared = mlp["router"]["experts"], mlp.get("shared")
                names = {"router": "mlp.router"}
                for e in range(n_expert):
                    names[f"expert{e}_up"], names[f"expert{e}_down"] = f"mlp.e{e}.up", f"mlp.e{e}.down"
                if shared is not None:
                    names.update({"shared_up": "mlp.shared.up", "shared_down": "mlp.shared.down"})
                parts["feed_forward"] = PartSpec("routed_experts", dict(
                    width=c, n_expert=n_expert, top=mlp["router"]["top"], inner=mlp["expert"]["ff"],
                    activation="erf", renorm=False, shared_inner=shared["ff"] if shared is not None else 0,
                    shared_activation="erf"), _refs(p, names))
        parts["depth_mix"] = PartSpec("depth_weighted_average", dict(n_levels=i + 2),
                                      {"weights": TensorRef(p + "dwa")})
        layers.append(LayerSpec("post_norm_depth_mix", parts, args=dict(alpha=cfg.postln_alpha)))
        schedule.append(ScheduleEntry(i, cache_of=kv_from))
    return ModelSpec(
        width=c,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, width=c), {"table": TensorRef("embed")}),
        position=None,
        layers=layers,
        schedule=schedule,
        final_norm=PartSpec("rmsnorm", dict(width=c, eps=eps), {"weight": TensorRef("final.norm")}),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab, width=c), {"weight": TensorRef("head")}),
        max_positions=None,
    )
