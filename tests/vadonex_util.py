"""Helpers of the Vadonex tests: small configurations, model folders with seeded weights made so that
faults show, and the error measure."""
import json
import os

import torch


def attention_layer(heads=2, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=32, window=24, rot_dims=None,
                    base=10000.0, kv_from=None, scale=None, mlp=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank,
             scale=scale if scale is not None else (dim + rot_dim) ** -0.5,
             rot=dict(base=base, dims=rot_dim if rot_dims is None else rot_dims))
    if window:
        m["mask"] = dict(size=window)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m, mlp=mlp)


def delta_layer(heads=2, dim=16, decay_rank=8, mlp=None):
    return dict(type="general_delta", mixer=dict(heads=heads, dim=dim, decay_rank=decay_rank), mlp=mlp)


def dense(ff=48):
    return dict(kind="dense", ff=ff)


def moe(experts=6, top=2, ff=24, shared=16):
    out = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))
    if shared:
        out["shared"] = dict(ff=shared)
    return out


def config(layers, vocab=200, width=64, alpha=1.7, eps=1e-5):
    return dict(architecture="Vadonex", vocab=vocab, width=width, postln_alpha=alpha, norm=dict(eps=eps),
                layers=layers)


def write_model(cfg_dict, out_dir, dtype=torch.float32, seed=1, sharpen=8.0, long_memory=False):
    """A model folder from the product's random-weights rule, then reshaped so that faults show: unit-sized
    embeddings, queries and keys scaled so that the softmax leans on single keys (a wrong key, window edge or
    position then moves the logits), decay biases spread so that some channels remember for hundreds of
    tokens (``long_memory``: all of them, and hardly anything is removed), a decisive router, activation numbers
    away from zero, depth weights of ordinary size."""
    from nanoinfer_b200.config import VadonexConfig
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture
    from nanoinfer_b200.weights import random_tensors, write_safetensors

    cfg = VadonexConfig.from_dict(json.loads(json.dumps(cfg_dict)))
    model = Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)
    tensors = random_tensors(model, seed, 0.02, torch.float32)
    g = torch.Generator().manual_seed(seed + 99)
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if name == "embed":
            t *= 50.0
        elif leaf in ("mix.uq", "mix.uk"):
            t *= sharpen
        elif leaf == "mix.dkv":
            i = int(name[1:].split(".")[0])
            kr = cfg.layers[i]["mixer"]["kv_rank"]
            t[kr:] *= sharpen
        elif leaf == "mix.w0":
            t.copy_(torch.rand(t.shape, generator=g) * 6.0 - 5.0)
            if long_memory:
                t.copy_(torch.rand(t.shape, generator=g) * 2.0 - 8.0)
        elif leaf in ("mix.w1", "mix.w2", "mix.a", "mix.g"):
            t *= 10.0
        elif leaf == "mix.a.b":
            t.copy_(torch.randn(t.shape, generator=g) - (6.0 if long_memory else 0.0))
        elif leaf == "mlp.router":
            t *= 25.0
        elif leaf == "mlp.act":
            t.copy_(torch.randn(t.shape, generator=g))
        elif leaf == "dwa":
            t.copy_((torch.rand(t.shape, generator=g) * 0.8 + 0.3) / t.numel() * torch.sign(torch.randn(t.shape, generator=g) + 1.0))
        elif leaf.startswith("mlp.") and leaf.endswith((".up", ".down")):
            t *= 5.0
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(cfg.to_dict(), fh)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), {k: v.to(dtype) for k, v in tensors.items()})
    return out_dir


def rel_err(got: torch.Tensor, ref: torch.Tensor) -> float:
    """The largest over rows of rms(difference with its mean taken off) / rms(reference with its mean taken off)."""
    got, ref = got.double().cpu(), ref.double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-12)).max())


#: bounds on ``rel_err`` of logits: 32-bit, and bfloat16 matrices with 32-bit sums
TOL = {"float32": 2e-4, "bfloat16": 6e-2}

#: in bfloat16 a row is left out of a comparison when the plain model's router chose between two experts
#: whose scores lie closer than this (relative): rounding may then choose the other one
CLOSE_CALL = 0.03


def clear_rows(plain, dtype) -> torch.Tensor:
    """After ``plain.logits(tokens)``: which positions a comparison in ``dtype`` may rest on: in bfloat16 all
    but those at which some router of the plain model made a close call (what a flipped choice at one
    position does to later ones through the cache and the state stays far below the bound)."""
    if dtype == "float32":
        return torch.ones_like(plain.router_margin, dtype=torch.bool)
    return plain.router_margin >= CLOSE_CALL
