"""Helpers of the Mulavik tests: small configurations, model folders with seeded weights made so that faults
show, and the error measure."""
import json
import os

import torch


def attention_layer(heads=4, kv_heads=2, dim=16, vdim=16, rot_dims=8, base=10000.0, scale=None, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale if scale is not None else dim ** -0.5)
    if rot_dims is not None:
        m["rot"] = dict(base=base, dims=rot_dims)
    return dict(type="attention", mixer=m, mlp=mlp)


def memory_layer(heads=2, dim=16, vdim=24, gate_cap=15.0, mlp=None):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=gate_cap), mlp=mlp)


def dense(ff=48):
    return dict(kind="dense", ff=ff)


def moe(experts=6, top=2, ff=24, shared=16):
    out = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))
    if shared:
        out["shared"] = dict(ff=shared)
    return out


def config(layers, vocab=200, width=64, scale=6.0, eps=1e-5):
    return dict(architecture="Mulavik", vocab=vocab, width=width, embedding=dict(scale=scale), norm=dict(eps=eps),
                layers=layers)


def write_model(cfg_dict, out_dir, dtype=torch.float32, seed=1, sharpen=8.0, long_memory=False):
    """A model folder from the product's random-weights rule, then reshaped so that faults show: embeddings of
    ordinary size, queries and keys scaled so that the softmax leans on single keys or, where all scores are
    negative, on the sink (a wrong key, position or a sink left out then moves the logits); gate biases of the
    matrix memory spread so that some heads forget within a few tokens and others remember for hundreds
    (``long_memory``: all remember); a decisive router; the sublayers' matrices large enough that their outputs
    are far from zero before the norm that follows them."""
    from nanoinfer_b200.config import MulavikConfig
    from nanoinfer_b200.models.model import Model
    from nanoinfer_b200.registry import get_architecture
    from nanoinfer_b200.weights import random_tensors, write_safetensors

    cfg = MulavikConfig.from_dict(json.loads(json.dumps(cfg_dict)))
    model = Model(get_architecture(cfg.architecture).build_spec(cfg), cfg)
    tensors = random_tensors(model, seed, 0.02, torch.float32)
    g = torch.Generator().manual_seed(seed + 99)
    for name, t in tensors.items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        i = int(name[1:].split(".")[0]) if leaf != name else -1
        kind = cfg.layers[i]["type"] if i >= 0 else None
        if name == "embed":
            t *= 50.0 / abs(cfg.embedding_scale)
        elif kind == "attention" and leaf in ("mix.q", "mix.k"):
            t *= sharpen
        elif kind == "mlstm" and leaf in ("mix.q", "mix.k", "mix.v"):
            t *= 5.0
        elif leaf in ("mix.i", "mix.f", "mix.g"):
            t *= 10.0
        elif leaf == "mix.i.b":
            t.copy_(torch.randn(t.shape, generator=g) * 2.0)
        elif leaf == "mix.f.b":
            t.copy_(torch.rand(t.shape, generator=g) * 8.0 - 2.0)
            if long_memory:
                t.copy_(torch.rand(t.shape, generator=g) * 2.0 + 7.0)
        elif leaf == "mlp.router":
            t *= 25.0
        elif leaf == "mlp.shared.sg":
            t *= 10.0
        elif leaf.startswith("mlp.") and leaf.endswith((".up", ".down", ".gate")):
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


def row_errs(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per row: rms(difference with its mean taken off) / rms(reference with its mean taken off)."""
    got, ref = got.double().cpu(), ref.double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-12)


#: bounds on ``rel_err`` of logits: 32-bit, and bfloat16 matrices with 32-bit sums
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def assert_close(errs: torch.Tensor, dtype: str, what: str = "") -> None:
    """32-bit: every position within the bound.  bfloat16: the test weights are made to lean on single keys and
    the matrix memory's sums cancel, so rounding is amplified many times at a position in a hundred: the median
    stays below half the bound, at most one position in twenty-five (or two) lies over it, none far over it.  (A wrong
    key, state or expert moves every position behind it by about 1.)"""
    errs = errs.flatten()
    if dtype == "float32":
        assert float(errs.max()) <= TOL[dtype], f"{what}: {float(errs.max()):.3e} at {int(errs.argmax())}"
        return
    over = int((errs > TOL[dtype]).sum())
    assert float(errs.median()) <= TOL[dtype] / 2, f"{what}: median {float(errs.median()):.3e}"
    assert over <= max(2, len(errs) // 25), f"{what}: {over} of {len(errs)} positions over {TOL[dtype]}"
    assert float(errs.max()) <= 5 * TOL[dtype], f"{what}: {float(errs.max()):.3e} at {int(errs.argmax())}"
