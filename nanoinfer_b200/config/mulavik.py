"""Mulavik's configuration: a list of layers, each with a mixer of one of two kinds (attention with a softmax
sink, or the matrix memory of xLSTM) and an optional feed-forward of one of two kinds, read from the nested keys
of its config.json:

    {"architecture": "Mulavik", "vocab": V, "width": C, "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [{"type": "mlstm", "mixer": {"heads": H, "dim": d, "vdim": v, "gate_cap": c}, "mlp": ...},
                {"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": s,
                           "rot": {"base": b, "dims": n}},
                 "mlp": ...}]}
    mlp: null | {"kind": "dense", "ff": F}
             | {"kind": "moe", "router": {"experts": E, "top": K}, "expert": {"ff": F}, "shared": {"ff": Fs}}

Every size and constant comes from the file.  ``kv_heads`` defaults to ``heads``, a missing ``rot`` means no
rotation, a missing or null ``shared`` no shared expert.
"""
from __future__ import annotations

import dataclasses
from typing import ClassVar, List, Tuple

from .base import ConfigError, ModelConfig, field
from .vadonex import _get

MIXER_KINDS = ("attention", "mlstm")
MLP_KINDS = ("dense", "moe")


def _positive(d, path, kind, bad, where, **kw):
    v = _get(d, path, kind, bad, where, **kw)
    if v is not None and not v > 0:
        bad.append(f"{where}.{path} must be positive, got {v}")
    return v


@dataclasses.dataclass
class MulavikConfig(ModelConfig):
    architecture_names: ClassVar[Tuple[str, ...]] = ("Mulavik",)

    vocab: int = field()
    width: int = field()
    layers: list = field()
    norm: dict = field()
    embedding: dict = field()

    def validate(self) -> None:
        bad: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            bad.append("vocab and width must be positive")
        _positive(self.norm, "eps", float, bad, "norm")
        _get(self.embedding, "scale", float, bad, "embedding")
        if not self.layers:
            bad.append("layers: at least one layer is needed")
        for i, layer in enumerate(self.layers):
            w = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                bad.append(f"{w}: expected an object with 'type', 'mixer' and 'mlp'")
                continue
            kind, m = layer.get("type"), layer["mixer"]
            if kind not in MIXER_KINDS:
                bad.append(f"{w}.type {kind!r} is not one of {MIXER_KINDS}")
                continue
            heads = _positive(m, "heads", int, bad, f"{w}.mixer")
            dim = _positive(m, "dim", int, bad, f"{w}.mixer")
            _positive(m, "vdim", int, bad, f"{w}.mixer")
            if kind == "attention":
                g = _positive(m, "kv_heads", int, bad, f"{w}.mixer", default=heads)
                if isinstance(heads, int) and isinstance(g, int) and g > 0 and heads % g:
                    bad.append(f"{w}.mixer.heads {heads} must be a multiple of kv_heads {g}")
                _get(m, "scale", float, bad, f"{w}.mixer")
                if m.get("rot") is not None:
                    _positive(m, "rot.base", float, bad, f"{w}.mixer")
                    dims = _get(m, "rot.dims", int, bad, f"{w}.mixer")
                    if isinstance(dims, int) and isinstance(dim, int) and (dims < 0 or dims % 2 or dims > dim):
                        bad.append(f"{w}.mixer.rot.dims {dims} must be even and at most dim {dim}")
            else:
                _positive(m, "gate_cap", float, bad, f"{w}.mixer")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                bad.append(f"{w}.mlp.kind must be one of {MLP_KINDS} (or mlp null)")
                continue
            if mlp["kind"] == "dense":
                _positive(mlp, "ff", int, bad, f"{w}.mlp")
            else:
                e = _positive(mlp, "router.experts", int, bad, f"{w}.mlp")
                k = _get(mlp, "router.top", int, bad, f"{w}.mlp")
                _positive(mlp, "expert.ff", int, bad, f"{w}.mlp")
                if isinstance(e, int) and isinstance(k, int) and not 0 < k <= e:
                    bad.append(f"{w}.mlp.router.top {k} must be between 1 and experts {e}")
                if mlp.get("shared") is not None:
                    _positive(mlp, "shared.ff", int, bad, f"{w}.mlp")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def embedding_scale(self) -> float:
        return float(self.embedding["scale"])

    @property
    def n_layer(self) -> int:
        return len(self.layers)

    def to_dict(self):
        return {"architecture": self.architecture_names[0], "vocab": self.vocab, "width": self.width,
                "embedding": dict(self.embedding), "norm": dict(self.norm), "layers": self.layers}
