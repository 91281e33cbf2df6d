"""Vadonex's configuration: a list of layers, each with a mixer of one of two kinds and an optional
feed-forward of one of two kinds, read from the nested keys of its config.json:

    {"architecture": "Vadonex", "vocab": V, "width": C, "postln_alpha": a, "norm": {"eps": e},
     "layers": [{"type": "general_delta", "mixer": {"heads": H, "dim": d}, "mlp": ...},
                {"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "rot_dim": r, "vdim": v, "q_rank": q, "kv_rank": k,
                           "scale": s, "mask": {"size": w}, "rot": {"base": b, "dims": n}, "kv_from": j},
                 "mlp": ...}]}
    mlp: null | {"kind": "dense", "ff": F}
             | {"kind": "moe", "router": {"experts": E, "top": K}, "expert": {"ff": F}, "shared": {"ff": Fs}}

Every size and constant comes from the file.  The one size the file does not give, the rank of a
general_delta layer's decay projection, is read from the shape of that layer's tensor when a model
folder is loaded (``sizes_from_tensors``); a configuration written by this package carries it as
``mixer.decay_rank``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, List, Optional, Tuple

from .base import ConfigError, ModelConfig, field

MIXER_KINDS = ("latent_attention", "general_delta")
MLP_KINDS = ("dense", "moe")


def _get(d: Dict[str, Any], path: str, kind, problems: List[str], where: str, default=dataclasses.MISSING):
    """d[a][b]... for a dotted path, checked to be of ``kind`` (int, float); problems are collected."""
    cur: Any = d
    for key in path.split("."):
        if not isinstance(cur, dict) or key not in cur or cur[key] is None:
            if default is dataclasses.MISSING:
                problems.append(f"{where}.{path}: required key is missing")
                return None
            return default
        cur = cur[key]
    if kind is int and (isinstance(cur, bool) or not isinstance(cur, int)):
        problems.append(f"{where}.{path}: expected int, got {cur!r}")
        return None
    if kind is float:
        if isinstance(cur, bool) or not isinstance(cur, (int, float)):
            problems.append(f"{where}.{path}: expected a number, got {cur!r}")
            return None
        return float(cur)
    return cur


@dataclasses.dataclass
class VadonexConfig(ModelConfig):
    architecture_names: ClassVar[Tuple[str, ...]] = ("Vadonex",)

    vocab: int = field()
    width: int = field()
    layers: list = field()
    norm: dict = field()
    postln_alpha: float = field()

    def validate(self) -> None:
        bad: List[str] = []
        if self.vocab <= 0 or self.width <= 0:
            bad.append("vocab and width must be positive")
        eps = _get(self.norm, "eps", float, bad, "norm")
        if eps is not None and not eps > 0.0:
            bad.append(f"norm.eps must be positive, got {eps}")
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
            sizes = ["heads", "dim"] + (["rot_dim", "vdim", "q_rank", "kv_rank"] if kind == "latent_attention" else [])
            for key in sizes:
                v = _get(m, key, int, bad, f"{w}.mixer")
                if v is not None and (v < 0 or (v == 0 and key not in ("dim", "rot_dim"))):
                    bad.append(f"{w}.mixer.{key} must be positive, got {v}")
            if kind == "latent_attention":
                _get(m, "scale", float, bad, f"{w}.mixer")
                size = _get(m, "mask.size", int, bad, f"{w}.mixer", default=0)
                if size is not None and size < 0:
                    bad.append(f"{w}.mixer.mask.size must not be negative")
                if "rot" in m and m["rot"] is not None:
                    _get(m, "rot.base", float, bad, f"{w}.mixer")
                    dims = _get(m, "rot.dims", int, bad, f"{w}.mixer")
                    rd = m.get("rot_dim")
                    if isinstance(dims, int) and isinstance(rd, int) and (dims % 2 or dims > rd):
                        bad.append(f"{w}.mixer.rot.dims {dims} must be even and at most rot_dim {rd}")
                j = m.get("kv_from")
                if j is not None:
                    ok = isinstance(j, int) and not isinstance(j, bool) and 0 <= j < i and \
                        isinstance(self.layers[j], dict) and self.layers[j].get("type") == "latent_attention" and \
                        isinstance(self.layers[j].get("mixer"), dict) and self.layers[j]["mixer"].get("kv_from") is None
                    if not ok:
                        bad.append(f"{w}.mixer.kv_from must name an earlier latent_attention layer that has a "
                                   f"cache of its own, got {j!r}")
                    else:
                        o = self.layers[j]["mixer"]
                        if any(o.get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                            bad.append(f"{w}.mixer: kv_rank, rot_dim and rot must equal those of layer {j}")
            else:
                r = _get(m, "decay_rank", int, bad, f"{w}.mixer", default=None)
                if r is not None and r <= 0:
                    bad.append(f"{w}.mixer.decay_rank must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                bad.append(f"{w}.mlp.kind must be one of {MLP_KINDS} (or mlp null)")
                continue
            if mlp["kind"] == "dense":
                _get(mlp, "ff", int, bad, f"{w}.mlp")
            else:
                e = _get(mlp, "router.experts", int, bad, f"{w}.mlp")
                k = _get(mlp, "router.top", int, bad, f"{w}.mlp")
                _get(mlp, "expert.ff", int, bad, f"{w}.mlp")
                if isinstance(e, int) and isinstance(k, int) and not 0 < k <= e:
                    bad.append(f"{w}.mlp.router.top {k} must be between 1 and experts {e}")
                if mlp.get("shared") is not None:
                    _get(mlp, "shared.ff", int, bad, f"{w}.mlp")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    @property
    def n_layer(self) -> int:
        return len(self.layers)

    def sizes_from_tensors(self, shapes: Dict[str, Tuple[int, ...]]) -> None:
        """Sizes that only the checkpoint's tensor shapes give: the decay projection's rank of every
        general_delta layer (rows of ``l<i>.mix.w1``)."""
        for i, layer in enumerate(self.layers):
            if layer["type"] == "general_delta" and layer["mixer"].get("decay_rank") is None:
                shape = shapes.get(f"l{i}.mix.w1")
                if shape is not None and len(shape) == 2:
                    layer["mixer"]["decay_rank"] = int(shape[0])

    def to_dict(self):
        return {"architecture": self.architecture_names[0], "vocab": self.vocab, "width": self.width,
                "postln_alpha": self.postln_alpha, "norm": dict(self.norm), "layers": self.layers}
