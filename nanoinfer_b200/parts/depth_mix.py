"""A weighted average over depth: what goes on to the next layer is sum_j weights[j] * level_j over the
embedding's output (level 0) and the results of all layers so far, the layer's own among them.  The part
owns the weights; the arrangement that holds it keeps the levels and does the sum in its last kernel."""
from __future__ import annotations

from typing import List

from .base import INIT_NORMAL, VECTOR, DepthMix, ParamSpec, register_depth_mix


@register_depth_mix("depth_weighted_average")
class DepthWeightedAverage(DepthMix):
    def __init__(self, n_levels: int):
        if n_levels < 2:
            raise ValueError("a depth average reads at least the embedding's output and one layer's result")
        self.n_levels = int(n_levels)

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec("weights", (self.n_levels,), VECTOR, INIT_NORMAL)]
