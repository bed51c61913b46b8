"""Mixers side by side on one input.

Every branch is a mixer of any registered kind and reads the same rows; each branch's result is
RMS-normed over the model width with a weight of its own, and the mean of those is the mixer's
result (one kernel).  The branches' caches travel under one cache id as a ``CompositeCacheSpec``:
pages for the branches that keep keys and values, the request's slot row for those with state.
"""
from __future__ import annotations

from typing import Dict

from .base import MIXERS, CompositeCacheSpec, ParamSpec, Part, register_mixer


@register_mixer("parallel")
class ParallelMixer(Part):
    kernels = ("sandwich",)

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        if not spec.branches or len(spec.names) != len(spec.branches) or len(set(spec.names)) != len(spec.names):
            raise ValueError("a parallel mixer needs branches, each with a name of its own")
        self.branches = [MIXERS.build(b, rt) for b in spec.branches]
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)

    @classmethod
    def params(cls, spec) -> Dict[str, ParamSpec]:
        return {f"{n}_out": ParamSpec((spec.hidden_size,), role="vector", init="ones") for n in spec.names}

    def children(self) -> Dict[str, Part]:
        return dict(zip(self.spec.names, self.branches))

    def load(self, tensors):
        self.weights = [tensors[f"{n}_out"] for n in self.spec.names]

    def cache_spec(self):
        return CompositeCacheSpec(tuple(b.cache_spec() for b in self.branches))

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        ys = [b.forward(x, ctx, cache[i], writes_cache) for i, b in enumerate(self.branches)]
        out = self.rt.empty(*ys[0].shape)
        self.rt.ops.branch_mean(ys, self.weights, self.spec.eps, out)
        return out
