"""Mixers made of other mixers."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import kernels
from ..runtime import Runtime
from .registry import part_class, register_mixer
from .spec import MixerSumSpec, TensorDecl


class MixerSum:
    """Two mixers side by side on the same rows: left_scale * left(h) + right_scale * right(h) (see
    :class:`~inferrs_b200.parts.spec.MixerSumSpec`).  Both are built from the registry like any mixer and get the
    layer's cache id: one of them may keep pages of keys and values, one a per-request state."""

    @staticmethod
    def _classes(spec: MixerSumSpec):
        return [(m, part_class("mixer", m)) for m in (spec.left, spec.right)]

    @staticmethod
    def declare(spec: MixerSumSpec) -> List[TensorDecl]:
        return [d for m, cls in MixerSum._classes(spec) for d in cls.declare(m)]

    @staticmethod
    def _one_need(spec: MixerSumSpec, which: str):
        needs = [n for n in (getattr(cls, which)(m) for m, cls in MixerSum._classes(spec)) if n is not None]
        if len(needs) > 1:
            raise ValueError(f"two mixers side by side share one cache id: only one of them may have a {which}")
        return needs[0] if needs else None

    @staticmethod
    def cache_need(spec: MixerSumSpec):
        return MixerSum._one_need(spec, "cache_need")

    @staticmethod
    def state_need(spec: MixerSumSpec):
        return MixerSum._one_need(spec, "state_need")

    @staticmethod
    def side_states(spec: MixerSumSpec):
        """What the two mixers keep beside their own state (a convolution's inputs), each under its own description."""
        return [pair for m, cls in MixerSum._classes(spec) if hasattr(cls, "side_states") for pair in cls.side_states(m)]

    @staticmethod
    def writes_cache(spec: MixerSumSpec) -> bool:
        return all(cls.writes_cache(m) if hasattr(cls, "writes_cache") else True
                   for m, cls in MixerSum._classes(spec)
                   if cls.cache_need(m) is not None or cls.state_need(m) is not None)

    def __init__(self, spec: MixerSumSpec, weights: Dict[str, torch.Tensor], rt: Runtime):
        self.spec, self.rt = spec, rt
        self.left, self.right = (cls(m, weights, rt) for m, cls in self._classes(spec))

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.left, "graph_safe", False) and getattr(self.right, "graph_safe", False))

    def forward(self, ctx, cache_id: int, h):
        a = self.left.forward(ctx, cache_id, h)
        b = self.right.forward(ctx, cache_id, h)
        out = torch.empty_like(a)
        kernels.scaled_sum(a, self.spec.left_scale, b, self.spec.right_scale, out)
        return out


register_mixer("mixer_sum", MixerSum)
