"""Mixers made of other mixers."""
from __future__ import annotations

from .. import ops
from ..errors import ConfigError
from .base import CacheNeed, LayerCache, Mixer, build_part, part_class, register_part
from .spec import PartSpec, TensorSpec


class ParallelMixers(Mixer):
    """Two mixers run on one input, their outputs added with a constant each: out = left_scale * left(x) + right_scale * right(x).

    params: ``left``, ``right`` (PartSpecs of mixers; their tensors lie under ``<prefix>.left`` and ``<prefix>.right``), ``left_scale``, ``right_scale``.
    What the two keep between steps is one need: at most one of them may keep pages, and their per-request states lie one behind the
    other in the layer's state.  The sum is 32-bit inside."""

    capturable = True

    @classmethod
    def _children(cls, spec: PartSpec):
        return [(name, spec[name], part_class("mixer", spec[name])) for name in ("left", "right")]

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [t for name, child, kind in cls._children(spec) for t in kind.tensor_specs(child, f"{prefix}.{name}")]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        from dataclasses import replace

        needs = [kind.cache_need(child) for _, child, kind in cls._children(spec)]
        paged = [need for need in needs if need.kind == "pages"]
        if len(paged) > 1:
            raise ConfigError("two mixers on one input: only one of them may keep pages")
        pages = replace(paged[0], state_shape=()) if paged else CacheNeed()
        return pages.with_state(sum(need.state_words() for need in needs))   # the left mixer's words, then the right one's

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.left = build_part("mixer", spec["left"], f"{prefix}.left", weights, runtime)
        self.right = build_part("mixer", spec["right"], f"{prefix}.right", weights, runtime)
        self.left_scale, self.right_scale = float(spec.get("left_scale", 1.0)), float(spec.get("right_scale", 1.0))
        self.needs = [kind.cache_need(child) for _, child, kind in self._children(spec)]
        self.hidden = int(spec["hidden_size"])

    def _cache_of(self, index: int, cache: LayerCache) -> LayerCache:
        need = self.needs[index]
        before = sum(n.state_words() for n in self.needs[:index])
        state = cache.state[:, before : before + need.state_words()] if need.state_words() else None
        if need.kind == "pages":
            return LayerCache(need, cache.writes, cache.pages, cache.block_table, cache.page_size, state, cache.plane_pages)
        return LayerCache(need, cache.writes, None, None, 0, state)

    def forward(self, x, ctx, cache: LayerCache):
        ws, dtype = self.runtime.workspace, self.runtime.dtype
        left = self.left.forward(x, ctx, self._cache_of(0, cache))
        right = self.right.forward(x, ctx, self._cache_of(1, cache))
        if left.data_ptr() == right.data_ptr():
            raise ConfigError(f"{self.prefix}: both mixers write one workspace buffer; give one of them an out_buffer of its own")
        ops.scaled_sum(left, right, self.left_scale, self.right_scale, right)
        return right


register_part("mixer", "parallel_mixers", ParallelMixers)
