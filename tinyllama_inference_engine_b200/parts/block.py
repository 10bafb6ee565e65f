"""How the parts of one layer are arranged."""
from __future__ import annotations

import torch

from .base import Block, CacheNeed, LayerCache, build_part, norm_then_part, part_class, register_part
from .spec import PartSpec, TensorSpec


class PreNormResidualBlock(Block):
    """x -> x + mixer(norm(x)) -> x + feed_forward(norm(x))  (src/model.cpp:112-207).

    params: ``mixer``, ``feed_forward``, ``mixer_norm``, ``feed_forward_norm``
    (PartSpecs) and the tensor-name suffix of each (``*_name``).  ``feed_forward`` may be
    None: the layer is then x -> x + mixer(norm(x)) alone.  Optional ``token_input`` (a PartSpec of that category, with
    ``token_input_name``): after the sublayers the part adds what it makes of the tokens themselves into the finished stream.
    The hidden state travels as (32-bit residual, output not yet added): each norm
    adds the pending output into the residual before normalising, which is the
    reference's separate add kernel (src/cuda/kernels.cu:208-215) fused into its
    norm (:67-84).
    """

    _SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"), ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))

    capturable = True

    @classmethod
    def _slots(cls, spec: PartSpec):
        """The block's (slot, category) pairs; a block whose ``feed_forward`` is None is its first sublayer alone."""
        slots = [pair for pair in cls._SLOTS if spec.get("feed_forward") is not None or not pair[0].startswith("feed_forward")]
        return slots + ([("token_input", "token_input")] if spec.get("token_input") is not None else [])

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        specs: list[TensorSpec] = []
        for slot, category in cls._slots(spec):
            child = spec[slot]
            specs += part_class(category, child).tensor_specs(child, f"{prefix}.{spec[slot + '_name']}")
        return specs

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return part_class("mixer", spec["mixer"]).cache_need(spec["mixer"])

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.feed_forward = self.feed_forward_norm = self.token_input = None
        for slot, category in self._slots(spec):
            setattr(self, slot, build_part(category, spec[slot], f"{prefix}.{spec[slot + '_name']}", weights, runtime))

    accepts_next_norm = True

    @property
    def first_norm(self):
        return self.mixer_norm

    def forward(self, residual, pending, ctx, cache: LayerCache, next_norm=None):
        from .. import ops

        fused = residual.shape[0] <= ops.fused_rows_limit(self.runtime.dtype, residual.device)
        if self.token_input is not None:
            next_norm = None   # the stream still changes after the last sublayer: nobody prepares the next norm from it
        if self.feed_forward is None:
            pending = norm_then_part(self.mixer_norm, self.mixer, residual, pending, fused, next_norm, ctx, cache)
        else:
            pending = norm_then_part(self.mixer_norm, self.mixer, residual, pending, fused, self.feed_forward_norm, ctx, cache)
            pending = norm_then_part(self.feed_forward_norm, self.feed_forward, residual, pending, fused, next_norm, ctx)
        if self.token_input is not None:
            self.token_input.forward(residual, ctx, pending)   # completes the residual with what is pending, then adds its own
            pending = None
        return residual, pending


class StreamVectorBlock(Block):
    """x -> x + vector: a learned vector, one row of a table, joins every row of the stream (what a model adds before each pass
    of a run of layers that it repeats).  It keeps nothing between steps and is no layer of its own in a trace.

    params: ``tensor`` (the table's full name), ``rows``, ``size``, ``row`` (which row this block adds)."""

    capturable = True
    traced = False

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(spec["tensor"], (spec["rows"], spec["size"]), std=0.5)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.vector = weights.get(spec["tensor"], torch.float32)[int(spec["row"])].contiguous()

    def forward(self, residual, pending, ctx, cache: LayerCache):
        from .. import ops

        ops.add_row_vector(residual, pending, self.vector)
        return residual, None


class SandwichNormBlock(Block):
    """x -> x + post(mixer(pre(x))) -> x + post'(feed_forward(pre'(x))): a norm before every sublayer and another on its output,
    before that joins the stream.

    params: ``mixer``, ``feed_forward`` (or None), and the four norms ``mixer_norm``, ``mixer_post_norm``, ``feed_forward_norm``,
    ``feed_forward_post_norm`` (PartSpecs of a norm kind that offers ``join``), each with its tensor-name suffix (``*_name``).
    Optional ``mixer_filter`` / ``feed_forward_filter`` (PartSpecs of category ``input_filter``, with ``*_name``): what stands between a
    sublayer's first norm and the sublayer (a short convolution over time); what they keep per request lies behind the mixer's own
    state in the layer's state.
    A branch's norm, its sum into the 32-bit stream and the norm that reads the stream next are one kernel (``Norm.join``); the norm
    that follows the block's last sublayer is the next block's first one, which the block is told (``next_norm``) and hands over
    finished, as a prepared norm, if it is of the same kind.
    """

    _SLOTS = (("mixer_norm", "norm"), ("mixer_filter", "input_filter"), ("mixer", "mixer"), ("mixer_post_norm", "norm"), ("feed_forward_norm", "norm"),
              ("feed_forward_filter", "input_filter"), ("feed_forward", "feed_forward"), ("feed_forward_post_norm", "norm"))

    capturable = True
    accepts_next_norm = True

    @classmethod
    def _slots(cls, spec: PartSpec):
        slots = [pair for pair in cls._SLOTS if spec.get("feed_forward") is not None or not pair[0].startswith("feed_forward")]
        return [pair for pair in slots if pair[1] != "input_filter" or spec.get(pair[0]) is not None]

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        specs: list[TensorSpec] = []
        for slot, category in cls._slots(spec):
            child = spec[slot]
            specs += part_class(category, child).tensor_specs(child, f"{prefix}.{spec[slot + '_name']}")
        return specs

    @classmethod
    def _filter_words(cls, spec: PartSpec) -> list[int]:
        return [part_class(category, spec[slot]).state_words(spec[slot]) for slot, category in cls._slots(spec) if category == "input_filter"]

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        need = part_class("mixer", spec["mixer"]).cache_need(spec["mixer"])
        return need.with_state(sum(cls._filter_words(spec)))

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.feed_forward = self.feed_forward_norm = self.feed_forward_post_norm = self.mixer_filter = self.feed_forward_filter = None
        for slot, category in self._slots(spec):
            setattr(self, slot, build_part(category, spec[slot], f"{prefix}.{spec[slot + '_name']}", weights, runtime))
        # the layer's state: [the mixer's own words | the first filter's | the second filter's]
        self.mixer_need = part_class("mixer", spec["mixer"]).cache_need(spec["mixer"])
        self.mixer_words = self.mixer_need.state_words()
        self.filter_offsets, at = {}, self.mixer_words
        for slot, category in self._slots(spec):
            if category == "input_filter":
                self.filter_offsets[slot] = at
                at += part_class(category, spec[slot]).state_words(spec[slot])
        self.filtered = at > self.mixer_words

    @property
    def first_norm(self):
        return self.mixer_norm

    @staticmethod
    def _joinable(norm, following) -> bool:
        return (following is not None and type(following) is type(norm) and following.eps == norm.eps and following.size == norm.size
                and getattr(following, "groups", 1) == getattr(norm, "groups", 1))

    def _mixer_cache(self, cache: LayerCache) -> LayerCache:
        """The layer's cache as the mixer declared it: without the words the filters keep behind the mixer's."""
        if not self.filtered:
            return cache
        state = cache.state[:, : self.mixer_words] if self.mixer_words else None
        return LayerCache(self.mixer_need, cache.writes, cache.pages, cache.block_table, cache.page_size, state, cache.plane_pages)

    def forward(self, residual, pending, ctx, cache: LayerCache, next_norm=None):
        from .. import ops

        if isinstance(pending, ops.LazyNorm) and pending.weight is self.mixer_norm.weight and pending.prepared is not None:
            x = pending.prepared[0]   # the block before left this block's first norm finished
        else:
            x = self.mixer_norm.forward(residual, None if isinstance(pending, ops.LazyNorm) else pending)
        if self.mixer_filter is not None:
            x = self.mixer_filter.forward(x, ctx, cache.state, self.filter_offsets["mixer_filter"])
        branch = self.mixer.forward(x, ctx, self._mixer_cache(cache))
        last = self.mixer_post_norm
        if self.feed_forward is not None:
            x = self.mixer_post_norm.join(residual, branch, self.feed_forward_norm)
            if self.feed_forward_filter is not None:
                x = self.feed_forward_filter.forward(x, ctx, cache.state, self.filter_offsets["feed_forward_filter"])
            branch = self.feed_forward.forward(x, ctx)
            last = self.feed_forward_post_norm
        if self._joinable(last, next_norm):
            ready = last.join(residual, branch, next_norm)
            handle = ops.LazyNorm(residual, next_norm.weight, next_norm.eps, None, lambda: ready)
            handle.prepared = (ready,)
            return residual, handle
        last.join(residual, branch, None)
        return residual, None


class StreamInputMixBlock(Block):
    """x -> W [x ; x0]: the stream and the embedding's output x0 (the token's table row times a constant), side by side, through one
    product that gives the new stream (what a model does before each pass of a run of layers that it repeats).  It keeps nothing
    between steps and is no layer of its own in a trace.  The embedding's output is made again from the step's token ids.

    params: ``tensor`` (W's full name, [size, 2 size], the stream's columns first), ``size``, ``table`` (the embedding table's name),
    ``vocab_size``, ``scale`` (the embedding's constant), ``turn`` (which of the block's two output buffers this run writes: runs that
    follow one another alternate)."""

    capturable = True
    traced = False

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        size = spec["size"]
        return [TensorSpec(spec["tensor"], (size, 2 * size), std=(2 * size) ** -0.5), TensorSpec(spec["table"], (spec["vocab_size"], size), std=1.0)]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.size, self.scale, self.turn = int(spec["size"]), float(spec.get("scale", 1.0)), int(spec.get("turn", 0)) % 2
        self.weight = weights.get(spec["tensor"], runtime.dtype).contiguous()
        self.table = weights.get(spec["table"], runtime.dtype).contiguous()

    def forward(self, residual, pending, ctx, cache: LayerCache):
        from .. import ops

        if pending is not None:
            ops.add_(residual, pending)
        ws, rows = self.runtime.workspace, residual.shape[0]
        both = ws.get("stream_and_input", rows, 2 * self.size, self.runtime.dtype)
        ops.stream_with_embedding(residual, self.table, ctx.token_ids, self.scale, both)
        mixed = ws.get(f"stream_mixed_{self.turn}", rows, self.size, torch.float32)
        ops.linear(both, self.weight, mixed)
        return mixed, None


register_part("block", "pre_norm_residual", PreNormResidualBlock)
register_part("block", "sandwich_norm", SandwichNormBlock)
register_part("block", "stream_input_mix", StreamInputMixBlock)
register_part("block", "stream_vector", StreamVectorBlock)
