"""The two ends of a model: token embedding and output head."""
from __future__ import annotations

import torch

from .. import ops
from .base import Part, register_part
from .spec import PartSpec, TensorSpec


def _tensor_name(spec: PartSpec) -> str:
    """The part's own tensor: ``tensor`` if the spec names it in full, else ``<name>.weight``."""
    return spec.get("tensor") or f"{spec['name']}.weight"


class TokenEmbedding(Part):
    """hidden = table[token], a row copy without scaling (src/model.cpp:94-97).

    params: ``vocab_size``, ``hidden_size``, ``name`` (the tensor is ``<name>.weight``, or ``tensor`` in full).  The row is widened into the
    32-bit residual stream by a gather kernel (the reference copies one row per token
    with a device memcpy, src/cuda/model.cu:572-576).
    """

    capturable = True
    category = "embedding"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(_tensor_name(spec), (spec["vocab_size"], spec["hidden_size"]))]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.table = weights.get(_tensor_name(spec), runtime.dtype).contiguous()
        self.hidden = int(spec["hidden_size"])

    def forward(self, token_ids, ctx=None):
        residual = self.runtime.workspace.get("residual", token_ids.shape[0], self.hidden, torch.float32)
        ops.embedding(self.table, token_ids, residual)
        return residual


class PositionedEmbedding(Part):
    """hidden = norm(table[token] * scale + places[position]): a learned vector per position added to the token's row, the sum
    normalised before the first layer.

    params: ``vocab_size``, ``hidden_size``, ``tensor`` (the token table's name), optional ``positions`` = {``tensor``,
    ``max_positions``} (the table of position vectors [max_positions, hidden]; positions count from 0 in each request),
    optional ``norm`` = {``tensor``, ``eps``} (an RMS norm of the sum with its own weight), optional ``scale`` (1.0).
    Sum, statistics and result are 32-bit: the result is the residual stream.  One kernel.
    """

    capturable = True
    category = "embedding"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden = spec["hidden_size"]
        specs = [TensorSpec(_tensor_name(spec), (spec["vocab_size"], hidden), std=1.0)]
        if spec.get("positions"):
            specs.append(TensorSpec(spec["positions"]["tensor"], (spec["positions"]["max_positions"], hidden), std=0.5))
        if spec.get("norm"):
            specs.append(TensorSpec(spec["norm"]["tensor"], (hidden,), init="norm", std=0.1))
        return specs

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden = int(spec["hidden_size"])
        self.table = weights.get(_tensor_name(spec), runtime.dtype).contiguous()
        places, norm = spec.get("positions"), spec.get("norm")
        self.places = weights.get(places["tensor"], runtime.dtype).contiguous() if places else None
        self.norm_weight = weights.get(norm["tensor"], torch.float32).contiguous() if norm else None
        self.eps = float(norm["eps"]) if norm else 0.0
        self.scale = float(spec.get("scale", 1.0))

    def forward(self, token_ids, ctx=None):
        residual = self.runtime.workspace.get("residual", token_ids.shape[0], self.hidden, torch.float32)
        ops.embedding_positions(self.table, self.places, token_ids, None if ctx is None else ctx.positions, self.norm_weight, self.eps, residual, self.scale)
        return residual


class PairEmbedding(Part):
    """hidden = norm(table[token] * scale + pairs[(previous token * mul_prev + token * mul_cur) mod buckets]): beside the token's own row a row of
    a second table chosen by the token and the one before it; a request's first token reads that table's last row (number ``buckets``).

    params: ``vocab_size``, ``hidden_size``, ``tensor`` (the token table's name), optional ``scale`` (1.0), optional ``pairs`` = {``tensor``, ``buckets``,
    ``mul_prev``, ``mul_cur``} (the second table, [buckets + 1, hidden]), optional ``norm`` = {``tensor``, ``eps``, ``groups``} (an RMS norm of the sum over
    ``groups`` equal parts of the row).  The token before a step's first row belongs to the request: one word of per-request state, which the
    cache manager keeps like a mixer's.  Sum, statistics and result are 32-bit: the result is the residual stream.
    """

    capturable = True
    category = "embedding"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        hidden = spec["hidden_size"]
        specs = [TensorSpec(_tensor_name(spec), (spec["vocab_size"], hidden), std=1.0)]
        if spec.get("pairs"):
            specs.append(TensorSpec(spec["pairs"]["tensor"], (spec["pairs"]["buckets"] + 1, hidden), std=1.0))
        if spec.get("norm"):
            specs.append(TensorSpec(spec["norm"]["tensor"], (hidden,), init="norm", std=0.1))
        return specs

    @classmethod
    def cache_need(cls, spec: PartSpec):
        from .base import CacheNeed

        return CacheNeed("state", state_shape=(1,)) if spec.get("pairs") else CacheNeed()

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        self.hidden = int(spec["hidden_size"])
        self.table = weights.get(_tensor_name(spec), runtime.dtype).contiguous()
        pairs, norm = spec.get("pairs"), spec.get("norm")
        self.pairs = weights.get(pairs["tensor"], runtime.dtype).contiguous() if pairs else None
        self.buckets, self.mul_prev, self.mul_cur = (int(pairs[k]) for k in ("buckets", "mul_prev", "mul_cur")) if pairs else (1, 0, 0)
        self.norm_weight = weights.get(norm["tensor"], torch.float32).contiguous() if norm else None
        self.eps = float(norm["eps"]) if norm else 0.0
        self.groups = int(norm.get("groups", 1) or 1) if norm else 1
        self.scale = float(spec.get("scale", 1.0))

    def forward(self, token_ids, ctx=None, cache=None):
        residual = self.runtime.workspace.get("residual", token_ids.shape[0], self.hidden, torch.float32)
        ops.pair_embedding(self.table, self.pairs, ctx, None if cache is None else cache.state, 0, self.norm_weight, self.eps, self.scale, residual,
                           self.buckets, self.mul_prev, self.mul_cur, self.groups)
        return residual


class LinearHead(Part):
    """logits = W . normed, 32-bit out, for the wanted rows only (src/model.cpp:217-225).

    params: ``vocab_size``, ``hidden_size``, ``name``, ``tied_to`` (name of the
    embedding table, or None).  With ``tied_to`` the head's own tensor is optional:
    a checkpoint that stores it anyway is read as it is, one that does not makes the
    head alias the embedding table.  The reference refuses tied checkpoints
    (src/model_config.cpp:72).  A head whose ``tensor`` is the embedding table's own name is that table.
    Optional ``scale``: the logits are multiplied by it (32-bit, after the product).
    """

    capturable = True
    category = "head"

    @classmethod
    def tensor_specs(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        return [TensorSpec(_tensor_name(spec), (spec["vocab_size"], spec["hidden_size"]), optional=bool(spec.get("tied_to")))]

    def __init__(self, spec, prefix, weights, runtime):
        super().__init__(spec, prefix, weights, runtime)
        own = _tensor_name(spec)
        source = own if not spec.get("tied_to") or weights.has(own) else f"{spec['tied_to']}.weight"
        self.weight = weights.get(source, runtime.dtype).contiguous()
        self.vocab = int(spec["vocab_size"])
        self.scale = float(spec.get("scale", 1.0) or 1.0)

    def forward(self, normed_rows):
        """``normed_rows`` is the normalised hidden state of the wanted rows, or an ops.LazyNorm of it."""
        rows = normed_rows.shape[0]
        logits = torch.empty((rows, self.vocab), dtype=torch.float32, device=self.weight.device)
        if isinstance(normed_rows, ops.LazyNorm):
            ops.norm_linear(normed_rows, self.weight, logits)
        else:
            ops.linear(normed_rows, self.weight, logits)
        if self.scale != 1.0:
            ops.scale_rows(logits, self.scale)
        return logits


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("embedding", "positioned_embedding", PositionedEmbedding)
register_part("embedding", "pair_embedding", PairEmbedding)
register_part("head", "linear_head", LinearHead)
