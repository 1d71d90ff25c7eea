"""The two ends of the model: token ids in, logits out.

``embedding``: h[t] = table[ids[t]] as float32 rows of the residual stream (times the record's
``scale``, 1 by default, and repeated ``copies`` times for a residual kept as several streams); an id
outside the table is reported through the error word (thanhauco/rust-inference
src/ops/embedding.rs:10-42).

``linear`` head: logits = x W^T, no bias, float32 out of the float32 accumulator
(src/models/qwen3.rs:166-171, 286); a record may give a factor on the logits and a soft-cap
(cap * tanh(logits / cap)) applied after it.  When the model ties its embeddings the head is
given the embedding's table instead of a tensor of its own.

Another architecture registers other kinds (a scaled embedding, a head with a soft-cap or a bias)
with ``@register_embedding`` / ``@register_head`` and names them in its ``ModelSpec``.

Interfaces: embedding ``__call__(ids, ctx) -> float32 [tokens, hidden]`` (``ctx`` is the step's
:class:`~.base.StepContext`: an embedding that adds learned positions reads ``ctx.tok_pos``) and
``table`` (what a tied head shares); head ``__call__(x) -> float32 [rows, vocab]``, ``load(tensors)``
where ``tensors["weight"]`` is its own tensor or the embedding's table.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import CacheRequest, Part
from .registry import ParamInfo, register_embedding, register_head


@register_embedding("embedding")
class TokenEmbedding(Part):
    graph_safe = True

    @classmethod
    def param_infos(cls, spec):
        return {"weight": ParamInfo((spec.vocab_size, spec.hidden_size), "matrix")}

    def load(self, tensors):
        self.table = tensors["weight"]

    def weight_bytes(self):
        return self.table.numel() * self.table.element_size()

    def __call__(self, ids, ctx=None):
        return ops.embed(ids, self.table, getattr(self.spec, "scale", 1.0), getattr(self.spec, "copies", 1))


@register_embedding("pair_hash")
class PairHashEmbedding(Part):
    """Token rows plus rows of a hashed table of (previous token, token) pairs; the previous token of a step's first
    token is per-sequence state (one int32 per cache slot), which the part asks the cache for."""
    graph_safe = True

    @classmethod
    def param_infos(cls, spec):
        return {"weight": ParamInfo((spec.vocab_size, spec.hidden_size), "matrix"),
                spec.pairs_name: ParamInfo((spec.buckets + 1, spec.hidden_size), "matrix")}

    def load(self, tensors):
        self.table = tensors["weight"]
        self.pairs = tensors[self.spec.pairs_name]

    def weight_bytes(self):
        return (self.table.numel() + self.pairs.numel()) * self.table.element_size()

    def cache_request(self):
        return CacheRequest(state_shape=(1,), state_dtype=torch.int32)

    def __call__(self, ids, ctx, cache):
        s = self.spec
        return ops.embed_pair_hash(ids, self.table, self.pairs, cache.state.view(-1), ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                                   ctx.seq_start, s.mul_prev, s.mul_cur, single=ctx.decode_only)


@register_head("linear")
class LinearHead(Part):
    graph_safe = True

    @classmethod
    def param_infos(cls, spec):
        return {"weight": ParamInfo((spec.vocab_size, spec.hidden_size), "matrix")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def reads_first(self):
        return self.weight

    def __call__(self, x):
        z = ops.scale_(ops.linear(x, self.weight, out_dtype=torch.float32), getattr(self.spec, "scale", 1.0))
        return ops.softcap_(z, getattr(self.spec, "softcap", 0.0))
