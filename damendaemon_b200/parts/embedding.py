"""Embeddings: from the step's token ids to the float32 residual stream.

'tokens': x[t] = table[id[t]] * scale (+ the position encoding's own table at the token's position, if it has one:
damendaemon/gpt2.py:46), one fused gather; the position encoding may then act on x (``on_embedding``).
'tokens_pairs': x[t] = table[id[t]] + pairs[(id[t-1] * mul_prev + id[t] * mul_cur) mod buckets] (the pair table's last row
for a sequence's first token), one gather; the id before a step's first token of a request is per-request state, which
the embedding declares like a mixer does (``cache_needs``) and finds at a cache site of its own.
"""
from __future__ import annotations

from .. import kernels
from .interfaces import Embedding
from .registry import register_embedding
from ..cache.manager import RequestState
from .spec import TensorDecl


@register_embedding("tokens")
class TokenEmbedding(Embedding):
    def __init__(self, spec, weights, runtime):
        self.spec, self.table = spec, weights[spec.table]

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.table, (spec.vocab_size, spec.width), "table")]

    def forward(self, ctx, position):
        x = kernels.embed(ctx.token_ids, ctx.positions, self.table, position.embedding_table(), scale=self.spec.scale)
        return position.on_embedding(x, ctx)


@register_embedding("tokens_pairs")
class TokenPairEmbedding(Embedding):
    def __init__(self, spec, weights, runtime):
        if spec.buckets < 1 or spec.mul_prev < 0 or spec.mul_cur < 0:
            raise ValueError("a pair table needs at least one bucket and multipliers that are not negative")
        self.spec, self.table, self.pairs = spec, weights[spec.table], weights[spec.pair_table]

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.table, (spec.vocab_size, spec.width), "table"),
                TensorDecl(spec.pair_table, (spec.buckets + 1, spec.width), "table")]

    @staticmethod
    def cache_needs(spec):
        return [RequestState((), "int32", name="last_id")]

    def forward(self, ctx, position, cache=None):
        if cache is None or "last_id" not in (cache.named or {}):
            raise ValueError("the pair embedding needs its per-request state (the id before a step's first token)")
        x = kernels.embed_pairs(ctx.token_ids, ctx.positions, ctx.token_entry, ctx.entry_start, ctx.entry_slot, self.table,
                                self.pairs, cache.named["last_id"], self.spec.mul_prev, self.spec.mul_cur)
        return position.on_embedding(x, ctx)
