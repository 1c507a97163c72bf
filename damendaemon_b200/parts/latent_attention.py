"""Attention over a compressed latent: one small row per token is its key for every head and holds its value.

One fused projection gives the queries (per head [plain | rotated]) and the token's down projection [latent | a key part
that all heads share]. ``kernels.latent_prepare`` norms the latent, rotates the shared key part and the queries' rotated
parts, and writes the token's row [normed latent | rotated key part] straight into the request's page: that row is all
the cache keeps. The plain part of a score, q . (W_uk c), is computed as (W_uk^T q) . c: every head's plain query is
taken through its own transposed key matrix (``kernels.per_head_linear``), so the attention runs over the cached rows
as they are, with one shared key/value "head" whose values are the first ``rank`` elements of its keys, and a sink in
the softmax: in bfloat16 on the tensor cores (``kernels.attention_latent``: a tile's query rows are (token, head) pairs
that share every key tile), in float32 or at sizes that kernel does not take on the general kernel. The result, a weighted sum of latent rows per head, becomes the head's value through W_uv (the same
per-head product), then the output projection adds into the stream in its epilogue. The transposed key matrices
[heads, rank, head_dim] are made once, when the part is built.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import PagedRows
from .interfaces import Mixer
from .linear import linear
from .positions import rotary_frequencies
from .registry import register_mixer
from .spec import TensorDecl


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        s = spec
        if s.rank + s.rot_dim > 512:
            raise ValueError(f"a latent row of {s.rank} + {s.rot_dim} is not supported (together at most 512)")
        if s.rotary is None or s.rotary.dims > s.rot_dim or s.rotary.dims % 2 or not s.rotary.interleaved or s.rotary.blend is not None:
            raise ValueError("the rotated part takes a plain rotation of neighbouring pairs over at most rot_dim dimensions")
        key = s.query_weight + "+" + s.down_weight
        self.proj_w = weights[key]
        if self.proj_w.shape[0] % 8:
            pad = torch.zeros((-self.proj_w.shape[0] % 8, self.proj_w.shape[1]), dtype=self.proj_w.dtype, device=self.proj_w.device)
            self.proj_w = weights[key] = torch.cat([self.proj_w, pad], dim=0)
        self.q_width = s.n_heads * (s.head_dim + s.rot_dim)
        self.latent_norm = weights[s.latent_norm]
        # W_uk [heads * head_dim, rank] -> per head its transpose [rank, head_dim]; W_uv [heads * value_dim, rank] per head
        self.key_t = weights[s.up_key_weight].view(s.n_heads, s.head_dim, s.rank).transpose(1, 2).contiguous()
        self.value_up = weights[s.up_value_weight].view(s.n_heads, s.value_dim, s.rank).contiguous()
        self.out_w = weights[s.out_weight]
        self.sink = weights[s.sink] if s.sink else None
        freqs, _ = rotary_frequencies(s.rotary)
        self.freqs = freqs.to(torch.float32).to(runtime.device)

    @staticmethod
    def tensor_decls(spec):
        s = spec
        q, down = s.n_heads * (s.head_dim + s.rot_dim), s.rank + s.rot_dim
        decls = [TensorDecl(s.query_weight + "+" + s.down_weight, (q + down, s.width), "matrix", False,
                            ((s.query_weight, (q, s.width)), (s.down_weight, (down, s.width)))),
                 TensorDecl(s.latent_norm, (s.rank,), "vector"),
                 TensorDecl(s.up_key_weight, (s.n_heads * s.head_dim, s.rank), "matrix"),
                 TensorDecl(s.up_value_weight, (s.n_heads * s.value_dim, s.rank), "matrix"),
                 TensorDecl(s.out_weight, (s.width, s.n_heads * s.value_dim), "matrix")]
        if s.sink:
            decls.append(TensorDecl(s.sink, (s.n_heads,), "vector"))
        return decls

    @staticmethod
    def cache_needs(spec):
        return [PagedRows(spec.rank + spec.rot_dim)]

    def forward(self, y, residual, ctx, cache, position):
        s = self.spec
        if not cache.writable:
            raise ValueError("the latent attention mixer writes its own cache")
        proj = linear(self.runtime, y, self.proj_w)
        q, down = proj[:, :self.q_width], proj[:, self.q_width:self.q_width + s.rank + s.rot_dim]
        table = ctx.block_table(cache.group)
        kernels.latent_prepare(q, down, self.latent_norm, s.norm_eps, self.freqs, ctx.token_entry, ctx.positions, table,
                               cache.kv, s.n_heads, s.head_dim, s.rot_dim, s.rank)
        # every head's query against the cached rows: [W_uk^T q_plain | q_rotated]
        q_rows = kernels.per_head_linear(q, self.key_t, s.head_dim + s.rot_dim, tail=s.rot_dim)
        if self.runtime.attention != "rows" and kernels.attention_latent_supported(s.rank + s.rot_dim, s.rank, q_rows.dtype):
            # tensor-core tiles of (token, head) pairs; a step of single tokens cuts its keys so that the GPU fills
            splits = kernels.attention_latent_splits(ctx.n_tokens, ctx.n_entries, s.n_heads, ctx.split_context, q_rows.device) \
                if ctx.decode_only else 1
            mixed = kernels.attention_latent(q_rows, cache.kv, ctx.entry_start, ctx.entry_pos0, table, s.n_heads, s.rank,
                                             s.scale, n_splits=splits, sink=self.sink)
        else:
            mixed = kernels.attention_rows(q_rows, cache.kv, ctx.token_entry, ctx.positions, table, s.n_heads, s.scale,
                                           n_splits=ctx.key_splits(s.n_heads), kv_heads=1, v_dim=s.rank, sink=self.sink,
                                           values_in_keys=True)
        attended = kernels.per_head_linear(mixed, self.value_up, s.rank)
        return linear(self.runtime, attended, self.out_w, residual=residual, out_dtype=residual.dtype, out=residual)
