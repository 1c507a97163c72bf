"""The attention mixer: fused QKV projection, cache write, paged causal attention, output
projection with the residual add in its epilogue (damendaemon/gpt2.py:48-61).

Heads, key/value groups, head size, scale and window are parameters of the spec, and so
are: a value head of another size than a key head; a chunked mask (positions in chunks
counted from the start of the sequence, nothing seen across a border); a gate per head,
sigmoid of one more projection of the mixer's input, on the head's output before the
output projection (its rows are joined to the fused projection); a rotary position
encoding of the mixer's own; an RMS norm over every query head and every key head before
that rotation (one kernel does both); no keys and values of its own (the mixer then
projects queries only and reads the cache of another stop of the run order through its own
mask); first keys that stay visible behind the window, capped scores and a sink in the softmax (a learned number per
head in the denominator); values blended with those an earlier mixer computed for the same tokens (one learned weight,
the blended values are what is cached); values that are the keys as projected (no value projection: the key projection's
rows are joined to the fused product a second time, so the values are the unnormed, unrotated keys bit for bit); a norm of
queries and keys over the whole projection instead of per head; a gate per element of the attended output; a unit term in
the softmax's denominator. The kernels read keys and values from the cache pages only, so
a portion of a prompt sees earlier portions exactly as a decoded token sees its context.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import PagedKeyValues
from .paged_attention import prompt_key_block
from .interfaces import Mixer
from .linear import linear
from .registry import POSITIONS, lookup, register_mixer
from .spec import TensorDecl


def _joined(names):
    """The key of a tensor that the checkpoint holds whole (its name) or in pieces (their names joined)."""
    return names if isinstance(names, str) else "+".join(names)


def _projection(spec):
    """(names of the pieces of the fused projection, or its one name; the key the joined tensor is found under)."""
    names = spec.qkv_weight
    if not spec.own_keys_values:
        if isinstance(names, str) or len(names) != 1:
            raise ValueError("a mixer without keys and values of its own names its query projection alone")
        names = tuple(names)
    if spec.values_are_keys:
        if isinstance(names, str) or len(names) != 2 or not spec.own_keys_values:
            raise ValueError("a mixer whose values are its keys names its query and key projections (and no third)")
        names = (names[0], names[1], names[1])        # the key projection's rows a second time: the values
    if spec.gate_weight:
        if isinstance(names, str):
            raise ValueError("a gate's rows are joined to separate query, key and value projections")
        names = tuple(names) + (spec.gate_weight,)
    return names, _joined(names)


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        self.qkv_w = weights[_projection(spec)[1]]
        if self.qkv_w.shape[0] % 8:
            # the attention kernels read the projection's rows in 16-byte pieces: rows of zeros after a gate's few
            # make the row stride a multiple of eight elements (their outputs are never read)
            pad = torch.zeros((-self.qkv_w.shape[0] % 8, self.qkv_w.shape[1]), dtype=self.qkv_w.dtype, device=self.qkv_w.device)
            self.qkv_w = weights[_projection(spec)[1]] = torch.cat([self.qkv_w, pad], dim=0)
        self.qkv_b = weights[_joined(spec.qkv_bias)] if spec.qkv_bias else None
        if self.qkv_b is not None and self.qkv_b.numel() < self.qkv_w.shape[0]:
            self.qkv_b = torch.cat([self.qkv_b, self.qkv_b.new_zeros(self.qkv_w.shape[0] - self.qkv_b.numel())])
        self.out_w = weights[spec.out_weight]
        self.out_b = weights[spec.out_bias] if spec.out_bias else None
        self.value_dim = spec.value_dim or spec.head_dim
        self.q_width = spec.n_heads * spec.head_dim
        self.kv_width = spec.n_kv_heads * spec.head_dim if spec.own_keys_values else 0
        self.v_width = spec.n_kv_heads * self.value_dim if spec.own_keys_values else 0
        self.query_norm = weights[spec.query_norm] if spec.query_norm else None
        self.key_norm = weights[spec.key_norm] if spec.key_norm else None
        if self.key_norm is not None and not spec.own_keys_values:
            raise ValueError("a mixer without keys of its own has no key norm")
        plain = self.value_dim == spec.head_dim
        if spec.head_dim > 256 or self.value_dim > 256:
            raise ValueError(f"head sizes {spec.head_dim} and {self.value_dim} are not supported (at most 256)")
        if spec.gate_weight and spec.qkv_bias:
            raise ValueError("a gated attention with projection biases is not supported")
        self.rotary = None if spec.rotary is None else lookup(POSITIONS, spec.rotary, "position encoding")(spec.rotary, weights, runtime)
        self.sink = weights[spec.sink] if spec.sink else None
        if spec.unit_sink:
            if spec.sink:
                raise ValueError("a unit term in the softmax's denominator and a learned sink do not go together")
            self.sink = torch.zeros(spec.n_heads, dtype=torch.float32, device=runtime.device)      # exp(0) = 1
        if spec.values_are_keys and self.value_dim != spec.head_dim:
            raise ValueError("values that are the keys have the keys' size")
        if spec.gate_per_element and not spec.gate_weight:
            raise ValueError("a gate per element needs the gate's projection")
        self.gate_width = 0 if not spec.gate_weight else (spec.n_heads * self.value_dim if spec.gate_per_element else spec.n_heads)
        self.value_mix = weights[spec.value_mix] if spec.value_mix else None
        if (spec.value_mix or spec.value_mix_source) and not spec.own_keys_values:
            raise ValueError("values are blended only by a mixer with values of its own")
        if spec.keep_first < 0 or (spec.softcap is not None and spec.softcap <= 0):
            raise ValueError("keep_first must not be negative and a score cap must be positive")
        # what the attention kernels are told beside heads, scale and window
        self.mask = dict(chunk=spec.chunk, value_dim=None if plain else self.value_dim, keep_first=spec.keep_first,
                         softcap=spec.softcap, sink=self.sink, exact_weights=spec.exact_weights)
        # (the tcgen05 prompt kernel takes a sink, none of the others)
        plain = plain and not spec.keep_first and not spec.softcap and not spec.exact_weights
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads cannot share {spec.n_kv_heads} key/value heads")
        # where this mixer likes a prompt to be cut: the key block of its prompt kernel, if that kernel takes its sizes
        self.portion_multiple = 1
        if runtime.dtype == torch.bfloat16 and runtime.attention == "auto" and runtime.gemm != "simt" and plain:
            self.portion_multiple = prompt_key_block(spec.n_heads, spec.n_kv_heads, spec.head_dim, runtime.page_size, runtime.dtype)

    @staticmethod
    def tensor_decls(spec):
        q, kv = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        v = spec.n_kv_heads * (spec.value_dim or spec.head_dim)
        if not spec.own_keys_values:
            kv = v = 0
        attended = spec.n_heads * (spec.value_dim or spec.head_dim)
        gate = 0 if not spec.gate_weight else (attended if spec.gate_per_element else spec.n_heads)
        total = q + kv + v + gate
        io = spec.stored_in_out
        matrix = lambda n: (spec.width, n) if io else (n, spec.width)
        # one fused projection in the checkpoint, or separate query, key and value (and gate) projections joined at load
        names, key = _projection(spec)
        shapes = (matrix(q), matrix(kv), matrix(v), matrix(gate)) if spec.own_keys_values else (matrix(q), matrix(gate))
        pieces = () if isinstance(names, str) else tuple(zip(names, shapes))
        decls = [TensorDecl(key, matrix(total), "matrix", io, pieces),
                 TensorDecl(spec.out_weight, (attended, spec.width) if io else (spec.width, attended), "matrix", io)]
        if spec.qkv_bias:
            pieces = () if isinstance(spec.qkv_bias, str) else tuple(zip(spec.qkv_bias, ((q,), (kv,), (v,))))
            decls.append(TensorDecl(_joined(spec.qkv_bias), (total,), "vector", False, pieces))
        if spec.out_bias:
            decls.append(TensorDecl(spec.out_bias, (spec.width,), "vector"))
        for name, heads in ((spec.query_norm, spec.n_heads), (spec.key_norm, spec.n_kv_heads)):
            if name:
                decls.append(TensorDecl(name, (heads * spec.head_dim if spec.norm_whole_projection else spec.head_dim,), "vector"))
        if spec.sink:
            decls.append(TensorDecl(spec.sink, (spec.n_heads,), "vector"))
        if spec.value_mix:
            decls.append(TensorDecl(spec.value_mix, (), "vector"))
        return decls

    @staticmethod
    def cache_needs(spec):
        if not spec.own_keys_values:
            return []
        value_dim = None if spec.value_dim in (None, spec.head_dim) else spec.value_dim
        # the cache keeps what the widest mask that reads it needs (other stops may read it through masks of their own)
        kept = spec.window if spec.keep_window is None else (None if spec.keep_window == "all" else int(spec.keep_window))
        return [PagedKeyValues(spec.n_kv_heads, spec.head_dim, kept, value_dim, spec.chunk,
                               spec.keep_first if kept is not None or spec.chunk is not None else 0)]

    def forward(self, y, residual, ctx, cache, position):
        s = self.spec
        qkv = linear(self.runtime, y, self.qkv_w, self.qkv_b)
        q = qkv[:, :self.q_width]
        k = v = None
        if s.own_keys_values:
            k = qkv[:, self.q_width:self.q_width + self.kv_width]
            v = qkv[:, self.q_width + self.kv_width:self.q_width + self.kv_width + self.v_width]
        elif cache.writable:
            raise ValueError("a mixer without keys and values of its own must read another stop's cache (RunEntry.cache_of)")
        gate = qkv[:, self.q_width + self.kv_width + self.v_width:][:, :self.gate_width] if s.gate_weight else None
        q, k = position.on_query_key(q, k, ctx)
        if s.norm_whole_projection:
            # the norm over all heads at once and the rotation, one pass (values that are the keys were projected a
            # second time and stay as they are)
            if self.rotary is not None and self.rotary.magnitude != 1.0:
                raise ValueError("a norm over the whole projection takes plain rotary frequencies (no scaled cosines)")
            kernels.wide_norm_rotary(q, k, ctx.positions, self.query_norm, self.key_norm, s.head_norm_eps, s.n_heads,
                                     s.n_kv_heads if k is not None else 0, s.head_dim,
                                     freqs=None if self.rotary is None else self.rotary.freqs,
                                     interleaved=True if self.rotary is None else self.rotary.spec.interleaved)
        elif self.query_norm is not None or self.key_norm is not None or (k is None and self.rotary is not None):
            # the heads' norm and the rotation in one pass over the projection's output (the normed value is rotated as
            # float32); a rotation that also scales cosine and sine follows as a pass of its own
            fused = self.rotary is not None and self.rotary.magnitude == 1.0
            kernels.head_norm_rotary(q, k, ctx.positions, self.query_norm, self.key_norm, s.head_norm_eps, s.n_heads,
                                     s.n_kv_heads if k is not None else 0, s.head_dim,
                                     freqs=self.rotary.freqs if fused else None,
                                     interleaved=self.rotary.spec.interleaved if fused else True)
            if self.rotary is not None and not fused:
                if k is None:
                    raise ValueError("a rotation with scaled cosines needs keys of the mixer's own")
                q, k = self.rotary.on_query_key(q, k, ctx)
        elif self.rotary is not None:
            q, k = self.rotary.on_query_key(q, k, ctx)
        if s.value_mix_source:
            ctx.shared["values_to_mix"] = v          # later mixers of this step blend their values with these
        elif self.value_mix is not None:
            first = ctx.shared.get("values_to_mix")
            if first is None or first.shape != v.shape:
                raise ValueError("values are blended with those of an earlier mixer of the same step and shape; none was left")
            kernels.blend_rows(v, first, self.value_mix)
        attended = ctx.attend(q, k, v, cache, s.n_heads, s.scale, s.window, gate=None if s.gate_per_element else gate, **self.mask)
        if s.gate_per_element:
            kernels.sigmoid_gate(attended, gate)
        return linear(self.runtime, attended, self.out_w, self.out_b, residual=residual, out_dtype=residual.dtype,
                      out=residual)
