"""The gated-delta mixer: a linear-attention state per head that every token first decays per key channel, then corrects
towards its value (the delta rule) and reads.

One fused projection gives q, k, v, the two low-rank inputs (of the decay and of the output gate) and beta; two small
products take the low-rank inputs up (float32 results). ``kernels.delta_prepare`` makes the recurrence's float32 operands
(short causal convolutions with silu, unit queries and keys, decay, beta); the convolution's last inputs and the state S
are per-request state (a state without a name for S, one named 'conv'), so a portion of a prompt continues exactly where
the portion before stopped. ``kernels.delta_rule`` runs the recurrence, ``kernels.delta_finish`` norms and gates the
read-out, and the output projection adds into the stream in its epilogue. Everything between the projections' outputs
and the operand of the output projection is float32.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import RequestState
from .interfaces import Mixer
from .linear import linear
from .registry import register_mixer
from .spec import TensorDecl


def _pieces(spec):
    """(checkpoint name, rows) of the fused projection's pieces, in the order they lie in its output."""
    s = spec
    qk, v = s.n_kv_heads * s.head_dim, s.n_heads * s.value_dim
    return ((s.query_weight, qk), (s.key_weight, qk), (s.value_weight, v), (s.decay_down, s.decay_rank),
            (s.gate_down, s.gate_rank), (s.beta_weight, s.n_heads))


def _conv_names(spec):
    return tuple(n + ".conv" for n in (spec.query_weight, spec.key_weight, spec.value_weight))


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        s = spec
        if s.n_heads % s.n_kv_heads:
            raise ValueError(f"{s.n_heads} heads cannot share {s.n_kv_heads} query/key heads")
        if s.head_dim > 256:
            raise ValueError(f"a delta-rule head of {s.head_dim} is not supported (at most 256)")
        if s.conv_taps < 1:
            raise ValueError("a convolution needs at least one tap")
        key = "+".join(n for n, _ in _pieces(s))
        self.proj_w = weights[key]
        if self.proj_w.shape[0] % 8:
            pad = torch.zeros((-self.proj_w.shape[0] % 8, self.proj_w.shape[1]), dtype=self.proj_w.dtype, device=self.proj_w.device)
            self.proj_w = weights[key] = torch.cat([self.proj_w, pad], dim=0)
        self.channels = 2 * s.n_kv_heads * s.head_dim + s.n_heads * s.value_dim
        self.conv_w = weights["+".join(_conv_names(s))]
        self.decay_up, self.gate_up = weights[s.decay_up], weights[s.gate_up]
        self.decay_log, self.decay_bias = weights[s.decay_log], weights[s.decay_bias]
        self.out_norm, self.out_w = weights[s.out_norm], weights[s.out_weight]

    @staticmethod
    def tensor_decls(spec):
        s = spec
        pieces = _pieces(s)
        qk, v = s.n_kv_heads * s.head_dim, s.n_heads * s.value_dim
        return [TensorDecl("+".join(n for n, _ in pieces), (sum(r for _, r in pieces), s.width), "matrix", False,
                           tuple((n, (r, s.width)) for n, r in pieces)),
                TensorDecl("+".join(_conv_names(s)), (2 * qk + v, s.conv_taps), "vector", False,
                           tuple(zip(_conv_names(s), ((qk, s.conv_taps), (qk, s.conv_taps), (v, s.conv_taps))))),
                TensorDecl(s.decay_up, (s.n_heads * s.head_dim, s.decay_rank), "matrix"),
                TensorDecl(s.gate_up, (v, s.gate_rank), "matrix"),
                TensorDecl(s.decay_log, (s.n_heads,), "vector"),
                TensorDecl(s.decay_bias, (s.n_heads * s.head_dim,), "vector"),
                TensorDecl(s.out_norm, (s.value_dim,), "vector"),
                TensorDecl(s.out_weight, (s.width, v), "matrix")]

    @staticmethod
    def cache_needs(spec):
        s = spec
        channels = 2 * s.n_kv_heads * s.head_dim + s.n_heads * s.value_dim
        needs = [RequestState(kernels.delta_state_shape(s.n_heads, s.head_dim, s.value_dim), "float32")]
        if s.conv_taps > 1:
            needs.append(RequestState((s.conv_taps - 1, channels), "float32", name="conv"))
        return needs

    def _low_rank(self, proj, start, rank, up):
        """The float32 result of the second product of a low-rank pair; its input is a column slice of the fused projection's
        output (copied where the slice does not start on a 16-byte boundary, which the tensor-core product needs)."""
        x = proj[:, start:start + rank]
        if (x.data_ptr() % 16 or rank % 8) and x.dtype == torch.bfloat16:
            x = x.clone(memory_format=torch.contiguous_format)      # (a single row counts as contiguous wherever it starts)
        return linear(self.runtime, x, up, out_dtype=torch.float32)

    def forward(self, y, residual, ctx, cache, position):
        s, c = self.spec, self.channels
        if cache.state is None or (s.conv_taps > 1 and "conv" not in (cache.named or {})):
            raise ValueError("the gated-delta mixer needs its per-request state (a stop of the run order with a cache of its own)")
        proj = linear(self.runtime, y, self.proj_w)
        step_in = self._low_rank(proj, c, s.decay_rank, self.decay_up)
        gate = self._low_rank(proj, c + s.decay_rank, s.gate_rank, self.gate_up)
        beta_at = c + s.decay_rank + s.gate_rank
        conv_state = cache.named["conv"] if s.conv_taps > 1 else proj.new_zeros((1, 0, c), dtype=torch.float32)
        q, k, v, decay, beta = kernels.delta_prepare(proj, proj[:, beta_at:beta_at + s.n_heads], step_in, self.conv_w, conv_state,
                                                     self.decay_log, self.decay_bias, ctx.token_entry, ctx.entry_start,
                                                     ctx.entry_slot, s.n_heads, s.n_kv_heads, s.head_dim, s.value_dim)
        if s.conv_taps > 1:
            kernels.conv_state_update(proj, conv_state, ctx.entry_start, ctx.entry_slot)
        o = kernels.delta_rule(q, k, v, decay, beta, ctx.entry_start, ctx.entry_slot, cache.state, s.n_heads, s.n_kv_heads,
                               s.head_dim, s.value_dim)
        mixed = kernels.delta_finish(o, gate, self.out_norm, s.n_heads, s.norm_eps, proj.dtype)
        return linear(self.runtime, mixed, self.out_w, residual=residual, out_dtype=residual.dtype, out=residual)
