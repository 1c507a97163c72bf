"""The state-space mixer: a recurrent state per head with a scalar decay, fed through a short causal convolution.

One projection gives [z | x | B | C | dt]. x, B and C pass the convolution (``kernels.conv_channels``: the taps - 1 inputs
before a step's first token are per-request state named 'conv') and silu, as float32; ``kernels.state_space_scan`` runs
S <- exp(-exp(A) dt) S + dt B x^T, y = S^T C + D x per head from the request's float32 state (a state without a name), with
dt = softplus(dt + bias) computed there in float32; ``kernels.gated_group_norm`` multiplies y by silu(z), norms it in equal
stretches, weights it and rounds once, to the operand of the output projection, whose epilogue adds into the stream. A
portion of a prompt continues exactly where the portion before stopped.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import RequestState
from .interfaces import Mixer
from .linear import linear
from .registry import register_mixer
from .spec import TensorDecl


def _sizes(spec):
    inner = spec.n_heads * spec.value_dim
    channels = inner + 2 * spec.groups * spec.state
    return inner, channels, inner + channels + spec.n_heads


@register_mixer("state_space")
class StateSpace(Mixer):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        s = spec
        if s.n_heads % s.groups:
            raise ValueError(f"{s.n_heads} heads cannot share {s.groups} groups of B and C")
        self.inner, self.channels, rows = _sizes(s)
        if self.inner % s.norm_groups:
            raise ValueError(f"{self.inner} channels do not fall into {s.norm_groups} equal stretches")
        if s.conv_taps < 1:
            raise ValueError("a convolution needs at least one tap")
        kernels.state_space_state_shape(s.n_heads, s.state, s.value_dim)        # raises for sizes the kernel does not take
        self.in_w = weights[s.in_weight]
        if self.in_w.shape[0] % 8:
            # rows of zeros make the projection's row stride a multiple of eight elements (their outputs are never read)
            pad = torch.zeros((-self.in_w.shape[0] % 8, self.in_w.shape[1]), dtype=self.in_w.dtype, device=self.in_w.device)
            self.in_w = weights[s.in_weight] = torch.cat([self.in_w, pad], dim=0)
        self.conv_w, self.conv_b = weights[s.conv_weight], weights[s.conv_bias]
        self.dt_bias, self.decay_log, self.skip = weights[s.dt_bias], weights[s.decay_log], weights[s.skip]
        self.out_norm, self.out_w = weights[s.out_norm], weights[s.out_weight]

    @staticmethod
    def tensor_decls(spec):
        s = spec
        inner, channels, rows = _sizes(s)
        return [TensorDecl(s.in_weight, (rows, s.width), "matrix"),
                TensorDecl(s.conv_weight, (channels, s.conv_taps), "vector"),
                TensorDecl(s.conv_bias, (channels,), "vector"),
                TensorDecl(s.dt_bias, (s.n_heads,), "vector"),
                TensorDecl(s.decay_log, (s.n_heads,), "vector"),
                TensorDecl(s.skip, (s.n_heads,), "vector"),
                TensorDecl(s.out_norm, (inner,), "vector"),
                TensorDecl(s.out_weight, (s.width, inner), "matrix")]

    @staticmethod
    def cache_needs(spec):
        s = spec
        needs = [RequestState(kernels.state_space_state_shape(s.n_heads, s.state, s.value_dim), "float32")]
        if s.conv_taps > 1:
            needs.append(RequestState((s.conv_taps - 1, _sizes(s)[1]), "float32", name="conv"))
        return needs

    def forward(self, y, residual, ctx, cache, position):
        s, inner, channels = self.spec, self.inner, self.channels
        if cache.state is None or (s.conv_taps > 1 and "conv" not in (cache.named or {})):
            raise ValueError("the state-space mixer needs its per-request state (a stop of the run order with a cache of its own)")
        proj = linear(self.runtime, y, self.in_w)
        z, xbc_in, dt = proj[:, :inner], proj[:, inner:inner + channels], proj[:, inner + channels:inner + channels + s.n_heads]
        conv_state = cache.named["conv"] if s.conv_taps > 1 else proj.new_zeros((1, 0, channels), dtype=torch.float32)
        xbc = kernels.conv_channels(xbc_in, self.conv_w, self.conv_b, conv_state, ctx.token_entry, ctx.entry_start, ctx.entry_slot,
                                    activation="silu")
        if s.conv_taps > 1:
            kernels.conv_state_update(xbc_in, conv_state, ctx.entry_start, ctx.entry_slot)
        read = kernels.state_space_scan(xbc, dt, self.dt_bias, self.decay_log, self.skip, ctx.entry_start, ctx.entry_slot, cache.state,
                                        s.n_heads, s.groups, s.state, s.value_dim)
        mixed = kernels.gated_group_norm(read, z, self.out_norm, s.norm_groups, s.norm_eps, proj.dtype)
        return linear(self.runtime, mixed, self.out_w, residual=residual, out_dtype=residual.dtype, out=residual)
