"""The gated linear recurrence mixer: a decaying state per channel whose decay and input gate depend on the token.

One projection (with its biases) gives the two branches [g | u_in]. u = conv(u_in) (``kernels.conv_channels`` with a
bias and no activation; the taps - 1 inputs before a step's first token are per-request state named 'conv') as float32;
``kernels.recurrence_gates`` computes, per part of the channels, r = sigmoid(Ra u + ba), i = sigmoid(Ri u + bi),
a = exp(-gain r softplus(lam)) (handed on as 1 - a) and the drive sqrt(1 - a^2) i u as float32 sums; ``kernels.linear_scan`` runs
S <- a S + drive from the request's float32 state (a state without a name) and writes S * gelu_tanh(g), rounded once, as the
operand of the output projection, whose epilogue adds into the stream.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import RequestState
from .interfaces import Mixer
from .linear import linear
from .registry import register_mixer
from .spec import TensorDecl


@register_mixer("linear_recurrence")
class LinearRecurrence(Mixer):
    graph_safe = True

    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        s = spec
        if s.inner % s.blocks:
            raise ValueError(f"{s.inner} channels do not fall into {s.blocks} equal parts")
        if s.conv_taps < 1:
            raise ValueError("a convolution needs at least one tap")
        key = s.gate_weight + "+" + s.in_weight
        self.proj_w, self.proj_b = weights[key], weights[s.gate_bias + "+" + s.in_bias]
        if self.proj_w.shape[0] % 8:
            pad = -self.proj_w.shape[0] % 8
            self.proj_w = weights[key] = torch.cat([self.proj_w, self.proj_w.new_zeros((pad, self.proj_w.shape[1]))], dim=0)
            self.proj_b = torch.cat([self.proj_b, self.proj_b.new_zeros(pad)])
        self.conv_w, self.conv_b = weights[s.conv_weight], weights[s.conv_bias]
        self.wa, self.ba = weights[s.decay_gate], weights[s.decay_gate_bias].reshape(-1)
        self.wi, self.bi = weights[s.input_gate], weights[s.input_gate_bias].reshape(-1)
        self.lam, self.out_w = weights[s.decay_param], weights[s.out_weight]

    @staticmethod
    def tensor_decls(spec):
        s = spec
        part = s.inner // s.blocks
        return [TensorDecl(s.gate_weight + "+" + s.in_weight, (2 * s.inner, s.width), "matrix", False,
                           ((s.gate_weight, (s.inner, s.width)), (s.in_weight, (s.inner, s.width)))),
                TensorDecl(s.gate_bias + "+" + s.in_bias, (2 * s.inner,), "vector", False,
                           ((s.gate_bias, (s.inner,)), (s.in_bias, (s.inner,)))),
                TensorDecl(s.conv_weight, (s.inner, s.conv_taps), "vector"),
                TensorDecl(s.conv_bias, (s.inner,), "vector"),
                # the gates are part of the recurrence: their matrices stay float32 whatever the engine's dtype
                TensorDecl(s.decay_gate, (s.blocks, part, part), "vector"),
                TensorDecl(s.decay_gate_bias, (s.blocks, part), "vector"),
                TensorDecl(s.input_gate, (s.blocks, part, part), "vector"),
                TensorDecl(s.input_gate_bias, (s.blocks, part), "vector"),
                TensorDecl(s.decay_param, (s.inner,), "vector"),
                TensorDecl(s.out_weight, (s.width, s.inner), "matrix")]

    @staticmethod
    def cache_needs(spec):
        needs = [RequestState((spec.inner,), "float32")]
        if spec.conv_taps > 1:
            needs.append(RequestState((spec.conv_taps - 1, spec.inner), "float32", name="conv"))
        return needs

    def forward(self, y, residual, ctx, cache, position):
        s = self.spec
        if cache.state is None or (s.conv_taps > 1 and "conv" not in (cache.named or {})):
            raise ValueError("the linear recurrence needs its per-request state (a stop of the run order with a cache of its own)")
        proj = linear(self.runtime, y, self.proj_w, self.proj_b)
        gate, u_in = proj[:, :s.inner], proj[:, s.inner:2 * s.inner]
        conv_state = cache.named["conv"] if s.conv_taps > 1 else proj.new_zeros((1, 0, s.inner), dtype=torch.float32)
        u = kernels.conv_channels(u_in, self.conv_w, self.conv_b, conv_state, ctx.token_entry, ctx.entry_start, ctx.entry_slot)
        if s.conv_taps > 1:
            kernels.conv_state_update(u_in, conv_state, ctx.entry_start, ctx.entry_slot)
        fade, drive = kernels.recurrence_gates(u, self.wa, self.ba, self.wi, self.bi, self.lam, s.gain)      # fade = 1 - a
        mixed = kernels.linear_scan(fade, drive, gate, ctx.entry_start, ctx.entry_slot, cache.state, activation="gelu_tanh")
        return linear(self.runtime, mixed, self.out_w, residual=residual, out_dtype=residual.dtype, out=residual)
