"""Norms. LayerNorm with weight and optional bias (damendaemon/starcoder.py:53-55); RMS norm,
x / sqrt(mean(x^2) + eps) * (offset + weight), with the offset a parameter of the spec, and optionally in groups:
the row in equal consecutive stretches, each divided by its own root mean square; a norm without statistics,
tanh(alpha x) * weight + bias with one learned number alpha."""
from __future__ import annotations

from .. import kernels
from .interfaces import Norm
from .registry import register_norm
from .spec import TensorDecl


@register_norm("layernorm")
class LayerNorm(Norm):
    def __init__(self, spec, weights, runtime):
        self.spec, self.runtime = spec, runtime
        self.gamma = weights[spec.weight]
        self.beta = weights[spec.bias] if spec.bias else None

    @staticmethod
    def tensor_decls(spec):
        decls = [TensorDecl(spec.weight, (spec.width,), "vector")]
        if spec.bias:
            decls.append(TensorDecl(spec.bias, (spec.width,), "vector"))
        return decls

    def forward(self, x, row_index=None, out_dtype=None):
        return kernels.layernorm(x, self.gamma, self.beta, self.spec.eps, out_dtype or self.runtime.dtype, row_index)


@register_norm("rmsnorm")
class RmsNorm(Norm):
    def __init__(self, spec, weights, runtime):
        if spec.bias:
            raise ValueError("an RMS norm has no bias")
        if spec.groups < 1 or spec.width % spec.groups:
            raise ValueError(f"a row of {spec.width} does not fall into {spec.groups} equal stretches")
        self.spec, self.runtime = spec, runtime
        self.weight = weights[spec.weight]

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.weight, (spec.width,), "vector")]

    def forward(self, x, row_index=None, out_dtype=None):
        return kernels.rmsnorm(x, self.weight, self.spec.eps, out_dtype or self.runtime.dtype, row_index,
                               offset=self.spec.weight_offset, groups=self.spec.groups)

    def forward_shifted(self, x, shift, state, ctx):
        """The norm of every row blended with the norm of the token before it (kernels.rmsnorm_shift), one kernel."""
        return kernels.rmsnorm_shift(x, self.weight, self.spec.eps, self.runtime.dtype, shift, state, ctx.token_entry,
                                     ctx.entry_start, ctx.entry_slot, offset=self.spec.weight_offset, groups=self.spec.groups)


@register_norm("tanh")
class TanhNorm(Norm):
    """tanh(alpha * x) * weight + bias: no mean, no variance, so a row needs no reduction."""

    def __init__(self, spec, weights, runtime):
        if not spec.bias or not spec.alpha:
            raise ValueError("a tanh norm has a weight, a bias and the number alpha")
        self.spec, self.runtime = spec, runtime
        self.weight, self.bias = weights[spec.weight], weights[spec.bias]
        self.alpha = weights[spec.alpha].reshape(1)

    @staticmethod
    def tensor_decls(spec):
        return [TensorDecl(spec.weight, (spec.width,), "vector"), TensorDecl(spec.bias, (spec.width,), "vector"),
                TensorDecl(spec.alpha, (), "vector")]

    def forward(self, x, row_index=None, out_dtype=None):
        return kernels.tanh_norm(x, self.alpha, self.weight, self.bias, out_dtype or self.runtime.dtype, row_index)
