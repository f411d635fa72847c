"""Norms.  RMSNorm with learned weights: y = x / sqrt(mean(x^2) + eps) * (gamma + offset)
(crates/nncpu/src/kernels/scalar.rs:270-292), computed in 32-bit.  ``offset`` is 0 for weights stored around
one and 1 for weights stored around zero."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.params import ParamSpec
from .base import Norm, NormRequest, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec):
        self.size, self.eps, self.name = spec.size, spec.eps, spec.name
        self.tensor = spec.name + spec.suffix
        self.offset = float(spec.offset)
        self.gamma = None

    def params(self):
        return [ParamSpec(self.tensor, (self.size,), init=("normal" if self.offset else "one_plus_normal", 0.1))]

    def bind(self, tensors, rt):
        self.rt = rt
        self.gamma = tensors[self.tensor]

    def forward(self, ctx, residual, rows=None):
        n = residual.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.size)
        with self.rt.phase("norm"):
            ops.rmsnorm(residual, self.gamma, self.eps, out, rows, gamma_offset=self.offset)
        return out

    def add_into(self, ctx, x, residual) -> None:
        """residual += norm(x): the norm that closes a sublayer (32-bit, one pass over both)."""
        with self.rt.phase("norm"):
            ops.rmsnorm(x, self.gamma, self.eps, residual, gamma_offset=self.offset, accumulate=True)

    def request(self, ctx, residual):
        """In a bfloat16 run the products around this norm can carry it: the few-token products at up to 16
        tokens, the tensor-core products of whole prompts (a launch, and at many tokens a pass over the residual
        stream, less)."""
        if (self.offset != 0.0 or self.rt.dtype != torch.bfloat16 or self.size % 16 or residual.dtype != torch.float32
                or not self.rt.fuses_norms(ctx.n_tokens, self.size)):
            return None
        return NormRequest(self, residual, self.gamma, self.eps, self.size)


@register_norm("layernorm")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * w + b over the row, var the mean of the squared deviations from the mean;
    32-bit.  It does not ride on the products around it (they carry sums of squares, not means)."""

    def __init__(self, spec):
        self.size, self.eps, self.name = spec.size, spec.eps, spec.name
        self.tensor = spec.name + spec.suffix
        self.bias_tensor = self.tensor + spec.bias_suffix
        self.gamma = self.beta = None

    def params(self):
        return [ParamSpec(self.tensor, (self.size,), init=("one_plus_normal", 0.1)),
                ParamSpec(self.bias_tensor, (self.size,), init=("normal", 0.1))]

    def bind(self, tensors, rt):
        self.rt = rt
        self.gamma, self.beta = tensors[self.tensor], tensors[self.bias_tensor]

    def forward(self, ctx, residual, rows=None):
        n = residual.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.size)
        with self.rt.phase("norm"):
            ops.layernorm(residual, self.gamma, self.beta, self.eps, out, rows)
        return out

    def request(self, ctx, residual):
        """A kernel that closes a sublayer with a norm of its own (``ops.branch_norm_add``) holds the stream's new rows in
        registers and can leave this norm's output in the same pass: the request asks for that (``wants_output``)."""
        if residual.dtype != torch.float32 or not ops.branch_norm_add_takes_norm(self.size):
            return None
        return NormRequest(self, residual, self.gamma, self.eps, self.size, wants_output=True)

    def closing(self, out):
        """What ``ops.branch_norm_add`` takes as ``then_norm`` to leave this norm's output in ``out``."""
        return (self.gamma, self.beta, self.eps, out)
