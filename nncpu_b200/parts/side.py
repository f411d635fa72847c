"""A per-layer input from the token itself, added to the stream at the end of a layer.

With x the stream, e the layer's ``dim`` lanes of the token's row in a table shared by all layers, and m the layer's
residual weight:

    g = gelu_tanh(W_gate x) * e,   y = W_proj g,   x <- x + m * y / sqrt(mean(y^2) + eps) * w

The gate's product reads the stream itself, not a norm of it: rounded to the run's element type where a bfloat16 run
multiplies on the tensor cores, and as it is in a step of a few tokens, whose gate is one launch (product, activation,
gating).
The activation, the gating, the norm and the sum are 32-bit.  A layer that runs several times in a schedule uses the
same lanes every time.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.params import ParamSpec
from .base import Part, norm_output_buffer


class TokenSide(Part):
    def __init__(self, spec):
        self.spec = spec

    def params(self):
        s = self.spec
        return [ParamSpec(f"{s.name}.gate", (s.dim, s.hidden_size)),
                ParamSpec(f"{s.name}.proj", (s.hidden_size, s.dim)),
                ParamSpec(f"{s.name}.norm", (s.hidden_size,), init=("one_plus_normal", 0.1))]

    def table_param(self) -> ParamSpec:
        """The table all layers share; the model lists it once."""
        s = self.spec
        return ParamSpec(s.table, (s.vocab_size, s.table_width), init=("normal", 1.0))

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        self.w_gate, self.w_proj, self.w_norm = (tensors[f"{s.name}.{n}"] for n in ("gate", "proj", "norm"))
        self.table = tensors[s.table]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_gate, self.w_proj))

    def forward(self, ctx, residual, mult: float, then=None) -> None:
        """``then``: the request of the norm that reads the stream next; the closing kernel can leave its output."""
        s, rt = self.spec, self.rt
        n = residual.shape[0]
        with rt.scope():
            g = rt.empty(n, s.dim)
            if n <= ops.GATE_ROWS_MAX_TOKENS:
                # a few tokens: the gate's product, the activation and the gating in one launch (a warp a row of the
                # matrix, which is read once for all tokens; the stream is read as it is)
                with rt.phase("side_gate", self.w_gate, n):
                    ops.token_gate_rows(residual, self.w_gate, self.table, ctx.tok_ids, s.col, g)
            else:
                if rt.dtype == torch.float32:
                    x = residual
                else:
                    x = rt.empty(n, s.hidden_size)
                    with rt.phase("side_gate"):
                        ops.concat_rows(residual, None, x)
                z = rt.empty(n, s.dim, dtype=torch.float32)
                with rt.phase("side_gate", self.w_gate, n):
                    rt.linear(x, self.w_gate, None, z)
                with rt.phase("side_gate"):
                    ops.token_gate(z, self.table, ctx.tok_ids, s.col, g)
            y = rt.empty(n, s.hidden_size, dtype=torch.float32)
            with rt.phase("side_proj", self.w_proj, n):
                rt.linear(g, self.w_proj, None, y)
            with rt.phase("norm", nbytes=12.0 * y.numel()):
                if then is not None and then.wants_output and hasattr(then.norm, "closing") and then.residual is residual:
                    out = norm_output_buffer(ctx, rt, residual.shape)
                    ops.branch_norm_add(residual, y, self.w_norm, None, None, s.eps, mult, then_norm=then.norm.closing(out))
                    then.output = out
                else:
                    ops.branch_norm_add(residual, y, self.w_norm, None, None, s.eps, mult)
