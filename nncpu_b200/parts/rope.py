"""Rotary position embedding, half-split pairing (i, i + rotary_dim/2):
angle_i = float32(position) * scale * theta^(-2i/rotary_dim)
(crates/nncpu/src/kernels/mod.rs:687-737).

The inverse frequencies are computed once in float64 and rounded to float32;
the cosines and sines of a step's positions are computed once per step in
32-bit and shared by every layer that uses the same encoding.

"rope_pairs" has the same table; its mixers turn the neighbouring lanes (2i, 2i + 1) by entry i instead.  Both take
frequencies rescaled between two wavelengths (``PositionSpec.scaling_*``): the rescaled frequencies replace the plain
ones when the weights are bound, and cos and sin are multiplied by one more number when the table is made.
"""
from __future__ import annotations

import math

import torch

from ..errors import BadFormat
from ..kernels import ops
from .base import PositionEncoding, register_position


RAMP_FLOOR = 0.001      # the least width of the ramp between the two wavelengths
STRETCH_SLOPE = 0.1     # cos and sin are multiplied by STRETCH_SLOPE * ln(factor) + 1


@register_position("rope_neox")
class RopeNeox(PositionEncoding):
    tables_by_pair = True

    def __init__(self, spec):
        if spec.rotary_dim % 2 or spec.rotary_dim <= 0:
            raise BadFormat(f"rotary size {spec.rotary_dim} must be even and positive")
        self.spec = spec
        self.half = spec.rotary_dim // 2
        self.inv_freq = None

    def bind(self, tensors, rt):
        self.rt = rt
        s = self.spec
        i = torch.arange(self.half, dtype=torch.float64)
        inv = torch.pow(torch.tensor(float(s.theta), dtype=torch.float64), -2.0 * i / s.rotary_dim)
        self.stretch = 1.0
        if s.scaling_factor > 0.0:
            # pairs whose wavelength lies between the two limits are blended towards a frequency `factor` times lower
            def pair_of(turns: float) -> float:
                return s.rotary_dim * math.log(s.scaling_original / (2.0 * math.pi * turns)) / (2.0 * math.log(s.theta))
            lo = max(math.floor(pair_of(s.scaling_fast)), 0)
            hi = min(math.ceil(pair_of(s.scaling_slow)), s.rotary_dim - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, RAMP_FLOOR), 0.0, 1.0)
            inv = inv / s.scaling_factor * ramp + inv * (1.0 - ramp)
            self.stretch = STRETCH_SLOPE * math.log(s.scaling_factor) + 1.0
        self.inv_freq = inv.to(torch.float32).to(rt.device)

    def tables(self, ctx, by_pair: bool = False):
        """float32 [n_tokens, half, 2] of (cos, sin), or with ``by_pair`` the same
        values as [half, n_tokens, 2]; memoised in the step."""
        key = ("rope", self.spec, by_pair)
        t = ctx.memo.get(key)
        if t is None:
            shape = (self.half, ctx.n_tokens, 2) if by_pair else (ctx.n_tokens, self.half, 2)
            t = self.rt.empty(*shape, dtype=torch.float32, keep=True)     # every later layer of the step reads it
            ops.rope_table(ctx.tok_pos, self.inv_freq, t, self.spec.position_scale, by_pair, self.stretch)
            ctx.memo[key] = t
        return t


@register_position("rope_pairs")
class RopePairs(RopeNeox):
    """The same angles for the neighbouring lanes (2i, 2i + 1).  Its mixers read the table by token."""
    tables_by_pair = False
