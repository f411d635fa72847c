"""The gated delta rule: a recurrent mixer that keeps, per sequence and head, a state S of ``key_dim`` x
``value_dim`` 32-bit floats, and the last inputs of its short convolutions, in the cache's state area.

With h the mixer's input, H heads, G query/key heads (head a of H uses query/key head a // (H / G)), d = key_dim,
e = value_dim, and conv_T a causal convolution over time per channel (T taps, the last one the current token's, zeros
before the sequence's start):

    q = silu(conv_T(W_q h)),  k = silu(conv_T(W_k h))       [G, d]     then q <- q / |q| * d^(-1/2),  k <- k / |k|
    v = silu(conv_T(W_v h))                                  [H, e]     (|x| = sqrt(sum x^2 + 1e-6) per head)
    beta = sigmoid(W_b h),   g = exp(-exp(A_log) * softplus(W_a h + dt_bias))        one of each per head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q                  (the read-out sees the write)
    out = W_o concat_heads(o / rms(o) * w_norm * silu(W_g h))

The six projections of h are one product (their rows stacked); it runs in the run's element type with 32-bit
accumulators and its results stay float32.  Convolutions, activations, unit vectors, decays, the recurrence and the
norm are 32-bit in both run types.  The recurrence walks a sequence's tokens in order with a fixed order of operations
per (sequence, head, column) that follows from the layer's sizes alone, so a prompt cut into portions, a batch of
unequal sequences and a prompt decoded token by token give the same bits.
"""
from __future__ import annotations

import torch

from ..cache import StateRequest
from ..errors import UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from .base import Mixer, register_mixer

MAX_KEY_DIM = 1024     # the scan kernel spreads a column's rows over the 32 lanes of a warp, 32 rows a lane
MAX_TAPS = 32


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    accepts_deferred_norm = True    # x goes to Runtime.linear alone

    def __init__(self, spec, reads_other_cache: bool = False):
        if reads_other_cache:
            raise UnsupportedModel(f"{spec.name}: a recurrent mixer keeps no keys and values that another layer could read")
        if spec.key_dim > MAX_KEY_DIM:
            raise UnsupportedModel(f"{spec.name}: {spec.key_dim} key channels a head (at most {MAX_KEY_DIM})")
        if not 1 <= spec.conv <= MAX_TAPS:
            raise UnsupportedModel(f"{spec.name}: convolutions of {spec.conv} taps (1 to {MAX_TAPS})")
        if spec.n_heads % spec.n_kv_heads:
            raise UnsupportedModel(f"{spec.name}: {spec.n_heads} heads over {spec.n_kv_heads} query/key heads")
        s = self.spec = spec
        self.qk_size = s.n_kv_heads * s.key_dim
        self.v_size = s.n_heads * s.value_dim
        self.channels = 2 * self.qk_size + self.v_size              # what the convolutions run over
        self.gate_col = self.channels                               # the output gate's logits follow them in a row
        self.proj_size = self.channels + self.v_size + 2 * s.n_heads
        self.state_floats = s.n_heads * s.key_dim * s.value_dim     # S of every head, then the convolutions' inputs
        self.conv_floats = (s.conv - 1) * self.channels

    def state_request(self):
        return StateRequest((self.state_floats + self.conv_floats,), torch.float32)

    def params(self):
        s = self.spec
        return [ParamSpec(f"{s.name}.q", (self.qk_size, s.hidden_size)),
                ParamSpec(f"{s.name}.q.conv", (self.qk_size, s.conv), init=("normal", 0.5)),
                ParamSpec(f"{s.name}.k", (self.qk_size, s.hidden_size)),
                ParamSpec(f"{s.name}.k.conv", (self.qk_size, s.conv), init=("normal", 0.5)),
                ParamSpec(f"{s.name}.v", (self.v_size, s.hidden_size)),
                ParamSpec(f"{s.name}.v.conv", (self.v_size, s.conv), init=("normal", 0.5)),
                ParamSpec(f"{s.name}.b", (s.n_heads, s.hidden_size)),
                ParamSpec(f"{s.name}.a", (s.n_heads, s.hidden_size)),
                ParamSpec(f"{s.name}.A_log", (s.n_heads,), init=("normal", 0.5)),
                ParamSpec(f"{s.name}.dt_bias", (s.n_heads,), init=("normal", 0.5)),
                ParamSpec(f"{s.name}.g", (self.v_size, s.hidden_size)),
                ParamSpec(f"{s.name}.norm", (s.value_dim,), init=("one_plus_normal", 0.1)),
                ParamSpec(f"{s.name}.o", (s.hidden_size, self.v_size))]

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        # rows of the one product: q, k, v (the convolutions' channels), the output gate, beta's logits, the decays' inputs
        ws = [tensors.pop(f"{s.name}.{n}") for n in ("q", "k", "v", "g", "b", "a")]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        del ws
        self.w_conv = torch.cat([tensors.pop(f"{s.name}.{n}.conv") for n in ("q", "k", "v")], dim=0).contiguous()
        self.a_log, self.dt_bias = tensors[f"{s.name}.A_log"], tensors[f"{s.name}.dt_bias"]
        self.w_o, self.w_norm = tensors[f"{s.name}.o"], tensors[f"{s.name}.norm"]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_conv, self.w_o))

    def forward(self, ctx, x, residual, cache):
        s, rt = self.spec, self.rt
        n, H, G, d, e = x.shape[0], s.n_heads, s.n_kv_heads, s.key_dim, s.value_dim
        proj = rt.empty(n, self.proj_size, dtype=torch.float32)
        with rt.phase("delta_proj", self.w_in, n):
            rt.linear(x, self.w_in, None, proj)
        gated = rt.empty(n, self.v_size)
        state_bytes = 8.0 * ctx.n_seqs * self.state_floats          # read and written once a step
        xc = rt.empty(n, self.channels, dtype=torch.float32)
        gb = rt.empty(n, 2 * H, dtype=torch.float32)
        o = rt.empty(n, self.v_size, dtype=torch.float32)
        with rt.phase("delta_conv", nbytes=4.0 * (proj.numel() + xc.numel())):
            ops.delta_prepare(proj, self.w_conv, cache.state, self.state_floats, ctx.tok_seq, ctx.seq_slots, ctx.cu_seqlens,
                              self.a_log, self.dt_bias, xc, gb, ctx.n_seqs, H, G, d, e, s.conv,
                              one_token_each=ctx.is_decode)
        with rt.phase("delta_scan", nbytes=state_bytes + 4.0 * (xc.numel() + o.numel()), flops=6.0 * n * H * d * e):
            ops.delta_scan(xc, gb, cache.state, ctx.seq_slots, ctx.cu_seqlens, o, ctx.n_seqs, H, G, d, e)
        with rt.phase("delta_gate"):
            ops.gla_output(o, proj, self.w_norm, s.eps, gated, H, d, e, gate_col=self.gate_col)
        with rt.phase("delta_out", self.w_o, n):
            rt.linear(gated, self.w_o, None, residual, accumulate=not getattr(ctx, "branch_is_fresh", False),
                      then_norm=getattr(ctx, "next_norm", None))
