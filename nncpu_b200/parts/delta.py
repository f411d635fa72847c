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

With ``channel_decay`` the decay is one number per head AND key channel, acting on the rows of S,

    g = exp(-exp(A_log_h) * softplus(W_a2 (W_a1 h) + dt_bias))      laid out [H, d]:   S <- diag(g) S

and the output gate is sigmoid(W_g2 (W_g1 h)) (laid out [H, e]) in place of silu(W_g h); both go through a low rank that
the file's tensors give.  The two low-rank inputs W_a1 h and W_g1 h are one product (rows stacked), and each second
matrix is bound with zero columns for the other's lanes.

The six projections of h are one product (their rows stacked); it runs in the run's element type with 32-bit
accumulators and its results stay float32.  Convolutions, activations, unit vectors, decays, the recurrence and the
norm are 32-bit in both run types.  The recurrence walks a sequence's tokens in order with a fixed order of operations
per (sequence, head, column) that follows from the layer's sizes alone, so a prompt cut into portions, a batch of
unequal sequences and a prompt decoded token by token give the same bits.
"""
from __future__ import annotations

import torch

from ..cache import StateRequest
from ..errors import BadFormat, UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from .base import Mixer, register_mixer

MAX_KEY_DIM = 1024     # the scan kernel spreads a column's rows over the 32 lanes of a warp, 32 rows a lane
MAX_TAPS = 32


@register_mixer("gated_delta")
class GatedDelta(Mixer):
    accepts_deferred_norm = True    # x goes to Runtime.linear alone
    scales_output = True            # ctx.out_scale rides on the heads' norm-and-gate stage, before the output product

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
        self.channel = bool(s.channel_decay)
        self.accepts_deferred_norm = not self.channel      # (its input goes to two products then)
        # per-head decays: the gate's logits, beta's and the decays' inputs follow the channels; per-channel decays:
        # beta's logits alone (the gate and the decays come out of their low-rank products)
        self.proj_size = self.channels + (s.n_heads if self.channel else self.v_size + 2 * s.n_heads)
        self.state_floats = s.n_heads * s.key_dim * s.value_dim     # S of every head, then the convolutions' inputs
        self.conv_floats = (s.conv - 1) * self.channels

    def state_request(self):
        return StateRequest((self.state_floats + self.conv_floats,), torch.float32)

    def params(self):
        s = self.spec
        if self.channel:
            return [ParamSpec(f"{s.name}.q", (self.qk_size, s.hidden_size)),
                    ParamSpec(f"{s.name}.q.conv", (self.qk_size, s.conv), init=("normal", 0.5)),
                    ParamSpec(f"{s.name}.k", (self.qk_size, s.hidden_size)),
                    ParamSpec(f"{s.name}.k.conv", (self.qk_size, s.conv), init=("normal", 0.5)),
                    ParamSpec(f"{s.name}.v", (self.v_size, s.hidden_size)),
                    ParamSpec(f"{s.name}.v.conv", (self.v_size, s.conv), init=("normal", 0.5)),
                    ParamSpec(f"{s.name}.b", (s.n_heads, s.hidden_size)),
                    ParamSpec(f"{s.name}.A_log", (s.n_heads,), init=("normal", 0.5)),
                    ParamSpec(f"{s.name}.norm", (s.value_dim,), init=("one_plus_normal", 0.1)),
                    ParamSpec(f"{s.name}.a1", (s.decay_rank or -1, s.hidden_size)),
                    ParamSpec(f"{s.name}.a2", (s.n_heads * s.key_dim, s.decay_rank or -1), init=("normal", 0.2)),
                    ParamSpec(f"{s.name}.dt_bias", (s.n_heads * s.key_dim,), init=("normal", 0.5)),
                    ParamSpec(f"{s.name}.g1", (s.gate_rank or -1, s.hidden_size)),
                    ParamSpec(f"{s.name}.g2", (self.v_size, s.gate_rank or -1), init=("normal", 0.2)),
                    ParamSpec(f"{s.name}.o", (s.hidden_size, self.v_size))]
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
        # (per-channel decays: q, k, v and beta's logits)
        ws = [tensors.pop(f"{s.name}.{n}") for n in (("q", "k", "v", "b") if self.channel else ("q", "k", "v", "g", "b", "a"))]
        self.w_in = torch.cat(ws, dim=0).contiguous()
        del ws
        self.w_conv = torch.cat([tensors.pop(f"{s.name}.{n}.conv") for n in ("q", "k", "v")], dim=0).contiguous()
        self.a_log, self.dt_bias = tensors[f"{s.name}.A_log"], tensors[f"{s.name}.dt_bias"]
        self.w_o, self.w_norm = tensors[f"{s.name}.o"], tensors[f"{s.name}.norm"]
        self.w_low = self.w_a2 = self.w_g2 = None
        if self.channel:
            a1, a2 = tensors.pop(f"{s.name}.a1"), tensors.pop(f"{s.name}.a2")
            g1, g2 = tensors.pop(f"{s.name}.g1"), tensors.pop(f"{s.name}.g2")
            if a1.shape[0] != a2.shape[1] or g1.shape[0] != g2.shape[1]:
                raise BadFormat(f"{s.name}: a1/a2 or g1/g2 do not share their rank")
            ra, rg = a1.shape[0], g1.shape[0]
            # one product makes both low-rank inputs; each second matrix gets zero columns for the other's lanes (and
            # up to a multiple of 8 lanes, which the tensor-core products want)
            pad = (-(ra + rg)) % 8
            self.low_size = ra + rg + pad
            self.w_low = torch.cat([a1, g1, a1.new_zeros(pad, a1.shape[1])], dim=0).contiguous()
            self.w_a2 = torch.cat([a2, a2.new_zeros(a2.shape[0], rg + pad)], dim=1).contiguous()
            self.w_g2 = torch.cat([g2.new_zeros(g2.shape[0], ra), g2, g2.new_zeros(g2.shape[0], pad)], dim=1).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_conv, self.w_o, self.w_low, self.w_a2, self.w_g2)
                   if t is not None)

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
        if self.channel:
            low = rt.empty(n, self.low_size)
            z = rt.empty(n, H * d, dtype=torch.float32)              # the decays' logits, then the decays
            gate = rt.empty(n, self.v_size, dtype=torch.float32)
            with rt.phase("delta_low", self.w_low, n):
                rt.linear(x, self.w_low, None, low)
                rt.linear(low, self.w_a2, self.dt_bias, z)
                rt.linear(low, self.w_g2, None, gate)
            with rt.phase("delta_conv", nbytes=4.0 * (proj.numel() + xc.numel() + 2 * z.numel())):
                ops.delta_prepare(proj, self.w_conv, cache.state, self.state_floats, ctx.tok_seq, ctx.seq_slots,
                                  ctx.cu_seqlens, self.a_log, None, xc, gb, ctx.n_seqs, H, G, d, e, s.conv,
                                  one_token_each=ctx.is_decode, beta_col=self.channels, chan_z=z)
            with rt.phase("delta_scan", nbytes=state_bytes + 4.0 * (xc.numel() + o.numel() + z.numel()),
                          flops=8.0 * n * H * d * e):
                ops.delta_scan(xc, gb, cache.state, ctx.seq_slots, ctx.cu_seqlens, o, ctx.n_seqs, H, G, d, e, chan_g=z)
            with rt.phase("delta_gate"):
                ops.gla_output(o, gate, self.w_norm, s.eps, gated, H, d, e, gate_col=0, gate="sigmoid",
                               out_scale=float(getattr(ctx, "out_scale", 1.0)))
            with rt.phase("delta_out", self.w_o, n):
                rt.linear(gated, self.w_o, None, residual, accumulate=not getattr(ctx, "branch_is_fresh", False),
                          then_norm=getattr(ctx, "next_norm", None))
            return
        with rt.phase("delta_conv", nbytes=4.0 * (proj.numel() + xc.numel())):
            ops.delta_prepare(proj, self.w_conv, cache.state, self.state_floats, ctx.tok_seq, ctx.seq_slots, ctx.cu_seqlens,
                              self.a_log, self.dt_bias, xc, gb, ctx.n_seqs, H, G, d, e, s.conv,
                              one_token_each=ctx.is_decode)
        with rt.phase("delta_scan", nbytes=state_bytes + 4.0 * (xc.numel() + o.numel()), flops=6.0 * n * H * d * e):
            ops.delta_scan(xc, gb, cache.state, ctx.seq_slots, ctx.cu_seqlens, o, ctx.n_seqs, H, G, d, e)
        with rt.phase("delta_gate"):
            ops.gla_output(o, proj, self.w_norm, s.eps, gated, H, d, e, gate_col=self.gate_col,
                           out_scale=float(getattr(ctx, "out_scale", 1.0)))
        with rt.phase("delta_out", self.w_o, n):
            rt.linear(gated, self.w_o, None, residual, accumulate=not getattr(ctx, "branch_is_fresh", False),
                      then_norm=getattr(ctx, "next_norm", None))
