"""Retention, and two mixers side by side.

**Retention** is linear attention with ONE fixed decay per head and neither softmax nor denominator: a recurrent
mixer that keeps, per sequence and head, a state S of ``key_dim`` x ``value_dim`` 32-bit floats in the cache's state
area.  With h the mixer's input, per head a (d = key_dim, e = value_dim, R the rotation by the token's position):

    q = R(W_q h),   k = R(W_k h) * d^(-1/2),   v = W_v h
    S_t = decay_a * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t
    out = W_o (concat_heads(o / rms(o)) * silu(W_g h))

It is gated linear attention's recurrence with a constant in place of the per-channel decays, and runs on those
kernels (``gla_scan`` for the tokens of a prompt, ``gla_step`` for a decode step, both told the heads' decays); what
is its own is the kernel before them, which rotates q and k in place on the 32-bit projections and scales k.  The four
projections of h are one product with 32-bit results; rotation angles, the recurrence, the state and the heads' norm
are 32-bit in both run types.

**A pair of mixers** reads the same input with both and adds ``weight`` times the sum of their outputs to the stream,
each first RMS-normed over the model width with a plain weight of its own.  The two write into 32-bit branches of
their own; one kernel norms both and adds them to the stream.  What the two keep from step to step is one cache
user's: keys and values of the one, state of the other.
"""
from __future__ import annotations

import torch

from ..cache import StateRequest
from ..errors import UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from . import base
from .base import Mixer, register_mixer

MAX_KEY_DIM = 512      # a lane of the scan kernel keeps one column of a head's state in registers


@register_mixer("retention")
class Retention(Mixer):
    def __init__(self, spec, reads_other_cache: bool = False):
        if reads_other_cache:
            raise UnsupportedModel(f"{spec.name}: a recurrent mixer keeps no keys and values that another layer could read")
        if spec.key_dim > MAX_KEY_DIM:
            raise UnsupportedModel(f"{spec.name}: {spec.key_dim} key channels a head (at most {MAX_KEY_DIM})")
        if len(spec.decays) != spec.n_heads:
            raise UnsupportedModel(f"{spec.name}: {len(spec.decays)} decays for {spec.n_heads} heads")
        self.spec = spec
        self.qk_size = spec.n_heads * spec.key_dim
        self.v_size = spec.n_heads * spec.value_dim
        self.position = None if spec.position is None else base.build("position", spec.position)
        if self.position is not None and 2 * self.position.half > spec.key_dim:
            raise UnsupportedModel(f"{spec.name}: {2 * self.position.half} rotated lanes of a head's {spec.key_dim}")

    def state_request(self):
        s = self.spec
        return StateRequest((s.n_heads, s.key_dim, s.value_dim), torch.float32)

    def params(self):
        s = self.spec
        return [ParamSpec(f"{s.name}.q", (self.qk_size, s.hidden_size)),
                ParamSpec(f"{s.name}.k", (self.qk_size, s.hidden_size)),
                ParamSpec(f"{s.name}.v", (self.v_size, s.hidden_size)),
                ParamSpec(f"{s.name}.g", (self.v_size, s.hidden_size)),
                ParamSpec(f"{s.name}.o", (s.hidden_size, self.v_size))]

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        ws = [tensors.pop(f"{s.name}.{n}") for n in ("q", "k", "v", "g")]
        self.w_qkvg = torch.cat(ws, dim=0).contiguous()
        del ws
        self.w_o = tensors[f"{s.name}.o"]
        # the decays enter 32-bit arithmetic as the nearest floats of the configuration's numbers
        self.decays = torch.tensor([float(a) for a in s.decays], dtype=torch.float32, device=self.w_o.device)
        if self.position is not None:
            self.position.bind(tensors, rt)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkvg, self.w_o))

    def forward(self, ctx, x, residual, cache):
        s, rt = self.spec, self.rt
        n, H, d, e = x.shape[0], s.n_heads, s.key_dim, s.value_dim
        proj = rt.empty(n, 2 * (self.qk_size + self.v_size), dtype=torch.float32)
        with rt.phase("ret_proj", self.w_qkvg, n):
            rt.linear(x, self.w_qkvg, None, proj)
        with rt.phase("ret_rope"):
            cos_sin = None if self.position is None else self.position.tables(ctx)
        gated = rt.empty(n, self.v_size)
        state_bytes = 8.0 * ctx.n_seqs * H * d * e                   # read and written once a step
        if ctx.is_decode and e <= 1024:
            # one token per sequence: rotation, recurrence, norm and gate in one launch that streams the state once
            with rt.phase("ret_scan", nbytes=state_bytes + 4.0 * proj.numel() + gated.numel() * gated.element_size()):
                ops.gla_step(proj, None, cache.state, ctx.seq_slots, None, s.eps, gated, H, d, e, 1.0, 1.0,
                             head_decay=self.decays, cos_sin=cos_sin, k_scale=d ** -0.5)
        else:
            with rt.phase("ret_rope", nbytes=16.0 * n * self.qk_size):
                ops.retention_prepare(proj, cos_sin, H, d, d ** -0.5)
            o = rt.empty(n, self.v_size, dtype=torch.float32)
            with rt.phase("ret_scan", nbytes=state_bytes + 4.0 * (proj.numel() + o.numel()), flops=4.0 * n * H * d * e):
                ops.gla_scan(proj, None, cache.state, ctx.seq_slots, ctx.cu_seqlens, o, ctx.n_seqs, H, d, e, 1.0, 1.0,
                             head_decay=self.decays)
            with rt.phase("ret_gate"):
                ops.gla_output(o, proj, None, s.eps, gated, H, d, e)
        with rt.phase("ret_out", self.w_o, n):
            rt.linear(gated, self.w_o, None, residual, accumulate=not getattr(ctx, "branch_is_fresh", False))


@register_mixer("mixer_pair")
class MixerPair(Mixer):
    scales_output = True        # what it adds to the stream is multiplied by ctx.out_scale
    closes_stream = True        # its last kernel holds the stream's new rows: it can leave the layer norm that follows

    def __init__(self, spec, reads_other_cache: bool = False):
        self.spec = spec
        kwargs = {"reads_other_cache": True} if reads_other_cache else {}
        self.left = base.build("mixer", spec.left, **kwargs)
        self.right = base.build("mixer", spec.right, **kwargs)
        kv, st = [m.kv_request() for m in (self.left, self.right)], [m.state_request() for m in (self.left, self.right)]
        if all(r is not None for r in kv) or all(r is not None for r in st):
            raise UnsupportedModel(f"{spec.name}: the two mixers of a pair share one cache user, so at most one of them "
                                   "may keep keys and values and at most one a state")
        self._kv = kv[0] if kv[0] is not None else kv[1]
        self._state = st[0] if st[0] is not None else st[1]

    def kv_request(self):
        return self._kv

    def state_request(self):
        return self._state

    def params(self):
        s = self.spec
        return (self.left.params() + self.right.params()
                + [ParamSpec(f"{s.name}.left.out", (s.hidden_size,), init=("one_plus_normal", 0.1)),
                   ParamSpec(f"{s.name}.right.out", (s.hidden_size,), init=("one_plus_normal", 0.1))])

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        self.left.bind(tensors, rt)
        self.right.bind(tensors, rt)
        self.w_left, self.w_right = tensors[f"{s.name}.left.out"], tensors[f"{s.name}.right.out"]

    def weight_bytes(self):
        return self.left.weight_bytes() + self.right.weight_bytes()

    def forward(self, ctx, x, residual, cache):
        s, rt = self.spec, self.rt
        if getattr(ctx, "branch_is_fresh", False):
            raise UnsupportedModel(f"{s.name}: a pair of mixers adds into the stream it is given")
        scale = float(getattr(ctx, "out_scale", 1.0))
        then = getattr(ctx, "next_norm", None)
        a = rt.empty(*residual.shape, dtype=torch.float32)
        b = rt.empty(*residual.shape, dtype=torch.float32)
        ctx.next_norm = None                # neither mixer's last product is the last write into the stream
        ctx.branch_is_fresh, ctx.out_scale = True, 1.0
        try:
            with rt.scope():
                self.left.forward(ctx, x, a, cache)
            with rt.scope():
                self.right.forward(ctx, x, b, cache)
        finally:
            ctx.branch_is_fresh, ctx.out_scale = False, scale
        with rt.phase("norm", nbytes=16.0 * residual.numel()):
            if then is not None and then.wants_output and hasattr(then.norm, "closing") and then.residual is residual:
                out = base.norm_output_buffer(ctx, rt, residual.shape)
                ops.branch_norm_add(residual, a, self.w_left, b, self.w_right, s.eps, scale * s.weight,
                                    then_norm=then.norm.closing(out))
                then.output = out
            else:
                ops.branch_norm_add(residual, a, self.w_left, b, self.w_right, s.eps, scale * s.weight)
