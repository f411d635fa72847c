"""Arrangements of parts in a layer.  "prenorm":
x += mixer(norm1(x)); x += feed_forward(norm2(x))
(crates/nncpu/src/model/forward.rs:735-803 without the Gemma post-norms).
"sandwich" norms each sublayer's output as well; "parallel" lets both sublayers read the stream as it enters
the layer: x += mixer(norm1(x)) + feed_forward(norm2(x)).
The residual stream stays in float32 from the embedding to the final norm.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.params import ParamSpec
from . import base
from .base import Block, NormRequest, register_block
from .side import TokenSide


@register_block("prenorm")
class PreNormBlock(Block):
    """x += m * mixer(norm1(x)); x += m * feed_forward(norm2(x)); then, if the layer has one, its per-layer token input
    (``parts.side``).  m = ``residual_mult``.  With m = 1 the sublayers add into the stream themselves.  With another m
    a sublayer that says ``scales_output`` is told the factor (``ctx.out_scale``) and still adds into the stream; any
    other writes into a 32-bit branch of its own (told that it is fresh, so its last product writes instead of adding)
    which one kernel adds to the stream times m.  A layer may go without a feed-forward (its second norm is then not
    used, and its tensors are not asked for)."""

    def __init__(self, spec, reads_other_cache: bool = False):
        self.norm1 = base.build("norm", spec.norm1)
        kwargs = {"reads_other_cache": True} if reads_other_cache else {}
        self.mixer = base.build("mixer", spec.mixer, **kwargs)
        self.feed_forward = None if spec.feed_forward is None else base.build("feed_forward", spec.feed_forward)
        self.norm2 = None if self.feed_forward is None else base.build("norm", spec.norm2)
        self.mult = float(spec.residual_mult)
        self.side = None if spec.side is None else TokenSide(spec.side)
        self._parts = tuple(p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward, self.side) if p is not None)
        # a layer without a feed-forward may still name its second norm: its tensors are then optional and not used
        self._spare = (base.build("norm", spec.norm2).params()
                       if (self.feed_forward is None and spec.norm2 is not None) else [])

    def params(self):
        spare = [ParamSpec(p.name, p.shape, required=False, init=p.init) for p in self._spare]
        return [p for part in self._parts for p in part.params()] + spare

    def bind(self, tensors, rt):
        self.rt = rt
        for part in self._parts:
            part.bind(tensors, rt)

    def weight_bytes(self):
        return sum(part.weight_bytes() for part in self._parts)

    def cache_requests(self):
        return [(self.mixer.kv_request(), self.mixer.state_request())]

    def entry_norm_request(self, ctx, residual):
        req = self.norm1.request(ctx, residual)
        if req is not None and req.wants_output:     # a finished output: whatever the mixer is, it can read it
            return req
        return req if self.mixer.accepts_deferred_norm else None

    @staticmethod
    def _finished(norm, ctx, residual, request):
        """``norm``'s output: what the part that wrote the stream last left, if it fulfilled this very norm's request for
        a finished output; else the norm's own kernel."""
        if request is not None and request.norm is norm and request.output is not None:
            return request.output
        return norm.forward(ctx, residual)

    @staticmethod
    def _normed(norm, consumer, ctx, residual, request):
        """``norm``'s output for ``consumer``: what the writer of the residual left, if it fulfilled the request
        of this very norm and the consumer takes it unfinished; else the norm's own kernel."""
        if request is not None and request.norm is norm and request.output is not None:
            return request.output           # finished, by a kernel that closed the sublayer before
        if (request is not None and request.norm is norm and request.result is not None
                and consumer.accepts_deferred_norm):
            return request.result
        return norm.forward(ctx, residual)

    def _scaled(self, ctx, part, residual, run):
        """x += m * part(...) for m != 1: ``run(out)`` makes the part add into (or, for a fresh branch, write) ``out``."""
        if getattr(part, "scales_output", False):
            ctx.out_scale = self.mult
            try:
                run(residual)
            finally:
                ctx.out_scale = 1.0
            return
        branch = self.rt.empty(*residual.shape, dtype=torch.float32)
        ctx.branch_is_fresh = True
        try:
            run(branch)
        finally:
            ctx.branch_is_fresh = False
        with self.rt.phase("norm", nbytes=12.0 * residual.numel()):
            ops.stream_axpy(residual, branch, self.mult)

    def forward(self, ctx, residual, caches):
        # At a few tokens the norms ride on the products around them: the block before may have left norm1's
        # input (ctx.next_norm), the mixer's last product is asked for norm2's, and the feed-forward's last
        # product for the first norm of the block that follows (ctx.after_block).
        handed, after = ctx.next_norm, ctx.after_block
        ctx.next_norm = ctx.after_block = None
        ff = self.feed_forward
        if self.mult != 1.0 or self.side is not None:
            # the sublayers' products are not the last writes into the stream: no norm rides on them
            # (a mixer that closes with a kernel of its own, and the side part, can leave the norm that follows them)
            asked = None
            with self.rt.scope():
                x = self._finished(self.norm1, ctx, residual, handed)
                if ff is not None and getattr(self.mixer, "closes_stream", False):
                    asked = self.norm2.request(ctx, residual)
                    if asked is not None and not asked.wants_output:
                        asked = None
                ctx.next_norm = asked
                if self.mult != 1.0:
                    self._scaled(ctx, self.mixer, residual, lambda out: self.mixer.forward(ctx, x, out, caches[0]))
                else:
                    self.mixer.forward(ctx, x, residual, caches[0])
                ctx.next_norm = None
            if ff is not None:
                with self.rt.scope():
                    x = self._finished(self.norm2, ctx, residual, asked)
                    if self.mult != 1.0:
                        self._scaled(ctx, ff, residual, lambda out: ff.forward(ctx, x, out))
                    else:
                        ff.forward(ctx, x, residual)
            if self.side is not None:
                self.side.forward(ctx, residual, self.mult, then=after)
            ctx.next_norm = after       # the block that follows finds its request there, fulfilled or not
            return
        with self.rt.scope():       # the mixer's temporaries are done with when the feed-forward starts
            x = self._normed(self.norm1, self.mixer, ctx, residual, handed)
            asked = self.norm2.request(ctx, residual) if (ff is not None and ff.accepts_deferred_norm) else None
            ctx.next_norm = asked if ff is not None else after
            self.mixer.forward(ctx, x, residual, caches[0])
            if ff is not None:
                ctx.next_norm = None
        if ff is not None:
            with self.rt.scope():
                x = self._normed(self.norm2, ff, ctx, residual, asked)
                ctx.next_norm = after
                ff.forward(ctx, x, residual)
        # ctx.next_norm stays: the block that follows finds its request there, fulfilled or not


@register_block("sandwich")
class SandwichBlock(Block):
    """A norm before and after each sublayer: x += norm1_post(mixer(norm1(x))), then, if the layer has a
    feed-forward, x += norm2_post(feed_forward(norm2(x))).  A sublayer writes its output into a float32 branch
    of its own, and the closing norm adds its result into the residual stream; the norm that opens whatever follows
    (the block's own feed-forward, or the next block when it is of this kind too) runs in the same pass."""

    def __init__(self, spec, reads_other_cache: bool = False):
        kwargs = {"reads_other_cache": True} if reads_other_cache else {}
        self.norm1 = base.build("norm", spec.norm1)
        self.mixer = base.build("mixer", spec.mixer, **kwargs)
        self.norm1_post = base.build("norm", spec.norm1_post)
        self.feed_forward = None if spec.feed_forward is None else base.build("feed_forward", spec.feed_forward)
        self.norm2 = self.norm2_post = None
        if self.feed_forward is not None:
            self.norm2 = base.build("norm", spec.norm2)
            self.norm2_post = base.build("norm", spec.norm2_post)
        self._parts = tuple(p for p in (self.norm1, self.mixer, self.norm1_post, self.norm2, self.feed_forward,
                                        self.norm2_post) if p is not None)

    def params(self):
        return [p for part in self._parts for p in part.params()]

    def bind(self, tensors, rt):
        self.rt = rt
        for part in self._parts:
            part.bind(tensors, rt)

    def weight_bytes(self):
        return sum(part.weight_bytes() for part in self._parts)

    def cache_requests(self):
        return [(self.mixer.kv_request(), self.mixer.state_request())]

    def entry_norm_request(self, ctx, residual):
        n = self.norm1
        return NormRequest(n, residual, n.gamma, n.eps, n.size, wants_output=True)

    def _close(self, ctx, norm_post, branch, residual, then, out):
        """residual += norm_post(branch); and, in the same pass where the sizes allow it, ``out`` = then(residual), the
        norm that opens what follows.  Returns whether ``out`` was written."""
        if (then is not None and out is not None and hasattr(then, "offset") and then.size == norm_post.size
                and then.gamma.dtype == norm_post.gamma.dtype and ops.rmsnorm_pair_supported(then.size)
                and residual.dtype == torch.float32):
            with self.rt.phase("norm"):
                ops.rmsnorm_pair(branch, residual, norm_post.gamma, norm_post.offset, norm_post.eps, then.gamma,
                                 then.offset, then.eps, out)
            return True
        norm_post.add_into(ctx, branch, residual)
        return False

    def _branch(self, ctx, residual, run, x):
        """A sublayer's output in a branch of its own.  The parts add into what they are given; told that the branch
        is fresh, their last product writes instead, which saves clearing it."""
        branch = self.rt.empty(*residual.shape, dtype=residual.dtype)
        ctx.branch_is_fresh = True
        try:
            run(x, branch)
        finally:
            ctx.branch_is_fresh = False
        return branch

    def _next_input(self, ctx, residual):
        """Where the first norm of the block that follows is left: two buffers of the step take turns."""
        turn = ctx.memo.get("sandwich_turn", 0)
        ctx.memo["sandwich_turn"] = 1 - turn
        key = ("sandwich_x", turn)
        buf = ctx.memo.get(key)
        if buf is None:
            buf = ctx.memo[key] = self.rt.empty(*residual.shape, keep=True)
        return buf

    def forward(self, ctx, residual, caches):
        rt = self.rt
        handed, after = ctx.next_norm, ctx.after_block
        ctx.next_norm = ctx.after_block = None      # these norms do not ride on the products around them
        wanted = after if (after is not None and after.wants_output) else None
        nxt = self._next_input(ctx, residual) if wanted is not None else None
        ff = self.feed_forward
        with rt.scope():
            x2 = rt.empty(*residual.shape) if ff is not None else None      # outlives the mixer's temporaries
            with rt.scope():
                if handed is not None and handed.norm is self.norm1 and handed.output is not None:
                    x = handed.output               # the block before left it with its closing norm
                else:
                    x = self.norm1.forward(ctx, residual)
                branch = self._branch(ctx, residual, lambda x, out: self.mixer.forward(ctx, x, out, caches[0]), x)
                if ff is not None:
                    if not self._close(ctx, self.norm1_post, branch, residual, self.norm2, x2):
                        x2 = None
                elif wanted is not None and self._close(ctx, self.norm1_post, branch, residual, wanted.norm, nxt):
                    wanted.output = nxt
                else:
                    self._close(ctx, self.norm1_post, branch, residual, None, None)
            if ff is not None:
                with rt.scope():
                    x = x2 if x2 is not None else self.norm2.forward(ctx, residual)
                    branch = self._branch(ctx, residual, lambda x, out: ff.forward(ctx, x, out), x)
                    if wanted is not None and self._close(ctx, self.norm2_post, branch, residual, wanted.norm, nxt):
                        wanted.output = nxt
                    else:
                        self._close(ctx, self.norm2_post, branch, residual, None, None)
        ctx.next_norm = after       # the block that follows finds its request there, fulfilled or not


@register_block("parallel")
class ParallelBlock(Block):
    """Both sublayers read the stream as it enters the layer: x += mixer(norm1(x)) + feed_forward(norm2(x)).

    The two norms are of the same rows, so they run as one kernel that takes the sum of squares once; both outputs are
    made before the mixer adds into the stream.  A layer without a feed-forward has the mixer alone (a ``norm2``
    tensor that its file may still hold is accepted and not used).  A layer with a feed-forward and no second norm has
    ONE norm: x += mixer(h) + feed_forward(h) with h = norm1(x).  The sublayers add into the 32-bit stream one
    after the other."""

    def __init__(self, spec, reads_other_cache: bool = False):
        kwargs = {"reads_other_cache": True} if reads_other_cache else {}
        self.norm1 = base.build("norm", spec.norm1)
        self.mixer = base.build("mixer", spec.mixer, **kwargs)
        self.feed_forward = None if spec.feed_forward is None else base.build("feed_forward", spec.feed_forward)
        # with a feed-forward and no second norm, both sublayers read the one norm's output
        self.norm2 = None if (self.feed_forward is None or spec.norm2 is None) else base.build("norm", spec.norm2)
        self.one_norm = self.feed_forward is not None and spec.norm2 is None
        # a layer without a feed-forward may still name its second norm: the tensor is then optional
        self._spare = spec.norm2.name + spec.norm2.suffix if (self.feed_forward is None and spec.norm2 is not None) else None
        self._parts = tuple(p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None)

    def params(self):
        p = [q for part in self._parts for q in part.params()]
        if self._spare is not None:
            p.append(ParamSpec(self._spare, (self.norm1.size,), required=False, init=("one_plus_normal", 0.1)))
        return p

    def bind(self, tensors, rt):
        self.rt = rt
        for part in self._parts:
            part.bind(tensors, rt)

    def weight_bytes(self):
        return sum(part.weight_bytes() for part in self._parts)

    def cache_requests(self):
        return [(self.mixer.kv_request(), self.mixer.state_request())]

    def _norms(self, ctx, residual):
        n1, n2, rt = self.norm1, self.norm2, self.rt
        if n2 is None:
            x1 = n1.forward(ctx, residual)
            return x1, (x1 if self.one_norm else None)
        if (getattr(n1, "offset", 1.0) == 0.0 and getattr(n2, "offset", 1.0) == 0.0 and n1.size == n2.size
                and n1.gamma.dtype == n2.gamma.dtype and residual.dtype == torch.float32):
            x1, x2 = rt.empty(*residual.shape), rt.empty(*residual.shape)
            with rt.phase("norm"):
                ops.rmsnorm_dual(residual, n1.gamma, n1.eps, n2.gamma, n2.eps, x1, x2)
            return x1, x2
        return n1.forward(ctx, residual), n2.forward(ctx, residual)

    def forward(self, ctx, residual, caches):
        ctx.next_norm = ctx.after_block = None      # two norms read what this block leaves: they run as a kernel
        with self.rt.scope():
            x1, x2 = self._norms(ctx, residual)
            with self.rt.scope():
                self.mixer.forward(ctx, x1, residual, caches[0])
            if self.feed_forward is not None:
                with self.rt.scope():
                    self.feed_forward.forward(ctx, x2, residual)
