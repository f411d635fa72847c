"""Grouped-query attention over the paged cache: projections (with optional
biases, added before the per-head norms), optional per-head q/k norm, optional
position encoding, append of k and v to the entry's pages, causal attention
over all earlier keys or a window of them, output projection added to the
residual stream (crates/nncpu/src/model/forward.rs:197-439).

q, k and v projections are stored as one matrix so the input is read once.
An entry that reads another entry's cache has no k/v projection at all
(crates/nncpu/src/model/forward.rs:210,240-255).

Options a spec may switch on: value heads of another size than the query/key heads (``v_head_dim``), a
distance bias per head (``slope_base`` b: head h of H takes 2^(-b (h + 1) / H) * (i - j) off the scaled score
of query i and key j), and a query temperature (the query at position p times
1 + coef * ln(floor((p + 1) / every) + 1)).  Scores, bias and softmax are 32-bit.  Which earlier keys a query sees is
``window`` (the last n up to itself) or ``chunk`` (those of its own block of n positions, blocks counted from position
0 of the sequence) or neither (all); the kernels know it as one number, ``ops.key_span``.

Further options: ``values_are_keys`` (no value projection: a position's value is its key as projected, before norm and
rotation), ``sink`` (a learned logit per head whose exponential joins the softmax's denominator), ``out_gate`` (the
concatenated heads times sigmoid(W_g h), lane by lane, before the output projection; W_g's rows ride in the q/k/v
product) and ``out_bias``.
"""
from __future__ import annotations

import torch

from .. import perf
from ..cache import KVRequest
from ..errors import UnsupportedModel
from ..kernels import ops
from ..weights.params import ParamSpec
from . import base
from .base import Mixer, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    accepts_deferred_norm = True    # x goes to Runtime.linear, which finishes a norm's unfinished output

    def __init__(self, spec, reads_other_cache: bool = False):
        s = self.spec = spec
        self.shared_kv = reads_other_cache
        if s.n_heads % s.n_kv_heads:
            raise UnsupportedModel(f"{s.name}: {s.n_heads} heads over {s.n_kv_heads} key/value heads")
        if s.qk_norm is not None and s.qk_norm.kind != "rmsnorm":
            raise UnsupportedModel(f"{s.name}: per-head norm of kind {s.qk_norm.kind!r} is not supported")
        if s.tensor_names not in ("proj", "short"):
            raise UnsupportedModel(f"{s.name}: tensor names of style {s.tensor_names!r}")
        self.v_dim = s.v_head_dim or s.head_dim
        if s.values_are_keys and self.v_dim != s.head_dim:
            raise UnsupportedModel(f"{s.name}: values that are the keys have {s.head_dim} lanes, not {self.v_dim}")
        self.q_size = s.n_heads * s.head_dim
        self.kv_size = 0 if reads_other_cache else s.n_kv_heads * s.head_dim
        self.v_size = 0 if (reads_other_cache or s.values_are_keys) else s.n_kv_heads * self.v_dim
        self.out_size = s.n_heads * self.v_dim
        self.gate_size = self.out_size if s.out_gate else 0
        self.gate_col = self.q_size + self.kv_size + self.v_size      # the gate's logits follow the heads in a row
        # Value heads of their own size are known to the 32-bit kernel alone.  A distance bias or a query temperature
        # keeps a prompt step off the fused q/k/v epilogue of the projection (which knows neither): the temperature is
        # applied where q is made (in a decode step: inside the attention kernel that starts from the projections),
        # the bias inside the attention kernels (tcgen05 for prompts, mma.sync for decode steps and short portions).
        # Values that are the keys and an output gate keep a prompt step off that epilogue too (it appends a value of
        # its own and knows no rows of gate logits); a decode step has them inside the attention kernel that starts
        # from the projections.  A sink is a matter of the attention kernels alone, and all of them take it; the one
        # design that has sinks has the other two as well, so a sink keeps to their path.
        self.plain_core = self.v_dim != s.head_dim
        self.unfused = (self.plain_core or s.slope_base != 0.0 or s.q_temp_coef != 0.0 or s.values_are_keys or s.sink
                        or s.out_gate)
        self.q_temp = (s.q_temp_coef, s.q_temp_every) if s.q_temp_coef != 0.0 else None
        self.position = None if s.position is None else base.build("position", s.position)
        self.span = ops.key_span(s.window, s.chunk)     # what the kernels take as their ``window``

    def kv_request(self):
        s = self.spec
        return None if self.shared_kv else KVRequest(s.n_kv_heads, s.head_dim, s.window,
                                                     0 if self.v_dim == s.head_dim else self.v_dim, chunk=s.chunk)

    def _proj_names(self):
        if self.shared_kv:
            return ["q_proj"]
        return ["q_proj", "k_proj"] if self.spec.values_are_keys else ["q_proj", "k_proj", "v_proj"]

    def _tensor(self, proj: str, bias: bool = False) -> str:
        """The file's name of a projection's matrix or bias."""
        s = self.spec
        if s.tensor_names == "short":
            return f"{s.name}.{proj[0]}" + (".b" if bias else "")
        return f"{s.name}.{proj}." + ("bias" if bias else "weight")

    def _norm_tensor(self, which: str) -> str:
        s = self.spec
        if s.tensor_names == "short":
            return f"{s.qk_norm.name}.{which}.norm"
        return f"{s.qk_norm.name}.{which}_norm.weight"

    def params(self):
        s, p = self.spec, []
        sizes = {"q_proj": self.q_size, "k_proj": self.kv_size, "v_proj": self.v_size}
        for n in self._proj_names():
            p.append(ParamSpec(self._tensor(n), (sizes[n], s.hidden_size)))
            if s.qkv_bias:
                p.append(ParamSpec(self._tensor(n, bias=True), (sizes[n],)))
        p.append(ParamSpec(self._tensor("o_proj"), (s.hidden_size, self.out_size)))
        if s.out_bias or s.out_bias_optional:
            p.append(ParamSpec(self._tensor("o_proj", bias=True), (s.hidden_size,), required=s.out_bias))
        if s.qk_norm is not None:
            p.append(ParamSpec(self._norm_tensor("q"), (s.head_dim,), init=("one_plus_normal", 0.1)))
            if not self.shared_kv:
                p.append(ParamSpec(self._norm_tensor("k"), (s.head_dim,), init=("one_plus_normal", 0.1)))
        if s.sink:
            p.append(ParamSpec(f"{s.name}.sink", (s.n_heads,), init=("normal", 1.0)))
        if s.out_gate:
            p.append(ParamSpec(f"{s.name}.g", (self.gate_size, s.hidden_size)))
        return p

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        names = self._proj_names()
        ws = [tensors.pop(self._tensor(n)) for n in names]
        if s.out_gate:
            ws.append(tensors.pop(f"{s.name}.g"))       # the gate's logits come out of the same product
        self.w_qkv = ws[0] if len(ws) == 1 else torch.cat(ws, dim=0).contiguous()
        del ws
        self.b_qkv = None
        if s.qkv_bias:
            bs = [tensors.pop(self._tensor(n, bias=True)) for n in names]
            if s.out_gate:
                bs.append(torch.zeros(self.gate_size, dtype=bs[0].dtype, device=bs[0].device))   # the gate has no bias
            self.b_qkv = bs[0] if len(bs) == 1 else torch.cat(bs, dim=0).contiguous()
        # the sink logits enter 32-bit softmax arithmetic
        self.sinks = tensors[f"{s.name}.sink"].to(torch.float32).contiguous() if s.sink else None
        self.w_o = tensors[self._tensor("o_proj")]
        self.b_o = tensors.get(self._tensor("o_proj", bias=True))
        self.q_gamma = self.k_gamma = None
        if s.qk_norm is not None:
            self.q_gamma = tensors[self._norm_tensor("q")]
            self.k_gamma = tensors.get(self._norm_tensor("k"))
        if self.position is not None:
            self.position.bind(tensors, rt)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_qkv, self.w_o))

    def forward(self, ctx, x, residual, cache):
        s, rt = self.spec, self.rt
        n = x.shape[0]
        eps = s.qk_norm.eps if s.qk_norm else 0.0
        attn = rt.empty(n, self.out_size)
        if self._fused_qkv(x, cache):
            # a prompt: norm, rotation and the cache append happen in the projection's epilogue, on its
            # float32 accumulators; its threads are tokens, so the rotation table is laid out by pair
            q = rt.empty(n, self.q_size)
            with rt.phase("attn_rope"):
                cos_sin = None if self.position is None else self.position.tables(ctx, by_pair=True)
            norm_in = None
            if isinstance(x, base.DeferredNorm):      # the norm before rides on this product
                x, norm_in = x.x_gamma, (x.bins, x.request.eps)
            with rt.phase("attn_qkv", self.w_qkv, n):
                ops.linear_tc_qkv(x, self.w_qkv, self.q_gamma, self.k_gamma, eps, cos_sin, ctx.tok_seq, ctx.tok_pos,
                                  cache.block_table, cache.k_pages, cache.v_pages, q, rt.workspace, s.n_heads,
                                  s.n_kv_heads, s.head_dim, norm_in=norm_in)
            with self._core_phase(ctx, cache):
                self._attend(ctx, q, cache, attn)
        else:
            # the projections stay in float32 until the per-head norm and the rotation have been applied
            qkv = rt.empty(n, self.q_size + self.kv_size + self.v_size + self.gate_size, dtype=torch.float32)
            with rt.phase("attn_qkv", self.w_qkv, n):
                rt.linear(x, self.w_qkv, self.b_qkv, qkv)
            with rt.phase("attn_rope"):
                cos_sin = None if self.position is None else self.position.tables(ctx)
            if self._decode_from_projections(ctx, cache):
                # a decode step: norm, rotation and append are the attention kernel's own first steps, the sink's term
                # and the output gate its last
                with self._core_phase(ctx, cache):
                    n_splits, scratch = self._decode_splits(ctx)
                    ops.attention_decode_mma_from_qkv(qkv, self.q_gamma, self.k_gamma, eps, cos_sin, cache.k_pages,
                                                      cache.v_pages, not self.shared_kv, cache.block_table, ctx.tok_seq,
                                                      ctx.tok_pos, attn, scratch, s.n_heads, s.n_kv_heads, s.head_dim,
                                                      s.scale, self.span, n_splits, s.slope_base, self.q_temp,
                                                      sinks=self.sinks, values_are_keys=s.values_are_keys,
                                                      gated=s.out_gate)
            else:
                q = rt.empty(n, self.q_size)
                with rt.phase("attn_rope"):
                    ops.qk_norm_rope_append(qkv, self.q_gamma, self.k_gamma, eps, cos_sin, ctx.tok_seq, ctx.tok_pos,
                                            cache.block_table, cache.k_pages, cache.v_pages, q, s.n_heads,
                                            0 if self.shared_kv else s.n_kv_heads, s.head_dim, self.v_dim, self.q_temp,
                                            values_are_keys=s.values_are_keys)
                with self._core_phase(ctx, cache):
                    self._attend(ctx, q, cache, attn)
                if s.out_gate:      # (the decode kernel that starts from the projections applies the gate itself)
                    with rt.phase("attn_gate"):
                        ops.sigmoid_gate(attn, qkv, self.gate_col)
        with rt.phase("attn_out", self.w_o, n):
            # the last write into the residual stream: it may leave the next norm its input
            rt.linear(attn, self.w_o, self.b_o, residual, accumulate=not getattr(ctx, "branch_is_fresh", False),
                      then_norm=getattr(ctx, "next_norm", None))

    def _core_phase(self, ctx, cache):
        """The profiler's scope of the attention itself: every token streams the keys and values of its span
        (crates/nncpu/src/model/forward.rs:382-386)."""
        if not perf.enabled():
            return perf._NULL
        s = self.spec
        keys = ctx.span_sum(s.window, s.chunk)
        return self.rt.phase("attn_core", nbytes=1.0 * keys * s.n_kv_heads * (s.head_dim + self.v_dim) * cache.k_pages.element_size(),
                             flops=2.0 * keys * (self.q_size + self.out_size))

    def _decode_from_projections(self, ctx, cache) -> bool:
        """Whether this step's attention can start from the float32 projections: a decode step on the tensor-core
        kernel, every lane of a head rotated (or none), norm weights of one type."""
        s = self.spec
        return (not self.plain_core and ctx.is_decode and self.rt.dtype == torch.bfloat16 and cache.k_pages.dtype == torch.bfloat16
                and ops.attention_mma_supported(s.n_heads, s.n_kv_heads, s.head_dim)
                and s.n_heads // s.n_kv_heads <= 16
                and (self.position is None or self.position.half * 2 == s.head_dim)
                and (self.q_gamma is None or self.k_gamma is None or self.q_gamma.dtype == self.k_gamma.dtype))

    def _decode_splits(self, ctx):
        """Splits of every token's keys in a decode step, and the scratch their merge needs (None: they merge
        inside a thread-block cluster)."""
        s = self.spec
        limit = s.window or s.chunk
        longest = min(ctx.max_kv_len, limit) if limit > 0 else ctx.max_kv_len
        n_splits = ops.attention_decode_splits(ctx.n_tokens, s.n_kv_heads, longest, self.rt.sm_count)
        floats = 0 if n_splits <= ops.DECODE_CLUSTER_MAX_SPLITS else ops.attention_decode_scratch_floats(
            ctx.n_tokens, s.n_heads, s.n_kv_heads, s.head_dim, n_splits)
        return n_splits, (self.rt.empty(floats, dtype=torch.float32) if floats else None)

    def _fused_qkv(self, x, cache) -> bool:
        s = self.spec
        if isinstance(x, base.DeferredNorm):
            x = x.x_gamma
        return (not self.unfused and not self.shared_kv and self.b_qkv is None and x.dtype == torch.bfloat16
                and self.w_qkv.dtype == torch.bfloat16 and cache.k_pages.dtype == torch.bfloat16
                and (self.position is None or (self.position.tables_by_pair and self.position.half * 2 == s.head_dim))
                and ops.linear_tc_qkv_supported(x, s.n_heads, s.n_kv_heads, s.head_dim))

    def _attend(self, ctx, q, cache, attn):
        """bfloat16 with a head size the tensor-core kernels take: split-key
        decode, tcgen05 prefill for prompts, mma.sync prefill for a few tokens
        per sequence; everything else: the 32-bit kernel."""
        s = self.spec
        if (self.plain_core
                or not ops.attention_mma_supported(s.n_heads, s.n_kv_heads, s.head_dim, q, cache.k_pages, attn)):
            ops.attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.tok_seq, ctx.tok_pos, attn,
                          s.n_heads, s.n_kv_heads, s.head_dim, s.scale, self.span, self.v_dim, s.slope_base, self.sinks)
        elif ctx.is_decode:
            n_splits, scratch = self._decode_splits(ctx)
            ops.attention_decode_mma(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.tok_seq, ctx.tok_pos,
                                     attn, scratch, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, self.span, n_splits,
                                     s.slope_base, self.sinks)
        elif ctx.n_tokens >= 32 * ctx.n_seqs and ops.attention_prefill_tc_supported(
                s.n_heads, s.n_kv_heads, s.head_dim, q, cache.k_pages, attn):
            # prompts: 128-row tiles on the tcgen05 tensor cores
            ops.attention_prefill_tc(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.cu_seqlens, ctx.tok_pos,
                                     attn, self.rt.workspace.status, ctx.n_seqs, s.n_heads, s.n_kv_heads, s.head_dim,
                                     s.scale, self.span, s.slope_base, self.sinks)
        else:
            # a few new tokens per sequence: 64-row tiles
            ops.attention_prefill_mma(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.cu_seqlens, ctx.tok_pos,
                                      attn, ctx.n_seqs, s.n_heads, s.n_kv_heads, s.head_dim, s.scale, self.span,
                                      s.slope_base, self.sinks)
