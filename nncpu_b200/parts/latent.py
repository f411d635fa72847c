"""Latent attention: the keys and values of all heads are products of ONE vector per position, and that vector
is all the cache keeps.

With h the mixer's input, H heads of d query/key lanes and e value lanes, and a latent of r lanes:

    q = W_q h                                  [H, d]
    c = rmsnorm(W_dkv h) * w_norm              [r]          (kept per position)
    k_a = W_uk[a] c,  v_a = W_uv[a] c          per head a
    s_a(i, j) = (q_a(i) . k_a(j)) * scale,  j <= i;  softmax over j;  o_a = sum_j p_a(i, j) v_a(j)
    out = W_o concat_a(sigmoid(g_a) o_a),  g = W_g h         (the gate only with ``head_gate``)

The products with W_uk and W_uv are moved to the query side, so that no key or value of a head is ever made:
q'_a = W_uk[a]^T q_a (r lanes) gives q_a . k_a(j) = q'_a . c(j), and sum_j p(j) v_a(j) = W_uv[a] (sum_j p(j) c(j)).
What runs over the cache is therefore attention of H query heads on one key/value head of r lanes whose values
are its keys: the paged attention kernels of the ordinary attention part, on a cache group that has key pages only.
The projections of h are one product; q, the latent and the gate logits stay float32 until the norm, q' and the
sigmoid have been computed in 32-bit.

Options of the spec.  ``rot_dim`` R > 0: a head's query has R more lanes after its d unrotated ones, W_dkv has R more
rows (not normed), and those R lanes, rotated by the position part (neighbouring lanes in pairs), are one key part
that all heads share: s_a(i, j) = (q_a . k_a(j) + qr_a(i) . kr(j)) * scale.  The kept row is then [c, kr] (r + R
lanes), the query in latent space [q'_a, qr_a], and the values are the row's first r lanes: the product with W_uv
leaves the row's other lanes out.  ``q_rank``: queries go through a latent of their own, q = W_uq rmsnorm(W_dq h).
``sink``: a learned logit per head in the softmax's denominator.  A layer that reads another layer's cache has no
W_dkv and appends nothing.
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

MAX_LATENT = 1024       # the 32-bit attention kernel keeps a head's output lanes in registers, eight a thread;
                        # a kept row (the latent and the shared rotated key part) may be this long


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    accepts_deferred_norm = True    # x goes to Runtime.linear, which finishes a norm's unfinished output

    def __init__(self, spec, reads_other_cache: bool = False):
        s = self.spec = spec
        self.shared_kv = reads_other_cache
        self.row = s.latent_dim + s.rot_dim             # lanes of a kept row, and of a head's query in latent space
        if self.row > MAX_LATENT:
            raise UnsupportedModel(f"{spec.name}: a kept row of {self.row} lanes (at most {MAX_LATENT})")
        if s.rot_dim and s.position is None:
            raise UnsupportedModel(f"{spec.name}: {s.rot_dim} rotated lanes and no rotation")
        self.q_size = s.n_heads * (s.head_dim + s.rot_dim)
        self.q_part = s.q_rank or self.q_size           # what the input product makes of the queries
        # the queries leave the input product as a matrix of their own unless they sit at the front of its rows, ready
        # for the per-head product (no rotated lanes, no latent of their own)
        self.q_apart = s.rot_dim > 0 and not s.q_rank
        self.kv_part = 0 if reads_other_cache else self.row
        self.gate_size = s.n_heads if s.head_gate else 0
        self.lat_col = 0 if self.q_apart else self.q_part
        self.gate_col = self.lat_col + self.kv_part
        self.proj_size = self.gate_col + self.gate_size
        self.out_size = s.n_heads * s.v_head_dim
        self.position = None if s.position is None else base.build("position", s.position)

    def kv_request(self):
        return None if self.shared_kv else KVRequest(1, self.row, keys_only=True)

    def params(self):
        s = self.spec
        p = []
        if s.q_rank:
            p += [ParamSpec(f"{s.name}.dq", (s.q_rank, s.hidden_size)),
                  ParamSpec(f"{s.name}.dq.norm", (s.q_rank,), init=("one_plus_normal", 0.1)),
                  ParamSpec(f"{s.name}.uq", (self.q_size, s.q_rank), init=("normal", 0.05))]
        else:
            p.append(ParamSpec(f"{s.name}.q", (self.q_size, s.hidden_size)))
        if not self.shared_kv:
            p += [ParamSpec(f"{s.name}.dkv", (self.row, s.hidden_size)),
                  ParamSpec(f"{s.name}.dkv.norm", (s.latent_dim,), init=("one_plus_normal", 0.1))]
        p += [ParamSpec(f"{s.name}.uk", (s.n_heads * s.head_dim, s.latent_dim), init=("normal", 0.05)),
              ParamSpec(f"{s.name}.uv", (self.out_size, s.latent_dim), init=("normal", 0.05))]
        if s.head_gate:
            p.append(ParamSpec(f"{s.name}.g", (s.n_heads, s.hidden_size), init=("normal", 0.05)))
        if s.sink:
            p.append(ParamSpec(f"{s.name}.sink", (s.n_heads,), init=("normal", 1.0)))
        p.append(ParamSpec(f"{s.name}.o", (s.hidden_size, self.out_size)))
        return p

    def bind(self, tensors, rt):
        s, self.rt = self.spec, rt
        H, r = s.n_heads, s.latent_dim
        w_q = tensors.pop(f"{s.name}.dq" if s.q_rank else f"{s.name}.q")
        self.w_q = w_q if self.q_apart else None
        ws = [] if self.q_apart else [w_q]
        if not self.shared_kv:
            ws.append(tensors.pop(f"{s.name}.dkv"))
        if s.head_gate:
            ws.append(tensors.pop(f"{s.name}.g"))
        # rows: the queries (or their latent), the latent and the shared key part, the gate logits
        self.w_in = None if not ws else (ws[0] if len(ws) == 1 else torch.cat(ws, dim=0).contiguous())
        del ws, w_q
        self.w_qnorm = tensors[f"{s.name}.dq.norm"] if s.q_rank else None
        self.w_uq = tensors[f"{s.name}.uq"] if s.q_rank else None
        self.w_norm = None if self.shared_kv else tensors[f"{s.name}.dkv.norm"]
        # head a's W_uk[a] is [d, r]; q' = W_uk[a]^T q needs it as [r, d] (out, in)
        self.w_uk_t = tensors.pop(f"{s.name}.uk").view(H, s.head_dim, r).transpose(1, 2).contiguous()
        w_uv = tensors[f"{s.name}.uv"].view(H, s.v_head_dim, r)
        # The values are the kept row's first r lanes.  Where only the row's whole width suits the tensor cores, W_uv
        # gets columns of zeros for the row's other lanes; else the product reads r lanes of every head and steps on.
        self.uv_padded = s.rot_dim > 0 and r % 64 != 0 and self.row % 64 == 0
        if self.uv_padded:
            w_uv = torch.cat([w_uv, torch.zeros(H, s.v_head_dim, s.rot_dim, dtype=w_uv.dtype, device=w_uv.device)],
                             dim=2).contiguous()
        self.w_uv = w_uv
        self.w_o = tensors[f"{s.name}.o"]
        self.sinks = tensors[f"{s.name}.sink"].to(torch.float32).contiguous() if s.sink else None
        if self.position is not None:
            self.position.bind(tensors, rt)

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_q, self.w_uq, self.w_uk_t, self.w_uv, self.w_o)
                   if t is not None)

    def forward(self, ctx, x, residual, cache):
        s, rt = self.spec, self.rt
        n, H, r, R, d, W = x.shape[0], s.n_heads, s.latent_dim, s.rot_dim, s.head_dim, self.row
        if isinstance(x, base.DeferredNorm) and self.q_apart:
            x = x.finish(ctx)           # two products read it
        proj = None
        if self.w_in is not None:
            proj = rt.empty(n, self.proj_size, dtype=torch.float32)
            with rt.phase("attn_qkv", self.w_in, n):
                rt.linear(x, self.w_in, None, proj)
        fast = self._tensor_core_attention(cache)
        lat_dt = torch.bfloat16 if fast else torch.float32
        q_lat, o_lat, heads = rt.empty(n, H * W, dtype=lat_dt), rt.empty(n, H * W, dtype=lat_dt), rt.empty(n, self.out_size)
        # the two per-head products run on the tensor cores where the sizes allow it (the queries are rounded to
        # bfloat16 for that, where a kernel passes over the row anyway), else in 32-bit on the CUDA cores
        q16 = rt.empty(n, self.q_size, dtype=torch.bfloat16)
        absorb_tc = fast and ops.linear_heads_tc_supported(q16, 0, self.w_uk_t, q_lat, d + R)
        expand_tc = fast and ops.linear_heads_tc_supported(o_lat, 0, self.w_uv, heads, W)
        with rt.phase("attn_rope"):
            cos_sin = self.position.tables(ctx) if R else None
        separate_q = bool(s.q_rank) or self.q_apart        # q is (or becomes) a matrix of its own, not the front of proj
        cq = rt.empty(n, s.q_rank) if s.q_rank else None
        if proj is not None and (not self.shared_kv or s.q_rank or (absorb_tc and not separate_q)):
            with rt.phase("attn_rope"):
                ops.latent_append(proj, self.lat_col, self.w_norm, s.eps, ctx.tok_seq, ctx.tok_pos, cache.block_table,
                                  None if self.shared_kv else cache.k_pages,
                                  q16 if (absorb_tc and not separate_q) else None, rot_dim=R, cos_sin=cos_sin,
                                  q_norm=(self.w_qnorm, 0, s.q_rank, cq) if s.q_rank else None)
        if separate_q:
            q = rt.empty(n, self.q_size, dtype=torch.float32)
            with rt.phase("attn_q", self.w_uq if s.q_rank else self.w_q, n):
                if s.q_rank:
                    rt.linear(cq, self.w_uq, None, q)
                else:
                    rt.linear(x, self.w_q, None, q)
            if R or absorb_tc:
                with rt.phase("attn_rope"):
                    ops.latent_query(q, cos_sin, q_lat, H, d, R, r, q16 if absorb_tc else None)
        else:
            q = proj
        with rt.phase("attn_absorb", self.w_uk_t, n):
            if absorb_tc:
                ops.linear_heads_tc(q16, self.w_uk_t, q_lat, rt.workspace, x_step=d + R, out_step=W)
            else:
                ops.linear_heads(q, 0, self.w_uk_t, q_lat, x_step=d + R, out_step=W)
        with self._core_phase(ctx, cache):
            self._attend(ctx, q_lat, cache, o_lat, fast)
        gate = proj if s.head_gate else None
        with rt.phase("attn_expand", self.w_uv, n):
            if expand_tc:
                ops.linear_heads_tc(o_lat, self.w_uv, heads, rt.workspace, gate=gate, gate_col=self.gate_col, x_step=W)
            else:
                ops.linear_heads(o_lat, 0, self.w_uv, heads, gate=gate, gate_col=self.gate_col, x_step=W)
        with rt.phase("attn_out", self.w_o, n):
            rt.linear(heads, self.w_o, None, residual, accumulate=not getattr(ctx, "branch_is_fresh", False),
                      then_norm=getattr(ctx, "next_norm", None))

    def _tensor_core_attention(self, cache) -> bool:
        s = self.spec
        return (self.rt.dtype == torch.bfloat16 and cache.k_pages.dtype == torch.bfloat16
                and ops.attention_mma_supported(s.n_heads, 1, self.row))

    def _core_phase(self, ctx, cache):
        if not perf.enabled():
            return perf._NULL
        s = self.spec
        keys = ctx.span_sum()
        return self.rt.phase("attn_core", nbytes=1.0 * keys * self.row * cache.k_pages.element_size(),
                             flops=4.0 * keys * s.n_heads * self.row)

    def _attend(self, ctx, q, cache, out, fast: bool):
        """H query heads on the one key/value head of the kept rows, values = keys."""
        s, rt = self.spec, self.rt
        H, r = s.n_heads, self.row
        pages = cache.k_pages
        if not fast:
            ops.attention(q, pages, pages, cache.block_table, ctx.tok_seq, ctx.tok_pos, out, H, 1, r, s.scale,
                          sinks=self.sinks)
        elif ctx.is_decode:
            n_splits = ops.attention_decode_splits(ctx.n_tokens, 1, ctx.max_kv_len, rt.sm_count)
            floats = 0 if n_splits <= ops.DECODE_CLUSTER_MAX_SPLITS else ops.attention_decode_scratch_floats(
                ctx.n_tokens, H, 1, r, n_splits)
            scratch = rt.empty(floats, dtype=torch.float32) if floats else None
            ops.attention_decode_mma(q, pages, pages, cache.block_table, ctx.tok_seq, ctx.tok_pos, out, scratch, H, 1, r,
                                     s.scale, 0, n_splits, 0.0, self.sinks)
        elif ctx.n_tokens >= 32 * ctx.n_seqs and ops.attention_prefill_tc_supported(H, 1, r, q, pages, out):
            ops.attention_prefill_tc(q, pages, pages, cache.block_table, ctx.cu_seqlens, ctx.tok_pos, out,
                                     rt.workspace.status, ctx.n_seqs, H, 1, r, s.scale, 0, 0.0, self.sinks)
        else:
            ops.attention_prefill_mma(q, pages, pages, cache.block_table, ctx.cu_seqlens, ctx.tok_pos, out, ctx.n_seqs,
                                      H, 1, r, s.scale, 0, 0.0, self.sinks)
