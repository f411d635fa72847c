"""Python faces of the CUDA kernels: one function per kernel, taking torch
tensors on the GPU and launching on torch's current stream.

Nothing here computes: every function checks what only Python can see
(devices, element types, contiguity), then calls the C entry point, which
checks sizes and either launches or refuses with a message.
"""
from __future__ import annotations

import ctypes
import functools
from typing import Optional

import torch

from ..errors import ExtensionError, InvalidArgument
from . import library

_DT = {torch.float32: 0, torch.bfloat16: 1}
_vp = ctypes.c_void_p


def _code(t: Optional[torch.Tensor]) -> int:
    if t is None:
        return 0
    try:
        return _DT[t.dtype]
    except KeyError:
        raise InvalidArgument(f"kernels take float32 or bfloat16 tensors, not {t.dtype}") from None


def _ptr(t: Optional[torch.Tensor]):
    # asked several times per launch (a prompt step of a few tokens is bound by the host): the usual case first
    if t is None:
        return None             # a null pointer
    if t.is_cuda and t.is_contiguous():
        return _vp(t.data_ptr())
    if t.is_meta and _dry:
        return None             # a pass over shapes alone: nothing is launched, so nothing is pointed at
    if not t.is_cuda:
        raise ExtensionError("the kernels run on the GPU: a tensor on the CPU was passed, and there is no CPU path")
    raise InvalidArgument("kernels take contiguous tensors")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream of the current device as a raw handle (the short way when torch offers it: this is
    asked once per kernel launch)."""
    if _raw_stream is not None:
        return _vp(_raw_stream(torch._C._cuda_getDevice()))
    return _vp(torch.cuda.current_stream().cuda_stream)


_launches = 0
_dry = False


class shapes_only:
    """Inside, every function of this module checks its arguments and launches nothing: a forward pass over
    shape-only (``meta``) tensors, which the engine runs once to learn how much memory a step needs."""

    def __enter__(self):
        global _dry
        self.before, _dry = _dry, True

    def __exit__(self, *exc):
        global _dry
        _dry = self.before
        return False



def launch_count() -> int:
    """Kernels of this library launched so far in this process, graph replays included."""
    return _launches


def add_launches(n: int) -> None:
    """A CUDA graph that holds ``n`` of this library's kernels was replayed."""
    global _launches
    _launches += n


_last_fn = ""      # the entry point that launched last (a hint for launches that can overlap with their like)


_entry_points = {}     # (library, function) -> (the function, its library): found once


def _call(libname: str, fn: str, *args) -> None:
    global _launches, _last_fn
    found = _entry_points.get((libname, fn))
    if found is None:
        lib = library.load(libname)
        found = _entry_points[libname, fn] = (getattr(lib, fn), lib)
    if _dry:
        return
    _last_fn = ""
    if found[0](*args) != 0:
        raise ExtensionError(found[1].last_error().decode())
    _launches += 1
    _last_fn = fn


def launch_overlap(on: bool) -> None:
    """Whether kernels that can do so are launched to start while the kernel before them ends: a few-token
    product after another one (it asks for its first weights before it waits for that one's results), the
    tensor-core products (their set-up; up to 64 tokens also their first weight tiles), prefill attention (its
    set-up) and the norms between them.
    On by default; off, every kernel waits for the one before it to be over, and the results are the same bits."""
    for name in ("linear_skinny", "gemm_sm100", "generic", "attention_tc"):
        getattr(library.load(name), f"nncpu_launch_overlap_{name}")(ctypes.c_int(1 if on else 0))


_l = ctypes.c_long      # a C long: strides in elements

_i = int      # a C int: ctypes passes a Python int as one (sizes, counts, flags, type codes; booleans become 0 or 1)


def _f(v) -> ctypes.c_float:
    return ctypes.c_float(float(v))


def embed(table, ids, out, scale: float = 1.0, pos_table=None, positions=None) -> None:
    """out[t] = table[ids[t]] * scale; out is float32 [n, hidden]; ids int32.  With ``pos_table`` [n_pos, hidden]
    (learned position vectors) and ``positions`` int32 [n]: out[t] += pos_table[positions[t]], not scaled."""
    n, hidden = out.shape
    assert out.dtype == torch.float32 and ids.dtype == torch.int32 and ids.numel() >= n
    n_pos = 0
    if pos_table is not None:
        n_pos = pos_table.shape[0]
        assert pos_table.shape[1] == hidden and positions.dtype == torch.int32 and positions.numel() >= n
    _call("generic", "nncpu_embed", _ptr(table), _i(_code(table)), _ptr(ids), _ptr(out), _i(n), _i(hidden),
          _i(table.shape[0]), _f(scale), _ptr(pos_table), _i(_code(pos_table)),
          _ptr(positions if pos_table is not None else None), _i(n_pos), _stream())


def rmsnorm(x, gamma, eps: float, out, rows=None, gamma_offset: float = 0.0, accumulate: bool = False) -> None:
    """out[r] = rmsnorm(x[rows[r]] or x[r]) * (gamma + gamma_offset) over the last axis; with ``accumulate``
    the result is added to ``out`` (the norm that closes a sublayer adds into the residual stream)."""
    dim = x.shape[-1]
    n_rows = out.numel() // dim
    assert gamma is None or gamma.numel() == dim
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() >= n_rows)
    _call("generic", "nncpu_rmsnorm", _ptr(x), _i(_code(x)), _ptr(gamma), _i(_code(gamma)), _ptr(out),
          _i(_code(out)), _ptr(rows), _i(n_rows), _i(dim), _f(eps), _f(gamma_offset), _i(accumulate), _stream())


def layernorm(x, weight, bias, eps: float, out, rows=None) -> None:
    """out = (x - mean) / sqrt(var + eps) * weight + bias per row, var the mean of the squared deviations; x float32,
    32-bit arithmetic.  ``rows`` (int32) picks the input rows."""
    n = out.shape[0]
    dim = x.shape[1]
    assert x.dtype == torch.float32 and x.is_contiguous() and out.shape == (n, dim)
    assert weight.numel() == dim and bias.numel() == dim and weight.dtype == bias.dtype
    assert rows is None or (rows.dtype == torch.int32 and rows.numel() == n)
    _call("generic", "nncpu_layernorm", _ptr(x), _ptr(weight), _ptr(bias), _i(_code(weight)), _ptr(out), _i(_code(out)),
          _ptr(rows), _i(n), _i(dim), _f(eps), _stream())


def pair_embed(table, ids, tok_seq, tok_pos, cu_seqlens, seq_slots, last, out, buckets: int, mul_prev: int,
               mul_cur: int) -> None:
    """out[t] += table[(prev * mul_prev + id * mul_cur) mod buckets] with prev the token before token t in its
    sequence, and table[buckets] for a sequence's first token.  ``last`` int32 [slots + 1, 1] holds every sequence's
    last token from step to step: it is read for a step's first tokens and left at the step's last ones."""
    n, hidden = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and table.shape == (buckets + 1, hidden)
    assert ids.dtype == tok_seq.dtype == tok_pos.dtype == cu_seqlens.dtype == seq_slots.dtype == torch.int32
    assert last.dtype == torch.int32 and last.is_contiguous() and ids.numel() >= n
    _call("generic", "nncpu_pair_embed", _ptr(table), _i(_code(table)), _ptr(ids), _ptr(tok_seq), _ptr(tok_pos),
          _ptr(cu_seqlens), _ptr(seq_slots), _ptr(last), _ptr(out), _i(n), _i(hidden), _l(buckets), _l(mul_prev),
          _l(mul_cur), _stream())


def concat_rows(a, b, out) -> None:
    """out = [a, b] along the last axis in ``out``'s element type (``b`` None: a conversion of ``a``); a, b float32."""
    n, dim = a.shape
    assert a.dtype == torch.float32 and a.is_contiguous() and out.is_contiguous()
    assert b is None or (b.dtype == torch.float32 and b.shape == a.shape and b.is_contiguous())
    assert out.shape == (n, dim * (1 if b is None else 2))
    _call("generic", "nncpu_concat_rows", _ptr(a), _ptr(b), _ptr(out), _i(_code(out)), _i(n), _i(dim), _stream())


def stream_axpy(x, y, alpha: float) -> None:
    """x += alpha * y, float32."""
    assert x.dtype == y.dtype == torch.float32 and x.shape == y.shape and x.is_contiguous() and y.is_contiguous()
    _call("generic", "nncpu_stream_axpy", _ptr(x), _ptr(y), _f(alpha), _l(x.numel()), _stream())


def branch_norm_add_takes_norm(dim: int) -> bool:
    """Whether ``branch_norm_add`` can leave the layer norm that follows (``then_norm``) for rows of ``dim`` lanes."""
    return dim > 0 and dim % 4 == 0 and dim <= 8192


def branch_norm_add(x, a, wa, b, wb, eps: float, alpha: float, then_norm=None) -> None:
    """x += alpha * (rmsnorm(a) * wa + rmsnorm(b) * wb) row by row (``b`` None: the first term alone; a weight None:
    ones); x, a, b float32.  ``then_norm`` = (weight, bias, eps, out): the layer norm of the new rows is left in ``out``
    in the same pass (where ``branch_norm_add_takes_norm`` says so)."""
    n, dim = x.shape
    ln_w = ln_b = ln_out = None
    ln_eps = 0.0
    if then_norm is not None:
        ln_w, ln_b, ln_eps, ln_out = then_norm
        assert branch_norm_add_takes_norm(dim) and ln_out.shape == x.shape and ln_out.is_contiguous()
        assert ln_w.numel() == ln_b.numel() == dim and ln_w.dtype == ln_b.dtype
    assert x.dtype == a.dtype == torch.float32 and a.shape == x.shape and x.is_contiguous() and a.is_contiguous()
    assert b is None or (b.dtype == torch.float32 and b.shape == x.shape and b.is_contiguous())
    assert wa is None or wa.numel() == dim
    assert wb is None or (wb.numel() == dim and (wa is None or wa.dtype == wb.dtype))
    w = wa if wa is not None else wb
    _call("generic", "nncpu_branch_norm_add", _ptr(x), _ptr(a), _ptr(wa), _ptr(b), _ptr(wb), _i(_code(w)), _f(eps),
          _f(alpha), _i(n), _i(dim), _ptr(ln_w), _ptr(ln_b), _i(_code(ln_w)), _f(ln_eps), _ptr(ln_out), _i(_code(ln_out)),
          _stream())


def relu2(x, out, scale: float = 1.0) -> None:
    """out = scale * max(x, 0)^2; x float32."""
    assert x.dtype == torch.float32 and x.shape == out.shape and x.is_contiguous() and out.is_contiguous()
    _call("generic", "nncpu_unary_act", _ptr(x), _ptr(out), _i(_code(out)), _l(x.numel()), _i(0), _f(scale), _stream())


GATE_ROWS_MAX_TOKENS = 16


def token_gate_rows(x, w, table, ids, col: int, out) -> None:
    """out[t, j] = gelu_tanh(w[j] . x[t]) * table[ids[t], col + j] for a step of up to ``GATE_ROWS_MAX_TOKENS`` tokens
    in one launch: the product, the activation and the gating.  x float32 [n, width] (read as it is), w [dim, width]."""
    n, width = x.shape
    dim = w.shape[0]
    assert n <= GATE_ROWS_MAX_TOKENS and x.dtype == torch.float32 and x.is_contiguous()
    assert w.shape == (dim, width) and w.is_contiguous() and out.shape == (n, dim) and out.is_contiguous()
    assert table.dim() == 2 and table.is_contiguous() and 0 <= col and col + dim <= table.shape[1]
    assert ids.dtype == torch.int32 and ids.numel() >= n
    _call("generic", "nncpu_token_gate_rows", _ptr(x), _ptr(w), _i(_code(w)), _ptr(table), _i(_code(table)), _ptr(ids),
          _i(table.shape[1]), _i(col), _ptr(out), _i(_code(out)), _i(n), _i(width), _i(dim), _stream())


def token_gate(z, table, ids, col: int, out) -> None:
    """out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col + j]: lanes of a per-token table gate a projection; z float32."""
    n, dim = z.shape
    assert z.dtype == torch.float32 and z.is_contiguous() and out.shape == z.shape and out.is_contiguous()
    assert table.dim() == 2 and table.is_contiguous() and 0 <= col and col + dim <= table.shape[1]
    assert ids.dtype == torch.int32 and ids.numel() >= n
    _call("generic", "nncpu_token_gate", _ptr(z), _ptr(table), _i(_code(table)), _ptr(ids), _i(table.shape[1]), _i(col),
          _ptr(out), _i(_code(out)), _i(n), _i(dim), _stream())


def rmsnorm_pair_supported(dim: int) -> bool:
    return dim > 0 and dim % 4 == 0 and dim <= 8192


def rmsnorm_pair(branch, residual, gamma1, offset1: float, eps1: float, gamma2, offset2: float, eps2: float, out) -> None:
    """residual += rmsnorm(branch) * (gamma1 + offset1), then out = rmsnorm(residual) * (gamma2 + offset2): the norm
    that closes a sublayer and the one that opens the next in one pass.  branch and residual float32 [n, dim]."""
    n, dim = residual.shape
    assert branch.shape == residual.shape == out.shape and branch.dtype == residual.dtype == torch.float32
    assert gamma1.numel() == gamma2.numel() == dim and gamma1.dtype == gamma2.dtype
    _call("generic", "nncpu_rmsnorm_pair", _ptr(branch), _ptr(residual), _ptr(gamma1), _f(offset1), _f(eps1), _ptr(gamma2),
          _f(offset2), _f(eps2), _i(_code(gamma1)), _ptr(out), _i(_code(out)), _i(n), _i(dim), _stream())


def linear_simt(x, w, bias, out, accumulate: bool = False) -> None:
    """out (+)= x . w^T + bias on CUDA cores in 32-bit; any sizes and element types."""
    m, k = x.shape
    n = w.shape[0]
    assert w.shape[1] == k and out.shape == (m, n)
    _call("generic", "nncpu_linear_simt", _ptr(x), _i(_code(x)), _ptr(w), _i(_code(w)), _ptr(bias),
          _i(_code(bias)), _ptr(out), _i(_code(out)), _i(m), _i(n), _i(k), _i(k), _i(n), _i(accumulate), _stream())


def linear_tc_supported(m: int, n: int, k: int) -> bool:
    return m > 0 and k % 8 == 0


class GemmWorkspace:
    """Device memory the tensor-core kernels need besides their operands:
    scratch for the partial tiles of products that deal their k-blocks out
    evenly, and the status word that a kernel sets when a bounded wait ran
    out.  Launches that share a workspace must not overlap on the GPU (one
    stream)."""

    def __init__(self, device):
        lib = library.load("gemm_sm100")
        lib.nncpu_linear_tc_scratch_floats.restype = ctypes.c_long
        self.scratch = torch.empty(lib.nncpu_linear_tc_scratch_floats(), dtype=torch.float32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)


# Which kernel a tensor-core product runs with, where a measurement or a test wants another than its sizes would get.
PLANS = {"auto": 0, "even_from_17": 1, "never_even": 2, "no_pairs": 4, "narrow_units": 8}

EPILOGUES = {"plain": 0, "swiglu": 1}


_ACTIVATIONS = {"xielu": 1, "gelu_tanh": 2, "swish_clamp": 3, "relu2": 4}


def _activation(activation):
    """``activation`` None, or (kind, a, b).  With the plain epilogue ("xielu", a, b), a = softplus(p) and
    b = 1/2 + softplus(q) ready-made, or ("relu2", a, 0), a times the square of relu: applied to the product's result after
    the bias (no accumulation).  With the
    gated epilogue the gate's activation in place of SiLU: ("gelu_tanh", 0, 0) or ("swish_clamp", limit, 0), see
    ``gated_act``."""
    if activation is None:
        return _i(0), _f(0.0), _f(0.0)
    kind, a, b = activation
    if kind not in _ACTIVATIONS:
        raise InvalidArgument(f"a product cannot apply the activation {kind!r}")
    return _i(_ACTIVATIONS[kind]), _f(a), _f(b)


@functools.lru_cache(maxsize=4096)
def linear_tc_fuses_norms(m: int, n: int) -> bool:
    """Whether the tensor-core product of ``m`` tokens with ``n`` output features can carry the norms around it
    (``linear_tc``'s ``norm_out`` and ``norm_in``): the products of whole prompts."""
    return bool(library.load("gemm_sm100").nncpu_linear_tc_fuses_norms(m, n))


@functools.lru_cache(maxsize=4096)
def linear_tc_norm_roles(m: int, n: int, k: int) -> int:
    """Which norms the tensor-core product of ``m`` tokens, ``n`` output features and width ``k`` can carry: bit 0 the
    norm before it (``norm_in``), bit 1 the norm after it (``norm_out``).  Whole prompts both; 17 to 64 tokens the
    norm before, and the norm after where a cluster shares every output tile."""
    return int(library.load("gemm_sm100").nncpu_linear_tc_norm_roles(m, n, k))


def linear_tc(x, w, bias, out, workspace: GemmWorkspace, accumulate: bool = False, epilogue: str = "plain",
              plan: str = "auto", norm_out=None, norm_in=None, activation=None) -> None:
    """out (+)= x . w^T + bias on the tensor cores; x and w bfloat16.  With
    ``epilogue="swiglu"`` the rows of w hold gate and up rows interleaved in
    blocks of 8 and out [m, n/2] receives silu(gate) * up.  ``plan``: "auto",
    or for measurements and tests "even_from_17" (17 to 64 tokens deal their
    k-blocks out evenly like 65 to 256), "never_even", "no_pairs".

    Where ``linear_tc_norm_roles(m, n, k)`` says so, the product can carry the RMS norms around it as
    ``linear_skinny`` does: ``norm_out = (xg, gamma, bins, bins_clear)`` and ``norm_in = (bins, eps)`` with accumulators of
    ``NORM_ROW_WORDS`` 64-bit words per row (int64 [m, NORM_ROW_WORDS])."""
    m, k = x.shape
    n = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert w.shape[1] == k and out.shape == (m, n // 2 if epilogue == "swiglu" else n)
    xg = gamma = bins_out = bins_clear = bins_in = None
    eps = 0.0
    if norm_out is not None:
        xg, gamma, bins_out, bins_clear = norm_out
        assert xg.dtype == torch.bfloat16 and xg.shape == (m, n) and xg.is_contiguous() and gamma.numel() == n
        assert bins_out.dtype == torch.int64 and bins_out.shape == (m, NORM_ROW_WORDS) and bins_out.is_contiguous()
        assert bins_clear is None or (bins_clear.dtype == torch.int64 and bins_clear.shape == (m, NORM_ROW_WORDS))
    if norm_in is not None:
        bins_in, eps = norm_in
        assert bins_in.dtype == torch.int64 and bins_in.shape == (m, NORM_ROW_WORDS) and bins_in.is_contiguous()
    _call("gemm_sm100", "nncpu_linear_tc", _ptr(x), _ptr(w), _ptr(bias), _i(_code(bias)), _ptr(out),
          _i(_code(out)), _i(m), _i(n), _i(k), _i(x.stride(0)), _i(out.shape[1]), _i(accumulate), _i(EPILOGUES[epilogue]),
          _i(PLANS[plan]), _ptr(xg), _ptr(gamma), _i(_code(gamma)), _ptr(bins_out), _ptr(bins_clear), _ptr(bins_in),
          _f(eps), *_activation(activation), _ptr(workspace.scratch), _ptr(workspace.status), _stream())


def linear_tc_wait_probe(x, w, out, workspace: GemmWorkspace, limit_ms: int = 5) -> None:
    """The library's check of its own failure path: one tile of x [128, K] . w [256, K]^T whose copies are
    expected to bring more bytes than they do, with every wait limited to ``limit_ms``.  The kernel gives up in
    order, frees what it holds and sets the workspace's status word; ``out`` is not written."""
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype == torch.float32
    assert x.shape[0] == 128 and w.shape[0] == 256 and x.shape[1] == w.shape[1] and out.shape == (128, 256)
    _call("gemm_sm100", "nncpu_linear_tc_wait_probe", _ptr(x), _ptr(w), _ptr(out), _i(x.shape[1]), _i(limit_ms),
          _ptr(workspace.status), _stream())


def linear_tc_qkv_supported(x, n_heads: int, n_kv: int, head_dim: int) -> bool:
    """Whether the q/k/v projection of these tokens can run with its epilogue fused."""
    lib = library.load("gemm_sm100")
    return x.dtype == torch.bfloat16 and bool(
        lib.nncpu_linear_tc_qkv_supported(x.shape[0], x.shape[1], x.stride(0), n_heads, n_kv, head_dim))


def linear_tc_qkv(x, w_qkv, q_gamma, k_gamma, eps, cos_sin, tok_seq, tok_pos, block_table, k_pages, v_pages, q_out,
                  workspace: GemmWorkspace, n_heads: int, n_kv: int, head_dim: int, norm_in=None) -> None:
    """x . w_qkv^T with the per-head norm, the rotation and the stores fused into the product's epilogue:
    queries to ``q_out``, keys and values to the tokens' rows of the cache pages.  bfloat16 throughout,
    32-bit accumulators, norm and rotation.  ``cos_sin`` is the rotation table laid out by pair:
    float32 [head_dim / 2, tokens, 2].  ``norm_in = (bins, eps)``: ``x`` holds the rows of the norm before the
    projection times gamma, and the rows' scales are applied to the accumulators (as in ``linear_tc``)."""
    m, k = x.shape
    bins_in, norm_eps = norm_in if norm_in is not None else (None, 0.0)
    assert bins_in is None or (bins_in.dtype == torch.int64 and bins_in.shape == (m, NORM_ROW_WORDS))
    assert w_qkv.shape == ((n_heads + 2 * n_kv) * head_dim, k) and q_out.shape == (m, n_heads * head_dim)
    assert x.dtype == w_qkv.dtype == q_out.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16
    assert q_out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert k_pages.shape[1:] == (n_kv, 64, head_dim) and v_pages.shape == k_pages.shape
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (head_dim // 2, m, 2))
    assert q_gamma is None or k_gamma is None or q_gamma.dtype == k_gamma.dtype
    g = q_gamma if q_gamma is not None else k_gamma
    _call("gemm_sm100", "nncpu_linear_tc_qkv", _ptr(x), _ptr(w_qkv), _i(m), _i(k), _i(x.stride(0)), _ptr(q_out),
          _ptr(k_pages), _ptr(v_pages), _ptr(q_gamma), _ptr(k_gamma), _i(_code(g)), _f(eps), _ptr(cos_sin),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(block_table), _i(block_table.shape[1]), _i(n_heads), _i(n_kv),
          _i(head_dim), _ptr(bins_in), _f(norm_eps), _ptr(workspace.status), _stream())


SKINNY_MAX_TOKENS = 16
CLUSTER_MAX_TOKENS = 64    # up to here a tensor-core product's weights are the 128-row operand of one tile row


def linear_skinny(x, w, bias, out, accumulate: bool = False, epilogue: str = "plain", norm_out=None,
                  norm_in=None, activation=None) -> None:
    """The same product for at most 16 tokens: a stream over the weights that
    uses every SM, with no scratch memory.

    The product can carry the RMS norms around it.  ``norm_out = (xg, gamma, bins, bins_clear)``: besides ``out``
    it leaves ``xg`` (bfloat16 [m, n]) = out * gamma and adds the sums of squares of out's rows into ``bins`` (int64
    [NORM_WORDS], zero before the call: exact accumulators that do not depend on the order of additions);
    ``bins_clear`` (or None) is another such block, which is set to zero.  ``norm_in = (bins, eps)``: ``x`` holds
    such rows times gamma, and the result is multiplied by 1 / sqrt(sum / k + eps) per row before bias and
    activation."""
    m, k = x.shape
    n = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    assert w.shape[1] == k and out.shape == (m, n // 2 if epilogue == "swiglu" else n)
    xg = gamma = bins_out = bins_clear = bins_in = None
    eps = 0.0
    if norm_out is not None:
        xg, gamma, bins_out, bins_clear = norm_out
        assert xg.dtype == torch.bfloat16 and xg.shape == (m, n) and gamma.numel() == n
        assert bins_out.dtype == torch.int64 and bins_out.numel() == NORM_WORDS
        assert bins_clear is None or (bins_clear.dtype == torch.int64 and bins_clear.numel() == NORM_WORDS)
    if norm_in is not None:
        assert norm_out is None, "a product is a norm's producer or its consumer"
        bins_in, eps = norm_in
        assert bins_in.dtype == torch.int64 and bins_in.numel() == NORM_WORDS
    # a product that follows another one may start while that one ends (see launch_overlap)
    after_skinny = _last_fn == "nncpu_linear_skinny"
    _call("linear_skinny", "nncpu_linear_skinny", _ptr(x), _ptr(w), _ptr(bias), _i(_code(bias)), _ptr(out),
          _i(_code(out)), _i(m), _i(n), _i(k), _i(k), _i(out.shape[1]), _i(accumulate), _i(EPILOGUES[epilogue]),
          _ptr(xg), _ptr(gamma), _i(_code(gamma)), _ptr(bins_out), _ptr(bins_clear), _ptr(bins_in), _f(eps),
          *_activation(activation), _i(after_skinny), _stream())


def linear_skinny_force_warps(warps: int) -> None:
    """For measurements and tests: the few-token product runs as blocks of 8 or of 4 warps whatever the sizes;
    0: chosen by the sizes (4 warps where 16-row blocks number more than two per SM and at most four)."""
    library.load("linear_skinny").nncpu_linear_skinny_force_warps(ctypes.c_int(int(warps)))


NORM_ROW_WORDS = 16  # 64-bit words of one row's accumulator: 8 bins, a word that says "not finite", spare
NORM_WORDS = 256    # the accumulators of one norm of a few-token step: 16 rows


def rope_table(positions, inv_freq, out, position_scale: float = 1.0, by_pair: bool = False, stretch: float = 1.0) -> None:
    """out[t, i] = stretch * (cos, sin)(positions[t] * position_scale * inv_freq[i]); out float32 [n, half, 2], or with
    ``by_pair`` [half, n, 2] holding the same values as out[i, t]."""
    if by_pair:
        half, n, two = out.shape
    else:
        n, half, two = out.shape
    assert two == 2 and out.dtype == torch.float32 and inv_freq.dtype == torch.float32
    assert inv_freq.numel() == half and positions.dtype == torch.int32 and positions.numel() >= n
    _call("generic", "nncpu_rope_table", _ptr(positions), _ptr(inv_freq), _ptr(out), _i(n), _i(half),
          _f(position_scale), _i(by_pair), _f(stretch), _stream())


def qk_norm_rope_append(qkv, q_gamma, k_gamma, eps, cos_sin, tok_seq, tok_pos, block_table, k_pages, v_pages,
                        q_out, n_heads: int, n_kv: int, head_dim: int, v_head_dim: int = 0, q_temp=None,
                        values_are_keys: bool = False) -> None:
    """Per-head norm and rotation of q and k, and the append of k and v to
    their pages.  ``n_kv`` 0: qkv holds q only and nothing is appended.  ``v_head_dim``: lanes of a value
    head when they differ from ``head_dim``.  ``q_temp = (coef, every)``: the query at position p is
    multiplied by 1 + coef * ln(floor((p + 1) / every) + 1).  ``values_are_keys``: the rows hold no value heads, a
    position's value is its key as projected (before norm and rotation).  A row may be longer than its heads."""
    n = q_out.shape[0]
    rot_half = 0 if cos_sin is None else cos_sin.shape[1]
    v_head_dim = v_head_dim or head_dim
    coef, every = q_temp if q_temp is not None else (0.0, 1)
    assert qkv.shape[0] == n and q_out.shape == (n, n_heads * head_dim) and qkv.is_contiguous()
    assert qkv.shape[1] >= (n_heads + n_kv) * head_dim + (0 if values_are_keys else n_kv * v_head_dim)
    assert q_gamma is None or k_gamma is None or q_gamma.dtype == k_gamma.dtype
    g = q_gamma if q_gamma is not None else k_gamma
    bt_stride = block_table.shape[1] if block_table is not None else 0
    _call("generic", "nncpu_qk_norm_rope_append", _ptr(qkv), _i(_code(qkv)), _ptr(q_gamma), _ptr(k_gamma),
          _i(_code(g)), _f(eps), _ptr(cos_sin), _i(rot_half), _ptr(tok_seq), _ptr(tok_pos), _ptr(block_table),
          _i(bt_stride), _ptr(k_pages), _ptr(v_pages), _i(_code(k_pages)), _ptr(q_out), _i(_code(q_out)), _i(n),
          _i(n_heads), _i(n_kv), _i(head_dim), _i(v_head_dim), _f(coef), _i(every), _i(qkv.shape[1]),
          _i(values_are_keys), _stream())


def key_span(window: int = 0, chunk: int = 0) -> int:
    """The one number by which every attention kernel knows which earlier keys a query sees (their ``window``
    argument): ``window`` > 0, the last ``window`` keys up to the query, as it is; ``chunk`` > 0, the keys of the
    query's own block of ``chunk`` positions (blocks counted from position 0 of the sequence), as ``-chunk``; 0: all."""
    if window < 0 or chunk < 0 or (window and chunk):
        raise InvalidArgument(f"a mixer's keys are limited by a window ({window}) or by blocks ({chunk}), not both")
    return window if window else -chunk


def attention(q, k_pages, v_pages, block_table, tok_seq, tok_pos, out, n_heads: int, n_kv: int, head_dim: int,
              scale: float, window: int = 0, v_head_dim: int = 0, slope_base: float = 0.0, sinks=None) -> None:
    """Causal attention of each token over its sequence's pages.  ``window``: see ``key_span`` (here and in the
    other attention kernels).  ``v_head_dim``: lanes of a value head (and of
    the output) when they differ from ``head_dim``.  ``slope_base`` b != 0: head h takes
    2^(-b (h + 1) / n_heads) * (query position - key position) off its scaled scores.  ``sinks`` (float32
    [n_heads]): exp(sinks[h]) joins the denominator of head h's softmax (here and in the other attention kernels)."""
    n = q.shape[0]
    v_head_dim = v_head_dim or head_dim
    assert q.shape == (n, n_heads * head_dim) and out.shape == (n, n_heads * v_head_dim)
    assert k_pages.dtype == v_pages.dtype and block_table.dtype == torch.int32
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == n_heads)
    _call("generic", "nncpu_attention", _ptr(q), _i(_code(q)), _ptr(k_pages), _ptr(v_pages), _i(_code(k_pages)),
          _ptr(block_table), _i(block_table.shape[1]), _ptr(tok_seq), _ptr(tok_pos), _ptr(out), _i(_code(out)),
          _i(n), _i(n_heads), _i(n_kv), _i(head_dim), _i(v_head_dim), _f(scale), _i(window), _f(slope_base), _ptr(sinks),
          _stream())


def attention_mma_supported(n_heads: int, n_kv: int, head_dim: int, *tensors) -> bool:
    """The tensor-core attention kernels take bfloat16 q, cache and output with
    head size 64 or 128 (where more than 16 query heads share a key/value head, several blocks of the decode
    kernel take a part of them each)."""
    return (head_dim in (64, 128) and n_kv > 0 and n_heads % n_kv == 0
            and all(t.dtype == torch.bfloat16 for t in tensors))


# How decode attention cuts a sequence's keys into splits: the kernel's launch bounds let two of its blocks run on
# an SM at once, and a split shorter than this many keys costs more in merging than it gains.
DECODE_BLOCKS_PER_SM = 2
DECODE_MIN_KEYS_PER_SPLIT = 256
DECODE_CLUSTER_MAX_SPLITS = 8      # up to here the splits merge inside a thread-block cluster, without scratch


def attention_decode_splits(n_tokens: int, n_kv: int, longest: int, sm_count: int) -> int:
    """As many splits as keep every block of the grid running at once (never a second wave), each with at
    least ``DECODE_MIN_KEYS_PER_SPLIT`` keys of the longest sequence.  Up to twice what a cluster merges is cut
    back to what it merges: one launch instead of two costs less than the finer cut gains (one sequence of 3 072
    keys: 8 splits in a cluster 9.1 us, 12 through scratch and a merge kernel 9.3 us before the kernel boundary)."""
    pairs = max(1, n_tokens * n_kv)
    n = max(1, min(DECODE_BLOCKS_PER_SM * sm_count // pairs, longest // DECODE_MIN_KEYS_PER_SPLIT))
    return DECODE_CLUSTER_MAX_SPLITS if DECODE_CLUSTER_MAX_SPLITS < n <= 2 * DECODE_CLUSTER_MAX_SPLITS else n


def attention_decode_scratch_floats(n_tok: int, n_heads: int, n_kv: int, head_dim: int, n_splits: int) -> int:
    return 0 if n_splits <= 1 else n_tok * n_kv * n_splits * (n_heads // n_kv) * (head_dim + 2)


def attention_decode_mma(q, k_pages, v_pages, block_table, tok_seq, tok_pos, out, scratch, n_heads: int, n_kv: int,
                         head_dim: int, scale: float, window: int, n_splits: int, slope_base: float = 0.0,
                         sinks=None) -> None:
    """One token per sequence; each token's keys are cut into ``n_splits``
    splits that run in parallel.  With ``scratch`` (float32,
    ``attention_decode_scratch_floats`` elements) a second kernel merges them;
    with ``scratch`` None and at most 8 splits they form a thread-block
    cluster and merge through distributed shared memory.  ``sinks`` as in ``attention``: the term joins where the
    splits merge, once."""
    n = q.shape[0]
    assert q.shape == (n, n_heads * head_dim) and out.shape == q.shape
    assert scratch is None or scratch.dtype == torch.float32
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == n_heads)
    _call("attention_mma", "nncpu_attention_decode_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
          _i(block_table.shape[1]), _ptr(tok_seq), _ptr(tok_pos), _ptr(out), _ptr(scratch),
          ctypes.c_long(0 if scratch is None else scratch.numel()), _i(n), _i(n_heads), _i(n_kv), _i(head_dim),
          _f(scale), _i(window), _i(n_splits), _f(slope_base), _ptr(sinks), _stream())


def attention_decode_mma_from_qkv(qkv, q_gamma, k_gamma, eps, cos_sin, k_pages, v_pages, append: bool, block_table,
                                  tok_seq, tok_pos, out, scratch, n_heads: int, n_kv: int, head_dim: int, scale: float,
                                  window: int, n_splits: int, slope_base: float = 0.0, q_temp=None, sinks=None,
                                  values_are_keys: bool = False, gated: bool = False) -> None:
    """Decode attention that starts from the float32 projections ``qkv`` [n, per_tok * head_dim] (q heads, then with
    ``append`` the k and v heads): every block makes its queries itself (per-head norm, rotation by ``cos_sin``
    [n, head_dim / 2, 2]), and with ``append`` the token's key and value are made, written to the cache and used.
    One launch in place of ``qk_norm_rope_append`` and ``attention_decode_mma``, with the same arithmetic;
    ``slope_base``, ``q_temp`` and ``sinks`` as there.  ``values_are_keys``: the rows hold no v heads, a token's value
    is its key as projected.  ``gated``: n_heads more heads of logits end the rows, and the output is multiplied lane by
    lane by their sigmoid (in place of ``sigmoid_gate``)."""
    n = out.shape[0]
    per_tok = n_heads + (((1 if values_are_keys else 2) * n_kv) if append else 0) + (n_heads if gated else 0)
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == n_heads)
    assert qkv.dtype == torch.float32 and qkv.shape == (n, per_tok * head_dim) and qkv.is_contiguous()
    assert out.shape == (n, n_heads * head_dim) and out.dtype == torch.bfloat16
    assert k_pages.dtype == v_pages.dtype == torch.bfloat16 and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (n, head_dim // 2, 2))
    assert q_gamma is None or k_gamma is None or q_gamma.dtype == k_gamma.dtype
    assert scratch is None or scratch.dtype == torch.float32
    g = q_gamma if q_gamma is not None else k_gamma
    _call("attention_mma", "nncpu_attention_decode_mma_from_qkv", _ptr(qkv), _ptr(q_gamma), _ptr(k_gamma), _i(_code(g)),
          _f(eps), _ptr(cos_sin), _ptr(k_pages), _ptr(v_pages), _i(append), _ptr(block_table), _i(block_table.shape[1]),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(out), _ptr(scratch), ctypes.c_long(0 if scratch is None else scratch.numel()),
          _i(n), _i(n_heads), _i(n_kv), _i(head_dim), _f(scale), _i(window), _i(n_splits), _f(slope_base),
          _f(q_temp[0] if q_temp else 0.0), _i(q_temp[1] if q_temp else 1), _ptr(sinks), _i(values_are_keys), _i(gated),
          _stream())


def attention_prefill_mma(q, k_pages, v_pages, block_table, cu_seqlens, tok_pos, out, n_seqs: int, n_heads: int,
                          n_kv: int, head_dim: int, scale: float, window: int, slope_base: float = 0.0,
                          sinks=None) -> None:
    """Any number of new tokens per sequence, at consecutive positions.  ``slope_base`` and ``sinks`` as in
    ``attention``."""
    n = q.shape[0]
    assert q.shape == (n, n_heads * head_dim) and out.shape == q.shape and cu_seqlens.numel() >= n_seqs + 1
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == n_heads)
    _call("attention_mma", "nncpu_attention_prefill_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
          _i(block_table.shape[1]), _ptr(cu_seqlens), _ptr(tok_pos), _ptr(out), _i(n), _i(n_seqs), _i(n_heads),
          _i(n_kv), _i(head_dim), _f(scale), _i(window), _f(slope_base), _ptr(sinks), _stream())


def attention_prefill_tc_supported(n_heads: int, n_kv: int, head_dim: int, *tensors) -> bool:
    """Whether the tcgen05 prefill kernel takes these sizes (and these tensors: all bfloat16)."""
    lib = library.load("attention_tc")
    return bool(lib.nncpu_attention_prefill_tc_supported(n_heads, n_kv, head_dim)) and \
        all(t.dtype == torch.bfloat16 for t in tensors)


def attention_prefill_tc(q, k_pages, v_pages, block_table, cu_seqlens, tok_pos, out, status, n_seqs: int,
                         n_heads: int, n_kv: int, head_dim: int, scale: float, window: int, slope_base: float = 0.0,
                         sinks=None) -> None:
    """Prefill attention on the tcgen05 tensor cores: any number of new tokens per sequence, at consecutive
    positions; ``status`` is an int32 word on the device that receives a code if a bounded wait runs out.
    ``slope_base`` and ``sinks`` as in ``attention``."""
    assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == n_heads)
    n = q.shape[0]
    assert q.shape == (n, n_heads * head_dim) and out.shape == q.shape and cu_seqlens.numel() >= n_seqs + 1
    assert q.is_contiguous() and out.is_contiguous() and k_pages.is_contiguous() and v_pages.is_contiguous()
    assert k_pages.shape[1:] == (n_kv, 64, head_dim) and v_pages.shape == k_pages.shape
    assert status.dtype == torch.int32
    _call("attention_tc", "nncpu_attention_prefill_tc", _ptr(q), _ptr(k_pages), _ptr(v_pages), _i(k_pages.shape[0]),
          _ptr(block_table), _i(block_table.shape[1]), _ptr(cu_seqlens), _ptr(tok_pos), _ptr(out), _i(n), _i(n_seqs),
          _i(n_heads), _i(n_kv), _i(head_dim), _f(scale), _i(window), _f(slope_base), _ptr(sinks),
          _ptr(status), _stream())


GATED_ACTS = {"silu": 0, "gelu_tanh": 1, "swish_clamp": 2}


def gated_act(gate_up, out, kind: str = "silu", limit: float = 0.0) -> None:
    """out[t, i] = act(gate_up[t, i], gate_up[t, I + i]) in 32-bit.  ``kind`` "silu": silu(g) u; "gelu_tanh":
    g/2 (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) u; "swish_clamp": with g' = min(g, limit) and
    u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1)."""
    n, inter = out.shape
    assert gate_up.shape == (n, 2 * inter)
    _call("generic", "nncpu_gated_act", _ptr(gate_up), _i(_code(gate_up)), _ptr(out), _i(_code(out)), _i(n),
          _i(inter), _i(GATED_ACTS[kind]), _f(limit), _stream())


def swiglu(gate_up, out) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    gated_act(gate_up, out, "silu")


def stream_add(x, rows=None, vec=None) -> None:
    """x[t] += rows[t] + vec: float32 x and rows [n, dim], vec [dim] of either element type; either may be None."""
    n, dim = x.shape
    assert x.dtype == torch.float32 and (rows is None or (rows.shape == x.shape and rows.dtype == torch.float32))
    assert vec is None or vec.numel() == dim
    _call("generic", "nncpu_stream_add", _ptr(x), _ptr(rows), _ptr(vec), _i(_code(vec)), _i(n), _i(dim), _stream())


def rmsnorm_dual(x, gamma1, eps1: float, gamma2, eps2: float, out1, out2) -> None:
    """out1 = rmsnorm(x) * gamma1 and out2 = rmsnorm(x) * gamma2 in one pass over float32 x [n, dim]."""
    n, dim = x.shape
    assert x.dtype == torch.float32 and out1.shape == out2.shape == x.shape and out1.dtype == out2.dtype
    assert gamma1.numel() == gamma2.numel() == dim and gamma1.dtype == gamma2.dtype
    _call("generic", "nncpu_rmsnorm_dual", _ptr(x), _ptr(gamma1), _ptr(gamma2), _i(_code(gamma1)), _f(eps1), _f(eps2),
          _ptr(out1), _ptr(out2), _i(_code(out1)), _i(n), _i(dim), _stream())


def linear_heads(x, x_col: int, w, out, out_col: int = 0, gate=None, gate_col: int = 0, x_step: int = 0,
                 out_step: int = 0) -> None:
    """One product per head: out[t, out_col + b * N : ... + N] = x[t, x_col + b * K : ... + K] . w[b]^T for the heads
    b of w [B, N, K]; x and out are row-major matrices whose rows hold the heads side by side.  With ``gate``
    (float32 [n, *]) row t of head b is multiplied by sigmoid(gate[t, gate_col + b]).  32-bit on CUDA cores.
    ``x_step`` / ``out_step``: lanes from one head to the next in a row of x / out when a head there is wider than K / N
    (only the first K lanes are read, only the first N written)."""
    B, N, K = w.shape
    m = x.shape[0]
    x_step, out_step = x_step or K, out_step or N
    assert out.shape[0] == m and x.shape[1] >= x_col + (B - 1) * x_step + K and out.shape[1] >= out_col + (B - 1) * out_step + N
    assert x.is_contiguous() and out.is_contiguous()
    assert gate is None or (gate.dtype == torch.float32 and gate.shape[0] == m and gate.is_contiguous())
    xe, oe = x.element_size(), out.element_size()
    _call("generic", "nncpu_linear_heads", _vp(x.data_ptr() + x_col * xe) if not (x.is_meta and _dry) else None,
          _i(_code(x)), _ptr(w), _i(_code(w)),
          _vp(out.data_ptr() + out_col * oe) if not (out.is_meta and _dry) else None, _i(_code(out)), _i(m), _i(N), _i(K),
          _i(B), _i(x.shape[1]), _i(out.shape[1]), _i(x_step), _i(out_step), _ptr(gate),
          _i(0 if gate is None else gate.shape[1]), _i(gate_col), _stream())


def linear_heads_tc_supported(x, x_col: int, w, out, x_step: int = 0) -> bool:
    """Whether ``linear_heads_tc`` takes these operands: bfloat16 x and w, a head's K a multiple of 64, 16-byte steps."""
    B, N, K = w.shape
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and out.dtype in (torch.bfloat16, torch.float32)
            and x_col == 0 and K % 64 == 0 and x.shape[1] % 8 == 0 and (x_step or K) % 8 == 0)


def linear_heads_tc(x, w, out, workspace: GemmWorkspace, gate=None, gate_col: int = 0, x_step: int = 0,
                    out_step: int = 0) -> None:
    """``linear_heads`` on the tcgen05 tensor cores (the grouped product with the heads as groups): x [n, >= B K]
    bfloat16 with the heads side by side from column 0, w [B, N, K] bfloat16, out [n, >= B N] from column 0.
    ``x_step`` / ``out_step`` as in ``linear_heads``."""
    B, N, K = w.shape
    m = x.shape[0]
    x_step, out_step = x_step or K, out_step or N
    assert linear_heads_tc_supported(x, 0, w, out, x_step) and out.shape[0] == m
    assert x.shape[1] >= (B - 1) * x_step + K and out.shape[1] >= (B - 1) * out_step + N
    assert gate is None or (gate.dtype == torch.float32 and gate.shape[0] == m and gate.is_contiguous())
    _call("gemm_sm100", "nncpu_linear_tc_heads", _ptr(x), _ptr(w), _ptr(out), _i(_code(out)), _i(m), _i(N), _i(K), _i(B),
          _i(x.shape[1]), _i(out.shape[1]), _i(x_step), _i(out_step), _ptr(gate), _i(0 if gate is None else gate.shape[1]),
          _i(gate_col), _ptr(workspace.status), _stream())


def latent_append(proj, col: int, gamma, eps: float, tok_seq, tok_pos, block_table, pages, q_out=None, rot_dim: int = 0,
                  cos_sin=None, q_norm=None) -> None:
    """pages[row of token t] = rmsnorm(proj[t, col : col + rank]) * gamma: the one vector per position that latent
    attention keeps.  proj float32; pages [n_pages, 1, PAGE, rank + rot_dim].  With ``q_out`` (bfloat16 [n, q_size])
    the first q_size columns of proj are left there rounded to bfloat16.  ``rot_dim`` > 0: the rot_dim lanes after the
    latent's in proj are a key part that all heads share; its first 2 * cos_sin.shape[1] lanes are rotated in
    neighbouring pairs by ``cos_sin`` [n, pairs, 2] and it follows the latent in the page row.  ``pages`` None: the
    layer reads another layer's cache, nothing is appended.  ``q_norm = (gamma, col, rank, out)``: the queries' own
    latent at that column is normed into ``out`` [n, rank]."""
    n = proj.shape[0]
    assert proj.dtype == torch.float32 and proj.is_contiguous()
    rank = gamma.numel() if gamma is not None else 1
    if pages is not None:
        assert pages.shape[1] == 1 and pages.shape[-1] == rank + rot_dim
    assert q_out is None or (q_out.dtype == torch.bfloat16 and q_out.shape[0] == n and q_out.shape[1] <= proj.shape[1])
    rot_half = 0 if cos_sin is None else cos_sin.shape[1]
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (n, rot_half, 2))
    qg, qcol, qrank, cq = q_norm if q_norm is not None else (None, 0, 0, None)
    assert q_norm is None or (cq.shape == (n, qrank) and qg.numel() == qrank and cq.is_contiguous()
                              and (gamma is None or qg.dtype == gamma.dtype))
    g = gamma if gamma is not None else qg
    _call("generic", "nncpu_latent_append", _ptr(proj), _i(proj.shape[1]), _i(col), _ptr(gamma), _i(_code(g)), _f(eps),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(block_table), _i(0 if block_table is None else block_table.shape[1]),
          _ptr(pages), _i(_code(pages)), _i(n), _i(rank), _ptr(q_out), _i(0 if q_out is None else q_out.shape[1]),
          _i(rot_dim), _ptr(cos_sin), _i(rot_half), _ptr(qg), _i(qcol), _i(qrank), _ptr(cq), _i(_code(cq)), _stream())


def latent_query(q, cos_sin, q_lat, n_heads: int, head_dim: int, rot_dim: int, rank: int, q16=None) -> None:
    """The rotated part of latent attention's queries: q float32 [n, H (head_dim + rot_dim)] holds per head head_dim
    unrotated lanes, then rot_dim lanes whose first 2 * cos_sin.shape[1] are rotated in neighbouring pairs by ``cos_sin``
    [n, pairs, 2]; they go to q_lat[t, head, rank : rank + rot_dim] (rows of H (rank + rot_dim) lanes).  With ``q16``
    (bfloat16, q's shape) q is also left there rounded."""
    n = q.shape[0]
    rot_half = 0 if cos_sin is None else cos_sin.shape[1]
    assert q.dtype == torch.float32 and q.shape == (n, n_heads * (head_dim + rot_dim)) and q.is_contiguous()
    assert q_lat.shape == (n, n_heads * (rank + rot_dim)) and q_lat.is_contiguous()
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (n, rot_half, 2))
    assert q16 is None or (q16.dtype == torch.bfloat16 and q16.shape == q.shape and q16.is_contiguous())
    _call("generic", "nncpu_latent_query", _ptr(q), _i(n), _i(n_heads), _i(head_dim), _i(rot_dim), _ptr(cos_sin),
          _i(rot_half), _ptr(q_lat), _i(_code(q_lat)), _i(rank), _ptr(q16), _stream())


def sigmoid_gate(x, gate, col: int) -> None:
    """x[t, i] *= sigmoid(gate[t, col + i]) in 32-bit; x [n, width] in either element type, gate float32 [n, >= col + width]."""
    n, width = x.shape
    assert gate.dtype == torch.float32 and gate.shape[0] == n and gate.shape[1] >= col + width
    assert x.is_contiguous() and gate.is_contiguous()
    _call("generic", "nncpu_sigmoid_gate", _ptr(x), _i(_code(x)), _ptr(gate), _i(gate.shape[1]), _i(col), _i(n), _i(width),
          _stream())


def _route_mode(scoring):
    """``scoring`` None: the softmax over the chosen logits alone.  ("all", n_groups, keep, scale): scores are the
    softmax over all experts; the experts form ``n_groups`` equal groups of neighbours whose score is their best
    expert's, and only experts of the ``keep`` best groups can be chosen (``n_groups`` <= 1: no groups); the weights
    are the chosen scores divided by their sum (+ 1e-20), times ``scale``."""
    if scoring is None:
        return _i(0), _i(1), _i(1), _f(1.0)
    kind, n_groups, keep, scale = scoring
    if kind != "all":
        raise InvalidArgument(f"a router cannot score by {kind!r}")
    return _i(1), _i(max(1, n_groups)), _i(max(1, keep)), _f(scale)


def moe_route(logits, top: int, ids, weights, scoring=None) -> None:
    """Per row of float32 logits [n, E]: ids [n, top] (int32) of the largest logits in descending order (the lower
    index wins a tie) and weights [n, top] (float32), the softmax over those logits alone, or what ``scoring`` says
    (see ``_route_mode``)."""
    n, E = logits.shape
    assert logits.dtype == torch.float32 and ids.dtype == torch.int32 and weights.dtype == torch.float32
    assert ids.shape == weights.shape == (n, top)
    _call("generic", "nncpu_moe_route", _ptr(logits), _i(n), _i(E), _i(top), _ptr(ids), _ptr(weights),
          *_route_mode(scoring), _stream())


def moe_router_fits(n_experts: int, width: int) -> bool:
    """Whether ``moe_router`` takes these sizes (a token's input and logits in one block's shared memory)."""
    return 0 < n_experts <= 1024 and (width + 2 * n_experts) * 4 <= 48 * 1024


def moe_router(x, w, bias, top: int, ids, weights, scoring=None) -> None:
    """The router in one launch: logits = x . w^T + bias in 32-bit, then ``moe_route``'s choice and weights."""
    n, width = x.shape
    E = w.shape[0]
    assert w.shape == (E, width) and (bias is None or bias.numel() == E) and ids.shape == weights.shape == (n, top)
    assert ids.dtype == torch.int32 and weights.dtype == torch.float32
    _call("generic", "nncpu_moe_router", _ptr(x), _i(_code(x)), _ptr(w), _i(_code(w)), _ptr(bias), _i(_code(bias)), _i(n),
          _i(E), _i(top), _i(width), _ptr(ids), _ptr(weights), *_route_mode(scoring), _stream())


def moe_experts(x, w_gate, w_up, w_down, ids, weights, act, out, kind: str, limit: float = 0.0) -> None:
    """out[t] += sum_c weights[t, c] * W_down[e] act(W_gate[e] x_t, W_up[e] x_t) with e = ids[t, c].  Weights are
    [E, ff, width] (gate, up) and [E, width, ff] (down); with ``w_up`` None, ``w_gate`` is [E, 2 ff, width] with an
    expert's gate and up rows interleaved in blocks of 8 (the layout of the grouped product).  ``act`` [n * top, ff] is
    scratch in the run's type; out is the float32 stream.  Every token reads its experts' rows itself: the kernel for
    few tokens and for every size and type."""
    n, width = x.shape
    E, ff = w_down.shape[0], w_down.shape[2]
    top = ids.shape[1]
    assert w_down.shape == (E, width, ff) and w_gate.dtype == w_down.dtype
    assert w_gate.shape == ((E, 2 * ff, width) if w_up is None else (E, ff, width))
    assert w_up is None or (w_up.shape == (E, ff, width) and w_up.dtype == w_gate.dtype)
    assert act.shape == (n * top, ff) and out.shape == (n, width) and out.dtype == torch.float32
    _call("generic", "nncpu_moe_experts", _ptr(x), _i(_code(x)), _ptr(w_gate), _ptr(w_up), _ptr(w_down), _i(_code(w_gate)),
          _ptr(ids), _ptr(weights), _ptr(act), _i(_code(act)), _ptr(out), _i(n), _i(top), _i(width), _i(ff), _i(E),
          _i(GATED_ACTS[kind]), _f(limit), _stream())


def moe_plan_tiles(n_slots: int, n_experts: int) -> int:
    """The most 128-row tiles a grouped product over ``n_slots`` rows in ``n_experts`` groups can have."""
    return (n_slots + 127) // 128 + n_experts


def moe_plan(ids, n_experts: int, row_of_slot, slot_of_row, plan) -> None:
    """Sorts the token slots (row-major ``ids`` [n, top]) by expert: ``row_of_slot`` / ``slot_of_row`` (int32 [n * top])
    map slots to rows and back, and ``plan`` (int32 [1 + 3 * moe_plan_tiles]) receives the number of 128-row tiles and
    per tile its expert, first row and its expert's last row + 1, for ``linear_tc_grouped``."""
    S = ids.numel()
    mt = moe_plan_tiles(S, n_experts)
    assert ids.dtype == row_of_slot.dtype == slot_of_row.dtype == plan.dtype == torch.int32
    assert row_of_slot.numel() == slot_of_row.numel() == S and plan.numel() == 1 + 3 * mt and plan.is_contiguous()
    base, dry = (0 if plan.is_meta else plan.data_ptr()), plan.is_meta and _dry
    at = lambda k: None if dry else _vp(base + 4 * k)
    _call("generic", "nncpu_moe_plan", _ptr(ids), _i(S), _i(n_experts), _ptr(row_of_slot), _ptr(slot_of_row), at(0), at(1),
          at(1 + mt), at(1 + 2 * mt), _i(mt), _stream())


def moe_gather(x, slot_of_row, top: int, xs) -> None:
    """xs[row] = x[slot_of_row[row] // top] as bfloat16: the tokens' rows in the order of the grouped product."""
    S, width = xs.shape
    assert xs.dtype == torch.bfloat16 and x.shape[1] == width and slot_of_row.numel() == S
    _call("generic", "nncpu_moe_gather", _ptr(x), _i(_code(x)), _ptr(slot_of_row), _i(top), _ptr(xs), _i(S), _i(width), _stream())


def moe_combine(y, row_of_slot, weights, out) -> None:
    """out[t] += sum_c weights[t, c] * y[row_of_slot[t * top + c]], choices in their order; out float32."""
    n, top = weights.shape
    assert out.dtype == torch.float32 and out.shape == (n, y.shape[1]) and row_of_slot.numel() == n * top
    _call("generic", "nncpu_moe_combine", _ptr(y), _i(_code(y)), _ptr(row_of_slot), _ptr(weights), _ptr(out), _i(n), _i(top),
          _i(out.shape[1]), _stream())


def linear_tc_grouped(xs, w, out, plan, n_experts: int, workspace: GemmWorkspace, epilogue: str = "plain",
                      activation=None) -> None:
    """out[r] = xs[r] . w[e]^T for the rows r of expert e, on the tcgen05 tensor cores; xs [S, K] bfloat16 sorted by
    expert (``moe_plan``), w [E, N, K] bfloat16.  With ``epilogue="swiglu"`` every expert's rows are gate and up rows
    interleaved in blocks of 8 and out [S, N / 2] receives act(gate) * up (``activation`` as in ``linear_tc``)."""
    S, K = xs.shape
    E, N, _ = w.shape
    mt = moe_plan_tiles(S, n_experts)
    assert E == n_experts and w.shape[2] == K and xs.dtype == w.dtype == torch.bfloat16 and w.is_contiguous()
    assert out.shape == (S, N // 2 if epilogue == "swiglu" else N) and plan.numel() == 1 + 3 * mt
    base, dry = (0 if plan.is_meta else plan.data_ptr()), plan.is_meta and _dry
    at = lambda k: None if dry else _vp(base + 4 * k)
    act, a, _b = _activation(activation)
    _call("gemm_sm100", "nncpu_linear_tc_grouped", _ptr(xs), _ptr(w), _ptr(out), _i(_code(out)), _i(S), _i(N), _i(K), _i(E),
          _i(K), _i(out.shape[1]), _i(EPILOGUES[epilogue]), act, a, at(0), at(1), at(1 + mt), at(1 + 2 * mt), _i(mt),
          _ptr(workspace.status), _stream())


def xielu(x, params, out) -> None:
    """out = xIELU(x) elementwise with the two learned numbers ``params`` = (p, q): for z > 0
    softplus(p) z^2 + z/2, else (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2; computed in 32-bit."""
    assert x.shape == out.shape and params.numel() == 2 and x.is_contiguous() and out.is_contiguous()
    _call("generic", "nncpu_xielu", _ptr(x), _i(_code(x)), _ptr(params), _i(_code(params)), _ptr(out), _i(_code(out)),
          ctypes.c_long(x.numel()), _stream())


def softcap(x, cap: float) -> None:
    """x <- cap * tanh(x / cap) in place; x float32."""
    assert x.dtype == torch.float32 and x.is_contiguous()
    _call("generic", "nncpu_softcap", _ptr(x), ctypes.c_long(x.numel()), _f(cap), _stream())


def gla_decay(z, tau: float) -> None:
    """z <- sigmoid(z)^(1/tau) in place (float32): the decays of gated linear attention from their logits."""
    assert z.dtype == torch.float32 and z.is_contiguous()
    _call("recurrent", "nncpu_gla_decay", _ptr(z), ctypes.c_long(z.numel()), _f(tau), _stream())


def gla_step(proj, z, state, seq_slots, weight, eps: float, out, n_heads: int, d: int, e: int, q_scale: float,
             tau: float, head_decay=None, cos_sin=None, k_scale: float = 1.0) -> None:
    """A decode step of gated linear attention, one token per sequence: the recurrence on ``state`` (as ``gla_scan``
    with sequences of one token, ``z`` holding logits), then the heads' norm, weight and gate (as ``gla_output``),
    in one launch.  ``out`` [n, H e] in float32 or bfloat16.  ``head_decay`` (float32 [H]): one fixed decay per head
    in place of the decays from ``z`` (which may then be None); ``weight`` None: ones.  ``cos_sin`` (float32
    [n, half, 2]): q and k are rotated on the way in as ``retention_prepare`` rotates them; k is multiplied by ``k_scale``."""
    n = out.shape[0]
    assert proj.dtype == state.dtype == torch.float32 and (z is None or z.dtype == torch.float32)
    assert proj.shape == (n, 2 * n_heads * (d + e)) and out.shape == (n, n_heads * e)
    assert (z is not None and z.shape == (n, n_heads * d)) or (head_decay is not None and head_decay.dtype == torch.float32
                                                               and head_decay.numel() == n_heads)
    assert state.shape[1:] == (n_heads, d, e) and state.is_contiguous() and proj.is_contiguous()
    assert weight is None or weight.numel() == e
    assert seq_slots.dtype == torch.int32 and seq_slots.numel() >= n
    _call("recurrent", "nncpu_gla_step", _ptr(proj), _i(proj.shape[1]), _ptr(z), _ptr(state), _ptr(seq_slots),
          _ptr(weight), _i(_code(weight)), _f(eps), _ptr(out), _i(_code(out)), _i(n), _i(n_heads), _i(d), _i(e),
          _f(q_scale), _f(tau), _ptr(head_decay), _ptr(cos_sin), _i(0 if cos_sin is None else cos_sin.shape[1]),
          _f(k_scale), _stream())


def gla_scan_force_columns(cpl: int) -> None:
    """For measurements and tests: the scan runs with 2 or 4 columns of the state per lane whatever the grid's size;
    0: chosen by the grid (2, with twice the warps, where the blocks would not fill the GPU four times over)."""
    library.load("recurrent").nncpu_gla_scan_force_columns(ctypes.c_int(int(cpl)))


def gla_scan(proj, z, state, seq_slots, cu_seqlens, o, n_seqs: int, n_heads: int, d: int, e: int, q_scale: float,
             tau: float, decays_given: bool = False, head_decay=None) -> None:
    """Gated linear attention's recurrence over the step's tokens, sequence by sequence in order.  ``proj``
    float32 [n, 2 H d + 2 H e] holds q, k, v and the output gate per token, ``z`` float32 [n, H d] the decay
    logits (with ``decays_given`` the decays themselves, as ``gla_decay`` leaves them); ``state`` float32 [slots, H, d, e] is read and left updated for the slots in ``seq_slots`` (a negative
    slot: a padding sequence, zeros out); ``o`` float32 [n, H e] receives S_t^T q_t.  ``head_decay`` (float32 [H]):
    one fixed decay per head for every key channel and token; ``z`` is then not read and may be None."""
    n = o.shape[0]
    assert proj.dtype == state.dtype == o.dtype == torch.float32 and (z is None or z.dtype == torch.float32)
    assert proj.shape == (n, 2 * n_heads * (d + e)) and o.shape == (n, n_heads * e)
    assert (z is not None and z.shape == (n, n_heads * d)) or (head_decay is not None and head_decay.dtype == torch.float32
                                                               and head_decay.numel() == n_heads)
    assert state.shape[1:] == (n_heads, d, e) and state.is_contiguous() and proj.is_contiguous()
    assert seq_slots.dtype == torch.int32 and cu_seqlens.dtype == torch.int32 and cu_seqlens.numel() >= n_seqs + 1
    _call("recurrent", "nncpu_gla_scan", _ptr(proj), _i(proj.shape[1]), _ptr(z), _ptr(state), _ptr(seq_slots),
          _ptr(cu_seqlens), _ptr(o), _i(n_seqs), _i(n_heads), _i(d), _i(e), _f(q_scale), _f(tau), _i(decays_given),
          _ptr(head_decay), _stream())


OUTPUT_GATES = {"silu": 0, "sigmoid": 1}


def gla_output(o, proj, weight, eps: float, out, n_heads: int, d: int, e: int, gate_col: int = -1,
               gate: str = "silu", out_scale: float = 1.0) -> None:
    """out[t, h] = o[t, h] / rms(o[t, h]) * weight * silu(g[t, h]) with g the H e lanes of ``proj``'s rows from column
    ``gate_col`` (default: after 2 H d + H e lanes, where gated linear attention keeps them).  ``weight`` None: ones;
    ``gate`` "sigmoid": sigmoid(g) in place of silu(g); the whole times ``out_scale``."""
    n = o.shape[0]
    assert o.dtype == proj.dtype == torch.float32 and o.shape == (n, n_heads * e) and out.shape == o.shape
    assert weight is None or weight.numel() == e
    _call("recurrent", "nncpu_gla_output", _ptr(o), _ptr(proj), _i(proj.shape[1]),
          _i(gate_col if gate_col >= 0 else 2 * n_heads * d + n_heads * e),
          _ptr(weight), _i(_code(weight)), _f(eps), _ptr(out), _i(_code(out)), _i(n), _i(n_heads), _i(e),
          _i(OUTPUT_GATES[gate]), _f(out_scale), _stream())


def retention_prepare(proj, cos_sin, n_heads: int, d: int, k_scale: float) -> None:
    """In place on ``proj`` float32 [n, >= 2 H d], whose rows begin with q (H d) and k (H d): both are rotated by the
    token's position (``cos_sin`` float32 [n, half, 2]: the pairs (i, i + half) of a head's first 2 half lanes; None:
    no rotation), then k is multiplied by ``k_scale``.  What retention's recurrence reads."""
    n = proj.shape[0]
    half = 0 if cos_sin is None else cos_sin.shape[1]
    assert proj.dtype == torch.float32 and proj.is_contiguous() and proj.shape[1] >= 2 * n_heads * d
    assert cos_sin is None or (cos_sin.dtype == torch.float32 and cos_sin.shape == (n, half, 2) and cos_sin.is_contiguous())
    _call("recurrent", "nncpu_retention_prepare", _ptr(proj), _i(proj.shape[1]), _ptr(cos_sin), _i(half), _i(n),
          _i(n_heads), _i(d), _f(k_scale), _stream())


def delta_prepare(proj, conv_w, state, conv_col: int, tok_seq, seq_slots, cu_seqlens, a_log, dt_bias, xc, gb, n_seqs: int,
                  n_heads: int, n_kv: int, d: int, e: int, taps: int, one_token_each: bool = False, beta_col: int = -1,
                  chan_z=None) -> None:
    """What the gated delta rule's recurrence reads, from the projections: ``proj`` float32 [n, >= C + H e + 2 H] holds
    per token q (G d), k (G d), v (H e) (the C channels of the short convolutions), the output gate's logits (H e), the
    logits of beta (H) and the decays' inputs (H).  ``xc`` float32 [n, C] receives silu(conv(.)) with q and k made unit
    vectors per head (q also times d^-1/2), ``gb`` float32 [n, 2 H] the decays exp(-exp(A_log) softplus(a + dt_bias))
    and then beta = sigmoid(b).  ``conv_w`` [C, taps]; ``state`` float32 [slots, L] holds from lane ``conv_col`` of a
    slot's row [taps - 1, C]: the sequence's last inputs; it is left advanced by the step's tokens.
    ``one_token_each``: every sequence of the step brings exactly one token (the kept inputs then advance inside the one
    kernel; otherwise a second kernel advances them after all tokens have read them).
    ``beta_col``: the column of ``proj`` where beta's logits start (default C + H e; the decays' inputs follow them).
    ``chan_z`` float32 [n, H d]: a decay per head and key channel; it holds softplus's argument (bias included) and
    receives exp(-exp(A_log_h) softplus(.)) in place; ``proj`` then has no decay inputs, ``dt_bias`` is not read and
    ``gb``'s decays are ones."""
    n = xc.shape[0]
    C = 2 * n_kv * d + n_heads * e
    if beta_col < 0:
        beta_col = C + n_heads * e
    assert proj.dtype == xc.dtype == gb.dtype == state.dtype == torch.float32 and proj.is_contiguous()
    assert proj.shape[0] == n and proj.shape[1] >= beta_col + (1 if chan_z is not None else 2) * n_heads and xc.shape == (n, C)
    assert chan_z is None or (chan_z.dtype == torch.float32 and chan_z.shape == (n, n_heads * d) and chan_z.is_contiguous())
    assert gb.shape == (n, 2 * n_heads) and conv_w.shape == (C, taps) and conv_w.is_contiguous()
    assert state.dim() == 2 and state.shape[1] >= conv_col + (taps - 1) * C and state.is_contiguous()
    assert a_log.numel() == n_heads and (chan_z is not None or (dt_bias.numel() == n_heads and a_log.dtype == dt_bias.dtype))
    assert tok_seq.dtype == seq_slots.dtype == cu_seqlens.dtype == torch.int32 and cu_seqlens.numel() >= n_seqs + 1
    _call("recurrent", "nncpu_delta_prepare", _ptr(proj), _i(proj.shape[1]), _ptr(conv_w), _i(_code(conv_w)),
          None if (state.is_meta and _dry) else _vp(state.data_ptr() + 4 * conv_col), _l(state.shape[1]), _ptr(tok_seq), _ptr(seq_slots), _ptr(cu_seqlens), _ptr(a_log),
          _ptr(dt_bias), _i(_code(a_log)),
          _ptr(xc), _ptr(gb), _i(n), _i(n_seqs), _i(n_heads), _i(n_kv), _i(d), _i(e), _i(taps), _f(d ** -0.5),
          _i(one_token_each), _i(beta_col), _ptr(chan_z), _stream())


def delta_scan_force(lanes: int = 0, columns: int = 0) -> None:
    """For measurements: the delta rule's scan runs with ``lanes`` lanes a column (a power of two from 4 to 32, before
    the doubling that goes with two columns a lane) and 1 or 2 ``columns`` a lane, whatever the layer's sizes; 0: by the
    launcher's rule."""
    lib = library.load("recurrent")
    lib.nncpu_delta_scan_force_lanes(ctypes.c_int(int(lanes)))
    lib.nncpu_delta_scan_force_columns(ctypes.c_int(int(columns)))


def delta_scan(xc, gb, state, seq_slots, cu_seqlens, o, n_seqs: int, n_heads: int, n_kv: int, d: int, e: int,
               chan_g=None) -> None:
    """The gated delta rule over the step's tokens, sequence by sequence in order: per head S <- g S;
    u = beta (v - S^T k); S <- S + k u^T; o = S^T q, with q, k, v from ``xc`` and g, beta from ``gb`` as
    ``delta_prepare`` leaves them.  ``state`` float32 [slots, >= H d e] (a slot's [H, d, e] in the first lanes of its
    row) is read and left updated for the slots in
    ``seq_slots`` (negative: a padding sequence, zeros out); ``o`` float32 [n, H e].  ``chan_g`` float32 [n, H d]: a
    decay per head and key channel, S <- diag(g) S, in place of ``gb``'s one per head."""
    n = o.shape[0]
    assert chan_g is None or (chan_g.dtype == torch.float32 and chan_g.shape == (n, n_heads * d) and chan_g.is_contiguous())
    assert xc.dtype == gb.dtype == state.dtype == o.dtype == torch.float32
    assert xc.shape == (n, 2 * n_kv * d + n_heads * e) and gb.shape == (n, 2 * n_heads) and o.shape == (n, n_heads * e)
    assert state.dim() == 2 and state.shape[1] >= n_heads * d * e and state.is_contiguous()
    assert xc.is_contiguous() and gb.is_contiguous()
    assert seq_slots.dtype == torch.int32 and cu_seqlens.dtype == torch.int32 and cu_seqlens.numel() >= n_seqs + 1
    _call("recurrent", "nncpu_delta_scan", _ptr(xc), _ptr(gb), _ptr(chan_g), _ptr(state), _l(state.shape[1]), _ptr(seq_slots), _ptr(cu_seqlens), _ptr(o),
          _i(n_seqs), _i(n_heads), _i(n_kv), _i(d), _i(e), _stream())


def gather_rows(x, rows, out) -> None:
    n, dim = out.shape
    assert x.dtype == torch.float32 and out.dtype == torch.float32 and rows.dtype == torch.int32
    _call("generic", "nncpu_gather_rows", _ptr(x), _ptr(rows), _ptr(out), _i(n), _i(dim), _stream())


def argmax(logits, out) -> None:
    """out[r] = the first largest of logits[r]; logits float32 [n, vocab], out int32 [n]."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.numel() >= n
    lib = library.load("generic")
    lib.nncpu_argmax_scratch_bytes.restype = ctypes.c_long
    need = lib.nncpu_argmax_scratch_bytes(_i(n), _i(vocab))      # long rows are searched in chunks
    scratch = torch.empty(need, dtype=torch.uint8, device=logits.device) if need else None
    _call("generic", "nncpu_argmax", _ptr(logits), _ptr(out), _i(n), _i(vocab), _ptr(scratch), ctypes.c_long(need),
          _stream())


def topk(logits, vals, ids) -> None:
    """The k = vals.shape[1] best entries of every row by (logit descending, id
    ascending), NaN as -inf, in no particular order: vals float32 [n, k], ids int32 [n, k]."""
    n, vocab = logits.shape
    k = vals.shape[1]
    assert logits.dtype == torch.float32 and vals.dtype == torch.float32 and ids.dtype == torch.int32
    assert vals.shape == (n, k) and ids.shape == (n, k)
    _call("generic", "nncpu_topk", _ptr(logits), _ptr(vals), _ptr(ids), _i(n), _i(vocab), _i(k), _stream())


def sample_chain(logits, u, out, top_k: int, temperature: float, top_p: float, min_p: float) -> None:
    """The whole chain on the device for 0 < top_k <= 1024: out[r] = the token drawn from row r with the
    uniform u[r] (float64 in [0, 1)) after top-k, top-p, min-p and temperature, in rank order."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and u.dtype == torch.float64 and out.dtype == torch.int32
    assert u.numel() >= n and out.numel() >= n
    lib = library.load("generic")
    lib.nncpu_sample_chain_scratch_bytes.restype = ctypes.c_long
    need = lib.nncpu_sample_chain_scratch_bytes(_i(n), _i(vocab))   # long rows: candidates found by the whole GPU
    scratch = torch.empty(need, dtype=torch.uint8, device=logits.device) if need else None
    _call("generic", "nncpu_sample_chain", _ptr(logits), _ptr(u), _ptr(out), _i(n), _i(vocab), _i(top_k),
          _f(temperature), _f(top_p), _f(min_p), _ptr(scratch), ctypes.c_long(need), _stream())


def row_exp_sum(logits, out) -> None:
    """out[r] (float64) = sum over the row of exp(logit - the row's largest logit), NaN as -inf."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.float64 and out.shape == (n,)
    _call("generic", "nncpu_row_exp_sum", _ptr(logits), _ptr(out), _i(n), _i(vocab), _stream())


def sample_temperature(logits, uniforms, out, temperature: float) -> None:
    """One draw per row at ``temperature`` over the whole vocabulary in id
    order; uniforms float64 [n] in [0, 1)."""
    n, vocab = logits.shape
    assert logits.dtype == torch.float32 and uniforms.dtype == torch.float64 and out.dtype == torch.int32
    lib = library.load("generic")
    lib.nncpu_sample_temperature_scratch_bytes.restype = ctypes.c_long
    need = lib.nncpu_sample_temperature_scratch_bytes(_i(n), _i(vocab))   # long rows are summed in chunks
    scratch = torch.empty(need, dtype=torch.uint8, device=logits.device) if need else None
    _call("generic", "nncpu_sample_temperature", _ptr(logits), _ptr(uniforms), _ptr(out), _i(n), _i(vocab),
          _f(temperature), _ptr(scratch), ctypes.c_long(need), _stream())
