// Kernels that take every size and both element types (float and bfloat16,
// chosen per tensor at run time) and compute in 32-bit: the whole float32 path
// of the model runs on them, and the bfloat16 path uses them wherever no
// specialised kernel applies.  Plain CUDA cores, no reduced-precision matrix
// mode anywhere in this file.
//
// The arithmetic follows ZacWalk/nncpu's scalar kernels:
//   RMSNorm            crates/nncpu/src/kernels/scalar.rs:270-292
//   rotary embedding   crates/nncpu/src/kernels/mod.rs:687-737
//   attention          crates/nncpu/src/kernels/scalar.rs:444-548 (online softmax, scale after the dot)
//   SiLU gate          crates/nncpu/src/kernels/scalar.rs:102-106,146-150
//   argmax             crates/nncpu/src/model/forward.rs:1003-1011 (first largest)
//   temperature draw   crates/nncpu/src/session/sample.rs:186-200

#include <math.h>

#define NN_LIB generic
#define NN_LAUNCH_OVERLAP
#include "common.cuh"

// ---------------------------------------------------------------------------
// Embedding rows: out[t, :] = table[ids[t], :] * scale, float32 out.
// A negative id (a padded row) gives zeros.  With a table of learned position
// vectors, out[t, :] += pos_table[pos[t], :] (not scaled); a position beyond
// the table gives NaN rows, which nobody can mistake for a result.
// ---------------------------------------------------------------------------
__global__ void embed_kernel(const void* __restrict__ table, int table_dt, const int* __restrict__ ids,
                             float* __restrict__ out, int hidden, float scale, const void* __restrict__ pos_table,
                             int pos_dt, const int* __restrict__ pos, int n_pos) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const int p = pos_table != nullptr ? pos[t] : 0;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = 0.0f;
        if (id >= 0) {
            v = ld_f(table, (size_t)id * hidden + i, table_dt) * scale;
            if (pos_table != nullptr)
                v = (p >= 0 && p < n_pos) ? v + ld_f(pos_table, (size_t)p * hidden + i, pos_dt) : __int_as_float(0x7FC00000);
        }
        out[(size_t)t * hidden + i] = v;
    }
}

extern "C" int nncpu_embed(const void* table, int table_dt, const int* ids, float* out, int n_tok, int hidden,
                           int vocab, float scale, const void* pos_table, int pos_dt, const int* pos, int n_pos,
                           void* stream) {
    NN_CHECK(n_tok >= 0 && hidden > 0 && vocab > 0, "embed: n_tok %d, hidden %d, vocab %d", n_tok, hidden, vocab);
    NN_CHECK(pos_table == nullptr || (pos != nullptr && n_pos > 0), "embed: a position table without positions");
    if (n_tok == 0) return 0;
    embed_kernel<<<n_tok, 256, 0, (cudaStream_t)stream>>>(table, table_dt, ids, out, hidden, scale, pos_table, pos_dt,
                                                          pos, n_pos);
    NN_LAUNCH_OK("embed");
    return 0;
}

// ---------------------------------------------------------------------------
// RMSNorm over the last axis: y = (x * scale) * (gamma + gamma_offset),
// scale = 1 / sqrt(mean(x^2) + eps).  `rows` (optional) picks input rows, so
// the final norm runs only on the rows whose logits are wanted.  gamma_offset
// is 1 for weights that are stored around zero.  With `accumulate` the result
// is added to y (a norm that closes a sublayer: y is the residual stream).
// ---------------------------------------------------------------------------
__global__ void rmsnorm_kernel(const void* __restrict__ x, int x_dt, const void* __restrict__ gamma, int g_dt,
                               void* __restrict__ y, int y_dt, const int* __restrict__ rows, int dim, float eps,
                               float gamma_offset, int accumulate) {
    __shared__ float scratch[33];
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    if (r_in < 0) {
        if (!accumulate)
            for (int i = threadIdx.x; i < dim; i += blockDim.x) st_f(y, (size_t)r_out * dim + i, y_dt, 0.0f);
        return;
    }
    const size_t base = (size_t)r_in * dim;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = ld_f(x, base + i, x_dt);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss * (1.0f / (float)dim) + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = ld_f(x, base + i, x_dt) * scale;
        if (gamma) v *= ld_f(gamma, i, g_dt) + gamma_offset;
        const size_t at = (size_t)r_out * dim + i;
        st_f(y, at, y_dt, accumulate ? ld_f(y, at, y_dt) + v : v);
    }
}

// The common case, float32 rows of a width that is a multiple of 4 and at most 256 * 4 * kVec: every
// thread keeps its part of the row in registers between the sum of squares and the scaling, so the
// row is read once, 16 bytes at a time.
template <int kVec>
__global__ void __launch_bounds__(256)
rmsnorm_f32_kernel(const float* __restrict__ x, const void* __restrict__ gamma, int g_dt, void* __restrict__ y,
                   int y_dt, const int* __restrict__ rows, int dim, float eps, float gamma_offset, int accumulate) {
    __shared__ float scratch[33];
    // launched to start while the kernel before it ends: the product that follows may set itself up meanwhile
    let_next_kernel_start();
    wait_for_previous_kernels();
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    const int n4 = dim >> 2;
    float4 v[kVec];
    float ss = 0.0f;
    if (r_in >= 0) {
        const float4* src = reinterpret_cast<const float4*>(x + (size_t)r_in * dim);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
            const int i = threadIdx.x + j * 256;
            v[j] = i < n4 ? src[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
            ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    } else {
#pragma unroll
        for (int j = 0; j < kVec; ++j) v[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    ss = block_sum(ss, scratch);
    const float scale = r_in >= 0 ? 1.0f / sqrtf(ss * (1.0f / (float)dim) + eps) : 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        float o[4] = {v[j].x * scale, v[j].y * scale, v[j].z * scale, v[j].w * scale};
        if (gamma) {
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] *= ld_f(gamma, 4 * i + e, g_dt) + gamma_offset;
        }
        const size_t at = (size_t)r_out * dim + 4 * i;
        if (accumulate) {          // float32 y (checked by the launcher): the norm is added to what y holds
            if (r_in < 0) continue;
            const float4 was = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(y) + at);
            o[0] += was.x; o[1] += was.y; o[2] += was.z; o[3] += was.w;
        }
        if (y_dt == DT_BF16) {
            __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + at) = *reinterpret_cast<uint2*>(h);
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + at) = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

extern "C" int nncpu_rmsnorm(const void* x, int x_dt, const void* gamma, int g_dt, void* y, int y_dt,
                             const int* rows, int n_rows, int dim, float eps, float gamma_offset, int accumulate,
                             void* stream) {
    NN_CHECK(n_rows >= 0 && dim > 0, "rmsnorm: %d rows of %d", n_rows, dim);
    NN_CHECK(!accumulate || x != y, "rmsnorm: a norm cannot be added to its own input");
    if (n_rows == 0) return 0;
    if ((!accumulate || y_dt == DT_F32) && x_dt == DT_F32 && dim % 4 == 0 && dim >= 1024 && dim <= 256 * 4 * 8 && (uintptr_t)x % 16 == 0 &&
        (uintptr_t)y % 16 == 0) {
        const float* xf = (const float*)x;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)n_rows);
        cfg.blockDim = dim3(256);
        cfg.stream = (cudaStream_t)stream;
        cudaLaunchAttribute attr[1];
        cfg.attrs = attr;
        cfg.numAttrs = overlap_attribute(attr);
        const auto kernel = dim <= 256 * 4 * 2 ? rmsnorm_f32_kernel<2> : dim <= 256 * 4 * 4 ? rmsnorm_f32_kernel<4> : rmsnorm_f32_kernel<8>;
        const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, xf, gamma, g_dt, y, y_dt, rows, dim, eps, gamma_offset,
                                                 accumulate);
        NN_CHECK(e == cudaSuccess, "rmsnorm: launch failed: %s", cudaGetErrorString(e));
        return 0;
    }
    int threads = dim >= 2048 ? 512 : (dim >= 512 ? 256 : (dim >= 128 ? 128 : 32));
    rmsnorm_kernel<<<n_rows, threads, 0, (cudaStream_t)stream>>>(x, x_dt, gamma, g_dt, y, y_dt, rows, dim, eps,
                                                                 gamma_offset, accumulate);
    NN_LAUNCH_OK("rmsnorm");
    return 0;
}

// ---------------------------------------------------------------------------
// The two norms that meet between two sublayers of a "sandwich" layer, in one pass:
//     r <- r + norm(b) * (g1 + off1)      (the norm that closes a sublayer, added to the residual stream r)
//     y  = norm(r) * (g2 + off2)          (the norm that opens the next sublayer)
// b and r are float32 rows of `dim`; a thread keeps its part of the row in registers between the two sums, so
// b and r are read once and r and y written once.  dim <= 256 * 4 * kVec, a multiple of 4.
// ---------------------------------------------------------------------------
template <int kVec>
__global__ void __launch_bounds__(256)
rmsnorm_pair_kernel(const float* __restrict__ b, float* __restrict__ r, const void* __restrict__ g1, float off1,
                    const void* __restrict__ g2, float off2, int g_dt, void* __restrict__ y, int y_dt, int dim,
                    float eps1, float eps2) {
    __shared__ float scratch[33];
    const int row = blockIdx.x, n4 = dim >> 2;
    float4 v[kVec];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < n4 ? reinterpret_cast<const float4*>(b + (size_t)row * dim)[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float s1 = 1.0f / sqrtf(ss * (1.0f / (float)dim) + eps1);
    float ss2 = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        float4* at = reinterpret_cast<float4*>(r + (size_t)row * dim) + i;
        const float4 was = *at;
        float o[4] = {v[j].x * s1, v[j].y * s1, v[j].z * s1, v[j].w * s1};
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] *= ld_f(g1, 4 * i + e, g_dt) + off1;
        v[j] = make_float4(was.x + o[0], was.y + o[1], was.z + o[2], was.w + o[3]);
        *at = v[j];
        ss2 = fmaf(v[j].x, v[j].x, ss2); ss2 = fmaf(v[j].y, v[j].y, ss2);
        ss2 = fmaf(v[j].z, v[j].z, ss2); ss2 = fmaf(v[j].w, v[j].w, ss2);
    }
    ss2 = block_sum(ss2, scratch);
    const float s2 = 1.0f / sqrtf(ss2 * (1.0f / (float)dim) + eps2);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        float o[4] = {v[j].x * s2, v[j].y * s2, v[j].z * s2, v[j].w * s2};
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] *= ld_f(g2, 4 * i + e, g_dt) + off2;
        const size_t at = (size_t)row * dim + 4 * i;
        if (y_dt == DT_BF16) {
            __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + at) = *reinterpret_cast<uint2*>(h);
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + at) = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

extern "C" int nncpu_rmsnorm_pair_supported(int dim) { return dim > 0 && dim % 4 == 0 && dim <= 256 * 4 * 8; }

extern "C" int nncpu_rmsnorm_pair(const float* b, float* r, const void* g1, float off1, float eps1, const void* g2,
                                  float off2, float eps2, int g_dt, void* y, int y_dt, int n_rows, int dim, void* stream) {
    NN_CHECK(n_rows >= 0 && nncpu_rmsnorm_pair_supported(dim), "rmsnorm_pair: %d rows of %d", n_rows, dim);
    NN_CHECK((uintptr_t)b % 16 == 0 && (uintptr_t)r % 16 == 0 && (uintptr_t)y % 16 == 0 && b != r,
             "rmsnorm_pair: rows must be 16-byte aligned and the branch must not be the stream");
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dim <= 256 * 4) rmsnorm_pair_kernel<1><<<n_rows, 256, 0, st>>>(b, r, g1, off1, g2, off2, g_dt, y, y_dt, dim, eps1, eps2);
    else if (dim <= 256 * 4 * 2) rmsnorm_pair_kernel<2><<<n_rows, 256, 0, st>>>(b, r, g1, off1, g2, off2, g_dt, y, y_dt, dim, eps1, eps2);
    else if (dim <= 256 * 4 * 4) rmsnorm_pair_kernel<4><<<n_rows, 256, 0, st>>>(b, r, g1, off1, g2, off2, g_dt, y, y_dt, dim, eps1, eps2);
    else rmsnorm_pair_kernel<8><<<n_rows, 256, 0, st>>>(b, r, g1, off1, g2, off2, g_dt, y, y_dt, dim, eps1, eps2);
    NN_LAUNCH_OK("rmsnorm_pair");
    return 0;
}

// ---------------------------------------------------------------------------
// C[M, N] (+)= A[M, K] . W[N, K]^T + bias[N], 32-bit multiply-add on CUDA
// cores.  Each output element is summed over k in ascending order by one
// thread, so a row's result does not depend on which other rows are present.
// ---------------------------------------------------------------------------
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
linear_simt_kernel(const void* __restrict__ A, int a_dt, const void* __restrict__ W, int w_dt,
                   const void* __restrict__ bias, int b_dt, void* __restrict__ C, int c_dt, int M, int N, int K,
                   int lda, int ldc, int accumulate) {
    constexpr int NT = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += NT) {
            const int r = e / BK, c = e % BK;
            const int m = m0 + r, k = k0 + c;
            As[c][r] = (m < M && k < K) ? ld_f(A, (size_t)m * lda + k, a_dt) : 0.0f;
        }
        for (int e = tid; e < BN * BK; e += NT) {
            const int r = e / BK, c = e % BK;
            const int n = n0 + r, k = k0 + c;
            Ws[c][r] = (n < N && k < K) ? ld_f(W, (size_t)n * K + k, w_dt) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += ld_f(bias, n, b_dt);
            const size_t o = (size_t)m * ldc + n;
            if (accumulate) v += ld_f(C, o, c_dt);
            st_f(C, o, c_dt, v);
        }
    }
}

extern "C" int nncpu_linear_simt(const void* A, int a_dt, const void* W, int w_dt, const void* bias, int b_dt,
                                 void* C, int c_dt, int M, int N, int K, int lda, int ldc, int accumulate,
                                 void* stream) {
    NN_CHECK(M >= 0 && N > 0 && K > 0 && lda >= K && ldc >= N, "linear: M %d, N %d, K %d, lda %d, ldc %d", M, N,
             K, lda, ldc);
    if (M == 0) return 0;
    if (M <= 16) {
        dim3 grid((N + 63) / 64, (M + 15) / 16);
        linear_simt_kernel<16, 64, 32, 2, 2><<<grid, 256, 0, (cudaStream_t)stream>>>(
            A, a_dt, W, w_dt, bias, b_dt, C, c_dt, M, N, K, lda, ldc, accumulate);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64);
        linear_simt_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, (cudaStream_t)stream>>>(
            A, a_dt, W, w_dt, bias, b_dt, C, c_dt, M, N, K, lda, ldc, accumulate);
    }
    NN_LAUNCH_OK("linear");
    return 0;
}

// ---------------------------------------------------------------------------
// Rotation table of a step: cs[t, i] = stretch * (cos, sin)(float(pos_t) * pos_scale * inv_freq[i]), or with
// by_pair the same values laid out [i, t] for readers whose lanes are tokens.
// Computed once per step and read by every layer that shares the encoding.
// ---------------------------------------------------------------------------
__global__ void rope_table_kernel(const int* __restrict__ pos, const float* __restrict__ inv_freq,
                                  float2* __restrict__ cs, int n_tok, int half, float pos_scale, int by_pair,
                                  float stretch) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tok * half) return;
    const int t = by_pair ? idx % n_tok : idx / half, i = by_pair ? idx / n_tok : idx % half;
    const float theta = ((float)pos[t] * pos_scale) * inv_freq[i];
    float s, c;
    sincosf(theta, &s, &c);
    cs[idx] = stretch == 1.0f ? make_float2(c, s) : make_float2(c * stretch, s * stretch);
}

extern "C" int nncpu_rope_table(const int* pos, const float* inv_freq, float* cs, int n_tok, int half,
                                float pos_scale, int by_pair, float stretch, void* stream) {
    NN_CHECK(n_tok >= 0 && half > 0, "rope_table: %d tokens, %d pairs", n_tok, half);
    if (n_tok == 0) return 0;
    const int total = n_tok * half;
    NN_CHECK((uintptr_t)cs % 8 == 0, "rope_table: the table must be 8-byte aligned (it is written as cos/sin pairs)");
    rope_table_kernel<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>(pos, inv_freq, (float2*)cs, n_tok,
                                                                             half, pos_scale, by_pair, stretch);
    NN_LAUNCH_OK("rope_table");
    return 0;
}

// ---------------------------------------------------------------------------
// Per-head q/k RMSNorm, rotation, and the append of k and v to the cache.
// qkv [n_tok, (n_heads + n_kv) * hd + n_kv * vd] holds q heads, then k heads,
// then v heads (of vd lanes each).  One warp per (token, head).  q goes to
// q_out [n_tok, n_heads * hd]; k (normed, rotated) and v (raw) go to their page
// rows.  With n_kv == 0 the mixer reads another layer's cache and only q is
// processed.  A query temperature (temp_coef != 0) multiplies the query at
// position p by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1).
// With v_from_k the rows hold no v heads: a value head is the key head of the
// same number as projected (raw), and vd == hd.  A row is ld elements long
// (it may hold more than the heads: a gate's logits after them).
// ---------------------------------------------------------------------------
__global__ void qk_norm_rope_append_kernel(const void* __restrict__ qkv, int in_dt, const void* __restrict__ q_gamma,
                                           const void* __restrict__ k_gamma, int g_dt, float eps,
                                           const float2* __restrict__ cs, int rot_half,
                                           const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                           const int* __restrict__ block_table, int bt_stride,
                                           void* __restrict__ k_pages, void* __restrict__ v_pages, int kv_dt,
                                           void* __restrict__ q_out, int q_dt, int n_tok, int n_heads, int n_kv,
                                           int hd, int vd, float temp_coef, int temp_every, int ld, int v_from_k) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tok = n_heads + 2 * n_kv;
    const long item = (long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (long)n_tok * per_tok) return;
    const int t = (int)(item / per_tok), h = (int)(item % per_tok);
    const int seq = tok_seq[t];
    const bool is_q = h < n_heads, is_k = !is_q && h < n_heads + n_kv;
    const int len = (is_q || is_k) ? hd : vd;
    const size_t row = (size_t)ld;
    float* x = smem + warp * max(hd, vd);
    const size_t in_base = (size_t)t * row + ((is_q || is_k) ? (size_t)h * hd
                                                              : v_from_k ? (size_t)(h - n_kv) * hd
                                                              : (size_t)(n_heads + n_kv) * hd + (size_t)(h - n_heads - n_kv) * vd);
    const void* gamma = is_q ? q_gamma : (is_k ? k_gamma : nullptr);

    float ss = 0.0f;
    for (int i = lane; i < len; i += 32) {
        const float v = ld_f(qkv, in_base + i, in_dt);
        x[i] = v;
        ss = fmaf(v, v, ss);
    }
    if (gamma) {
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss * (1.0f / (float)hd) + eps);
        for (int i = lane; i < hd; i += 32) x[i] = (x[i] * scale) * ld_f(gamma, i, g_dt);
    }
    __syncwarp();
    if ((is_q || is_k) && cs != nullptr) {
        for (int i = lane; i < rot_half; i += 32) {
            const float2 c = cs[(size_t)t * rot_half + i];
            const float a = x[i], b = x[i + rot_half];
            x[i] = c.x * a - c.y * b;
            x[i + rot_half] = c.y * a + c.x * b;
        }
        __syncwarp();
    }
    if (is_q) {
        float temp = 1.0f;
        if (temp_coef != 0.0f) temp = 1.0f + temp_coef * logf((float)((tok_pos[t] + 1) / temp_every) + 1.0f);
        const size_t o = (size_t)t * n_heads * hd + (size_t)h * hd;
        for (int i = lane; i < hd; i += 32) st_f(q_out, o + i, q_dt, x[i] * temp);
        return;
    }
    if (seq < 0) return;  // a padded row owns no place in the cache
    const int pos = tok_pos[t];
    const int page = block_table[(size_t)seq * bt_stride + pos / kPage];
    if (page < 0) return;
    const int kvh = is_k ? h - n_heads : h - n_heads - n_kv;
    const size_t o = (((size_t)page * n_kv + kvh) * kPage + pos % kPage) * len;
    void* dst = is_k ? k_pages : v_pages;
    for (int i = lane; i < len; i += 32) st_f(dst, o + i, kv_dt, x[i]);
}

// The bfloat16 run's case: float32 projections in, bfloat16 q and cache out, the whole head rotated,
// head size 64 or 128.  A lane holds EPL = hd / 32 neighbouring lanes of the head, so lanes 0-15 hold
// the first half and lanes 16-31 the second: a rotation pair sits in lanes i and i + 16.
template <int EPL>
__global__ void __launch_bounds__(256)
qk_norm_rope_append_fast_kernel(const float* __restrict__ qkv, const void* __restrict__ q_gamma,
                                const void* __restrict__ k_gamma, int g_dt, float eps, const float2* __restrict__ cs,
                                const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                                const int* __restrict__ block_table, int bt_stride, __nv_bfloat16* __restrict__ k_pages,
                                __nv_bfloat16* __restrict__ v_pages, __nv_bfloat16* __restrict__ q_out, int n_tok,
                                int n_heads, int n_kv, float temp_coef, int temp_every, int ld, int v_from_k) {
    constexpr int hd = 32 * EPL, half = hd / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_tok = n_heads + 2 * n_kv;
    const long item = (long)blockIdx.x * 8 + warp;
    if (item >= (long)n_tok * per_tok) return;
    const int t = (int)(item / per_tok), h = (int)(item % per_tok);
    const bool is_q = h < n_heads, is_k = !is_q && h < n_heads + n_kv;
    const float* src = qkv + (size_t)t * ld + (size_t)((!is_q && !is_k && v_from_k) ? h - n_kv : h) * hd + lane * EPL;
    float x[EPL];
    if (EPL == 4) {
        const float4 v = *reinterpret_cast<const float4*>(src);
        x[0] = v.x; x[1] = v.y; x[2 % EPL] = v.z; x[3 % EPL] = v.w;
    } else {
        const float2 v = *reinterpret_cast<const float2*>(src);
        x[0] = v.x; x[1] = v.y;
    }
    const void* gamma = is_q ? q_gamma : (is_k ? k_gamma : nullptr);
    if (gamma) {
        float ss = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) ss = fmaf(x[e], x[e], ss);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss * (1.0f / (float)hd) + eps);
#pragma unroll
        for (int e = 0; e < EPL; ++e) x[e] = (x[e] * scale) * ld_f(gamma, lane * EPL + e, g_dt);
    }
    if ((is_q || is_k) && cs != nullptr) {
        const int i0 = (lane & 15) * EPL;   // index of the rotation pair
#pragma unroll
        for (int e = 0; e < EPL; ++e) {
            const float other = __shfl_xor_sync(0xffffffffu, x[e], 16);
            const float2 c = cs[(size_t)t * half + i0 + e];
            x[e] = lane < 16 ? c.x * x[e] - c.y * other : c.y * other + c.x * x[e];
        }
    }
    __nv_bfloat16* dst;
    if (is_q) {
        if (temp_coef != 0.0f) {       // the query temperature of the token's position
            const float temp = 1.0f + temp_coef * logf((float)((tok_pos[t] + 1) / temp_every) + 1.0f);
#pragma unroll
            for (int e = 0; e < EPL; ++e) x[e] *= temp;
        }
        dst = q_out + ((size_t)t * n_heads + h) * hd;
    } else {
        const int seq = tok_seq[t];
        if (seq < 0) return;
        const int pos = tok_pos[t];
        const int page = block_table[(size_t)seq * bt_stride + pos / kPage];
        if (page < 0) return;
        const int kvh = is_k ? h - n_heads : h - n_heads - n_kv;
        dst = (is_k ? k_pages : v_pages) + (((size_t)page * n_kv + kvh) * kPage + pos % kPage) * hd;
    }
    if (EPL == 4) {
        __nv_bfloat162 o[2] = {__floats2bfloat162_rn(x[0], x[1]), __floats2bfloat162_rn(x[2 % EPL], x[3 % EPL])};
        *reinterpret_cast<uint2*>(dst + lane * 4) = *reinterpret_cast<uint2*>(o);
    } else {
        *reinterpret_cast<__nv_bfloat162*>(dst + lane * 2) = __floats2bfloat162_rn(x[0], x[1]);
    }
}

extern "C" int nncpu_qk_norm_rope_append(const void* qkv, int in_dt, const void* q_gamma, const void* k_gamma,
                                         int g_dt, float eps, const float* cs, int rot_half, const int* tok_seq,
                                         const int* tok_pos, const int* block_table, int bt_stride, void* k_pages,
                                         void* v_pages, int kv_dt, void* q_out, int q_dt, int n_tok, int n_heads,
                                         int n_kv, int hd, int vd, float temp_coef, int temp_every, int ld, int v_from_k,
                                         void* stream) {
    NN_CHECK(n_tok >= 0 && n_heads > 0 && n_kv >= 0 && hd > 0 && vd > 0, "qk_norm_rope_append: sizes");
    NN_CHECK(!v_from_k || vd == hd, "qk_norm_rope_append: values that are the keys have the keys' size, not %d", vd);
    NN_CHECK(ld >= (n_heads + n_kv) * hd + (v_from_k ? 0 : n_kv * vd), "qk_norm_rope_append: rows of %d elements", ld);
    NN_CHECK(vd <= 1024, "qk_norm_rope_append: value size %d is above 1024", vd);
    NN_CHECK(temp_coef == 0.0f || temp_every > 0, "qk_norm_rope_append: a query temperature every %d positions", temp_every);
    NN_CHECK((cs == nullptr || hd % 2 == 0) && 2 * rot_half <= hd, "qk_norm_rope_append: head size %d with %d rotated pairs", hd,
             rot_half);
    NN_CHECK((uintptr_t)cs % 8 == 0, "qk_norm_rope_append: the rotation table must be 8-byte aligned (cos/sin pairs)");
    NN_CHECK(hd <= 1024, "qk_norm_rope_append: head size %d is above 1024", hd);
    if (n_tok == 0) return 0;
    if (in_dt == DT_F32 && q_dt == DT_BF16 && (n_kv == 0 || kv_dt == DT_BF16) && (hd == 64 || hd == 128) && vd == hd &&
        (cs == nullptr || 2 * rot_half == hd) && (uintptr_t)qkv % 16 == 0 && (uintptr_t)q_out % 16 == 0 && ld % 4 == 0) {
        const long n_items = (long)n_tok * (n_heads + 2 * n_kv);
        const unsigned n_blocks = (unsigned)((n_items + 7) / 8);
        if (hd == 128)
            qk_norm_rope_append_fast_kernel<4><<<n_blocks, 256, 0, (cudaStream_t)stream>>>(
                (const float*)qkv, q_gamma, k_gamma, g_dt, eps, (const float2*)cs, tok_seq, tok_pos, block_table,
                bt_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)q_out, n_tok, n_heads, n_kv,
                temp_coef, temp_every, ld, v_from_k);
        else
            qk_norm_rope_append_fast_kernel<2><<<n_blocks, 256, 0, (cudaStream_t)stream>>>(
                (const float*)qkv, q_gamma, k_gamma, g_dt, eps, (const float2*)cs, tok_seq, tok_pos, block_table,
                bt_stride, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, (__nv_bfloat16*)q_out, n_tok, n_heads, n_kv,
                temp_coef, temp_every, ld, v_from_k);
        NN_LAUNCH_OK("qk_norm_rope_append");
        return 0;
    }
    const int warps = 4;
    const long items = (long)n_tok * (n_heads + 2 * n_kv);
    const long blocks = (items + warps - 1) / warps;
    qk_norm_rope_append_kernel<<<(unsigned)blocks, warps * 32, warps * (hd > vd ? hd : vd) * sizeof(float),
                                 (cudaStream_t)stream>>>(
        qkv, in_dt, q_gamma, k_gamma, g_dt, eps, (const float2*)cs, rot_half, tok_seq, tok_pos, block_table,
        bt_stride, k_pages, v_pages, kv_dt, q_out, q_dt, n_tok, n_heads, n_kv, hd, vd, temp_coef, temp_every, ld, v_from_k);
    NN_LAUNCH_OK("qk_norm_rope_append");
    return 0;
}

// ---------------------------------------------------------------------------
// Attention of every (token, head) over the cache of the token's sequence:
// keys first..pos with first = first_visible_key(pos, window): a sliding window (window > 0), blocks of
// -window positions (window < 0) or every earlier key (0).
// One block per (token, head) walks the span in chunks of 128 keys with an
// online softmax; the chunk boundaries are fixed by the span alone, so the
// result does not depend on the batch or on how tokens were cut into steps.
// Values have vd lanes a head (the output too).  With slope_base != 0 head h
// takes slope_h * (pos - key) off its scaled scores, slope_h = 2^(-slope_base (h + 1) / n_heads).
// With sinks (float32 [n_heads]) the softmax's denominator of head h also holds exp(sinks[h]): a term without
// key or value, not scaled, counted once.
// ---------------------------------------------------------------------------
constexpr int kAttnThreads = 128;

__global__ void __launch_bounds__(kAttnThreads)
attention_kernel(const void* __restrict__ q, int q_dt, const void* __restrict__ k_pages,
                 const void* __restrict__ v_pages, int kv_dt, const int* __restrict__ block_table, int bt_stride,
                 const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, void* __restrict__ out,
                 int out_dt, int n_heads, int n_kv, int hd, int vd, float scale, int window, float slope_base,
                 const float* __restrict__ sinks) {
    extern __shared__ float smem[];
    float* qs = smem;                       // hd
    float* p = smem + hd;                   // kAttnThreads
    long long* row = (long long*)(p + kAttnThreads);  // kAttnThreads element offsets of the chunk's rows
    __shared__ float scratch[33];

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int seq = tok_seq[t];
    const size_t q_base = (size_t)t * n_heads * hd + (size_t)h * hd;
    const size_t out_base = (size_t)t * n_heads * vd + (size_t)h * vd;
    if (seq < 0) {
        for (int d = tid; d < vd; d += kAttnThreads) st_f(out, out_base + d, out_dt, 0.0f);
        return;
    }
    const float slope = slope_base != 0.0f ? exp2f(-slope_base * (float)(h + 1) / (float)n_heads) : 0.0f;
    const int pos = tok_pos[t];
    const int first = first_visible_key(pos, window);
    const int kvh = h / (n_heads / n_kv);
    for (int d = tid; d < hd; d += kAttnThreads) qs[d] = ld_f(q, q_base + d, q_dt);
    __syncthreads();

    float m = -INFINITY, l = 0.0f;
    float acc[8];  // lanes d = tid + 128 * j, vd <= 1024
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.0f;

    for (int k0 = first; k0 <= pos; k0 += kAttnThreads) {
        const int key = k0 + tid;
        float s = -INFINITY;
        long long off = -1;
        if (key <= pos) {
            const int page = block_table[(size_t)seq * bt_stride + key / kPage];
            off = ((long long)page * n_kv + kvh) * kPage + key % kPage;      // the key's row in its pages
            float dot = 0.0f;
            for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], ld_f(k_pages, (size_t)off * hd + d, kv_dt), dot);
            s = dot * scale - slope * (float)(pos - key);
        }
        const float m_new = fmaxf(m, block_max(s, scratch));
        const float w = key <= pos ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);  // 0 on the first chunk
        l = l * corr + block_sum(w, scratch);
        m = m_new;
        p[tid] = w;
        row[tid] = off;
        __syncthreads();
        const int n_keys = min(kAttnThreads, pos + 1 - k0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int d = tid + kAttnThreads * j;
            if (d < vd) {
                float a = acc[j] * corr;
                for (int i = 0; i < n_keys; ++i) a = fmaf(p[i], ld_f(v_pages, (size_t)row[i] * vd + d, kv_dt), a);
                acc[j] = a;
            }
        }
        __syncthreads();
    }
    if (sinks != nullptr) l += expf(sinks[h] - m);      // the maximum is that of the keys: a query sees itself at least
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int d = tid + kAttnThreads * j;
        if (d < vd) st_f(out, out_base + d, out_dt, acc[j] * inv);
    }
}

extern "C" int nncpu_attention(const void* q, int q_dt, const void* k_pages, const void* v_pages, int kv_dt,
                               const int* block_table, int bt_stride, const int* tok_seq, const int* tok_pos,
                               void* out, int out_dt, int n_tok, int n_heads, int n_kv, int hd, int vd, float scale,
                               int window, float slope_base, const float* sinks, void* stream) {
    NN_CHECK(n_tok >= 0 && n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0,
             "attention: %d heads over %d key/value heads", n_heads, n_kv);
    NN_CHECK(hd > 0 && hd <= 1024, "attention: head size %d must be positive and at most 1024", hd);
    NN_CHECK(vd > 0 && vd <= 1024, "attention: value size %d must be positive and at most 1024", vd);
    if (n_tok == 0) return 0;
    const size_t smem = (hd + kAttnThreads) * sizeof(float) + kAttnThreads * sizeof(long long) + 8;
    dim3 grid(n_tok, n_heads);
    attention_kernel<<<grid, kAttnThreads, smem, (cudaStream_t)stream>>>(q, q_dt, k_pages, v_pages, kv_dt,
                                                                         block_table, bt_stride, tok_seq, tok_pos,
                                                                         out, out_dt, n_heads, n_kv, hd, vd, scale,
                                                                         window, slope_base, sinks);
    NN_LAUNCH_OK("attention");
    return 0;
}

// ---------------------------------------------------------------------------
// Gated activation: out[t, i] = act(gu[t, i], gu[t, inter + i]) with act one of gated_act_f's kinds
// (silu(g) u; the tanh form of GELU times u; the clamped g sigmoid(1.702 g) (u + 1)), in 32-bit.
// ---------------------------------------------------------------------------
__global__ void gated_act_kernel(const void* __restrict__ gu, int in_dt, void* __restrict__ out, int out_dt,
                                 long n_tok, int inter, int kind, float limit) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tok * inter) return;
    const long t = idx / inter;
    const int i = (int)(idx % inter);
    const float g = ld_f(gu, (size_t)t * 2 * inter + i, in_dt);
    const float u = ld_f(gu, (size_t)t * 2 * inter + inter + i, in_dt);
    st_f(out, (size_t)idx, out_dt, gated_act_f(g, u, kind, limit));
}

extern "C" int nncpu_gated_act(const void* gu, int in_dt, void* out, int out_dt, int n_tok, int inter, int kind,
                               float limit, void* stream) {
    NN_CHECK(n_tok >= 0 && inter > 0, "gated activation: %d tokens of %d", n_tok, inter);
    NN_CHECK(kind >= kGateSilu && kind <= kGateSwishClamp, "gated activation: kind %d", kind);
    if (n_tok == 0) return 0;
    const long total = (long)n_tok * inter;
    gated_act_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gu, in_dt, out, out_dt, n_tok,
                                                                                         inter, kind, limit);
    NN_LAUNCH_OK("gated activation");
    return 0;
}

// ---------------------------------------------------------------------------
// xIELU, an activation with two learned numbers (p, q) = params[0..1]:
//   z > 0:  softplus(p) z^2 + z / 2
//   z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2
// softplus and the activation are computed in 32-bit whatever the tensors hold.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

__global__ void xielu_kernel(const void* __restrict__ x, int in_dt, const void* __restrict__ params, int p_dt,
                             void* __restrict__ out, int out_dt, long n) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const float a_pos = softplus_f(ld_f(params, 0, p_dt));
    const float a_neg = 0.5f + softplus_f(ld_f(params, 1, p_dt));
    const float z = ld_f(x, (size_t)idx, in_dt);
    st_f(out, (size_t)idx, out_dt, xielu_f(z, a_pos, a_neg));
}

// The prompt's case: float32 in, bfloat16 out, four elements a thread (16 bytes in, 8 out).
__global__ void __launch_bounds__(256)
xielu_f32_bf16_kernel(const float4* __restrict__ x, const void* __restrict__ params, int p_dt,
                      uint2* __restrict__ out, long n4) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n4) return;
    const float a_pos = softplus_f(ld_f(params, 0, p_dt));
    const float a_neg = 0.5f + softplus_f(ld_f(params, 1, p_dt));
    const float4 v = x[idx];
    const float z[4] = {v.x, v.y, v.z, v.w};
    float y[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
        y[e] = xielu_f(z[e], a_pos, a_neg);
    __nv_bfloat162 h[2] = {__floats2bfloat162_rn(y[0], y[1]), __floats2bfloat162_rn(y[2], y[3])};
    out[idx] = *reinterpret_cast<uint2*>(h);
}

extern "C" int nncpu_xielu(const void* x, int in_dt, const void* params, int p_dt, void* out, int out_dt, long n,
                           void* stream) {
    NN_CHECK(n >= 0 && params != nullptr, "xielu: %ld elements", n);
    if (n == 0) return 0;
    if (in_dt == DT_F32 && out_dt == DT_BF16 && n % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 8 == 0) {
        xielu_f32_bf16_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            (const float4*)x, params, p_dt, (uint2*)out, n / 4);
        NN_LAUNCH_OK("xielu");
        return 0;
    }
    xielu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, in_dt, params, p_dt, out, out_dt, n);
    NN_LAUNCH_OK("xielu");
    return 0;
}

// ---------------------------------------------------------------------------
// Soft cap in place: x <- cap * tanh(x / cap), float32.
// ---------------------------------------------------------------------------
__global__ void softcap_kernel(float* __restrict__ x, long n, float cap) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) x[idx] = cap * tanhf(x[idx] / cap);
}

extern "C" int nncpu_softcap(float* x, long n, float cap, void* stream) {
    NN_CHECK(n >= 0 && cap > 0.0f, "softcap: %ld elements, cap %g", n, cap);
    if (n == 0) return 0;
    softcap_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, n, cap);
    NN_LAUNCH_OK("softcap");
    return 0;
}

// ---------------------------------------------------------------------------
// Gather rows: out[r, :] = x[rows[r], :] (float32), zeros for a negative row.
// ---------------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int dim) {
    const int r = blockIdx.x, src = rows[r];
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
        out[(size_t)r * dim + i] = src < 0 ? 0.0f : x[(size_t)src * dim + i];
}

extern "C" int nncpu_gather_rows(const float* x, const int* rows, float* out, int n_rows, int dim, void* stream) {
    NN_CHECK(n_rows >= 0 && dim > 0, "gather_rows: %d rows of %d", n_rows, dim);
    if (n_rows == 0) return 0;
    gather_rows_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, rows, out, dim);
    NN_LAUNCH_OK("gather_rows");
    return 0;
}

// ---------------------------------------------------------------------------
// Greedy choice: the first largest logit of each row.  NaN never wins.
// ---------------------------------------------------------------------------
__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int vocab) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int n_warps = blockDim.x >> 5;
        bv = lane < n_warps ? best_v[lane] : -INFINITY;
        bi = lane < n_warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
    }
}

// A long row in two steps: blocks (chunk, row) each leave the first largest of their chunk, then one warp per row
// picks among the chunks by the same rule.  One block per row walks 150 000 logits in 33 us whatever the
// number of rows; cut into 32 chunks the two kernels take a few microseconds.
constexpr int kArgmaxChunks = 32;

__global__ void argmax_chunk_kernel(const float* __restrict__ logits, float* __restrict__ part_v,
                                    int* __restrict__ part_i, int vocab) {
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    const float* row = logits + (size_t)blockIdx.y * vocab;
    const int len = (vocab + kArgmaxChunks - 1) / kArgmaxChunks;
    const int begin = blockIdx.x * len, end = min(vocab, begin + len);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int n_warps = blockDim.x >> 5;
        bv = lane < n_warps ? best_v[lane] : -INFINITY;
        bi = lane < n_warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            part_v[blockIdx.y * kArgmaxChunks + blockIdx.x] = bv;
            part_i[blockIdx.y * kArgmaxChunks + blockIdx.x] = bi;
        }
    }
}

__global__ void argmax_pick_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i,
                                   int* __restrict__ out) {
    static_assert(kArgmaxChunks == 32, "one lane per chunk");
    const int lane = threadIdx.x;
    float bv = part_v[blockIdx.x * kArgmaxChunks + lane];
    int bi = part_i[blockIdx.x * kArgmaxChunks + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
}

// Bytes of scratch that nncpu_argmax wants for rows this long (0: none).
extern "C" long nncpu_argmax_scratch_bytes(int n_rows, int vocab) {
    return vocab >= 8192 ? (long)n_rows * kArgmaxChunks * 8 : 0;
}

extern "C" int nncpu_argmax(const float* logits, int* out, int n_rows, int vocab, void* scratch, long scratch_bytes,
                            void* stream) {
    NN_CHECK(n_rows >= 0 && vocab > 0, "argmax: %d rows of %d", n_rows, vocab);
    if (n_rows == 0) return 0;
    const long need = nncpu_argmax_scratch_bytes(n_rows, vocab);
    if (need > 0 && scratch != nullptr && scratch_bytes >= need) {
        float* part_v = (float*)scratch;
        int* part_i = (int*)(part_v + (size_t)n_rows * kArgmaxChunks);
        argmax_chunk_kernel<<<dim3(kArgmaxChunks, n_rows), 256, 0, (cudaStream_t)stream>>>(logits, part_v, part_i, vocab);
        NN_LAUNCH_OK("argmax (chunks)");
        argmax_pick_kernel<<<n_rows, 32, 0, (cudaStream_t)stream>>>(part_v, part_i, out);
        NN_LAUNCH_OK("argmax (pick)");
        return 0;
    }
    argmax_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(logits, out, vocab);
    NN_LAUNCH_OK("argmax");
    return 0;
}

// ---------------------------------------------------------------------------
// The k best logits of each row in the sampler's ranking: higher logit first,
// then lower id; NaN counts as -inf (crates/nncpu/src/session/sample.rs:69-88,
// 130-152, where a k-element heap makes the same selection).  A radix select
// over the order-preserving integer image of the floats finds the k-th value,
// then everything above it and the lowest ids at it are gathered.  The k
// candidates come out unordered; the host sorts them (k is small).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t float_order(float v) {
    if (!(v == v)) v = -INFINITY;
    const uint32_t u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// The selection by radix, for a block of 1024 threads: vals and ids (global or shared memory) receive the k
// candidates of `row` in no particular order.  Works for every row and every k.
__device__ void select_topk_radix(const float* __restrict__ row, int vocab, int k, float* vals, int* ids) {
    __shared__ int hist[256];
    __shared__ uint32_t prefix_s;
    __shared__ int need_s, n_out;
    __shared__ int seg[1024];
    const int tid = threadIdx.x, nt = blockDim.x;
    // radix select, most significant byte first: after 4 rounds `prefix` is the image of the k-th largest value
    uint32_t prefix = 0, mask = 0;
    int need = k;   // how many of the values matching `prefix` so far are still wanted
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256; i += nt) hist[i] = 0;
        __syncthreads();
        for (int i = tid; i < vocab; i += nt) {
            const uint32_t u = float_order(row[i]);
            if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255], 1);
        }
        __syncthreads();
        if (tid == 0) {
            int bin = 255, left = need;
            for (; bin > 0; --bin) {
                if (hist[bin] >= left) break;
                left -= hist[bin];
            }
            prefix_s = prefix | ((uint32_t)bin << shift);
            need_s = left;
        }
        __syncthreads();
        prefix = prefix_s;
        need = need_s;
        mask |= 255u << shift;
        __syncthreads();
    }
    // `need` values equal to the k-th value are wanted: the ones with the lowest ids.  Threads own
    // contiguous id ranges so that a scan over the threads counts ties in id order.
    const int per = (vocab + nt - 1) / nt;
    const int lo = min(vocab, tid * per), hi = min(vocab, lo + per);
    int ties = 0;
    for (int i = lo; i < hi; ++i) ties += float_order(row[i]) == prefix;
    seg[tid] = ties;
    if (tid == 0) n_out = 0;
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int i = 0; i < nt; ++i) { const int c = seg[i]; seg[i] = run; run += c; }
    }
    __syncthreads();
    int tie_rank = seg[tid];
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        const uint32_t u = float_order(v);
        bool take = u > prefix;
        if (u == prefix) take = tie_rank++ < need;
        if (take) {
            const int at = atomicAdd(&n_out, 1);
            if (at < k) { vals[at] = (v == v) ? v : -INFINITY; ids[at] = i; }
        }
    }
    __syncthreads();
}

// Ascending bitonic sort of key[0 .. n2) by a block of at least n2 threads; n2 a power of two.
__device__ void sort_keys(unsigned long long* key, int n2) {
    const int tid = threadIdx.x;
    for (int size = 2; size <= n2; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            if (tid < n2) {
                const int other = tid ^ stride;
                if (other > tid) {
                    const bool up = (tid & size) == 0;
                    const unsigned long long a = key[tid], b = key[other];
                    if ((a > b) == up) { key[tid] = b; key[other] = a; }
                }
            }
            __syncthreads();
        }
    }
}

// (descending logit, ascending id) as one ascending 64-bit key, and back.
__device__ __forceinline__ unsigned long long rank_key(float v, int id) {
    return ((unsigned long long)(~float_order(v)) << 32) | (uint32_t)id;
}
__device__ __forceinline__ float key_value(unsigned long long key) {
    const uint32_t image = ~(uint32_t)(key >> 32);
    return __uint_as_float((image & 0x80000000u) ? (image & 0x7fffffffu) : ~image);
}

// The quick way to the k candidates, which serves the rows a language model produces: the candidates lie within
// 16 of the row's largest logit.  One pass finds the largest, one counts the logits of that range in 1024 bins
// (few logits share a bin there, so the counters do not collide), one gathers everything down to the bin that
// holds the k-th, and a sort of those few puts the k best first.  `key` is scratch for 1024 keys.  Returns
// false, having written nothing, when the range holds fewer than k logits or the gathered ones do not fit:
// then the radix selection does the job.  On success vals and ids are in rank order.
__device__ bool select_topk_near_max(const float* __restrict__ row, int vocab, int k, float* vals, int* ids,
                                     unsigned long long* key) {
    constexpr int kBins = 1024;
    constexpr float kRange = 16.0f, kPerUnit = kBins / kRange;
    __shared__ int fine[kBins];
    __shared__ float red[33];
    __shared__ int cut_bin, n_in, n_got;
    const int tid = threadIdx.x, nt = blockDim.x;
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += nt) {
        const float v = row[i];
        if (v == v) mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    if (!(mx > -INFINITY) || mx == INFINITY) return false;
    for (int i = tid; i < kBins; i += nt) fine[i] = 0;
    __syncthreads();
    for (int i = tid; i < vocab; i += nt) {
        const float d = mx - row[i];
        if (d < kRange) atomicAdd(&fine[(int)(d * kPerUnit)], 1);   // false for NaN
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0, b = 0;
        for (; b < kBins; ++b) {
            run += fine[b];
            if (run >= k) break;
        }
        cut_bin = b;
        n_in = run;
        n_got = 0;
    }
    __syncthreads();
    const int cut = cut_bin, n = n_in;
    if (cut >= kBins || n > 1024) return false;
    for (int i = tid; i < vocab; i += nt) {
        const float v = row[i];
        const float d = mx - v;
        if (d < kRange && (int)(d * kPerUnit) <= cut) key[atomicAdd(&n_got, 1)] = rank_key(v, i);
    }
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    __syncthreads();
    for (int i = n + tid; i < n2; i += nt) key[i] = ~0ull;
    __syncthreads();
    sort_keys(key, n2);
    if (tid < k) {
        vals[tid] = key_value(key[tid]);
        ids[tid] = (int)(uint32_t)key[tid];
    }
    __syncthreads();
    return true;
}

// The k candidates of `row` in vals and ids; `*sorted` tells whether they came out in rank order.
__device__ void select_topk(const float* __restrict__ row, int vocab, int k, float* vals, int* ids,
                            unsigned long long* key, bool* sorted) {
    *sorted = select_topk_near_max(row, vocab, k, vals, ids, key);
    if (!*sorted) select_topk_radix(row, vocab, k, vals, ids);
}

__global__ void __launch_bounds__(1024)
topk_kernel(const float* __restrict__ logits, float* __restrict__ out_vals, int* __restrict__ out_ids, int vocab, int k) {
    __shared__ unsigned long long key[1024];
    bool sorted;
    select_topk(logits + (size_t)blockIdx.x * vocab, vocab, k, out_vals + (size_t)blockIdx.x * k,
                out_ids + (size_t)blockIdx.x * k, key, &sorted);
}

// ---------------------------------------------------------------------------
// The same candidates for long rows, found by the whole GPU instead of one block per row: a block per
// (chunk, row) for each of the three passes of the quick way (largest logit; counts in 1024 bins within 16 of
// it; gather down to the bin of the k-th), a small kernel between the last two that finds that bin, and the
// chain's kernel then sorts what was gathered.  Per row the scratch holds: the chunks' largest logits, the
// bins, three numbers (the cut bin or -1, how many logits lie down to it, how many were gathered) and 1024 keys.
// ---------------------------------------------------------------------------
constexpr int kPickChunks = 32;
constexpr int kPickBins = 1024;
constexpr float kPickRange = 16.0f, kPickPerUnit = kPickBins / kPickRange;

struct PickScratch {
    float chunk_max[kPickChunks];
    int bins[kPickBins];
    int cut, n_in, n_got, pad;
    unsigned long long key[1024];
};

__device__ __forceinline__ void chunk_span(int vocab, int& begin, int& end) {
    const int len = (vocab + kPickChunks - 1) / kPickChunks;
    begin = blockIdx.x * len;
    end = min(vocab, begin + len);
}

__global__ void __launch_bounds__(256)
pick_max_kernel(const float* __restrict__ logits, PickScratch* __restrict__ scratch, int vocab) {
    __shared__ float red[33];
    PickScratch& sc = scratch[blockIdx.y];
    int begin, end;
    chunk_span(vocab, begin, end);
    const float* row = logits + (size_t)blockIdx.y * vocab;
    float mx = -INFINITY;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        if (v == v) mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    if (threadIdx.x == 0) sc.chunk_max[blockIdx.x] = mx;
    // this block's share of the row's bins and numbers starts at zero
    for (int i = threadIdx.x; i < kPickBins / kPickChunks; i += blockDim.x) sc.bins[blockIdx.x * (kPickBins / kPickChunks) + i] = 0;
    if (blockIdx.x == 0 && threadIdx.x == 0) sc.cut = sc.n_in = sc.n_got = 0;
}

__device__ __forceinline__ float row_max_of_chunks(const PickScratch& sc) {
    float mx = -INFINITY;
#pragma unroll 8
    for (int c = 0; c < kPickChunks; ++c) mx = fmaxf(mx, sc.chunk_max[c]);
    return mx;
}

__global__ void __launch_bounds__(256)
pick_count_kernel(const float* __restrict__ logits, PickScratch* __restrict__ scratch, int vocab) {
    __shared__ int fine[kPickBins];
    PickScratch& sc = scratch[blockIdx.y];
    const float mx = row_max_of_chunks(sc);
    if (!(mx > -INFINITY) || mx == INFINITY) return;
    int begin, end;
    chunk_span(vocab, begin, end);
    const float* row = logits + (size_t)blockIdx.y * vocab;
    for (int i = threadIdx.x; i < kPickBins; i += blockDim.x) fine[i] = 0;
    __syncthreads();
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float d = mx - row[i];
        if (d < kPickRange) atomicAdd(&fine[(int)(d * kPickPerUnit)], 1);   // false for NaN
    }
    __syncthreads();
    for (int i = threadIdx.x; i < kPickBins; i += blockDim.x)
        if (fine[i]) atomicAdd(&sc.bins[i], fine[i]);
}

// One block of 1024 threads per row: the bin that holds the k-th logit from the top, by a prefix sum over the bins.
__global__ void __launch_bounds__(kPickBins)
pick_cut_kernel(PickScratch* __restrict__ scratch, int k) {
    __shared__ int warp_total[32];
    PickScratch& sc = scratch[blockIdx.x];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mine = sc.bins[tid];
    int run = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, run, o);
        if (lane >= o) run += t;
    }
    if (lane == 31) warp_total[warp] = run;
    __syncthreads();
    if (warp == 0) {
        int t = warp_total[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, t, o);
            if (lane >= o) t += v;
        }
        warp_total[lane] = t;
    }
    __syncthreads();
    run += warp > 0 ? warp_total[warp - 1] : 0;     // logits in bins 0 .. tid
    // the first bin whose running count reaches k; none, or too many to gather: -1 (the chain's kernel selects by radix)
    if (run >= k && run - mine < k) {
        sc.cut = run <= 1024 ? tid : -1;
        sc.n_in = run;
    }
    if (tid == kPickBins - 1 && run < k) sc.cut = -1;
}

__global__ void __launch_bounds__(256)
pick_gather_kernel(const float* __restrict__ logits, PickScratch* __restrict__ scratch, int vocab) {
    PickScratch& sc = scratch[blockIdx.y];
    const int cut = sc.cut;
    const float mx = row_max_of_chunks(sc);
    if (cut < 0 || !(mx > -INFINITY) || mx == INFINITY) return;
    int begin, end;
    chunk_span(vocab, begin, end);
    const float* row = logits + (size_t)blockIdx.y * vocab;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const float v = row[i];
        const float d = mx - v;
        if (d < kPickRange && (int)(d * kPickPerUnit) <= cut) sc.key[atomicAdd(&sc.n_got, 1)] = rank_key(v, i);
    }
}

// ---------------------------------------------------------------------------
// The whole sampling chain of one row on the device, for 0 < top-k <= 1024: the k candidates, their ranking
// (higher logit first, then lower id), top-p and min-p on the distribution at temperature 1, temperature over
// the survivors and the draw in rank order from u[row], uniform in [0, 1)
// (crates/nncpu/src/session/sample.rs:121-201).  After the selection and a bitonic sort one thread walks the
// few candidates with the arithmetic of the reference: 32-bit weights, 64-bit sums.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
sample_chain_kernel(const float* __restrict__ logits, const double* __restrict__ u, int* __restrict__ out, int vocab,
                    int k, float temperature, float top_p, float min_p, const PickScratch* __restrict__ picked) {
    __shared__ float c_val[1024];
    __shared__ int c_id[1024];
    __shared__ unsigned long long key[1024];
    const int tid = threadIdx.x;
    bool sorted;
    if (picked != nullptr && picked[blockIdx.x].cut >= 0) {
        // the candidates were gathered by the kernels before this one: sort them, the k best come first
        const PickScratch& sc = picked[blockIdx.x];
        const int n = sc.n_in;
        int n2 = 1;
        while (n2 < n) n2 <<= 1;
        if (tid < n2) key[tid] = tid < n ? sc.key[tid] : ~0ull;
        __syncthreads();
        sort_keys(key, n2);
        if (tid < k) {
            c_val[tid] = key_value(key[tid]);
            c_id[tid] = (int)(uint32_t)key[tid];
        }
        __syncthreads();
        sorted = true;
    } else {
        select_topk(logits + (size_t)blockIdx.x * vocab, vocab, k, c_val, c_id, key, &sorted);
    }
    if (!sorted) {
        // ascending by (descending logit, ascending id); the padding sorts last
        int n2 = 1;
        while (n2 < k) n2 <<= 1;
        if (tid < n2) key[tid] = tid < k ? rank_key(c_val[tid], c_id[tid]) : ~0ull;
        __syncthreads();
        sort_keys(key, n2);
        if (tid < k) {
            c_val[tid] = key_value(key[tid]);
            c_id[tid] = (int)(uint32_t)key[tid];
        }
        __syncthreads();
    }
    if (tid != 0) return;
    const float top = c_val[0];
    if (!(top > -INFINITY) || top == INFINITY) {   // nothing finite to draw from
        out[blockIdx.x] = c_id[0];
        return;
    }
    // weights at temperature 1
    double total = 0.0;
    for (int i = 0; i < k; ++i) total += (double)expf(c_val[i] - top);
    int keep = k;
    if (top_p > 0.0f && top_p < 1.0f) {
        double cum = 0.0;
        for (int i = 0; i < k; ++i) {
            cum += (double)expf(c_val[i] - top) / total;
            if (cum >= (double)top_p) { keep = i + 1; break; }
        }
    }
    if (min_p > 0.0f) {
        const float floor_ = min_p * 1.0f;   // the best candidate's weight is exp(0) = 1
        int i = 1;
        while (i < keep && expf(c_val[i] - top) >= floor_) ++i;
        keep = i;
    }
    const double inv_t = 1.0 / (double)temperature;
    double sum_t = 0.0;
    for (int i = 0; i < keep; ++i) sum_t += (double)(float)exp((double)(c_val[i] - top) * inv_t);
    double r = u[blockIdx.x] * sum_t;
    int chosen = c_id[keep - 1];
    for (int i = 0; i < keep; ++i) {
        r -= (double)(float)exp((double)(c_val[i] - top) * inv_t);
        if (r <= 0.0) { chosen = c_id[i]; break; }
    }
    out[blockIdx.x] = chosen;
}

// Bytes of scratch with which nncpu_sample_chain finds the candidates of long rows by the whole GPU (0: rows
// are short, one block per row does it all).
extern "C" long nncpu_sample_chain_scratch_bytes(int n_rows, int vocab) {
    return vocab >= 8192 ? (long)n_rows * (long)sizeof(PickScratch) : 0;
}

extern "C" int nncpu_sample_chain(const float* logits, const double* u, int* out, int n_rows, int vocab, int top_k,
                                  float temperature, float top_p, float min_p, void* scratch, long scratch_bytes,
                                  void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    NN_CHECK(n_rows >= 0 && vocab > 0, "sample_chain: %d rows of %d", n_rows, vocab);
    NN_CHECK(top_k > 0 && top_k <= 1024 && top_k <= vocab, "sample_chain: top-k %d is outside 1..min(1024, %d)", top_k, vocab);
    NN_CHECK(temperature > 0.0f && temperature < INFINITY, "sample_chain: temperature %g", (double)temperature);
    NN_CHECK(top_p >= 0.0f && top_p <= 1.0f && min_p >= 0.0f && min_p <= 1.0f, "sample_chain: top-p %g, min-p %g",
             (double)top_p, (double)min_p);
    if (n_rows == 0) return 0;
    PickScratch* picked = nullptr;
    const long need = nncpu_sample_chain_scratch_bytes(n_rows, vocab);
    if (need > 0 && scratch != nullptr && scratch_bytes >= need && ((uintptr_t)scratch % 8) == 0) {
        picked = (PickScratch*)scratch;
        const dim3 grid(kPickChunks, n_rows);
        pick_max_kernel<<<grid, 256, 0, stream>>>(logits, picked, vocab);
        NN_LAUNCH_OK("sample_chain (largest)");
        pick_count_kernel<<<grid, 256, 0, stream>>>(logits, picked, vocab);
        NN_LAUNCH_OK("sample_chain (count)");
        pick_cut_kernel<<<n_rows, kPickBins, 0, stream>>>(picked, top_k);
        NN_LAUNCH_OK("sample_chain (cut)");
        pick_gather_kernel<<<grid, 256, 0, stream>>>(logits, picked, vocab);
        NN_LAUNCH_OK("sample_chain (gather)");
    }
    sample_chain_kernel<<<n_rows, 1024, 0, stream>>>(logits, u, out, vocab, top_k, temperature, top_p, min_p, picked);
    NN_LAUNCH_OK("sample_chain");
    return 0;
}

// Per row: sum over the vocabulary of exp(logit - largest logit), NaN as -inf: the denominator of the
// distribution at temperature 1, which top-p and min-p are measured on.
__global__ void __launch_bounds__(1024)
row_exp_sum_kernel(const float* __restrict__ logits, double* __restrict__ out_sum, int vocab) {
    __shared__ float red_f[32];
    __shared__ double red_d[32];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float m = -INFINITY;
    for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v == v) m = fmaxf(m, v);
    }
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red_f[warp] = m;
    __syncthreads();
    m = red_f[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, red_f[w]);
    double s = 0.0;
    for (int i = tid; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v == v && v != -INFINITY) s += (double)expf(v - m);
    }
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red_d[warp] = s;
    __syncthreads();
    if (tid == 0) {
        double t = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red_d[w];
        out_sum[blockIdx.x] = t;
    }
}

extern "C" int nncpu_row_exp_sum(const float* logits, double* out_sum, int n_rows, int vocab, void* stream) {
    NN_CHECK(n_rows >= 0 && vocab > 0, "row_exp_sum: %d rows of %d", n_rows, vocab);
    if (n_rows == 0) return 0;
    row_exp_sum_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(logits, out_sum, vocab);
    NN_LAUNCH_OK("row_exp_sum");
    return 0;
}

extern "C" int nncpu_topk(const float* logits, float* out_vals, int* out_ids, int n_rows, int vocab, int k, void* stream) {
    NN_CHECK(n_rows >= 0 && vocab > 0 && k > 0 && k <= vocab, "topk: %d rows of %d, k %d", n_rows, vocab, k);
    if (n_rows == 0) return 0;
    topk_kernel<<<n_rows, 1024, 0, (cudaStream_t)stream>>>(logits, out_vals, out_ids, vocab, k);
    NN_LAUNCH_OK("topk");
    return 0;
}

// ---------------------------------------------------------------------------
// Temperature draw over the whole vocabulary, in token-id order:
// p_i = exp((l_i - max) / T) in double, r = u * sum(p), the first i whose
// running sum reaches r.  NaN counts as -inf.  `u[row]` is uniform in [0, 1).
// ---------------------------------------------------------------------------
__global__ void sample_kernel(const float* __restrict__ logits, const double* __restrict__ u,
                              int* __restrict__ out, int vocab, float inv_temp) {
    __shared__ float scratch[33];
    __shared__ double part[1024];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int tid = threadIdx.x, nt = blockDim.x;
    float mx = -INFINITY;
    for (int i = tid; i < vocab; i += nt) {
        const float v = row[i];
        if (v == v) mx = fmaxf(mx, v);
    }
    mx = block_max(mx, scratch);
    if (!(mx > -INFINITY) || mx == INFINITY) {  // nothing finite to draw from: the first largest
        if (tid == 0) {
            int best = 0;
            for (int i = 1; i < vocab; ++i) if (row[i] > row[best] || (row[best] != row[best] && row[i] == row[i])) best = i;
            out[blockIdx.x] = best;
        }
        return;
    }
    // thread `tid` owns the contiguous ids [lo, hi)
    const int per = (vocab + nt - 1) / nt;
    const int lo = min(vocab, tid * per), hi = min(vocab, lo + per);
    double s = 0.0;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v == v) s += exp((double)(v - mx) * (double)inv_temp);
    }
    part[tid] = s;
    __syncthreads();
    if (tid == 0) {
        double total = 0.0;
        for (int i = 0; i < nt; ++i) total += part[i];
        double r = u[blockIdx.x] * total;
        int owner = nt - 1;
        for (int i = 0; i < nt; ++i) {
            if (r - part[i] <= 0.0 && part[i] > 0.0) { owner = i; break; }
            r -= part[i];
        }
        // walk the owner's ids; the last id with weight is the fallback
        const int olo = min(vocab, owner * per), ohi = min(vocab, olo + per);
        int pick = -1, last = -1;
        for (int i = olo; i < ohi; ++i) {
            const float v = row[i];
            if (!(v == v)) continue;
            const double w = exp((double)(v - mx) * (double)inv_temp);
            if (w > 0.0) last = i;
            r -= w;
            if (r <= 0.0 && w > 0.0) { pick = i; break; }
        }
        if (pick < 0) pick = last;
        if (pick < 0) {  // rounding pushed r past the end: the last id with weight anywhere
            for (int i = vocab - 1; i >= 0; --i) {
                const float v = row[i];
                if (v == v && exp((double)(v - mx) * (double)inv_temp) > 0.0) { pick = i; break; }
            }
        }
        out[blockIdx.x] = pick < 0 ? 0 : pick;
    }
}

// The same draw for long rows in three kernels: the chunks' largest logits (pick_max_kernel), the chunks' sums
// of weights, and a block per row that finds the chunk in which the running sum reaches r and walks that chunk
// alone.  Per row the scratch is a PickScratch; the chunk sums lie where its keys would.
__global__ void __launch_bounds__(256)
sample_chunk_sum_kernel(const float* __restrict__ logits, PickScratch* __restrict__ scratch, int vocab, float inv_temp) {
    __shared__ double red[8];
    PickScratch& sc = scratch[blockIdx.y];
    const float mx = row_max_of_chunks(sc);
    int begin, end;
    chunk_span(vocab, begin, end);
    const float* row = logits + (size_t)blockIdx.y * vocab;
    double s = 0.0;
    if (mx > -INFINITY && mx != INFINITY) {
        for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            const float v = row[i];
            if (v == v) s += exp((double)(v - mx) * (double)inv_temp);
        }
    }
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
        reinterpret_cast<double*>(sc.key)[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(256)
sample_chunk_draw_kernel(const float* __restrict__ logits, const double* __restrict__ u, int* __restrict__ out,
                         const PickScratch* __restrict__ scratch, int vocab, float inv_temp) {
    __shared__ double part[256];
    const PickScratch& sc = scratch[blockIdx.x];
    const float* row = logits + (size_t)blockIdx.x * vocab;
    const int tid = threadIdx.x, nt = blockDim.x;
    const float mx = row_max_of_chunks(sc);
    if (!(mx > -INFINITY) || mx == INFINITY) {  // nothing finite to draw from: the first largest
        if (tid == 0) {
            int best = 0;
            for (int i = 1; i < vocab; ++i) if (row[i] > row[best] || (row[best] != row[best] && row[i] == row[i])) best = i;
            out[blockIdx.x] = best;
        }
        return;
    }
    // the chunk in which the running sum, in id order, reaches r; the last chunk with weight if rounding ran past the end
    const double* chunk_sum = reinterpret_cast<const double*>(sc.key);
    double total = 0.0;
    for (int c = 0; c < kPickChunks; ++c) total += chunk_sum[c];
    double r = u[blockIdx.x] * total;
    int chunk = -1, last_chunk = -1;
    for (int c = 0; c < kPickChunks; ++c) {
        if (chunk_sum[c] > 0.0) last_chunk = c;
        if (r - chunk_sum[c] <= 0.0 && chunk_sum[c] > 0.0) { chunk = c; break; }
        r -= chunk_sum[c];
    }
    if (chunk < 0) {      // past the end: the last id with weight
        chunk = last_chunk;
        r = INFINITY;
    }
    if (chunk < 0) {      // no weight anywhere (cannot be: the largest logit has weight 1)
        if (tid == 0) out[blockIdx.x] = 0;
        return;
    }
    const int len = (vocab + kPickChunks - 1) / kPickChunks;
    const int begin = chunk * len, end = min(vocab, begin + len);
    // thread `tid` owns the contiguous ids [lo, hi) of the chunk
    const int per = (end - begin + nt - 1) / nt;
    const int lo = min(end, begin + tid * per), hi = min(end, lo + per);
    double s = 0.0;
    for (int i = lo; i < hi; ++i) {
        const float v = row[i];
        if (v == v) s += exp((double)(v - mx) * (double)inv_temp);
    }
    part[tid] = s;
    __syncthreads();
    if (tid != 0) return;
    int owner = -1, last_owner = -1;
    for (int i = 0; i < nt; ++i) {
        if (part[i] > 0.0) last_owner = i;
        if (r - part[i] <= 0.0 && part[i] > 0.0) { owner = i; break; }
        r -= part[i];
    }
    if (owner < 0) {
        owner = last_owner;
        r = INFINITY;
    }
    int pick = -1, last = -1;
    if (owner >= 0) {
        const int olo = min(end, begin + owner * per), ohi = min(end, olo + per);
        for (int i = olo; i < ohi; ++i) {
            const float v = row[i];
            if (!(v == v)) continue;
            const double w = exp((double)(v - mx) * (double)inv_temp);
            if (w > 0.0) last = i;
            r -= w;
            if (r <= 0.0 && w > 0.0) { pick = i; break; }
        }
    }
    if (pick < 0) pick = last;
    out[blockIdx.x] = pick < 0 ? 0 : pick;
}

extern "C" long nncpu_sample_temperature_scratch_bytes(int n_rows, int vocab) {
    return vocab >= 8192 ? (long)n_rows * (long)sizeof(PickScratch) : 0;
}

extern "C" int nncpu_sample_temperature(const float* logits, const double* u, int* out, int n_rows, int vocab,
                                        float temperature, void* scratch, long scratch_bytes, void* stream_) {
    cudaStream_t stream = (cudaStream_t)stream_;
    NN_CHECK(n_rows >= 0 && vocab > 0, "sample: %d rows of %d", n_rows, vocab);
    NN_CHECK(temperature > 0.0f && isfinite(temperature), "sample: temperature %g must be positive", temperature);
    if (n_rows == 0) return 0;
    const long need = nncpu_sample_temperature_scratch_bytes(n_rows, vocab);
    if (need > 0 && scratch != nullptr && scratch_bytes >= need && ((uintptr_t)scratch % 8) == 0) {
        PickScratch* sc = (PickScratch*)scratch;
        const dim3 grid(kPickChunks, n_rows);
        pick_max_kernel<<<grid, 256, 0, stream>>>(logits, sc, vocab);
        NN_LAUNCH_OK("sample (largest)");
        sample_chunk_sum_kernel<<<grid, 256, 0, stream>>>(logits, sc, vocab, 1.0f / temperature);
        NN_LAUNCH_OK("sample (sums)");
        sample_chunk_draw_kernel<<<n_rows, 256, 0, stream>>>(logits, u, out, sc, vocab, 1.0f / temperature);
        NN_LAUNCH_OK("sample (draw)");
        return 0;
    }
    sample_kernel<<<n_rows, 1024, 0, stream>>>(logits, u, out, vocab, 1.0f / temperature);
    NN_LAUNCH_OK("sample");
    return 0;
}

// ---------------------------------------------------------------------------
// x[t, :] += rows[t, :] + vec[:]: what a schedule adds to the residual stream
// before a run of layers (an earlier state of the stream, a learned vector).
// Either addend may be null.  32-bit.
// ---------------------------------------------------------------------------
__global__ void stream_add_kernel(float* __restrict__ x, const float* __restrict__ rows, const void* __restrict__ vec,
                                  int vec_dt, long total, int dim) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    float v = x[idx];
    if (rows) v += rows[idx];
    if (vec) v += ld_f(vec, (size_t)(idx % dim), vec_dt);
    x[idx] = v;
}

extern "C" int nncpu_stream_add(float* x, const float* rows, const void* vec, int vec_dt, int n_tok, int dim,
                                void* stream) {
    NN_CHECK(n_tok >= 0 && dim > 0, "stream add: %d rows of %d", n_tok, dim);
    if (n_tok == 0 || (rows == nullptr && vec == nullptr)) return 0;
    const long total = (long)n_tok * dim;
    stream_add_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, rows, vec, vec_dt, total, dim);
    NN_LAUNCH_OK("stream add");
    return 0;
}

// ---------------------------------------------------------------------------
// Two norms of the same rows in one pass (a layer whose sublayers both read the
// stream as it enters the layer): y1 = x * scale1 * gamma1, y2 = x * scale2 * gamma2
// with scale = 1 / sqrt(mean(x^2) + eps).  x float32; the sum of squares is taken once.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rmsnorm_dual_kernel(const float* __restrict__ x, const void* __restrict__ g1, const void* __restrict__ g2, int g_dt,
                    float eps1, float eps2, void* __restrict__ y1, void* __restrict__ y2, int y_dt, int dim) {
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * dim;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = x[base + i];
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float mean = ss * (1.0f / (float)dim);
    const float s1 = 1.0f / sqrtf(mean + eps1), s2 = 1.0f / sqrtf(mean + eps2);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float v = x[base + i];
        st_f(y1, base + i, y_dt, (v * s1) * ld_f(g1, i, g_dt));
        st_f(y2, base + i, y_dt, (v * s2) * ld_f(g2, i, g_dt));
    }
}

// The common case: a width that is a multiple of 4 and at most 256 * 4 * kVec; every thread keeps its part of the row
// in registers between the sum of squares and the two scalings, so the row is read once, 16 bytes at a time.
template <int kVec>
__global__ void __launch_bounds__(256)
rmsnorm_dual_f32_kernel(const float* __restrict__ x, const void* __restrict__ g1, const void* __restrict__ g2, int g_dt,
                        float eps1, float eps2, void* __restrict__ y1, void* __restrict__ y2, int y_dt, int dim) {
    __shared__ float scratch[33];
    const int n4 = dim >> 2;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)blockIdx.x * dim);
    float4 v[kVec];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        v[j] = i < n4 ? src[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = block_sum(ss, scratch);
    const float mean = ss * (1.0f / (float)dim);
    const float s1 = 1.0f / sqrtf(mean + eps1), s2 = 1.0f / sqrtf(mean + eps2);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        const float in[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        const size_t at = (size_t)blockIdx.x * dim + 4 * i;
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            const void* g = which ? g2 : g1;
            void* y = which ? y2 : y1;
            const float sc = which ? s2 : s1;
            float o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = (in[e] * sc) * ld_f(g, 4 * i + e, g_dt);
            if (y_dt == DT_BF16) {
                __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
                *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + at) = *reinterpret_cast<uint2*>(h);
            } else {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + at) = make_float4(o[0], o[1], o[2], o[3]);
            }
        }
    }
}

extern "C" int nncpu_rmsnorm_dual(const float* x, const void* g1, const void* g2, int g_dt, float eps1, float eps2,
                                  void* y1, void* y2, int y_dt, int n_rows, int dim, void* stream) {
    NN_CHECK(n_rows >= 0 && dim > 0, "rmsnorm (two outputs): %d rows of %d", n_rows, dim);
    if (n_rows == 0) return 0;
    if (dim % 4 == 0 && dim >= 512 && dim <= 256 * 4 * 8 && (uintptr_t)x % 16 == 0 && (uintptr_t)y1 % 16 == 0 &&
        (uintptr_t)y2 % 16 == 0) {
        const auto kernel = dim <= 256 * 4 * 2 ? rmsnorm_dual_f32_kernel<2> : dim <= 256 * 4 * 4 ? rmsnorm_dual_f32_kernel<4>
                                                                                                    : rmsnorm_dual_f32_kernel<8>;
        kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, g1, g2, g_dt, eps1, eps2, y1, y2, y_dt, dim);
        NN_LAUNCH_OK("rmsnorm (two outputs)");
        return 0;
    }
    rmsnorm_dual_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, g1, g2, g_dt, eps1, eps2, y1, y2, y_dt, dim);
    NN_LAUNCH_OK("rmsnorm (two outputs)");
    return 0;
}

// ---------------------------------------------------------------------------
// One small product per head: C[m, b, :] = A[m, b, :] . W[b]^T for b < n_batch, with A [M, lda] holding head b's
// K lanes at column b * a_step, W [n_batch, N, K] and C [M, ldc] taking head b's N lanes at column b * c_step.
// With `gate` [M, gate_ld] (32-bit logits) row m of head b is multiplied by sigmoid(gate[m, gate_col + b]).
// 32-bit multiply-add on CUDA cores, k ascending per output element.
// ---------------------------------------------------------------------------
template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
linear_heads_kernel(const void* __restrict__ A, int a_dt, const void* __restrict__ W, int w_dt, void* __restrict__ C,
                    int c_dt, int M, int N, int K, int lda, int ldc, int a_step, int c_step,
                    const float* __restrict__ gate, int gate_ld, int gate_col) {
    constexpr int NT = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x, b = blockIdx.z;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const size_t a0 = (size_t)b * a_step, w0 = (size_t)b * N * K, c0 = (size_t)b * c_step;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += NT) {
            const int r = e / BK, c = e % BK;
            const int m = m0 + r, k = k0 + c;
            As[c][r] = (m < M && k < K) ? ld_f(A, a0 + (size_t)m * lda + k, a_dt) : 0.0f;
        }
        for (int e = tid; e < BN * BK; e += NT) {
            const int r = e / BK, c = e % BK;
            const int n = n0 + r, k = k0 + c;
            Ws[c][r] = (n < N && k < K) ? ld_f(W, w0 + (size_t)n * K + k, w_dt) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
        const float g = gate ? 1.0f / (1.0f + expf(0.0f - gate[(size_t)m * gate_ld + gate_col + b])) : 1.0f;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) st_f(C, c0 + (size_t)m * ldc + n, c_dt, acc[i][j] * g);
        }
    }
}

extern "C" int nncpu_linear_heads(const void* A, int a_dt, const void* W, int w_dt, void* C, int c_dt, int M, int N,
                                  int K, int n_batch, int lda, int ldc, int a_step, int c_step, const float* gate,
                                  int gate_ld, int gate_col, void* stream) {
    NN_CHECK(M >= 0 && N > 0 && K > 0 && n_batch > 0 && n_batch <= 65535, "per-head product: M %d, N %d, K %d, %d heads",
             M, N, K, n_batch);
    NN_CHECK(lda >= (n_batch - 1) * a_step + K && ldc >= (n_batch - 1) * c_step + N && a_step >= 0 && c_step >= N,
             "per-head product: row strides %d / %d for %d heads of %d / %d lanes", lda, ldc, n_batch, K, N);
    NN_CHECK(gate == nullptr || gate_ld >= gate_col + n_batch, "per-head product: gate stride %d", gate_ld);
    if (M == 0) return 0;
    if (M <= 16) {
        dim3 grid((N + 63) / 64, (M + 15) / 16, n_batch);
        linear_heads_kernel<16, 64, 32, 2, 2><<<grid, 256, 0, (cudaStream_t)stream>>>(
            A, a_dt, W, w_dt, C, c_dt, M, N, K, lda, ldc, a_step, c_step, gate, gate_ld, gate_col);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64, n_batch);
        NN_CHECK(grid.y <= 65535, "per-head product: %d rows", M);
        linear_heads_kernel<64, 64, 16, 4, 4><<<grid, 256, 0, (cudaStream_t)stream>>>(
            A, a_dt, W, w_dt, C, c_dt, M, N, K, lda, ldc, a_step, c_step, gate, gate_ld, gate_col);
    }
    NN_LAUNCH_OK("per-head product");
    return 0;
}

// ---------------------------------------------------------------------------
// Latent attention keeps one vector per position: c = rmsnorm(z) * gamma of `rank` lanes, where z sits at column
// `col` of the rows of proj [n_tok, ld] (32-bit).  It goes to the token's row of the key pages (one key/value head);
// the same pages serve as values.  One block per token.  With q_out (bfloat16 [n_tok, q_size]) the
// first q_size columns of the token's row (the queries) are copied there rounded to bfloat16, for the per-head
// products on the tensor cores.
// With rot_dim > 0 the row of proj holds rot_dim more lanes right after z: a key part that all heads share.  Its first
// 2 * rot_half lanes are rotated in neighbouring pairs (2i, 2i + 1) by cs[t, i] = (cos, sin), the rest pass, and the
// part follows c in the page row, which is rank + rot_dim lanes long.  With pages null the layer reads another layer's
// cache and nothing is appended.
// With qn_gamma the queries' own latent is normed too: cq_out[t] = rmsnorm(proj[t, qn_col : qn_col + qn_rank]) * qn_gamma.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
latent_append_kernel(const float* __restrict__ proj, int ld, int col, const void* __restrict__ gamma, int g_dt,
                     float eps, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
                     const int* __restrict__ block_table, int bt_stride, void* __restrict__ pages, int kv_dt,
                     int rank, __nv_bfloat16* __restrict__ q_out, int q_size, int rot_dim,
                     const float2* __restrict__ cs, int rot_half, const void* __restrict__ qn_gamma, int qn_col,
                     int qn_rank, void* __restrict__ cq_out, int cq_dt) {
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    if (q_out != nullptr)
        for (int i = threadIdx.x; i < q_size; i += blockDim.x)
            q_out[(size_t)t * q_size + i] = __float2bfloat16_rn(proj[(size_t)t * ld + i]);
    if (qn_gamma != nullptr) {
        const float* zq = proj + (size_t)t * ld + qn_col;
        float sq = 0.0f;
        for (int i = threadIdx.x; i < qn_rank; i += blockDim.x) sq = fmaf(zq[i], zq[i], sq);
        sq = block_sum(sq, scratch);
        const float sc = 1.0f / sqrtf(sq * (1.0f / (float)qn_rank) + eps);
        for (int i = threadIdx.x; i < qn_rank; i += blockDim.x)
            st_f(cq_out, (size_t)t * qn_rank + i, cq_dt, (zq[i] * sc) * ld_f(qn_gamma, i, g_dt));
    }
    const int seq = tok_seq[t];
    if (seq < 0 || pages == nullptr) return;   // a padded row owns no place in the cache
    const float* z = proj + (size_t)t * ld + col;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < rank; i += blockDim.x) ss = fmaf(z[i], z[i], ss);
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss * (1.0f / (float)rank) + eps);
    const int pos = tok_pos[t];
    const int page = block_table[(size_t)seq * bt_stride + pos / kPage];
    if (page < 0) return;
    const size_t o = ((size_t)page * kPage + pos % kPage) * (size_t)(rank + rot_dim);
    for (int i = threadIdx.x; i < rank; i += blockDim.x) st_f(pages, o + i, kv_dt, (z[i] * scale) * ld_f(gamma, i, g_dt));
    const float* zr = z + rank;
    for (int i = threadIdx.x; i < rot_half; i += blockDim.x) {
        const float2 c = cs[(size_t)t * rot_half + i];
        const float u = zr[2 * i], v = zr[2 * i + 1];
        st_f(pages, o + rank + 2 * i, kv_dt, c.x * u - c.y * v);
        st_f(pages, o + rank + 2 * i + 1, kv_dt, c.x * v + c.y * u);
    }
    for (int i = 2 * rot_half + threadIdx.x; i < rot_dim; i += blockDim.x) st_f(pages, o + rank + i, kv_dt, zr[i]);
}

extern "C" int nncpu_latent_append(const float* proj, int ld, int col, const void* gamma, int g_dt, float eps,
                                   const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride,
                                   void* pages, int kv_dt, int n_tok, int rank, void* q_out, int q_size, int rot_dim,
                                   const float* cs, int rot_half, const void* qn_gamma, int qn_col, int qn_rank,
                                   void* cq_out, int cq_dt, void* stream) {
    NN_CHECK(n_tok >= 0 && rank > 0 && col >= 0 && rot_dim >= 0 && (pages == nullptr || ld >= col + rank + rot_dim),
             "latent append: %d tokens, rank %d + %d at column %d of %d", n_tok, rank, rot_dim, col, ld);
    NN_CHECK(q_out == nullptr || (q_size > 0 && q_size <= ld), "latent append: %d query lanes of a row of %d", q_size, ld);
    NN_CHECK(rot_half >= 0 && 2 * rot_half <= rot_dim && (rot_half == 0 || cs != nullptr) && (uintptr_t)cs % 8 == 0,
             "latent append: %d rotated pairs of %d lanes", rot_half, rot_dim);
    NN_CHECK(qn_gamma == nullptr || (qn_rank > 0 && qn_col >= 0 && qn_col + qn_rank <= ld && cq_out != nullptr),
             "latent append: a query latent of %d lanes at column %d of %d", qn_rank, qn_col, ld);
    if (n_tok == 0) return 0;
    latent_append_kernel<<<n_tok, 128, 0, (cudaStream_t)stream>>>(proj, ld, col, gamma, g_dt, eps, tok_seq, tok_pos,
                                                                  block_table, bt_stride, pages, kv_dt, rank,
                                                                  (__nv_bfloat16*)q_out, q_size, rot_dim,
                                                                  (const float2*)cs, rot_half, qn_gamma, qn_col, qn_rank,
                                                                  cq_out, cq_dt);
    NN_LAUNCH_OK("latent append");
    return 0;
}

// ---------------------------------------------------------------------------
// The queries of latent attention with a rotated part: q [n_tok, n_heads * (hd + rot_dim)] (32-bit) holds, head by
// head, hd unrotated lanes and then rot_dim lanes of which the first 2 * rot_half are rotated in neighbouring pairs
// by cs[t, i].  The rotated part goes to q_lat[t, head, rank : rank + rot_dim] (rows of n_heads * (rank + rot_dim)
// lanes; the first `rank` lanes of a head are the per-head product's to fill).  With q16 the whole row of q is also
// left there rounded to bfloat16, for that product on the tensor cores.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
latent_query_kernel(const float* __restrict__ q, int n_heads, int hd, int rot_dim, const float2* __restrict__ cs,
                    int rot_half, void* __restrict__ q_lat, int lat_dt, int rank, __nv_bfloat16* __restrict__ q16) {
    const int t = blockIdx.x;
    const int per = hd + rot_dim;
    const float* row = q + (size_t)t * n_heads * per;
    if (q16 != nullptr)
        for (int i = threadIdx.x; i < n_heads * per; i += blockDim.x)
            q16[(size_t)t * n_heads * per + i] = __float2bfloat16_rn(row[i]);
    const size_t o = (size_t)t * n_heads * (rank + rot_dim);
    for (int idx = threadIdx.x; idx < n_heads * rot_half; idx += blockDim.x) {
        const int a = idx / rot_half, i = idx % rot_half;
        const float2 c = cs[(size_t)t * rot_half + i];
        const float u = row[a * per + hd + 2 * i], v = row[a * per + hd + 2 * i + 1];
        st_f(q_lat, o + (size_t)a * (rank + rot_dim) + rank + 2 * i, lat_dt, c.x * u - c.y * v);
        st_f(q_lat, o + (size_t)a * (rank + rot_dim) + rank + 2 * i + 1, lat_dt, c.x * v + c.y * u);
    }
    const int rest = rot_dim - 2 * rot_half;
    for (int idx = threadIdx.x; idx < n_heads * rest; idx += blockDim.x) {
        const int a = idx / rest, i = 2 * rot_half + idx % rest;
        st_f(q_lat, o + (size_t)a * (rank + rot_dim) + rank + i, lat_dt, row[a * per + hd + i]);
    }
}

extern "C" int nncpu_latent_query(const float* q, int n_tok, int n_heads, int hd, int rot_dim, const float* cs,
                                  int rot_half, void* q_lat, int lat_dt, int rank, void* q16, void* stream) {
    NN_CHECK(n_tok >= 0 && n_heads > 0 && hd > 0 && rot_dim >= 0 && rank > 0, "latent query: sizes");
    NN_CHECK(rot_half >= 0 && 2 * rot_half <= rot_dim && (rot_half == 0 || cs != nullptr) && (uintptr_t)cs % 8 == 0,
             "latent query: %d rotated pairs of %d lanes", rot_half, rot_dim);
    if (n_tok == 0) return 0;
    latent_query_kernel<<<n_tok, 128, 0, (cudaStream_t)stream>>>(q, n_heads, hd, rot_dim, (const float2*)cs, rot_half,
                                                                 q_lat, lat_dt, rank, (__nv_bfloat16*)q16);
    NN_LAUNCH_OK("latent query");
    return 0;
}

// ---------------------------------------------------------------------------
// An elementwise gate: x[t, i] *= sigmoid(g[t, col + i]) for i < width; x in either element type, g 32-bit with
// rows of ld lanes.  The sigmoid and the product are 32-bit.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(void* __restrict__ x, int x_dt, const float* __restrict__ g, int ld, int col, long n_tok, int width) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tok * width) return;
    const long t = idx / width;
    const int i = (int)(idx % width);
    const float z = g[(size_t)t * ld + col + i];
    st_f(x, idx, x_dt, ld_f(x, idx, x_dt) * (1.0f / (1.0f + expf(0.0f - z))));
}

extern "C" int nncpu_sigmoid_gate(void* x, int x_dt, const float* g, int ld, int col, int n_tok, int width, void* stream) {
    NN_CHECK(n_tok >= 0 && width > 0 && col >= 0 && ld >= col + width, "sigmoid gate: %d lanes at column %d of %d", width, col, ld);
    if (n_tok == 0) return 0;
    const long total = (long)n_tok * width;
    sigmoid_gate_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, x_dt, g, ld, col, n_tok, width);
    NN_LAUNCH_OK("sigmoid gate");
    return 0;
}

// ---------------------------------------------------------------------------
// Routed experts.
//   route: per token the `top` largest of its n_experts router logits (the lower index wins a tie), in descending
//     order, and the softmax over those logits alone.  One warp per token, 32-bit.
//   gate/up: for slot s = (token t, choice c) with expert e: act[s, j] = gated_act(Wg[e, j] . h_t, Wu[e, j] . h_t).
//   down: out[t, i] += sum_c weight[t, c] * (Wd[e_c, i] . act[(t, c)]), choices added in their order.
// The two products keep a warp on an output feature, lanes across k, and add in a fixed order, so a token's result
// does not depend on the batch.  They serve every size and element type; weights are [n_experts, rows, cols].
// ---------------------------------------------------------------------------
constexpr int kRouteMaxExperts = 1024;

// One warp picks the top of z[0 .. n_experts) (shared memory; taken entries are overwritten).
__device__ __forceinline__ void route_top(float* z, int n_experts, int top, int* __restrict__ ids,
                                          float* __restrict__ weights, int lane) {
    float z_first = 0.0f, sum = 0.0f;
    for (int c = 0; c < top; ++c) {
        float best = -INFINITY;
        int at = n_experts;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }   // NaN never wins; -inf only by index order
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= n_experts) at = 0;            // nothing but NaN is left: garbage in, an expert that exists out
        if (c == 0) z_first = best;
        const float w = expf(best - z_first);
        sum += w;
        if (lane == 0) {
            ids[c] = at;
            weights[c] = w;
            z[at] = __int_as_float(0x7FC00000);   // taken: NaN loses every comparison above
        }
        __syncwarp();
    }
    const float inv = 1.0f / sum;
    for (int c = lane; c < top; c += 32) weights[c] *= inv;
}

// Scores over ALL experts: s = softmax(z).  The experts form n_groups equal groups of neighbours; a group's score is its
// largest score, and only experts of the `keep` best groups can be chosen (n_groups <= 1: no groups).  The weights of the
// chosen are their scores divided by the sum of the chosen scores (+ 1e-20), times `scale`.  One warp; z is overwritten;
// gbuf holds n_groups floats.  The softmax does not change an order, so groups and experts are picked by their logits.
__device__ __forceinline__ void route_top_all(float* z, float* gbuf, int n_experts, int top, int n_groups, int keep,
                                              float scale, int* __restrict__ ids, float* __restrict__ weights, int lane) {
    float zmax = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float den = 0.0f;
    for (int e = lane; e < n_experts; e += 32) den += expf(z[e] - zmax);
    den = warp_sum(den);
    if (n_groups > 1 && keep < n_groups) {
        const int per = n_experts / n_groups;
        for (int g = lane; g < n_groups; g += 32) {
            float m = -INFINITY;
            for (int j = 0; j < per; ++j) m = fmaxf(m, z[g * per + j]);
            gbuf[g] = m;
        }
        __syncwarp();
        for (int c = 0; c < keep; ++c) {
            float best = -INFINITY;
            int at = n_groups;
            for (int g = lane; g < n_groups; g += 32) {
                const float v = gbuf[g];
                if (v > best || (v == best && g < at)) { best = v; at = g; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (at < n_groups && lane == 0) gbuf[at] = __int_as_float(0x7FC00000);    // kept: NaN marks it
            __syncwarp();
        }
        for (int e = lane; e < n_experts; e += 32)
            if (gbuf[e / per] == gbuf[e / per]) z[e] = __int_as_float(0x7FC00000);      // not kept: cannot be chosen
        __syncwarp();
    }
    float sum = 0.0f;
    for (int c = 0; c < top; ++c) {
        float best = -INFINITY;
        int at = n_experts;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = z[e];
            if (v > best || (v == best && e < at)) { best = v; at = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= n_experts) at = 0;
        const float w = expf(best - zmax) / den;
        sum += w;
        if (lane == 0) {
            ids[c] = at;
            weights[c] = w;
            z[at] = __int_as_float(0x7FC00000);
        }
        __syncwarp();
    }
    const float inv = scale / (sum + 1e-20f);
    for (int c = lane; c < top; c += 32) weights[c] *= inv;
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, int n_tok, int n_experts, int top, int* __restrict__ ids,
                 float* __restrict__ weights, int all_scores, int n_groups, int keep, float scale) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= n_tok) return;
    float* z = smem + (size_t)warp * (n_experts + n_groups);
    for (int e = lane; e < n_experts; e += 32) z[e] = logits[(size_t)t * n_experts + e];
    __syncwarp();
    if (all_scores)
        route_top_all(z, z + n_experts, n_experts, top, n_groups, keep, scale, ids + (size_t)t * top,
                      weights + (size_t)t * top, lane);
    else
        route_top(z, n_experts, top, ids + (size_t)t * top, weights + (size_t)t * top, lane);
}

// Whether a choice among groups can be made: equal groups, and the kept ones hold enough experts.
static bool route_groups_ok(int n_experts, int top, int n_groups, int keep) {
    if (n_groups <= 1) return true;
    return n_experts % n_groups == 0 && keep >= 1 && keep <= n_groups && (long)keep * (n_experts / n_groups) >= top;
}

extern "C" int nncpu_moe_route(const float* logits, int n_tok, int n_experts, int top, int* ids, float* weights,
                               int all_scores, int n_groups, int keep, float scale, void* stream) {
    NN_CHECK(n_tok >= 0 && n_experts > 0 && n_experts <= kRouteMaxExperts && top > 0 && top <= n_experts,
             "router: %d tokens, the top %d of %d experts (at most %d)", n_tok, top, n_experts, kRouteMaxExperts);
    NN_CHECK(all_scores ? route_groups_ok(n_experts, top, n_groups, keep) : n_groups <= 1,
             "router: the %d best of %d groups of %d experts for the top %d", keep, n_groups, n_experts, top);
    if (n_tok == 0) return 0;
    if (n_groups < 1) n_groups = 1;
    const size_t smem = (size_t)4 * (n_experts + n_groups) * sizeof(float);
    moe_route_kernel<<<(n_tok + 3) / 4, 128, smem, (cudaStream_t)stream>>>(logits, n_tok, n_experts, top, ids, weights,
                                                                          all_scores, n_groups, keep, scale);
    NN_LAUNCH_OK("router");
    return 0;
}

// A warp's dot product of a weight row with a vector held in shared memory as floats.
__device__ __forceinline__ float warp_dot(const void* __restrict__ w, size_t row_at, int w_dt, const float* __restrict__ x,
                                          int k, int lane) {
    float acc = 0.0f;
    if (w_dt == DT_BF16 && (k & 7) == 0 && (row_at & 7) == 0) {
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(w) + row_at);
        const int n8 = k >> 3;
        // four 16-byte loads of a lane are asked for before the first is used
        for (int i0 = lane; i0 < n8; i0 += 128) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = i0 + 32 * u < n8 ? src[i0 + 32 * u] : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (i0 + 32 * u >= n8) break;
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[u]);
                const float* xs = x + 8 * (i0 + 32 * u);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    acc = fmaf(f.x, xs[2 * j], acc);
                    acc = fmaf(f.y, xs[2 * j + 1], acc);
                }
            }
        }
    } else {
        for (int i = lane; i < k; i += 32) acc = fmaf(ld_f(w, row_at + i, w_dt), x[i], acc);
    }
    return warp_sum(acc);
}

// The router in one launch: z = W_r x + b in 32-bit (a warp per expert's row, lanes across k), then the choice.
// One block per token; x [n_tok, width] of either type, W_r [n_experts, width], b [n_experts].
__global__ void __launch_bounds__(256)
moe_router_kernel(const void* __restrict__ x, int x_dt, const void* __restrict__ w, int w_dt, const void* __restrict__ bias,
                  int b_dt, int n_tok, int per_block, int n_experts, int top, int width, int* __restrict__ ids,
                  float* __restrict__ weights, int all_scores, int n_groups, int keep, float scale) {
    extern __shared__ float smem[];          // a token's input, then its logits
    float* z = smem + width;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    // a block takes `per_block` tokens one after the other, so that the router's rows come from L1 after the first
    for (int t = blockIdx.x * per_block; t < min(n_tok, (int)(blockIdx.x + 1) * per_block); ++t) {
        for (int i = threadIdx.x; i < width; i += blockDim.x) smem[i] = ld_f(x, (size_t)t * width + i, x_dt);
        __syncthreads();
        for (int e = warp; e < n_experts; e += n_warps) {
            const float d = warp_dot(w, (size_t)e * width, w_dt, smem, width, lane);
            if (lane == 0) z[e] = d + (bias ? ld_f(bias, e, b_dt) : 0.0f);
        }
        __syncthreads();
        if (warp == 0) {
            if (all_scores)
                route_top_all(z, z + n_experts, n_experts, top, n_groups, keep, scale, ids + (size_t)t * top,
                              weights + (size_t)t * top, lane);
            else
                route_top(z, n_experts, top, ids + (size_t)t * top, weights + (size_t)t * top, lane);
        }
        __syncthreads();
    }
}

extern "C" int nncpu_moe_router_fits(int n_experts, int width) {
    return n_experts > 0 && n_experts <= kRouteMaxExperts && (size_t)(width + 2 * n_experts) * 4 <= 48 * 1024;
}

extern "C" int nncpu_moe_router(const void* x, int x_dt, const void* w, int w_dt, const void* bias, int b_dt, int n_tok,
                                int n_experts, int top, int width, int* ids, float* weights, int all_scores, int n_groups,
                                int keep, float scale, void* stream) {
    NN_CHECK(n_tok >= 0 && width > 0 && top > 0 && top <= n_experts && nncpu_moe_router_fits(n_experts, width),
             "router: %d tokens of %d, the top %d of %d experts", n_tok, width, top, n_experts);
    NN_CHECK(all_scores ? route_groups_ok(n_experts, top, n_groups, keep) : n_groups <= 1,
             "router: the %d best of %d groups of %d experts for the top %d", keep, n_groups, n_experts, top);
    if (n_tok == 0) return 0;
    if (n_groups < 1) n_groups = 1;
    // One token a block: with several a block the router's rows did not stay in L1 and the grid got too small
    // (2 048 tokens of 4 096 lanes, 16 experts: 88 us a launch with one token a block, 124 us with eight).
    const int per_block = 1;
    moe_router_kernel<<<(n_tok + per_block - 1) / per_block, 256, (size_t)(width + n_experts + n_groups) * 4, (cudaStream_t)stream>>>(
        x, x_dt, w, w_dt, bias, b_dt, n_tok, per_block, n_experts, top, width, ids, weights, all_scores, n_groups, keep, scale);
    NN_LAUNCH_OK("router");
    return 0;
}

constexpr int kMoeWarps = 8;

__global__ void __launch_bounds__(kMoeWarps * 32)
moe_gate_up_kernel(const void* __restrict__ x, int x_dt, const void* __restrict__ wg, const void* __restrict__ wu,
                   int w_dt, const int* __restrict__ ids, void* __restrict__ act, int act_dt, int top, int width, int ff,
                   int n_experts, int kind, float limit) {
    // wu null: wg holds [n_experts, 2 ff, width] with an expert's gate and up rows interleaved in blocks of 8 (the
    // layout of the tensor-core products' gated epilogue): gate row j is row 16 (j / 8) + j % 8, up row j eight below
    extern __shared__ float smem[];          // the token's input as floats
    const int s = blockIdx.x, t = s / top;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = ids[s];
    for (int i = threadIdx.x; i < width; i += blockDim.x) smem[i] = ld_f(x, (size_t)t * width + i, x_dt);
    __syncthreads();
    if (e < 0 || e >= n_experts) return;
    const bool mixed = wu == nullptr;
    const size_t w0 = (size_t)e * ff * width * (mixed ? 2 : 1);
    for (int j = blockIdx.y * kMoeWarps + warp; j < ff; j += gridDim.y * kMoeWarps) {
        const size_t row = mixed ? (size_t)(((j >> 3) << 4) + (j & 7)) : (size_t)j;
        const float g = warp_dot(wg, w0 + row * width, w_dt, smem, width, lane);
        const float u = mixed ? warp_dot(wg, w0 + (row + 8) * width, w_dt, smem, width, lane)
                              : warp_dot(wu, w0 + row * width, w_dt, smem, width, lane);
        if (lane == 0) st_f(act, (size_t)s * ff + j, act_dt, gated_act_f(g, u, kind, limit));
    }
}

__global__ void __launch_bounds__(kMoeWarps * 32)
moe_down_kernel(const void* __restrict__ act, int act_dt, const void* __restrict__ wd, int w_dt,
                const int* __restrict__ ids, const float* __restrict__ weights, float* __restrict__ out, int top,
                int width, int ff, int n_experts) {
    extern __shared__ float smem[];          // the token's top * ff activations as floats
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < top * ff; i += blockDim.x) smem[i] = ld_f(act, (size_t)t * top * ff + i, act_dt);
    __syncthreads();
    for (int i = blockIdx.y * kMoeWarps + warp; i < width; i += gridDim.y * kMoeWarps) {
        float sum = 0.0f;
        for (int c = 0; c < top; ++c) {
            const int e = ids[(size_t)t * top + c];
            if (e < 0 || e >= n_experts) continue;
            const float d = warp_dot(wd, ((size_t)e * width + i) * ff, w_dt, smem + (size_t)c * ff, ff, lane);
            sum = fmaf(weights[(size_t)t * top + c], d, sum);
        }
        if (lane == 0) out[(size_t)t * width + i] += sum;
    }
}

extern "C" int nncpu_moe_experts(const void* x, int x_dt, const void* wg, const void* wu, const void* wd, int w_dt,
                                 const int* ids, const float* weights, void* act, int act_dt, float* out, int n_tok,
                                 int top, int width, int ff, int n_experts, int kind, float limit, void* stream) {
    NN_CHECK(n_tok >= 0 && top > 0 && width > 0 && ff > 0 && n_experts > 0, "experts: %d tokens, top %d, %d x %d, %d experts",
             n_tok, top, width, ff, n_experts);
    NN_CHECK(kind >= kGateSilu && kind <= kGateSwishClamp, "experts: activation kind %d", kind);
    NN_CHECK(wu != nullptr || ff % 8 == 0, "experts: interleaved gate and up rows need a multiple of 8 of them (%d)", ff);
    constexpr size_t kMost = 200 * 1024;
    NN_CHECK((size_t)width * 4 <= kMost && (size_t)top * ff * 4 <= kMost,
             "experts: a token's %d inputs or %d x %d activations do not fit the shared memory of this kernel", width, top, ff);
    if (n_tok == 0) return 0;
    static bool configured[64] = {};
    if (first_use_on_this_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(moe_gate_up_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMost);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(moe_down_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMost);
        NN_CHECK(e == cudaSuccess, "experts: cannot reserve %zu bytes of shared memory: %s", kMost, cudaGetErrorString(e));
    }
    const long slots = (long)n_tok * top;
    NN_CHECK(slots < (1l << 31), "experts: %ld token slots", slots);
    // few tokens: more blocks per token, so that the weights' stream is spread over the SMs
    const int split_up = (int)max(1l, min((long)(ff + kMoeWarps - 1) / kMoeWarps, 1024 / max(1l, slots)));
    const int split_down = (int)max(1l, min((long)(width + kMoeWarps - 1) / kMoeWarps, 1024 / max(1l, (long)n_tok)));
    moe_gate_up_kernel<<<dim3((unsigned)slots, split_up), kMoeWarps * 32, (size_t)width * 4, (cudaStream_t)stream>>>(
        x, x_dt, wg, wu, w_dt, ids, act, act_dt, top, width, ff, n_experts, kind, limit);
    NN_LAUNCH_OK("experts (gate and up)");
    moe_down_kernel<<<dim3(n_tok, split_down), kMoeWarps * 32, (size_t)top * ff * 4, (cudaStream_t)stream>>>(
        act, act_dt, wd, w_dt, ids, weights, out, top, width, ff, n_experts);
    NN_LAUNCH_OK("experts (down)");
    return 0;
}

// ---------------------------------------------------------------------------
// Routed experts for many tokens: the token slots (token, choice) are sorted by expert, the experts' products run
// as one grouped product on the tensor cores (gemm_sm100.cu), and the choices of a token are added up afterwards.
//   plan: counts the slots of every expert, gives every slot a row (its expert's rows follow one another; the order
//     inside an expert is whatever the atomics give, which changes no result: a row's product does not depend on its
//     place), and lists the 128-row tiles of the grouped product.  One block.
//   gather: xs[row] = x[slot_of_row[row] / top].
//   combine: out[t] += sum_c weight[t, c] * y[row_of_slot[t * top + c]], choices in their order.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int n_slots, int n_experts, int* __restrict__ row_of_slot,
                int* __restrict__ slot_of_row, int* __restrict__ n_tiles, int* __restrict__ tile_group,
                int* __restrict__ tile_row0, int* __restrict__ tile_row_end, int max_tiles) {
    extern __shared__ int plan_smem[];
    int* count = plan_smem;
    int* offset = plan_smem + n_experts;
    int* cursor = plan_smem + 2 * n_experts;
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) count[e] = cursor[e] = 0;
    __syncthreads();
    for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
        const int e = ids[s];
        if (e >= 0 && e < n_experts) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0, tiles = 0;
        for (int e = 0; e < n_experts; ++e) {
            offset[e] = acc;
            for (int r = 0; r < count[e]; r += 128, ++tiles) {
                if (tiles < max_tiles) {
                    tile_group[tiles] = e;
                    tile_row0[tiles] = acc + r;
                    tile_row_end[tiles] = acc + count[e];
                }
            }
            acc += count[e];
        }
        *n_tiles = tiles < max_tiles ? tiles : max_tiles;
    }
    __syncthreads();
    for (int s = threadIdx.x; s < n_slots; s += blockDim.x) {
        const int e = ids[s];
        if (e < 0 || e >= n_experts) { row_of_slot[s] = -1; continue; }
        const int row = offset[e] + atomicAdd(&cursor[e], 1);
        row_of_slot[s] = row;
        slot_of_row[row] = s;
    }
}

extern "C" int nncpu_moe_plan(const int* ids, int n_slots, int n_experts, int* row_of_slot, int* slot_of_row,
                              int* n_tiles, int* tile_group, int* tile_row0, int* tile_row_end, int max_tiles,
                              void* stream) {
    NN_CHECK(n_slots > 0 && n_experts > 0 && n_experts <= kRouteMaxExperts && max_tiles >= (n_slots + 127) / 128 + n_experts,
             "experts (plan): %d slots, %d experts, room for %d tiles", n_slots, n_experts, max_tiles);
    moe_plan_kernel<<<1, 1024, (size_t)3 * n_experts * sizeof(int), (cudaStream_t)stream>>>(
        ids, n_slots, n_experts, row_of_slot, slot_of_row, n_tiles, tile_group, tile_row0, tile_row_end, max_tiles);
    NN_LAUNCH_OK("experts (plan)");
    return 0;
}

__global__ void __launch_bounds__(256)
moe_gather_kernel(const void* __restrict__ x, int x_dt, const int* __restrict__ slot_of_row, int top,
                  __nv_bfloat16* __restrict__ xs, int width) {
    const int row = blockIdx.x;
    const int t = slot_of_row[row] / top;
    if (x_dt == DT_BF16 && (width & 7) == 0) {
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(x) + (size_t)t * width);
        uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)row * width);
        for (int i = threadIdx.x; i < (width >> 3); i += blockDim.x) dst[i] = src[i];
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x)
            xs[(size_t)row * width + i] = __float2bfloat16_rn(ld_f(x, (size_t)t * width + i, x_dt));
    }
}

extern "C" int nncpu_moe_gather(const void* x, int x_dt, const int* slot_of_row, int top, void* xs, int n_slots,
                                int width, void* stream) {
    NN_CHECK(n_slots > 0 && top > 0 && width > 0, "experts (gather): %d slots of %d", n_slots, width);
    moe_gather_kernel<<<n_slots, 256, 0, (cudaStream_t)stream>>>(x, x_dt, slot_of_row, top, (__nv_bfloat16*)xs, width);
    NN_LAUNCH_OK("experts (gather)");
    return 0;
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const void* __restrict__ y, int y_dt, const int* __restrict__ row_of_slot,
                   const float* __restrict__ weights, float* __restrict__ out, int top, int width) {
    const int t = blockIdx.x;
    if (y_dt == DT_F32 && (width & 3) == 0) {
        // 16 bytes a thread; the choices' rows are asked for one after the other and added in their order
        const float* yf = reinterpret_cast<const float*>(y);
        for (int i = threadIdx.x; i < (width >> 2); i += blockDim.x) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            for (int c = 0; c < top; ++c) {
                const int row = row_of_slot[(size_t)t * top + c];
                if (row < 0) continue;
                const float w = weights[(size_t)t * top + c];
                const float4 v = reinterpret_cast<const float4*>(yf + (size_t)row * width)[i];
                sum.x = fmaf(w, v.x, sum.x); sum.y = fmaf(w, v.y, sum.y);
                sum.z = fmaf(w, v.z, sum.z); sum.w = fmaf(w, v.w, sum.w);
            }
            float4* o = reinterpret_cast<float4*>(out + (size_t)t * width) + i;
            float4 was = *o;
            was.x += sum.x; was.y += sum.y; was.z += sum.z; was.w += sum.w;
            *o = was;
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float sum = 0.0f;
        for (int c = 0; c < top; ++c) {
            const int row = row_of_slot[(size_t)t * top + c];
            if (row >= 0) sum = fmaf(weights[(size_t)t * top + c], ld_f(y, (size_t)row * width + i, y_dt), sum);
        }
        out[(size_t)t * width + i] += sum;
    }
}

extern "C" int nncpu_moe_combine(const void* y, int y_dt, const int* row_of_slot, const float* weights, float* out,
                                 int n_tok, int top, int width, void* stream) {
    NN_CHECK(n_tok > 0 && top > 0 && width > 0, "experts (combine): %d tokens of %d", n_tok, width);
    moe_combine_kernel<<<n_tok, 256, 0, (cudaStream_t)stream>>>(y, y_dt, row_of_slot, weights, out, top, width);
    NN_LAUNCH_OK("experts (combine)");
    return 0;
}

// ---------------------------------------------------------------------------
// Layer norm over the last axis with weight and bias: y = (x - mean) / sqrt(var + eps) * w + b, where var is the
// mean of the squared deviations from the mean (two passes: the mean first, then the deviations).  x float32;
// `rows` (optional) picks input rows; a negative row gives zeros.  32-bit throughout.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
layernorm_kernel(const float* __restrict__ x, const void* __restrict__ w, const void* __restrict__ b, int p_dt,
                 void* __restrict__ y, int y_dt, const int* __restrict__ rows, int dim, float eps) {
    __shared__ float scratch[33];
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    if (r_in < 0) {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) st_f(y, (size_t)r_out * dim + i, y_dt, 0.0f);
        return;
    }
    const float* src = x + (size_t)r_in * dim;
    float s = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) s += src[i];
    const float mean = block_sum(s, scratch) * (1.0f / (float)dim);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float c = src[i] - mean;
        ss = fmaf(c, c, ss);
    }
    const float scale = 1.0f / sqrtf(block_sum(ss, scratch) * (1.0f / (float)dim) + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = (src[i] - mean) * scale;
        if (w) v *= ld_f(w, i, p_dt);
        if (b) v += ld_f(b, i, p_dt);
        st_f(y, (size_t)r_out * dim + i, y_dt, v);
    }
}

// The common case, rows of a width that is a multiple of 4 and at most 256 * 4 * kVec: every thread keeps its part of
// the row in registers between the mean, the deviations and the scaling, so the row is read once, 16 bytes at a time.
template <int kVec>
__global__ void __launch_bounds__(256)
layernorm_f32_kernel(const float* __restrict__ x, const void* __restrict__ w, const void* __restrict__ b, int p_dt,
                     void* __restrict__ y, int y_dt, const int* __restrict__ rows, int dim, float eps) {
    __shared__ float scratch[33];
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    const int n4 = dim >> 2;
    float4 v[kVec];
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        v[j] = (r_in >= 0 && i < n4) ? reinterpret_cast<const float4*>(x + (size_t)r_in * dim)[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = block_sum(s, scratch) * (1.0f / (float)dim);
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        if (threadIdx.x + j * 256 >= n4) continue;
        v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
        ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
    }
    const float scale = r_in >= 0 ? 1.0f / sqrtf(block_sum(ss, scratch) * (1.0f / (float)dim) + eps) : 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        float o[4] = {v[j].x * scale, v[j].y * scale, v[j].z * scale, v[j].w * scale};
        if (r_in >= 0) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                if (w) o[e] *= ld_f(w, 4 * i + e, p_dt);
                if (b) o[e] += ld_f(b, 4 * i + e, p_dt);
            }
        }
        const size_t at = (size_t)r_out * dim + 4 * i;
        if (y_dt == DT_BF16) {
            __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(y) + at) = *reinterpret_cast<uint2*>(h);
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(y) + at) = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

extern "C" int nncpu_layernorm(const float* x, const void* w, const void* b, int p_dt, void* y, int y_dt,
                               const int* rows, int n_rows, int dim, float eps, void* stream) {
    NN_CHECK(n_rows >= 0 && dim > 0, "layernorm: %d rows of %d", n_rows, dim);
    if (n_rows == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (dim % 4 == 0 && dim <= 256 * 4 * 8 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)y % 16) == 0) {
        if (dim <= 1024) layernorm_f32_kernel<1><<<n_rows, 256, 0, st>>>(x, w, b, p_dt, y, y_dt, rows, dim, eps);
        else if (dim <= 2048) layernorm_f32_kernel<2><<<n_rows, 256, 0, st>>>(x, w, b, p_dt, y, y_dt, rows, dim, eps);
        else if (dim <= 4096) layernorm_f32_kernel<4><<<n_rows, 256, 0, st>>>(x, w, b, p_dt, y, y_dt, rows, dim, eps);
        else layernorm_f32_kernel<8><<<n_rows, 256, 0, st>>>(x, w, b, p_dt, y, y_dt, rows, dim, eps);
        NN_LAUNCH_OK("layernorm");
        return 0;
    }
    layernorm_kernel<<<n_rows, 256, 0, (cudaStream_t)stream>>>(x, w, b, p_dt, y, y_dt, rows, dim, eps);
    NN_LAUNCH_OK("layernorm");
    return 0;
}

// ---------------------------------------------------------------------------
// A hashed embedding of the pair (previous token, token): out[t, :] += table[row, :] with
// row = (prev * mul_prev + id * mul_cur) mod buckets, and row = buckets (the table's last row) for a sequence's first
// token.  The previous token of a step's first token is what `last` [slots + 1] holds for the sequence's slot; the
// block of that token also leaves the sequence's last token of this step there (it is the only block that reads or
// writes the slot's entry in the step).  A token of no sequence (tok_seq < 0) is left as it is.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
pair_embed_kernel(const void* __restrict__ table, int table_dt, const int* __restrict__ ids,
                  const int* __restrict__ tok_seq, const int* __restrict__ tok_pos, const int* __restrict__ cu_seqlens,
                  const int* __restrict__ seq_slots, int* last, float* __restrict__ out, int hidden, long long buckets,
                  long long mul_prev, long long mul_cur) {
    __shared__ int s_prev;
    const int t = blockIdx.x;
    const int seq = tok_seq[t];
    if (seq < 0) return;
    const int slot = seq_slots[seq];
    if (slot < 0) return;
    const int first = cu_seqlens[seq];
    const int id = ids[t];
    if (threadIdx.x == 0) {
        if (t > first) {
            s_prev = ids[t - 1];
        } else {
            s_prev = tok_pos[t] == 0 ? -1 : last[slot];
            last[slot] = ids[cu_seqlens[seq + 1] - 1];
        }
    }
    __syncthreads();
    const int prev = s_prev;
    const long long row = prev < 0 ? buckets : ((long long)prev * mul_prev + (long long)id * mul_cur) % buckets;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        out[(size_t)t * hidden + i] += ld_f(table, (size_t)row * hidden + i, table_dt);
}

extern "C" int nncpu_pair_embed(const void* table, int table_dt, const int* ids, const int* tok_seq, const int* tok_pos,
                                const int* cu_seqlens, const int* seq_slots, int* last, float* out, int n_tok,
                                int hidden, long buckets, long mul_prev, long mul_cur, void* stream) {
    NN_CHECK(n_tok >= 0 && hidden > 0 && buckets > 0 && mul_prev >= 0 && mul_cur >= 0,
             "pair embedding: %d tokens of %d, %ld buckets", n_tok, hidden, buckets);
    if (n_tok == 0) return 0;
    pair_embed_kernel<<<n_tok, 256, 0, (cudaStream_t)stream>>>(table, table_dt, ids, tok_seq, tok_pos, cu_seqlens,
                                                               seq_slots, last, out, hidden, buckets, mul_prev, mul_cur);
    NN_LAUNCH_OK("pair embedding");
    return 0;
}

// ---------------------------------------------------------------------------
// out[t, :] = [a[t, :], b[t, :]] in the element type of out (b may be null: a plain conversion).  a, b float32.
// ---------------------------------------------------------------------------
__global__ void concat_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, void* __restrict__ out,
                                   int out_dt, long total, int dim) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int wide = b ? 2 * dim : dim;
    const long t = idx / wide;
    const int i = (int)(idx % wide);
    st_f(out, (size_t)idx, out_dt, i < dim ? a[(size_t)t * dim + i] : b[(size_t)t * dim + i - dim]);
}

extern "C" int nncpu_concat_rows(const float* a, const float* b, void* out, int out_dt, int n_tok, int dim, void* stream) {
    NN_CHECK(n_tok >= 0 && dim > 0, "concat: %d rows of %d", n_tok, dim);
    if (n_tok == 0) return 0;
    const long total = (long)n_tok * dim * (b ? 2 : 1);
    concat_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, b, out, out_dt, total, dim);
    NN_LAUNCH_OK("concat");
    return 0;
}

// ---------------------------------------------------------------------------
// x[t, :] += alpha * y[t, :] (float32): a sublayer's branch joins the residual stream with a weight.
// ---------------------------------------------------------------------------
__global__ void stream_axpy_kernel(float* __restrict__ x, const float* __restrict__ y, float alpha, long total) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) x[idx] = fmaf(alpha, y[idx], x[idx]);
}

extern "C" int nncpu_stream_axpy(float* x, const float* y, float alpha, long total, void* stream) {
    NN_CHECK(total >= 0, "axpy: %ld elements", total);
    if (total == 0) return 0;
    stream_axpy_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, y, alpha, total);
    NN_LAUNCH_OK("axpy");
    return 0;
}

// ---------------------------------------------------------------------------
// x[t, :] += alpha * (a[t, :] / rms(a[t]) * wa + b[t, :] / rms(b[t]) * wb): one or two branches (b may be null), each
// RMS-normed over the row (eps inside the root) with a plain weight (null: ones), join the residual stream.  32-bit.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
branch_norm_add_kernel(float* __restrict__ x, const float* __restrict__ a, const void* __restrict__ wa,
                       const float* __restrict__ b, const void* __restrict__ wb, int w_dt, float eps, float alpha, int dim) {
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * dim;
    float sa = 0.0f, sb = 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float va = a[base + i];
        sa = fmaf(va, va, sa);
        if (b) {
            const float vb = b[base + i];
            sb = fmaf(vb, vb, sb);
        }
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, scratch) * (1.0f / (float)dim) + eps);
    const float rb = b ? 1.0f / sqrtf(block_sum(sb, scratch) * (1.0f / (float)dim) + eps) : 0.0f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = (a[base + i] * ra) * (wa ? ld_f(wa, i, w_dt) : 1.0f);
        if (b) v += (b[base + i] * rb) * (wb ? ld_f(wb, i, w_dt) : 1.0f);
        x[base + i] = fmaf(alpha, v, x[base + i]);
    }
}

// The common case, rows of a width that is a multiple of 4 and at most 256 * 4 * kVec: the branches' rows stay in
// registers between the sums of squares and the scaling, so every row is read once.  With ln_out the layer norm that
// reads the stream next (weight ln_w, bias ln_b, ln_eps) is left there in the same pass: the new row is in registers.
template <int kVec, bool kTwo>
__global__ void __launch_bounds__(256)
branch_norm_add_f32_kernel(float* __restrict__ x, const float* __restrict__ a, const void* __restrict__ wa,
                           const float* __restrict__ b, const void* __restrict__ wb, int w_dt, float eps, float alpha, int dim,
                           const void* __restrict__ ln_w, const void* __restrict__ ln_b, int ln_dt, float ln_eps,
                           void* __restrict__ ln_out, int ln_out_dt) {
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * dim;
    const int n4 = dim >> 2;
    float4 va[kVec], vb[kTwo ? kVec : 1];
    float sa = 0.0f, sb = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        va[j] = i < n4 ? reinterpret_cast<const float4*>(a + base)[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        sa = fmaf(va[j].x, va[j].x, sa); sa = fmaf(va[j].y, va[j].y, sa);
        sa = fmaf(va[j].z, va[j].z, sa); sa = fmaf(va[j].w, va[j].w, sa);
        if (kTwo) {
            vb[j] = i < n4 ? reinterpret_cast<const float4*>(b + base)[i] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            sb = fmaf(vb[j].x, vb[j].x, sb); sb = fmaf(vb[j].y, vb[j].y, sb);
            sb = fmaf(vb[j].z, vb[j].z, sb); sb = fmaf(vb[j].w, vb[j].w, sb);
        }
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, scratch) * (1.0f / (float)dim) + eps);
    const float rb = kTwo ? 1.0f / sqrtf(block_sum(sb, scratch) * (1.0f / (float)dim) + eps) : 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        const float pa[4] = {va[j].x, va[j].y, va[j].z, va[j].w};
        float4 was = reinterpret_cast<float4*>(x + base)[i];
        float o[4] = {was.x, was.y, was.z, was.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float v = (pa[e] * ra) * (wa ? ld_f(wa, 4 * i + e, w_dt) : 1.0f);
            if (kTwo) {
                const float pb = e == 0 ? vb[j].x : e == 1 ? vb[j].y : e == 2 ? vb[j].z : vb[j].w;
                v += (pb * rb) * (wb ? ld_f(wb, 4 * i + e, w_dt) : 1.0f);
            }
            o[e] = fmaf(alpha, v, o[e]);
        }
        reinterpret_cast<float4*>(x + base)[i] = make_float4(o[0], o[1], o[2], o[3]);
        va[j] = make_float4(o[0], o[1], o[2], o[3]);        // the new row, for the norm that follows
    }
    if (ln_out == nullptr) return;
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j)
        if (threadIdx.x + j * 256 < n4) s += (va[j].x + va[j].y) + (va[j].z + va[j].w);
    const float mean = block_sum(s, scratch) * (1.0f / (float)dim);
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        if (threadIdx.x + j * 256 >= n4) continue;
        va[j].x -= mean; va[j].y -= mean; va[j].z -= mean; va[j].w -= mean;
        ss = fmaf(va[j].x, va[j].x, ss); ss = fmaf(va[j].y, va[j].y, ss);
        ss = fmaf(va[j].z, va[j].z, ss); ss = fmaf(va[j].w, va[j].w, ss);
    }
    const float scale = 1.0f / sqrtf(block_sum(ss, scratch) * (1.0f / (float)dim) + ln_eps);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
        const int i = threadIdx.x + j * 256;
        if (i >= n4) continue;
        float o[4] = {va[j].x * scale, va[j].y * scale, va[j].z * scale, va[j].w * scale};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (ln_w) o[e] *= ld_f(ln_w, 4 * i + e, ln_dt);
            if (ln_b) o[e] += ld_f(ln_b, 4 * i + e, ln_dt);
        }
        const size_t at = base + 4 * i;
        if (ln_out_dt == DT_BF16) {
            __nv_bfloat162 h[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(ln_out) + at) = *reinterpret_cast<uint2*>(h);
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(ln_out) + at) = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

extern "C" int nncpu_branch_norm_add_takes_norm(int dim) { return dim > 0 && dim % 4 == 0 && dim <= 256 * 4 * 8; }

extern "C" int nncpu_branch_norm_add(float* x, const float* a, const void* wa, const float* b, const void* wb, int w_dt,
                                     float eps, float alpha, int n_tok, int dim, const void* ln_w, const void* ln_b,
                                     int ln_dt, float ln_eps, void* ln_out, int ln_out_dt, void* stream) {
    NN_CHECK(n_tok >= 0 && dim > 0 && a != nullptr, "branch norm: %d rows of %d", n_tok, dim);
    const bool vec = dim % 4 == 0 && dim <= 256 * 4 * 8 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)a % 16) == 0 &&
                     ((uintptr_t)b % 16) == 0 && ((uintptr_t)ln_out % 16) == 0;
    NN_CHECK(ln_out == nullptr || vec, "branch norm: a norm after rows of %d (a multiple of 4 up to 8192, 16-byte aligned)", dim);
    if (n_tok == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    if (vec) {
#define NN_BRANCH(V)                                                                                                  \
        do {                                                                                                          \
            if (b) branch_norm_add_f32_kernel<V, true><<<n_tok, 256, 0, st>>>(x, a, wa, b, wb, w_dt, eps, alpha, dim, ln_w, ln_b, ln_dt, ln_eps, ln_out, ln_out_dt);  \
            else branch_norm_add_f32_kernel<V, false><<<n_tok, 256, 0, st>>>(x, a, wa, b, wb, w_dt, eps, alpha, dim, ln_w, ln_b, ln_dt, ln_eps, ln_out, ln_out_dt);   \
        } while (0)
        if (dim <= 1024) NN_BRANCH(1);
        else if (dim <= 2048) NN_BRANCH(2);
        else if (dim <= 4096) NN_BRANCH(4);
        else NN_BRANCH(8);
#undef NN_BRANCH
        NN_LAUNCH_OK("branch norm");
        return 0;
    }
    branch_norm_add_kernel<<<n_tok, 256, 0, (cudaStream_t)stream>>>(x, a, wa, b, wb, w_dt, eps, alpha, dim);
    NN_LAUNCH_OK("branch norm");
    return 0;
}

// ---------------------------------------------------------------------------
// Elementwise activations of one product's 32-bit result: kind 0 `a` times the square of relu.
// ---------------------------------------------------------------------------
__global__ void unary_act_kernel(const float* __restrict__ x, void* __restrict__ out, int out_dt, long n, int kind, float a) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    st_f(out, (size_t)idx, out_dt, plain_act_f(x[idx], kind == 0 ? kActRelu2 : kActNone, a, 0.0f));
}

extern "C" int nncpu_unary_act(const float* x, void* out, int out_dt, long n, int kind, float a, void* stream) {
    NN_CHECK(n >= 0 && kind == 0, "activation: %ld elements, kind %d", n, kind);
    if (n == 0) return 0;
    unary_act_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, out, out_dt, n, kind, a);
    NN_LAUNCH_OK("activation");
    return 0;
}

// ---------------------------------------------------------------------------
// A token's own lanes gate a small projection: out[t, j] = gelu_tanh(z[t, j]) * table[ids[t], col + j], j < dim, with
// `table` [vocab, ld] holding a part of `dim` lanes per layer.  z float32; a negative id gives zeros.
// ---------------------------------------------------------------------------
__global__ void token_gate_kernel(const float* __restrict__ z, const void* __restrict__ table, int table_dt,
                                  const int* __restrict__ ids, int ld, int col, void* __restrict__ out, int out_dt,
                                  long total, int dim) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const long t = idx / dim;
    const int j = (int)(idx % dim), id = ids[t];
    const float e = id >= 0 ? ld_f(table, (size_t)id * ld + col + j, table_dt) : 0.0f;
    st_f(out, (size_t)idx, out_dt, gelu_tanh_f(z[idx]) * e);
}

// The same for a step of a few tokens, with the product in front of it: out[t, j] = gelu_tanh(W[j] . x[t]) *
// table[ids[t], col + j].  A warp owns one (row j of W [dim, width], token t) pair and asks for its whole share of the
// row and of the token before it multiplies (a chain of dependent loads from memory is what such a small product would
// otherwise wait for); a row is read from memory once and by the other tokens' warps from L2.  x float32
// [n_tok, width] is read as it is (not rounded).
constexpr int kGateRowsMaxTokens = 16;
constexpr int kGateRowsChunk = 8;          // 16-byte pieces of a row that a lane has in flight

__global__ void __launch_bounds__(256)
token_gate_rows_kernel(const float* __restrict__ x, const void* __restrict__ w, int w_dt, const void* __restrict__ table,
                       int table_dt, const int* __restrict__ ids, int ld, int col, void* __restrict__ out, int out_dt,
                       int width, int dim) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * 8 + warp, t = blockIdx.y;
    if (j >= dim) return;
    float s = 0.0f;
    if (w_dt == DT_BF16 && (width & 7) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
        const uint4* row = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(w) + (size_t)j * width);
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)t * width);
        const int n8 = width >> 3;
        for (int c0 = 0; c0 < n8; c0 += 32 * kGateRowsChunk) {
            uint4 wv[kGateRowsChunk];
            float4 xa[kGateRowsChunk], xb[kGateRowsChunk];
#pragma unroll
            for (int k = 0; k < kGateRowsChunk; ++k) {
                const int c = c0 + lane + 32 * k;
                const bool in = c < n8;
                wv[k] = in ? row[c] : make_uint4(0, 0, 0, 0);
                xa[k] = in ? xr[2 * c] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                xb[k] = in ? xr[2 * c + 1] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
#pragma unroll
            for (int k = 0; k < kGateRowsChunk; ++k) {
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&wv[k]);
                const float2 f0 = __bfloat1622float2(h2[0]), f1 = __bfloat1622float2(h2[1]);
                const float2 f2 = __bfloat1622float2(h2[2]), f3 = __bfloat1622float2(h2[3]);
                s = fmaf(f0.x, xa[k].x, s); s = fmaf(f0.y, xa[k].y, s); s = fmaf(f1.x, xa[k].z, s); s = fmaf(f1.y, xa[k].w, s);
                s = fmaf(f2.x, xb[k].x, s); s = fmaf(f2.y, xb[k].y, s); s = fmaf(f3.x, xb[k].z, s); s = fmaf(f3.y, xb[k].w, s);
            }
        }
    } else {
        for (int i = lane; i < width; i += 32) s = fmaf(ld_f(w, (size_t)j * width + i, w_dt), x[(size_t)t * width + i], s);
    }
    const float z = warp_sum(s);
    if (lane == 0) {
        const int id = ids[t];
        const float e = id >= 0 ? ld_f(table, (size_t)id * ld + col + j, table_dt) : 0.0f;
        st_f(out, (size_t)t * dim + j, out_dt, gelu_tanh_f(z) * e);
    }
}

extern "C" int nncpu_token_gate_rows(const float* x, const void* w, int w_dt, const void* table, int table_dt,
                                     const int* ids, int ld, int col, void* out, int out_dt, int n_tok, int width, int dim,
                                     void* stream) {
    NN_CHECK(n_tok >= 0 && n_tok <= kGateRowsMaxTokens && width > 0 && dim > 0 && col >= 0 && col + dim <= ld,
             "token gate (few tokens): %d tokens (at most %d) of %d, lanes %d..%d of %d", n_tok, kGateRowsMaxTokens, width,
             col, col + dim, ld);
    if (n_tok == 0) return 0;
    token_gate_rows_kernel<<<dim3((dim + 7) / 8, n_tok), 256, 0, (cudaStream_t)stream>>>(x, w, w_dt, table, table_dt, ids, ld,
                                                                                        col, out, out_dt, width, dim);
    NN_LAUNCH_OK("token gate (few tokens)");
    return 0;
}

extern "C" int nncpu_token_gate(const float* z, const void* table, int table_dt, const int* ids, int ld, int col,
                                void* out, int out_dt, int n_tok, int dim, void* stream) {
    NN_CHECK(n_tok >= 0 && dim > 0 && col >= 0 && col + dim <= ld, "token gate: lanes %d..%d of %d", col, col + dim, ld);
    if (n_tok == 0) return 0;
    const long total = (long)n_tok * dim;
    token_gate_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(z, table, table_dt, ids, ld, col,
                                                                                       out, out_dt, total, dim);
    NN_LAUNCH_OK("token gate");
    return 0;
}
