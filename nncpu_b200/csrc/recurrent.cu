// Recurrent mixers: layers that carry a fixed-size state per sequence from token to token instead of keys
// and values per position.  The state lives in 32-bit floats in the cache's state area, one row per sequence
// slot; everything that enters the recurrence (decays, their logarithms and exponentials) is computed in 32-bit.
//
// Gated linear attention.  Per head, with a state S of d rows (key channels) and e columns (value channels):
//     a_t = sigmoid(z_t)^(1/tau)                 (a decay per key channel, from the gate logits z_t)
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T
//     o_t = S_t^T q_t
// The columns of S do not depend on one another, so a block owns a few of them, keeps them in registers and walks
// the tokens of its sequence in order; q, k and a of a token are shared by the block through shared memory.  The
// order of operations of a (sequence, head, column) does not depend on how the sequence was cut into steps or on
// what else the step holds, so the results are the same bits.  Per token the recurrence costs 2 d e multiply-adds
// a head whatever the arrangement, and 32-bit multiply-adds run on the CUDA cores, so the kernel's job is to keep
// every SM's lanes busy with them.

#include <math.h>

#define NN_LIB recurrent
#include "common.cuh"

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

// Two 32-bit multiply-adds in one instruction (sm_100 has them for pairs of floats in a 64-bit register): each half is
// an ordinary fused multiply-add with round-to-nearest, so results are those of two fmaf calls.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

// The decays of a prompt's tokens, made once for all the blocks that read them: z <- sigmoid(z)^(1/tau) in place.
__global__ void gla_decay_kernel(float* __restrict__ z, long n, float inv_tau) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) z[idx] = expf(log_sigmoid_f(z[idx]) * inv_tau);
}

extern "C" int nncpu_gla_decay(float* z, long n, float tau, void* stream) {
    NN_CHECK(n >= 0 && tau > 0.0f, "gla_decay: %ld elements, tau %g", n, tau);
    if (n == 0) return 0;
    gla_decay_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(z, n, 1.0f / tau);
    NN_LAUNCH_OK("gla_decay");
    return 0;
}

// proj [n_tok, row] float32 holds per token q (H*d), k (H*d), v (H*e), g (H*e); z [n_tok, H*d] float32 the
// decay logits (or, with decays_given, the decays themselves).  state [n_slots + 1, H, d, e]; seq_slots[s] < 0 marks a padding sequence: its rows of o are zero
// and no state is touched.  o [n_tok, H*e] float32.
//
// A block of four warps owns 16 columns of one head's state for one sequence, a warp four of them.  A lane keeps
// the rows i = 32 ii + lane of its warp's four columns in registers (DMAX / 32 x 4 numbers): what it reads of a
// token from shared memory, (a, k, q) of its rows, serves four columns, and shared memory is what bounds this
// kernel.  A lane's partial dot products of a whole group of tokens are added over the warp in one go by a
// butterfly that halves what a lane carries while it doubles the rows that covers.  a, k, q and v of a group of tokens are
// staged once per block in shared memory (two buffers that take turns: one barrier a group); the next group's
// loads are issued before this group's arithmetic.
constexpr int kScanCols = 16;       // columns of the state a block owns
constexpr int kScanGroup = 8;       // tokens staged at a time

// CPL columns a lane: 4 (four warps a block) where there are blocks enough to fill the GPU several times over, 2
// (eight warps a block, twice the warps for the same state) where there are not: a warp's token is a chain of
// dependent instructions, and an SM needs warps to put into one another's waits.
template <int DMAX, int CPL>
__global__ void __launch_bounds__(32 * kScanCols / CPL)
gla_scan_kernel(const float* __restrict__ proj, int row, const float* __restrict__ z, float* __restrict__ state,
                const int* __restrict__ seq_slots, const int* __restrict__ cu_seqlens, float* __restrict__ o, int H,
                int d, int e, float q_scale, float inv_tau, int decays_given, const float* __restrict__ head_decay) {
    constexpr int DR = DMAX / 32;                             // rows of its columns that a lane keeps
    constexpr int TB = DMAX <= 128 ? kScanGroup : DMAX <= 256 ? kScanGroup / 2 : kScanGroup / 4;   // tokens a group (shared memory: 2 TB DMAX 16 bytes)
    constexpr int kScanThreads = 32 * kScanCols / CPL;
    constexpr int PER = TB * DMAX / kScanThreads;             // (token, key channel) pairs a thread stages
    constexpr int N = CPL * TB;                               // partial sums a lane carries through a group
    __shared__ float4 shared[2][TB][DMAX];                    // (a, k, q, -) of the group under way and of the next
    __shared__ float shared_v[2][TB][kScanCols];              // v of the block's columns
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int j0 = blockIdx.z * kScanCols + warp * CPL;       // this warp's first column
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    const int slot = seq_slots[seq];
    if (slot < 0) {
        if (lane < CPL && j0 + lane < e)
            for (int t = t0; t < t1; ++t) o[(size_t)t * H * e + (size_t)h * e + j0 + lane] = 0.0f;
        return;
    }
    float* s_head = state + ((size_t)slot * H + h) * (size_t)d * e;
    float2 S[DR][CPL / 2];          // pairs of neighbouring columns: the recurrence runs on two at a time
#pragma unroll
    for (int ii = 0; ii < DR; ++ii) {
        const int i = ii * 32 + lane;
#pragma unroll
        for (int c = 0; c < CPL; c += 2) {
            S[ii][c / 2].x = (i < d && j0 + c < e) ? s_head[(size_t)i * e + j0 + c] : 0.0f;
            S[ii][c / 2].y = (i < d && j0 + c + 1 < e) ? s_head[(size_t)i * e + j0 + c + 1] : 0.0f;
        }
    }
    const size_t q_at = (size_t)h * d, k_at = (size_t)H * d + (size_t)h * d, v_at = 2 * (size_t)H * d + (size_t)h * e;
    // The tokens come in groups of TB: a group's q, k, v and decay logits are fetched into registers while the group
    // before it is worked on, turned into (a, k, q) and put into the shared buffer that is free; one barrier a group.
    float nq[PER], nk[PER], nz[PER], nv = 0.0f;
    const int v_tt = tid / kScanCols, v_col = tid % kScanCols;      // the v that this thread stages (TB * 16 of them)
    auto fetch = [&](int g0) {
        const int nt = min(TB, t1 - g0);
#pragma unroll
        for (int c = 0; c < PER; ++c) {
            const int idx = tid + kScanThreads * c;
            const int tt = idx / DMAX, i = idx % DMAX;
            if (tt < nt && i < d) {
                const float* p = proj + (size_t)(g0 + tt) * row;
                nq[c] = p[q_at + i];
                nk[c] = p[k_at + i];
                nz[c] = head_decay ? head_decay[h] : z[(size_t)(g0 + tt) * H * d + (size_t)h * d + i];
            }
        }
        const int col = blockIdx.z * kScanCols + v_col;
        nv = (tid < TB * kScanCols && v_tt < nt && col < e) ? proj[(size_t)(g0 + v_tt) * row + v_at + col] : 0.0f;
    };
    if (t0 < t1) fetch(t0);
    int buf = 0;
    for (int g0 = t0; g0 < t1; g0 += TB, buf ^= 1) {
        const int nt = min(TB, t1 - g0);
#pragma unroll
        for (int c = 0; c < PER; ++c) {
            const int idx = tid + kScanThreads * c;
            const int tt = idx / DMAX, i = idx % DMAX;
            // rows beyond d hold zeros: they keep their part of the state at zero and add nothing
            shared[buf][tt][i] = (tt < nt && i < d) ? make_float4(decays_given ? nz[c] : expf(log_sigmoid_f(nz[c]) * inv_tau),
                                                                  nk[c], nq[c] * q_scale, 0.0f)
                                                    : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        if (tid < TB * kScanCols) shared_v[buf][v_tt][v_col] = nv;
        __syncthreads();      // the other buffer was read before its readers came here
        if (g0 + TB < t1) fetch(g0 + TB);
        // the group's arithmetic first, token by token: x[4 tt + c] is this lane's part of o[tt] in column c
        float x[N];
#pragma unroll
        for (int tt = 0; tt < TB; ++tt) {
            float2 xs[CPL / 2];
#pragma unroll
            for (int k = 0; k < CPL / 2; ++k) xs[k] = make_float2(0.0f, 0.0f);
            if (tt < nt) {
                float2 v[CPL / 2];
#pragma unroll
                for (int k = 0; k < CPL / 2; ++k)
                    v[k] = make_float2(shared_v[buf][tt][warp * CPL + 2 * k], shared_v[buf][tt][warp * CPL + 2 * k + 1]);
                float4 c[DR];       // all of the token's loads first: they do not wait for one another
#pragma unroll
                for (int ii = 0; ii < DR; ++ii) c[ii] = shared[buf][tt][ii * 32 + lane];
#pragma unroll
                for (int ii = 0; ii < DR; ++ii) {
                    const float2 a2 = make_float2(c[ii].x, c[ii].x), k2 = make_float2(c[ii].y, c[ii].y);
                    const float2 q2 = make_float2(c[ii].z, c[ii].z);
#pragma unroll
                    for (int k = 0; k < CPL / 2; ++k) {
                        // S <- a S + k v; x += S q (each half: fmaf(a, S, k * v) with the product rounded, as before)
                        const float2 kv = fma2(k2, v[k], make_float2(-0.0f, -0.0f));
                        S[ii][k] = fma2(a2, S[ii][k], kv);
                        xs[k] = fma2(S[ii][k], q2, xs[k]);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < CPL / 2; ++k) {
                x[CPL * tt + 2 * k] = xs[k].x;
                x[CPL * tt + 2 * k + 1] = xs[k].y;
            }
        }
        // then one sum over the warp for all of them: at every stage a lane hands half of what it carries to the
        // lane m away and adds what it gets to the half it keeps, so that in the end lane n % N holds sum number n
        // (N - 1 shuffles for N sums, and the shuffles of a stage do not wait for one another)
#pragma unroll
        for (int m = N / 2; m >= 1; m >>= 1) {
            const bool up = lane & m;
#pragma unroll
            for (int k = 0; k < m; ++k) {
                const float got = __shfl_xor_sync(0xffffffffu, up ? x[k] : x[k + m], m);
                x[k] = (up ? x[k + m] : x[k]) + got;
            }
        }
#pragma unroll
        for (int m = N; m < 32; m <<= 1) x[0] += __shfl_xor_sync(0xffffffffu, x[0], m);
        {
            const int n = lane % N, tt = n / CPL, col = j0 + n % CPL;
            if (lane < N && tt < nt && col < e) o[(size_t)(g0 + tt) * H * e + (size_t)h * e + col] = x[0];
        }
    }
#pragma unroll
    for (int ii = 0; ii < DR; ++ii) {
        const int i = ii * 32 + lane;
#pragma unroll
        for (int c = 0; c < CPL; ++c)
            if (i < d && j0 + c < e) s_head[(size_t)i * e + j0 + c] = (c & 1) ? S[ii][c / 2].y : S[ii][c / 2].x;
    }
}

static int g_scan_cpl = 0;     // 0: by the grid's size; 2 or 4: forced (measurements and tests)
extern "C" void nncpu_gla_scan_force_columns(int cpl) { g_scan_cpl = (cpl == 2 || cpl == 4) ? cpl : 0; }

extern "C" int nncpu_gla_scan(const float* proj, int row, const float* z, float* state, const int* seq_slots,
                              const int* cu_seqlens, float* o, int n_seqs, int H, int d, int e, float q_scale,
                              float tau, int decays_given, const float* head_decay, void* stream) {
    // head_decay [H] (optional): one fixed decay per head for every key channel and token; z is then not read
    if (head_decay != nullptr) decays_given = 1;
    NN_CHECK(n_seqs >= 0 && H > 0 && d > 0 && e > 0, "gla_scan: %d sequences, %d heads of %d x %d", n_seqs, H, d, e);
    NN_CHECK(d <= 512, "gla_scan: %d key channels a head (at most 512)", d);
    NN_CHECK(row >= 2 * H * d + 2 * H * e, "gla_scan: rows of %d floats for %d heads of %d x %d", row, H, d, e);
    NN_CHECK(tau > 0.0f, "gla_scan: tau %g", tau);
    NN_CHECK(H <= 65535 && (e + kScanCols - 1) / kScanCols <= 65535, "gla_scan: grid");
    if (n_seqs == 0) return 0;
    dim3 grid(n_seqs, H, (e + kScanCols - 1) / kScanCols);
    const float inv_tau = 1.0f / tau;
    cudaStream_t st = (cudaStream_t)stream;
    int sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const long blocks = (long)grid.x * grid.y * grid.z;
    const bool narrow = g_scan_cpl == 2 || (g_scan_cpl == 0 && blocks < 4L * sms);
#define NN_SCAN(DMAX)                                                                                               \
    do {                                                                                                            \
        if (narrow)                                                                                                 \
            gla_scan_kernel<DMAX, 2><<<grid, 32 * kScanCols / 2, 0, st>>>(proj, row, z, state, seq_slots, cu_seqlens, o, H, d, \
                                                                          e, q_scale, inv_tau, decays_given, head_decay); \
        else                                                                                                        \
            gla_scan_kernel<DMAX, 4><<<grid, 32 * kScanCols / 4, 0, st>>>(proj, row, z, state, seq_slots, cu_seqlens, o, H, d, \
                                                                          e, q_scale, inv_tau, decays_given, head_decay); \
    } while (0)
    if (d <= 32) NN_SCAN(32);
    else if (d <= 64) NN_SCAN(64);
    else if (d <= 128) NN_SCAN(128);
    else if (d <= 256) NN_SCAN(256);
    else NN_SCAN(512);
#undef NN_SCAN
    NN_LAUNCH_OK("gla_scan");
    return 0;
}

// The mixer's output stage: every head's o is divided by its root mean square over the e value channels (eps
// inside the root), multiplied by the weight w [e] that the heads share (null: ones) and by silu(g), the gate of its
// channel (gate_kind 1: by sigmoid(g)), and by out_scale.
// One warp per (token, head); out [n_tok, H*e] in the run's element type.
__global__ void __launch_bounds__(256)
gla_output_kernel(const float* __restrict__ o, const float* __restrict__ proj, int row, int g_at,
                  const void* __restrict__ w, int w_dt, float eps, void* __restrict__ out, int out_dt, long n_items,
                  int H, int e, int gate_kind, float out_scale) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 8 + warp;
    if (item >= n_items) return;
    const long t = item / H;
    const int h = (int)(item % H);
    const float* src = o + (size_t)t * H * e + (size_t)h * e;
    float ss = 0.0f;
    for (int j = lane; j < e; j += 32) ss = fmaf(src[j], src[j], ss);
    ss = warp_sum(ss);
    const float scale = out_scale / sqrtf(ss * (1.0f / (float)e) + eps);
    const float* g = proj + (size_t)t * row + g_at + (size_t)h * e;
    for (int j = lane; j < e; j += 32) {
        const float gate = g[j];
        const float y = (src[j] * scale) * (w ? ld_f(w, j, w_dt) : 1.0f);
        const float sg = 1.0f / (1.0f + expf(-gate));         // gate_kind 0: silu(gate), 1: sigmoid(gate)
        st_f(out, (size_t)t * H * e + (size_t)h * e + j, out_dt, y * (gate_kind == 1 ? sg : gate * sg));
    }
}

extern "C" int nncpu_gla_output(const float* o, const float* proj, int row, int g_at, const void* w, int w_dt,
                                float eps, void* out, int out_dt, int n_tok, int H, int e, int gate_kind, float out_scale,
                                void* stream) {
    NN_CHECK(n_tok >= 0 && H > 0 && e > 0 && g_at >= 0 && g_at + H * e <= row, "gla_output: sizes");
    if (n_tok == 0) return 0;
    const long n_items = (long)n_tok * H;
    gla_output_kernel<<<(unsigned)((n_items + 7) / 8), 256, 0, (cudaStream_t)stream>>>(o, proj, row, g_at, w, w_dt, eps,
                                                                                       out, out_dt, n_items, H, e, gate_kind, out_scale);
    NN_LAUNCH_OK("gla_output");
    return 0;
}

// One token per sequence (a decode step): recurrence, norm and gate in one launch.  A block owns a (sequence, head)
// pair; thread j owns column j of the state and streams its d rows through once, rows being contiguous over the
// columns, so a step reads and writes the state at full width and nothing of it stays in registers.  The decays, k
// and q of the token are shared through shared memory; the head's sum of squares is a block sum.  A negative slot
// (padding) gives zeros and touches no state.  Threads: e rounded up to a warp (e <= 1024).
template <int kThreads, int kInFlight>
__global__ void __launch_bounds__(kThreads)
gla_step_kernel(const float* __restrict__ proj, int row, const float* __restrict__ z, float* __restrict__ state,
                const int* __restrict__ seq_slots, const void* __restrict__ w, int w_dt, float eps,
                void* __restrict__ out, int out_dt, int H, int d, int e, float q_scale, float inv_tau,
                const float* __restrict__ head_decay, const float* __restrict__ cos_sin, int half, float k_scale) {
    extern __shared__ float4 akq[];          // d entries of (a, k, q, -)
    __shared__ float scratch[33];
    const int t = blockIdx.x, h = blockIdx.y, j = threadIdx.x;
    const int slot = seq_slots[t];
    const size_t out_at = (size_t)t * H * e + (size_t)h * e + j;
    if (slot < 0) {
        if (j < e) st_f(out, out_at, out_dt, 0.0f);
        return;
    }
    const float* p = proj + (size_t)t * row;
    for (int i = j; i < d; i += blockDim.x) {
        const float* qp = p + (size_t)h * d;
        const float* kp = qp + (size_t)H * d;
        float qv = qp[i], kv = kp[i];
        if (cos_sin != nullptr && i < 2 * half) {
            // retention: q and k are rotated by the token's position on the way in (the pair (u, v) = lanes (i, i + half)
            // becomes (u c - v s, v c + u s)), with the operations of the kernel that rotates a prompt's rows in place
            const int ii = i < half ? i : i - half;
            const float c = cos_sin[((size_t)t * half + ii) * 2], sn = cos_sin[((size_t)t * half + ii) * 2 + 1];
            const float qo = qp[i < half ? i + half : i - half], ko = kp[i < half ? i + half : i - half];
            qv = i < half ? qv * c - qo * sn : qv * c + qo * sn;
            kv = i < half ? kv * c - ko * sn : kv * c + ko * sn;
        }
        akq[i] = make_float4(head_decay ? head_decay[h] : expf(log_sigmoid_f(z[(size_t)t * H * d + (size_t)h * d + i]) * inv_tau),
                             kv * k_scale, qv * q_scale, 0.0f);
    }
    __syncthreads();
    float acc = 0.0f;
    if (j < e) {
        const float v = p[2 * (size_t)H * d + (size_t)h * e + j];
        float* col = state + (((size_t)slot * H + h) * d) * e + j;
        int i = 0;
        // kInFlight rows in flight: a step of few sequences is bound by the loads' latency, and a block of up to 256
        // threads has the registers for 32 of them (a block of 1 024 threads has 64 registers a thread: 8)
        for (; i + kInFlight <= d; i += kInFlight) {
            float s[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) s[u] = col[(size_t)(i + u) * e];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const float4 c = akq[i + u];
                s[u] = fmaf(c.x, s[u], c.y * v);
                acc = fmaf(s[u], c.z, acc);
                col[(size_t)(i + u) * e] = s[u];
            }
        }
        for (; i < d; ++i) {
            const float4 c = akq[i];
            const float s = fmaf(c.x, col[(size_t)i * e], c.y * v);
            acc = fmaf(s, c.z, acc);
            col[(size_t)i * e] = s;
        }
    }
    const float ss = block_sum(j < e ? acc * acc : 0.0f, scratch);
    if (j < e) {
        const float scale = 1.0f / sqrtf(ss * (1.0f / (float)e) + eps);
        const float gate = p[2 * (size_t)H * d + (size_t)H * e + (size_t)h * e + j];
        st_f(out, out_at, out_dt, ((acc * scale) * (w ? ld_f(w, j, w_dt) : 1.0f)) * (gate / (1.0f + expf(-gate))));
    }
}

extern "C" int nncpu_gla_step(const float* proj, int row, const float* z, float* state, const int* seq_slots,
                              const void* w, int w_dt, float eps, void* out, int out_dt, int n_tok, int H, int d, int e,
                              float q_scale, float tau, const float* head_decay, const float* cos_sin, int half, float k_scale,
                              void* stream) {
    // cos_sin [n_tok, half, 2] (optional): q and k are rotated on the way in; k is multiplied by k_scale (1: as it is)
    NN_CHECK(cos_sin == nullptr || (half > 0 && 2 * half <= d), "gla_step: %d rotated lanes of %d", 2 * half, d);
    NN_CHECK(n_tok >= 0 && H > 0 && H <= 65535 && d > 0 && e > 0, "gla_step: %d tokens, %d heads of %d x %d", n_tok, H, d, e);
    NN_CHECK(e <= 1024, "gla_step: %d value channels a head (at most 1024)", e);
    NN_CHECK(d <= 2048, "gla_step: %d key channels a head (at most 2048)", d);
    NN_CHECK(row >= 2 * H * d + 2 * H * e && tau > 0.0f, "gla_step: rows of %d floats, tau %g", row, tau);
    if (n_tok == 0) return 0;
    const int threads = (e + 31) / 32 * 32;
    int sms = 148;
    {
        int dev = 0;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    // few blocks: each thread keeps 32 loads in flight (one block an SM); many blocks: 8, and the SM's other blocks
    // fill the waits (batch 8 of 8 heads 20 -> 11 us with 32; batch 64 of 16 heads 57 us with 8, 78 with 32)
    if (threads <= 256 && (long)n_tok * H <= 2L * sms)
        gla_step_kernel<256, 32><<<dim3(n_tok, H), threads, (size_t)d * sizeof(float4), (cudaStream_t)stream>>>(
            proj, row, z, state, seq_slots, w, w_dt, eps, out, out_dt, H, d, e, q_scale, 1.0f / tau, head_decay, cos_sin, half, k_scale);
    else if (threads <= 256)
        gla_step_kernel<256, 8><<<dim3(n_tok, H), threads, (size_t)d * sizeof(float4), (cudaStream_t)stream>>>(
            proj, row, z, state, seq_slots, w, w_dt, eps, out, out_dt, H, d, e, q_scale, 1.0f / tau, head_decay, cos_sin, half, k_scale);
    else
        gla_step_kernel<1024, 8><<<dim3(n_tok, H), threads, (size_t)d * sizeof(float4), (cudaStream_t)stream>>>(
            proj, row, z, state, seq_slots, w, w_dt, eps, out, out_dt, H, d, e, q_scale, 1.0f / tau, head_decay, cos_sin, half, k_scale);
    NN_LAUNCH_OK("gla_step");
    return 0;
}

// Retention: linear attention with ONE fixed decay per head, S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t: the
// recurrence of gated linear attention with a constant in place of the per-channel decays (gla_scan and gla_step take
// `head_decay`).  What comes before it: q and k of every head are rotated by the token's position (the pairs (i, i +
// half) of a head's first 2 half lanes by the table's (cos, sin) [n_tok, half, 2]; the rest pass), then k is
// multiplied by k_scale.  In place, on the rows of proj [n_tok, row] that hold q (H d) and then k (H d).
__global__ void __launch_bounds__(256)
retention_prepare_kernel(float* __restrict__ proj, int row, const float* __restrict__ cos_sin, int half, long total,
                         int H, int d, float k_scale) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int i = (int)(idx % d);
    const long th = idx / d;
    const int h = (int)(th % H);
    const long t = th / H;
    float* q = proj + (size_t)t * row + (size_t)h * d;
    float* k = q + (size_t)H * d;
    if (i < half) {
        const float c = cos_sin[((size_t)t * half + i) * 2], sn = cos_sin[((size_t)t * half + i) * 2 + 1];
        const float qu = q[i], qv = q[i + half], ku = k[i], kv = k[i + half];
        q[i] = qu * c - qv * sn;
        q[i + half] = qv * c + qu * sn;
        k[i] = (ku * c - kv * sn) * k_scale;
        k[i + half] = (kv * c + ku * sn) * k_scale;
    } else if (i >= 2 * half) {
        k[i] *= k_scale;
    }
}

extern "C" int nncpu_retention_prepare(float* proj, int row, const float* cos_sin, int half, int n_tok, int H, int d,
                                       float k_scale, void* stream) {
    NN_CHECK(n_tok >= 0 && H > 0 && d > 0 && half >= 0 && 2 * half <= d && row >= 2 * H * d,
             "retention: %d heads of %d lanes, %d of them rotated, rows of %d", H, d, 2 * half, row);
    NN_CHECK(half == 0 || cos_sin != nullptr, "retention: a rotation without its table");
    if (n_tok == 0) return 0;
    const long total = (long)n_tok * H * d;
    retention_prepare_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(proj, row, cos_sin, half,
                                                                                             total, H, d, k_scale);
    NN_LAUNCH_OK("retention prepare");
    return 0;
}

// ---------------------------------------------------------------------------
// The gated delta rule.  Per head, with a state S of d rows (key channels) and e columns (value channels), a decay
// g and a write strength beta per token and head, unit vectors k and q (q also times d^-1/2):
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
// q and k have G heads (head h of H uses q/k head h / (H / G)), v has H.  Before that, q, k and v each pass a causal
// convolution over time per channel (taps weights a channel, the last one the current token's, zeros before the
// sequence's start) and SiLU.  The last taps - 1 inputs of the convolutions are per-sequence state, like S.
//
// The rows of proj [n_tok, ld] (32-bit) hold, in this order: q (G d), k (G d), v (H e), the output gate's logits (H e),
// the logits of beta (H), the decays' inputs (H).  The first C = 2 G d + H e of them are the convolutions' channels;
// A slot's state and its convolution inputs may be parts of one row per slot: both are addressed as base + slot *
// slot_stride floats.  conv_state [taps - 1, C] of a slot holds, for a sequence of n tokens so far, the inputs of positions n - (taps - 1)
// .. n - 1 (zeros before position 0).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float softplus_r(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

constexpr float kUnitEps = 1e-6f;     // inside the root that makes q and k unit vectors
constexpr int kMaxTaps = 32;

// One warp per (token, item): G query heads, G key heads, H value heads, one item for the token's H decays and
// write strengths, and (with a decay per key channel) H more items, one per head's d decays.  xc [n_tok, C] receives the convolved, activated (and for q, k: normalised) channels, gb [n_tok,
// 2 H] the decays g and then the strengths beta.  A token of no sequence (tok_seq < 0) gets zeros.  With kShiftHere
// (every sequence of the step brings ONE token, so a channel's kept inputs are read by one lane of one warp alone) that
// lane also advances the channel's kept inputs by the token, which saves the launch of the kernel below.
template <bool kShiftHere>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const float* __restrict__ proj, int ld, const void* __restrict__ conv_w, int w_dt,
                     float* conv_state, long slot_stride, const int* __restrict__ tok_seq,
                     const int* __restrict__ seq_slots, const int* __restrict__ cu_seqlens,
                     const void* __restrict__ a_log, const void* __restrict__ dt_bias, int p_dt,
                     float* __restrict__ xc, float* __restrict__ gb, long n_items, int H, int G, int d, int e, int taps,
                     float q_scale, int beta_col, float* __restrict__ chan_z) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long item = (long)blockIdx.x * 8 + warp;
    if (item >= n_items) return;
    const int per_tok = 2 * G + H + 1 + (chan_z ? H : 0);
    const int t = (int)(item / per_tok), it = (int)(item % per_tok);
    const int C = 2 * G * d + H * e;
    const int seq = tok_seq[t];
    const int slot = seq < 0 ? -1 : seq_slots[seq];
    if (it > 2 * G + H) {       // (a decay per key channel) one more item per head: its d decays from their logits, in place
        const int h = it - (2 * G + H + 1);
        float* zz = chan_z + ((size_t)t * H + h) * d;
        const float rate = expf(ld_f(a_log, h, p_dt));
        for (int i = lane; i < d; i += 32) zz[i] = slot >= 0 ? expf(0.0f - rate * softplus_r(zz[i])) : 0.0f;
        return;
    }
    if (it == 2 * G + H) {
        for (int h = lane; h < H; h += 32) {
            float g = 0.0f, beta = 0.0f;
            if (slot >= 0) {
                const float* p = proj + (size_t)t * ld + beta_col;
                beta = 1.0f / (1.0f + expf(0.0f - p[h]));
                g = chan_z ? 1.0f : expf(0.0f - expf(ld_f(a_log, h, p_dt)) * softplus_r(p[H + h] + ld_f(dt_bias, h, p_dt)));
            }
            gb[(size_t)t * 2 * H + h] = g;
            gb[(size_t)t * 2 * H + H + h] = beta;
        }
        return;
    }
    const bool is_v = it >= 2 * G;
    const int len = is_v ? e : d;
    const int ch0 = is_v ? 2 * G * d + (it - 2 * G) * e : it * d;
    float* dst = xc + (size_t)t * C + ch0;
    if (slot < 0) {
        for (int i = lane; i < len; i += 32) dst[i] = 0.0f;
        return;
    }
    const int local = t - cu_seqlens[seq];          // the token's place among its sequence's tokens of this step
    float* st = conv_state + (size_t)slot * slot_stride;
    const float* __restrict__ st_kept = st;     // what the kernel that does not advance the kept inputs reads them through
    float ss = 0.0f;
    for (int i = lane; i < len; i += 32) {
        const int ch = ch0 + i;
        float acc = 0.0f;
        for (int j = 0; j < taps; ++j) {
            const int at = local - (taps - 1) + j;
            const float x = at >= 0 ? proj[(size_t)(t - local + at) * ld + ch]
                                    : (kShiftHere ? st : st_kept)[(size_t)(taps - 1 + at) * C + ch];
            acc = fmaf(ld_f(conv_w, (size_t)ch * taps + j, w_dt), x, acc);
        }
        const float y = acc / (1.0f + expf(0.0f - acc));
        dst[i] = y;
        ss = fmaf(y, y, ss);
        if (kShiftHere && taps > 1) {       // local is 0: the kept inputs move up by one, the token's input comes last
            for (int s = 0; s + 2 < taps; ++s) st[(size_t)s * C + ch] = st[(size_t)(s + 1) * C + ch];
            st[(size_t)(taps - 2) * C + ch] = proj[(size_t)t * ld + ch];
        }
    }
    if (is_v) return;
    ss = warp_sum(ss);
    const float scale = (1.0f / sqrtf(ss + kUnitEps)) * (it < G ? q_scale : 1.0f);
    __syncwarp();
    for (int i = lane; i < len; i += 32) dst[i] *= scale;      // a lane rereads what it wrote itself
}

// The convolutions' state after the step: one thread per (sequence, channel) shifts its taps - 1 inputs.
__global__ void __launch_bounds__(256)
delta_conv_state_kernel(const float* __restrict__ proj, int ld, float* __restrict__ conv_state, long slot_stride,
                        const int* __restrict__ seq_slots, const int* __restrict__ cu_seqlens, int n_seqs, int C, int taps) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * C) return;
    const int seq = (int)(idx / C), ch = (int)(idx % C);
    const int slot = seq_slots[seq];
    if (slot < 0) return;
    const int t0 = cu_seqlens[seq], n = cu_seqlens[seq + 1] - t0;
    float* st = conv_state + (size_t)slot * slot_stride + ch;
    float keep[kMaxTaps];
    for (int s = 0; s < taps - 1; ++s) {
        const int at = n - (taps - 1) + s;          // the step's token that lands in place s (negative: an older one)
        keep[s] = at >= 0 ? proj[(size_t)(t0 + at) * ld + ch] : st[(size_t)(taps - 1 + at) * C];
    }
    for (int s = 0; s < taps - 1; ++s) st[(size_t)s * C] = keep[s];
}

extern "C" int nncpu_delta_prepare(const float* proj, int ld, const void* conv_w, int w_dt, float* conv_state,
                                   long slot_stride, const int* tok_seq, const int* seq_slots, const int* cu_seqlens, const void* a_log,
                                   const void* dt_bias, int p_dt, float* xc, float* gb, int n_tok, int n_seqs, int H,
                                   int G, int d, int e, int taps, float q_scale, int one_token_each, int beta_col,
                                   float* chan_z, void* stream) {
    // beta_col: where a row of proj holds the H logits of beta (the H decay inputs follow them unless chan_z is given:
    // float [n_tok, H d] logits of a decay per head and key channel, turned into the decays in place)
    NN_CHECK(n_tok >= 0 && n_seqs >= 0 && H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0,
             "delta prepare: %d heads over %d query/key heads of %d x %d", H, G, d, e);
    NN_CHECK(taps >= 1 && taps <= kMaxTaps, "delta prepare: %d taps (1 to %d)", taps, kMaxTaps);
    const int C = 2 * G * d + H * e;
    NN_CHECK(beta_col >= C && ld >= beta_col + (chan_z ? 1 : 2) * H, "delta prepare: rows of %d floats", ld);
    if (n_tok == 0) return 0;
    const long n_items = (long)n_tok * (2 * G + H + 1 + (chan_z ? H : 0));
    if (one_token_each)
        delta_prepare_kernel<true><<<(unsigned)((n_items + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
            proj, ld, conv_w, w_dt, conv_state, slot_stride, tok_seq, seq_slots, cu_seqlens, a_log, dt_bias, p_dt, xc, gb, n_items, H,
            G, d, e, taps, q_scale, beta_col, chan_z);
    else
        delta_prepare_kernel<false><<<(unsigned)((n_items + 7) / 8), 256, 0, (cudaStream_t)stream>>>(
            proj, ld, conv_w, w_dt, conv_state, slot_stride, tok_seq, seq_slots, cu_seqlens, a_log, dt_bias, p_dt, xc, gb, n_items, H,
            G, d, e, taps, q_scale, beta_col, chan_z);
    NN_LAUNCH_OK("delta prepare");
    if (taps > 1 && n_seqs > 0 && !one_token_each) {
        const long total = (long)n_seqs * C;
        delta_conv_state_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            proj, ld, conv_state, slot_stride, seq_slots, cu_seqlens, n_seqs, C, taps);
        NN_LAUNCH_OK("delta conv state");
    }
    return 0;
}

__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_one_() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// The recurrence over the step's tokens, sequence by sequence in order.  The columns of S do not depend on one
// another.  A block of four warps owns 4 * 32 / R columns of one head's state for one sequence; R lanes share a column,
// lane r of them keeping DR rows in registers (the groups of four rows 4 (c R + r) .. + 3, c < DR / 4: the R lanes of
// a column read R neighbouring 16-byte pieces of k and of q from shared memory with one load), so that S^T k costs DR
// multiply-adds and log2(R) shuffles a token, the only exchange on the chain from token to token (the sum for o is
// off that chain).  k, q, v,
// g and beta of a group of tokens are staged in shared memory by asynchronous copies, the next group's in flight under
// this group's arithmetic.  The order of operations of a (sequence, head, column) does not depend on how the sequence
// was cut into steps or on what else the step holds.  A negative slot (padding): zeros out, no state touched.
// Tokens a group: what two buffers of the default shared memory hold.  With a decay per key channel (CH) a buffer
// also holds the tokens' decays.
__host__ __device__ constexpr int delta_group(int DP, bool CH) {
    return CH ? (DP <= 128 ? 8 : DP <= 256 ? 4 : DP <= 512 ? 2 : 1) : (DP <= 256 ? 8 : (DP <= 512 ? 4 : 2));
}

// CH: the decay is one number per head and key channel (gch [n_tok, H d]), S <- diag(g) S, instead of one per head.
// (With a decay per key channel and up to 16 rows a lane the kernel is held to the registers of four blocks an SM, as
// the per-head variant has them by itself: with three, a step of many sequences took 1.9 times the per-head kernel's
// time instead of the 1.3 times of its instructions.)
template <int DR, int R, int CPL, bool CH>
__global__ void __launch_bounds__(128, (CH && DR * CPL <= 16) ? 4 : 1)
delta_scan_kernel(const float* __restrict__ xc, const float* __restrict__ gb, const float* __restrict__ gch,
                  float* __restrict__ state,
                  long slot_stride, const int* __restrict__ seq_slots, const int* __restrict__ cu_seqlens, float* __restrict__ o, int H,
                  int G, int d, int e) {
    static_assert(DR % 4 == 0, "a lane keeps whole groups of four rows");
    constexpr int DP = DR * R;                      // rows the lanes cover (>= d; the rest hold zeros)
    constexpr int CW = CPL * 32 / R;                // columns a warp: CPL neighbouring ones a lane
    constexpr int COLS = 4 * CW;                    // columns a block
    constexpr int TB = delta_group(DP, CH);         // tokens a group
    // floats a buffer: k, q (, decays) [TB][DP], v [TB][COLS], (g, beta) [TB]; a whole number of 16-byte pieces, so that
    // the second buffer's rows of k, q and decays start on 16-byte borders like the first one's
    constexpr int BUF = (TB * ((CH ? 3 : 2) * DP + COLS + 2) + 3) / 4 * 4;
    extern __shared__ __align__(16) float dsm_[];
    const int seq = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, r = lane % R;
    auto row_of = [&](int ii) { return ((ii >> 2) * R + r) * 4 + (ii & 3); };      // the row that S[.][ii] holds
    const int col_local = warp * CW + (lane / R) * CPL, col0 = blockIdx.z * COLS, col = col0 + col_local;
    const int t0 = cu_seqlens[seq], t1 = cu_seqlens[seq + 1];
    const int slot = seq_slots[seq];
    const int C = 2 * G * d + H * e;
    const bool wide = (d & 3) == 0 && (C & 3) == 0 && (reinterpret_cast<uintptr_t>(xc) & 15) == 0;
    if (slot < 0) {
        if (r == 0)
            for (int t = t0; t < t1; ++t)
#pragma unroll
                for (int cc = 0; cc < CPL; ++cc)
                    if (col + cc < e) o[(size_t)t * H * e + (size_t)h * e + col + cc] = 0.0f;
        return;
    }
    const int kvh = h / (H / G);
    const size_t q_at = (size_t)kvh * d, k_at = (size_t)G * d + (size_t)kvh * d, v_at = 2 * (size_t)G * d + (size_t)h * e;
    float* s_head = state + (size_t)slot * slot_stride + (size_t)h * d * e;
    float S[CPL][DR];
#pragma unroll
    for (int ii = 0; ii < DR; ++ii) {
        const int i = row_of(ii);
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) S[cc][ii] = (i < d && col + cc < e) ? s_head[(size_t)i * e + col + cc] : 0.0f;
    }
    for (int i = tid; i < 2 * BUF; i += 128) dsm_[i] = 0.0f;      // rows beyond d and columns beyond e stay zero
    __syncthreads();
    auto stage = [&](int g0, int buf) {
        const int nt = min(TB, t1 - g0);
        float* kb = dsm_ + buf * BUF;
        float* qb = kb + TB * DP;
        float* gcb = qb + TB * DP;                   // (CH) the tokens' decays per key channel
        float* vb = gcb + (CH ? TB * DP : 0);
        float* gbb = vb + TB * COLS;
        if (CH) {
            const bool wide_g = (d & 3) == 0 && (reinterpret_cast<uintptr_t>(gch) & 15) == 0;
            if (wide_g) {
                const int d4 = d >> 2;
                for (int idx = tid; idx < nt * d4; idx += 128) {
                    const int tt = idx / d4, i = (idx % d4) << 2;
                    cp_async16_(gcb + tt * DP + i, gch + ((size_t)(g0 + tt) * H + h) * d + i);
                }
            } else {
                for (int idx = tid; idx < nt * d; idx += 128) {
                    const int tt = idx / d, i = idx % d;
                    cp_async4(gcb + tt * DP + i, gch + ((size_t)(g0 + tt) * H + h) * d + i);
                }
            }
        }
        if (wide) {          // rows of xc start on 16-byte borders, and so do the heads in them
            const int d4 = d >> 2;
            for (int idx = tid; idx < nt * d4; idx += 128) {
                const int tt = idx / d4, i = (idx % d4) << 2;
                const float* src = xc + (size_t)(g0 + tt) * C;
                cp_async16_(kb + tt * DP + i, src + k_at + i);
                cp_async16_(qb + tt * DP + i, src + q_at + i);
            }
        } else {
            for (int idx = tid; idx < nt * d; idx += 128) {
                const int tt = idx / d, i = idx % d;
                const float* src = xc + (size_t)(g0 + tt) * C;
                cp_async4(kb + tt * DP + i, src + k_at + i);
                cp_async4(qb + tt * DP + i, src + q_at + i);
            }
        }
        for (int idx = tid; idx < nt * COLS; idx += 128) {
            const int tt = idx / COLS, c = idx % COLS;
            if (col0 + c < e) cp_async4(vb + tt * COLS + c, xc + (size_t)(g0 + tt) * C + v_at + col0 + c);
        }
        for (int idx = tid; idx < nt * 2; idx += 128) {
            const int tt = idx >> 1, w = idx & 1;
            cp_async4(gbb + tt * 2 + w, gb + (size_t)(g0 + tt) * 2 * H + (size_t)w * H + h);
        }
    };
    if (t0 < t1) stage(t0, 0);
    cp_async_commit_();
    int buf = 0;
    for (int g0 = t0; g0 < t1; g0 += TB, buf ^= 1) {
        if (g0 + TB < t1) stage(g0 + TB, buf ^ 1);
        cp_async_commit_();
        cp_async_wait_one_();        // this group's copies have landed (the next group's may still fly)
        __syncthreads();
        const int nt = min(TB, t1 - g0);
        const float* kb = dsm_ + buf * BUF;
        const float* qb = kb + TB * DP;
        const float* gcb = qb + TB * DP;             // (CH) the tokens' decays per key channel
        const float* vb = gcb + (CH ? TB * DP : 0);
        const float* gbb = vb + TB * COLS;
        // One token: the chain from token to token is S^T k (DR multiply-adds in four sums, log2(R) shuffles), u, and
        // the update of S, once per column of the lane: the lane's columns are independent chains that share the
        // loads of k and q and fill one another's waits.  The lane's parts of o = S^T q are left in os; their sums
        // over the lanes are off the chain.
        auto token = [&](int tt, float (&os)[CPL]) {
            const float g = gbb[tt * 2], beta = gbb[tt * 2 + 1];
            float kk[DR];
            float p[CPL][4];
#pragma unroll
            for (int cc = 0; cc < CPL; ++cc) p[cc][0] = p[cc][1] = p[cc][2] = p[cc][3] = 0.0f;
#pragma unroll
            for (int c = 0; c < DR / 4; ++c) {
                const float4 k4 = *reinterpret_cast<const float4*>(kb + tt * DP + (c * R + r) * 4);
                kk[4 * c] = k4.x; kk[4 * c + 1] = k4.y; kk[4 * c + 2] = k4.z; kk[4 * c + 3] = k4.w;
                if (CH) {        // S^T k of the decayed state: the rows' decays go with k
                    const float4 g4 = *reinterpret_cast<const float4*>(gcb + tt * DP + (c * R + r) * 4);
                    const float kg[4] = {k4.x * g4.x, k4.y * g4.y, k4.z * g4.z, k4.w * g4.w};
#pragma unroll
                    for (int cc = 0; cc < CPL; ++cc)
#pragma unroll
                        for (int j = 0; j < 4; ++j) p[cc][j] = fmaf(kg[j], S[cc][4 * c + j], p[cc][j]);
                } else {
#pragma unroll
                    for (int cc = 0; cc < CPL; ++cc)
#pragma unroll
                        for (int j = 0; j < 4; ++j) p[cc][j] = fmaf(kk[4 * c + j], S[cc][4 * c + j], p[cc][j]);
                }
            }
            float ks[CPL], u[CPL];
#pragma unroll
            for (int cc = 0; cc < CPL; ++cc) ks[cc] = (p[cc][0] + p[cc][1]) + (p[cc][2] + p[cc][3]);
#pragma unroll
            for (int m = 1; m < R; m <<= 1)
#pragma unroll
                for (int cc = 0; cc < CPL; ++cc) ks[cc] += __shfl_xor_sync(0xffffffffu, ks[cc], m);
            // S^T k of the decayed state is g times that of the old one
#pragma unroll
            for (int cc = 0; cc < CPL; ++cc) u[cc] = beta * (vb[tt * COLS + col_local + cc] - g * ks[cc]);
            float a[CPL][4];
#pragma unroll
            for (int cc = 0; cc < CPL; ++cc) a[cc][0] = a[cc][1] = a[cc][2] = a[cc][3] = 0.0f;
#pragma unroll
            for (int c = 0; c < DR / 4; ++c) {
                const float4 q4 = *reinterpret_cast<const float4*>(qb + tt * DP + (c * R + r) * 4);
                const float qq[4] = {q4.x, q4.y, q4.z, q4.w};
                float gg[4] = {g, g, g, g};
                if (CH) {
                    const float4 g4 = *reinterpret_cast<const float4*>(gcb + tt * DP + (c * R + r) * 4);
                    gg[0] = g4.x; gg[1] = g4.y; gg[2] = g4.z; gg[3] = g4.w;
                }
#pragma unroll
                for (int cc = 0; cc < CPL; ++cc)
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        S[cc][4 * c + j] = fmaf(gg[j], S[cc][4 * c + j], kk[4 * c + j] * u[cc]);
                        a[cc][j] = fmaf(qq[j], S[cc][4 * c + j], a[cc][j]);
                    }
            }
#pragma unroll
            for (int cc = 0; cc < CPL; ++cc) os[cc] = (a[cc][0] + a[cc][1]) + (a[cc][2] + a[cc][3]);
        };
        if (nt == TB) {
            // a whole group, unrolled: the next token's loads issue under this token's chain, and the sums for o of
            // all its tokens are added over the lanes together, as independent chains (the same additions in the same
            // order as one by one)
            float os[TB][CPL];
#pragma unroll
            for (int tt = 0; tt < TB; ++tt) token(tt, os[tt]);
#pragma unroll
            for (int m = 1; m < R; m <<= 1)
#pragma unroll
                for (int tt = 0; tt < TB; ++tt)
#pragma unroll
                    for (int cc = 0; cc < CPL; ++cc) os[tt][cc] += __shfl_xor_sync(0xffffffffu, os[tt][cc], m);
            if (r == 0) {
#pragma unroll
                for (int tt = 0; tt < TB; ++tt)
#pragma unroll
                    for (int cc = 0; cc < CPL; ++cc)
                        if (col + cc < e) o[(size_t)(g0 + tt) * H * e + (size_t)h * e + col + cc] = os[tt][cc];
            }
        } else {
            for (int tt = 0; tt < nt; ++tt) {
                float os[CPL];
                token(tt, os);
#pragma unroll
                for (int m = 1; m < R; m <<= 1)
#pragma unroll
                    for (int cc = 0; cc < CPL; ++cc) os[cc] += __shfl_xor_sync(0xffffffffu, os[cc], m);
                if (r == 0)
#pragma unroll
                    for (int cc = 0; cc < CPL; ++cc)
                        if (col + cc < e) o[(size_t)(g0 + tt) * H * e + (size_t)h * e + col + cc] = os[cc];
            }
        }
        __syncthreads();             // the buffer is free for the group after next
    }
#pragma unroll
    for (int ii = 0; ii < DR; ++ii) {
        const int i = row_of(ii);
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc)
            if (i < d && col + cc < e) s_head[(size_t)i * e + col + cc] = S[cc][ii];
    }
}

template <int DR, int R, int CPL>
static int launch_delta_scan(const float* xc, const float* gb, const float* gch, float* state, long slot_stride, const int* seq_slots, const int* cu_seqlens,
                             float* o, int n_seqs, int H, int G, int d, int e, cudaStream_t st) {
    constexpr int DP = DR * R, COLS = 4 * (CPL * 32 / R);
    constexpr size_t smem = (size_t)2 * ((delta_group(DP, false) * (2 * DP + COLS + 2) + 3) / 4 * 4) * sizeof(float);
    constexpr size_t smem_ch = (size_t)2 * ((delta_group(DP, true) * (3 * DP + COLS + 2) + 3) / 4 * 4) * sizeof(float);
    static_assert(smem <= 48 * 1024 && smem_ch <= 48 * 1024, "the staging buffers fit the default shared memory");
    dim3 grid(n_seqs, H, (e + COLS - 1) / COLS);
    if (gch != nullptr)
        delta_scan_kernel<DR, R, CPL, true><<<grid, 128, smem_ch, st>>>(xc, gb, gch, state, slot_stride, seq_slots, cu_seqlens, o, H, G, d, e);
    else
        delta_scan_kernel<DR, R, CPL, false><<<grid, 128, smem, st>>>(xc, gb, gch, state, slot_stride, seq_slots, cu_seqlens, o, H, G, d, e);
    return 0;
}

// Blocks of one sequence that the choice of lanes a column aims for: two thirds of the SMs of a 148-SM part.
constexpr long kDeltaBlocksWanted = 96;
static int g_delta_lanes = 0;    // a measurement's override of the lanes a column (0: the rule below)
static int g_delta_cpl = 0;      // and of the columns a lane (0: the rule below)
extern "C" void nncpu_delta_scan_force_lanes(int lanes) { g_delta_lanes = lanes; }
extern "C" void nncpu_delta_scan_force_columns(int cpl) { g_delta_cpl = cpl; }

extern "C" int nncpu_delta_scan(const float* xc, const float* gb, const float* gch, float* state, long slot_stride, const int* seq_slots,
                                const int* cu_seqlens, float* o, int n_seqs, int H, int G, int d, int e, void* stream) {
    // gch (optional): float [n_tok, H d], a decay per head and key channel; the per-head decays of gb are then not used
    NN_CHECK(n_seqs >= 0 && H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0, "delta scan: %d sequences, %d heads of %d x %d",
             n_seqs, H, d, e);
    NN_CHECK(d <= 1024, "delta scan: %d key channels a head (at most 1024)", d);
    NN_CHECK(H <= 65535 && e <= 65535 * 16, "delta scan: grid");
    if (n_seqs == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    // R lanes share a column (R * DR rows cover d).  Few lanes a column mean few shuffles and few warps; a sequence alone
    // in a step (a prompt) then leaves most of the GPU idle while every warp walks a chain of dependent instructions
    // a token.  So R grows until ONE sequence's blocks cover most of the SMs (measured: 2 048 tokens of one sequence,
    // 16 heads of 128 x 128: 577 us with 4 lanes, 464 with 8; 64 sequences of one token: 48 against 54).  R follows
    // from the layer's sizes alone, never from the step: with R the order in which a column's products are added
    // changes, and a sequence's numbers must not depend on what else the step holds.
    const int DP = d <= 32 ? 32 : d <= 64 ? 64 : d <= 128 ? 128 : d <= 256 ? 256 : d <= 512 ? 512 : 1024;
    int R = DP / 32 < 4 ? 4 : DP / 32;
    if (g_delta_lanes >= R && g_delta_lanes <= 32 && g_delta_lanes <= DP / 4 && (g_delta_lanes & (g_delta_lanes - 1)) == 0)
        R = g_delta_lanes;
    else
        while (R < 32 && R * 2 <= DP / 4 && (long)H * ((e + 128 / R - 1) / (128 / R)) < kDeltaBlocksWanted) R *= 2;
    // Two columns a lane with twice the lanes a column: the same blocks, warps and registers, but a warp then walks
    // two independent chains that share their loads of k and q.  It pays where the blocks suffice without more lanes
    // (32 heads of 128 x 128: 8 sequences of 512 tokens 847 -> 556 us, one of 2 048 tokens 591 -> 551 us), not where
    // the lanes were raised to get blocks (16 heads, lanes raised to 8: 455 us with one column a lane, 513 with two).
    int CPL = (R == (DP / 32 < 4 ? 4 : DP / 32) && 2 * R <= 32 && 2 * R <= DP / 4) ? 2 : 1;
    if (g_delta_cpl == 1 || g_delta_cpl == 2) CPL = (g_delta_cpl == 2 && 2 * R <= 32 && 2 * R <= DP / 4) ? 2 : 1;
    if (CPL == 2) R *= 2;
#define NN_DELTA(DP_, R_)                                                                                              \
    if (DP == DP_ && R == R_ && CPL == 1)                                                                              \
        launch_delta_scan<DP_ / R_, R_, 1>(xc, gb, gch, state, slot_stride, seq_slots, cu_seqlens, o, n_seqs, H, G, d, e, st); \
    if (DP == DP_ && R == R_ && CPL == 2)                                                                              \
        launch_delta_scan<DP_ / R_, R_, 2>(xc, gb, gch, state, slot_stride, seq_slots, cu_seqlens, o, n_seqs, H, G, d, e, st);
    NN_DELTA(32, 4) NN_DELTA(32, 8)
    NN_DELTA(64, 4) NN_DELTA(64, 8) NN_DELTA(64, 16)
    NN_DELTA(128, 4) NN_DELTA(128, 8) NN_DELTA(128, 16) NN_DELTA(128, 32)
    NN_DELTA(256, 8) NN_DELTA(256, 16) NN_DELTA(256, 32)
    NN_DELTA(512, 16) NN_DELTA(512, 32)
    NN_DELTA(1024, 32)
#undef NN_DELTA
    NN_LAUNCH_OK("delta scan");
    return 0;
}
