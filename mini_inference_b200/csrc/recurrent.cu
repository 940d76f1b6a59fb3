// Matrix-state recurrences: a decayed outer-product accumulation ("lightning") and a gated delta rule with one decay
// per key channel, both over a float32 state S [heads, key_dim, value_dim] that lives in a request's state slot.
//
// The columns of S never mix: every update is "row factors times S, plus key times a row vector", and the read-out
// is S^T q.  So a column is given to LANES = 4 lanes of a warp that hold its rows (row r belongs to lane r % 4) in
// registers for the whole entry; a warp holds 8 neighbouring columns (a 32-byte piece of every row, so that loading
// and storing the state moves whole sectors), a block 32.  A block walks the tokens of ONE entry (a prompt portion or
// a single decoded token) of ONE head in order, staging a few tokens' q, k (g) and v at a time in shared memory; the
// two dot products of a token are finished with two shuffles each.  Everything is float32.
//
// Before the delta rule runs, a kernel per token applies the short causal convolutions (reading the inputs before
// the entry's first token from the state slot), silu, the unit norms of q and k, the sigmoid of beta and the decay
// exp(-exp(A_log) softplus(a + dt_bias)); a small kernel then moves the convolutions' last inputs into the slot.
#include "common.cuh"
#include <math.h>

using namespace mi;

namespace {

constexpr int LANES = 4;          // lanes per column
constexpr int COLS = 32;          // columns per block (4 warps x 8)
constexpr int SCAN_THREADS = 128;

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + expf(-x)); }

struct ScanIds {
    int qs, n, slot, h, l, col, colv, wcol;
};

__device__ __forceinline__ ScanIds scan_ids(const int* seg_q_start, const int* seg_slot, int V) {
    ScanIds s;
    const int seg = blockIdx.x;
    s.qs = seg_q_start[seg];
    s.n = seg_q_start[seg + 1] - s.qs;
    s.slot = seg_slot[seg];
    s.h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    s.l = lane >> 3;
    s.wcol = warp * 8 + (lane & 7);
    s.col = blockIdx.z * COLS + s.wcol;
    s.colv = s.col < V;
    return s;
}

// ------------------------------------------------------------------ lightning: S <- decay S + k v^T; o = S^T q
// p [T, ldp] holds q | k | v (before silu) at columns 0, H D, 2 H D.  grid (entries, heads, ceil(V / 32)).
template <typename T, int RP>
__global__ void __launch_bounds__(SCAN_THREADS) lightning_scan_kernel(
        const T* __restrict__ p, int ldp, const float* __restrict__ decay, float* __restrict__ state, long long state_stride,
        float* __restrict__ out, const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot, int H, int D, int V, int TC) {
    extern __shared__ float sm[];
    float* qsm = sm;                      // [TC, D]
    float* ksm = qsm + TC * D;            // [TC, D]
    float* vsm = ksm + TC * D;            // [TC, COLS]
    const ScanIds id = scan_ids(seg_q_start, seg_slot, V);
    float* S = state + (long long)id.slot * state_stride + (long long)id.h * D * V;
    float s[RP];
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int r = id.l + LANES * i;
        s[i] = (r < D && id.colv) ? S[(size_t)r * V + id.col] : 0.f;
    }
    const float dec = decay[id.h];
    for (int t0 = 0; t0 < id.n; t0 += TC) {
        const int nt = min(TC, id.n - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * D; idx += SCAN_THREADS) {
            const int tt = idx / D, d = idx - tt * D;
            const T* row = p + (size_t)(id.qs + t0 + tt) * ldp + (size_t)id.h * D + d;
            qsm[idx] = silu(to_f32(row[0]));
            ksm[idx] = silu(to_f32(row[(size_t)H * D]));
        }
        for (int idx = threadIdx.x; idx < nt * COLS; idx += SCAN_THREADS) {
            const int tt = idx / COLS, c = idx - tt * COLS, cc = blockIdx.z * COLS + c;
            vsm[idx] = cc < V ? silu(to_f32(p[(size_t)(id.qs + t0 + tt) * ldp + (size_t)2 * H * D + (size_t)id.h * V + cc])) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vv = vsm[tt * COLS + id.wcol];
            const float* kk = ksm + tt * D;
            const float* qq = qsm + tt * D;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < RP; ++i) {
                const int r = id.l + LANES * i;
                if (r < D) {
                    s[i] = fmaf(dec, s[i], kk[r] * vv);
                    acc = fmaf(s[i], qq[r], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (id.l == 0 && id.colv) out[(size_t)(id.qs + t0 + tt) * H * V + (size_t)id.h * V + id.col] = acc;
        }
    }
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int r = id.l + LANES * i;
        if (r < D && id.colv) S[(size_t)r * V + id.col] = s[i];
    }
}

// ------------------------------------------------------------------ delta rule with a decay per key channel
// prep float32 [T, ld]: q [KV D] | k [KV D] | v [H V] | beta [H] | g [H D] (what delta_prepare_kernel wrote).
//   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (the read-out sees the token's own write)
template <int RP>
__global__ void __launch_bounds__(SCAN_THREADS) delta_scan_kernel(
        const float* __restrict__ prep, int ld, float* __restrict__ state, long long state_stride, float* __restrict__ out,
        const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot, int H, int KV, int D, int V, int TC) {
    extern __shared__ float sm[];
    float* qsm = sm;
    float* ksm = qsm + TC * D;
    float* gsm = ksm + TC * D;
    float* vsm = gsm + TC * D;            // [TC, COLS]
    float* bsm = vsm + TC * COLS;         // [TC]
    const ScanIds id = scan_ids(seg_q_start, seg_slot, V);
    const int kvh = id.h / (H / KV);
    const int C = 2 * KV * D + H * V;
    float* S = state + (long long)id.slot * state_stride + (long long)id.h * D * V;
    float s[RP];
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int r = id.l + LANES * i;
        s[i] = (r < D && id.colv) ? S[(size_t)r * V + id.col] : 0.f;
    }
    for (int t0 = 0; t0 < id.n; t0 += TC) {
        const int nt = min(TC, id.n - t0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < nt * D; idx += SCAN_THREADS) {
            const int tt = idx / D, d = idx - tt * D;
            const float* row = prep + (size_t)(id.qs + t0 + tt) * ld;
            qsm[idx] = row[kvh * D + d];
            ksm[idx] = row[KV * D + kvh * D + d];
            gsm[idx] = row[C + H + id.h * D + d];
        }
        for (int idx = threadIdx.x; idx < nt * COLS; idx += SCAN_THREADS) {
            const int tt = idx / COLS, c = idx - tt * COLS, cc = blockIdx.z * COLS + c;
            vsm[idx] = cc < V ? prep[(size_t)(id.qs + t0 + tt) * ld + 2 * KV * D + id.h * V + cc] : 0.f;
        }
        for (int tt = threadIdx.x; tt < nt; tt += SCAN_THREADS) bsm[tt] = prep[(size_t)(id.qs + t0 + tt) * ld + C + id.h];
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float vv = vsm[tt * COLS + id.wcol], beta = bsm[tt];
            const float* kk = ksm + tt * D;
            const float* qq = qsm + tt * D;
            const float* gg = gsm + tt * D;
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < RP; ++i) {
                const int r = id.l + LANES * i;
                if (r < D) {
                    s[i] *= gg[r];
                    dot = fmaf(s[i], kk[r], dot);
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 8);
            dot += __shfl_xor_sync(0xffffffffu, dot, 16);
            const float u = beta * (vv - dot);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < RP; ++i) {
                const int r = id.l + LANES * i;
                if (r < D) {
                    s[i] = fmaf(kk[r], u, s[i]);
                    acc = fmaf(s[i], qq[r], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 8);
            acc += __shfl_xor_sync(0xffffffffu, acc, 16);
            if (id.l == 0 && id.colv) out[(size_t)(id.qs + t0 + tt) * H * V + (size_t)id.h * V + id.col] = acc;
        }
    }
#pragma unroll
    for (int i = 0; i < RP; ++i) {
        const int r = id.l + LANES * i;
        if (r < D && id.colv) S[(size_t)r * V + id.col] = s[i];
    }
}

// ------------------------------------------------------------------ what enters the delta rule, per token
// p [T, ldp]: q | k | v (C = 2 KV D + H V channels that pass the convolution) | beta logits [H] | ...
// a [T, lda]: decay logits [H D].  conv [C, taps], the last tap multiplies the current token.  The inputs of the
// taps - 1 positions before an entry's first token are rows of hist = state[slot] + hist_off, [taps - 1, C]
// (zeros for a request's first entry: the slot is zeroed when it is claimed).
template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ p, int ldp, const T* __restrict__ a, int lda,
                                     const float* __restrict__ conv, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                     const float* __restrict__ state, long long state_stride, long long hist_off,
                                     float* __restrict__ out, int ldo, const int* __restrict__ token_seg,
                                     const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
                                     int H, int KV, int D, int V, int taps, float unit_eps) {
    extern __shared__ float y[];          // [C]
    const int t = blockIdx.x, seg = token_seg[t], qs = seg_q_start[seg], r = t - qs;
    const int C = 2 * KV * D + H * V;
    const float* hist = state + (long long)seg_slot[seg] * state_stride + hist_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int off = r - (taps - 1 - j);
            const float x = off >= 0 ? to_f32(p[(size_t)(qs + off) * ldp + c]) : hist[(size_t)(taps - 1 + off) * C + c];
            acc = fmaf(conv[(size_t)c * taps + j], x, acc);
        }
        y[c] = silu(acc);
    }
    __syncthreads();
    float* o = out + (size_t)t * ldo;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int hd = warp; hd < 2 * KV; hd += warps) {          // unit vectors; q is also scaled by D^-1/2
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) ss += y[hd * D + d] * y[hd * D + d];
        float inv = 1.f / sqrtf(warp_sum(ss) + unit_eps);
        if (hd < KV) inv *= rsqrtf((float)D);
        for (int d = lane; d < D; d += 32) o[hd * D + d] = y[hd * D + d] * inv;
    }
    for (int c = 2 * KV * D + threadIdx.x; c < C; c += blockDim.x) o[c] = y[c];
    for (int h = threadIdx.x; h < H; h += blockDim.x) o[C + h] = sigmoidf(to_f32(p[(size_t)t * ldp + C + h]));
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
        const float x = to_f32(a[(size_t)t * lda + i]) + dt_bias[i];
        const float sp = x > 20.f ? x : log1pf(expf(x));
        o[C + H + i] = expf(-expf(A_log[i / D]) * sp);
    }
}

// hist[j] <- input at (entry's end - (taps - 1) + j), j = 0 .. taps - 2; a thread owns a channel and goes up in j, so an
// entry shorter than taps - 1 shifts its own rows safely.
template <typename T>
__global__ void conv_tail_kernel(const T* __restrict__ p, int ldp, float* __restrict__ state, long long state_stride, long long hist_off,
                                 const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot, int C, int taps) {
    const int seg = blockIdx.x, qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs;
    float* hist = state + (long long)seg_slot[seg] * state_stride + hist_off;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= C) return;
    for (int j = 0; j < taps - 1; ++j) {
        const int src = n - (taps - 1) + j;
        hist[(size_t)j * C + c] = src >= 0 ? to_f32(p[(size_t)(qs + src) * ldp + c]) : hist[(size_t)(taps - 1 + src) * C + c];
    }
}

inline int pick_chunk(int floats_per_token) {      // tokens staged at a time: 16, or 8 when 16 would pass 48 KB
    return floats_per_token * 16 * 4 <= 48 * 1024 ? 16 : 8;
}

}  // namespace

MI_EXPORT int mi_lightning_scan(const void* p, int ldp, const float* decay, float* state, long long state_stride, float* out,
                                const int* seg_q_start, const int* seg_slot, int num_segs, int H, int D, int V, int dtype,
                                cudaStream_t stream) {
    if (num_segs == 0) return 0;
    if (D > 256 || H > 65535) return -2;
    const int TC = pick_chunk(2 * D + COLS);
    const size_t smem = (size_t)TC * (2 * D + COLS) * sizeof(float);
    dim3 grid(num_segs, H, (V + COLS - 1) / COLS);
#define GO(T, RP) lightning_scan_kernel<T, RP><<<grid, SCAN_THREADS, smem, stream>>>((const T*)p, ldp, decay, state, state_stride, out, \
                                                                                      seg_q_start, seg_slot, H, D, V, TC)
#define PICK(T) do { if (D <= 32) GO(T, 8); else if (D <= 64) GO(T, 16); else if (D <= 128) GO(T, 32); else GO(T, 64); } while (0)
    if (dtype == MI_BF16) PICK(__nv_bfloat16); else PICK(float);
#undef PICK
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_delta_scan(const float* prep, int ld, float* state, long long state_stride, float* out, const int* seg_q_start,
                            const int* seg_slot, int num_segs, int H, int KV, int D, int V, cudaStream_t stream) {
    if (num_segs == 0) return 0;
    if (D > 256 || H > 65535) return -2;
    const int TC = pick_chunk(3 * D + COLS + 1);
    const size_t smem = (size_t)TC * (3 * D + COLS + 1) * sizeof(float);
    dim3 grid(num_segs, H, (V + COLS - 1) / COLS);
#define GO(RP) delta_scan_kernel<RP><<<grid, SCAN_THREADS, smem, stream>>>(prep, ld, state, state_stride, out, seg_q_start, seg_slot, H, KV, D, V, TC)
    if (D <= 32) GO(8); else if (D <= 64) GO(16); else if (D <= 128) GO(32); else GO(64);
#undef GO
    return (int)cudaGetLastError();
}

MI_EXPORT int mi_delta_prepare(const void* p, int ldp, const void* a, int lda, const float* conv, const float* A_log, const float* dt_bias,
                               float* state, long long state_stride, long long hist_off, float* out, int ldo, const int* token_seg,
                               const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int H, int KV, int D, int V, int taps,
                               float unit_eps, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    const int C = 2 * KV * D + H * V;
    const size_t smem = (size_t)C * sizeof(float);
    if (smem > 200 * 1024) return -2;
    if (dtype == MI_BF16) {
        auto k = delta_prepare_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<T_, 256, smem, stream>>>((const __nv_bfloat16*)p, ldp, (const __nv_bfloat16*)a, lda, conv, A_log, dt_bias, state, state_stride,
                                     hist_off, out, ldo, token_seg, seg_q_start, seg_slot, H, KV, D, V, taps, unit_eps);
    } else {
        auto k = delta_prepare_kernel<float>;
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        k<<<T_, 256, smem, stream>>>((const float*)p, ldp, (const float*)a, lda, conv, A_log, dt_bias, state, state_stride, hist_off, out, ldo,
                                     token_seg, seg_q_start, seg_slot, H, KV, D, V, taps, unit_eps);
    }
    int err = (int)cudaGetLastError();
    if (err || taps <= 1) return err;
    dim3 grid(num_segs, (C + 255) / 256);
    if (dtype == MI_BF16)
        conv_tail_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)p, ldp, state, state_stride, hist_off, seg_q_start, seg_slot, C, taps);
    else
        conv_tail_kernel<float><<<grid, 256, 0, stream>>>((const float*)p, ldp, state, state_stride, hist_off, seg_q_start, seg_slot, C, taps);
    return (int)cudaGetLastError();
}
