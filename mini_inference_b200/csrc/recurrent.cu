// Matrix-state recurrences: a decayed outer-product accumulation ("lightning") and a gated delta rule with one decay
// per key channel, both over a float32 state S [heads, key_dim, value_dim] that lives in a request's state slot.
//
// The columns of S never mix: every update is "row factors times S, plus key times a row vector", and the read-out
// is S^T q.  So a PAIR of neighbouring columns is given to LN lanes of a warp that hold its rows in registers for the
// whole entry (lane l owns the rows 4 (l + LN g) + e, g = 0 .. NG-1, e = 0 .. 3: groups of four neighbouring rows, so
// that the lanes fetch a token's q, k and g from shared memory as full wavefronts of 16-byte loads, and each fetched
// number serves two columns).  With LN = 8 a warp holds 4 pairs = 8 neighbouring columns (a 32-byte piece of every
// row: loading and storing the state moves whole sectors) and a block 32: the form for decode steps.  For prompt
// portions what counts is the chain of dependent instructions per token, so LN grows to 16 or 32 (one group of four
// rows per lane) and eight times as many warps share a head.  A block
// walks the tokens of ONE entry (a prompt portion or a single decoded token) of ONE head in order.  What a token
// brings (q, k, g, its 32 values, beta: float32, written by a prologue kernel) is staged a few tokens at a time in
// one of two shared-memory buffers with cp.async, the next chunk travelling while the current one is worked on.  The
// delta rule's S^T k of a token's two columns is finished together with log2(LN) + 1 shuffles, since the update needs it;
// the partial sums of the read-out S^T q wait in shared memory and are added up (in lane order) and stored, coalesced,
// once per chunk.  Everything is float32.
//
// Prologue kernels, one small block per (token, unit): lightning: silu of q, k, v.  Delta rule: the short causal
// convolutions (the inputs before an entry's first token come from the state slot), silu, the unit norms of q and k,
// sigmoid(beta logits), and the decay exp(-exp(A_log) softplus(a + dt_bias)); a last kernel then moves the
// convolutions' newest inputs into the slot.
#include "common.cuh"
#include <math.h>

using namespace mi;

namespace {

constexpr int SCAN_THREADS = 128;
// LN lanes share a pair of columns (8: a warp holds 4 pairs, the state moves in 32-byte pieces, few blocks: decode steps,
// where the state's bytes are the cost; 16 or 32: fewer rows per lane, so a token's chain of dependent instructions is
// shorter and more warps share the work: prompt portions, where the tokens' latency is the cost).  Columns per block:
constexpr int cols_of(int LN) { return 4 * (32 / LN) * 2; }

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + expf(-x)); }

__device__ __forceinline__ void cp16(float* dst, const float* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" :: "r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N) : "memory"); }

// Where the scan finds a token's numbers in its float32 row (ld floats per token).
struct ScanLayout {
    int ld, q_off, k_off, v_off, g_off, b_off;      // q/k: + kv_head * D; v: + head * V; g: + head * D; beta: + head
};

// One chunk of nt tokens into a buffer: q, k (g) rows of Dp floats (D copied, the rest stays zero), v [COLS], beta.
template <bool DELTA, int COLS>
__device__ __forceinline__ void stage_chunk(float* buf, int Dp, int TC, const float* __restrict__ prep, const ScanLayout L,
                                            int tok0, int nt, int h, int kvh, int D, int V, int col0, bool vec) {
    float* qsm = buf;
    float* ksm = qsm + TC * Dp;
    float* gsm = ksm + TC * Dp;                               // DELTA only
    float* vsm = DELTA ? gsm + TC * Dp : ksm + TC * Dp;       // [TC, COLS]
    float* bsm = vsm + TC * COLS;                             // [TC] (DELTA only)
    const int ncol = min(COLS, V - col0);
    if (vec) {
        const int dq = D >> 2, vq = ncol >> 2;
        for (int idx = threadIdx.x; idx < nt * dq; idx += SCAN_THREADS) {
            const int tt = idx / dq, c = (idx - tt * dq) << 2;
            const float* row = prep + (size_t)(tok0 + tt) * L.ld;
            cp16(qsm + tt * Dp + c, row + L.q_off + kvh * D + c);
            cp16(ksm + tt * Dp + c, row + L.k_off + kvh * D + c);
            if (DELTA) cp16(gsm + tt * Dp + c, row + L.g_off + h * D + c);
        }
        for (int idx = threadIdx.x; idx < nt * vq; idx += SCAN_THREADS) {
            const int tt = idx / vq, c = (idx - tt * vq) << 2;
            cp16(vsm + tt * COLS + c, prep + (size_t)(tok0 + tt) * L.ld + L.v_off + h * V + col0 + c);
        }
    } else {
        for (int idx = threadIdx.x; idx < nt * D; idx += SCAN_THREADS) {
            const int tt = idx / D, c = idx - tt * D;
            const float* row = prep + (size_t)(tok0 + tt) * L.ld;
            qsm[tt * Dp + c] = row[L.q_off + kvh * D + c];
            ksm[tt * Dp + c] = row[L.k_off + kvh * D + c];
            if (DELTA) gsm[tt * Dp + c] = row[L.g_off + h * D + c];
        }
        for (int idx = threadIdx.x; idx < nt * ncol; idx += SCAN_THREADS) {
            const int tt = idx / ncol, c = idx - tt * ncol;
            vsm[tt * COLS + c] = prep[(size_t)(tok0 + tt) * L.ld + L.v_off + h * V + col0 + c];
        }
    }
    if (DELTA)
        for (int tt = threadIdx.x; tt < nt; tt += SCAN_THREADS) bsm[tt] = prep[(size_t)(tok0 + tt) * L.ld + L.b_off + h];
}

// Sums a0 and a1 over the LN row lanes of a column pair (the low lane bits) with log2(LN) + 1 shuffles; every lane gets both.
template <int LN>
__device__ __forceinline__ float2 reduce_pair(float a0, float a1, int l) {
    const bool odd = l & 1;
    float keep = odd ? a1 : a0;
    keep += __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1);
#pragma unroll
    for (int o = 2; o < LN; o <<= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
    const float other = __shfl_xor_sync(0xffffffffu, keep, 1);
    return odd ? make_float2(other, keep) : make_float2(keep, other);
}

// grid (entries, heads, ceil(V / cols_of(LN))).  DELTA:  S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.
// otherwise:  S <- decay[h] S + k v^T; o = S^T q.   NG: groups of four rows per lane (key_dim <= 4 LN NG).
template <bool DELTA, int LN, int NG>
__global__ void __launch_bounds__(SCAN_THREADS) state_scan_kernel(
        const float* __restrict__ prep, const ScanLayout L, const float* __restrict__ decay, float* __restrict__ state,
        long long state_stride, float* __restrict__ out, const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
        int H, int KV, int D, int V, int TC, int vec) {
    extern __shared__ __align__(16) float sm[];
    constexpr int LANES = LN, COLS = cols_of(LN), Dp = 4 * LN * NG;
    const int buf_floats = TC * ((DELTA ? 3 : 2) * Dp + COLS + (DELTA ? 1 : 0));
    const int buf_stride = (buf_floats + 3) & ~3;
    float* part = sm + 2 * buf_stride;                         // [TC, COLS, LN + 1] partial sums of the read-out
    const int seg = blockIdx.x, h = blockIdx.y, kvh = h / (H / KV);
    const int qs = seg_q_start[seg], n = seg_q_start[seg + 1] - qs, slot = seg_slot[seg];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int l = lane & (LANES - 1), wcol = (warp * (32 / LANES) + lane / LANES) * 2, col0 = blockIdx.z * COLS, col = col0 + wcol;
    const bool v0 = col < V, v1 = col + 1 < V;
    for (int i = threadIdx.x; i < 2 * buf_stride; i += SCAN_THREADS) sm[i] = 0.f;       // the pads beyond D (and V) stay zero
    float* S = state + (long long)slot * state_stride + (long long)h * D * V;
    __syncthreads();
    // the first chunk's copies start before the state is fetched, so that the two waits for global memory overlap
    const int chunks = (n + TC - 1) / TC;
    stage_chunk<DELTA, COLS>(sm, Dp, TC, prep, L, qs, min(TC, n), h, kvh, D, V, col0, (vec & 1) != 0);
    cp_commit();
    float s0[4 * NG], s1[4 * NG];
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = 4 * (l + LANES * g) + e;
            if (vec & 2) {                                     // even V and slot size: a pair of columns is one 8-byte access
                const float2 t = (r < D && v0) ? *reinterpret_cast<const float2*>(S + (size_t)r * V + col) : make_float2(0.f, 0.f);
                s0[4 * g + e] = t.x; s1[4 * g + e] = t.y;
            } else {
                s0[4 * g + e] = (r < D && v0) ? S[(size_t)r * V + col] : 0.f;
                s1[4 * g + e] = (r < D && v1) ? S[(size_t)r * V + col + 1] : 0.f;
            }
        }
    const float dec = DELTA ? 0.f : decay[h];
    for (int c = 0; c < chunks; ++c) {
        const int t0 = c * TC, nt = min(TC, n - t0);
        if (c + 1 < chunks) {
            stage_chunk<DELTA, COLS>(sm + ((c + 1) & 1) * buf_stride, Dp, TC, prep, L, qs + t0 + TC, min(TC, n - t0 - TC), h, kvh, D, V, col0, (vec & 1) != 0);
            cp_commit();
            cp_wait<1>();
        } else {
            cp_wait<0>();
        }
        __syncthreads();
        const float* buf = sm + (c & 1) * buf_stride;
        const float* qsm = buf;
        const float* ksm = qsm + TC * Dp;
        const float* gsm = ksm + TC * Dp;
        const float* vsm = DELTA ? gsm + TC * Dp : ksm + TC * Dp;
        const float* bsm = vsm + TC * COLS;
        // two partial sums per dot product and column keep the chains of dependent additions short
        for (int tt = 0; tt < nt; ++tt) {
            const float2 vv = *reinterpret_cast<const float2*>(vsm + tt * COLS + wcol);
            const float4* kk = reinterpret_cast<const float4*>(ksm + tt * Dp) + l;
            const float4* qq = reinterpret_cast<const float4*>(qsm + tt * Dp) + l;
            float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;                 // a: first column, b: second column
            if (DELTA) {
                const float4* gg = reinterpret_cast<const float4*>(gsm + tt * Dp) + l;
                float d0 = 0.f, d1 = 0.f, e0 = 0.f, e1 = 0.f;
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float4 gv = gg[LANES * g], kv = kk[LANES * g];
                    s0[4 * g] *= gv.x; s0[4 * g + 1] *= gv.y; s0[4 * g + 2] *= gv.z; s0[4 * g + 3] *= gv.w;
                    s1[4 * g] *= gv.x; s1[4 * g + 1] *= gv.y; s1[4 * g + 2] *= gv.z; s1[4 * g + 3] *= gv.w;
                    d0 = fmaf(s0[4 * g], kv.x, d0); d1 = fmaf(s0[4 * g + 1], kv.y, d1);
                    d0 = fmaf(s0[4 * g + 2], kv.z, d0); d1 = fmaf(s0[4 * g + 3], kv.w, d1);
                    e0 = fmaf(s1[4 * g], kv.x, e0); e1 = fmaf(s1[4 * g + 1], kv.y, e1);
                    e0 = fmaf(s1[4 * g + 2], kv.z, e0); e1 = fmaf(s1[4 * g + 3], kv.w, e1);
                }
                const float2 dot = reduce_pair<LN>(d0 + d1, e0 + e1, l);
                const float beta = bsm[tt];
                const float u0 = beta * (vv.x - dot.x), u1 = beta * (vv.y - dot.y);
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float4 kv = kk[LANES * g], qv = qq[LANES * g];
                    s0[4 * g] = fmaf(kv.x, u0, s0[4 * g]); s0[4 * g + 1] = fmaf(kv.y, u0, s0[4 * g + 1]);
                    s0[4 * g + 2] = fmaf(kv.z, u0, s0[4 * g + 2]); s0[4 * g + 3] = fmaf(kv.w, u0, s0[4 * g + 3]);
                    s1[4 * g] = fmaf(kv.x, u1, s1[4 * g]); s1[4 * g + 1] = fmaf(kv.y, u1, s1[4 * g + 1]);
                    s1[4 * g + 2] = fmaf(kv.z, u1, s1[4 * g + 2]); s1[4 * g + 3] = fmaf(kv.w, u1, s1[4 * g + 3]);
                    a0 = fmaf(s0[4 * g], qv.x, a0); a1 = fmaf(s0[4 * g + 1], qv.y, a1);
                    a0 = fmaf(s0[4 * g + 2], qv.z, a0); a1 = fmaf(s0[4 * g + 3], qv.w, a1);
                    b0 = fmaf(s1[4 * g], qv.x, b0); b1 = fmaf(s1[4 * g + 1], qv.y, b1);
                    b0 = fmaf(s1[4 * g + 2], qv.z, b0); b1 = fmaf(s1[4 * g + 3], qv.w, b1);
                }
            } else {
#pragma unroll
                for (int g = 0; g < NG; ++g) {
                    const float4 kv = kk[LANES * g], qv = qq[LANES * g];
                    s0[4 * g] = fmaf(dec, s0[4 * g], kv.x * vv.x); s0[4 * g + 1] = fmaf(dec, s0[4 * g + 1], kv.y * vv.x);
                    s0[4 * g + 2] = fmaf(dec, s0[4 * g + 2], kv.z * vv.x); s0[4 * g + 3] = fmaf(dec, s0[4 * g + 3], kv.w * vv.x);
                    s1[4 * g] = fmaf(dec, s1[4 * g], kv.x * vv.y); s1[4 * g + 1] = fmaf(dec, s1[4 * g + 1], kv.y * vv.y);
                    s1[4 * g + 2] = fmaf(dec, s1[4 * g + 2], kv.z * vv.y); s1[4 * g + 3] = fmaf(dec, s1[4 * g + 3], kv.w * vv.y);
                    a0 = fmaf(s0[4 * g], qv.x, a0); a1 = fmaf(s0[4 * g + 1], qv.y, a1);
                    a0 = fmaf(s0[4 * g + 2], qv.z, a0); a1 = fmaf(s0[4 * g + 3], qv.w, a1);
                    b0 = fmaf(s1[4 * g], qv.x, b0); b1 = fmaf(s1[4 * g + 1], qv.y, b1);
                    b0 = fmaf(s1[4 * g + 2], qv.z, b0); b1 = fmaf(s1[4 * g + 3], qv.w, b1);
                }
            }
            // the read-out feeds nothing back: its partial sums wait in shared memory until the chunk's tokens are done
            part[(tt * COLS + wcol) * (LANES + 1) + l] = a0 + a1;
            part[(tt * COLS + wcol + 1) * (LANES + 1) + l] = b0 + b1;
        }
        __syncthreads();                                       // partial sums complete; the staging buffer is free for the chunk after the next
        for (int o = threadIdx.x; o < nt * COLS; o += SCAN_THREADS) {
            const int tt = o / COLS, ci = o - tt * COLS;
            const float* pp = part + o * (LANES + 1);
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < LANES; ++i) acc += pp[i];
            if (col0 + ci < V) out[(size_t)(qs + t0 + tt) * H * V + (size_t)h * V + col0 + ci] = acc;
        }
    }
#pragma unroll
    for (int g = 0; g < NG; ++g)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = 4 * (l + LANES * g) + e;
            if (vec & 2) {
                if (r < D && v0) *reinterpret_cast<float2*>(S + (size_t)r * V + col) = make_float2(s0[4 * g + e], s1[4 * g + e]);
            } else {
                if (r < D && v0) S[(size_t)r * V + col] = s0[4 * g + e];
                if (r < D && v1) S[(size_t)r * V + col + 1] = s1[4 * g + e];
            }
        }
}

template <bool DELTA>
int launch_scan(const float* prep, ScanLayout L, const float* decay, float* state, long long state_stride, float* out,
                const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int H, int KV, int D, int V, cudaStream_t stream) {
    if (num_segs == 0) return 0;
    if (D > 256 || H > 65535) return -2;
    // entries of many tokens: as many lanes per column pair as leave a lane one group of four rows (up to a warp);
    // decode steps: 8 lanes, so that a warp moves the state in whole sectors
    int LN = 8;
    if (T_ > 4 * num_segs) LN = D > 64 ? 32 : D > 32 ? 16 : 8;
    const int NG = (D + 4 * LN - 1) / (4 * LN);
    const int COLS = cols_of(LN);
    const int per_token = (DELTA ? 3 : 2) * 4 * LN * NG + COLS + 1;
    const int per_chunk_token = 2 * per_token + COLS * (LN + 1);          // two staging buffers and the partial sums
    const int TC = T_ <= 4 * num_segs ? 4 : per_chunk_token * 16 * 4 <= 96 * 1024 ? 16 : per_chunk_token * 8 * 4 <= 96 * 1024 ? 8 : 4;   // decode steps: small buffers, more blocks per SM
    const size_t smem = (2 * (size_t)((TC * per_token + 3) & ~3) + (size_t)TC * COLS * (LN + 1)) * sizeof(float);
    // 16-byte copies need every piece on a 16-byte boundary: sizes and offsets in multiples of four floats
    const int vec = (((uintptr_t)prep % 16 == 0 && D % 4 == 0 && V % 4 == 0 && L.ld % 4 == 0 && L.q_off % 4 == 0 && L.k_off % 4 == 0 &&
                     L.v_off % 4 == 0 && (!DELTA || L.g_off % 4 == 0)) ? 1 : 0)
                  | ((V % 2 == 0 && state_stride % 2 == 0 && (uintptr_t)state % 8 == 0) ? 2 : 0);      // bit 1: the state in 8-byte pairs
    dim3 grid(num_segs, H, (V + COLS - 1) / COLS);
#define GO(LN_, N) do { \
        auto kern = state_scan_kernel<DELTA, LN_, N>; \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
        kern<<<grid, SCAN_THREADS, smem, stream>>>(prep, L, decay, state, state_stride, out, seg_q_start, seg_slot, H, KV, D, V, TC, vec); } while (0)
    if (LN == 32) { if (NG == 1) GO(32, 1); else GO(32, 2); }
    else if (LN == 16) GO(16, 1);
    else { if (NG == 1) GO(8, 1); else if (NG == 2) GO(8, 2); else if (NG == 4) GO(8, 4); else GO(8, 8); }
#undef GO
    return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ lightning prologue: out = silu(p[:, :n]) in float32
template <typename T>
__global__ void silu_f32_kernel(const T* __restrict__ p, int ldp, float* __restrict__ out, int n) {
    const T* row = p + (size_t)blockIdx.x * ldp;
    float* o = out + (size_t)blockIdx.x * n;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) o[i] = silu(to_f32(row[i]));
}

// ------------------------------------------------------------------ retention prologue: rotate q and k, scale k, all to float32
// p [T, ldp] = q [H D] | k [H D] | v [H V].  The first 2 * half coordinates of every q and k head are turned in the
// rotate-half layout (coordinate i pairs with i + half; angle = position * inv_freq[i], float32), the rest pass;
// k is then multiplied by k_scale.  out [T, 2 H D + H V] float32.
template <typename T>
__global__ void rotate_f32_kernel(const T* __restrict__ p, int ldp, float* __restrict__ out, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, int half, float k_scale, int H, int D, int V) {
    const T* row = p + (size_t)blockIdx.x * ldp;
    const int HD = H * D, n = 2 * HD + H * V;
    float* o = out + (size_t)blockIdx.x * n;
    const float pos = (float)positions[blockIdx.x];
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        float v = to_f32(row[i]);
        if (i < 2 * HD) {
            const int d = i % D;
            if (d < 2 * half) {
                const bool low = d < half;
                const float other = to_f32(row[low ? i + half : i - half]);
                float sn, cs;
                sincosf(pos * inv_freq[low ? d : d - half], &sn, &cs);
                v = low ? v * cs - other * sn : v * cs + other * sn;
            }
            if (i >= HD) v *= k_scale;
        }
        o[i] = v;
    }
}

// ------------------------------------------------------------------ delta-rule prologue, one block per (token, unit)
// p [T, ldp]: q | k | v (C = 2 KV D + H V channels that pass the convolution) | beta logits [H] | ...
// a [T, lda]: decay logits [H D].  conv [C, taps], the last tap multiplies the current token.  The inputs of the
// taps - 1 positions before an entry's first token are rows of hist = state[slot] + hist_off, [taps - 1, C]
// (zeros for a request's first entry: the slot is zeroed when it is claimed).
// Units: 0 .. 2 KV - 1 a q or k head (convolution, silu, unit norm; q also * D^-1/2); then H value heads
// (convolution, silu); then H decay heads; then one unit for all beta.  out [T, ldo]: q | k | v | g | beta (ldo may pad).
template <typename T>
__device__ __forceinline__ float conv_silu(const T* __restrict__ p, int ldp, const float* __restrict__ conv, const float* __restrict__ hist,
                                           int C, int taps, int qs, int r, int c) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
        const int off = r - (taps - 1 - j);
        const float x = off >= 0 ? to_f32(p[(size_t)(qs + off) * ldp + c]) : hist[(size_t)(taps - 1 + off) * C + c];
        acc = fmaf(conv[(size_t)c * taps + j], x, acc);
    }
    return silu(acc);
}

template <typename T>
__global__ void delta_prepare_kernel(const T* __restrict__ p, int ldp, const T* __restrict__ a, int lda,
                                     const float* __restrict__ conv, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                     const float* __restrict__ state, long long state_stride, long long hist_off,
                                     float* __restrict__ out, int ldo, const int* __restrict__ token_seg,
                                     const int* __restrict__ seg_q_start, const int* __restrict__ seg_slot,
                                     int H, int KV, int D, int V, int taps, float unit_eps, int T_, int toks) {
    __shared__ float scratch[32];
    const int unit = blockIdx.y;
    const int C = 2 * KV * D + H * V;
    for (int t = blockIdx.x * toks; t < min(T_, (int)(blockIdx.x + 1) * toks); ++t) {      // a block takes a unit of a few neighbouring tokens
    const int seg = token_seg[t], qs = seg_q_start[seg], r = t - qs;
    const float* hist = state + (long long)seg_slot[seg] * state_stride + hist_off;
    float* o = out + (size_t)t * ldo;
    if (unit < 2 * KV) {
        const int c0 = unit * D;
        float ss = 0.f;
        for (int d = threadIdx.x; d < D; d += 128) { const float y = conv_silu(p, ldp, conv, hist, C, taps, qs, r, c0 + d); ss += y * y; }
        float inv = 1.f / sqrtf(block_sum<128>(ss, scratch) + unit_eps);
        if (unit < KV) inv *= rsqrtf((float)D);
        for (int d = threadIdx.x; d < D; d += 128) o[c0 + d] = conv_silu(p, ldp, conv, hist, C, taps, qs, r, c0 + d) * inv;
    } else if (unit < 2 * KV + H) {
        const int c0 = 2 * KV * D + (unit - 2 * KV) * V;
        for (int i = threadIdx.x; i < V; i += 128) o[c0 + i] = conv_silu(p, ldp, conv, hist, C, taps, qs, r, c0 + i);
    } else if (unit < 2 * KV + 2 * H) {
        const int hh = unit - 2 * KV - H;
        const float rate = expf(A_log[hh]);
        for (int d = threadIdx.x; d < D; d += 128) {
            const float x = to_f32(a[(size_t)t * lda + hh * D + d]) + dt_bias[hh * D + d];
            const float sp = x > 20.f ? x : log1pf(expf(x));
            o[C + hh * D + d] = expf(-rate * sp);
        }
    } else {
        for (int h = threadIdx.x; h < H; h += 128) o[C + H * D + h] = sigmoidf(to_f32(p[(size_t)t * ldp + C + h]));
    }
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

}  // namespace

// p [T, ldp] = q | k | v before silu (2 H D + H V columns); prep: float32 scratch [T, 2 H D + H V]; out float32 [T, H V].
MI_EXPORT int mi_lightning_scan(const void* p, int ldp, float* prep, const float* decay, float* state, long long state_stride, float* out,
                                const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int H, int D, int V, int dtype,
                                cudaStream_t stream) {
    if (num_segs == 0 || T_ == 0) return 0;
    const int n = 2 * H * D + H * V;
    dim3 pgrid(T_, T_ >= 256 ? 1 : min(8, (n + 255) / 256));
    if (dtype == MI_BF16) silu_f32_kernel<__nv_bfloat16><<<pgrid, 256, 0, stream>>>((const __nv_bfloat16*)p, ldp, prep, n);
    else silu_f32_kernel<float><<<pgrid, 256, 0, stream>>>((const float*)p, ldp, prep, n);
    int err = (int)cudaGetLastError();
    if (err) return err;
    ScanLayout L{n, 0, H * D, 2 * H * D, 0, 0};
    return launch_scan<false>(prep, L, decay, state, state_stride, out, seg_q_start, seg_slot, T_, num_segs, H, H, D, V, stream);
}

// p [T, ldp] = q | k | v as projected; inv_freq: half frequencies (nullptr or half = 0: no rotation).  Otherwise as mi_lightning_scan.
MI_EXPORT int mi_retention_scan(const void* p, int ldp, float* prep, const int* positions, const float* inv_freq, int half, float k_scale,
                                const float* decay, float* state, long long state_stride, float* out, const int* seg_q_start,
                                const int* seg_slot, int T_, int num_segs, int H, int D, int V, int dtype, cudaStream_t stream) {
    if (num_segs == 0 || T_ == 0) return 0;
    if (2 * half > D) return -2;
    const int n = 2 * H * D + H * V;
    dim3 pgrid(T_, T_ >= 256 ? 1 : min(8, (n + 255) / 256));
    if (dtype == MI_BF16) rotate_f32_kernel<__nv_bfloat16><<<pgrid, 256, 0, stream>>>((const __nv_bfloat16*)p, ldp, prep, positions, inv_freq, inv_freq ? half : 0, k_scale, H, D, V);
    else rotate_f32_kernel<float><<<pgrid, 256, 0, stream>>>((const float*)p, ldp, prep, positions, inv_freq, inv_freq ? half : 0, k_scale, H, D, V);
    int err = (int)cudaGetLastError();
    if (err) return err;
    ScanLayout L{n, 0, H * D, 2 * H * D, 0, 0};
    return launch_scan<false>(prep, L, decay, state, state_stride, out, seg_q_start, seg_slot, T_, num_segs, H, H, D, V, stream);
}

MI_EXPORT int mi_delta_scan(const float* prep, int ld, float* state, long long state_stride, float* out, const int* seg_q_start,
                            const int* seg_slot, int T_, int num_segs, int H, int KV, int D, int V, cudaStream_t stream) {
    const int C = 2 * KV * D + H * V;
    ScanLayout L{ld, 0, KV * D, 2 * KV * D, C, C + H * D};
    return launch_scan<true>(prep, L, nullptr, state, state_stride, out, seg_q_start, seg_slot, T_, num_segs, H, KV, D, V, stream);
}

MI_EXPORT int mi_delta_prepare(const void* p, int ldp, const void* a, int lda, const float* conv, const float* A_log, const float* dt_bias,
                               float* state, long long state_stride, long long hist_off, float* out, int ldo, const int* token_seg,
                               const int* seg_q_start, const int* seg_slot, int T_, int num_segs, int H, int KV, int D, int V, int taps,
                               float unit_eps, int dtype, cudaStream_t stream) {
    if (T_ == 0) return 0;
    const int C = 2 * KV * D + H * V;
    const int units = 2 * KV + 2 * H + 1;
    if (units > 65535) return -2;
    const int toks = T_ >= 1024 ? 8 : 1;
    dim3 pgrid((T_ + toks - 1) / toks, units);
    if (dtype == MI_BF16)
        delta_prepare_kernel<__nv_bfloat16><<<pgrid, 128, 0, stream>>>((const __nv_bfloat16*)p, ldp, (const __nv_bfloat16*)a, lda, conv, A_log, dt_bias,
                                                                       state, state_stride, hist_off, out, ldo, token_seg, seg_q_start, seg_slot,
                                                                       H, KV, D, V, taps, unit_eps, T_, toks);
    else
        delta_prepare_kernel<float><<<pgrid, 128, 0, stream>>>((const float*)p, ldp, (const float*)a, lda, conv, A_log, dt_bias, state, state_stride,
                                                               hist_off, out, ldo, token_seg, seg_q_start, seg_slot, H, KV, D, V, taps, unit_eps, T_, toks);
    int err = (int)cudaGetLastError();
    if (err || taps <= 1) return err;
    dim3 grid(num_segs, (C + 255) / 256);
    if (dtype == MI_BF16)
        conv_tail_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)p, ldp, state, state_stride, hist_off, seg_q_start, seg_slot, C, taps);
    else
        conv_tail_kernel<float><<<grid, 256, 0, stream>>>((const float*)p, ldp, state, state_stride, hist_off, seg_q_start, seg_slot, C, taps);
    return (int)cudaGetLastError();
}
