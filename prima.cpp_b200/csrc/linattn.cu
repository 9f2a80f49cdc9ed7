// prima.cpp_b200/csrc/linattn.cu — linear attention with a fixed decay per head (declaration and semantics: layers.h, launch_decay_attn):
//     S_t = decay_h S_{t-1} + k_t v_t^T,   y_t = S_t^T q_t          S [dim][vdim] fp32 per (sequence slot, head)
// with an optional SiLU on q, k, v and a factor on k applied while the inputs are staged.  The recurrence, the state and everything that
// enters it are fp32.  Two kernels, as for the Mamba-2 scan (mixers.cu): the state in registers for dim <= 256, in shared memory above.
#include <cuda_runtime.h>
#include <math.h>

#include "layers.h"
#include "mixers.cuh"

namespace pb {
namespace {

struct DecayIO {
    const float * qkv;
    int64_t ld;
    int q_off, k_off, v_off;
};
__device__ __forceinline__ float in_act(float v, int act) { return act ? silu_f(v) : v; }

// A CTA owns one head and 16 value columns.  LN lanes share a column: thread (pl = tid / LN, ng = tid % LN) keeps S[n][column pl] for
// n = ng, ng + LN, ... (NREG values), so a token costs each thread NREG fused steps and the column one LN-lane shuffle reduction, and
// the CTA's 16 LN / 32 warps hide each other's latencies.  Tokens are walked in chunks of 16 whose k, q and v rows go through registers
// into shared memory: the loads of the next chunk are issued before the current chunk's recurrence and land while it runs; two CTA
// barriers per chunk, none per token.
constexpr int DCHUNK = 16, DCOLS = 16;
template <int NREG, int LN>
__global__ void __launch_bounds__(DCOLS * LN) k_decay_attn_reg(DecayIO io, const int32_t * __restrict__ slot, const int32_t * __restrict__ off, DecayAttnParams p,
                                                               const float * __restrict__ decay, float * __restrict__ state, int64_t slot_stride,
                                                               float * __restrict__ y) {
    extern __shared__ float sm[];
    constexpr int NT = DCOLS * LN;                                 // threads
    constexpr int NV = (DCHUNK * DCOLS + NT - 1) / NT;             // staged v elements per thread
    const int N = p.dim, P = p.vdim, inner = p.heads * p.vdim;
    const int ptiles = (P + DCOLS - 1) / DCOLS;
    const int h = blockIdx.x / ptiles, pt = blockIdx.x - h * ptiles, e = blockIdx.y;
    const int tid = threadIdx.x, pl = tid / LN, ng = tid % LN;
    const int pcol = pt * DCOLS + pl;
    const bool pok = pcol < P;
    float * Ks = sm;                        // [DCHUNK][N]
    float * Qs = Ks + DCHUNK * N;           // [DCHUNK][N]
    float * Vs = Qs + DCHUNK * N;           // [DCHUNK][DCOLS]
    float * gst = state + (int64_t) slot[e] * slot_stride + (int64_t) h * N * P;
    float S[NREG];
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int nn = ng + LN * j;
        S[j] = (pok && nn < N) ? gst[(int64_t) nn * P + pcol] : 0.f;
    }
    const float dec = decay[h];
    const int t0 = off[e], n = off[e + 1] - t0;
    // staged element i = tid + NT k of a chunk: (token i / N, entry i % N) of k and q (N <= LN NREG, so k < NREG); (token i / 16, column i % 16) of v
    float rk[NREG], rq[NREG], rv[NV];
    auto fetch = [&](int c0) {
        const int nc = min(DCHUNK, n - c0);
#pragma unroll
        for (int k = 0; k < NREG; k++) {
            const int i = tid + NT * k;
            if (i < nc * N) {
                const int tt = i / N, nn = i - tt * N;
                const float * row = io.qkv + (int64_t) (t0 + c0 + tt) * io.ld + h * N + nn;
                rk[k] = row[io.k_off];
                rq[k] = row[io.q_off];
            }
        }
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int i = tid + NT * k, tt = i / DCOLS, pp = i - tt * DCOLS;
            rv[k] = (tt < nc && pt * DCOLS + pp < P) ? io.qkv[(int64_t) (t0 + c0 + tt) * io.ld + io.v_off + h * P + pt * DCOLS + pp] : 0.f;
        }
    };
    if (n > 0) fetch(0);
    for (int c0 = 0; c0 < n; c0 += DCHUNK) {
        const int nc = min(DCHUNK, n - c0);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < NREG; k++) {
            const int i = tid + NT * k;
            if (i < nc * N) {
                Ks[i] = in_act(rk[k], p.act) * p.k_scale;
                Qs[i] = in_act(rq[k], p.act);
            }
        }
#pragma unroll
        for (int k = 0; k < NV; k++)
            if (tid + NT * k < DCHUNK * DCOLS) Vs[tid + NT * k] = in_act(rv[k], p.act);
        __syncthreads();
        if (c0 + DCHUNK < n) fetch(c0 + DCHUNK);
        for (int tt = 0; tt < nc; tt++) {
            const float xv = Vs[tt * DCOLS + pl];
            const float * Kr = Ks + tt * N, * Qr = Qs + tt * N;
            float acc = 0.f;
#pragma unroll
            for (int j = 0; j < NREG; j++) {
                const int nn = ng + LN * j;
                if (nn < N) {
                    S[j] = fmaf(dec, S[j], Kr[nn] * xv);
                    acc = fmaf(S[j], Qr[nn], acc);
                }
            }
#pragma unroll
            for (int o = 1; o < LN; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (ng == 0 && pok) y[(int64_t) (t0 + c0 + tt) * inner + h * P + pcol] = acc;
        }
    }
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int nn = ng + LN * j;
        if (pok && nn < N) gst[(int64_t) nn * P + pcol] = S[j];
    }
}

// one CTA per (head, 64 value columns, entry); the state tile S [N][64] lives in shared memory for the whole entry
constexpr int SCOLS = 64;
__global__ void __launch_bounds__(256) k_decay_attn_smem(DecayIO io, const int32_t * __restrict__ slot, const int32_t * __restrict__ off, DecayAttnParams p,
                                                         const float * __restrict__ decay, float * __restrict__ state, int64_t slot_stride,
                                                         float * __restrict__ y) {
    extern __shared__ float sm[];
    const int N = p.dim, P = p.vdim, inner = p.heads * p.vdim;
    const int ptiles = (P + SCOLS - 1) / SCOLS;
    const int h = blockIdx.x / ptiles, pt = blockIdx.x - h * ptiles, e = blockIdx.y;
    const int c0 = pt * SCOLS, nc = min(SCOLS, P - c0);
    float * S = sm;                // [N][SCOLS]
    float * ks = S + N * SCOLS;    // [N]
    float * qs = ks + N;           // [N]
    float * vs = qs + N;           // [SCOLS]
    float * part = vs + SCOLS;     // [4][SCOLS]
    float * gst = state + (int64_t) slot[e] * slot_stride + (int64_t) h * N * P;
    for (int i = threadIdx.x; i < N * SCOLS; i += blockDim.x) {
        const int nn = i / SCOLS, cc = i - nn * SCOLS;
        S[i] = cc < nc ? gst[(int64_t) nn * P + c0 + cc] : 0.f;
    }
    const float dec = decay[h];
    const int t0 = off[e], n = off[e + 1] - t0;
    const int cc = threadIdx.x & (SCOLS - 1), q4 = threadIdx.x / SCOLS;   // column, quarter of the rows
    for (int lt = 0; lt < n; lt++) {
        const float * row = io.qkv + (int64_t) (t0 + lt) * io.ld;
        __syncthreads();
        for (int i = threadIdx.x; i < N; i += blockDim.x) {
            ks[i] = in_act(row[io.k_off + h * N + i], p.act) * p.k_scale;
            qs[i] = in_act(row[io.q_off + h * N + i], p.act);
        }
        for (int i = threadIdx.x; i < SCOLS; i += blockDim.x) vs[i] = i < nc ? in_act(row[io.v_off + h * P + c0 + i], p.act) : 0.f;
        __syncthreads();
        float acc = 0.f;
        const float xv = vs[cc];
        for (int nn = q4; nn < N; nn += 4) {
            const float s = fmaf(dec, S[nn * SCOLS + cc], ks[nn] * xv);
            S[nn * SCOLS + cc] = s;
            acc = fmaf(s, qs[nn], acc);
        }
        part[q4 * SCOLS + cc] = acc;
        __syncthreads();
        if (threadIdx.x < nc) y[(int64_t) (t0 + lt) * inner + h * P + c0 + threadIdx.x] =
            (part[threadIdx.x] + part[SCOLS + threadIdx.x]) + (part[2 * SCOLS + threadIdx.x] + part[3 * SCOLS + threadIdx.x]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < N * SCOLS; i += blockDim.x) {
        const int nn = i / SCOLS, c2 = i - nn * SCOLS;
        if (c2 < nc) gst[(int64_t) nn * P + c0 + c2] = S[i];
    }
}

}  // namespace

int launch_decay_attn(const float * qkv, int64_t ld, int q_off, int k_off, int v_off, const BatchView & b, const DecayAttnParams & p, const float * decay,
                      float * state, int64_t slot_stride, float * y, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (p.heads <= 0 || p.dim <= 0 || p.vdim <= 0 || !decay || !state) return (int) cudaErrorInvalidValue;
    const DecayIO io{qkv, ld, q_off, k_off, v_off};
    if (p.dim <= 256) {
        // lanes per column by the size of a key: 8 (dim <= 32), 16 (<= 64), 32 above; each lane then holds 1, 2, 4 or 8 state values of its column
        const int ln = p.dim <= 32 ? 8 : p.dim <= 64 ? 16 : 32;
        const int nreg = (p.dim + ln - 1) / ln;
        const size_t smem = ((size_t) 2 * DCHUNK * p.dim + DCHUNK * DCOLS) * sizeof(float);
        const dim3 grid((unsigned) (p.heads * ((p.vdim + DCOLS - 1) / DCOLS)), (unsigned) b.n_entries);
#define PB_DECAY(NR, LNV) return ck_launch([&] { k_decay_attn_reg<NR, LNV><<<grid, DCOLS * LNV, smem, st>>>(io, b.slot, b.off, p, decay, state, slot_stride, y); })
#define PB_DECAY_LN(LNV)           \
    do {                           \
        if (nreg <= 1) PB_DECAY(1, LNV); \
        if (nreg <= 2) PB_DECAY(2, LNV); \
        if (nreg <= 4) PB_DECAY(4, LNV); \
        PB_DECAY(8, LNV);          \
    } while (0)
        if (ln == 8) PB_DECAY_LN(8);
        if (ln == 16) PB_DECAY_LN(16);
        PB_DECAY_LN(32);
#undef PB_DECAY_LN
#undef PB_DECAY
    }
    const size_t smem = ((size_t) p.dim * SCOLS + 2 * (size_t) p.dim + 5 * SCOLS) * sizeof(float);
    if (smem > 220 * 1024) return (int) cudaErrorInvalidValue;
    int rc = raise_smem(k_decay_attn_smem, smem);
    if (rc) return rc;
    const dim3 grid((unsigned) (p.heads * ((p.vdim + SCOLS - 1) / SCOLS)), (unsigned) b.n_entries);
    return ck_launch([&] { k_decay_attn_smem<<<grid, 256, smem, st>>>(io, b.slot, b.off, p, decay, state, slot_stride, y); });
}

}  // namespace pb
