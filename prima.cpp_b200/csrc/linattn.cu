// prima.cpp_b200/csrc/linattn.cu — linear attention with a fixed decay per head (declaration and semantics: layers.h, launch_decay_attn):
//     S_t = decay_h S_{t-1} + k_t v_t^T,   y_t = S_t^T q_t          S [dim][vdim] fp32 per (sequence slot, head)
// with an optional SiLU on q, k, v and a factor on k applied while the inputs are staged.  The recurrence, the state and everything that
// enters it are fp32.  Two kernels, as for the Mamba-2 scan (mixers.cu): the state in registers for dim <= 128, in shared memory above.
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

// A CTA of 128 threads owns one head and 32 value columns; thread (pl = tid / 8, ng = tid % 8) keeps S[n][column] for columns pl and
// pl + 16 and n = ng, ng + 8, ... (2 x NREG values).  Tokens are walked in chunks of 16 whose k, q and v rows are staged in shared
// memory by the whole CTA (two CTA barriers per chunk, none per token); y needs one 8-lane shuffle reduction per token.
constexpr int DCHUNK = 16, DCOLS = 32;
template <int NREG>
__global__ void __launch_bounds__(128) k_decay_attn_reg(DecayIO io, const int32_t * __restrict__ slot, const int32_t * __restrict__ off, DecayAttnParams p,
                                                        const float * __restrict__ decay, float * __restrict__ state, int64_t slot_stride,
                                                        float * __restrict__ y) {
    extern __shared__ float sm[];
    const int N = p.dim, P = p.vdim, inner = p.heads * p.vdim;
    const int ptiles = (P + DCOLS - 1) / DCOLS;
    const int h = blockIdx.x / ptiles, pt = blockIdx.x - h * ptiles, e = blockIdx.y;
    const int tid = threadIdx.x, pl = tid >> 3, ng = tid & 7;
    const int pcol = pt * DCOLS + pl, pcol1 = pcol + 16;
    const bool pok = pcol < P, pok1 = pcol1 < P;
    float * Ks = sm;                        // [DCHUNK][N]
    float * Qs = Ks + DCHUNK * N;           // [DCHUNK][N]
    float * Vs = Qs + DCHUNK * N;           // [DCHUNK][DCOLS]
    float * gst = state + (int64_t) slot[e] * slot_stride + (int64_t) h * N * P;
    float S[NREG], S1[NREG];
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int nn = ng + 8 * j;
        S[j] = (pok && nn < N) ? gst[(int64_t) nn * P + pcol] : 0.f;
        S1[j] = (pok1 && nn < N) ? gst[(int64_t) nn * P + pcol1] : 0.f;
    }
    const float dec = decay[h];
    const int t0 = off[e], n = off[e + 1] - t0;
    for (int c0 = 0; c0 < n; c0 += DCHUNK) {
        const int nc = min(DCHUNK, n - c0);
        __syncthreads();
        for (int i = tid; i < nc * N; i += 128) {
            const int tt = i / N, nn = i - tt * N;
            const float * row = io.qkv + (int64_t) (t0 + c0 + tt) * io.ld + h * N + nn;
            Ks[i] = in_act(row[io.k_off], p.act) * p.k_scale;
            Qs[i] = in_act(row[io.q_off], p.act);
        }
        for (int i = tid; i < nc * DCOLS; i += 128) {
            const int tt = i / DCOLS, pp = i - tt * DCOLS;
            Vs[i] = pt * DCOLS + pp < P ? in_act(io.qkv[(int64_t) (t0 + c0 + tt) * io.ld + io.v_off + h * P + pt * DCOLS + pp], p.act) : 0.f;
        }
        __syncthreads();
        for (int tt = 0; tt < nc; tt++) {
            const float xv = Vs[tt * DCOLS + pl], xv1 = Vs[tt * DCOLS + pl + 16];
            const float * Kr = Ks + tt * N, * Qr = Qs + tt * N;
            float acc = 0.f, acc1 = 0.f;
#pragma unroll
            for (int j = 0; j < NREG; j++) {
                const int nn = ng + 8 * j;
                if (nn < N) {
                    const float kv = Kr[nn], qv = Qr[nn];
                    S[j] = fmaf(dec, S[j], kv * xv);
                    S1[j] = fmaf(dec, S1[j], kv * xv1);
                    acc = fmaf(S[j], qv, acc);
                    acc1 = fmaf(S1[j], qv, acc1);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 4);
            if (ng == 0 && pok) y[(int64_t) (t0 + c0 + tt) * inner + h * P + pcol] = acc;
            if (ng == 0 && pok1) y[(int64_t) (t0 + c0 + tt) * inner + h * P + pcol1] = acc1;
        }
    }
#pragma unroll
    for (int j = 0; j < NREG; j++) {
        const int nn = ng + 8 * j;
        if (pok && nn < N) gst[(int64_t) nn * P + pcol] = S[j];
        if (pok1 && nn < N) gst[(int64_t) nn * P + pcol1] = S1[j];
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
    if (p.dim <= 128) {
        const size_t smem = ((size_t) 2 * DCHUNK * p.dim + DCHUNK * DCOLS) * sizeof(float);
        const dim3 grid((unsigned) (p.heads * ((p.vdim + DCOLS - 1) / DCOLS)), (unsigned) b.n_entries);
        const int nreg = (p.dim + 7) / 8;
#define PB_DECAY(NR) return ck_launch([&] { k_decay_attn_reg<NR><<<grid, 128, smem, st>>>(io, b.slot, b.off, p, decay, state, slot_stride, y); })
        if (nreg <= 1) PB_DECAY(1);
        if (nreg <= 2) PB_DECAY(2);
        if (nreg <= 4) PB_DECAY(4);
        if (nreg <= 8) PB_DECAY(8);
        PB_DECAY(16);
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
