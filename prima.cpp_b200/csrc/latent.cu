// prima.cpp_b200/csrc/latent.cu — the steps of softmax attention over a low-rank latent around the shared attention kernels of mixers.cu
// (declarations and semantics: layers.h).  A sequence slot caches per position one row [normed latent (kv_rank) | rotated key part
// (rot_dim) that all heads share].  Prompts expand keys and values from the latent with dense products and run the prompt attention
// kernel with the shared key tail; a decode step folds the key up-projection into the query (qa = W_uk^T q), so that a cache row is
// the key of every head as it stands and its latent part the value, walks the rows split over many CTAs, and applies the value
// up-projection to the merged weighted sum of latents.  Norms, positions, angles, scores, weights and rotations are fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

#include "layers.h"
#include "mixers.cuh"

namespace pb {
namespace {

// rotates the pair (u, v) = (x[i], x[i + half]) by the angle pos * freq[i]; cos and sin carry the factor mag
__device__ __forceinline__ void turn(float u, float v, int pos, float f, float mag, float & ou, float & ov) {
    const float ang = (float) pos * f;
    const float c = cosf(ang) * mag, s = sinf(ang) * mag;
    ou = u * c - v * s;
    ov = v * c + u * s;
}

template <typename OT>
__global__ void __launch_bounds__(256) k_latent_prep(const float * __restrict__ proj, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                                     const int32_t * __restrict__ pos0, const int32_t * __restrict__ entry_of, LatentParams p,
                                                     const float * __restrict__ wq, const float * __restrict__ wkv, const float * __restrict__ freq, float eps,
                                                     OT * __restrict__ cq, float * __restrict__ cache, int64_t slot_stride) {
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int pos = pos0[e] + (t - off[e]);
    const int C = latent_proj_cols(p), Rq = p.q_rank, R = p.kv_rank, Dr = p.rot_dim;
    const float * row = proj + (int64_t) t * C;
    float s = 0.f;
    for (int i = threadIdx.x; i < Rq; i += blockDim.x) s = fmaf(row[i], row[i], s);
    const float invq = 1.f / sqrtf(block_sum(s, red) / (float) Rq + eps);
    for (int i = threadIdx.x; i < Rq; i += blockDim.x) put(cq, (int64_t) t * Rq + i, row[i] * invq * wq[i]);
    if (!p.own_kv) return;
    const float * kv = row + Rq + p.heads * p.vdim;
    s = 0.f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) s = fmaf(kv[i], kv[i], s);
    const float invk = 1.f / sqrtf(block_sum(s, red) / (float) R + eps);
    float * crow = cache + (int64_t) slot[e] * slot_stride + (int64_t) pos * (R + Dr);
    for (int i = threadIdx.x; i < R; i += blockDim.x) crow[i] = kv[i] * invk * wkv[i];
    const int half = p.rot_dims / 2;
    for (int i = threadIdx.x; i < Dr; i += blockDim.x) {
        if (i < half) {
            float a, b;
            turn(kv[R + i], kv[R + i + half], pos, freq[i], p.rot_mag, a, b);
            crow[R + i] = a;
            crow[R + i + half] = b;
        } else if (i >= 2 * half) {
            crow[R + i] = kv[R + i];
        }
    }
}

__global__ void k_latent_rope_q(float * __restrict__ q, const int32_t * __restrict__ off, const int32_t * __restrict__ pos0,
                                const int32_t * __restrict__ entry_of, LatentParams p, const float * __restrict__ freq) {
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int pos = pos0[e] + (t - off[e]);
    const int half = p.rot_dims / 2, DQ = p.dim + p.rot_dim;
    float * row = q + (int64_t) t * p.heads * DQ;
    for (int i = threadIdx.x; i < p.heads * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        float * r = row + h * DQ + p.dim;
        float a, b;
        turn(r[j], r[j + half], pos, freq[j], p.rot_mag, a, b);
        r[j] = a;
        r[j + half] = b;
    }
}

template <typename OT>
__global__ void k_latent_gather(const float * __restrict__ cache, int64_t slot_stride, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                const int32_t * __restrict__ pos0, const int32_t * __restrict__ entry_of, LatentParams p, OT * __restrict__ lat,
                                float * __restrict__ kr) {
    const int t = blockIdx.x;
    const int e = entry_of[t];
    const int pos = pos0[e] + (t - off[e]);
    const int R = p.kv_rank, Dr = p.rot_dim;
    const float * crow = cache + (int64_t) slot[e] * slot_stride + (int64_t) pos * (R + Dr);
    for (int i = threadIdx.x; i < R; i += blockDim.x) put(lat, (int64_t) t * R + i, crow[i]);
    for (int i = threadIdx.x; i < Dr; i += blockDim.x) kr[(int64_t) t * Dr + i] = crow[R + i];
}

// CTA (head, token, 128 latent entries): qa[r] = sum_d W_uk[h * dim + d][r] q[d]; thread r walks a column of the head's block (coalesced
// over r, eight loads in flight)
template <typename WT>
__global__ void __launch_bounds__(128) k_latent_absorb_q(const float * __restrict__ q, const int32_t * __restrict__ off, const int32_t * __restrict__ pos0,
                                                         const int32_t * __restrict__ entry_of, const WT * __restrict__ wuk, LatentParams p,
                                                         const float * __restrict__ freq, float * __restrict__ qa) {
    extern __shared__ float qs[];   // [dim]
    const int h = blockIdx.x, t = blockIdx.y;
    const int D = p.dim, Dr = p.rot_dim, R = p.kv_rank;
    const float * qr = q + ((int64_t) t * p.heads + h) * (D + Dr);
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qr[d];
    __syncthreads();
    float * out = qa + ((int64_t) t * p.heads + h) * (R + Dr);
    const WT * w = wuk + (int64_t) h * D * R;
    const int r = blockIdx.z * 128 + threadIdx.x;
    if (r < R) {
        float acc = 0.f;
        int d = 0;
        for (; d + 7 < D; d += 8) {
            float wv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) wv[u] = ld_f(w, (int64_t) (d + u) * R + r);
#pragma unroll
            for (int u = 0; u < 8; u++) acc = fmaf(wv[u], qs[d + u], acc);
        }
        for (; d < D; d++) acc = fmaf(ld_f(w, (int64_t) d * R + r), qs[d], acc);
        out[r] = acc;
    }
    if (blockIdx.z == 0) {   // the rotated part, turned here by the token's position
        const int e = entry_of[t], pos = pos0[e] + (t - off[e]), half = p.rot_dims / 2;
        for (int i = threadIdx.x; i < Dr; i += blockDim.x) {
            if (i < half) {
                float a, b;
                turn(qr[D + i], qr[D + i + half], pos, freq[i], p.rot_mag, a, b);
                out[R + i] = a;
                out[R + i + half] = b;
            } else if (i >= 2 * half) {
                out[R + i] = qr[D + i];
            }
        }
    }
}

// one CTA per (head, token): a warp per output row of the head's block of W_uv, lanes split the latent
template <typename WT, typename OT>
__global__ void __launch_bounds__(256) k_latent_up_v(const float * __restrict__ olat, const WT * __restrict__ wuv, LatentParams p,
                                                     const float * __restrict__ gate, int64_t ldg, OT * __restrict__ out) {
    extern __shared__ float os[];   // [kv_rank]
    const int h = blockIdx.x, t = blockIdx.y;
    const int R = p.kv_rank, DV = p.vdim;
    const float * orow = olat + ((int64_t) t * p.heads + h) * R;
    for (int r = threadIdx.x; r < R; r += blockDim.x) os[r] = orow[r];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int dv = warp; dv < DV; dv += (int) (blockDim.x >> 5)) {
        const float acc = wsum(dot_lane8(wuv + ((int64_t) h * DV + dv) * R, os, R, lane));
        if (lane == 0) put(out, (int64_t) t * p.heads * DV + h * DV + dv, acc * sigmoid_f(gate[(int64_t) t * ldg + h * DV + dv]));
    }
}

// Decode attention over the latent cache, split over the rows: CTA (split, entry, group of 16 heads) walks its share of the slot's rows
// in tiles of 16 staged in shared memory.  Thread (head, row) scores one cache row against one head's folded query (the whole row is
// the key), the 16 lanes of a head keep its running max / sum, and every thread accumulates two latent columns of all 16 heads (the
// value is the row's latent part) -- a row is read once for all heads of the group.  Partial (sum, max, normaliser) per split go to
// `part` [entry][split][head][kv_rank + 2]; k_latent_merge_up_v combines them.  The share of a split depends on the sequence's own
// length only, so a token's result does not depend on the batch around it.
constexpr int LT_ROWS = 16, LT_HEADS = 16;
__global__ void __launch_bounds__(256) k_latent_decode_split(const float * __restrict__ qa, const int32_t * __restrict__ slot, const int32_t * __restrict__ off,
                                                             const int32_t * __restrict__ pos0, LatentParams p, const float * __restrict__ cache,
                                                             int64_t slot_stride, int splits, float * __restrict__ part) {
    extern __shared__ float sm[];
    const int s = blockIdx.x, e = blockIdx.y, h0 = blockIdx.z * LT_HEADS;
    const int H = p.heads, R = p.kv_rank, RW = R + p.rot_dim, RWP = RW | 1;
    const int nh = min(LT_HEADS, H - h0);
    float * tile = sm;                        // [LT_ROWS][RWP]
    float * qs = tile + LT_ROWS * RWP;        // [LT_HEADS][RW]
    float * P = qs + LT_HEADS * RW;           // [LT_HEADS][LT_ROWS]
    float * mrun = P + LT_HEADS * LT_ROWS;    // [LT_HEADS] running max, then running sum, then this tile's factor on what was gathered before
    float * lrun = mrun + LT_HEADS;
    float * corr = lrun + LT_HEADS;
    const int tid = threadIdx.x, hl = tid >> 4, r = tid & 15;
    const int rows_used = pos0[e] + 1;        // the token's own row is in the cache already
    const int per = ((rows_used + splits - 1) / splits + LT_ROWS - 1) / LT_ROWS * LT_ROWS;
    const int r_lo = s * per, r_hi = min(rows_used, r_lo + per);
    const float * qrow = qa + ((int64_t) off[e] * H + h0) * RW;
    for (int i0 = tid; i0 < nh * RW; i0 += 256 * 8) {   // eight loads in flight per thread
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) { const int i = i0 + 256 * u; v[u] = i < nh * RW ? qrow[i] : 0.f; }
#pragma unroll
        for (int u = 0; u < 8; u++) { const int i = i0 + 256 * u; if (i < nh * RW) qs[i] = v[u] * p.scale; }
    }
    if (tid < LT_HEADS) { mrun[tid] = -INFINITY; lrun[tid] = 0.f; }
    float acc[LT_HEADS][2];
#pragma unroll
    for (int h = 0; h < LT_HEADS; h++) acc[h][0] = acc[h][1] = 0.f;
    const float * crow = cache + (int64_t) slot[e] * slot_stride;
    const bool c0ok = tid < R, c1ok = tid + 256 < R;
    for (int r0 = r_lo; r0 < r_hi; r0 += LT_ROWS) {
        const int nr = min(LT_ROWS, r_hi - r0);
        __syncthreads();
        {   // the tile's rows are one contiguous piece of the cache: eight loads per thread in flight before the first store
            const float * src = crow + (int64_t) r0 * RW;
            const int n_src = nr * RW, n_all = LT_ROWS * RW;
            for (int i0 = tid; i0 < n_all; i0 += 256 * 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; u++) { const int i = i0 + 256 * u; v[u] = i < n_src ? src[i] : 0.f; }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int i = i0 + 256 * u;
                    if (i < n_all) { const int rr = i / RW; tile[rr * RWP + (i - rr * RW)] = v[u]; }
                }
            }
        }
        __syncthreads();
        float sc = -INFINITY;
        if (hl < nh && r < nr) {
            const float * q = qs + hl * RW, * k = tile + r * RWP;
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            int d = 0;
            for (; d + 3 < RW; d += 4) {
                a0 = fmaf(q[d], k[d], a0); a1 = fmaf(q[d + 1], k[d + 1], a1);
                a2 = fmaf(q[d + 2], k[d + 2], a2); a3 = fmaf(q[d + 3], k[d + 3], a3);
            }
            for (; d < RW; d++) a0 = fmaf(q[d], k[d], a0);
            sc = (a0 + a1) + (a2 + a3);
        }
        float tmax = sc;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
        const float mo = mrun[hl];
        const float mn = fmaxf(mo, tmax);
        const float pv = sc == -INFINITY ? 0.f : expf(sc - mn);
        float ps = pv;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        P[hl * LT_ROWS + r] = pv;
        __syncwarp();
        if (r == 0) {
            const float c = mn == -INFINITY ? 1.f : (mo == -INFINITY ? 0.f : expf(mo - mn));
            lrun[hl] = lrun[hl] * c + ps;
            mrun[hl] = mn;
            corr[hl] = c;
        }
        __syncthreads();
#pragma unroll
        for (int h = 0; h < LT_HEADS; h++) { const float c = corr[h]; acc[h][0] *= c; acc[h][1] *= c; }
        for (int rr = 0; rr < nr; rr++) {
            const float v0 = c0ok ? tile[rr * RWP + tid] : 0.f, v1 = c1ok ? tile[rr * RWP + tid + 256] : 0.f;
#pragma unroll
            for (int h = 0; h < LT_HEADS; h++) {
                const float pw = P[h * LT_ROWS + rr];
                acc[h][0] = fmaf(pw, v0, acc[h][0]);
                acc[h][1] = fmaf(pw, v1, acc[h][1]);
            }
        }
    }
    float * pp = part + (((int64_t) e * splits + s) * H + h0) * (R + 2);
#pragma unroll
    for (int h = 0; h < LT_HEADS; h++) {
        if (h < nh) {
            if (c0ok) pp[(int64_t) h * (R + 2) + tid] = acc[h][0];
            if (c1ok) pp[(int64_t) h * (R + 2) + tid + 256] = acc[h][1];
        }
    }
    __syncthreads();
    if (tid < nh) { pp[(int64_t) tid * (R + 2) + R] = mrun[tid]; pp[(int64_t) tid * (R + 2) + R + 1] = lrun[tid]; }
}

// CTA (head, entry, half of the value rows): the splits' partial sums become the weighted sum of latents (both halves compute it), then
// a warp per output row of the head's block of W_uv (lanes split the latent) and the output gate.  Up to 64 splits: a lane of warp 0
// weighs splits lane and lane + 32.
template <typename WT, typename OT>
__global__ void __launch_bounds__(256) k_latent_merge_up_v(const float * __restrict__ part, int splits, const int32_t * __restrict__ off, const WT * __restrict__ wuv,
                                                           LatentParams p, const float * __restrict__ gate, int64_t ldg, OT * __restrict__ out) {
    extern __shared__ float os[];   // [kv_rank], then [64] weights of the splits
    const int h = blockIdx.x, e = blockIdx.y, t = off[e];
    const int R = p.kv_rank, DV = p.vdim, H = p.heads;
    float * w = os + R;
    const float * pe = part + ((int64_t) e * splits * H + h) * (R + 2);
    const int64_t stride = (int64_t) H * (R + 2);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp == 0) {
        const bool ok0 = lane < splits, ok1 = lane + 32 < splits;
        const float m0 = ok0 ? pe[lane * stride + R] : -INFINITY, m1 = ok1 ? pe[(lane + 32) * stride + R] : -INFINITY;
        const float l0 = ok0 ? pe[lane * stride + R + 1] : 0.f, l1 = ok1 ? pe[(lane + 32) * stride + R + 1] : 0.f;
        const float M = wmax(fmaxf(m0, m1));
        const float f0 = m0 == -INFINITY ? 0.f : expf(m0 - M), f1 = m1 == -INFINITY ? 0.f : expf(m1 - M);
        const float L = wsum(l0 * f0 + l1 * f1);
        w[lane] = L > 0.f ? f0 / L : 0.f;
        w[lane + 32] = L > 0.f ? f1 / L : 0.f;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        float a = 0.f;
        int s = 0;
        for (; s + 7 < splits; s += 8) {   // eight loads in flight
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; u++) v[u] = pe[(s + u) * stride + r];
#pragma unroll
            for (int u = 0; u < 8; u++) a = fmaf(w[s + u], v[u], a);
        }
        for (; s < splits; s++) a = fmaf(w[s], pe[s * stride + r], a);
        os[r] = a;
    }
    __syncthreads();
    const int dv_lo = blockIdx.z * ((DV + 1) / 2), dv_hi = min(DV, dv_lo + (DV + 1) / 2);
    for (int dv = dv_lo + warp; dv < dv_hi; dv += (int) (blockDim.x >> 5)) {
        const float acc = wsum(dot_lane8(wuv + ((int64_t) h * DV + dv) * R, os, R, lane));
        if (lane == 0) put(out, (int64_t) t * H * DV + h * DV + dv, acc * sigmoid_f(gate[(int64_t) t * ldg + h * DV + dv]));
    }
}

}  // namespace

static bool latent_ok(const LatentParams & p) {
    return p.heads > 0 && p.dim > 0 && p.rot_dim >= 0 && p.vdim > 0 && p.kv_rank > 0 && p.q_rank > 0 && p.rot_dims >= 0 && p.rot_dims <= p.rot_dim &&
           p.rot_dims % 2 == 0;
}

int launch_latent_prep(const float * proj, const BatchView & b, const LatentParams & p, const float * wq, const float * wkv, const float * freq, float eps,
                       void * cq, int otype, float * cache, int64_t slot_stride, cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    if (!latent_ok(p) || (p.own_kv && (!cache || !wkv))) return (int) cudaErrorInvalidValue;
    return ck_launch([&] {
        if (otype == T_BF16)
            k_latent_prep<__nv_bfloat16><<<b.n_tokens, 256, 0, st>>>(proj, b.slot, b.off, b.pos0, b.entry_of, p, wq, wkv, freq, eps, (__nv_bfloat16 *) cq, cache,
                                                                     slot_stride);
        else k_latent_prep<float><<<b.n_tokens, 256, 0, st>>>(proj, b.slot, b.off, b.pos0, b.entry_of, p, wq, wkv, freq, eps, (float *) cq, cache, slot_stride);
    });
}
int launch_latent_rope_q(float * q, const BatchView & b, const LatentParams & p, const float * freq, cudaStream_t st) {
    if (b.n_tokens <= 0 || p.rot_dims < 2) return 0;
    if (!latent_ok(p)) return (int) cudaErrorInvalidValue;
    return ck_launch([&] { k_latent_rope_q<<<b.n_tokens, 128, 0, st>>>(q, b.off, b.pos0, b.entry_of, p, freq); });
}
int launch_latent_gather(const float * cache, int64_t slot_stride, const BatchView & b, const LatentParams & p, void * lat, int otype, float * kr,
                         cudaStream_t st) {
    if (b.n_tokens <= 0) return 0;
    return ck_launch([&] {
        if (otype == T_BF16)
            k_latent_gather<__nv_bfloat16><<<b.n_tokens, 128, 0, st>>>(cache, slot_stride, b.slot, b.off, b.pos0, b.entry_of, p, (__nv_bfloat16 *) lat, kr);
        else k_latent_gather<float><<<b.n_tokens, 128, 0, st>>>(cache, slot_stride, b.slot, b.off, b.pos0, b.entry_of, p, (float *) lat, kr);
    });
}
int launch_latent_absorb_q(const float * q, const BatchView & b, const void * wuk, int wtype, const LatentParams & p, const float * freq, float * qa,
                           cudaStream_t st) {
    const int n_tokens = b.n_tokens;
    if (n_tokens <= 0) return 0;
    if (!latent_ok(p)) return (int) cudaErrorInvalidValue;
    const dim3 grid((unsigned) p.heads, (unsigned) n_tokens, (unsigned) ((p.kv_rank + 127) / 128));
    const size_t smem = (size_t) p.dim * sizeof(float);
    return ck_launch([&] {
        if (wtype == T_BF16) k_latent_absorb_q<__nv_bfloat16><<<grid, 128, smem, st>>>(q, b.off, b.pos0, b.entry_of, (const __nv_bfloat16 *) wuk, p, freq, qa);
        else k_latent_absorb_q<float><<<grid, 128, smem, st>>>(q, b.off, b.pos0, b.entry_of, (const float *) wuk, p, freq, qa);
    });
}
int launch_latent_up_v(const float * olat, const void * wuv, int wtype, const LatentParams & p, const float * gate, int64_t ldg, void * out, int otype,
                       int n_tokens, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (!latent_ok(p)) return (int) cudaErrorInvalidValue;
    const dim3 grid((unsigned) p.heads, (unsigned) n_tokens);
    const size_t smem = (size_t) p.kv_rank * sizeof(float);
    return ck_launch([&] {
        if (wtype == T_BF16) {
            if (otype == T_BF16) k_latent_up_v<__nv_bfloat16, __nv_bfloat16><<<grid, 256, smem, st>>>(olat, (const __nv_bfloat16 *) wuv, p, gate, ldg, (__nv_bfloat16 *) out);
            else k_latent_up_v<__nv_bfloat16, float><<<grid, 256, smem, st>>>(olat, (const __nv_bfloat16 *) wuv, p, gate, ldg, (float *) out);
        } else {
            if (otype == T_BF16) k_latent_up_v<float, __nv_bfloat16><<<grid, 256, smem, st>>>(olat, (const float *) wuv, p, gate, ldg, (__nv_bfloat16 *) out);
            else k_latent_up_v<float, float><<<grid, 256, smem, st>>>(olat, (const float *) wuv, p, gate, ldg, (float *) out);
        }
    });
}

int launch_latent_decode(const float * qa, const BatchView & b, const LatentParams & p, const float * cache, int64_t slot_stride, int splits, float * part,
                         const void * wuv, int wtype, const float * gate, int64_t ldg, void * out, int otype, cudaStream_t st) {
    if (b.n_entries <= 0) return 0;
    if (!latent_ok(p) || p.kv_rank > 512 || splits < 1 || splits > 64 || !part || b.n_tokens != b.n_entries) return (int) cudaErrorInvalidValue;
    const int RW = latent_row(p);
    const size_t smem = ((size_t) LT_ROWS * (RW | 1) + (size_t) LT_HEADS * RW + LT_HEADS * LT_ROWS + 3 * LT_HEADS) * sizeof(float);
    int rc = raise_smem(k_latent_decode_split, smem);
    if (rc) return rc;
    const dim3 grid((unsigned) splits, (unsigned) b.n_entries, (unsigned) ((p.heads + LT_HEADS - 1) / LT_HEADS));
    rc = ck_launch([&] { k_latent_decode_split<<<grid, 256, smem, st>>>(qa, b.slot, b.off, b.pos0, p, cache, slot_stride, splits, part); });
    if (rc) return rc;
    const dim3 grid2((unsigned) p.heads, (unsigned) b.n_entries, 2);
    const size_t smem2 = ((size_t) p.kv_rank + 64) * sizeof(float);
    return ck_launch([&] {
        if (wtype == T_BF16) {
            if (otype == T_BF16) k_latent_merge_up_v<__nv_bfloat16, __nv_bfloat16><<<grid2, 256, smem2, st>>>(part, splits, b.off, (const __nv_bfloat16 *) wuv, p, gate, ldg, (__nv_bfloat16 *) out);
            else k_latent_merge_up_v<__nv_bfloat16, float><<<grid2, 256, smem2, st>>>(part, splits, b.off, (const __nv_bfloat16 *) wuv, p, gate, ldg, (float *) out);
        } else {
            if (otype == T_BF16) k_latent_merge_up_v<float, __nv_bfloat16><<<grid2, 256, smem2, st>>>(part, splits, b.off, (const float *) wuv, p, gate, ldg, (__nv_bfloat16 *) out);
            else k_latent_merge_up_v<float, float><<<grid2, 256, smem2, st>>>(part, splits, b.off, (const float *) wuv, p, gate, ldg, (float *) out);
        }
    });
}

}  // namespace pb
