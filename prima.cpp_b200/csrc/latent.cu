// prima.cpp_b200/csrc/latent.cu — the steps of softmax attention over a low-rank latent around the shared attention kernels of mixers.cu
// (declarations and semantics: layers.h).  A sequence slot caches per position one row [normed latent (kv_rank) | rotated key part
// (rot_dim) that all heads share].  Prompts expand keys and values from the latent with dense products and run the prompt attention
// kernel with the shared key tail; a decode step folds the key up-projection into the query (qa = W_uk^T q), runs the decode
// attention kernel with ONE key / value head whose key is the whole cache row and whose value is its latent part, and applies the value
// up-projection to the weighted sum of latents.  Norms, positions, angles and rotations are fp32.
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

// one CTA per (head, token): qa[r] = sum_d W_uk[h * dim + d][r] q[d]; thread r walks a column of the head's block (coalesced over r)
template <typename WT>
__global__ void __launch_bounds__(256) k_latent_absorb_q(const float * __restrict__ q, const WT * __restrict__ wuk, LatentParams p, float * __restrict__ qa) {
    extern __shared__ float qs[];   // [dim]
    const int h = blockIdx.x, t = blockIdx.y;
    const int D = p.dim, Dr = p.rot_dim, R = p.kv_rank;
    const float * qr = q + ((int64_t) t * p.heads + h) * (D + Dr);
    for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = qr[d];
    __syncthreads();
    float * out = qa + ((int64_t) t * p.heads + h) * (R + Dr);
    const WT * w = wuk + (int64_t) h * D * R;
    for (int r = threadIdx.x; r < R; r += blockDim.x) {
        float acc = 0.f;
        for (int d = 0; d < D; d++) acc = fmaf(ld_f(w, (int64_t) d * R + r), qs[d], acc);
        out[r] = acc;
    }
    for (int i = threadIdx.x; i < Dr; i += blockDim.x) out[R + i] = qr[D + i];
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
        const WT * w = wuv + ((int64_t) h * DV + dv) * R;
        float acc = 0.f;
        for (int r = lane; r < R; r += 32) acc = fmaf(ld_f(w, r), os[r], acc);
        acc = wsum(acc);
        if (lane == 0) put(out, (int64_t) t * p.heads * DV + h * DV + dv, acc * sigmoid_f(gate[(int64_t) t * ldg + h * DV + dv]));
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
int launch_latent_absorb_q(const float * q, const void * wuk, int wtype, const LatentParams & p, float * qa, int n_tokens, cudaStream_t st) {
    if (n_tokens <= 0) return 0;
    if (!latent_ok(p)) return (int) cudaErrorInvalidValue;
    const dim3 grid((unsigned) p.heads, (unsigned) n_tokens);
    const size_t smem = (size_t) p.dim * sizeof(float);
    return ck_launch([&] {
        if (wtype == T_BF16) k_latent_absorb_q<__nv_bfloat16><<<grid, 256, smem, st>>>(q, (const __nv_bfloat16 *) wuk, p, qa);
        else k_latent_absorb_q<float><<<grid, 256, smem, st>>>(q, (const float *) wuk, p, qa);
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

}  // namespace pb
