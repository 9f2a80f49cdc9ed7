// prima.cpp_b200/csrc/mixers.cuh — device helpers shared by the kernels of the layer-list engine (mixers.cu, linattn.cu, latent.cu,
// moe.cu): typed stores, warp / CTA reductions, activations, and the launch bookkeeping of their host-side launchers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

extern std::atomic<uint64_t> g_launches;

namespace pb {
namespace {

__device__ __forceinline__ void put(float * p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void put(__nv_bfloat16 * p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// sum over the CTA (blockDim.x a multiple of 32, <= 1024); every thread gets the result; `red` is 33 floats of shared memory
__device__ __forceinline__ float block_sum(float v, float * red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = wsum(v);
    __syncthreads();   // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float s = lane < nw ? red[lane] : 0.f;
        s = wsum(s);
        if (lane == 0) red[32] = s;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }
__device__ __forceinline__ float sigmoid_f(float v) { return 1.f / (1.f + expf(-v)); }

__device__ __forceinline__ float ld_f(const float * p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ld_f(const __nv_bfloat16 * p, int64_t i) { return __bfloat162float(p[i]); }

// a lane's share of sum_i a[i] * b[i], i = lane, lane + 32, ...; a in global memory (eight loads in flight), b in shared memory
template <typename T>
__device__ __forceinline__ float dot_lane8(const T * __restrict__ a, const float * b, int n, int lane) {
    float acc = 0.f;
    int i = lane;
    for (; i + 7 * 32 < n; i += 8 * 32) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = ld_f(a, i + 32 * u);
#pragma unroll
        for (int u = 0; u < 8; u++) acc = fmaf(v[u], b[i + 32 * u], acc);
    }
    for (; i < n; i += 32) acc = fmaf(ld_f(a, i), b[i], acc);
    return acc;
}

template <typename F> int ck_launch(F && f) {
    g_launches++;
    f();
    return (int) cudaGetLastError();
}
template <typename K> int raise_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return 0;
    return (int) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) bytes);
}

}  // namespace
}  // namespace pb
