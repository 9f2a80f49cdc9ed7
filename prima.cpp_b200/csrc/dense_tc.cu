// prima.cpp_b200/csrc/dense_tc.cu — bf16 dense product for prompts on the 5th-generation tensor cores:
//   C[t][n] = alpha * sum_k A[t][k] W[n][k] (+ bias[n]) (+ resid[t][n]),   A [T][K], W [N][K] row-major bf16, C f32.
// One CTA computes a tile of 128 weight rows x BN tokens: tcgen05.mma kind::f16 (bf16 operands, M = 128, N = BN, K = 16) with the fp32
// accumulator in TMEM, both operands staged from their row-major global layout into the swizzle-128B K-major shared-memory image by
// 16-byte cp.async pieces (4 producer warps, 4 stages of 64 k), one elected thread issuing the MMAs, tcgen05.commit handing stages back,
// and all 8 warps reading the accumulator out with tcgen05.ld for the epilogue (lane = weight row, so a warp stores 32 consecutive
// floats of one token's row).  K is never split: an output element is one fixed-order sum.  Every wait is bounded (common.cuh).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "launch.h"
#include "layers.h"

extern std::atomic<uint64_t> g_launches;

namespace pb {
namespace {

constexpr int TC_BM = 128, TC_BK = 64, TC_STAGES = 4, TC_LAG = 2, TC_PRODUCERS = 128, TC_THREADS = 256;

struct TcCtl {
    uint64_t full[TC_STAGES], empty[TC_STAGES], acc_ready;
    uint32_t tmem_base;
    int abort;
};

struct TcParams {
    const __nv_bfloat16 * A; int64_t lda;
    const __nv_bfloat16 * W; int64_t ldw;
    float * C; int64_t ldc;
    const float * bias; const float * resid; int64_t ldr;
    float alpha;
    int T, N, K;
    int * abort_flag;
    // grouped: rows [grp_start[g], + grp_count[g]) of A times the g-th matrix of W (grp_w_stride elements apart) into the same rows of C.
    // The counts live on the device: blockIdx.y numbers the token tiles of all groups in a row (group 0's tiles, then group 1's, ...), the
    // grid has room for the most tiles there can be (rows / BN + groups) and a CTA past the last tile leaves at once.
    const int32_t * grp_start; const int32_t * grp_count; int64_t grp_w_stride; int groups;
};

__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {   // K-major, SWIZZLE_128B: rows of 128 B, 8-row groups 1024 B apart
    uint64_t d = (uint64_t) ((saddr >> 4) & 0x3FFF);
    d |= (uint64_t) 1 << 16;
    d |= (uint64_t) (1024 >> 4) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) 2 << 61;
    return d;
}
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t * bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 16 bytes global -> shared; bytes = 0 writes zeros (rows / k beyond the matrix)
__device__ __forceinline__ void cp16(uint32_t dst, const void * src, uint32_t bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}

// rows [r0, r0 + ROWS) x k [k0, k0 + 64) of a row-major bf16 matrix -> swizzle-128B image at `dst` (1024-byte aligned)
template <int ROWS>
__device__ __forceinline__ void stage_rows(uint32_t dst, const __nv_bfloat16 * M, int64_t ld, int r0, int nrows, int k0, int K, int p) {
#pragma unroll
    for (int j = 0; j < ROWS * 8 / TC_PRODUCERS; j++) {
        const int i = p + TC_PRODUCERS * j;
        const int row = i >> 3, c = i & 7;
        const bool ok = r0 + row < nrows && k0 + c * 8 < K;
        const __nv_bfloat16 * src = ok ? M + (int64_t) (r0 + row) * ld + k0 + c * 8 : M;
        cp16(dst + (uint32_t) ((row >> 3) * 1024 + (row & 7) * 128 + ((c ^ (row & 7)) << 4)), src, ok ? 16u : 0u);
    }
}

template <int BN>
__global__ void __launch_bounds__(TC_THREADS, 1) k_dense_tc(const __grid_constant__ TcParams P) {
    const __nv_bfloat16 * Am = P.A, * Wm = P.W;
    float * Cm = P.C;
    int Tn = P.T, tile_y = blockIdx.y;
    if (P.grp_count) {
        int g = 0;
        for (; g < P.groups; g++) {
            const int nt = (P.grp_count[g] + BN - 1) / BN;
            if (tile_y < nt) break;
            tile_y -= nt;
        }
        if (g >= P.groups) return;   // the whole CTA, before any barrier or TMEM allocation
        Tn = P.grp_count[g];
        const int64_t r0 = P.grp_start[g];
        Am += r0 * P.lda; Cm += r0 * P.ldc; Wm += (int64_t) g * P.grp_w_stride;
    }
    extern __shared__ uint8_t smem_raw[];
    uint8_t * smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    constexpr int A_BYTES = TC_BM * 128, B_BYTES = BN * 128, STAGE = A_BYTES + B_BYTES;
    TcCtl * ctl = reinterpret_cast<TcCtl *>(smem + TC_STAGES * STAGE);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TC_BM, t0 = tile_y * BN;
    const int nk = (P.K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TC_STAGES; i++) { mbar_init(&ctl->full[i], TC_PRODUCERS); mbar_init(&ctl->empty[i], 1); }
        mbar_init(&ctl->acc_ready, 1);
        ctl->abort = 0;
        mbar_fence_init();
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctl->tmem_base)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = *(volatile uint32_t *) &ctl->tmem_base;
    volatile int * cta_abort = &ctl->abort;

    if (warp < 4) {
        // ---- producers: stage u of A (weights) and B (activations) into ring slot u % 4 ----
        const int p = threadIdx.x;
        int signalled = 0;
        auto signal = [&](int u) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the copies above are read by the tensor core's async proxy
            mbar_arrive(&ctl->full[u % TC_STAGES]);
        };
        for (int u = 0; u < nk; u++) {
            const int s = u % TC_STAGES;
            if (u >= TC_STAGES) mbar_wait(&ctl->empty[s], (uint32_t) ((u / TC_STAGES - 1) & 1), cta_abort, P.abort_flag);
            const uint32_t base = smem_u32(smem + s * STAGE);
            stage_rows<TC_BM>(base, Wm, P.ldw, n0, P.N, u * TC_BK, P.K, p);
            stage_rows<BN>(base + A_BYTES, Am, P.lda, t0, Tn, u * TC_BK, P.K, p);
            asm volatile("cp.async.commit_group;" ::: "memory");
            if (u - signalled >= TC_LAG) {
                asm volatile("cp.async.wait_group 2;" ::: "memory");
                signal(signalled++);
            }
        }
        while (signalled < nk) {
            if (nk - 1 - signalled >= 1) asm volatile("cp.async.wait_group 1;" ::: "memory");
            else asm volatile("cp.async.wait_group 0;" ::: "memory");
            signal(signalled++);
        }
    } else if (warp == 4) {
        // ---- one thread issues the MMAs ----
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (BN >> 3) << 17) | ((uint32_t) (TC_BM >> 4) << 24);
            for (int u = 0; u < nk; u++) {
                const int s = u % TC_STAGES;
                mbar_wait(&ctl->full[s], (uint32_t) ((u / TC_STAGES) & 1), cta_abort, P.abort_flag);
                fence_after();
                const uint64_t da = desc_sw128(smem_u32(smem + s * STAGE)), db = desc_sw128(smem_u32(smem + s * STAGE + A_BYTES));
#pragma unroll
                for (int k = 0; k < TC_BK / 16; k++) mma_bf16(tmem, da + 2 * k, db + 2 * k, idesc, (uint32_t) ((u | k) != 0));
                mma_commit(&ctl->empty[s]);        // arrives once the MMAs above have read the stage
            }
            mma_commit(&ctl->acc_ready);
        }
        __syncwarp();
    }
    // ---- epilogue: every warp reads its TMEM quadrant (lanes = weight rows), warps 0-3 the first half of the tokens, 4-7 the second ----
    mbar_wait(&ctl->acc_ready, 0u, cta_abort, P.abort_flag);
    fence_after();
    {
        const int quad = warp & 3, half = warp >> 2;
        const int n = n0 + quad * 32 + lane;
        const float bias = (P.bias && n < P.N) ? P.bias[n] : 0.f;
        for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 16) {
            if (t0 + c0 >= Tn) break;                                   // uniform over the warp
            uint32_t v[16];
            const uint32_t taddr = tmem + ((uint32_t) (quad * 32) << 16) + (uint32_t) c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
                  "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                : "r"(taddr)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (n < P.N && !*cta_abort) {
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int t = t0 + c0 + i;
                    if (t < Tn) {
                        float y = P.alpha * __uint_as_float(v[i]) + bias;
                        if (P.resid) y += P.resid[(int64_t) t * P.ldr + n];
                        Cm[(int64_t) t * P.ldc + n] = y;
                    }
                }
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == 4) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BN) : "memory");
    }
}

template <int BN> constexpr size_t tc_smem() { return 1024 + (size_t) TC_STAGES * (TC_BM * 128 + BN * 128) + sizeof(TcCtl) + 64; }

template <int BN>
int launch_tc(const TcParams & P, cudaStream_t st) {
    static FuncAttrCache cache;
    cudaError_t e = ensure_dyn_smem(cache, (const void *) k_dense_tc<BN>, tc_smem<BN>(), BN == 256);
    if (e != cudaSuccess) return (int) e;
    const dim3 grid((unsigned) ((P.N + TC_BM - 1) / TC_BM), (unsigned) ((P.T + BN - 1) / BN + (P.grp_count ? P.groups : 0)));
    g_launches++;
    k_dense_tc<BN><<<grid, TC_THREADS, tc_smem<BN>(), st>>>(P);
    return (int) cudaGetLastError();
}

}  // namespace

bool dense_tc_ok(int T, int N, int K, int64_t lda, int64_t ldw, const void * A, const void * W) {
    static const bool off = getenv("PB200_NO_DENSE_TC") != nullptr;   // A/B: the CUDA-core tile kernel instead
    return !off && T > 0 && N > 0 && K >= 8 && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 && ((uintptr_t) A & 15) == 0 && ((uintptr_t) W & 15) == 0;
}

int launch_dense_tc(const __nv_bfloat16 * A, int64_t lda, const __nv_bfloat16 * W, int64_t ldw, float * C, int64_t ldc, int T, int N, int K, const float * bias,
                    const float * resid, int64_t ldr, float alpha, cudaStream_t st) {
    TcParams P{A, lda, W, ldw, C, ldc, bias, resid, ldr, alpha, T, N, K, abort_flag(), nullptr, nullptr, 0, 0};
    return T <= 64 ? launch_tc<64>(P, st) : T <= 128 ? launch_tc<128>(P, st) : launch_tc<256>(P, st);
}

int launch_dense_tc_grouped(const __nv_bfloat16 * A, int64_t lda, const __nv_bfloat16 * W, int64_t ldw, int64_t w_stride, float * C, int64_t ldc,
                            const int32_t * start, const int32_t * count, int groups, int max_rows, int N, int K, cudaStream_t st) {
    if (groups <= 0 || max_rows <= 0) return 0;
    // T bounds the grid only (all groups together hold max_rows rows); the kernel reads each group's own count
    TcParams P{A, lda, W, ldw, C, ldc, nullptr, nullptr, 0, 1.f, max_rows, N, K, abort_flag(), start, count, w_stride, groups};
    const int avg = (max_rows + groups - 1) / groups;   // the token tile follows the expected rows of a group
    return avg <= 64 ? launch_tc<64>(P, st) : avg <= 128 ? launch_tc<128>(P, st) : launch_tc<256>(P, st);
}

}  // namespace pb
