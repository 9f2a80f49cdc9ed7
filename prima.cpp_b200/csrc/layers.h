// prima.cpp_b200/csrc/layers.h — launchers of the dense (f32 / bf16 weight) products and of the sequence mixers that the layer-list
// engine (layers.cu) is built from: windowed attention with kept first tokens, soft-capped scores and a per-head output gate; the
// Mamba-2 state-space mixer (short causal convolution, selective scan, gated grouped RMS norm); weight-only layer norm with the
// residual add; tanh-GELU gating.  Every constant of a mechanism is a parameter, nothing is tied to one model.
// All launchers enqueue on `stream` and return a cudaError_t as int (0 = success).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pb {

enum : int { T_BF16 = 30 };   // enum ggml_type value of bfloat16

// ---- ragged batch: the tokens of all entries lie back to back; entry e owns tokens [off[e], off[e+1]) of sequence slot slot[e],
// at positions pos0[e] .. pos0[e] + n - 1 ----
struct BatchView {
    int n_entries = 0;
    int n_tokens = 0;
    int max_n = 0;                 // longest entry
    const int32_t * slot = nullptr;   // device [n_entries]
    const int32_t * off = nullptr;    // device [n_entries + 1]
    const int32_t * pos0 = nullptr;   // device [n_entries]
    const int32_t * entry_of = nullptr;   // device [n_tokens]
};

// ---- dense products ----
// C[t][n] = alpha * sum_k A[t][k] * W[n][k] (+ bias[n]) (+ resid[t][n]);  A and W share `type` (T_F32: true fp32 multiply-add;
// T_BF16: bf16 operands, fp32 accumulation), C / bias / resid are f32.  resid may alias C.  lda / ldw / ldc / ldr in elements.
// The result of a row does not depend on the other rows of the call beyond the choice between the small-batch and the tiled kernel.
int launch_dense(int type, const void * A, int64_t lda, const void * W, int64_t ldw, float * C, int64_t ldc, int T, int N, int K,
                 const float * bias, const float * resid, int64_t ldr, float alpha, cudaStream_t stream);
// 1: the tensor-core kernel takes this shape (bf16, aligned K / strides); informational (bench, tests)
int dense_uses_tensor_cores(int type, int T, int N, int K, int64_t lda, int64_t ldw);

// ---- element-wise / norms; `otype` (T_F32 | T_BF16) is the type of an activation that feeds a dense product ----
int launch_embed(const void * table, int type, int width, const int32_t * tokens, int n_tokens, float * x, float * x_copy, cudaStream_t stream);
int launch_cast(const float * x, void * y, int otype, int64_t n, cudaStream_t stream);
// y[r] = (x[row] - mean) / sqrt(var + eps) * w, row = rows ? rows[r] : r; var = mean of squared deviations
int launch_layernorm(const float * x, const int32_t * rows, const float * w, float eps, void * y, int otype, int n_rows, int width, cudaStream_t stream);
// x[t] += layernorm(m[t]) * w      (the post-norm of a sublayer and the residual sum, fp32)
int launch_layernorm_residual(const float * m, const float * w, float eps, float * x, int n_rows, int width, cudaStream_t stream);
// both at once: x[t] += layernorm(m[t]) * wa, then y[t] = layernorm(x[t]) * wb (the next sublayer's input)
int launch_layernorm_residual_next(const float * m, const float * wa, const float * wb, float eps, float * x, void * y, int otype, int n_rows, int width,
                                   cudaStream_t stream);
// y[t][j] = gelu_tanh(gu[t][j]) * gu[t][ff + j]       gu: [T][2 ff] f32
int launch_gelu_mul(const float * gu, void * y, int otype, int n_tokens, int ff, cudaStream_t stream);
// out[r] = first index of the maximum of logits[r][0..n)
int launch_argmax_rows(const float * logits, int n, int n_rows, int32_t * out, cudaStream_t stream);

// ---- attention with a sliding window and kept first tokens ----
struct AttnParams {
    int heads = 0, kv_heads = 0, dim = 0, vdim = 0;
    float scale = 1.f;
    float softcap = 0.f;      // > 0: score <- softcap * tanh(score / softcap)
    int window = 0;           // position i sees j <= i with i - j < window ...   (<= 0: every earlier position)
    int keep_first = 0;       // ... or j < keep_first
    int cache_rows = 0;       // rows per slot: positions < keep_first at their own row, later ones in a ring over the rest
};
__host__ __device__ inline int attn_qkvg_cols(const AttnParams & a) { return a.heads * a.dim + a.kv_heads * a.dim + a.kv_heads * a.vdim + a.heads; }
// rows of a slot's cache so that every position a later token may still see is present, capped at n_ctx
inline int attn_cache_rows(int window, int keep_first, int n_ctx) {
    if (window <= 0) return n_ctx;
    const int64_t need = (int64_t) keep_first + window;
    return (int) (need < n_ctx ? need : n_ctx);
}
// qkvg: [T][q | k | v | gate] f32 (one fused projection).  Stores the K / V rows that later tokens can still see.
// kcache / vcache: base of the layer run's cache, slot s at + s * slot_stride floats; rows of kv_heads*dim / kv_heads*vdim floats.
int launch_attn_kv_store(const float * qkvg, const BatchView & b, const AttnParams & a, float * kcache, float * vcache, int64_t slot_stride,
                         cudaStream_t stream);
// entries that start at position 0: keys and values are read from the batch itself
int launch_attn_window_prefill(const float * qkvg, const BatchView & b, const AttnParams & a, void * out, int otype, cudaStream_t stream);
// one-token entries: keys and values come from the cache (the token's own row already stored)
int launch_attn_window_decode(const float * qkvg, const BatchView & b, const AttnParams & a, const float * kcache, const float * vcache,
                              int64_t slot_stride, void * out, int otype, cudaStream_t stream);

// ---- Mamba-2 ----
struct Mamba2Params {
    int heads = 0, vdim = 0, state = 0, groups = 0, conv = 0, norm_groups = 0;
};
__host__ __device__ inline int mamba2_inner(const Mamba2Params & p) { return p.heads * p.vdim; }
__host__ __device__ inline int mamba2_conv_channels(const Mamba2Params & p) { return p.heads * p.vdim + 2 * p.groups * p.state; }
__host__ __device__ inline int mamba2_in_cols(const Mamba2Params & p) { return 2 * p.heads * p.vdim + 2 * p.groups * p.state + p.heads; }
// u: [T][z | x | B | C | dt] f32 (the input projection).  xbc[t][c] = silu(bias[c] + sum_d w[c][taps-1-d] * in(t - d)), inputs before
// the entry's first token come from the slot's convolution state [taps-1][channels] (zeros for a new sequence); then the state is
// advanced to the entry's last taps-1 inputs.
int launch_mamba2_conv(const float * u, const BatchView & b, const Mamba2Params & p, const float * w, const float * bias, float * conv_state,
                       int64_t slot_stride, float * xbc, cudaStream_t stream);
// selective scan per (entry, head) over the entry's tokens, state S [state][vdim] f32 per head carried in ssm_state:
//   dt = softplus(dt_raw + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x
int launch_mamba2_scan(const float * u, const float * xbc, const BatchView & b, const Mamba2Params & p, const float * dt_bias, const float * A_log,
                       const float * D, float * ssm_state, int64_t slot_stride, float * y, cudaStream_t stream);
// out[t] = rms_norm_by_group(y[t] * silu(z[t])) * w      (z = first inner columns of u)
int launch_mamba2_gate_norm(const float * y, const float * u, const Mamba2Params & p, const float * w, float eps, void * out, int otype, int n_tokens,
                            cudaStream_t stream);

}  // namespace pb
