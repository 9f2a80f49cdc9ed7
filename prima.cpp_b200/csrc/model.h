// prima.cpp_b200/csrc/model.h — the model object behind the C ABI (include/prima_b200.h), shared by the engines:
// engine.cu (k-quant transformer family: llama, qwen2) and layers.cu (layer-list family: a configuration file lists the layers).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "../../include/prima_b200.h"
#include "launch.h"

namespace pb {

struct LayerList;   // layers.cu

struct Tensor {
    void * data = nullptr;
    int type = -1;
    int64_t N = 0, K = 0;
    size_t bytes = 0;
};

struct Layer {
    float *attn_norm = nullptr, *ffn_norm = nullptr;
    Tensor wq, wk, wv, wo, gate, up, down;
    float *bq = nullptr, *bk = nullptr, *bv = nullptr;
};

struct ActBuf {
    ActQ q{};
    void * base = nullptr;
    int64_t K = 0;
};

}  // namespace pb

struct pb200_model {
    pb200_hparams hp{};
    int device = 0, l0 = 0, l1 = 0;
    bool with_embd = false, with_head = false, finalized = false, use_graph = true;
    cudaStream_t stream = nullptr;
    pb::Tensor tok_embd, output;
    float *output_norm = nullptr, *rope_ff = nullptr;
    std::vector<pb::Layer> layers;   // index il - l0
    __half *kcache = nullptr, *vcache = nullptr;
    float *x_in = nullptr, *x_a = nullptr, *x_b = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *g = nullptr, *u = nullptr,
          *xn = nullptr, *x_out = nullptr, *logits = nullptr;
    pb::ActBuf actE, actQD, actF;
    unsigned int * gbar = nullptr;     // grid-barrier state of the distributed GEMV prologues (2 words, self-resetting)
    int32_t * tokpos_dev = nullptr;    // [0] token, [1] pos
    int32_t * tokpos_host = nullptr;   // pinned
    float * logits_host = nullptr;     // pinned
    pb::RopeParams rp{};
    int n_seq = 1;                      // independent sequences with their own KV cache / token / position (the pipeline keeps one per stage in flight)
    std::vector<cudaGraphExec_t> graph_exec;   // one captured step per sequence slot
    int32_t * sample_dev = nullptr;     // [n_seq] greedy token of the last step (pb200_argmax_seq)
    uint64_t launches_per_step = 0;
    int64_t weight_bytes = 0;
    std::vector<void *> allocs;
    bool profiling = false;
    // prompt-processing (prefill) scratch, grown on demand
    struct Prefill {
        int T = 0;
        float *x0 = nullptr, *x1 = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *g = nullptr, *u = nullptr;
        void * ws = nullptr;
        int32_t *tok = nullptr, *pos = nullptr;
        std::vector<void *> allocs;
    } pf;
    std::vector<cudaEvent_t> prof_ev;
    std::vector<int64_t> prof_bytes;
    size_t prof_n = 0;
    pb::LayerList * ll = nullptr;   // set for architectures of the layer-list family (layers.cu); the k-quant transformer fields above stay unused then

    int alloc(void ** p, size_t bytes) {
        bytes = (bytes + 255) / 256 * 256;
        cudaError_t e = cudaMalloc(p, bytes);
        if (e != cudaSuccess) return (int) e;
        allocs.push_back(*p);
        return 0;
    }
};

