// The loaded model as the decode and the M-token step see it.
#pragma once
#include "decode_kernel.cuh"

#include <vector>

namespace mi {
// device buffers of the M-token step (all [tokens][...], token-major)
struct VerifyBufs {
    int cap = 0;                       // tokens the buffers hold
    float* X = nullptr;                // residual stream [M][E]
    float* Y = nullptr;                // projection output [M][max(qkv_rows, 2FF, E)]
    float* qkv = nullptr;              // [M][qkv_rows (padded)] after bias and RoPE, packed row order
    int8_t* xq = nullptr; __half* xd = nullptr;         // q8_0 of the normed input [M][E]
    float* att = nullptr; int8_t* att_q = nullptr; __half* att_d = nullptr;   // [M][NQ]
    int8_t* act_q = nullptr; __half* act_d = nullptr;   // [M][FF]
    float* logits = nullptr;           // [M][V]
    int* tokens = nullptr; int* out = nullptr;          // [M]
    int* pos0 = nullptr;               // first position of the pass (device resident so that the launch sequence is position-free)
    void* graph[51] = {};              // cudaGraphExec_t of the pass per M, and the scratch addresses each was built with
    const void* graph_part[51] = {}; const void* graph_cnt[51] = {};
    bool warm[51] = {};                // index: M + 17 * attention regime (see verify.cu)
    double* attn_part = nullptr; unsigned* attn_cnt = nullptr;   // [M][NH][max_chunks][HD+2], [M][NH]
    unsigned long long* amax_key = nullptr; unsigned* amax_cnt = nullptr;   // [M] argmax scratch, self-clearing
    float* margins = nullptr;          // [M] greedy logit minus the runner-up
};
}

struct mi_model {
    int device = 0;
    int L = 0, E = 0, FF = 0, NH = 0, NKV = 0, HD = 0, KVD = 0, V = 0, G = 0;
    float eps = 1e-6f, rope_base = 1e6f;
    int max_seq = 0, grid = 0, max_chunks = 0, attn_ctas = 0;
    int tp_rank = 0, tp_world = 1;
    bool tied = false;
    int requantized = 0;                  // matrices that were stored in another block format and re-quantized at load
    int64_t weight_bytes_q4 = 0;          // algorithmic q4_0 bytes streamed per token (18 bytes / 32 weights)
    std::vector<void*> allocs;            // everything cudaMalloc'ed for this model
    std::vector<mi::Job> jobs;
    mi::DecodeParams P{};                     // device pointers filled in; per-call fields set at launch
    int* d_in_tokens = nullptr; int in_capacity = 0;
    int* d_out_tokens = nullptr; int out_capacity = 0;
    // kernel-sequence engine as a replayed CUDA graph (decode.cu, step_graph): one graph per context range, the control
    // block the graph's first and last node read (device memory, refilled per call), the step's token and margin
    void* step_graph[4] = {}; unsigned long long step_graph_wait[4] = {};
    void* d_seq_ctl = nullptr; int* d_step_out = nullptr; float* d_step_margin = nullptr;
    int stop_token = -1;                  // see mi_model_set_stop_token
    int last_count = 0;                   // steps (tokens) the last decode / generate call produced: fewer than asked after a stop
    float* d_margins = nullptr; int last_steps = 0;   // top-1 minus top-2 logit of every step of the last decode call
    size_t smem = 0;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    unsigned long long* prof_buf = nullptr;
    float* best_buf = nullptr;           // {best logit value, greedy token (int bits)}
    int qkv_rows = 0;
    int* tp_flags = nullptr;              // host-driven peer exchange: flags, epoch, gathered argmax candidates (see tp_peer.cu)
    void* tp_peer[8][3] = {};             // per rank: exchange block, (unused), flag block (own entries = local pointers)
    unsigned long long errors_seen = 0;   // value of the context's error count when this model last cleared its counters
    bool tp_peer_on = false;
    std::vector<void*> ipc_opened;        // peer mappings to close
    int* d_pos = nullptr;                 // [2]: device-resident position for position-free launch sequences; the tag epoch
    std::vector<mi_weight> views;         // [4L+1] whole matrices in job order (QKV, O, gate/up, down per layer; lm_head), for the M-token step
    std::vector<mi::LayerPtrs> layer_ptrs;    // host copy of the per-layer norm / bias pointers
    mi::VerifyBufs vb;                    // buffers of the M-token step, allocated on first use
};


namespace mi {

template <typename T>
int dev_alloc(mi_ctx* ctx, mi_model* m, T** p, size_t n, bool zero = true) {
    *p = nullptr;
    if (n == 0) n = 1;
    cudaError_t e = cudaMalloc((void**)p, n * sizeof(T));
    if (e != cudaSuccess) return set_error(ctx, MI_ERR_NOMEM, "model: cudaMalloc(%zu) failed: %s", n * sizeof(T), cudaGetErrorString(e));
    m->allocs.push_back(*p);
    if (zero) {
        // the fill runs on the legacy stream, which the context's own (non-blocking) stream does not wait for:
        // finish it here, before anything enqueued later can write the buffer
        e = cudaMemset(*p, 0, n * sizeof(T));
        if (e == cudaSuccess) e = cudaStreamSynchronize(cudaStreamLegacy);
        if (e != cudaSuccess) return set_error(ctx, MI_ERR_CUDA, "model: cudaMemset failed");
    }
    return MI_OK;
}

}  // namespace mi
