// Model and inference-state containers of the device-resident forward pass, shared between runtime.cu (which
// owns them) and the measurement harnesses in bench_probes.cu.
#pragma once
#include <vector>

#include "internal.cuh"
#include "../../include/lspk_runtime.h"

namespace lspk {

struct DevNorm {
    void* g = nullptr;
    int is_bf16 = 0;
    int K = 0;
};

struct DevLayer {
    lspk_weight_t proj[7] = {};
    DevNorm norm[4];
};

struct DevTable {
    int kind = -1;
    void* data = nullptr;
    float* scale = nullptr;
};

struct Model {
    lspk_model_config cfg;
    std::vector<DevLayer> layers;
    DevNorm final_norm;
    DevTable emb, head;
    bool finalized = false;
    size_t bytes = 0;
    int D() const { return cfg.hidden_size / cfg.num_heads; }
    int kv_dim() const { return cfg.num_kv_heads * D(); }
};

struct State {
    Model* m = nullptr;
    int t_max = 0, batch = 1, kv_fp16 = 1;
    int cap_rows = 0;                 // rows the scratch buffers hold
    void *cache_k = nullptr, *cache_v = nullptr;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    float* rope_cur = nullptr;        // [batch][D]: cos | sin rows of each sequence's current position (decode step)
    bool rope_cur_valid = false;      // true while the kernels of a decode step are being enqueued
    int* ctl = nullptr;               // device: pos[batch], token[batch], step
    unsigned long long* best = nullptr;   // device: argmax keys [batch]
    int* tokens_out = nullptr;        // device: [t_max * batch]
    float *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *attn = nullptr, *inter = nullptr, *inter2 = nullptr;
    float *logits = nullptr;          // [max(batch, 8), V]
    int logits_rows = 0;
    int8_t *xq_h = nullptr, *xq_i = nullptr;
    float* xs = nullptr;
    int* tok_rows = nullptr;          // device token ids for a prefill chunk
    int* h_int = nullptr;             // pinned staging for ints
    float* h_logits = nullptr;        // pinned staging for logits
    std::vector<int> host_pos;
    // Host-fed single step without copy operations (one sequence, no logits): the step's first kernel reads the token
    // from mapped pinned memory, its last kernel stores (step number << 32 | next token) there with one 8-byte store
    // and the host polls that word instead of waiting for the stream.
    int* io_tok = nullptr;                 // mapped pinned: token in (host pointer)
    unsigned long long* io_pkt = nullptr;  // mapped pinned: packet out (host pointer)
    int* io_tok_dev = nullptr;             // the same two words as the device sees them
    unsigned long long* io_pkt_dev = nullptr;
    unsigned* io_seq_dev = nullptr;        // device: steps of this kind finished so far
    unsigned io_seq = 0;                   // host: the same count
    cudaGraphExec_t graph[3] = {nullptr, nullptr, nullptr};   // [0] no logits store, [1] with logits, [2] host-fed step
    unsigned graph_gen[3] = {0, 0, 0};   // scratch_generation() at capture: a later move of library scratch voids the graph
    int graph_nodes = 0;
    size_t bytes = 0;
    size_t kv_elem() const { return kv_fp16 ? 2 : 4; }
    size_t layer_stride() const { return (size_t)t_max * m->kv_dim(); }            // elements
    size_t seq_stride() const { return layer_stride() * m->cfg.num_layers; }       // elements
};

// runtime.cu: one transformer layer for `rows` rows held in the state's scratch buffers (see its definition).
int run_layer(State* s, int li, int rows, bool per_row_seq, int seq, bool skip_attention = false);
size_t table_bytes(int kind, int V, int H);

}  // namespace lspk
