// Decode runtime for the hybrid configuration: embedding -> layers (Mamba-2 or MoE, in the order
// they were added) -> final RMSNorm -> tied bf16 LM head with greedy argmax.  One decode step of
// all sequences is captured into a CUDA graph; chained greedy decode replays it with the argmax of
// a step feeding the next on the device.  No counterpart in the reference.
#include <string.h>
#include <vector>

#include "internal.cuh"
#include "../../include/lspk_hybrid.h"

namespace lspk {

struct HybridLayer {
    Mamba* mamba = nullptr;
    Moe* moe = nullptr;
};

struct Hybrid {
    int H = 0, V = 0;
    float eps = 1e-5f;
    std::vector<HybridLayer> layers;
    uint16_t* emb = nullptr;
    uint16_t* final_norm = nullptr;
    size_t bytes = 0;
};

struct HybridState {
    Hybrid* m = nullptr;
    int batch = 1, max_steps = 0;
    std::vector<float*> layer_state;      // per Mamba layer: [batch][state_floats]
    std::vector<size_t> layer_state_bytes;
    int* ctl = nullptr;                   // pos[batch], token[batch], step
    unsigned long long* best = nullptr;
    int* tokens_out = nullptr;
    float *x = nullptr, *logits = nullptr;
    int* h_int = nullptr;
    float* h_logits = nullptr;
    cudaGraphExec_t graph = nullptr;
    unsigned graph_gen = 0;           // scratch_generation() at capture
    int graph_nodes = 0;
    size_t bytes = 0;
};

static int enqueue_hybrid_step(HybridState* s) {
    Hybrid* m = s->m;
    const int B = s->batch;
    if (int rc = launch_embed(s->ctl + B, B, 0, m->emb, nullptr, s->x, m->H, m->V)) return rc;
    size_t li_m = 0;
    for (auto& L : m->layers) {
        if (L.mamba) {
            if (int rc = mamba_step(L.mamba, s->x, s->layer_state[li_m], s->ctl, B)) return rc;
            ++li_m;
        } else {
            if (int rc = moe_forward(L.moe, s->x, B, nullptr, nullptr, nullptr, nullptr, nullptr)) return rc;
        }
    }
    if (B == 1) {
        if (int rc = lm_head_launch(0, m->emb, nullptr, s->x, s->logits, 1, m->V, m->H, m->final_norm, 1, m->eps, s->best))
            return rc;
    } else {
        // several sequences: the LM head returns each row's greedy choice itself (logits only where its
        // tensor-core form does not apply and a row argmax has to read them)
        if (int rc = lm_head_launch(0, m->emb, nullptr, s->x, (m->H % 32) ? s->logits : nullptr, B, m->V, m->H,
                                    m->final_norm, 1, m->eps, s->best))
            return rc;
    }
    return launch_finish_step(s->ctl, s->best, s->tokens_out, B, s->max_steps);
}

static int hybrid_build_graph(HybridState* s) {
    if (s->graph && s->graph_gen == scratch_generation()) return LSPK_OK;
    // A graph whose scratch addresses went stale (another state made a layer's buffers grow) is captured
    // again; every buffer is already large enough for this state then, and the kernels' attributes are set.
    const bool recapture = s->graph != nullptr;
    if (recapture) {
        LSPK_CUDA(cudaStreamSynchronize(stream()));
        cudaGraphExecDestroy(s->graph);
        s->graph = nullptr;
    }
    // scratch of every layer is sized before capture (allocation is not allowed while capturing)
    for (auto& L : s->m->layers) {
        if (L.mamba) { if (int rc = mamba_reserve(L.mamba, s->batch)) return rc; }
        else { if (int rc = moe_reserve(L.moe, s->batch)) return rc; }
    }
    if (!recapture) {
        // A plain run first: sets kernel attributes, sizes the shared scratch and surfaces launch errors.  It
        // advances the recurrent state, so it is only done on a freshly reset state, which is reset again afterwards.
        if (int rc = enqueue_hybrid_step(s)) return rc;
        LSPK_CUDA(cudaStreamSynchronize(stream()));
        if (int rc = lspk_hybrid_state_reset(reinterpret_cast<lspk_hybrid_state_t>(s))) return rc;
    }
    cudaGraph_t g = nullptr;
    LSPK_CUDA(cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_hybrid_step(s);
    cudaError_t e = cudaStreamEndCapture(stream(), &g);
    if (rc) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "hybrid graph capture failed: %s", cudaGetErrorString(e));
    size_t n = 0;
    cudaGraphGetNodes(g, nullptr, &n);
    s->graph_nodes = (int)n;
    e = cudaGraphInstantiate(&s->graph, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "hybrid graph instantiate failed: %s", cudaGetErrorString(e));
    s->graph_gen = scratch_generation();
    return LSPK_OK;
}

}  // namespace lspk

using namespace lspk;

extern "C" {

lspk_hybrid_t lspk_hybrid_create(int hidden, int vocab, float eps) {
    if (ensure_init()) return nullptr;
    if (hidden < 8 || (hidden & 7) || vocab < 1) {
        fail(LSPK_ERR_ARG, "lspk_hybrid_create: hidden must be a positive multiple of 8, vocab positive");
        return nullptr;
    }
    Hybrid* h = new Hybrid();
    h->H = hidden;
    h->V = vocab;
    h->eps = eps;
    return reinterpret_cast<lspk_hybrid_t>(h);
}

int lspk_hybrid_add_mamba(lspk_hybrid_t hh, lspk_mamba_t layer) {
    LSPK_REQUIRE(hh && layer, "lspk_hybrid_add_mamba: null argument");
    HybridLayer L;
    L.mamba = reinterpret_cast<Mamba*>(layer);
    reinterpret_cast<Hybrid*>(hh)->layers.push_back(L);
    return LSPK_OK;
}

int lspk_hybrid_add_moe(lspk_hybrid_t hh, lspk_moe_t layer) {
    LSPK_REQUIRE(hh && layer, "lspk_hybrid_add_moe: null argument");
    HybridLayer L;
    L.moe = reinterpret_cast<Moe*>(layer);
    reinterpret_cast<Hybrid*>(hh)->layers.push_back(L);
    return LSPK_OK;
}

int lspk_hybrid_set_embedding(lspk_hybrid_t hh, const uint16_t* emb_bf16_host, const uint16_t* final_norm_gamma) {
    LSPK_REQUIRE(hh && emb_bf16_host && final_norm_gamma, "lspk_hybrid_set_embedding: null argument");
    Hybrid* h = reinterpret_cast<Hybrid*>(hh);
    const size_t eb = (size_t)h->V * h->H * 2;
    if (h->emb) cudaFree(h->emb);
    if (h->final_norm) cudaFree(h->final_norm);
    LSPK_CUDA(cudaMalloc((void**)&h->emb, eb));
    LSPK_CUDA(cudaMemcpy(h->emb, emb_bf16_host, eb, cudaMemcpyHostToDevice));
    LSPK_CUDA(cudaMalloc((void**)&h->final_norm, (size_t)h->H * 2));
    LSPK_CUDA(cudaMemcpy(h->final_norm, final_norm_gamma, (size_t)h->H * 2, cudaMemcpyHostToDevice));
    h->bytes += eb + (size_t)h->H * 2;
    return LSPK_OK;
}

int lspk_hybrid_free(lspk_hybrid_t hh) {
    if (!hh) return LSPK_OK;
    Hybrid* h = reinterpret_cast<Hybrid*>(hh);
    cudaStreamSynchronize(stream());
    for (auto& L : h->layers) {
        if (L.mamba) lspk_mamba_free(reinterpret_cast<lspk_mamba_t>(L.mamba));
        if (L.moe) lspk_moe_free(reinterpret_cast<lspk_moe_t>(L.moe));
    }
    cudaFree(h->emb);
    cudaFree(h->final_norm);
    delete h;
    return LSPK_OK;
}

size_t lspk_hybrid_device_bytes(lspk_hybrid_t hh) {
    if (!hh) return 0;
    Hybrid* h = reinterpret_cast<Hybrid*>(hh);
    size_t b = h->bytes;
    for (auto& L : h->layers)
        b += L.mamba ? lspk_mamba_device_bytes(reinterpret_cast<lspk_mamba_t>(L.mamba))
                     : lspk_moe_device_bytes(reinterpret_cast<lspk_moe_t>(L.moe));
    return b;
}

lspk_hybrid_state_t lspk_hybrid_state_create(lspk_hybrid_t hh, int batch, int max_steps) {
    Hybrid* h = reinterpret_cast<Hybrid*>(hh);
    if (!h || !h->emb || h->layers.empty() || batch < 1 || batch > 1024 || max_steps < 1) {
        fail(LSPK_ERR_ARG, "lspk_hybrid_state_create: bad arguments (embedding set? layers added?)");
        return nullptr;
    }
    HybridState* s = new HybridState();
    s->m = h;
    s->batch = batch;
    s->max_steps = max_steps;
    cudaError_t e = cudaSuccess;
    auto alloc = [&](void** p, size_t bytes) {
        if (e != cudaSuccess) return;
        e = cudaMalloc(p, bytes);
        s->bytes += bytes;
    };
    for (auto& L : h->layers) {
        if (!L.mamba) continue;
        float* st = nullptr;
        const size_t bytes = (size_t)batch * mamba_state_floats(L.mamba) * 4;
        alloc((void**)&st, bytes);
        s->layer_state.push_back(st);
        s->layer_state_bytes.push_back(bytes);
    }
    const int lrows = batch > 8 ? batch : 8;
    alloc((void**)&s->ctl, (size_t)(2 * batch + 1) * 4);
    alloc((void**)&s->best, (size_t)batch * 8);
    alloc((void**)&s->tokens_out, (size_t)max_steps * batch * 4);
    alloc((void**)&s->x, (size_t)batch * h->H * 4);
    alloc((void**)&s->logits, (size_t)lrows * h->V * 4);
    if (e == cudaSuccess) e = cudaMallocHost((void**)&s->h_int, (size_t)(max_steps * batch + 2 * batch + 16) * 4);
    if (e == cudaSuccess) e = cudaMallocHost((void**)&s->h_logits, (size_t)batch * h->V * 4);
    if (e != cudaSuccess || lspk_hybrid_state_reset(reinterpret_cast<lspk_hybrid_state_t>(s)) != LSPK_OK) {
        fail(LSPK_ERR_CUDA, "lspk_hybrid_state_create: %s", cudaGetErrorString(e));
        lspk_hybrid_state_free(reinterpret_cast<lspk_hybrid_state_t>(s));
        return nullptr;
    }
    return reinterpret_cast<lspk_hybrid_state_t>(s);
}

int lspk_hybrid_state_reset(lspk_hybrid_state_t sh) {
    HybridState* s = reinterpret_cast<HybridState*>(sh);
    LSPK_REQUIRE(s, "lspk_hybrid_state_reset: null state");
    for (size_t i = 0; i < s->layer_state.size(); ++i)
        LSPK_CUDA(cudaMemsetAsync(s->layer_state[i], 0, s->layer_state_bytes[i], stream()));
    LSPK_CUDA(cudaMemsetAsync(s->ctl, 0, (size_t)(2 * s->batch + 1) * 4, stream()));
    LSPK_CUDA(cudaMemsetAsync(s->best, 0, (size_t)s->batch * 8, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    return LSPK_OK;
}

int lspk_hybrid_state_free(lspk_hybrid_state_t sh) {
    if (!sh) return LSPK_OK;
    HybridState* s = reinterpret_cast<HybridState*>(sh);
    cudaStreamSynchronize(stream());
    if (s->graph) cudaGraphExecDestroy(s->graph);
    for (float* p : s->layer_state) cudaFree(p);
    void* dev[] = {s->ctl, s->best, s->tokens_out, s->x, s->logits};
    for (void* p : dev) cudaFree(p);
    if (s->h_int) cudaFreeHost(s->h_int);
    if (s->h_logits) cudaFreeHost(s->h_logits);
    delete s;
    return LSPK_OK;
}

int lspk_hybrid_step(lspk_hybrid_state_t sh, const int* tokens_host, float* logits_host, int* next_tokens_host) {
    HybridState* s = reinterpret_cast<HybridState*>(sh);
    LSPK_REQUIRE(s && tokens_host, "lspk_hybrid_step: null argument");
    const int B = s->batch, V = s->m->V;
    if (int rc = hybrid_build_graph(s)) return rc;
    memcpy(s->h_int, tokens_host, (size_t)B * 4);
    LSPK_CUDA(cudaMemcpyAsync(s->ctl + B, s->h_int, (size_t)B * 4, cudaMemcpyHostToDevice, stream()));
    LSPK_CUDA(cudaGraphLaunch(s->graph, stream()));
    if (logits_host)
        LSPK_CUDA(cudaMemcpyAsync(s->h_logits, s->logits, (size_t)B * V * 4, cudaMemcpyDeviceToHost, stream()));
    if (next_tokens_host)
        LSPK_CUDA(cudaMemcpyAsync(s->h_int + B, s->ctl + B, (size_t)B * 4, cudaMemcpyDeviceToHost, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    if (logits_host) memcpy(logits_host, s->h_logits, (size_t)B * V * 4);
    if (next_tokens_host) memcpy(next_tokens_host, s->h_int + B, (size_t)B * 4);
    return LSPK_OK;
}

int lspk_hybrid_decode_greedy(lspk_hybrid_state_t sh, const int* first_tokens_host, int n_steps, int* tokens_out_host) {
    HybridState* s = reinterpret_cast<HybridState*>(sh);
    LSPK_REQUIRE(s && first_tokens_host && tokens_out_host && n_steps >= 1 && n_steps <= s->max_steps,
                 "lspk_hybrid_decode_greedy: bad arguments (n_steps must not exceed max_steps)");
    const int B = s->batch;
    if (int rc = hybrid_build_graph(s)) return rc;
    memcpy(s->h_int, first_tokens_host, (size_t)B * 4);
    s->h_int[B] = 0;
    LSPK_CUDA(cudaMemcpyAsync(s->ctl + B, s->h_int, (size_t)(B + 1) * 4, cudaMemcpyHostToDevice, stream()));
    for (int i = 0; i < n_steps; ++i) LSPK_CUDA(cudaGraphLaunch(s->graph, stream()));
    LSPK_CUDA(cudaMemcpyAsync(s->h_int, s->tokens_out, (size_t)n_steps * B * 4, cudaMemcpyDeviceToHost, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    memcpy(tokens_out_host, s->h_int, (size_t)n_steps * B * 4);
    return LSPK_OK;
}

int lspk_hybrid_prefill(lspk_hybrid_state_t sh, const int* tokens_host, int T, int* next_tokens_host) {
    HybridState* s = reinterpret_cast<HybridState*>(sh);
    LSPK_REQUIRE(s && tokens_host && T >= 1, "lspk_hybrid_prefill: bad arguments");
    const int B = s->batch;
    if (int rc = hybrid_build_graph(s)) return rc;
    // one graph replay per prompt position; the token ids of all positions are staged once
    std::vector<int> all(tokens_host, tokens_host + (size_t)T * B);
    int* d_tokens = nullptr;
    LSPK_CUDA(cudaMalloc((void**)&d_tokens, (size_t)T * B * 4));
    cudaError_t e = cudaMemcpyAsync(d_tokens, all.data(), (size_t)T * B * 4, cudaMemcpyHostToDevice, stream());
    for (int t = 0; t < T && e == cudaSuccess; ++t) {
        e = cudaMemcpyAsync(s->ctl + B, d_tokens + (size_t)t * B, (size_t)B * 4, cudaMemcpyDeviceToDevice, stream());
        if (e == cudaSuccess) e = cudaGraphLaunch(s->graph, stream());
    }
    if (e == cudaSuccess && next_tokens_host)
        e = cudaMemcpyAsync(s->h_int, s->ctl + B, (size_t)B * 4, cudaMemcpyDeviceToHost, stream());
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream());
    cudaFree(d_tokens);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "lspk_hybrid_prefill: %s", cudaGetErrorString(e));
    if (next_tokens_host) memcpy(next_tokens_host, s->h_int, (size_t)B * 4);
    return LSPK_OK;
}

int lspk_hybrid_step_kernel_count(lspk_hybrid_state_t sh) {
    HybridState* s = reinterpret_cast<HybridState*>(sh);
    return s ? s->graph_nodes : 0;
}

}  // extern "C"
