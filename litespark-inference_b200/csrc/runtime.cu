// Device-resident forward pass: model and inference-state containers, the decode step (one
// CUDA graph of fused kernels), chunked prefill and chained greedy decode.
//
// Restates the host loop of litespark_inference/torchless/runtime.py (forward_one :171-282,
// _forward_prefill_hidden :285-436, generate :669-697, falcon_forward_one :735-817) as a
// sequence of kernel launches; the per-op arithmetic lives in linear.cu / rows.cu /
// attention.cu / lm_head.cu.
#include <string.h>
#include <vector>

#include "runtime_internal.cuh"

namespace lspk {

// ---- small kernels of the forward pass ---------------------------------------------------

// x[r, :] = embedding row of token[r] as fp32 (bf16 / int8*scale / int4*scale), the lookup of
// runtime.py:151-168.
// When rope_cur is given, also copies the rope factors of row r's position into rope_cur[r] (cos | sin),
// so that the attention kernels of the step find them at a fixed address instead of behind the position.
__global__ void embed_kernel(const int* __restrict__ tokens, int kind, const void* __restrict__ emb,
                             const float* __restrict__ scale, float* __restrict__ x, int H, int V,
                             const int* __restrict__ pos, const float* __restrict__ rope_cos,
                             const float* __restrict__ rope_sin, float* __restrict__ rope_cur, int half,
                             int tokens_in_host_memory) {
    grid_dependency_launch();
    grid_dependency_wait();
    const int r = blockIdx.x;
    if (rope_cur) {
        const int ps = pos[r];
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            rope_cur[(size_t)r * 2 * half + i] = rope_cos[(size_t)ps * half + i];
            rope_cur[(size_t)r * 2 * half + half + i] = rope_sin[(size_t)ps * half + i];
        }
    }
    int tok;
    if (tokens_in_host_memory) asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(tok) : "l"(tokens + r) : "memory");
    else tok = tokens[r];
    tok = min(max(tok, 0), V - 1);
    float* dst = x + (size_t)r * H;
    if (kind == 0) {
        const uint16_t* row = reinterpret_cast<const uint16_t*>(emb) + (size_t)tok * H;
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = bf16_bits_to_f32(row[i]);
    } else if (kind == 1) {
        const int8_t* row = reinterpret_cast<const int8_t*>(emb) + (size_t)tok * H;
        const float s = scale[tok];
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __fmul_rn((float)row[i], s);
    } else {
        const uint8_t* row = reinterpret_cast<const uint8_t*>(emb) + (size_t)tok * (H / 2);
        const float s = scale[tok];
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const uint8_t b = row[i >> 1];
            const int nib = (i & 1) ? ((int8_t)b >> 4) : ((int8_t)(b << 4) >> 4);
            dst[i] = __fmul_rn((float)nib, s);
        }
    }
}

// First-maximum argmax of each logits row (np.argmax semantics), used when the LM head's fused
// argmax does not apply (more than one row).
__global__ void argmax_rows_kernel(const float* __restrict__ logits, int V, unsigned long long* __restrict__ best) {
    grid_dependency_launch();
    grid_dependency_wait();
    __shared__ unsigned long long sb[32];
    const float* row = logits + (size_t)blockIdx.x * V;
    unsigned long long b = 0ull;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        uint32_t u = __float_as_uint(row[i]);
        u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
        const unsigned long long key = ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
        b = key > b ? key : b;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
        b = other > b ? other : b;
    }
    if ((threadIdx.x & 31) == 0) sb[threadIdx.x >> 5] = b;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) b = sb[w] > b ? sb[w] : b;
        best[blockIdx.x] = b;
    }
}

// End of a decode step: turn the argmax keys into token ids, make them the next step's input,
// append them to the output list, advance every position, clear the keys.
// host_pkt (optional, one sequence): mapped host word that receives (count of host-fed steps << 32 | token) in one
// 8-byte store, so that a host that sees the count has the token.
__global__ void finish_step_kernel(int* __restrict__ ctl, unsigned long long* __restrict__ best,
                                   int* __restrict__ tokens_out, int batch, int out_cap,
                                   unsigned long long* host_pkt, unsigned* host_seq) {
    grid_dependency_launch();
    grid_dependency_wait();
    const int b = threadIdx.x;
    if (b < batch) {
        const int tok = (int)(0xffffffffu - (uint32_t)(best[b] & 0xffffffffull));
        best[b] = 0ull;
        const int step = ctl[2 * batch];
        ctl[batch + b] = tok;
        if (step < out_cap) tokens_out[(size_t)step * batch + b] = tok;
        ctl[b] += 1;
        if (host_pkt && b == 0) {
            const unsigned seq = *host_seq + 1u;
            *host_seq = seq;
            const unsigned long long pkt = ((unsigned long long)seq << 32) | (unsigned long long)(uint32_t)tok;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(host_pkt), "l"(pkt) : "memory");
        }
    }
    __syncthreads();
    if (b == 0) ctl[2 * batch] += 1;
}

__global__ void advance_pos_kernel(int* __restrict__ ctl, int seq, int by) {
    grid_dependency_launch();
    grid_dependency_wait();
    if (threadIdx.x == 0) ctl[seq] += by;
}

// ---- launch wrappers shared with the hybrid runtime (kernels must be launched from this file) ----
int launch_embed(const int* tokens, int rows, int kind, const void* emb, const float* scale, float* x, int H, int V) {
    LSPK_CUDA(launch(embed_kernel, dim3(rows), dim3(256), 0, true, tokens, kind, emb, scale, x, H, V, (const int*)nullptr,
                     (const float*)nullptr, (const float*)nullptr, (float*)nullptr, 0, 0));
    return LSPK_OK;
}
int launch_argmax_rows(const float* logits, int rows, int V, unsigned long long* best) {
    LSPK_CUDA(launch(argmax_rows_kernel, dim3(rows), dim3(1024), 0, true, logits, V, best));
    return LSPK_OK;
}
int launch_finish_step(int* ctl, unsigned long long* best, int* tokens_out, int batch, int out_cap) {
    LSPK_CUDA(launch(finish_step_kernel, dim3(1), dim3(((batch + 31) / 32) * 32), 0, true, ctl, best, tokens_out,
                     batch, out_cap, (unsigned long long*)nullptr, (unsigned*)nullptr));
    return LSPK_OK;
}

// ---- helpers -------------------------------------------------------------------------------

static int dev_alloc(void** p, size_t bytes, size_t* tally) {
    LSPK_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    if (tally) *tally += bytes;
    return LSPK_OK;
}

size_t table_bytes(int kind, int V, int H) {
    return kind == 0 ? (size_t)V * H * 2 : kind == 1 ? (size_t)V * H : (size_t)V * (H / 2);
}

static int upload_table(DevTable& t, int kind, const void* host, const float* scale_host, int V, int H, size_t* tally) {
    LSPK_REQUIRE(kind >= 0 && kind <= 2 && host, "embedding: bad arguments");
    LSPK_REQUIRE(kind == 0 || scale_host, "embedding: int8/int4 tables need the per-row scale");
    if (t.data) { cudaFree(t.data); t.data = nullptr; }
    if (t.scale) { cudaFree(t.scale); t.scale = nullptr; }
    if (int rc = dev_alloc(&t.data, table_bytes(kind, V, H), tally)) return rc;
    LSPK_CUDA(cudaMemcpy(t.data, host, table_bytes(kind, V, H), cudaMemcpyHostToDevice));
    if (kind != 0) {
        if (int rc = dev_alloc((void**)&t.scale, (size_t)V * 4, tally)) return rc;
        LSPK_CUDA(cudaMemcpy(t.scale, scale_host, (size_t)V * 4, cudaMemcpyHostToDevice));
    }
    t.kind = kind;
    return LSPK_OK;
}

// One transformer layer for `rows` rows held in the state's scratch buffers.
//   one row: norm + quantiser fused into the linear kernels;
//   otherwise rows go through the batched norm+quantise kernel once and the linear kernels (eight-row
//   tensor-core tiles below 32 rows, the tcgen05 GEMM from there) take the int8 prologue.
//   per_row_seq: rows are different sequences (batched decode) instead of consecutive positions.
int run_layer(State* s, int li, int rows, bool per_row_seq, int seq, bool skip_attention) {
    Model* m = s->m;
    const lspk_model_config& c = m->cfg;
    const DevLayer& L = m->layers[li];
    const int H = c.hidden_size, I = c.intermediate_size;
    const bool bitnet = c.arch == 0;
    // fp32 rows go to the linear layer as they are: one row is normalised and quantised inside the GEMV;
    // more rows are quantised once, by one kernel, straight into the activation layout of the kernel that
    // takes them (eight-row tiles below 32 rows, the tcgen05 GEMM from there).  The library scratch this
    // uses is sized by the warm-up run that precedes every graph capture.
    const bool fused_quant = true;
    const float eps = c.rms_norm_eps;

    auto linear = [&](int n_mats, const int* which, float* const* outs, const float* src, int8_t* src_q,
                      const DevNorm* norm, int K, int epilogue) -> int {
        lspk_linear_args a = {};
        for (int i = 0; i < n_mats; ++i) {
            a.w[i] = L.proj[which[i]];
            a.out[i] = outs[i];
        }
        a.n_mats = n_mats;
        a.M = rows;
        a.epilogue = epilogue;
        a.eps = eps;
        if (fused_quant) {
            a.x_f32 = src;
            if (norm) {
                a.prologue = LSPK_PRO_RMSNORM_QUANT;
                a.gamma = norm->g;
                a.gamma_is_bf16 = norm->is_bf16;
            } else {
                a.prologue = LSPK_PRO_QUANT;
            }
        } else {
            int rc = norm ? lspk_rmsnorm_quantize_rows(src, norm->g, norm->is_bf16, src_q, s->xs, rows, K, eps)
                          : lspk_quantize_rows(src, src_q, s->xs, rows, K);
            if (rc) return rc;
            a.prologue = LSPK_PRO_INT8;
            a.x_i8 = src_q;
            a.x_scales = s->xs;
        }
        return lspk_linear(&a);
    };

    // attention block
    {
        const int which[3] = {LSPK_PROJ_Q, LSPK_PROJ_K, LSPK_PROJ_V};
        float* outs[3] = {s->q, s->k, s->v};
        if (int rc = linear(3, which, outs, s->x, s->xq_h, &L.norm[LSPK_NORM_INPUT], H, LSPK_EPI_STORE)) return rc;
    }
    if (!skip_attention) {
        AttnParams p = {};
        p.q = s->q;
        p.k_cur = s->k;
        p.v_cur = s->v;
        p.out = s->attn;
        const size_t off = (size_t)li * s->layer_stride() + (per_row_seq ? 0 : (size_t)seq * s->seq_stride());
        p.cache_k = (char*)s->cache_k + off * s->kv_elem();
        p.cache_v = (char*)s->cache_v + off * s->kv_elem();
        p.rope_cos = s->rope_cos;
        p.rope_sin = s->rope_sin;
        p.rope_cur = s->rope_cur_valid ? s->rope_cur : nullptr;
        p.pos_ptr = s->ctl + (per_row_seq ? 0 : seq);
        p.pos_per_row = per_row_seq ? 1 : 0;
        p.cache_seq_stride = per_row_seq ? s->seq_stride() : 0;
        p.T = rows;
        p.Q = c.num_heads;
        p.KV = c.num_kv_heads;
        p.D = m->D();
        p.t_max = s->t_max;
        p.fused = (per_row_seq || rows == 1) ? 1 : 0;
        if (int rc = attention_launch(p, s->kv_fp16)) return rc;
    }
    {
        const int which[1] = {LSPK_PROJ_O};
        float* outs[1] = {s->x};
        if (int rc = linear(1, which, outs, s->attn, s->xq_h, bitnet ? &L.norm[LSPK_NORM_ATTN_SUB] : nullptr, H,
                            LSPK_EPI_ADD)) return rc;
    }
    // MLP block: gate and up as one call with the gate (ReLU^2 or SiLU) as its epilogue at every row count
    {
        const int which[2] = {LSPK_PROJ_GATE, LSPK_PROJ_UP};
        float* outs[2] = {s->inter, nullptr};
        if (int rc = linear(2, which, outs, s->x, s->xq_h, &L.norm[LSPK_NORM_POST_ATTN], H,
                            bitnet ? LSPK_EPI_RELU2_MUL : LSPK_EPI_SILU_MUL)) return rc;
    }
    {
        const int which[1] = {LSPK_PROJ_DOWN};
        float* outs[1] = {s->x};
        if (int rc = linear(1, which, outs, s->inter, s->xq_i, bitnet ? &L.norm[LSPK_NORM_FFN_SUB] : nullptr, I,
                            LSPK_EPI_ADD)) return rc;
    }
    return LSPK_OK;
}

// The kernels of one decode step for every sequence of the state (enqueued on the stream;
// captured into a graph by the caller).
static int enqueue_step(State* s, bool store_logits, bool host_io = false) {
    Model* m = s->m;
    const lspk_model_config& c = m->cfg;
    const int B = s->batch, H = c.hidden_size, V = c.vocab_size;
    LSPK_CUDA(launch(embed_kernel, dim3(B), dim3(256), 0, true, host_io ? (const int*)s->io_tok_dev : (const int*)(s->ctl + B),
                     m->emb.kind, (const void*)m->emb.data, (const float*)m->emb.scale, s->x, H, V, (const int*)s->ctl,
                     (const float*)s->rope_cos, (const float*)s->rope_sin, s->rope_cur, m->D() / 2, host_io ? 1 : 0));
    s->rope_cur_valid = true;
    for (int li = 0; li < c.num_layers; ++li)
        if (int rc = run_layer(s, li, B, B > 1, 0)) {
            s->rope_cur_valid = false;
            return rc;
        }
    s->rope_cur_valid = false;
    const DevTable& head = m->head.data ? m->head : m->emb;
    if (B == 1) {
        if (int rc = lm_head_launch(head.kind, head.data, head.scale, s->x, store_logits ? s->logits : nullptr, 1, V, H,
                                    m->final_norm.g, m->final_norm.is_bf16, c.rms_norm_eps, s->best)) return rc;
    } else {
        // the greedy choice of every row comes out of the LM head itself (bf16 table) or of a row argmax it
        // launches (int8 / int4 tables); logits are written only where something reads them
        const bool need_logits = store_logits || head.kind != 0 || (H % 32) != 0;
        if (int rc = lm_head_launch(head.kind, head.data, head.scale, s->x, need_logits ? s->logits : nullptr, B, V, H,
                                    m->final_norm.g, m->final_norm.is_bf16, c.rms_norm_eps, s->best)) return rc;
    }
    LSPK_CUDA(launch(finish_step_kernel, dim3(1), dim3(((B + 31) / 32) * 32), 0, true, s->ctl, s->best,
                     s->tokens_out, B, s->t_max, host_io ? s->io_pkt_dev : (unsigned long long*)nullptr,
                     host_io ? s->io_seq_dev : (unsigned*)nullptr));
    return LSPK_OK;
}

static int build_graph(State* s, int variant) {
    if (s->graph[variant] && s->graph_gen[variant] == scratch_generation()) return LSPK_OK;
    if (s->graph[variant]) {
        // library scratch whose addresses the graph holds was moved by a later call (a larger prefill, a
        // state of another batch size): capture again
        LSPK_CUDA(cudaStreamSynchronize(stream()));
        cudaGraphExecDestroy(s->graph[variant]);
        s->graph[variant] = nullptr;
    }
    // First run the step once outside capture: it sets the kernels' shared-memory attributes
    // (not allowed while capturing) and surfaces launch errors directly.  The warm-up must not
    // change the state: save and restore the control block around it.
    const int nctl = 2 * s->batch + 1;
    std::vector<int> saved(nctl);
    LSPK_CUDA(cudaMemcpyAsync(saved.data(), s->ctl, nctl * sizeof(int), cudaMemcpyDeviceToHost, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    if (int rc = enqueue_step(s, variant == 1, variant == 2)) return rc;
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    LSPK_CUDA(cudaMemcpyAsync(s->ctl, saved.data(), nctl * sizeof(int), cudaMemcpyHostToDevice, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    if (variant == 2) s->io_seq += 1;          // the warm-up step counted itself on the device

    cudaGraph_t g = nullptr;
    LSPK_CUDA(cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal));
    int rc = enqueue_step(s, variant == 1, variant == 2);
    cudaError_t e = cudaStreamEndCapture(stream(), &g);
    if (rc) {
        if (g) cudaGraphDestroy(g);
        return rc;
    }
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    size_t n = 0;
    cudaGraphGetNodes(g, nullptr, &n);
    s->graph_nodes = (int)n;
    e = cudaGraphInstantiate(&s->graph[variant], g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
    s->graph_gen[variant] = scratch_generation();
    return LSPK_OK;
}

}  // namespace lspk

using namespace lspk;

extern "C" {

lspk_model_t lspk_model_create(const lspk_model_config* cfg) {
    if (ensure_init()) return nullptr;
    if (!cfg || cfg->hidden_size <= 0 || cfg->num_layers <= 0 || cfg->num_heads <= 0 || cfg->num_kv_heads <= 0 ||
        cfg->intermediate_size <= 0 || cfg->vocab_size <= 0 || cfg->hidden_size % cfg->num_heads ||
        cfg->num_heads % cfg->num_kv_heads || (cfg->arch != 0 && cfg->arch != 1)) {
        fail(LSPK_ERR_ARG, "lspk_model_create: bad configuration");
        return nullptr;
    }
    const int D = cfg->hidden_size / cfg->num_heads;
    if (D != 64 && D != 128 && D != 256) {
        fail(LSPK_ERR_ARG, "lspk_model_create: head_dim %d not supported (64, 128, 256)", D);
        return nullptr;
    }
    Model* m = new Model();
    m->cfg = *cfg;
    m->layers.resize(cfg->num_layers);
    return reinterpret_cast<lspk_model_t>(m);
}

int lspk_model_set_projection(lspk_model_t h, int layer, int which, const uint8_t* packed_host, int N, int K,
                              float scale) {
    LSPK_REQUIRE(h, "lspk_model_set_projection: null model");
    Model* m = reinterpret_cast<Model*>(h);
    LSPK_REQUIRE(layer >= 0 && layer < m->cfg.num_layers && which >= 0 && which < 7,
                 "lspk_model_set_projection: layer/which out of range");
    const int H = m->cfg.hidden_size, I = m->cfg.intermediate_size, kv = m->kv_dim();
    const int wantN[7] = {H, kv, kv, H, I, I, H};
    const int wantK[7] = {H, H, H, H, H, H, I};
    LSPK_REQUIRE(N == wantN[which] && K == wantK[which], "lspk_model_set_projection: shape %dx%d, expected %dx%d", N,
                 K, wantN[which], wantK[which]);
    lspk_weight_t w = lspk_upload_packed(packed_host, N, K, scale);
    if (!w) return LSPK_ERR_CUDA;
    DevLayer& L = m->layers[layer];
    if (L.proj[which]) lspk_weight_free(L.proj[which]);
    L.proj[which] = w;
    m->bytes += reinterpret_cast<Weight*>(w)->bytes;
    return LSPK_OK;
}

int lspk_model_set_projection_bf16(lspk_model_t h, int layer, int which, const uint16_t* w_bf16_host, int N, int K,
                                   double absmean) {
    LSPK_REQUIRE(h, "lspk_model_set_projection_bf16: null model");
    Model* m = reinterpret_cast<Model*>(h);
    LSPK_REQUIRE(layer >= 0 && layer < m->cfg.num_layers && which >= 0 && which < 7,
                 "lspk_model_set_projection_bf16: layer/which out of range");
    const int H = m->cfg.hidden_size, I = m->cfg.intermediate_size, kv = m->kv_dim();
    const int wantN[7] = {H, kv, kv, H, I, I, H};
    const int wantK[7] = {H, H, H, H, H, H, I};
    LSPK_REQUIRE(N == wantN[which] && K == wantK[which], "lspk_model_set_projection_bf16: shape %dx%d, expected %dx%d",
                 N, K, wantN[which], wantK[which]);
    lspk_weight_t w = lspk_upload_bf16_ternary(w_bf16_host, N, K, absmean);
    if (!w) return LSPK_ERR_CUDA;
    DevLayer& L = m->layers[layer];
    if (L.proj[which]) lspk_weight_free(L.proj[which]);
    L.proj[which] = w;
    m->bytes += reinterpret_cast<Weight*>(w)->bytes;
    return LSPK_OK;
}

int lspk_model_set_norm(lspk_model_t h, int layer, int which, const void* gamma_host, int is_bf16, int K) {
    LSPK_REQUIRE(h && gamma_host, "lspk_model_set_norm: null argument");
    Model* m = reinterpret_cast<Model*>(h);
    DevNorm* n = nullptr;
    if (which == LSPK_NORM_FINAL) {
        n = &m->final_norm;
    } else {
        LSPK_REQUIRE(layer >= 0 && layer < m->cfg.num_layers && which >= 0 && which < 4,
                     "lspk_model_set_norm: layer/which out of range");
        n = &m->layers[layer].norm[which];
    }
    const int want = which == LSPK_NORM_FFN_SUB ? m->cfg.intermediate_size : m->cfg.hidden_size;
    LSPK_REQUIRE(K == want, "lspk_model_set_norm: length %d, expected %d", K, want);
    if (n->g) cudaFree(n->g);
    const size_t bytes = (size_t)K * (is_bf16 ? 2 : 4);
    if (int rc = dev_alloc(&n->g, bytes, &m->bytes)) return rc;
    LSPK_CUDA(cudaMemcpy(n->g, gamma_host, bytes, cudaMemcpyHostToDevice));
    n->is_bf16 = is_bf16;
    n->K = K;
    return LSPK_OK;
}

int lspk_model_set_embedding(lspk_model_t h, int kind, const void* emb_host, const float* scale_host) {
    LSPK_REQUIRE(h, "lspk_model_set_embedding: null model");
    Model* m = reinterpret_cast<Model*>(h);
    return upload_table(m->emb, kind, emb_host, scale_host, m->cfg.vocab_size, m->cfg.hidden_size, &m->bytes);
}

int lspk_model_set_lm_head(lspk_model_t h, int kind, const void* head_host, const float* scale_host) {
    LSPK_REQUIRE(h, "lspk_model_set_lm_head: null model");
    Model* m = reinterpret_cast<Model*>(h);
    return upload_table(m->head, kind, head_host, scale_host, m->cfg.vocab_size, m->cfg.hidden_size, &m->bytes);
}

int lspk_model_finalize(lspk_model_t h) {
    LSPK_REQUIRE(h, "lspk_model_finalize: null model");
    Model* m = reinterpret_cast<Model*>(h);
    const bool bitnet = m->cfg.arch == 0;
    for (int li = 0; li < m->cfg.num_layers; ++li) {
        for (int w = 0; w < 7; ++w)
            if (!m->layers[li].proj[w]) return fail(LSPK_ERR_STATE, "model: layer %d projection %d not set", li, w);
        for (int n = 0; n < (bitnet ? 4 : 2); ++n)
            if (!m->layers[li].norm[n].g) return fail(LSPK_ERR_STATE, "model: layer %d norm %d not set", li, n);
    }
    if (!m->final_norm.g) return fail(LSPK_ERR_STATE, "model: final norm not set");
    if (!m->emb.data) return fail(LSPK_ERR_STATE, "model: embedding not set");
    const int kind = (m->head.data ? m->head : m->emb).kind;
    const int E = kind == 0 ? 8 : kind == 1 ? 16 : 32;
    LSPK_REQUIRE(m->cfg.hidden_size % E == 0, "model: hidden_size must be a multiple of %d for this LM-head format", E);
    m->finalized = true;
    return LSPK_OK;
}

size_t lspk_model_device_bytes(lspk_model_t h) { return h ? reinterpret_cast<Model*>(h)->bytes : 0; }

lspk_weight_t lspk_model_projection(lspk_model_t h, int layer, int which) {
    if (!h) return nullptr;
    Model* m = reinterpret_cast<Model*>(h);
    if (layer < 0 || layer >= m->cfg.num_layers || which < 0 || which >= 7) return nullptr;
    return m->layers[layer].proj[which];
}

int lspk_model_free(lspk_model_t h) {
    if (!h) return LSPK_OK;
    Model* m = reinterpret_cast<Model*>(h);
    cudaStreamSynchronize(stream());
    for (auto& L : m->layers) {
        for (auto& w : L.proj) lspk_weight_free(w);
        for (auto& n : L.norm) cudaFree(n.g);
    }
    cudaFree(m->final_norm.g);
    cudaFree(m->emb.data);
    cudaFree(m->emb.scale);
    cudaFree(m->head.data);
    cudaFree(m->head.scale);
    delete m;
    return LSPK_OK;
}

lspk_state_t lspk_state_create(lspk_model_t h, int t_max, int batch, int kv_fp16, const float* rope_cos,
                               const float* rope_sin) {
    if (ensure_init()) return nullptr;
    Model* m = reinterpret_cast<Model*>(h);
    if (!m || !m->finalized || t_max < 1 || batch < 1 || batch > 1024 || !rope_cos || !rope_sin) {
        fail(LSPK_ERR_ARG, "lspk_state_create: bad arguments (model finalised? t_max=%d batch=%d)", t_max, batch);
        return nullptr;
    }
    State* s = new State();
    s->m = m;
    s->t_max = t_max;
    s->batch = batch;
    s->kv_fp16 = kv_fp16 ? 1 : 0;
    s->host_pos.assign(batch, 0);
    const lspk_model_config& c = m->cfg;
    const int H = c.hidden_size, I = c.intermediate_size, V = c.vocab_size, D = m->D(), kv = m->kv_dim();
    s->cap_rows = batch > 128 ? batch : 128;
    s->logits_rows = batch > 8 ? batch : 8;
    const size_t cache_bytes = (size_t)batch * s->seq_stride() * s->kv_elem();
    const size_t R = s->cap_rows;
    int rc = 0;
    rc |= dev_alloc(&s->cache_k, cache_bytes, &s->bytes);
    rc |= dev_alloc(&s->cache_v, cache_bytes, &s->bytes);
    rc |= dev_alloc((void**)&s->rope_cos, (size_t)t_max * (D / 2) * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->rope_sin, (size_t)t_max * (D / 2) * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->rope_cur, (size_t)batch * D * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->ctl, (size_t)(2 * batch + 1) * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->best, (size_t)batch * 8, &s->bytes);
    rc |= dev_alloc((void**)&s->tokens_out, (size_t)t_max * batch * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->x, R * H * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->q, R * H * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->k, R * kv * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->v, R * kv * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->attn, R * H * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->inter, R * I * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->inter2, R * I * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->logits, (size_t)s->logits_rows * V * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->xq_h, R * H, &s->bytes);
    rc |= dev_alloc((void**)&s->xq_i, R * I, &s->bytes);
    rc |= dev_alloc((void**)&s->xs, R * 4, &s->bytes);
    rc |= dev_alloc((void**)&s->tok_rows, R * 4, &s->bytes);
    if (!rc && cudaMallocHost((void**)&s->h_int, (size_t)(t_max * batch + R + 16) * 4) != cudaSuccess) rc = 1;
    if (!rc && cudaMallocHost((void**)&s->h_logits, (size_t)s->logits_rows * V * 4) != cudaSuccess) rc = 1;
    if (!rc && batch == 1) {
        // the two words of the host-fed step (see State): mapped pinned memory and its device alias
        void *io = nullptr, *io_dev = nullptr;
        if (cudaHostAlloc(&io, 64, cudaHostAllocMapped) != cudaSuccess) rc = 1;
        if (!rc && cudaHostGetDevicePointer(&io_dev, io, 0) != cudaSuccess) rc = 1;
        if (io) {
            memset(io, 0, 64);
            s->io_pkt = static_cast<unsigned long long*>(io);
            s->io_tok = reinterpret_cast<int*>(static_cast<char*>(io) + 16);
        }
        if (!rc) {
            s->io_pkt_dev = static_cast<unsigned long long*>(io_dev);
            s->io_tok_dev = reinterpret_cast<int*>(static_cast<char*>(io_dev) + 16);
            rc |= dev_alloc((void**)&s->io_seq_dev, 4, &s->bytes);
            if (!rc && cudaMemset(s->io_seq_dev, 0, 4) != cudaSuccess) rc = 1;
        }
    }
    if (!rc) {
        cudaError_t e = cudaMemset(s->cache_k, 0, cache_bytes);
        if (e == cudaSuccess) e = cudaMemset(s->cache_v, 0, cache_bytes);
        if (e == cudaSuccess) e = cudaMemset(s->ctl, 0, (size_t)(2 * batch + 1) * 4);
        if (e == cudaSuccess) e = cudaMemset(s->best, 0, (size_t)batch * 8);
        if (e == cudaSuccess) e = cudaMemcpy(s->rope_cos, rope_cos, (size_t)t_max * (D / 2) * 4, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(s->rope_sin, rope_sin, (size_t)t_max * (D / 2) * 4, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaDeviceSynchronize();   // the memsets ran on the default stream
        if (e != cudaSuccess) rc = 1;
    }
    if (rc) {
        fail(LSPK_ERR_CUDA, "lspk_state_create: allocation failed (%s)", cudaGetErrorString(cudaGetLastError()));
        lspk_state_free(reinterpret_cast<lspk_state_t>(s));
        return nullptr;
    }
    return reinterpret_cast<lspk_state_t>(s);
}

int lspk_state_free(lspk_state_t h) {
    if (!h) return LSPK_OK;
    State* s = reinterpret_cast<State*>(h);
    cudaStreamSynchronize(stream());
    for (auto& g : s->graph)
        if (g) cudaGraphExecDestroy(g);
    void* dev[] = {s->cache_k, s->cache_v, s->rope_cos, s->rope_sin, s->rope_cur, s->ctl, s->best, s->tokens_out, s->x, s->q, s->k,
                   s->v, s->attn, s->inter, s->inter2, s->logits, s->xq_h, s->xq_i, s->xs, s->tok_rows};
    for (void* p : dev) cudaFree(p);
    if (s->h_int) cudaFreeHost(s->h_int);
    if (s->h_logits) cudaFreeHost(s->h_logits);
    if (s->io_pkt) cudaFreeHost(s->io_pkt);
    cudaFree(s->io_seq_dev);
    delete s;
    return LSPK_OK;
}

int lspk_state_get_pos(lspk_state_t h, int seq) {
    State* s = reinterpret_cast<State*>(h);
    if (!s || seq < 0 || seq >= s->batch) return -1;
    return s->host_pos[seq];
}

int lspk_state_set_pos(lspk_state_t h, int seq, int pos) {
    State* s = reinterpret_cast<State*>(h);
    LSPK_REQUIRE(s && seq >= 0 && seq < s->batch && pos >= 0 && pos <= s->t_max, "lspk_state_set_pos: out of range");
    s->h_int[0] = pos;
    LSPK_CUDA(cudaMemcpyAsync(s->ctl + seq, s->h_int, 4, cudaMemcpyHostToDevice, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    s->host_pos[seq] = pos;
    return LSPK_OK;
}

size_t lspk_state_device_bytes(lspk_state_t h) { return h ? reinterpret_cast<State*>(h)->bytes : 0; }

int lspk_state_read_kv(lspk_state_t h, int seq, int layer, int n_pos, float* k_host, float* v_host) {
    State* s = reinterpret_cast<State*>(h);
    LSPK_REQUIRE(s && seq >= 0 && seq < s->batch && layer >= 0 && layer < s->m->cfg.num_layers && n_pos >= 0 &&
                 n_pos <= s->t_max, "lspk_state_read_kv: out of range");
    const size_t n = (size_t)n_pos * s->m->kv_dim();
    const size_t off = (size_t)seq * s->seq_stride() + (size_t)layer * s->layer_stride();
    std::vector<unsigned char> tmp(n * s->kv_elem());
    for (int which = 0; which < 2; ++which) {
        float* dst = which ? v_host : k_host;
        if (!dst) continue;
        const char* src = (const char*)(which ? s->cache_v : s->cache_k) + off * s->kv_elem();
        LSPK_CUDA(cudaMemcpyAsync(tmp.data(), src, n * s->kv_elem(), cudaMemcpyDeviceToHost, stream()));
        LSPK_CUDA(cudaStreamSynchronize(stream()));
        if (s->kv_fp16) {
            const __half* hp = reinterpret_cast<const __half*>(tmp.data());
            for (size_t i = 0; i < n; ++i) dst[i] = __half2float(hp[i]);
        } else {
            memcpy(dst, tmp.data(), n * 4);
        }
    }
    return LSPK_OK;
}

int lspk_forward_step(lspk_state_t h, const int* tokens_host, float* logits_host, int* next_tokens_host) {
    State* s = reinterpret_cast<State*>(h);
    LSPK_REQUIRE(s && tokens_host, "lspk_forward_step: null argument");
    const int B = s->batch, V = s->m->cfg.vocab_size;
    for (int b = 0; b < B; ++b)
        if (s->host_pos[b] >= s->t_max)
            return fail(LSPK_ERR_STATE, "inference state exhausted: pos=%d >= t_max=%d", s->host_pos[b], s->t_max);
    if (B == 1 && !logits_host && next_tokens_host && s->io_seq_dev) {
        // One sequence, token id in, token id out: no copy operations and no stream wait.  The step's first kernel
        // reads the token from mapped pinned memory; its last kernel stores (count << 32 | next token) there.
        *(volatile int*)s->io_tok = tokens_host[0];
        if (int rc = build_graph(s, 2)) return rc;
        const unsigned want = ++s->io_seq;
        LSPK_CUDA(cudaGraphLaunch(s->graph[2], stream()));
        unsigned long long pkt = 0;
        for (unsigned spins = 1;; ++spins) {
            pkt = *(volatile unsigned long long*)s->io_pkt;
            if ((unsigned)(pkt >> 32) == want) break;
            if ((spins & 0x3fffu) == 0) {
                // every so often ask the driver: an error ends the wait, and so does a stream that has finished
                // without the packet showing the expected count (host and device counts out of step)
                const cudaError_t q = cudaStreamQuery(stream());
                if (q == cudaErrorNotReady) continue;
                pkt = *(volatile unsigned long long*)s->io_pkt;
                if (q == cudaSuccess && (unsigned)(pkt >> 32) == want) break;
                s->io_seq = (unsigned)(pkt >> 32);
                if (q != cudaSuccess) return fail(LSPK_ERR_CUDA, "lspk_forward_step: %s", cudaGetErrorString(q));
                return fail(LSPK_ERR_STATE, "lspk_forward_step: step %u finished without its result packet", want);
            }
        }
        next_tokens_host[0] = (int)(uint32_t)pkt;
        s->host_pos[0] += 1;
        return LSPK_OK;
    }
    const int variant = (logits_host || B > 1) ? 1 : 0;
    if (int rc = build_graph(s, variant)) return rc;
    memcpy(s->h_int, tokens_host, (size_t)B * 4);
    LSPK_CUDA(cudaMemcpyAsync(s->ctl + B, s->h_int, (size_t)B * 4, cudaMemcpyHostToDevice, stream()));
    LSPK_CUDA(cudaGraphLaunch(s->graph[variant], stream()));
    if (logits_host)
        LSPK_CUDA(cudaMemcpyAsync(s->h_logits, s->logits, (size_t)B * V * 4, cudaMemcpyDeviceToHost, stream()));
    if (next_tokens_host)
        LSPK_CUDA(cudaMemcpyAsync(s->h_int + B, s->ctl + B, (size_t)B * 4, cudaMemcpyDeviceToHost, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    if (logits_host) memcpy(logits_host, s->h_logits, (size_t)B * V * 4);
    if (next_tokens_host) memcpy(next_tokens_host, s->h_int + B, (size_t)B * 4);
    for (int b = 0; b < B; ++b) s->host_pos[b] += 1;
    return LSPK_OK;
}

int lspk_decode_greedy(lspk_state_t h, const int* first_tokens_host, int n_steps, int* tokens_out_host) {
    State* s = reinterpret_cast<State*>(h);
    LSPK_REQUIRE(s && first_tokens_host && tokens_out_host && n_steps >= 1, "lspk_decode_greedy: bad arguments");
    const int B = s->batch;
    LSPK_REQUIRE(n_steps <= s->t_max, "lspk_decode_greedy: n_steps exceeds the output buffer (t_max)");
    for (int b = 0; b < B; ++b)
        if (s->host_pos[b] + n_steps > s->t_max)
            return fail(LSPK_ERR_STATE, "inference state exhausted: pos=%d + %d steps > t_max=%d", s->host_pos[b],
                        n_steps, s->t_max);
    const int variant = B > 1 ? 1 : 0;
    if (int rc = build_graph(s, variant)) return rc;
    memcpy(s->h_int, first_tokens_host, (size_t)B * 4);
    s->h_int[B] = 0;   // step counter
    LSPK_CUDA(cudaMemcpyAsync(s->ctl + B, s->h_int, (size_t)(B + 1) * 4, cudaMemcpyHostToDevice, stream()));
    for (int i = 0; i < n_steps; ++i) LSPK_CUDA(cudaGraphLaunch(s->graph[variant], stream()));
    LSPK_CUDA(cudaMemcpyAsync(s->h_int, s->tokens_out, (size_t)n_steps * B * 4, cudaMemcpyDeviceToHost, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    memcpy(tokens_out_host, s->h_int, (size_t)n_steps * B * 4);
    for (int b = 0; b < B; ++b) s->host_pos[b] += n_steps;
    return LSPK_OK;
}

int lspk_forward_prefill(lspk_state_t h, int seq, const int* tokens_host, int T, float* last_logits_host,
                         float* all_logits_host, int* next_token_host) {
    State* s = reinterpret_cast<State*>(h);
    LSPK_REQUIRE(s && tokens_host && T >= 1, "lspk_forward_prefill: bad arguments");
    LSPK_REQUIRE(seq >= 0 && seq < s->batch, "lspk_forward_prefill: sequence index out of range");
    Model* m = s->m;
    const lspk_model_config& c = m->cfg;
    const int H = c.hidden_size, V = c.vocab_size;
    if (s->host_pos[seq] + T > s->t_max)
        return fail(LSPK_ERR_STATE, "prefill would exceed t_max: pos=%d T=%d t_max=%d", s->host_pos[seq], T, s->t_max);
    const DevTable& head = m->head.data ? m->head : m->emb;
    for (int t0 = 0; t0 < T; t0 += s->cap_rows) {
        const int rows = (T - t0) < s->cap_rows ? (T - t0) : s->cap_rows;
        memcpy(s->h_int, tokens_host + t0, (size_t)rows * 4);
        LSPK_CUDA(cudaMemcpyAsync(s->tok_rows, s->h_int, (size_t)rows * 4, cudaMemcpyHostToDevice, stream()));
        if (int rc = launch_embed(s->tok_rows, rows, m->emb.kind, m->emb.data, m->emb.scale, s->x, H, V)) return rc;
        for (int li = 0; li < c.num_layers; ++li)
            if (int rc = run_layer(s, li, rows, false, seq)) return rc;
        if (all_logits_host) {
            for (int r0 = 0; r0 < rows; r0 += s->logits_rows) {
                const int rr = (rows - r0) < s->logits_rows ? (rows - r0) : s->logits_rows;
                if (int rc = lm_head_launch(head.kind, head.data, head.scale, s->x + (size_t)r0 * H, s->logits, rr, V, H,
                                            m->final_norm.g, m->final_norm.is_bf16, c.rms_norm_eps, nullptr)) return rc;
                LSPK_CUDA(cudaMemcpyAsync(s->h_logits, s->logits, (size_t)rr * V * 4, cudaMemcpyDeviceToHost, stream()));
                LSPK_CUDA(cudaStreamSynchronize(stream()));
                memcpy(all_logits_host + (size_t)(t0 + r0) * V, s->h_logits, (size_t)rr * V * 4);
            }
        }
        const bool last_chunk = t0 + rows >= T;
        const bool want_last = last_chunk && (last_logits_host || next_token_host);
        if (want_last) {
            LSPK_CUDA(cudaMemsetAsync(s->best, 0, 8, stream()));
            if (int rc = lm_head_launch(head.kind, head.data, head.scale, s->x + (size_t)(rows - 1) * H, s->logits, 1, V, H,
                                        m->final_norm.g, m->final_norm.is_bf16, c.rms_norm_eps, s->best)) return rc;
            LSPK_CUDA(cudaMemcpyAsync(s->h_logits, s->logits, (size_t)V * 4, cudaMemcpyDeviceToHost, stream()));
            LSPK_CUDA(cudaMemcpyAsync(s->h_int + s->cap_rows, s->best, 8, cudaMemcpyDeviceToHost, stream()));
            LSPK_CUDA(cudaMemsetAsync(s->best, 0, 8, stream()));     // the decode step expects cleared keys
        }
        LSPK_CUDA(launch(advance_pos_kernel, dim3(1), dim3(32), 0, true, s->ctl, seq, rows));
        LSPK_CUDA(cudaStreamSynchronize(stream()));     // the pinned staging is reused by the next chunk
        s->host_pos[seq] += rows;
        if (want_last) {
            if (last_logits_host) memcpy(last_logits_host, s->h_logits, (size_t)V * 4);
            if (next_token_host) {
                unsigned long long key = 0;
                memcpy(&key, s->h_int + s->cap_rows, 8);
                *next_token_host = (int)(0xffffffffu - (uint32_t)(key & 0xffffffffull));
            }
        }
    }
    return LSPK_OK;
}

int lspk_state_step_kernel_count(lspk_state_t h) {
    State* s = reinterpret_cast<State*>(h);
    if (!s) return 0;
    return s->graph_nodes;
}

}  // extern "C"
