// Host-pointer drop-ins: the symbol set the reference's ctypes loader binds
// (litespark_inference/torchless/kernel.py:227-322) under the tag `sm100`.  Each call stages its
// host arguments into device scratch buffers, runs the same CUDA kernels the device-resident
// API uses, and copies the result back before returning.  Failures are recorded (see
// lspk_last_error) because, like the reference, these functions have no status return.
#include <map>
#include <mutex>
#include <string.h>

#include "internal.cuh"

namespace lspk {

// ---- growable device scratch slots ------------------------------------------------------
enum { S_X = 0, S_XS, S_Y, S_A, S_B, S_G, S_EMB, S_ESC, S_COUNT };
static void* g_slot[S_COUNT] = {};
static size_t g_slot_bytes[S_COUNT] = {};
static std::mutex g_compat_mu;

static void* slot(int i, size_t bytes) {
    if (bytes > g_slot_bytes[i]) {
        if (g_slot[i]) cudaFree(g_slot[i]);
        g_slot[i] = nullptr;
        size_t want = bytes + bytes / 4 + 256;
        if (cudaMalloc(&g_slot[i], want) != cudaSuccess) {
            g_slot_bytes[i] = 0;
            fail(LSPK_ERR_CUDA, "device scratch allocation of %zu bytes failed", want);
            return nullptr;
        }
        g_slot_bytes[i] = want;
    }
    return g_slot[i];
}

static bool up(void* dst, const void* src, size_t bytes) {
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream());
    if (e != cudaSuccess) { fail(LSPK_ERR_CUDA, "host->device copy failed: %s", cudaGetErrorString(e)); return false; }
    return true;
}
static bool down(void* dst, const void* src, size_t bytes) {
    cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream());
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream());
    if (e != cudaSuccess) { fail(LSPK_ERR_CUDA, "device->host copy failed: %s", cudaGetErrorString(e)); return false; }
    return true;
}

// ---- registry of resident weights / embeddings keyed by host address ------------------------
struct PackedEntry { lspk_weight_t w; int N, K; };
struct EmbEntry { void* emb; float* scale; int kind, V, H; };
static std::map<const void*, PackedEntry> g_packed;
static std::map<const void*, EmbEntry> g_emb;

static size_t emb_bytes(int kind, int V, int H) {
    return kind == 0 ? (size_t)V * H * 2 : kind == 1 ? (size_t)V * H : (size_t)V * (H / 2);
}

// Shared body of _m1 / _mT / _prefill.
static void matmul_host(const int8_t* x, const float* x_scales, const uint8_t* packed_w, float w_scale,
                        float* y, int T, int N, int K) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    if (ensure_init()) return;
    if (!x || !x_scales || !packed_w || !y || T < 1 || N < 1 || K < 4 || (K & 3)) {
        fail(LSPK_ERR_ARG, "matmul_lut_sm100: bad arguments (T=%d N=%d K=%d)", T, N, K);
        return;
    }
    lspk_weight_t w = nullptr;
    bool temp = false;
    auto it = g_packed.find(packed_w);
    if (it != g_packed.end() && it->second.N == N && it->second.K == K) {
        w = it->second.w;
    } else {
        w = lspk_upload_packed(packed_w, N, K, w_scale);
        temp = true;
    }
    if (!w) return;
    reinterpret_cast<Weight*>(w)->scale = w_scale;
    int8_t* dx = (int8_t*)slot(S_X, (size_t)T * K);
    float* dxs = (float*)slot(S_XS, (size_t)T * 4);
    float* dy = (float*)slot(S_Y, (size_t)T * N * 4);
    if (dx && dxs && dy && up(dx, x, (size_t)T * K) && up(dxs, x_scales, (size_t)T * 4)) {
        lspk_linear_args a = {};
        a.w[0] = w;
        a.out[0] = dy;
        a.n_mats = 1;
        a.M = T;
        a.prologue = LSPK_PRO_INT8;
        a.epilogue = LSPK_EPI_STORE;
        a.x_i8 = dx;
        a.x_scales = dxs;
        if (lspk_linear(&a) == LSPK_OK) down(y, dy, (size_t)T * N * 4);
    }
    if (temp) {
        cudaStreamSynchronize(stream());
        lspk_weight_free(w);
    }
}

static void rows_host(const float* x, const void* gamma, int gamma_is_bf16, float* out_f32, int8_t* out_i8,
                      float* scales, int T, int K, float eps, int mode) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    if (ensure_init()) return;
    if (!x || T < 1 || K < 1) { fail(LSPK_ERR_ARG, "row helper: bad arguments (T=%d K=%d)", T, K); return; }
    const size_t n = (size_t)T * K;
    float* dx = (float*)slot(S_A, n * 4);
    void* dg = gamma ? slot(S_G, (size_t)K * (gamma_is_bf16 ? 2 : 4)) : nullptr;
    float* dof = (mode & 2) ? nullptr : (float*)slot(S_B, n * 4);
    int8_t* doi = (mode & 2) ? (int8_t*)slot(S_X, n) : nullptr;
    float* dsc = (mode & 2) ? (float*)slot(S_XS, (size_t)T * 4) : nullptr;
    if (!dx || (gamma && !dg) || (!(mode & 2) && !dof) || ((mode & 2) && (!doi || !dsc))) return;
    if (!up(dx, x, n * 4)) return;
    if (gamma && !up(dg, gamma, (size_t)K * (gamma_is_bf16 ? 2 : 4))) return;
    int rc;
    if (mode == 2) rc = lspk_quantize_rows(dx, doi, dsc, T, K);
    else if (mode == 1) rc = lspk_rmsnorm_rows(dx, dg, gamma_is_bf16, dof, T, K, eps);
    else rc = lspk_rmsnorm_quantize_rows(dx, dg, gamma_is_bf16, doi, dsc, T, K, eps);
    if (rc != LSPK_OK) return;
    if (mode & 2) {
        cudaMemcpyAsync(out_i8, doi, n, cudaMemcpyDeviceToHost, stream());
        down(scales, dsc, (size_t)T * 4);
    } else {
        down(out_f32, dof, n * 4);
    }
}

static void lm_head_host(int kind, const void* emb, const float* emb_scale, const float* x, float* logits,
                         int V, int H) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    if (ensure_init()) return;
    if (!emb || !x || !logits || V < 1 || H < 1 || (kind != 0 && !emb_scale)) {
        fail(LSPK_ERR_ARG, "lm_head_sm100: bad arguments (V=%d H=%d)", V, H);
        return;
    }
    const void* demb = nullptr;
    const float* dsc = nullptr;
    auto it = g_emb.find(emb);
    if (it != g_emb.end() && it->second.kind == kind && it->second.V == V && it->second.H == H) {
        demb = it->second.emb;
        dsc = it->second.scale;
    } else {
        void* e = slot(S_EMB, emb_bytes(kind, V, H));
        if (!e || !up(e, emb, emb_bytes(kind, V, H))) return;
        demb = e;
        if (kind != 0) {
            float* s = (float*)slot(S_ESC, (size_t)V * 4);
            if (!s || !up(s, emb_scale, (size_t)V * 4)) return;
            dsc = s;
        }
    }
    float* dx = (float*)slot(S_A, (size_t)H * 4);
    float* dl = (float*)slot(S_Y, (size_t)V * 4);
    if (!dx || !dl || !up(dx, x, (size_t)H * 4)) return;
    if (lspk_lm_head(kind, demb, dsc, dx, dl, 1, V, H) == LSPK_OK) down(logits, dl, (size_t)V * 4);
}

}  // namespace lspk

using namespace lspk;

extern "C" {

void matmul_lut_sm100_m1(const int8_t* x, const uint8_t* packed_w, float w_scale, float x_scale, float* y,
                         int N, int K) {
    matmul_host(x, &x_scale, packed_w, w_scale, y, 1, N, K);
}

void matmul_lut_sm100_mT(const int8_t* x, const float* x_scales, const uint8_t* packed_w, float w_scale,
                         float* y, int T, int N, int K) {
    matmul_host(x, x_scales, packed_w, w_scale, y, T, N, K);
}

void matmul_lut_sm100_prefill(const int8_t* x, const uint8_t* packed_w, float w_scale, const float* x_scale,
                              float* y, int M, int N, int K) {
    matmul_host(x, x_scale, packed_w, w_scale, y, M, N, K);
}

float quantize_activation_sm100(const float* x, int8_t* out, int K) {
    float s = 0.0f;
    rows_host(x, nullptr, 0, nullptr, out, &s, 1, K, 0.0f, 2);
    return s;
}
void quantize_activation_batched_sm100(const float* x, int8_t* out, float* scales, int T, int K) {
    rows_host(x, nullptr, 0, nullptr, out, scales, T, K, 0.0f, 2);
}

void rmsnorm_bf16gamma_fp32_sm100(const float* x, const uint16_t* gamma, float* out, int K, float eps) {
    rows_host(x, gamma, 1, out, nullptr, nullptr, 1, K, eps, 1);
}
void rmsnorm_fp32gamma_fp32_sm100(const float* x, const float* gamma, float* out, int K, float eps) {
    rows_host(x, gamma, 0, out, nullptr, nullptr, 1, K, eps, 1);
}
void rmsnorm_bf16gamma_fp32_batched_sm100(const float* x, const uint16_t* gamma, float* out, int T, int K, float eps) {
    rows_host(x, gamma, 1, out, nullptr, nullptr, T, K, eps, 1);
}
void rmsnorm_fp32gamma_fp32_batched_sm100(const float* x, const float* gamma, float* out, int T, int K, float eps) {
    rows_host(x, gamma, 0, out, nullptr, nullptr, T, K, eps, 1);
}

float rmsnorm_quantize_bf16gamma_sm100(const float* x, const uint16_t* gamma, int8_t* out_i8, float* tmp, int K,
                                       float eps) {
    (void)tmp;
    float s = 0.0f;
    rows_host(x, gamma, 1, nullptr, out_i8, &s, 1, K, eps, 3);
    return s;
}
void rmsnorm_quantize_bf16gamma_batched_sm100(const float* x, const uint16_t* gamma, int8_t* out_i8, float* scales,
                                              float* tmp, int T, int K, float eps) {
    (void)tmp;
    rows_host(x, gamma, 1, nullptr, out_i8, scales, T, K, eps, 3);
}

void relu2_mul_fp32_batched_sm100(const float* gate, const float* up_, float* out, int T, int K) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    if (ensure_init()) return;
    if (!gate || !up_ || !out || T < 1 || K < 1) { fail(LSPK_ERR_ARG, "relu2_mul_sm100: bad arguments"); return; }
    const size_t n = (size_t)T * K;
    float* dg = (float*)slot(S_A, n * 4);
    float* du = (float*)slot(S_B, n * 4);
    float* dout = (float*)slot(S_Y, n * 4);
    if (!dg || !du || !dout || !up(dg, gate, n * 4) || !up(du, up_, n * 4)) return;
    if (lspk_relu2_mul_rows(dg, du, dout, T, K) == LSPK_OK) down(out, dout, n * 4);
}
void relu2_mul_fp32_sm100(const float* gate, const float* up_, float* out, int K) {
    relu2_mul_fp32_batched_sm100(gate, up_, out, 1, K);
}

void add_inplace_fp32_sm100(float* a, const float* b, int K) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    if (ensure_init()) return;
    if (!a || !b || K < 1) { fail(LSPK_ERR_ARG, "add_inplace_sm100: bad arguments"); return; }
    float* da = (float*)slot(S_A, (size_t)K * 4);
    float* db = (float*)slot(S_B, (size_t)K * 4);
    if (!da || !db || !up(da, a, (size_t)K * 4) || !up(db, b, (size_t)K * 4)) return;
    if (lspk_add_rows(da, db, (size_t)K) == LSPK_OK) down(a, da, (size_t)K * 4);
}

void lm_head_bf16_fp32_sm100(const uint16_t* emb, const float* x, float* logits, int V, int H) {
    lm_head_host(0, emb, nullptr, x, logits, V, H);
}
void lm_head_int8_fp32_sm100(const int8_t* emb, const float* emb_scale, const float* x, float* logits, int V, int H) {
    lm_head_host(1, emb, emb_scale, x, logits, V, H);
}
void lm_head_int4_fp32_sm100(const uint8_t* emb, const float* emb_scale, const float* x, float* logits, int V, int H) {
    lm_head_host(2, emb, emb_scale, x, logits, V, H);
}

int matmul_lut_sm100_has_omp(void) { return 0; }
int matmul_lut_sm100_max_threads(void) { return lspk_sm_count(); }

int lspk_register_packed(const uint8_t* packed_host, int N, int K) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    if (int rc = ensure_init()) return rc;
    lspk_weight_t w = lspk_upload_packed(packed_host, N, K, 1.0f);
    if (!w) return LSPK_ERR_CUDA;
    auto it = g_packed.find(packed_host);
    if (it != g_packed.end()) lspk_weight_free(it->second.w);
    g_packed[packed_host] = PackedEntry{w, N, K};
    return LSPK_OK;
}

int lspk_register_embedding(int kind, const void* emb_host, const float* emb_scale_host, int V, int H) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(emb_host && kind >= 0 && kind <= 2 && V > 0 && H > 0, "lspk_register_embedding: bad arguments");
    LSPK_REQUIRE(kind == 0 || emb_scale_host, "lspk_register_embedding: int8/int4 need the scale vector");
    EmbEntry e = {};
    e.kind = kind; e.V = V; e.H = H;
    LSPK_CUDA(cudaMalloc(&e.emb, emb_bytes(kind, V, H)));
    LSPK_CUDA(cudaMemcpy(e.emb, emb_host, emb_bytes(kind, V, H), cudaMemcpyHostToDevice));
    if (kind != 0) {
        LSPK_CUDA(cudaMalloc((void**)&e.scale, (size_t)V * 4));
        LSPK_CUDA(cudaMemcpy(e.scale, emb_scale_host, (size_t)V * 4, cudaMemcpyHostToDevice));
    }
    auto it = g_emb.find(emb_host);
    if (it != g_emb.end()) { cudaFree(it->second.emb); cudaFree(it->second.scale); }
    g_emb[emb_host] = e;
    return LSPK_OK;
}

int lspk_unregister(const void* host_ptr) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    auto it = g_packed.find(host_ptr);
    if (it != g_packed.end()) { lspk_weight_free(it->second.w); g_packed.erase(it); }
    auto ie = g_emb.find(host_ptr);
    if (ie != g_emb.end()) { cudaFree(ie->second.emb); cudaFree(ie->second.scale); g_emb.erase(ie); }
    return LSPK_OK;
}

int lspk_unregister_all(void) {
    std::lock_guard<std::mutex> lk(g_compat_mu);
    for (auto& kv : g_packed) lspk_weight_free(kv.second.w);
    g_packed.clear();
    for (auto& kv : g_emb) { cudaFree(kv.second.emb); cudaFree(kv.second.scale); }
    g_emb.clear();
    return LSPK_OK;
}

}  // extern "C"
