// Packed-expert ternary MoE layer (top-2 softmax router, squared-ReLU experts).
//
// No counterpart in the reference.  Per token:  h = RMSNorm(x);  p = softmax(Wr h);  the two largest
// p (ties to the lower index) renormalised to sum one;  for each routed expert e:
// y_e = down_e(quant(SubLN_e(relu(gate_e q)^2 * up_e q))), q = quant(h) computed once;
// x += w_0 y_0 + w_1 y_1.
//
// Kernel sequence (all on the library stream, no host synchronisation):
//   moe_router_kernel        one CTA per token: norm, quantise, router logits, softmax, top-2
//   moe_group_kernel         rows (token, slot) listed per expert, ascending
//   ternary_linear_kernel    expert-grouped launch, gate/up pair, ReLU^2 epilogue  (grid.z = expert)
//   moe_subnorm_quant_kernel per routed row: RMSNorm with the row's expert's weights + quantiser
//   ternary_linear_kernel    expert-grouped launch, down projection
//   moe_combine_kernel       x += w_0 y_0 + w_1 y_1
// The expert matrices live in one device buffer [expert][gate|up|down] in the device chunk layout;
// an expert with no routed row costs no weight traffic.
#include <vector>

#include "internal.cuh"
#include "ternary_core.cuh"
#include "../../include/lspk_hybrid.h"

namespace lspk {

constexpr int kMoeThreads = 256;
constexpr int kMaxExperts = 32;

struct Moe {
    int E = 0, H = 0, I = 0;
    float eps = 1e-5f;
    uint4* w = nullptr;              // [E][3][mat_chunks] device layout
    size_t mat_stride = 0;           // uint4 units per matrix
    int groups_gu = 0, chunks_gu = 0, groups_d = 0, chunks_d = 0;
    float* scales = nullptr;         // [E][3]
    float* router = nullptr;         // [E][H]
    uint16_t* norm = nullptr;        // [H]
    uint16_t* sub_norm = nullptr;    // [E][I]
    // per-call scratch, sized for cap_B token rows
    int cap_B = 0;
    int8_t *xq = nullptr, *xq2 = nullptr;
    float *xs = nullptr, *xs2 = nullptr, *selw = nullptr, *inter = nullptr, *ydown = nullptr;
    int *sel = nullptr, *counts = nullptr, *rows = nullptr;
    size_t bytes = 0;
};

// One CTA per token row.
__global__ void __launch_bounds__(kMoeThreads)
moe_router_kernel(const float* __restrict__ x, const uint16_t* __restrict__ gamma, const float* __restrict__ router,
                  int8_t* __restrict__ xq, float* __restrict__ xs, int* __restrict__ sel, float* __restrict__ selw,
                  int H, int E, float eps) {
    extern __shared__ __align__(16) float hs[];           // [H] normalised row
    __shared__ float red[32];
    __shared__ float s_logit[kMaxExperts][kMoeThreads / 32];
    grid_dependency_launch();
    grid_dependency_wait();
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* src = x + (size_t)t * H;
    float ssq = 0.0f;
    for (int k = tid; k < H; k += kMoeThreads) {
        const float v = src[k];
        hs[k] = v;
        ssq = fmaf(v, v, ssq);
    }
    ssq = block_sum(ssq, red);
    const float rrms = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, (float)H), eps)));
    float amax = 0.0f;
    for (int k = tid; k < H; k += kMoeThreads) {
        const float v = __fmul_rn(__fmul_rn(hs[k], rrms), bf16_bits_to_f32(gamma[k]));
        hs[k] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    amax = block_max(amax, red);
    const float scale = quant_scale_from_absmax(amax);
    const float inv = __frcp_rn(scale);
    const int tail_start = H & ~15;
    for (int k = tid; k < H; k += kMoeThreads) {
        int q;
        if (k < tail_start) {
            q = (int)quant_rne_sat(__fmul_rn(hs[k], inv));
        } else {
            q = max(-127, min(127, (int)roundf(__fmul_rn(hs[k], inv))));
        }
        xq[(size_t)t * H + k] = (int8_t)q;
    }
    if (tid == 0) xs[t] = scale;
    // router logits: every thread holds a partial of each expert's dot product
    for (int e = 0; e < E; ++e) {
        const float* wr = router + (size_t)e * H;
        float acc = 0.0f;
        for (int k = tid; k < H; k += kMoeThreads) acc = fmaf(hs[k], wr[k], acc);
        acc = warp_sum(acc);
        if (lane == 0) s_logit[e][warp] = acc;
    }
    __syncthreads();
    if (tid == 0) {
        float logit[kMaxExperts], mx = -INFINITY;
        for (int e = 0; e < E; ++e) {
            float a = 0.0f;
            for (int w = 0; w < kMoeThreads / 32; ++w) a += s_logit[e][w];
            logit[e] = a;
            mx = fmaxf(mx, a);
        }
        float sum = 0.0f;
        for (int e = 0; e < E; ++e) {
            logit[e] = expf(logit[e] - mx);
            sum += logit[e];
        }
        int i0 = 0, i1 = -1;
        float p0 = -1.0f, p1 = -1.0f;
        for (int e = 0; e < E; ++e) {
            const float pe = __fdiv_rn(logit[e], sum);
            if (pe > p0) {
                p1 = p0; i1 = i0;
                p0 = pe; i0 = e;
            } else if (pe > p1) {
                p1 = pe; i1 = e;
            }
        }
        const float den = __fadd_rn(p0, p1);
        sel[2 * t] = i0;
        sel[2 * t + 1] = i1;
        selw[2 * t] = __fdiv_rn(p0, den);
        selw[2 * t + 1] = __fdiv_rn(p1, den);
    }
}

// rows[e][0..counts[e]) = the routed rows (2*token + slot) of expert e, ascending.
__global__ void moe_group_kernel(const int* __restrict__ sel, int n_rows, int E, int* __restrict__ counts,
                                 int* __restrict__ rows, int rows_stride) {
    grid_dependency_launch();
    grid_dependency_wait();
    const int e = threadIdx.x;
    if (e < E) {
        int c = 0;
        for (int r = 0; r < n_rows; ++r)
            if (sel[r] == e) rows[(size_t)e * rows_stride + c++] = r;
        counts[e] = c;
    }
}

// One CTA per routed row: RMSNorm with the weights of the row's expert, then the int8 quantiser.
__global__ void __launch_bounds__(kMoeThreads)
moe_subnorm_quant_kernel(const float* __restrict__ inter, const int* __restrict__ sel, const uint16_t* __restrict__ gamma,
                         int8_t* __restrict__ out, float* __restrict__ scales, int K, float eps) {
    extern __shared__ __align__(16) float vs[];
    __shared__ float red[32];
    grid_dependency_launch();
    grid_dependency_wait();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* src = inter + (size_t)r * K;
    const uint16_t* g = gamma + (size_t)sel[r] * K;
    float ssq = 0.0f;
    for (int k = tid; k < K; k += kMoeThreads) {
        const float v = src[k];
        vs[k] = v;
        ssq = fmaf(v, v, ssq);
    }
    ssq = block_sum(ssq, red);
    const float rrms = __frcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, (float)K), eps)));
    float amax = 0.0f;
    for (int k = tid; k < K; k += kMoeThreads) {
        const float v = __fmul_rn(__fmul_rn(vs[k], rrms), bf16_bits_to_f32(g[k]));
        vs[k] = v;
        amax = fmaxf(amax, fabsf(v));
    }
    amax = block_max(amax, red);
    const float scale = quant_scale_from_absmax(amax);
    const float inv = __frcp_rn(scale);
    const int tail_start = K & ~15;
    for (int k = tid; k < K; k += kMoeThreads) {
        int q;
        if (k < tail_start) {
            q = (int)quant_rne_sat(__fmul_rn(vs[k], inv));
        } else {
            q = max(-127, min(127, (int)roundf(__fmul_rn(vs[k], inv))));
        }
        out[(size_t)r * K + k] = (int8_t)q;
    }
    if (tid == 0) scales[r] = scale;
}

__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ selw,
                                   int H) {
    grid_dependency_launch();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const float w0 = selw[2 * t], w1 = selw[2 * t + 1];
    const float* y0 = y + (size_t)(2 * t) * H;
    const float* y1 = y0 + H;
    for (int k = threadIdx.x; k < H; k += blockDim.x)
        x[(size_t)t * H + k] = __fadd_rn(x[(size_t)t * H + k], __fadd_rn(__fmul_rn(w0, y0[k]), __fmul_rn(w1, y1[k])));
}

static int moe_alloc(void** p, size_t bytes, Moe* m) {
    LSPK_CUDA(cudaMalloc(p, bytes ? bytes : 16));
    m->bytes += bytes;
    return LSPK_OK;
}

// Make the per-call scratch large enough for B token rows (allocates; call before any graph capture).
int moe_reserve(Moe* m, int B) {
    if (B <= m->cap_B) return LSPK_OK;
    void* old[] = {m->xq, m->xq2, m->xs, m->xs2, m->selw, m->inter, m->ydown, m->sel, m->counts, m->rows};
    for (void* p : old) cudaFree(p);
    const size_t R = 2 * (size_t)B;
    int rc = 0;
    rc |= moe_alloc((void**)&m->xq, (size_t)B * m->H, m);
    rc |= moe_alloc((void**)&m->xs, (size_t)B * 4, m);
    rc |= moe_alloc((void**)&m->sel, R * 4, m);
    rc |= moe_alloc((void**)&m->selw, R * 4, m);
    rc |= moe_alloc((void**)&m->counts, (size_t)m->E * 4, m);
    rc |= moe_alloc((void**)&m->rows, (size_t)m->E * R * 4, m);
    rc |= moe_alloc((void**)&m->inter, R * m->I * 4, m);
    rc |= moe_alloc((void**)&m->xq2, R * m->I, m);
    rc |= moe_alloc((void**)&m->xs2, R * 4, m);
    rc |= moe_alloc((void**)&m->ydown, R * m->H * 4, m);
    if (rc) return rc;
    m->cap_B = B;
    return LSPK_OK;
}

int moe_forward(Moe* m, float* x, int B, int32_t* sel_out, float* selw_out, int32_t* acc_gate, int32_t* acc_up,
                int32_t* acc_down) {
    LSPK_REQUIRE(m && x && B >= 1, "moe_forward: bad arguments");
    if (int rc = moe_reserve(m, B)) return rc;
    const int H = m->H, I = m->I, E = m->E, R = 2 * B;
    static bool attr_set = false;
    if (!attr_set) {
        LSPK_CUDA(cudaFuncSetAttribute(moe_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(moe_subnorm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set = true;
    }
    LSPK_CUDA(launch(moe_router_kernel, dim3(B), dim3(kMoeThreads), (size_t)H * 4, true, (const float*)x,
                     (const uint16_t*)m->norm, (const float*)m->router, m->xq, m->xs, m->sel, m->selw, H, E, m->eps));
    LSPK_CUDA(launch(moe_group_kernel, dim3(1), dim3(32), 0, true, (const int*)m->sel, R, E, m->counts, m->rows, R));

    const int ctas = 2 * sm_count() / (E < 4 ? E : 4);     // a few experts are active; keep each one's grid wide
    LinearParams p = {};
    p.trace = nullptr;
    p.prologue = LSPK_PRO_INT8;
    p.stream_weights = 0;
    p.grp_counts = m->counts;
    p.grp_rows = m->rows;
    p.grp_rows_stride = R;
    p.grp_w_stride = 3 * m->mat_stride;
    p.grp_scales = m->scales;
    p.M = R;
    // gate / up
    p.K = H;
    p.chunks = m->chunks_gu;
    p.n_seg = 2;
    p.total_groups = m->groups_gu;
    p.epilogue = LSPK_EPI_RELU2_MUL;
    p.seg[0] = LinearSeg{m->w, m->inter, acc_gate, I, m->groups_gu, 1.0f, 0};
    p.seg[1] = LinearSeg{m->w + m->mat_stride, nullptr, acc_up, I, m->groups_gu, 1.0f, 1};
    p.x_i8 = m->xq;
    p.x_scales = m->xs;
    p.grp_in_shift = 1;                // routed row 2*token + slot reads token's activations
    if (int rc = linear_launch_params(p, 8, true, true, ctas < m->groups_gu ? ctas : m->groups_gu, 1, E)) return rc;
    // SubLN + quantiser per routed row, with the row's expert's norm weights
    LSPK_CUDA(launch(moe_subnorm_quant_kernel, dim3(R), dim3(kMoeThreads), (size_t)I * 4, true, (const float*)m->inter,
                     (const int*)m->sel, (const uint16_t*)m->sub_norm, m->xq2, m->xs2, I, m->eps));
    // down
    p.K = I;
    p.chunks = m->chunks_d;
    p.n_seg = 1;
    p.total_groups = m->groups_d;
    p.epilogue = LSPK_EPI_STORE;
    p.seg[0] = LinearSeg{m->w + 2 * m->mat_stride, m->ydown, acc_down, H, m->groups_d, 1.0f, 2};
    p.x_i8 = m->xq2;
    p.x_scales = m->xs2;
    p.grp_in_shift = 0;
    if (int rc = linear_launch_params(p, 8, false, true, ctas < m->groups_d ? ctas : m->groups_d, 1, E)) return rc;
    LSPK_CUDA(launch(moe_combine_kernel, dim3(B), dim3(256), 0, true, x, (const float*)m->ydown, (const float*)m->selw, H));
    if (sel_out) LSPK_CUDA(cudaMemcpyAsync(sel_out, m->sel, (size_t)R * 4, cudaMemcpyDeviceToDevice, stream()));
    if (selw_out) LSPK_CUDA(cudaMemcpyAsync(selw_out, m->selw, (size_t)R * 4, cudaMemcpyDeviceToDevice, stream()));
    return LSPK_OK;
}

}  // namespace lspk

using namespace lspk;

extern "C" {

lspk_moe_t lspk_moe_create(int n_experts, int hidden, int inter, const uint8_t* experts_packed_host,
                           const float* scales_host, const float* router_host, const uint16_t* norm_gamma_host,
                           const uint16_t* sub_norm_gamma_host, float eps) {
    if (ensure_init()) return nullptr;
    if (n_experts < 2 || n_experts > kMaxExperts || hidden < 4 || inter < 4 || (hidden & 3) || (inter & 3) ||
        !experts_packed_host || !scales_host || !router_host || !norm_gamma_host || !sub_norm_gamma_host) {
        fail(LSPK_ERR_ARG, "lspk_moe_create: bad arguments (experts=%d hidden=%d inter=%d)", n_experts, hidden, inter);
        return nullptr;
    }
    Moe* m = new Moe();
    m->E = n_experts;
    m->H = hidden;
    m->I = inter;
    m->eps = eps;
    m->groups_gu = (inter + kRowsPerGroup - 1) / kRowsPerGroup;
    m->chunks_gu = (hidden + kWeightsPerChunk - 1) / kWeightsPerChunk;
    m->groups_d = (hidden + kRowsPerGroup - 1) / kRowsPerGroup;
    m->chunks_d = (inter + kWeightsPerChunk - 1) / kWeightsPerChunk;
    const size_t gu_chunks = (size_t)m->groups_gu * m->chunks_gu * kRowsPerGroup;
    const size_t d_chunks = (size_t)m->groups_d * m->chunks_d * kRowsPerGroup;
    m->mat_stride = gu_chunks > d_chunks ? gu_chunks : d_chunks;
    const size_t host_mat = (size_t)inter * hidden / 4;
    uint8_t* staging = nullptr;
    cudaError_t e = cudaMalloc((void**)&m->w, (size_t)n_experts * 3 * m->mat_stride * 16);
    if (e == cudaSuccess) e = cudaMalloc((void**)&staging, host_mat);
    for (int ex = 0; ex < n_experts && e == cudaSuccess; ++ex) {
        for (int which = 0; which < 3 && e == cudaSuccess; ++which) {
            const uint8_t* src = experts_packed_host + ((size_t)ex * 3 + which) * host_mat;
            e = cudaMemcpyAsync(staging, src, host_mat, cudaMemcpyHostToDevice, stream());
            uint4* dst = m->w + ((size_t)ex * 3 + which) * m->mat_stride;
            if (e == cudaSuccess)
                e = which < 2 ? retile_to_device_launch(staging, dst, inter, hidden / 4, m->groups_gu, m->chunks_gu)
                              : retile_to_device_launch(staging, dst, hidden, inter / 4, m->groups_d, m->chunks_d);
            if (e == cudaSuccess) e = cudaStreamSynchronize(stream());
        }
    }
    if (staging) cudaFree(staging);
    m->bytes = (size_t)n_experts * 3 * m->mat_stride * 16;
    auto up = [&](void** dst, const void* src, size_t bytes) {
        if (e != cudaSuccess) return;
        e = cudaMalloc(dst, bytes);
        if (e == cudaSuccess) e = cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice);
        m->bytes += bytes;
    };
    up((void**)&m->scales, scales_host, (size_t)n_experts * 3 * 4);
    up((void**)&m->router, router_host, (size_t)n_experts * hidden * 4);
    up((void**)&m->norm, norm_gamma_host, (size_t)hidden * 2);
    up((void**)&m->sub_norm, sub_norm_gamma_host, (size_t)n_experts * inter * 2);
    if (e != cudaSuccess) {
        fail(LSPK_ERR_CUDA, "lspk_moe_create: %s", cudaGetErrorString(e));
        lspk_moe_free(reinterpret_cast<lspk_moe_t>(m));
        return nullptr;
    }
    return reinterpret_cast<lspk_moe_t>(m);
}

int lspk_moe_free(lspk_moe_t h) {
    if (!h) return LSPK_OK;
    Moe* m = reinterpret_cast<Moe*>(h);
    cudaStreamSynchronize(stream());
    void* dev[] = {m->w, m->scales, m->router, m->norm, m->sub_norm, m->xq, m->xq2, m->xs, m->xs2, m->selw,
                   m->inter, m->ydown, m->sel, m->counts, m->rows};
    for (void* p : dev) cudaFree(p);
    delete m;
    return LSPK_OK;
}

size_t lspk_moe_device_bytes(lspk_moe_t h) { return h ? reinterpret_cast<Moe*>(h)->bytes : 0; }

int lspk_moe_forward(lspk_moe_t h, float* x_dev, int B, int32_t* sel_out, float* selw_out, int32_t* acc_gate_out,
                     int32_t* acc_up_out, int32_t* acc_down_out) {
    if (int rc = ensure_init()) return rc;
    return moe_forward(reinterpret_cast<Moe*>(h), x_dev, B, sel_out, selw_out, acc_gate_out, acc_up_out, acc_down_out);
}

}  // extern "C"
