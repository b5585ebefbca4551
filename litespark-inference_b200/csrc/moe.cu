// Packed-expert ternary MoE layer (top-2 softmax router, squared-ReLU experts).
//
// No counterpart in the reference.  Per token:  h = RMSNorm(x);  p = softmax(Wr h);  the two largest
// p (ties to the lower index) renormalised to sum one;  for each routed expert e:
// y_e = down_e(quant(SubLN_e(relu(gate_e q)^2 * up_e q))), q = quant(h) computed once;
// x += w_0 y_0 + w_1 y_1.
//
// Kernel sequence (all on the library stream, no host synchronisation):
//   moe_router_kernel        one CTA per token: norm, quantise, router logits, softmax, top-2
//   moe_group_kernel         rows (token, slot) listed per expert, ascending (more than one token;
//                            the router kernel lists a single token's two rows itself)
//   ternary_linear_mma_kernel expert-grouped launch, gate/up pair, ReLU^2 epilogue  (grid.z = expert)
//   row_norm_quant_kernel    per routed row: RMSNorm with the row's expert's weights + quantiser
//   ternary_linear_mma_kernel expert-grouped launch, down projection
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

// One CTA per token row: RMSNorm, quantiser, router logits (one warp per expert, round-robin), softmax
// and top-2 inside warp 0.  With a single token (gridDim.x == 1) the per-expert row lists are written
// here as well, which saves the grouping kernel.  H is a multiple of 4 (checked at creation).
__global__ void __launch_bounds__(kMoeThreads)
moe_router_kernel(const float* __restrict__ x, const uint16_t* __restrict__ gamma, const float* __restrict__ router,
                  int8_t* __restrict__ xq, float* __restrict__ xs, int* __restrict__ sel, float* __restrict__ selw,
                  int* __restrict__ counts, int* __restrict__ rows, int rows_stride, int H, int E, float eps) {
    extern __shared__ __align__(16) float hs[];           // [H] normalised row
    __shared__ __align__(16) float red[16];
    __shared__ float s_logit[kMaxExperts];
    grid_dependency_launch();
    grid_dependency_wait();
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int H4 = H >> 2;
    const float4* src4 = reinterpret_cast<const float4*>(x + (size_t)t * H);
    float4* hs4 = reinterpret_cast<float4*>(hs);
    float ssq = 0.0f;
    for (int i = tid; i < H4; i += kMoeThreads) {
        const float4 v = src4[i];
        hs4[i] = v;
        ssq = fmaf(v.x, v.x, ssq);
        ssq = fmaf(v.y, v.y, ssq);
        ssq = fmaf(v.z, v.z, ssq);
        ssq = fmaf(v.w, v.w, ssq);
    }
    ssq = warp_sum(ssq);
    if (lane == 0) red[warp] = ssq;
    __syncthreads();
    {
        const float4 a = *reinterpret_cast<const float4*>(red), b = *reinterpret_cast<const float4*>(red + 4);
        ssq = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
    }
    const float rrms = rcp_rn(__fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, (float)H), eps)));
    float amax = 0.0f;
    for (int i = tid; i < H4; i += kMoeThreads) {
        float4 v = hs4[i];
        const uint2 gb = *reinterpret_cast<const uint2*>(gamma + 4 * i);
        v.x = __fmul_rn(__fmul_rn(v.x, rrms), __uint_as_float(gb.x << 16));
        v.y = __fmul_rn(__fmul_rn(v.y, rrms), __uint_as_float(gb.x & 0xffff0000u));
        v.z = __fmul_rn(__fmul_rn(v.z, rrms), __uint_as_float(gb.y << 16));
        v.w = __fmul_rn(__fmul_rn(v.w, rrms), __uint_as_float(gb.y & 0xffff0000u));
        hs4[i] = v;
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    {
        const uint32_t u = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
        if (lane == 0) red[8 + warp] = __uint_as_float(u);
        __syncthreads();                                   // also publishes the normalised row
        const float4 a = *reinterpret_cast<const float4*>(red + 8), b = *reinterpret_cast<const float4*>(red + 12);
        amax = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
    }
    const float scale = quant_scale_from_absmax(amax);
    const float inv = rcp_rn(scale);
    const int tail_start = H & ~15;
    uint32_t* xq4 = reinterpret_cast<uint32_t*>(xq + (size_t)t * H);
    for (int i = tid; i < H4; i += kMoeThreads) {
        const float4 v = hs4[i];
        const float f[4] = {v.x, v.y, v.z, v.w};
        uint32_t word = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            int q;
            if (4 * i < tail_start) q = (int)quant_rne_sat(__fmul_rn(f[e], inv));
            else q = max(-127, min(127, (int)roundf(__fmul_rn(f[e], inv))));
            word |= ((uint32_t)q & 0xffu) << (8 * e);
        }
        xq4[i] = word;
    }
    if (tid == 0) xs[t] = scale;
    // router logits: warp w takes experts w, w + 8, ...
    for (int e = warp; e < E; e += kMoeThreads / 32) {
        const float4* wr4 = reinterpret_cast<const float4*>(router + (size_t)e * H);
        float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        for (int i = lane; i < H4; i += 32) {
            const float4 h = hs4[i], w = __ldg(wr4 + i);
            a0 = fmaf(h.x, w.x, a0);
            a1 = fmaf(h.y, w.y, a1);
            a2 = fmaf(h.z, w.z, a2);
            a3 = fmaf(h.w, w.w, a3);
        }
        const float acc = warp_sum((a0 + a1) + (a2 + a3));
        if (lane == 0) s_logit[e] = acc;
    }
    __syncthreads();
    if (warp == 0) {
        // softmax over the experts (E <= 32: one lane each), then the two largest (ties to the lower index)
        const bool valid = lane < E;
        const float l = valid ? s_logit[lane] : -INFINITY;
        const float mx = warp_max(l);
        const float ex = valid ? expf(l - mx) : 0.0f;
        const float sum = warp_sum(ex);
        const float pe = valid ? __fdiv_rn(ex, sum) : 0.0f;
        // probabilities are in [0, 1]: bits + 1 orders them and leaves 0 for "no candidate"
        const uint32_t key = valid ? __float_as_uint(pe) + 1u : 0u;
        const uint32_t k0 = __reduce_max_sync(0xffffffffu, key);
        const int i0 = (int)__reduce_min_sync(0xffffffffu, key == k0 ? (uint32_t)lane : 32u);
        const uint32_t key1 = lane == i0 ? 0u : key;
        const uint32_t k1 = __reduce_max_sync(0xffffffffu, key1);
        const int i1 = (int)__reduce_min_sync(0xffffffffu, (key1 == k1 && lane != i0) ? (uint32_t)lane : 32u);
        const float p0 = __shfl_sync(0xffffffffu, pe, i0), p1 = __shfl_sync(0xffffffffu, pe, i1);
        const float den = __fadd_rn(p0, p1);
        if (lane == 0) {
            sel[2 * t] = i0;
            sel[2 * t + 1] = i1;
            selw[2 * t] = __fdiv_rn(p0, den);
            selw[2 * t + 1] = __fdiv_rn(p1, den);
        }
        if (gridDim.x == 1 && valid) {
            // single token: routed row 0 goes to expert i0, routed row 1 to expert i1
            counts[lane] = (lane == i0 || lane == i1) ? 1 : 0;
            if (lane == i0) rows[(size_t)lane * rows_stride] = 0;
            if (lane == i1) rows[(size_t)lane * rows_stride] = 1;
        }
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
    void** old[] = {(void**)&m->xq, (void**)&m->xq2, (void**)&m->xs, (void**)&m->xs2, (void**)&m->selw,
                    (void**)&m->inter, (void**)&m->ydown, (void**)&m->sel, (void**)&m->counts, (void**)&m->rows};
    for (void** p : old) {
        cudaFree(*p);
        *p = nullptr;
    }
    m->cap_B = 0;               // nothing is held until every buffer below exists
    scratch_moved();
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
        attr_set = true;
    }
    LSPK_CUDA(launch(moe_router_kernel, dim3(B), dim3(kMoeThreads), (size_t)H * 4, true, (const float*)x,
                     (const uint16_t*)m->norm, (const float*)m->router, m->xq, m->xs, m->sel, m->selw, m->counts, m->rows, R,
                     H, E, m->eps));
    if (B > 1)      // a single token's two rows are listed by the router kernel itself
        LSPK_CUDA(launch(moe_group_kernel, dim3(1), dim3(32), 0, true, (const int*)m->sel, R, E, m->counts, m->rows, R));

    if (B == 1) {
        // A single token: its two experts' products are one-row products whose matrices the router has just chosen.
        // Both experts of a stage go through ONE launch of the streamed batch (linear_stream.cu), which reads the
        // expert indices on the device; same integer arithmetic as the eight-row kernel, so the same bits.
        static StreamParams sp;
        sp.n = 2;
        for (int slot = 0; slot < 2; ++slot) {
            StreamItem& it = sp.it[slot];
            it = StreamItem{};
            it.w[0] = m->w;
            it.w[1] = m->w + m->mat_stride;
            it.sel = m->sel + slot;
            it.sel_stride = 3 * m->mat_stride;
            it.sel_scales = m->scales;
            it.scale_idx[0] = 0;
            it.scale_idx[1] = 1;
            it.out = m->inter + (size_t)slot * I;
            it.acc[0] = acc_gate ? acc_gate + (size_t)slot * I : nullptr;
            it.acc[1] = acc_up ? acc_up + (size_t)slot * I : nullptr;
            it.x = m->xq;
            it.xs = m->xs;
            it.N = I;
            it.K = H;
            it.chunks = m->chunks_gu;
            it.groups = m->groups_gu;
            it.nm = 2;
            it.epilogue = LSPK_EPI_RELU2_MUL;
        }
        if (int rc = stream_launch(&sp)) return rc;
        if (int rc = norm_quant_rows_selected(m->inter, m->sub_norm, m->sel, m->xq2, m->xs2, R, I, m->eps)) return rc;
        for (int slot = 0; slot < 2; ++slot) {
            StreamItem& it = sp.it[slot];
            it = StreamItem{};
            it.w[0] = m->w + 2 * m->mat_stride;
            it.sel = m->sel + slot;
            it.sel_stride = 3 * m->mat_stride;
            it.sel_scales = m->scales;
            it.scale_idx[0] = 2;
            it.scale_idx[1] = 2;
            it.out = m->ydown + (size_t)slot * H;
            it.acc[0] = acc_down ? acc_down + (size_t)slot * H : nullptr;
            it.x = m->xq2 + (size_t)slot * I;
            it.xs = m->xs2 + slot;
            it.N = H;
            it.K = I;
            it.chunks = m->chunks_d;
            it.groups = m->groups_d;
            it.nm = 1;
            it.epilogue = LSPK_EPI_STORE;
        }
        if (int rc = stream_launch(&sp)) return rc;
        LSPK_CUDA(launch(moe_combine_kernel, dim3(B), dim3(256), 0, true, x, (const float*)m->ydown, (const float*)m->selw, H));
        if (sel_out) LSPK_CUDA(cudaMemcpyAsync(sel_out, m->sel, (size_t)R * 4, cudaMemcpyDeviceToDevice, stream()));
        if (selw_out) LSPK_CUDA(cudaMemcpyAsync(selw_out, m->selw, (size_t)R * 4, cudaMemcpyDeviceToDevice, stream()));
        return LSPK_OK;
    }

    // At most min(E, R) experts have rows; CTAs of the others leave at once.  Two resident CTAs per SM
    // over the experts that can be active keeps enough weight bytes in flight.
    const int active = E < R ? E : R;
    int ctas = (2 * sm_count() + active - 1) / active;
    // The expert products stream tens of megabytes per launch: the weights go through the bulk-copy ring of the
    // eight-row kernel, three stages deep where they fit.  CTAs per SM follow from the ring's size.
    const int knob_bulk = 3;
    auto bulk_ctas = [&](int chunks, bool pair, int Kp, int* stages) -> int {
        int st = knob_bulk > 4 ? 4 : knob_bulk;
        const size_t stage = (size_t)chunks * 256 * (pair ? 2 : 1);
        const size_t base = (size_t)8 * mma_row_stride(Kp) + (size_t)8 * 8 * 16 * (pair ? 2 : 1) * 4 + 8 * 8 + 64 + 256;
        while (st > 1 && base + st * stage > 110 * 1024) --st;
        *stages = st;
        const size_t smem = base + st * stage + 1024;
        int per_sm = (int)((227 * 1024) / smem);
        if (per_sm < 1) per_sm = 1;
        if (per_sm > 3) per_sm = 3;
        return (per_sm * sm_count() + active - 1) / active;
    };
    LinearParams p = {};
    p.error_flag = device_wait_flag();
    p.trace = trace_buffer();
    p.trace_cap = trace_capacity();
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
    if (knob_bulk > 0) ctas = bulk_ctas(p.chunks, true, p.chunks * kWeightsPerChunk, &p.bulk_stages);
    if (int rc = linear_launch_params(p, 8, true, true, ctas < m->groups_gu ? ctas : m->groups_gu, 1, E)) return rc;
    // SubLN + quantiser per routed row, with the row's expert's norm weights
    if (int rc = norm_quant_rows_selected(m->inter, m->sub_norm, m->sel, m->xq2, m->xs2, R, I, m->eps)) return rc;
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
    if (knob_bulk > 0) ctas = bulk_ctas(p.chunks, false, p.chunks * kWeightsPerChunk, &p.bulk_stages);
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
