// Mamba-2 selective-state-update decode step (one group, depthwise conv of width 4).
//
// No counterpart in the reference.  Per sequence and step:
//   zxbcdt = in_proj(quant(RMSNorm(x)))                       ternary linear, fused prologue
//   xBC    = SiLU(conv1d_step(xBC) + bias)                     ring of the last four conv inputs
//   dt = softplus(dt + dt_bias);  dA = exp(dt * A_h)
//   state[h,p,n] = state * dA + (dt * x[h,p]) * B[n];  y[h,p] = sum_n state * C[n] + D_h * x[h,p]
//   out = out_proj(quant(RMSNorm(y * SiLU(z))));  x += out      ternary linear, residual epilogue
// The state update is the HBM-bound part: the fp32 state [heads, head_dim, d_state] (2.6 MB per
// sequence and layer at 80 x 64 x 128) is read and written once per step.  One CTA owns half a head (32 rows of
// 128 states, 16 KB in and out; grid = 2 * heads x sequences) or, for four and more sequences, a whole head.
#include "internal.cuh"
#include "../../include/lspk_hybrid.h"

namespace lspk {

struct Mamba {
    lspk_mamba_config cfg;
    int d_inner = 0, conv_dim = 0, in_out = 0;
    lspk_weight_t in_proj = nullptr, out_proj = nullptr;
    float *conv_w = nullptr, *conv_b = nullptr, *A = nullptr, *dt_bias = nullptr, *D = nullptr;
    uint16_t *norm = nullptr, *gnorm = nullptr;
    int cap_B = 0;
    float *zx = nullptr, *v = nullptr;      // [B][in_out], [B][d_inner]
    size_t bytes = 0;
    size_t state_floats() const { return (size_t)conv_dim * 4 + (size_t)cfg.nheads * cfg.headdim * cfg.d_state; }
};

__device__ __forceinline__ float silu_f(float v) { return __fdiv_rn(v, __fadd_rn(expf(-v), 1.0f)); }

// P = head_dim = 64, N = d_state = 128.  A CTA of 256 threads owns ROWS rows of one head (32: half a head, grid
// 2 * heads x sequences; 64: a whole head, grid heads x sequences); 8 threads share a row, a thread holds 16 state
// values of each of its ROWS / 32 rows.  Whole-head CTAs keep twice the state bytes in flight per thread and run
// the B / C convolution once per head instead of twice: the form for several sequences, where the launch is bound
// by HBM; with one sequence the half-head form covers more SMs.  Same arithmetic per element in both.
template <int ROWS>
__global__ void __launch_bounds__(256, ROWS == 64 ? 4 : 1)
mamba2_ssu_kernel(const float* __restrict__ zx, float* __restrict__ state, const int* __restrict__ pos_ptr,
                  const float* __restrict__ conv_w, const float* __restrict__ conv_b, const float* __restrict__ A,
                  const float* __restrict__ dt_bias, const float* __restrict__ Dskip, float* __restrict__ vout,
                  int d_inner, int conv_dim, int in_out, size_t state_floats) {
    constexpr int P = 64, N = 128, RS = ROWS / 32;       // RS: rows per thread
    static_assert(ROWS == 32 || ROWS == 64, "a CTA owns half a head or a whole one");
    __shared__ float xs_s[ROWS];
    // B and C with four floats of padding after every 16: the eight threads of a row read 16-byte pieces 80 bytes
    // apart, which fall into eight different bank groups (64 bytes apart they collide four ways)
    constexpr int NPAD = N + N / 16 * 4;
    __shared__ __align__(16) float B_s[NPAD];
    __shared__ __align__(16) float C_s[NPAD];
    const int b = blockIdx.y, hh = blockIdx.x, head = ROWS == 64 ? hh : hh >> 1, p0 = ROWS == 64 ? 0 : (hh & 1) * ROWS;
    const int tid = threadIdx.x;
    grid_dependency_launch();
    grid_dependency_wait();
    // This thread's state values are requested first thing after the dependency wait, ahead of the convolution's
    // loads, so that their trip to HBM (16 KB per 32 rows each way, the bulk of the bytes) runs under the
    // convolution.  Not before the wait: the state was written by this kernel one decode step ago, and with
    // programmatic launch nothing orders code in front of the wait after a kernel that is not the direct
    // predecessor (in a short chain -- a single layer stepped in a loop -- that kernel may still be running).
    float4 st[RS][4];
    float4* srow[RS];
    {
        float* ssm0 = state + (size_t)b * state_floats + (size_t)conv_dim * 4;
#pragma unroll
        for (int rr = 0; rr < RS; ++rr) {
            srow[rr] = reinterpret_cast<float4*>(ssm0 + ((size_t)(head * P + p0 + 32 * rr + (tid >> 3)) * N + (tid & 7) * 16));
#pragma unroll
            for (int q = 0; q < 4; ++q) st[rr][q] = srow[rr][q];
        }
    }
    const float* zrow = zx + (size_t)b * in_out;
    const float* xbc_raw = zrow + d_inner;
    const float* dt_raw = zrow + d_inner + conv_dim;
    float* ring = state + (size_t)b * state_floats;              // [conv_dim][4]
    // behind the ring: the state matrices [heads][P][N] (srow above)
    const int pos = pos_ptr[b];
    const int slot = pos & 3;
    // per-head scalars and this thread's gate inputs: requested here so that their round trip overlaps the
    // convolution's (they are used after the barrier below)
    const float dt_in = dt_raw[head], dt_b = dt_bias[head], a_head = A[head], d_head = Dskip[head];
    float z_gate[RS];
#pragma unroll
    for (int rr = 0; rr < RS; ++rr) z_gate[rr] = (tid & 7) == 0 ? zrow[head * P + p0 + 32 * rr + (tid >> 3)] : 0.0f;

    // depthwise conv step + SiLU for the channels this CTA needs: its ROWS x-channels, all of B and C.  A thread
    // takes channel index tid and, the first ROWS + 2 N - 256 threads, a second one; everything both need (the
    // newest input, the bias, the four taps as one 16-byte load, the four ring slots as another) is requested
    // before either is computed, so the two cost one trip to memory, not two.
    constexpr int NCH2 = ROWS + 2 * N - 256;     // channels beyond one per thread
    static_assert(NCH2 > 0 && NCH2 <= 256, "one or two channels per thread");
    const bool second = tid < NCH2;
    int cch[2];
    float newv[2], bias[2];
    float4 taps[2], hist[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        const int idx = tid + 256 * k;
        cch[k] = idx < ROWS ? head * P + p0 + idx : d_inner + (idx - ROWS);
        if (k == 0 || second) {
            newv[k] = xbc_raw[cch[k]];
            bias[k] = conv_b[cch[k]];
            taps[k] = *reinterpret_cast<const float4*>(conv_w + (size_t)cch[k] * 4);
            hist[k] = *reinterpret_cast<const float4*>(ring + (size_t)cch[k] * 4);
        }
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
        if (k == 0 || second) {
            const int idx = tid + 256 * k;
            const float h4[4] = {hist[k].x, hist[k].y, hist[k].z, hist[k].w};
            const float w4[4] = {taps[k].x, taps[k].y, taps[k].z, taps[k].w};
            float acc = bias[k];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int sl = (pos - 3 + j) & 3;
                const float hv = sl == 0 ? h4[0] : sl == 1 ? h4[1] : sl == 2 ? h4[2] : h4[3];
                acc = __fadd_rn(acc, __fmul_rn(w4[j], hv));
            }
            acc = __fadd_rn(acc, __fmul_rn(w4[3], newv[k]));
            const float act = silu_f(acc);
            if (idx < ROWS) xs_s[idx] = act;
            else if (idx < ROWS + N) B_s[(idx - ROWS) + ((idx - ROWS) >> 4) * 4] = act;
            else C_s[(idx - ROWS - N) + ((idx - ROWS - N) >> 4) * 4] = act;
            // the newest input replaces the oldest slot; nobody reads that slot during this step
            if (idx < ROWS || hh == 0) ring[(size_t)cch[k] * 4 + slot] = newv[k];
        }
    }
    __syncthreads();

    const float dv = __fadd_rn(dt_in, dt_b);
    const float dt = dv > 20.0f ? dv : log1pf(expf(dv));
    const float dA = expf(__fmul_rn(dt, a_head));
    const int seg = tid & 7;
#pragma unroll
    for (int rr = 0; rr < RS; ++rr) {
        const int p = 32 * rr + (tid >> 3);
        const float xv = xs_s[p];
        const float dtx = __fmul_rn(dt, xv);
        float ysum = 0.0f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 Bv = *reinterpret_cast<const float4*>(B_s + seg * 20 + q * 4);
            const float4 Cv = *reinterpret_cast<const float4*>(C_s + seg * 20 + q * 4);
            float4 s4 = st[rr][q];
            s4.x = __fadd_rn(__fmul_rn(s4.x, dA), __fmul_rn(dtx, Bv.x));
            s4.y = __fadd_rn(__fmul_rn(s4.y, dA), __fmul_rn(dtx, Bv.y));
            s4.z = __fadd_rn(__fmul_rn(s4.z, dA), __fmul_rn(dtx, Bv.z));
            s4.w = __fadd_rn(__fmul_rn(s4.w, dA), __fmul_rn(dtx, Bv.w));
            ysum = fmaf(s4.x, Cv.x, ysum);
            ysum = fmaf(s4.y, Cv.y, ysum);
            ysum = fmaf(s4.z, Cv.z, ysum);
            ysum = fmaf(s4.w, Cv.w, ysum);
            srow[rr][q] = s4;
        }
        ysum += __shfl_xor_sync(0xffffffffu, ysum, 4);
        ysum += __shfl_xor_sync(0xffffffffu, ysum, 2);
        ysum += __shfl_xor_sync(0xffffffffu, ysum, 1);
        if (seg == 0) {
            const int ch = head * P + p0 + p;
            const float y = __fadd_rn(ysum, __fmul_rn(d_head, xv));
            vout[(size_t)b * d_inner + ch] = __fmul_rn(y, silu_f(z_gate[rr]));
        }
    }
}

size_t mamba_state_floats(const Mamba* m) { return m->state_floats(); }

int mamba_reserve(Mamba* m, int B) {
    if (B <= m->cap_B) return LSPK_OK;
    cudaFree(m->zx);
    cudaFree(m->v);
    m->zx = m->v = nullptr;
    m->cap_B = 0;
    scratch_moved();
    LSPK_CUDA(cudaMalloc((void**)&m->zx, (size_t)B * m->in_out * 4));
    LSPK_CUDA(cudaMalloc((void**)&m->v, (size_t)B * m->d_inner * 4));
    m->bytes += (size_t)B * (m->in_out + m->d_inner) * 4;
    m->cap_B = B;
    return LSPK_OK;
}

int mamba_step(Mamba* m, float* x, float* state, const int* pos, int B) {
    LSPK_REQUIRE(m && x && state && pos && B >= 1, "mamba_step: bad arguments");
    LSPK_REQUIRE((reinterpret_cast<uintptr_t>(state) & 15) == 0, "mamba_step: the state buffer must be 16-byte aligned");
    if (int rc = mamba_reserve(m, B)) return rc;
    lspk_linear_args a = {};
    a.w[0] = m->in_proj;
    a.out[0] = m->zx;
    a.n_mats = 1;
    a.M = B;
    a.prologue = LSPK_PRO_RMSNORM_QUANT;
    a.epilogue = LSPK_EPI_STORE;
    a.x_f32 = x;
    a.gamma = m->norm;
    a.gamma_is_bf16 = 1;
    a.eps = m->cfg.eps;
    // several rows: linear_cuda_core quantises them once, straight into the eight-row kernel's tile layout
    if (int rc = linear_cuda_core(&a)) return rc;
    if (B >= 4)
        LSPK_CUDA(launch(mamba2_ssu_kernel<64>, dim3(m->cfg.nheads, B), dim3(256), 0, true, (const float*)m->zx, state, pos,
                         (const float*)m->conv_w, (const float*)m->conv_b, (const float*)m->A, (const float*)m->dt_bias,
                         (const float*)m->D, m->v, m->d_inner, m->conv_dim, m->in_out, m->state_floats()));
    else
        LSPK_CUDA(launch(mamba2_ssu_kernel<32>, dim3(m->cfg.nheads * 2, B), dim3(256), 0, true, (const float*)m->zx, state, pos,
                         (const float*)m->conv_w, (const float*)m->conv_b, (const float*)m->A, (const float*)m->dt_bias,
                         (const float*)m->D, m->v, m->d_inner, m->conv_dim, m->in_out, m->state_floats()));
    lspk_linear_args o = {};
    o.w[0] = m->out_proj;
    o.out[0] = x;
    o.n_mats = 1;
    o.M = B;
    o.prologue = LSPK_PRO_RMSNORM_QUANT;
    o.epilogue = LSPK_EPI_ADD;
    o.x_f32 = m->v;
    o.gamma = m->gnorm;
    o.gamma_is_bf16 = 1;
    o.eps = m->cfg.eps;
    return linear_cuda_core(&o);
}

}  // namespace lspk

using namespace lspk;

extern "C" {

lspk_mamba_t lspk_mamba_create(const lspk_mamba_config* cfg, const uint8_t* in_proj_packed, float in_scale,
                               const uint8_t* out_proj_packed, float out_scale, const float* conv_w,
                               const float* conv_b, const float* A, const float* dt_bias, const float* D,
                               const uint16_t* norm_gamma, const uint16_t* gated_norm_gamma) {
    if (ensure_init()) return nullptr;
    if (!cfg || !in_proj_packed || !out_proj_packed || !conv_w || !conv_b || !A || !dt_bias || !D || !norm_gamma ||
        !gated_norm_gamma) {
        fail(LSPK_ERR_ARG, "lspk_mamba_create: null argument");
        return nullptr;
    }
    if (cfg->headdim != 64 || cfg->d_state != 128 || cfg->conv_width != 4 || cfg->nheads < 1 || cfg->hidden < 4 ||
        (cfg->hidden & 3)) {
        fail(LSPK_ERR_ARG, "lspk_mamba_create: this kernel is built for head_dim 64, d_state 128, conv width 4");
        return nullptr;
    }
    Mamba* m = new Mamba();
    m->cfg = *cfg;
    m->d_inner = cfg->nheads * cfg->headdim;
    m->conv_dim = m->d_inner + 2 * cfg->d_state;
    m->in_out = 2 * m->d_inner + 2 * cfg->d_state + cfg->nheads;
    m->in_proj = lspk_upload_packed(in_proj_packed, m->in_out, cfg->hidden, in_scale);
    m->out_proj = lspk_upload_packed(out_proj_packed, cfg->hidden, m->d_inner, out_scale);
    cudaError_t e = (m->in_proj && m->out_proj) ? cudaSuccess : cudaErrorMemoryAllocation;
    auto up = [&](void** dst, const void* src, size_t bytes) {
        if (e != cudaSuccess) return;
        e = cudaMalloc(dst, bytes);
        if (e == cudaSuccess) e = cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice);
        m->bytes += bytes;
    };
    up((void**)&m->conv_w, conv_w, (size_t)m->conv_dim * 4 * 4);
    up((void**)&m->conv_b, conv_b, (size_t)m->conv_dim * 4);
    up((void**)&m->A, A, (size_t)cfg->nheads * 4);
    up((void**)&m->dt_bias, dt_bias, (size_t)cfg->nheads * 4);
    up((void**)&m->D, D, (size_t)cfg->nheads * 4);
    up((void**)&m->norm, norm_gamma, (size_t)cfg->hidden * 2);
    up((void**)&m->gnorm, gated_norm_gamma, (size_t)m->d_inner * 2);
    if (e != cudaSuccess) {
        fail(LSPK_ERR_CUDA, "lspk_mamba_create: %s", cudaGetErrorString(e));
        lspk_mamba_free(reinterpret_cast<lspk_mamba_t>(m));
        return nullptr;
    }
    size_t wb = 0;
    lspk_weight_shape(m->in_proj, nullptr, nullptr, nullptr, &wb);
    m->bytes += wb;
    lspk_weight_shape(m->out_proj, nullptr, nullptr, nullptr, &wb);
    m->bytes += wb;
    return reinterpret_cast<lspk_mamba_t>(m);
}

int lspk_mamba_free(lspk_mamba_t h) {
    if (!h) return LSPK_OK;
    Mamba* m = reinterpret_cast<Mamba*>(h);
    cudaStreamSynchronize(stream());
    lspk_weight_free(m->in_proj);
    lspk_weight_free(m->out_proj);
    void* dev[] = {m->conv_w, m->conv_b, m->A, m->dt_bias, m->D, m->norm, m->gnorm, m->zx, m->v};
    for (void* p : dev) cudaFree(p);
    delete m;
    return LSPK_OK;
}

size_t lspk_mamba_device_bytes(lspk_mamba_t h) { return h ? reinterpret_cast<Mamba*>(h)->bytes : 0; }
size_t lspk_mamba_state_floats(lspk_mamba_t h) { return h ? reinterpret_cast<Mamba*>(h)->state_floats() : 0; }

int lspk_mamba_step(lspk_mamba_t h, float* x_dev, float* state_dev, const int* pos_dev, int B) {
    if (int rc = ensure_init()) return rc;
    return mamba_step(reinterpret_cast<Mamba*>(h), x_dev, state_dev, pos_dev, B);
}

}  // extern "C"
