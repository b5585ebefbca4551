// Row-wise helpers on device-resident fp32 rows: activation quantiser, RMSNorm, fused
// RMSNorm + quantiser, ReLU^2 gate and residual add.  One CTA per token row.
//
// Replace quantize_activation(_batched) (matmul_lut_avx512_extern_c.cpp:425-466, 1098-1109),
// rmsnorm_{bf16,fp32}gamma_fp32(_batched) (:590-650, 1074-1096),
// rmsnorm_quantize_bf16gamma(_batched) (:975-1067), relu2_mul_fp32(_batched) (:653-670,
// 1111-1123) and add_inplace_fp32 (:1127-1137).
#include "common.cuh"

namespace lspk {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float gamma_at(const void* gamma, int is_bf16, int k) {
    return is_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(gamma)[k])
                   : reinterpret_cast<const float*>(gamma)[k];
}

// mode bit 0: apply RMSNorm first; bit 1: quantise (else write fp32 rows to out_f32).
// The normalised row is staged in shared memory (K floats) between the passes.
__global__ void __launch_bounds__(kRowThreads)
row_norm_quant_kernel(const float* __restrict__ x, const void* __restrict__ gamma, int gamma_is_bf16,
                      float* __restrict__ out_f32, int8_t* __restrict__ out_i8,
                      float* __restrict__ scales, int K, float eps, int mode) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* xs = reinterpret_cast<float*>(smem_raw);
    __shared__ float red[32];
    grid_dependency_launch();
    grid_dependency_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* src = x + (size_t)t * K;
    const bool norm = mode & 1, quant = mode & 2;

    float ssq = 0.0f;
    for (int k = tid; k < K; k += kRowThreads) {
        const float v = src[k];
        xs[k] = v;
        ssq = fmaf(v, v, ssq);
    }
    float amax = 0.0f;
    if (norm) {
        ssq = block_sum(ssq, red);
        const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, (float)K), eps)));
        for (int k = tid; k < K; k += kRowThreads) {
            const float v = __fmul_rn(__fmul_rn(xs[k], rrms), gamma_at(gamma, gamma_is_bf16, k));
            if (quant) xs[k] = v; else out_f32[(size_t)t * K + k] = v;
            amax = fmaxf(amax, fabsf(v));
        }
    } else {
        for (int k = tid; k < K; k += kRowThreads) amax = fmaxf(amax, fabsf(xs[k]));
    }
    if (!quant) return;
    amax = block_max(amax, red);
    const float scale = quant_scale_from_absmax(amax);
    const float inv = __fdiv_rn(1.0f, scale);
    const int tail_start = K & ~15;
    for (int k = tid; k < K; k += kRowThreads) {
        int q;
        if (k < tail_start) {
            q = quant_one(xs[k], inv);
        } else {
            q = (int)roundf(__fmul_rn(xs[k], inv));
            q = max(-127, min(127, q));
        }
        out_i8[(size_t)t * K + k] = (int8_t)q;
    }
    if (tid == 0) scales[t] = scale;
}

// `out` may alias `gate` (in-place gating): no restrict qualifiers.
__global__ void relu2_mul_kernel(const float* gate, const float* up, float* out, size_t n) {
    grid_dependency_launch();
    grid_dependency_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float g = fmaxf(gate[i], 0.0f);
        out[i] = __fmul_rn(__fmul_rn(g, g), up[i]);
    }
}

__global__ void add_kernel(float* __restrict__ a, const float* __restrict__ b, size_t n) {
    grid_dependency_launch();
    grid_dependency_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        a[i] = __fadd_rn(a[i], b[i]);
}

static int launch_rows(const float* x, const void* gamma, int gamma_is_bf16, float* out_f32, int8_t* out_i8,
                       float* scales, int T, int K, float eps, int mode) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(x && T >= 1 && K >= 1, "row helper: bad arguments (T=%d K=%d)", T, K);
    const size_t smem = (size_t)K * sizeof(float);
    LSPK_REQUIRE(smem <= 200 * 1024, "row helper: K=%d too large", K);
    static bool attr_set = false;
    if (!attr_set) {
        LSPK_CUDA(cudaFuncSetAttribute(row_norm_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set = true;
    }
    LSPK_CUDA(launch(row_norm_quant_kernel, dim3(T), dim3(kRowThreads), smem, true, x, gamma, gamma_is_bf16,
                     out_f32, out_i8, scales, K, eps, mode));
    return LSPK_OK;
}

static int grid_for(size_t n, int block) {
    size_t g = (n + block - 1) / block;
    const size_t cap = (size_t)sm_count() * 8;
    return (int)(g < cap ? (g ? g : 1) : cap);
}

}  // namespace lspk

using namespace lspk;

extern "C" {

int lspk_quantize_rows(const float* x, int8_t* out, float* scales, int T, int K) {
    LSPK_REQUIRE(out && scales, "lspk_quantize_rows: null output");
    return launch_rows(x, nullptr, 0, nullptr, out, scales, T, K, 0.0f, 2);
}

int lspk_rmsnorm_rows(const float* x, const void* gamma, int gamma_is_bf16, float* out, int T, int K, float eps) {
    LSPK_REQUIRE(gamma && out, "lspk_rmsnorm_rows: null argument");
    return launch_rows(x, gamma, gamma_is_bf16, out, nullptr, nullptr, T, K, eps, 1);
}

int lspk_rmsnorm_quantize_rows(const float* x, const void* gamma, int gamma_is_bf16, int8_t* out, float* scales,
                               int T, int K, float eps) {
    LSPK_REQUIRE(gamma && out && scales, "lspk_rmsnorm_quantize_rows: null argument");
    return launch_rows(x, gamma, gamma_is_bf16, nullptr, out, scales, T, K, eps, 3);
}

int lspk_relu2_mul_rows(const float* gate, const float* up, float* out, int T, int K) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(gate && up && out && T >= 1 && K >= 1, "lspk_relu2_mul_rows: bad arguments");
    const size_t n = (size_t)T * K;
    LSPK_CUDA(launch(relu2_mul_kernel, dim3(grid_for(n, 256)), dim3(256), 0, true, gate, up, out, n));
    return LSPK_OK;
}

int lspk_add_rows(float* a, const float* b, size_t n) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(a && b && n >= 1, "lspk_add_rows: bad arguments");
    LSPK_CUDA(launch(add_kernel, dim3(grid_for(n, 256)), dim3(256), 0, true, a, b, n));
    return LSPK_OK;
}

}  // extern "C"
