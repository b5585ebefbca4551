// Row-wise helpers on device-resident fp32 rows: activation quantiser, RMSNorm, fused
// RMSNorm + quantiser, ReLU^2 gate and residual add.  One CTA per token row.
//
// Replace quantize_activation(_batched) (matmul_lut_avx512_extern_c.cpp:425-466, 1098-1109),
// rmsnorm_{bf16,fp32}gamma_fp32(_batched) (:590-650, 1074-1096),
// rmsnorm_quantize_bf16gamma(_batched) (:975-1067), relu2_mul_fp32(_batched) (:653-670,
// 1111-1123) and add_inplace_fp32 (:1127-1137).
#include "internal.cuh"
#include "ternary_core.cuh"

namespace lspk {

constexpr int kRowThreads = 256;     // eight warps: the lanes of the canonical sum-of-squares order

__device__ __forceinline__ float silu_gate(float z) { return __fdiv_rn(z, __fadd_rn(expf(-z), 1.0f)); }

__device__ __forceinline__ float gamma_at(const void* gamma, int is_bf16, int k) {
    return is_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(gamma)[k])
                   : reinterpret_cast<const float*>(gamma)[k];
}

// Combines the threads' canonical sum-of-squares values (ternary_core.cuh: thread = lane of the 256-lane group)
// over the CTA.  Two barriers: `red` can be reused right after.
__device__ __forceinline__ float row_ssq_combine(float lane_value, float* red) {
    static_assert(kRowThreads == 256, "the canonical order has 256 lanes");
    const float v = warp_sum(lane_value);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    const float total = canonical_ssq_combine(red);
    __syncthreads();
    return total;
}

// mode bit 0: apply RMSNorm first; bit 1: quantise (else write fp32 rows to out_f32).
// gate != nullptr: the row is x * SiLU(gate) (the gated norm of the Mamba-2 block) before anything else.
// perm_kp > 0 (VEC only): the int8 row is written in the layout the tensor-core kernels read: perm_kp bytes (K
// rounded up to 64, zero padded) with the 4x4 index transpose inside every 16-element block, rows perm_stride
// bytes apart; sums (optional) receives the sum of the row's int8 values.
// The normalised row is staged in shared memory (K floats) between the passes.  VEC: K is a
// multiple of 4 and every pointer 16-byte aligned, so the passes move four elements at a time.
template <bool VEC>
__global__ void __launch_bounds__(kRowThreads)
row_norm_quant_kernel(const float* __restrict__ x, const float* __restrict__ gate, const void* __restrict__ gamma_base,
                      const int* __restrict__ gamma_sel, int gamma_is_bf16, float* __restrict__ out_f32,
                      int8_t* __restrict__ out_i8, float* __restrict__ scales, int K, float eps, int mode, int perm_kp,
                      int perm_stride, int* __restrict__ sums) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* xs = reinterpret_cast<float*>(smem_raw);
    __shared__ float red[32];
    grid_dependency_launch();
    grid_dependency_wait();
    const int t = blockIdx.x, tid = threadIdx.x;
    const float* src = x + (size_t)t * K;
    const float* gsrc = gate ? gate + (size_t)t * K : nullptr;
    // gamma_sel: row t uses the gamma_sel[t]-th vector of K norm weights (per-expert sub-norms)
    const void* gamma = gamma_base;
    if (gamma_sel) gamma = reinterpret_cast<const char*>(gamma_base) + (size_t)gamma_sel[t] * K * (gamma_is_bf16 ? 2 : 4);
    const bool norm = mode & 1, quant = mode & 2;
    const int tail_start = K & ~15;

    if (VEC) {
        const int K4 = K >> 2;
        const float4* src4 = reinterpret_cast<const float4*>(src);
        float4* xs4 = reinterpret_cast<float4*>(xs);
        // first pass in the canonical order of the sum of squares: thread = lane, 16-element blocks tid, tid + 256,
        // ...; element e of a block goes into partial e % 4 (a float4's .x/.y/.z/.w are e % 4 = 0..3)
        float amax = 0.0f;
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
        for (int b4 = tid * 4; b4 < K4; b4 += kRowThreads * 4) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int i = b4 + q;
                if (i < K4) {
                    float4 v = src4[i];
                    if (gsrc) {
                        const float4 gz = reinterpret_cast<const float4*>(gsrc)[i];
                        v.x = __fmul_rn(v.x, silu_gate(gz.x));
                        v.y = __fmul_rn(v.y, silu_gate(gz.y));
                        v.z = __fmul_rn(v.z, silu_gate(gz.z));
                        v.w = __fmul_rn(v.w, silu_gate(gz.w));
                    }
                    xs4[i] = v;
                    ss[0] = fmaf(v.x, v.x, ss[0]);
                    ss[1] = fmaf(v.y, v.y, ss[1]);
                    ss[2] = fmaf(v.z, v.z, ss[2]);
                    ss[3] = fmaf(v.w, v.w, ss[3]);
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                }
            }
        }
        if (norm) {
            const float ssq = row_ssq_combine((ss[0] + ss[1]) + (ss[2] + ss[3]), red);
            const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, (float)K), eps)));
            amax = 0.0f;
            for (int i = tid; i < K4; i += kRowThreads) {
                float4 v = xs4[i];
                const int k = i << 2;
                v.x = __fmul_rn(__fmul_rn(v.x, rrms), gamma_at(gamma, gamma_is_bf16, k));
                v.y = __fmul_rn(__fmul_rn(v.y, rrms), gamma_at(gamma, gamma_is_bf16, k + 1));
                v.z = __fmul_rn(__fmul_rn(v.z, rrms), gamma_at(gamma, gamma_is_bf16, k + 2));
                v.w = __fmul_rn(__fmul_rn(v.w, rrms), gamma_at(gamma, gamma_is_bf16, k + 3));
                if (quant) xs4[i] = v; else reinterpret_cast<float4*>(out_f32 + (size_t)t * K)[i] = v;
                amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
            }
        }
        if (!quant) return;
        amax = block_max(amax, red);
        const float scale = quant_scale_from_absmax(amax);
        const float inv = __fdiv_rn(1.0f, scale);
        auto quant4 = [&](int i) -> uint32_t {
            const float4 v = xs4[i];
            const float f[4] = {v.x, v.y, v.z, v.w};
            uint32_t word = 0;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int q;
                if ((i << 2) < tail_start) {
                    q = quant_one(f[e], inv);
                } else {
                    q = (int)roundf(__fmul_rn(f[e], inv));
                    q = max(-127, min(127, q));
                }
                word |= ((uint32_t)q & 0xffu) << (8 * e);
            }
            return word;
        };
        if (perm_kp > 0) {
            // one quarter of a 16-element block per thread (all threads busy); the four lanes of a block
            // exchange their words and lane q assembles output word q = byte q of the four quarters
            uint32_t* dst = reinterpret_cast<uint32_t*>(out_i8 + (size_t)t * perm_stride);
            const int P4 = perm_kp >> 2;
            const int lane = tid & 31, q = lane & 3, base = lane & ~3;
            int sumx = 0;
            for (int i0 = 0; i0 < P4; i0 += kRowThreads) {          // uniform trip count: shuffles need whole warps
                const int i = i0 + tid;
                const uint32_t mine = i < K4 ? quant4(i) : 0u;
                sumx = __dp4a((int)mine, 0x01010101, sumx);
                const uint32_t w0 = __shfl_sync(0xffffffffu, mine, base + 0), w1 = __shfl_sync(0xffffffffu, mine, base + 1);
                const uint32_t w2 = __shfl_sync(0xffffffffu, mine, base + 2), w3 = __shfl_sync(0xffffffffu, mine, base + 3);
                const uint32_t sel = 0x4440u + 0x1111u * (uint32_t)q;      // byte q of the first operand, byte q of the second
                const uint32_t lo = __byte_perm(w0, w1, sel & 0x00ffu), hi = __byte_perm(w2, w3, sel & 0x00ffu);
                if (i < P4) dst[i] = __byte_perm(lo, hi, 0x5410);
            }
            if (sums) {                                    // uniform branch: every thread of the block takes it
                sumx = __reduce_add_sync(0xffffffffu, sumx);
                int* redi = reinterpret_cast<int*>(red);
                if (lane == 0) redi[tid >> 5] = sumx;
                __syncthreads();
                if (tid == 0) {
                    int total = 0;
                    for (int w = 0; w < kRowThreads / 32; ++w) total += redi[w];
                    sums[t] = total;
                }
            }
        } else {
            uint32_t* dst = reinterpret_cast<uint32_t*>(out_i8 + (size_t)t * K);
            for (int i = tid; i < K4; i += kRowThreads) dst[i] = quant4(i);
        }
        if (tid == 0) scales[t] = scale;
        return;
    }

    for (int k = tid; k < K; k += kRowThreads) {
        float v = src[k];
        if (gsrc) v = __fmul_rn(v, silu_gate(gsrc[k]));
        xs[k] = v;
    }
    float amax = 0.0f;
    if (norm) {
        __syncthreads();
        const float ssq = row_ssq_combine(canonical_ssq_lane(xs, K, tid), red);
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

// Row quantiser for rows of up to 4096 * NB elements, everything in registers: a thread owns the 16-element blocks
// tid, tid + 256 (the lanes of the canonical sum-of-squares order), loads them once, and -- having whole blocks --
// writes the permuted layout of the tensor-core kernels without any exchange between lanes.  The norm weights
// do not depend on the previous kernel and are requested before the dependency wait (unless they are selected
// per row by device data).  Same arithmetic, step for step, as the fused prologue of the one-row GEMV.
//   norm      apply RMSNorm (gamma, eps) before the quantiser
//   perm_kp   > 0: write perm_kp bytes per row (K rounded up to 64, zero padded) in the permuted layout, rows
//             perm_stride bytes apart, and optionally the sum of the row's int8 values; 0: natural order [T, K]
template <int NB>
__global__ void __launch_bounds__(kRowThreads)
row_quant_regs_kernel(const float* __restrict__ x, const float* __restrict__ gate, const void* __restrict__ gamma_base,
                      const int* __restrict__ gamma_sel, int gamma_is_bf16, int8_t* __restrict__ out_i8,
                      float* __restrict__ scales, int K, float eps, int norm, int perm_kp, int perm_stride,
                      int* __restrict__ sums) {
    __shared__ __align__(16) float red[32];
    const int t = blockIdx.x, tid = threadIdx.x;
    float gm[NB][16];
    auto load_gamma = [&](const void* gamma) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int k0 = (tid + nb * kRowThreads) * 16;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int k = k0 + q * 4;
                float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (k < K) {
                    if (gamma_is_bf16) {
                        const uint2 gb = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(gamma) + k));
                        gv.x = __uint_as_float(gb.x << 16);
                        gv.y = __uint_as_float(gb.x & 0xffff0000u);
                        gv.z = __uint_as_float(gb.y << 16);
                        gv.w = __uint_as_float(gb.y & 0xffff0000u);
                    } else {
                        gv = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(gamma) + k));
                    }
                }
                gm[nb][q * 4 + 0] = gv.x;
                gm[nb][q * 4 + 1] = gv.y;
                gm[nb][q * 4 + 2] = gv.z;
                gm[nb][q * 4 + 3] = gv.w;
            }
        }
    };
    if (norm && !gamma_sel) load_gamma(gamma_base);
    grid_dependency_launch();
    grid_dependency_wait();
    if (norm && gamma_sel)
        load_gamma(reinterpret_cast<const char*>(gamma_base) + (size_t)gamma_sel[t] * K * (gamma_is_bf16 ? 2 : 4));

    const float* src = x + (size_t)t * K;
    float v[NB][16];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        const int k0 = (tid + nb * kRowThreads) * 16;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k0 + q * 4 < K) t4 = *reinterpret_cast<const float4*>(src + k0 + q * 4);
            v[nb][q * 4 + 0] = t4.x;
            v[nb][q * 4 + 1] = t4.y;
            v[nb][q * 4 + 2] = t4.z;
            v[nb][q * 4 + 3] = t4.w;
        }
    }
    if (gate) {
        const float* gsrc = gate + (size_t)t * K;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int k0 = (tid + nb * kRowThreads) * 16;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                if (k0 + q * 4 < K) t4 = *reinterpret_cast<const float4*>(gsrc + k0 + q * 4);
                v[nb][q * 4 + 0] = __fmul_rn(v[nb][q * 4 + 0], silu_gate(t4.x));
                v[nb][q * 4 + 1] = __fmul_rn(v[nb][q * 4 + 1], silu_gate(t4.y));
                v[nb][q * 4 + 2] = __fmul_rn(v[nb][q * 4 + 2], silu_gate(t4.z));
                v[nb][q * 4 + 3] = __fmul_rn(v[nb][q * 4 + 3], silu_gate(t4.w));
            }
        }
    }
    if (norm) {
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 16; ++e) ss[e & 3] = fmaf(v[nb][e], v[nb][e], ss[e & 3]);
        const float ssq = row_ssq_combine((ss[0] + ss[1]) + (ss[2] + ss[3]), red);
        const float rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, (float)K), eps)));
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int e = 0; e < 16; ++e) v[nb][e] = __fmul_rn(__fmul_rn(v[nb][e], rrms), gm[nb][e]);
    }
    float amax = 0.0f;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(v[nb][e]));
    amax = block_max(amax, red);
    const float scale = quant_scale_from_absmax(amax);
    const float inv = __fdiv_rn(1.0f, scale);
    const int tail_start = K & ~15;
    const int limit = perm_kp > 0 ? perm_kp : K;
    int sumx = 0;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
        const int k0 = (tid + nb * kRowThreads) * 16;
        if (k0 < limit) {
            uint32_t a[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t word = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int k = k0 + q * 4 + e;
                    int qv = 0;
                    if (k < tail_start) {
                        qv = quant_one(v[nb][q * 4 + e], inv);
                    } else if (k < K) {
                        qv = max(-127, min(127, (int)roundf(__fmul_rn(v[nb][q * 4 + e], inv))));
                    }
                    word |= ((uint32_t)qv & 0xffu) << (8 * e);
                }
                a[q] = word;
                sumx = __dp4a((int)word, 0x01010101, sumx);
            }
            if (perm_kp > 0) {
                uint32_t o0, o1, o2, o3;
                transpose4x4_bytes(a[0], a[1], a[2], a[3], o0, o1, o2, o3);
                *reinterpret_cast<uint4*>(out_i8 + (size_t)t * perm_stride + k0) = make_uint4(o0, o1, o2, o3);
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (k0 + q * 4 < K) *reinterpret_cast<uint32_t*>(out_i8 + (size_t)t * K + k0 + q * 4) = a[q];
            }
        }
    }
    if (sums) {                                        // uniform branch
        sumx = __reduce_add_sync(0xffffffffu, sumx);
        int* redi = reinterpret_cast<int*>(red);
        if ((tid & 31) == 0) redi[tid >> 5] = sumx;
        __syncthreads();
        if (tid == 0) {
            int total = 0;
            for (int w = 0; w < kRowThreads / 32; ++w) total += redi[w];
            sums[t] = total;
        }
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
                       float* scales, int T, int K, float eps, int mode, const float* gate = nullptr,
                       const int* gamma_sel = nullptr, int perm_kp = 0, int perm_stride = 0, int* sums = nullptr) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(x && T >= 1 && K >= 1, "row helper: bad arguments (T=%d K=%d)", T, K);
    const size_t smem = (size_t)K * sizeof(float);
    LSPK_REQUIRE(smem <= 200 * 1024, "row helper: K=%d too large", K);
    static bool attr_set = false;
    if (!attr_set) {
        LSPK_CUDA(cudaFuncSetAttribute(row_norm_quant_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(row_norm_quant_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set = true;
    }
    auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    const bool vec = (K % 4 == 0) && aligned(x) && aligned(out_f32) && aligned(out_i8) && aligned(gamma) && aligned(gate) &&
                     (!gamma_sel || K % 8 == 0);
    LSPK_REQUIRE(perm_kp == 0 || vec, "row helper: the permuted output needs K %% 4 == 0 and 16-byte aligned buffers");
    // quantising rows of up to 8192 elements: the register-resident kernel
    if (vec && (mode & 2) && K <= 8192 && (perm_kp == 0 || perm_kp <= 8192)) {
        const int pstride = perm_stride > 0 ? perm_stride : perm_kp;
        const cudaError_t e = K <= 4096 && perm_kp <= 4096
            ? launch(row_quant_regs_kernel<1>, dim3(T), dim3(kRowThreads), 0, true, x, gate, gamma, gamma_sel, gamma_is_bf16,
                     out_i8, scales, K, eps, mode & 1, perm_kp, pstride, sums)
            : launch(row_quant_regs_kernel<2>, dim3(T), dim3(kRowThreads), 0, true, x, gate, gamma, gamma_sel, gamma_is_bf16,
                     out_i8, scales, K, eps, mode & 1, perm_kp, pstride, sums);
        if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "row quantiser launch failed: %s", cudaGetErrorString(e));
        return LSPK_OK;
    }
    LSPK_CUDA(launch(vec ? row_norm_quant_kernel<true> : row_norm_quant_kernel<false>, dim3(T), dim3(kRowThreads), smem,
                     true, x, gate, gamma, gamma_sel, gamma_is_bf16, out_f32, out_i8, scales, K, eps, mode, vec ? perm_kp : 0,
                     perm_stride > 0 ? perm_stride : perm_kp, sums));
    return LSPK_OK;
}

// For more than one token row, quantising inside the linear kernel would make every CTA repeat the
// norm + quantiser of all rows (three passes over M*K floats per CTA): run it once here into the
// caller's scratch and switch the call to the int8 prologue.  One row keeps the fused prologue.
int split_row_prologue(lspk_linear_args* a, int K, int8_t* q_scratch, float* scale_scratch) {
    if (a->M <= 1) return LSPK_OK;
    int mode;
    const float* gate = nullptr;
    if (a->prologue == LSPK_PRO_QUANT) mode = 2;
    else if (a->prologue == LSPK_PRO_RMSNORM_QUANT) mode = 3;
    else if (a->prologue == LSPK_PRO_GATED_RMSNORM_QUANT) { mode = 3; gate = a->gate_f32; }
    else return LSPK_OK;
    if (int rc = launch_rows(a->x_f32, a->gamma, a->gamma_is_bf16, nullptr, q_scratch, scale_scratch, a->M, K, a->eps, mode,
                             gate))
        return rc;
    a->prologue = LSPK_PRO_INT8;
    a->x_i8 = q_scratch;
    a->x_scales = scale_scratch;
    a->x_f32 = nullptr;
    a->gate_f32 = nullptr;
    return LSPK_OK;
}

// RMSNorm + quantiser of T rows where row t takes the gamma_sel[t]-th weight vector (bf16, K each).
int norm_quant_rows_selected(const float* x, const void* gamma_bf16, const int* gamma_sel, int8_t* out, float* scales,
                             int T, int K, float eps) {
    return launch_rows(x, gamma_bf16, 1, nullptr, out, scales, T, K, eps, 3, nullptr, gamma_sel);
}

// Quantise fp32 rows (QUANT, RMSNORM_QUANT or GATED_RMSNORM_QUANT prologue of `a`) straight into the permuted,
// padded activation layout of the tensor-core kernels: rows `stride` bytes apart (0: Kp), optionally with the
// per-row sums of the int8 values.  *done = 0 when the vector path cannot run (shape / alignment).
int quantize_rows_permuted(const lspk_linear_args* a, int K, int Kp, int8_t* out_perm, float* scales, int* done,
                           int stride, int* sums) {
    *done = 0;
    auto aligned = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if ((K % 4) || !aligned(a->x_f32) || !aligned(a->gamma) || !aligned(out_perm) || !aligned(a->gate_f32) || (stride & 15))
        return LSPK_OK;
    int mode;
    const float* gate = nullptr;
    if (a->prologue == LSPK_PRO_QUANT) mode = 2;
    else if (a->prologue == LSPK_PRO_RMSNORM_QUANT) mode = 3;
    else if (a->prologue == LSPK_PRO_GATED_RMSNORM_QUANT) { mode = 3; gate = a->gate_f32; }
    else return LSPK_OK;
    if (int rc = launch_rows(a->x_f32, a->gamma, a->gamma_is_bf16, nullptr, out_perm, scales, a->M, K, a->eps, mode, gate,
                             nullptr, Kp, stride, sums))
        return rc;
    *done = 1;
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
