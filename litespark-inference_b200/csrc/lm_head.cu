// LM-head GEMV: logits[t, v] = sum_h dequant(E[v, h]) * x[t, h]  (* emb_scale[v] for int8/int4).
// The embedding table is the largest tensor streamed per token (656.7 MB in bf16 at V=128256,
// H=2560), so this is a pure HBM-streaming kernel: one warp per vocabulary row, 16-byte loads,
// up to 5 loads in flight per lane, x staged once per CTA in shared memory in an order that makes
// each lane's 16-byte shared loads conflict-free.  Optionally fuses the final RMSNorm in front
// (every CTA renormalises the H-vector itself) and a greedy argmax behind (first maximum wins,
// like np.argmax).
//
// Replaces lm_head_bf16_fp32 / lm_head_int8_fp32 / lm_head_int4_fp32
// (matmul_lut_avx512_extern_c.cpp:470-498, 501-525, 535-587).
#include <stdlib.h>

#include "common.cuh"

namespace lspk {

constexpr int kLmThreads = 256;
constexpr int kLmWarps = kLmThreads / 32;
constexpr int kLmMaxT = 8;

template <int KIND> struct EmbTraits;
template <> struct EmbTraits<0> { static constexpr int E = 8;  };   // bf16: 8 values per 16 bytes
template <> struct EmbTraits<1> { static constexpr int E = 16; };   // int8
template <> struct EmbTraits<2> { static constexpr int E = 32; };   // int4, low nibble first

template <int KIND>
__device__ __forceinline__ void decode4(const uint4& c, int s, float f[4]) {
    // the s-th group of four consecutive values of a 16-byte chunk
    const uint32_t w[4] = {c.x, c.y, c.z, c.w};
    if (KIND == 0) {
        const uint32_t a = w[(s * 2) & 3], b = w[(s * 2 + 1) & 3];
        f[0] = __uint_as_float(a << 16);
        f[1] = __uint_as_float(a & 0xffff0000u);
        f[2] = __uint_as_float(b << 16);
        f[3] = __uint_as_float(b & 0xffff0000u);
    } else if (KIND == 1) {
        const uint32_t a = w[s & 3];
#pragma unroll
        for (int e = 0; e < 4; ++e) f[e] = (float)((int)(a << (24 - 8 * e)) >> 24);
    } else {
        const uint32_t a = (w[(s >> 1) & 3] >> ((s & 1) * 16)) & 0xffffu;   // two bytes = four nibbles
#pragma unroll
        for (int e = 0; e < 4; ++e) f[e] = (float)((int)(a << (28 - 4 * e)) >> 28);
    }
}

__device__ __forceinline__ unsigned long long argmax_key(float v, int idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);       // order-preserving map to unsigned
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)idx);
}

// TT: rows of x handled per launch (1 for decode, up to kLmMaxT otherwise); INFL: 16-byte loads in
// flight per lane and vocabulary row (10 covers a 2560-wide bf16 row in one batch); RW: vocabulary
// rows a warp works on at once.  With several rows of x the kernel would be bound by shared-memory
// reads of x (32 bytes per row of x and 16-byte chunk of the table); a warp that holds RW table
// rows reuses every x value it fetched RW times.
template <int KIND, int TT, int INFL, int RW>
__global__ void __launch_bounds__(kLmThreads)
lm_head_kernel(const uint4* __restrict__ emb, const float* __restrict__ emb_scale,
               const float* __restrict__ x, float* __restrict__ logits, int T, int V, int H,
               const void* __restrict__ norm_gamma, int gamma_is_bf16, float eps,
               unsigned long long* __restrict__ best_key) {
    constexpr int E = EmbTraits<KIND>::E;
    constexpr int S = E / 4;                       // float4 groups per chunk
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float4* xs4 = reinterpret_cast<float4*>(smem_raw);   // [T][S][nchunks]
    __shared__ float red[32];
    __shared__ unsigned long long s_best[kLmWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nchunks = H / E;                     // host guarantees H % E == 0

    grid_dependency_launch();
    grid_dependency_wait();

    for (int t = 0; t < T; ++t) {
        const float* xr = x + (size_t)t * H;
        float rrms = 1.0f;
        if (norm_gamma) {
            float ssq = 0.0f;
            for (int k = tid; k < H; k += kLmThreads) ssq = fmaf(xr[k], xr[k], ssq);
            ssq = block_sum(ssq, red);
            rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, (float)H), eps)));
        }
        float* dst = reinterpret_cast<float*>(xs4 + (size_t)t * S * nchunks);
        for (int k = tid; k < H; k += kLmThreads) {
            float v = xr[k];
            if (norm_gamma) {
                const float gm = gamma_is_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(norm_gamma)[k])
                                               : reinterpret_cast<const float*>(norm_gamma)[k];
                v = __fmul_rn(__fmul_rn(v, rrms), gm);
            }
            const int c = k / E, s = (k % E) / 4, e = k & 3;
            dst[((size_t)s * nchunks + c) * 4 + e] = v;
        }
    }
    __syncthreads();

    unsigned long long best = 0ull;
    const size_t row_chunks = (size_t)nchunks;
    for (int v0 = (blockIdx.x * kLmWarps + warp) * RW; v0 < V; v0 += gridDim.x * kLmWarps * RW) {
        float acc[TT][RW];
#pragma unroll
        for (int t = 0; t < TT; ++t)
#pragma unroll
            for (int r = 0; r < RW; ++r) acc[t][r] = 0.0f;
        for (int c0 = lane; c0 < nchunks; c0 += 32 * INFL) {
            uint4 buf[RW][INFL];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                if (RW == 1 || v0 + r < V) {
                    const uint4* row = emb + (size_t)(v0 + r) * row_chunks;
#pragma unroll
                    for (int u = 0; u < INFL; ++u) {
                        const int c = c0 + 32 * u;
                        if (c < nchunks) buf[r][u] = __ldcs(row + c);
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < INFL; ++u) buf[r][u] = make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < INFL; ++u) {
                const int c = c0 + 32 * u;
                if (c < nchunks) {
#pragma unroll
                    for (int s = 0; s < S; ++s) {
                        float f[RW][4];
#pragma unroll
                        for (int r = 0; r < RW; ++r) decode4<KIND>(buf[r][u], s, f[r]);
#pragma unroll
                        for (int t = 0; t < TT; ++t) {
                            if (TT == 1 || t < T) {
                                const float4 xv = xs4[((size_t)t * S + s) * nchunks + c];
#pragma unroll
                                for (int r = 0; r < RW; ++r) {
                                    acc[t][r] = fmaf(f[r][0], xv.x, acc[t][r]);
                                    acc[t][r] = fmaf(f[r][1], xv.y, acc[t][r]);
                                    acc[t][r] = fmaf(f[r][2], xv.z, acc[t][r]);
                                    acc[t][r] = fmaf(f[r][3], xv.w, acc[t][r]);
                                }
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < RW; ++r) {
            const int v = v0 + r;
            if (RW > 1 && v >= V) break;
            const float sc = (KIND == 0) ? 1.0f : emb_scale[v];
#pragma unroll
            for (int t = 0; t < TT; ++t) {
                if (TT == 1 || t < T) {
                    float rr = warp_sum(acc[t][r]);
                    if (KIND != 0) rr = __fmul_rn(sc, rr);
                    if (lane == 0) {
                        if (logits) logits[(size_t)t * V + v] = rr;
                        if (best_key && t == 0) {
                            const unsigned long long key = argmax_key(rr, v);
                            best = key > best ? key : best;
                        }
                    }
                }
            }
        }
    }
    if (best_key) {
        if (lane == 0) s_best[warp] = best;
        __syncthreads();
        if (tid == 0) {
            unsigned long long b = s_best[0];
#pragma unroll
            for (int w = 1; w < kLmWarps; ++w) b = s_best[w] > b ? s_best[w] : b;
            atomicMax(best_key, b);
        }
    }
}

// norm_gamma / best_key may be null.  T <= kLmMaxT per launch; larger T is tiled here.
int lm_head_launch(int kind, const void* emb, const float* emb_scale, const float* x, float* logits,
                   int T, int V, int H, const void* norm_gamma, int gamma_is_bf16, float eps,
                   unsigned long long* best_key) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(emb && x && T >= 1 && V >= 1 && H >= 1, "lm_head: bad arguments");
    LSPK_REQUIRE(kind >= 0 && kind <= 2, "lm_head: kind must be 0 (bf16), 1 (int8) or 2 (int4)");
    LSPK_REQUIRE(kind == 0 || emb_scale, "lm_head: int8/int4 need emb_scale");
    const int E = kind == 0 ? 8 : kind == 1 ? 16 : 32;
    LSPK_REQUIRE(H % E == 0, "lm_head: H=%d must be a multiple of %d for this embedding format", H, E);
    LSPK_REQUIRE(((uintptr_t)emb & 15) == 0, "lm_head: embedding must be 16-byte aligned");
    const int rows_per_cta = kLmWarps;
    int grid = (V + rows_per_cta - 1) / rows_per_cta;
    const int cap = sm_count() * 4;
    if (grid > cap) grid = cap;
    const uint4* e4 = reinterpret_cast<const uint4*>(emb);
    for (int t0 = 0; t0 < T; t0 += kLmMaxT) {
        const int tt = (T - t0) < kLmMaxT ? (T - t0) : kLmMaxT;
        const size_t smem = (size_t)tt * H * sizeof(float);
        LSPK_REQUIRE(smem <= 200 * 1024, "lm_head: H=%d too large", H);
        const float* xt = x + (size_t)t0 * H;
        float* lt = logits ? logits + (size_t)t0 * V : nullptr;
        unsigned long long* bk = t0 == 0 ? best_key : nullptr;
        cudaError_t e = cudaSuccess;
#define LSPK_LM_LAUNCH(KIND, TT, INFL, RW)                                                                  \
        do {                                                                                                \
            static bool attr_set = false;                                                                   \
            auto kern = lm_head_kernel<KIND, TT, INFL, RW>;                                                   \
            if (!attr_set) {                                                                                \
                e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);     \
                attr_set = (e == cudaSuccess);                                                              \
            }                                                                                               \
            if (e == cudaSuccess)                                                                           \
                e = launch(kern, dim3(grid), dim3(kLmThreads), smem, true, e4, emb_scale, xt, lt, tt, V, H,  \
                           norm_gamma, gamma_is_bf16, eps, bk);                                             \
        } while (0)
        if (tt == 1) {
            if (kind == 0) LSPK_LM_LAUNCH(0, 1, 10, 1);
            else if (kind == 1) LSPK_LM_LAUNCH(1, 1, 5, 1);
            else LSPK_LM_LAUNCH(2, 1, 3, 1);
        } else {
            // measured at V = 128256, H = 2560, 8 rows (loads in flight, table rows per warp): (4,1) 396 us,
            // (4,2) 315, (3,4) 482, (6,2) 514, (2,4) 255: with eight rows the kernel is bound by its
            // fused multiply-adds and registers, not by loads in flight
            if (kind == 0) LSPK_LM_LAUNCH(0, kLmMaxT, 2, 4);
            else if (kind == 1) LSPK_LM_LAUNCH(1, kLmMaxT, 2, 2);
            else LSPK_LM_LAUNCH(2, kLmMaxT, 1, 2);
        }
#undef LSPK_LM_LAUNCH
        if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "lm_head launch failed: %s", cudaGetErrorString(e));
    }
    return LSPK_OK;
}

}  // namespace lspk

extern "C" int lspk_lm_head(int kind, const void* emb, const float* emb_scale, const float* x, float* logits,
                            int T, int V, int H) {
    LSPK_REQUIRE(logits, "lspk_lm_head: null logits");
    return lspk::lm_head_launch(kind, emb, emb_scale, x, logits, T, V, H, nullptr, 0, 0.0f, nullptr);
}
