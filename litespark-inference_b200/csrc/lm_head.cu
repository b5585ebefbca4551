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

#include "internal.cuh"

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

// ---- several rows of x against a bf16 table on the warp-level tensor cores -------------------------
// With 2..16 rows of x the CUDA-core kernel above is bound by its fused multiply-adds (V * H * T of them)
// and by shared-memory reads of x.  Here a warp owns 16 table rows (the MMA's M side), the rows of x are
// the N side (one or two tiles of eight), and the table bytes go from global memory straight into A
// fragments: lane (g, t) loads 16 bytes of row g and of row g + 8 per 32-wide K step; which eight k's a
// lane holds is a permutation of K that the x fragments repeat, so no shuffle is needed.
// x stays fp32-exact: it is split into three bf16 terms (x = hi + mid + lo up to 2^-24 |x|), each product
// bf16 x bf16 is exact in the fp32 accumulator, so the result differs from the fp32 dot product only in
// summation order, like every other reduction here.
constexpr int kLmmStepsInFlight = 6;      // 32-wide K steps of table data in flight per lane (12 x 16 bytes)

__device__ __forceinline__ void mma_bf16_16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t bf16_rn_bits(float v) {          // round to nearest even, as a 16-bit pattern
    const uint32_t u = __float_as_uint(v);
    return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}

// NT: tiles of eight rows of x (1 or 2) a CTA holds.  Shared memory: [3 terms][8 * NT rows][H + 32] bf16.
// passes: more rows than a CTA holds are served side by side in ONE launch: CTA b takes the row block b % passes
// and the table tiles of position b / passes, so the CTAs that need the same table rows run next to each other
// and the table comes from HBM once (the second reader finds it in L2).
template <int NT>
__global__ void __launch_bounds__(kLmThreads)
lm_head_mma_kernel(const uint4* __restrict__ emb, const float* __restrict__ x, float* __restrict__ logits, int T_all, int V,
                   int H, const void* __restrict__ norm_gamma, int gamma_is_bf16, float eps,
                   unsigned long long* __restrict__ best_keys, int passes) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    uint16_t* xs = reinterpret_cast<uint16_t*>(smem_raw);
    __shared__ float red[32];
    __shared__ unsigned long long s_best[kLmWarps][8 * NT];
    unsigned long long best[NT][2];                          // greedy argmax keys of tokens 8 n + 2 t4 + {0, 1}
#pragma unroll
    for (int n = 0; n < NT; ++n) best[n][0] = best[n][1] = 0ull;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    constexpr int R = 8 * NT;
    const int pass = (int)blockIdx.x % passes, cta = (int)blockIdx.x / passes, ncta = (int)gridDim.x / passes;
    const int T = min(R, T_all - pass * R);                // rows of this CTA's block
    x += (size_t)pass * R * H;
    if (logits) logits += (size_t)pass * R * V;
    if (best_keys) best_keys += pass * R;
    const int ld = H + 32;                                 // row stride in bf16: 64 bytes of padding make the quarter-warp 16-byte loads conflict-free
    const int steps = H / 32;                              // host guarantees H % 32 == 0
    const size_t row_chunks = (size_t)H / 8;

    // table rows of this warp's first tile can be requested before the activations exist
    auto tile_of = [&](int i) { return (cta * kLmWarps + warp) + i * ncta * kLmWarps; };
    uint4 buf[kLmmStepsInFlight][2];
    auto request = [&](int v0, int s0) {
#pragma unroll
        for (int u = 0; u < kLmmStepsInFlight; ++u) {
            const int sidx = s0 + u;
            if (sidx < steps) {
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int v = v0 + g + 8 * hh;
                    buf[u][hh] = v < V ? __ldcs(emb + (size_t)v * row_chunks + (size_t)sidx * 4 + t4) : make_uint4(0, 0, 0, 0);
                }
            }
        }
    };
    int tile = tile_of(0);
    if (tile * 16 < V) request(tile * 16, 0);

    grid_dependency_launch();
    grid_dependency_wait();

    // rows of x (optionally RMS-normalised) -> three bf16 terms in shared memory
    for (int r = 0; r < R; ++r) {
        if (r < T) {
            const float* xr = x + (size_t)r * H;
            float rrms = 1.0f;
            if (norm_gamma) {
                float ssq = 0.0f;
                for (int k = tid; k < H; k += kLmThreads) ssq = fmaf(xr[k], xr[k], ssq);
                ssq = block_sum(ssq, red);
                rrms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ssq, (float)H), eps)));
            }
            for (int k = tid; k < H; k += kLmThreads) {
                float v = xr[k];
                if (norm_gamma) {
                    const float gm = gamma_is_bf16 ? bf16_bits_to_f32(reinterpret_cast<const uint16_t*>(norm_gamma)[k])
                                                   : reinterpret_cast<const float*>(norm_gamma)[k];
                    v = __fmul_rn(__fmul_rn(v, rrms), gm);
                }
                const uint32_t hi = bf16_rn_bits(v);
                const float r1 = v - __uint_as_float(hi << 16);
                const uint32_t mid = bf16_rn_bits(r1);
                const float r2 = r1 - __uint_as_float(mid << 16);
                const uint32_t lo = bf16_rn_bits(r2);
                xs[(size_t)(0 * R + r) * ld + k] = (uint16_t)hi;
                xs[(size_t)(1 * R + r) * ld + k] = (uint16_t)mid;
                xs[(size_t)(2 * R + r) * ld + k] = (uint16_t)lo;
            }
        } else {
            for (int k = tid; k < H; k += kLmThreads) {
                xs[(size_t)(0 * R + r) * ld + k] = 0;
                xs[(size_t)(1 * R + r) * ld + k] = 0;
                xs[(size_t)(2 * R + r) * ld + k] = 0;
            }
        }
    }
    __syncthreads();

    for (int it = 0; tile * 16 < V; ++it) {
        const int v0 = tile * 16;
        float acc[NT][4];
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[n][c] = 0.0f;
        for (int s0 = 0; s0 < steps; s0 += kLmmStepsInFlight) {
            uint4 cur[kLmmStepsInFlight][2];
#pragma unroll
            for (int u = 0; u < kLmmStepsInFlight; ++u) {
                cur[u][0] = buf[u][0];
                cur[u][1] = buf[u][1];
            }
            // next batch of this tile, or the first batch of the next tile, goes out before the math
            if (s0 + kLmmStepsInFlight < steps) {
                request(v0, s0 + kLmmStepsInFlight);
            } else {
                const int nt = tile_of(it + 1);
                if (nt * 16 < V) request(nt * 16, 0);
            }
#pragma unroll
            for (int u = 0; u < kLmmStepsInFlight; ++u) {
                const int sidx = s0 + u;
                if (sidx < steps) {
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
#pragma unroll
                        for (int term = 0; term < 3; ++term) {
                            // this lane's B data: token row (8 n + g), k = 32 sidx + 8 t4 .. + 7
                            const uint4 b = *reinterpret_cast<const uint4*>(
                                xs + (size_t)(term * R + 8 * n + g) * ld + (size_t)sidx * 32 + t4 * 8);
                            mma_bf16_16816(acc[n], cur[u][0].x, cur[u][1].x, cur[u][0].y, cur[u][1].y, b.x, b.y);
                            mma_bf16_16816(acc[n], cur[u][0].z, cur[u][1].z, cur[u][0].w, cur[u][1].w, b.z, b.w);
                        }
                    }
                }
            }
        }
        // C fragment: c0, c1 = (table row g, tokens 2 t4, 2 t4 + 1), c2, c3 = (table row g + 8, same tokens)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int v = v0 + g + 8 * (c >> 1);
                const int tok = 8 * n + 2 * t4 + (c & 1);
                if (v < V && tok < T) {
                    if (logits) logits[(size_t)tok * V + v] = acc[n][c];
                    const unsigned long long key = argmax_key(acc[n][c], v);
                    best[n][c & 1] = key > best[n][c & 1] ? key : best[n][c & 1];
                }
            }
        tile = tile_of(it + 1);
    }
    if (best_keys) {
        // lanes with the same t4 hold the same tokens: combine over g, then over the warps, one atomic per token
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                unsigned long long k = best[n][e];
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) {
                    const unsigned long long other = __shfl_xor_sync(0xffffffffu, k, o);
                    k = other > k ? other : k;
                }
                if (g == 0) s_best[warp][8 * n + 2 * t4 + e] = k;
            }
        __syncthreads();
        if (tid < 8 * NT && tid < T) {
            unsigned long long k = s_best[0][tid];
#pragma unroll
            for (int w = 1; w < kLmWarps; ++w) k = s_best[w][tid] > k ? s_best[w][tid] : k;
            atomicMax(best_keys + tid, k);
        }
    }
}

// norm_gamma / best_key may be null; best_key points at T keys (one greedy argmax per row of x, combined with
// atomicMax: the caller clears them).  Larger T is tiled here.
int lm_head_launch(int kind, const void* emb, const float* emb_scale, const float* x, float* logits,
                   int T, int V, int H, const void* norm_gamma, int gamma_is_bf16, float eps,
                   unsigned long long* best_key) {
    if (int rc = ensure_init()) return rc;
    unsigned long long* const best_key_in = best_key;
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
    if (kind == 0 && T > 1 && H % 32 == 0 && (logits || best_key)) {
        // several rows against the bf16 table: tensor-core kernel.  A CTA holds sixteen rows where their three bf16
        // terms fit the shared memory (H <= 2100), else eight; more rows than that are row blocks served side by
        // side in one launch (the kernel's `passes`), so the table is read from HBM once
        const int nt = ((size_t)3 * 16 * (H + 32) * 2 <= 200 * 1024 && T > 8) ? 2 : 1;
        const int rows_per_cta = 8 * nt;
        const int passes = (T + rows_per_cta - 1) / rows_per_cta;
        const size_t smem = (size_t)3 * rows_per_cta * (H + 32) * 2;
        LSPK_REQUIRE(smem <= 200 * 1024, "lm_head: H=%d too large for %d rows", H, rows_per_cta);
        LSPK_REQUIRE(passes <= sm_count(), "lm_head: too many rows (%d) for one launch", T);
        int per_pass = (V + 16 * kLmWarps - 1) / (16 * kLmWarps);
        if (per_pass > sm_count() / passes) per_pass = sm_count() / passes;
        const int mgrid = per_pass * passes;
        static bool attr1 = false, attr2 = false;
        cudaError_t e = cudaSuccess;
        if (nt == 1) {
            if (!attr1) e = cudaFuncSetAttribute(lm_head_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            attr1 = attr1 || e == cudaSuccess;
            if (e == cudaSuccess)
                e = launch(lm_head_mma_kernel<1>, dim3(mgrid), dim3(kLmThreads), smem, true, e4, x, logits, T, V, H, norm_gamma,
                           gamma_is_bf16, eps, best_key, passes);
        } else {
            if (!attr2) e = cudaFuncSetAttribute(lm_head_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            attr2 = attr2 || e == cudaSuccess;
            if (e == cudaSuccess)
                e = launch(lm_head_mma_kernel<2>, dim3(mgrid), dim3(kLmThreads), smem, true, e4, x, logits, T, V, H, norm_gamma,
                           gamma_is_bf16, eps, best_key, passes);
        }
        if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "lm_head (mma) launch failed: %s", cudaGetErrorString(e));
        return LSPK_OK;
    }
    // several rows with a greedy choice wanted, on the CUDA-core kernels: logits are stored and a row argmax follows
    const bool argmax_after = T > 1 && best_key != nullptr;
    LSPK_REQUIRE(!argmax_after || logits, "lm_head: several rows with argmax need a logits buffer for this table format");
    if (argmax_after) best_key = nullptr;
    unsigned long long* const keys_after = argmax_after ? const_cast<unsigned long long*>(best_key_in) : nullptr;
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
    if (keys_after) return launch_argmax_rows(logits, T, V, keys_after);
    return LSPK_OK;
}

}  // namespace lspk

extern "C" int lspk_lm_head(int kind, const void* emb, const float* emb_scale, const float* x, float* logits,
                            int T, int V, int H) {
    LSPK_REQUIRE(logits, "lspk_lm_head: null logits");
    return lspk::lm_head_launch(kind, emb, emb_scale, x, logits, T, V, H, nullptr, 0, 0.0f, nullptr);
}
