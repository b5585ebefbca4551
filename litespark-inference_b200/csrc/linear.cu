// Ternary linear layer on CUDA cores: y[m, n] = float(sum_k w[n,k] * xq[m,k]) * (xscale[m] * wscale),
// with the activation quantiser (and optionally the RMSNorm in front of it) fused in as a prologue and
// the residual add / ReLU^2 gate fused as epilogue.  The kernel is written for MT token rows per CTA
// tile; only MT = 1 (the decode GEMV) is instantiated: two and more rows go to the tensor-core kernels
// (linear_mma.cu, gemm_tc.cu), expert-grouped launches to linear_mma.cu.
//
// Replaces matmul_lut_avx512_m1 / _mT (matmul_lut_avx512_extern_c.cpp:150-236, 258-339) and,
// through the prologue / epilogue switches, quantize_activation (:425-466),
// rmsnorm_quantize_bf16gamma (:975-1048), relu2_mul_fp32 (:653-670) and add_inplace_fp32
// (:1127-1137).
//
// Work split: one CTA owns one group of 16 output rows (for the ReLU^2 pairing: row group g of
// the gate matrix and of the up matrix).  Lanes 0-15 / 16-31 of a warp hold the 16 rows for an
// even / odd 64-weight chunk, so every warp-wide 16-byte load is one contiguous 512-byte span
// of the device layout.  The 8 warps stride over the chunks of the row group.  A lane decodes
// a packed word with four masks (no shifts): the four 2-bit fields stay at their bit offset
// and are accumulated in four separate int32 sums that are scaled back by exact shifts at the
// end.  Like the reference the codes stay unsigned {0,1,2}; sum(x) is subtracted once per row.
#include <stdlib.h>

#include "internal.cuh"
#include "ternary_core.cuh"

namespace lspk {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

// Reductions over the eight warps of a CTA.  One barrier each: the result is read back from `slot`
// (8 floats, 16-byte aligned) by every thread, so two consecutive reductions need two slots.
static_assert(kWarps == 8, "cta8_* reductions assume eight warps");
__device__ __forceinline__ float cta8_sum(float v, float* slot) {
    v = warp_sum(v);
    if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
    __syncthreads();
    const float4 a = *reinterpret_cast<const float4*>(slot), b = *reinterpret_cast<const float4*>(slot + 4);
    return ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
}
// v >= 0: non-negative floats order like their bit patterns, so the warp stage is one integer redux
__device__ __forceinline__ float cta8_max_nonneg(float v, float* slot) {
    const uint32_t u = __reduce_max_sync(0xffffffffu, __float_as_uint(v));
    if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = __uint_as_float(u);
    __syncthreads();
    const float4 a = *reinterpret_cast<const float4*>(slot), b = *reinterpret_cast<const float4*>(slot + 4);
    return fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
}

// MT      token rows per CTA tile
// NI      16-byte weight loads per lane per batch (covers K <= 4096 at 4, K <= 8192 at 8 in one batch)
// NB      16-element activation blocks a thread owns in the fp32 prologue (K <= 4096 * NB)
// PAIR    gate/up pairing (two weight streams, gated epilogue)
// GROUPED expert-grouped launch: blockIdx.z is the expert; its row list and row count are read from
//         device arrays, its weights and scales are found by stride (packed-expert MoE GEMV)
template <int MT, int NI, int NB, bool PAIR, bool GROUPED>
#ifdef LSPK_LINEAR_MIN_BLOCKS
__global__ void __launch_bounds__(kThreads, LSPK_LINEAR_MIN_BLOCKS)
#else
__global__ void __launch_bounds__(kThreads)
#endif
ternary_linear_kernel(const __grid_constant__ LinearParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int Kp = p.chunks * kWeightsPerChunk;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane & 15, h = lane >> 4;

    int8_t* xq = reinterpret_cast<int8_t*>(smem_raw);                 // [MT][Kp] permuted int8
    int* part = reinterpret_cast<int*>(xq + (size_t)MT * Kp);          // [PAIR?2:1][warps][MT][16]
    constexpr int kPartInts = kWarps * MT * 16 * (PAIR ? 2 : 1);
    float* redf = reinterpret_cast<float*>(part + kPartInts);          // [32] reduction scratch
    float* s_scale = redf + 32;                                        // [MT]
    int* s_sumx = reinterpret_cast<int*>(s_scale + MT);                // [MT][warps] partial sums of x
    const int z = GROUPED ? blockIdx.z : 0;
    const size_t w_off = GROUPED ? (size_t)z * p.grp_w_stride : 0;

    // ---- row groups of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ... (flat over the segments) ----
    auto locate = [&](int flat, int& seg_i, int& grp) {
        seg_i = 0;
        grp = flat;
        if (!PAIR) {
            while (seg_i < p.n_seg - 1 && grp >= p.seg[seg_i].groups) {
                grp -= p.seg[seg_i].groups;
                ++seg_i;
            }
        }
    };
    auto load_batch = [&](int seg_i, int grp, int base, uint4* dst_a, uint4* dst_b) {
        const uint4* wa_base = p.seg[seg_i].w + w_off + (size_t)grp * p.chunks * kRowsPerGroup + r;
        const uint4* wb_base = PAIR ? (p.seg[1].w + w_off + (size_t)grp * p.chunks * kRowsPerGroup + r) : nullptr;
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const int j = 2 * (warp + kWarps * (base + i)) + h;
            if (j < p.chunks) {
                // read-once weights bypass the L2 replacement queue so that the KV cache, the
                // activations and the norm weights stay resident from token to token
                if (p.stream_weights) {
                    dst_a[i] = __ldcs(wa_base + (size_t)j * kRowsPerGroup);
                    if (PAIR) dst_b[i] = __ldcs(wb_base + (size_t)j * kRowsPerGroup);
                } else {
                    dst_a[i] = __ldg(wa_base + (size_t)j * kRowsPerGroup);
                    if (PAIR) dst_b[i] = __ldg(wb_base + (size_t)j * kRowsPerGroup);
                }
            }
        }
    };
    PhaseTrace tr;
    tr.begin(p.trace, p.trace_cap, 1);
    tr.mark();                                   // 0: entry
    const int pairs = (p.chunks + 1) / 2;
    const bool one_batch = kWarps * NI >= pairs;     // a row group's weights fit one register batch
    const bool fp32_in = p.prologue != LSPK_PRO_INT8;
    const bool normed = p.prologue == LSPK_PRO_RMSNORM_QUANT || p.prologue == LSPK_PRO_GATED_RMSNORM_QUANT;

    int flat0 = blockIdx.x, s0, g0;
    locate(flat0, s0, g0);

    // ---- everything that does not depend on the previous kernel is requested first: the first
    //      batch of packed weights and the norm weights (neither is written by the forward pass).
    //      An expert-grouped launch cannot: whether this expert has any row is device data. ----
    uint4 wa[NI], wb[PAIR ? NI : 1];
    uint4 na[NI], nb_[PAIR ? NI : 1];                // the next row group's first batch
    if (!GROUPED) load_batch(s0, g0, 0, wa, wb);
    float gm[NB][16];
    if (normed) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            const int k0 = (tid + nb * kThreads) * 16;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int k = k0 + q * 4;
                float4 gv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (k < p.K) {
                    if (p.gamma_is_bf16) {
                        const uint2 gb = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p.gamma) + k));
                        gv.x = __uint_as_float(gb.x << 16);
                        gv.y = __uint_as_float(gb.x & 0xffff0000u);
                        gv.z = __uint_as_float(gb.y << 16);
                        gv.w = __uint_as_float(gb.y & 0xffff0000u);
                    } else {
                        gv = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.gamma) + k));
                    }
                }
                gm[nb][q * 4 + 0] = gv.x;
                gm[nb][q * 4 + 1] = gv.y;
                gm[nb][q * 4 + 2] = gv.z;
                gm[nb][q * 4 + 3] = gv.w;
            }
        }
    }
    grid_dependency_launch();
    grid_dependency_wait();
    tr.mark();                                   // 1: predecessor finished

    const int M_eff = GROUPED ? p.grp_counts[z] : p.M;
    const int* rows = GROUPED ? p.grp_rows + (size_t)z * p.grp_rows_stride : nullptr;
    const int out_m = tid >> 4, out_r = tid & 15;
    const int tail_start = p.K & ~15;      // the reference's scalar-tail rounding rule applies from here
    bool first_tile = true;

    // Plain launches give every row tile its own CTA (grid.y), so this loop runs once for them (and the
    // compiler is told so: register lifetimes end with the single pass); expert-grouped launches, whose
    // row count is device data, walk their tiles here.
    for (int m0 = blockIdx.y * MT; m0 < M_eff; m0 += gridDim.y * MT) {
        const int mt = min(MT, M_eff - m0);
        auto out_row = [&](int m) -> int { return GROUPED ? rows[m0 + m] : m0 + m; };
        auto in_row = [&](int m) -> int { return GROUPED ? (rows[m0 + m] >> p.grp_in_shift) : m0 + m; };
        int flat = flat0, s = s0, g = g0;
        // residual value of this thread's output element (ADD epilogue), requested as early as possible
        auto residual_of = [&](int seg_i, int grp) -> float {
            if (p.epilogue != LSPK_EPI_ADD || tid >= MT * 16 || out_m >= mt) return 0.0f;
            const int n = grp * kRowsPerGroup + out_r;
            if (n >= p.seg[seg_i].N) return 0.0f;
            return p.seg[seg_i].out[(size_t)out_row(out_m) * p.seg[seg_i].N + n];
        };
        float resid = residual_of(s, g);
        if (GROUPED || !first_tile) load_batch(s, g, 0, wa, wb);
        first_tile = false;

        // ---- prologue: this tile's activations -> permuted int8 rows in shared memory ---------------
        for (int m = 0; m < mt; ++m) {
            int8_t* xq_row = xq + (size_t)m * Kp;
            int sumx = 0;
            float scale = 1.0f;
            if (!fp32_in) {
                const int8_t* src = p.x_i8 + (size_t)in_row(m) * p.K;
                for (int b = tid; b < Kp / 16; b += kThreads) {
                    uint32_t a[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int k = b * 16 + q * 4;
                        a[q] = (k < p.K) ? *reinterpret_cast<const uint32_t*>(src + k) : 0u;
                        sumx = __dp4a((int)a[q], 0x01010101, sumx);
                    }
                    uint32_t o0, o1, o2, o3;
                    transpose4x4_bytes(a[0], a[1], a[2], a[3], o0, o1, o2, o3);
                    *reinterpret_cast<uint4*>(xq_row + b * 16) = make_uint4(o0, o1, o2, o3);
                }
                scale = p.x_scales[in_row(m)];
            } else {
                // every thread keeps its 16-element blocks in registers through all three passes
                const float* src = p.x_f32 + (size_t)in_row(m) * p.K;
                float v[NB][16];
                float ssq = 0.0f;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int k0 = (tid + nb * kThreads) * 16;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (k0 + q * 4 < p.K) t4 = *reinterpret_cast<const float4*>(src + k0 + q * 4);
                        v[nb][q * 4 + 0] = t4.x;
                        v[nb][q * 4 + 1] = t4.y;
                        v[nb][q * 4 + 2] = t4.z;
                        v[nb][q * 4 + 3] = t4.w;
                    }
                }
                if (p.prologue == LSPK_PRO_GATED_RMSNORM_QUANT) {
                    // v = x * SiLU(gate), SiLU(g) = g / (1 + exp(-g)); each step a single rounding
                    const float* gsrc = p.gate_f32 + (size_t)in_row(m) * p.K;
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const int k0 = (tid + nb * kThreads) * 16;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            float4 t4 = make_float4(0.f, 0.f, 0.f, 0.f);
                            if (k0 + q * 4 < p.K) t4 = *reinterpret_cast<const float4*>(gsrc + k0 + q * 4);
                            const float gg[4] = {t4.x, t4.y, t4.z, t4.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float sg = __fdiv_rn(gg[e], __fadd_rn(expf(-gg[e]), 1.0f));
                                v[nb][q * 4 + e] = __fmul_rn(v[nb][q * 4 + e], sg);
                            }
                        }
                    }
                }
                if (normed) {
                    float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
                        for (int e = 0; e < 16; ++e) ss[e & 3] = fmaf(v[nb][e], v[nb][e], ss[e & 3]);
                    tr.mark();                       // 2: x arrived, local squares summed
                    ssq = cta8_sum((ss[0] + ss[1]) + (ss[2] + ss[3]), redf);
                    tr.mark();                       // 3: sum of squares reduced
                    // __frcp_rn is the correctly rounded reciprocal, i.e. exactly 1.0f / x
                    const float mean = p.rcp_K != 0.0f ? div_const_rn(ssq, (float)p.K, p.rcp_K) : __fdiv_rn(ssq, (float)p.K);
                    const float rrms = rcp_rn(__fsqrt_rn(__fadd_rn(mean, p.eps)));
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
                tr.mark();                           // 4: normalised, local absmax
                amax = cta8_max_nonneg(amax, redf + 8);
                tr.mark();                           // 5: absmax reduced
                scale = quant_scale_from_absmax(amax);
                const float inv = rcp_rn(scale);
                const bool tap = (p.xq_out != nullptr) && blockIdx.x == 0;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int b = tid + nb * kThreads;
                    const int k0 = b * 16;
                    if (k0 < Kp) {
                        uint32_t o0, o1, o2, o3;
                        if (k0 + 16 <= tail_start) {
                            // |v * inv| <= 127 by construction of inv, so the saturation of the reference's
                            // conversion never acts and round-to-nearest-even can be taken from the adder:
                            // v + 1.5 * 2^23 leaves the integer in the low mantissa byte.  The words are
                            // packed directly in the transposed order the dot products read.
                            uint32_t t[16];
#pragma unroll
                            for (int e = 0; e < 16; ++e)
                                t[e] = __float_as_uint(__fadd_rn(__fmul_rn(v[nb][e], inv), 12582912.0f));
                            o0 = pack4_bytes(t[0], t[4], t[8], t[12]);
                            o1 = pack4_bytes(t[1], t[5], t[9], t[13]);
                            o2 = pack4_bytes(t[2], t[6], t[10], t[14]);
                            o3 = pack4_bytes(t[3], t[7], t[11], t[15]);
                            if (tap) {
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    *reinterpret_cast<uint32_t*>(p.xq_out + (size_t)out_row(m) * p.K + k0 + q * 4) =
                                        pack4_bytes(t[q * 4], t[q * 4 + 1], t[q * 4 + 2], t[q * 4 + 3]);
                            }
                        } else {
                            // block that reaches past the last multiple of 16: the reference's scalar tail
                            // (round half away from zero, clamp to +-127), zeros beyond K
                            uint32_t a[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t word = 0;
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int k = k0 + q * 4 + e;
                                    int qv = 0;
                                    if (k < tail_start) {
                                        qv = (int)quant_rne_sat(__fmul_rn(v[nb][q * 4 + e], inv));
                                    } else if (k < p.K) {
                                        qv = max(-127, min(127, (int)roundf(__fmul_rn(v[nb][q * 4 + e], inv))));
                                    }
                                    word |= ((uint32_t)qv & 0xffu) << (8 * e);
                                }
                                a[q] = word;
                                if (tap && k0 + q * 4 < p.K)
                                    *reinterpret_cast<uint32_t*>(p.xq_out + (size_t)out_row(m) * p.K + k0 + q * 4) = word;
                            }
                            transpose4x4_bytes(a[0], a[1], a[2], a[3], o0, o1, o2, o3);
                        }
                        sumx = __dp4a((int)o0, 0x01010101, sumx);
                        sumx = __dp4a((int)o1, 0x01010101, sumx);
                        sumx = __dp4a((int)o2, 0x01010101, sumx);
                        sumx = __dp4a((int)o3, 0x01010101, sumx);
                        *reinterpret_cast<uint4*>(xq_row + k0) = make_uint4(o0, o1, o2, o3);
                    }
                }
            }
            // sum(x): per-warp partials; the output threads add the eight of them
            sumx = __reduce_add_sync(0xffffffffu, sumx);
            if (lane == 0) s_sumx[m * kWarps + warp] = sumx;
            if (tid == 0) {
                s_scale[m] = scale;
                if (p.xscale_out && blockIdx.x == 0) p.xscale_out[out_row(m)] = scale;
            }
        }
        tr.mark();                                   // 6: quantised rows written
        __syncthreads();
        tr.mark();                                   // 7: activations visible to all warps

        // ---- loop over this CTA's row groups: integer dot products, reduction, epilogue ----------------
        while (true) {
            const int next_flat = flat + gridDim.x;
            const bool has_next = next_flat < p.total_groups;
            int ns = 0, ng = 0;
            float next_resid = 0.0f;
            if (has_next) {
                locate(next_flat, ns, ng);
                if (one_batch) load_batch(ns, ng, 0, na, nb_);       // in flight while this group is computed
                next_resid = residual_of(ns, ng);
            }

            int acc_a[MT][4], acc_b[PAIR ? MT : 1][4];
#pragma unroll
            for (int m = 0; m < MT; ++m)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    acc_a[m][c] = 0;
                    if (PAIR) acc_b[m][c] = 0;
                }
            for (int base = 0;; ) {
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int j = 2 * (warp + kWarps * (base + i)) + h;
                    if (j < p.chunks) {
#pragma unroll
                        for (int m = 0; m < MT; ++m) {
                            if (MT == 1 || m < mt) {
                                const int4* xp = reinterpret_cast<const int4*>(xq + (size_t)m * Kp + (size_t)j * 64);
                                chunk_dot(wa[i], xp, acc_a[m]);
                                if (PAIR) chunk_dot(wb[i], xp, acc_b[m]);
                            }
                        }
                    }
                }
                base += NI;
                if (kWarps * base >= pairs) break;
                load_batch(s, g, base, wa, wb);
            }

            tr.mark();                               // 8+: dot products of a row group done
            // fields -> one int, odd/even chunk halves by shuffle, warps through shared memory
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                int v = acc_a[m][0] + (acc_a[m][1] >> 2) + (acc_a[m][2] >> 4) + (acc_a[m][3] >> 6);
                v += __shfl_down_sync(0xffffffffu, v, 16);
                if (h == 0) part[(warp * MT + m) * 16 + r] = v;
                if (PAIR) {
                    int u = acc_b[m][0] + (acc_b[m][1] >> 2) + (acc_b[m][2] >> 4) + (acc_b[m][3] >> 6);
                    u += __shfl_down_sync(0xffffffffu, u, 16);
                    if (h == 0) part[kWarps * MT * 16 + (warp * MT + m) * 16 + r] = u;
                }
            }
            __syncthreads();

            if (tid < MT * 16) {
                const LinearSeg& sg = p.seg[s];
                const int n = g * kRowsPerGroup + out_r;
                if (out_m < mt && n < sg.N) {
                    int va = 0, vb = 0, sx = 0;
#pragma unroll
                    for (int w = 0; w < kWarps; ++w) {
                        va += part[(w * MT + out_m) * 16 + out_r];
                        if (PAIR) vb += part[kWarps * MT * 16 + (w * MT + out_m) * 16 + out_r];
                        sx += s_sumx[out_m * kWarps + w];
                    }
                    va -= sx;
                    const size_t o = (size_t)out_row(out_m) * sg.N + n;
                    if (sg.acc_out) sg.acc_out[o] = va;
                    const float wsa = GROUPED ? p.grp_scales[z * 3 + sg.scale_idx] : sg.w_scale;
                    const float ya = __fmul_rn((float)va, __fmul_rn(s_scale[out_m], wsa));
                    if (PAIR) {
                        vb -= sx;
                        if (p.seg[1].acc_out) p.seg[1].acc_out[o] = vb;
                        const float wsb = GROUPED ? p.grp_scales[z * 3 + p.seg[1].scale_idx] : p.seg[1].w_scale;
                        const float yb = __fmul_rn((float)vb, __fmul_rn(s_scale[out_m], wsb));
                        if (p.epilogue == LSPK_EPI_SILU_MUL) {
                            // the reference's Falcon gate (runtime.py:726-732): g / (1 + exp(-g)) * u
                            sg.out[o] = __fmul_rn(__fdiv_rn(ya, __fadd_rn(expf(-ya), 1.0f)), yb);
                        } else {
                            const float gpos = fmaxf(ya, 0.0f);
                            sg.out[o] = __fmul_rn(__fmul_rn(gpos, gpos), yb);
                        }
                    } else if (p.epilogue == LSPK_EPI_ADD) {
                        sg.out[o] = __fadd_rn(resid, ya);
                    } else {
                        sg.out[o] = ya;
                    }
                }
            }
            tr.mark();                               // 9+: row group reduced and stored
            __syncthreads();                         // `part` (and, at the end of a tile, xq) is rewritten next
            if (!has_next) break;
            flat = next_flat;
            s = ns;
            g = ng;
            resid = next_resid;
            if (one_batch) {
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    wa[i] = na[i];
                    if (PAIR) wb[i] = nb_[i];
                }
            } else {
                load_batch(s, g, 0, wa, wb);
            }
        }
        if (!GROUPED) break;
    }
    tr.end();
}

static size_t linear_smem_bytes(int MT, int Kp, bool pair) {
    size_t b = (size_t)MT * Kp;
    b += (size_t)kWarps * MT * 16 * (pair ? 2 : 1) * 4;
    b += 32 * 4 + MT * 4 + MT * kWarps * 4;
    return b;
}
template <int MT, int NI, int NB, bool PAIR, bool GROUPED>
static cudaError_t launch_linear(const LinearParams& p, dim3 grid, size_t smem) {
    static bool attr_set = false;
    auto kern = ternary_linear_kernel<MT, NI, NB, PAIR, GROUPED>;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    return launch(kern, grid, dim3(kThreads), smem, true, p);
}

template <int MT>
static cudaError_t launch_linear_mt(const LinearParams& p, dim3 grid, bool pair, size_t smem) {
    if (p.chunks <= 64)
        return pair ? launch_linear<MT, 4, 1, true, false>(p, grid, smem) : launch_linear<MT, 4, 1, false, false>(p, grid, smem);
    if (p.chunks <= 128)
        return pair ? launch_linear<MT, 8, 2, true, false>(p, grid, smem) : launch_linear<MT, 8, 2, false, false>(p, grid, smem);
    return pair ? launch_linear<MT, 8, 8, true, false>(p, grid, smem) : launch_linear<MT, 8, 8, false, false>(p, grid, smem);
}

int linear_launch_params(const LinearParams& p, int mt, bool pair, bool grouped, int grid_x, int grid_y, int grid_z) {
    // more than one token row per tile (and every expert-grouped launch): the eight-row mma kernel
    if (mt > 1 || grouped) return linear_mma_launch(p, pair, grouped, grid_x, grid_y, grid_z);
    const int Kp = p.chunks * kWeightsPerChunk;
    const size_t smem = linear_smem_bytes(1, Kp, pair);
    LSPK_REQUIRE(smem <= 200 * 1024 && p.chunks <= 512, "linear: K=%d too large (limit 32768)", p.K);
    const dim3 grid(grid_x, grid_y, grid_z);
    const cudaError_t e = launch_linear_mt<1>(p, grid, pair, smem);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "linear launch failed: %s", cudaGetErrorString(e));
    return LSPK_OK;
}

// Host-side validation + launch of the CUDA-core kernel.  Used by lspk_linear and by the
// forward pass.
int linear_cuda_core(const lspk_linear_args* a) {
    LSPK_REQUIRE(a, "linear: null args");
    LSPK_REQUIRE(a->n_mats >= 1 && a->n_mats <= 3, "linear: n_mats must be 1..3 (got %d)", a->n_mats);
    LSPK_REQUIRE(a->M >= 1, "linear: M must be >= 1 (got %d)", a->M);
    const bool pair = a->epilogue == LSPK_EPI_RELU2_MUL || a->epilogue == LSPK_EPI_SILU_MUL;
    LSPK_REQUIRE(!pair || a->n_mats == 2, "linear: the gated epilogues take exactly two matrices (gate, up)");
    LinearParams p = {};
    const Weight* w0 = reinterpret_cast<const Weight*>(a->w[0]);
    LSPK_REQUIRE(w0, "linear: null weight");
    // Several rows of fp32 input: normalise + quantise them once in their own kernel (fused into the
    // product, every CTA would repeat that work for all rows) and continue with the int8 prologue.
    lspk_linear_args split;
    const int* tiled_sums = nullptr;
    if (a->M > 1 && a->prologue != LSPK_PRO_INT8) {
        LSPK_REQUIRE(a->prologue >= LSPK_PRO_QUANT && a->prologue <= LSPK_PRO_GATED_RMSNORM_QUANT,
                     "linear: unknown prologue %d", a->prologue);
        LSPK_REQUIRE(a->x_f32, "linear: fp32 prologue needs x_f32");
        LSPK_REQUIRE(a->prologue == LSPK_PRO_QUANT || a->gamma, "linear: RMSNORM_QUANT prologue needs gamma");
        LSPK_REQUIRE(a->prologue != LSPK_PRO_GATED_RMSNORM_QUANT || a->gate_f32,
                     "linear: GATED_RMSNORM_QUANT prologue needs gate_f32");
        split = *a;
        int8_t* q = nullptr;
        float* sc = nullptr;
        int* sums = nullptr;
        const int Kp = w0->chunks * kWeightsPerChunk, rs = mma_row_stride(Kp);
        if (int rc = quant_scratch((size_t)a->M, (size_t)rs, &q, &sc, &sums)) return rc;
        int tiled = 0;
        // below the tensor-core GEMM's threshold the rows go to the eight-row kernel: quantise them straight into
        // its tile layout (a plain copy there); the natural-order rows are produced only when the caller wants them
        if (!a->xq_out)
            if (int rc = quantize_rows_permuted(a, w0->K, Kp, q, sc, &tiled, rs, sums)) return rc;
        if (tiled) {
            split.prologue = kProInt8Tiled;
            split.x_i8 = q;
            split.x_scales = sc;
            split.x_f32 = nullptr;
            split.gate_f32 = nullptr;
            tiled_sums = sums;
        } else {
            if (int rc = split_row_prologue(&split, w0->K, q, sc)) return rc;
            if (a->xq_out) LSPK_CUDA(cudaMemcpyAsync(a->xq_out, q, (size_t)a->M * w0->K, cudaMemcpyDeviceToDevice, stream()));
        }
        if (a->xscale_out) LSPK_CUDA(cudaMemcpyAsync(a->xscale_out, sc, (size_t)a->M * 4, cudaMemcpyDeviceToDevice, stream()));
        split.xq_out = nullptr;
        split.xscale_out = nullptr;
        a = &split;
    }
    p.K = w0->K;
    p.chunks = w0->chunks;
    p.n_seg = a->n_mats;
    int groups = 0;
    for (int i = 0; i < a->n_mats; ++i) {
        const Weight* w = reinterpret_cast<const Weight*>(a->w[i]);
        LSPK_REQUIRE(w && w->K == p.K, "linear: matrices must share K");
        LSPK_REQUIRE(pair ? (i == 1 || a->out[i] != nullptr) : a->out[i] != nullptr, "linear: null output");
        LSPK_REQUIRE(!pair || w->N == w0->N, "linear: gate and up must have the same N");
        p.seg[i] = LinearSeg{w->dev, a->out[i], a->acc_out[i], w->N, w->groups, w->scale, i};
        groups += w->groups;
    }
    if (pair) groups = w0->groups;
    p.total_groups = groups;
    p.M = a->M;
    p.prologue = a->prologue;
    p.epilogue = a->epilogue;
    p.x_f32 = a->x_f32;
    p.rcp_K = fma_division_ok((float)w0->K) ? 1.0f / (float)w0->K : 0.0f;
    p.gate_f32 = a->gate_f32;
    p.x_i8 = a->x_i8;
    p.x_scales = a->x_scales;
    p.x_sums = tiled_sums;
    p.gamma = a->gamma;
    p.gamma_is_bf16 = a->gamma_is_bf16;
    p.eps = a->eps;
    p.xq_out = a->xq_out;
    p.xscale_out = a->xscale_out;
    p.trace = trace_buffer();
    p.trace_cap = trace_capacity();
    p.error_flag = device_wait_flag();
    switch (a->prologue) {
        case kProInt8Tiled:                      // set above, never by a caller
            LSPK_REQUIRE(tiled_sums != nullptr, "linear: unknown prologue %d", a->prologue);
            break;
        case LSPK_PRO_INT8:
            LSPK_REQUIRE(a->x_i8 && a->x_scales, "linear: INT8 prologue needs x_i8 and x_scales");
            break;
        case LSPK_PRO_GATED_RMSNORM_QUANT:
            LSPK_REQUIRE(a->gate_f32, "linear: GATED_RMSNORM_QUANT prologue needs gate_f32");
            /* fallthrough */
        case LSPK_PRO_RMSNORM_QUANT:
            LSPK_REQUIRE(a->gamma, "linear: RMSNORM_QUANT prologue needs gamma");
            /* fallthrough */
        case LSPK_PRO_QUANT:
            LSPK_REQUIRE(a->x_f32, "linear: fp32 prologue needs x_f32");
            break;
        default:
            return fail(LSPK_ERR_ARG, "linear: unknown prologue %d", a->prologue);
    }
    LSPK_REQUIRE(a->epilogue >= 0 && a->epilogue <= 3, "linear: unknown epilogue %d", a->epilogue);
    const int MT = a->M == 1 ? 1 : 8;
    // At most two CTAs per SM when there is a single token tile (measured best on B200: the prologue
    // runs once per CTA, which then loops over its row groups).  With several token tiles the grid's
    // second dimension already fills the machine.
    const int tiles = (a->M + MT - 1) / MT;
    p.stream_weights = tiles == 1 ? 1 : 0;
    int ctas = groups;
    const int per_wave = tiles == 1 ? 2 * sm_count() : (2 * sm_count() + tiles - 1) / tiles;
    if (ctas > per_wave) ctas = per_wave > 0 ? per_wave : 1;
    return linear_launch_params(p, MT, pair, false, ctas, tiles, 1);
}

}  // namespace lspk

using namespace lspk;

static int g_force_path = 0;   // 0 auto, 1 CUDA-core only, 2 tensor-core only

extern "C" int lspk_linear_force_path(int path) {
    LSPK_REQUIRE(path >= 0 && path <= 2, "lspk_linear_force_path: path must be 0, 1 or 2");
    g_force_path = path;
    return LSPK_OK;
}

extern "C" int lspk_linear(const lspk_linear_args* a) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(a, "lspk_linear: null args");
    if (a->prologue != LSPK_PRO_INT8) {
        LSPK_REQUIRE(((uintptr_t)a->x_f32 & 15) == 0 && ((uintptr_t)a->gate_f32 & 15) == 0,
                     "lspk_linear: x_f32 / gate_f32 must be 16-byte aligned");
        LSPK_REQUIRE((a->prologue != LSPK_PRO_RMSNORM_QUANT && a->prologue != LSPK_PRO_GATED_RMSNORM_QUANT) ||
                         ((uintptr_t)a->gamma & (a->gamma_is_bf16 ? 7 : 15)) == 0,
                     "lspk_linear: gamma must be 8-byte (bf16) / 16-byte (fp32) aligned");
    } else {
        LSPK_REQUIRE(((uintptr_t)a->x_i8 & 3) == 0, "lspk_linear: x_i8 must be 4-byte aligned");
    }
    if (g_force_path != 1) {
        int handled = 0;
        if (int rc = linear_tensor_core(a, &handled)) return rc;
        if (handled) return LSPK_OK;
        if (g_force_path == 2) return fail(LSPK_ERR_ARG, "lspk_linear: shape not supported by the tensor-core path");
    }
    return linear_cuda_core(a);
}
