// Ternary linear layer for 2..8 int8 token rows per tile on the warp-level int8 tensor-core path
// (mma.sync.m16n8k32.u8.s8): the weights of a 16-row group are the MMA's M side, up to eight
// token rows its N side, so streaming a packed matrix once serves eight tokens for the instruction
// count the one-token kernel spends on one.  Same contract and epilogues as
// ternary_linear_kernel in linear.cu (matmul_lut_avx512_mT, matmul_lut_avx512_extern_c.cpp:258-339,
// plus the fused helpers); this is the path of the small batches: speculative validation, several
// sequences decoded in lock step, the rows an expert receives in the MoE layer.
//
// Operand mapping (no re-layout: the device chunk layout is read as is).  The 256-byte tile of
// "16 rows x one 64-weight chunk" is 64 words; lane l of a warp loads word l (row l/4, the
// (l%4)-th 16-weight word of the chunk) and word 32+l (row l/4 + 8).  Masking a packed word with
// 0x03030303 << 2j leaves four codes (weights 16t + {j, 4+j, 8+j, 12+j}, scaled by 4^j) in the
// byte positions of an A-fragment register; two consecutive chunks give the two K halves of one
// m16n8k32 step.  The int8 activations sit in shared memory in the same transposed 16-element
// blocks the one-token kernel uses, so lane (token l/4, word l%4) gets its four B registers for
// the four masks with one 16-byte load per chunk.  One accumulator set per mask keeps the scales
// apart; they are combined with exact shifts at the end.  Codes stay unsigned, sum(x) is
// subtracted per row: all integer, bit-exact.
#include <stdlib.h>

#include "internal.cuh"
#include "ternary_core.cuh"

namespace lspk {

constexpr int kMThreads = 256;
constexpr int kMWarps = kMThreads / 32;
constexpr int kMT = 8;            // token rows per tile (the MMA's N)
constexpr int kMNI = 4;           // chunk pairs whose weights a lane keeps in flight

__device__ __forceinline__ void mma_u8s8(int c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Row stride of the activation tile in shared memory (mma_row_stride, internal.cuh): Kp rounded so that
// consecutive rows start 64 bytes apart modulo 128, which makes the quarter-warp 16-byte loads (two tokens x
// four words) conflict-free.

// BULK: the packed weights of the CTA's row groups arrive in a shared-memory ring by bulk asynchronous copies
// (one thread requests up to p.bulk_stages groups ahead, each a contiguous block of the device layout) instead of
// per-lane register loads.  For launches that stream tens of megabytes (the expert-grouped MoE products): the
// bytes in flight per SM then do not depend on registers or on where the CTA is in its reduction.
constexpr int kMBulkStages = 4;
constexpr int kMIssuers = 4;                          // warps whose lane 0 requests a quarter of each stage
constexpr unsigned kMBulkSpinLimit = 1u << 22;
// Pre-tiled int8 rows (the row quantiser's output, already in the tile's layout) arrive by bulk copies in
// segments of 16 chunks along K, one mbarrier per segment, so the MMAs of the first segment start while the
// later ones are still on their way; every wait on a segment ends at a clock deadline.
constexpr int kMXSegChunks = 16;                     // chunks per segment = what the 8 warps consume per step
constexpr int kMXSegMax = 24;                        // covers K up to 24576
constexpr long long kMXWaitCycles = 1ll << 31;
static_assert(kMWarps == kMT && kMXSegMax <= 32, "row staging maps warp -> row and lane -> segment");

template <bool PAIR, bool GROUPED, bool BULK>
__global__ void __launch_bounds__(kMThreads)
ternary_linear_mma_kernel(const __grid_constant__ LinearParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int Kp = p.chunks * kWeightsPerChunk;
    const int rs = mma_row_stride(Kp);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gid = lane >> 2, t4 = lane & 3;

    int8_t* xq = reinterpret_cast<int8_t*>(smem_raw);                         // [kMT][rs] permuted int8
    int* part = reinterpret_cast<int*>(xq + (size_t)kMT * rs);                 // [PAIR?2:1][warps][kMT][16]
    constexpr int kPartInts = kMWarps * kMT * 16 * (PAIR ? 2 : 1);
    float* s_scale = reinterpret_cast<float*>(part + kPartInts);               // [kMT]
    int* s_sumx = reinterpret_cast<int*>(s_scale + kMT);                       // [kMT]
    unsigned char* ring_base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(s_sumx + kMT) + 127) & ~uintptr_t(127));
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_base);                   // [kMBulkStages]
    uint32_t* ring = reinterpret_cast<uint32_t*>(ring_base + 128);             // [stages][PAIR?2:1][chunks*64 words]
    const int grp_words = p.chunks * 64;
    const int stage_words = grp_words * (PAIR ? 2 : 1);

    const int z = GROUPED ? blockIdx.z : 0;
    const size_t w_off = GROUPED ? (size_t)z * p.grp_w_stride : 0;
    const int pairs = (p.chunks + 1) / 2;

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
    // weights of chunk pair (warp + 8*(base+i)) of a row group: for each of the two chunks the words of
    // row gid and of row gid+8 -> 4 words per pair (8 with the gate/up pairing)
    auto load_batch = [&](int seg_i, int grp, int base, uint32_t (*dst_a)[4], uint32_t (*dst_b)[4]) {
        const uint32_t* wa = reinterpret_cast<const uint32_t*>(p.seg[seg_i].w + w_off + (size_t)grp * p.chunks * kRowsPerGroup);
        const uint32_t* wb = PAIR ? reinterpret_cast<const uint32_t*>(p.seg[1].w + w_off + (size_t)grp * p.chunks * kRowsPerGroup)
                                  : nullptr;
#pragma unroll
        for (int i = 0; i < kMNI; ++i) {
            const int pr = warp + kMWarps * (base + i);
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int j = 2 * pr + c;
                uint32_t a_lo = 0x55555555u, a_hi = 0x55555555u, b_lo = 0x55555555u, b_hi = 0x55555555u;
                if (j < p.chunks) {
                    const size_t o = (size_t)j * 64 + lane;           // 64 words per 16-row chunk tile
                    if (p.stream_weights) {
                        a_lo = __ldcs(wa + o);
                        a_hi = __ldcs(wa + o + 32);
                        if (PAIR) { b_lo = __ldcs(wb + o); b_hi = __ldcs(wb + o + 32); }
                    } else {
                        a_lo = __ldg(wa + o);
                        a_hi = __ldg(wa + o + 32);
                        if (PAIR) { b_lo = __ldg(wb + o); b_hi = __ldg(wb + o + 32); }
                    }
                }
                dst_a[i][c * 2] = a_lo;
                dst_a[i][c * 2 + 1] = a_hi;
                if (PAIR) {
                    dst_b[i][c * 2] = b_lo;
                    dst_b[i][c * 2 + 1] = b_hi;
                }
            }
        }
    };

    int flat0 = blockIdx.x, s0, g0;
    locate(flat0, s0, g0);
    uint32_t wa[kMNI][4], wb[PAIR ? kMNI : 1][4];
    PhaseTrace tr;
    tr.begin(p.trace, p.trace_cap, 3);
    tr.mark();                                          // 0: entry
    if (!GROUPED && !BULK) load_batch(s0, g0, 0, wa, wb);       // weights never depend on the previous kernel
    __shared__ __align__(8) uint64_t xbars[kMXSegMax];
    const int nxseg = (p.chunks + kMXSegChunks - 1) / kMXSegChunks;
    // CTA-uniform: a full tile of pre-tiled rows, one token tile per CTA
    const bool x_async = !GROUPED && !BULK && p.prologue == kProInt8Tiled && nxseg <= kMXSegMax &&
                         p.M - (int)blockIdx.y * kMT >= kMT;
    if (x_async) {
        if (tid < nxseg) {
            mbar_init(&xbars[tid], kMT);
            fence_mbar_init();
        }
        __syncthreads();
    }
    grid_dependency_launch();
    grid_dependency_wait();
    tr.mark();                                          // 1: predecessor finished

    const int M_eff = GROUPED ? p.grp_counts[z] : p.M;
    const int* rows = GROUPED ? p.grp_rows + (size_t)z * p.grp_rows_stride : nullptr;
    const int out_m = tid >> 4, out_r = tid & 15;
    bool first_tile = true;

    // BULK: the CTA's work as one sequence: for every token tile, every row group of this CTA
    const int ngrp_cta = (int)blockIdx.x < p.total_groups ? (p.total_groups - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int tile_step = (int)gridDim.y * kMT;
    const int ntile_cta = M_eff > (int)blockIdx.y * kMT ? (M_eff - 1 - (int)blockIdx.y * kMT) / tile_step + 1 : 0;
    const int total_it = BULK ? ngrp_cta * ntile_cta : 0;
    // Request part `part` (of kMIssuers equal pieces) of sequence element it_ into its stage.  The pieces of a stage
    // are requested by different warps: one thread gets a bulk copy out only every few hundred cycles, which would
    // otherwise sit on the CTA's critical path once per row group.
    auto issue_it = [&](int it_, int part) {
        int ss, gg;
        locate((int)blockIdx.x + (it_ % ngrp_cta) * (int)gridDim.x, ss, gg);
        const int st = it_ % p.bulk_stages;
        const uint32_t bytes = (uint32_t)grp_words * 4u / kMIssuers;             // chunks * 64: a multiple of 16
        uint32_t* dst = ring + (size_t)st * stage_words + (size_t)part * (bytes / 4u);
        mbar_expect_tx(&bars[st], bytes * (PAIR ? 2u : 1u));
        const uint4* src_a = p.seg[ss].w + w_off + (size_t)gg * p.chunks * kRowsPerGroup + (size_t)part * (bytes / 16u);
        bulk_load_stream(dst, src_a, bytes, &bars[st]);
        if (PAIR)
            bulk_load_stream(dst + grp_words,
                             p.seg[1].w + w_off + (size_t)gg * p.chunks * kRowsPerGroup + (size_t)part * (bytes / 16u), bytes,
                             &bars[st]);
    };
    int it = 0;
    int wait_failed = 0;
    bool give_up = false;                              // CTA-uniform: a bounded wait ran out somewhere in the CTA
    if (BULK) {
        if (tid == 0) {
            for (int st = 0; st < p.bulk_stages; ++st) mbar_init(&bars[st], kMIssuers);
            fence_mbar_init();
            for (int i = 0; i < p.bulk_stages && i < total_it; ++i)
                for (int part = 0; part < kMIssuers; ++part) issue_it(i, part);
        }
        // the barriers are used after the __syncthreads that follows the prologue of the first tile
    }

    for (int m0 = blockIdx.y * kMT; m0 < M_eff; m0 += gridDim.y * kMT) {
        const int mt = min(kMT, M_eff - m0);
        auto out_row = [&](int m) -> int { return GROUPED ? rows[m0 + m] : m0 + m; };
        auto in_row = [&](int m) -> int { return GROUPED ? (rows[m0 + m] >> p.grp_in_shift) : m0 + m; };
        int flat = flat0, s = s0, g = g0;
        auto residual_of = [&](int seg_i, int grp) -> float {
            if (p.epilogue != LSPK_EPI_ADD || tid >= kMT * 16 || out_m >= mt) return 0.0f;
            const int n = grp * kRowsPerGroup + out_r;
            if (n >= p.seg[seg_i].N) return 0.0f;
            return p.seg[seg_i].out[(size_t)out_row(out_m) * p.seg[seg_i].N + n];
        };
        float resid = BULK ? 0.0f : residual_of(s, g);
        if (!BULK && (GROUPED || !first_tile)) load_batch(s, g, 0, wa, wb);
        first_tile = false;

        // ---- prologue: the tile's rows -> permuted int8 rows in shared memory ------------------------------
        if (x_async) {
            // lane s of warp m requests segment s of row m (a contiguous run of the pre-tiled buffer): the eight
            // warps issue side by side, a thread's own copies go out one after the other, nearest segment first
            if (lane < nxseg) {
                const int c0 = lane * kMXSegChunks;
                const uint32_t bytes = (uint32_t)(min(p.chunks, c0 + kMXSegChunks) - c0) * 64u;
                const size_t off = (size_t)warp * rs + (size_t)c0 * 64;            // kMWarps == kMT: warp = row
                mbar_expect_tx(&xbars[lane], bytes);
                bulk_load(xq + off, p.x_i8 + (size_t)m0 * rs + off, bytes, &xbars[lane]);
            }
            if (tid < kMT) {
                s_scale[tid] = p.x_scales[m0 + tid];
                s_sumx[tid] = p.x_sums[m0 + tid];
            }
        } else if (p.prologue == kProInt8Tiled) {
            // rows already permuted and spaced like the shared-memory tile: a plain 16-byte copy
            const int chunks_per_row = rs / 16;
            const uint4* src = reinterpret_cast<const uint4*>(p.x_i8 + (size_t)m0 * rs);
            uint4* dst = reinterpret_cast<uint4*>(xq);
            for (int i = tid; i < kMT * chunks_per_row; i += kMThreads)
                dst[i] = (i / chunks_per_row) < mt ? src[i] : make_uint4(0, 0, 0, 0);
            if (tid < kMT) {
                s_scale[tid] = tid < mt ? p.x_scales[m0 + tid] : 0.0f;
                s_sumx[tid] = tid < mt ? p.x_sums[m0 + tid] : 0;
            }
        } else {
            // plain int8 rows: one warp per row, a single pass of independent loads
            const int m = warp;                                  // kMWarps == kMT
            int8_t* xq_row = xq + (size_t)m * rs;
            const int nblk = Kp / 16;
            if (m >= mt) {
                for (int b = lane; b < nblk; b += 32) *reinterpret_cast<uint4*>(xq_row + b * 16) = make_uint4(0, 0, 0, 0);
                if (lane == 0) { s_scale[m] = 0.0f; s_sumx[m] = 0; }
            } else {
                const int8_t* src = p.x_i8 + (size_t)in_row(m) * p.K;
                int sumx = 0;
                if ((p.K & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                    // whole 16-element blocks, 16-byte aligned: one load per block, four blocks in flight per lane
                    const uint4* src4 = reinterpret_cast<const uint4*>(src);
                    const int kblk = p.K >> 4;
#pragma unroll 4
                    for (int b = lane; b < nblk; b += 32) {
                        uint4 a = make_uint4(0, 0, 0, 0);
                        if (b < kblk) a = src4[b];
                        sumx = __dp4a((int)a.x, 0x01010101, sumx);
                        sumx = __dp4a((int)a.y, 0x01010101, sumx);
                        sumx = __dp4a((int)a.z, 0x01010101, sumx);
                        sumx = __dp4a((int)a.w, 0x01010101, sumx);
                        uint32_t o0, o1, o2, o3;
                        transpose4x4_bytes(a.x, a.y, a.z, a.w, o0, o1, o2, o3);
                        *reinterpret_cast<uint4*>(xq_row + b * 16) = make_uint4(o0, o1, o2, o3);
                    }
                } else {
#pragma unroll 2
                    for (int b = lane; b < nblk; b += 32) {
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
                }
                sumx = warp_sum(sumx);
                if (lane == 0) { s_scale[m] = p.x_scales[in_row(m)]; s_sumx[m] = sumx; }
            }
        }
        tr.mark();                                                 // 2: rows staged (or requested)
        if (!x_async) __syncthreads();
        tr.mark();                                                 // 3: activations visible
        bool x_pending = x_async;                                  // the first row group waits segment by segment
        const long long x_deadline = x_async ? clock64() + kMXWaitCycles : 0;

        // ---- row groups of this CTA ---------------------------------------------------------------------
        while (true) {
            const int next_flat = flat + gridDim.x;
            const bool has_next = next_flat < p.total_groups;
            int ns = 0, ng = 0;
            float next_resid = 0.0f;
            if (has_next) {
                locate(next_flat, ns, ng);
                next_resid = residual_of(ns, ng);
            }
            int acc_a[4][4], acc_b[PAIR ? 4 : 1][4];
#pragma unroll
            for (int f = 0; f < 4; ++f)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    acc_a[f][c] = 0;
                    if (PAIR) acc_b[f][c] = 0;
                }
            const int8_t* xrow = xq + (size_t)gid * rs;            // B operand: token gid
            if (BULK) {
                const int st = it % p.bulk_stages;
                const uint32_t parity = (uint32_t)(it / p.bulk_stages) & 1u;
                bool arrived = false;
                for (unsigned i = 0; i < kMBulkSpinLimit && !arrived; ++i) arrived = mbar_try_wait(&bars[st], parity);
                wait_failed |= arrived ? 0 : 1;
                const uint32_t* sa = ring + (size_t)st * stage_words + lane;
#pragma unroll 2
                for (int pr = warp; pr < pairs; pr += kMWarps) {
                    const int j0 = 2 * pr;
                    const bool two = j0 + 1 < p.chunks;
                    const uint4 x0 = *reinterpret_cast<const uint4*>(xrow + (size_t)(4 * j0 + t4) * 16);
                    uint4 x1 = make_uint4(0, 0, 0, 0);
                    if (two) x1 = *reinterpret_cast<const uint4*>(xrow + (size_t)(4 * (j0 + 1) + t4) * 16);
                    const uint32_t xb0[4] = {x0.x, x0.y, x0.z, x0.w};
                    const uint32_t xb1[4] = {x1.x, x1.y, x1.z, x1.w};
                    const uint32_t a0 = sa[j0 * 64], a1 = sa[j0 * 64 + 32];
                    const uint32_t a2 = two ? sa[(j0 + 1) * 64] : 0x55555555u, a3 = two ? sa[(j0 + 1) * 64 + 32] : 0x55555555u;
                    uint32_t b0 = 0, b1 = 0, b2 = 0, b3 = 0;
                    if (PAIR) {
                        b0 = sa[grp_words + j0 * 64];
                        b1 = sa[grp_words + j0 * 64 + 32];
                        b2 = two ? sa[grp_words + (j0 + 1) * 64] : 0x55555555u;
                        b3 = two ? sa[grp_words + (j0 + 1) * 64 + 32] : 0x55555555u;
                    }
#pragma unroll
                    for (int f = 0; f < 4; ++f) {
                        const uint32_t mask = 0x03030303u << (2 * f);
                        mma_u8s8(acc_a[f], a0 & mask, a1 & mask, a2 & mask, a3 & mask, xb0[f], xb1[f]);
                        if (PAIR) mma_u8s8(acc_b[f], b0 & mask, b1 & mask, b2 & mask, b3 & mask, xb0[f], xb1[f]);
                    }
                }
            } else
            for (int base = 0;; ) {
#pragma unroll
                for (int i = 0; i < kMNI; ++i) {
                    const int pr = warp + kMWarps * (base + i);
                    if (pr < pairs) {
                        const int j0 = 2 * pr;
                        if (x_pending) {                           // segment base+i holds chunks j0, j0+1
                            while (!mbar_try_wait(&xbars[base + i], 0)) {
                                if (clock64() > x_deadline) {
                                    wait_failed = 1;
                                    break;
                                }
                            }
                        }
                        // four masks' B registers of chunk j0 and of chunk j0+1 (zeros past the last chunk)
                        const uint4 x0 = *reinterpret_cast<const uint4*>(xrow + (size_t)(4 * j0 + t4) * 16);
                        uint4 x1 = make_uint4(0, 0, 0, 0);
                        if (j0 + 1 < p.chunks) x1 = *reinterpret_cast<const uint4*>(xrow + (size_t)(4 * (j0 + 1) + t4) * 16);
                        const uint32_t xb0[4] = {x0.x, x0.y, x0.z, x0.w};
                        const uint32_t xb1[4] = {x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                        for (int f = 0; f < 4; ++f) {
                            const uint32_t mask = 0x03030303u << (2 * f);
                            mma_u8s8(acc_a[f], wa[i][0] & mask, wa[i][1] & mask, wa[i][2] & mask, wa[i][3] & mask,
                                     xb0[f], xb1[f]);
                            if (PAIR)
                                mma_u8s8(acc_b[f], wb[i][0] & mask, wb[i][1] & mask, wb[i][2] & mask, wb[i][3] & mask,
                                         xb0[f], xb1[f]);
                        }
                    }
                }
                base += kMNI;
                if (kMWarps * base >= pairs) break;
                load_batch(s, g, base, wa, wb);
            }
            tr.mark();                                             // 4+: MMAs of a row group done
            if (!BULK && has_next) load_batch(ns, ng, 0, wa, wb);  // in flight during the reduction below

            // masks -> one int; C fragment: c0,c1 = (row gid, tokens 2*t4, 2*t4+1), c2,c3 = (row gid+8, same)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int row = gid + ((c >> 1) << 3);
                const int tok = 2 * t4 + (c & 1);
                const int v = acc_a[0][c] + (acc_a[1][c] >> 2) + (acc_a[2][c] >> 4) + (acc_a[3][c] >> 6);
                part[(warp * kMT + tok) * 16 + row] = v;
                if (PAIR) {
                    const int u = acc_b[0][c] + (acc_b[1][c] >> 2) + (acc_b[2][c] >> 4) + (acc_b[3][c] >> 6);
                    part[kMWarps * kMT * 16 + (warp * kMT + tok) * 16 + row] = u;
                }
            }
            if (BULK) {
                // every warp is done with this stage: request the element bulk_stages ahead into it.  A wait that
                // ran out ends the CTA once its outstanding copies (bounded wait again) have landed.
                if (__syncthreads_or(wait_failed)) {
                    if (tid == 0) {
                        if (p.error_flag) atomicExch(p.error_flag, LSPK_ERR_DEVICE_WAIT);
                        for (int k = it + 1; k < it + p.bulk_stages && k < total_it; ++k) {
                            bool done = false;
                            for (unsigned i = 0; i < kMBulkSpinLimit && !done; ++i)
                                done = mbar_try_wait(&bars[k % p.bulk_stages], (uint32_t)(k / p.bulk_stages) & 1u);
                        }
                    }
                    give_up = true;
                } else {
                    if (lane == 0 && warp < kMIssuers && it + p.bulk_stages < total_it) issue_it(it + p.bulk_stages, warp);
                    ++it;
                }
            } else if (x_pending) {
                x_pending = false;
                if (__syncthreads_or(wait_failed)) {
                    // a segment never arrived: report, give the copies in flight one more bounded wait, leave
                    if (tid == 0) {
                        if (p.error_flag) atomicExch(p.error_flag, LSPK_ERR_DEVICE_WAIT);
                        const long long dl = clock64() + kMXWaitCycles;
                        for (int k = 0; k < nxseg; ++k)
                            while (!mbar_try_wait(&xbars[k], 0) && clock64() <= dl) {}
                    }
                    give_up = true;
                }
            } else {
                __syncthreads();
            }
            if (give_up) break;

            if (tid < kMT * 16) {
                const LinearSeg& sg = p.seg[s];
                const int n = g * kRowsPerGroup + out_r;
                if (out_m < mt && n < sg.N) {
                    int va = 0, vb = 0;
#pragma unroll
                    for (int w = 0; w < kMWarps; ++w) {
                        va += part[(w * kMT + out_m) * 16 + out_r];
                        if (PAIR) vb += part[kMWarps * kMT * 16 + (w * kMT + out_m) * 16 + out_r];
                    }
                    const int sx = s_sumx[out_m];
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
                            sg.out[o] = __fmul_rn(__fdiv_rn(ya, __fadd_rn(expf(-ya), 1.0f)), yb);
                        } else {
                            const float gpos = fmaxf(ya, 0.0f);
                            sg.out[o] = __fmul_rn(__fmul_rn(gpos, gpos), yb);
                        }
                    } else if (p.epilogue == LSPK_EPI_ADD) {
                        sg.out[o] = __fadd_rn(BULK ? sg.out[o] : resid, ya);
                    } else {
                        sg.out[o] = ya;
                    }
                }
            }
            tr.mark();                                             // 5+: row group stored
            __syncthreads();                       // `part` (and, at the end of a tile, xq) is rewritten next
            if (!has_next) break;
            flat = next_flat;
            s = ns;
            g = ng;
            resid = next_resid;
        }
        if (give_up) break;
        if (!GROUPED) break;
    }
    tr.end();
}

template <bool PAIR, bool GROUPED, bool BULK = false>
static cudaError_t launch_mma(const LinearParams& p, dim3 grid, size_t smem) {
    static bool attr_set = false;
    auto kern = ternary_linear_mma_kernel<PAIR, GROUPED, BULK>;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    return launch(kern, grid, dim3(kMThreads), smem, true, p);
}

// Launch the eight-row kernel.  K is limited by the shared-memory activation tile (8 rows of K bytes).
// Rows arrive quantised (INT8 prologue); fp32 rows are quantised once by the row kernel beforehand.
int linear_mma_launch(const LinearParams& p, bool pair, bool grouped, int grid_x, int grid_y, int grid_z) {
    LSPK_REQUIRE(p.prologue == LSPK_PRO_INT8 || (p.prologue == kProInt8Tiled && !grouped),
                 "linear: the eight-row kernel takes int8 rows (prologue %d)", p.prologue);
    const int Kp = p.chunks * kWeightsPerChunk;
    size_t smem = (size_t)kMT * mma_row_stride(Kp) + (size_t)kMWarps * kMT * 16 * (pair ? 2 : 1) * 4 + kMT * 8 + 64;
    LSPK_REQUIRE(smem <= 200 * 1024, "linear: K=%d too large for the 8-row activation tile (limit about 24000)", p.K);
    const dim3 grid(grid_x, grid_y, grid_z);
    if (p.bulk_stages > 0) {
        // expert-grouped launches only (set by the MoE layer): ring behind the tile
        LSPK_REQUIRE(grouped && p.bulk_stages <= kMBulkStages, "linear (mma): bulk ring is for expert-grouped launches");
        smem += 256 + (size_t)p.bulk_stages * p.chunks * 256 * (pair ? 2 : 1);
        LSPK_REQUIRE(smem <= 200 * 1024, "linear (mma): bulk ring too large");
        cudaError_t e = pair ? launch_mma<true, true, true>(p, grid, smem) : launch_mma<false, true, true>(p, grid, smem);
        if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "linear (mma, bulk) launch failed: %s", cudaGetErrorString(e));
        return LSPK_OK;
    }
    cudaError_t e = grouped ? (pair ? launch_mma<true, true>(p, grid, smem) : launch_mma<false, true>(p, grid, smem))
                            : (pair ? launch_mma<true, false>(p, grid, smem) : launch_mma<false, false>(p, grid, smem));
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "linear (mma) launch failed: %s", cudaGetErrorString(e));
    return LSPK_OK;
}

}  // namespace lspk
