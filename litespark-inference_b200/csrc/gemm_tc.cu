// Prefill path of the ternary linear layer on the 5th-generation tensor cores (tcgen05).
//
//   acc[t, n] = sum_k w[n, k] * xq[t, k]      int8 x int8 -> int32 in tensor memory (exact)
//   y[t, n]   = float(acc) * (xscale[t] * wscale)
//
// Replaces, for many token rows, what the reference does with its batched kernel
// (matmul_lut_avx512_mT, matmul_lut_avx512_extern_c.cpp:258-339) and, as the tensor-unit analogue,
// its AMX tile GEMM (matmul_amx_int8_mT_v2, :819-933).
//
// One CTA owns 128 output features (the MMA's M side: one TMEM lane per feature) and TN token rows
// (the MMA's N side: one TMEM column per token).  Per 128-wide K block, through a 4-stage ring:
//   warp 0      TMA: 4 KB of packed 2-bit weights (128 rows x 32 bytes of the device chunk layout)
//               and the TN x 128-byte tile of int8 activations (128-byte swizzle) -> shared memory
//   warps 2-5   expand the packed rows to signed int8 {-1,0,+1} in the canonical K-major,
//               128-byte-swizzled operand layout (thread = weight row; one packed word -> 16 bytes)
//   warp 1      one thread issues 4 x tcgen05.mma.kind::i8 (M=128, N=TN, K=32) per block and
//               commits the stage back to the producer
// then warps 2-9 read the accumulators with tcgen05.ld (two warps per quarter of the TMEM lanes, alternate
// 32-column slabs; warps 6-9 exist only for this) and write fp32 (and, if asked, the int32).
// The activations are stored with the 4x4 index transpose inside every 16-element block that the
// masked decode of a packed word implies (same trick as the CUDA-core kernel), so a packed word
// expands with 4 x (shift, and, byte-subtract) and lands as one aligned 16-byte chunk.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records an error code, stops issuing
// work, drains its own copies, frees its tensor memory and returns.
#include <cuda.h>
#include <stdlib.h>

#include "internal.cuh"

namespace lspk {

constexpr int kTcThreads = 320;          // 10 warps: TMA, MMA, 4 x expand + epilogue, 4 x epilogue only
constexpr int kTcStages = 4;
constexpr int kTcBK = 128;               // K elements per pipeline block
constexpr int kTcRows = 128;             // output features per CTA
constexpr unsigned kSpinLimit = 1u << 22;

// One matrix of a launch: the matrices of a call (q/k/v; gate/up) share the activations and are covered by one
// grid, matrix i owning the output-feature tiles [tile0, tile0 + ceil(N / 128)) of gridDim.x.
struct TcSeg {
    float* out;
    int32_t* acc_out;
    int32_t* split_ws;       // K split / gated pairing: this CTA's K range stores its int32 partial sums in slice
                             // blockIdx.z of this workspace ([splits][M, N]); the finish kernel adds the slices
    float w_scale;
    int N;
    int tile0;
};
struct TcParams {
    TcSeg seg[3];
    int n_seg;
    const float* x_scales;
    int M, K;
    int k_blocks;            // K blocks of the whole product
    int kb_per_split;        // K blocks per CTA along gridDim.z (== k_blocks when K is not split)
    int epilogue;            // LSPK_EPI_STORE or LSPK_EPI_ADD
    int* error_flag;
    unsigned long long* trace;   // optional phase trace: one record per role of CTA (0,0,0) (ids 10, 11, 12)
    int trace_cap;
};

// ---- PTX wrappers (mbarrier and fences: common.cuh) --------------------------------------------
// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when the limit is reached or
// another thread already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (unsigned i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major operand, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart (stride field 64), leading field 1, descriptor version 1.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                                // leading byte offset (unused for this layout)
    d |= (uint64_t)(1024 >> 4) << 32;                      // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                // version
    d |= (uint64_t)2 << 61;                                // SWIZZLE_128B
    return d;
}

template <int TN>
__global__ void __launch_bounds__(kTcThreads)
ternary_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                       const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_x,
                       const __grid_constant__ TcParams p) {
    constexpr int kPackedBytes = kTcRows * kTcBK / 4;       // 4096
    constexpr int kATileBytes = kTcRows * kTcBK;            // 16384
    constexpr int kBTileBytes = TN * kTcBK;
    constexpr int kStageBytes = kPackedBytes + kATileBytes + kBTileBytes;
    constexpr uint32_t kTmemCols = TN < 32 ? 32 : TN;       // power of two >= 32
    // instruction descriptor: D = s32, A = B = signed int8, both K-major, N = TN, M = 128
    constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((128u >> 4) << 24);

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_w[kTcStages];     // packed weights of the stage have landed
    __shared__ __align__(8) uint64_t full_tma[kTcStages];   // activation tile of the stage has landed
    __shared__ __align__(8) uint64_t full_a[kTcStages];
    __shared__ __align__(8) uint64_t empty[kTcStages];
    __shared__ __align__(8) uint64_t acc_ready;
    __shared__ uint32_t tmem_base_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int sgi = 0;
    if (p.n_seg > 1 && (int)blockIdx.x >= p.seg[1].tile0) sgi = 1;
    if (p.n_seg > 2 && (int)blockIdx.x >= p.seg[2].tile0) sgi = 2;
    const TcSeg& sg = p.seg[sgi];
    const CUtensorMap* map_w = sgi == 0 ? &map_w0 : sgi == 1 ? &map_w1 : &map_w2;
    const int n0 = ((int)blockIdx.x - sg.tile0) * kTcRows;
    const int m0 = blockIdx.y * TN;
    // K split: this CTA's K blocks are [kb0, kb0 + nkb)
    const int kb0 = blockIdx.z * p.kb_per_split;
    const int nkb = min(p.kb_per_split, p.k_blocks - kb0);

    auto a_tile = [&](int s) { return smem + (size_t)s * kStageBytes; };
    auto b_tile = [&](int s) { return smem + (size_t)s * kStageBytes + kATileBytes; };
    auto packed = [&](int s) { return smem + (size_t)s * kStageBytes + kATileBytes + kBTileBytes; };

    if (tid == 0) {
        abort_flag = 0;
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(&full_w[s], 1);
            mbar_init(&full_tma[s], 1);
            mbar_init(&full_a[s], 4);                      // one arrival per expansion warp
            mbar_init(&empty[s], 1);
        }
        mbar_init(&acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_slot;
    volatile int* abortp = &abort_flag;

    grid_dependency_launch();
    // The packed weights do not depend on the previous kernel: the producer requests the first ring of them, and
    // the expansion warps turn them into operand tiles, while that kernel is still running.  Whoever touches the
    // activations, the scales or the outputs waits for it first.
    auto load_weights = [&](int kb) {
        const int s = kb % kTcStages;
        mbar_expect_tx(&full_w[s], kPackedBytes);
        // inner coordinate in 4-byte units (a K block is 2 chunks x 16 rows x 16 bytes = 128 units per row
        // group), outer coordinate = row group
        tma_load_2d(packed(s), map_w, (kb0 + kb) * 128, n0 / kRowsPerGroup, &full_w[s]);
    };

    if (warp == 0) {
        // ---------------- producer ------------------------------------------------------------
        if (lane == 0) {
            PhaseTrace tr;
            tr.begin(p.trace, p.trace_cap, 10, 0);
            const int early = min(nkb, kTcStages);
            for (int kb = 0; kb < early; ++kb) load_weights(kb);
            grid_dependency_wait();
            int issued = 0;
            for (int kb = 0; kb < nkb; ++kb) {
                if ((kb & 1) == 0) tr.mark();              // before the wait for blocks 0, 2, 4, ...
                const int s = kb % kTcStages;
                if (kb >= kTcStages && !mbar_wait(&empty[s], ((kb / kTcStages) - 1) & 1, abortp)) break;
                if (*abortp) break;
                if (kb >= early) load_weights(kb);
                mbar_expect_tx(&full_tma[s], kBTileBytes);
                tma_load_2d(b_tile(s), &map_x, (kb0 + kb) * kTcBK, m0, &full_tma[s]);
                ++issued;
            }
            tr.end();
            if (*abortp) {
                // drain: wait (bounded) for every copy this thread started
                const int w_issued = issued > early ? issued : early;
                for (int kb = 0; kb < w_issued; ++kb) {
                    const int s = kb % kTcStages;
                    if (kb + kTcStages >= w_issued)
                        for (unsigned i = 0; i < kSpinLimit && !mbar_try_wait(&full_w[s], (kb / kTcStages) & 1); ++i) {}
                }
                for (int kb = 0; kb < issued; ++kb) {
                    const int s = kb % kTcStages;
                    if (kb + kTcStages >= issued)
                        for (unsigned i = 0; i < kSpinLimit && !mbar_try_wait(&full_tma[s], (kb / kTcStages) & 1); ++i) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ------------------------------------------------------------
        if (lane == 0) {
            PhaseTrace tr;
            tr.begin(p.trace, p.trace_cap, 11, 32);
            grid_dependency_wait();
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                if ((kb & 1) == 0) tr.mark();
                const int s = kb % kTcStages;
                const uint32_t ph = (kb / kTcStages) & 1;
                ok = mbar_wait(&full_tma[s], ph, abortp) && mbar_wait(&full_a[s], ph, abortp);
                if (!ok) break;
                tc_fence_after();
                const uint64_t da = umma_desc_sw128(smem_u32(a_tile(s)));
                const uint64_t db = umma_desc_sw128(smem_u32(b_tile(s)));
#pragma unroll
                for (int k4 = 0; k4 < kTcBK / 32; ++k4) {
                    const uint32_t accumulate = (kb | k4) ? 1u : 0u;
                    // advancing 32 int8 along K = 32 bytes = 2 descriptor address units
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem_base), "l"(da + (uint64_t)(k4 * 2)), "l"(db + (uint64_t)(k4 * 2)), "r"(kIdesc),
                        "r"(accumulate)
                        : "memory");
                }
                // frees the stage for the producer once the MMAs above have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                 smem_u32(&empty[s]))
                             : "memory");
            }
            // On the regular path this tells the epilogue warps that every MMA has completed.  After an abort
            // nobody waits on it any more (they saw the abort flag), and the same commit + one bounded wait makes
            // sure that no MMA issued above is still in flight when the tensor memory is freed below.
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_u32(&acc_ready))
                         : "memory");
            if (!ok)
                for (unsigned i = 0; i < kSpinLimit && !mbar_try_wait(&acc_ready, 0); ++i) {}
            tr.end();
        }
    } else {
        // ---------------- expand packed weights -> int8 operand tile, then epilogue ---------------
        const int row = tid - 64;                         // 0..127: weight row inside the CTA tile
        const int gi = row >> 4, rr = row & 15;
        bool ok = true;
        PhaseTrace tr;
        tr.begin(p.trace, p.trace_cap, 12, 64);
        // warps 6-9 take no part in the expansion: they double the warps that drain the accumulators afterwards
        for (int kb = 0; kb < (warp < 6 ? nkb : 0) && ok; ++kb) {
            if ((kb & 7) == 0 && kb < 24) tr.mark();
            const int s = kb % kTcStages;
            // warp-uniform: every lane polls with its own counter, and the barrier below needs the whole warp
            ok = __all_sync(0xffffffffu, mbar_wait(&full_w[s], (kb / kTcStages) & 1, abortp));
            if (!ok) break;
            const unsigned char* pk = packed(s);
            unsigned char* arow = a_tile(s) + (size_t)(row >> 3) * 1024 + (size_t)(row & 7) * 128;
#pragma unroll
            for (int c = 0; c < 2; ++c) {                  // the two 64-weight chunks of this K block
                const uint4 w = *reinterpret_cast<const uint4*>(pk + gi * 512 + c * 256 + rr * 16);
                const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    uint4 o;
                    o.x = __vsub4(words[m] & 0x03030303u, 0x01010101u);
                    o.y = __vsub4((words[m] >> 2) & 0x03030303u, 0x01010101u);
                    o.z = __vsub4((words[m] >> 4) & 0x03030303u, 0x01010101u);
                    o.w = __vsub4((words[m] >> 6) & 0x03030303u, 0x01010101u);
                    const int chunk = c * 4 + m;           // 16-byte chunk index inside the 128-byte row
                    *reinterpret_cast<uint4*>(arow + ((chunk ^ (row & 7)) << 4)) = o;
                }
            }
            fence_async_smem();                            // generic-proxy writes -> visible to the tensor unit
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_a[s]);        // 4 arrivals per stage instead of 128
        }
        // epilogue: TMEM lane = weight row, column = token
        grid_dependency_wait();                            // scales, residual and outputs belong to the chain
        tr.mark();                                         // all blocks expanded
        __syncwarp();
        if (ok) ok = mbar_wait(&acc_ready, 0, abortp);
        tr.mark();                                         // accumulators complete
        ok = __all_sync(0xffffffffu, ok);              // the tensor-memory loads below need the whole warp
        if (ok) {
            tc_fence_after();
            const int quarter = warp & 3;                  // TMEM lanes this warp may read
            const int n = n0 + quarter * 32 + lane;
#pragma unroll 1
            // two warps share a quarter of the TMEM lanes: they take alternate 32-column slabs
            for (int cb = warp < 6 ? 0 : 1; cb < TN / 32; cb += 2) {
                uint32_t v[32];
                tr.mark();                                 // previous slab stored
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(cb * 32);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                      "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
                      "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
                      "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tr.mark();                                 // a 32-column slab of accumulators is in registers
                const int t0 = m0 + cb * 32;
                const int jmax = min(32, p.M - t0);        // token rows of this slab that exist
                // scale of token row t0 + lane (one coalesced load; handed round by shuffles below)
                const float my_scale = (!sg.split_ws && lane < jmax) ? __fmul_rn(__ldg(p.x_scales + t0 + lane), sg.w_scale) : 0.0f;
                float sc[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) sc[j] = __shfl_sync(0xffffffffu, my_scale, j);
                if (n < sg.N && jmax > 0) {
                    const size_t o0 = (size_t)t0 * sg.N + n;
                    if (sg.split_ws) {
                        // partial sums of this K range: exact in int32, slice blockIdx.z of the workspace
                        int32_t* wsp = sg.split_ws + (size_t)blockIdx.z * p.M * sg.N + o0;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < jmax) wsp[(size_t)j * sg.N] = (int)v[j];
                    } else {
                        float* outp = sg.out + o0;
                        if (sg.acc_out) {
                            int32_t* accp = sg.acc_out + o0;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < jmax) accp[(size_t)j * sg.N] = (int)v[j];
                        }
                        // every load of the slab before its first store: the stores may alias the residual as far
                        // as the compiler knows, and would otherwise serialise 32 round trips
                        if (p.epilogue == LSPK_EPI_ADD) {
                            float res[32];
#pragma unroll
                            for (int j = 0; j < 32; ++j) res[j] = j < jmax ? outp[(size_t)j * sg.N] : 0.0f;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < jmax)
                                    outp[(size_t)j * sg.N] = __fadd_rn(res[j], __fmul_rn((float)(int)v[j], sc[j]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (j < jmax) outp[(size_t)j * sg.N] = __fmul_rn((float)(int)v[j], sc[j]);
                        }
                    }
                }
            }
        }
        tr.end();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    if (tid == 0 && abort_flag && p.error_flag) atomicExch(p.error_flag, LSPK_ERR_DEVICE_WAIT);
}

// K split: int32 sums of all K ranges -> fp32 outputs (rescale, residual add or the gated pairing), and the
// raw accumulators where asked for.  Up to three matrices of one call are finished by one launch; for the
// gated epilogues segment 0 is the gate and segment 1 the up projection (same N), and only out[0] is written.
struct FinishSeg {
    const int32_t* ws;       // [splits][M, N]
    float* out;
    int32_t* acc_out;
    float w_scale;
    int N;
    int splits;
};
struct FinishParams {
    FinishSeg seg[3];
    int n_seg;
    int M;
    int epilogue;
    const float* x_scales;
};

// Sum of one element over the K-range slices (at most 8): all loads issued before the first add.
__device__ __forceinline__ int sum_slices(const int32_t* first, size_t slice, int splits) {
    int v[8];
#pragma unroll
    for (int z = 0; z < 8; ++z) v[z] = z < splits ? first[(size_t)z * slice] : 0;
    return ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
}

__global__ void splitk_finish_kernel(const FinishParams p) {
    grid_dependency_launch();
    grid_dependency_wait();
    const bool pair = p.epilogue == LSPK_EPI_RELU2_MUL || p.epilogue == LSPK_EPI_SILU_MUL;
    const int n_seg = pair ? 1 : p.n_seg;
    for (int sgi = 0; sgi < n_seg; ++sgi) {
        const FinishSeg sg = p.seg[sgi];
        const size_t total = (size_t)p.M * sg.N;
        for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
            const int t = (int)(i / sg.N);
            const int a = sum_slices(sg.ws + i, total, sg.splits);
            if (sg.acc_out) sg.acc_out[i] = a;
            const float xs = p.x_scales[t];
            const float y = __fmul_rn((float)a, __fmul_rn(xs, sg.w_scale));
            if (pair) {
                const int b = sum_slices(p.seg[1].ws + i, total, p.seg[1].splits);
                if (p.seg[1].acc_out) p.seg[1].acc_out[i] = b;
                const float u = __fmul_rn((float)b, __fmul_rn(xs, p.seg[1].w_scale));
                if (p.epilogue == LSPK_EPI_SILU_MUL) {
                    sg.out[i] = __fmul_rn(__fdiv_rn(y, __fadd_rn(expf(-y), 1.0f)), u);
                } else {
                    const float gpos = fmaxf(y, 0.0f);
                    sg.out[i] = __fmul_rn(__fmul_rn(gpos, gpos), u);
                }
            } else {
                sg.out[i] = p.epilogue == LSPK_EPI_ADD ? __fadd_rn(sg.out[i], y) : y;
            }
        }
    }
}

// int8 rows [M, K] in natural order -> [M, Kp] with the 4x4 transpose inside every 16-element block
// (Kp = K rounded up to 64, zero padded), the order the expanded weights come out in.
__global__ void permute_rows_kernel(const int8_t* __restrict__ src, int8_t* __restrict__ dst, int M, int K, int Kp) {
    grid_dependency_launch();
    grid_dependency_wait();
    const size_t total = (size_t)M * Kp;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(i / Kp), kp = (int)(i % Kp);
        const int k = perm_index(kp);                      // the transpose is its own inverse
        dst[i] = k < K ? src[(size_t)t * K + k] : (int8_t)0;
    }
}

// ---- host side -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
    return fn;
}

struct TcScratch {
    int8_t *xq = nullptr, *xq_perm = nullptr;
    float* xs = nullptr;
    int* err = nullptr;
    int32_t* split_ws = nullptr;
    int* xsum = nullptr;
    size_t cap_xq = 0, cap_perm = 0, cap_xs = 0, cap_ws = 0, cap_xsum = 0;
};
static TcScratch g_tc;

static int grow(void** p, size_t* cap, size_t need) {
    if (need <= *cap) return LSPK_OK;
    // cudaFree waits for the device, so no kernel in flight still uses the old buffer; graphs that hold its
    // address are re-captured by their owners (scratch_generation)
    if (*p) cudaFree(*p);
    *p = nullptr;
    *cap = 0;
    scratch_moved();
    LSPK_CUDA(cudaMalloc(p, need + need / 4 + 256));
    *cap = need + need / 4 + 256;
    return LSPK_OK;
}

// Library-owned int8 rows + scales for callers that hand fp32 rows to a many-row product.  Grows with
// cudaMalloc: the first call of a given size must happen outside stream capture.
int quant_scratch(size_t M, size_t K, int8_t** q, float** s, int** sums) {
    if (int rc = grow((void**)&g_tc.xq, &g_tc.cap_xq, M * K)) return rc;
    if (int rc = grow((void**)&g_tc.xs, &g_tc.cap_xs, M * 4)) return rc;
    *q = g_tc.xq;
    *s = g_tc.xs;
    if (sums) {
        if (int rc = grow((void**)&g_tc.xsum, &g_tc.cap_xsum, M * 4)) return rc;
        *sums = g_tc.xsum;
    }
    return LSPK_OK;
}

template <int TN>
static cudaError_t launch_tc(const CUtensorMap* mw, const CUtensorMap& mx, const TcParams& p, dim3 grid) {
    constexpr size_t smem = (size_t)kTcStages * (kTcRows * kTcBK / 4 + kTcRows * kTcBK + TN * kTcBK) + 1024;
    static bool attr_set = false;
    auto kern = ternary_gemm_tc_kernel<TN>;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    return launch(kern, grid, dim3(kTcThreads), smem, true, mw[0], mw[1], mw[2], mx, p);
}

// Tensor-core path.  Handles STORE / ADD epilogues of one or several matrices sharing the input (each matrix is
// its own GEMM launch) and the gated gate/up pairings (two GEMMs into the int32 workspace, gate applied by the
// finish kernel).
int linear_tensor_core(const lspk_linear_args* a, int* handled) {
    *handled = 0;
    if (a->M < 32) return LSPK_OK;
    const bool pair = a->epilogue == LSPK_EPI_RELU2_MUL || a->epilogue == LSPK_EPI_SILU_MUL;
    if (a->epilogue != LSPK_EPI_STORE && a->epilogue != LSPK_EPI_ADD && !pair) return LSPK_OK;
    if (pair && a->n_mats != 2) return LSPK_OK;
    if (a->prologue == LSPK_PRO_GATED_RMSNORM_QUANT) return LSPK_OK;
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return LSPK_OK;
    const Weight* w0 = reinterpret_cast<const Weight*>(a->w[0]);
    if (!w0) return LSPK_OK;
    const int M = a->M, K = w0->K, Kp = w0->chunks * kWeightsPerChunk;

    // ---- activations: int8 rows + scales, then the permuted, padded copy the tensor map reads ----
    const int8_t* xq = a->x_i8;
    const float* xs = a->x_scales;
    if (int rc = grow((void**)&g_tc.xq_perm, &g_tc.cap_perm, (size_t)M * Kp)) return rc;
    g_tc.err = device_wait_flag();
    int permuted = 0;
    if (a->prologue != LSPK_PRO_INT8) {
        if (int rc = grow((void**)&g_tc.xs, &g_tc.cap_xs, (size_t)M * 4)) return rc;
        xs = g_tc.xs;
        // fp32 rows: one kernel quantises straight into the permuted layout (unless the caller wants the
        // natural-order int8 rows back as well)
        if (!a->xq_out)
            if (int rc = quantize_rows_permuted(a, K, Kp, g_tc.xq_perm, g_tc.xs, &permuted)) return rc;
        if (!permuted) {
            if (int rc = grow((void**)&g_tc.xq, &g_tc.cap_xq, (size_t)M * K)) return rc;
            int rc = a->prologue == LSPK_PRO_RMSNORM_QUANT
                         ? lspk_rmsnorm_quantize_rows(a->x_f32, a->gamma, a->gamma_is_bf16, g_tc.xq, g_tc.xs, M, K, a->eps)
                         : lspk_quantize_rows(a->x_f32, g_tc.xq, g_tc.xs, M, K);
            if (rc) return rc;
            xq = g_tc.xq;
        }
    }
    if (!permuted) {
        const size_t total = (size_t)M * Kp;
        int grid = (int)((total + 255) / 256);
        if (grid > sm_count() * 8) grid = sm_count() * 8;
        LSPK_CUDA(launch(permute_rows_kernel, dim3(grid), dim3(256), 0, true, xq, g_tc.xq_perm, M, K, Kp));
    }
    if (a->xq_out) LSPK_CUDA(cudaMemcpyAsync(a->xq_out, xq, (size_t)M * K, cudaMemcpyDeviceToDevice, stream()));
    if (a->xscale_out) LSPK_CUDA(cudaMemcpyAsync(a->xscale_out, xs, (size_t)M * 4, cudaMemcpyDeviceToDevice, stream()));

    // ---- one grid for all matrices of the call: output-feature tiles of matrix 0, 1, 2 side by side in grid.x --
    const int k_blocks = (Kp + kTcBK - 1) / kTcBK;
    int n_tiles[3] = {0, 0, 0}, total_tiles = 0;
    for (int i = 0; i < a->n_mats; ++i) {
        const Weight* w = reinterpret_cast<const Weight*>(a->w[i]);
        LSPK_REQUIRE(w && w->K == K && (a->out[i] || (pair && i == 1)),
                     "linear (tensor-core): matrices must share K and have outputs");
        LSPK_REQUIRE(!pair || w->N == w0->N, "linear (tensor-core): gate and up must have the same N");
        n_tiles[i] = (w->N + kTcRows - 1) / kTcRows;
        total_tiles += n_tiles[i];
    }
    // Token rows per CTA tile.  A K block costs about the same whatever the tile's width (the loop is bound by
    // its handshakes, not by the tensor pipe), so 256 rows per tile halve the work when the grid still fills
    // the machine or the K loop is long; otherwise more, narrower tiles win.
    const bool wide = M > 128 && (total_tiles * ((M + 255) / 256) * 2 > sm_count() || k_blocks >= 32);
    const int TN = wide ? 256 : M > 64 ? 128 : M > 32 ? 64 : 32;
    const int m_tiles = (M + TN - 1) / TN;
    CUtensorMap mx;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)Kp, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)Kp};
        const cuuint32_t box[2] = {(cuuint32_t)kTcBK, (cuuint32_t)TN};
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&mx, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, g_tc.xq_perm, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(LSPK_ERR_CUDA, "tensor map (activations) failed: %d", (int)r);
    }
    // K split when the output tiles alone leave most SMs idle: every CTA then streams a fraction of the bytes and
    // runs a fraction of the K loop; the partial sums of a K range go to their own slice of an int32 workspace
    // and the finish kernel adds the slices (exact).  The gated pairing always goes through the workspace: its
    // epilogue needs both products of an element.
    int sp = 1;
    if (total_tiles * m_tiles * 2 <= sm_count()) {
        sp = sm_count() / (total_tiles * m_tiles);
        if (sp > 8) sp = 8;
        if (sp > k_blocks / 2) sp = k_blocks / 2;                       // at least two K blocks per CTA
        if (sp < 1) sp = 1;
    }
    const int kb_per = (k_blocks + sp - 1) / sp;
    const int splits = (k_blocks + kb_per - 1) / kb_per;                // no CTA without work
    const bool via_ws = splits > 1 || pair;
    size_t ws_off[3] = {0, 0, 0}, ws_total = 0;
    if (via_ws) {
        for (int i = 0; i < a->n_mats; ++i) {
            const Weight* w = reinterpret_cast<const Weight*>(a->w[i]);
            ws_off[i] = ws_total;
            ws_total += (size_t)M * w->N * splits;
        }
        if (int rc = grow((void**)&g_tc.split_ws, &g_tc.cap_ws, ws_total * 4)) return rc;
    }
    CUtensorMap mw[3];
    TcParams p = {};
    FinishParams fp = {};
    fp.M = M;
    fp.epilogue = a->epilogue;
    fp.x_scales = xs;
    size_t finish_elems = 0;
    int tile0 = 0;
    for (int i = 0; i < a->n_mats; ++i) {
        const Weight* w = reinterpret_cast<const Weight*>(a->w[i]);
        const cuuint64_t row_words = (cuuint64_t)w->chunks * 64;          // 4-byte units per row group
        const cuuint64_t dims[2] = {row_words, (cuuint64_t)w->groups};
        const cuuint64_t strides[1] = {row_words * 4};
        const cuuint32_t box[2] = {128, 8};                               // 512 bytes x 8 row groups
        const cuuint32_t estr[2] = {1, 1};
        CUresult r = enc(&mw[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, w->dev, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(LSPK_ERR_CUDA, "tensor map (weights) failed: %d", (int)r);
        p.seg[i] = TcSeg{a->out[i], a->acc_out[i], via_ws ? g_tc.split_ws + ws_off[i] : nullptr, w->scale, w->N, tile0};
        tile0 += n_tiles[i];
        if (via_ws) {
            fp.seg[fp.n_seg++] = FinishSeg{g_tc.split_ws + ws_off[i], a->out[i], a->acc_out[i], w->scale, w->N, splits};
            finish_elems += (size_t)M * w->N;
        }
    }
    for (int i = a->n_mats; i < 3; ++i) mw[i] = mw[0];
    p.n_seg = a->n_mats;
    p.x_scales = xs;
    p.M = M;
    p.K = K;
    p.k_blocks = k_blocks;
    p.kb_per_split = kb_per;
    p.epilogue = a->epilogue;
    p.error_flag = g_tc.err;
    p.trace = trace_buffer();
    p.trace_cap = trace_capacity();
    {
        const dim3 grid(total_tiles, m_tiles, splits);
        cudaError_t e = TN == 256 ? launch_tc<256>(mw, mx, p, grid)
                       : TN == 128 ? launch_tc<128>(mw, mx, p, grid)
                       : TN == 64 ? launch_tc<64>(mw, mx, p, grid)
                                  : launch_tc<32>(mw, mx, p, grid);
        if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "tensor-core GEMM launch failed: %s", cudaGetErrorString(e));
    }
    if (fp.n_seg > 0) {
        if (pair) finish_elems /= 2;
        int fgrid = (int)((finish_elems / (size_t)fp.n_seg + 255) / 256);
        if (fgrid > sm_count() * 4) fgrid = sm_count() * 4;
        if (fgrid < 1) fgrid = 1;
        cudaError_t e = launch(splitk_finish_kernel, dim3(fgrid), dim3(256), 0, true, fp);
        if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "tensor-core finish launch failed: %s", cudaGetErrorString(e));
    }
    *handled = 1;
    return LSPK_OK;
}

// Reads (and clears) the device-side wait-expiry flag of the tensor-core kernel.
int tensor_core_check_error() {
    g_tc.err = device_wait_flag();
    if (!g_tc.err) return LSPK_OK;
    int v = 0;
    LSPK_CUDA(cudaMemcpyAsync(&v, g_tc.err, 4, cudaMemcpyDeviceToHost, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    if (v) {
        cudaMemsetAsync(g_tc.err, 0, 4, stream());
        return fail(LSPK_ERR_DEVICE_WAIT, "a bounded device-side wait expired (tensor-core GEMM or bulk-copy GEMV)");
    }
    return LSPK_OK;
}

// Exercises the expiry path of the bounded waits without any other kernel's help: one thread polls an mbarrier
// that nothing will ever arrive on, a given number of times, then raises the wait flag and returns (the context
// stays usable; lspk_tc_check_error reports LSPK_ERR_DEVICE_WAIT once).
__global__ void wait_expiry_probe_kernel(int* flag, unsigned polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
        bool arrived = false;
        for (unsigned i = 0; i < polls && !arrived; ++i) arrived = mbar_try_wait(&bar, 0);
        if (!arrived && flag) atomicExch(flag, LSPK_ERR_DEVICE_WAIT);
    }
}

int expire_one_wait(unsigned polls) {
    int* flag = device_wait_flag();
    LSPK_REQUIRE(flag, "lspk_debug_expire_wait: library not initialised");
    LSPK_CUDA(launch(wait_expiry_probe_kernel, dim3(1), dim3(32), 0, false, flag, polls));
    return LSPK_OK;
}

}  // namespace lspk

extern "C" int lspk_tc_check_error(void) { return lspk::tensor_core_check_error(); }

extern "C" int lspk_debug_expire_wait(int polls) {
    if (int rc = lspk::ensure_init()) return rc;
    LSPK_REQUIRE(polls >= 1 && polls <= (1 << 16), "lspk_debug_expire_wait: polls must be in 1..65536");
    return lspk::expire_one_wait((unsigned)polls);
}
