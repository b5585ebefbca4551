// Many independent one-row ternary products in ONE launch (lspk_linear_batch).
//
// The reference's kernel benchmark calls matmul_lut_*_m1 in a loop over matrices that do not depend on one
// another (benchmark_kernel.py, the per-shape timing loops; kernel matmul_lut_avx512_m1,
// matmul_lut_avx512_extern_c.cpp:150-236).  On the GPU a launch per matrix pays a ramp every time: a 4.4 MB
// matrix is 0.7 us of HBM time, shorter than the fill and drain of a kernel.  Here the whole list is one
// stream of bytes: the row groups of all products form one flat sequence of units; every CTA of a persistent
// grid (one per SM) takes a contiguous range of it.  Six warps of the CTA do nothing but request the range's
// stages, in order (stage q by warp q % 6), into a ring of eighteen 10 KB slots in shared memory (cp.async.bulk +
// mbarrier, across product boundaries); twelve consumer warps take the units round-robin, each computing its unit alone.  A range touches
// one or two products, so a CTA installs one or two vectors.
//
//   unit   = 16 output rows of one product (both matrices of a gated gate/up pair), cut along K into stages of
//            at most 10 KB; a warp accumulates a unit's stages in registers and stores its 16 results itself:
//            no CTA-wide barrier per unit, only one per product (when the next activation vector is installed)
//   vector = the int8 activations of product i + 1 are fetched into registers while product i is computed, then
//            byte-transposed into the other of two shared-memory slots
// The arithmetic per row is integer throughout and equal to the one-row kernel's (masked 2-bit fields at their bit
// offset, dp4a, exact shifts, sum(x) subtracted once), so results are bit-identical to lspk_linear.  Every wait is
// bounded by one deadline in SM cycles (about a second for the whole CTA): on expiry the warp raises the
// library's wait flag and leaves its ring alone; the other warps stop computing but keep waiting for the copies
// already requested for them, and all keep the CTA's barriers company until the kernel ends.
#include "internal.cuh"
#include "ternary_core.cuh"

namespace lspk {

constexpr int kSConsumers = 12;                  // warps that compute
// Warps that only request copies (one lane each; stage q belongs to warp q % kSProducers).  One thread gets a
// bulk copy out every ~500 cycles, i.e. 20 bytes per cycle and SM with 10 KB stages: measured on the gate shape,
// 1 / 2 / 4 / 6 requesting warps reach 0.60 / 0.75 / 0.87 / 0.93 of the measured HBM copy rate.
constexpr int kSProducers = 6;
constexpr int kSThreads = 32 * (kSConsumers + kSProducers);
constexpr int kSSlots = 18;                      // stages of the CTA's ring (shared by all consumer warps)
constexpr int kSStageChunks = 40;                // 16-row x 16-byte chunks per stage (all matrices of a unit)
constexpr int kSStageBytes = kSStageChunks * kRowsPerGroup * 16;   // 10240: 180 KB of ring per SM
constexpr int kSMaxItems = kStreamMaxItems;
constexpr int kSMaxKp = kStreamMaxKp;
constexpr long long kSBudgetCycles = 1ll << 31;  // SM cycles (about a second) after which every wait of a CTA gives up

__device__ __forceinline__ void consumer_barrier() {      // the consumer warps only (the requesting warps never join)
    asm volatile("bar.sync 1, %0;" ::"n"(32 * kSConsumers) : "memory");
}

__global__ void __launch_bounds__(kSThreads, 1)
ternary_gemv_stream_kernel(const __grid_constant__ StreamParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint4* ring = reinterpret_cast<uint4*>(smem_raw);                                   // [slots][stage]
    int8_t* xq = reinterpret_cast<int8_t*>(smem_raw + (size_t)kSSlots * kSStageBytes);  // [2][kSMaxKp]
    __shared__ __align__(8) uint64_t full[kSSlots], empty[kSSlots];
    __shared__ int s_seq[kSSlots];               // 1 + the number of the last stage requested into each slot (0: none yet)
    __shared__ int s_sumx[2][kSConsumers];
    __shared__ float s_scale[2];
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // this CTA's range of units [u_lo, u_hi) and the products it touches [i_lo, i_hi]
    const int per_cta = (p.total_units + (int)gridDim.x - 1) / (int)gridDim.x;
    const int u_lo = min((int)blockIdx.x * per_cta, p.total_units), u_hi = min(u_lo + per_cta, p.total_units);
    int i_lo = 0, i_hi = -1;
    if (u_lo < u_hi) {
        while (u_lo >= p.it[i_lo].unit0 + p.it[i_lo].groups) ++i_lo;
        i_hi = i_lo;
        while (u_hi - 1 >= p.it[i_hi].unit0 + p.it[i_hi].groups) ++i_hi;
    }
    // stage number (over the whole call) of the first stage of this CTA's first unit
    const int q_lo = i_hi >= i_lo ? p.it[i_lo].q0 + (u_lo - p.it[i_lo].unit0) * p.it[i_lo].sub : 0;

    // Every wait below is bounded by one deadline for the whole CTA, in SM cycles: whatever goes wrong, the kernel
    // is over about a second later.
    const long long deadline = clock64() + kSBudgetCycles;
    auto expired = [&]() { return clock64() > deadline || *(volatile int*)&s_abort != 0; };
    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < kSSlots; ++s) {
            s_seq[s] = 0;
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        fence_mbar_init();
    }
    __syncthreads();
    grid_dependency_launch();
    auto expert_of = [&](const StreamItem& it) -> size_t { return it.sel ? (size_t)*(volatile const int*)it.sel : 0; };

    if (warp >= kSConsumers) {
        const int pw = warp - kSConsumers;
        if (p.wait_for_predecessor) grid_dependency_wait();      // which matrices to stream is the previous kernel's output
        // ---------------- producers: lane 0 of warp pw requests stages pw, pw + kSProducers, ... as slots come free --
        // (the weights do not depend on whatever ran before, so this starts at once)
        if (lane == 0 && i_hi >= i_lo) {
            uint64_t policy;
            asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
            int q = 0;
            bool ok = true;
            for (int i = i_lo; i <= i_hi && ok; ++i) {
                const StreamItem& it = p.it[i];
                const int g_first = max(u_lo, it.unit0) - it.unit0, g_end = min(u_hi, it.unit0 + it.groups) - it.unit0;
                const int nm = it.nm, chunks = it.chunks, cps = it.cps, sub = it.sub;
                const size_t w_off = expert_of(it) * it.sel_stride;
                const uint4* ua = it.w[0] + w_off + (size_t)g_first * chunks * kRowsPerGroup;
                const uint4* ub = nm == 2 ? it.w[1] + w_off + (size_t)g_first * chunks * kRowsPerGroup : nullptr;
                for (int g = g_first; g < g_end && ok; ++g) {
                    for (int s = 0; s < sub; ++s, ++q) {
                        if (q % kSProducers != pw) continue;
                        const int slot = q % kSSlots;
                        if (q >= kSSlots) {          // the slot's previous occupant has to be consumed first
                            const uint32_t parity = (uint32_t)(q / kSSlots - 1) & 1u;
                            bool freed = mbar_try_wait(&empty[slot], parity);
                            while (!freed && !expired()) freed = mbar_try_wait(&empty[slot], parity);
                            if (!freed) {
                                ok = false;
                                break;
                            }
                        }
                        const int c0 = s * cps, c1 = min(c0 + cps, chunks);
                        const uint32_t bytes = (uint32_t)(c1 - c0) * kRowsPerGroup * 16u;
                        uint4* dst = ring + (size_t)slot * (kSStageBytes / 16);
                        mbar_expect_tx(&full[slot], bytes * (uint32_t)nm);
                        bulk_load_policy(dst, ua + (size_t)c0 * kRowsPerGroup, bytes, &full[slot], policy);
                        if (nm == 2)
                            bulk_load_policy(dst + (size_t)(c1 - c0) * kRowsPerGroup, ub + (size_t)c0 * kRowsPerGroup, bytes,
                                             &full[slot], policy);
                        // Tell the consumers that stage q's phase of full[slot] is now the current one.  A consumer
                        // must not test a phase parity before the previous use of the slot has completed (the test
                        // would succeed at once on the stale phase); the release observed above implies that it has.
                        __threadfence_block();
                        *(volatile int*)&s_seq[slot] = q + 1;
                    }
                    ua += (size_t)chunks * kRowsPerGroup;
                    if (nm == 2) ub += (size_t)chunks * kRowsPerGroup;
                }
            }
            if (!ok && !*(volatile int*)&s_abort) {               // a consumer did not free its slot in time
                s_abort = 1;
                if (p.error_flag) atomicExch(p.error_flag, LSPK_ERR_DEVICE_WAIT);
            }
        }
        return;      // consumers wait for everything that was requested
    }

    // ---------------- consumers: warp w takes units u_lo + w, u_lo + w + 12, ... ----------------------------------
    const int r = lane & 15, h = lane >> 4;
    grid_dependency_wait();

    // activation vector of product `i`: this thread's 16-byte blocks (at most two), raw, into registers
    constexpr int kXB = (kSMaxKp / 16 + 32 * kSConsumers - 1) / (32 * kSConsumers);
    uint32_t raw[kXB][4];
    auto fetch_x = [&](int i) {
        const StreamItem& it = p.it[i];
        const int Kp = it.chunks * kWeightsPerChunk;
#pragma unroll
        for (int u = 0; u < kXB; ++u) {
            const int k0 = (tid + u * 32 * kSConsumers) * 16;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int k = k0 + q * 4;
                raw[u][q] = (k0 < Kp && k < it.K) ? *reinterpret_cast<const uint32_t*>(it.x + k) : 0u;
            }
        }
    };
    auto install_x = [&](int i) {                 // registers -> transposed int8 row in slot i & 1, partial sum(x)
        const StreamItem& it = p.it[i];
        const int Kp = it.chunks * kWeightsPerChunk;
        int8_t* dst = xq + (size_t)(i & 1) * kSMaxKp;
        int sumx = 0;
#pragma unroll
        for (int u = 0; u < kXB; ++u) {
            const int k0 = (tid + u * 32 * kSConsumers) * 16;
            if (k0 < Kp) {
                uint32_t o0, o1, o2, o3;
                transpose4x4_bytes(raw[u][0], raw[u][1], raw[u][2], raw[u][3], o0, o1, o2, o3);
                sumx = __dp4a((int)o0, 0x01010101, sumx);
                sumx = __dp4a((int)o1, 0x01010101, sumx);
                sumx = __dp4a((int)o2, 0x01010101, sumx);
                sumx = __dp4a((int)o3, 0x01010101, sumx);
                *reinterpret_cast<uint4*>(dst + k0) = make_uint4(o0, o1, o2, o3);
            }
        }
        sumx = __reduce_add_sync(0xffffffffu, sumx);
        if (lane == 0) s_sumx[i & 1][warp] = sumx;
        if (tid == 0) s_scale[i & 1] = it.xs[0];
    };
    if (i_hi >= i_lo) {
        fetch_x(i_lo);
        install_x(i_lo);
    }
    consumer_barrier();

    bool dead = false;                           // a wait of this warp ran out: it leaves the ring alone from here on
    bool skip = false;                           // another warp gave up: keep draining the ring, compute nothing
    int unit = u_lo + warp;
    for (int i = i_lo; i <= i_hi; ++i) {
        if (i < i_hi) fetch_x(i + 1);            // in flight while product i is computed
        const StreamItem& it = p.it[i];
        const int8_t* xrow = xq + (size_t)(i & 1) * kSMaxKp;
        int sx = 0;
#pragma unroll
        for (int w = 0; w < kSConsumers; ++w) sx += s_sumx[i & 1][w];
        const float xscale = s_scale[i & 1];
        float ws0 = it.ws[0], ws1 = it.ws[1];
        if (it.sel) {
            const size_t e = expert_of(it);
            ws0 = it.sel_scales[3 * e + it.scale_idx[0]];
            ws1 = it.sel_scales[3 * e + it.scale_idx[1]];
        }
        const int unit_end = min(u_hi, it.unit0 + it.groups);
        for (; !dead && unit < unit_end; unit += kSConsumers) {
            const int g = unit - it.unit0;
            int acc_a[4] = {0, 0, 0, 0}, acc_b[4] = {0, 0, 0, 0};
            for (int s = 0; s < it.sub; ++s) {
                const int q = it.q0 + g * it.sub + s - q_lo;       // this stage's number in the CTA's sequence
                const int slot = q % kSSlots;
                const uint32_t parity = (uint32_t)(q / kSSlots) & 1u;
                // first the request (see the producer), then the data
                bool arrived = *(volatile int*)&s_seq[slot] > q;
                while (!arrived && !(clock64() > deadline)) arrived = *(volatile int*)&s_seq[slot] > q;
                if (arrived) {
                    arrived = mbar_try_wait(&full[slot], parity);
                    while (!arrived && !(clock64() > deadline)) arrived = mbar_try_wait(&full[slot], parity);
                }
                if (!__all_sync(0xffffffffu, arrived)) {
                    dead = true;
                    if (lane == 0) {
                        s_abort = 1;
                        if (p.error_flag) atomicExch(p.error_flag, LSPK_ERR_DEVICE_WAIT);
                    }
                    break;
                }
                const int c0 = s * it.cps, c1 = min(c0 + it.cps, it.chunks);
                const uint4* sa = ring + (size_t)slot * (kSStageBytes / 16);
                const uint4* sb = sa + (size_t)(c1 - c0) * kRowsPerGroup;
                // this half-warp's chunks c0 + h, c0 + h + 2, ...: constant strides from here on (32 uint4 of weights,
                // 128 bytes of activations per step), so the unrolled loop addresses everything by immediates
                const int nit = skip ? 0 : (c1 - c0 - h + 1) >> 1;
                const uint4* wp = sa + h * kRowsPerGroup + r;
                const int4* xp = reinterpret_cast<const int4*>(xrow + (size_t)(c0 + h) * 64);
                if (it.nm == 2) {
                    const uint4* wq = sb + h * kRowsPerGroup + r;
#pragma unroll 4
                    for (int t = 0; t < nit; ++t) {
                        chunk_dot(wp[t * 2 * kRowsPerGroup], xp + t * 8, acc_a);
                        chunk_dot(wq[t * 2 * kRowsPerGroup], xp + t * 8, acc_b);
                    }
                } else {
#pragma unroll 4
                    for (int t = 0; t < nit; ++t) chunk_dot(wp[t * 2 * kRowsPerGroup], xp + t * 8, acc_a);
                }
                // hand the slot back to the producer: every lane has read it
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);
            }
            if (dead || skip) continue;
            int va = acc_a[0] + (acc_a[1] >> 2) + (acc_a[2] >> 4) + (acc_a[3] >> 6);
            va += __shfl_down_sync(0xffffffffu, va, 16);
            int vb = 0;
            if (it.nm == 2) {
                vb = acc_b[0] + (acc_b[1] >> 2) + (acc_b[2] >> 4) + (acc_b[3] >> 6);
                vb += __shfl_down_sync(0xffffffffu, vb, 16);
            }
            const int n = g * kRowsPerGroup + r;
            if (h == 0 && n < it.N) {
                va -= sx;
                if (it.acc[0]) it.acc[0][n] = va;
                const float ya = __fmul_rn((float)va, __fmul_rn(xscale, ws0));
                if (it.nm == 2) {
                    vb -= sx;
                    if (it.acc[1]) it.acc[1][n] = vb;
                    const float yb = __fmul_rn((float)vb, __fmul_rn(xscale, ws1));
                    if (it.epilogue == LSPK_EPI_SILU_MUL) {
                        it.out[n] = __fmul_rn(__fdiv_rn(ya, __fadd_rn(expf(-ya), 1.0f)), yb);
                    } else {
                        const float gpos = fmaxf(ya, 0.0f);
                        it.out[n] = __fmul_rn(__fmul_rn(gpos, gpos), yb);
                    }
                } else if (it.epilogue == LSPK_EPI_ADD) {
                    it.out[n] = __fadd_rn(it.out[n], ya);
                } else {
                    it.out[n] = ya;
                }
            }
        }
        if (i < i_hi) install_x(i + 1);
        consumer_barrier();
        // After an abort elsewhere in the CTA this warp still waits for (and releases) every stage requested for it,
        // so that no copy lands in shared memory after the CTA has gone; it only stops computing.
        if (*(volatile int*)&s_abort) skip = true;
    }
}

static size_t stream_smem_bytes() { return (size_t)kSSlots * kSStageBytes + 2 * (size_t)kSMaxKp; }

int stream_launch(StreamParams* p) {
    LSPK_REQUIRE(p && p->n >= 1 && p->n <= kSMaxItems, "streamed batch: 1..%d products per launch", kSMaxItems);
    p->error_flag = device_wait_flag();
    p->wait_for_predecessor = 0;
    int unit0 = 0, q0 = 0;
    for (int i = 0; i < p->n; ++i) {
        StreamItem& it = p->it[i];
        LSPK_REQUIRE(it.chunks * kWeightsPerChunk <= kSMaxKp, "streamed batch: product %d: K=%d too long (limit %d)", i, it.K, kSMaxKp);
        it.unit0 = unit0;
        it.q0 = q0;
        it.cps = kSStageChunks / it.nm;
        it.sub = (it.chunks + it.cps - 1) / it.cps;
        unit0 += it.groups;
        q0 += it.groups * it.sub;
        if (it.sel) p->wait_for_predecessor = 1;
    }
    p->total_units = unit0;
    static bool attr_set = false;
    const size_t smem = stream_smem_bytes();
    if (!attr_set) {
        LSPK_CUDA(cudaFuncSetAttribute(ternary_gemv_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set = true;
    }
    // one CTA per SM as soon as there are two units for each: a short batch is bound by how many SMs pull on it
    // (an SM takes in about 76 GB/s through the copy engine), not by idle consumer warps
    int ctas = (unit0 + 1) / 2;
    if (ctas > sm_count()) ctas = sm_count();
    if (ctas < 1) ctas = 1;
    LSPK_CUDA(launch(ternary_gemv_stream_kernel, dim3(ctas), dim3(kSThreads), smem, true, *p));
    return LSPK_OK;
}

}  // namespace lspk

using namespace lspk;

extern "C" int lspk_linear_batch(const lspk_linear_args* args, int n) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(args && n >= 1 && n <= kSMaxItems, "lspk_linear_batch: 1..%d products per call (got %d)", kSMaxItems, n);
    static StreamParams p;                        // 10 KB: kept off the stack; calls are serialised by the caller
    p.n = n;
    for (int i = 0; i < n; ++i) {
        const lspk_linear_args& a = args[i];
        const bool pair = a.epilogue == LSPK_EPI_RELU2_MUL || a.epilogue == LSPK_EPI_SILU_MUL;
        LSPK_REQUIRE(a.M == 1, "lspk_linear_batch: product %d has %d rows (one-row products only)", i, a.M);
        LSPK_REQUIRE(a.prologue == LSPK_PRO_INT8 && a.x_i8 && a.x_scales,
                     "lspk_linear_batch: product %d: int8 activations + scale in (quantise fp32 rows first with "
                     "lspk_quantize_rows / lspk_rmsnorm_quantize_rows)", i);
        LSPK_REQUIRE(((uintptr_t)a.x_i8 & 3) == 0, "lspk_linear_batch: product %d: x_i8 must be 4-byte aligned", i);
        LSPK_REQUIRE(a.epilogue >= 0 && a.epilogue <= 3, "lspk_linear_batch: product %d: unknown epilogue", i);
        LSPK_REQUIRE(a.n_mats == (pair ? 2 : 1), "lspk_linear_batch: product %d: one matrix, or gate + up for a gated epilogue", i);
        const Weight* w0 = reinterpret_cast<const Weight*>(a.w[0]);
        LSPK_REQUIRE(w0 && a.out[0], "lspk_linear_batch: product %d: null weight or output", i);
        LSPK_REQUIRE(w0->chunks * kWeightsPerChunk <= kSMaxKp, "lspk_linear_batch: product %d: K=%d too long (limit %d)", i, w0->K, kSMaxKp);
        StreamItem& it = p.it[i];
        it = StreamItem{};
        it.w[0] = w0->dev;
        it.ws[0] = w0->scale;
        it.acc[0] = a.acc_out[0];
        it.nm = pair ? 2 : 1;
        if (pair) {
            const Weight* w1 = reinterpret_cast<const Weight*>(a.w[1]);
            LSPK_REQUIRE(w1 && w1->K == w0->K && w1->N == w0->N, "lspk_linear_batch: product %d: gate and up must have the same shape", i);
            it.w[1] = w1->dev;
            it.ws[1] = w1->scale;
            it.acc[1] = a.acc_out[1];
        }
        it.out = a.out[0];
        it.x = a.x_i8;
        it.xs = a.x_scales;
        it.N = w0->N;
        it.K = w0->K;
        it.chunks = w0->chunks;
        it.groups = w0->groups;
        it.epilogue = a.epilogue;
    }
    return stream_launch(&p);
}
