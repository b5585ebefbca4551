// Measurement-only kernels and entry points (declared in include/lspk_bench.h, loaded by bench.py; no product
// path calls anything in this file).
//
// Hand-off probe: what does it cost to pass a 10 KB activation vector from the CTAs that produce it to every
// CTA that consumes it, the step a decode pass repeats about 150 times per token?  One cooperative launch runs
// `iters` rounds; in every round each CTA reads the whole vector of the previous round, reduces it over the CTA
// (what an RMSNorm prologue does) and CTA b < 160 writes its 16-element slice of the next vector.  Two ways of
// knowing that the previous round's data has arrived:
//   mode 0  tagged packets: every element travels as one 64-bit word (fp32 value | round number << 32), written
//           and read with single 64-bit accesses; a reader polls its own 16 packets until they carry the round
//           it expects.  No fence, no counter: one store and one load between producer and consumer.
//   mode 1  counter barrier: plain fp32 stores, then one thread per CTA does a release-add on a global counter
//           and polls it with acquire loads until all CTAs of the round have arrived; plain loads follow.
// Every poll loop is bounded; when a bound is reached the CTA raises the error word and all CTAs leave.
#include <cooperative_groups.h>

#include "runtime_internal.cuh"
#include "../../include/lspk_bench.h"
#include "../../include/lspk_tp.h"

namespace lspk {

constexpr int kProbeVec = 2560;                 // elements of the vector (BitNet-2B hidden size)
constexpr int kProbeWriters = kProbeVec / 16;   // CTAs that write a slice
constexpr unsigned kProbeSpinLimit = 1u << 20;

__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add_u32(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(256) handoff_probe_kernel(unsigned long long* buf_a, unsigned long long* buf_b,
                                                            float* plain_a, float* plain_b, unsigned* counter,
                                                            int* error_word, int iters, int mode, unsigned tag0,
                                                            unsigned long long* cycles_out) {
    __shared__ float red[32];
    __shared__ int s_fail;
    const int tid = threadIdx.x;
    if (tid == 0) s_fail = 0;
    __syncthreads();
    const long long t_begin = clock64();
    for (int it = 1; it <= iters; ++it) {
        const unsigned want = tag0 + (unsigned)it - 1u;          // round whose output is read now
        float acc = 0.0f;
        if (mode == 0) {
            const unsigned long long* src = (it & 1) ? buf_a : buf_b;
            if (tid < kProbeWriters) {
                const unsigned long long* mine = src + tid * 16;
                unsigned long long v[16];
                bool ok = false;
                for (unsigned spin = 0; spin < kProbeSpinLimit && !ok; ++spin) {
                    // the first packet alone is polled; the other fifteen of the slice were written by the same
                    // half warp in the same instruction and are checked once it has arrived
                    v[0] = ld_relaxed_u64(mine);
                    if ((unsigned)(v[0] >> 32) - want > 0x7fffffffu) {       // tag < want
                        if ((spin & 63u) == 63u && *(volatile int*)error_word) break;
                        continue;
                    }
                    ok = true;
#pragma unroll
                    for (int e = 1; e < 16; ++e) {
                        v[e] = ld_relaxed_u64(mine + e);
                        ok = ok && ((unsigned)(v[e] >> 32) - want <= 0x7fffffffu);
                    }
                }
                if (!ok) s_fail = 1;
#pragma unroll
                for (int e = 0; e < 16; ++e) acc += __uint_as_float((unsigned)v[e]);
            }
        } else {
            const float* src = (it & 1) ? plain_a : plain_b;
            if (tid < kProbeWriters) {
                const float4* mine = reinterpret_cast<const float4*>(src) + tid * 4;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 v = __ldcg(mine + q);
                    acc += (v.x + v.y) + (v.z + v.w);
                }
            }
        }
        acc = block_sum(acc, red);
        if (s_fail) {
            if (tid == 0) atomicExch(error_word, LSPK_ERR_DEVICE_WAIT);
            break;
        }
        if (blockIdx.x < kProbeWriters && tid < 16) {
            const float o = acc * 1e-6f + (float)tid;
            if (mode == 0) {
                unsigned long long* dst = ((it & 1) ? buf_b : buf_a) + blockIdx.x * 16 + tid;
                st_relaxed_u64(dst, (unsigned long long)__float_as_uint(o) | ((unsigned long long)(tag0 + (unsigned)it) << 32));
            } else {
                float* dst = ((it & 1) ? plain_b : plain_a) + blockIdx.x * 16 + tid;
                __stcg(dst, o);
            }
        }
        if (mode == 1) {
            __syncthreads();
            if (tid == 0) {
                red_release_add_u32(counter, 1u);
                const unsigned target = (tag0 + (unsigned)it) * gridDim.x;
                bool ok = false;
                for (unsigned spin = 0; spin < kProbeSpinLimit && !ok; ++spin) {
                    ok = ld_acquire_u32(counter) - target <= 0x7fffffffu;
                    if (!ok && (spin & 63u) == 63u && *(volatile int*)error_word) break;
                }
                if (!ok) s_fail = 1;
            }
            __syncthreads();
            if (s_fail) {
                if (tid == 0) atomicExch(error_word, LSPK_ERR_DEVICE_WAIT);
                break;
            }
        }
    }
    if (cycles_out && blockIdx.x == 0 && tid == 0) cycles_out[0] = (unsigned long long)(clock64() - t_begin);
}

}  // namespace lspk

using namespace lspk;

extern "C" int lspk_bench_handoff(int grid, int iters, int mode, float* us_per_round_out, double* cycles_per_round_out) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(grid >= kProbeWriters && grid <= 4 * sm_count() && iters >= 1 && (mode == 0 || mode == 1) && us_per_round_out,
                 "lspk_bench_handoff: grid must be 160 .. 4 x SM count, mode 0 or 1");
    int per_sm = 0;
    LSPK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, handoff_probe_kernel, 256, 0));
    LSPK_REQUIRE(grid <= per_sm * sm_count(), "lspk_bench_handoff: %d CTAs cannot be resident together (%d per SM)", grid, per_sm);
    unsigned char* mem = nullptr;
    const size_t packets = (size_t)kProbeVec * 8, plain = (size_t)kProbeVec * 4;
    const size_t total = 2 * packets + 2 * plain + 256;
    LSPK_CUDA(cudaMalloc((void**)&mem, total));
    LSPK_CUDA(cudaMemsetAsync(mem, 0, total, stream()));
    unsigned long long* buf_a = reinterpret_cast<unsigned long long*>(mem);
    unsigned long long* buf_b = buf_a + kProbeVec;
    float* plain_a = reinterpret_cast<float*>(mem + 2 * packets);
    float* plain_b = plain_a + kProbeVec;
    unsigned* counter = reinterpret_cast<unsigned*>(mem + 2 * packets + 2 * plain);
    int* error_word = reinterpret_cast<int*>(counter + 4);
    unsigned long long* cycles = reinterpret_cast<unsigned long long*>(counter + 8);
    int rc = LSPK_OK;
    float ms = 0.0f;
    unsigned tag0 = 0;
    for (int pass = 0; pass < 2 && rc == LSPK_OK; ++pass) {          // first pass warms up
        // all CTAs have to be resident together: a cooperative launch refuses to start otherwise
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(256);
        cfg.stream = stream();
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeCooperative;
        attr[0].val.cooperative = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (pass == 1) rc = lspk_timer_start();
        if (rc) break;
        cudaError_t e = cudaLaunchKernelEx(&cfg, handoff_probe_kernel, buf_a, buf_b, plain_a, plain_b, counter, error_word,
                                           iters, mode, tag0, cycles);
        if (e != cudaSuccess) {
            rc = fail(LSPK_ERR_CUDA, "hand-off probe launch failed: %s", cudaGetErrorString(e));
            break;
        }
        if (pass == 1) rc = lspk_timer_stop(&ms);
        tag0 += (unsigned)iters;
    }
    int err = 0;
    unsigned long long cyc = 0;
    if (rc == LSPK_OK && cudaMemcpy(&err, error_word, 4, cudaMemcpyDeviceToHost) != cudaSuccess) rc = fail(LSPK_ERR_CUDA, "copy failed");
    if (rc == LSPK_OK && cudaMemcpy(&cyc, cycles, 8, cudaMemcpyDeviceToHost) != cudaSuccess) rc = fail(LSPK_ERR_CUDA, "copy failed");
    cudaFree(mem);
    if (rc) return rc;
    if (err) return fail(LSPK_ERR_DEVICE_WAIT, "hand-off probe: a bounded wait ran out");
    *us_per_round_out = ms * 1000.0f / (float)iters;
    if (cycles_per_round_out) *cycles_per_round_out = (double)cyc / iters;
    return LSPK_OK;
}

// ---- Cluster probe ---------------------------------------------------------------------------------------------
// What a decode step confined to ONE thread-block cluster could do: (1) how many bytes per second the SMs of a
// cluster pull from global memory through rings of bulk copies (the weight stream), and (2) what an exchange of a
// small vector between all CTAs of the cluster costs (each CTA stores its slice into every peer's shared memory,
// then one cluster barrier), the hand-off that a kernel boundary provides between grid-wide stages.
namespace lspk {

constexpr int kCpStage = 16384;              // bytes per ring stage
constexpr int kCpStages = 8;
constexpr unsigned kCpSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t cluster_nctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_rank(const void* smem_ptr, uint32_t rank) {
    uint32_t a = smem_u32(smem_ptr), out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(a), "r"(rank));
    return out;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// mode 0: stream `stages_per_cta` stages of 16 KB per CTA through the ring, no exchange
// mode 1: `rounds` exchanges of a 2560-float vector (slices by rank), no streaming
// mode 2: both: an exchange after every `stages_per_round` stages
// + 4: four warps request the stages (stage k by lane 0 of warp k % 4) instead of one thread requesting all of them
__global__ void __launch_bounds__(256, 1)
cluster_probe_kernel(const unsigned char* __restrict__ src, size_t src_bytes, int stages_per_cta, int rounds,
                     int stages_per_round, int mode, int* error_word, float* sink) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* ring = smem_raw;                                   // [kCpStages][kCpStage]
    float* vec = reinterpret_cast<float*>(smem_raw + kCpStages * kCpStage);   // [2][2560] double-buffered vector
    __shared__ __align__(8) uint64_t bars[kCpStages];
    __shared__ int s_fail;
    const int tid = threadIdx.x;
    const uint32_t rank = cluster_ctarank(), nrank = cluster_nctarank();
    const size_t cta_lin = blockIdx.x;
    const int issuers = (mode & 4) ? 4 : 1;
    mode &= 3;
    if (tid == 0) {
        s_fail = 0;
        for (int s = 0; s < kCpStages; ++s) mbar_init(&bars[s], 1);
        fence_mbar_init();
    }
    __syncthreads();
    cluster_sync_all();                                              // every CTA of the cluster has started
    const int n_stages = mode == 1 ? 0 : stages_per_cta;
    const size_t base = (cta_lin * (size_t)stages_per_cta * kCpStage) % (src_bytes - (size_t)stages_per_cta * kCpStage);
    auto issue = [&](int k) {
        const int s = k % kCpStages;
        mbar_expect_tx(&bars[s], kCpStage);
        bulk_load_stream(ring + (size_t)s * kCpStage, src + ((base + (size_t)k * kCpStage) & ~(size_t)15), kCpStage, &bars[s]);
    };
    const bool issuer = (tid & 31) == 0 && (tid >> 5) < issuers;      // stage k is requested by warp k % issuers
    if (issuer)
        for (int k = tid >> 5; k < kCpStages && k < n_stages; k += issuers) issue(k);
    float acc = 0.0f;
    int done_rounds = 0;
    const int slice = 2560 / (int)nrank;                              // floats of the vector this CTA produces
    auto exchange = [&]() {
        // every thread of this CTA stores part of the CTA's slice into every peer's copy of the vector
        float* dst = vec + (size_t)(done_rounds & 1) * 2560;
        for (int i = tid; i < slice * (int)nrank; i += 256) {
            const uint32_t peer = (uint32_t)(i / slice);
            const int e = (int)rank * slice + (i % slice);
            st_cluster_f32(map_to_rank(dst + e, peer), acc + (float)e);
        }
        cluster_sync_all();
        // consume: reduce the whole vector (what a norm prologue does)
        float v = 0.0f;
        for (int i = tid; i < 2560; i += 256) v += dst[i];
        acc += v * 1e-9f;
        ++done_rounds;
    };
    for (int k = 0; k < n_stages; ++k) {
        const int s = k % kCpStages;
        const uint32_t parity = (uint32_t)(k / kCpStages) & 1u;
        bool ok = false;
        for (unsigned spin = 0; spin < kCpSpinLimit && !ok; ++spin) ok = mbar_try_wait(&bars[s], parity);
        if (!ok) s_fail = 1;
        // touch the stage: one 16-byte read per thread, four times (what a dot product reads once)
        const uint4* st = reinterpret_cast<const uint4*>(ring + (size_t)s * kCpStage);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 w = st[tid + q * 256];
            acc += __uint_as_float((w.x ^ w.y ^ w.z ^ w.w) & 0x007fffffu);
        }
        __syncthreads();
        if (s_fail) break;
        if (issuer && (k + kCpStages) % issuers == (tid >> 5) && k + kCpStages < n_stages) issue(k + kCpStages);
        if (mode == 2 && (k + 1) % stages_per_round == 0) exchange();
    }
    if (mode == 1)
        for (int r = 0; r < rounds; ++r) exchange();
    if (s_fail && tid == 0) atomicExch(error_word, LSPK_ERR_DEVICE_WAIT);
    // copies still in flight after a failed wait: bounded drain
    if (s_fail && tid == 0)
        for (int s = 0; s < kCpStages; ++s)
            for (unsigned spin = 0; spin < kCpSpinLimit && !mbar_try_wait(&bars[s], 0) && !mbar_try_wait(&bars[s], 1); ++spin) {}
    cluster_sync_all();                                              // no CTA leaves while peers may still store into it
    if (sink && acc == 123.456f) sink[0] = acc;
}

}  // namespace lspk

extern "C" int lspk_bench_cluster(int cluster_size, int n_clusters, int stages_per_cta, int rounds, int stages_per_round,
                                  int mode, float* ms_out) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE((cluster_size == 1 || cluster_size == 2 || cluster_size == 4 || cluster_size == 8 || cluster_size == 16) &&
                     n_clusters >= 1 && cluster_size * n_clusters <= sm_count() && mode >= 0 && (mode & 3) <= 2 && mode <= 6 && ms_out &&
                     stages_per_cta >= 1 && stages_per_cta <= 65536 && rounds >= 1 && stages_per_round >= 1,
                 "lspk_bench_cluster: bad arguments");
    const size_t src_bytes = 1ull << 30;
    unsigned char* src = nullptr;
    int* err = nullptr;
    LSPK_CUDA(cudaMalloc((void**)&src, src_bytes));
    LSPK_CUDA(cudaMalloc((void**)&err, 16));
    LSPK_CUDA(cudaMemsetAsync(src, 1, src_bytes, stream()));
    LSPK_CUDA(cudaMemsetAsync(err, 0, 16, stream()));
    const size_t smem = (size_t)kCpStages * kCpStage + 2 * 2560 * 4;
    cudaError_t e = cudaFuncSetAttribute(cluster_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess && cluster_size > 8)
        e = cudaFuncSetAttribute(cluster_probe_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    int rc = LSPK_OK;
    if (e != cudaSuccess) rc = fail(LSPK_ERR_CUDA, "cluster probe: attribute failed: %s", cudaGetErrorString(e));
    for (int pass = 0; pass < 2 && rc == LSPK_OK; ++pass) {
        if (pass == 1) rc = lspk_timer_start();
        if (rc) break;
        e = launch_cluster(cluster_probe_kernel, dim3(cluster_size * n_clusters), dim3(256), smem, false, dim3(cluster_size, 1, 1),
                           (const unsigned char*)src, src_bytes, stages_per_cta, rounds, stages_per_round, mode, err, (float*)nullptr);
        if (e != cudaSuccess) {
            rc = fail(LSPK_ERR_CUDA, "cluster probe launch failed: %s", cudaGetErrorString(e));
            break;
        }
        if (pass == 1) rc = lspk_timer_stop(ms_out);
    }
    int flag = 0;
    if (rc == LSPK_OK && cudaMemcpy(&flag, err, 4, cudaMemcpyDeviceToHost) != cudaSuccess) rc = fail(LSPK_ERR_CUDA, "copy failed");
    cudaFree(src);
    cudaFree(err);
    if (rc) return rc;
    if (flag) return fail(LSPK_ERR_DEVICE_WAIT, "cluster probe: a bounded wait ran out");
    return LSPK_OK;
}


// ---- Timing harnesses of the decode step's pieces (graph replays, CUDA events) ---------------------------------
namespace lspk {

// Takes part in a dependency chain and does what a decode kernel does at its boundaries: every CTA
// reads a 10 KB vector the previous kernel wrote (16 floats per thread, 160 threads), reduces over
// the CTA, and writes its 64-float slice of the next vector.  Measures the floor cost of a kernel
// boundary plus the first read of freshly written data (see lspk_bench_launch_floor).
//   mode bit 0: trigger dependents early; bits 1-2: load flavour (0 plain, 1 .cg, 2 volatile);
//   bit 3: store flavour (0 plain, 1 .cg); bit 4: skip the vector traffic (empty kernel)
__global__ void chain_probe_kernel(int* __restrict__ sink, const float* __restrict__ vin, float* __restrict__ vout,
                                   int mode, unsigned long long* trace, int trace_cap) {
    __shared__ float red[32];
    PhaseTrace tr;
    tr.begin(trace, trace_cap, 5);
    tr.mark();
    if (mode & 1) grid_dependency_launch();
    grid_dependency_wait();
    tr.mark();                                   // 1: predecessor finished
    if (!(mode & 16)) {
        const int tid = threadIdx.x, lf = (mode >> 1) & 3;
        float acc = 0.0f;
        if (tid < 160) {
            const float4* src = reinterpret_cast<const float4*>(vin) + tid * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float4 v;
                if (lf == 1) v = __ldcg(src + q);
                else if (lf == 2) asm volatile("ld.volatile.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(src + q));
                else v = src[q];
                acc += (v.x + v.y) + (v.z + v.w);
            }
        }
        tr.mark();                               // 2: this thread's 64 bytes arrived
        acc = block_sum(acc, red);
        tr.mark();                               // 3: all warps' data arrived and reduced
        if (tid < 64 && blockIdx.x < 160) {
            const float o = acc * 1e-3f + (float)tid;
            float* dst = vout + blockIdx.x * 64 + tid;
            if (mode & 8) __stcg(dst, o); else *dst = o;
        }
    }
    if (sink && threadIdx.x == 0 && blockIdx.x == 0) sink[0] += 1;
    tr.end();
}

}  // namespace lspk

extern "C" {

// Replay, `reps` times, a graph holding only the ternary linear launches of one decode step of a
// single-sequence state (4 per layer: q/k/v, o, gate/up, down -- the attention kernel left out),
// and report the CUDA-event time, the number of linear launches and the algorithmic bytes they
// move (packed weights + fp32 input + fp32 output per launch).
int lspk_bench_linears(lspk_state_t h, int reps, float* ms_out, int* launches_out, double* bytes_out) {
    State* s = reinterpret_cast<State*>(h);
    LSPK_REQUIRE(s && s->batch == 1 && reps >= 1 && ms_out, "lspk_bench_linears: needs a single-sequence state");
    Model* m = s->m;
    const lspk_model_config& c = m->cfg;
    static cudaGraphExec_t exec = nullptr;
    static State* exec_for = nullptr;
    auto enqueue = [&]() -> int {
        if (int rc = launch_embed(s->ctl + 1, 1, m->emb.kind, m->emb.data, m->emb.scale, s->x, c.hidden_size, c.vocab_size))
            return rc;
        for (int li = 0; li < c.num_layers; ++li)
            if (int rc = run_layer(s, li, 1, false, 0, true)) return rc;
        return LSPK_OK;
    };
    if (!exec || exec_for != s) {
        if (exec) cudaGraphExecDestroy(exec);
        exec = nullptr;
        if (int rc = enqueue()) return rc;
        LSPK_CUDA(cudaStreamSynchronize(stream()));
        cudaGraph_t g = nullptr;
        LSPK_CUDA(cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal));
        int rc = enqueue();
        cudaError_t e = cudaStreamEndCapture(stream(), &g);
        if (rc) return rc;
        if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        e = cudaGraphInstantiate(&exec, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
        exec_for = s;
    }
    LSPK_CUDA(cudaGraphLaunch(exec, stream()));          // warm
    if (int rc = lspk_timer_start()) return rc;
    for (int i = 0; i < reps; ++i) LSPK_CUDA(cudaGraphLaunch(exec, stream()));
    if (int rc = lspk_timer_stop(ms_out)) return rc;
    const double H = c.hidden_size, I = c.intermediate_size, KV = m->kv_dim();
    const double per_layer = (H * H / 4 + 2 * KV * H / 4 + 4 * H + 4 * (H + 2 * KV))      // q/k/v
                           + (H * H / 4 + 4 * H + 4 * H)                                   // o
                           + (2 * I * H / 4 + 4 * H + 4 * I)                               // gate/up
                           + (H * I / 4 + 4 * I + 4 * H);                                  // down
    if (launches_out) *launches_out = 4 * c.num_layers;
    if (bytes_out) *bytes_out = per_layer * c.num_layers;
    return LSPK_OK;
}

// Time `reps` LM-head launches (final norm + argmax fused, no logits store) of a single-sequence state.
int lspk_bench_lm_head(lspk_state_t h, int reps, float* ms_out, double* bytes_out) {
    State* s = reinterpret_cast<State*>(h);
    LSPK_REQUIRE(s && s->batch == 1 && reps >= 1 && ms_out, "lspk_bench_lm_head: needs a single-sequence state");
    Model* m = s->m;
    const lspk_model_config& c = m->cfg;
    const DevTable& head = m->head.data ? m->head : m->emb;
    auto once = [&]() -> int {
        return lm_head_launch(head.kind, head.data, head.scale, s->x, nullptr, 1, c.vocab_size, c.hidden_size,
                              m->final_norm.g, m->final_norm.is_bf16, c.rms_norm_eps, s->best);
    };
    if (int rc = once()) return rc;
    if (int rc = lspk_timer_start()) return rc;
    for (int i = 0; i < reps; ++i)
        if (int rc = once()) return rc;
    if (int rc = lspk_timer_stop(ms_out)) return rc;
    LSPK_CUDA(cudaMemsetAsync(s->best, 0, 8, stream()));
    if (bytes_out) *bytes_out = (double)table_bytes(head.kind, c.vocab_size, c.hidden_size) + 4.0 * c.hidden_size;
    return LSPK_OK;
}

// Time the fused-quantiser linear product y = W_i (quant x) over `n_w` device copies of a matrix,
// visited round-robin so that consecutive launches read different HBM (defeats the L2 when the
// copies together exceed it).  One pass over all copies is captured into a graph and replayed.
int lspk_bench_linear_copies(const lspk_weight_t* w, int n_w, const float* x_f32, float* y, int M, int reps,
                             float* ms_out) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(w && n_w >= 1 && x_f32 && y && M >= 1 && reps >= 1 && ms_out, "lspk_bench_linear_copies: bad arguments");
    auto enqueue = [&]() -> int {
        for (int i = 0; i < n_w; ++i) {
            lspk_linear_args a = {};
            a.w[0] = w[i];
            a.out[0] = y;
            a.n_mats = 1;
            a.M = M;
            a.prologue = LSPK_PRO_QUANT;
            a.epilogue = LSPK_EPI_STORE;
            a.x_f32 = x_f32;
            if (int rc = lspk_linear(&a)) return rc;
        }
        return LSPK_OK;
    };
    if (int rc = enqueue()) return rc;                   // sizes scratch, sets kernel attributes
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    cudaGraph_t g = nullptr;
    cudaGraphExec_t exec = nullptr;
    LSPK_CUDA(cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal));
    int rc = enqueue();
    cudaError_t e = cudaStreamEndCapture(stream(), &g);
    if (rc) return rc;
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
    cudaGraphLaunch(exec, stream());
    rc = lspk_timer_start();
    for (int i = 0; i < reps && !rc; ++i)
        if (cudaGraphLaunch(exec, stream()) != cudaSuccess) rc = fail(LSPK_ERR_CUDA, "graph launch failed");
    if (!rc) rc = lspk_timer_stop(ms_out);
    cudaStreamSynchronize(stream());
    cudaGraphExecDestroy(exec);
    return rc;
}

// The same product, but the launches of one pass do not depend on one another: they are captured on
// `n_streams` forked streams (round-robin, one output buffer per stream), so the graph holds independent
// kernel nodes and the GPU may overlap them.  This is the amortised single-GEMV figure: what the kernel
// streams when it is not a link in a dependency chain.  y must hold n_streams * N floats.
int lspk_bench_linear_copies_independent(const lspk_weight_t* w, const lspk_weight_t* w_up, int n_w, const float* x_f32,
                                         float* y, int M, int reps, int n_streams, int int8_input, float* ms_out) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(w && n_w >= 1 && x_f32 && y && M == 1 && reps >= 1 && ms_out && n_streams >= 1 && n_streams <= 16,
                 "lspk_bench_linear_copies_independent: bad arguments (one row only: more rows share library scratch)");
    const Weight* w0 = reinterpret_cast<const Weight*>(w[0]);
    const size_t y_stride = (size_t)M * w0->N;
    // int8_input: the reference kernel's own contract (matmul_lut_*_m1 takes the quantised vector and its
    // scale); x is quantised once, outside the timed region
    int8_t* xq = nullptr;
    float* xs = nullptr;
    if (int8_input) {
        LSPK_CUDA(cudaMalloc((void**)&xq, (size_t)w0->K + 16));
        LSPK_CUDA(cudaMalloc((void**)&xs, 16));
        if (int rc = lspk_quantize_rows(x_f32, xq, xs, 1, w0->K)) return rc;
    }
    auto one = [&](int i, float* out) -> int {
        lspk_linear_args a = {};
        a.w[0] = w[i];
        a.out[0] = out;
        a.n_mats = 1;
        a.M = M;
        a.epilogue = LSPK_EPI_STORE;
        if (w_up) {                                       // the fused gate/up launch of a feed-forward block
            a.w[1] = w_up[i];
            a.n_mats = 2;
            a.epilogue = LSPK_EPI_RELU2_MUL;
        }
        if (int8_input) {
            a.prologue = LSPK_PRO_INT8;
            a.x_i8 = xq;
            a.x_scales = xs;
        } else {
            a.prologue = LSPK_PRO_QUANT;
            a.x_f32 = x_f32;
        }
        return lspk_linear(&a);
    };
    if (int rc = one(0, y)) return rc;                    // sets kernel attributes
    // one graph holds several passes over the matrices, so that the fork and join of a replay weigh little
    const int passes = n_w >= 256 ? 1 : (256 + n_w - 1) / n_w;
    LSPK_CUDA(cudaStreamSynchronize(main_stream()));
    cudaStream_t side[16] = {};
    cudaEvent_t fork = nullptr, join[16] = {};
    int rc = LSPK_OK;
    cudaError_t e = cudaEventCreateWithFlags(&fork, cudaEventDisableTiming);
    for (int s = 0; s < n_streams && e == cudaSuccess; ++s) {
        e = cudaStreamCreateWithFlags(&side[s], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&join[s], cudaEventDisableTiming);
    }
    cudaGraph_t g = nullptr;
    cudaGraphExec_t exec = nullptr;
    if (e == cudaSuccess) e = cudaStreamBeginCapture(main_stream(), cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
        cudaEventRecord(fork, main_stream());
        for (int s = 0; s < n_streams; ++s) cudaStreamWaitEvent(side[s], fork, 0);
        const bool pdl_was = pdl_enabled();
        lspk_set_pdl(0);                                  // no programmatic edges: plain independent nodes
        for (int i = 0; i < n_w * passes && rc == LSPK_OK; ++i) {
            set_stream_override(side[i % n_streams]);
            rc = one(i % n_w, y + (size_t)(i % n_streams) * y_stride);
        }
        set_stream_override(nullptr);
        lspk_set_pdl(pdl_was ? 1 : 0);
        for (int s = 0; s < n_streams; ++s) {
            cudaEventRecord(join[s], side[s]);
            cudaStreamWaitEvent(main_stream(), join[s], 0);
        }
        e = cudaStreamEndCapture(main_stream(), &g);
    }
    if (e == cudaSuccess && rc == LSPK_OK) e = cudaGraphInstantiate(&exec, g, 0);
    if (g) cudaGraphDestroy(g);
    if (e == cudaSuccess && rc == LSPK_OK) {
        cudaGraphLaunch(exec, main_stream());
        rc = lspk_timer_start();
        for (int i = 0; i < reps && !rc; ++i)
            if (cudaGraphLaunch(exec, main_stream()) != cudaSuccess) rc = fail(LSPK_ERR_CUDA, "graph launch failed");
        if (!rc) rc = lspk_timer_stop(ms_out);
        if (!rc) *ms_out /= (float)passes;                // time of reps passes over the n_w matrices
        cudaStreamSynchronize(main_stream());
    }
    if (exec) cudaGraphExecDestroy(exec);
    for (int s = 0; s < n_streams; ++s) {
        if (join[s]) cudaEventDestroy(join[s]);
        if (side[s]) cudaStreamDestroy(side[s]);
    }
    if (fork) cudaEventDestroy(fork);
    if (xq) cudaFree(xq);
    if (xs) cudaFree(xs);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "independent-launch benchmark failed: %s", cudaGetErrorString(e));
    return rc;
}

// Floor cost of a dependent kernel boundary: replay a graph of `n_kernels` kernels of `grid` CTAs x
// 256 threads that do no work, each depending on the previous one, and report the time of `reps` replays.
int lspk_bench_launch_floor(int n_kernels, int grid, int reps, float* ms_out) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(n_kernels >= 1 && grid >= 1 && reps >= 1 && ms_out, "lspk_bench_launch_floor: bad arguments");
    int* sink = nullptr;
    LSPK_CUDA(cudaMalloc(&sink, 16 + 2 * 10240 * 4));
    LSPK_CUDA(cudaMemset(sink, 0, 16 + 2 * 10240 * 4));
    float* va = reinterpret_cast<float*>(sink + 4);
    float* vb = va + 10240;
    const int mode = 17;                                  // empty kernels, early trigger
    LSPK_CUDA(cudaDeviceSynchronize());
    cudaGraph_t g = nullptr;
    cudaGraphExec_t exec = nullptr;
    LSPK_CUDA(cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal));
    cudaError_t le = cudaSuccess;
    for (int i = 0; i < n_kernels && le == cudaSuccess; ++i)
        le = launch(chain_probe_kernel, dim3(grid), dim3(256), 0, true, sink, (const float*)((i & 1) ? vb : va), (i & 1) ? va : vb, mode,
                    trace_buffer(), trace_capacity());
    cudaError_t e = cudaStreamEndCapture(stream(), &g);
    if (le != cudaSuccess || e != cudaSuccess) {
        cudaFree(sink);
        return fail(LSPK_ERR_CUDA, "launch-floor capture failed: %s", cudaGetErrorString(le != cudaSuccess ? le : e));
    }
    e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) {
        cudaFree(sink);
        return fail(LSPK_ERR_CUDA, "launch-floor instantiate failed: %s", cudaGetErrorString(e));
    }
    cudaGraphLaunch(exec, stream());
    int rc = lspk_timer_start();
    for (int i = 0; i < reps && !rc; ++i)
        if (cudaGraphLaunch(exec, stream()) != cudaSuccess) rc = fail(LSPK_ERR_CUDA, "graph launch failed");
    if (!rc) rc = lspk_timer_stop(ms_out);
    cudaStreamSynchronize(stream());
    cudaGraphExecDestroy(exec);
    cudaFree(sink);
    return rc;
}

// Time `reps` replays of a graph holding `n_blocks` such MLP blocks over distinct weight triples.
// inter_full == NULL: the gathers go through the peer windows (lspk_tp_mlp_block_peer) instead of NCCL.
int lspk_tp_bench_mlp(const lspk_weight_t* gate_r, const lspk_weight_t* up_r, const lspk_weight_t* down_r, int n_blocks,
                      const float* x_dev, const void* norm_gamma_bf16, const void* sub_norm_gamma_bf16, float eps,
                      float* inter_slice, float* inter_full, float* down_slice, float* y_full, int reps, float* ms_out) {
    LSPK_REQUIRE(gate_r && up_r && down_r && n_blocks >= 1 && reps >= 1 && ms_out, "lspk_tp_bench_mlp: bad arguments");
    auto enqueue = [&]() -> int {
        for (int i = 0; i < n_blocks; ++i) {
            const int rc = inter_full
                ? lspk_tp_mlp_block(gate_r[i], up_r[i], down_r[i], x_dev, norm_gamma_bf16, sub_norm_gamma_bf16, eps,
                                    inter_slice, inter_full, down_slice, y_full)
                : lspk_tp_mlp_block_peer(gate_r[i], up_r[i], down_r[i], x_dev, norm_gamma_bf16, sub_norm_gamma_bf16, eps,
                                         inter_slice, down_slice);
            if (rc) return rc;
        }
        return LSPK_OK;
    };
    if (int rc = enqueue()) return rc;
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    cudaGraph_t g = nullptr;
    cudaGraphExec_t exec = nullptr;
    LSPK_CUDA(cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal));
    int rc = enqueue();
    cudaError_t e = cudaStreamEndCapture(stream(), &g);
    if (rc) return rc;
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(&exec, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
    cudaGraphLaunch(exec, stream());
    rc = lspk_timer_start();
    for (int i = 0; i < reps && !rc; ++i)
        if (cudaGraphLaunch(exec, stream()) != cudaSuccess) rc = fail(LSPK_ERR_CUDA, "graph launch failed");
    if (!rc) rc = lspk_timer_stop(ms_out);
    cudaStreamSynchronize(stream());
    cudaGraphExecDestroy(exec);
    return rc;
}


}  // extern "C"
