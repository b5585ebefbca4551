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

#include "internal.cuh"
#include "../../include/lspk_bench.h"

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
