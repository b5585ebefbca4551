// Shared device/host helpers for the sm_100a ternary-matmul library.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/lspk_sm100.h"

namespace lspk {

// ---- sticky error state (host) -------------------------------------------------
void set_error(const char* fmt, ...);
int  fail(int code, const char* fmt, ...);          // records the message, returns code
cudaStream_t stream();                              // the library's launch stream
cudaStream_t main_stream();                         // the same, ignoring a measurement override
void set_stream_override(cudaStream_t s);           // measurement aid: route launches to another stream (nullptr: off)
bool pdl_enabled();                                 // programmatic dependent launch on/off
int  sm_count();
int  ensure_init();                                 // bind to a GPU on first use
// Library-owned device scratch (the row quantiser's buffers, the K-split workspace, the per-layer buffers of
// the MoE and Mamba blocks) grows by free + malloc, which moves it.  A CUDA graph captured earlier holds the
// old addresses, so whoever moves scratch bumps this counter and every graph owner compares it with the value
// it recorded at capture and re-captures when they differ.
unsigned scratch_generation();
void scratch_moved();

#define LSPK_CUDA(expr)                                                              \
    do {                                                                             \
        cudaError_t _e = (expr);                                                     \
        if (_e != cudaSuccess)                                                       \
            return ::lspk::fail(LSPK_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,       \
                                cudaGetErrorString(_e), __FILE__, __LINE__);         \
    } while (0)

#define LSPK_REQUIRE(cond, ...)                                                      \
    do {                                                                             \
        if (!(cond)) return ::lspk::fail(LSPK_ERR_ARG, __VA_ARGS__);                 \
    } while (0)

// ---- device layout of one ternary matrix ---------------------------------------
// The reference stores uint8 [N, K/4], weight k of row n at bits 2*(k%4) of byte k/4.
// On the device the same bytes are regrouped (no bit is changed) into 16-byte chunks
// (64 weights) ordered [row-group of 16][chunk index along K][row within group], so that
// 32 lanes reading "16 rows x 2 consecutive chunks" touch one contiguous 512-byte span.
// Rows are padded to a multiple of 16 and K to a multiple of 64 with code 1 (weight 0).
constexpr int kRowsPerGroup = 16;
constexpr int kWeightsPerChunk = 64;

struct Weight {
    uint4* dev;        // [groups][chunks][16] chunks of 16 bytes
    int N, K;          // logical shape
    int groups;        // ceil(N / 16)
    int chunks;        // ceil(K / 64)
    float scale;       // per-tensor weight scale
    size_t bytes;      // groups * chunks * 16 * 16
};

// ---- launch helper: optional programmatic dependent launch ----------------------
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                          bool allow_pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    if (allow_pdl && pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Same, for a kernel whose CTAs form thread-block clusters of `cluster` CTAs.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, bool allow_pdl,
                                  dim3 cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[2];
    int n = 0;
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster.x;
    attr[n].val.clusterDim.y = cluster.y;
    attr[n].val.clusterDim.z = cluster.z;
    ++n;
    if (allow_pdl && pdl_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ---- optional in-kernel phase trace (measurement aid) -------------------------------------------
// When a trace buffer is installed (lspk_trace_begin), CTA 0 of every traced kernel appends one
// record of kTraceWords 64-bit words: [kernel id, globaltimer at entry, SM clock at up to 12 phase
// marks, globaltimer at exit].  Word 0 of the buffer is the record counter.
// Device int that kernels with bounded waits set to LSPK_ERR_DEVICE_WAIT when a wait runs out (a word of the
// library image whose address lspk_init looks up; read and cleared by lspk_tc_check_error).
int* device_wait_flag();
int  bound_device();                                // ordinal of the GPU the library is bound to, -1 before

constexpr int kTraceWords = 16;
unsigned long long* trace_buffer();       // device pointer or nullptr
int trace_capacity();                     // records

#ifdef __CUDACC__
struct PhaseTrace {
    unsigned long long* rec;
    int n;
    // the recording thread is thread `thread` of block (0, 0, 0)
    __device__ __forceinline__ void begin(unsigned long long* buf, int cap, int kernel_id, int thread = 0) {
        rec = nullptr;
        n = 0;
        if (buf && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == thread) {
            const unsigned long long slot = atomicAdd(buf, 1ull);
            if (slot < (unsigned long long)cap) {
                rec = buf + 1 + slot * kTraceWords;
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                rec[0] = (unsigned long long)kernel_id;
                rec[1] = t;
                for (int i = 2; i < kTraceWords; ++i) rec[i] = 0;
                n = 2;
            }
        }
    }
    __device__ __forceinline__ void mark() {
        if (rec && n < kTraceWords - 1) rec[n++] = (unsigned long long)clock64();
    }
    __device__ __forceinline__ void end() {
        if (rec) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            rec[kTraceWords - 1] = t;
        }
    }
};
#endif

#ifdef __CUDACC__
// ---- device helpers --------------------------------------------------------------

// ---- mbarrier / bulk-copy wrappers -----------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a phase (try_wait may park the thread for a while before it answers).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// Contiguous global -> shared copy by the copy engine (both addresses 16-byte aligned, bytes a multiple of
// 16), completion counted on `bar`; the lines are marked evict-first in L2 (read-once weight stream).
__device__ __forceinline__ void bulk_load_stream(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// The same with a cache policy made once by the caller (createpolicy is an instruction of its own).
__device__ __forceinline__ void bulk_load_policy(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Wait until the kernels this launch depends on have completed and their writes are
// visible.  A no-op when the launch carries no programmatic dependency.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Allow the next kernel in the stream to start launching (it still waits, in its own
// grid_dependency_wait, for this grid to finish before touching what this grid writes).
__device__ __forceinline__ void grid_dependency_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// 4-way byte dot product, unsigned a (weight codes) x signed b (activations), s32 accumulate.
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
    return __uint_as_float(((uint32_t)b) << 16);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide reductions.  `red` is a shared array of at least 32 elements; every thread
// of the block must call; the result is returned to every thread.  Two barriers each, so
// the same `red` can be reused by consecutive calls.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.0f;
    r = warp_sum(r);
    __syncthreads();
    return r;
}
__device__ __forceinline__ int block_sum(int v, int* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    int r = (lane < nw) ? red[lane] : 0;
    r = warp_sum(r);
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    __syncthreads();
    return r;
}

// Per-token absmax int8 quantiser, the arithmetic of the reference's vector path
// (quantize_activation_avx512, matmul_lut_avx512_extern_c.cpp:443-456): every step is a
// single correctly rounded fp32 operation, round-half-even conversion, saturation to
// [-128, 127].
// a / d, correctly rounded, for a divisor whose correctly rounded reciprocal rcp_d = 1.0f / d is at
// hand: q = a * rcp_d is within one ulp of the quotient, the residual a - q * d is exact in a fused
// multiply-add, and q + r * rcp_d then rounds to the true quotient (Markstein's division theorem; it
// needs a divisor whose significand is not all ones -- see fma_division_ok -- and no overflow or
// underflow, hence the range test).  Checked against a / d for every float in [1e-30, 1e30] for
// 127 and for the K values of the model shapes.  Three dependent instructions instead of the
// division subroutine, which sits on the critical path of every fused quantiser.
__device__ __forceinline__ float div_const_rn(float a, float d, float rcp_d) {
    if (!(a >= 1e-30f && a <= 1e30f)) return __fdiv_rn(a, d);
    const float q = __fmul_rn(a, rcp_d);
    const float r = __fmaf_rn(-q, d, a);
    return __fmaf_rn(r, rcp_d, q);
}
// 1 / b, correctly rounded (== __frcp_rn(b) == 1.0f / b): hardware approximation (within one ulp)
// followed by two residual corrections; from any start within two ulps the second one lands on the
// correctly rounded reciprocal unless b's significand is all ones (checked for every float in
// [1e-30, 1e30]); those and out-of-range inputs take the library routine.
__device__ __forceinline__ float rcp_rn(float b) {
    if (!(b >= 1e-30f && b <= 1e30f) || (__float_as_uint(b) & 0x7fffffu) == 0x7fffffu) return __frcp_rn(b);
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(b));
    float r = __fmaf_rn(-b, y, 1.0f);
    y = __fmaf_rn(r, y, y);
    r = __fmaf_rn(-b, y, 1.0f);
    return __fmaf_rn(r, y, y);
}
__device__ __forceinline__ float quant_scale_from_absmax(float absmax) {
    if (absmax < 1e-5f) absmax = 1e-5f;
    return div_const_rn(absmax, 127.0f, 1.0f / 127.0f);
}
__device__ __forceinline__ int quant_one(float v, float inv_scale) {
    int q = __float2int_rn(__fmul_rn(v, inv_scale));
    return max(-128, min(127, q));
}

// Position of activation k inside the permuted int8 row kept in shared memory.  Within each
// 16-element block the 4x4 index grid is transposed, so that the 32-bit word (16*blk + 4*j)
// holds activations 16*blk + {j, 4+j, 8+j, 12+j}: exactly the four activations that multiply
// the four 2-bit fields at bit offset 2*j of the four bytes of a packed weight word.
__device__ __forceinline__ int perm_index(int k) {
    return (k & ~15) | ((k & 3) << 2) | ((k >> 2) & 3);
}
#endif  // __CUDACC__

// Host side: may division by d use div_const_rn (significand of d not all ones)?
inline bool fma_division_ok(float d) {
    uint32_t u;
    memcpy(&u, &d, 4);
    return d > 0.0f && (u & 0x7fffffu) != 0x7fffffu;
}

}  // namespace lspk
