// RoPE + KV-cache write + causal grouped-query attention on device-resident rows.
//
// Replaces the numpy section of the reference's forward pass: apply_rope / rope tables
// (litespark_inference/torchless/ops.py:40-67), the cache write and the
// scores -> softmax -> weighted sum of runtime.py:224-245 (decode) and :381-407 (prefill).
// Arithmetic order follows the reference: split-half rotation with separately rounded
// products, scores scaled by 1/sqrt(D) after the dot product, max-subtracted softmax,
// probabilities normalised before the V product.  Query head h reads KV head h / (Q / KV).
//
// Cache layout is the reference's: [layer][position][kv_head][D], in fp32 or fp16.
#include "internal.cuh"

namespace lspk {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;

template <typename KVT> __device__ __forceinline__ float kv_load(const KVT* p);
template <> __device__ __forceinline__ float kv_load<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float kv_load<__half>(const __half* p) { return __half2float(*p); }
template <typename KVT> __device__ __forceinline__ KVT kv_make(float v);
template <> __device__ __forceinline__ float kv_make<float>(float v) { return v; }
template <> __device__ __forceinline__ __half kv_make<__half>(float v) { return __float2half_rn(v); }
template <typename KVT> __device__ __forceinline__ float kv_round(float v);
template <> __device__ __forceinline__ float kv_round<float>(float v) { return v; }
template <> __device__ __forceinline__ float kv_round<__half>(float v) { return __half2float(__float2half_rn(v)); }

__device__ __forceinline__ float rope_elem(const float* row, int d, int half, const float* cos_row,
                                           const float* sin_row) {
    const int i = d < half ? d : d - half;
    const float x1 = row[i], x2 = row[half + i];
    const float c = cos_row[i], s = sin_row[i];
    return d < half ? __fsub_rn(__fmul_rn(x1, c), __fmul_rn(x2, s))
                    : __fadd_rn(__fmul_rn(x1, s), __fmul_rn(x2, c));
}


// Rotate q in place and write rotated k and raw v into the cache, for T rows.
template <typename KVT>
__global__ void __launch_bounds__(kAttnThreads) rope_store_kernel(const AttnParams p) {
    grid_dependency_launch();
    grid_dependency_wait();
    extern __shared__ __align__(16) float rs_smem[];     // (Q + KV) * D raw q and k of this row
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = p.pos_per_row ? p.pos_ptr[t] : p.pos_ptr[0] + t;
    const int D = p.D, half = D / 2;
    const int qd = p.Q * D, kd = p.KV * D;
    float* qrow = p.q + (size_t)t * qd;
    const float* krow = p.k_cur + (size_t)t * kd;
    const float* vrow = p.v_cur + (size_t)t * kd;
    for (int i = tid; i < qd; i += kAttnThreads) rs_smem[i] = qrow[i];
    for (int i = tid; i < kd; i += kAttnThreads) rs_smem[qd + i] = krow[i];
    __syncthreads();
    const float* cr = p.rope_cos + (size_t)pos * half;
    const float* sr = p.rope_sin + (size_t)pos * half;
    for (int i = tid; i < qd; i += kAttnThreads) {
        const int hd = i / D, d = i % D;
        qrow[i] = rope_elem(rs_smem + hd * D, d, half, cr, sr);
    }
    KVT* ck = reinterpret_cast<KVT*>(p.cache_k) + (size_t)t * p.cache_seq_stride + (size_t)pos * kd;
    KVT* cv = reinterpret_cast<KVT*>(p.cache_v) + (size_t)t * p.cache_seq_stride + (size_t)pos * kd;
    for (int i = tid; i < kd; i += kAttnThreads) {
        const int hd = i / D, d = i % D;
        ck[i] = kv_make<KVT>(rope_elem(rs_smem + qd + hd * D, d, half, cr, sr));
        cv[i] = kv_make<KVT>(vrow[i]);
    }
}

// 16 bytes of cache row -> fp32 values (8 halves or 4 floats).
template <typename KVT> struct KvVec;
template <> struct KvVec<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& c, float* f) {
        const __half2* h = reinterpret_cast<const __half2*>(&c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 v = __half22float2(h[i]);
            f[2 * i] = v.x;
            f[2 * i + 1] = v.y;
        }
    }
};
template <> struct KvVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& c, float* f) {
        f[0] = __uint_as_float(c.x);
        f[1] = __uint_as_float(c.y);
        f[2] = __uint_as_float(c.z);
        f[3] = __uint_as_float(c.w);
    }
};

// One CTA per (query head, row).  Built for latency, not bandwidth (one head's K and V are at
// most a few hundred KB): every phase issues all of its global loads before using any of them.
//   scores : one thread per key; the key row is read with 16-byte loads, up to 16 in flight.
//   softmax: two block reductions.
//   values : D/VEC threads per key (16 bytes of the value row each), 256/(D/VEC) key groups,
//            8 loads in flight per thread; group partials are summed through shared memory.
template <typename KVT, int D>
__global__ void __launch_bounds__(kAttnThreads) attention_kernel(const AttnParams p) {
    constexpr int VEC = KvVec<KVT>::N;          // cache elements per 16-byte load
    constexpr int NCH = D / VEC;                // 16-byte chunks per cache row
    constexpr int TPK = NCH;                    // threads per key in the value phase
    constexpr int NG = kAttnThreads / TPK;      // key groups in the value phase
    constexpr int KB = NCH < 16 ? NCH : 16;     // chunks per batch in the score phase
    extern __shared__ __align__(16) float at_smem[];
    float* qs = at_smem;                  // [D] rotated query
    float* ks = qs + D;                   // [D] rotated current key (fused mode)
    float* vs = ks + D;                   // [D] current value (fused mode)
    float* raw = vs + D;                  // [2*D] raw q and k before rotation (fused mode)
    float* part = raw + 2 * D;            // [NG][D] value partial sums
    float* sc = part + NG * D;            // [n] scores / probabilities
    __shared__ float red[32];
    PhaseTrace tr;
    tr.begin(p.trace, p.trace_cap, 2);
    tr.mark();                                   // 0: entry

    grid_dependency_launch();
    grid_dependency_wait();
    tr.mark();                                   // 1: predecessor finished

    const int h = blockIdx.x, t = blockIdx.y;
    const int tid = threadIdx.x;
    const int G = p.Q / p.KV, kvh = h / G;
    const int pos = p.pos_per_row ? p.pos_ptr[t] : p.pos_ptr[0] + t;
    const int n = pos + 1;
    const int half = D / 2;
    const int kd = p.KV * D;
    KVT* ck = reinterpret_cast<KVT*>(p.cache_k) + (size_t)t * p.cache_seq_stride + (size_t)kvh * D;
    KVT* cv = reinterpret_cast<KVT*>(p.cache_v) + (size_t)t * p.cache_seq_stride + (size_t)kvh * D;
    const float* qrow = p.q + (size_t)t * p.Q * D + (size_t)h * D;

    // ---- request everything up front: the row's own q/k/v and rope factors, this thread's key
    //      row for the score phase and its first 16 value chunks for the value phase ----------------
    constexpr int VB0 = 16;                     // value chunks requested before the scores exist
    const int g = tid / TPK, c = tid % TPK;
    float q_raw = 0.0f, k_raw = 0.0f, vr = 0.0f, cr = 0.0f, sr = 0.0f;
    if (tid < D) {
        q_raw = qrow[tid];
        if (p.fused) {
            const int i = tid < half ? tid : tid - half;
            k_raw = p.k_cur[(size_t)t * kd + (size_t)kvh * D + tid];
            vr = p.v_cur[(size_t)t * kd + (size_t)kvh * D + tid];
            cr = p.rope_cos[(size_t)pos * half + i];
            sr = p.rope_sin[(size_t)pos * half + i];
        }
    }
    uint4 kbuf[KB];
    const bool k_from_cache = tid < n && !(p.fused && tid == pos);
    if (k_from_cache) {
        const uint4* kp = reinterpret_cast<const uint4*>(ck + (size_t)tid * kd);
#pragma unroll
        for (int b = 0; b < KB; ++b) kbuf[b] = kp[b];
    }
    uint4 vbuf[VB0];
#pragma unroll
    for (int b = 0; b < VB0; ++b) {
        const int i = g + b * NG;
        if (i < n && !(p.fused && i == pos)) vbuf[b] = *(reinterpret_cast<const uint4*>(cv + (size_t)i * kd) + c);
    }

    if (p.fused) {
        if (tid < D) {
            raw[tid] = q_raw;
            raw[D + tid] = k_raw;
        }
        __syncthreads();
        if (tid < D) {
            const int i = tid < half ? tid : tid - half;
            const float q1 = raw[i], q2 = raw[half + i], k1 = raw[D + i], k2 = raw[D + half + i];
            float qr, kr;
            if (tid < half) {
                qr = __fsub_rn(__fmul_rn(q1, cr), __fmul_rn(q2, sr));
                kr = __fsub_rn(__fmul_rn(k1, cr), __fmul_rn(k2, sr));
            } else {
                qr = __fadd_rn(__fmul_rn(q1, sr), __fmul_rn(q2, cr));
                kr = __fadd_rn(__fmul_rn(k1, sr), __fmul_rn(k2, cr));
            }
            qs[tid] = qr;
            ks[tid] = kv_round<KVT>(kr);
            vs[tid] = kv_round<KVT>(vr);
            if (h % G == 0) {
                ck[(size_t)pos * kd + tid] = kv_make<KVT>(kr);
                cv[(size_t)pos * kd + tid] = kv_make<KVT>(vr);
            }
        }
    } else {
        if (tid < D) qs[tid] = q_raw;
    }
    __syncthreads();
    tr.mark();                                   // 2: q/k rotated (own loads arrived)

    // ---- scores: thread per key ------------------------------------------------------------------
    const float inv_sqrt_d = 1.0f / sqrtf((float)D);
    for (int i = tid; i < n; i += kAttnThreads) {
        float dot = 0.0f;
        if (p.fused && i == pos) {
#pragma unroll 8
            for (int d = 0; d < D; ++d) dot = fmaf(qs[d], ks[d], dot);
        } else {
            const uint4* kp = reinterpret_cast<const uint4*>(ck + (size_t)i * kd);
#pragma unroll
            for (int b0 = 0; b0 < NCH; b0 += KB) {
                if (b0 > 0 || i != tid) {
#pragma unroll
                    for (int b = 0; b < KB; ++b) kbuf[b] = kp[b0 + b];
                }
#pragma unroll
                for (int b = 0; b < KB; ++b) {
                    float f[VEC];
                    KvVec<KVT>::unpack(kbuf[b], f);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) dot = fmaf(qs[(b0 + b) * VEC + e], f[e], dot);
                }
            }
        }
        sc[i] = __fmul_rn(dot, inv_sqrt_d);
    }
    tr.mark();                                   // 3: own score done (key row arrived)
    __syncthreads();
    tr.mark();                                   // 4: all scores visible

    // ---- softmax over sc[0..n) -----------------------------------------------------------------------
    float mx = -INFINITY;
    for (int i = tid; i < n; i += kAttnThreads) mx = fmaxf(mx, sc[i]);
    mx = block_max(mx, red);
    float sum = 0.0f;
    for (int i = tid; i < n; i += kAttnThreads) {
        const float e = expf(sc[i] - mx);
        sc[i] = e;
        sum += e;
    }
    sum = block_sum(sum, red);
    for (int i = tid; i < n; i += kAttnThreads) sc[i] = __fdiv_rn(sc[i], sum);
    __syncthreads();
    tr.mark();                                   // 5: softmax done

    // ---- weighted sum of values: TPK threads per key, NG key groups ---------------------------------
    float o[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) o[e] = 0.0f;
    auto accumulate = [&](int i, const uint4& chunk) {
        const float pi = sc[i];
        float f[VEC];
        if (p.fused && i == pos) {
#pragma unroll
            for (int e = 0; e < VEC; ++e) f[e] = vs[c * VEC + e];
        } else {
            KvVec<KVT>::unpack(chunk, f);
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = fmaf(pi, f[e], o[e]);
    };
#pragma unroll
    for (int b = 0; b < VB0; ++b) {
        const int i = g + b * NG;
        if (i < n) accumulate(i, vbuf[b]);
    }
    constexpr int VB = 8;                                   // loads in flight per thread afterwards
    for (int i0 = g + VB0 * NG; i0 < n; i0 += NG * VB) {
        uint4 buf[VB];
#pragma unroll
        for (int b = 0; b < VB; ++b) {
            const int i = i0 + b * NG;
            if (i < n && !(p.fused && i == pos))
                buf[b] = *(reinterpret_cast<const uint4*>(cv + (size_t)i * kd) + c);
        }
#pragma unroll
        for (int b = 0; b < VB; ++b) {
            const int i = i0 + b * NG;
            if (i < n) accumulate(i, buf[b]);
        }
    }
    tr.mark();                                   // 6: values accumulated
#pragma unroll
    for (int e = 0; e < VEC; ++e) part[g * D + c * VEC + e] = o[e];
    __syncthreads();
    if (tid < D) {
        float r = 0.0f;
#pragma unroll
        for (int w = 0; w < NG; ++w) r += part[w * D + tid];
        p.out[(size_t)t * p.Q * D + (size_t)h * D + tid] = r;
    }
    tr.mark();                                   // 7: output stored
    tr.end();
}

template <typename KVT>
static int attention_launch_t(const AttnParams& p) {
    const int D = p.D;
    constexpr int VEC = 16 / (int)sizeof(KVT);
    const size_t smem = (size_t)(5 * D + kAttnThreads * VEC + p.t_max) * sizeof(float);
    LSPK_REQUIRE(smem <= 200 * 1024, "attention: t_max=%d too large for the shared score buffer", p.t_max);
    static bool attr_set = false;
    if (!attr_set) {
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(rope_store_kernel<KVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set = true;
    }
    if (!p.fused) {
        const size_t rs = (size_t)(p.Q + p.KV) * D * sizeof(float);
        LSPK_CUDA(launch(rope_store_kernel<KVT>, dim3(p.T), dim3(kAttnThreads), rs, true, p));
    }
    const dim3 grid(p.Q, p.T);
    cudaError_t e;
    if (D == 64) e = launch(attention_kernel<KVT, 64>, grid, dim3(kAttnThreads), smem, true, p);
    else if (D == 128) e = launch(attention_kernel<KVT, 128>, grid, dim3(kAttnThreads), smem, true, p);
    else e = launch(attention_kernel<KVT, 256>, grid, dim3(kAttnThreads), smem, true, p);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
    return LSPK_OK;
}

int attention_launch(const AttnParams& p_in, int kv_is_fp16) {
    AttnParams p = p_in;
    p.trace = trace_buffer();
    p.trace_cap = trace_capacity();
    LSPK_REQUIRE(p.D == 64 || p.D == 128 || p.D == 256, "attention: head_dim must be 64, 128 or 256 (got %d)", p.D);
    LSPK_REQUIRE(p.Q % p.KV == 0, "attention: num_heads must be a multiple of num_kv_heads");
    LSPK_REQUIRE(!p.fused || p.T == 1 || p.pos_per_row, "attention: the fused form needs rows that do not attend to each other");
    return kv_is_fp16 ? attention_launch_t<__half>(p) : attention_launch_t<float>(p);
}

}  // namespace lspk
