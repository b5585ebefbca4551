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
#include <cooperative_groups.h>
#include <stdlib.h>

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
    extern __shared__ __align__(16) float rs_smem[];     // (Q + KV) * D raw q and k of this row, cos | sin, raw v
    const int t = blockIdx.x, tid = threadIdx.x;
    const int pos = p.pos_per_row ? p.pos_ptr[t] : p.pos_ptr[0] + t;
    const int D = p.D, half = D / 2;
    const int qd = p.Q * D, kd = p.KV * D;
    float* qrow = p.q + (size_t)t * qd;
    const float* krow = p.k_cur + (size_t)t * kd;
    const float* vrow = p.v_cur + (size_t)t * kd;
    // everything this row reads goes to shared memory first: the stores below may alias the inputs as far as
    // the compiler knows, and loads interleaved with them would each wait for the store before
    float* cr = rs_smem + qd + kd;
    float* sr = cr + half;
    float* vs = sr + half;
    for (int i = tid; i < qd; i += kAttnThreads) rs_smem[i] = qrow[i];
    for (int i = tid; i < kd; i += kAttnThreads) {
        rs_smem[qd + i] = krow[i];
        vs[i] = vrow[i];
    }
    for (int i = tid; i < half; i += kAttnThreads) {
        cr[i] = p.rope_cos[(size_t)pos * half + i];
        sr[i] = p.rope_sin[(size_t)pos * half + i];
    }
    __syncthreads();
    for (int i = tid; i < qd; i += kAttnThreads) {
        const int hd = i / D, d = i % D;
        qrow[i] = rope_elem(rs_smem + hd * D, d, half, cr, sr);
    }
    KVT* ck = reinterpret_cast<KVT*>(p.cache_k) + (size_t)t * p.cache_seq_stride + (size_t)pos * kd;
    KVT* cv = reinterpret_cast<KVT*>(p.cache_v) + (size_t)t * p.cache_seq_stride + (size_t)pos * kd;
    for (int i = tid; i < kd; i += kAttnThreads) {
        const int hd = i / D, d = i % D;
        ck[i] = kv_make<KVT>(rope_elem(rs_smem + qd + hd * D, d, half, cr, sr));
        cv[i] = kv_make<KVT>(vs[i]);
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

// Order-preserving map float -> uint32 (and back), so that a maximum over possibly negative floats
// can use the integer warp reduction.
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ordered_to_float(uint32_t u) {
    return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// One CTA per (query head, row).  Built for latency, not bandwidth (one head's K and V are at
// most a few hundred KB): every phase issues all of its global loads before using any of them,
// and every cache row is read by a group of adjacent lanes, 16 bytes each, so that a warp-wide
// load touches whole 128-byte lines (a thread-per-key layout costs one L1 wavefront per lane
// per load and was bound by exactly that).
//   scores : TPK lanes per key; each lane's partial dot products for SB keys are combined with a
//            halving exchange (SB + ... shuffles instead of SB * log2(TPK)), leaving lane c with
//            the finished score of key c.
//   softmax: two single-barrier block reductions.
//   values : TPK lanes per key, NG key groups, 16 loads requested before the scores exist and
//            8 in flight per thread afterwards; group partials are summed through shared memory.
// VB0: value chunks a thread requests before the scores exist (16 hides the latency when a launch has few
// CTAs; with many rows a small number keeps the registers low enough for two CTAs per SM).
template <typename KVT, int D, int VB0>
__global__ void __launch_bounds__(kAttnThreads) attention_kernel(const AttnParams p) {
    constexpr int VEC = KvVec<KVT>::N;          // cache elements per 16-byte load
    constexpr int NCH = D / VEC;                // 16-byte chunks per cache row
    constexpr int TPK = NCH > 32 ? 32 : NCH;    // lanes per key
    constexpr int CPT = NCH / TPK;              // chunks per lane (2 only for fp32 rows of 256)
    constexpr int NG = kAttnThreads / TPK;      // key groups
    constexpr int SBCAP = VB0 >= 16 ? 16 : 8;    // fewer key rows in flight in the many-CTA variant (registers)
    constexpr int SB = (TPK < SBCAP ? TPK : SBCAP) / CPT;   // keys per group whose rows are in flight together
    constexpr int KPB = NG * SB;                // keys per batch of the score phase
    static_assert(kAttnWarps == 8, "block reductions assume eight warps");
    extern __shared__ __align__(16) float at_smem[];
    float* qs = at_smem;                  // [D] rotated query
    float* ks = qs + D;                   // [D] rotated current key (fused mode)
    float* vs = ks + D;                   // [D] current value (fused mode)
    float* raw = vs + D;                  // [2*D] raw q and k before rotation (fused mode)
    float* part = raw + 2 * D;            // [NG][D] value partial sums
    float* sc = part + NG * D;            // [n] scores / probabilities
    __shared__ __align__(16) float red[16];
    PhaseTrace tr;
    tr.begin(p.trace, p.trace_cap, 2);
    tr.mark();                                   // 0: entry

    grid_dependency_launch();
    grid_dependency_wait();
    tr.mark();                                   // 1: predecessor finished

    const int h = blockIdx.x, t = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.Q / p.KV, kvh = h / G;
    const int pos = p.pos_per_row ? p.pos_ptr[t] : p.pos_ptr[0] + t;
    const int n = pos + 1;
    const int half = D / 2;
    const int kd = p.KV * D;
    KVT* ck = reinterpret_cast<KVT*>(p.cache_k) + (size_t)t * p.cache_seq_stride + (size_t)kvh * D;
    KVT* cv = reinterpret_cast<KVT*>(p.cache_v) + (size_t)t * p.cache_seq_stride + (size_t)kvh * D;
    const float* qrow = p.q + (size_t)t * p.Q * D + (size_t)h * D;

    // ---- request everything up front: the row's own q/k/v and rope factors, the key rows of the
    //      first score batch and the first 16 value chunks of this thread ---------------------------
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
    uint4 kbuf[SB][CPT];
    auto request_keys = [&](int base) {
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int i = base + g + j * NG;
            if (i < n && !(p.fused && i == pos)) {
                const uint4* kp = reinterpret_cast<const uint4*>(ck + (size_t)i * kd);
#pragma unroll
                for (int u = 0; u < CPT; ++u) kbuf[j][u] = kp[c + u * TPK];
            }
        }
    };
    request_keys(0);
    uint4 vbuf[VB0 / CPT][CPT];
#pragma unroll
    for (int b = 0; b < VB0 / CPT; ++b) {
        const int i = g + b * NG;
        if (i < n && !(p.fused && i == pos)) {
#pragma unroll
            for (int u = 0; u < CPT; ++u) vbuf[b][u] = *(reinterpret_cast<const uint4*>(cv + (size_t)i * kd) + c + u * TPK);
        }
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

    // ---- scores ------------------------------------------------------------------------------------
    const float inv_sqrt_d = 1.0f / sqrtf((float)D);
    float qreg[CPT][VEC];
#pragma unroll
    for (int u = 0; u < CPT; ++u)
#pragma unroll
        for (int e = 0; e < VEC; ++e) qreg[u][e] = qs[(c + u * TPK) * VEC + e];
    for (int base = 0; base < n; base += KPB) {
        if (base > 0) request_keys(base);
        float dotp[SB];
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int i = base + g + j * NG;
            float d = 0.0f;
            if (i < n) {
#pragma unroll
                for (int u = 0; u < CPT; ++u) {
                    float f[VEC];
                    if (p.fused && i == pos) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) f[e] = ks[(c + u * TPK) * VEC + e];
                    } else {
                        KvVec<KVT>::unpack(kbuf[j][u], f);
                    }
#pragma unroll
                    for (int e = 0; e < VEC; ++e) d = fmaf(qreg[u][e], f[e], d);
                }
            }
            dotp[j] = d;
        }
        // combine the TPK lanes of a key: plain exchange while more lanes than keys remain, then each
        // step halves the keys a lane still carries; lane c ends with the sum for key c % SB
#pragma unroll
        for (int o = TPK / 2; o >= 1; o >>= 1) {
            if (o >= SB) {
#pragma unroll
                for (int j = 0; j < SB; ++j) dotp[j] += __shfl_xor_sync(0xffffffffu, dotp[j], o);
            } else {
                const bool upper = (c & o) != 0;
#pragma unroll
                for (int k = 0; k < o; ++k) {
                    const float send = upper ? dotp[k] : dotp[k + o];
                    const float keep = upper ? dotp[k + o] : dotp[k];
                    dotp[k] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
        }
        if (c < SB) {
            const int i = base + g + c * NG;
            if (i < n) sc[i] = __fmul_rn(dotp[0], inv_sqrt_d);
        }
    }
    tr.mark();                                   // 3: own scores done (key rows arrived)
    __syncthreads();
    tr.mark();                                   // 4: all scores visible

    // ---- softmax over sc[0..n) -----------------------------------------------------------------------
    float mx = -INFINITY;
    for (int i = tid; i < n; i += kAttnThreads) mx = fmaxf(mx, sc[i]);
    {
        const uint32_t u = __reduce_max_sync(0xffffffffu, float_to_ordered(mx));
        if (lane == 0) red[warp] = ordered_to_float(u);
        __syncthreads();
        const float4 a = *reinterpret_cast<const float4*>(red), b = *reinterpret_cast<const float4*>(red + 4);
        mx = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
    }
    float sum = 0.0f;
    for (int i = tid; i < n; i += kAttnThreads) {
        const float e = expf(sc[i] - mx);
        sc[i] = e;
        sum += e;
    }
    {
        sum = warp_sum(sum);
        if (lane == 0) red[8 + warp] = sum;
        __syncthreads();
        const float4 a = *reinterpret_cast<const float4*>(red + 8), b = *reinterpret_cast<const float4*>(red + 12);
        sum = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
    }
    for (int i = tid; i < n; i += kAttnThreads) sc[i] = __fdiv_rn(sc[i], sum);
    __syncthreads();
    tr.mark();                                   // 5: softmax done

    // ---- weighted sum of values: TPK lanes per key, NG key groups -----------------------------------
    float o[CPT][VEC];
#pragma unroll
    for (int u = 0; u < CPT; ++u)
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[u][e] = 0.0f;
    auto accumulate = [&](int i, const uint4* chunk) {
        const float pi = sc[i];
#pragma unroll
        for (int u = 0; u < CPT; ++u) {
            float f[VEC];
            if (p.fused && i == pos) {
#pragma unroll
                for (int e = 0; e < VEC; ++e) f[e] = vs[(c + u * TPK) * VEC + e];
            } else {
                KvVec<KVT>::unpack(chunk[u], f);
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[u][e] = fmaf(pi, f[e], o[u][e]);
        }
    };
#pragma unroll
    for (int b = 0; b < VB0 / CPT; ++b) {
        const int i = g + b * NG;
        if (i < n) accumulate(i, vbuf[b]);
    }
    constexpr int VB = 8 / CPT;                             // keys in flight per thread afterwards
    for (int i0 = g + (VB0 / CPT) * NG; i0 < n; i0 += NG * VB) {
        uint4 buf[VB][CPT];
#pragma unroll
        for (int b = 0; b < VB; ++b) {
            const int i = i0 + b * NG;
            if (i < n && !(p.fused && i == pos)) {
#pragma unroll
                for (int u = 0; u < CPT; ++u) buf[b][u] = *(reinterpret_cast<const uint4*>(cv + (size_t)i * kd) + c + u * TPK);
            }
        }
#pragma unroll
        for (int b = 0; b < VB; ++b) {
            const int i = i0 + b * NG;
            if (i < n) accumulate(i, buf[b]);
        }
    }
    tr.mark();                                   // 6: values accumulated
#pragma unroll
    for (int u = 0; u < CPT; ++u)
#pragma unroll
        for (int e = 0; e < VEC; ++e) part[g * D + (c + u * TPK) * VEC + e] = o[u][e];
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

// Decode form: the keys of one (query head, row) are split over a thread-block cluster of kSplit
// CTAs, CTA r taking keys r, r + kSplit, ...  One head's K and V rows (100 KB at 200 positions) pulled
// through a single SM bound the one-CTA form; eight SMs share them here, and the three scalars/vectors
// the softmax needs from all keys (maximum, sum, output partials) cross the cluster through
// distributed shared memory in ONE exchange: every CTA forms a softmax over its own keys (own maximum,
// own sum, unnormalised output) and rank 0 merges the pieces with the weights exp(m_r - M) -- the same
// function as the one-CTA form, rounded in a different order (compared within tolerance).  Only for rows that do not attend to each
// other (a single row, or one sequence per row): the row's own key and value come from registers /
// shared memory, the cache rows are written by the CTA that owns position `pos` (head h % G == 0).
constexpr int kSplit = 8;

// The order of every floating-point sum is defined for kAttnThreads (256) threads: key groups of TPK lanes, one
// partial output per group, exponentials summed per thread, warp and eight-warp tree.  NT: threads the CTA really
// has.  Launches over several sequences have far more clusters than the machine holds at once; their instantiation
// runs 128 threads per CTA (twice the CTAs per SM), each thread group standing in for two of the defined groups
// with an accumulator apiece, each thread for two of the defined threads in the sum of exponentials: every result
// bit is the same, so a sequence's tokens do not depend on what it is batched with.  MINB: CTAs per SM the
// register budget is held to.
template <typename KVT, int D, int NT = kAttnThreads, int MINB = 1>
__global__ void __launch_bounds__(NT, MINB) attention_split_kernel(const AttnParams p) {
    namespace cg = cooperative_groups;
    constexpr int VEC = KvVec<KVT>::N;
    constexpr int NCH = D / VEC;
    constexpr int TPK = NCH > 32 ? 32 : NCH;    // lanes per key
    constexpr int CPT = NCH / TPK;              // chunks per lane
    constexpr int VG = kAttnThreads / TPK;      // key groups the sums are defined over
    constexpr int NG = NT / TPK;                // key groups this CTA has
    constexpr int ACC = VG / NG;                // defined groups per real group (1 or 2): slot j belongs to g + NG * (j % ACC)
    constexpr int SB = 4 / CPT;                 // keys per group in flight (requested before pos is known)
    constexpr int KPB = NG * SB;                // local keys per batch
    static_assert(NT == kAttnThreads || (NT * 2 == kAttnThreads && NT >= D && SB % 2 == 0), "half-size CTAs: D <= NT, even SB");
    extern __shared__ __align__(16) float at_smem[];
    float* qs = at_smem;                  // [D] rotated query
    float* ks = qs + D;                   // [D] rotated current key
    float* vs = ks + D;                   // [D] current value
    float* raw = vs + D;                  // [2*D] raw q and k before rotation
    float* part = raw + 2 * D;            // [VG][D] value partial sums of this CTA
    float* fin = part + VG * D;           // [kSplit][D] CTA partials, gathered in rank 0
    float* sc = fin + kSplit * D;         // [local keys] scores / probabilities
    __shared__ __align__(16) float cl_max[kSplit], cl_sum[kSplit];
    __shared__ __align__(16) float red[16];
    cg::cluster_group cluster = cg::this_cluster();
    const int r = (int)cluster.block_rank();
    PhaseTrace tr;
    tr.begin(p.trace, p.trace_cap, 2);
    tr.mark();                                   // 0: entry
    // Shared memory of another CTA of the cluster may only be touched once that CTA has started: every CTA
    // announces itself here and the matching wait sits just before the first remote store, off the critical path.
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    grid_dependency_launch();
    grid_dependency_wait();
    tr.mark();                                   // 1: predecessor finished

    const int h = blockIdx.x, t = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = p.Q / p.KV, kvh = h / G;
    const int half = D / 2;
    const int kd = p.KV * D;
    KVT* ck = reinterpret_cast<KVT*>(p.cache_k) + (size_t)t * p.cache_seq_stride + (size_t)kvh * D;
    KVT* cv = reinterpret_cast<KVT*>(p.cache_v) + (size_t)t * p.cache_seq_stride + (size_t)kvh * D;
    const float* qrow = p.q + (size_t)t * p.Q * D + (size_t)h * D;
    const int g = tid / TPK, c = tid % TPK;

    // ---- requests that do not need the position: q, the row's k and v, and the first batch of this
    //      CTA's key and value rows (any row below t_max is allocated; rows past the position are
    //      never used) ---------------------------------------------------------------------------------
    const int pos = p.pos_per_row ? p.pos_ptr[t] : p.pos_ptr[0] + t;
    float q_raw = 0.0f, k_raw = 0.0f, vr = 0.0f, cr = 0.0f, sr = 0.0f;
    if (tid < D) {
        q_raw = qrow[tid];
        k_raw = p.k_cur[(size_t)t * kd + (size_t)kvh * D + tid];
        vr = p.v_cur[(size_t)t * kd + (size_t)kvh * D + tid];
        if (p.rope_cur) {
            const int i = tid < half ? tid : tid - half;
            cr = p.rope_cur[(size_t)t * D + i];
            sr = p.rope_cur[(size_t)t * D + half + i];
        }
    }
    uint4 kbuf[SB][CPT], vbuf[SB][CPT];
#pragma unroll
    for (int j = 0; j < SB; ++j) {
        const int i = r + kSplit * (g + j * NG);
        if (i < p.t_max) {
#pragma unroll
            for (int u = 0; u < CPT; ++u) {
                kbuf[j][u] = *(reinterpret_cast<const uint4*>(ck + (size_t)i * kd) + c + u * TPK);
                vbuf[j][u] = *(reinterpret_cast<const uint4*>(cv + (size_t)i * kd) + c + u * TPK);
            }
        }
    }
    // ---- now the position: rope factors, rotation, cache write ----------------------------------------
    const int n = pos + 1;
    const int n_local = n > r ? (n - r + kSplit - 1) / kSplit : 0;     // keys r, r + kSplit, ... below n
    const bool owner = (pos % kSplit) == r;
    if (tid < D && !p.rope_cur) {
        const int i = tid < half ? tid : tid - half;
        cr = p.rope_cos[(size_t)pos * half + i];
        sr = p.rope_sin[(size_t)pos * half + i];
    }
    if (tid < D) {
        raw[tid] = q_raw;
        raw[D + tid] = k_raw;
    }
    __syncthreads();                             // the rotation pairs element i with i + half
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
        if (owner && h % G == 0) {
            ck[(size_t)pos * kd + tid] = kv_make<KVT>(kr);
            cv[(size_t)pos * kd + tid] = kv_make<KVT>(vr);
        }
    }
    __syncthreads();
    tr.mark();                                   // 2: q/k rotated

    // ---- scores of this CTA's keys -------------------------------------------------------------------------
    const float inv_sqrt_d = 1.0f / sqrtf((float)D);
    float qreg[CPT][VEC];
#pragma unroll
    for (int u = 0; u < CPT; ++u)
#pragma unroll
        for (int e = 0; e < VEC; ++e) qreg[u][e] = qs[(c + u * TPK) * VEC + e];
    float mx = -INFINITY;
    for (int base = 0; base < n_local; base += KPB) {
        if (base > 0) {
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                const int i = r + kSplit * (base + g + j * NG);
                if (i < n && i != pos) {
#pragma unroll
                    for (int u = 0; u < CPT; ++u)
                        kbuf[j][u] = *(reinterpret_cast<const uint4*>(ck + (size_t)i * kd) + c + u * TPK);
                }
            }
        }
        float dotp[SB];
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int i = r + kSplit * (base + g + j * NG);
            float d = 0.0f;
            if (i < n) {
#pragma unroll
                for (int u = 0; u < CPT; ++u) {
                    float f[VEC];
                    if (i == pos) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) f[e] = ks[(c + u * TPK) * VEC + e];
                    } else {
                        KvVec<KVT>::unpack(kbuf[j][u], f);
                    }
#pragma unroll
                    for (int e = 0; e < VEC; ++e) d = fmaf(qreg[u][e], f[e], d);
                }
            }
            dotp[j] = d;
        }
#pragma unroll
        for (int o = TPK / 2; o >= 1; o >>= 1) {
            if (o >= SB) {
#pragma unroll
                for (int j = 0; j < SB; ++j) dotp[j] += __shfl_xor_sync(0xffffffffu, dotp[j], o);
            } else {
                const bool upper = (c & o) != 0;
#pragma unroll
                for (int k = 0; k < o; ++k) {
                    const float send = upper ? dotp[k] : dotp[k + o];
                    const float keep = upper ? dotp[k + o] : dotp[k];
                    dotp[k] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                }
            }
        }
        if (c < SB) {
            const int jl = base + g + c * NG;                    // local key index
            if (r + kSplit * jl < n) {
                const float s = __fmul_rn(dotp[0], inv_sqrt_d);
                sc[jl] = s;
                mx = fmaxf(mx, s);
            }
        }
    }
    tr.mark();                                   // 3: own scores done

    // ---- this CTA's maximum, exponentials relative to it, and their sum ------------------------------------
    {
        const uint32_t u = __reduce_max_sync(0xffffffffu, float_to_ordered(mx));
        if (lane == 0) red[warp] = ordered_to_float(u);
        if (NT < kAttnThreads && tid < 8 - NT / 32) red[NT / 32 + tid] = -INFINITY;      // the warps this CTA does not have
        __syncthreads();
        const float4 a = *reinterpret_cast<const float4*>(red), b = *reinterpret_cast<const float4*>(red + 4);
        mx = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
    }
    float sum = 0.0f, sum_hi = 0.0f;              // defined thread tid, and (half-size CTAs) defined thread tid + NT
    for (int j = tid; j < n_local; j += kAttnThreads) {
        const float e = expf(sc[j] - mx);
        sc[j] = e;
        sum += e;
    }
    if (NT < kAttnThreads) {
        for (int j = tid + NT; j < n_local; j += kAttnThreads) {
            const float e = expf(sc[j] - mx);
            sc[j] = e;
            sum_hi += e;
        }
    }
    {
        sum = warp_sum(sum);
        if (lane == 0) red[8 + warp] = sum;
        if (NT < kAttnThreads) {
            sum_hi = warp_sum(sum_hi);
            if (lane == 0) red[8 + NT / 32 + warp] = sum_hi;
        }
        __syncthreads();                          // also publishes sc[] to the value phase
        const float4 a = *reinterpret_cast<const float4*>(red + 8), b = *reinterpret_cast<const float4*>(red + 12);
        sum = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
    }
    tr.mark();                                   // 4: local softmax terms done

    // ---- unnormalised weighted sum of this CTA's values ------------------------------------------------------
    float o[ACC][CPT][VEC];
#pragma unroll
    for (int a = 0; a < ACC; ++a)
#pragma unroll
        for (int u = 0; u < CPT; ++u)
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[a][u][e] = 0.0f;
    for (int base = 0; base < n_local; base += KPB) {
        if (base > 0) {
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                const int i = r + kSplit * (base + g + j * NG);
                if (i < n && i != pos) {
#pragma unroll
                    for (int u = 0; u < CPT; ++u)
                        vbuf[j][u] = *(reinterpret_cast<const uint4*>(cv + (size_t)i * kd) + c + u * TPK);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int jl = base + g + j * NG;
            const int i = r + kSplit * jl;
            if (i < n) {
                const float pi = sc[jl];
#pragma unroll
                for (int u = 0; u < CPT; ++u) {
                    float f[VEC];
                    if (i == pos) {
#pragma unroll
                        for (int e = 0; e < VEC; ++e) f[e] = vs[(c + u * TPK) * VEC + e];
                    } else {
                        KvVec<KVT>::unpack(vbuf[j][u], f);
                    }
#pragma unroll
                    for (int e = 0; e < VEC; ++e) o[j % ACC][u][e] = fmaf(pi, f[e], o[j % ACC][u][e]);
                }
            }
        }
    }
    tr.mark();                                   // 5: values accumulated
#pragma unroll
    for (int a = 0; a < ACC; ++a)
#pragma unroll
        for (int u = 0; u < CPT; ++u)
#pragma unroll
            for (int e = 0; e < VEC; ++e) part[(g + a * NG) * D + (c + u * TPK) * VEC + e] = o[a][u][e];
    __syncthreads();
    // ---- hand (maximum, sum, partial output) to rank 0, which merges the kSplit softmax pieces --------------
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");      // every CTA of the cluster is running
    if (tid < D) {
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < VG; ++w) acc += part[w * D + tid];
        cluster.map_shared_rank(fin, 0)[r * D + tid] = acc;
    }
    if (tid == 0) {
        cluster.map_shared_rank(cl_max, 0)[r] = mx;
        cluster.map_shared_rank(cl_sum, 0)[r] = sum;
    }
    cluster.sync();
    tr.mark();                                   // 6: cluster exchange done
    if (r == 0 && tid < D) {
        // softmax over all keys from the pieces: weights exp(m_r - M), denominators and outputs rescaled
        float M = cl_max[0];
#pragma unroll
        for (int w = 1; w < kSplit; ++w) M = fmaxf(M, cl_max[w]);
        float L = 0.0f, acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kSplit; ++w) {
            const float wgt = expf(cl_max[w] - M);               // 0 for a piece without keys (maximum -inf)
            L = fmaf(cl_sum[w], wgt, L);
            acc = fmaf(fin[w * D + tid], wgt, acc);
        }
        p.out[(size_t)t * p.Q * D + (size_t)h * D + tid] = __fdiv_rn(acc, L);
    }
    tr.mark();                                   // 7: output stored
    tr.end();
}

// Prefill form: kRows consecutive query rows of one head per CTA (rows of one sequence, already rotated,
// keys and values already in the cache).  Every key / value row is fetched once for the kRows queries
// instead of once per query; row r attends keys 0 .. pos0 + t0 + r.  Same lane layout as the one-row
// kernel (TPK lanes per cache row, halving exchange for the dot products).
constexpr int kRows = 4;

template <typename KVT, int D>
__global__ void __launch_bounds__(kAttnThreads) attention_rows_kernel(const AttnParams p) {
    constexpr int VEC = KvVec<KVT>::N;
    constexpr int NCH = D / VEC;
    constexpr int TPK = NCH > 32 ? 32 : NCH;
    constexpr int CPT = NCH / TPK;
    constexpr int NG = kAttnThreads / TPK;
    constexpr int SB = (TPK < 8 ? TPK : 8) / CPT;      // keys per group in flight
    constexpr int KPB = NG * SB;
    extern __shared__ __align__(16) float at_smem[];
    float* qs = at_smem;                           // [kRows][D]
    float* part = qs + kRows * D;                  // [NG][kRows][D] value partial sums
    float* sc = part + NG * kRows * D;             // [kRows][n_stride] scores / probabilities
    __shared__ __align__(16) float red[2][kRows][8];
    grid_dependency_launch();
    grid_dependency_wait();

    const int h = blockIdx.x, t0 = blockIdx.y * kRows;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nrows = min(kRows, p.T - t0);
    const int G = p.Q / p.KV, kvh = h / G;
    const int pos0 = p.pos_ptr[0] + t0;            // position of this CTA's first row
    const int n_max = pos0 + nrows;                // keys 0 .. n_max - 1 are needed by some row
    const int n_stride = (p.t_max + 3) & ~3;
    const int kd = p.KV * D;
    const KVT* ck = reinterpret_cast<const KVT*>(p.cache_k) + (size_t)kvh * D;
    const KVT* cv = reinterpret_cast<const KVT*>(p.cache_v) + (size_t)kvh * D;
    const int g = tid / TPK, c = tid % TPK;

    for (int i = tid; i < kRows * D; i += kAttnThreads) {
        const int r = i / D, d = i % D;
        qs[i] = r < nrows ? p.q[(size_t)(t0 + r) * p.Q * D + (size_t)h * D + d] : 0.0f;
    }
    __syncthreads();

    // ---- scores -----------------------------------------------------------------------------------------
    const float inv_sqrt_d = 1.0f / sqrtf((float)D);
    float mx[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) mx[r] = -INFINITY;
    for (int base = 0; base < n_max; base += KPB) {
        uint4 kbuf[SB][CPT];
#pragma unroll
        for (int j = 0; j < SB; ++j) {
            const int i = base + g + j * NG;
            if (i < n_max) {
                const uint4* kp = reinterpret_cast<const uint4*>(ck + (size_t)i * kd);
#pragma unroll
                for (int u = 0; u < CPT; ++u) kbuf[j][u] = kp[c + u * TPK];
            }
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float qreg[CPT][VEC];
#pragma unroll
            for (int u = 0; u < CPT; ++u)
#pragma unroll
                for (int e = 0; e < VEC; ++e) qreg[u][e] = qs[r * D + (c + u * TPK) * VEC + e];
            float dotp[SB];
#pragma unroll
            for (int j = 0; j < SB; ++j) {
                const int i = base + g + j * NG;
                float d = 0.0f;
                if (i < n_max) {
#pragma unroll
                    for (int u = 0; u < CPT; ++u) {
                        float f[VEC];
                        KvVec<KVT>::unpack(kbuf[j][u], f);
#pragma unroll
                        for (int e = 0; e < VEC; ++e) d = fmaf(qreg[u][e], f[e], d);
                    }
                }
                dotp[j] = d;
            }
#pragma unroll
            for (int o = TPK / 2; o >= 1; o >>= 1) {
                if (o >= SB) {
#pragma unroll
                    for (int j = 0; j < SB; ++j) dotp[j] += __shfl_xor_sync(0xffffffffu, dotp[j], o);
                } else {
                    const bool upper = (c & o) != 0;
#pragma unroll
                    for (int k = 0; k < o; ++k) {
                        const float send = upper ? dotp[k] : dotp[k + o];
                        const float keep = upper ? dotp[k + o] : dotp[k];
                        dotp[k] = keep + __shfl_xor_sync(0xffffffffu, send, o);
                    }
                }
            }
            if (c < SB) {
                const int i = base + g + c * NG;
                if (i <= pos0 + r && r < nrows) {            // causal: row r sees keys up to its own position
                    const float sv = __fmul_rn(dotp[0], inv_sqrt_d);
                    sc[r * n_stride + i] = sv;
                    mx[r] = fmaxf(mx[r], sv);
                }
            }
        }
    }
    // ---- softmax of every row: one barrier for the kRows maxima, one for the sums ----------------------------
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const uint32_t u = __reduce_max_sync(0xffffffffu, float_to_ordered(mx[r]));
        if (lane == 0) red[0][r][warp] = ordered_to_float(u);
    }
    __syncthreads();
    float sum[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const float4 a = *reinterpret_cast<const float4*>(red[0][r]), b = *reinterpret_cast<const float4*>(red[0][r] + 4);
        mx[r] = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(a.z, a.w)), fmaxf(fmaxf(b.x, b.y), fmaxf(b.z, b.w)));
        sum[r] = 0.0f;
        if (r < nrows) {
            for (int i = tid; i <= pos0 + r; i += kAttnThreads) {
                const float e = expf(sc[r * n_stride + i] - mx[r]);
                sc[r * n_stride + i] = e;
                sum[r] += e;
            }
        }
        const float ws = warp_sum(sum[r]);
        if (lane == 0) red[1][r][warp] = ws;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        const float4 a = *reinterpret_cast<const float4*>(red[1][r]), b = *reinterpret_cast<const float4*>(red[1][r] + 4);
        const float total = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
        if (r < nrows)
            for (int i = tid; i <= pos0 + r; i += kAttnThreads) sc[r * n_stride + i] = __fdiv_rn(sc[r * n_stride + i], total);
    }
    __syncthreads();

    // ---- weighted sums of values -----------------------------------------------------------------------------
    float o[kRows][CPT][VEC];
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
        for (int u = 0; u < CPT; ++u)
#pragma unroll
            for (int e = 0; e < VEC; ++e) o[r][u][e] = 0.0f;
    constexpr int VB = 8 / CPT;
    for (int i0 = g; i0 < n_max; i0 += NG * VB) {
        uint4 buf[VB][CPT];
#pragma unroll
        for (int b = 0; b < VB; ++b) {
            const int i = i0 + b * NG;
            if (i < n_max) {
#pragma unroll
                for (int u = 0; u < CPT; ++u) buf[b][u] = *(reinterpret_cast<const uint4*>(cv + (size_t)i * kd) + c + u * TPK);
            }
        }
#pragma unroll
        for (int b = 0; b < VB; ++b) {
            const int i = i0 + b * NG;
            if (i < n_max) {
#pragma unroll
                for (int u = 0; u < CPT; ++u) {
                    float f[VEC];
                    KvVec<KVT>::unpack(buf[b][u], f);
#pragma unroll
                    for (int r = 0; r < kRows; ++r) {
                        if (i <= pos0 + r) {
                            const float pi = sc[r * n_stride + i];
#pragma unroll
                            for (int e = 0; e < VEC; ++e) o[r][u][e] = fmaf(pi, f[e], o[r][u][e]);
                        }
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
        for (int u = 0; u < CPT; ++u)
#pragma unroll
            for (int e = 0; e < VEC; ++e) part[(g * kRows + r) * D + (c + u * TPK) * VEC + e] = o[r][u][e];
    __syncthreads();
    for (int i = tid; i < nrows * D; i += kAttnThreads) {
        const int r = i / D, d = i % D;
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < NG; ++w) acc += part[(w * kRows + r) * D + d];
        p.out[(size_t)(t0 + r) * p.Q * D + (size_t)h * D + d] = acc;
    }
}

template <typename KVT>
static int attention_launch_t(const AttnParams& p) {
    const int D = p.D;
    constexpr int VEC = 16 / (int)sizeof(KVT);
    const int nch = D / VEC, tpk = nch > 32 ? 32 : nch;
    const size_t smem = (size_t)(5 * D + (kAttnThreads / tpk) * D + p.t_max) * sizeof(float);
    LSPK_REQUIRE(smem <= 200 * 1024, "attention: t_max=%d too large for the shared score buffer", p.t_max);
    static bool attr_set = false;
    if (!attr_set) {
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 64, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 128, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 256, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 64, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 128, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(attention_kernel<KVT, 256, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        LSPK_CUDA(cudaFuncSetAttribute(rope_store_kernel<KVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set = true;
    }
    if (!p.fused) {
        const size_t rs = (size_t)((p.Q + 2 * p.KV) * D + D) * sizeof(float);
        LSPK_CUDA(launch(rope_store_kernel<KVT>, dim3(p.T), dim3(kAttnThreads), rs, true, p));
    }
    if (!p.fused && !p.pos_per_row && p.T >= 2 * kRows) {
        // many consecutive rows of one sequence: kRows query rows per CTA share every key / value row they fetch
        const int nch2 = D / VEC, tpk2 = nch2 > 32 ? 32 : nch2;
        const size_t sm = (size_t)(kRows * D + (kAttnThreads / tpk2) * kRows * D + kRows * ((p.t_max + 3) & ~3)) * sizeof(float);
        if (sm <= 200 * 1024) {
            static bool rows_attr_set = false;
            if (!rows_attr_set) {
                LSPK_CUDA(cudaFuncSetAttribute(attention_rows_kernel<KVT, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                LSPK_CUDA(cudaFuncSetAttribute(attention_rows_kernel<KVT, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                LSPK_CUDA(cudaFuncSetAttribute(attention_rows_kernel<KVT, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
                rows_attr_set = true;
            }
            const dim3 rgrid(p.Q, (p.T + kRows - 1) / kRows);
            cudaError_t re;
            if (D == 64) re = launch(attention_rows_kernel<KVT, 64>, rgrid, dim3(kAttnThreads), sm, true, p);
            else if (D == 128) re = launch(attention_rows_kernel<KVT, 128>, rgrid, dim3(kAttnThreads), sm, true, p);
            else re = launch(attention_rows_kernel<KVT, 256>, rgrid, dim3(kAttnThreads), sm, true, p);
            if (re != cudaSuccess) return fail(LSPK_ERR_CUDA, "attention (rows) launch failed: %s", cudaGetErrorString(re));
            return LSPK_OK;
        }
    }
    if (p.fused) {
        // decode rows: keys split over a cluster of kSplit CTAs.  Every decode launch takes this kernel, whatever
        // the number of sequences, so that a sequence's attention sums are formed in the same order alone and in a
        // batch (its tokens do not depend on what it is batched with).
        const int nch = D / VEC, tpk = nch > 32 ? 32 : nch;
        const int local_keys = (p.t_max + kSplit - 1) / kSplit + 1;
        const size_t sm = (size_t)(5 * D + (kAttnThreads / tpk) * D + kSplit * D + local_keys) * sizeof(float);
        static bool split_attr_set = false;
        if (!split_attr_set) {
            LSPK_CUDA(cudaFuncSetAttribute(attention_split_kernel<KVT, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            LSPK_CUDA(cudaFuncSetAttribute(attention_split_kernel<KVT, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            LSPK_CUDA(cudaFuncSetAttribute(attention_split_kernel<KVT, 128, kAttnThreads / 2, 6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            LSPK_CUDA(cudaFuncSetAttribute(attention_split_kernel<KVT, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            split_attr_set = true;
        }
        LSPK_REQUIRE(sm <= 200 * 1024, "attention: t_max=%d too large for the shared score buffer", p.t_max);
        const dim3 sgrid(p.Q, p.T, kSplit), cl(1, 1, kSplit);
        cudaError_t se;
        if (D == 64) se = launch_cluster(attention_split_kernel<KVT, 64>, sgrid, dim3(kAttnThreads), sm, true, cl, p);
        else if (D == 128 && p.T >= 4) se = launch_cluster(attention_split_kernel<KVT, 128, kAttnThreads / 2, 6>, sgrid, dim3(kAttnThreads / 2), sm, true, cl, p);
        else if (D == 128) se = launch_cluster(attention_split_kernel<KVT, 128>, sgrid, dim3(kAttnThreads), sm, true, cl, p);
        else se = launch_cluster(attention_split_kernel<KVT, 256>, sgrid, dim3(kAttnThreads), sm, true, cl, p);
        if (se != cudaSuccess) return fail(LSPK_ERR_CUDA, "attention (split) launch failed: %s", cudaGetErrorString(se));
        return LSPK_OK;
    }
    const dim3 grid(p.Q, p.T);
    cudaError_t e;
    const bool many = p.Q * p.T > 2 * sm_count();      // enough CTAs to hide latency by themselves
    if (D == 64) e = many ? launch(attention_kernel<KVT, 64, 2>, grid, dim3(kAttnThreads), smem, true, p)
                          : launch(attention_kernel<KVT, 64, 16>, grid, dim3(kAttnThreads), smem, true, p);
    else if (D == 128) e = many ? launch(attention_kernel<KVT, 128, 2>, grid, dim3(kAttnThreads), smem, true, p)
                                : launch(attention_kernel<KVT, 128, 16>, grid, dim3(kAttnThreads), smem, true, p);
    else e = many ? launch(attention_kernel<KVT, 256, 2>, grid, dim3(kAttnThreads), smem, true, p)
                  : launch(attention_kernel<KVT, 256, 16>, grid, dim3(kAttnThreads), smem, true, p);
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
