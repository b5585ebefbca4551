// Device building blocks shared by the ternary kernels: activation byte transpose, the masked
// dp4a decode of one 64-weight chunk, and the int8 quantiser primitives.
#pragma once
#include "common.cuh"

namespace lspk {

__device__ __forceinline__ void transpose4x4_bytes(uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                   uint32_t& o0, uint32_t& o1, uint32_t& o2, uint32_t& o3) {
    const uint32_t t0 = __byte_perm(a0, a1, 0x5140), t1 = __byte_perm(a2, a3, 0x5140);
    const uint32_t t2 = __byte_perm(a0, a1, 0x7362), t3 = __byte_perm(a2, a3, 0x7362);
    o0 = __byte_perm(t0, t1, 0x5410);
    o1 = __byte_perm(t0, t1, 0x7632);
    o2 = __byte_perm(t2, t3, 0x5410);
    o3 = __byte_perm(t2, t3, 0x7632);
}

// Accumulate one 16-byte weight chunk (64 weights) against the matching 64 permuted activations.
__device__ __forceinline__ void chunk_dot(const uint4& wv, const int4* __restrict__ xp, int acc[4]) {
    const uint32_t w[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        const int4 xv = xp[m];
        acc[0] = dp4a_us(w[m] & 0x03030303u, xv.x, acc[0]);
        acc[1] = dp4a_us(w[m] & 0x0C0C0C0Cu, xv.y, acc[1]);
        acc[2] = dp4a_us(w[m] & 0x30303030u, xv.z, acc[2]);
        acc[3] = dp4a_us(w[m] & 0xC0C0C0C0u, xv.w, acc[3]);
    }
}

// Sum of squares of a row in the ONE summation order every kernel of the library uses, so that a row normalised
// by the fused prologue of the one-row GEMV, by the row kernel in front of the many-row products or by a prefill
// comes out bit-identical (a sum that rounds differently flips int8 activations, and a deep network amplifies
// that into different tokens).  The order: the row is cut into 16-element blocks; block b belongs to lane
// b % 256 of a 256-lane group; a lane walks its blocks in increasing order and, inside a block, adds element e
// into partial e % 4 with a fused multiply-add; the lane's value is (p0 + p1) + (p2 + p3); lanes combine through
// the xor-shuffle tree of warp_sum and the eight warps as ((w0 + w1) + (w2 + w3)) + ((w4 + w5) + (w6 + w7)).
// canonical_ssq_lane returns the value of lane `lane256` for a row of K floats readable at `row` (shared or
// global memory; elements at and beyond K count as zero).
__device__ __forceinline__ float canonical_ssq_lane(const float* __restrict__ row, int K, int lane256) {
    float ss[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = lane256 * 16; k0 < K; k0 += 256 * 16) {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const float v = (k0 + e < K) ? row[k0 + e] : 0.0f;
            ss[e & 3] = fmaf(v, v, ss[e & 3]);
        }
    }
    return (ss[0] + ss[1]) + (ss[2] + ss[3]);
}
// Combines the eight warp sums (warp w's value at slot[w]) in the canonical order.
__device__ __forceinline__ float canonical_ssq_combine(const float* slot) {
    return ((slot[0] + slot[1]) + (slot[2] + slot[3])) + ((slot[4] + slot[5]) + (slot[6] + slot[7]));
}

// fp32 -> int8 with round-half-even and saturation to [-128, 127] in one instruction: the pair
// _mm512_cvtps_epi32 + _mm512_cvtsepi32_epi8 of the reference quantiser.
__device__ __forceinline__ uint32_t quant_rne_sat(float v) {
    int r;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
    return (uint32_t)r;
}
__device__ __forceinline__ uint32_t pack4_bytes(uint32_t q0, uint32_t q1, uint32_t q2, uint32_t q3) {
    return __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
}


}  // namespace lspk
