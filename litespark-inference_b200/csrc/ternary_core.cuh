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
