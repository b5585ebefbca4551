/*
 * CPU oracle for the ternary-matmul hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic of the reference's torchless kernel
 * (litespark_inference/kernels/x86_64/matmul_lut_avx512_extern_c.cpp).  It is
 * written so that, for the shapes the tests use, every result is bit-identical
 * to the reference's AVX-512 build: integer paths are exact by construction,
 * and the fp32 reductions follow the reference's 16-lane accumulate-then-tree
 * order (lane t owns elements t, t+16, t+32, ... combined with a fused
 * multiply-add; lanes are then folded 16 -> 8 -> 4 -> 2 -> 1).
 *
 * Nothing in the shipped library links or calls this file.  It is used by the
 * tests, by the smoke check and by the benchmark's CPU-baseline leg.
 *
 * Build: see oracle/Makefile (gcc -O2 -ffp-contract=off -fopenmp).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#if defined(_OPENMP)
#include <omp.h>
#endif

/* ---- helpers ----------------------------------------------------------- */

/* Fold 16 fp32 lanes the way GCC's _mm512_reduce_add_ps does:
 * (i, i+8) -> 8 lanes, (i, i+4) -> 4 lanes, (i, i+2) -> 2 lanes, then [0]+[1].
 * Used by every fp32 reduction of the reference
 * (matmul_lut_avx512_extern_c.cpp:51-53, hsum_f32_x16). */
static float fold16_add(const float a[16]) {
    float t8[8], t4[4], t2[2];
    for (int i = 0; i < 8; ++i) t8[i] = a[i + 8] + a[i];
    for (int i = 0; i < 4; ++i) t4[i] = t8[i + 4] + t8[i];
    t2[0] = t4[0] + t4[2];
    t2[1] = t4[1] + t4[3];
    return t2[0] + t2[1];
}

static inline float bf16_bits_to_f32(uint16_t b) {
    uint32_t u = ((uint32_t)b) << 16;
    float f;
    memcpy(&f, &u, sizeof f);
    return f;
}

static inline int32_t sat_i8_from_rne(float v) {
    /* _mm512_cvtps_epi32 (round-half-even under the default MXCSR) followed by
     * _mm512_cvtsepi32_epi8 (signed saturation to [-128, 127]);
     * matmul_lut_avx512_extern_c.cpp:451-456. */
    float r = nearbyintf(v);
    if (r > 127.0f) return 127;
    if (r < -128.0f) return -128;
    return (int32_t)r;
}

static inline int32_t tail_i8_from_round(float v) {
    /* Scalar tail of the reference quantiser (K % 16 leftovers): std::round
     * (half away from zero) and clamp to [-127, 127];
     * matmul_lut_avx512_extern_c.cpp:458-464. */
    int32_t iv = (int32_t)roundf(v);
    if (iv > 127) iv = 127;
    if (iv < -127) iv = -127;
    return iv;
}

/* ---- ternary matmul ---------------------------------------------------- */

/* Exact int32 accumulator of one packed row against one int8 activation row:
 * sum_k code(n,k) * x[k], code in {0,1,2} = weight + 1.
 * Packing: byte kb of a row holds weights 4kb..4kb+3 at bit offsets 0,2,4,6
 * (litespark_inference/torchless/pack.py:4-6). */
static inline int32_t row_code_dot(const uint8_t* row, const int8_t* x, int Kb) {
    int32_t s = 0;
    for (int kb = 0; kb < Kb; ++kb) {
        const uint8_t b = row[kb];
        const int8_t* xx = x + 4 * kb;
        s += (int32_t)((b >> 0) & 3) * xx[0];
        s += (int32_t)((b >> 2) & 3) * xx[1];
        s += (int32_t)((b >> 4) & 3) * xx[2];
        s += (int32_t)((b >> 6) & 3) * xx[3];
    }
    return s;
}

static inline int32_t sum_i8(const int8_t* x, int K) {
    int32_t s = 0;
    for (int k = 0; k < K; ++k) s += x[k];
    return s;
}

/* acc[t, n] = sum_k w[n,k] * x[t,k] with w = code - 1 (the value the
 * reference forms as `sum - sum_x`, matmul_lut_avx512_extern_c.cpp:234,336).
 * Any T (the reference's x86 batched kernel refuses T > 64, :266; callers of
 * the real reference must chunk, this restatement does not need to). */
void oracle_ternary_acc_i32(const int8_t* x, const uint8_t* packed_w,
                            int32_t* acc, int T, int N, int K) {
    const int Kb = K >> 2;
    #pragma omp parallel for schedule(static) if (N >= 64)
    for (int n = 0; n < N; ++n) {
        const uint8_t* row = packed_w + (ptrdiff_t)n * Kb;
        for (int t = 0; t < T; ++t) {
            const int8_t* xt = x + (ptrdiff_t)t * K;
            acc[(ptrdiff_t)t * N + n] = row_code_dot(row, xt, Kb) - sum_i8(xt, K);
        }
    }
}

/* matmul_lut_avx512_m1 (matmul_lut_avx512_extern_c.cpp:150-236):
 * y[n] = float(acc[n]) * (x_scale * w_scale), the two scales multiplied first. */
void oracle_matmul_lut_m1(const int8_t* x, const uint8_t* packed_w,
                          float w_scale, float x_scale, float* y, int N, int K) {
    const int Kb = K >> 2;
    const float out_scale = x_scale * w_scale;
    const int32_t sx = sum_i8(x, K);
    #pragma omp parallel for schedule(static) if (N >= 64)
    for (int n = 0; n < N; ++n) {
        const int32_t s = row_code_dot(packed_w + (ptrdiff_t)n * Kb, x, Kb);
        y[n] = (float)(s - sx) * out_scale;
    }
}

/* matmul_lut_avx512_mT (matmul_lut_avx512_extern_c.cpp:258-339), any T. */
void oracle_matmul_lut_mT(const int8_t* x, const float* x_scales,
                          const uint8_t* packed_w, float w_scale, float* y,
                          int T, int N, int K) {
    const int Kb = K >> 2;
    #pragma omp parallel for schedule(static) if (N >= 64)
    for (int n = 0; n < N; ++n) {
        const uint8_t* row = packed_w + (ptrdiff_t)n * Kb;
        for (int t = 0; t < T; ++t) {
            const int8_t* xt = x + (ptrdiff_t)t * K;
            const int32_t s = row_code_dot(row, xt, Kb) - sum_i8(xt, K);
            const float scale_t = x_scales[t] * w_scale;
            y[(ptrdiff_t)t * N + n] = (float)s * scale_t;
        }
    }
}

/* ---- activation quantiser ---------------------------------------------- */

/* quantize_activation_avx512 (matmul_lut_avx512_extern_c.cpp:425-466). */
float oracle_quantize_activation(const float* x, int8_t* out, int K) {
    float absmax = 0.0f;
    for (int k = 0; k < K; ++k) {
        const float a = fabsf(x[k]);
        if (a > absmax) absmax = a;
    }
    if (absmax < 1e-5f) absmax = 1e-5f;
    const float scale = absmax / 127.0f;
    const float inv_scale = 1.0f / scale;
    const int K16 = K & ~15;
    for (int k = 0; k < K16; ++k) out[k] = (int8_t)sat_i8_from_rne(x[k] * inv_scale);
    for (int k = K16; k < K; ++k) out[k] = (int8_t)tail_i8_from_round(x[k] * inv_scale);
    return scale;
}

void oracle_quantize_activation_batched(const float* x, int8_t* out,
                                        float* scales, int T, int K) {
    for (int t = 0; t < T; ++t)
        scales[t] = oracle_quantize_activation(x + (ptrdiff_t)t * K,
                                               out + (ptrdiff_t)t * K, K);
}

/* ---- RMSNorm ------------------------------------------------------------ */

/* Sum of squares in the reference's order
 * (matmul_lut_avx512_extern_c.cpp:597-604): 16 lanes of fused multiply-adds,
 * folded, then the scalar tail added one element at a time. */
static float ssq_ref_order(const float* x, int K) {
    float lane[16];
    for (int i = 0; i < 16; ++i) lane[i] = 0.0f;
    const int K16 = K & ~15;
    for (int k = 0; k < K16; k += 16)
        for (int i = 0; i < 16; ++i) lane[i] = fmaf(x[k + i], x[k + i], lane[i]);
    float s = fold16_add(lane);
    for (int k = K16; k < K; ++k) s += x[k] * x[k];
    return s;
}

static inline float rrms_of(const float* x, int K, float eps) {
    return 1.0f / sqrtf(ssq_ref_order(x, K) / (float)K + eps);
}

/* rmsnorm_bf16gamma_fp32_avx512 (:590-622): out = (x * rrms) * gamma. */
void oracle_rmsnorm_bf16gamma(const float* x, const uint16_t* gamma, float* out,
                              int K, float eps) {
    const float rrms = rrms_of(x, K, eps);
    for (int k = 0; k < K; ++k) out[k] = (x[k] * rrms) * bf16_bits_to_f32(gamma[k]);
}

/* rmsnorm_fp32gamma_fp32_avx512 (:625-650). */
void oracle_rmsnorm_fp32gamma(const float* x, const float* gamma, float* out,
                              int K, float eps) {
    const float rrms = rrms_of(x, K, eps);
    for (int k = 0; k < K; ++k) out[k] = (x[k] * rrms) * gamma[k];
}

void oracle_rmsnorm_bf16gamma_batched(const float* x, const uint16_t* gamma,
                                      float* out, int T, int K, float eps) {
    for (int t = 0; t < T; ++t)
        oracle_rmsnorm_bf16gamma(x + (ptrdiff_t)t * K, gamma, out + (ptrdiff_t)t * K, K, eps);
}

void oracle_rmsnorm_fp32gamma_batched(const float* x, const float* gamma,
                                      float* out, int T, int K, float eps) {
    for (int t = 0; t < T; ++t)
        oracle_rmsnorm_fp32gamma(x + (ptrdiff_t)t * K, gamma, out + (ptrdiff_t)t * K, K, eps);
}

/* rmsnorm_quantize_bf16gamma_avx512 (:975-1048): RMSNorm into tmp, then the
 * quantiser of :425-466 applied to tmp. */
float oracle_rmsnorm_quantize_bf16gamma(const float* x, const uint16_t* gamma,
                                        int8_t* out_i8, float* tmp, int K, float eps) {
    oracle_rmsnorm_bf16gamma(x, gamma, tmp, K, eps);
    return oracle_quantize_activation(tmp, out_i8, K);
}

void oracle_rmsnorm_quantize_bf16gamma_batched(const float* x, const uint16_t* gamma,
                                               int8_t* out_i8, float* scales, float* tmp,
                                               int T, int K, float eps) {
    for (int t = 0; t < T; ++t)
        scales[t] = oracle_rmsnorm_quantize_bf16gamma(
            x + (ptrdiff_t)t * K, gamma, out_i8 + (ptrdiff_t)t * K,
            tmp + (ptrdiff_t)t * K, K, eps);
}

/* ---- element-wise ------------------------------------------------------- */

/* relu2_mul_fp32_avx512 (:653-670): (max(g,0) * max(g,0)) * u. */
void oracle_relu2_mul(const float* gate, const float* up, float* out, int K) {
    for (int k = 0; k < K; ++k) {
        float g = gate[k];
        if (!(g > 0.0f)) g = 0.0f;
        out[k] = (g * g) * up[k];
    }
}

void oracle_relu2_mul_batched(const float* gate, const float* up, float* out, int T, int K) {
    oracle_relu2_mul(gate, up, out, T * K);
}

/* add_inplace_fp32_avx512 (:1127-1137). */
void oracle_add_inplace(float* a, const float* b, int K) {
    for (int k = 0; k < K; ++k) a[k] = a[k] + b[k];
}

/* ---- LM head ------------------------------------------------------------ */

/* lm_head_bf16_fp32_avx512 (:470-498). */
void oracle_lm_head_bf16(const uint16_t* emb, const float* x, float* logits, int V, int H) {
    const int H16 = H & ~15;
    #pragma omp parallel for schedule(static) if (V >= 64)
    for (int v = 0; v < V; ++v) {
        const uint16_t* row = emb + (ptrdiff_t)v * H;
        float lane[16];
        for (int i = 0; i < 16; ++i) lane[i] = 0.0f;
        for (int h = 0; h < H16; h += 16)
            for (int i = 0; i < 16; ++i)
                lane[i] = fmaf(bf16_bits_to_f32(row[h + i]), x[h + i], lane[i]);
        float tail = 0.0f;
        for (int h = H16; h < H; ++h) tail += bf16_bits_to_f32(row[h]) * x[h];
        logits[v] = tail + fold16_add(lane);
    }
}

/* lm_head_int8_fp32_avx512 (:501-525). */
void oracle_lm_head_int8(const int8_t* emb, const float* emb_scale, const float* x,
                         float* logits, int V, int H) {
    const int H16 = H & ~15;
    #pragma omp parallel for schedule(static) if (V >= 64)
    for (int v = 0; v < V; ++v) {
        const int8_t* row = emb + (ptrdiff_t)v * H;
        float lane[16];
        for (int i = 0; i < 16; ++i) lane[i] = 0.0f;
        for (int h = 0; h < H16; h += 16)
            for (int i = 0; i < 16; ++i)
                lane[i] = fmaf((float)row[h + i], x[h + i], lane[i]);
        float tail = 0.0f;
        for (int h = H16; h < H; ++h) tail += (float)row[h] * x[h];
        logits[v] = emb_scale[v] * (tail + fold16_add(lane));
    }
}

/* lm_head_int4_fp32_avx512 (:535-587): two signed nibbles per byte, low nibble
 * first; 32 columns per step feed the same 16 lanes twice (columns h..h+15,
 * then h+16..h+31). */
void oracle_lm_head_int4(const uint8_t* emb, const float* emb_scale, const float* x,
                         float* logits, int V, int H) {
    const int H32 = H & ~31;
    #pragma omp parallel for schedule(static) if (V >= 64)
    for (int v = 0; v < V; ++v) {
        const uint8_t* row = emb + (ptrdiff_t)v * (H / 2);
        float lane[16];
        for (int i = 0; i < 16; ++i) lane[i] = 0.0f;
        for (int h = 0; h < H32; h += 32) {
            float w[32];
            for (int i = 0; i < 16; ++i) {
                const uint8_t b = row[(h >> 1) + i];
                w[2 * i]     = (float)(int8_t)(((b & 0x0F) ^ 8) - 8);
                w[2 * i + 1] = (float)(int8_t)((((b >> 4) & 0x0F) ^ 8) - 8);
            }
            for (int i = 0; i < 16; ++i) lane[i] = fmaf(w[i], x[h + i], lane[i]);
            for (int i = 0; i < 16; ++i) lane[i] = fmaf(w[16 + i], x[h + 16 + i], lane[i]);
        }
        float tail = 0.0f;
        for (int h = H32; h < H; h += 2) {
            const uint8_t b = row[h >> 1];
            const int8_t lo = (int8_t)((int8_t)(b << 4) >> 4);
            const int8_t hi = (int8_t)((int8_t)b >> 4);
            tail += (float)lo * x[h];
            if (h + 1 < H) tail += (float)hi * x[h + 1];
        }
        logits[v] = emb_scale[v] * (tail + fold16_add(lane));
    }
}

int oracle_max_threads(void) {
#if defined(_OPENMP)
    return omp_get_max_threads();
#else
    return 1;
#endif
}
