/*
 * lspk_hybrid.h -- the two decode blocks of the hybrid (Mamba-2 + ternary MoE) configuration and a
 * decode runtime that alternates them.
 *
 * No counterpart in the reference (it has no MoE and no state-space code); the blocks are defined by
 * the benchmark configuration: 8 ternary experts with a top-2 fp32 softmax router and squared-ReLU
 * FFNs stored as ONE packed buffer [expert][gate|up|down][rows, K/4] in the reference's 2-bit packing
 * (litespark_inference/torchless/pack.py:16-45), and Mamba-2 layers (heads x head_dim, d_state,
 * one group, depthwise conv of width 4) with ternary in/out projections.  Every ternary product
 * runs through the same decode / dp4a code as lspk_linear and is bit-exact against the reference's
 * matmul_lut_avx512_m1 on the selected expert's slice.
 */
#ifndef LSPK_HYBRID_H_
#define LSPK_HYBRID_H_

#include "lspk_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- packed-expert MoE layer -------------------------------------------------------------- */
typedef struct lspk_moe_s* lspk_moe_t;

/* experts_packed_host: uint8 [E][3][I*H/4]: gate [I, H/4], up [I, H/4], down [H, I/4] per expert.
 * scales_host: fp32 [E][3].  router_host: fp32 [E, H].  norm_gamma / sub_norm_gamma: bf16 bits,
 * [H] and [E, I].  Re-tiles every matrix into the device layout (one device buffer). */
lspk_moe_t lspk_moe_create(int n_experts, int hidden, int inter, const uint8_t* experts_packed_host,
                           const float* scales_host, const float* router_host,
                           const uint16_t* norm_gamma_host, const uint16_t* sub_norm_gamma_host, float eps);
int lspk_moe_free(lspk_moe_t m);
size_t lspk_moe_device_bytes(lspk_moe_t m);

/* One MoE layer for B token rows held on the device: x[B, H] (fp32) is updated in place,
 *   x += sum over the two routed experts of w_e * down_e(SubLN(relu(gate_e h)^2 * up_e h)),  h = RMSNorm(x).
 * Routing, grouping of rows by expert, the expert GEMVs (indexed by expert id from a device array, no
 * host sync) and the weighted sum all run as kernels on the library stream.
 * Optional taps (device pointers, may be NULL): sel_out int32 [B,2], selw_out fp32 [B,2],
 * acc_gate_out / acc_up_out int32 [B*2, I], acc_down_out int32 [B*2, H] (row = 2*token + slot). */
int lspk_moe_forward(lspk_moe_t m, float* x_dev, int B, int32_t* sel_out, float* selw_out,
                     int32_t* acc_gate_out, int32_t* acc_up_out, int32_t* acc_down_out);

/* ---- Mamba-2 decode step ------------------------------------------------------------------- */
typedef struct lspk_mamba_s* lspk_mamba_t;

typedef struct {
    int hidden, nheads, headdim, d_state, conv_width;   /* d_inner = nheads*headdim; conv_dim = d_inner + 2*d_state */
    float eps;
} lspk_mamba_config;

/* in_proj: packed [2*d_inner + 2*d_state + nheads, hidden/4]; out_proj: packed [hidden, d_inner/4];
 * conv_w fp32 [conv_dim, conv_width], conv_b fp32 [conv_dim]; A, dt_bias, D fp32 [nheads];
 * norm_gamma bf16 [hidden]; gated_norm_gamma bf16 [d_inner]. */
lspk_mamba_t lspk_mamba_create(const lspk_mamba_config* cfg, const uint8_t* in_proj_packed, float in_scale,
                               const uint8_t* out_proj_packed, float out_scale, const float* conv_w,
                               const float* conv_b, const float* A, const float* dt_bias, const float* D,
                               const uint16_t* norm_gamma, const uint16_t* gated_norm_gamma);
int lspk_mamba_free(lspk_mamba_t m);
size_t lspk_mamba_device_bytes(lspk_mamba_t m);
size_t lspk_mamba_state_floats(lspk_mamba_t m);     /* per sequence: conv ring + SSM state, in floats */

/* One decode step for B sequences: x[B, H] updated in place (residual added).  state_dev: fp32
 * [B][lspk_mamba_state_floats] zero-initialised by the caller at sequence start; pos_dev: int32 [B]
 * step index of each sequence (selects the slot of the conv ring). */
int lspk_mamba_step(lspk_mamba_t m, float* x_dev, float* state_dev, const int* pos_dev, int B);

/* ---- hybrid decode runtime ------------------------------------------------------------------ */
typedef struct lspk_hybrid_s* lspk_hybrid_t;
typedef struct lspk_hybrid_state_s* lspk_hybrid_state_t;

lspk_hybrid_t lspk_hybrid_create(int hidden, int vocab, float eps);
int lspk_hybrid_add_mamba(lspk_hybrid_t h, lspk_mamba_t layer);      /* layers run in the order added; */
int lspk_hybrid_add_moe(lspk_hybrid_t h, lspk_moe_t layer);          /* the model takes ownership      */
int lspk_hybrid_set_embedding(lspk_hybrid_t h, const uint16_t* emb_bf16_host, const uint16_t* final_norm_gamma);
int lspk_hybrid_free(lspk_hybrid_t h);
size_t lspk_hybrid_device_bytes(lspk_hybrid_t h);

lspk_hybrid_state_t lspk_hybrid_state_create(lspk_hybrid_t h, int batch, int max_steps);
int lspk_hybrid_state_free(lspk_hybrid_state_t s);
int lspk_hybrid_state_reset(lspk_hybrid_state_t s);
/* One decode step for every sequence: tokens in; optional logits [B, V] and greedy next tokens out. */
int lspk_hybrid_step(lspk_hybrid_state_t s, const int* tokens_host, float* logits_host, int* next_tokens_host);
/* n_steps chained greedy steps on the device (argmax feeds the next step); tokens_out_host [n_steps, B]. */
int lspk_hybrid_decode_greedy(lspk_hybrid_state_t s, const int* first_tokens_host, int n_steps, int* tokens_out_host);
/* Feed a prompt (one sequence at a time would break lock step, so: the same number of tokens for
 * every sequence, tokens_host [T, B]); the recurrence makes this a loop of T steps on the device. */
int lspk_hybrid_prefill(lspk_hybrid_state_t s, const int* tokens_host, int T, int* next_tokens_host);
int lspk_hybrid_step_kernel_count(lspk_hybrid_state_t s);

#ifdef __cplusplus
}
#endif
#endif /* LSPK_HYBRID_H_ */
