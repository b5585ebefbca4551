/*
 * lspk_runtime.h -- device-resident forward pass built on the kernels of lspk_sm100.h.
 *
 * Mirrors the host runtime of the reference (litespark_inference/torchless/runtime.py):
 *   InferState / init_state          (runtime.py:59-111)   -> lspk_state_create
 *   forward_one                      (runtime.py:171-282)  -> lspk_forward_step
 *   forward_prefill[_all_logits]     (runtime.py:285-489)  -> lspk_forward_prefill
 *   generate (greedy loop)           (runtime.py:669-697)  -> lspk_decode_greedy
 *   falcon_forward_one               (runtime.py:735-817)  -> same entry points, arch = 1
 * Weights, activations and the KV cache stay on the GPU; the host passes token ids in and gets
 * logits and/or the greedy next token back.  One decode step is a single CUDA-graph launch.
 */
#ifndef LSPK_RUNTIME_H_
#define LSPK_RUNTIME_H_

#include "lspk_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct lspk_model_s* lspk_model_t;
typedef struct lspk_state_s* lspk_state_t;

typedef struct {
    int hidden_size, num_layers, num_heads, num_kv_heads, intermediate_size, vocab_size;
    float rms_norm_eps;
    int arch;   /* 0: BitNet b1.58 (sub-norms, ReLU^2 gate, tied head); 1: Falcon-E (SiLU gate, no sub-norms) */
} lspk_model_config;

enum { LSPK_PROJ_Q = 0, LSPK_PROJ_K, LSPK_PROJ_V, LSPK_PROJ_O, LSPK_PROJ_GATE, LSPK_PROJ_UP, LSPK_PROJ_DOWN };
enum { LSPK_NORM_INPUT = 0, LSPK_NORM_POST_ATTN, LSPK_NORM_ATTN_SUB, LSPK_NORM_FFN_SUB, LSPK_NORM_FINAL };

/* Model construction: host arrays in the reference's formats (model.py:26-110) are uploaded
 * once; packed projections are re-tiled to the device layout on the way. */
lspk_model_t lspk_model_create(const lspk_model_config* cfg);
int lspk_model_set_projection(lspk_model_t m, int layer, int which, const uint8_t* packed_host,
                              int N, int K, float scale);
/* Same from bf16 master weights, ternarised on the device (lspk_upload_bf16_ternary). */
int lspk_model_set_projection_bf16(lspk_model_t m, int layer, int which, const uint16_t* w_bf16_host,
                                   int N, int K, double absmean);
int lspk_model_set_norm(lspk_model_t m, int layer, int which, const void* gamma_host, int is_bf16, int K);
/* kind: 0 bf16 bits [V,H], 1 int8 [V,H] + scale[V], 2 int4 [V,H/2] + scale[V].  The same table is
 * the LM head unless lspk_model_set_lm_head supplies an untied one. */
int lspk_model_set_embedding(lspk_model_t m, int kind, const void* emb_host, const float* scale_host);
int lspk_model_set_lm_head(lspk_model_t m, int kind, const void* head_host, const float* scale_host);
int lspk_model_finalize(lspk_model_t m);          /* checks that every tensor is present */
size_t lspk_model_device_bytes(lspk_model_t m);
/* Projection handle for direct use with lspk_linear (tests, micro-benchmarks). */
lspk_weight_t lspk_model_projection(lspk_model_t m, int layer, int which);
int lspk_model_free(lspk_model_t m);

/* Inference state for `batch` independent sequences (KV cache [batch][layer][t_max][kv][D]).
 * rope_cos / rope_sin: host fp32 [t_max, D/2], computed by the caller exactly as the reference's
 * rope_tables (ops.py:40-50) so that the rotation uses bit-identical tables. */
lspk_state_t lspk_state_create(lspk_model_t m, int t_max, int batch, int kv_fp16,
                               const float* rope_cos, const float* rope_sin);
int lspk_state_free(lspk_state_t s);
int lspk_state_get_pos(lspk_state_t s, int seq);
int lspk_state_set_pos(lspk_state_t s, int seq, int pos);    /* rollback / reuse (runtime.py:629) */
size_t lspk_state_device_bytes(lspk_state_t s);
/* Copy one sequence's cache slice [layer][0..n_pos) to the host as fp32 (tests). */
int lspk_state_read_kv(lspk_state_t s, int seq, int layer, int n_pos, float* k_host, float* v_host);

/* One decode step for every sequence of the state: tokens_host[batch] in, optionally
 * logits_host[batch, V] and next_tokens_host[batch] (greedy argmax, first maximum) out.
 * Returns LSPK_ERR_STATE when a cache is full (the reference raises RuntimeError, runtime.py:183).
 * With one sequence and no logits requested the step runs without copy operations: the token is read by the
 * step's first kernel from mapped pinned memory and the next token comes back in one 8-byte store that the call
 * polls for (no stream synchronisation). */
int lspk_forward_step(lspk_state_t s, const int* tokens_host, float* logits_host, int* next_tokens_host);

/* Feed T tokens of sequence `seq` at once (any T >= 1; processed in row chunks).  Outputs, each
 * optional: last_logits_host[V], all_logits_host[T, V], next_token_host (argmax of the last row). */
int lspk_forward_prefill(lspk_state_t s, int seq, const int* tokens_host, int T,
                         float* last_logits_host, float* all_logits_host, int* next_token_host);

/* Greedy decode of n_steps tokens for every sequence with no host round trip between steps: the
 * argmax of step i is the input of step i+1 on the device.  first_tokens_host[batch] starts it;
 * tokens_out_host[n_steps, batch] receives the generated ids (the argmax after each step). */
int lspk_decode_greedy(lspk_state_t s, const int* first_tokens_host, int n_steps, int* tokens_out_host);

/* Number of kernel launches contained in one decode step (graph nodes), for reporting. */
int lspk_state_step_kernel_count(lspk_state_t s);

/* Test aid for the bounded device-side waits: launches one thread that polls an mbarrier nothing arrives on
 * `polls` times (1..65536), gives up, and raises the library's wait flag; the next lspk_tc_check_error then
 * returns LSPK_ERR_DEVICE_WAIT once and clears it.  Nothing faults and the context stays usable. */
int lspk_debug_expire_wait(int polls);
#ifdef __cplusplus
}
#endif
#endif /* LSPK_RUNTIME_H_ */
