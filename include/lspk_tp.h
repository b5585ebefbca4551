/*
 * lspk_tp.h -- optional tensor-parallel (row-split) variant of the MLP projections.
 *
 * No counterpart in the reference (single process, no communication backend).  Each of g ranks
 * (one process per GPU) holds N/g output rows of gate/up and of down, computes its slice with the
 * ordinary ternary linear kernel and all-gathers the fp32 slices with NCCL over NVLink.  Rows are
 * independent, so the gathered vectors are bit-identical to the unsplit products.
 */
#ifndef LSPK_TP_H_
#define LSPK_TP_H_

#include "lspk_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif

int lspk_tp_unique_id(char* out128);                       /* rank 0: 128-byte NCCL id to share */
int lspk_tp_init(const char* id128, int rank, int world);  /* after lspk_init(device) on every rank */
int lspk_tp_rank(void);
int lspk_tp_world(void);
int lspk_tp_allgather_f32(const float* send_dev, float* recv_dev, size_t count_per_rank);
int lspk_tp_finalize(void);

/* One layer's MLP block at batch 1 with row-split weights (see csrc/tp.cu). */
int lspk_tp_mlp_block(lspk_weight_t gate_r, lspk_weight_t up_r, lspk_weight_t down_r, const float* x_dev,
                      const void* norm_gamma_bf16, const void* sub_norm_gamma_bf16, float eps, float* inter_slice,
                      float* inter_full, float* down_slice, float* y_full);
#ifdef __cplusplus
}
#endif
#endif /* LSPK_TP_H_ */
