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

/* The same exchange over peer memory (csrc/tp_peer.cu): every rank creates one window (a device buffer holding
 * the gathered gate product [I] and the gathered down product [H] as 64-bit packets, value | exchange number),
 * hands its 64-byte CUDA IPC handle to the other ranks of the node by any host channel, and opens theirs.
 * lspk_tp_exchange is one launch: four CTAs store this rank's slice (which = 0: I / world floats of the gate
 * product, 1: H / world floats of the down product) into every window, one 8-byte store per element, and a fifth
 * polls, with a bound, the packets of its own window until every rank's slice of this exchange is there and
 * writes the plain fp32 vector.  When the
 * bound runs out the library's wait flag is raised (lspk_tc_check_error returns LSPK_ERR_DEVICE_WAIT) and the
 * stream carries on: a rank that never arrives costs an error code, not a hang. */
int lspk_tp_window_create(int rank, int world, int I, int H, void* ipc_handle64_out);
int lspk_tp_window_open(int rank, const void* ipc_handle64);
int lspk_tp_window_close(void);
int lspk_tp_window_set_poll_limit(unsigned polls);          /* loads of a packet before the wait for it gives up */
/* Test aid for the bounded wait: the next lspk_tp_exchange stores nothing, as if this rank's peers were gone, so
 * its wait polls packets that nothing renews, gives up and raises the wait flag.  Nothing faults. */
int lspk_tp_debug_drop_next_arrival(void);
const float* lspk_tp_window_vector(int which);              /* device pointer of a gathered vector in the local window */
int lspk_tp_exchange(const float* slice_dev, int which);
/* lspk_tp_mlp_block with both gathers through the windows; the gathered down product stays in the window. */
int lspk_tp_mlp_block_peer(lspk_weight_t gate_r, lspk_weight_t up_r, lspk_weight_t down_r, const float* x_dev,
                           const void* norm_gamma_bf16, const void* sub_norm_gamma_bf16, float eps, float* inter_slice,
                           float* down_slice);
#ifdef __cplusplus
}
#endif
#endif /* LSPK_TP_H_ */
