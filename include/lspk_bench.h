/*
 * lspk_bench.h -- measurement-only entry points of the sm_100a library.
 *
 * Nothing here is part of the drop-in boundary and no product path calls it: these are the timing harnesses
 * that bench.py drives (CUDA-event timings of graph replays and of probe kernels).  They have no counterpart
 * in the reference, whose benchmark (benchmark_kernel.py) times its kernels from Python.
 */
#ifndef LSPK_BENCH_H_
#define LSPK_BENCH_H_

#include "lspk_runtime.h"
#include "lspk_tp.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Cost of handing a 2560-element activation vector from its producers to every consumer CTA inside ONE
 * persistent (cooperative) launch of `grid` CTAs, `iters` rounds back to back.  mode 0: each element is a
 * 64-bit packet (value | round tag), consumers poll the packets themselves; mode 1: plain stores, a
 * release/acquire counter barrier, plain loads.  Reports microseconds per round (CUDA events) and SM cycles
 * per round as seen by CTA 0.  Every device-side wait is bounded; LSPK_ERR_DEVICE_WAIT if one runs out. */
int lspk_bench_handoff(int grid, int iters, int mode, float* us_per_round_out, double* cycles_per_round_out);

/* What a decode step confined to one thread-block cluster could do.  `n_clusters` clusters of `cluster_size`
 * CTAs (one CTA per SM, 1..16 per cluster) run side by side.  mode 0: each CTA pulls `stages_per_cta` stages of
 * 16 KB from a 1 GB buffer through a ring of eight bulk copies; mode 1: `rounds` exchanges of a 2560-float
 * vector (every CTA stores its slice into every peer's shared memory, one cluster barrier, every CTA reduces the
 * vector); mode 2: an exchange after every `stages_per_round` stages; + 4: four warps take turns
 * requesting the stages instead of one thread requesting all of them.  Reports CUDA-event milliseconds. */
int lspk_bench_cluster(int cluster_size, int n_clusters, int stages_per_cta, int rounds, int stages_per_round, int mode,
                       float* ms_out);

/* Single-sequence states.  lspk_bench_linears replays a graph of just the
 * ternary linear launches of one decode step (4 per layer) `reps` times; lspk_bench_lm_head times the
 * LM-head kernel alone.  Both report CUDA-event milliseconds and the algorithmic bytes of ONE pass. */
int lspk_bench_linears(lspk_state_t s, int reps, float* ms_out, int* launches_out, double* bytes_out);
int lspk_bench_lm_head(lspk_state_t s, int reps, float* ms_out, double* bytes_out);
/* Time y = W_i (quant x) over n_w device copies of one matrix visited round-robin (reps passes). */
int lspk_bench_linear_copies(const lspk_weight_t* w, int n_w, const float* x_f32, float* y, int M, int reps,
                             float* ms_out);
/* Floor cost of a kernel boundary: a graph of n_kernels empty dependent kernels, replayed reps times. */
int lspk_bench_launch_floor(int n_kernels, int grid, int reps, float* ms_out);
/* lspk_bench_linear_copies with the launches of a pass on n_streams forked streams (independent graph nodes):
 * the amortised throughput of the kernel outside a dependency chain.  y holds n_streams * M * N floats.
 * int8_input != 0: x is quantised once beforehand and the launches take the int8 vector + scale, which is the
 * contract of the reference's matmul_lut_*_m1; 0: every launch quantises x itself (fused prologue).
 * w_up != NULL: launch i is the gated pair (w[i], w_up[i]) with the ReLU^2 epilogue. */
int lspk_bench_linear_copies_independent(const lspk_weight_t* w, const lspk_weight_t* w_up, int n_w, const float* x_f32,
                                         float* y, int M, int reps, int n_streams, int int8_input, float* ms_out);

/* CUDA-event time of `reps` replays of a graph of n_blocks MLP blocks over distinct weight triples.
 * inter_full == NULL: the two gathers of every block go through the peer windows instead of NCCL. */
int lspk_tp_bench_mlp(const lspk_weight_t* gate_r, const lspk_weight_t* up_r, const lspk_weight_t* down_r, int n_blocks,
                      const float* x_dev, const void* norm_gamma_bf16, const void* sub_norm_gamma_bf16, float eps,
                      float* inter_slice, float* inter_full, float* down_slice, float* y_full, int reps, float* ms_out);

#ifdef __cplusplus
}
#endif
#endif /* LSPK_BENCH_H_ */
