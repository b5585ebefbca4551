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

#ifdef __cplusplus
extern "C" {
#endif

/* Cost of handing a 2560-element activation vector from its producers to every consumer CTA inside ONE
 * persistent (cooperative) launch of `grid` CTAs, `iters` rounds back to back.  mode 0: each element is a
 * 64-bit packet (value | round tag), consumers poll the packets themselves; mode 1: plain stores, a
 * release/acquire counter barrier, plain loads.  Reports microseconds per round (CUDA events) and SM cycles
 * per round as seen by CTA 0.  Every device-side wait is bounded; LSPK_ERR_DEVICE_WAIT if one runs out. */
int lspk_bench_handoff(int grid, int iters, int mode, float* us_per_round_out, double* cycles_per_round_out);

#ifdef __cplusplus
}
#endif
#endif /* LSPK_BENCH_H_ */
