/*
 * lspk_sm100.h -- C ABI of the sm_100a (B200) ternary-matmul library.
 *
 * Two groups of entry points:
 *
 *  (1) HOST-POINTER DROP-INS.  Same names, argument order and meaning as the symbols the
 *      reference's ctypes loader binds (litespark_inference/torchless/kernel.py:227-322),
 *      with the architecture tag `sm100` in place of `avx512` / `avx2` / `neon`.  Every
 *      pointer is a host pointer; the call copies inputs to the GPU, runs the CUDA kernel,
 *      copies the result back and returns when the result is in host memory.  Like the
 *      reference they return void / a value; a failure is recorded and can be read with
 *      lspk_last_error() / lspk_error_count().
 *
 *  (2) DEVICE-RESIDENT API.  Weights, activations and the KV cache live in GPU memory;
 *      pointers are device pointers obtained from lspk_malloc (or any CUDA allocation of the
 *      same context).  Every function returns an int status (0 = LSPK_OK).
 *
 * There is no CPU fallback: every entry point fails with LSPK_ERR_NO_DEVICE when no sm_100
 * GPU is usable.
 */
#ifndef LSPK_SM100_H_
#define LSPK_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    LSPK_OK = 0,
    LSPK_ERR_ARG = 1,        /* bad shape / null pointer / unsupported size */
    LSPK_ERR_CUDA = 2,       /* a CUDA runtime call failed; message has the detail */
    LSPK_ERR_NO_DEVICE = 3,  /* no usable GPU */
    LSPK_ERR_STATE = 4,      /* KV cache exhausted, model not finalised, ... */
    LSPK_ERR_NCCL = 5,
    LSPK_ERR_DEVICE_WAIT = 6 /* a bounded device-side wait ran out */
};

/* ------------------------------------------------------------------------------------ */
/* Library state                                                                         */
/* ------------------------------------------------------------------------------------ */
int lspk_init(int device);              /* select the GPU for this process; idempotent   */
int lspk_device_count(void);
int lspk_mem_info(size_t* free_bytes, size_t* total_bytes);   /* cudaMemGetInfo of the bound GPU */
int lspk_sm_count(void);
const char* lspk_last_error(void);      /* last recorded message ("" if none)            */
int lspk_error_count(void);             /* number of failures recorded so far            */
void lspk_clear_error(void);
int lspk_set_pdl(int enabled);          /* programmatic dependent launch between kernels */
int lspk_sync(void);                    /* wait for everything queued on the stream      */

void* lspk_malloc(size_t bytes);        /* device memory; NULL on failure                */
int lspk_free(void* dev);
void* lspk_host_alloc(size_t bytes);    /* pinned host memory                            */
int lspk_host_free(void* host);
int lspk_h2d(void* dev, const void* host, size_t bytes);   /* stream-ordered, then waits */
int lspk_d2h(void* host, const void* dev, size_t bytes);
int lspk_h2d_async(void* dev, const void* host, size_t bytes);
int lspk_d2h_async(void* host, const void* dev, size_t bytes);
int lspk_memset(void* dev, int value, size_t bytes);
int lspk_flush_l2(void);                /* overwrite a buffer larger than L2             */

/* CUDA-event timer on the library's stream: start, enqueue work, stop -> milliseconds.   */
int lspk_timer_start(void);
int lspk_timer_stop(float* ms_out);

/* In-kernel phase trace (measurement aid): after lspk_trace_begin, CTA 0 of each traced kernel
 * appends a record of 16 uint64 words [kernel id, globaltimer ns at entry, SM clock at phase marks
 * ..., globaltimer ns at exit]; lspk_trace_read copies the records out and clears the counter.
 * Kernels captured into a CUDA graph before lspk_trace_begin do not record; a later call with the same or a
 * smaller max_records keeps the buffer (graphs captured in between stay valid), a larger one replaces it. */
int lspk_trace_begin(int max_records);
int lspk_trace_read(unsigned long long* host_out, int max_records, int* n_out);

/* ------------------------------------------------------------------------------------ */
/* (a) Packed-weight upload: reference layout <-> device layout                          */
/*     Reference layout: uint8 [N, K/4], byte = (w0+1)|(w1+1)<<2|(w2+1)<<4|(w3+1)<<6       */
/*     (litespark_inference/torchless/pack.py:16-45; model.py:26-49 PackedProjection).    */
/*     Plays the role the reference gives transpose_packed_to_amx_vnni                    */
/*     (matmul_lut_avx512_extern_c.cpp:942-961): a load-time re-tiling for the hardware.  */
/* ------------------------------------------------------------------------------------ */
typedef struct lspk_weight_s* lspk_weight_t;
lspk_weight_t lspk_upload_packed(const uint8_t* packed_host, int N, int K, float w_scale);
/* The load-time quantiser on the device (quantize_ternary_absmean, torchless/quantize.py:24-60, then
 * pack_ternary_4_per_byte, pack.py:16-45): bf16 master weights [N, K] are ternarised with
 * t = clip(rint(w * float32(1 / absmean)), -1, 1), packed and re-tiled without leaving the GPU.  absmean
 * = mean |W| is computed by the host in the reference's summation order and passed in as a double;
 * the handle's scale is float32(absmean). */
lspk_weight_t lspk_upload_bf16_ternary(const uint16_t* w_bf16_host, int N, int K, double absmean);
int lspk_download_packed(lspk_weight_t w, uint8_t* packed_host_out);   /* exact inverse   */
int lspk_weight_free(lspk_weight_t w);
int lspk_weight_shape(lspk_weight_t w, int* N, int* K, float* scale, size_t* device_bytes);

/* ------------------------------------------------------------------------------------ */
/* (b)(c) Ternary GEMV / small-batch GEMM on device-resident data                         */
/* ------------------------------------------------------------------------------------ */
/* Prologue: what the kernel does to its input before the integer dot products.           */
enum { LSPK_PRO_INT8 = 0,        /* x is int8 [M,K] with per-row fp32 scales (a5/a6 contract) */
       LSPK_PRO_QUANT = 1,       /* x is fp32: per-token absmax int8 quantiser fused (a4)     */
       LSPK_PRO_RMSNORM_QUANT = 2,/* x is fp32: RMSNorm(gamma, eps) then quantiser (a10)       */
       LSPK_PRO_GATED_RMSNORM_QUANT = 3 /* x * SiLU(gate_f32), then RMSNorm and quantiser (Mamba-2 output norm) */ };
/* Epilogue: what happens to y = float(acc) * (x_scale * w_scale).                         */
enum { LSPK_EPI_STORE = 0,       /* out = y                                               */
       LSPK_EPI_ADD = 1,         /* out += y            (residual add, a12)                */
       LSPK_EPI_RELU2_MUL = 2,   /* two matrices (gate, up): out = max(g,0)^2 * u  (a11)   */
       LSPK_EPI_SILU_MUL = 3     /* two matrices (gate, up): out = g / (1 + exp(-g)) * u    */ };

typedef struct {
    /* up to three matrices that share the input (q/k/v, or gate/up); rows are independent */
    lspk_weight_t w[3];
    float* out[3];               /* fp32 [M, N_i] row-major (RELU2_MUL: only out[0], [M,N])  */
    int n_mats;
    int M;                       /* token rows, any M >= 1                                  */
    int prologue, epilogue;
    const float* x_f32;          /* [M,K] for QUANT / RMSNORM_QUANT                         */
    const int8_t* x_i8;          /* [M,K] for INT8                                          */
    const float* x_scales;       /* [M] device array for INT8                               */
    const void* gamma;           /* [K] bf16 bits (uint16) or fp32 for RMSNORM_QUANT        */
    int gamma_is_bf16;
    float eps;
    /* optional taps for parity tests (may be NULL) */
    int32_t* acc_out[3];         /* int32 [M, N_i]: the exact integer accumulators          */
    int8_t* xq_out;              /* int8 [M,K]: the quantised activations the kernel used   */
    float* xscale_out;           /* fp32 [M]                                                */
    const float* gate_f32;       /* [M,K] for GATED_RMSNORM_QUANT                           */
} lspk_linear_args;

#define LSPK_MAX_GEMV_M 8
/* Replaces matmul_lut_{tag}_m1 / _mT (matmul_lut_avx512_extern_c.cpp:150-236, 258-339) plus
 * the helpers fused around them.  Any M >= 1.  One row: the dp4a GEMV with the prologue fused in.
 * 2..31 rows: tiles of LSPK_MAX_GEMV_M rows on the warp-level int8 tensor cores (mma.sync).  From 32
 * rows: the TMA + tcgen05 GEMM (all four epilogues; the gated prologue stays on the tile kernel).
 * With more than one row of fp32 input the rows are normalised + quantised once, by a separate kernel,
 * into library scratch that grows with cudaMalloc: make the first call of a new size outside stream
 * capture.  The kernels request the packed weights and gamma before they wait for the work queued ahead of them
 * on the library stream: both must be complete in memory when the call is made (the upload functions of this
 * header synchronise); activations, residuals and outputs are ordered after everything queued before. */
int lspk_linear(const lspk_linear_args* a);
int lspk_linear_force_path(int path);   /* 0 auto, 1 CUDA-core kernel only, 2 tcgen05 only */
/* n independent one-row products in ONE launch: product i is args[i], which must have M == 1 and the int8
 * prologue (x_i8 + x_scales: the contract of the reference's matmul_lut_{tag}_m1, matmul_lut_avx512_extern_c.cpp:
 * 150-236; quantise fp32 rows first with lspk_quantize_rows / lspk_rmsnorm_quantize_rows), one matrix with the
 * STORE / ADD epilogue or a gate + up pair with a gated epilogue, up to 96 products, K up to 8192.  For callers
 * that loop over matrices which do not depend on one another (the reference's kernel benchmark does; so do the
 * experts of a mixture layer): the row groups of all products form one stream that a persistent grid, one CTA
 * per SM, pulls through a shared-memory ring of bulk asynchronous copies (six requesting warps, twelve computing
 * warps), so that no product pays a kernel's fill and drain.  The outputs must not be inputs of other products of the same call.  Results are bit-identical to
 * lspk_linear.  Every device-side wait is bounded; an expiry is reported by lspk_tc_check_error. */
int lspk_linear_batch(const lspk_linear_args* args, int n);
/* The tcgen05 kernel bounds every device-side wait; this reads and clears its expiry flag
 * (LSPK_ERR_DEVICE_WAIT if a wait ran out since the last call).  Synchronises the stream. */
int lspk_tc_check_error(void);

/* ------------------------------------------------------------------------------------ */
/* Element-wise helpers on device-resident rows (batched over T rows)                     */
/* ------------------------------------------------------------------------------------ */
int lspk_quantize_rows(const float* x, int8_t* out, float* scales, int T, int K);           /* a4  */
int lspk_rmsnorm_rows(const float* x, const void* gamma, int gamma_is_bf16, float* out,
                      int T, int K, float eps);                                              /* a9  */
int lspk_rmsnorm_quantize_rows(const float* x, const void* gamma, int gamma_is_bf16,
                               int8_t* out, float* scales, int T, int K, float eps);         /* a10 */
int lspk_relu2_mul_rows(const float* gate, const float* up, float* out, int T, int K);      /* a11 */
int lspk_add_rows(float* a, const float* b, size_t n);                                       /* a12 */

/* LM head GEMV on device-resident rows; kind: 0 bf16, 1 int8 (+scale), 2 int4 (+scale). a13 */
int lspk_lm_head(int kind, const void* emb, const float* emb_scale, const float* x,
                 float* logits, int T, int V, int H);

/* ------------------------------------------------------------------------------------ */
/* Host-pointer drop-ins (tag sm100).  kernel.py line of the binding each one replaces:   */
/* ------------------------------------------------------------------------------------ */
/* kernel.py:234-236  matmul_lut_{T}_m1 */
void matmul_lut_sm100_m1(const int8_t* x, const uint8_t* packed_w, float w_scale, float x_scale,
                         float* y, int N, int K);
/* kernel.py:247-251  matmul_lut_{T}_mT (x86 argument order).  Any T >= 1: the reference's
 * x86 kernel silently does nothing for T > 64 (matmul_lut_avx512_extern_c.cpp:266); this one
 * computes every row. */
void matmul_lut_sm100_mT(const int8_t* x, const float* x_scales, const uint8_t* packed_w,
                         float w_scale, float* y, int T, int N, int K);
/* kernel.py:252-256  matmul_lut_{T}_prefill (arm argument order) */
void matmul_lut_sm100_prefill(const int8_t* x, const uint8_t* packed_w, float w_scale,
                              const float* x_scale, float* y, int M, int N, int K);
/* kernel.py:295-297, 289-291 */
float quantize_activation_sm100(const float* x, int8_t* out, int K);
void quantize_activation_batched_sm100(const float* x, int8_t* out, float* scales, int T, int K);
/* kernel.py:307-312, 283-288 */
void rmsnorm_bf16gamma_fp32_sm100(const float* x, const uint16_t* gamma, float* out, int K, float eps);
void rmsnorm_fp32gamma_fp32_sm100(const float* x, const float* gamma, float* out, int K, float eps);
void rmsnorm_bf16gamma_fp32_batched_sm100(const float* x, const uint16_t* gamma, float* out,
                                          int T, int K, float eps);
void rmsnorm_fp32gamma_fp32_batched_sm100(const float* x, const float* gamma, float* out,
                                          int T, int K, float eps);
/* kernel.py:273-279.  `tmp` (caller scratch in the reference) is accepted and left untouched. */
float rmsnorm_quantize_bf16gamma_sm100(const float* x, const uint16_t* gamma, int8_t* out_i8,
                                       float* tmp, int K, float eps);
void rmsnorm_quantize_bf16gamma_batched_sm100(const float* x, const uint16_t* gamma, int8_t* out_i8,
                                              float* scales, float* tmp, int T, int K, float eps);
/* kernel.py:313-315, 292-294 */
void relu2_mul_fp32_sm100(const float* gate, const float* up, float* out, int K);
void relu2_mul_fp32_batched_sm100(const float* gate, const float* up, float* out, int T, int K);
/* kernel.py:316-318 */
void add_inplace_fp32_sm100(float* a, const float* b, int K);
/* kernel.py:298-306 */
void lm_head_bf16_fp32_sm100(const uint16_t* emb, const float* x, float* logits, int V, int H);
void lm_head_int8_fp32_sm100(const int8_t* emb, const float* emb_scale, const float* x,
                             float* logits, int V, int H);
void lm_head_int4_fp32_sm100(const uint8_t* emb, const float* emb_scale, const float* x,
                             float* logits, int V, int H);
/* kernel.py:319-320.  has_omp reports 0 (no OpenMP anywhere); max_threads reports the SM count. */
int matmul_lut_sm100_has_omp(void);
int matmul_lut_sm100_max_threads(void);

/* Same product as matmul_lut_sm100_m1, for callers that cannot allocate device memory at call time
 * (a server that handed all GPU memory to its own pool at start-up; a loop that must stay out of the
 * CUDA allocator's lock).  It has no counterpart in the reference, whose kernels work in host memory.
 * All device scratch (staging of the packed rows, their re-tiled copy, x and y) lives in one
 * file-scope device array of LSPK_NOALLOC_SCRATCH_BYTES that every GPU loading the library holds
 * until exit; the call makes no cudaMalloc / cudaFree.  Host pointers in and out, like the drop-in.
 * Returns LSPK_OK, or LSPK_ERR_ARG when the matrix does not fit the array (about N*K/2 + K + 4N
 * bytes are needed: 6912 x 2560 fits, 6912 x 6912 does not).
 * If the library is not yet bound to a GPU, the first call binds it (lspk_init: one stream, two events,
 * no device allocation: the word its bounded waits report through is also part of the library image)
 * and looks up the array's device address: make that first call before any stream capture begins.  The
 * call makes the bound GPU current for the calling thread.  Every call reuses the same
 * array, and the array keeps what the previous call left; nothing needs clearing because each call
 * overwrites what it reads.  Calls are serialised on the host and run on one stream; work issued by
 * other means that touched the array at the same time on the GPU would race with them. */
#define LSPK_NOALLOC_SCRATCH_BYTES (12u << 20)
int matmul_lut_sm100_m1_noalloc(const int8_t* x, const uint8_t* packed_w, float w_scale, float x_scale,
                                float* y, int N, int K);

/* Weight residency for the drop-ins.  By default a drop-in uploads the packed matrix (or the
 * embedding) on every call.  Registering a host buffer keeps a device copy keyed by its
 * address: later drop-in calls given the same pointer and shape skip the upload.  The caller
 * promises not to modify a registered buffer.  (No counterpart in the reference, whose
 * kernels read host memory directly.) */
int lspk_register_packed(const uint8_t* packed_host, int N, int K);
int lspk_register_embedding(int kind, const void* emb_host, const float* emb_scale_host, int V, int H);
int lspk_unregister(const void* host_ptr);
int lspk_unregister_all(void);

#ifdef __cplusplus
}
#endif
#endif /* LSPK_SM100_H_ */
