// Declarations shared between the translation units of the library (not part of the C ABI).
#pragma once
#include "common.cuh"

namespace lspk {

// layout.cu: reference byte layout (device copy) -> device chunk layout, on the library stream.
cudaError_t retile_to_device_launch(const uint8_t* src_dev, uint4* dst_dev, int N, int Kb, int groups, int chunks);

// linear.cu: kernel parameters (filled by linear_cuda_core, or directly by the MoE layer for its
// expert-grouped launches).
struct LinearSeg {
    const uint4* w;
    float* out;
    int32_t* acc_out;
    int N;
    int groups;
    float w_scale;
    int scale_idx;         // grouped mode: index of this matrix inside an expert's scale triple
};

// Internal prologue of the eight-row kernel: int8 rows already in its shared-memory layout (permuted 16-element
// blocks, rows mma_row_stride(Kp) bytes apart) with their sums, so that a tile is a plain copy.
constexpr int kProInt8Tiled = 16;

struct LinearParams {
    LinearSeg seg[3];
    int n_seg;
    int total_groups;      // row groups over all segments (of one matrix for the gated pairing)
    int K, chunks;
    int M;
    int prologue, epilogue;
    const float* x_f32;
    const float* gate_f32; // GATED_RMSNORM_QUANT: x is multiplied by SiLU(gate) before the norm
    const int8_t* x_i8;
    const float* x_scales;
    const int* x_sums;     // tiled int8 prologue: sum of each row's int8 values
    const void* gamma;
    int gamma_is_bf16;
    float eps;
    float rcp_K;           // 1.0f / K when division by K may use the fused multiply-add form, else 0
    int8_t* xq_out;
    float* xscale_out;
    int stream_weights;    // 1: weights are read once by this launch -> evict-first loads
    int bulk_stages;       // > 0 (expert-grouped launches of the eight-row kernel): weight ring of this many stages
    int* error_flag;       // set to LSPK_ERR_DEVICE_WAIT when a bounded wait of that variant runs out
    unsigned long long* trace;
    int trace_cap;
    // ---- expert-grouped mode (blockIdx.z = expert): rows and their count come from device arrays ----
    const int* grp_counts;     // [experts] rows routed to each expert
    const int* grp_rows;       // [experts][grp_rows_stride] output row of each routed row
    int grp_rows_stride;
    int grp_in_shift;          // input row = output row >> shift (1: two routed rows share one input row)
    size_t grp_w_stride;       // uint4 units between consecutive experts' copies of a matrix
    const float* grp_scales;   // [experts][3] weight scales
};

// linear_mma.cu: the eight-row tile kernel (mma.sync int8), also used for expert-grouped launches.
// Quantise (and normalise) M > 1 rows once into caller scratch and turn the call into an int8-prologue one.
int split_row_prologue(lspk_linear_args* a, int K, int8_t* q_scratch, float* scale_scratch);
// Library-owned scratch for that (grown with cudaMalloc: size it once outside stream capture).
int quant_scratch(size_t M, size_t K, int8_t** q, float** s, int** sums = nullptr);
// rows.cu: fp32 rows -> int8 rows in the tensor-core GEMM's permuted, padded layout (one kernel instead of
// quantise + permute); *done = 0 when the shape / alignment does not allow it.
int quantize_rows_permuted(const lspk_linear_args* a, int K, int Kp, int8_t* out_perm, float* scales, int* done,
                           int stride = 0, int* sums = nullptr);
// rows.cu: RMSNorm + quantiser of T rows, row t with the gamma_sel[t]-th bf16 weight vector.
int norm_quant_rows_selected(const float* x, const void* gamma_bf16, const int* gamma_sel, int8_t* out, float* scales,
                             int T, int K, float eps);
int linear_mma_launch(const LinearParams& p, bool pair, bool grouped, int grid_x, int grid_y, int grid_z);
__host__ __device__ inline int mma_row_stride(int Kp) { return (Kp % 128 == 0) ? Kp + 64 : Kp; }

// Launch the CUDA-core kernel with fully prepared parameters.  mt: rows per CTA tile (1, 2, 4 or 8).
int linear_launch_params(const LinearParams& p, int mt, bool pair, bool grouped, int grid_x, int grid_y, int grid_z);

// linear.cu: validate + launch the CUDA-core ternary linear kernel on the library stream.
int linear_cuda_core(const lspk_linear_args* a);

// gemm_tc.cu: tcgen05 tensor-core path for large M.  Returns LSPK_OK and sets *handled = 1 when it
// ran; leaves *handled = 0 when the shape is outside what it supports.
int linear_tensor_core(const lspk_linear_args* a, int* handled);

// lm_head.cu
int lm_head_launch(int kind, const void* emb, const float* emb_scale, const float* x, float* logits,
                   int T, int V, int H, const void* norm_gamma, int gamma_is_bf16, float eps,
                   unsigned long long* best_key);

// runtime.cu: small kernels of a decode step, shared with the hybrid runtime.
//   ctl layout: pos[batch], token[batch], step counter.
int launch_embed(const int* tokens, int rows, int kind, const void* emb, const float* scale, float* x, int H, int V);
int launch_argmax_rows(const float* logits, int rows, int V, unsigned long long* best);
int launch_finish_step(int* ctl, unsigned long long* best, int* tokens_out, int batch, int out_cap);

// moe.cu / mamba.cu: layer objects of the hybrid configuration.
struct Moe;
struct Mamba;
int moe_reserve(Moe* m, int B);
int moe_forward(Moe* m, float* x, int B, int32_t* sel_out, float* selw_out, int32_t* acc_gate, int32_t* acc_up,
                int32_t* acc_down);
int mamba_reserve(Mamba* m, int B);
int mamba_step(Mamba* m, float* x, float* state, const int* pos, int B);
size_t mamba_state_floats(const Mamba* m);

// attention.cu
struct AttnParams {
    float* q;              // [T, Q*D] fp32; rotated in place by the rope kernel / read raw when fused
    const float* k_cur;    // [T, KV*D] fp32 projections of the rows being processed
    const float* v_cur;    // [T, KV*D]
    float* out;            // [T, Q*D]
    void* cache_k;         // this layer's [t_max, KV, D] (of sequence 0)
    void* cache_v;
    const float* rope_cos; // [t_max, D/2]
    const float* rope_sin;
    const float* rope_cur; // optional [T][D]: cos | sin of each row's position at a fixed address (decode step)
    const int* pos_ptr;    // device ints: position of row 0, or one position per row
    int pos_per_row;       // 0: rows are consecutive positions of one sequence; 1: one sequence per row
    size_t cache_seq_stride;  // elements between the caches of consecutive sequences (pos_per_row)
    int T, Q, KV, D, t_max;
    int fused;             // 1: rotate + cache write inside the attention kernel (independent rows)
    unsigned long long* trace;
    int trace_cap;
};
int attention_launch(const AttnParams& p, int kv_is_fp16);

// One product of a streamed batch (linear_stream.cu).  The caller fills everything above the line; stream_launch
// fills the rest.  With `sel` set the product's matrices are chosen on the device: expert e = *sel (written by an
// earlier kernel of the stream), matrices w[m] + e * sel_stride, scales sel_scales[3 * e + scale_idx[m]].
struct StreamItem {
    const uint4* w[2];
    float* out;
    int32_t* acc[2];
    const int8_t* x;
    const float* xs;
    float ws[2];
    int N, K, chunks, groups;
    int nm;            // matrices per unit: 1, or 2 for the gated pairing
    int epilogue;
    const int* sel;
    size_t sel_stride; // uint4 units
    const float* sel_scales;
    int scale_idx[2];
    // ---- filled by stream_launch ----
    int unit0;         // flat index of this product's first unit
    int q0;            // flat index of this product's first stage
    int cps;           // chunks per stage and matrix
    int sub;           // stages per unit
};
constexpr int kStreamMaxItems = 96;
constexpr int kStreamMaxKp = 8192;               // longest row (K rounded up to 64)
struct StreamParams {
    StreamItem it[kStreamMaxItems];
    int n;
    int total_units;
    int* error_flag;
    int wait_for_predecessor;   // the requesting warps may not start before the previous kernel has finished (sel)
};
// Launch the streamed batch described by p->it[0 .. p->n) on the library stream.
int stream_launch(StreamParams* p);

}  // namespace lspk
