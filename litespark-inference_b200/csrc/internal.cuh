// Declarations shared between the translation units of the library (not part of the C ABI).
#pragma once
#include "common.cuh"

namespace lspk {

// layout.cu: reference byte layout (device copy) -> device chunk layout, on the library stream.
cudaError_t retile_to_device_launch(const uint8_t* src_dev, uint4* dst_dev, int N, int Kb, int groups, int chunks);

// linear.cu: validate + launch the CUDA-core ternary linear kernel on the library stream.
int linear_cuda_core(const lspk_linear_args* a);

// gemm_tc.cu: tcgen05 tensor-core path for large M.  Returns LSPK_OK and sets *handled = 1 when it
// ran; leaves *handled = 0 when the shape is outside what it supports.
int linear_tensor_core(const lspk_linear_args* a, int* handled);

// lm_head.cu
int lm_head_launch(int kind, const void* emb, const float* emb_scale, const float* x, float* logits,
                   int T, int V, int H, const void* norm_gamma, int gamma_is_bf16, float eps,
                   unsigned long long* best_key);

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
    const int* pos_ptr;    // device ints: position of row 0, or one position per row
    int pos_per_row;       // 0: rows are consecutive positions of one sequence; 1: one sequence per row
    size_t cache_seq_stride;  // elements between the caches of consecutive sequences (pos_per_row)
    int T, Q, KV, D, t_max;
    int fused;             // 1: rotate + cache write inside the attention kernel (independent rows)
    unsigned long long* trace;
    int trace_cap;
};
int attention_launch(const AttnParams& p, int kv_is_fp16);

}  // namespace lspk
