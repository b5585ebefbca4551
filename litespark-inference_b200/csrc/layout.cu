// Packed-weight upload: reference byte layout [N, K/4]  <->  device chunk layout
// [row-group of 16][chunk along K][row in group] x 16 bytes.  Pure byte regrouping.
#include "common.cuh"

namespace lspk {

// One thread per 16-byte device chunk.  `src` is the reference layout (row stride Kb bytes).
// Bytes outside the logical matrix become 0x55: four codes of value 1, i.e. weight 0.
__global__ void retile_to_device_kernel(const uint8_t* __restrict__ src, uint4* __restrict__ dst,
                                        int N, int Kb, int groups, int chunks) {
    const long long total = (long long)groups * chunks * kRowsPerGroup;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(idx % kRowsPerGroup);
        const long long gj = idx / kRowsPerGroup;
        const int j = (int)(gj % chunks);
        const int g = (int)(gj / chunks);
        const int n = g * kRowsPerGroup + r;
        uint32_t w[4];
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            uint32_t v = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int kb = j * 16 + m * 4 + b;
                uint32_t byte = 0x55u;
                if (n < N && kb < Kb) byte = src[(size_t)n * Kb + kb];
                v |= byte << (8 * b);
            }
            w[m] = v;
        }
        dst[idx] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// Inverse: one thread per reference byte.
__global__ void retile_to_reference_kernel(const uint8_t* __restrict__ dev_bytes,
                                           uint8_t* __restrict__ dst, int N, int Kb, int chunks) {
    const long long total = (long long)N * Kb;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int n = (int)(idx / Kb);
        const int kb = (int)(idx % Kb);
        const int g = n / kRowsPerGroup, r = n % kRowsPerGroup;
        const int j = kb / 16, off = kb % 16;
        const size_t chunk = ((size_t)g * chunks + j) * kRowsPerGroup + r;
        dst[idx] = dev_bytes[chunk * 16 + off];
    }
}

// Launch the re-tiling kernel on the library stream (both pointers are device pointers).
cudaError_t retile_to_device_launch(const uint8_t* src_dev, uint4* dst_dev, int N, int Kb, int groups, int chunks) {
    const long long total = (long long)groups * chunks * kRowsPerGroup;
    const int block = 256;
    const int grid = (int)((total + block - 1) / block < 65535 ? (total + block - 1) / block : 65535);
    retile_to_device_kernel<<<grid, block, 0, stream()>>>(src_dev, dst_dev, N, Kb, groups, chunks);
    return cudaGetLastError();
}


// bf16 master weights [N, K] (row-major) -> ternary codes, four per byte in the reference layout
// [N, K/4].  t = clip(rint(w * inv), -1, 1) with rint = round-half-even, as the reference's host
// quantiser does in fp32 (quantize.py:24-60); code = t + 1.  K is a multiple of 4, so a byte never
// straddles two rows and the kernel is a flat map over bytes.
__global__ void ternarize_pack_kernel(const uint16_t* __restrict__ w, uint8_t* __restrict__ packed, long long n_bytes,
                                      float inv) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_bytes; i += (long long)gridDim.x * blockDim.x) {
        const uint2 four = *reinterpret_cast<const uint2*>(w + 4 * i);
        const float f[4] = {__uint_as_float(four.x << 16), __uint_as_float(four.x & 0xffff0000u),
                            __uint_as_float(four.y << 16), __uint_as_float(four.y & 0xffff0000u)};
        uint32_t byte = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float t = fminf(fmaxf(rintf(__fmul_rn(f[e], inv)), -1.0f), 1.0f);
            byte |= (uint32_t)((int)t + 1) << (2 * e);
        }
        packed[i] = (uint8_t)byte;
    }
}

}  // namespace lspk

using namespace lspk;

extern "C" {

lspk_weight_t lspk_upload_packed(const uint8_t* packed_host, int N, int K, float w_scale) {
    if (ensure_init()) return nullptr;
    if (!packed_host || N <= 0 || K <= 0 || (K & 3)) {
        fail(LSPK_ERR_ARG, "lspk_upload_packed: need N > 0, K > 0, K %% 4 == 0 (got N=%d K=%d)", N, K);
        return nullptr;
    }
    const int Kb = K / 4;
    Weight* w = new Weight();
    w->N = N;
    w->K = K;
    w->groups = (N + kRowsPerGroup - 1) / kRowsPerGroup;
    w->chunks = (K + kWeightsPerChunk - 1) / kWeightsPerChunk;
    w->scale = w_scale;
    w->bytes = (size_t)w->groups * w->chunks * kRowsPerGroup * 16;
    w->dev = nullptr;
    uint8_t* staging = nullptr;
    cudaError_t e = cudaMalloc(&w->dev, w->bytes);
    if (e == cudaSuccess) e = cudaMalloc(&staging, (size_t)N * Kb);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(staging, packed_host, (size_t)N * Kb, cudaMemcpyHostToDevice, stream());
    if (e == cudaSuccess) {
        const long long total = (long long)w->groups * w->chunks * kRowsPerGroup;
        const int block = 256;
        const int grid = (int)((total + block - 1) / block < 65535 ? (total + block - 1) / block : 65535);
        retile_to_device_kernel<<<grid, block, 0, stream()>>>(staging, w->dev, N, Kb, w->groups, w->chunks);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream());
    if (staging) cudaFree(staging);
    if (e != cudaSuccess) {
        fail(LSPK_ERR_CUDA, "lspk_upload_packed: %s", cudaGetErrorString(e));
        if (w->dev) cudaFree(w->dev);
        delete w;
        return nullptr;
    }
    return reinterpret_cast<lspk_weight_t>(w);
}

lspk_weight_t lspk_upload_bf16_ternary(const uint16_t* w_bf16_host, int N, int K, double absmean) {
    if (ensure_init()) return nullptr;
    if (!w_bf16_host || N <= 0 || K <= 0 || (K & 3) || !(absmean > 0.0)) {
        fail(LSPK_ERR_ARG, "lspk_upload_bf16_ternary: need N > 0, K > 0, K %% 4 == 0, absmean > 0 (got N=%d K=%d)", N, K);
        return nullptr;
    }
    // the reference multiplies fp32 weights by float32(1 / absmean) and hands float32(absmean) to its kernels
    const float inv = (float)(1.0 / absmean);
    const float scale = (float)absmean;
    const int Kb = K / 4;
    Weight* w = new Weight();
    w->N = N;
    w->K = K;
    w->groups = (N + kRowsPerGroup - 1) / kRowsPerGroup;
    w->chunks = (K + kWeightsPerChunk - 1) / kWeightsPerChunk;
    w->scale = scale;
    w->bytes = (size_t)w->groups * w->chunks * kRowsPerGroup * 16;
    w->dev = nullptr;
    uint16_t* master = nullptr;
    uint8_t* staging = nullptr;
    cudaError_t e = cudaMalloc(&w->dev, w->bytes);
    if (e == cudaSuccess) e = cudaMalloc(&master, (size_t)N * K * 2);
    if (e == cudaSuccess) e = cudaMalloc(&staging, (size_t)N * Kb);
    if (e == cudaSuccess) e = cudaMemcpyAsync(master, w_bf16_host, (size_t)N * K * 2, cudaMemcpyHostToDevice, stream());
    if (e == cudaSuccess) {
        const long long n_bytes = (long long)N * Kb;
        const int block = 256;
        long long g = (n_bytes + block - 1) / block;
        const long long cap = (long long)sm_count() * 16;
        ternarize_pack_kernel<<<(int)(g < cap ? g : cap), block, 0, stream()>>>(master, staging, n_bytes, inv);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) {
        const long long total = (long long)w->groups * w->chunks * kRowsPerGroup;
        const int block = 256;
        const int grid = (int)((total + block - 1) / block < 65535 ? (total + block - 1) / block : 65535);
        retile_to_device_kernel<<<grid, block, 0, stream()>>>(staging, w->dev, N, Kb, w->groups, w->chunks);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream());
    if (master) cudaFree(master);
    if (staging) cudaFree(staging);
    if (e != cudaSuccess) {
        fail(LSPK_ERR_CUDA, "lspk_upload_bf16_ternary: %s", cudaGetErrorString(e));
        if (w->dev) cudaFree(w->dev);
        delete w;
        return nullptr;
    }
    return reinterpret_cast<lspk_weight_t>(w);
}

int lspk_download_packed(lspk_weight_t h, uint8_t* packed_host_out) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(h && packed_host_out, "lspk_download_packed: null argument");
    Weight* w = reinterpret_cast<Weight*>(h);
    const int Kb = w->K / 4;
    uint8_t* staging = nullptr;
    LSPK_CUDA(cudaMalloc(&staging, (size_t)w->N * Kb));
    const long long total = (long long)w->N * Kb;
    const int block = 256;
    const int grid = (int)((total + block - 1) / block < 65535 ? (total + block - 1) / block : 65535);
    retile_to_reference_kernel<<<grid, block, 0, stream()>>>(
        reinterpret_cast<const uint8_t*>(w->dev), staging, w->N, Kb, w->chunks);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(packed_host_out, staging, (size_t)w->N * Kb, cudaMemcpyDeviceToHost, stream());
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream());
    cudaFree(staging);
    if (e != cudaSuccess) return fail(LSPK_ERR_CUDA, "lspk_download_packed: %s", cudaGetErrorString(e));
    return LSPK_OK;
}

int lspk_weight_free(lspk_weight_t h) {
    if (!h) return LSPK_OK;
    Weight* w = reinterpret_cast<Weight*>(h);
    if (w->dev) cudaFree(w->dev);
    delete w;
    return LSPK_OK;
}

int lspk_weight_shape(lspk_weight_t h, int* N, int* K, float* scale, size_t* device_bytes) {
    LSPK_REQUIRE(h, "lspk_weight_shape: null handle");
    Weight* w = reinterpret_cast<Weight*>(h);
    if (N) *N = w->N;
    if (K) *K = w->K;
    if (scale) *scale = w->scale;
    if (device_bytes) *device_bytes = w->bytes;
    return LSPK_OK;
}

}  // extern "C"
