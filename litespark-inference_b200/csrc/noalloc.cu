// Ternary GEMV for callers that must not allocate device memory.
//
// Some hosts of this library cannot go through the CUDA allocator at call time: an inference
// server that reserved all of the GPU's memory for its own pool at start-up (so a cudaMalloc from
// a plug-in fails or fragments the pool), or a latency-critical loop that may not take the
// allocator's device-wide lock and its implicit synchronisation.  The ordinary host-pointer entry
// point, matmul_lut_sm100_m1, grows device staging buffers on demand and uploads the packed matrix
// into freshly allocated memory.  The variant below does the same work with every byte of device
// scratch taken from one fixed array that is part of the library image.
#include <mutex>

#include "internal.cuh"

namespace lspk {

// All device scratch of the no-allocation GEMV.  Resident on every GPU that loads the library,
// from load until process exit.
static __device__ __align__(256) unsigned char g_noalloc_scratch[LSPK_NOALLOC_SCRATCH_BYTES];

static std::mutex g_noalloc_mu;
static unsigned char* g_noalloc_dev = nullptr;     // device address of the array on the GPU the library is bound to

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace lspk

using namespace lspk;

extern "C" int matmul_lut_sm100_m1_noalloc(const int8_t* x, const uint8_t* packed_w, float w_scale, float x_scale,
                                           float* y, int N, int K) {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(x && packed_w && y && N >= 1 && K >= 4 && (K & 3) == 0,
                 "matmul_lut_sm100_m1_noalloc: bad arguments (N=%d K=%d)", N, K);

    // carve the fixed array: raw packed rows | re-tiled rows | x | x_scale | y
    const int Kb = K / 4;
    const int groups = (N + kRowsPerGroup - 1) / kRowsPerGroup;
    const int chunks = (K + kWeightsPerChunk - 1) / kWeightsPerChunk;
    const size_t raw_bytes = align_up((size_t)N * Kb, 256);
    const size_t tiled_bytes = (size_t)groups * chunks * kRowsPerGroup * 16;
    const size_t x_bytes = align_up((size_t)K, 256);
    const size_t y_bytes = align_up((size_t)N * 4, 256);
    const size_t need = raw_bytes + tiled_bytes + x_bytes + 256 + y_bytes;
    if (need > (size_t)LSPK_NOALLOC_SCRATCH_BYTES)
        return fail(LSPK_ERR_ARG,
                    "matmul_lut_sm100_m1_noalloc: a %d x %d matrix needs %zu bytes of device scratch; the built-in "
                    "array holds %zu (use matmul_lut_sm100_m1, which allocates, for larger matrices)",
                    N, K, need, (size_t)LSPK_NOALLOC_SCRATCH_BYTES);

    // The array's name is only a host-side handle here: the device address has to be asked for, with
    // the right device current.  The library's stream lives on the GPU the library is bound to, so that
    // GPU is made current for the calling thread (which may never have selected one) before the lookup
    // and for every copy and launch below.
    LSPK_CUDA(cudaSetDevice(bound_device()));
    if (!g_noalloc_dev) {
        void* p = nullptr;
        LSPK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
        g_noalloc_dev = static_cast<unsigned char*>(p);
    }
    unsigned char* base = g_noalloc_dev;
    uint8_t* d_raw = base;
    uint4* d_tiled = reinterpret_cast<uint4*>(base + raw_bytes);
    int8_t* d_x = reinterpret_cast<int8_t*>(base + raw_bytes + tiled_bytes);
    float* d_xs = reinterpret_cast<float*>(base + raw_bytes + tiled_bytes + x_bytes);
    float* d_y = reinterpret_cast<float*>(base + raw_bytes + tiled_bytes + x_bytes + 256);

    // Nothing in the array has to start at zero: every byte a kernel reads below is written first
    // in this same call (the re-tiling kernel also writes the padding of the tiled copy).
    LSPK_CUDA(cudaMemcpyAsync(d_raw, packed_w, (size_t)N * Kb, cudaMemcpyHostToDevice, stream()));
    LSPK_CUDA(cudaMemcpyAsync(d_x, x, (size_t)K, cudaMemcpyHostToDevice, stream()));
    LSPK_CUDA(cudaMemcpyAsync(d_xs, &x_scale, sizeof(float), cudaMemcpyHostToDevice, stream()));
    LSPK_CUDA(retile_to_device_launch(d_raw, d_tiled, N, Kb, groups, chunks));

    Weight w;
    w.dev = d_tiled;
    w.N = N;
    w.K = K;
    w.groups = groups;
    w.chunks = chunks;
    w.scale = w_scale;
    w.bytes = tiled_bytes;
    lspk_linear_args a = {};
    a.w[0] = reinterpret_cast<lspk_weight_t>(&w);
    a.out[0] = d_y;
    a.n_mats = 1;
    a.M = 1;
    a.prologue = LSPK_PRO_INT8;
    a.epilogue = LSPK_EPI_STORE;
    a.x_i8 = d_x;
    a.x_scales = d_xs;
    if (int rc = linear_cuda_core(&a)) return rc;
    LSPK_CUDA(cudaMemcpyAsync(y, d_y, (size_t)N * 4, cudaMemcpyDeviceToHost, stream()));
    LSPK_CUDA(cudaStreamSynchronize(stream()));
    return LSPK_OK;
}
