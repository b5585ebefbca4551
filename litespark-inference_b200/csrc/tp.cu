// Tensor-parallel plumbing: an NCCL all-gather of fp32 row slices on the library stream.
//
// The reference is single-process; this is the optional row-split variant of the MLP projections:
// each rank holds N/g output rows of gate/up (and of down), computes its slice with the ordinary
// linear kernel and all-gathers the slices (rows are independent, so the gathered vector is
// bit-identical to the unsplit product).  NCCL is loaded at run time (dlopen) so that the library
// itself has no link dependency on it.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include "internal.cuh"
#include "../../include/lspk_tp.h"

namespace lspk {

struct NcclApi {
    void* so = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
};
static NcclApi g_nccl;
static ncclComm_t g_comm = nullptr;
static int g_tp_rank = 0, g_tp_world = 1;

static int nccl_load() {
    if (g_nccl.so) return LSPK_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        g_nccl.so = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.so) break;
    }
    if (!g_nccl.so) return fail(LSPK_ERR_NCCL, "cannot load libnccl: %s", dlerror());
    g_nccl.GetUniqueId = reinterpret_cast<decltype(&ncclGetUniqueId)>(dlsym(g_nccl.so, "ncclGetUniqueId"));
    g_nccl.CommInitRank = reinterpret_cast<decltype(&ncclCommInitRank)>(dlsym(g_nccl.so, "ncclCommInitRank"));
    g_nccl.AllGather = reinterpret_cast<decltype(&ncclAllGather)>(dlsym(g_nccl.so, "ncclAllGather"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(&ncclCommDestroy)>(dlsym(g_nccl.so, "ncclCommDestroy"));
    g_nccl.GetErrorString = reinterpret_cast<decltype(&ncclGetErrorString)>(dlsym(g_nccl.so, "ncclGetErrorString"));
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllGather || !g_nccl.CommDestroy || !g_nccl.GetErrorString) {
        dlclose(g_nccl.so);
        g_nccl = NcclApi();
        return fail(LSPK_ERR_NCCL, "libnccl lacks a required symbol");
    }
    return LSPK_OK;
}

#define LSPK_NCCL(expr)                                                                              \
    do {                                                                                             \
        ncclResult_t _r = (expr);                                                                    \
        if (_r != ncclSuccess) return fail(LSPK_ERR_NCCL, "%s failed: %s", #expr, g_nccl.GetErrorString(_r)); \
    } while (0)

}  // namespace lspk

using namespace lspk;

extern "C" {

int lspk_tp_unique_id(char* out128) {
    LSPK_REQUIRE(out128, "lspk_tp_unique_id: null buffer");
    if (int rc = nccl_load()) return rc;
    ncclUniqueId id;
    LSPK_NCCL(g_nccl.GetUniqueId(&id));
    static_assert(sizeof(id) == 128, "ncclUniqueId is expected to be 128 bytes");
    memcpy(out128, &id, 128);
    return LSPK_OK;
}

int lspk_tp_init(const char* id128, int rank, int world) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(id128 && world >= 1 && rank >= 0 && rank < world, "lspk_tp_init: bad arguments");
    if (int rc = nccl_load()) return rc;
    LSPK_REQUIRE(!g_comm, "lspk_tp_init: already initialised");
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    LSPK_NCCL(g_nccl.CommInitRank(&g_comm, world, id, rank));
    g_tp_rank = rank;
    g_tp_world = world;
    return LSPK_OK;
}

int lspk_tp_rank(void) { return g_tp_rank; }
int lspk_tp_world(void) { return g_tp_world; }

int lspk_tp_allgather_f32(const float* send_dev, float* recv_dev, size_t count_per_rank) {
    LSPK_REQUIRE(send_dev && recv_dev && count_per_rank >= 1, "lspk_tp_allgather_f32: bad arguments");
    if (g_tp_world == 1 || !g_comm) {
        if (send_dev != recv_dev)
            LSPK_CUDA(cudaMemcpyAsync(recv_dev, send_dev, count_per_rank * 4, cudaMemcpyDeviceToDevice, stream()));
        return LSPK_OK;
    }
    LSPK_NCCL(g_nccl.AllGather(send_dev, recv_dev, count_per_rank, ncclFloat32, g_comm, stream()));
    return LSPK_OK;
}

int lspk_tp_finalize(void) {
    if (g_comm) {
        cudaStreamSynchronize(stream());
        g_nccl.CommDestroy(g_comm);
        g_comm = nullptr;
    }
    g_tp_rank = 0;
    g_tp_world = 1;
    return LSPK_OK;
}

// Row-split MLP block of one layer at batch 1, as one enqueue (capturable):
//   inter_slice = relu(gate_r h)^2 * (up_r h), h = quant(RMSNorm(x))      [I/g]
//   inter       = all-gather(inter_slice)                                   [I]
//   down_slice  = down_r quant(RMSNorm(inter))                              [H/g]
//   y           = all-gather(down_slice)                                    [H]
// gate_r / up_r / down_r are this rank's row slices uploaded as ordinary weight handles.
int lspk_tp_mlp_block(lspk_weight_t gate_r, lspk_weight_t up_r, lspk_weight_t down_r, const float* x_dev,
                      const void* norm_gamma_bf16, const void* sub_norm_gamma_bf16, float eps, float* inter_slice,
                      float* inter_full, float* down_slice, float* y_full) {
    if (int rc = ensure_init()) return rc;
    const Weight* wg = reinterpret_cast<const Weight*>(gate_r);
    const Weight* wd = reinterpret_cast<const Weight*>(down_r);
    LSPK_REQUIRE(wg && up_r && wd && x_dev && inter_slice && inter_full && down_slice && y_full,
                 "lspk_tp_mlp_block: null argument");
    lspk_linear_args a = {};
    a.w[0] = gate_r;
    a.w[1] = up_r;
    a.out[0] = inter_slice;
    a.n_mats = 2;
    a.M = 1;
    a.prologue = LSPK_PRO_RMSNORM_QUANT;
    a.epilogue = LSPK_EPI_RELU2_MUL;
    a.x_f32 = x_dev;
    a.gamma = norm_gamma_bf16;
    a.gamma_is_bf16 = 1;
    a.eps = eps;
    if (int rc = linear_cuda_core(&a)) return rc;
    if (int rc = lspk_tp_allgather_f32(inter_slice, inter_full, (size_t)wg->N)) return rc;
    lspk_linear_args d = {};
    d.w[0] = down_r;
    d.out[0] = down_slice;
    d.n_mats = 1;
    d.M = 1;
    d.prologue = LSPK_PRO_RMSNORM_QUANT;
    d.epilogue = LSPK_EPI_STORE;
    d.x_f32 = inter_full;
    d.gamma = sub_norm_gamma_bf16;
    d.gamma_is_bf16 = 1;
    d.eps = eps;
    if (int rc = linear_cuda_core(&d)) return rc;
    return lspk_tp_allgather_f32(down_slice, y_full, (size_t)wd->N);
}

}  // extern "C"
