// Tensor-parallel exchange over peer memory instead of a collective library.
//
// The NCCL all-gather of tp.cu moves 27.6 KB and 10.2 KB per MLP block: pure latency (a collective launch per
// message).  Here every rank owns a WINDOW -- one device buffer that all other ranks of the node map through
// CUDA IPC -- holding the two gathered vectors and two arrival counters.  After a projection a small kernel
// stores this rank's slice into every rank's window with plain stores through the mapped pointers, fences at
// system scope and adds one to each rank's counter; before the next projection a one-thread kernel waits until
// its own counter shows that every rank's slice has arrived.  The wait is bounded: when it runs out it raises the
// library's wait flag (lspk_tc_check_error -> LSPK_ERR_DEVICE_WAIT) and returns, so a rank that never arrives
// costs its peers an error code, not a hang.  No collective library, no multicast, nothing but stores, one
// atomic per peer and loads of local memory.
//
// Window layout (floats): [0, I) gathered gate product, [I, I + H) gathered down product, then two 64-bit
// arrival counters and two 64-bit epoch words (which exchange of its kind this is: the counters only grow, so
// the same graph can be replayed).
#include <string.h>

#include "internal.cuh"
#include "../../include/lspk_tp.h"

namespace lspk {

constexpr int kTpMaxWorld = 8;
constexpr int kTpScatterCtas = 4;

struct PeerWindow {
    void* local = nullptr;                 // this rank's window (cudaMalloc)
    void* peer[kTpMaxWorld] = {};          // every rank's window as seen from here (peer[rank] == local)
    bool opened[kTpMaxWorld] = {};
    size_t bytes = 0;
    int I = 0, H = 0, rank = 0, world = 1;
    unsigned poll_limit = 1u << 22;
};
static PeerWindow g_win;
static bool g_drop_next = false;           // test hook: the next exchange stores nothing (its wait must run out)

struct PeerPtrs {
    float* data[kTpMaxWorld];
    unsigned long long* counter[kTpMaxWorld];
};

// Store `n` floats of this rank's slice at `offset` floats into every rank's window, then tell every rank.
__global__ void __launch_bounds__(256) tp_scatter_kernel(const float* __restrict__ slice, int n, PeerPtrs peers, int world) {
    grid_dependency_launch();
    grid_dependency_wait();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = slice[i];
        for (int r = 0; r < world; ++r) peers.data[r][i] = v;
    }
    __threadfence_system();                // this thread's stores are visible to every GPU before the count below
    __syncthreads();
    if (threadIdx.x == 0)
        for (int r = 0; r < world; ++r) atomicAdd_system(peers.counter[r], 1ull);
}

// One thread: this is exchange number ++epoch of its kind; wait until all arrivals of that many exchanges are in.
__global__ void tp_wait_kernel(unsigned long long* counter, unsigned long long* epoch, unsigned long long per_exchange,
                               unsigned poll_limit, int* error_flag) {
    grid_dependency_launch();
    grid_dependency_wait();
    if (threadIdx.x == 0) {
        const unsigned long long target = (*epoch += 1ull) * per_exchange;
        bool ok = false;
        for (unsigned i = 0; i < poll_limit && !ok; ++i) {
            unsigned long long v;
            asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(counter) : "memory");
            ok = v >= target;
        }
        if (!ok && error_flag) atomicExch(error_flag, LSPK_ERR_DEVICE_WAIT);
    }
}

static size_t window_floats(int I, int H) { return (size_t)I + H; }
static unsigned long long* counter_of(void* base, int I, int H, int which) {
    return reinterpret_cast<unsigned long long*>(reinterpret_cast<float*>(base) + ((window_floats(I, H) + 3) & ~(size_t)3)) + which;
}
static unsigned long long* epoch_of(void* base, int I, int H, int which) { return counter_of(base, I, H, 2 + which); }

// which: 0 = gate product (offset 0, I floats in all), 1 = down product (offset I, H floats in all)
static int exchange(const float* slice, int which) {
    const PeerWindow& w = g_win;
    const int total = which == 0 ? w.I : w.H, n = total / w.world;
    PeerPtrs pp = {};
    for (int r = 0; r < w.world; ++r) {
        LSPK_REQUIRE(w.peer[r], "tensor-parallel window of rank %d has not been opened", r);
        pp.data[r] = reinterpret_cast<float*>(w.peer[r]) + (which == 0 ? 0 : w.I) + (size_t)w.rank * n;
        pp.counter[r] = counter_of(w.peer[r], w.I, w.H, which);
    }
    if (g_drop_next) g_drop_next = false;
    else LSPK_CUDA(launch(tp_scatter_kernel, dim3(kTpScatterCtas), dim3(256), 0, true, slice, n, pp, w.world));
    LSPK_CUDA(launch(tp_wait_kernel, dim3(1), dim3(32), 0, true, counter_of(w.local, w.I, w.H, which),
                     epoch_of(w.local, w.I, w.H, which), (unsigned long long)w.world * kTpScatterCtas, w.poll_limit,
                     device_wait_flag()));
    return LSPK_OK;
}

}  // namespace lspk

using namespace lspk;

extern "C" {

int lspk_tp_window_create(int rank, int world, int I, int H, void* ipc_handle64_out) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(world >= 1 && world <= kTpMaxWorld && rank >= 0 && rank < world && I >= world && H >= world &&
                     I % world == 0 && H % world == 0 && ipc_handle64_out,
                 "lspk_tp_window_create: bad arguments (world 1..%d, I and H divisible by it)", kTpMaxWorld);
    LSPK_REQUIRE(!g_win.local, "lspk_tp_window_create: a window already exists (close it first)");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are expected to be 64 bytes");
    const size_t bytes = ((window_floats(I, H) + 3) & ~(size_t)3) * 4 + 4 * 8;
    void* p = nullptr;
    LSPK_CUDA(cudaMalloc(&p, bytes));
    LSPK_CUDA(cudaMemset(p, 0, bytes));
    LSPK_CUDA(cudaDeviceSynchronize());
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(LSPK_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
    }
    memcpy(ipc_handle64_out, &h, 64);
    g_win = PeerWindow();
    g_win.local = p;
    g_win.bytes = bytes;
    g_win.I = I;
    g_win.H = H;
    g_win.rank = rank;
    g_win.world = world;
    g_win.peer[rank] = p;
    return LSPK_OK;
}

int lspk_tp_window_open(int rank, const void* ipc_handle64) {
    LSPK_REQUIRE(g_win.local && rank >= 0 && rank < g_win.world && rank != g_win.rank && ipc_handle64,
                 "lspk_tp_window_open: create the local window first; rank must be another rank of the group");
    LSPK_REQUIRE(!g_win.peer[rank], "lspk_tp_window_open: rank %d is already open", rank);
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle64, 64);
    void* p = nullptr;
    LSPK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    g_win.peer[rank] = p;
    g_win.opened[rank] = true;
    return LSPK_OK;
}

int lspk_tp_window_close(void) {
    if (!g_win.local) return LSPK_OK;
    cudaStreamSynchronize(stream());
    for (int r = 0; r < kTpMaxWorld; ++r)
        if (g_win.opened[r]) cudaIpcCloseMemHandle(g_win.peer[r]);
    cudaFree(g_win.local);
    g_win = PeerWindow();
    return LSPK_OK;
}

int lspk_tp_window_set_poll_limit(unsigned polls) {
    LSPK_REQUIRE(polls >= 1, "lspk_tp_window_set_poll_limit: at least one poll");
    g_win.poll_limit = polls;
    return LSPK_OK;
}

int lspk_tp_debug_drop_next_arrival(void) {
    g_drop_next = true;
    return LSPK_OK;
}

const float* lspk_tp_window_vector(int which) {
    if (!g_win.local || which < 0 || which > 1) return nullptr;
    return reinterpret_cast<const float*>(g_win.local) + (which == 0 ? 0 : g_win.I);
}

int lspk_tp_exchange(const float* slice_dev, int which) {
    LSPK_REQUIRE(g_win.local && slice_dev && (which == 0 || which == 1), "lspk_tp_exchange: bad arguments / no window");
    return exchange(slice_dev, which);
}

// The MLP block of lspk_tp_mlp_block with both gathers done through the peer windows.  The gathered down
// product is left in the window (lspk_tp_window_vector(1)).
int lspk_tp_mlp_block_peer(lspk_weight_t gate_r, lspk_weight_t up_r, lspk_weight_t down_r, const float* x_dev,
                           const void* norm_gamma_bf16, const void* sub_norm_gamma_bf16, float eps, float* inter_slice,
                           float* down_slice) {
    if (int rc = ensure_init()) return rc;
    LSPK_REQUIRE(g_win.local, "lspk_tp_mlp_block_peer: no window (lspk_tp_window_create)");
    const Weight* wg = reinterpret_cast<const Weight*>(gate_r);
    const Weight* wd = reinterpret_cast<const Weight*>(down_r);
    LSPK_REQUIRE(wg && up_r && wd && x_dev && inter_slice && down_slice, "lspk_tp_mlp_block_peer: null argument");
    LSPK_REQUIRE(wg->N * g_win.world == g_win.I && wd->N * g_win.world == g_win.H && wd->K == g_win.I,
                 "lspk_tp_mlp_block_peer: slices %d / %d do not match the window (%d, %d over %d ranks)", wg->N, wd->N,
                 g_win.I, g_win.H, g_win.world);
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
    if (int rc = exchange(inter_slice, 0)) return rc;
    lspk_linear_args d = {};
    d.w[0] = down_r;
    d.out[0] = down_slice;
    d.n_mats = 1;
    d.M = 1;
    d.prologue = LSPK_PRO_RMSNORM_QUANT;
    d.epilogue = LSPK_EPI_STORE;
    d.x_f32 = lspk_tp_window_vector(0);
    d.gamma = sub_norm_gamma_bf16;
    d.gamma_is_bf16 = 1;
    d.eps = eps;
    if (int rc = linear_cuda_core(&d)) return rc;
    return exchange(down_slice, 1);
}

}  // extern "C"
