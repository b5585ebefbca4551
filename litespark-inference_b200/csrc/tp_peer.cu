// Tensor-parallel exchange over peer memory instead of a collective library.
//
// The NCCL all-gather of tp.cu moves 27.6 KB and 10.2 KB per MLP block: pure latency (a collective launch per
// message).  Here every rank owns a WINDOW -- one device buffer that all other ranks of the node map through
// CUDA IPC.  After a projection a small kernel stores this rank's slice into every rank's window as 64-bit
// packets (fp32 value | number of this exchange << 32), each with one 8-byte store through the mapped pointer:
// no fence, no atomic, no flag, because the value and the evidence that it is new travel in the same store.
// One more CTA of the same launch polls the packets of its own window until every one carries the current
// exchange number and writes the plain fp32 vector the next projection reads.  The polling is bounded: when
// it runs out the kernel raises the library's wait flag (lspk_tc_check_error -> LSPK_ERR_DEVICE_WAIT) and
// returns, so a rank that never arrives costs its peers an error code, not a hang.  No collective library, no
// multicast: plain stores to peer memory and loads of local memory.
//
// Window layout: [I packets: gathered gate product][H packets: gathered down product] (written by every rank),
// then, used locally only, the two plain fp32 vectors and the two exchange counters (how many exchanges of each
// kind are complete; kept on the device so that the same CUDA graph can be replayed).
#include <string.h>

#include "internal.cuh"
#include "../../include/lspk_tp.h"

namespace lspk {

constexpr int kTpMaxWorld = 8;
constexpr int kTpScatterCtas = 4;
constexpr int kTpUnpackThreads = 1024;

struct PeerWindow {
    void* local = nullptr;                 // this rank's window (cudaMalloc)
    void* peer[kTpMaxWorld] = {};          // every rank's window as seen from here (peer[rank] == local)
    bool opened[kTpMaxWorld] = {};
    size_t bytes = 0;
    int I = 0, H = 0, rank = 0, world = 1;
    unsigned poll_limit = 1u << 20;
};
static PeerWindow g_win;
static bool g_drop_next = false;           // test hook: the next exchange stores nothing (its wait must run out)

struct PeerPtrs {
    unsigned long long* dst[kTpMaxWorld];  // this rank's segment of the packet vector in every rank's window
};

// One launch per exchange.  CTAs 0 .. kTpScatterCtas-1 store `n` floats of this rank's slice into every rank's window
// as (value, exchange number) packets; the last CTA waits until every packet of this window's vector carries the
// current exchange number, writes the plain vector and counts the exchange as done.  The waiting CTA depends on
// the storing CTAs of the OTHER ranks' launches and on those of its own launch, which wait for nobody, so the
// launch cannot block itself.  The count is advanced only after every packet of this rank has arrived, i.e.
// after every storing thread has read it.
__global__ void __launch_bounds__(kTpUnpackThreads)
tp_exchange_kernel(const float* __restrict__ slice, int n, PeerPtrs peers, int world, int scatter_on,
                   const unsigned long long* __restrict__ packets, float* __restrict__ plain, int total,
                   unsigned* done_count, unsigned poll_limit, int* error_flag) {
    grid_dependency_launch();
    grid_dependency_wait();
    const unsigned want = *reinterpret_cast<volatile unsigned*>(done_count) + 1u;
    if (blockIdx.x < kTpScatterCtas) {
        if (!scatter_on) return;
        const unsigned long long tag = (unsigned long long)want << 32;
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += kTpScatterCtas * blockDim.x) {
            const unsigned long long pkt = tag | (unsigned long long)__float_as_uint(slice[i]);
            for (int r = 0; r < world; ++r)
                asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(peers.dst[r] + i), "l"(pkt) : "memory");
        }
        return;
    }
    __syncthreads();                       // every thread has read the count before thread 0 advances it below
    bool ok = true;
    // eight packets per thread and round: all their loads are in flight together, so a round costs one trip to
    // memory, and only the packets that have not arrived yet are asked for again
    for (int base = threadIdx.x; base < total; base += 8 * blockDim.x) {
        unsigned long long pkt[8];
        unsigned missing = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (base + k * (int)blockDim.x < total) missing |= 1u << k;
        for (unsigned poll = 0; poll < poll_limit && missing; ++poll) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (missing & (1u << k))
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(pkt[k]) : "l"(packets + base + k * (int)blockDim.x) : "memory");
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if ((missing & (1u << k)) && (unsigned)(pkt[k] >> 32) == want) missing &= ~(1u << k);
        }
        ok = ok && missing == 0;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (base + k * (int)blockDim.x < total) plain[base + k * (int)blockDim.x] = __uint_as_float((unsigned)pkt[k]);
    }
    const int all_ok = __syncthreads_and(ok ? 1 : 0);
    if (threadIdx.x == 0) {
        if (!all_ok && error_flag) atomicExch(error_flag, LSPK_ERR_DEVICE_WAIT);
        *done_count = want;
    }
}

// byte offsets inside a window
static size_t off_packets(int I, int which) { return which == 0 ? 0 : (size_t)I * 8; }
static size_t off_plain(int I, int H, int which) { return (size_t)(I + H) * 8 + (which == 0 ? 0 : (size_t)I * 4); }
static size_t off_counts(int I, int H) { return ((size_t)(I + H) * 12 + 15) & ~(size_t)15; }
static size_t window_bytes(int I, int H) { return off_counts(I, H) + 16; }

// which: 0 = gate product (I floats in all), 1 = down product (H floats in all)
static int exchange(const float* slice, int which) {
    const PeerWindow& w = g_win;
    const int total = which == 0 ? w.I : w.H, n = total / w.world;
    char* base = static_cast<char*>(w.local);
    unsigned* done = reinterpret_cast<unsigned*>(base + off_counts(w.I, w.H)) + which;
    PeerPtrs pp = {};
    for (int r = 0; r < w.world; ++r) {
        LSPK_REQUIRE(w.peer[r], "tensor-parallel window of rank %d has not been opened", r);
        pp.dst[r] = reinterpret_cast<unsigned long long*>(static_cast<char*>(w.peer[r]) + off_packets(w.I, which)) + (size_t)w.rank * n;
    }
    const int scatter_on = g_drop_next ? 0 : 1;
    g_drop_next = false;
    LSPK_CUDA(launch(tp_exchange_kernel, dim3(kTpScatterCtas + 1), dim3(kTpUnpackThreads), 0, true, slice, n, pp, w.world,
                     scatter_on, (const unsigned long long*)(base + off_packets(w.I, which)),
                     reinterpret_cast<float*>(base + off_plain(w.I, w.H, which)), total, done, w.poll_limit,
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
    const size_t bytes = window_bytes(I, H);
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
    return reinterpret_cast<const float*>(static_cast<char*>(g_win.local) + off_plain(g_win.I, g_win.H, which));
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
