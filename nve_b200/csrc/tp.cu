// Tensor-parallel context: one symmetric buffer per rank ({partial sum, epoch} slots + per-CTA launch counters),
// exported with CUDA IPC and mapped by every peer, so that the row-parallel GEMVs (o_proj, down_proj) can
// all-reduce their output inside the kernel: partial rows are pushed to every rank with plain 8-byte peer
// stores over NVLink / NVSwitch and each rank polls only its own memory (gemv_w4.cu).
//
// The reference project has no multi-GPU path; this file has no counterpart there.
//
// Protocol (host side, once):  every rank calls nve_b200_tp_create -> exchanges the 64-byte handles through any
// host channel (the Python side uses torch.distributed) -> every rank calls nve_b200_tp_connect with all
// handles in rank order.  No multicast / multimem objects are created: peers are reached with ordinary
// stores, and every device-side wait is bounded (an expired wait sets the error word read by
// nve_b200_tp_error).
#include <string.h>

#include "gemv_w4.cuh"

namespace nve {

namespace {
struct TpHost {
    TpDev dev = {};
    void* local = nullptr;            // base of this rank's allocation
    void* peer_base[kTpMaxWorld] = {};
    size_t bytes = 0;
    bool connected = false;
};
TpHost g_tp;

// allocation: [counters kTpMaxCtas u32][error word, padded to 256 B][slots: 2 parities x world x rows_cap x 8 B]
constexpr size_t kCounterBytes = kTpMaxCtas * sizeof(unsigned);
constexpr size_t kErrOffset = kCounterBytes;
constexpr size_t kBufOffset = kCounterBytes + 256;

void fill_rank(TpDev& d, int r, void* base) {
    d.ll[r] = reinterpret_cast<uint2*>(static_cast<unsigned char*>(base) + kBufOffset);
}
}  // namespace

const TpDev& tp_device_ctx() {
    static const TpDev none = {};
    return g_tp.connected ? g_tp.dev : none;
}

}  // namespace nve

using namespace nve;

extern "C" int nve_b200_tp_create(int rank, int world, int max_rows, void* handle_out) {
    if (world < 2 || world > kTpMaxWorld || rank < 0 || rank >= world || max_rows <= 0 || handle_out == nullptr)
        return set_status(NVE_ERR_BAD_SHAPE);
    if (g_tp.local != nullptr) return set_status(NVE_ERR_BAD_SHAPE);  // one context per process
    const size_t bytes = kBufOffset + 2 * static_cast<size_t>(world) * max_rows * sizeof(uint2);
    void* base = nullptr;
    cudaError_t e = cudaMalloc(&base, bytes);
    if (e == cudaSuccess) e = cudaMemset(base, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, base);
    if (e != cudaSuccess) {
        if (base) cudaFree(base);
        return set_cuda_status(e);
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    memcpy(handle_out, &h, 64);
    g_tp.local = base;
    g_tp.bytes = bytes;
    g_tp.dev = {};
    g_tp.dev.world = world;
    g_tp.dev.rank = rank;
    g_tp.dev.rows_cap = max_rows;
    g_tp.dev.err = reinterpret_cast<int*>(static_cast<unsigned char*>(base) + kErrOffset);
    g_tp.dev.counter = reinterpret_cast<unsigned*>(base);
    fill_rank(g_tp.dev, rank, base);
    return set_status(NVE_OK);
}

extern "C" int nve_b200_tp_connect(const void* handles) {
    if (g_tp.local == nullptr || handles == nullptr) return set_status(NVE_ERR_BAD_POINTER);
    const unsigned char* hb = static_cast<const unsigned char*>(handles);
    for (int r = 0; r < g_tp.dev.world; r++) {
        if (r == g_tp.dev.rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, hb + 64 * r, 64);
        void* base = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return set_cuda_status(e);
        g_tp.peer_base[r] = base;
        fill_rank(g_tp.dev, r, base);
    }
    g_tp.connected = true;
    return set_status(NVE_OK);
}

extern "C" int nve_b200_tp_world(void) { return g_tp.connected ? g_tp.dev.world : 0; }

extern "C" int nve_b200_tp_error(int reset) {
    if (g_tp.local == nullptr) return 0;
    int v = 0;
    cudaError_t e = cudaMemcpy(&v, g_tp.dev.err, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { set_cuda_status(e); return -1; }
    if (reset && v != 0) cudaMemset(g_tp.dev.err, 0, sizeof(int));
    return v;
}

extern "C" int nve_b200_tp_destroy(void) {
    if (g_tp.local == nullptr) return set_status(NVE_OK);
    cudaDeviceSynchronize();
    for (int r = 0; r < kTpMaxWorld; r++) {
        if (g_tp.peer_base[r] != nullptr) {
            cudaIpcCloseMemHandle(g_tp.peer_base[r]);
            g_tp.peer_base[r] = nullptr;
        }
    }
    cudaFree(g_tp.local);
    g_tp = TpHost();
    return set_status(NVE_OK);
}
