// Host-side runtime of libnve_kernels.so: status bookkeeping, device queries, the process-global
// decode-graph manager and the device-to-device copy helper.
//
// The graph manager keeps the protocol of cuda/nve_kernels.cu:1230-1299 of the reference project
// (init / begin_capture / end_capture / launch / ready / destroy, pinned pos and seq_len scalars copied
// to device scalars by the first two nodes of the captured graph) so that src/decode_graph.rs can drive
// it unchanged.
#include <atomic>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"

namespace nve {

static thread_local int t_status = NVE_OK;
static thread_local int t_cuda_error = 0;
static std::atomic<unsigned long long> g_launches{0};
static std::atomic<int> g_pdl{0};

int set_status(int code) {
    t_status = code;
    return code;
}

int set_cuda_status(cudaError_t err) {
    if (err == cudaSuccess) return set_status(NVE_OK);
    t_cuda_error = static_cast<int>(err);
    return set_status(NVE_ERR_CUDA);
}

void count_launch(int n) { g_launches.fetch_add(static_cast<unsigned long long>(n), std::memory_order_relaxed); }

bool pdl_enabled() { return g_pdl.load(std::memory_order_relaxed) != 0; }

int check_launch() { return set_cuda_status(cudaPeekAtLastError()); }

int sm_count() {
    static std::mutex mu;
    static int cached[64];
    static bool have[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
        have[dev] = true;
    }
    return cached[dev];
}

int ensure_dynamic_smem(const void* kernel, int bytes) {
    static std::mutex mu;
    static std::vector<std::pair<int, const void*>> done;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_cuda_status(e);
    std::lock_guard<std::mutex> lock(mu);
    for (const auto& d : done)
        if (d.first == dev && d.second == kernel) return NVE_OK;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return set_cuda_status(e);
    done.emplace_back(dev, kernel);
    return NVE_OK;
}

}  // namespace nve

using namespace nve;

extern "C" int nve_b200_last_status(void) { return t_status; }
extern "C" int nve_b200_last_cuda_error(void) { return t_cuda_error; }
extern "C" const char* nve_b200_version(void) { return "nve-b200 0.1 sm_100a"; }
extern "C" unsigned long long nve_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
extern "C" int nve_b200_set_pdl(int enabled) { return g_pdl.exchange(enabled ? 1 : 0); }

extern "C" void nve_d2d_copy(void* dst, const void* src, size_t bytes, nve_stream_t stream) {
    set_cuda_status(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
}

// ---------------------------------------------------------------------------------------------
// Decode-graph manager
// ---------------------------------------------------------------------------------------------
namespace {
struct GraphState {
    cudaGraphExec_t exec = nullptr;
    cudaStream_t cap_stream = nullptr;
    int* pin_pos = nullptr;
    int* pin_seqlen = nullptr;
    int* dev_pos = nullptr;
    int* dev_seqlen = nullptr;
    int ready = 0;
    bool capturing = false;
    unsigned long long launches_at_begin = 0;
    unsigned long long kernels_in_graph = 0;
};
GraphState g_graph;
}  // namespace

extern "C" void nve_graph_init(void) {
    GraphState& g = g_graph;
    if (g.cap_stream != nullptr) return;  // idempotent
    cudaError_t e = cudaStreamCreateWithFlags(&g.cap_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMallocHost(reinterpret_cast<void**>(&g.pin_pos), sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost(reinterpret_cast<void**>(&g.pin_seqlen), sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&g.dev_pos), sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&g.dev_seqlen), sizeof(int));
    if (e == cudaSuccess) {
        *g.pin_pos = 0;
        *g.pin_seqlen = 1;
        e = cudaMemset(g.dev_pos, 0, sizeof(int));
    }
    if (e == cudaSuccess) {
        const int one = 1;
        e = cudaMemcpy(g.dev_seqlen, &one, sizeof(int), cudaMemcpyHostToDevice);
    }
    g.ready = 0;
    set_cuda_status(e);
}

extern "C" const int* nve_graph_d_pos(void) { return g_graph.dev_pos; }
extern "C" const int* nve_graph_d_seqlen(void) { return g_graph.dev_seqlen; }
extern "C" nve_stream_t nve_graph_capture_stream(void) { return g_graph.cap_stream; }

extern "C" void nve_graph_begin_capture(void) {
    GraphState& g = g_graph;
    g.ready = 0;
    if (g.cap_stream == nullptr) {
        set_status(NVE_ERR_BAD_POINTER);
        return;
    }
    cudaError_t e = cudaStreamSynchronize(g.cap_stream);
    // Thread-local capture mode: other threads of the host program may keep using CUDA while this
    // thread records; calls made by the capturing thread itself are checked exactly as in global mode.
    if (e == cudaSuccess) e = cudaStreamBeginCapture(g.cap_stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
        g.capturing = true;
        g.launches_at_begin = g_launches.load(std::memory_order_relaxed);
        // The scalar copies are the first nodes, so every replay starts by refreshing pos / seq_len.
        e = cudaMemcpyAsync(g.dev_pos, g.pin_pos, sizeof(int), cudaMemcpyHostToDevice, g.cap_stream);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(g.dev_seqlen, g.pin_seqlen, sizeof(int), cudaMemcpyHostToDevice, g.cap_stream);
    }
    set_cuda_status(e);
}

extern "C" void nve_graph_end_capture(void) {
    GraphState& g = g_graph;
    if (g.exec != nullptr) {
        cudaGraphExecDestroy(g.exec);
        g.exec = nullptr;
    }
    if (!g.capturing) {
        set_status(NVE_ERR_BAD_SHAPE);
        return;
    }
    g.capturing = false;
    g.kernels_in_graph = g_launches.load(std::memory_order_relaxed) - g.launches_at_begin;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(g.cap_stream, &graph);
    if (e == cudaSuccess && graph != nullptr) {
        e = cudaGraphInstantiate(&g.exec, graph, 0);
        cudaGraphDestroy(graph);
    }
    g.ready = (e == cudaSuccess && g.exec != nullptr) ? 1 : 0;
    set_cuda_status(e);
}

extern "C" void nve_graph_launch(int pos, int seq_len, nve_stream_t stream) {
    GraphState& g = g_graph;
    if (!g.ready || g.exec == nullptr) {  // the reference silently skips (cuda/nve_kernels.cu:1281)
        set_status(NVE_ERR_BAD_SHAPE);
        return;
    }
    *g.pin_pos = pos;
    *g.pin_seqlen = seq_len;
    // every replay runs the kernels recorded between begin_capture and end_capture
    count_launch(static_cast<int>(g.kernels_in_graph));
    set_cuda_status(cudaGraphLaunch(g.exec, static_cast<cudaStream_t>(stream)));
}

extern "C" int nve_graph_ready(void) { return g_graph.ready; }

extern "C" void nve_graph_destroy(void) {
    GraphState& g = g_graph;
    g.ready = 0;
    if (g.exec) { cudaGraphExecDestroy(g.exec); g.exec = nullptr; }
    if (g.cap_stream) { cudaStreamDestroy(g.cap_stream); g.cap_stream = nullptr; }
    if (g.pin_pos) { cudaFreeHost(g.pin_pos); g.pin_pos = nullptr; }
    if (g.pin_seqlen) { cudaFreeHost(g.pin_seqlen); g.pin_seqlen = nullptr; }
    if (g.dev_pos) { cudaFree(g.dev_pos); g.dev_pos = nullptr; }
    if (g.dev_seqlen) { cudaFree(g.dev_seqlen); g.dev_seqlen = nullptr; }
    g.capturing = false;
}
