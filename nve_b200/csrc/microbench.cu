// Standalone kernel microbenchmark behind the reference's nve_run_microbench entry point
// (cuda/nve_kernels.cu:1306-1413): event-timed loops over the decode kernels for one model shape, printed
// as microseconds per call.  Unlike the reference it also times the quantized GEMVs and reports the
// algorithmic GB/s of each (weights that fit in L2 are re-read from L2, which the printout says).
#include <stdio.h>

#include <vector>

#include "common.cuh"

namespace {

struct DevBuf {
    void* p = nullptr;
    explicit DevBuf(size_t bytes) {
        if (cudaMalloc(&p, bytes) != cudaSuccess) p = nullptr;
        else cudaMemset(p, 0x11, bytes);
    }
    ~DevBuf() { if (p) cudaFree(p); }
    template <typename T> T* as() const { return static_cast<T*>(p); }
};

template <typename F> float time_us(F&& fn, int iters, cudaStream_t st) {
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    for (int i = 0; i < 3; i++) fn();
    cudaEventRecord(a, st);
    for (int i = 0; i < iters; i++) fn();
    cudaEventRecord(b, st);
    cudaEventSynchronize(b);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    return ms * 1000.0f / static_cast<float>(iters);
}

}  // namespace

extern "C" void nve_run_microbench(int hidden, int intermediate, int num_heads, int num_kv_heads, int head_dim, int iters) {
    if (hidden <= 0 || intermediate <= 0 || num_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || iters <= 0 ||
        (hidden % 32) != 0 || (intermediate % 32) != 0) {
        printf("nve_run_microbench: unsupported shape\n");
        return;
    }
    cudaStream_t st = nullptr;
    const size_t N = static_cast<size_t>(intermediate), K = static_cast<size_t>(hidden);
    DevBuf x(K * 2), w(K * 2), o(N * 2 > K * 2 ? N * 2 : K * 2), xq(K), xs(K / 32 * 4);
    DevBuf nib(N * K / 2), sc(N * K / 32 * 4), dense(N * K * 2);
    DevBuf q(static_cast<size_t>(num_heads) * head_dim * 2), k(static_cast<size_t>(num_kv_heads) * head_dim * 2),
        cs(static_cast<size_t>(head_dim)), sn(static_cast<size_t>(head_dim));
    if (!x.p || !w.p || !o.p || !xq.p || !xs.p || !nib.p || !sc.p || !dense.p || !q.p || !k.p || !cs.p || !sn.p) {
        printf("nve_run_microbench: allocation failed\n");
        return;
    }
    cudaMemset(x.p, 0, K * 2);
    cudaMemset(sc.p, 0, N * K / 32 * 4);
    cudaMemset(xs.p, 0, K / 32 * 4);

    const double w4_bytes = static_cast<double>(N) * K * 0.625;
    const float t_norm = time_us([&] { nve_rms_norm_f16(x.as<uint16_t>(), w.as<uint16_t>(), o.as<uint16_t>(), hidden, 1e-5f, st); }, iters, st);
    const float t_rope = time_us([&] { nve_rope_f16_decode(q.as<uint16_t>(), k.as<uint16_t>(), cs.as<uint16_t>(), sn.as<uint16_t>(), num_heads, num_kv_heads, head_dim, st); }, iters, st);
    const float t_f16 = time_us([&] { nve_matvec_f16(x.as<uint16_t>(), dense.as<uint16_t>(), o.as<uint16_t>(), intermediate, hidden, st); }, iters, st);
    const float t_q8 = time_us([&] { nve_quantize_f16_q8(x.as<uint16_t>(), xq.as<int8_t>(), xs.as<float>(), hidden, st); }, iters, st);
    const float t_w4a8 = time_us([&] { nve_matvec_w4a8(xq.as<int8_t>(), xs.as<float>(), nib.as<uint8_t>(), sc.as<float>(), o.as<uint16_t>(), intermediate, hidden, st); }, iters, st);
    const float t_w4a16 = time_us([&] { nve_matvec_w4a16(x.as<uint16_t>(), nib.as<uint8_t>(), sc.as<float>(), nullptr, o.as<uint16_t>(), intermediate, hidden, st); }, iters, st);
    cudaError_t e = cudaDeviceSynchronize();

    printf("nve microbench (hidden=%d intermediate=%d heads=%d/%d head_dim=%d iters=%d)%s\n", hidden, intermediate,
           num_heads, num_kv_heads, head_dim, iters, e == cudaSuccess ? "" : "  [CUDA error]");
    printf("  rms_norm_f16        %9.3f us/call\n", t_norm);
    printf("  rope_f16_decode     %9.3f us/call\n", t_rope);
    printf("  quantize_f16_q8     %9.3f us/call\n", t_q8);
    printf("  matvec_f16  [%dx%d] %9.3f us/call  %8.1f GB/s\n", intermediate, hidden, t_f16, N * K * 2.0 / t_f16 * 1e-3);
    printf("  matvec_w4a8 [%dx%d] %9.3f us/call  %8.1f GB/s\n", intermediate, hidden, t_w4a8, w4_bytes / t_w4a8 * 1e-3);
    printf("  matvec_w4a16[%dx%d] %9.3f us/call  %8.1f GB/s\n", intermediate, hidden, t_w4a16, w4_bytes / t_w4a16 * 1e-3);
    printf("  (one matrix re-read every call: a matrix smaller than the L2 cache is served from L2, not HBM)\n");
    fflush(stdout);
}
