// Stand-alone microbenchmark (not part of libnve_kernels.so): the load pattern of the W4 GEMV (one 16-byte nibble
// load and one 4-byte scale load per lane and quantisation block, two rows x four column sets per warp item, 296
// CTAs of 256 threads, register double buffering) with the arithmetic replaced by a dial of dependent integer
// instructions per block.  Shows at how many instructions per block the kernel stops being bound by HBM and starts
// being bound by instruction issue.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o gemv_load_pattern gemv_load_pattern.cu && ./gemv_load_pattern
#include <cstdio>
#include <cuda_runtime.h>
#include <stdint.h>
__device__ __forceinline__ unsigned long long gt() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ uint4 ldnc(const void* p) { uint4 v; asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x),"=r"(v.y),"=r"(v.z),"=r"(v.w) : "l"(p)); return v; }
__device__ __forceinline__ float ldf(const void* p) { float v; asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p)); return v; }
// N rows x K: nibbles [N, K/2], scales [N, K/32] f32; 296 CTAs x 256 threads; item = 2 rows x 4 column sets
template <int WORK, bool SCALES> __global__ void __launch_bounds__(256, 2) k(const unsigned char* nib, const float* sc, int N, int K, unsigned long long* out, float* sink) {
    const int nb = K / 32, S = nb / 32, CG = S / 4;
    const int tiles = N / 2;
    const int tb = (long long)tiles * blockIdx.x / gridDim.x, te = (long long)tiles * (blockIdx.x + 1) / gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned long long t0 = gt();
    float acc = 0.f;
    const int items = (te - tb) * CG;
    uint4 w[8]; float s[8];
    auto load = [&](int q) {
        const int t = tb + q / CG, cg = q % CG;
        #pragma unroll
        for (int r = 0; r < 2; r++) {
            const long long b0 = (long long)(t * 2 + r) * nb + cg * 128 + lane;
            #pragma unroll
            for (int c = 0; c < 4; c++) {
                w[c * 2 + r] = ldnc(nib + (b0 + c * 32) * 16);
                if (SCALES) s[c * 2 + r] = ldf(sc + b0 + c * 32); else s[c*2+r] = 1.f;
            }
        }
    };
    int q = warp;
    if (q < items) load(q);
    while (q < items) {
        float a = 0.f;
        #pragma unroll
        for (int j = 0; j < 8; j++) {
            unsigned x = w[j].x ^ w[j].y ^ w[j].z ^ w[j].w;
            #pragma unroll
            for (int i = 0; i < WORK; i++) x = __dp4a((int)x, 0x01020304, (int)(x >> 3)) ^ (x & 0x0F0F0F0Fu);
            a += s[j] * (float)(int)x;
        }
        q += 8;
        if (q < items) load(q);
        #pragma unroll
        for (int m = 16; m > 0; m >>= 1) a += __shfl_xor_sync(0xffffffffu, a, m);
        acc += a;
    }
    __syncthreads();
    unsigned long long t1 = gt();
    if (threadIdx.x == 0) out[blockIdx.x] = t1 - t0;
    if (acc == 1234.5f) *sink = acc;
}
template <int WORK, bool SCALES> void run(const char* name, unsigned char* nib, float* sc, int N, int K, int layers, unsigned long long* out, float* sink) {
    size_t nbytes = (size_t)N * K / 2, sbytes = (size_t)N * K / 32 * 4;
    double best = 1e9;
    unsigned long long h[296];
    for (int rep = 0; rep < 3; rep++) for (int l = 0; l < layers; l++) {
        k<WORK, SCALES><<<296, 256>>>(nib + l * nbytes, sc + l * (sbytes / 4), N, K, out, sink);
        cudaDeviceSynchronize();
        cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
        unsigned long long mx = 0; for (int i = 0; i < 296; i++) if (h[i] > mx) mx = h[i];
        if (mx < best) best = mx;
    }
    double bytes = nbytes + (SCALES ? sbytes : 0);
    printf("%-28s N=%d K=%d: %.2f us  %.0f GB/s\n", name, N, K, best / 1e3, bytes / best);
}
int main() {
    const int N = 28672, K = 4096, layers = 4;
    unsigned char* nib; float* sc; cudaMalloc(&nib, (size_t)N * K / 2 * layers); cudaMalloc(&sc, (size_t)N * K / 32 * 4 * layers);
    cudaMemset(nib, 0x55, (size_t)N * K / 2 * layers); cudaMemset(sc, 0, (size_t)N * K / 32 * 4 * layers);
    unsigned long long* out; cudaMalloc(&out, 296 * 8); float* sink; cudaMalloc(&sink, 4);
    run<0, true>("loads only (nib+scales)", nib, sc, N, K, layers, out, sink);
    run<0, false>("loads only (nibbles)", nib, sc, N, K, layers, out, sink);
    run<4, true>("+ ~10 instr per block", nib, sc, N, K, layers, out, sink);
    run<12, true>("+ ~30 instr per block", nib, sc, N, K, layers, out, sink);
    run<20, true>("+ ~50 instr per block", nib, sc, N, K, layers, out, sink);
    printf("%s\n", cudaGetErrorString(cudaGetLastError()));
    return 0;
}
