// Stand-alone microbenchmark (not part of libnve_kernels.so): how fast does a GEMV-like read stream run from DRAM and
// from an L2-resident region on this GPU, and what does an L2 prefetch issued earlier / at the same time do to it?
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o l2_prefetch_stream l2_prefetch_stream.cu && ./l2_prefetch_stream
//
// One CTA of 512 threads per SM; every warp keeps 8 x 16 bytes per lane in flight (512 contiguous bytes per warp
// load), the access pattern of the W4 GEMV without its arithmetic.  Regions rotate through a 1 GiB arena so that
// nothing is L2-resident by accident.  mode 0: no prefetch; 1: cp.async.bulk.prefetch.L2; 2: prefetch.global.L2 per
// 128-byte line; `wait` is the time between issuing the prefetch and starting the read.
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include <stdint.h>
__device__ __forceinline__ unsigned long long gt() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ uint4 ldnc(const void* p) { uint4 v; asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x),"=r"(v.y),"=r"(v.z),"=r"(v.w) : "l"(p)); return v; }
// mode 0: no prefetch; 1: bulk prefetch; 2: per-line prefetch.global.L2
__global__ void __launch_bounds__(512,1) k(const unsigned char* buf, size_t bytes, int mode, unsigned wait_ns, unsigned long long* out, unsigned* sink) {
    const size_t per = bytes / gridDim.x;   // multiple of 8192 assumed
    const unsigned char* mine = buf + per * blockIdx.x;
    unsigned long long t0 = gt();
    if (mode == 1) {
        if (threadIdx.x < 16) {
            size_t chunk = per / 16;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" :: "l"(mine + chunk * threadIdx.x), "r"((unsigned)chunk) : "memory");
        }
    } else if (mode == 2) {
        for (size_t o = (size_t)threadIdx.x * 128; o < per; o += 512 * 128)
            asm volatile("prefetch.global.L2 [%0];" :: "l"(mine + o));
    }
    while (gt() - t0 < wait_ns) { }
    __syncthreads();
    unsigned long long t1 = gt();
    unsigned acc = 0;
    // each thread: 8 x 16B loads in flight per iteration, coalesced 512B per warp-load
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (size_t o = (size_t)warp * 4096; o < per; o += 16 * 4096) {
        uint4 v[8];
        #pragma unroll
        for (int j = 0; j < 8; j++) v[j] = ldnc(mine + o + j * 512 + lane * 16);
        #pragma unroll
        for (int j = 0; j < 8; j++) acc += v[j].x ^ v[j].y ^ v[j].z ^ v[j].w;
    }
    __syncthreads();
    unsigned long long t2 = gt();
    if (threadIdx.x == 0) { out[blockIdx.x * 2] = t1 - t0; out[blockIdx.x * 2 + 1] = t2 - t1; }
    if (acc == 0x12345678u) *sink = acc;
}
int main() {
    const size_t total = 1ull << 30;   // 1 GiB arena, rotate regions so nothing is L2-resident by accident
    unsigned char* buf; cudaMalloc(&buf, total); cudaMemset(buf, 1, total);
    unsigned long long* out; cudaMalloc(&out, 148 * 16); unsigned* sink; cudaMalloc(&sink, 4);
    unsigned long long h[296];
    size_t region_off = 0;
    for (size_t mb : {8, 16, 32, 64, 96}) {
        size_t bytes = (mb << 20) / (148 * 65536) * (148 * 65536);
        for (int mode = 0; mode < 3; mode++) {
            for (unsigned wait_us : {0u, 10u, 30u}) {
                if (mode == 0 && wait_us) continue;
                double best = 1e9, avgmax = 0; int reps = 5;
                for (int r = 0; r < reps; r++) {
                    region_off = (region_off + (128ull << 20)) % (total - (128ull << 20));
                    k<<<148, 512>>>(buf + region_off, bytes, mode, wait_us * 1000, out, sink);
                    cudaDeviceSynchronize();
                    cudaMemcpy(h, out, 148 * 16, cudaMemcpyDeviceToHost);
                    unsigned long long mx = 0; for (int i = 0; i < 148; i++) if (h[2*i+1] > mx) mx = h[2*i+1];
                    if (mx < best) best = mx; avgmax += mx;
                }
                printf("region %3zu MB mode %d wait %2u us: read phase max-over-CTAs best %.1f us (%.0f GB/s) avg %.1f us\n", mb, mode, wait_us, best / 1e3, bytes / best, avgmax / reps / 1e3);
            }
        }
    }
    cudaError_t e = cudaGetLastError(); printf("status %s\n", cudaGetErrorString(e));
    return 0;
}
