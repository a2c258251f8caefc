// Stand-alone microbenchmark (not part of libnve_kernels.so): cost of a device-wide barrier over one 512-thread CTA per
// SM (cooperative launch), for the variants considered for the persistent decode step.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o grid_barrier grid_barrier.cu && ./grid_barrier
//
// mode 0: arrival counter, red.release + ld.acquire polling (the form decode_step.cu uses); 1: + nanosleep backoff;
// 2: relaxed polling + fence; 3: sense reversal, generation flag on its own line; 4: 3 + backoff; 5: two-level tree.
// work 0: barriers back to back; work 10: 0.2 - 1.2 us of skewed spinning per CTA between barriers.
// Every run is bounded by its iteration count; nothing waits on a flag that is never set.
#include <cstdio>
#include <cuda_runtime.h>
#include <stdint.h>
__device__ __forceinline__ unsigned long long gt() { unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ unsigned long long ldacq(const unsigned long long* p) { unsigned long long v; asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ unsigned long long ldrlx(const unsigned long long* p) { unsigned long long v; asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void redrel(unsigned long long* p) { asm volatile("red.release.gpu.global.add.u64 [%0], 1;" :: "l"(p) : "memory"); }
__device__ __forceinline__ unsigned long long atomrel(unsigned long long* p) { unsigned long long v; asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], 1;" : "=l"(v) : "l"(p) : "memory"); return v; }
__device__ __forceinline__ void strel(unsigned long long* p, unsigned long long v) { asm volatile("st.release.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory"); }

template <int MODE> __device__ __forceinline__ void barrier(unsigned long long* ctr, unsigned long long* flag, unsigned long long& target, unsigned long long& gen) {
    __syncthreads();
    if (threadIdx.x == 0) {
        if (MODE == 0) { target += gridDim.x; redrel(ctr); while (ldacq(ctr) < target) {} }
        if (MODE == 1) { target += gridDim.x; redrel(ctr); while (ldacq(ctr) < target) { __nanosleep(40); } }
        if (MODE == 2) { target += gridDim.x; redrel(ctr); while (ldrlx(ctr) < target) { } __threadfence(); }
        if (MODE == 3) {  // sense reversal: last arriver publishes the generation on another line
            gen++; target += gridDim.x;
            unsigned long long old = atomrel(ctr);
            if (old + 1 == target) strel(flag, gen);
            else while (ldacq(flag) < gen) {}
        }
        if (MODE == 4) {  // as 3 with backoff
            gen++; target += gridDim.x;
            unsigned long long old = atomrel(ctr);
            if (old + 1 == target) strel(flag, gen);
            else while (ldacq(flag) < gen) { __nanosleep(40); }
        }
        if (MODE == 5) {  // two-level: 8 group counters on separate lines, then root
            // group g = blockIdx.x % 8 ; ctr[g*32] ; root ctr[8*32]
            gen++;
            const int grp = blockIdx.x & 7;
            const unsigned gsize = (gridDim.x + 7 - grp) / 8;
            unsigned long long old = atomrel(ctr + grp * 32);
            if (old + 1 == gen * gsize) {
                unsigned long long o2 = atomrel(ctr + 8 * 32);
                if (o2 + 1 == gen * 8) strel(flag, gen);
            }
            while (ldacq(flag) < gen) {}
        }
    }
    __syncthreads();
}
template <int MODE> __global__ void __launch_bounds__(512,1) k(unsigned long long* ctr, unsigned long long* flag, int iters, unsigned long long* out, int work) {
    unsigned long long target = 0, gen = 0;
    barrier<MODE>(ctr, flag, target, gen);
    unsigned long long t0 = gt();
    for (int i = 0; i < iters; i++) {
        if (work) { // a little skewed work: spin blockIdx-dependent
            unsigned long long s = gt(); while (gt() - s < (unsigned)(200 + (blockIdx.x * 37 % 100) * work)) {}
        }
        barrier<MODE>(ctr, flag, target, gen);
    }
    unsigned long long t1 = gt();
    if (threadIdx.x == 0 && blockIdx.x == 0) out[0] = t1 - t0;
}
template <int MODE> void run(unsigned long long* mem, unsigned long long* out, int work) {
    cudaMemset(mem, 0, 8192);
    void* args[] = {&mem, nullptr, nullptr, &out, &work};
    unsigned long long* flag = mem + 512; int iters = 200;
    args[1] = &flag; args[2] = &iters;
    cudaError_t e = cudaLaunchCooperativeKernel((void*)k<MODE>, dim3(148), dim3(512), args, 0, 0);
    cudaDeviceSynchronize();
    unsigned long long h; cudaMemcpy(&h, out, 8, cudaMemcpyDeviceToHost);
    printf("mode %d work %d: %.2f us per barrier (%s)\n", MODE, work, h / 1e3 / iters, cudaGetErrorString(e == cudaSuccess ? cudaGetLastError() : e));
}
int main() {
    unsigned long long* mem; cudaMalloc(&mem, 8192); unsigned long long* out; cudaMalloc(&out, 64);
    for (int work : {0, 10}) {
        run<0>(mem, out, work); run<1>(mem, out, work); run<2>(mem, out, work); run<3>(mem, out, work); run<4>(mem, out, work); run<5>(mem, out, work);
    }
    return 0;
}
