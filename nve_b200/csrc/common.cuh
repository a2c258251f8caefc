// Shared device/host helpers for the sm_100a kernels of libnve_kernels.so.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nve_kernels.h"

namespace nve {

constexpr int kWarp = 32;
constexpr int kBlockK = 32;  // weights per quantisation block (src/quantize.rs:20)

// ---------------------------------------------------------------------------------------------
// Host-side status bookkeeping (defined in runtime.cu)
// ---------------------------------------------------------------------------------------------
int set_status(int code);                 // records and returns `code`
int set_cuda_status(cudaError_t err);     // records NVE_ERR_CUDA (or NVE_OK) and returns it
void count_launch(int n = 1);             // bumps the process-wide launch counter
int sm_count();                           // multiprocessors of the current device (cached per device)
bool pdl_enabled();
int check_launch();                       // cudaPeekAtLastError -> status
// Raise a kernel's dynamic shared-memory limit to `bytes` once per (device, kernel); legal during capture.
int ensure_dynamic_smem(const void* kernel, int bytes);

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// ---------------------------------------------------------------------------------------------
// 16-bit activation types
// ---------------------------------------------------------------------------------------------
template <int DT> struct Act16;
template <> struct Act16<NVE_DT_F16> {
    using T = __half;
    __device__ static __forceinline__ float to_f32(uint16_t v) { return __half2float(__ushort_as_half(v)); }
    __device__ static __forceinline__ uint16_t from_f32(float v) { return __half_as_ushort(__float2half_rn(v)); }
};
template <> struct Act16<NVE_DT_BF16> {
    using T = __nv_bfloat16;
    __device__ static __forceinline__ float to_f32(uint16_t v) { return __uint_as_float(static_cast<uint32_t>(v) << 16); }
    __device__ static __forceinline__ uint16_t from_f32(float v) {
        return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    }
};

// Store one result element in the requested output type.
template <int DT> __device__ __forceinline__ void store_out(void* base, long long i, float v);
template <> __device__ __forceinline__ void store_out<NVE_DT_F16>(void* base, long long i, float v) {
    static_cast<uint16_t*>(base)[i] = Act16<NVE_DT_F16>::from_f32(v);
}
template <> __device__ __forceinline__ void store_out<NVE_DT_BF16>(void* base, long long i, float v) {
    static_cast<uint16_t*>(base)[i] = Act16<NVE_DT_BF16>::from_f32(v);
}
template <> __device__ __forceinline__ void store_out<NVE_DT_F32>(void* base, long long i, float v) {
    static_cast<float*>(base)[i] = v;
}
template <int DT> __device__ __forceinline__ float load_out(const void* base, long long i);
template <> __device__ __forceinline__ float load_out<NVE_DT_F16>(const void* base, long long i) {
    return Act16<NVE_DT_F16>::to_f32(static_cast<const uint16_t*>(base)[i]);
}
template <> __device__ __forceinline__ float load_out<NVE_DT_BF16>(const void* base, long long i) {
    return Act16<NVE_DT_BF16>::to_f32(static_cast<const uint16_t*>(base)[i]);
}
template <> __device__ __forceinline__ float load_out<NVE_DT_F32>(const void* base, long long i) {
    return static_cast<const float*>(base)[i];
}

// ---------------------------------------------------------------------------------------------
// Loads
// ---------------------------------------------------------------------------------------------
// 128-bit streaming load of read-once weight data: no L1 allocation, so the activations stay cached.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_stream_f32(const void* p) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// The same loads at a compile-time byte offset from a base address: the offset goes into the instruction's immediate
// field, so the loads of one row of an item share one 64-bit address computation.
template <int OFF> __device__ __forceinline__ uint4 ld_stream_u4_off(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p), "n"(OFF));
    return v;
}
template <int OFF> __device__ __forceinline__ float ld_stream_f32_off(const void* p) {
    float v;
    asm volatile("ld.global.nc.L1::no_allocate.f32 %0, [%1+%2];" : "=f"(v) : "l"(p), "n"(OFF));
    return v;
}

// dp4a with an unsigned first operand (raw nibbles 0..15) and a signed second operand (int8 codes).
__device__ __forceinline__ int dp4a_us(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// System-scope 8-byte accesses for slots that another GPU writes over NVLink (peer mappings): value (low word) and
// epoch (high word) travel in ONE aligned 64-bit access, which is single-copy atomic, so the reader needs no
// separate flag and can never pair a new epoch with an old value.
__device__ __forceinline__ void st_relaxed_sys_slot(uint2* p, uint32_t value, uint32_t epoch) {
    const unsigned long long w = (static_cast<unsigned long long>(epoch) << 32) | value;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_relaxed_sys_slot(const uint2* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2(static_cast<uint32_t>(w), static_cast<uint32_t>(w >> 32));
}

// Programmatic dependent launch: wait for the producer grid's memory / allow the consumer grid to start.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------
// Warp reductions with a fixed, documented order (xor butterfly 16, 8, 4, 2, 1).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}

// Sum R per-lane values across the warp, R a power of two <= 32.  On return a[0] of lane L holds the
// total of row multi_row_of<R>(L).  Every row's total is the same balanced tree over lanes
// (pairs L^16, then ^8, ^4, ^2, ^1), so the result does not depend on R.
template <int R> __device__ __forceinline__ void warp_sum_multi(float (&a)[R], int lane) {
    int m = 16;
#pragma unroll
    for (int n = R; n > 1; n >>= 1) {
        const int half = n >> 1;
        const bool up = (lane & m) != 0;
#pragma unroll
        for (int i = 0; i < half; i++) {
            float send = up ? a[i] : a[i + half];
            float keep = up ? a[i + half] : a[i];
            a[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
        }
        m >>= 1;
    }
    for (; m > 0; m >>= 1) a[0] += __shfl_xor_sync(0xffffffffu, a[0], m);
}
// Row whose total lane L holds after warp_sum_multi<R>.
template <int R> __device__ __forceinline__ int multi_row_of(int lane) {
    int row = 0;
    int m = 16;
#pragma unroll
    for (int n = R; n > 1; n >>= 1) {
        row = row + ((lane & m) ? (n >> 1) : 0);
        m >>= 1;
    }
    return row;
}
// True on exactly one lane per row (the lowest lane holding that row).
template <int R> __device__ __forceinline__ bool multi_row_writer(int lane) {
    constexpr int kLowMask = (32 / R) - 1;
    return (lane & kLowMask) == 0;
}

// ---------------------------------------------------------------------------------------------
// Counter-based synthetic generator (same integer recipe as the test oracle).
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
constexpr unsigned long long kGolden = 0x9E3779B97F4A7C15ull;
constexpr unsigned long long kStreamMul = 0xD6E8FEB86659FD93ull;
__host__ __device__ __forceinline__ unsigned long long gen_state(unsigned long long seed, unsigned long long stream_id) {
    return mix64(seed ^ (stream_id * kStreamMul));
}
__host__ __device__ __forceinline__ float gen_normal(unsigned long long st, unsigned long long i) {
    unsigned long long a = mix64(st + (2 * i + 1) * kGolden);
    unsigned long long b = mix64(st + (2 * i + 2) * kGolden);
    int s = 0;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        s += static_cast<int>((a >> (16 * j)) & 0xFFFFull);
        s += static_cast<int>((b >> (16 * j)) & 0xFFFFull);
    }
    // 0x1.3988e2p-16f = 1/sqrt(8*(65536^2-1)/12): unit variance for a sum of eight uniform u16
    return static_cast<float>(s - 262140) * 0x1.3988e2p-16f;
}

// 16-bit fixed point of one 32-wide group held by the 4 threads of a quad (8 values each): v = rint(x * 32767 / amax),
// split into an unsigned low-byte plane and a signed high-byte plane (the form the W4A16 GEMV multiplies with dp4a).
// Returns the group's scale; `sum` is the sum of the group's 32 codes.
__device__ __forceinline__ float x16_quad_convert(const float (&xe)[8], uint32_t& l0, uint32_t& l1, uint32_t& h0, uint32_t& h1,
                                                  int& sum) {
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(xe[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float scale = amax > 0.0f ? __fdiv_rn(amax, 32767.0f) : 1.0f;
    if (!(amax <= 3.0e38f)) scale = __int_as_float(0x7FC00000);
    const float inv = __fdiv_rn(1.0f, scale);
    l0 = l1 = h0 = h1 = 0;
    sum = 0;
#pragma unroll
    for (int e = 0; e < 8; e++) {
        int q = __float2int_rn(__fmul_rn(xe[e], inv));
        q = max(-32767, min(32767, q));
        sum += q;
        const uint32_t lo8 = static_cast<uint32_t>(q) & 0xFFu;
        const uint32_t hi8 = static_cast<uint32_t>(q >> 8) & 0xFFu;
        if (e < 4) { l0 |= lo8 << (8 * e); h0 |= hi8 << (8 * e); }
        else { l1 |= lo8 << (8 * (e - 4)); h1 |= hi8 << (8 * (e - 4)); }
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    return scale;
}

}  // namespace nve
