// Element-wise activation arithmetic shared by the stand-alone activation kernels (act_quant.cu) and the
// persistent decode-step kernel (decode_step.cu): int8 group quantisation, the 16-bit fixed-point planes of the
// W4A16 GEMV, SiLU*up.  Every operation that decides an int8 code or a 16-bit result is an IEEE-rounded
// intrinsic in a fixed order, so all users produce the same bits.
#pragma once
#include "common.cuh"

namespace nve {

__device__ __forceinline__ void unpack8(const uint4& raw, uint16_t (&h)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        h[2 * j] = static_cast<uint16_t>(w[j] & 0xFFFFu);
        h[2 * j + 1] = static_cast<uint16_t>(w[j] >> 16);
    }
}
__device__ __forceinline__ uint4 pack8(const uint16_t (&h)[8]) {
    uint4 r;
    r.x = h[0] | (static_cast<uint32_t>(h[1]) << 16);
    r.y = h[2] | (static_cast<uint32_t>(h[3]) << 16);
    r.z = h[4] | (static_cast<uint32_t>(h[5]) << 16);
    r.w = h[6] | (static_cast<uint32_t>(h[7]) << 16);
    return r;
}

// int8 codes of the 8 values of this thread; the 4 threads of a quad hold one 32-wide group.
//   scale = amax > 0 ? amax/127 : 1 ; q = clamp(rint(v * (1/scale)), -127, 127)   (cuda/nve_kernels.cu:712-745)
// With `awq_inv` (the per-column divisor a weight matrix was pre-scaled by, src/quantize.rs:271-304) the values
// are multiplied by it first, so that the W4A8 route sees the same activations as the W4A16 one.
__device__ __forceinline__ float quantize_quad_codes(const float (&v)[8], uint32_t& lo, uint32_t& hi, int& sum) {
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    lo = 0;
    hi = 0;
    sum = 0;
#pragma unroll
    for (int e = 0; e < 8; e++) {
        int q = __float2int_rn(__fmul_rn(v[e], inv));
        q = max(-127, min(127, q));
        sum += q;
        const uint32_t byte = static_cast<uint32_t>(q) & 0xFFu;
        if (e < 4) lo |= byte << (8 * e);
        else hi |= byte << (8 * (e - 4));
    }
    return scale;
}

// Quantise the 8 values of this thread and store codes / scale to global arrays.
__device__ __forceinline__ void quantize_quad(const float (&v)[8], int8_t* xq, float* scales, long long chunk,
                                              bool active) {
    uint32_t lo, hi;
    int sum;
    const float scale = quantize_quad_codes(v, lo, hi, sum);
    if (active) {
        reinterpret_cast<uint2*>(xq)[chunk] = make_uint2(lo, hi);
        if ((chunk & 3) == 0) scales[chunk >> 2] = scale;
    }
}

// Write the 16-bit fixed-point planes of the 8 values of this thread (the 4 threads of a quad hold one group).
__device__ __forceinline__ void x16_quad(const float (&v)[8], uint8_t* xlo, int8_t* xhi, float* scales, long long chunk,
                                         bool active) {
    uint32_t l0, l1, h0, h1;
    int sum;
    const float scale = x16_quad_convert(v, l0, l1, h0, h1, sum);
    if (active) {
        reinterpret_cast<uint2*>(xlo)[chunk] = make_uint2(l0, l1);
        reinterpret_cast<uint2*>(xhi)[chunk] = make_uint2(h0, h1);
        if ((chunk & 3) == 0) scales[chunk >> 2] = scale;
    }
}

__device__ __forceinline__ float silu_mul_f32(float g, float u) {
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), u);
}

}  // namespace nve
