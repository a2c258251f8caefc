// Weight-side helpers: dense f16 GEMV, full dequantisation, on-device Q4 quantisation and repacking,
// and the synthetic input generator.
//
// Replaces cuda/nve_kernels.cu:273-314 (nve_matvec_f16) and :397-433 (nve_dequant_w4a16) of the reference
// project, and moves src/quantize.rs:711-731 (quantize_block_q4) and :437-463 (extract_for_gpu) onto the
// device with bit-identical results.
#include "common.cuh"

namespace nve {

// ---------------------------------------------------------------------------------------------
// Dense f16 GEMV: one warp per row, 128-bit loads when aligned.
// ---------------------------------------------------------------------------------------------
template <bool VEC> __global__ void __launch_bounds__(256) matvec_f16_kernel(const uint16_t* x, const uint16_t* W,
                                                                              uint16_t* out, int N, int K) {
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= N) return;
    const uint16_t* w = W + static_cast<long long>(row) * K;
    float acc = 0.0f;
    if constexpr (VEC) {
        for (int c = lane; c < K / 8; c += 32) {
            const uint4 wv = ld_stream_u4(w + c * 8);
            const uint4 xv = reinterpret_cast<const uint4*>(x)[c];
            const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
            const uint32_t xx[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                acc = fmaf(Act16<NVE_DT_F16>::to_f32(ww[j] & 0xFFFFu), Act16<NVE_DT_F16>::to_f32(xx[j] & 0xFFFFu), acc);
                acc = fmaf(Act16<NVE_DT_F16>::to_f32(ww[j] >> 16), Act16<NVE_DT_F16>::to_f32(xx[j] >> 16), acc);
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(Act16<NVE_DT_F16>::to_f32(w[k]), Act16<NVE_DT_F16>::to_f32(x[k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[row] = Act16<NVE_DT_F16>::from_f32(acc);
}

// ---------------------------------------------------------------------------------------------
// Dequantisation: one thread per 16-byte block -> 32 outputs (4 x 128-bit stores).
// ---------------------------------------------------------------------------------------------
template <int ODT> __global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* nibbles, const float* scales,
                                                                          const float* awq, uint16_t* out,
                                                                          long long total_blocks, int nb) {
    const long long blk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk >= total_blocks) return;
    const uint4 w = ld_stream_u4(nibbles + blk * 16);
    const float sc = scales[blk];
    const int b = static_cast<int>(blk % nb);
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
    uint16_t h[32];
#pragma unroll
    for (int j = 0; j < 4; j++) {
#pragma unroll
        for (int t = 0; t < 4; t++) {
            const int lo = static_cast<int>((wv[j] >> (8 * t)) & 0xFu) - 8;
            const int hi = static_cast<int>((wv[j] >> (8 * t + 4)) & 0xFu) - 8;
            float vlo = __fmul_rn(static_cast<float>(lo), sc);
            float vhi = __fmul_rn(static_cast<float>(hi), sc);
            if (awq != nullptr) {
                vlo = __fmul_rn(vlo, awq[b * 32 + 4 * j + t]);
                vhi = __fmul_rn(vhi, awq[b * 32 + 16 + 4 * j + t]);
            }
            h[4 * j + t] = Act16<ODT>::from_f32(vlo);
            h[16 + 4 * j + t] = Act16<ODT>::from_f32(vhi);
        }
    }
    uint4* dst = reinterpret_cast<uint4*>(out + blk * 32);
#pragma unroll
    for (int v = 0; v < 4; v++) {
        uint4 o;
        o.x = h[8 * v + 0] | (static_cast<uint32_t>(h[8 * v + 1]) << 16);
        o.y = h[8 * v + 2] | (static_cast<uint32_t>(h[8 * v + 3]) << 16);
        o.z = h[8 * v + 4] | (static_cast<uint32_t>(h[8 * v + 5]) << 16);
        o.w = h[8 * v + 6] | (static_cast<uint32_t>(h[8 * v + 7]) << 16);
        dst[v] = o;
    }
}

template <int ODT> __global__ void dequant_scalar_kernel(const uint8_t* nibbles, const float* scales, const float* awq,
                                                          uint16_t* out, long long total, int K) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long blk = i / 32;
    const int pos = static_cast<int>(i % 32);
    const uint8_t bv = nibbles[blk * 16 + (pos & 15)];
    const int nib = (pos < 16) ? (bv & 0xF) : (bv >> 4);
    float v = __fmul_rn(static_cast<float>(nib - 8), scales[blk]);
    if (awq != nullptr) v = __fmul_rn(v, awq[i % K]);
    out[i] = Act16<ODT>::from_f32(v);
}

// ---------------------------------------------------------------------------------------------
// On-device Q4 quantisation (bit-identical to the host quantizer of the reference project):
//   amax = max|v| ; scale = amax > 0 ? amax/7 : 0 ; inv = scale > 0 ? 1/scale : 0
//   q = clamp(round_half_away(v*inv), -8, 7) + 8 ; device byte j = q[j] | q[j+16] << 4
// One thread per block of 32 weights.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int round_half_away_sat(float v) {
    if (v != v) return 0;                 // NaN -> 0, as a saturating float->int8 cast gives
    const float r = roundf(v);            // half away from zero
    return static_cast<int>(fminf(fmaxf(r, -128.0f), 127.0f));
}

__global__ void __launch_bounds__(256) q4_quantize_kernel(const float* W, const float* awq_scales, uint8_t* nibbles,
                                                          float* scales, long long total_blocks, int nb) {
    const long long blk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk >= total_blocks) return;
    const int b = static_cast<int>(blk % nb);
    float v[32];
    const float4* src = reinterpret_cast<const float4*>(W + blk * 32);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float4 f = src[i];
        v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
    }
    if (awq_scales != nullptr) {
#pragma unroll
        for (int e = 0; e < 32; e++) v[e] = __fmul_rn(v[e], awq_scales[b * 32 + e]);
    }
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 32; e++) {
        const float a = fabsf(v[e]);
        if (a > amax) amax = a;  // NaN never wins, matching f32::max folding from 0
    }
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 7.0f) : 0.0f;
    const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
    uint32_t packed[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; j++) {
        int q0 = round_half_away_sat(__fmul_rn(v[j], inv));
        int q1 = round_half_away_sat(__fmul_rn(v[j + 16], inv));
        q0 = max(-8, min(7, q0)) + 8;
        q1 = max(-8, min(7, q1)) + 8;
        packed[j >> 2] |= static_cast<uint32_t>(q0 | (q1 << 4)) << (8 * (j & 3));
    }
    reinterpret_cast<uint4*>(nibbles)[blk] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    scales[blk] = scale;
}

// CPU block (f32 scale + 16 bytes of {2i, 2i+1}) -> device layout.
__global__ void __launch_bounds__(256) q4_repack_kernel(const uint8_t* cpu_blocks, uint8_t* nibbles, float* scales,
                                                        long long total_blocks) {
    const long long blk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (blk >= total_blocks) return;
    const uint8_t* src = cpu_blocks + blk * 20;
    uint8_t raw[20];
#pragma unroll
    for (int i = 0; i < 5; i++) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(src + 4 * i);  // blocks are 20 bytes: 4-byte aligned
        raw[4 * i] = w & 0xFF; raw[4 * i + 1] = (w >> 8) & 0xFF; raw[4 * i + 2] = (w >> 16) & 0xFF; raw[4 * i + 3] = w >> 24;
    }
    uint32_t sbits = raw[0] | (raw[1] << 8) | (raw[2] << 16) | (static_cast<uint32_t>(raw[3]) << 24);
    scales[blk] = __uint_as_float(sbits);
    uint8_t* dst = nibbles + blk * 16;
#pragma unroll
    for (int j = 0; j < 16; j++) {
        const int h = j >> 1;
        const uint8_t ej = (j & 1) ? (raw[4 + h] >> 4) : (raw[4 + h] & 0xF);
        const uint8_t ej16 = (j & 1) ? (raw[4 + h + 8] >> 4) : (raw[4 + h + 8] & 0xF);
        dst[j] = static_cast<uint8_t>(ej | (ej16 << 4));
    }
}

// ---------------------------------------------------------------------------------------------
// Synthetic generator
// ---------------------------------------------------------------------------------------------
template <int ODT> __global__ void __launch_bounds__(256) fill_normal_kernel(void* out, long long n, unsigned long long st,
                                                                              unsigned long long first, float scale) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = __fmul_rn(gen_normal(st, first + static_cast<unsigned long long>(i)), scale);
    store_out<ODT>(out, i, v);
}

static unsigned grid_for(long long n, int block) { return static_cast<unsigned>((n + block - 1) / block); }

}  // namespace nve

using namespace nve;

extern "C" void nve_matvec_f16(const uint16_t* x, const uint16_t* W, uint16_t* out, int N, int K, nve_stream_t stream) {
    if (!x || !W || !out) { set_status(NVE_ERR_BAD_POINTER); return; }
    if (N <= 0 || K <= 0) { set_status(NVE_ERR_BAD_SHAPE); return; }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool vec = (K % 8) == 0 && aligned(x, 16) && aligned(W, 16);
    const int wpb = 8;
    if (vec) matvec_f16_kernel<true><<<(N + wpb - 1) / wpb, wpb * 32, 0, st>>>(x, W, out, N, K);
    else matvec_f16_kernel<false><<<(N + wpb - 1) / wpb, wpb * 32, 0, st>>>(x, W, out, N, K);
    count_launch();
    check_launch();
}

extern "C" int nve_b200_dequant_w4a16(const uint8_t* nibbles, const float* scales, const float* awq, void* out, int N,
                                      int K, int out_dtype, nve_stream_t stream) {
    if (!nibbles || !scales || !out) return set_status(NVE_ERR_BAD_POINTER);
    if (N <= 0 || K <= 0 || (K % 32) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    if (out_dtype != NVE_DT_F16 && out_dtype != NVE_DT_BF16) return set_status(NVE_ERR_BAD_DTYPE);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long blocks = static_cast<long long>(N) * (K / 32);
    uint16_t* o = static_cast<uint16_t*>(out);
    if (aligned(nibbles, 16) && aligned(out, 16)) {
        if (out_dtype == NVE_DT_F16) dequant_kernel<NVE_DT_F16><<<grid_for(blocks, 256), 256, 0, st>>>(nibbles, scales, awq, o, blocks, K / 32);
        else dequant_kernel<NVE_DT_BF16><<<grid_for(blocks, 256), 256, 0, st>>>(nibbles, scales, awq, o, blocks, K / 32);
    } else {
        const long long total = blocks * 32;
        if (out_dtype == NVE_DT_F16) dequant_scalar_kernel<NVE_DT_F16><<<grid_for(total, 256), 256, 0, st>>>(nibbles, scales, awq, o, total, K);
        else dequant_scalar_kernel<NVE_DT_BF16><<<grid_for(total, 256), 256, 0, st>>>(nibbles, scales, awq, o, total, K);
    }
    count_launch();
    return check_launch();
}

extern "C" void nve_dequant_w4a16(const uint8_t* nibbles, const float* scales, const float* awq, uint16_t* out, int N,
                                  int K, nve_stream_t stream) {
    nve_b200_dequant_w4a16(nibbles, scales, awq, out, N, K, NVE_DT_F16, stream);
}

extern "C" int nve_b200_q4_quantize(const float* W, const float* awq_scales, uint8_t* nibbles, float* scales, int N, int K,
                                    nve_stream_t stream) {
    if (!W || !nibbles || !scales) return set_status(NVE_ERR_BAD_POINTER);
    if (N <= 0 || K <= 0 || (K % 32) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    if (!aligned(W, 16) || !aligned(nibbles, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    const long long blocks = static_cast<long long>(N) * (K / 32);
    q4_quantize_kernel<<<grid_for(blocks, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(W, awq_scales, nibbles, scales,
                                                                                            blocks, K / 32);
    count_launch();
    return check_launch();
}

extern "C" int nve_b200_q4_repack_blocks(const uint8_t* cpu_blocks, uint8_t* nibbles, float* scales, int N, int K,
                                         nve_stream_t stream) {
    if (!cpu_blocks || !nibbles || !scales) return set_status(NVE_ERR_BAD_POINTER);
    if (N <= 0 || K <= 0 || (K % 32) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    if (!aligned(cpu_blocks, 4)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    const long long blocks = static_cast<long long>(N) * (K / 32);
    q4_repack_kernel<<<grid_for(blocks, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(cpu_blocks, nibbles, scales, blocks);
    count_launch();
    return check_launch();
}

extern "C" int nve_b200_fill_normal(float* out, long long n, unsigned long long seed, unsigned long long stream_id,
                                    unsigned long long first, float scale, nve_stream_t stream) {
    if (!out) return set_status(NVE_ERR_BAD_POINTER);
    if (n <= 0) return set_status(NVE_ERR_BAD_SHAPE);
    fill_normal_kernel<NVE_DT_F32><<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        out, n, gen_state(seed, stream_id), first, scale);
    count_launch();
    return check_launch();
}

extern "C" int nve_b200_fill_normal_16(void* out, long long n, unsigned long long seed, unsigned long long stream_id,
                                       unsigned long long first, float scale, int dtype, nve_stream_t stream) {
    if (!out) return set_status(NVE_ERR_BAD_POINTER);
    if (n <= 0) return set_status(NVE_ERR_BAD_SHAPE);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned long long s = gen_state(seed, stream_id);
    if (dtype == NVE_DT_F16) fill_normal_kernel<NVE_DT_F16><<<grid_for(n, 256), 256, 0, st>>>(out, n, s, first, scale);
    else if (dtype == NVE_DT_BF16) fill_normal_kernel<NVE_DT_BF16><<<grid_for(n, 256), 256, 0, st>>>(out, n, s, first, scale);
    else return set_status(NVE_ERR_BAD_DTYPE);
    count_launch();
    return check_launch();
}
