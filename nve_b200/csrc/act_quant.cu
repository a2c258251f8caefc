// Activation-side kernels of the decode path: per-group int8 quantisation, RMSNorm, SiLU*up, residual add,
// LayerNorm, and the fused forms RMSNorm->quantise and SiLU*up->quantise.
//
// Replaces cuda/nve_kernels.cu:26-76 (RMSNorm), :82-134 (LayerNorm), :712-757 (quantize_f16_q8),
// :955-969 (add_inplace) and :978-995 (silu_mul) of the reference project; the fused forms have no
// counterpart there (the reference launches the two kernels back to back, src/gpu_layer.rs:658,946).
//
// All arithmetic that decides an int8 code or a 16-bit result uses IEEE-rounded operations in a fixed
// order, so that a host restatement can reproduce the bits:
//   quantise : amax over the group; scale = amax > 0 ? amax/127 : 1; q = clamp(rint(x * (1/scale)), +-127)
//   RMSNorm  : 256 threads; thread t adds x^2 (fma chain) over the 8-element chunks t, t+256, ... in
//              ascending element order; xor-butterfly per warp; the 8 warp sums added in ascending order;
//              r = 1/sqrt(sum/n + eps); out = round16((x*r)*w)
#include "act_ops.cuh"

namespace nve {

constexpr int kActThreads = 256;

// Load / store one 8-element chunk; the scalar path also handles a ragged tail (elements >= n read as 0).
template <bool VEC> __device__ __forceinline__ void load_chunk(const uint16_t* p, long long c, int n, uint16_t (&h)[8]) {
    if constexpr (VEC) {
        unpack8(reinterpret_cast<const uint4*>(p)[c], h);
    } else {
#pragma unroll
        for (int e = 0; e < 8; e++) h[e] = (c * 8 + e < n) ? p[c * 8 + e] : static_cast<uint16_t>(0);
    }
}
template <bool VEC> __device__ __forceinline__ void store_chunk(uint16_t* p, long long c, int n, const uint16_t (&h)[8]) {
    if constexpr (VEC) {
        reinterpret_cast<uint4*>(p)[c] = pack8(h);
    } else {
#pragma unroll
        for (int e = 0; e < 8; e++)
            if (c * 8 + e < n) p[c * 8 + e] = h[e];
    }
}

template <int DT> __global__ void __launch_bounds__(kActThreads) quantize_q8_kernel(const uint16_t* x, int8_t* xq,
                                                                                     float* scales, int K,
                                                                                     const float* awq_inv) {
    pdl_wait();
    const long long chunk = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const bool active = chunk * 8 < K;
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) {
        uint16_t h[8];
        load_chunk<true>(x, chunk, K, h);
#pragma unroll
        for (int e = 0; e < 8; e++) v[e] = Act16<DT>::to_f32(h[e]);
        if (awq_inv != nullptr) {  // activations of an AWQ pre-scaled matrix: x[k] * awq_inv[k] before the absmax
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], awq_inv[chunk * 8 + e]);
        }
    }
    pdl_launch_dependents();
    quantize_quad(v, xq, scales, chunk, active);
}

// Scalar fallback for unaligned pointers: one thread per group.
template <int DT> __global__ void quantize_q8_scalar_kernel(const uint16_t* x, int8_t* xq, float* scales, int K,
                                                           const float* awq_inv) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= K / 32) return;
    auto val = [&](int e) {
        const float v = Act16<DT>::to_f32(x[g * 32 + e]);
        return awq_inv != nullptr ? __fmul_rn(v, awq_inv[g * 32 + e]) : v;
    };
    float amax = 0.0f;
    for (int e = 0; e < 32; e++) amax = fmaxf(amax, fabsf(val(e)));
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    scales[g] = scale;
    for (int e = 0; e < 32; e++) {
        int q = __float2int_rn(__fmul_rn(val(e), inv));
        xq[g * 32 + e] = static_cast<int8_t>(max(-127, min(127, q)));
    }
}

// Sum of squares with the documented order; returns the total on every thread.
template <int DT, bool VEC> __device__ __forceinline__ float sum_squares(const uint16_t* x, int n) {
    __shared__ float warp_part[kActThreads / 32];
    const int chunks = (n + 7) / 8;
    float acc = 0.0f;
    for (int c = threadIdx.x; c < chunks; c += kActThreads) {
        uint16_t h[8];
        load_chunk<VEC>(x, c, n, h);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float v = Act16<DT>::to_f32(h[e]);
            acc = __fmaf_rn(v, v, acc);
        }
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    float total = warp_part[0];
#pragma unroll
    for (int w = 1; w < kActThreads / 32; w++) total = __fadd_rn(total, warp_part[w]);
    return total;
}

// RMSNorm, optionally followed by the int8 quantisation of the rounded result.  Single CTA.
template <int DT, bool VEC, bool QUANT>
__global__ void __launch_bounds__(kActThreads) rmsnorm_kernel(const uint16_t* x, const uint16_t* w, uint16_t* out,
                                                              int8_t* xq, float* scales, int n, float eps) {
    // one CTA per row of n values (a single row in every form but nve_b200_rms_norm_rows)
    x += static_cast<long long>(blockIdx.x) * n;
    if (out != nullptr) out += static_cast<long long>(blockIdx.x) * n;
    pdl_wait();
    const float total = sum_squares<DT, VEC>(x, n);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(n)), eps)));
    pdl_launch_dependents();
    const int chunks = (n + 7) / 8;
    // all threads of a quad iterate together so that the group maximum can use shuffles
    const int iters = (chunks + kActThreads - 1) / kActThreads;
    for (int it = 0; it < iters; it++) {
        const int c = it * kActThreads + threadIdx.x;
        const bool active = c < chunks;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (active) {
            uint16_t hx[8], hw[8], ho[8];
            load_chunk<VEC>(x, c, n, hx);
            load_chunk<VEC>(w, c, n, hw);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float o = __fmul_rn(__fmul_rn(Act16<DT>::to_f32(hx[e]), r), Act16<DT>::to_f32(hw[e]));
                ho[e] = Act16<DT>::from_f32(o);
                v[e] = Act16<DT>::to_f32(ho[e]);
            }
            if (out != nullptr) store_chunk<VEC>(out, c, n, ho);
        }
        if constexpr (QUANT) quantize_quad(v, xq, scales, c, active);
    }
}

// x[row] += delta[row] (the residual add, stored in place with add_inplace_kernel's arithmetic) followed by the RMSNorm
// of the updated row into out: one launch for the pair of launches between two projections of a batched layer.  The
// CTA reads back what it stored (ordered by the CTA barrier), so the bits are those of the two separate kernels.
template <int DT> __global__ void __launch_bounds__(kActThreads) add_rmsnorm_rows_kernel(uint16_t* x, const uint16_t* delta,
                                                                                         const uint16_t* w, uint16_t* out, int n,
                                                                                         float eps) {
    x += static_cast<long long>(blockIdx.x) * n;
    delta += static_cast<long long>(blockIdx.x) * n;
    out += static_cast<long long>(blockIdx.x) * n;
    pdl_wait();
    const int chunks = n / 8;
    for (int c = threadIdx.x; c < chunks; c += kActThreads) {
        uint16_t hd[8], hs[8];
        load_chunk<true>(x, c, n, hd);
        load_chunk<true>(delta, c, n, hs);
#pragma unroll
        for (int e = 0; e < 8; e++) hd[e] = Act16<DT>::from_f32(__fadd_rn(Act16<DT>::to_f32(hd[e]), Act16<DT>::to_f32(hs[e])));
        store_chunk<true>(x, c, n, hd);
    }
    __syncthreads();
    const float total = sum_squares<DT, true>(x, n);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(n)), eps)));
    pdl_launch_dependents();
    for (int c = threadIdx.x; c < chunks; c += kActThreads) {
        uint16_t hx[8], hw[8], ho[8];
        load_chunk<true>(x, c, n, hx);
        load_chunk<true>(w, c, n, hw);
#pragma unroll
        for (int e = 0; e < 8; e++)
            ho[e] = Act16<DT>::from_f32(__fmul_rn(__fmul_rn(Act16<DT>::to_f32(hx[e]), r), Act16<DT>::to_f32(hw[e])));
        store_chunk<true>(out, c, n, ho);
    }
}

// QUANT: 0 = 16-bit output only, 1 = + int8 codes (W4A8 route), 2 = + 16-bit fixed-point planes (W4A16 route; `awq`,
// if given, multiplies each element first, as the W4A16 GEMV's own staging does).
template <int DT, int QUANT>
__global__ void __launch_bounds__(kActThreads) silu_mul_kernel(const uint16_t* gate, const uint16_t* up, uint16_t* out,
                                                               int8_t* xq, float* scales, int n, uint8_t* xlo,
                                                               const float* awq) {
    pdl_wait();
    const long long c = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const bool active = c * 8 < n;
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (active) {
        uint16_t hg[8], hu[8], ho[8];
        load_chunk<true>(gate, c, n, hg);
        load_chunk<true>(up, c, n, hu);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            ho[e] = Act16<DT>::from_f32(silu_mul_f32(Act16<DT>::to_f32(hg[e]), Act16<DT>::to_f32(hu[e])));
            v[e] = Act16<DT>::to_f32(ho[e]);
        }
        if (out != nullptr) store_chunk<true>(out, c, n, ho);
    }
    pdl_launch_dependents();
    if constexpr (QUANT == 1) quantize_quad(v, xq, scales, c, active);
    if constexpr (QUANT == 2) {
        if (active && awq != nullptr) {
#pragma unroll
            for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], awq[c * 8 + e]);
        }
        x16_quad(v, xlo, xq, scales, c, active);
    }
}

template <int DT> __global__ void silu_mul_scalar_kernel(uint16_t* gate, const uint16_t* up, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) gate[i] = Act16<DT>::from_f32(silu_mul_f32(Act16<DT>::to_f32(gate[i]), Act16<DT>::to_f32(up[i])));
}

template <int DT, bool VEC> __global__ void __launch_bounds__(kActThreads) add_inplace_kernel(uint16_t* dst, const uint16_t* src,
                                                                                             int n) {
    pdl_wait();
    const long long c = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (c * 8 >= n) return;
    uint16_t hd[8], hs[8];
    load_chunk<VEC>(dst, c, n, hd);
    load_chunk<VEC>(src, c, n, hs);
#pragma unroll
    for (int e = 0; e < 8; e++) hd[e] = Act16<DT>::from_f32(__fadd_rn(Act16<DT>::to_f32(hd[e]), Act16<DT>::to_f32(hs[e])));
    store_chunk<VEC>(dst, c, n, hd);
}

// LayerNorm with optional bias (cuda/nve_kernels.cu:82-118 arithmetic: var = E[x^2] - mean^2).
__global__ void __launch_bounds__(kActThreads) layer_norm_kernel(const uint16_t* x, const uint16_t* w, const uint16_t* bias,
                                                                 uint16_t* out, int n, float eps) {
    __shared__ float s_sum[kActThreads / 32], s_sq[kActThreads / 32];
    float a = 0.0f, b = 0.0f;
    for (int i = threadIdx.x; i < n; i += kActThreads) {
        const float v = Act16<NVE_DT_F16>::to_f32(x[i]);
        a += v;
        b = __fmaf_rn(v, v, b);
    }
    a = warp_sum(a);
    b = warp_sum(b);
    if ((threadIdx.x & 31) == 0) {
        s_sum[threadIdx.x >> 5] = a;
        s_sq[threadIdx.x >> 5] = b;
    }
    __syncthreads();
    float ta = 0.0f, tb = 0.0f;
#pragma unroll
    for (int k = 0; k < kActThreads / 32; k++) {
        ta += s_sum[k];
        tb += s_sq[k];
    }
    const float mean = ta / static_cast<float>(n);
    const float var = tb / static_cast<float>(n) - mean * mean;
    const float istd = __fdiv_rn(1.0f, __fsqrt_rn(var + eps));
    for (int i = threadIdx.x; i < n; i += kActThreads) {
        const float v = (Act16<NVE_DT_F16>::to_f32(x[i]) - mean) * istd;
        const float bb = bias != nullptr ? Act16<NVE_DT_F16>::to_f32(bias[i]) : 0.0f;
        out[i] = Act16<NVE_DT_F16>::from_f32(v * Act16<NVE_DT_F16>::to_f32(w[i]) + bb);
    }
}

static int launch_cfg(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int grid, cudaStream_t stream) {
    cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kActThreads);
    cfg.stream = stream;
    if (pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return 0;
}

template <int DT>
static int quantize_q8_impl(const void* x, int8_t* xq, float* scales, int K, cudaStream_t st, const float* awq_inv = nullptr) {
    if (!x || !xq || !scales) return set_status(NVE_ERR_BAD_POINTER);
    if (K <= 0 || (K % 32) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    const uint16_t* x16 = static_cast<const uint16_t*>(x);
    if (aligned(x, 16) && aligned(xq, 8)) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attr[1];
        launch_cfg(cfg, attr, (K / 8 + kActThreads - 1) / kActThreads, st);
        cudaError_t e = cudaLaunchKernelEx(&cfg, quantize_q8_kernel<DT>, x16, xq, scales, K, awq_inv);
        count_launch();
        return set_cuda_status(e);
    }
    quantize_q8_scalar_kernel<DT><<<(K / 32 + 127) / 128, 128, 0, st>>>(x16, xq, scales, K, awq_inv);
    count_launch();
    return check_launch();
}

template <int DT, bool QUANT>
static int rmsnorm_impl(const void* x, const void* w, void* out, int8_t* xq, float* scales, int n, float eps,
                        cudaStream_t st, int rows = 1) {
    if (!x || !w) return set_status(NVE_ERR_BAD_POINTER);
    if (n <= 0 || rows <= 0 || (QUANT && rows != 1)) return set_status(NVE_ERR_BAD_SHAPE);
    if (QUANT) {
        if (!xq || !scales) return set_status(NVE_ERR_BAD_POINTER);
        if ((n % 32) != 0) return set_status(NVE_ERR_BAD_SHAPE);
        if (!aligned(xq, 8)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    } else if (!out) {
        return set_status(NVE_ERR_BAD_POINTER);
    }
    const bool vec = (n % 8) == 0 && aligned(x, 16) && aligned(w, 16) && (out == nullptr || aligned(out, 16));
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, rows, st);
    const uint16_t* x16 = static_cast<const uint16_t*>(x);
    const uint16_t* w16 = static_cast<const uint16_t*>(w);
    uint16_t* o16 = static_cast<uint16_t*>(out);
    cudaError_t e = vec ? cudaLaunchKernelEx(&cfg, rmsnorm_kernel<DT, true, QUANT>, x16, w16, o16, xq, scales, n, eps)
                        : cudaLaunchKernelEx(&cfg, rmsnorm_kernel<DT, false, QUANT>, x16, w16, o16, xq, scales, n, eps);
    count_launch();
    return set_cuda_status(e);
}

template <int DT, int QUANT>
static int silu_mul_impl(const void* gate, const void* up, void* out, int8_t* xq, float* scales, int n, cudaStream_t st,
                         uint8_t* xlo = nullptr, const float* awq = nullptr) {
    if (!gate || !up) return set_status(NVE_ERR_BAD_POINTER);
    if (n <= 0) return set_status(NVE_ERR_BAD_SHAPE);
    const bool vec = (n % 8) == 0 && aligned(gate, 16) && aligned(up, 16) && (out == nullptr || aligned(out, 16));
    if (QUANT) {
        if (!xq || !scales) return set_status(NVE_ERR_BAD_POINTER);
        if ((n % 32) != 0) return set_status(NVE_ERR_BAD_SHAPE);
        if (!vec || !aligned(xq, 8)) return set_status(NVE_ERR_BAD_ALIGNMENT);
        if (QUANT == 2 && (!xlo || !aligned(xlo, 8))) return set_status(xlo ? NVE_ERR_BAD_ALIGNMENT : NVE_ERR_BAD_POINTER);
    }
    if (!vec) {
        if (out != gate) return set_status(NVE_ERR_BAD_ALIGNMENT);
        silu_mul_scalar_kernel<DT><<<(n + 255) / 256, 256, 0, st>>>(static_cast<uint16_t*>(out),
                                                                     static_cast<const uint16_t*>(up), n);
        count_launch();
        return check_launch();
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, (n / 8 + kActThreads - 1) / kActThreads, st);
    cudaError_t e = cudaLaunchKernelEx(&cfg, silu_mul_kernel<DT, QUANT>, static_cast<const uint16_t*>(gate),
                                       static_cast<const uint16_t*>(up), static_cast<uint16_t*>(out), xq, scales, n, xlo, awq);
    count_launch();
    return set_cuda_status(e);
}

template <int DT> static int add_inplace_impl(void* dst, const void* src, int n, cudaStream_t st) {
    if (!dst || !src) return set_status(NVE_ERR_BAD_POINTER);
    if (n <= 0) return set_status(NVE_ERR_BAD_SHAPE);
    const bool vec = (n % 8) == 0 && aligned(dst, 16) && aligned(src, 16);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, ((n + 7) / 8 + kActThreads - 1) / kActThreads, st);
    uint16_t* d = static_cast<uint16_t*>(dst);
    const uint16_t* s = static_cast<const uint16_t*>(src);
    cudaError_t e = vec ? cudaLaunchKernelEx(&cfg, add_inplace_kernel<DT, true>, d, s, n)
                        : cudaLaunchKernelEx(&cfg, add_inplace_kernel<DT, false>, d, s, n);
    count_launch();
    return set_cuda_status(e);
}

}  // namespace nve

using namespace nve;

#define NVE_DISPATCH_16(dtype, expr_f16, expr_bf16)     \
    ((dtype) == NVE_DT_F16 ? (expr_f16) : ((dtype) == NVE_DT_BF16 ? (expr_bf16) : set_status(NVE_ERR_BAD_DTYPE)))

extern "C" int nve_b200_quantize_q8(const void* x, int8_t* xq, float* scales, int K, int x_dtype, nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(x_dtype, quantize_q8_impl<NVE_DT_F16>(x, xq, scales, K, st),
                           quantize_q8_impl<NVE_DT_BF16>(x, xq, scales, K, st));
}

extern "C" int nve_b200_quantize_q8_awq(const void* x, const float* awq_inv, int8_t* xq, float* scales, int K, int x_dtype,
                                        nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(x_dtype, quantize_q8_impl<NVE_DT_F16>(x, xq, scales, K, st, awq_inv),
                           quantize_q8_impl<NVE_DT_BF16>(x, xq, scales, K, st, awq_inv));
}

extern "C" void nve_quantize_f16_q8(const uint16_t* x, int8_t* xq, float* scales, int K, nve_stream_t stream) {
    quantize_q8_impl<NVE_DT_F16>(x, xq, scales, K, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_rms_norm(const void* x, const void* weight, void* out, int n, float eps, int dtype,
                                 nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(dtype, (rmsnorm_impl<NVE_DT_F16, false>(x, weight, out, nullptr, nullptr, n, eps, st)),
                           (rmsnorm_impl<NVE_DT_BF16, false>(x, weight, out, nullptr, nullptr, n, eps, st)));
}

/* RMSNorm of every row of x [rows, n] with one weight vector (the reference runs its kernel once per token in prefill,
 * src/gpu_layer.rs:137): one launch, a CTA per row, each row bit-identical to nve_b200_rms_norm on it. */
extern "C" int nve_b200_rms_norm_rows(const void* x, const void* weight, void* out, int rows, int n, float eps, int dtype,
                                      nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(dtype, (rmsnorm_impl<NVE_DT_F16, false>(x, weight, out, nullptr, nullptr, n, eps, st, rows)),
                           (rmsnorm_impl<NVE_DT_BF16, false>(x, weight, out, nullptr, nullptr, n, eps, st, rows)));
}

template <int DT> static int add_rmsnorm_rows_impl(void* x, const void* delta, const void* weight, void* out, int rows, int n, float eps,
                                                   cudaStream_t st) {
    if (!x || !delta || !weight || !out) return set_status(NVE_ERR_BAD_POINTER);
    if (rows <= 0 || rows > 65535 || n <= 0 || (n % 8) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    if (!aligned(x, 16) || !aligned(delta, 16) || !aligned(weight, 16) || !aligned(out, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    launch_cfg(cfg, attr, rows, st);
    cudaError_t e = cudaLaunchKernelEx(&cfg, add_rmsnorm_rows_kernel<DT>, static_cast<uint16_t*>(x), static_cast<const uint16_t*>(delta),
                                       static_cast<const uint16_t*>(weight), static_cast<uint16_t*>(out), n, eps);
    count_launch();
    return set_cuda_status(e);
}

extern "C" int nve_b200_add_rms_norm_rows(void* x, const void* delta, const void* weight, void* out, int rows, int n, float eps,
                                          int dtype, nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(dtype, (add_rmsnorm_rows_impl<NVE_DT_F16>(x, delta, weight, out, rows, n, eps, st)),
                           (add_rmsnorm_rows_impl<NVE_DT_BF16>(x, delta, weight, out, rows, n, eps, st)));
}

extern "C" void nve_rms_norm_f16(const uint16_t* x, const uint16_t* weight, uint16_t* out, int n, float eps,
                                 nve_stream_t stream) {
    rmsnorm_impl<NVE_DT_F16, false>(x, weight, out, nullptr, nullptr, n, eps, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_rmsnorm_quantize_q8(const void* x, const void* weight, void* normed_out, int8_t* xq,
                                            float* scales, int n, float eps, int dtype, nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(dtype, (rmsnorm_impl<NVE_DT_F16, true>(x, weight, normed_out, xq, scales, n, eps, st)),
                           (rmsnorm_impl<NVE_DT_BF16, true>(x, weight, normed_out, xq, scales, n, eps, st)));
}

extern "C" int nve_b200_silu_mul_quantize_q8(const void* gate, const void* up, void* mid_out, int8_t* xq, float* scales,
                                             int n, int dtype, nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(dtype, (silu_mul_impl<NVE_DT_F16, 1>(gate, up, mid_out, xq, scales, n, st)),
                           (silu_mul_impl<NVE_DT_BF16, 1>(gate, up, mid_out, xq, scales, n, st)));
}

extern "C" int nve_b200_silu_mul_x16(const void* gate, const void* up, void* mid_out, uint8_t* x_lo, int8_t* x_hi,
                                     float* x_scales, const float* awq, int n, int dtype, nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(dtype, (silu_mul_impl<NVE_DT_F16, 2>(gate, up, mid_out, x_hi, x_scales, n, st, x_lo, awq)),
                           (silu_mul_impl<NVE_DT_BF16, 2>(gate, up, mid_out, x_hi, x_scales, n, st, x_lo, awq)));
}

extern "C" int nve_b200_silu_mul(void* gate, const void* up, int n, int dtype, nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(dtype, (silu_mul_impl<NVE_DT_F16, 0>(gate, up, gate, nullptr, nullptr, n, st)),
                           (silu_mul_impl<NVE_DT_BF16, 0>(gate, up, gate, nullptr, nullptr, n, st)));
}

extern "C" void nve_silu_mul_f16(uint16_t* gate, const uint16_t* up, int n, nve_stream_t stream) {
    silu_mul_impl<NVE_DT_F16, 0>(gate, up, gate, nullptr, nullptr, n, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_add_inplace(void* dst, const void* src, int n, int dtype, nve_stream_t stream) {
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return NVE_DISPATCH_16(dtype, add_inplace_impl<NVE_DT_F16>(dst, src, n, st), add_inplace_impl<NVE_DT_BF16>(dst, src, n, st));
}

extern "C" void nve_add_inplace_f16(uint16_t* dst, const uint16_t* src, int n, nve_stream_t stream) {
    add_inplace_impl<NVE_DT_F16>(dst, src, n, static_cast<cudaStream_t>(stream));
}

extern "C" void nve_layer_norm_f16(const uint16_t* x, const uint16_t* weight, const uint16_t* bias, uint16_t* out, int n,
                                   float eps, nve_stream_t stream) {
    if (!x || !weight || !out) { set_status(NVE_ERR_BAD_POINTER); return; }
    if (n <= 0) { set_status(NVE_ERR_BAD_SHAPE); return; }
    layer_norm_kernel<<<1, kActThreads, 0, static_cast<cudaStream_t>(stream)>>>(x, weight, bias, out, n, eps);
    count_launch();
    check_launch();
}
