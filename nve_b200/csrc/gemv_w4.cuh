// Device code shared by the W4 GEMV kernels: parameters, shared-memory layout, activation staging and the
// per-block integer dot product.  See gemv_w4.cu for the description of the algorithm.
#pragma once
#include "act_ops.cuh"

namespace nve {

constexpr int kGemvThreads = 256;  // 8 warps
constexpr int kPartFloats = 4096;  // shared-memory floats for column-set partial sums
constexpr int kMaxGemvSmem = 200 * 1024;  // dynamic shared memory a GEMV CTA may ask for

// Tensor-parallel context as the kernels see it.  Every rank owns a "low-latency" buffer of 8-byte slots
// {f32 partial sum, u32 epoch}, indexed [parity][source rank][row]; a rank PUSHES its partial rows into the
// buffers of all ranks (its own included) with single 8-byte stores and then polls only its own, local buffer
// until the slots carry the current epoch.  Data and flag travel in one store, so no fence and no round trip
// is needed.  world <= 1 disables it.
constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxCtas = 1024;
struct TpDev {
    int world;
    int rank;
    int rows_cap;                 // rows per [parity][source] plane
    uint2* ll[kTpMaxWorld];       // rank r's buffer (own memory for `rank`, CUDA-IPC peer mappings otherwise)
    unsigned* counter;            // local [kTpMaxCtas]: all-reduce launches seen by each CTA index
    int* err;                     // local error word (0 = ok)
};

struct GemvParams {
    const uint8_t* nib[3];
    const float* sc[3];
    void* out[3];
    const void* res[3];
    int row_end[3];  // cumulative row ends of the (up to three) matrices
    int n_total;     // rows over all matrices
    int K;
    int nb;          // K / 32
    int S;           // column sets = ceil(nb / 32)
    const int8_t* xq;   // W4A8 codes
    const float* xs;    // W4A8 scales
    const void* x16;    // W4A16 activations
    const uint8_t* xlo; // W4A16 activations already in fixed point: low-byte plane (high bytes in xq, scales in xs)
    const float* awq;   // optional per-column multiplier (W4A16)
    const void* norm_w; // RMSNorm weight of the fused prologue (16-bit, same type as x16)
    float eps;
    int32_t* idot;      // debug: per-block integer dots [n_total, nb]
    int paired;         // gate/up with SiLU*up in the epilogue: a tile holds R/2 gate rows (matrix 0) and the R/2 up
                        // rows (matrix 1) of the same indices; out[0] receives silu(gate) * up, [row_end[0]] values
    // paired form only: the CTA that completes a 32-wide group of silu(gate)*up values converts the group for the
    // down projection (pq_mode 1: int8 codes + scale, 2: 16-bit fixed-point planes + scale), so that no separate
    // activation kernel and no per-CTA quantiser prologue is needed.  pq_cnt[g] counts the values written to group g
    // (32 per launch, never reset; the test is on the count modulo 32, so the wrap of the 32-bit counter is harmless).
    int pq_mode;
    unsigned* pq_cnt;
    int8_t* pq_xq;      // int8 codes (mode 1) / high-byte plane (mode 2)
    uint8_t* pq_xlo;    // low-byte plane (mode 2)
    float* pq_xs;       // per-group scales
    const float* pq_awq; // optional per-column multiplier of the down projection (mode 2)
    TpDev tp;           // all-reduce of the (single) output over the tensor-parallel ranks
};

template <int PLANES> struct XTile {
    uint4 lo[PLANES];
    uint4 hi[PLANES];
    float xs;
    int bias;
};

__device__ __forceinline__ void locate(const GemvParams& p, int grow, const uint8_t*& nib, const float*& sc, int& lrow,
                                       int& lend) {
    if (grow < p.row_end[0]) {
        nib = p.nib[0]; sc = p.sc[0]; lrow = grow; lend = p.row_end[0];
    } else if (grow < p.row_end[1]) {
        nib = p.nib[1]; sc = p.sc[1]; lrow = grow - p.row_end[0]; lend = p.row_end[1] - p.row_end[0];
    } else {
        nib = p.nib[2]; sc = p.sc[2]; lrow = grow - p.row_end[1]; lend = p.row_end[2] - p.row_end[1];
    }
}

// Exact integer dot of one 32-weight block with the staged activations: sum_e (q_e - 8) * x_e.
// Low nibbles are masked out; high nibbles are used in place (as 16*q) and the factor 16 is removed by one
// arithmetic shift, exact because that partial sum is a multiple of 16.
template <int PLANES> __device__ __forceinline__ int block_dot(const uint4& w, const XTile<PLANES>& x) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
    if constexpr (PLANES == 1) {
        const int xl[4] = {(int)x.lo[0].x, (int)x.lo[0].y, (int)x.lo[0].z, (int)x.lo[0].w};
        const int xh[4] = {(int)x.hi[0].x, (int)x.hi[0].y, (int)x.hi[0].z, (int)x.hi[0].w};
        int acc_lo = 0, acc_hi = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc_lo = dp4a_us(wv[j] & 0x0F0F0F0Fu, xl[j], acc_lo);
            acc_hi = dp4a_us(wv[j] & 0xF0F0F0F0u, xh[j], acc_hi);
        }
        return acc_lo + (acc_hi >> 4) - x.bias;
    } else {
        // plane 0: unsigned low bytes, plane 1: signed high bytes of the 16-bit fixed-point activations
        const uint32_t l0[4] = {x.lo[0].x, x.lo[0].y, x.lo[0].z, x.lo[0].w};
        const uint32_t h0[4] = {x.hi[0].x, x.hi[0].y, x.hi[0].z, x.hi[0].w};
        const int l1[4] = {(int)x.lo[1].x, (int)x.lo[1].y, (int)x.lo[1].z, (int)x.lo[1].w};
        const int h1[4] = {(int)x.hi[1].x, (int)x.hi[1].y, (int)x.hi[1].z, (int)x.hi[1].w};
        int lo_lo = 0, lo_hi = 0, hi_lo = 0, hi_hi = 0;  // <activation byte plane>_<nibble half>
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t nl = wv[j] & 0x0F0F0F0Fu;
            const uint32_t nh = wv[j] & 0xF0F0F0F0u;
            lo_lo = dp4a_uu(nl, l0[j], lo_lo);
            lo_hi = dp4a_uu(nh, h0[j], lo_hi);
            hi_lo = dp4a_us(nl, l1[j], hi_lo);
            hi_hi = dp4a_us(nh, h1[j], hi_hi);
        }
        return (hi_lo + (hi_hi >> 4)) * 256 + lo_lo + (lo_hi >> 4) - x.bias;
    }
}

// Shared-memory layout: planes[PLANES][2][nbp] uint4, xs[nbp] f32, bias[nbp] i32, part[kPartFloats] f32
template <int PLANES> struct Smem {
    uint4* plane;  // index ((pl * 2 + half) * nbp + b)
    float* xs;
    int* bias;
    float* part;
    int nbp;
    __device__ Smem(unsigned char* base, int nbp_) : nbp(nbp_) {
        plane = reinterpret_cast<uint4*>(base);
        xs = reinterpret_cast<float*>(plane + static_cast<size_t>(PLANES) * 2 * nbp);
        bias = reinterpret_cast<int*>(xs + nbp);
        part = reinterpret_cast<float*>(bias + nbp);
    }
};

inline size_t gemv_smem_bytes(int planes, int S) {
    const size_t nbp = static_cast<size_t>(S) * kWarp;
    return nbp * (32 * planes + 8) + kPartFloats * sizeof(float);
}

// Stage the caller's int8 codes (W4A8).
__device__ __forceinline__ void stage_q8(const GemvParams& p, Smem<1>& sm) {
#pragma unroll 2
    for (int b = threadIdx.x; b < sm.nbp; b += kGemvThreads) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo;
        float xs = 0.0f;
        int bias = 0;
        if (b < p.nb) {
            const uint4* src = reinterpret_cast<const uint4*>(p.xq + static_cast<long long>(b) * 32);
            lo = src[0];
            hi = src[1];
            xs = p.xs != nullptr ? p.xs[b] : 1.0f;
            int sum = 0;
            sum = __dp4a((int)lo.x, 0x01010101, sum); sum = __dp4a((int)lo.y, 0x01010101, sum);
            sum = __dp4a((int)lo.z, 0x01010101, sum); sum = __dp4a((int)lo.w, 0x01010101, sum);
            sum = __dp4a((int)hi.x, 0x01010101, sum); sum = __dp4a((int)hi.y, 0x01010101, sum);
            sum = __dp4a((int)hi.z, 0x01010101, sum); sum = __dp4a((int)hi.w, 0x01010101, sum);
            bias = 8 * sum;
        }
        sm.plane[b] = lo;
        sm.plane[sm.nbp + b] = hi;
        sm.xs[b] = xs;
        sm.bias[b] = bias;
    }
}

// ---- chunk-wise staging -------------------------------------------------------------------------------
// A chunk is 8 consecutive activations held by one thread; the 4 threads of a quad hold one 32-wide block.
// Plane words of chunk c = 4b + j: half j/2 of block b, bytes (j%2)*8 .. (j%2)*8+7 of that 16-byte half.

template <int PLANES> __device__ __forceinline__ void store_chunk_planes(Smem<PLANES>& sm, int c, int pl, uint32_t w0,
                                                                        uint32_t w1) {
    const int b = c >> 2, j = c & 3;
    uint2* dst = reinterpret_cast<uint2*>(&sm.plane[(pl * 2 + (j >> 1)) * sm.nbp + b]);
    dst[j & 1] = make_uint2(w0, w1);
}

// W4A8 codes from 8 already-rounded 16-bit values per thread (same arithmetic as the stand-alone quantizer:
// scale = amax > 0 ? amax/127 : 1 ; q = clamp(rint(v * (1/scale)), -127, 127)).
__device__ __forceinline__ void stage_chunk_q8(Smem<1>& sm, int c, const float (&v)[8], bool active) {
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(v[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    uint32_t w0 = 0, w1 = 0;
    int sum = 0;
#pragma unroll
    for (int e = 0; e < 8; e++) {
        int q = __float2int_rn(__fmul_rn(v[e], inv));
        q = max(-127, min(127, q));
        sum += q;
        const uint32_t byte = static_cast<uint32_t>(q) & 0xFFu;
        if (e < 4) w0 |= byte << (8 * e);
        else w1 |= byte << (8 * (e - 4));
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (active) {
        store_chunk_planes<1>(sm, c, 0, w0, w1);
        if ((c & 3) == 0) {
            sm.xs[c >> 2] = scale;
            sm.bias[c >> 2] = 8 * sum;
        }
    }
}

// W4A16: 16-bit fixed-point planes from 8 f32 values per thread.
//   amax = max|xe| over the block ; scale = amax > 0 ? amax / 32767 : 1 ; v = clamp(rint(xe * (1/scale)), +-32767)
//   low plane = v & 0xFF (unsigned), high plane = v >> 8 (signed) ; bias = 8 * sum(v)
// A non-finite amax makes the scale NaN so that the affected outputs are NaN, as an f32 path would give.
__device__ __forceinline__ void stage_chunk_x16(Smem<2>& sm, int c, const float (&xe)[8], bool active) {
    uint32_t l0, l1, h0, h1;
    int sum;
    const float scale = x16_quad_convert(xe, l0, l1, h0, h1, sum);
    if (active) {
        store_chunk_planes<2>(sm, c, 0, l0, l1);
        store_chunk_planes<2>(sm, c, 1, h0, h1);
        if ((c & 3) == 0) {
            sm.xs[c >> 2] = scale;
            sm.bias[c >> 2] = 8 * sum;
        }
    }
}

// W4A16 activations that a producer kernel already converted to the two byte planes (nve_b200_silu_mul_x16):
// a straight copy, plus the group's code sum for the bias term.
__device__ __forceinline__ void stage_x16_planes(const GemvParams& p, Smem<2>& sm) {
#pragma unroll 2
    for (int b = threadIdx.x; b < p.nb; b += kGemvThreads) {
        const uint4* lo = reinterpret_cast<const uint4*>(p.xlo + static_cast<long long>(b) * 32);
        const uint4* hi = reinterpret_cast<const uint4*>(p.xq + static_cast<long long>(b) * 32);
        const uint4 l0 = lo[0], l1 = lo[1], h0 = hi[0], h1 = hi[1];
        int ul = 0, sh = 0;
        const uint32_t lw[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w};
        const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int j = 0; j < 8; j++) {
            ul = dp4a_uu(lw[j], 0x01010101u, ul);
            sh = __dp4a(static_cast<int>(hw[j]), 0x01010101, sh);
        }
        sm.plane[0 * sm.nbp + b] = l0;
        sm.plane[1 * sm.nbp + b] = l1;
        sm.plane[2 * sm.nbp + b] = h0;
        sm.plane[3 * sm.nbp + b] = h1;
        sm.xs[b] = p.xs[b];
        sm.bias[b] = 8 * (sh * 256 + ul);
    }
}

__device__ __forceinline__ void load8(const uint16_t* p, int c, uint16_t (&h)[8]) {
    const uint4 raw = reinterpret_cast<const uint4*>(p)[c];
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        h[2 * j] = static_cast<uint16_t>(w[j] & 0xFFFFu);
        h[2 * j + 1] = static_cast<uint16_t>(w[j] >> 16);
    }
}

// Zero the padding blocks [nb, nbp) so that idle lanes contribute exactly 0.
template <int PLANES> __device__ __forceinline__ void zero_padding(const GemvParams& p, Smem<PLANES>& sm) {
    for (int b = p.nb + threadIdx.x; b < sm.nbp; b += kGemvThreads) {
#pragma unroll
        for (int q = 0; q < PLANES * 2; q++) sm.plane[q * sm.nbp + b] = make_uint4(0, 0, 0, 0);
        sm.xs[b] = 0.0f;
        sm.bias[b] = 0;
    }
}

// Barrier over the kGemvThreads (256) threads that stage activations and compute; the TMA kernel has one more
// warp (the producer) that must not take part.
__device__ __forceinline__ void consumer_barrier() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

// RMSNorm weights of the fused prologue held in registers: they are static, so the kernel fetches them before it
// waits for its predecessor (they are cold in L2 by the time a layer comes round again: a DRAM round trip that
// would otherwise sit on the critical path between the wait and the first dot product).  Covers K <= 8192.
constexpr int kNormRegChunks = 4;  // 8-element chunks per thread
struct NormRegs {
    uint4 w[kNormRegChunks];
};
__device__ __forceinline__ void load_norm_regs(const GemvParams& p, NormRegs& nr) {
    const int chunks = p.K >> 3;
#pragma unroll
    for (int j = 0; j < kNormRegChunks; j++) {
        const int c = j * kGemvThreads + threadIdx.x;
        nr.w[j] = make_uint4(0, 0, 0, 0);
        if (c < chunks && chunks <= kNormRegChunks * kGemvThreads) nr.w[j] = reinterpret_cast<const uint4*>(p.norm_w)[c];
    }
}
// Stage the activations.  PRO = 0: the caller's vector (int8 codes for W4A8, 16-bit values for W4A16).
// PRO = 2: the caller's 16-bit vector, quantised here (W4A8: the int8 codes of the stand-alone quantiser).
// PRO = 1: RMSNorm of the caller's 16-bit vector first, in the library's fixed order (256 threads; thread t
// adds x^2 over the 8-element chunks t, t+256, ... ; xor butterfly per warp; warp sums added in ascending
// order; r = 1/sqrt(sum/n + eps); o = round16((x*r)*w)), then quantised exactly as the separate kernels do.
template <int PLANES, int XDT, int PRO> __device__ __forceinline__ void stage_activations(const GemvParams& p,
                                                                                           Smem<PLANES>& sm,
                                                                                           const NormRegs& nr) {
    zero_padding<PLANES>(p, sm);
    if constexpr (PLANES == 1 && PRO == 0) {
        stage_q8(p, sm);
        return;
    } else {
        if constexpr (PLANES == 2 && PRO == 0) {
            if (p.xlo != nullptr) {  // uniform over the grid
                stage_x16_planes(p, sm);
                return;
            }
        }
        const uint16_t* x = static_cast<const uint16_t*>(p.x16);
        const int chunks = p.K >> 3;
        float r = 1.0f;
        if constexpr (PRO == 1) {
            if (chunks <= kNormRegChunks * kGemvThreads) {
                // Register-resident form: the vector is read once (all loads in flight together), the norm weights
                // came in before the dependency wait.  Same arithmetic and the same summation order as below.
                __shared__ float warp_part_r[kGemvThreads / 32];
                uint4 xr[kNormRegChunks];
#pragma unroll
                for (int j = 0; j < kNormRegChunks; j++) {
                    const int c = j * kGemvThreads + threadIdx.x;
                    xr[j] = make_uint4(0, 0, 0, 0);
                    if (c < chunks) xr[j] = reinterpret_cast<const uint4*>(x)[c];
                }
                float acc = 0.0f;
#pragma unroll
                for (int j = 0; j < kNormRegChunks; j++) {
                    if (j * kGemvThreads + static_cast<int>(threadIdx.x) < chunks) {
                        uint16_t h[8];
                        unpack8(xr[j], h);
#pragma unroll
                        for (int e = 0; e < 8; e++) {
                            const float v = Act16<XDT>::to_f32(h[e]);
                            acc = __fmaf_rn(v, v, acc);
                        }
                    }
                }
                acc = warp_sum(acc);
                if ((threadIdx.x & 31) == 0) warp_part_r[threadIdx.x >> 5] = acc;
                consumer_barrier();
                float total = warp_part_r[0];
#pragma unroll
                for (int w = 1; w < kGemvThreads / 32; w++) total = __fadd_rn(total, warp_part_r[w]);
                r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.K)), p.eps)));
                const int iters_r = (chunks + kGemvThreads - 1) / kGemvThreads;
#pragma unroll
                for (int j = 0; j < kNormRegChunks; j++) {
                    if (j < iters_r) {  // uniform over the CTA: the quad shuffles inside stage_chunk_* need whole warps
                        const int c = j * kGemvThreads + threadIdx.x;
                        const bool active = c < chunks;
                        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                        if (active) {
                            uint16_t h[8], hw[8];
                            unpack8(xr[j], h);
                            unpack8(nr.w[j], hw);
#pragma unroll
                            for (int e = 0; e < 8; e++) {
                                const float o = __fmul_rn(__fmul_rn(Act16<XDT>::to_f32(h[e]), r), Act16<XDT>::to_f32(hw[e]));
                                v[e] = Act16<XDT>::to_f32(Act16<XDT>::from_f32(o));
                            }
                            if (p.awq != nullptr) {  // W4A16 always; W4A8 only through the *_awq entry point
#pragma unroll
                                for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], p.awq[c * 8 + e]);
                            }
                        }
                        if constexpr (PLANES == 1) stage_chunk_q8(sm, c, v, active);
                        else stage_chunk_x16(sm, c, v, active);
                    }
                }
                return;
            }
        }
        if constexpr (PRO == 1) {
            __shared__ float warp_part[kGemvThreads / 32];
            float acc = 0.0f;
            for (int c = threadIdx.x; c < chunks; c += kGemvThreads) {
                uint16_t h[8];
                load8(x, c, h);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const float v = Act16<XDT>::to_f32(h[e]);
                    acc = __fmaf_rn(v, v, acc);
                }
            }
            acc = warp_sum(acc);
            if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
            consumer_barrier();
            float total = warp_part[0];
#pragma unroll
            for (int w = 1; w < kGemvThreads / 32; w++) total = __fadd_rn(total, warp_part[w]);
            r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(p.K)), p.eps)));
        }
        const int iters = (chunks + kGemvThreads - 1) / kGemvThreads;
        for (int it = 0; it < iters; it++) {
            const int c = it * kGemvThreads + threadIdx.x;
            const bool active = c < chunks;
            float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (active) {
                uint16_t h[8];
                load8(x, c, h);
                if constexpr (PRO == 1) {
                    uint16_t hw[8];
                    load8(static_cast<const uint16_t*>(p.norm_w), c, hw);
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const float o = __fmul_rn(__fmul_rn(Act16<XDT>::to_f32(h[e]), r), Act16<XDT>::to_f32(hw[e]));
                        v[e] = Act16<XDT>::to_f32(Act16<XDT>::from_f32(o));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = Act16<XDT>::to_f32(h[e]);
                }
                if (p.awq != nullptr) {
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], p.awq[c * 8 + e]);
                }
            }
            if constexpr (PLANES == 1) stage_chunk_q8(sm, c, v, active);
            else stage_chunk_x16(sm, c, v, active);
        }
    }
}


// Device view of the process's tensor-parallel context (tp.cu); world == 0 when none is connected.
const TpDev& tp_device_ctx();

}  // namespace nve
