// Batch-1 GEMVs over 4-bit group-32 weights: W4A8 (int8 activations) and W4A16 (16-bit activations).
//
// Replaces cuda/nve_kernels.cu:784-894 (nve_matvec_w4a8), :330-388 (nve_matvec_w4a16) and :607-700
// (nve_qkv_matvec_w4a16) of the reference project.  Not a port: the work decomposition, the
// activation staging and the integer formulation of W4A16 are specific to this library.
//
// One kernel template serves both precisions.
//   * A CTA owns a contiguous range of 4-row tiles and first stages the activation vector in shared
//     memory as int8 "planes", split so that lane l of a warp reads 16 consecutive bytes (no bank
//     conflicts):
//       W4A8  : one plane = the caller's int8 codes; per block the f32 scale and 8*sum(codes).
//       W4A16 : the 16-bit activations (times awq when given) are converted per 32-wide block to a
//               16-bit fixed-point value v = rint(x * 32767/amax), stored as a signed high byte plane and
//               an unsigned low byte plane, so the dot product stays on the integer dp4a pipe and is
//               exact in int32; the only approximation is the fixed-point step amax/65534 per element,
//               far below the 16-bit rounding of the output.
//   * A warp task is (4 rows) x (32 consecutive blocks = 1024 weights per row): every lane issues one
//     128-bit load of packed nibbles and one 32-bit load of the block scale per row, i.e. 512 contiguous
//     bytes per row per warp.  The next task's loads are issued before the current one is reduced.
//   * Per lane: 8 (W4A8) or 16 (W4A16) dp4a on raw nibbles 0..15, minus the precomputed 8*sum(x) bias,
//     one int->float conversion and one multiply by (weight scale * activation scale).
//   * The 32 lane values of a (row, column-set) are added by a fixed xor butterfly and stored to shared
//     memory; a final pass adds the column-set partials of each row in ascending order.  The result is
//     therefore independent of grid size and warp scheduling, and bit-reproducible.
//
// Algorithmic bytes per launch: N*K/2 nibbles + N*K/8 scale bytes + activations + outputs.
#include "common.cuh"

namespace nve {

constexpr int kRows = 4;           // rows per warp task
constexpr int kGemvThreads = 256;  // 8 warps
constexpr int kPartFloats = 4096;  // shared-memory floats for column-set partial sums
constexpr int kMaxGemvSmem = 200 * 1024;  // dynamic shared memory a GEMV CTA may ask for

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
    int tiles;       // ceil(n_total / kRows)
    const int8_t* xq;   // W4A8 codes
    const float* xs;    // W4A8 scales
    const void* x16;    // W4A16 activations
    const float* awq;   // optional per-column multiplier (W4A16)
    const void* norm_w; // RMSNorm weight of the fused prologue (16-bit, same type as x16)
    float eps;
    int32_t* idot;      // debug: per-block integer dots [n_total, nb]
};

template <int PLANES> struct XTile {
    uint4 lo[PLANES];
    uint4 hi[PLANES];
    float xs;
    int bias;
};

struct WTile {
    uint4 w[kRows];
    float s[kRows];
    int row0;   // global first row of the tile
    int b;      // block index of this lane (may be >= nb: lane idle)
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

__device__ __forceinline__ void load_wtile(const GemvParams& p, int tile, int s, int lane, WTile& t) {
    t.row0 = tile * kRows;
    t.b = s * kWarp + lane;
    const uint8_t* nib;
    const float* sc;
    int lrow, lend;
    locate(p, t.row0, nib, sc, lrow, lend);
    const bool lane_ok = t.b < p.nb;
#pragma unroll
    for (int r = 0; r < kRows; r++) {
        // rows past the end of a matrix are clamped for the load and discarded at the store
        const int row = min(lrow + r, lend - 1);
        if (lane_ok) {
            t.w[r] = ld_stream_u4(nib + (static_cast<long long>(row) * p.nb + t.b) * 16);
            t.s[r] = ld_stream_f32(sc + static_cast<long long>(row) * p.nb + t.b);
        } else {
            t.w[r] = make_uint4(0, 0, 0, 0);
            t.s[r] = 0.0f;
        }
    }
}

template <int PLANES> __device__ __forceinline__ int block_dot(const uint4& w, const XTile<PLANES>& x) {
    const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
    if constexpr (PLANES == 1) {
        const int xl[4] = {(int)x.lo[0].x, (int)x.lo[0].y, (int)x.lo[0].z, (int)x.lo[0].w};
        const int xh[4] = {(int)x.hi[0].x, (int)x.hi[0].y, (int)x.hi[0].z, (int)x.hi[0].w};
        int acc = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc = dp4a_us(wv[j] & 0x0F0F0F0Fu, xl[j], acc);
            acc = dp4a_us((wv[j] >> 4) & 0x0F0F0F0Fu, xh[j], acc);
        }
        return acc - x.bias;
    } else {
        // plane 0: unsigned low bytes, plane 1: signed high bytes of the 16-bit fixed-point activations
        const uint32_t l0[4] = {x.lo[0].x, x.lo[0].y, x.lo[0].z, x.lo[0].w};
        const uint32_t h0[4] = {x.hi[0].x, x.hi[0].y, x.hi[0].z, x.hi[0].w};
        const int l1[4] = {(int)x.lo[1].x, (int)x.lo[1].y, (int)x.lo[1].z, (int)x.lo[1].w};
        const int h1[4] = {(int)x.hi[1].x, (int)x.hi[1].y, (int)x.hi[1].z, (int)x.hi[1].w};
        int acc_lo = 0, acc_hi = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t nl = wv[j] & 0x0F0F0F0Fu;
            const uint32_t nh = (wv[j] >> 4) & 0x0F0F0F0Fu;
            acc_lo = dp4a_uu(nl, l0[j], acc_lo);
            acc_lo = dp4a_uu(nh, h0[j], acc_lo);
            acc_hi = dp4a_us(nl, l1[j], acc_hi);
            acc_hi = dp4a_us(nh, h1[j], acc_hi);
        }
        return acc_hi * 256 + acc_lo - x.bias;
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

static size_t gemv_smem_bytes(int planes, int S) {
    const size_t nbp = static_cast<size_t>(S) * kWarp;
    return nbp * (32 * planes + 8) + kPartFloats * sizeof(float);
}

// Stage the caller's int8 codes (W4A8).
__device__ __forceinline__ void stage_q8(const GemvParams& p, Smem<1>& sm) {
    for (int b = threadIdx.x; b < sm.nbp; b += blockDim.x) {
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
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 8; e++) amax = fmaxf(amax, fabsf(xe[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float scale = amax > 0.0f ? __fdiv_rn(amax, 32767.0f) : 1.0f;
    if (!(amax <= 3.0e38f)) scale = __int_as_float(0x7FC00000);
    const float inv = __fdiv_rn(1.0f, scale);
    uint32_t l0 = 0, l1 = 0, h0 = 0, h1 = 0;
    int sum = 0;
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
    if (active) {
        store_chunk_planes<2>(sm, c, 0, l0, l1);
        store_chunk_planes<2>(sm, c, 1, h0, h1);
        if ((c & 3) == 0) {
            sm.xs[c >> 2] = scale;
            sm.bias[c >> 2] = 8 * sum;
        }
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
    for (int b = p.nb + threadIdx.x; b < sm.nbp; b += blockDim.x) {
#pragma unroll
        for (int q = 0; q < PLANES * 2; q++) sm.plane[q * sm.nbp + b] = make_uint4(0, 0, 0, 0);
        sm.xs[b] = 0.0f;
        sm.bias[b] = 0;
    }
}

// Stage the activations.  PRO = 0: the caller's vector (int8 codes for W4A8, 16-bit values for W4A16).
// PRO = 1: RMSNorm of the caller's 16-bit vector first, in the library's fixed order (256 threads; thread t
// adds x^2 over the 8-element chunks t, t+256, ... ; xor butterfly per warp; warp sums added in ascending
// order; r = 1/sqrt(sum/n + eps); o = round16((x*r)*w)), then quantised exactly as the separate kernels do.
template <int PLANES, int XDT, int PRO> __device__ __forceinline__ void stage_activations(const GemvParams& p,
                                                                                           Smem<PLANES>& sm) {
    zero_padding<PLANES>(p, sm);
    if constexpr (PLANES == 1 && PRO == 0) {
        stage_q8(p, sm);
        return;
    } else {
        const uint16_t* x = static_cast<const uint16_t*>(p.x16);
        const int chunks = p.K >> 3;
        float r = 1.0f;
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
            __syncthreads();
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
                if constexpr (PLANES == 2) {
                    if (p.awq != nullptr) {
#pragma unroll
                        for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], p.awq[c * 8 + e]);
                    }
                }
            }
            if constexpr (PLANES == 1) stage_chunk_q8(sm, c, v, active);
            else stage_chunk_x16(sm, c, v, active);
        }
    }
}

template <int PLANES, int XDT, int ODT, bool IDOT, int PRO>
__global__ void __launch_bounds__(kGemvThreads, 2) gemv_w4_kernel(const GemvParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int W = blockDim.x >> 5;
    const int S = p.S;
    Smem<PLANES> sm(smem_raw, S * kWarp);

    const int tile_begin = static_cast<int>(static_cast<long long>(p.tiles) * blockIdx.x / gridDim.x);
    const int tile_end = static_cast<int>(static_cast<long long>(p.tiles) * (blockIdx.x + 1) / gridDim.x);
    const int chunk_tiles_max = max(1, kPartFloats / (kRows * S));
    const int dt = W / S, ds = W - dt * S;  // task stride W decomposed into (tiles, column sets)

    // Weights do not depend on the producer kernel: start streaming them before waiting for it.
    WTile cur, nxt;
    int t = warp / S, s = warp - (warp / S) * S;  // position inside the current chunk
    int chunk0 = tile_begin;
    int chunk_tiles = min(chunk_tiles_max, tile_end - chunk0);
    if (chunk_tiles > 0 && t < chunk_tiles) load_wtile(p, chunk0 + t, s, lane, cur);

    pdl_wait();
    stage_activations<PLANES, XDT, PRO>(p, sm);
    __syncthreads();
    pdl_launch_dependents();

    while (chunk_tiles > 0) {
        while (t < chunk_tiles) {
            // prefetch the warp's next task of this chunk
            int tn = t + dt, sn = s + ds;
            if (sn >= S) { sn -= S; tn++; }
            if (tn < chunk_tiles) load_wtile(p, chunk0 + tn, sn, lane, nxt);

            XTile<PLANES> x;
            const int bs = s * kWarp + lane;  // < nbp always
#pragma unroll
            for (int pl = 0; pl < PLANES; pl++) {
                x.lo[pl] = sm.plane[(pl * 2 + 0) * sm.nbp + bs];
                x.hi[pl] = sm.plane[(pl * 2 + 1) * sm.nbp + bs];
            }
            x.xs = sm.xs[bs];
            x.bias = sm.bias[bs];

            float a[kRows];
#pragma unroll
            for (int r = 0; r < kRows; r++) {
                const int I = block_dot<PLANES>(cur.w[r], x);
                if constexpr (IDOT) {
                    const int grow = cur.row0 + r;
                    if (grow < p.n_total && cur.b < p.nb) p.idot[static_cast<long long>(grow) * p.nb + cur.b] = I;
                    a[r] = 0.0f;
                } else {
                    a[r] = __fmul_rn(__fmul_rn(cur.s[r], x.xs), static_cast<float>(I));
                }
            }
            if constexpr (!IDOT) {
                warp_sum_multi<kRows>(a, lane);
                if (multi_row_writer<kRows>(lane)) {
                    sm.part[(t * kRows + multi_row_of<kRows>(lane)) * S + s] = a[0];
                }
            }
            cur = nxt;
            t = tn;
            s = sn;
        }
        __syncthreads();
        if constexpr (!IDOT) {
            // add the column-set partials of every row of the chunk in ascending order, then store
            const int rows = chunk_tiles * kRows;
            for (int i = threadIdx.x; i < rows; i += blockDim.x) {
                const int grow = chunk0 * kRows + i;
                if (grow >= p.n_total) continue;
                float y = sm.part[i * S];
                for (int c = 1; c < S; c++) y += sm.part[i * S + c];
                void* out;
                const void* res;
                int lrow;
                if (grow < p.row_end[0]) { out = p.out[0]; res = p.res[0]; lrow = grow; }
                else if (grow < p.row_end[1]) { out = p.out[1]; res = p.res[1]; lrow = grow - p.row_end[0]; }
                else { out = p.out[2]; res = p.res[2]; lrow = grow - p.row_end[1]; }
                if (res != nullptr) {
                    // same bits as a separate GEMV followed by the residual-add kernel
                    float yr = y;
                    if constexpr (ODT == NVE_DT_F16) yr = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(y));
                    if constexpr (ODT == NVE_DT_BF16) yr = Act16<NVE_DT_BF16>::to_f32(Act16<NVE_DT_BF16>::from_f32(y));
                    y = __fadd_rn(load_out<ODT>(res, lrow), yr);
                }
                store_out<ODT>(out, lrow, y);
            }
        }
        // next chunk
        chunk0 += chunk_tiles;
        chunk_tiles = min(chunk_tiles_max, tile_end - chunk0);
        __syncthreads();
        t = warp / S;
        s = warp - t * S;
        if (chunk_tiles > 0 && t < chunk_tiles) load_wtile(p, chunk0 + t, s, lane, cur);
    }
}

// Fallback for weight/activation pointers that are not 16-byte aligned (narrowed tensor views): one warp
// per row, byte loads, same arithmetic and the same summation tree per (row, column set).
template <int PLANES, int XDT, int ODT>
__global__ void gemv_w4_unaligned_kernel(const GemvParams p) {
    const int lane = threadIdx.x & 31;
    const int grow = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (grow >= p.n_total) return;
    const uint8_t* nib;
    const float* sc;
    int lrow, lend;
    locate(p, grow, nib, sc, lrow, lend);
    void* out = grow < p.row_end[0] ? p.out[0] : (grow < p.row_end[1] ? p.out[1] : p.out[2]);
    const void* res = grow < p.row_end[0] ? p.res[0] : (grow < p.row_end[1] ? p.res[1] : p.res[2]);
    float y = 0.0f;
    for (int s = 0; s < p.S; s++) {
        const int b = s * kWarp + lane;
        float v = 0.0f;
        if (b < p.nb) {
            const uint8_t* wb = nib + (static_cast<long long>(lrow) * p.nb + b) * 16;
            int I = 0;
            float xs;
            if constexpr (PLANES == 1) {
                int sum = 0;
                for (int j = 0; j < 16; j++) {
                    const int xl = p.xq[b * 32 + j], xh = p.xq[b * 32 + 16 + j];
                    I += (wb[j] & 0xF) * xl + (wb[j] >> 4) * xh;
                    sum += xl + xh;
                }
                I -= 8 * sum;
                xs = p.xs[b];
            } else {
                const uint16_t* x = static_cast<const uint16_t*>(p.x16);
                float xe[32];
                float amax = 0.0f;
                for (int e = 0; e < 32; e++) {
                    xe[e] = Act16<XDT>::to_f32(x[b * 32 + e]);
                    if (p.awq != nullptr) xe[e] = __fmul_rn(xe[e], p.awq[b * 32 + e]);
                    amax = fmaxf(amax, fabsf(xe[e]));
                }
                float scale = amax > 0.0f ? __fdiv_rn(amax, 32767.0f) : 1.0f;
                if (!(amax <= 3.0e38f)) scale = __int_as_float(0x7FC00000);
                const float inv = __fdiv_rn(1.0f, scale);
                for (int e = 0; e < 32; e++) {
                    int q = __float2int_rn(__fmul_rn(xe[e], inv));
                    q = max(-32767, min(32767, q));
                    const int nibv = (e < 16) ? (wb[e] & 0xF) : (wb[e - 16] >> 4);
                    I += (nibv - 8) * q;
                }
                xs = scale;
            }
            v = __fmul_rn(__fmul_rn(sc[static_cast<long long>(lrow) * p.nb + b], xs), static_cast<float>(I));
        }
        v = warp_sum(v);
        y = (s == 0) ? v : y + v;
    }
    if (lane == 0) {
        if (res != nullptr) {
            float yr = y;
            if constexpr (ODT == NVE_DT_F16) yr = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(y));
            if constexpr (ODT == NVE_DT_BF16) yr = Act16<NVE_DT_BF16>::to_f32(Act16<NVE_DT_BF16>::from_f32(y));
            y = __fadd_rn(load_out<ODT>(res, lrow), yr);
        }
        store_out<ODT>(out, lrow, y);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
template <typename Kern> static int launch_gemv(Kern kern, const GemvParams& p, int planes, cudaStream_t stream) {
    const size_t smem = gemv_smem_bytes(planes, p.S);
    if (smem > static_cast<size_t>(kMaxGemvSmem)) return set_status(NVE_ERR_TOO_LARGE);
    if (smem > 48 * 1024) {
        int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kMaxGemvSmem);
        if (st != NVE_OK) return st;
    }
    int grid = 2 * sm_count();
    if (grid > p.tiles) grid = p.tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    count_launch();
    return set_cuda_status(e);
}

static bool all_aligned(const GemvParams& p, int num_mats, int planes, int pro) {
    for (int m = 0; m < num_mats; m++)
        if (!aligned(p.nib[m], 16)) return false;
    if (pro == 1 && !aligned(p.norm_w, 16)) return false;
    if (planes == 1 && pro == 0) return aligned(p.xq, 16);
    return aligned(p.x16, 16);
}

template <int PLANES, int XDT, int ODT, int PRO> static int dispatch_aligned(const GemvParams& p, int num_mats, cudaStream_t st) {
    if (all_aligned(p, num_mats, PLANES, PRO)) return launch_gemv(gemv_w4_kernel<PLANES, XDT, ODT, false, PRO>, p, PLANES, st);
    if constexpr (PRO != 0) {
        return set_status(NVE_ERR_BAD_ALIGNMENT);  // the fused prologue needs 16-byte aligned vectors
    } else {
        const int wpb = 8;
        gemv_w4_unaligned_kernel<PLANES, XDT, ODT><<<(p.n_total + wpb - 1) / wpb, wpb * 32, 0, st>>>(p);
        count_launch();
        return check_launch();
    }
}

template <int PLANES, int XDT, int PRO> static int dispatch_out(const GemvParams& p, int num_mats, int odt, cudaStream_t st) {
    switch (odt) {
        case NVE_DT_F16: return dispatch_aligned<PLANES, XDT, NVE_DT_F16, PRO>(p, num_mats, st);
        case NVE_DT_BF16: return dispatch_aligned<PLANES, XDT, NVE_DT_BF16, PRO>(p, num_mats, st);
        case NVE_DT_F32: return dispatch_aligned<PLANES, XDT, NVE_DT_F32, PRO>(p, num_mats, st);
        default: return set_status(NVE_ERR_BAD_DTYPE);
    }
}

static int fill_params(GemvParams& p, const nve_b200_w4_matrix* mats, int num_mats, int K) {
    if (mats == nullptr) return NVE_ERR_BAD_POINTER;
    if (num_mats < 1 || num_mats > 3 || K <= 0 || (K % kBlockK) != 0) return NVE_ERR_BAD_SHAPE;
    long long total = 0;
    for (int m = 0; m < 3; m++) {
        if (m < num_mats) {
            if (mats[m].N <= 0) return NVE_ERR_BAD_SHAPE;
            if (!mats[m].nibbles || !mats[m].scales || !mats[m].out) return NVE_ERR_BAD_POINTER;
            // a 4-row tile must not straddle two matrices
            if (num_mats > 1 && m + 1 < num_mats && (mats[m].N % kRows) != 0) return NVE_ERR_BAD_SHAPE;
            total += mats[m].N;
            p.nib[m] = mats[m].nibbles; p.sc[m] = mats[m].scales; p.out[m] = mats[m].out; p.res[m] = mats[m].residual;
        } else {
            p.nib[m] = p.nib[0]; p.sc[m] = p.sc[0]; p.out[m] = p.out[0]; p.res[m] = p.res[0];
        }
        p.row_end[m] = static_cast<int>(total);
    }
    if (total > 0x7FFFFFF0ll) return NVE_ERR_BAD_SHAPE;
    p.n_total = static_cast<int>(total);
    p.K = K;
    p.nb = K / kBlockK;
    p.S = (p.nb + kWarp - 1) / kWarp;
    p.tiles = (p.n_total + kRows - 1) / kRows;
    p.xq = nullptr; p.xs = nullptr; p.x16 = nullptr; p.awq = nullptr; p.idot = nullptr;
    p.norm_w = nullptr; p.eps = 0.0f;
    return NVE_OK;
}

}  // namespace nve

using namespace nve;

extern "C" int nve_b200_matvec_w4a8_multi(const int8_t* xq, const float* xq_scales, const nve_b200_w4_matrix* mats,
                                          int num_mats, int K, int out_dtype, nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mats, num_mats, K);
    if (st != NVE_OK) return set_status(st);
    if (!xq || !xq_scales) return set_status(NVE_ERR_BAD_POINTER);
    p.xq = xq;
    p.xs = xq_scales;
    return dispatch_out<1, NVE_DT_F16, 0>(p, num_mats, out_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_matvec_w4a16_multi(const void* x, int x_dtype, const float* awq, const nve_b200_w4_matrix* mats,
                                           int num_mats, int K, int out_dtype, nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mats, num_mats, K);
    if (st != NVE_OK) return set_status(st);
    if (!x) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = x;
    p.awq = awq;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (x_dtype == NVE_DT_F16) return dispatch_out<2, NVE_DT_F16, 0>(p, num_mats, out_dtype, cs);
    if (x_dtype == NVE_DT_BF16) return dispatch_out<2, NVE_DT_BF16, 0>(p, num_mats, out_dtype, cs);
    return set_status(NVE_ERR_BAD_DTYPE);
}

extern "C" int nve_b200_w4a8_idot(const int8_t* xq, const uint8_t* nibbles, int32_t* I, int N, int K,
                                  nve_stream_t stream) {
    nve_b200_w4_matrix m = {nibbles, reinterpret_cast<const float*>(nibbles), I, nullptr, N};
    GemvParams p;
    int st = fill_params(p, &m, 1, K);
    if (st != NVE_OK) return set_status(st);
    if (!xq || !I) return set_status(NVE_ERR_BAD_POINTER);
    if (!aligned(nibbles, 16) || !aligned(xq, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    p.xq = xq;
    p.xs = nullptr;
    p.idot = I;
    return launch_gemv(gemv_w4_kernel<1, NVE_DT_F16, NVE_DT_F32, true, 0>, p, 1, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_rmsnorm_matvec_w4a8_multi(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                  const nve_b200_w4_matrix* mats, int num_mats, int K, int out_dtype,
                                                  nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mats, num_mats, K);
    if (st != NVE_OK) return set_status(st);
    if (!h || !norm_weight) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = h;
    p.norm_w = norm_weight;
    p.eps = eps;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (act_dtype == NVE_DT_F16) return dispatch_out<1, NVE_DT_F16, 1>(p, num_mats, out_dtype, cs);
    if (act_dtype == NVE_DT_BF16) return dispatch_out<1, NVE_DT_BF16, 1>(p, num_mats, out_dtype, cs);
    return set_status(NVE_ERR_BAD_DTYPE);
}

extern "C" int nve_b200_rmsnorm_matvec_w4a16_multi(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                   const float* awq, const nve_b200_w4_matrix* mats, int num_mats, int K,
                                                   int out_dtype, nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mats, num_mats, K);
    if (st != NVE_OK) return set_status(st);
    if (!h || !norm_weight) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = h;
    p.norm_w = norm_weight;
    p.eps = eps;
    p.awq = awq;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (act_dtype == NVE_DT_F16) return dispatch_out<2, NVE_DT_F16, 1>(p, num_mats, out_dtype, cs);
    if (act_dtype == NVE_DT_BF16) return dispatch_out<2, NVE_DT_BF16, 1>(p, num_mats, out_dtype, cs);
    return set_status(NVE_ERR_BAD_DTYPE);
}

// ---- reference-signature launchers ---------------------------------------------------------------

extern "C" void nve_matvec_w4a8(const int8_t* xq, const float* xq_scales, const uint8_t* nibbles, const float* wt_scales,
                                uint16_t* out, int N, int K, nve_stream_t stream) {
    nve_b200_w4_matrix m = {nibbles, wt_scales, out, nullptr, N};
    nve_b200_matvec_w4a8_multi(xq, xq_scales, &m, 1, K, NVE_DT_F16, stream);
}

extern "C" void nve_matvec_w4a16(const uint16_t* x, const uint8_t* nibbles, const float* scales, const float* awq,
                                 uint16_t* out, int N, int K, nve_stream_t stream) {
    nve_b200_w4_matrix m = {nibbles, scales, out, nullptr, N};
    nve_b200_matvec_w4a16_multi(x, NVE_DT_F16, awq, &m, 1, K, NVE_DT_F16, stream);
}

extern "C" void nve_qkv_matvec_w4a16(const uint16_t* x, const uint8_t* q_nibbles, const float* q_scales,
                                     const float* q_awq, int Nq, const uint8_t* k_nibbles, const float* k_scales,
                                     const float* k_awq, int Nk, const uint8_t* v_nibbles, const float* v_scales,
                                     const float* v_awq, int Nv, uint16_t* q_out, uint16_t* k_out, uint16_t* v_out, int K,
                                     nve_stream_t stream) {
    nve_b200_w4_matrix m[3] = {{q_nibbles, q_scales, q_out, nullptr, Nq},
                               {k_nibbles, k_scales, k_out, nullptr, Nk},
                               {v_nibbles, v_scales, v_out, nullptr, Nv}};
    // One launch when the three matrices share the activation multiplier and tile cleanly; otherwise three.
    const bool same_awq = (q_awq == k_awq) && (k_awq == v_awq);
    if (same_awq && Nq > 0 && Nk > 0 && Nv > 0 && (Nq % kRows) == 0 && (Nk % kRows) == 0) {
        nve_b200_matvec_w4a16_multi(x, NVE_DT_F16, q_awq, m, 3, K, NVE_DT_F16, stream);
        return;
    }
    const float* awqs[3] = {q_awq, k_awq, v_awq};
    for (int i = 0; i < 3; i++) {
        if (m[i].N > 0) nve_b200_matvec_w4a16_multi(x, NVE_DT_F16, awqs[i], &m[i], 1, K, NVE_DT_F16, stream);
    }
}
