// One decoded token through the whole layer stack in ONE persistent kernel.
//
// Replaces, as a single launch, the per-token kernel sequence that src/decode_graph.rs:206-343 records and
// src/gpu_layer.rs:633-997 issues eagerly (RMSNorm, q/k/v GEMV, RoPE, KV write, attention, o_proj, residual,
// RMSNorm, gate/up GEMV, SiLU*up, down GEMV, residual -- per layer), with per-layer W4A8 / W4A16 routing
// (src/gpu_layer.rs:1017-1025) and, optionally, the final RMSNorm + lm_head GEMV that the reference runs on
// the host (src/paged_model.rs:1424-1433).
//
// Design
//   * One CTA of 512 threads per SM, launched cooperatively so that all CTAs are co-resident.  The kernel walks
//     the phases of every layer; kernel boundaries become device-wide barriers (one 64-bit arrival counter,
//     release/acquire, every wait bounded by wall time -> error word, never a hang).
//   * Weights never depend on activations.  Before a CTA waits at the barrier in front of a GEMV phase, each of
//     its warps already has the first weight item of that phase in flight (8 x 128-bit + 8 x 32-bit loads per
//     lane), and a run-ahead stream of bulk L2 prefetches (`cp.async.bulk.prefetch.L2`) keeps DRAM busy across
//     barriers, attention and activation staging: demand loads of a phase then mostly hit L2.
//   * The activation vector of a phase is staged ONCE per SM (not once per 256-thread CTA as the stand-alone
//     GEMV does): RMSNorm + int8 / 16-bit fixed-point conversion into shared-memory planes by 512 threads.
//   * GEMV phases are warp-autonomous: a warp owns whole rows (R rows x all column groups, ascending), so there
//     is no shared-memory partial-sum exchange and no CTA barrier inside a phase.
//   * Arithmetic and summation order are those of the stand-alone kernels (gemv_w4.cu, act_quant.cu,
//     attn_decode.cu: same device functions), so the hidden state equals the six-launch-per-layer graph bit for
//     bit.
//
// Algorithmic bytes per token: every packed weight once (0.625 B per weight) + the valid K/V prefix once.
#include <algorithm>

#include "attn_core.cuh"
#include "gemv_w4.cuh"

namespace nve {

constexpr int kDsThreads = 512;
constexpr int kDsWarps = kDsThreads / 32;
constexpr unsigned long long kDsWaitNs = 100ull * 1000 * 1000;  // bound of every device-wide wait (wall time)

// Workspace carved out of the caller's buffer (offsets fixed by ds_layout()).
struct DsWork {
    unsigned long long* bar;  // arrival counter of the device-wide barrier (monotonic)
    int* err;                 // 0, or NVE_DS_ERR_* latched by an expired wait
    uint16_t* q;              // [nh*hd] f16
    uint16_t* k;              // [nkv*hd]
    uint16_t* v;
    void* parts;              // attention partials: [virtual clusters][kAdRanks] AdCtaPartial<hd, 2>
    uint16_t* attn;           // [nh*hd] f16
    int8_t* xq_a;             // int8 codes of attn (W4A8 route)
    float* xs_a;
    uint16_t* gate;           // [ffn] f16
    uint16_t* up;
    int8_t* xq_f;             // codes (W4A8) or high bytes (W4A16 fixed point) of silu(gate)*up
    uint8_t* xlo_f;           // low bytes (W4A16)
    float* xs_f;
};

struct DsParams {
    nve_b200_decode_model m;
    const nve_b200_decode_layer* layers;  // device array [num_layers]
    uint16_t* hidden;                     // [hidden] f16, updated in place
    const int* d_pos;
    const int* d_seq_len;
    DsWork w;
    unsigned long long wait_ns;
    long long pf_bytes;  // run-ahead distance of the L2 prefetch stream (0 = off)
    unsigned long long* trace;  // debugging aid: per phase 4 globaltimer stamps of CTA 0 and of the last CTA, or NULL
};

// ---------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned long long ds_globaltimer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Device-wide barrier: every CTA arrives once, thread 0 polls until all have.  The wait is bounded by wall
// time; when it expires (or another CTA's did) the error word is set and nothing waits any more, so the kernel
// runs to its end (with meaningless results) instead of hanging.
__device__ __forceinline__ void grid_barrier(const DsParams& p, unsigned long long& target) {
    target += gridDim.x;
    __syncthreads();
    if (threadIdx.x == 0) {
        red_release_add_u64(p.w.bar, 1ull);
        if (*reinterpret_cast<volatile int*>(p.w.err) == 0) {
            const unsigned long long t0 = ds_globaltimer();
            unsigned spins = 0;
            while (ld_acquire_u64(p.w.bar) < target) {
                if ((++spins & 63u) == 0u) {
                    if (*reinterpret_cast<volatile int*>(p.w.err) != 0) break;
                    if (ds_globaltimer() - t0 > p.wait_ns) {
                        atomicCAS(p.w.err, 0, NVE_ERR_TIMEOUT);
                        break;
                    }
                }
            }
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------------
// GEMV phase
// ---------------------------------------------------------------------------------------------
enum { kEpiF16 = 0, kEpiResidual = 1, kEpiF32 = 2 };

struct PhaseMats {
    const uint8_t* nib[3];
    const float* sc[3];
    void* out[3];
    int row_end[3];
    int n_total;
    int K, nb, S;
    int epi;
    int planes;  // 1 = W4A8, 2 = W4A16
};

struct WFlat {  // one warp item: R rows x C column sets (R*C = 8 blocks per lane), index c*R + r
    uint4 w[8];
    float s[8];
};

__device__ __forceinline__ int pm_rows_per_tile(const PhaseMats& pm) { return pm.S >= 3 ? 2 : (pm.S == 2 ? 4 : 8); }

__device__ __forceinline__ void pm_locate(const PhaseMats& pm, int grow, const uint8_t*& nib, const float*& sc, int& lrow,
                                          int& lend, int& mat) {
    if (grow < pm.row_end[0]) {
        nib = pm.nib[0]; sc = pm.sc[0]; lrow = grow; lend = pm.row_end[0]; mat = 0;
    } else if (grow < pm.row_end[1]) {
        nib = pm.nib[1]; sc = pm.sc[1]; lrow = grow - pm.row_end[0]; lend = pm.row_end[1] - pm.row_end[0]; mat = 1;
    } else {
        nib = pm.nib[2]; sc = pm.sc[2]; lrow = grow - pm.row_end[1]; lend = pm.row_end[2] - pm.row_end[1]; mat = 2;
    }
}

template <int R, int C>
__device__ __forceinline__ void ds_load_item(const PhaseMats& pm, int tile, int cg, int lane, WFlat& t) {
    const uint8_t* nib;
    const float* sc;
    int lrow, lend, mat;
    pm_locate(pm, tile * R, nib, sc, lrow, lend, mat);
#pragma unroll
    for (int r = 0; r < R; r++) {
        // rows past the end of a matrix are clamped for the load and discarded at the store
        const long long rb = static_cast<long long>(min(lrow + r, lend - 1)) * pm.nb;
#pragma unroll
        for (int c = 0; c < C; c++) {
            const int b = (cg * C + c) * kWarp + lane;
            if (b < pm.nb) {
                t.w[c * R + r] = ld_stream_u4(nib + (rb + b) * 16);
                t.s[c * R + r] = ld_stream_f32(sc + rb + b);
            } else {
                t.w[c * R + r] = make_uint4(0, 0, 0, 0);
                t.s[c * R + r] = 0.0f;
            }
        }
    }
}

// Tile range of this CTA for a phase.
__device__ __forceinline__ void pm_cta_tiles(const PhaseMats& pm, int& tb, int& te) {
    const int R = pm_rows_per_tile(pm);
    const int tiles = (pm.n_total + R - 1) / R;
    tb = static_cast<int>(static_cast<long long>(tiles) * blockIdx.x / gridDim.x);
    te = static_cast<int>(static_cast<long long>(tiles) * (blockIdx.x + 1) / gridDim.x);
}

// First item of this warp for the phase (issued before the barrier in front of the phase).
__device__ __forceinline__ void pm_load_first(const PhaseMats& pm, int warp, int lane, WFlat& it) {
    int tb, te;
    pm_cta_tiles(pm, tb, te);
    const int t = tb + warp;
    if (t >= te) return;
    if (pm.S >= 3) ds_load_item<2, 4>(pm, t, 0, lane, it);
    else if (pm.S == 2) ds_load_item<4, 2>(pm, t, 0, lane, it);
    else ds_load_item<8, 1>(pm, t, 0, lane, it);
}

template <int PLANES, int R, int C>
__device__ __forceinline__ void ds_run_gemv(const PhaseMats& pm, Smem<PLANES>& sm, const uint16_t* residual, int warp,
                                            int lane, WFlat& it) {
    const int S = pm.S;
    const int CG = (S + C - 1) / C;
    int tb, te;
    pm_cta_tiles(pm, tb, te);
    for (int t = tb + warp; t < te; t += kDsWarps) {
        float y = 0.0f;
        for (int cg = 0; cg < CG; cg++) {
            float a[R];
#pragma unroll
            for (int c = 0; c < C; c++) {
                const int bs = min((cg * C + c), S - 1) * kWarp + lane;  // < nbp; idle column sets carry zero weights
                XTile<PLANES> x;
#pragma unroll
                for (int pl = 0; pl < PLANES; pl++) {
                    x.lo[pl] = sm.plane[(pl * 2 + 0) * sm.nbp + bs];
                    x.hi[pl] = sm.plane[(pl * 2 + 1) * sm.nbp + bs];
                }
                x.xs = sm.xs[bs];
                x.bias = sm.bias[bs];
                const bool live = (cg * C + c) < S;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const int I = block_dot<PLANES>(it.w[c * R + r], x);
                    // per lane the C column sets of the group are added in ascending order, first term exact
                    const float v = live ? __fmul_rn(__fmul_rn(it.s[c * R + r], x.xs), static_cast<float>(I)) : 0.0f;
                    a[r] = (c == 0) ? v : __fadd_rn(a[r], v);
                }
            }
            // issue the next item's loads before reducing this one
            if (cg + 1 < CG) ds_load_item<R, C>(pm, t, cg + 1, lane, it);
            else if (t + kDsWarps < te) ds_load_item<R, C>(pm, t + kDsWarps, 0, lane, it);
            warp_sum_multi<R>(a, lane);
            y = (cg == 0) ? a[0] : __fadd_rn(y, a[0]);  // column groups of a row in ascending order
        }
        if (multi_row_writer<R>(lane)) {
            const int grow = t * R + multi_row_of<R>(lane);
            if (grow < pm.n_total) {
                const uint8_t* nib;
                const float* sc;
                int lrow, lend, mat;
                pm_locate(pm, grow, nib, sc, lrow, lend, mat);
                if (pm.epi == kEpiResidual) {
                    // same bits as a GEMV with f16 output followed by the residual-add kernel
                    const float yr = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(y));
                    const float h = __fadd_rn(Act16<NVE_DT_F16>::to_f32(__ldcg(residual + lrow)), yr);
                    static_cast<uint16_t*>(pm.out[mat])[lrow] = Act16<NVE_DT_F16>::from_f32(h);
                } else if (pm.epi == kEpiF32) {
                    static_cast<float*>(pm.out[mat])[lrow] = y;
                } else {
                    static_cast<uint16_t*>(pm.out[mat])[lrow] = Act16<NVE_DT_F16>::from_f32(y);
                }
            }
        }
    }
}

template <int PLANES>
__device__ __forceinline__ void ds_run_gemv_rc(const PhaseMats& pm, unsigned char* smem_raw, const uint16_t* residual,
                                               int warp, int lane, WFlat& it) {
    Smem<PLANES> sm(smem_raw, pm.S * kWarp);
    if (pm.S >= 3) ds_run_gemv<PLANES, 2, 4>(pm, sm, residual, warp, lane, it);
    else if (pm.S == 2) ds_run_gemv<PLANES, 4, 2>(pm, sm, residual, warp, lane, it);
    else ds_run_gemv<PLANES, 8, 1>(pm, sm, residual, warp, lane, it);
}

// ---------------------------------------------------------------------------------------------
// Activation staging by the 512 threads of the CTA (same arithmetic as gemv_w4.cuh stage_activations)
// ---------------------------------------------------------------------------------------------
template <int PLANES> __device__ __forceinline__ void ds_zero_padding(int nb, Smem<PLANES>& sm) {
    for (int b = nb + threadIdx.x; b < sm.nbp; b += kDsThreads) {
#pragma unroll
        for (int q = 0; q < PLANES * 2; q++) sm.plane[q * sm.nbp + b] = make_uint4(0, 0, 0, 0);
        sm.xs[b] = 0.0f;
        sm.bias[b] = 0;
    }
}

__device__ __forceinline__ void ds_load8(const uint16_t* p, int c, uint16_t (&h)[8]) {
    unpack8(__ldcg(reinterpret_cast<const uint4*>(p) + c), h);
}

constexpr int kDsStageIters = 2;                            // 8-element chunks per thread held in registers
constexpr int kDsMaxStageK = kDsStageIters * kDsThreads * 8;  // 8192: largest K of a 16-bit staged vector

// RMSNorm of x (K values, f16) in the library's fixed order, then int8 codes (PLANES 1) or 16-bit fixed-point
// planes (PLANES 2, after the optional awq multiply).  NORM = false: no normalisation (x is staged as it is).
// The vector is read once: every thread keeps its chunks in registers for the second pass and leaves a copy in
// `stash` so that the first 256 threads can take the sum of squares in the stand-alone kernel's order.
template <int PLANES, bool NORM>
__device__ __forceinline__ void ds_stage_f16(const uint16_t* x, const uint16_t* norm_w, float eps, const float* awq, int K,
                                             Smem<PLANES>& sm, float* warp_part, uint4* stash) {
    ds_zero_padding<PLANES>(K / kBlockK, sm);
    const int chunks = K >> 3;
    const int iters = (chunks + kDsThreads - 1) / kDsThreads;  // <= kDsStageIters (checked by the launcher)
    uint4 xr[kDsStageIters], wr[kDsStageIters];
#pragma unroll
    for (int it = 0; it < kDsStageIters; it++) {
        const int c = it * kDsThreads + threadIdx.x;
        xr[it] = make_uint4(0, 0, 0, 0);
        wr[it] = make_uint4(0, 0, 0, 0);
        if (it < iters && c < chunks) {
            xr[it] = __ldcg(reinterpret_cast<const uint4*>(x) + c);
            if constexpr (NORM) wr[it] = __ldg(reinterpret_cast<const uint4*>(norm_w) + c);
        }
    }
    float r = 1.0f;
    if constexpr (NORM) {
#pragma unroll
        for (int it = 0; it < kDsStageIters; it++) {
            const int c = it * kDsThreads + threadIdx.x;
            if (it < iters && c < chunks) stash[c] = xr[it];
        }
        __syncthreads();
        // sum of squares: thread t < 256 adds the chunks t, t+256, ... (fma chain, ascending), xor butterfly per
        // warp, the 8 warp sums in ascending order -- the order of the stand-alone RMSNorm kernel
        float acc = 0.0f;
        if (threadIdx.x < kGemvThreads) {
            for (int c = threadIdx.x; c < chunks; c += kGemvThreads) {
                uint16_t h[8];
                unpack8(stash[c], h);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const float v = Act16<NVE_DT_F16>::to_f32(h[e]);
                    acc = __fmaf_rn(v, v, acc);
                }
            }
        }
        acc = warp_sum(acc);
        if (threadIdx.x < kGemvThreads && (threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
        __syncthreads();
        float total = warp_part[0];
#pragma unroll
        for (int w = 1; w < kGemvThreads / 32; w++) total = __fadd_rn(total, warp_part[w]);
        r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(K)), eps)));
    }
#pragma unroll
    for (int it = 0; it < kDsStageIters; it++) {
        if (it < iters) {  // uniform over the CTA: the quad shuffles inside stage_chunk_* need whole warps
            const int c = it * kDsThreads + threadIdx.x;
            const bool active = c < chunks;
            float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (active) {
                uint16_t h[8];
                unpack8(xr[it], h);
                if constexpr (NORM) {
                    uint16_t hw[8];
                    unpack8(wr[it], hw);
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const float o = __fmul_rn(__fmul_rn(Act16<NVE_DT_F16>::to_f32(h[e]), r), Act16<NVE_DT_F16>::to_f32(hw[e]));
                        v[e] = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(o));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = Act16<NVE_DT_F16>::to_f32(h[e]);
                }
                if constexpr (PLANES == 2) {
                    if (awq != nullptr) {
#pragma unroll
                        for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], __ldg(awq + c * 8 + e));
                    }
                }
            }
            if constexpr (PLANES == 1) stage_chunk_q8(sm, c, v, active);
            else stage_chunk_x16(sm, c, v, active);
        }
    }
}

// int8 codes + scales written by an earlier phase (W4A8 o_proj / down_proj input).
__device__ __forceinline__ void ds_stage_q8(const int8_t* xq, const float* xs, int K, Smem<1>& sm) {
    const int nb = K / kBlockK;
    ds_zero_padding<1>(nb, sm);
    for (int b = threadIdx.x; b < nb; b += kDsThreads) {
        const uint4* src = reinterpret_cast<const uint4*>(xq + static_cast<long long>(b) * 32);
        const uint4 lo = __ldcg(src), hi = __ldcg(src + 1);
        int sum = 0;
        sum = __dp4a((int)lo.x, 0x01010101, sum); sum = __dp4a((int)lo.y, 0x01010101, sum);
        sum = __dp4a((int)lo.z, 0x01010101, sum); sum = __dp4a((int)lo.w, 0x01010101, sum);
        sum = __dp4a((int)hi.x, 0x01010101, sum); sum = __dp4a((int)hi.y, 0x01010101, sum);
        sum = __dp4a((int)hi.z, 0x01010101, sum); sum = __dp4a((int)hi.w, 0x01010101, sum);
        sm.plane[b] = lo;
        sm.plane[sm.nbp + b] = hi;
        sm.xs[b] = __ldcg(xs + b);
        sm.bias[b] = 8 * sum;
    }
}

// 16-bit fixed-point planes written by the SiLU phase (W4A16 down_proj input).
__device__ __forceinline__ void ds_stage_x16_planes(const uint8_t* xlo, const int8_t* xhi, const float* xs, int K,
                                                    Smem<2>& sm) {
    const int nb = K / kBlockK;
    ds_zero_padding<2>(nb, sm);
    for (int b = threadIdx.x; b < nb; b += kDsThreads) {
        const uint4* lo = reinterpret_cast<const uint4*>(xlo + static_cast<long long>(b) * 32);
        const uint4* hi = reinterpret_cast<const uint4*>(xhi + static_cast<long long>(b) * 32);
        const uint4 l0 = __ldcg(lo), l1 = __ldcg(lo + 1), h0 = __ldcg(hi), h1 = __ldcg(hi + 1);
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
        sm.xs[b] = __ldcg(xs + b);
        sm.bias[b] = 8 * (sh * 256 + ul);
    }
}

// ---------------------------------------------------------------------------------------------
// SiLU*up -> int8 codes (W4A8) or fixed-point planes (W4A16), spread over the grid one warp (32 chunks) at a time
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void ds_silu_phase(const DsParams& p, const nve_b200_decode_layer& ly, int warp, int lane) {
    const int n = p.m.ffn;
    const int chunks = n >> 3;
    const int warp_chunks = (chunks + 31) / 32;
    const float* awq = ly.awq[3];
    for (int j = warp * gridDim.x + blockIdx.x; j < warp_chunks; j += kDsWarps * gridDim.x) {
        const int c = j * 32 + lane;
        const bool active = c < chunks;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (active) {
            uint16_t hg[8], hu[8];
            ds_load8(p.w.gate, c, hg);
            ds_load8(p.w.up, c, hu);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const uint16_t ho = Act16<NVE_DT_F16>::from_f32(
                    silu_mul_f32(Act16<NVE_DT_F16>::to_f32(hg[e]), Act16<NVE_DT_F16>::to_f32(hu[e])));
                v[e] = Act16<NVE_DT_F16>::to_f32(ho);
            }
        }
        if (ly.use_w4a8) {
            quantize_quad(v, p.w.xq_f, p.w.xs_f, c, active);
        } else {
            if (active && awq != nullptr) {
#pragma unroll
                for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], __ldg(awq + c * 8 + e));
            }
            x16_quad(v, p.w.xlo_f, p.w.xq_f, p.w.xs_f, c, active);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Attention: partial pass (RoPE + KV write + per-slice online softmax) and the merge of the slices
// ---------------------------------------------------------------------------------------------
// A CTA runs two virtual CTAs of 256 threads side by side: the two query-head pairs 2u, 2u+1 on the same position
// slice (for the usual group size 4 they share the KV head, so the second reader hits L1/L2).
template <int HD>
__device__ __forceinline__ void ds_attn_partial(const DsParams& p, const nve_b200_decode_layer& ly, unsigned char* smem_raw,
                                                int seq_len, int pos) {
    constexpr int QH = 2;
    constexpr int DC = HD / 8;
    AdShared<HD, QH>* shs = reinterpret_cast<AdShared<HD, QH>*>(smem_raw);
    const int half = threadIdx.x / kAdThreads, tid = threadIdx.x % kAdThreads;
    AdShared<HD, QH>& sh = shs[half];
    const int groups = p.m.num_heads / p.m.num_kv_heads;
    const int clusters_per_kv = groups / QH;
    const int nvc = p.m.num_heads / QH;  // virtual clusters
    const int units = ((nvc + 1) / 2) * kAdRanks;
    const bool pos_ok = pos >= 0 && pos < p.m.max_seq;
    const int chunk = (seq_len + kAdRanks - 1) / kAdRanks;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int rank = u % kAdRanks;
        const int vc = (u / kAdRanks) * 2 + half;
        const bool live = vc < nvc;
        const int vcc = live ? vc : nvc - 1;  // an idle half repeats the last cluster's work and discards it
        const int kvh = vcc / clusters_per_kv;
        const int h0 = kvh * groups + (vcc % clusters_per_kv) * QH;
        const uint16_t* kh = ly.k_cache + static_cast<long long>(kvh) * p.m.max_seq * HD;
        const uint16_t* vh = ly.v_cache + static_cast<long long>(kvh) * p.m.max_seq * HD;
        attn_stage_q<HD, QH, true>(sh, tid, p.w.q, p.w.k, p.w.v, p.m.rope_cos, p.m.rope_sin, h0, kvh, pos, pos_ok);
        __syncthreads();
        const int t_begin = rank * chunk;
        const int t_end = min(seq_len, t_begin + chunk);
        if (live && pos_ok && rank == 0 && (vcc % clusters_per_kv) == 0 && tid < 2 * DC) {
            const int which = tid / DC, d = tid % DC;
            uint16_t* dst = (which == 0 ? ly.k_cache : ly.v_cache) + (static_cast<long long>(kvh) * p.m.max_seq + pos) * HD;
            reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(which == 0 ? sh.knew_s : sh.vnew_s)[d];
        }
        AdCtaPartial<HD, QH>* dst = static_cast<AdCtaPartial<HD, QH>*>(p.w.parts) + (static_cast<long long>(vcc) * kAdRanks + rank);
        attn_partial<HD, QH, true, false>(
            sh, tid, kh, vh, t_begin, t_end, pos, p.m.attn_scale, false, nullptr, [] { __syncthreads(); },
            [&](int h, int d, float mm, float ss, float a) {
                if (live) {
                    dst->acc[h][d] = a;
                    if (d == 0) { dst->m[h] = mm; dst->s[h] = ss; }
                }
            });
        __syncthreads();  // shared memory is reused by the next unit
    }
}

template <int HD>
__device__ __forceinline__ void ds_attn_merge(const DsParams& p, const nve_b200_decode_layer& ly) {
    constexpr int QH = 2;
    const int nvc = p.m.num_heads / QH;
    const int groups = p.m.num_heads / p.m.num_kv_heads;
    const int clusters_per_kv = groups / QH;
    for (int vc = blockIdx.x; vc < nvc; vc += gridDim.x) {
        const int kvh = vc / clusters_per_kv;
        const int h0 = kvh * groups + (vc % clusters_per_kv) * QH;
        const AdCtaPartial<HD, QH>* parts = static_cast<const AdCtaPartial<HD, QH>*>(p.w.parts) + static_cast<long long>(vc) * kAdRanks;
        for (int i = threadIdx.x; i < QH * HD; i += kDsThreads) {
            const int h = i / HD, d = i % HD;
            const uint16_t o16 = attn_merge_ranks<HD, QH>(parts, h, d);
            const long long oi = static_cast<long long>(h0 + h) * HD + d;
            p.w.attn[oi] = o16;
            if (ly.use_w4a8) {
                float scale;
                const int qv = attn_quantize_lane(o16, scale);
                p.w.xq_a[oi] = static_cast<int8_t>(qv);
                if ((threadIdx.x & 31) == 0) p.w.xs_a[oi >> 5] = scale;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Phase table
// ---------------------------------------------------------------------------------------------
enum { kPhQkv = 0, kPhAttn = 1, kPhMerge = 2, kPhO = 3, kPhGateUp = 4, kPhSilu = 5, kPhDown = 6, kPhPerLayer = 7 };

__device__ __forceinline__ bool ph_is_gemv(int kind) { return kind == kPhQkv || kind == kPhO || kind == kPhGateUp || kind == kPhDown; }

// Matrices of GEMV phase `kind` of layer `ly` (kind < 0: the lm_head).
__device__ __forceinline__ void pm_set(PhaseMats& pm, int m, const nve_b200_decode_layer* ly, int proj, void* out, int row_end) {
    pm.nib[m] = ly->nibbles[proj];
    pm.sc[m] = ly->scales[proj];
    pm.out[m] = out;
    pm.row_end[m] = row_end;
}

__device__ __forceinline__ void pm_build(const DsParams& p, const nve_b200_decode_layer* ly, int kind, PhaseMats& pm) {
    const int qd = p.m.num_heads * p.m.head_dim, kvd = p.m.num_kv_heads * p.m.head_dim;
    int K = p.m.hidden;
    pm.epi = kEpiF16;
    if (kind < 0) {
        pm.nib[0] = pm.nib[1] = pm.nib[2] = p.m.lm_nibbles;
        pm.sc[0] = pm.sc[1] = pm.sc[2] = p.m.lm_scales;
        pm.out[0] = pm.out[1] = pm.out[2] = p.m.logits;
        pm.row_end[0] = pm.row_end[1] = pm.row_end[2] = p.m.vocab;
        pm.epi = kEpiF32;
        pm.planes = p.m.lm_use_w4a8 ? 1 : 2;
    } else {
        if (kind == kPhQkv) {
            pm_set(pm, 0, ly, 0, p.w.q, qd);
            pm_set(pm, 1, ly, 1, p.w.k, qd + kvd);
            pm_set(pm, 2, ly, 2, p.w.v, qd + 2 * kvd);
        } else if (kind == kPhGateUp) {
            pm_set(pm, 0, ly, 4, p.w.gate, p.m.ffn);
            pm_set(pm, 1, ly, 5, p.w.up, 2 * p.m.ffn);
            pm_set(pm, 2, ly, 5, p.w.up, 2 * p.m.ffn);
        } else {
            const int proj = kind == kPhO ? 3 : 6;
            K = kind == kPhO ? qd : p.m.ffn;
            pm_set(pm, 0, ly, proj, p.hidden, p.m.hidden);
            pm_set(pm, 1, ly, proj, p.hidden, p.m.hidden);
            pm_set(pm, 2, ly, proj, p.hidden, p.m.hidden);
            pm.epi = kEpiResidual;
        }
        pm.planes = ly->use_w4a8 ? 1 : 2;
    }
    pm.n_total = pm.row_end[2];
    pm.K = K;
    pm.nb = K / kBlockK;
    pm.S = (pm.nb + kWarp - 1) / kWarp;
}

// ---------------------------------------------------------------------------------------------
// L2 prefetch stream: the GEMV phases in execution order form one byte stream; at the start of GEMV phase g every
// CTA makes sure that its own share of the stream up to `pf_bytes` beyond the end of phase g has been requested.
// A phase is cut into kPfSlabs slabs of each CTA's tile range; all CTAs advance the same (uniform) frontier.
// ---------------------------------------------------------------------------------------------
constexpr int kPfSlabs = 8;

struct PfState {
    int s;            // frontier: global slab index (GEMV index * kPfSlabs + slab)
    long long ahead;  // bytes of the stream requested beyond the end of the phase that is running
};

__device__ __forceinline__ long long pm_bytes(const PhaseMats& pm) {
    return static_cast<long long>(pm.n_total) * pm.nb * 20;  // 16 nibble bytes + one f32 scale per block
}

// Bytes of GEMV phase g (uniform arithmetic on the model's dimensions).
__device__ __forceinline__ long long pf_phase_bytes(const DsParams& p, int g) {
    const long long qd = static_cast<long long>(p.m.num_heads) * p.m.head_dim, kvd = static_cast<long long>(p.m.num_kv_heads) * p.m.head_dim;
    const long long H = p.m.hidden, F = p.m.ffn;
    if (g >= p.m.num_layers * 4) return static_cast<long long>(p.m.vocab) * H / 32 * 20;
    switch (g & 3) {
        case 0: return (qd + 2 * kvd) * H / 32 * 20;
        case 1: return H * qd / 32 * 20;
        case 2: return 2 * F * H / 32 * 20;
        default: return H * F / 32 * 20;
    }
}

__device__ __forceinline__ void pf_issue_slab(const PhaseMats& pm, int slab) {
    int tb, te;
    pm_cta_tiles(pm, tb, te);
    const int R = pm_rows_per_tile(pm);
    const int t0 = tb + static_cast<int>(static_cast<long long>(te - tb) * slab / kPfSlabs);
    const int t1 = tb + static_cast<int>(static_cast<long long>(te - tb) * (slab + 1) / kPfSlabs);
    const int r0 = t0 * R, r1 = min(t1 * R, pm.n_total);
    int mat_begin = 0;
#pragma unroll
    for (int m = 0; m < 3; m++) {
        const int mat_end = pm.row_end[m];
        const int a = max(r0, mat_begin), b = min(r1, mat_end);
        if (a < b) {
            const long long row0 = a - mat_begin, rows = b - a;
            const unsigned char* nb0 = pm.nib[m] + row0 * pm.nb * 16;
            l2_prefetch_bulk(nb0, static_cast<unsigned>(rows * pm.nb * 16));
            // scale rows are nb*4 bytes: round the range inwards to 16-byte boundaries
            const uintptr_t s0 = reinterpret_cast<uintptr_t>(pm.sc[m] + row0 * pm.nb);
            const uintptr_t s1 = s0 + static_cast<uintptr_t>(rows) * pm.nb * 4;
            const uintptr_t sa = (s0 + 15) & ~static_cast<uintptr_t>(15), sb = s1 & ~static_cast<uintptr_t>(15);
            if (sb > sa) l2_prefetch_bulk(reinterpret_cast<const void*>(sa), static_cast<unsigned>(sb - sa));
        }
        mat_begin = mat_end;
    }
}

// Called by one whole warp per CTA when GEMV phase g starts: the (uniform) frontier moves until `pf_bytes` of the
// stream beyond the end of phase g have been requested; the lanes issue the new slabs side by side.
__device__ __forceinline__ void pf_advance(const DsParams& p, PfState& pf, int g, int total_gemvs, int lane) {
    if (p.pf_bytes <= 0) return;
    if (pf.s < (g + 1) * kPfSlabs) {  // the frontier fell behind the running phase: restart right after it
        pf.s = (g + 1) * kPfSlabs;
        pf.ahead = 0;
    }
    const int s_begin = pf.s;
    while (pf.s < total_gemvs * kPfSlabs && pf.ahead < p.pf_bytes) {
        pf.ahead += pf_phase_bytes(p, pf.s / kPfSlabs) / kPfSlabs;
        pf.s++;
    }
    for (int s = s_begin + lane; s < pf.s; s += 32) {
        const int fg = s / kPfSlabs;
        PhaseMats pm;
        const int layer = fg / 4;
        if (layer < p.m.num_layers) {
            const int kind = (fg & 3) == 0 ? kPhQkv : ((fg & 3) == 1 ? kPhO : ((fg & 3) == 2 ? kPhGateUp : kPhDown));
            pm_build(p, p.layers + layer, kind, pm);
        } else {
            pm_build(p, nullptr, -1, pm);
        }
        pf_issue_slab(pm, s % kPfSlabs);
    }
}

// When phase g_next - 1 ends, the requested bytes of phase g_next stop counting as "ahead".
__device__ __forceinline__ void pf_retire(const DsParams& p, PfState& pf, int g_next) {
    const long long nb = pf_phase_bytes(p, g_next);
    const int done = pf.s - g_next * kPfSlabs;  // slabs of phase g_next already requested
    if (done >= kPfSlabs) pf.ahead -= nb;
    else if (done > 0) pf.ahead -= nb / kPfSlabs * done;
    if (pf.ahead < 0) pf.ahead = 0;
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(kDsThreads, 1) decode_step_kernel(const DsParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float warp_part[kGemvThreads / 32];
    __shared__ uint4 stash[kDsMaxStageK / 8];
    __shared__ unsigned long long bar_base_s;
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) bar_base_s = (ld_acquire_u64(p.w.bar) / gridDim.x) * gridDim.x;
    __syncthreads();
    unsigned long long bar_target = bar_base_s;

    int seq_len = *reinterpret_cast<const volatile int*>(p.d_seq_len);
    seq_len = max(0, min(seq_len, p.m.max_seq));
    const int pos = *reinterpret_cast<const volatile int*>(p.d_pos);

    const bool has_head = p.m.lm_nibbles != nullptr;
    const int layer_phases = p.m.num_layers * kPhPerLayer;
    const int total_phases = layer_phases + (has_head ? 1 : 0);
    const int total_gemvs = p.m.num_layers * 4 + (has_head ? 1 : 0);

    PfState pf = {0, 0};
    PhaseMats pm;
    WFlat item;
    pm_build(p, p.layers, kPhQkv, pm);
    pm_load_first(pm, warp, lane, item);
    int g = 0;  // index of the next GEMV phase

    for (int ph = 0; ph < total_phases; ph++) {
        const int layer = ph / kPhPerLayer;
        const int kind = ph < layer_phases ? ph % kPhPerLayer : -1;
        const nve_b200_decode_layer* ly = p.layers + min(layer, p.m.num_layers - 1);
        const bool tracer = p.trace != nullptr && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1);
        unsigned long long* tr = tracer ? p.trace + (static_cast<size_t>(blockIdx.x == 0 ? 0 : 1) * total_phases + ph) * 4 : nullptr;
        if (tracer) tr[0] = ds_globaltimer();
        if (ph > 0) grid_barrier(p, bar_target);
        if (tracer) tr[1] = ds_globaltimer();
        if (kind < 0 || ph_is_gemv(kind)) {
            // ---- stage the activation vector of the phase once for this SM
            const uint16_t* residual = nullptr;
            if (kind == kPhQkv || kind == kPhGateUp || kind < 0) {
                const uint16_t* nw = kind == kPhQkv ? ly->input_norm : (kind == kPhGateUp ? ly->post_attn_norm : p.m.final_norm);
                const float* awq = kind < 0 ? nullptr : ly->awq[kind == kPhQkv ? 0 : 2];
                if (pm.planes == 1) {
                    Smem<1> sm(smem_raw, pm.S * kWarp);
                    ds_stage_f16<1, true>(p.hidden, nw, p.m.norm_eps, nullptr, pm.K, sm, warp_part, stash);
                } else {
                    Smem<2> sm(smem_raw, pm.S * kWarp);
                    ds_stage_f16<2, true>(p.hidden, nw, p.m.norm_eps, awq, pm.K, sm, warp_part, stash);
                }
            } else if (kind == kPhO) {
                residual = p.hidden;
                if (pm.planes == 1) {
                    Smem<1> sm(smem_raw, pm.S * kWarp);
                    ds_stage_q8(p.w.xq_a, p.w.xs_a, pm.K, sm);
                } else {
                    Smem<2> sm(smem_raw, pm.S * kWarp);
                    ds_stage_f16<2, false>(p.w.attn, nullptr, 0.0f, ly->awq[1], pm.K, sm, warp_part, stash);
                }
            } else {  // down_proj
                residual = p.hidden;
                if (pm.planes == 1) {
                    Smem<1> sm(smem_raw, pm.S * kWarp);
                    ds_stage_q8(p.w.xq_f, p.w.xs_f, pm.K, sm);
                } else {
                    Smem<2> sm(smem_raw, pm.S * kWarp);
                    ds_stage_x16_planes(p.w.xlo_f, p.w.xq_f, p.w.xs_f, pm.K, sm);
                }
            }
            __syncthreads();
            if (tracer) tr[2] = ds_globaltimer();
            if (warp == kDsWarps - 1) pf_advance(p, pf, g, total_gemvs, lane);
            if (pm.planes == 1) ds_run_gemv_rc<1>(pm, smem_raw, residual, warp, lane, item);
            else ds_run_gemv_rc<2>(pm, smem_raw, residual, warp, lane, item);
            g++;
        } else if (kind == kPhAttn) {
            ds_attn_partial<HD>(p, *ly, smem_raw, seq_len, pos);
        } else if (kind == kPhMerge) {
            ds_attn_merge<HD>(p, *ly);
        } else {  // kPhSilu
            ds_silu_phase(p, *ly, warp, lane);
        }
        if (tracer) tr[3] = ds_globaltimer();
        // ---- the next GEMV phase's first weight item goes in flight before the barrier in front of it
        const int nph = ph + 1;
        if (nph < total_phases) {
            const int nkind = nph < layer_phases ? nph % kPhPerLayer : -1;
            if (nkind < 0 || ph_is_gemv(nkind)) {
                pm_build(p, nkind < 0 ? nullptr : p.layers + nph / kPhPerLayer, nkind, pm);
                pm_load_first(pm, warp, lane, item);
                pf_retire(p, pf, g);
            }
        }
    }
}

// A one-CTA kernel whose only job is to wait at a barrier that nobody else will reach: exercises the bounded wait.
__global__ void decode_step_wait_probe_kernel(DsParams p) {
    unsigned long long target = ld_acquire_u64(p.w.bar) + 1;  // as if one more CTA had to arrive
    grid_barrier(p, target);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
struct DsLayout {
    size_t off_bar, off_err, off_q, off_k, off_v, off_parts, off_attn, off_xq_a, off_xs_a, off_gate, off_up, off_xq_f,
        off_xlo_f, off_xs_f, total;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static DsLayout ds_layout(const nve_b200_decode_model& m) {
    DsLayout l;
    size_t o = 0;
    auto take = [&](size_t bytes) {
        const size_t at = o;
        o = align_up(o + bytes, 256);
        return at;
    };
    const size_t qd = static_cast<size_t>(m.num_heads) * m.head_dim, kvd = static_cast<size_t>(m.num_kv_heads) * m.head_dim;
    l.off_bar = take(8);
    l.off_err = take(4);
    l.off_q = take(qd * 2);
    l.off_k = take(kvd * 2);
    l.off_v = take(kvd * 2);
    const size_t part = (2 + 2 + 2 * static_cast<size_t>(m.head_dim)) * sizeof(float);  // AdCtaPartial<hd, 2>
    l.off_parts = take(static_cast<size_t>(m.num_heads / 2) * kAdRanks * part);
    l.off_attn = take(qd * 2);
    l.off_xq_a = take(qd);
    l.off_xs_a = take(qd / 32 * 4);
    l.off_gate = take(static_cast<size_t>(m.ffn) * 2);
    l.off_up = take(static_cast<size_t>(m.ffn) * 2);
    l.off_xq_f = take(m.ffn);
    l.off_xlo_f = take(m.ffn);
    l.off_xs_f = take(static_cast<size_t>(m.ffn) / 32 * 4);
    l.total = o;
    return l;
}

static int ds_check_model(const nve_b200_decode_model& m) {
    if (m.hidden <= 0 || m.ffn <= 0 || m.num_heads <= 0 || m.num_kv_heads <= 0 || m.num_layers <= 0 || m.max_seq <= 0)
        return NVE_ERR_BAD_SHAPE;
    if (m.head_dim != 64 && m.head_dim != 128) return NVE_ERR_BAD_SHAPE;
    if ((m.num_heads % m.num_kv_heads) != 0 || ((m.num_heads / m.num_kv_heads) % 2) != 0) return NVE_ERR_BAD_SHAPE;
    if ((m.hidden % 32) != 0 || (m.ffn % 32) != 0) return NVE_ERR_BAD_SHAPE;
    if (((m.num_heads * m.head_dim) % 8) != 0 || ((m.num_kv_heads * m.head_dim) % 8) != 0 || (m.ffn % 8) != 0 || (m.hidden % 8) != 0)
        return NVE_ERR_BAD_SHAPE;
    if (m.hidden > kDsMaxStageK || m.num_heads * m.head_dim > kDsMaxStageK) return NVE_ERR_TOO_LARGE;
    if (m.lm_nibbles != nullptr && (m.vocab <= 0 || !m.lm_scales || !m.final_norm || !m.logits)) return NVE_ERR_BAD_POINTER;
    if (!m.rope_cos || !m.rope_sin) return NVE_ERR_BAD_POINTER;
    return NVE_OK;
}

static size_t ds_smem_bytes(const nve_b200_decode_model& m) {
    const int kmax = std::max(m.hidden, std::max(m.ffn, m.num_heads * m.head_dim));
    const size_t S = (static_cast<size_t>(kmax) / 32 + 31) / 32;
    const size_t planes = S * 32 * (32 * 2 + 8);
    const size_t attn = 2 * (m.head_dim == 128 ? sizeof(AdShared<128, 2>) : sizeof(AdShared<64, 2>));
    return std::max(planes, attn);
}

static void ds_fill_work(DsWork& w, void* workspace, const DsLayout& l) {
    unsigned char* b = static_cast<unsigned char*>(workspace);
    w.bar = reinterpret_cast<unsigned long long*>(b + l.off_bar);
    w.err = reinterpret_cast<int*>(b + l.off_err);
    w.q = reinterpret_cast<uint16_t*>(b + l.off_q);
    w.k = reinterpret_cast<uint16_t*>(b + l.off_k);
    w.v = reinterpret_cast<uint16_t*>(b + l.off_v);
    w.parts = b + l.off_parts;
    w.attn = reinterpret_cast<uint16_t*>(b + l.off_attn);
    w.xq_a = reinterpret_cast<int8_t*>(b + l.off_xq_a);
    w.xs_a = reinterpret_cast<float*>(b + l.off_xs_a);
    w.gate = reinterpret_cast<uint16_t*>(b + l.off_gate);
    w.up = reinterpret_cast<uint16_t*>(b + l.off_up);
    w.xq_f = reinterpret_cast<int8_t*>(b + l.off_xq_f);
    w.xlo_f = reinterpret_cast<uint8_t*>(b + l.off_xlo_f);
    w.xs_f = reinterpret_cast<float*>(b + l.off_xs_f);
}

static long long g_ds_prefetch_bytes = 48ll << 20;
static unsigned long long* g_ds_trace = nullptr;

}  // namespace nve

using namespace nve;

extern "C" size_t nve_b200_decode_step_workspace_bytes(const nve_b200_decode_model* model) {
    if (model == nullptr || ds_check_model(*model) != NVE_OK) {
        set_status(NVE_ERR_BAD_SHAPE);
        return 0;
    }
    set_status(NVE_OK);
    return ds_layout(*model).total;
}

extern "C" int nve_b200_decode_step_init(void* workspace, size_t workspace_bytes, nve_stream_t stream) {
    if (workspace == nullptr || workspace_bytes < 512) return set_status(NVE_ERR_BAD_POINTER);
    if (!aligned(workspace, 256)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    // barrier counter and error word start at zero; the activation buffers need no initial value
    return set_cuda_status(cudaMemsetAsync(workspace, 0, 512, static_cast<cudaStream_t>(stream)));
}

extern "C" long long nve_b200_decode_step_set_prefetch(long long bytes) {
    const long long old = g_ds_prefetch_bytes;
    if (bytes >= 0) g_ds_prefetch_bytes = bytes;
    return old;
}

extern "C" int nve_b200_decode_step(const nve_b200_decode_model* model, const nve_b200_decode_layer* layers_dev,
                                    void* hidden, const int* d_pos, const int* d_seq_len, void* workspace,
                                    size_t workspace_bytes, nve_stream_t stream) {
    if (!model || !layers_dev || !hidden || !d_pos || !d_seq_len || !workspace) return set_status(NVE_ERR_BAD_POINTER);
    int st = ds_check_model(*model);
    if (st != NVE_OK) return set_status(st);
    if (!aligned(workspace, 256) || !aligned(hidden, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    const DsLayout l = ds_layout(*model);
    if (workspace_bytes < l.total) return set_status(NVE_ERR_TOO_LARGE);
    const size_t smem = ds_smem_bytes(*model);
    if (smem > static_cast<size_t>(kMaxGemvSmem)) return set_status(NVE_ERR_TOO_LARGE);
    DsParams p;
    p.m = *model;
    p.layers = layers_dev;
    p.hidden = static_cast<uint16_t*>(hidden);
    p.d_pos = d_pos;
    p.d_seq_len = d_seq_len;
    ds_fill_work(p.w, workspace, l);
    p.wait_ns = kDsWaitNs;
    p.pf_bytes = g_ds_prefetch_bytes;
    p.trace = g_ds_trace;
    const void* kern = model->head_dim == 128 ? reinterpret_cast<const void*>(decode_step_kernel<128>)
                                              : reinterpret_cast<const void*>(decode_step_kernel<64>);
    st = ensure_dynamic_smem(kern, kMaxGemvSmem);
    if (st != NVE_OK) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count());
    cfg.blockDim = dim3(kDsThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs co-resident, or the launch fails
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = model->head_dim == 128 ? cudaLaunchKernelEx(&cfg, decode_step_kernel<128>, p)
                                           : cudaLaunchKernelEx(&cfg, decode_step_kernel<64>, p);
    count_launch();
    return set_cuda_status(e);
}

extern "C" void nve_b200_decode_step_set_trace(unsigned long long* buf) { g_ds_trace = buf; }

extern "C" int nve_b200_decode_step_error(void* workspace, int reset) {
    if (workspace == nullptr) return -1;
    int v = 0;
    unsigned char* b = static_cast<unsigned char*>(workspace);
    // the error word sits at the second 256-byte slot of the workspace (see ds_layout)
    cudaError_t e = cudaMemcpy(&v, b + 256, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) { set_cuda_status(e); return -1; }
    if (reset && v != 0) cudaMemset(workspace, 0, 512);
    return v;
}

extern "C" int nve_b200_decode_step_wait_probe(void* workspace, unsigned long long wait_ns, nve_stream_t stream) {
    if (workspace == nullptr) return set_status(NVE_ERR_BAD_POINTER);
    if (wait_ns == 0 || wait_ns > kDsWaitNs) return set_status(NVE_ERR_BAD_SHAPE);
    DsParams p = {};
    unsigned char* b = static_cast<unsigned char*>(workspace);
    p.w.bar = reinterpret_cast<unsigned long long*>(b);
    p.w.err = reinterpret_cast<int*>(b + 256);
    p.wait_ns = wait_ns;
    decode_step_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
    count_launch();
    return check_launch();
}
