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
//   * Five phases (= five device-wide barriers) per layer: [RMSNorm + q/k/v], [RoPE + KV write + attention, the
//     CTA that finishes a head pair last merges its position slices], [o_proj + residual], [RMSNorm + gate/up with
//     SiLU*up in the epilogue: a warp owns gate row i and up row i], [down + residual].  The int8 / fixed-point
//     conversion of the attention output and of SiLU*up happens in the consumer's staging, once per SM.
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
    int* err;                 // 0, or NVE_ERR_TIMEOUT latched by an expired wait
    int* attn_cnt;            // per pair of head pairs: position slices finished (returns to 0 in every layer)
    uint16_t* q;              // [nh*hd] f16
    uint16_t* k;              // [nkv*hd]
    uint16_t* v;
    void* parts;              // attention partials: [virtual clusters][kAdRanks] AdCtaPartial<hd, 2>
    uint16_t* attn;           // [nh*hd] f16
    uint16_t* mid;            // [ffn] f16: silu(gate) * up
};

struct DsParams {
    nve_b200_decode_model m;
    const nve_b200_decode_layer* layers;  // device array [num_layers]
    uint16_t* hidden;                     // [hidden] f16, updated in place
    const int* d_pos;
    const int* d_seq_len;
    DsWork w;
    unsigned long long wait_ns;
    int pf_items;  // run-ahead distance of the L2 prefetch walk in items per warp (0 = off)
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
__device__ __forceinline__ void l2_prefetch_line(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }
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
enum { kEpiF16 = 0, kEpiResidual = 1, kEpiF32 = 2, kEpiSiluMul = 3 };

struct PhaseMats {
    const uint8_t* nib[3];
    const float* sc[3];
    void* out[3];
    int row_end[3];
    int n_total;
    int K, nb, S;
    int epi;
    int planes;  // 1 = W4A8, 2 = W4A16
    int paired;  // gate/up: a tile holds R/2 gate rows and the R/2 up rows of the same indices
    int tb, te;  // tile range of this CTA
};

struct WFlat {  // one warp item: R rows x C column sets (R*C = 8 blocks per lane), index c*R + r
    uint4 w[8];
    float s[8];
};

__device__ __forceinline__ int pm_rows_per_tile(const PhaseMats& pm) { return pm.S >= 3 ? 2 : (pm.S == 2 ? 4 : 8); }

__device__ __forceinline__ void pm_locate(const PhaseMats& pm, int grow, const uint8_t*& nib, const float*& sc, int& lrow,
                                          int& lend, void*& out) {
    if (grow < pm.row_end[0]) {
        nib = pm.nib[0]; sc = pm.sc[0]; lrow = grow; lend = pm.row_end[0]; out = pm.out[0];
    } else if (grow < pm.row_end[1]) {
        nib = pm.nib[1]; sc = pm.sc[1]; lrow = grow - pm.row_end[0]; lend = pm.row_end[1] - pm.row_end[0]; out = pm.out[1];
    } else {
        nib = pm.nib[2]; sc = pm.sc[2]; lrow = grow - pm.row_end[1]; lend = pm.row_end[2] - pm.row_end[1]; out = pm.out[2];
    }
}

// Tile range of this CTA for a phase (computed once when the phase is published).
__device__ __forceinline__ void pm_set_cta_tiles(PhaseMats& pm) {
    const int R = pm_rows_per_tile(pm);
    const int tiles = (pm.n_total + R - 1) / R;
    pm.tb = static_cast<int>(static_cast<long long>(tiles) * blockIdx.x / gridDim.x);
    pm.te = static_cast<int>(static_cast<long long>(tiles) * (blockIdx.x + 1) / gridDim.x);
}
__device__ __forceinline__ void pm_cta_tiles(const PhaseMats& pm, int& tb, int& te) {
    tb = pm.tb;
    te = pm.te;
}

struct ItemIt {
    int g;   // GEMV phase (execution order)
    int t;   // tile, or -1: not yet placed in phase g
    int cg;  // column group
};

// Row r of a tile: matrix pointers and the row's first block index (rows past the end of a matrix are clamped for
// the load and discarded at the store).
__device__ __forceinline__ void item_row(const PhaseMats& pm, int tile, int r, int R, const uint8_t*& nib, const float*& sc,
                                         long long& rb) {
    int lrow, lend;
    if (pm.paired) {
        const int half = R >> 1;
        const bool up = r >= half;
        nib = up ? pm.nib[1] : pm.nib[0];
        sc = up ? pm.sc[1] : pm.sc[0];
        lrow = tile * half + (up ? r - half : r);
        lend = pm.row_end[0];
    } else {
        void* out_unused;
        pm_locate(pm, tile * R, nib, sc, lrow, lend, out_unused);
        lrow += r;
    }
    rb = static_cast<long long>(min(lrow, lend - 1)) * pm.nb;
}

// Load one item into registers.  pf_tiles > 0: the lanes that own the first 16 bytes of a 128-byte line also ask L2
// for the same lines of the tile `pf_tiles` tiles further down this warp's sequence (same phase only; the rows of a
// matrix are evenly spaced, so that is a constant byte offset from the addresses computed for the load).
template <int R, int C>
__device__ __forceinline__ void ds_load_item(const PhaseMats& pm, int tile, int cg, int lane, WFlat& t, int pf_tiles = 0) {
    bool pf = pf_tiles > 0 && tile + pf_tiles * kDsWarps < pm.te;
    if (pf && !pm.paired && pm.row_end[0] != pm.n_total) {
        // several matrices in one launch: only when the far tile lies in the same matrix as this one
        const int r0 = tile * R, r1 = (tile + pf_tiles * kDsWarps) * R;
        const int m0 = r0 < pm.row_end[0] ? 0 : (r0 < pm.row_end[1] ? 1 : 2);
        const int m1 = r1 < pm.row_end[0] ? 0 : (r1 < pm.row_end[1] ? 1 : 2);
        pf = m0 == m1;
    }
    const long long pf_rows = static_cast<long long>(pf_tiles) * kDsWarps * (pm.paired ? R / 2 : R);
    // a full column group of full column sets: one address per row, the column sets at immediate offsets
    const bool full = (pm.nb & (kWarp - 1)) == 0 && (cg + 1) * C <= pm.S;
#pragma unroll
    for (int r = 0; r < R; r++) {
        const uint8_t* nib;
        const float* sc;
        long long rb;
        item_row(pm, tile, r, R, nib, sc, rb);
        if (full) {
            const long long b0 = rb + cg * (C * kWarp) + lane;
            const uint8_t* nrow = nib + b0 * 16;
            const float* srow = sc + b0;
            t.w[0 * R + r] = ld_stream_u4_off<0>(nrow);
            t.s[0 * R + r] = ld_stream_f32_off<0>(srow);
            if constexpr (C > 1) {
                t.w[1 * R + r] = ld_stream_u4_off<512>(nrow);
                t.s[1 * R + r] = ld_stream_f32_off<128>(srow);
            }
            if constexpr (C > 2) {
                t.w[2 * R + r] = ld_stream_u4_off<1024>(nrow);
                t.s[2 * R + r] = ld_stream_f32_off<256>(srow);
                t.w[3 * R + r] = ld_stream_u4_off<1536>(nrow);
                t.s[3 * R + r] = ld_stream_f32_off<384>(srow);
            }
            if (pf && (lane & 7) == 0) {
#pragma unroll
                for (int c = 0; c < C; c++) l2_prefetch_line(nrow + pf_rows * pm.nb * 16 + c * 512);
            }
            if (pf && lane == 0) {
#pragma unroll
                for (int c = 0; c < C; c++) l2_prefetch_line(srow + pf_rows * pm.nb + c * 32);
            }
            continue;
        }
#pragma unroll
        for (int c = 0; c < C; c++) {
            const int b = (cg * C + c) * kWarp + lane;
            if (b < pm.nb) {
                t.w[c * R + r] = ld_stream_u4(nib + (rb + b) * 16);
                t.s[c * R + r] = ld_stream_f32(sc + rb + b);
                if (pf && (lane & 7) == 0) l2_prefetch_line(nib + (rb + pf_rows * pm.nb + b) * 16);
                if (pf && lane == 0) l2_prefetch_line(sc + rb + pf_rows * pm.nb + b);
            } else {
                t.w[c * R + r] = make_uint4(0, 0, 0, 0);
                t.s[c * R + r] = 0.0f;
            }
        }
    }
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

// ---------------------------------------------------------------------------------------------
// L2 prefetch stream.  Weights never depend on activations, so every warp walks the sequence of its own future
// items -- across phase boundaries -- and asks for their cache lines (`prefetch.global.L2`) a fixed number of items
// ahead of the item it computes.  DRAM therefore stays busy while the CTA waits at a barrier or stages activations,
// and the register loads of an item mostly hit L2.  The matrices of the next kPmSlots - 1 GEMV phases are
// published in shared memory (pms[g % kPmSlots]) so that the walk can look that far.
// ---------------------------------------------------------------------------------------------
constexpr int kPmSlots = 4;

// The 40 cache lines of one item: lane l asks for 128-byte line l % 4 of nibble slot l / 4; lanes 0..7 for the
// scale line of slot l.
__device__ __forceinline__ void pf_item(const PhaseMats& pm, int tile, int cg, int lane) {
    const int R = pm_rows_per_tile(pm);
    const int C = 8 / R;
    {
        const int j = lane >> 2, c = j / R, r = j % R;
        const uint8_t* nib;
        const float* sc;
        long long rb;
        item_row(pm, tile, r, R, nib, sc, rb);
        const int b = (cg * C + c) * kWarp + (lane & 3) * 8;
        if (b < pm.nb) l2_prefetch_line(nib + (rb + b) * 16);
    }
    if (lane < 8) {
        const int c = lane / R, r = lane % R;
        const uint8_t* nib;
        const float* sc;
        long long rb;
        item_row(pm, tile, r, R, nib, sc, rb);
        const int b = (cg * C + c) * kWarp;
        if (b < pm.nb) l2_prefetch_line(sc + rb + b);
    }
}

// Ask L2 for this warp's first `items` items of a phase that has not started yet (called when the warp has finished
// the phase in front of it: the requests are served while the CTA waits at the barrier and stages activations).
__device__ __forceinline__ void pf_head(const PhaseMats& pm, int items, int warp, int lane) {
    const int C = pm.S >= 3 ? 4 : (pm.S == 2 ? 2 : 1);
    const int CG = (pm.S + C - 1) / C;
    int t = pm.tb + warp, cg = 0;
    for (int i = 0; i < items && t < pm.te; i++) {
        pf_item(pm, t, cg, lane);
        if (++cg >= CG) {
            cg = 0;
            t += kDsWarps;
        }
    }
}

template <int PLANES, int R, int C>
__device__ __forceinline__ void ds_run_gemv(const PhaseMats& pm, Smem<PLANES>& sm, const uint16_t* residual, int warp,
                                            int lane, WFlat& it, int dist) {
    const int S = pm.S;
    const int CG = (S + C - 1) / C;
    int tb, te;
    pm_cta_tiles(pm, tb, te);
    const int pf_tiles = dist > 0 ? (dist + CG - 1) / CG : 0;  // tiles ahead that cover `dist` items
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
            // issue the next item's loads before reducing this one, and keep the L2 prefetch walk `dist` items ahead
            if (cg + 1 < CG) ds_load_item<R, C>(pm, t, cg + 1, lane, it, pf_tiles);
            else if (t + kDsWarps < te) ds_load_item<R, C>(pm, t + kDsWarps, 0, lane, it, pf_tiles);
            warp_sum_multi<R>(a, lane);
            y = (cg == 0) ? a[0] : __fadd_rn(y, a[0]);  // column groups of a row in ascending order
        }
        if (pm.epi == kEpiSiluMul) {
            // lanes l and l ^ 16 hold gate row i and up row i: mid[i] = f16(silu(f16 gate) * f16 up), the bits of the
            // separate GEMV (f16 outputs) + SiLU*up kernels
            const float yu = __shfl_xor_sync(0xffffffffu, y, 16);
            if (multi_row_writer<R>(lane) && (lane & 16) == 0) {
                const int i = t * (R / 2) + multi_row_of<R>(lane);
                if (i < pm.row_end[0]) {
                    const float g = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(y));
                    const float u = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(yu));
                    static_cast<uint16_t*>(pm.out[0])[i] = Act16<NVE_DT_F16>::from_f32(silu_mul_f32(g, u));
                }
            }
        } else if (multi_row_writer<R>(lane)) {
            const int grow = t * R + multi_row_of<R>(lane);
            if (grow < pm.n_total) {
                const uint8_t* nib;
                const float* sc;
                int lrow, lend;
                void* out;
                pm_locate(pm, grow, nib, sc, lrow, lend, out);
                if (pm.epi == kEpiResidual) {
                    // same bits as a GEMV with f16 output followed by the residual-add kernel
                    const float yr = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(y));
                    const float h = __fadd_rn(Act16<NVE_DT_F16>::to_f32(__ldcg(residual + lrow)), yr);
                    static_cast<uint16_t*>(out)[lrow] = Act16<NVE_DT_F16>::from_f32(h);
                } else if (pm.epi == kEpiF32) {
                    static_cast<float*>(out)[lrow] = y;
                } else {
                    static_cast<uint16_t*>(out)[lrow] = Act16<NVE_DT_F16>::from_f32(y);
                }
            }
        }
    }
}

template <int PLANES>
__device__ __forceinline__ void ds_run_gemv_rc(const PhaseMats& pm, unsigned char* smem_raw, const uint16_t* residual,
                                               int warp, int lane, WFlat& it, int dist) {
    Smem<PLANES> sm(smem_raw, pm.S * kWarp);
    if (pm.S >= 3) ds_run_gemv<PLANES, 2, 4>(pm, sm, residual, warp, lane, it, dist);
    else if (pm.S == 2) ds_run_gemv<PLANES, 4, 2>(pm, sm, residual, warp, lane, it, dist);
    else ds_run_gemv<PLANES, 8, 1>(pm, sm, residual, warp, lane, it, dist);
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
constexpr int kDsMaxStageK = kDsStageIters * kDsThreads * 8;  // 8192: largest K of a vector that is RMS-normalised

// RMSNorm of x (K <= kDsMaxStageK values, f16) in the library's fixed order, then int8 codes (PLANES 1) or 16-bit
// fixed-point planes (PLANES 2, after the optional awq multiply).  The vector is read once: every thread keeps its
// chunks in registers for the second pass and leaves a copy in `stash` so that the first 256 threads can take the
// sum of squares in the stand-alone kernel's order.
template <int PLANES>
__device__ __forceinline__ void ds_stage_norm(const uint16_t* x, const uint16_t* norm_w, float eps, const float* awq, int K,
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
            wr[it] = __ldg(reinterpret_cast<const uint4*>(norm_w) + c);
            stash[c] = xr[it];
        }
    }
    __syncthreads();
    // sum of squares: thread t < 256 adds the chunks t, t+256, ... (fma chain, ascending), xor butterfly per warp,
    // the 8 warp sums in ascending order -- the order of the stand-alone RMSNorm kernel
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
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(total, static_cast<float>(K)), eps)));
#pragma unroll
    for (int it = 0; it < kDsStageIters; it++) {
        if (it < iters) {  // uniform over the CTA: the quad shuffles inside stage_chunk_* need whole warps
            const int c = it * kDsThreads + threadIdx.x;
            const bool active = c < chunks;
            float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (active) {
                uint16_t h[8], hw[8];
                unpack8(xr[it], h);
                unpack8(wr[it], hw);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const float o = __fmul_rn(__fmul_rn(Act16<NVE_DT_F16>::to_f32(h[e]), r), Act16<NVE_DT_F16>::to_f32(hw[e]));
                    v[e] = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(o));
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

// A 16-bit vector written by an earlier phase (attention output, SiLU*up) -> int8 codes (PLANES 1, the arithmetic of
// the stand-alone quantiser) or fixed-point planes (PLANES 2, after the optional awq multiply).  Any K.
template <int PLANES>
__device__ __forceinline__ void ds_stage_vec(const uint16_t* x, const float* awq, int K, Smem<PLANES>& sm) {
    ds_zero_padding<PLANES>(K / kBlockK, sm);
    const int chunks = K >> 3;
    const int iters = (chunks + kDsThreads - 1) / kDsThreads;
    for (int it0 = 0; it0 < iters; it0 += 4) {
        uint4 xr[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {  // up to four L2 loads in flight per thread
            const int c = (it0 + j) * kDsThreads + threadIdx.x;
            xr[j] = make_uint4(0, 0, 0, 0);
            if (it0 + j < iters && c < chunks) xr[j] = __ldcg(reinterpret_cast<const uint4*>(x) + c);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (it0 + j < iters) {
                const int c = (it0 + j) * kDsThreads + threadIdx.x;
                const bool active = c < chunks;
                float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (active) {
                    uint16_t h[8];
                    unpack8(xr[j], h);
#pragma unroll
                    for (int e = 0; e < 8; e++) v[e] = Act16<NVE_DT_F16>::to_f32(h[e]);
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
}

// ---------------------------------------------------------------------------------------------
// Attention phase: RoPE + KV write + per-slice online softmax; the CTA that completes the last slice of a pair of
// head pairs merges the slices (level 2), so no device-wide barrier separates the two steps.
// ---------------------------------------------------------------------------------------------
// A CTA runs two virtual CTAs of 256 threads side by side: the two query-head pairs 2u, 2u+1 on the same position
// slice (for the usual group size 4 they share the KV head, so the second reader hits L1/L2).
template <int HD>
__device__ __forceinline__ void ds_attn_phase(const DsParams& p, const nve_b200_decode_layer& ly, unsigned char* smem_raw,
                                              int seq_len, int pos, int* last_flag) {
    constexpr int QH = 2;
    constexpr int DC = HD / 8;
    AdShared<HD, QH>* shs = reinterpret_cast<AdShared<HD, QH>*>(smem_raw);
    const int half = threadIdx.x / kAdThreads, tid = threadIdx.x % kAdThreads;
    AdShared<HD, QH>& sh = shs[half];
    const int groups = p.m.num_heads / p.m.num_kv_heads;
    const int clusters_per_kv = groups / QH;
    const int nvc = p.m.num_heads / QH;  // virtual clusters (head pairs)
    const int units = ((nvc + 1) / 2) * kAdRanks;
    const bool pos_ok = pos >= 0 && pos < p.m.max_seq;
    const int chunk = (seq_len + kAdRanks - 1) / kAdRanks;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
        const int rank = u % kAdRanks;
        const int pair = u / kAdRanks;
        const int vc = pair * 2 + half;
        const bool live = vc < nvc;
        const int vcc = live ? vc : nvc - 1;  // an idle half repeats the last head pair's work and discards it
        const int kvh = vcc / clusters_per_kv;
        const int h0 = kvh * groups + (vcc % clusters_per_kv) * QH;
        const uint16_t* kh = ly.k_cache + static_cast<long long>(kvh) * p.m.max_seq * HD;
        const uint16_t* vh = ly.v_cache + static_cast<long long>(kvh) * p.m.max_seq * HD;
        attn_stage_q<HD, QH, true, true>(sh, tid, p.w.q, p.w.k, p.w.v, p.m.rope_cos, p.m.rope_sin, h0, kvh, pos, pos_ok);
        __syncthreads();
        const int t_begin = rank * chunk;
        const int t_end = min(seq_len, t_begin + chunk);
        if (live && pos_ok && rank == 0 && (vcc % clusters_per_kv) == 0 && tid < 2 * DC) {
            const int which = tid / DC, d = tid % DC;
            uint16_t* dst = (which == 0 ? ly.k_cache : ly.v_cache) + (static_cast<long long>(kvh) * p.m.max_seq + pos) * HD;
            reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(which == 0 ? sh.knew_s : sh.vnew_s)[d];
        }
        AdCtaPartial<HD, QH>* parts = static_cast<AdCtaPartial<HD, QH>*>(p.w.parts);
        AdCtaPartial<HD, QH>* dst = parts + (static_cast<long long>(vcc) * kAdRanks + rank);
        attn_partial<HD, QH, true, false>(
            sh, tid, kh, vh, t_begin, t_end, pos, p.m.attn_scale, false, nullptr, [] { __syncthreads(); },
            [&](int h, int d, float mm, float ss, float a) {
                if (live) {
                    __stcg(&dst->acc[h][d], a);
                    if (d == 0) { __stcg(&dst->m[h], mm); __stcg(&dst->s[h], ss); }
                }
            });
        // ---- count this slice; whoever completes the pair's last slice merges all of them
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            const int old = atomicAdd(p.w.attn_cnt + pair, 1);
            const int last = old == kAdRanks - 1;
            if (last) {
                p.w.attn_cnt[pair] = 0;  // ready for the next layer (a device-wide barrier comes first)
                __threadfence();
            }
            *last_flag = last;
        }
        __syncthreads();
        if (*last_flag && live) {
            for (int i = tid; i < QH * HD; i += kAdThreads) {
                const int h = i / HD, d = i % HD;
                const uint16_t o16 = attn_merge_ranks<HD, QH, true>(parts + static_cast<long long>(vcc) * kAdRanks, h, d);
                p.w.attn[static_cast<long long>(h0 + h) * HD + d] = o16;
            }
        }
        __syncthreads();  // shared memory (and the flag) are reused by the next unit
    }
}

// ---------------------------------------------------------------------------------------------
// Phase table
// ---------------------------------------------------------------------------------------------
enum { kPhQkv = 0, kPhAttn = 1, kPhO = 2, kPhGateUp = 3, kPhDown = 4, kPhPerLayer = 5 };

__device__ __forceinline__ bool ph_is_gemv(int kind) { return kind != kPhAttn; }

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
    pm.paired = 0;
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
            pm_set(pm, 0, ly, 4, p.w.mid, p.m.ffn);
            pm_set(pm, 1, ly, 5, p.w.mid, 2 * p.m.ffn);
            pm_set(pm, 2, ly, 5, p.w.mid, 2 * p.m.ffn);
            pm.paired = 1;
            pm.epi = kEpiSiluMul;
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
    pm_set_cta_tiles(pm);
}

// Matrices of GEMV phase g in execution order (four per layer, then the lm_head).
__device__ __forceinline__ void ds_build_gemv(const DsParams& p, int g, PhaseMats& pm) {
    const int layer = g >> 2;
    if (layer < p.m.num_layers) {
        const int kind = (g & 3) == 0 ? kPhQkv : ((g & 3) == 1 ? kPhO : ((g & 3) == 2 ? kPhGateUp : kPhDown));
        pm_build(p, p.layers + layer, kind, pm);
    } else {
        pm_build(p, nullptr, -1, pm);
    }
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
    __shared__ int last_flag_s;
    __shared__ PhaseMats pms[kPmSlots];
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

    // The matrices of GEMV phase g live in pms[g % kPmSlots]; thread 0 publishes phase g + kPmSlots - 1 while phase g
    // is staged, so the prefetch walk can look kPmSlots - 1 phases ahead.
    if (threadIdx.x == 0) {
        for (int i = 0; i < kPmSlots - 1 && i < total_gemvs; i++) ds_build_gemv(p, i, pms[i]);
    }
    __syncthreads();
    int g = 0;  // index of the next GEMV phase
    const int dist = p.pf_items;
    WFlat item;
    pm_load_first(pms[0], warp, lane, item);
    if (dist > 0) pf_head(pms[0], dist + 1, warp, lane);

    for (int ph = 0; ph < total_phases; ph++) {
        const int layer = ph / kPhPerLayer;
        const int kind = ph < layer_phases ? ph % kPhPerLayer : -1;
        const nve_b200_decode_layer* ly = p.layers + min(layer, p.m.num_layers - 1);
        const bool tracer = p.trace != nullptr && threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1);
        unsigned long long* tr = tracer ? p.trace + (static_cast<size_t>(blockIdx.x == 0 ? 0 : 1) * total_phases + ph) * 4 : nullptr;
        if (tracer) tr[0] = ds_globaltimer();
        if (ph > 0) grid_barrier(p, bar_target);
        if (tracer) tr[1] = ds_globaltimer();
        if (kind != kPhAttn) {
            const PhaseMats& pm = pms[g % kPmSlots];
            if (threadIdx.x == 0 && g + kPmSlots - 1 < total_gemvs) ds_build_gemv(p, g + kPmSlots - 1, pms[(g + kPmSlots - 1) % kPmSlots]);
            // ---- small read-only data that a later phase waits for goes to L2 now: the RMSNorm weight of the next
            // normalising phase (cold in L2 by the time its layer comes round), this CTA's K/V slice of the attention
            if (threadIdx.x == 32) {
                const unsigned nbytes = static_cast<unsigned>(p.m.hidden) * 2u;
                if (kind == kPhQkv && static_cast<int>(blockIdx.x) == (layer + 1) % static_cast<int>(gridDim.x))
                    l2_prefetch_bulk(ly->post_attn_norm, nbytes);
                if (kind == kPhGateUp && static_cast<int>(blockIdx.x) == (layer + 2) % static_cast<int>(gridDim.x)) {
                    if (layer + 1 < p.m.num_layers) l2_prefetch_bulk((ly + 1)->input_norm, nbytes);
                    else if (has_head) l2_prefetch_bulk(p.m.final_norm, nbytes);
                }
            }
            if (kind == kPhQkv && threadIdx.x >= 64 && threadIdx.x < 66) {
                const int groups = p.m.num_heads / p.m.num_kv_heads;
                const int nvc = p.m.num_heads / 2;
                const int units = ((nvc + 1) / 2) * kAdRanks;
                const int chunk = (seq_len + kAdRanks - 1) / kAdRanks;
                for (int u = blockIdx.x; u < units; u += gridDim.x) {
                    const int rank = u % kAdRanks;
                    const int vc = min((u / kAdRanks) * 2, nvc - 1);
                    const int kvh = vc / (groups / 2);
                    const int t0 = rank * chunk, t1 = min(seq_len, t0 + chunk);
                    if (t1 > t0) {
                        const uint16_t* base = (threadIdx.x == 64 ? ly->k_cache : ly->v_cache) +
                                               (static_cast<long long>(kvh) * p.m.max_seq + t0) * HD;
                        l2_prefetch_bulk(base, static_cast<unsigned>(t1 - t0) * HD * 2u);
                    }
                }
            }
            // ---- stage the activation vector of the phase once for this SM
            const uint16_t* residual = nullptr;
            const int planes = kind < 0 ? (p.m.lm_use_w4a8 ? 1 : 2) : (ly->use_w4a8 ? 1 : 2);
            const int K = kind == kPhO ? p.m.num_heads * p.m.head_dim : (kind == kPhDown ? p.m.ffn : p.m.hidden);
            const int nbp = ((K / kBlockK + kWarp - 1) / kWarp) * kWarp;
            if (kind == kPhQkv || kind == kPhGateUp || kind < 0) {
                const uint16_t* nw = kind == kPhQkv ? ly->input_norm : (kind == kPhGateUp ? ly->post_attn_norm : p.m.final_norm);
                const float* awq = kind < 0 ? nullptr : ly->awq[kind == kPhQkv ? 0 : 2];
                if (planes == 1) {
                    Smem<1> sm(smem_raw, nbp);
                    ds_stage_norm<1>(p.hidden, nw, p.m.norm_eps, nullptr, K, sm, warp_part, stash);
                } else {
                    Smem<2> sm(smem_raw, nbp);
                    ds_stage_norm<2>(p.hidden, nw, p.m.norm_eps, awq, K, sm, warp_part, stash);
                }
            } else {
                residual = p.hidden;
                const uint16_t* x = kind == kPhO ? p.w.attn : p.w.mid;
                if (planes == 1) {
                    Smem<1> sm(smem_raw, nbp);
                    ds_stage_vec<1>(x, nullptr, K, sm);
                } else {
                    Smem<2> sm(smem_raw, nbp);
                    ds_stage_vec<2>(x, ly->awq[kind == kPhO ? 1 : 3], K, sm);
                }
            }
            __syncthreads();
            if (tracer) tr[2] = ds_globaltimer();
            if (planes == 1) ds_run_gemv_rc<1>(pm, smem_raw, residual, warp, lane, item, dist);
            else ds_run_gemv_rc<2>(pm, smem_raw, residual, warp, lane, item, dist);
            g++;
            // this warp is done with the phase: the head of the next GEMV phase (and of the one after it when the
            // next one is short) is asked for now, to arrive while the CTA waits and stages
            if (dist > 0 && g < total_gemvs) {
                pf_head(pms[g % kPmSlots], dist + 1, warp, lane);
                if (g + 1 < total_gemvs && (g & 3) == 1) pf_head(pms[(g + 1) % kPmSlots], dist, warp, lane);
            }
        } else {
            ds_attn_phase<HD>(p, *ly, smem_raw, seq_len, pos, &last_flag_s);
        }
        if (tracer) tr[3] = ds_globaltimer();
        // ---- the next GEMV phase's first weight item goes in flight before the barrier in front of it
        const int nph = ph + 1;
        if (nph < total_phases && (nph >= layer_phases || nph % kPhPerLayer != kPhAttn))
            pm_load_first(pms[g % kPmSlots], warp, lane, item);
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
// Head of the workspace that must start at zero: barrier counter (+0), error word (+256), slice counters (+512).
constexpr size_t kDsControlBytes = 4096;

struct DsLayout {
    size_t off_bar, off_err, off_cnt, off_q, off_k, off_v, off_parts, off_attn, off_mid, total;
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
    l.off_cnt = take(kDsControlBytes - 512);  // one int per pair of head pairs
    l.off_q = take(qd * 2);
    l.off_k = take(kvd * 2);
    l.off_v = take(kvd * 2);
    const size_t part = (2 + 2 + 2 * static_cast<size_t>(m.head_dim)) * sizeof(float);  // AdCtaPartial<hd, 2>
    l.off_parts = take(static_cast<size_t>(m.num_heads / 2) * kAdRanks * part);
    l.off_attn = take(qd * 2);
    l.off_mid = take(static_cast<size_t>(m.ffn) * 2);
    l.total = o;
    return l;
}

static int ds_check_model(const nve_b200_decode_model& m) {
    if (m.hidden <= 0 || m.ffn <= 0 || m.num_heads <= 0 || m.num_kv_heads <= 0 || m.num_layers <= 0 || m.max_seq <= 0)
        return NVE_ERR_BAD_SHAPE;
    if (m.head_dim != 64 && m.head_dim != 128) return NVE_ERR_BAD_SHAPE;
    if (static_cast<size_t>(m.num_heads) * sizeof(int) > kDsControlBytes - 512) return NVE_ERR_TOO_LARGE;
    if ((m.num_heads % m.num_kv_heads) != 0 || ((m.num_heads / m.num_kv_heads) % 2) != 0) return NVE_ERR_BAD_SHAPE;
    if ((m.hidden % 32) != 0 || (m.ffn % 32) != 0) return NVE_ERR_BAD_SHAPE;
    if (((m.num_heads * m.head_dim) % 8) != 0 || ((m.num_kv_heads * m.head_dim) % 8) != 0 || (m.ffn % 8) != 0 || (m.hidden % 8) != 0)
        return NVE_ERR_BAD_SHAPE;
    if (m.hidden > kDsMaxStageK || m.num_heads * m.head_dim > kDsMaxStageK) return NVE_ERR_TOO_LARGE;
    if (m.lm_nibbles != nullptr && (m.vocab <= 0 || !m.lm_scales || !m.final_norm || !m.logits)) return NVE_ERR_BAD_POINTER;
    if (!m.rope_cos || !m.rope_sin) return NVE_ERR_BAD_POINTER;
    return NVE_OK;
}

// Dynamic shared memory: activation planes of a GEMV phase or the attention state.
static size_t ds_front_bytes(const nve_b200_decode_model& m) {
    const int kmax = std::max(m.hidden, std::max(m.ffn, m.num_heads * m.head_dim));
    const size_t S = (static_cast<size_t>(kmax) / 32 + 31) / 32;
    const size_t planes = S * 32 * (32 * 2 + 8);
    const size_t attn = 2 * (m.head_dim == 128 ? sizeof(AdShared<128, 2>) : sizeof(AdShared<64, 2>));
    return align_up(std::max(planes, attn), 128);
}
constexpr size_t kDsSmemBudget = 200 * 1024;  // dynamic shared memory the kernel may ask for (static use comes on top)

static void ds_fill_work(DsWork& w, void* workspace, const DsLayout& l) {
    unsigned char* b = static_cast<unsigned char*>(workspace);
    w.bar = reinterpret_cast<unsigned long long*>(b + l.off_bar);
    w.err = reinterpret_cast<int*>(b + l.off_err);
    w.attn_cnt = reinterpret_cast<int*>(b + l.off_cnt);
    w.q = reinterpret_cast<uint16_t*>(b + l.off_q);
    w.k = reinterpret_cast<uint16_t*>(b + l.off_k);
    w.v = reinterpret_cast<uint16_t*>(b + l.off_v);
    w.parts = b + l.off_parts;
    w.attn = reinterpret_cast<uint16_t*>(b + l.off_attn);
    w.mid = reinterpret_cast<uint16_t*>(b + l.off_mid);
}

static int g_ds_prefetch_items = 0;
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
    if (workspace == nullptr || workspace_bytes < kDsControlBytes) return set_status(NVE_ERR_BAD_POINTER);
    if (!aligned(workspace, 256)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    // barrier counter, error word and slice counters start at zero; the activation buffers need no initial value
    return set_cuda_status(cudaMemsetAsync(workspace, 0, kDsControlBytes, static_cast<cudaStream_t>(stream)));
}

extern "C" int nve_b200_decode_step_set_prefetch(int items) {
    const int old = g_ds_prefetch_items;
    if (items >= 0) g_ds_prefetch_items = items > 64 ? 64 : items;
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
    const size_t smem = ds_front_bytes(*model);
    if (smem > kDsSmemBudget) return set_status(NVE_ERR_TOO_LARGE);
    DsParams p;
    p.m = *model;
    p.layers = layers_dev;
    p.hidden = static_cast<uint16_t*>(hidden);
    p.d_pos = d_pos;
    p.d_seq_len = d_seq_len;
    ds_fill_work(p.w, workspace, l);
    p.wait_ns = kDsWaitNs;
    p.pf_items = g_ds_prefetch_items;
    p.trace = g_ds_trace;
    const void* kern = model->head_dim == 128 ? reinterpret_cast<const void*>(decode_step_kernel<128>)
                                              : reinterpret_cast<const void*>(decode_step_kernel<64>);
    st = ensure_dynamic_smem(kern, static_cast<int>(kDsSmemBudget));
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
    if (reset && v != 0) cudaMemset(workspace, 0, kDsControlBytes);
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
