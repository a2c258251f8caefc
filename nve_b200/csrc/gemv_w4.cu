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
//   * A column set is 32 consecutive blocks (1024 weights) of a row; lane l owns block l of it.  A warp item
//     is 2 rows x 4 column sets (8 blocks per lane; 4 x 2 or 8 x 1 when a row has only 2 or 1 column sets):
//     every lane issues eight 128-bit loads of packed nibbles and eight 32-bit loads of block scales at
//     once -- 512 contiguous bytes per row and column set -- so 16 warps keep about 80 KB in flight per SM.
//     The next item's loads are issued before the current one is reduced; the first item's before the
//     kernel waits for its producer (weights do not depend on it).
//   * Per lane and block: 8 (W4A8) or 16 (W4A16) dp4a on raw nibbles (the high nibbles stay in place as
//     16*q, removed by one exact shift), minus the precomputed 8*sum(x) bias, one int->float conversion and
//     one multiply by (weight scale * activation scale).
//   * Summation order (fixed, so results are bit-reproducible and independent of the launch geometry): per
//     lane the column sets of a group of four are added in ascending order; the 32 lane values of a
//     (row, group) are added by a xor butterfly (pairs l^16, ^8, ^4, ^2, ^1); the groups of a row are added
//     in ascending order.
//
// Algorithmic bytes per launch: N*K/2 nibbles + N*K/8 scale bytes + activations + outputs.
#include <type_traits>

#include "gemv_w4.cuh"

namespace nve {


constexpr unsigned kTpSpinLimit = 1u << 22;  // bounded wait for a peer's slot (local polls of >= 32 ns each)

// One warp item: R rows x C consecutive column sets (R * C = 8 blocks per lane), all 16 loads in flight at once.
template <int R, int C> struct WItem {
    uint4 w[C][R];
    float s[C][R];
    int row0;  // global first row
};

// EVEN: every row is a whole number of column groups of C full column sets (K % (1024 * C) == 0), so no lane and no
// column set of an item is ever idle and the bounds checks drop out.
template <int R, int C, bool PAIR, bool EVEN = false>
__device__ __forceinline__ void load_item(const GemvParams& p, int tile, int cg, int lane, WItem<R, C>& t) {
    t.row0 = tile * R;
    const uint8_t* nib0;
    const float* sc0;
    int lrow, lend;
    if constexpr (PAIR) {
        nib0 = p.nib[0]; sc0 = p.sc[0]; lrow = tile * (R / 2); lend = p.row_end[0];
    } else {
        locate(p, t.row0, nib0, sc0, lrow, lend);
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
        const uint8_t* nib = nib0;
        const float* sc = sc0;
        int row = lrow + r;
        if (PAIR && r >= R / 2) {  // second half of the tile: the up rows of the same indices
            nib = p.nib[1]; sc = p.sc[1]; row = lrow + r - R / 2;
        }
        // rows past the end of a matrix are clamped for the load and discarded at the store
        const long long rb = static_cast<long long>(min(row, lend - 1)) * p.nb;
        // a full column group of full column sets (always so with EVEN; otherwise e.g. 3 of the 4 groups of K = 14336)
        if (EVEN || ((p.nb & (kWarp - 1)) == 0 && (cg + 1) * C <= p.S)) {
            // one address per row; the C column sets of the item sit 512 (nibbles) / 128 (scales) bytes apart
            const long long b0 = rb + cg * (C * kWarp) + lane;
            const uint8_t* nrow = nib + b0 * 16;
            const float* srow = sc + b0;
            t.w[0][r] = ld_stream_u4_off<0>(nrow);
            t.s[0][r] = ld_stream_f32_off<0>(srow);
            if constexpr (C > 1) {
                t.w[1][r] = ld_stream_u4_off<512>(nrow);
                t.s[1][r] = ld_stream_f32_off<128>(srow);
            }
            if constexpr (C > 2) {
                t.w[2][r] = ld_stream_u4_off<1024>(nrow);
                t.s[2][r] = ld_stream_f32_off<256>(srow);
                t.w[3][r] = ld_stream_u4_off<1536>(nrow);
                t.s[3][r] = ld_stream_f32_off<384>(srow);
            }
        } else {
#pragma unroll
            for (int c = 0; c < C; c++) {
                const int b = (cg * C + c) * kWarp + lane;
                if (b < p.nb) {
                    t.w[c][r] = ld_stream_u4(nib + (rb + b) * 16);
                    t.s[c][r] = ld_stream_f32(sc + rb + b);
                } else {
                    t.w[c][r] = make_uint4(0, 0, 0, 0);
                    t.s[c][r] = 0.0f;
                }
            }
        }
    }
}

template <int PLANES, int XDT, int ODT, bool IDOT, int PRO, int R, int C, bool PAIR = false>
__global__ void __launch_bounds__(kGemvThreads, 2) gemv_w4_kernel(const GemvParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    constexpr int W = kGemvThreads / 32;
    const int S = p.S;
    const int CG = (S + C - 1) / C;  // column groups per row
    Smem<PLANES> sm(smem_raw, S * kWarp);

    const int tiles = (p.n_total + R - 1) / R;
    const int tile_begin = static_cast<int>(static_cast<long long>(tiles) * blockIdx.x / gridDim.x);
    const int tile_end = static_cast<int>(static_cast<long long>(tiles) * (blockIdx.x + 1) / gridDim.x);
    const int chunk_tiles_max = max(1, kPartFloats / (R * CG));

    // Weights do not depend on the producer kernel: start streaming them before waiting for it.
    WItem<R, C> it;
    int chunk0 = tile_begin;
    int chunk_tiles = min(chunk_tiles_max, tile_end - chunk0);
    // item index inside the chunk: q = tile * CG + column group; q advances by W per step, so (tile, column group) are
    // carried along instead of divided out for every item
    const int step_t = W / CG, step_c = W - step_t * CG;
    const int tl0 = warp / CG, cg0 = warp - tl0 * CG;
    int q = warp, tl = tl0, cg = cg0;
    if (chunk_tiles > 0 && q < chunk_tiles * CG) load_item<R, C, PAIR>(p, chunk0 + tl, cg, lane, it);

    NormRegs nr;
    if constexpr (PRO == 1) load_norm_regs(p, nr);  // static data: fetched before the dependency wait
    pdl_wait();
    // The residual of this thread's row of the first chunk comes in together with the activations instead of as a
    // dependent load at the very end of the CTA (one memory round trip less on the tail of every o / down launch).
    float res_pre = 0.0f;
    bool res_pre_ok = false;
    if constexpr (!IDOT && !PAIR) {
        const int grow = chunk0 * R + static_cast<int>(threadIdx.x);
        if (p.tp.world <= 1 && chunk_tiles > 0 && static_cast<int>(threadIdx.x) < chunk_tiles * R && grow < p.n_total) {
            const void* res;
            int lrow;
            if (grow < p.row_end[0]) { res = p.res[0]; lrow = grow; }
            else if (grow < p.row_end[1]) { res = p.res[1]; lrow = grow - p.row_end[0]; }
            else { res = p.res[2]; lrow = grow - p.row_end[1]; }
            if (res != nullptr) {
                res_pre = load_out<ODT>(res, lrow);
                res_pre_ok = true;
            }
        }
    }
    stage_activations<PLANES, XDT, PRO>(p, sm, nr);
    // tensor parallel: this launch's epoch is this CTA's own launch counter + 1; slots of the parity it selects
    // are used (a peer can be at most one all-reduce ahead, so two parities never collide)
    __shared__ unsigned tp_epoch_s;
    if (p.tp.world > 1 && threadIdx.x == 0) tp_epoch_s = p.tp.counter[blockIdx.x] + 1u;
    __syncthreads();
    pdl_launch_dependents();
    const bool tp_on = p.tp.world > 1;
    const unsigned tp_epoch = tp_on ? tp_epoch_s : 0u;
    // offset of the plane [parity][source = this rank] inside any rank's buffer
    const size_t tp_plane = (static_cast<size_t>(tp_epoch & 1u) * p.tp.world + p.tp.rank) * p.tp.rows_cap;

    bool first_chunk = true;
    // The streaming loop is compiled twice: with and without the bounds checks of ragged rows (see load_item).
    auto stream = [&](auto even_tag) {
    constexpr bool EVEN = decltype(even_tag)::value;
    while (chunk_tiles > 0) {
        const int n_items = chunk_tiles * CG;
        while (q < n_items) {
            float a[R];
#pragma unroll
            for (int c = 0; c < C; c++) {
                // < nbp; idle column sets carry zero weights
                const int bs = (EVEN ? (cg * C + c) : min((cg * C + c), S - 1)) * kWarp + lane;
                XTile<PLANES> x;
#pragma unroll
                for (int pl = 0; pl < PLANES; pl++) {
                    x.lo[pl] = sm.plane[(pl * 2 + 0) * sm.nbp + bs];
                    x.hi[pl] = sm.plane[(pl * 2 + 1) * sm.nbp + bs];
                }
                x.xs = sm.xs[bs];
                x.bias = sm.bias[bs];
                const bool live = EVEN || (cg * C + c) < S;
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const int I = block_dot<PLANES>(it.w[c][r], x);
                    if constexpr (IDOT) {
                        const int grow = it.row0 + r;
                        const int b = (cg * C + c) * kWarp + lane;
                        if (live && grow < p.n_total && b < p.nb) p.idot[static_cast<long long>(grow) * p.nb + b] = I;
                        a[r] = 0.0f;
                    } else {
                        // per lane the C column sets of the group are added in ascending order, first term exact
                        const float v = live ? __fmul_rn(__fmul_rn(it.s[c][r], x.xs), static_cast<float>(I)) : 0.0f;
                        a[r] = (c == 0) ? v : __fadd_rn(a[r], v);
                    }
                }
            }
            // issue the next item's loads before reducing this one
            const int qn = q + W;
            int tln = tl + step_t, cgn = cg + step_c;
            if (cgn >= CG) {
                cgn -= CG;
                tln++;
            }
            if (qn < n_items) load_item<R, C, PAIR, EVEN>(p, chunk0 + tln, cgn, lane, it);
            if constexpr (!IDOT) {
                warp_sum_multi<R>(a, lane);
                if (multi_row_writer<R>(lane)) sm.part[(tl * R + multi_row_of<R>(lane)) * CG + cg] = a[0];
            }
            q = qn;
            tl = tln;
            cg = cgn;
        }
        __syncthreads();
        if constexpr (!IDOT) {
            // add the column-group partials of every row of the chunk in ascending order, then store
            const int rows = chunk_tiles * R;
            if constexpr (PAIR) {
                // gate row and up row of one index sit in the same tile: out[j] = 16-bit silu(16-bit gate) * 16-bit up,
                // the bits of the GEMV (16-bit outputs) followed by the SiLU*up kernel
                constexpr int H = R / 2;
                for (int i = threadIdx.x; i < chunk_tiles * H; i += kGemvThreads) {
                    const int tl = i / H, j = i - tl * H;
                    const int idx = (chunk0 + tl) * H + j;
                    if (idx >= p.row_end[0]) continue;
                    const float* pg = sm.part + (tl * R + j) * CG;
                    const float* pu = sm.part + (tl * R + H + j) * CG;
                    float yg = pg[0], yu = pu[0];
                    for (int c = 1; c < CG; c++) {
                        yg = __fadd_rn(yg, pg[c]);
                        yu = __fadd_rn(yu, pu[c]);
                    }
                    if constexpr (ODT != NVE_DT_F32) {
                        const float g = Act16<ODT>::to_f32(Act16<ODT>::from_f32(yg));
                        const float u = Act16<ODT>::to_f32(Act16<ODT>::from_f32(yu));
                        store_out<ODT>(p.out[0], idx, silu_mul_f32(g, u));
                    }
                }
            } else {
            for (int i = threadIdx.x; i < rows; i += kGemvThreads) {
                const int grow = chunk0 * R + i;
                if (grow >= p.n_total) continue;
                float y = sm.part[i * CG];
                for (int c = 1; c < CG; c++) y = __fadd_rn(y, sm.part[i * CG + c]);
                if (tp_on) {  // push this rank's partial sum {value, epoch} to every rank; reduced after the last chunk
                    for (int r = 0; r < p.tp.world; r++)
                        st_relaxed_sys_slot(p.tp.ll[r] + tp_plane + grow, __float_as_uint(y), tp_epoch);
                    continue;
                }
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
                    const bool pre = res_pre_ok && first_chunk && i == static_cast<int>(threadIdx.x);
                    y = __fadd_rn(pre ? res_pre : load_out<ODT>(res, lrow), yr);
                }
                store_out<ODT>(out, lrow, y);
            }
            }
        }
        // next chunk
        first_chunk = false;
        chunk0 += chunk_tiles;
        chunk_tiles = min(chunk_tiles_max, tile_end - chunk0);
        __syncthreads();
        q = warp;
        tl = tl0;
        cg = cg0;
        if (chunk_tiles > 0 && q < chunk_tiles * CG) load_item<R, C, PAIR, EVEN>(p, chunk0 + tl, cg, lane, it);
    }

    };
    if ((p.nb % kWarp) == 0 && (S % C) == 0) stream(std::true_type{});
    else stream(std::false_type{});

    if constexpr (PAIR && !IDOT && ODT != NVE_DT_F32) {
        if (p.pq_mode != 0) {
            // ---- conversion of completed 32-wide groups of out[] for the down projection.  A CTA writes a contiguous
            // range of out[]; after its last store it adds, per group it touched, the number of values it wrote to
            // that group's counter.  Whoever brings a counter to a multiple of 32 wrote last: every value of the
            // group is visible (fence before the count, fence after it), and that CTA converts the group with the
            // arithmetic of the stand-alone activation kernels (same bits as SiLU*up + quantise).
            constexpr int H = R / 2;
            __threadfence();
            __syncthreads();
            if (warp == 0) {
                const int lo = tile_begin * H, hi = min(tile_end * H, p.row_end[0]);
                if (hi > lo) {
                    const int g_first = lo >> 5, g_last = (hi - 1) >> 5;
                    const int tq = lane & 3;
                    for (int gb = g_first; gb <= g_last; gb += 8) {
                        const int g = gb + (lane >> 2);
                        int mine = 0;
                        if (tq == 0 && g <= g_last) {
                            const unsigned n = static_cast<unsigned>(min(hi, (g + 1) * 32) - max(lo, g * 32));
                            const unsigned old = atomicAdd(p.pq_cnt + g, n);
                            mine = ((old + n) & 31u) == 0u;
                        }
                        mine = __shfl_sync(0xffffffffu, mine, lane & ~3);
                        if (__any_sync(0xffffffffu, mine)) {
                            __threadfence();
                            const long long chunk = static_cast<long long>(g) * 4 + tq;  // 8 values of the group
                            float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                            if (mine) {
                                const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(p.out[0]) + chunk);
                                uint16_t h[8];
                                unpack8(raw, h);
#pragma unroll
                                for (int e = 0; e < 8; e++) v[e] = Act16<ODT>::to_f32(h[e]);
                            }
                            if (p.pq_mode == 1) {
                                quantize_quad(v, p.pq_xq, p.pq_xs, chunk, mine != 0);
                            } else {
                                if (mine && p.pq_awq != nullptr) {
#pragma unroll
                                    for (int e = 0; e < 8; e++) v[e] = __fmul_rn(v[e], p.pq_awq[chunk * 8 + e]);
                                }
                                x16_quad(v, p.pq_xlo, p.pq_xq, p.pq_xs, chunk, mine != 0);
                            }
                        }
                    }
                }
            }
        }
    }

    if constexpr (!IDOT) {
        if (p.tp.world > 1) {
            // ---- fused all-reduce: every rank has pushed (or is pushing) its partial rows into this rank's buffer;
            // poll the local slots of this CTA's rows until they carry this epoch and add them in rank order.
            // Every rank adds in the same order, so the replicated result is bit-identical everywhere.
            if (threadIdx.x == 0) p.tp.counter[blockIdx.x] = tp_epoch;
            const int row_lo = tile_begin * R;
            const int row_hi = min(tile_end * R, p.n_total);
            const uint2* mine = p.tp.ll[p.tp.rank] + static_cast<size_t>(tp_epoch & 1u) * p.tp.world * p.tp.rows_cap;
            for (int grow = row_lo + threadIdx.x; grow < row_hi; grow += kGemvThreads) {
                float y = 0.0f;
                for (int r = 0; r < p.tp.world; r++) {
                    const uint2* slot = mine + static_cast<size_t>(r) * p.tp.rows_cap + grow;
                    uint2 v = ld_relaxed_sys_slot(slot);
                    for (unsigned spin = 0; v.y != tp_epoch && spin < kTpSpinLimit; spin++) {
                        __nanosleep(32);
                        v = ld_relaxed_sys_slot(slot);
                    }
                    // bounded wait expired: report which rank never arrived, do not hang, and poison the row so
                    // that a finite-check on the hidden state trips instead of a stale partial sum passing silently
                    if (v.y != tp_epoch) {
                        atomicExch(p.tp.err, 1 + r);
                        v.x = 0x7FC00000u;
                    }
                    const float part = __uint_as_float(v.x);
                    y = (r == 0) ? part : __fadd_rn(y, part);
                }
                const void* res = p.res[0];
                if (res != nullptr) {
                    float yr = y;
                    if constexpr (ODT == NVE_DT_F16) yr = Act16<NVE_DT_F16>::to_f32(Act16<NVE_DT_F16>::from_f32(y));
                    if constexpr (ODT == NVE_DT_BF16) yr = Act16<NVE_DT_BF16>::to_f32(Act16<NVE_DT_BF16>::from_f32(y));
                    y = __fadd_rn(load_out<ODT>(res, grow), yr);
                }
                store_out<ODT>(p.out[0], grow, y);
            }
        }
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
    float a = 0.0f;
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
        // same order as the main kernel: per lane the column sets of a group of four in ascending order,
        // xor butterfly over the lanes, then the groups in ascending order
        a = ((s & 3) == 0) ? v : __fadd_rn(a, v);
        if ((s & 3) == 3 || s == p.S - 1) {
            const float part = warp_sum(a);
            y = (s < 4) ? part : __fadd_rn(y, part);
        }
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
template <typename Kern> static int launch_gemv(Kern kern, const GemvParams& p, int planes, int rows_per_item, cudaStream_t stream) {
    const size_t smem = gemv_smem_bytes(planes, p.S);
    if (smem > static_cast<size_t>(kMaxGemvSmem)) return set_status(NVE_ERR_TOO_LARGE);
    if (smem > 48 * 1024) {
        int st = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), kMaxGemvSmem);
        if (st != NVE_OK) return st;
    }
    int grid = 2 * sm_count();
    const int tiles = (p.n_total + rows_per_item - 1) / rows_per_item;
    // The fused all-reduce numbers its launches with a per-CTA counter, so every all-reduce launch of a process must
    // have the same grid whatever its shape: CTAs without tiles still run (and count the launch).
    if (grid > tiles && p.tp.world <= 1) grid = tiles;
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
    return aligned(p.x16, 16);  // PRO 1 and 2 and W4A16 read the 16-bit vector
}

template <int PLANES, int XDT, int ODT, int PRO, bool PAIR = false>
static int dispatch_aligned(const GemvParams& p, int num_mats, cudaStream_t st) {
    if (all_aligned(p, num_mats, PLANES, PRO)) {
        // 8 blocks per lane and item: 2 rows x 4 column sets, or more rows when a row has fewer column sets
        if (p.S >= 3) return launch_gemv(gemv_w4_kernel<PLANES, XDT, ODT, false, PRO, 2, 4, PAIR>, p, PLANES, 2, st);
        if (p.S == 2) return launch_gemv(gemv_w4_kernel<PLANES, XDT, ODT, false, PRO, 4, 2, PAIR>, p, PLANES, 4, st);
        return launch_gemv(gemv_w4_kernel<PLANES, XDT, ODT, false, PRO, 8, 1, PAIR>, p, PLANES, 8, st);
    }
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
            // a row tile (up to 8 rows) must not straddle two matrices
            if (num_mats > 1 && m + 1 < num_mats && (mats[m].N % 8) != 0) return NVE_ERR_BAD_SHAPE;
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
    p.xq = nullptr; p.xs = nullptr; p.x16 = nullptr; p.xlo = nullptr; p.awq = nullptr; p.idot = nullptr;
    p.paired = 0;
    p.pq_mode = 0;
    p.pq_cnt = nullptr;
    p.pq_xq = nullptr;
    p.pq_xlo = nullptr;
    p.pq_xs = nullptr;
    p.pq_awq = nullptr;
    p.norm_w = nullptr; p.eps = 0.0f;
    p.tp.world = 0; p.tp.rank = 0; p.tp.rows_cap = 0; p.tp.err = nullptr;
    p.tp.counter = nullptr;
    for (int r = 0; r < kTpMaxWorld; r++) p.tp.ll[r] = nullptr;
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

extern "C" int nve_b200_matvec_w4a16_planes_multi(const uint8_t* x_lo, const int8_t* x_hi, const float* x_scales,
                                                  const nve_b200_w4_matrix* mats, int num_mats, int K, int out_dtype,
                                                  nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mats, num_mats, K);
    if (st != NVE_OK) return set_status(st);
    if (!x_lo || !x_hi || !x_scales) return set_status(NVE_ERR_BAD_POINTER);
    if (!aligned(x_lo, 16) || !aligned(x_hi, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    for (int m = 0; m < num_mats; m++)
        if (!aligned(mats[m].nibbles, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    p.xlo = x_lo;
    p.xq = x_hi;
    p.xs = x_scales;
    p.x16 = x_lo;  // only its alignment is looked at
    return dispatch_out<2, NVE_DT_F16, 0>(p, num_mats, out_dtype, static_cast<cudaStream_t>(stream));
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
    return launch_gemv(gemv_w4_kernel<1, NVE_DT_F16, NVE_DT_F32, true, 0, 2, 4>, p, 1, 2, static_cast<cudaStream_t>(stream));
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

extern "C" int nve_b200_rmsnorm_matvec_w4a8_awq_multi(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                      const float* awq_inv, const nve_b200_w4_matrix* mats, int num_mats,
                                                      int K, int out_dtype, nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mats, num_mats, K);
    if (st != NVE_OK) return set_status(st);
    if (!h || !norm_weight) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = h;
    p.norm_w = norm_weight;
    p.eps = eps;
    p.awq = awq_inv;
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

static int attach_tp(GemvParams& p);

// ---- gate/up with SiLU*up in the epilogue, down with the quantiser in the prologue (five launches per layer) ----
// Only the 16-bit output type equal to the activation type is built (the form the decode step uses).
template <int PLANES, int XDT, int PRO, bool PAIR = false>
static int dispatch_same_dt(const GemvParams& p, int num_mats, cudaStream_t st) {
    return dispatch_aligned<PLANES, XDT, XDT, PRO, PAIR>(p, num_mats, st);
}

static int fill_gateup(GemvParams& p, const nve_b200_w4_matrix* gate, const nve_b200_w4_matrix* up, void* mid_out, int K) {
    if (!gate || !up || !mid_out) return NVE_ERR_BAD_POINTER;
    if (gate->N != up->N || (gate->N % 8) != 0) return NVE_ERR_BAD_SHAPE;
    nve_b200_w4_matrix m[2] = {*gate, *up};
    m[0].out = mid_out; m[1].out = mid_out;  // the per-matrix outputs are not written in this form
    m[0].residual = nullptr; m[1].residual = nullptr;
    int st = fill_params(p, m, 2, K);
    if (st != NVE_OK) return st;
    p.paired = 1;
    return NVE_OK;
}

extern "C" int nve_b200_rmsnorm_gateup_silu_w4a8(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                 const float* awq_inv, const nve_b200_w4_matrix* gate,
                                                 const nve_b200_w4_matrix* up, void* mid_out, int K, nve_stream_t stream) {
    GemvParams p;
    int st = fill_gateup(p, gate, up, mid_out, K);
    if (st != NVE_OK) return set_status(st);
    if (!h || !norm_weight) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = h; p.norm_w = norm_weight; p.eps = eps; p.awq = awq_inv;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (act_dtype == NVE_DT_F16) return dispatch_same_dt<1, NVE_DT_F16, 1, true>(p, 2, cs);
    if (act_dtype == NVE_DT_BF16) return dispatch_same_dt<1, NVE_DT_BF16, 1, true>(p, 2, cs);
    return set_status(NVE_ERR_BAD_DTYPE);
}

extern "C" int nve_b200_rmsnorm_gateup_silu_w4a16(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                  const float* awq, const nve_b200_w4_matrix* gate,
                                                  const nve_b200_w4_matrix* up, void* mid_out, int K, nve_stream_t stream) {
    GemvParams p;
    int st = fill_gateup(p, gate, up, mid_out, K);
    if (st != NVE_OK) return set_status(st);
    if (!h || !norm_weight) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = h; p.norm_w = norm_weight; p.eps = eps; p.awq = awq;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (act_dtype == NVE_DT_F16) return dispatch_same_dt<2, NVE_DT_F16, 1, true>(p, 2, cs);
    if (act_dtype == NVE_DT_BF16) return dispatch_same_dt<2, NVE_DT_BF16, 1, true>(p, 2, cs);
    return set_status(NVE_ERR_BAD_DTYPE);
}

// The paired form that also leaves silu(gate)*up converted for the down projection (see the end of the kernel).
static int attach_pair_quant(GemvParams& p, int mode, unsigned* counters, int8_t* xq, uint8_t* xlo, float* xs, const float* awq) {
    if (!counters || !xq || !xs || (mode == 2 && !xlo)) return NVE_ERR_BAD_POINTER;
    if ((p.row_end[0] % 32) != 0) return NVE_ERR_BAD_SHAPE;
    if (!aligned(p.out[0], 16) || !aligned(xq, 8) || (xlo && !aligned(xlo, 8))) return NVE_ERR_BAD_ALIGNMENT;
    p.pq_mode = mode;
    p.pq_cnt = counters;
    p.pq_xq = xq;
    p.pq_xlo = xlo;
    p.pq_xs = xs;
    p.pq_awq = awq;
    return NVE_OK;
}

extern "C" int nve_b200_rmsnorm_gateup_silu_q8_w4a8(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                    const float* awq_inv, const nve_b200_w4_matrix* gate,
                                                    const nve_b200_w4_matrix* up, void* mid_out, int K, int8_t* mid_q,
                                                    float* mid_scales, unsigned* group_counters, nve_stream_t stream) {
    GemvParams p;
    int st = fill_gateup(p, gate, up, mid_out, K);
    if (st != NVE_OK) return set_status(st);
    if (!h || !norm_weight) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = h; p.norm_w = norm_weight; p.eps = eps; p.awq = awq_inv;
    st = attach_pair_quant(p, 1, group_counters, mid_q, nullptr, mid_scales, nullptr);
    if (st != NVE_OK) return set_status(st);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (act_dtype == NVE_DT_F16) return dispatch_same_dt<1, NVE_DT_F16, 1, true>(p, 2, cs);
    if (act_dtype == NVE_DT_BF16) return dispatch_same_dt<1, NVE_DT_BF16, 1, true>(p, 2, cs);
    return set_status(NVE_ERR_BAD_DTYPE);
}

extern "C" int nve_b200_rmsnorm_gateup_silu_x16_w4a16(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                      const float* awq, const nve_b200_w4_matrix* gate,
                                                      const nve_b200_w4_matrix* up, void* mid_out, int K, uint8_t* mid_lo,
                                                      int8_t* mid_hi, float* mid_scales, const float* down_awq,
                                                      unsigned* group_counters, nve_stream_t stream) {
    GemvParams p;
    int st = fill_gateup(p, gate, up, mid_out, K);
    if (st != NVE_OK) return set_status(st);
    if (!h || !norm_weight) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = h; p.norm_w = norm_weight; p.eps = eps; p.awq = awq;
    st = attach_pair_quant(p, 2, group_counters, mid_hi, mid_lo, mid_scales, down_awq);
    if (st != NVE_OK) return set_status(st);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (act_dtype == NVE_DT_F16) return dispatch_same_dt<2, NVE_DT_F16, 1, true>(p, 2, cs);
    if (act_dtype == NVE_DT_BF16) return dispatch_same_dt<2, NVE_DT_BF16, 1, true>(p, 2, cs);
    return set_status(NVE_ERR_BAD_DTYPE);
}

static int quantize_matvec_w4a8(const void* x, int x_dtype, const float* awq_inv, const nve_b200_w4_matrix* mats, int num_mats,
                                int K, bool allreduce, cudaStream_t cs) {
    GemvParams p;
    int st = fill_params(p, mats, num_mats, K);
    if (st != NVE_OK) return set_status(st);
    if (!x) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = x;
    p.awq = awq_inv;
    if (allreduce) {
        if (!all_aligned(p, num_mats, 1, 2)) return set_status(NVE_ERR_BAD_ALIGNMENT);
        st = attach_tp(p);
        if (st != NVE_OK) return set_status(st);
    }
    if (x_dtype == NVE_DT_F16) return dispatch_same_dt<1, NVE_DT_F16, 2>(p, num_mats, cs);
    if (x_dtype == NVE_DT_BF16) return dispatch_same_dt<1, NVE_DT_BF16, 2>(p, num_mats, cs);
    return set_status(NVE_ERR_BAD_DTYPE);
}

extern "C" int nve_b200_quantize_matvec_w4a8_multi(const void* x, int x_dtype, const float* awq_inv,
                                                   const nve_b200_w4_matrix* mats, int num_mats, int K, nve_stream_t stream) {
    return quantize_matvec_w4a8(x, x_dtype, awq_inv, mats, num_mats, K, false, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_quantize_matvec_w4a8_allreduce(const void* x, int x_dtype, const float* awq_inv,
                                                       const nve_b200_w4_matrix* mat, int K, nve_stream_t stream) {
    return quantize_matvec_w4a8(x, x_dtype, awq_inv, mat, 1, K, true, static_cast<cudaStream_t>(stream));
}

// ---- tensor-parallel GEMVs: y = all-reduce over the ranks of (W_shard . x_shard), optional residual ----------
static int attach_tp(GemvParams& p) {
    const TpDev& t = tp_device_ctx();
    if (t.world < 2) return NVE_ERR_BAD_POINTER;  // no connected tensor-parallel context
    if (p.n_total > t.rows_cap) return NVE_ERR_TOO_LARGE;
    if (2 * sm_count() > kTpMaxCtas) return NVE_ERR_TOO_LARGE;
    p.tp = t;
    return NVE_OK;
}

extern "C" int nve_b200_matvec_w4a8_allreduce(const int8_t* xq, const float* xq_scales, const nve_b200_w4_matrix* mat,
                                              int K, int out_dtype, nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mat, 1, K);
    if (st != NVE_OK) return set_status(st);
    if (!xq || !xq_scales) return set_status(NVE_ERR_BAD_POINTER);
    p.xq = xq;
    p.xs = xq_scales;
    if (!all_aligned(p, 1, 1, 0)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    st = attach_tp(p);
    if (st != NVE_OK) return set_status(st);
    return dispatch_out<1, NVE_DT_F16, 0>(p, 1, out_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_matvec_w4a16_planes_allreduce(const uint8_t* x_lo, const int8_t* x_hi, const float* x_scales,
                                                      const nve_b200_w4_matrix* mat, int K, int out_dtype,
                                                      nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mat, 1, K);
    if (st != NVE_OK) return set_status(st);
    if (!x_lo || !x_hi || !x_scales) return set_status(NVE_ERR_BAD_POINTER);
    p.xlo = x_lo;
    p.xq = x_hi;
    p.xs = x_scales;
    p.x16 = x_lo;  // only its alignment is looked at
    if (!aligned(x_hi, 16) || !all_aligned(p, 1, 2, 0)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    st = attach_tp(p);
    if (st != NVE_OK) return set_status(st);
    return dispatch_out<2, NVE_DT_F16, 0>(p, 1, out_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_matvec_w4a16_allreduce(const void* x, int x_dtype, const float* awq, const nve_b200_w4_matrix* mat,
                                               int K, int out_dtype, nve_stream_t stream) {
    GemvParams p;
    int st = fill_params(p, mat, 1, K);
    if (st != NVE_OK) return set_status(st);
    if (!x) return set_status(NVE_ERR_BAD_POINTER);
    p.x16 = x;
    p.awq = awq;
    if (!all_aligned(p, 1, 2, 0)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    st = attach_tp(p);
    if (st != NVE_OK) return set_status(st);
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (x_dtype == NVE_DT_F16) return dispatch_out<2, NVE_DT_F16, 0>(p, 1, out_dtype, cs);
    if (x_dtype == NVE_DT_BF16) return dispatch_out<2, NVE_DT_BF16, 0>(p, 1, out_dtype, cs);
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
    if (same_awq && Nq > 0 && Nk > 0 && Nv > 0 && (Nq % 8) == 0 && (Nk % 8) == 0) {
        nve_b200_matvec_w4a16_multi(x, NVE_DT_F16, q_awq, m, 3, K, NVE_DT_F16, stream);
        return;
    }
    const float* awqs[3] = {q_awq, k_awq, v_awq};
    for (int i = 0; i < 3; i++) {
        if (m[i].N > 0) nve_b200_matvec_w4a16_multi(x, NVE_DT_F16, awqs[i], &m[i], 1, K, NVE_DT_F16, stream);
    }
}
