// Batched W4A16 GEMM for narrow batches (M <= 32):  Y[M,N] = X[M,K] . W^T  with the packed weights streamed
// from HBM straight into registers, dequantised there and multiplied on the tensor cores with mma.sync.
//
// Same contract, work split and partial-tile layout as the tcgen05 kernel (gemm_w4a16_tc.cu), which it replaces
// where the batch is narrow: there the operation is a weight stream with a little arithmetic attached, and what
// bounds it is the number of instructions per weight and the bytes in flight per SM, not the tensor pipe.  The
// tcgen05 form pays for its pipeline (raw bytes -> shared memory -> registers -> tensor memory -> MMA, with an
// mbarrier hand-off at every arrow) about 4.5 instructions per weight; this form needs about 2 (1.75 of them the
// dequantisation itself) and no hand-off besides one CTA barrier per unit for the activation tile.
//
// Mapping.  A unit is 128 weight rows x 256 weights per row.  A CTA has 16 warps: warp w takes the 16 rows
// 16 (w & 7) .. +15 of the tile and the half w >> 3 of the unit's K range (128 weights per row).  The weight rows
// are the M dimension of mma.m16n8k16 (A operand), the batch is its N dimension (B operand, 8 batch rows per
// instruction), so one instruction covers 16 rows x 16 weights for 8 batch rows.
// The contraction index of an MMA can be permuted freely as long as both operands use the same permutation.
// Lane (g, t) = (lane / 4, lane % 4) loads one 16-byte group (32 weights, one scale) of row g and one of row g + 8,
// the groups t of the warp's 128-weight span, and feeds element 4j .. 4j+3 of its groups to MMA j (j < 4) and
// 16 + 4(j-4) .. +3 to MMA j >= 4: a 16-byte load per row is all the address arithmetic there is, and a warp-wide
// load touches 8 rows x 64 contiguous bytes.  The matching activations X[m][32t + ...] are staged once per CTA and
// unit in shared memory in exactly the order in which lanes read them (fragment-major: [K half][8-row batch
// group][quarter][lane] x 16 bytes), so the reads are conflict-free 128-bit loads.
// Weight loads run kDepth units ahead in registers (a ring that is unrolled, so the indices are static); the
// activation tiles run kXStages - 1 units ahead through cp.async.  One __syncthreads per unit publishes the next
// tile and retires the previous one.
// At the end of a segment (the part of a tile inside this CTA's run) the two K halves meet in a shared-memory
// tile, second half added to the first, and the tile is stored with coalesced rows -- to Y if the segment is the
// whole tile, else as an f32 partial tile for the reduce kernel, which adds the CTAs' partials in ascending K order.
// The result is reproducible for a given SM count; it differs from the tcgen05 kernel's in the order of the f32
// additions only (same f16 weights, same f16 activations).
#include "gemm_w4a16.cuh"

namespace nve {

constexpr int kMmaThreads = 512;
constexpr int kMmaWarps = kMmaThreads / 32;
constexpr int kXStages = 4;            // activation tiles in the shared-memory ring
constexpr int kTilePitch = kTileN + 4; // floats per batch row of the segment tile: lanes (g, t) hit 32 distinct banks

template <int NT> struct MmaCfg {
    static constexpr int kDepth = NT <= 2 ? 6 : 4;            // units of weights in flight per lane
    static constexpr int kChains = NT <= 2 ? 2 : 1;           // accumulator sets per batch group (even / odd MMAs)
    static constexpr int kStageBytes = NT * 8 * 512;          // one activation tile: NT*8 batch rows x 256 f16
    static constexpr int kSmemBytes = kXStages * kStageBytes + NT * 8 * kTilePitch * 4;
};

__device__ __forceinline__ void mma_f16_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 bytes global -> shared, or 16 zero bytes when `valid` is false (the source address must still be mapped)
__device__ __forceinline__ void cp_async_16_zfill(uint32_t dst, const void* src, bool valid) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}

template <int NT, int ODT>
__global__ void __launch_bounds__(kMmaThreads, 1) gemm_w4a16_mma_kernel(const GemmParams p) {
    using Cfg = MmaCfg<NT>;
    constexpr int D = Cfg::kDepth;
    extern __shared__ __align__(16) unsigned char smem[];
    float* sT = reinterpret_cast<float*>(smem + kXStages * Cfg::kStageBytes);  // [NT*8][kTilePitch]
    const uint32_t sX = s_addr(smem);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rt = warp & 7, kh = warp >> 3;
    const int SB = p.sb_per_tile;
    const int u0 = blockIdx.x * p.units_per_cta;
    const int n_units = min(p.units_per_cta, p.total_units - u0);
    const DequantConsts dc = make_dequant_consts();

    // ---- load cursor: the unit whose weights are requested next, kDepth units ahead of the arithmetic.  Its row
    // pointers are recomputed only when it enters a new tile; inside a tile a unit is 128 bytes of nibbles and 8
    // scales further along the row.
    const int kq = kh * 4 + t;  // this lane's group of 32 weights inside a unit
    int l_tile = u0 / SB, l_sbi = u0 - l_tile * SB;
    const uint8_t* wp[2] = {nullptr, nullptr};
    const float* sp[2] = {nullptr, nullptr};
    auto load_enter_tile = [&]() {
        if (l_tile >= p.tile_end[2]) return;
        int mi, n0;
        tile_locate(p, l_tile, mi, n0);
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const int n = min(n0 + 16 * rt + g + 8 * r, p.Nm[mi] - 1);
            wp[r] = p.nib[mi] + static_cast<long long>(n) * (p.K >> 1) + (l_sbi * 8 + kq) * 16;
            sp[r] = p.sc[mi] + static_cast<long long>(n) * p.nb + l_sbi * 8 + kq;
        }
    };
    load_enter_tile();
    uint4 wq[D][2];
    float ws[D][2];
    auto load_w = [&](uint4 (&q)[2], float (&sc)[2]) {
        if (l_sbi * 8 + kq < p.nb) {
#pragma unroll
            for (int r = 0; r < 2; r++) {
                q[r] = ld_stream_u4(wp[r]);
                sc[r] = ld_stream_f32(sp[r]);
            }
        } else {  // beyond the end of a K that is not a multiple of 256: q = 8 everywhere, zero weights
#pragma unroll
            for (int r = 0; r < 2; r++) {
                q[r] = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);
                sc[r] = 0.0f;
            }
        }
        l_sbi++;
        wp[0] += 128; wp[1] += 128;
        sp[0] += 8; sp[1] += 8;
        if (l_sbi == SB) {
            l_sbi = 0;
            l_tile++;
            load_enter_tile();
        }
    };
    // ---- activation tiles: unit j -> ring slot j % kXStages, fragment-major; batch rows >= M and K beyond the end
    // read zero.  A thread always copies the same pieces (batch row m, 16-byte piece c of the row's 512-byte span).
    constexpr int PP = (NT * 8 * 32 + kMmaThreads - 1) / kMmaThreads;
    const uint16_t* x_src[PP];
    uint32_t x_dst[PP];
    int x_k[PP];  // first K index of the piece inside a unit, or a value that fails every bounds test
#pragma unroll
    for (int i = 0; i < PP; i++) {
        const int idx = tid + i * kMmaThreads;
        const int m = idx >> 5, c = idx & 31;
        const bool mine = idx < NT * 8 * 32 && m < p.M;
        x_src[i] = p.X + (mine ? static_cast<long long>(m) * p.K + c * 8 : 0);
        x_k[i] = mine ? c * 8 : 0x40000000;
        const int xh = c >> 4, xt = (c >> 2) & 3, xq = c & 3;
        x_dst[i] = sX + ((((xh * NT + (m >> 3)) * 4 + xq) * 32 + (m & 7) * 4 + xt) << 4);
    }
    int x_sbi = u0 % SB;
    auto stage_x = [&](int j) {
        if (j < n_units) {
            const uint32_t slot = (j % kXStages) * Cfg::kStageBytes;
            const int k0 = x_sbi * 256;
#pragma unroll
            for (int i = 0; i < PP; i++) {
                if (PP * kMmaThreads == NT * 8 * 32 || tid + i * kMmaThreads < NT * 8 * 32) {
                    const bool valid = k0 + x_k[i] < p.K;
                    cp_async_16_zfill(x_dst[i] + slot, valid ? x_src[i] + k0 : p.X, valid);
                }
            }
            x_sbi = x_sbi + 1 == SB ? 0 : x_sbi + 1;
        }
        cp_async_commit();  // one group per unit, empty or not, so that the wait below counts units
    };

    // the weights do not depend on the previous kernel: they are requested before the grid dependency resolves
#pragma unroll
    for (int d = 0; d < D; d++)
        if (d < n_units) load_w(wq[d], ws[d]);
    pdl_wait();
#pragma unroll
    for (int st = 0; st < kXStages - 1; st++) stage_x(st);

    constexpr int C = Cfg::kChains;
    float acc[NT][C][4];
    auto zero_acc = [&]() {
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int c = 0; c < C; c++) acc[nt][c][0] = acc[nt][c][1] = acc[nt][c][2] = acc[nt][c][3] = 0.0f;
    };
    zero_acc();
    int seg = 0, seg_sbi0 = u0 % SB;
    int c_tile = u0 / SB, c_sbi = seg_sbi0;  // the unit the arithmetic is at

    for (int jb = 0; jb < n_units; jb += D) {
#pragma unroll
        for (int d = 0; d < D; d++) {
            const int j = jb + d;
            if (j >= n_units) break;
            cp_async_wait<kXStages - 2>();  // this thread's pieces of tile j have landed
            __syncthreads();                // everybody's have, and everybody is done with tile j - 1
            stage_x(j + kXStages - 1);      // into the slot of tile j - 1
            // ---- 16 rows x 128 weights x NT*8 batch rows
            {
                const unsigned char* xs = smem + (j % kXStages) * Cfg::kStageBytes + ((kh * NT * 4) * 32 + lane) * 16;
                const DequantScale s0 = make_dequant_scale(ws[d][0]), s1 = make_dequant_scale(ws[d][1]);
                const uint32_t* w0 = reinterpret_cast<const uint32_t*>(&wq[d][0]);
                const uint32_t* w1 = reinterpret_cast<const uint32_t*>(&wq[d][1]);
                uint4 xq[NT][4];
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int q = 0; q < 4; q++) xq[nt][q] = *reinterpret_cast<const uint4*>(xs + ((nt * 4 + q) * 32) * 16);
                // word w of the two rows -> MMA 2w (elements 4w..4w+3 of the group) and MMA 2w+1 (16+4w..16+4w+3);
                // the two go to different accumulator chains, so consecutive instructions do not wait for each other
#pragma unroll
                for (int w = 0; w < 4; w++) {
                    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
                    dequant_word(w0[w], s0, dc, a0, a2, b0, b2);
                    dequant_word(w1[w], s1, dc, a1, a3, b1, b3);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const uint4& lo = xq[nt][w >> 1];       // elements 8 (w/2) .. +7 hold 4w .. 4w+3
                        const uint4& hi = xq[nt][2 + (w >> 1)];  // and 16 + 4w .. 16 + 4w+3
                        if ((w & 1) == 0) {
                            mma_f16_m16n8k16(acc[nt][0], a0, a1, a2, a3, lo.x, lo.y);
                            mma_f16_m16n8k16(acc[nt][C - 1], b0, b1, b2, b3, hi.x, hi.y);
                        } else {
                            mma_f16_m16n8k16(acc[nt][0], a0, a1, a2, a3, lo.z, lo.w);
                            mma_f16_m16n8k16(acc[nt][C - 1], b0, b1, b2, b3, hi.z, hi.w);
                        }
                    }
                }
            }
            if (j + D < n_units) load_w(wq[d], ws[d]);
            // ---- end of a segment: the tile ends here, or the run does
            const bool tile_ends = c_sbi == SB - 1;
            if (tile_ends || j == n_units - 1) {
                int mi, n0;
                tile_locate(p, c_tile, mi, n0);
                const bool whole = seg_sbi0 == 0 && tile_ends;
                // lane (g, t) holds batch rows 8 nt + 2t, + 1 of output features 16 rt + g, + 8
                if (C == 2) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++)
#pragma unroll
                        for (int e = 0; e < 4; e++) acc[nt][0][e] = __fadd_rn(acc[nt][0][e], acc[nt][C - 1][e]);
                }
                __syncthreads();  // (the tile may still be read by the previous segment's stores)
                if (kh == 1) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        float* row = sT + (8 * nt + 2 * t) * kTilePitch + 16 * rt + g;
                        row[0] = acc[nt][0][0];
                        row[kTilePitch] = acc[nt][0][1];
                        row[8] = acc[nt][0][2];
                        row[kTilePitch + 8] = acc[nt][0][3];
                    }
                }
                __syncthreads();
                if (kh == 0) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        float* row = sT + (8 * nt + 2 * t) * kTilePitch + 16 * rt + g;
                        row[0] = __fadd_rn(acc[nt][0][0], row[0]);
                        row[kTilePitch] = __fadd_rn(acc[nt][0][1], row[kTilePitch]);
                        row[8] = __fadd_rn(acc[nt][0][2], row[8]);
                        row[kTilePitch + 8] = __fadd_rn(acc[nt][0][3], row[kTilePitch + 8]);
                    }
                }
                __syncthreads();
                const int Nloc = p.Nm[mi];
                float* part = p.partial + static_cast<long long>(2 * blockIdx.x + (seg > 0 ? 1 : 0)) * p.M * kTileN;
                for (int i = tid; i < p.M * kTileN; i += kMmaThreads) {
                    const int m = i >> 7, nl = i & (kTileN - 1);
                    const float y = sT[m * kTilePitch + nl];
                    if (!whole) part[i] = y;
                    else if (n0 + nl < Nloc) store_out<ODT>(p.Y[mi], static_cast<long long>(m) * Nloc + n0 + nl, y);
                }
                zero_acc();
                seg++;
                seg_sbi0 = 0;
            }
            c_sbi++;
            if (tile_ends) {
                c_sbi = 0;
                c_tile++;
            }
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();
}

template <int NT, int ODT> static int launch_gemm_mma(const GemmParams& p, cudaStream_t st) {
    auto kern = gemm_w4a16_mma_kernel<NT, ODT>;
    constexpr int smem = MmaCfg<NT>::kSmemBytes;
    int s = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem);
    if (s != NVE_OK) return s;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.total_units + p.units_per_cta - 1) / p.units_per_cta);
    cfg.blockDim = dim3(kMmaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    count_launch();
    if (e != cudaSuccess) return set_cuda_status(e);
    return NVE_OK;
}

template <int ODT> static bool gemm_mma_nt(const GemmParams& p, cudaStream_t st, int& status) {
    if (p.M <= 8) status = launch_gemm_mma<1, ODT>(p, st);
    else if (p.M <= 16) status = launch_gemm_mma<2, ODT>(p, st);
    else if (p.M <= 32) status = launch_gemm_mma<4, ODT>(p, st);
    else return false;
    return true;
}

bool gemm_mma_try(const GemmParams& p, int y_dtype, cudaStream_t st, int& status) {
    if (y_dtype == NVE_DT_F32) return gemm_mma_nt<NVE_DT_F32>(p, st, status);
    if (y_dtype == NVE_DT_F16) return gemm_mma_nt<NVE_DT_F16>(p, st, status);
    return gemm_mma_nt<NVE_DT_BF16>(p, st, status);
}

}  // namespace nve
