// Decode attention on the tensor cores, one cluster per KV head: RoPE + K/V write + single-query GQA attention +
// optional int8 quantisation of the output, the fused step between the q/k/v GEMV and o_proj of a decode layer
// (FUSED); the plain flash-decode form of the same arithmetic (nve_flash_decode_f16, the rows of a small causal
// block), so that the fused launch equals the un-fused launch sequence bit for bit; and a few independent sequences
// in one launch (batched decode).
//
// Same interface and the same place in the step as the clustered CUDA-core kernel (attn_decode.cu), which spends
// most of its time on dot products with shuffle reductions (about 1200 instructions per thread for 1024 positions).
// Here a cluster of 8 CTAs serves one KV head with ALL its G query heads (K and V are read once, not once per pair
// of heads); CTA `rank` owns the positions [rank*chunk, (rank+1)*chunk), its eight warps take 16-position tiles of
// them, and a tile is eight score MMAs and HD/8 output MMAs (attn_mma.cuh).  The first tile of every warp is loaded
// before the grid dependency resolves (the cache rows of earlier positions do not depend on the producer kernel);
// the row of the new token is taken from shared memory instead of the cache.  The eight warps' partials meet in
// shared memory; the CTAs of ranks 1..7 post their partial into rank 0's shared memory with asynchronous
// distributed-shared-memory stores that count their bytes on an mbarrier of rank 0 (st.async ... complete_tx) and
// leave; rank 0 waits for the bytes (bounded in time; an expired wait writes NaN so that the failure is visible),
// merges, normalises, stores and quantises.
// Probabilities are rounded to f16 for the second MMA and sums run in a different order, so results agree with the
// CUDA-core kernel within rounding, not bit for bit.
#include <cooperative_groups.h>

#include <cstddef>

#include "attn_mma.cuh"
#include "attn_params.cuh"

namespace cg = cooperative_groups;

namespace nve {

// Shared memory of a CTA.  q is kept as f16 in the order in which the MMA lanes read it: qf[kk][t * 8 + g] holds the
// four elements DPT*t + 4*kk .. +3 of head g's rotated q (rows g >= G stay zero), so that a lane's fragment load is
// one conflict-free 8-byte read per MMA.
template <int HD, int G> struct AdmShared {
    __align__(8) uint16_t qf[HD / 16][32][4];
    __align__(16) uint16_t knew_s[HD];
    __align__(16) uint16_t vnew_s[HD];
    float wm[kAmWarps][G], wl[kAmWarps][G];
    float wo[kAmWarps][G][am_wo_row(HD)];
};

__device__ __forceinline__ uint32_t adm_smem_addr(const void* ptr) { return static_cast<uint32_t>(__cvta_generic_to_shared(ptr)); }
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t adm_map_rank(uint32_t cta_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
    return r;
}
// posted 4-byte store into another CTA's shared memory that counts its bytes on that CTA's mbarrier when it lands
__device__ __forceinline__ void adm_st_async(uint32_t cluster_addr, float v, uint32_t cluster_mbar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(cluster_addr),
                 "r"(__float_as_uint(v)), "r"(cluster_mbar)
                 : "memory");
}
constexpr unsigned long long kAdmWaitLimitNs = 20ull * 1000 * 1000;  // a legitimate wait lasts a microsecond

template <int HD, int G> struct AdmSmem {
    AdmShared<HD, G> sh;
    AdCtaPartial<HD, G> parts[kAdRanks];
    __align__(8) unsigned long long pbar;
};

// With `rows` > 1 (batched decode) blockIdx.y selects one of several independent sequences: row b of q / k_new /
// v_new / out, the b-th K/V cache and the b-th position and length words.
// FUSED = false is the plain flash-decode form (nve_flash_decode_f16 and the rows of a small causal block): q is
// already rotated, nothing is written to the cache, the length is *d_seq_len or seq_len, and blockIdx.y selects one of
// `rows` query rows, row r reading q + r * row_stride and attending to seq_len + r positions.
template <int HD, int G, bool FUSED>
__global__ void __launch_bounds__(kAmThreads, 1) attn_decode_mma_kernel(const AttnParams pin) {
    AttnParams p = pin;
    int seq_len_row = p.seq_len;
    if constexpr (!FUSED) {
        p.q += static_cast<long long>(blockIdx.y) * p.row_stride;
        p.out += static_cast<long long>(blockIdx.y) * p.row_stride;
        seq_len_row += static_cast<int>(blockIdx.y);
    }
    if (FUSED && p.rows > 1) {
        const long long b = blockIdx.y;
        p.q += b * (static_cast<long long>(p.num_heads) * HD);
        p.out += b * (static_cast<long long>(p.num_heads) * HD);
        p.k_new += b * (static_cast<long long>(p.num_kv_heads) * HD);
        p.v_new += b * (static_cast<long long>(p.num_kv_heads) * HD);
        p.k_cache += b * p.cache_stride;
        p.v_cache += b * p.cache_stride;
        p.d_pos += b;
        p.d_seq_len += b;
    }
    constexpr int DC = HD / 8;
    constexpr int NT = HD / 8;
    static_assert((HD == 64 || HD == 128) && G >= 1 && G <= 8, "head_dim 64 or 128, up to 8 query heads per KV head");
    cg::cluster_group cluster = cg::this_cluster();
    constexpr int HALF = HD / 2, DPT = HD / 4;
    static_assert(HD <= kAmThreads, "one element of k and v per thread");
    extern __shared__ __align__(16) unsigned char adm_smem[];
    AdmSmem<HD, G>& sm = *reinterpret_cast<AdmSmem<HD, G>*>(adm_smem);
    AdmShared<HD, G>& sh = sm.sh;
    AdCtaPartial<HD, G>* parts = sm.parts;  // only rank 0's copy is used
    unsigned long long& pbar = sm.pbar;     // rank 0: counts the bytes of the other ranks' partials
    constexpr uint32_t kPartBytes = (G * HD + 2 * G) * 4;
    if (cluster.block_rank() == 0 && threadIdx.x == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(adm_smem_addr(&pbar)));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(adm_smem_addr(&pbar)), "r"((kAdRanks - 1) * kPartBytes)
                     : "memory");
    }
    // The cluster barrier: every CTA announces that it runs (and rank 0 that its mbarrier is set up), so that the
    // pushes into rank 0's shared memory never touch a CTA that has not started (matched by the wait in front of the push)
    cluster.barrier_arrive();

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int rank = static_cast<int>(cluster.block_rank());
    const int kvh = blockIdx.x / kAdCluster;
    const int h0 = kvh * G;
    const uint16_t* kh = p.k_cache + static_cast<long long>(kvh) * p.kv_stride * HD;
    const uint16_t* vh = p.v_cache + static_cast<long long>(kvh) * p.kv_stride * HD;

    // ---- before the wait: this warp's first tile, addressed with the position words as they are now (read again
    // after the wait; the tile is loaded again if they changed)
    const int pre_seq = max(0, min(p.d_seq_len != nullptr ? *p.d_seq_len : seq_len_row, p.kv_stride));
    const int pre_pos = FUSED ? *p.d_pos : -1;
    uint4 kr[2][HD / 32], vr[4][HD / 64];
    {
        const int pchunk = (pre_seq + kAdRanks - 1) / kAdRanks;
        const int pb = rank * pchunk, pe = min(pre_seq, pb + pchunk);
        const int p0 = pb + warp * 16;
        if (p0 < pe) am_load_tile<HD>(kh, vh, p0, pe - 1, g, t, kr, vr);
    }
    // the RoPE row of the guessed position does not depend on the producer either; rows g >= G of the q fragments are zero
    // this thread's element pairs (qe, qe + HALF) of the heads qh, qh + HPP, ... (those below G) ...
    constexpr int HPP = kAmThreads / HALF;        // heads covered by one pass of the CTA's threads
    constexpr int QI = (G + HPP - 1) / HPP;       // passes
    const int qe = tid % HALF, qh = tid / HALF;
    const bool spec_ok = pre_pos >= 0 && pre_pos < p.kv_stride;
    uint16_t c16 = 0, s16 = 0;
    if constexpr (FUSED) {
        c16 = p.cos_tab[static_cast<long long>(spec_ok ? pre_pos : 0) * HALF + qe];
        s16 = p.sin_tab[static_cast<long long>(spec_ok ? pre_pos : 0) * HALF + qe];
    }
    for (int i = tid; i < (HD / 16) * 32 * 2; i += kAmThreads) reinterpret_cast<uint32_t*>(sh.qf)[i] = 0;
    pdl_wait();
    // one round trip: the position words are read again while q, k and v of the new token come in; everything that
    // was addressed with the guess is redone in the rare case that the words changed
    uint16_t x0[QI], x1[QI];
#pragma unroll
    for (int j = 0; j < QI; j++) {
        const int h = qh + j * HPP;
        const uint16_t* qp = p.q + static_cast<long long>(h0 + (h < G ? h : 0)) * HD;
        x0[j] = qp[qe];
        x1[j] = qp[qe + HALF];
    }
    uint16_t k0 = 0, k1 = 0, vv = 0;
    if constexpr (FUSED) {
        const uint16_t* kp = p.k_new + static_cast<long long>(kvh) * HD;
        if (tid < HALF) {  // ... and, for the first HALF threads, of the new k
            k0 = kp[qe];
            k1 = kp[qe + HALF];
        }
        if (tid < HD) vv = p.v_new[static_cast<long long>(kvh) * HD + tid];
    }
    int seq_len = p.d_seq_len != nullptr ? *reinterpret_cast<const volatile int*>(p.d_seq_len) : seq_len_row;
    int pos = -1;
    if constexpr (FUSED) pos = *reinterpret_cast<const volatile int*>(p.d_pos);
    seq_len = max(0, min(seq_len, p.kv_stride));
    const bool pos_ok = FUSED && pos >= 0 && pos < p.kv_stride;
    const bool pre_ok = pre_seq == seq_len && pre_pos == pos;
    if (FUSED && pos != pre_pos) {  // uniform over the grid
        c16 = p.cos_tab[static_cast<long long>(pos_ok ? pos : 0) * HALF + qe];
        s16 = p.sin_tab[static_cast<long long>(pos_ok ? pos : 0) * HALF + qe];
    }
    __syncthreads();  // the zeros above are in place
    {
        // the rotation of attn_stage_q / the stand-alone RoPE kernel: same IEEE operations, same 16-bit rounding
        const float c = Act16<NVE_DT_F16>::to_f32(c16), sn = Act16<NVE_DT_F16>::to_f32(s16);
        auto rot = [&](uint16_t a, uint16_t b, uint16_t& r0, uint16_t& r1) {
            const float f0 = Act16<NVE_DT_F16>::to_f32(a), f1 = Act16<NVE_DT_F16>::to_f32(b);
            r0 = Act16<NVE_DT_F16>::from_f32(__fsub_rn(__fmul_rn(f0, c), __fmul_rn(f1, sn)));
            r1 = Act16<NVE_DT_F16>::from_f32(__fadd_rn(__fmul_rn(f0, sn), __fmul_rn(f1, c)));
        };
#pragma unroll
        for (int j = 0; j < QI; j++) {
            const int h = qh + j * HPP;
            if (h < G) {
                uint16_t r0 = x0[j], r1 = x1[j];
                if constexpr (FUSED) rot(x0[j], x1[j], r0, r1);
                const int d0 = qe, d1 = qe + HALF;  // dim d -> lane quarter t = d / DPT, MMA kk = (d % DPT) / 4, slot d % 4
                sh.qf[(d0 % DPT) / 4][(d0 / DPT) * 8 + h][d0 % 4] = r0;
                sh.qf[(d1 % DPT) / 4][(d1 / DPT) * 8 + h][d1 % 4] = r1;
            }
        }
        if constexpr (FUSED) {
            if (tid < HALF) rot(k0, k1, sh.knew_s[qe], sh.knew_s[qe + HALF]);
            if (tid < HD) sh.vnew_s[tid] = vv;
        }
    }
    __syncthreads();
    pdl_launch_dependents();
    // one CTA per KV head stores the new row; the tiles that cover `pos` take it from shared memory
    if (FUSED && pos_ok && rank == 0 && tid < 2 * DC) {
        const int which = tid / DC, d = tid % DC;
        uint16_t* dst = (which == 0 ? p.k_cache : p.v_cache) + (static_cast<long long>(kvh) * p.kv_stride + pos) * HD;
        reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(which == 0 ? sh.knew_s : sh.vnew_s)[d];
    }

    uint32_t qa[HD / 16][4];
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
        const uint2 f = *reinterpret_cast<const uint2*>(sh.qf[kk][t * 8 + g]);
        qa[kk][0] = f.x;
        qa[kk][1] = 0;
        qa[kk][2] = f.y;
        qa[kk][3] = 0;
    }
    float m = -1e30f, l = 0.0f;
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    const int chunk = (seq_len + kAdRanks - 1) / kAdRanks;
    const int t_begin = rank * chunk;
    const int t_end = min(seq_len, t_begin + chunk);
    bool have = pre_ok;  // the first tile is already in registers
    for (int p0 = t_begin + warp * 16; p0 < t_end; p0 += kAmWarps * 16) {
        if (!have) am_load_tile<HD>(kh, vh, p0, t_end - 1, g, t, kr, vr);
        have = false;
        if (pos_ok) am_patch_tile<HD>(sh.knew_s, sh.vnew_s, p0, pos, g, t, kr, vr);
        am_tile<HD>(qa, kr, vr, p0, t_end, p.scale, t, m, l, o);
    }

    // ---- level 1: the warps' partials meet in shared memory; level 2: every CTA's partial goes to rank 0
    am_store_warp_partial<HD, G>(sh, warp, g, t, m, l, o);
    __syncthreads();
    cluster.barrier_wait();  // all CTAs of the cluster run
    // Ranks 1..7 post their partial into rank 0's parts[rank] with asynchronous stores that count their bytes on rank
    // 0's mbarrier, and leave: no second cluster barrier, rank 0 waits for the bytes only.
    using Part = AdCtaPartial<HD, G>;
    const uint32_t remote = adm_map_rank(adm_smem_addr(&parts[rank]), 0);
    const uint32_t remote_bar = adm_map_rank(adm_smem_addr(&pbar), 0);
#pragma unroll
    for (int i = tid; i < G * HD; i += kAmThreads) {
        const int h = i / HD, d = i % HD;
        float mm, ss, a;
        am_merge_warps<HD, G>(sh, h, d, mm, ss, a);
        if (rank == 0) {
            parts[0].acc[h][d] = a;
            if (d == 0) {
                parts[0].m[h] = mm;
                parts[0].s[h] = ss;
            }
        } else {
            adm_st_async(remote + static_cast<uint32_t>(offsetof(Part, acc) + (h * HD + d) * 4), a, remote_bar);
            if (d == 0) {
                adm_st_async(remote + static_cast<uint32_t>(offsetof(Part, m) + h * 4), mm, remote_bar);
                adm_st_async(remote + static_cast<uint32_t>(offsetof(Part, s) + h * 4), ss, remote_bar);
            }
        }
    }
    if (rank != 0) return;
    __syncthreads();  // rank 0's own partial
    bool arrived = false;
    {
        const uint32_t bar = adm_smem_addr(&pbar);
        unsigned long long t0 = 0, tn = 0;
        for (int spin = 0; !arrived; spin++) {
            uint32_t done;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
                "selp.u32 %0, 1, 0, p;\n\t}"
                : "=r"(done)
                : "r"(bar)
                : "memory");
            arrived = done != 0;
            if (!arrived && (spin & 63) == 63) {  // bounded in time: a partial that never arrives poisons the output below
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tn));
                if (t0 == 0) t0 = tn;
                else if (tn - t0 > kAdmWaitLimitNs) break;
            }
        }
    }
#pragma unroll
    for (int i = tid; i < G * HD; i += kAmThreads) {
        const int h = i / HD, d = i % HD;
        float pm[kAdRanks], mm = -1e30f;
#pragma unroll
        for (int r = 0; r < kAdRanks; r++) {
            pm[r] = parts[r].m[h];
            mm = fmaxf(mm, pm[r]);
        }
        float ss = 0.0f, a = 0.0f;
#pragma unroll
        for (int r = 0; r < kAdRanks; r++) {  // ranks in ascending order
            const float c = __expf(pm[r] - mm);
            ss = fmaf(parts[r].s[h], c, ss);
            a = fmaf(parts[r].acc[h][d], c, a);
        }
        const uint16_t o16 = arrived ? Act16<NVE_DT_F16>::from_f32(ss > 0.0f ? a / ss : 0.0f) : static_cast<uint16_t>(0x7E00);  // NaN
        const long long oi = static_cast<long long>(h0 + h) * HD + d;
        p.out[oi] = o16;
        if (p.out_q != nullptr) {
            // i advances by whole warps and HD is a multiple of 32: the 32 lanes of a warp hold one group
            float scale;
            const int qv = attn_quantize_lane(o16, scale);
            p.out_q[oi] = static_cast<int8_t>(qv);
            if ((tid & 31) == 0) p.out_scales[oi >> 5] = scale;
        }
    }
}

template <int HD, int G, bool FUSED> static cudaError_t launch_adm_f(const AttnParams& p, cudaStream_t st) {
    constexpr int smem = static_cast<int>(sizeof(AdmSmem<HD, G>));
    if (ensure_dynamic_smem(reinterpret_cast<const void*>(attn_decode_mma_kernel<HD, G, FUSED>), smem) != NVE_OK) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.dynamicSmemBytes = smem;
    cfg.gridDim = dim3(p.num_kv_heads * kAdCluster, p.rows > 1 ? p.rows : 1);  // fused: sequences; else: query rows
    cfg.blockDim = dim3(kAmThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kAdCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (pdl_enabled()) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    return cudaLaunchKernelEx(&cfg, attn_decode_mma_kernel<HD, G, FUSED>, p);
}
template <int HD, int G> static cudaError_t launch_adm(const AttnParams& p, cudaStream_t st, bool fused) {
    return fused ? launch_adm_f<HD, G, true>(p, st) : launch_adm_f<HD, G, false>(p, st);
}

// Fused decode attention of one sequence; false when the shape is not covered (query heads per KV head other than
// 1, 2, 4 or 8, other head sizes): the caller then uses the CUDA-core kernel.
bool attn_decode_mma_try(const AttnParams& p, int head_dim, cudaStream_t st, cudaError_t& err, bool fused) {
    const int groups = p.num_heads / p.num_kv_heads;
    if (head_dim == 128) {
        switch (groups) {
            case 1: err = launch_adm<128, 1>(p, st, fused); return true;
            case 2: err = launch_adm<128, 2>(p, st, fused); return true;
            case 4: err = launch_adm<128, 4>(p, st, fused); return true;
            case 8: err = launch_adm<128, 8>(p, st, fused); return true;
            default: return false;
        }
    }
    if (head_dim == 64) {
        switch (groups) {
            case 1: err = launch_adm<64, 1>(p, st, fused); return true;
            case 2: err = launch_adm<64, 2>(p, st, fused); return true;
            case 4: err = launch_adm<64, 4>(p, st, fused); return true;
            case 8: err = launch_adm<64, 8>(p, st, fused); return true;
            default: return false;
        }
    }
    return false;
}

}  // namespace nve
