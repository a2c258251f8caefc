// Batched decode attention on the tensor cores: RoPE + K/V write + single-query GQA attention for MANY independent
// sequences in one launch, for batches large enough to fill the GPU without splitting a sequence.
//
// The clustered decode kernel (attn_decode.cu) is a latency design: eight CTAs share one sequence's positions and every
// thread does CUDA-core dot products with shuffles.  When it has to stream hundreds of MB of K/V (64 sequences x
// 4.2 MB) it is bound by its instruction count (1.9 TB/s).  Here one CTA owns one (sequence, KV head): all G query
// heads of the group, all positions, K/V read exactly once; the dot products q.K^T and p.V run as
// mma.sync.m16n8k16 (the G <= 8 heads are rows 0..G-1 of the 16-row A operand; the tensor pipe is far from a limit at
// this size, what counts is that one instruction replaces ~50).
//
// Operand layouts without any shuffle or shared-memory staging of K/V -- the contraction index of a dot product may be
// permuted freely as long as both operands use the same permutation, and so may the labels of the output columns:
//   * scores:  S[16 x 8 positions] += Qa[16 x 16] . Kb[16 x 8].  Lane (g = lane / 4, t = lane % 4) supplies K row
//     p0 + g, and for the kk-th MMA the four elements k = 2t, 2t+1, 2t+8, 2t+9 of the 16-wide slice.  Slice kk, slot
//     s of lane t is mapped to the physical dim DPT*t + 4*kk + s (DPT = HD/4): every lane reads DPT contiguous dims
//     (64 bytes at HD = 128) of its row with 128-bit loads; the q fragments use the same map.
//   * outputs: O[16 x 8 dims] += Pa[16 x 16 positions] . Vb[16 x 8].  Pa is the score fragment of two consecutive
//     position tiles converted to f16 (the usual register reuse); lane (g, t) supplies V rows p0 + {2t, 2t+1, 2t+8,
//     2t+9} and output column n = g of every dim tile j, which is mapped to the physical dim NT*g + j (NT = HD/8): the
//     lane reads NT contiguous dims (32 bytes at HD = 128) of its four rows and pairs them up with byte permutes.
// Eight warps take the 16-position tiles of the sequence round-robin, each with a private online-softmax state;
// their partials meet in shared memory at the end.  16 warps per SM x 8 KB of rows in flight per warp tile keep HBM
// busy without software pipelining.
#include "attn_core.cuh"
#include "attn_params.cuh"

namespace nve {

constexpr int kAmThreads = 256;
constexpr int kAmWarps = kAmThreads / 32;

template <int HD, int G> struct AmShared {
    float q_s[G][HD];
    __align__(16) uint16_t knew_s[HD];
    __align__(16) uint16_t vnew_s[HD];
    float wm[kAmWarps][G], wl[kAmWarps][G];
    float wo[kAmWarps][G][HD];
};

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

template <int HD, int G, bool FUSED>
__global__ void __launch_bounds__(kAmThreads, 2) attn_batch_mma_kernel(const AttnParams pin) {
    constexpr int DC = HD / 8;        // 16-byte chunks per row
    constexpr int DPT = HD / 4;       // dims of a K row per lane
    constexpr int KQ = DPT / 8;       // 128-bit loads per K row and lane
    constexpr int NT = HD / 8;        // output dim tiles = dims of a V row per lane
    constexpr int VQ = NT / 8;        // 128-bit loads per V row and lane
    constexpr int KK = HD / 16;       // MMAs per score tile
    static_assert(VQ >= 1 && KQ >= 1 && G >= 1 && G <= 8, "head_dim 64 or 128, up to 8 query heads per KV head");
    AttnParams p = pin;
    if constexpr (FUSED) {
        const long long b = blockIdx.y;
        p.q += b * (static_cast<long long>(p.num_heads) * HD);
        p.out += b * (static_cast<long long>(p.num_heads) * HD);
        p.k_new += b * (static_cast<long long>(p.num_kv_heads) * HD);
        p.v_new += b * (static_cast<long long>(p.num_kv_heads) * HD);
        p.k_cache += b * p.cache_stride;
        p.v_cache += b * p.cache_stride;
        p.d_pos += b;
        p.d_seq_len += b;
    } else {  // causal block: row blockIdx.y of q attends to seq_len + row positions of the one cache
        p.q += static_cast<long long>(blockIdx.y) * p.row_stride;
        p.out += static_cast<long long>(blockIdx.y) * p.row_stride;
    }
    __shared__ AmShared<HD, G> sh;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int kvh = blockIdx.x;
    const int h0 = kvh * G;
    uint16_t* kh = p.k_cache + static_cast<long long>(kvh) * p.kv_stride * HD;
    uint16_t* vh = p.v_cache + static_cast<long long>(kvh) * p.kv_stride * HD;

    pdl_wait();
    int seq_len;
    if constexpr (FUSED) {
        seq_len = max(0, min(*p.d_seq_len, p.kv_stride));
        const int pos = *p.d_pos;
        const bool pos_ok = pos >= 0 && pos < p.kv_stride;
        attn_stage_q<HD, G, true>(sh, tid, p.q, p.k_new, p.v_new, p.cos_tab, p.sin_tab, h0, kvh, pos, pos_ok);
        __syncthreads();
        pdl_launch_dependents();
        // the new row goes to the cache first and is read back from there like every other row (same CTA: the barrier
        // orders the store before the loads, which are ordinary coherent loads)
        if (pos_ok && tid < 2 * DC) {
            const int which = tid / DC, d = tid % DC;
            uint16_t* dst = (which == 0 ? kh : vh) + static_cast<long long>(pos) * HD;
            reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(which == 0 ? sh.knew_s : sh.vnew_s)[d];
        }
    } else {
        seq_len = max(0, min(p.seq_len + static_cast<int>(blockIdx.y), p.kv_stride));
        attn_stage_q<HD, G, false>(sh, tid, p.q, nullptr, nullptr, nullptr, nullptr, h0, kvh, 0, false);
        pdl_launch_dependents();
    }
    __syncthreads();

    // q fragments (rows g < G are heads, the other rows are zero)
    uint32_t qa[KK][4];
#pragma unroll
    for (int kk = 0; kk < KK; kk++) {
        qa[kk][1] = 0;
        qa[kk][3] = 0;
        if (g < G) {
            const float* qp = &sh.q_s[g][DPT * t + 4 * kk];
            qa[kk][0] = pack_f16x2(qp[0], qp[1]);  // exact: q_s holds f16-rounded values
            qa[kk][2] = pack_f16x2(qp[2], qp[3]);
        } else {
            qa[kk][0] = 0;
            qa[kk][2] = 0;
        }
    }

    float m = -1e30f, l = 0.0f;  // running maximum (equal on the four lanes of a row) and this lane's share of the sum
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    for (int p0 = warp * 16; p0 < seq_len; p0 += kAmWarps * 16) {
        const int last = seq_len - 1;
        // ---- loads of the tile: K rows p0 + g, p0 + 8 + g; V rows p0 + {2t, 2t+1, 2t+8, 2t+9}
        uint4 kr[2][KQ], vr[4][VQ];
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const uint16_t* row = kh + static_cast<long long>(min(p0 + 8 * r + g, last)) * HD + DPT * t;
#pragma unroll
            for (int i = 0; i < KQ; i++) kr[r][i] = *reinterpret_cast<const uint4*>(row + 8 * i);
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int pr = p0 + 2 * t + (r & 1) + 8 * (r >> 1);
            const uint16_t* row = vh + static_cast<long long>(min(pr, last)) * HD + NT * g;
#pragma unroll
            for (int i = 0; i < VQ; i++) vr[r][i] = *reinterpret_cast<const uint4*>(row + 8 * i);
        }
        // ---- scores of the two 8-position halves
        float s0[4] = {0, 0, 0, 0}, s1[4] = {0, 0, 0, 0};
#pragma unroll
        for (int kk = 0; kk < KK; kk++) {
            const uint32_t* k0 = reinterpret_cast<const uint32_t*>(&kr[0][0]);
            const uint32_t* k1 = reinterpret_cast<const uint32_t*>(&kr[1][0]);
            mma_f16_16816(s0, qa[kk], k0[2 * kk], k0[2 * kk + 1]);
            mma_f16_16816(s1, qa[kk], k1[2 * kk], k1[2 * kk + 1]);
        }
        // this lane's four scores of row g: positions p0 + 2t, +1 (s0[0], s0[1]) and p0 + 8 + 2t, +1 (s1[0], s1[1])
        float sc[4];
        sc[0] = p0 + 2 * t < seq_len ? s0[0] * p.scale : -1e30f;
        sc[1] = p0 + 2 * t + 1 < seq_len ? s0[1] * p.scale : -1e30f;
        sc[2] = p0 + 8 + 2 * t < seq_len ? s1[0] * p.scale : -1e30f;
        sc[3] = p0 + 9 + 2 * t < seq_len ? s1[1] * p.scale : -1e30f;
        float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);
        const float corr = __expf(m - m_new);
        float pe[4];
#pragma unroll
        for (int i = 0; i < 4; i++) pe[i] = sc[i] > -1e29f ? __expf(sc[i] - m_new) : 0.0f;
        l = l * corr + ((pe[0] + pe[1]) + (pe[2] + pe[3]));
        m = m_new;
#pragma unroll
        for (int j = 0; j < NT; j++) {
            o[j][0] *= corr;
            o[j][1] *= corr;
        }
        // ---- outputs: p (f16) . V
        uint32_t pa[4];
        pa[0] = pack_f16x2(pe[0], pe[1]);
        pa[1] = 0;
        pa[2] = pack_f16x2(pe[2], pe[3]);
        pa[3] = 0;
        const uint32_t* v0 = reinterpret_cast<const uint32_t*>(&vr[0][0]);  // row p0 + 2t
        const uint32_t* v1 = reinterpret_cast<const uint32_t*>(&vr[1][0]);  // row p0 + 2t + 1
        const uint32_t* v2 = reinterpret_cast<const uint32_t*>(&vr[2][0]);  // row p0 + 8 + 2t
        const uint32_t* v3 = reinterpret_cast<const uint32_t*>(&vr[3][0]);  // row p0 + 9 + 2t
#pragma unroll
        for (int j = 0; j < NT; j++) {
            // dim NT*g + j of the four rows: register j / 2, lower or upper half
            const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
            const uint32_t b0 = __byte_perm(v0[j >> 1], v1[j >> 1], sel);
            const uint32_t b1 = __byte_perm(v2[j >> 1], v3[j >> 1], sel);
            mma_f16_16816(o[j], pa, b0, b1);
        }
    }

    // ---- the warps' partials meet in shared memory: lane (g < G, t) holds head g, dims NT*(2t) + j and NT*(2t+1) + j
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (g < G) {
        if (t == 0) {
            sh.wm[warp][g] = m;
            sh.wl[warp][g] = l;
        }
#pragma unroll
        for (int j = 0; j < NT; j++) {
            sh.wo[warp][g][NT * (2 * t) + j] = o[j][0];
            sh.wo[warp][g][NT * (2 * t + 1) + j] = o[j][1];
        }
    }
    __syncthreads();
    for (int i = tid; i < G * HD; i += kAmThreads) {
        const int h = i / HD, d = i % HD;
        float mm = -1e30f;
#pragma unroll
        for (int w = 0; w < kAmWarps; w++) mm = fmaxf(mm, sh.wm[w][h]);
        float ss = 0.0f, a = 0.0f;
#pragma unroll
        for (int w = 0; w < kAmWarps; w++) {
            const float c = __expf(sh.wm[w][h] - mm);
            ss = fmaf(sh.wl[w][h], c, ss);
            a = fmaf(sh.wo[w][h][d], c, a);
        }
        const float inv = ss > 0.0f ? 1.0f / ss : 0.0f;
        p.out[static_cast<long long>(h0 + h) * HD + d] = Act16<NVE_DT_F16>::from_f32(a * inv);
    }
}

template <int HD, int G> static cudaError_t launch_am(const AttnParams& p, cudaStream_t st, bool fused) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p.num_kv_heads, p.rows);
    cfg.blockDim = dim3(kAmThreads);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return fused ? cudaLaunchKernelEx(&cfg, attn_batch_mma_kernel<HD, G, true>, p)
                 : cudaLaunchKernelEx(&cfg, attn_batch_mma_kernel<HD, G, false>, p);
}

bool attn_batch_mma_try(const AttnParams& p, int head_dim, cudaStream_t st, cudaError_t& err, bool fused) {
    const int groups = p.num_heads / p.num_kv_heads;
    if (head_dim == 128) {
        switch (groups) {
            case 1: err = launch_am<128, 1>(p, st, fused); return true;
            case 2: err = launch_am<128, 2>(p, st, fused); return true;
            case 4: err = launch_am<128, 4>(p, st, fused); return true;
            case 8: err = launch_am<128, 8>(p, st, fused); return true;
            default: return false;
        }
    }
    if (head_dim == 64) {
        switch (groups) {
            case 1: err = launch_am<64, 1>(p, st, fused); return true;
            case 2: err = launch_am<64, 2>(p, st, fused); return true;
            case 4: err = launch_am<64, 4>(p, st, fused); return true;
            case 8: err = launch_am<64, 8>(p, st, fused); return true;
            default: return false;
        }
    }
    return false;
}

}  // namespace nve
