// Tile arithmetic shared by the tensor-core attention kernels (attn_batch_mma.cu: many sequences, one CTA per
// sequence and KV head; attn_decode_mma.cu: one sequence, a cluster per KV head): one warp, one tile of 16 cached
// positions, all G <= 8 query heads of the KV head as rows of mma.sync.m16n8k16.  The operand layouts are described
// at the top of attn_batch_mma.cu.
#pragma once
#include "attn_core.cuh"

namespace nve {

constexpr int kAmThreads = 256;
constexpr int kAmWarps = kAmThreads / 32;

// The warps' output partials in shared memory: dim d of a head sits at am_wo_index(d) of a row of am_wo_row(HD)
// floats.  Lane (g, t) of a warp stores dims NT*(2t) + j and NT*(2t+1) + j of head g; with one float of skew per
// NT dims and rows of HD + 8 floats the 16 storing lanes hit 16 different banks.
__host__ __device__ constexpr int am_wo_row(int hd) { return hd + 8; }
template <int HD> __device__ __forceinline__ int am_wo_index(int d) { return d + d / (HD / 8); }

template <int HD, int G> struct AmShared {
    float q_s[G][HD];
    __align__(16) uint16_t knew_s[HD];
    __align__(16) uint16_t vnew_s[HD];
    float wm[kAmWarps][G], wl[kAmWarps][G];
    float wo[kAmWarps][G][am_wo_row(HD)];
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

// q fragments of lane (g, t) from the staged (rotated, f16-rounded) q rows: rows g < G are heads, the others zero
template <int HD, int G, class SH> __device__ __forceinline__ void am_q_fragments(const SH& sh, int g, int t, uint32_t (&qa)[HD / 16][4]) {
    constexpr int DPT = HD / 4, KK = HD / 16;
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
}

// Loads of the tile at p0: K rows p0 + g, p0 + 8 + g (dims DPT*t ..), V rows p0 + {2t, 2t+1, 2t+8, 2t+9} (dims
// NT*g ..); rows beyond `last` are clamped to it (their scores are masked by am_tile).
template <int HD> __device__ __forceinline__ void am_load_tile(const uint16_t* kh, const uint16_t* vh, int p0, int last, int g, int t,
                                                             uint4 (&kr)[2][HD / 32], uint4 (&vr)[4][HD / 64]) {
    constexpr int DPT = HD / 4, KQ = DPT / 8, NT = HD / 8, VQ = NT / 8;
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
}

// Rows of the tile that are position `pos` take the new token's k / v (f16, in shared memory) instead of what was
// loaded from the cache.
template <int HD> __device__ __forceinline__ void am_patch_tile(const uint16_t* knew_s, const uint16_t* vnew_s, int p0, int pos, int g, int t,
                                                              uint4 (&kr)[2][HD / 32], uint4 (&vr)[4][HD / 64]) {
    constexpr int DPT = HD / 4, KQ = DPT / 8, NT = HD / 8, VQ = NT / 8;
    if (pos < p0 || pos >= p0 + 16) return;
#pragma unroll
    for (int r = 0; r < 2; r++)
        if (p0 + 8 * r + g == pos) {
#pragma unroll
            for (int i = 0; i < KQ; i++) kr[r][i] = *reinterpret_cast<const uint4*>(knew_s + DPT * t + 8 * i);
        }
#pragma unroll
    for (int r = 0; r < 4; r++)
        if (p0 + 2 * t + (r & 1) + 8 * (r >> 1) == pos) {
#pragma unroll
            for (int i = 0; i < VQ; i++) vr[r][i] = *reinterpret_cast<const uint4*>(vnew_s + NT * g + 8 * i);
        }
}

// One tile into the warp's online-softmax state: m = running maximum of row g (equal on the four lanes of a row),
// l = this lane's share of the sum of exponentials, o[j] = columns of the weighted V sum (o[j][0], o[j][1]: row g).
template <int HD> __device__ __forceinline__ void am_tile(const uint32_t (&qa)[HD / 16][4], const uint4 (&kr)[2][HD / 32],
                                                        const uint4 (&vr)[4][HD / 64], int p0, int seq_len, float scale, int t,
                                                        float& m, float& l, float (&o)[HD / 8][4]) {
    constexpr int NT = HD / 8, KK = HD / 16;
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
    sc[0] = p0 + 2 * t < seq_len ? s0[0] * scale : -1e30f;
    sc[1] = p0 + 2 * t + 1 < seq_len ? s0[1] * scale : -1e30f;
    sc[2] = p0 + 8 + 2 * t < seq_len ? s1[0] * scale : -1e30f;
    sc[3] = p0 + 9 + 2 * t < seq_len ? s1[1] * scale : -1e30f;
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

// The warp's state -> shared memory: lane (g < G, t) holds head g, dims NT*(2t) + j and NT*(2t+1) + j.
template <int HD, int G, class SH> __device__ __forceinline__ void am_store_warp_partial(SH& sh, int warp, int g, int t, float m, float l,
                                                                                       const float (&o)[HD / 8][4]) {
    constexpr int NT = HD / 8;
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (g < G) {
        if (t == 0) {
            sh.wm[warp][g] = m;
            sh.wl[warp][g] = l;
        }
#pragma unroll
        for (int j = 0; j < NT; j++) {
            sh.wo[warp][g][(NT + 1) * (2 * t) + j] = o[j][0];  // = am_wo_index(NT * (2t) + j)
            sh.wo[warp][g][(NT + 1) * (2 * t + 1) + j] = o[j][1];
        }
    }
}
// Element (h, d) of the CTA's partial from the eight warps' (after a CTA barrier), warps in ascending order:
// mm = maximum, ss = sum of exponentials relative to it, a = weighted V sum relative to it.
template <int HD, int G, class SH> __device__ __forceinline__ void am_merge_warps(const SH& sh, int h, int d, float& mm, float& ss, float& a) {
    mm = -1e30f;
#pragma unroll
    for (int w = 0; w < kAmWarps; w++) mm = fmaxf(mm, sh.wm[w][h]);
    ss = 0.0f;
    a = 0.0f;
#pragma unroll
    for (int w = 0; w < kAmWarps; w++) {
        const float c = __expf(sh.wm[w][h] - mm);
        ss = fmaf(sh.wl[w][h], c, ss);
        a = fmaf(sh.wo[w][h][am_wo_index<HD>(d)], c, a);
    }
}

}  // namespace nve
