// Single-query GQA attention core shared by the clustered stand-alone kernel (attn_decode.cu) and the persistent
// decode-step kernel (decode_step.cu).  Both run exactly these device functions on the same decomposition, so
// their results are bit-identical:
//
//   * a "virtual CTA" is 256 threads = PL position lanes x DC dim chunks (DC = head_dim/8 lanes hold one 16-byte
//     slice of a row); it serves QH query heads that share one KV head and owns the positions
//     [rank*chunk, (rank+1)*chunk), chunk = ceil(seq_len / kAdRanks) (the stand-alone kernel's cluster of
//     kAdCluster CTAs runs kAdRanks / kAdCluster of them per CTA, the persistent kernel one per half CTA);
//   * every thread keeps a private online-softmax state over the positions t_begin + it*PL*4 + u*PL + pl;
//   * level 1: the PL lane states of a virtual CTA are merged in ascending lane order (attn_merge_lanes);
//   * level 2: the kAdRanks partials of a head are merged in ascending rank order (attn_merge_ranks).
//
// Every floating-point operation that feeds a result is an explicitly rounded intrinsic (no contraction), so the
// two callers cannot diverge through different instruction selection.
#pragma once
#include "common.cuh"

namespace nve {

constexpr int kAdRanks = 8;      // position slices per head
constexpr int kAdCluster = 8;    // CTAs per cluster of the stand-alone kernel (portable cluster size)
constexpr int kAdThreads = 256;  // threads of a virtual CTA
constexpr int kAdUnroll = 4;

__device__ __forceinline__ void unpack8_f32(const uint4& raw, float (&o)[8]) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
        o[2 * j] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(w[j] & 0xFFFFu));
        o[2 * j + 1] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(w[j] >> 16));
    }
}

// Partial result of one virtual CTA: per head the running maximum, the sum of exponentials and the weighted V sum.
template <int HD, int QH> struct AdCtaPartial {
    float m[QH];
    float s[QH];
    float acc[QH][HD];
};

// Shared memory of one virtual CTA.
template <int HD, int QH> struct AdShared {
    static constexpr int PL = kAdThreads / (HD / 8);
    float q_s[QH][HD];
    __align__(16) uint16_t knew_s[HD];
    __align__(16) uint16_t vnew_s[HD];
    float pm[PL][QH], ps[PL][QH];
    float pc[PL][QH];  // exp(pm - max over lanes): computed once per (lane, head) for the level-1 merge
    float pacc[PL][QH][HD];
};

// Stage q (rotated at `pos` in the fused form) and the rotated new k row / new v row of the KV head.
// tid in [0, 256).  The caller synchronises the virtual CTA afterwards.  L2ONLY: q / k_new / v_new were written by
// other CTAs of the same (persistent) kernel and are read past L1.
template <bool L2ONLY> __device__ __forceinline__ uint16_t attn_ld16(const uint16_t* p) {
    if constexpr (L2ONLY) return __ldcg(p);
    else return *p;
}
template <int HD, int QH, bool FUSED, bool L2ONLY = false, class SH = AdShared<HD, QH>>
__device__ __forceinline__ void attn_stage_q(SH& sh, int tid, const uint16_t* q, const uint16_t* k_new,
                                             const uint16_t* v_new, const uint16_t* cos_tab, const uint16_t* sin_tab,
                                             int h0, int kvh, int pos, bool pos_ok) {
    constexpr int HALF = HD / 2;
    if constexpr (FUSED) {
        const uint16_t* cr = cos_tab + static_cast<long long>(pos_ok ? pos : 0) * HALF;
        const uint16_t* sr = sin_tab + static_cast<long long>(pos_ok ? pos : 0) * HALF;
        for (int i = tid; i < QH * HALF; i += kAdThreads) {
            const int h = i / HALF, e = i % HALF;
            const uint16_t* qp = q + static_cast<long long>(h0 + h) * HD;
            const float c = Act16<NVE_DT_F16>::to_f32(cr[e]), s = Act16<NVE_DT_F16>::to_f32(sr[e]);
            const float x0 = Act16<NVE_DT_F16>::to_f32(attn_ld16<L2ONLY>(qp + e));
            const float x1 = Act16<NVE_DT_F16>::to_f32(attn_ld16<L2ONLY>(qp + e + HALF));
            const uint16_t r0 = Act16<NVE_DT_F16>::from_f32(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
            const uint16_t r1 = Act16<NVE_DT_F16>::from_f32(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
            sh.q_s[h][e] = Act16<NVE_DT_F16>::to_f32(r0);
            sh.q_s[h][e + HALF] = Act16<NVE_DT_F16>::to_f32(r1);
        }
        for (int e = tid; e < HALF; e += kAdThreads) {
            const uint16_t* kp = k_new + static_cast<long long>(kvh) * HD;
            const float c = Act16<NVE_DT_F16>::to_f32(cr[e]), s = Act16<NVE_DT_F16>::to_f32(sr[e]);
            const float x0 = Act16<NVE_DT_F16>::to_f32(attn_ld16<L2ONLY>(kp + e));
            const float x1 = Act16<NVE_DT_F16>::to_f32(attn_ld16<L2ONLY>(kp + e + HALF));
            sh.knew_s[e] = Act16<NVE_DT_F16>::from_f32(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
            sh.knew_s[e + HALF] = Act16<NVE_DT_F16>::from_f32(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
        }
        for (int e = tid; e < HD; e += kAdThreads) sh.vnew_s[e] = attn_ld16<L2ONLY>(v_new + static_cast<long long>(kvh) * HD + e);
    } else {
        for (int i = tid; i < QH * HD; i += kAdThreads)
            sh.q_s[i / HD][i % HD] = Act16<NVE_DT_F16>::to_f32(attn_ld16<L2ONLY>(q + static_cast<long long>(h0) * HD + i));
    }
}

// Rows fetched ahead of the dependency wait by the stand-alone kernel (two batches).
constexpr int kAdPre = 2;
struct AdPrefetch {
    uint4 k[kAdPre][kAdUnroll];
    uint4 v[kAdPre][kAdUnroll];
};

// The per-thread pass over the positions [t_begin, t_end) of this virtual CTA, then the level-1 merge of its PL
// lanes.  The merged partial of element i = tid, tid + 256, ... (< QH*HD) is handed to `sink(h, d, mm, ss, a)`.
// `sync()` synchronises the threads of the virtual CTA (all of them call this function together).
// kh / vh: cache rows of this KV head.  With FUSED the row at `pos` is taken from shared memory (the new token);
// `pre` holds rows loaded before the wait when `pre_ok` (same addresses as this pass would use).
template <int HD, int QH, bool FUSED, bool PRE, class Sync, class Sink>
__device__ __forceinline__ void attn_partial(AdShared<HD, QH>& sh, int tid, const uint16_t* kh, const uint16_t* vh,
                                             int t_begin, int t_end, int pos, float scale, bool pre_ok,
                                             const AdPrefetch* pre, Sync sync, Sink sink) {
    constexpr int DC = HD / 8;
    constexpr int PL = kAdThreads / DC;
    const int dc = tid % DC, pl = tid / DC;

    float qr[QH][8];
#pragma unroll
    for (int h = 0; h < QH; h++)
#pragma unroll
        for (int i = 0; i < 8; i++) qr[h][i] = sh.q_s[h][dc * 8 + i];

    float m[QH], s[QH], acc[QH][8];
#pragma unroll
    for (int h = 0; h < QH; h++) {
        m[h] = -1e30f;
        s[h] = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) acc[h][i] = 0.0f;
    }

    const int span = PL * kAdUnroll;
    const int iters = (max(0, t_end - t_begin) + span - 1) / span;  // uniform over the virtual CTA
    auto load = [&](int it, bool use_pre, int pre_idx, uint4 (&kraw)[kAdUnroll], uint4 (&vraw)[kAdUnroll]) {
#pragma unroll
        for (int u = 0; u < kAdUnroll; u++) {
            const int t = t_begin + it * span + u * PL + pl;
            const int tc = t < t_end ? t : t_begin;
            if (FUSED && tc == pos) {
                kraw[u] = reinterpret_cast<const uint4*>(sh.knew_s)[dc];
                vraw[u] = reinterpret_cast<const uint4*>(sh.vnew_s)[dc];
            } else if (PRE && use_pre) {
                kraw[u] = pre->k[pre_idx][u];
                vraw[u] = pre->v[pre_idx][u];
            } else {
                kraw[u] = ld_stream_u4(kh + static_cast<long long>(tc) * HD + dc * 8);
                vraw[u] = ld_stream_u4(vh + static_cast<long long>(tc) * HD + dc * 8);
            }
        }
    };
    auto reduce = [&](int it, const uint4 (&kraw)[kAdUnroll], const uint4 (&vraw)[kAdUnroll]) {
        bool valid[kAdUnroll];
#pragma unroll
        for (int u = 0; u < kAdUnroll; u++) valid[u] = t_begin + it * span + u * PL + pl < t_end;
        float sc[kAdUnroll][QH];
#pragma unroll
        for (int u = 0; u < kAdUnroll; u++) {
            float kf[8];
            unpack8_f32(kraw[u], kf);
#pragma unroll
            for (int h = 0; h < QH; h++) {
                float d = 0.0f;
#pragma unroll
                for (int i = 0; i < 8; i++) d = __fmaf_rn(qr[h][i], kf[i], d);
#pragma unroll
                for (int msk = DC / 2; msk > 0; msk >>= 1) d = __fadd_rn(d, __shfl_xor_sync(0xffffffffu, d, msk));
                sc[u][h] = valid[u] ? __fmul_rn(d, scale) : -1e30f;
            }
        }
#pragma unroll
        for (int h = 0; h < QH; h++) {
            float new_m = m[h];
#pragma unroll
            for (int u = 0; u < kAdUnroll; u++) new_m = fmaxf(new_m, sc[u][h]);
            const float corr = expf(__fsub_rn(m[h], new_m));
            float pe[kAdUnroll];
            float psum = 0.0f;
#pragma unroll
            for (int u = 0; u < kAdUnroll; u++) {
                pe[u] = valid[u] ? expf(__fsub_rn(sc[u][h], new_m)) : 0.0f;
                psum = __fadd_rn(psum, pe[u]);
            }
            s[h] = __fmaf_rn(s[h], corr, psum);
            m[h] = new_m;
#pragma unroll
            for (int i = 0; i < 8; i++) acc[h][i] = __fmul_rn(acc[h][i], corr);
#pragma unroll
            for (int u = 0; u < kAdUnroll; u++) {
                float vf[8];
                unpack8_f32(vraw[u], vf);
#pragma unroll
                for (int i = 0; i < 8; i++) acc[h][i] = __fmaf_rn(pe[u], vf[i], acc[h][i]);
            }
        }
    };

    {
        static_assert(kAdPre == 2, "the first two batches are peeled so that prefetched rows stay in registers");
        auto batch = [&](int it, bool use_pre, int pre_idx) {
            uint4 kraw[kAdUnroll], vraw[kAdUnroll];
            load(it, use_pre, pre_idx, kraw, vraw);
            reduce(it, kraw, vraw);
        };
        if (iters > 0) batch(0, pre_ok, 0);
        if (iters > 1) batch(1, pre_ok, 1);
        for (int it = kAdPre; it < iters; it++) batch(it, false, 0);
    }

    // ---- level 1: merge the position lanes of this virtual CTA in ascending lane order
#pragma unroll
    for (int h = 0; h < QH; h++) {
        if (dc == 0) { sh.pm[pl][h] = m[h]; sh.ps[pl][h] = s[h]; }
#pragma unroll
        for (int i = 0; i < 8; i++) sh.pacc[pl][h][dc * 8 + i] = acc[h][i];
    }
    sync();
    // the rescaling factor of a lane state is the same for all 8*DC elements of its head: one thread computes it
    if (tid < PL * QH) {
        const int l = tid / QH, h = tid % QH;
        float mm = -1e30f;
        for (int k = 0; k < PL; k++) mm = fmaxf(mm, sh.pm[k][h]);
        sh.pc[l][h] = expf(__fsub_rn(sh.pm[l][h], mm));
    }
    sync();
    for (int i = tid; i < QH * HD; i += kAdThreads) {
        const int h = i / HD, d = i % HD;
        float mm = -1e30f;
        for (int l = 0; l < PL; l++) mm = fmaxf(mm, sh.pm[l][h]);
        float ss = 0.0f, a = 0.0f;
        for (int l = 0; l < PL; l++) {
            const float c = sh.pc[l][h];
            ss = __fmaf_rn(sh.ps[l][h], c, ss);
            a = __fmaf_rn(sh.pacc[l][h][d], c, a);
        }
        sink(h, d, mm, ss, a);
    }
}

// Level 2 for element (h, d): merge the kAdRanks partials in ascending rank order and normalise; returns the
// 16-bit rounded output.  `parts` points at kAdRanks consecutive partials of the virtual cluster.
template <bool L2ONLY> __device__ __forceinline__ float attn_ldf(const float* p) {
    if constexpr (L2ONLY) return __ldcg(p);
    else return *p;
}
template <int HD, int QH, bool L2ONLY = false>
__device__ __forceinline__ uint16_t attn_merge_ranks(const AdCtaPartial<HD, QH>* parts, int h, int d) {
    float pm[kAdRanks], ps[kAdRanks], pa[kAdRanks];
#pragma unroll
    for (int r = 0; r < kAdRanks; r++) {  // all loads in flight together
        pm[r] = attn_ldf<L2ONLY>(&parts[r].m[h]);
        ps[r] = attn_ldf<L2ONLY>(&parts[r].s[h]);
        pa[r] = attn_ldf<L2ONLY>(&parts[r].acc[h][d]);
    }
    float mm = -1e30f;
#pragma unroll
    for (int r = 0; r < kAdRanks; r++) mm = fmaxf(mm, pm[r]);
    float ss = 0.0f, a = 0.0f;
#pragma unroll
    for (int r = 0; r < kAdRanks; r++) {
        const float c = expf(__fsub_rn(pm[r], mm));
        ss = __fmaf_rn(ps[r], c, ss);
        a = __fmaf_rn(pa[r], c, a);
    }
    const float inv = ss > 0.0f ? __fdiv_rn(1.0f, ss) : 0.0f;
    return Act16<NVE_DT_F16>::from_f32(__fmul_rn(a, inv));
}

// int8 code of one attention output element; the 32 lanes of the calling warp hold one 32-wide group.
// Returns the code; `scale` receives the group's scale (same arithmetic as the stand-alone quantiser).
__device__ __forceinline__ int attn_quantize_lane(uint16_t o16, float& scale) {
    const float v = Act16<NVE_DT_F16>::to_f32(o16);
    const float amax = warp_max(fabsf(v));
    scale = amax > 0.0f ? __fdiv_rn(amax, 127.0f) : 1.0f;
    int qv = __float2int_rn(__fmul_rn(v, __fdiv_rn(1.0f, scale)));
    return max(-127, min(127, qv));
}

}  // namespace nve
