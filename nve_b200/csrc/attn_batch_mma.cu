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
#include "attn_mma.cuh"
#include "attn_params.cuh"

namespace nve {

template <int HD, int G, bool FUSED>
__global__ void __launch_bounds__(kAmThreads, 2) attn_batch_mma_kernel(const AttnParams pin) {
    constexpr int DC = HD / 8;        // 16-byte chunks per row
    constexpr int NT = HD / 8;        // output dim tiles = dims of a V row per lane
    static_assert((HD == 64 || HD == 128) && G >= 1 && G <= 8, "head_dim 64 or 128, up to 8 query heads per KV head");
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

    uint32_t qa[HD / 16][4];
    am_q_fragments<HD, G>(sh, g, t, qa);

    float m = -1e30f, l = 0.0f;  // running maximum (equal on the four lanes of a row) and this lane's share of the sum
    float o[NT][4];
#pragma unroll
    for (int j = 0; j < NT; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;

    for (int p0 = warp * 16; p0 < seq_len; p0 += kAmWarps * 16) {
        uint4 kr[2][HD / 32], vr[4][HD / 64];
        am_load_tile<HD>(kh, vh, p0, seq_len - 1, g, t, kr, vr);
        am_tile<HD>(qa, kr, vr, p0, seq_len, p.scale, t, m, l, o);
    }

    // ---- the warps' partials meet in shared memory
    am_store_warp_partial<HD, G>(sh, warp, g, t, m, l, o);
    __syncthreads();
    for (int i = tid; i < G * HD; i += kAmThreads) {
        const int h = i / HD, d = i % HD;
        float mm, ss, a;
        am_merge_warps<HD, G>(sh, h, d, mm, ss, a);
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
