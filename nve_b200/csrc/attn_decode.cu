// Single-query GQA attention for decode, optionally fused with RoPE, the KV-cache write and the int8
// quantisation of its output.
//
// Replaces cuda/nve_kernels.cu:462-591 / :1075-1197 (flash decode) of the reference project and, in the
// fused form, also :1006-1065 (RoPE at a device position), :909-946 (KV scatter) and the activation
// quantiser call that precedes o_proj on the W4A8 route (src/gpu_layer.rs:697-741 in one launch).
//
// Design (head_dim 64 or 128; other sizes use the generic kernel in attn_glue.cu):
//   * A thread-block cluster of 8 CTAs serves QH query heads that share one KV head; CTA `rank` owns the
//     positions [rank*chunk, (rank+1)*chunk).  K and V rows are read once per cluster with 128-bit loads.
//   * 256 threads = PL position lanes x DC dim chunks (DC = head_dim/8 lanes hold one 16-byte slice of a
//     row).  Each thread loads K and V of 4 positions per iteration (8 loads in flight), reduces the QH dot
//     products over its DC lanes with xor shuffles and keeps a private online-softmax state.
//   * The 256 thread states are merged through shared memory; every CTA then pushes its partial into rank 0's
//     shared memory (distributed shared memory stores), arrives on the cluster barrier and leaves; rank 0 waits
//     and merges locally -- no global scratch, no second launch, no remote read round trip.
//   * Fused form: q and the new k are rotated in-kernel (same IEEE operations and 16-bit rounding as the
//     stand-alone RoPE kernel); the CTA that owns position `pos` takes the fresh k/v from shared memory
//     instead of the cache, and one CTA per KV head writes them to the cache.
#include <cooperative_groups.h>

#include <atomic>

#include "attn_core.cuh"
#include "attn_params.cuh"

namespace cg = cooperative_groups;

namespace nve {


// BATCH (fused form only): blockIdx.y selects one of several independent sequences -- row b of q / k_new / v_new / out,
// the b-th K/V cache and the b-th position and length words.
template <int HD, int QH, bool FUSED, bool BATCH = false>
__global__ void __launch_bounds__(kAdThreads) attn_decode_kernel(const AttnParams pin) {
    AttnParams p = pin;
    if constexpr (BATCH) {
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
    constexpr int DC = HD / 8;            // lanes per row
    constexpr int PL = kAdThreads / DC;   // position lanes
    cg::cluster_group cluster = cg::this_cluster();
    // Phase 1 of the cluster barrier: every CTA announces that it runs, so that the pushes into rank 0's shared
    // memory below never touch a CTA that has not started (matched by the wait in front of the push).
    cluster.barrier_arrive();

    __shared__ AdShared<HD, QH> sh;
    __shared__ AdCtaPartial<HD, QH> parts[kAdRanks];  // only rank 0's copy is used: every CTA pushes its partials there

    const int tid = threadIdx.x;
    const int dc = tid % DC, pl = tid / DC;
    const int rank = static_cast<int>(cluster.block_rank());
    const int cluster_id = blockIdx.x / kAdCluster;
    const int groups = p.num_heads / p.num_kv_heads;
    const int clusters_per_kv = groups / QH;
    const int kvh = cluster_id / clusters_per_kv;
    const int h0 = kvh * groups + (cluster_id % clusters_per_kv) * QH;  // first query head of this cluster

    const uint16_t* kh = p.k_cache + static_cast<long long>(kvh) * p.kv_stride * HD;
    const uint16_t* vh = p.v_cache + static_cast<long long>(kvh) * p.kv_stride * HD;
    const uint16_t* q_row = p.q;
    uint16_t* out_row = p.out;
    int seq_len_row = p.seq_len;
    if constexpr (!FUSED && !BATCH) {
        const int row = blockIdx.y;
        q_row += static_cast<long long>(row) * p.row_stride;
        out_row += static_cast<long long>(row) * p.row_stride;
        seq_len_row += row;
    }

    // Fused form: the cache rows of earlier positions were written by earlier steps, so the first batches of K/V
    // loads can be in flight while the kernel still waits for its predecessor (which produces q and the new k/v,
    // not the cache).  The scalars read here are only a guess used for addressing: they are read again after the
    // wait and the prefetched rows are dropped if anything differs.
    int pre_seq = -1, pre_pos = -2;
    AdPrefetch pre;
    if constexpr (FUSED) {
        pre_seq = max(0, min(*p.d_seq_len, p.kv_stride));
        pre_pos = *p.d_pos;
        const int pchunk = (pre_seq + kAdRanks - 1) / kAdRanks;
        const int pb = rank * pchunk, pe = min(pre_seq, pb + pchunk);
        const int safe = pb < p.kv_stride ? pb : 0;
#pragma unroll
        for (int b = 0; b < kAdPre; b++) {
#pragma unroll
            for (int u = 0; u < kAdUnroll; u++) {
                const int t = pb + b * (PL * kAdUnroll) + u * PL + pl;
                const int tc = t < pe ? t : safe;
                pre.k[b][u] = ld_stream_u4(kh + static_cast<long long>(tc) * HD + dc * 8);
                pre.v[b][u] = ld_stream_u4(vh + static_cast<long long>(tc) * HD + dc * 8);
            }
        }
    }
    pdl_wait();

    // The position scalars are read again now that the producer has finished; q / k / v / the RoPE row are staged
    // with the position read before the wait at the same time (one memory round trip instead of two) and staged again
    // in the rare case that the scalars changed in between.
    int seq_len = p.d_seq_len != nullptr ? *reinterpret_cast<const volatile int*>(p.d_seq_len) : seq_len_row;
    int pos = -1;
    if constexpr (FUSED) pos = *reinterpret_cast<const volatile int*>(p.d_pos);
    if constexpr (FUSED) {
        const bool spec_ok = pre_pos >= 0 && pre_pos < p.kv_stride;
        attn_stage_q<HD, QH, FUSED>(sh, tid, p.q, p.k_new, p.v_new, p.cos_tab, p.sin_tab, h0, kvh, pre_pos, spec_ok);
    }
    seq_len = max(0, min(seq_len, p.kv_stride));
    const bool pos_ok = FUSED && pos >= 0 && pos < p.kv_stride;
    const bool pre_ok = FUSED && pre_seq == seq_len && pre_pos == pos;
    if (!FUSED || pos != pre_pos) {  // uniform over the grid
        if constexpr (FUSED) __syncthreads();
        attn_stage_q<HD, QH, FUSED>(sh, tid, q_row, p.k_new, p.v_new, p.cos_tab, p.sin_tab, h0, kvh, pos, pos_ok);
    }
    __syncthreads();
    pdl_launch_dependents();

    const int chunk = (seq_len + kAdRanks - 1) / kAdRanks;
    // one CTA per KV head stores the new row; every CTA that covers `pos` reads it from shared memory
    if constexpr (FUSED) {
        if (pos_ok && rank == 0 && (cluster_id % clusters_per_kv) == 0 && tid < 2 * DC) {
            const int which = tid / DC, d = tid % DC;
            uint16_t* dst = (which == 0 ? p.k_cache : p.v_cache) + (static_cast<long long>(kvh) * p.kv_stride + pos) * HD;
            reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(which == 0 ? sh.knew_s : sh.vnew_s)[d];
        }
    }

    // push this CTA's partial into rank 0's shared memory (posted remote stores, no round trip); the level-1 merge
    // starts with a CTA barrier and the matching cluster wait rides on it (all CTAs of the cluster run by then)
    static_assert(kAdRanks == kAdCluster, "one position slice per CTA of the cluster");
    const int t_begin = rank * chunk;
    const int t_end = min(seq_len, t_begin + chunk);
    AdCtaPartial<HD, QH>* dst = cluster.map_shared_rank(&parts[rank], 0);
    bool first = true;
    attn_partial<HD, QH, FUSED, FUSED>(
        sh, tid, kh, vh, t_begin, t_end, pos, p.scale, pre_ok, &pre,
        [&] {
            __syncthreads();
            if (first) {
                cluster.barrier_wait();
                first = false;
            }
        },
        [&](int h, int d, float mm, float ss, float a) {
            dst->acc[h][d] = a;
            if (d == 0) { dst->m[h] = mm; dst->s[h] = ss; }
        });
    // phase 2: release the stores / acquire everybody's; only rank 0 has anything left to do
    cluster.barrier_arrive();
    if (rank != 0) return;
    cluster.barrier_wait();

    // ---- rank 0 merges the CTA partials from its own shared memory, normalises and stores
    for (int i = tid; i < QH * HD; i += kAdThreads) {
        const int h = i / HD, d = i % HD;
        const uint16_t o16 = attn_merge_ranks<HD, QH>(parts, h, d);
        const long long oi = static_cast<long long>(h0 + h) * HD + d;
        out_row[oi] = o16;
        if (p.out_q != nullptr) {
            // i advances by whole warps and HD is a multiple of 32: the 32 lanes of a warp hold one group
            float scale;
            const int qv = attn_quantize_lane(o16, scale);
            p.out_q[oi] = static_cast<int8_t>(qv);
            if ((tid & 31) == 0) p.out_scales[oi >> 5] = scale;
        }
    }
}

template <int HD, int QH, bool FUSED, bool BATCH = false> static cudaError_t launch_ad(const AttnParams& p, cudaStream_t st) {
    const int clusters = p.num_heads / QH;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(clusters * kAdCluster, (FUSED && !BATCH) ? 1 : max(1, p.rows));
    cfg.blockDim = dim3(kAdThreads);
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
    return cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, QH, FUSED, BATCH>, p);
}

// Returns false when the shape is not covered (the caller then uses the generic kernel).
template <bool FUSED, bool BATCH = false>
static bool attn_decode_dispatch(const AttnParams& p, int hd, cudaStream_t st, cudaError_t& err) {
    const int groups = p.num_heads / p.num_kv_heads;
    if (!aligned(p.k_cache, 16) || !aligned(p.v_cache, 16)) return false;
    const int qh = (groups % 2 == 0) ? 2 : 1;
    if (hd == 128) {
        err = qh == 2 ? launch_ad<128, 2, FUSED, BATCH>(p, st) : launch_ad<128, 1, FUSED, BATCH>(p, st);
        return true;
    }
    if (hd == 64) {
        err = qh == 2 ? launch_ad<64, 2, FUSED, BATCH>(p, st) : launch_ad<64, 1, FUSED, BATCH>(p, st);
        return true;
    }
    return false;
}

// 0: tensor-core kernels where they cover the shape (default); 1: always the CUDA-core kernel (nve_b200_set_attn_decode_kernel)
static std::atomic<int> g_attn_decode_kernel{0};

// Used by the reference-signature flash-decode entry points (attn_glue.cu).
bool attn_decode_try(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, uint16_t* out, int nh, int nkv, int seq_len,
                     const int* d_seq_len, int kv_stride, int hd, float scale, cudaStream_t st) {
    AttnParams p = {};
    p.q = q;
    p.k_cache = const_cast<uint16_t*>(kc);
    p.v_cache = const_cast<uint16_t*>(vc);
    p.d_seq_len = d_seq_len;
    p.seq_len = seq_len;
    p.out = out;
    p.num_heads = nh;
    p.num_kv_heads = nkv;
    p.kv_stride = kv_stride;
    p.scale = scale;
    cudaError_t e = cudaSuccess;
    const bool mma = g_attn_decode_kernel.load(std::memory_order_relaxed) == 0 && aligned(q, 16) && aligned(kc, 16) && aligned(vc, 16) &&
                     attn_decode_mma_try(p, hd, st, e, false);
    if (!mma && !attn_decode_dispatch<false>(p, hd, st, e)) return false;
    count_launch();
    set_cuda_status(e);
    return true;
}

}  // namespace nve

using namespace nve;

extern "C" int nve_b200_attn_decode_fused(const uint16_t* q, const uint16_t* k_new, const uint16_t* v_new, uint16_t* k_cache,
                                          uint16_t* v_cache, const uint16_t* cos_tab, const uint16_t* sin_tab,
                                          const int* d_pos, const int* d_seq_len, uint16_t* out, int8_t* out_q,
                                          float* out_scales, int num_heads, int num_kv_heads, int head_dim,
                                          int max_seq_len, float scale, nve_stream_t stream) {
    if (!q || !k_new || !v_new || !k_cache || !v_cache || !cos_tab || !sin_tab || !d_pos || !d_seq_len || !out)
        return set_status(NVE_ERR_BAD_POINTER);
    if ((out_q == nullptr) != (out_scales == nullptr)) return set_status(NVE_ERR_BAD_POINTER);
    if (num_heads <= 0 || num_kv_heads <= 0 || (num_heads % num_kv_heads) != 0 || max_seq_len <= 0)
        return set_status(NVE_ERR_BAD_SHAPE);
    if (head_dim != 64 && head_dim != 128) return set_status(NVE_ERR_BAD_SHAPE);
    if (!aligned(k_cache, 16) || !aligned(v_cache, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    AttnParams p = {};
    p.q = q; p.k_new = k_new; p.v_new = v_new; p.k_cache = k_cache; p.v_cache = v_cache;
    p.cos_tab = cos_tab; p.sin_tab = sin_tab; p.d_pos = d_pos; p.d_seq_len = d_seq_len; p.seq_len = 0;
    p.out = out; p.out_q = out_q; p.out_scales = out_scales;
    p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.kv_stride = max_seq_len; p.scale = scale;
    cudaError_t e = cudaSuccess;
    if (g_attn_decode_kernel.load(std::memory_order_relaxed) == 0 && aligned(q, 16) && aligned(k_new, 16) && aligned(v_new, 16) &&
        attn_decode_mma_try(p, head_dim, static_cast<cudaStream_t>(stream), e)) {
        count_launch();
        return set_cuda_status(e);
    }
    if (!attn_decode_dispatch<true>(p, head_dim, static_cast<cudaStream_t>(stream), e)) return set_status(NVE_ERR_BAD_SHAPE);
    count_launch();
    return set_cuda_status(e);
}

/* Which kernel nve_b200_attn_decode_fused launches: 0 (default) = the tensor-core kernel where it covers the shape
 * (head_dim 64 / 128, 1, 2, 4 or 8 query heads per KV head), 1 = always the CUDA-core kernel, whose output equals the
 * un-fused sequence RoPE -> K/V write -> nve_flash_decode_f16 bit for bit.  Process-wide; a captured graph keeps the
 * kernel it was recorded with.  Returns the previous setting. */
extern "C" int nve_b200_set_attn_decode_kernel(int mode) {
    return g_attn_decode_kernel.exchange(mode == 1 ? 1 : 0, std::memory_order_relaxed);
}

/* Causal attention of a block of S new positions against the cache (which already holds them): row r of q
 * [S, num_heads * head_dim] attends to positions [0, start_pos + r]; out has q's layout.  One launch.  Small blocks
 * (fewer than 64 (row, KV head) pairs) run the decode kernel with the row as second grid dimension, so every row
 * equals a nve_flash_decode_f16 call of that length bit for bit; larger ones run the tensor-core kernel of
 * attn_batch_mma.cu (one CTA per row and KV head, scores and outputs on mma.sync), equal to it within rounding. */
extern "C" int nve_b200_attn_prefill_causal(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out,
                                            int rows, int start_pos, int num_heads, int num_kv_heads, int head_dim,
                                            int max_seq_len, float scale, nve_stream_t stream) {
    if (!q || !k_cache || !v_cache || !out) return set_status(NVE_ERR_BAD_POINTER);
    if (rows <= 0 || rows > 65535 || start_pos < 0 || num_heads <= 0 || num_kv_heads <= 0 || (num_heads % num_kv_heads) != 0 ||
        max_seq_len <= 0 || start_pos + rows > max_seq_len)
        return set_status(NVE_ERR_BAD_SHAPE);
    if (head_dim != 64 && head_dim != 128) return set_status(NVE_ERR_BAD_SHAPE);
    if (!aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(q, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    AttnParams p = {};
    p.q = q;
    p.k_cache = const_cast<uint16_t*>(k_cache);
    p.v_cache = const_cast<uint16_t*>(v_cache);
    p.seq_len = start_pos + 1;
    p.out = out;
    p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.kv_stride = max_seq_len; p.scale = scale;
    p.rows = rows;
    p.row_stride = num_heads * head_dim;
    cudaError_t e = cudaSuccess;
    if (static_cast<long long>(rows) * num_kv_heads >= 64 && attn_batch_mma_try(p, head_dim, static_cast<cudaStream_t>(stream), e, false)) {
        count_launch();
        return set_cuda_status(e);
    }
    if (g_attn_decode_kernel.load(std::memory_order_relaxed) == 0 && attn_decode_mma_try(p, head_dim, static_cast<cudaStream_t>(stream), e, false)) {
        count_launch();
        return set_cuda_status(e);
    }
    if (!attn_decode_dispatch<false>(p, head_dim, static_cast<cudaStream_t>(stream), e)) return set_status(NVE_ERR_BAD_SHAPE);
    count_launch();
    return set_cuda_status(e);
}

/* nve_b200_attn_decode_fused for `batch` independent sequences in one launch: row b of q [batch, nh*hd] and of
 * k_new / v_new [batch, nkv*hd] belongs to sequence b, whose caches are k_cache / v_cache + b * nkv * max_seq_len * hd,
 * whose position is d_pos[b] and whose valid length is d_seq_len[b].  Small batches run the clustered kernel that
 * nve_b200_attn_decode_fused would run (row b bit-identical to a single-sequence call under the same
 * nve_b200_set_attn_decode_kernel setting), large ones the streaming tensor-core kernel of attn_batch_mma.cu. */
extern "C" int nve_b200_attn_decode_fused_batch(const uint16_t* q, const uint16_t* k_new, const uint16_t* v_new,
                                                uint16_t* k_cache, uint16_t* v_cache, const uint16_t* cos_tab,
                                                const uint16_t* sin_tab, const int* d_pos, const int* d_seq_len, uint16_t* out,
                                                int batch, int num_heads, int num_kv_heads, int head_dim, int max_seq_len,
                                                float scale, nve_stream_t stream) {
    if (!q || !k_new || !v_new || !k_cache || !v_cache || !cos_tab || !sin_tab || !d_pos || !d_seq_len || !out)
        return set_status(NVE_ERR_BAD_POINTER);
    if (batch <= 0 || batch > 65535 || num_heads <= 0 || num_kv_heads <= 0 || (num_heads % num_kv_heads) != 0 || max_seq_len <= 0)
        return set_status(NVE_ERR_BAD_SHAPE);
    if (head_dim != 64 && head_dim != 128) return set_status(NVE_ERR_BAD_SHAPE);
    if (!aligned(k_cache, 16) || !aligned(v_cache, 16) || !aligned(q, 16) || !aligned(k_new, 16) || !aligned(v_new, 16))
        return set_status(NVE_ERR_BAD_ALIGNMENT);
    AttnParams p = {};
    p.q = q; p.k_new = k_new; p.v_new = v_new; p.k_cache = k_cache; p.v_cache = v_cache;
    p.cos_tab = cos_tab; p.sin_tab = sin_tab; p.d_pos = d_pos; p.d_seq_len = d_seq_len; p.seq_len = 0;
    p.out = out;
    p.num_heads = num_heads; p.num_kv_heads = num_kv_heads; p.kv_stride = max_seq_len; p.scale = scale;
    p.rows = batch;
    p.cache_stride = static_cast<long long>(num_kv_heads) * max_seq_len * head_dim;
    cudaError_t e = cudaSuccess;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    // enough (sequence, head pair) units to fill every SM twice: one CTA per unit over all positions, streaming;
    // otherwise the clustered kernel, which splits a sequence's positions over eight CTAs
    // one CTA per (sequence, KV head) on the tensor cores (attn_batch_mma.cu) from 64 such units on: measured at 8
    // KV heads and context 1024, 8 sequences take 21 us there against 23 us on the clustered tensor-core kernel (29 us
    // on the CUDA-core one), 16 sequences 22 against 41, 64 sequences 63 against 188; below that the clustered
    // kernels, which split a sequence's positions over eight CTAs, are faster (2 sequences 8.7 us, 4 sequences 13.4 us)
    if (static_cast<long long>(batch) * num_kv_heads >= 64 && attn_batch_mma_try(p, head_dim, cs, e)) {
        count_launch();
        return set_cuda_status(e);
    }
    if (g_attn_decode_kernel.load(std::memory_order_relaxed) == 0 && attn_decode_mma_try(p, head_dim, cs, e)) {
        count_launch();
        return set_cuda_status(e);
    }
    if (!attn_decode_dispatch<true, true>(p, head_dim, cs, e)) return set_status(NVE_ERR_BAD_SHAPE);
    count_launch();
    return set_cuda_status(e);
}
