// Decode glue between the GEMVs: rotary embedding, KV-cache scatter and single-query attention.
//
// Replaces cuda/nve_kernels.cu:144-262 (RoPE decode/prefill), :1006-1065 (RoPE with device position),
// :909-946 (KV scatter), :462-591 and :1075-1197 (flash decode, static and device-length forms) of the
// reference project.
//
// Attention design: the reference runs one CTA per query head (32-64 CTAs).  Here every query head is
// served by a thread-block cluster of kFdCluster CTAs that split the sequence; each CTA keeps an online
// softmax state per warp, merges its warps in shared memory, and rank 0 of the cluster merges the CTA
// partials through distributed shared memory.  No global scratch and no second launch are needed.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace nve {

// ---------------------------------------------------------------------------------------------
// RoPE (half-split pairs i, i + hd/2), explicit IEEE rounding so that results are reproducible.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void rope_pair(uint16_t* ptr, int elem, int half_dim, float c, float s) {
    const float x0 = Act16<NVE_DT_F16>::to_f32(ptr[elem]);
    const float x1 = Act16<NVE_DT_F16>::to_f32(ptr[elem + half_dim]);
    ptr[elem] = Act16<NVE_DT_F16>::from_f32(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)));
    ptr[elem + half_dim] = Act16<NVE_DT_F16>::from_f32(__fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c)));
}

// tokens: 1 for decode.  Position of token t = start_pos + t, or *d_pos when d_pos != NULL.
// table_rows: true when cos/sin are [max_seq, hd/2] tables indexed by position; false when they are the
// single row for the current position.
__global__ void rope_kernel(uint16_t* q, uint16_t* k, const uint16_t* cos_t, const uint16_t* sin_t, int tokens,
                            int num_heads, int num_kv_heads, int head_dim, int start_pos, const int* d_pos,
                            bool table_rows) {
    pdl_wait();
    const int half_dim = head_dim / 2;
    const long long total_q = static_cast<long long>(tokens) * num_heads * half_dim;
    const long long total_k = static_cast<long long>(tokens) * num_kv_heads * half_dim;
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= total_q + total_k) return;
    const bool is_q = idx < total_q;
    const long long li = is_q ? idx : idx - total_q;
    const int heads = is_q ? num_heads : num_kv_heads;
    const int elem = static_cast<int>(li % half_dim);
    const int head = static_cast<int>((li / half_dim) % heads);
    const int tok = static_cast<int>(li / (static_cast<long long>(half_dim) * heads));
    int pos = start_pos + tok;
    if (d_pos != nullptr) pos = *d_pos;
    const long long trow = table_rows ? static_cast<long long>(pos) * half_dim : 0;
    const float c = Act16<NVE_DT_F16>::to_f32(cos_t[trow + elem]);
    const float s = Act16<NVE_DT_F16>::to_f32(sin_t[trow + elem]);
    uint16_t* base = (is_q ? q : k) + (static_cast<long long>(tok) * heads + head) * head_dim;
    rope_pair(base, elem, half_dim, c, s);
}

static void launch_rope(uint16_t* q, uint16_t* k, const uint16_t* c, const uint16_t* s, int tokens, int nh, int nkv,
                        int hd, int start_pos, const int* d_pos, bool table_rows, cudaStream_t st) {
    if (!q || !k || !c || !s) { set_status(NVE_ERR_BAD_POINTER); return; }
    if (tokens <= 0 || nh <= 0 || nkv < 0 || hd <= 0 || (hd & 1)) { set_status(NVE_ERR_BAD_SHAPE); return; }
    const long long total = static_cast<long long>(tokens) * (nh + nkv) * (hd / 2);
    const int block = 256;
    rope_kernel<<<static_cast<unsigned>((total + block - 1) / block), block, 0, st>>>(q, k, c, s, tokens, nh, nkv, hd,
                                                                                       start_pos, d_pos, table_rows);
    count_launch();
    check_launch();
}

// ---------------------------------------------------------------------------------------------
// KV scatter: cache[kvh, pos, :] = new[kvh, :]
// ---------------------------------------------------------------------------------------------
__global__ void kv_write_kernel(const uint16_t* k_new, uint16_t* k_cache, const uint16_t* v_new, uint16_t* v_cache,
                                const int* d_pos, int num_kv_heads, int head_dim, int max_seq_len) {
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= num_kv_heads * head_dim) return;
    const int pos = *d_pos;
    if (pos < 0 || pos >= max_seq_len) return;  // out-of-range position: skip instead of writing out of bounds
    const int kvh = i / head_dim, e = i - kvh * head_dim;
    const long long dst = (static_cast<long long>(kvh) * max_seq_len + pos) * head_dim + e;
    k_cache[dst] = k_new[i];
    v_cache[dst] = v_new[i];
}

// ---------------------------------------------------------------------------------------------
// Flash decode
// ---------------------------------------------------------------------------------------------
constexpr int kFdCluster = 8;  // CTAs per query head (portable cluster size)
constexpr int kFdWarps = 4;    // warps per CTA
constexpr int kFdMaxVe = 16;   // head_dim / 32 <= 16  (head_dim <= 512)

// Partial state of one CTA, read by rank 0 of its cluster through distributed shared memory.
struct FdPartial {
    float m;
    float s;
    float acc[kFdMaxVe * 32];
};

// Load VE consecutive 16-bit values as f32; one vector load when the caller guarantees alignment.
template <int VE, bool VEC> __device__ __forceinline__ void load_ve(const uint16_t* p, float (&o)[VE]) {
    if constexpr (VEC && VE == 2) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
        o[0] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(w & 0xFFFFu));
        o[1] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(w >> 16));
    } else if constexpr (VEC && VE == 4) {
        const uint2 w = *reinterpret_cast<const uint2*>(p);
        o[0] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(w.x & 0xFFFFu));
        o[1] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(w.x >> 16));
        o[2] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(w.y & 0xFFFFu));
        o[3] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(w.y >> 16));
    } else if constexpr (VEC && (VE % 8) == 0) {
#pragma unroll
        for (int v = 0; v < VE / 8; v++) {
            const uint4 w = reinterpret_cast<const uint4*>(p)[v];
            const uint32_t wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                o[v * 8 + 2 * j] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(wv[j] & 0xFFFFu));
                o[v * 8 + 2 * j + 1] = Act16<NVE_DT_F16>::to_f32(static_cast<uint16_t>(wv[j] >> 16));
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < VE; i++) o[i] = Act16<NVE_DT_F16>::to_f32(p[i]);
    }
}

template <int VE, bool VEC>
__global__ void __launch_bounds__(kFdWarps * 32) flash_decode_kernel(const uint16_t* q, const uint16_t* k_cache,
                                                                     const uint16_t* v_cache, uint16_t* out,
                                                                     int num_kv_heads, int groups, int seq_len_arg,
                                                                     const int* d_seq_len, int kv_stride, float scale) {
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ FdPartial cta_part;
    __shared__ float warp_m[kFdWarps], warp_s[kFdWarps];
    __shared__ float warp_acc[kFdWarps][VE * 32];

    pdl_wait();
    const int head_dim = VE * 32;
    const int h = blockIdx.x / kFdCluster;
    const int rank = static_cast<int>(cluster.block_rank());
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int kvh = h / groups;
    int seq_len = d_seq_len != nullptr ? *d_seq_len : seq_len_arg;
    seq_len = max(0, min(seq_len, kv_stride));

    // this lane owns elements [lane*VE, lane*VE + VE)
    float qr[VE];
#pragma unroll
    for (int i = 0; i < VE; i++) qr[i] = Act16<NVE_DT_F16>::to_f32(q[static_cast<long long>(h) * head_dim + lane * VE + i]);

    const uint16_t* kh = k_cache + static_cast<long long>(kvh) * kv_stride * head_dim;
    const uint16_t* vh = v_cache + static_cast<long long>(kvh) * kv_stride * head_dim;

    // positions are dealt round-robin in groups of 4 to the (rank, warp) pairs
    const int slot = rank * kFdWarps + warp;
    const int nslots = kFdCluster * kFdWarps;
    float m = -1e30f, s = 0.0f;
    float acc[VE];
#pragma unroll
    for (int i = 0; i < VE; i++) acc[i] = 0.0f;

    for (int t0 = slot * 4; t0 < seq_len; t0 += nslots * 4) {
        float kv[4][VE], vv[4][VE], dot[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int t = min(t0 + j, seq_len - 1);
            const uint16_t* kp = kh + static_cast<long long>(t) * head_dim + lane * VE;
            const uint16_t* vp = vh + static_cast<long long>(t) * head_dim + lane * VE;
            load_ve<VE, VEC>(kp, kv[j]);
            load_ve<VE, VEC>(vp, vv[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float d = 0.0f;
#pragma unroll
            for (int i = 0; i < VE; i++) d = fmaf(qr[i], kv[j][i], d);
            dot[j] = d;
        }
#pragma unroll
        for (int j = 0; j < 4; j++) dot[j] = warp_sum(dot[j]) * scale;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            if (t0 + j < seq_len) {
                const float new_m = fmaxf(m, dot[j]);
                const float corr = expf(m - new_m);
                const float e = expf(dot[j] - new_m);
#pragma unroll
                for (int i = 0; i < VE; i++) acc[i] = fmaf(e, vv[j][i], acc[i] * corr);
                s = fmaf(s, corr, e);
                m = new_m;
            }
        }
    }

    // merge the warps of this CTA
    if (lane == 0) { warp_m[warp] = m; warp_s[warp] = s; }
#pragma unroll
    for (int i = 0; i < VE; i++) warp_acc[warp][lane * VE + i] = acc[i];
    __syncthreads();
    if (warp == 0) {
        float mm = warp_m[0];
#pragma unroll
        for (int w = 1; w < kFdWarps; w++) mm = fmaxf(mm, warp_m[w]);
        float ss = 0.0f;
        float a[VE];
#pragma unroll
        for (int i = 0; i < VE; i++) a[i] = 0.0f;
#pragma unroll
        for (int w = 0; w < kFdWarps; w++) {
            const float c = expf(warp_m[w] - mm);
            ss = fmaf(warp_s[w], c, ss);
#pragma unroll
            for (int i = 0; i < VE; i++) a[i] = fmaf(warp_acc[w][lane * VE + i], c, a[i]);
        }
        if (lane == 0) { cta_part.m = mm; cta_part.s = ss; }
#pragma unroll
        for (int i = 0; i < VE; i++) cta_part.acc[lane * VE + i] = a[i];
    }
    cluster.sync();
    if (rank == 0 && warp == 0) {
        float pm[kFdCluster], mm = -1e30f;
#pragma unroll
        for (int r = 0; r < kFdCluster; r++) {
            const FdPartial* rp = cluster.map_shared_rank(&cta_part, r);
            pm[r] = rp->m;
            mm = fmaxf(mm, pm[r]);
        }
        float ss = 0.0f;
        float a[VE];
#pragma unroll
        for (int i = 0; i < VE; i++) a[i] = 0.0f;
#pragma unroll
        for (int r = 0; r < kFdCluster; r++) {
            const FdPartial* rp = cluster.map_shared_rank(&cta_part, r);
            const float c = expf(pm[r] - mm);
            ss = fmaf(rp->s, c, ss);
#pragma unroll
            for (int i = 0; i < VE; i++) a[i] = fmaf(rp->acc[lane * VE + i], c, a[i]);
        }
        const float inv = ss > 0.0f ? 1.0f / ss : 0.0f;
#pragma unroll
        for (int i = 0; i < VE; i++)
            out[static_cast<long long>(h) * head_dim + lane * VE + i] = Act16<NVE_DT_F16>::from_f32(a[i] * inv);
    }
    // keep every CTA's shared memory alive until rank 0 has read it
    cluster.sync();
}

template <int VE>
static cudaError_t launch_fd(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, uint16_t* out, int nh, int nkv,
                             int seq_len, const int* d_seq_len, int kv_stride, float scale, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(nh * kFdCluster);
    cfg.blockDim = dim3(kFdWarps * 32);
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kFdCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (pdl_enabled()) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    const bool vec = aligned(kc, 16) && aligned(vc, 16);
    if (vec)
        return cudaLaunchKernelEx(&cfg, flash_decode_kernel<VE, true>, q, kc, vc, out, nkv, nh / nkv, seq_len, d_seq_len,
                                  kv_stride, scale);
    return cudaLaunchKernelEx(&cfg, flash_decode_kernel<VE, false>, q, kc, vc, out, nkv, nh / nkv, seq_len, d_seq_len,
                              kv_stride, scale);
}

// Fast path for head_dim 64 / 128 (attn_decode.cu); returns false when the shape is not covered.
bool attn_decode_try(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, uint16_t* out, int nh, int nkv, int seq_len,
                     const int* d_seq_len, int kv_stride, int hd, float scale, cudaStream_t st);

static void flash_decode(const uint16_t* q, const uint16_t* kc, const uint16_t* vc, uint16_t* out, int nh, int nkv,
                         int seq_len, const int* d_seq_len, int kv_stride, int hd, float scale, cudaStream_t st) {
    if (!q || !kc || !vc || !out) { set_status(NVE_ERR_BAD_POINTER); return; }
    // same support envelope as the reference: head_dim a multiple of 32, at most 512
    if (hd <= 0 || (hd % 32) != 0 || hd / 32 > kFdMaxVe || nh <= 0 || nkv <= 0 || (nh % nkv) != 0 || kv_stride <= 0) {
        set_status(NVE_ERR_BAD_SHAPE);
        return;
    }
    if (attn_decode_try(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, hd, scale, st)) return;
    cudaError_t e;
    switch (hd / 32) {
        case 1: e = launch_fd<1>(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, scale, st); break;
        case 2: e = launch_fd<2>(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, scale, st); break;
        case 3: e = launch_fd<3>(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, scale, st); break;
        case 4: e = launch_fd<4>(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, scale, st); break;
        case 5: e = launch_fd<5>(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, scale, st); break;
        case 6: e = launch_fd<6>(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, scale, st); break;
        case 8: e = launch_fd<8>(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, scale, st); break;
        case 16: e = launch_fd<16>(q, kc, vc, out, nh, nkv, seq_len, d_seq_len, kv_stride, scale, st); break;
        default: set_status(NVE_ERR_BAD_SHAPE); return;
    }
    count_launch();
    set_cuda_status(e);
}

}  // namespace nve

using namespace nve;

extern "C" void nve_rope_f16_decode(uint16_t* q, uint16_t* k, const uint16_t* cos, const uint16_t* sin, int num_heads,
                                    int num_kv_heads, int head_dim, nve_stream_t stream) {
    launch_rope(q, k, cos, sin, 1, num_heads, num_kv_heads, head_dim, 0, nullptr, false, static_cast<cudaStream_t>(stream));
}

extern "C" void nve_rope_f16_prefill(uint16_t* q, uint16_t* k, const uint16_t* cos, const uint16_t* sin, int seq_len,
                                     int num_heads, int num_kv_heads, int head_dim, int start_pos, nve_stream_t stream) {
    launch_rope(q, k, cos, sin, seq_len, num_heads, num_kv_heads, head_dim, start_pos, nullptr, true,
                static_cast<cudaStream_t>(stream));
}

extern "C" void nve_rope_f16_decode_dyn(uint16_t* q, uint16_t* k, const uint16_t* cos_tab, const uint16_t* sin_tab,
                                        int num_heads, int num_kv_heads, int head_dim, const int* d_pos,
                                        nve_stream_t stream) {
    if (!d_pos) { set_status(NVE_ERR_BAD_POINTER); return; }
    launch_rope(q, k, cos_tab, sin_tab, 1, num_heads, num_kv_heads, head_dim, 0, d_pos, true,
                static_cast<cudaStream_t>(stream));
}

// cache[kvh, start_pos + s, :] = new[s, kvh, :] for a block of S new positions (K and V).
__global__ void kv_write_rows_kernel(const uint16_t* k_new, uint16_t* k_cache, const uint16_t* v_new, uint16_t* v_cache, int rows,
                                     int start_pos, int nkv, int hd, int max_seq) {
    pdl_wait();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long n = static_cast<long long>(rows) * nkv * hd;
    if (i >= n) return;
    const int d = static_cast<int>(i % hd);
    const int h = static_cast<int>((i / hd) % nkv);
    const int s = static_cast<int>(i / (static_cast<long long>(hd) * nkv));
    const long long dst = (static_cast<long long>(h) * max_seq + start_pos + s) * hd + d;
    k_cache[dst] = k_new[i];
    v_cache[dst] = v_new[i];
}

extern "C" int nve_b200_kv_cache_write_rows(const uint16_t* k_new, uint16_t* k_cache, const uint16_t* v_new, uint16_t* v_cache,
                                            int rows, int start_pos, int num_kv_heads, int head_dim, int max_seq_len,
                                            nve_stream_t stream) {
    if (!k_new || !k_cache || !v_new || !v_cache) return set_status(NVE_ERR_BAD_POINTER);
    if (rows <= 0 || start_pos < 0 || num_kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0 || start_pos + rows > max_seq_len)
        return set_status(NVE_ERR_BAD_SHAPE);
    const long long n = static_cast<long long>(rows) * num_kv_heads * head_dim;
    kv_write_rows_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        k_new, k_cache, v_new, v_cache, rows, start_pos, num_kv_heads, head_dim, max_seq_len);
    count_launch();
    return check_launch();
}

extern "C" void nve_kv_cache_write_f16(const uint16_t* k_new, uint16_t* k_cache, const uint16_t* v_new, uint16_t* v_cache,
                                       const int* d_pos, int num_kv_heads, int head_dim, int max_seq_len,
                                       nve_stream_t stream) {
    if (!k_new || !k_cache || !v_new || !v_cache || !d_pos) { set_status(NVE_ERR_BAD_POINTER); return; }
    if (num_kv_heads <= 0 || head_dim <= 0 || max_seq_len <= 0) { set_status(NVE_ERR_BAD_SHAPE); return; }
    const int n = num_kv_heads * head_dim;
    kv_write_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(k_new, k_cache, v_new, v_cache, d_pos,
                                                                                   num_kv_heads, head_dim, max_seq_len);
    count_launch();
    check_launch();
}

extern "C" void nve_flash_decode_f16(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out,
                                     int num_heads, int num_kv_heads, int seq_len, int head_dim, float scale,
                                     nve_stream_t stream) {
    if (seq_len <= 0) { set_status(NVE_ERR_BAD_SHAPE); return; }  // the reference skips the launch too
    flash_decode(q, k_cache, v_cache, out, num_heads, num_kv_heads, seq_len, nullptr, seq_len, head_dim, scale,
                 static_cast<cudaStream_t>(stream));
}

extern "C" void nve_flash_decode_dyn(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out,
                                     int num_heads, int num_kv_heads, const int* d_seq_len, int head_dim, float scale,
                                     int max_seq_len, nve_stream_t stream) {
    if (!d_seq_len) { set_status(NVE_ERR_BAD_POINTER); return; }
    flash_decode(q, k_cache, v_cache, out, num_heads, num_kv_heads, 0, d_seq_len, max_seq_len, head_dim, scale,
                 static_cast<cudaStream_t>(stream));
}
