// Launch parameters of the decode attention kernels (attn_decode.cu, attn_batch_mma.cu).
#pragma once
#include "common.cuh"

namespace nve {

struct AttnParams {
    const uint16_t* q;        // [nh, hd]
    const uint16_t* k_new;    // [nkv, hd] (fused form)
    const uint16_t* v_new;    // [nkv, hd]
    uint16_t* k_cache;        // [nkv, kv_stride, hd]
    uint16_t* v_cache;
    const uint16_t* cos_tab;  // [max_seq, hd/2]
    const uint16_t* sin_tab;
    const int* d_pos;         // fused form: position of the new token
    const int* d_seq_len;     // valid length (device scalar) or NULL
    int seq_len;              // valid length when d_seq_len == NULL
    uint16_t* out;            // [nh, hd] f16
    int8_t* out_q;            // optional int8 codes of out, group 32
    float* out_scales;        // [nh*hd/32]
    int num_heads, num_kv_heads, kv_stride;
    float scale;
    // un-fused form only: blockIdx.y selects one of `rows` query rows; row r reads q + r * row_stride, writes
    // out + r * row_stride and attends to seq_len + r positions (causal attention over a block of new positions)
    int rows, row_stride;
    // batched fused form: `rows` independent sequences; elements between consecutive K (or V) caches
    long long cache_stride;
};

// attn_batch_mma.cu: false when the shape is not covered (the caller then uses another kernel).  fused: `rows`
// independent sequences with RoPE and the K/V write inside; else the un-fused causal block described above.
bool attn_batch_mma_try(const AttnParams& p, int head_dim, cudaStream_t st, cudaError_t& err, bool fused = true);

// attn_decode_mma.cu: the fused decode attention of one sequence on the tensor cores; false when the shape is not
// covered.
bool attn_decode_mma_try(const AttnParams& p, int head_dim, cudaStream_t st, cudaError_t& err, bool fused = true);

}  // namespace nve
