/*
 * libnve_kernels.so -- C ABI of the B200 (sm_100a) quantized decode kernels for NVE.
 *
 * Part 1 re-declares, with identical names, argument order and meaning, every symbol the
 * reference project exports from cuda/nve_kernels.cu and binds in src/cuda_kernels.rs:57-289.
 * A library exporting these symbols is what the reference's build.rs:33-41 links when
 * NVE_KERNELS_PREBUILT points at its directory.  Each declaration cites the reference
 * definition it replaces (file:line in the reference project).
 *
 * Part 2 declares additive entry points (prefix nve_b200_) that the reference does not have:
 * status reporting, bf16/f32 I/O, fused prologues/epilogues, the batched tensor-core GEMM,
 * on-device weight preparation and tensor-parallel helpers.
 *
 * Conventions (same as the reference, src/cuda_kernels.rs:296-339):
 *   - every pointer is a raw device address owned by the caller unless stated otherwise;
 *   - 16-bit floats travel as uint16_t; int8 codes as int8_t; scales as float;
 *   - every launcher enqueues on `stream` and returns; NULL is the legacy default stream;
 *   - launchers allocate nothing and are legal inside stream capture;
 *   - the reference-signature launchers return void and silently skip unsupported shapes,
 *     as the reference does (cuda/nve_kernels.cu:582,1188); the reason is recorded and can be
 *     read with nve_b200_last_status().
 *
 * Weight format (src/quantize.rs:437-463, cuda/nve_kernels.cu:330-361):
 *   nibbles [N, K/2] u8 row-major, byte j of 32-wide block b = q[j] | q[j+16] << 4, q in [0,15],
 *   weight value = (q - 8) * scales[n, b];  scales [N, K/32] f32;  K % 32 == 0.
 */
#ifndef NVE_KERNELS_H
#define NVE_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported symbols (the library is built with hidden default visibility). */
#if defined(__GNUC__)
#define NVE_API __attribute__((visibility("default")))
#else
#define NVE_API
#endif

/* Opaque CUDA stream handle (cudaStream_t) so that C callers need no CUDA headers. */
typedef void* nve_stream_t;

/* ======================================================================================== */
/* Part 1: the reference ABI                                                                */
/* ======================================================================================== */

/* cuda/nve_kernels.cu:63-76.  out = f16(x * rsqrt(mean(x^2)+eps) * w), n elements. */
NVE_API void nve_rms_norm_f16(const uint16_t* x, const uint16_t* weight, uint16_t* out, int n, float eps,
                      nve_stream_t stream);

/* cuda/nve_kernels.cu:120-134.  LayerNorm with optional bias (bias may be NULL). */
NVE_API void nve_layer_norm_f16(const uint16_t* x, const uint16_t* weight, const uint16_t* bias, uint16_t* out, int n,
                        float eps, nve_stream_t stream);

/* cuda/nve_kernels.cu:182-200.  Half-split RoPE on q [nh,hd] and k [nkv,hd] in place; cos/sin [hd/2]. */
NVE_API void nve_rope_f16_decode(uint16_t* q, uint16_t* k, const uint16_t* cos, const uint16_t* sin, int num_heads,
                         int num_kv_heads, int head_dim, nve_stream_t stream);

/* cuda/nve_kernels.cu:246-262.  RoPE for seq_len tokens; tables [max_seq, hd/2]; q [seq,nh,hd]. */
NVE_API void nve_rope_f16_prefill(uint16_t* q, uint16_t* k, const uint16_t* cos, const uint16_t* sin, int seq_len,
                          int num_heads, int num_kv_heads, int head_dim, int start_pos, nve_stream_t stream);

/* cuda/nve_kernels.cu:1049-1065.  As nve_rope_f16_decode but the position is read from *d_pos and the
 * full tables [max_seq, hd/2] are passed. */
NVE_API void nve_rope_f16_decode_dyn(uint16_t* q, uint16_t* k, const uint16_t* cos_tab, const uint16_t* sin_tab,
                             int num_heads, int num_kv_heads, int head_dim, const int* d_pos,
                             nve_stream_t stream);

/* cuda/nve_kernels.cu:300-314.  Dense f16 GEMV out[N] = W[N,K] . x[K]. */
NVE_API void nve_matvec_f16(const uint16_t* x, const uint16_t* W, uint16_t* out, int N, int K, nve_stream_t stream);

/* cuda/nve_kernels.cu:373-388.  W4A16 GEMV: out[n] = f16(sum_k x[k] [*awq[k]] (q-8) scale[n,k/32]);
 * awq may be NULL. */
NVE_API void nve_matvec_w4a16(const uint16_t* x, const uint8_t* nibbles, const float* scales, const float* awq,
                      uint16_t* out, int N, int K, nve_stream_t stream);

/* cuda/nve_kernels.cu:420-433.  Full dequantisation W_f16[N,K] = (q-8)*scale [*awq[k]]. */
NVE_API void nve_dequant_w4a16(const uint8_t* nibbles, const float* scales, const float* awq, uint16_t* out, int N,
                       int K, nve_stream_t stream);

/* cuda/nve_kernels.cu:680-700.  W4A16 GEMV over three matrices sharing x, one launch. */
NVE_API void nve_qkv_matvec_w4a16(const uint16_t* x,
                          const uint8_t* q_nibbles, const float* q_scales, const float* q_awq, int Nq,
                          const uint8_t* k_nibbles, const float* k_scales, const float* k_awq, int Nk,
                          const uint8_t* v_nibbles, const float* v_scales, const float* v_awq, int Nv,
                          uint16_t* q_out, uint16_t* k_out, uint16_t* v_out, int K, nve_stream_t stream);

/* cuda/nve_kernels.cu:747-757.  Per-group-32 absmax int8 quantisation of f16 activations:
 * scale = amax > 0 ? amax/127 : 1 ; xq = clamp(rint(x / scale), -127, 127). */
NVE_API void nve_quantize_f16_q8(const uint16_t* x, int8_t* xq, float* scales, int K, nve_stream_t stream);

/* cuda/nve_kernels.cu:880-894.  W4A8 GEMV: out[n] = f16(sum_b wt_scales[n,b] * xq_scales[b] * I[n,b]),
 * I[n,b] = sum_e (q-8) * xq[32b+e] (exact int32). */
NVE_API void nve_matvec_w4a8(const int8_t* xq, const float* xq_scales, const uint8_t* nibbles, const float* wt_scales,
                     uint16_t* out, int N, int K, nve_stream_t stream);

/* cuda/nve_kernels.cu:574-591.  Single-query GQA attention; caches [nkv, seq_len, hd]; needs hd%32==0, hd<=512. */
NVE_API void nve_flash_decode_f16(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out,
                          int num_heads, int num_kv_heads, int seq_len, int head_dim, float scale,
                          nve_stream_t stream);

/* cuda/nve_kernels.cu:1177-1197.  As above with the length in *d_seq_len and caches [nkv, max_seq_len, hd]. */
NVE_API void nve_flash_decode_dyn(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out,
                          int num_heads, int num_kv_heads, const int* d_seq_len, int head_dim, float scale,
                          int max_seq_len, nve_stream_t stream);

/* cuda/nve_kernels.cu:931-946.  cache[kvh, *d_pos, :] = new[kvh, :] for K and V. */
NVE_API void nve_kv_cache_write_f16(const uint16_t* k_new, uint16_t* k_cache, const uint16_t* v_new, uint16_t* v_cache,
                            const int* d_pos, int num_kv_heads, int head_dim, int max_seq_len,
                            nve_stream_t stream);

/* cuda/nve_kernels.cu:963-969.  dst[i] = f16(f32(dst[i]) + f32(src[i])). */
NVE_API void nve_add_inplace_f16(uint16_t* dst, const uint16_t* src, int n, nve_stream_t stream);

/* cuda/nve_kernels.cu:989-995.  gate[i] = f16(silu(gate[i]) * up[i]). */
NVE_API void nve_silu_mul_f16(uint16_t* gate, const uint16_t* up, int n, nve_stream_t stream);

/* cuda/nve_kernels.cu:1203-1205.  Device-to-device async copy. */
NVE_API void nve_d2d_copy(void* dst, const void* src, size_t bytes, nve_stream_t stream);

/* cuda/nve_kernels.cu:1230-1299.  Process-global decode-graph manager: one capture stream, pinned
 * pos/seq_len scalars copied to device scalars by the first two nodes of the graph.
 * nve_graph_launch writes pos / seq_len into the pinned words at once and the replay reads them when its first two
 * nodes run: do not issue the next nve_graph_launch with other values before the previous replay has consumed them
 * (synchronise the stream, or at least wait for an event recorded after the previous launch) -- two replays
 * enqueued back to back can otherwise both read the later position.  The reference has the same property. */
NVE_API void nve_graph_init(void);
NVE_API void nve_graph_begin_capture(void);
NVE_API void nve_graph_end_capture(void);
NVE_API void nve_graph_launch(int pos, int seq_len, nve_stream_t stream);
NVE_API int nve_graph_ready(void);
NVE_API void nve_graph_destroy(void);
NVE_API const int* nve_graph_d_pos(void);
NVE_API const int* nve_graph_d_seqlen(void);
NVE_API nve_stream_t nve_graph_capture_stream(void);

/* cuda/nve_kernels.cu:1306-1413.  Event-timed microbenchmark of the decode kernels; prints to stdout. */
NVE_API void nve_run_microbench(int hidden, int intermediate, int num_heads, int num_kv_heads, int head_dim, int iters);

/* ======================================================================================== */
/* Part 2: additive entry points (no counterpart in the reference unless cited)             */
/* ======================================================================================== */

/* 16-bit / 32-bit element types accepted by the *_ex entry points. */
#define NVE_DT_F16 0
#define NVE_DT_BF16 1
#define NVE_DT_F32 2

/* Status codes.  Every nve_b200_* launcher returns one; 0 is success. */
#define NVE_OK 0
#define NVE_ERR_BAD_SHAPE 1      /* K % 32 != 0, non-positive sizes, unsupported head_dim ... */
#define NVE_ERR_BAD_POINTER 2    /* NULL where data is required */
#define NVE_ERR_BAD_ALIGNMENT 3  /* pointer not aligned for the kernel's vector accesses */
#define NVE_ERR_BAD_DTYPE 4
#define NVE_ERR_TOO_LARGE 5      /* exceeds a documented limit (shared memory, static scratch) */
#define NVE_ERR_CUDA 6           /* a CUDA runtime call failed; see nve_b200_last_cuda_error() */
#define NVE_ERR_TIMEOUT 7        /* a bounded device-side wait expired */

/* Status of the most recent launcher call on this thread (reference-signature calls included). */
NVE_API int nve_b200_last_status(void);
/* cudaError_t (as int) recorded with the last NVE_ERR_CUDA. */
NVE_API int nve_b200_last_cuda_error(void);
/* Library build tag, e.g. "nve-b200 sm_100a". */
NVE_API const char* nve_b200_version(void);
/* Number of kernels this library has launched from this process (all threads). */
NVE_API unsigned long long nve_b200_launch_count(void);
/* Enable (1) / disable (0) programmatic dependent launch on the GEMV launches; returns the old value. */
NVE_API int nve_b200_set_pdl(int enabled);

/* Activation quantizer with selectable input type (NVE_DT_F16 or NVE_DT_BF16); arithmetic as
 * nve_quantize_f16_q8 (cuda/nve_kernels.cu:712-745). */
NVE_API int nve_b200_quantize_q8(const void* x, int8_t* xq, float* scales, int K, int x_dtype, nve_stream_t stream);

/* The same quantiser for the activations of an AWQ pre-scaled matrix (src/quantize.rs:271-304 scales column k of the
 * weights by s[k] and the W4A16 kernels multiply x[k] by awq_inv[k] = 1/s[k]): x[k] * awq_inv[k] (f32 product) is what
 * gets quantised.  The reference drops the multiplier on its W4A8 route (nve_matvec_w4a8 has no such argument,
 * src/gpu_layer.rs:659); with this entry point the W4A8 route sees the activations the W4A16 route sees. */
NVE_API int nve_b200_quantize_q8_awq(const void* x, const float* awq_inv, int8_t* xq, float* scales, int K, int x_dtype,
                                     nve_stream_t stream);

/* Fused RMSNorm -> 16-bit round -> int8 quantisation (the two launches at src/gpu_layer.rs:1032-1038,658
 * in one).  normed_out may be NULL when only the codes are needed. */
NVE_API int nve_b200_rmsnorm_quantize_q8(const void* x, const void* weight, void* normed_out, int8_t* xq, float* scales,
                                 int n, float eps, int dtype, nve_stream_t stream);

/* RMSNorm with selectable 16-bit type (cuda/nve_kernels.cu:26-60 arithmetic, fixed summation order). */
NVE_API int nve_b200_rms_norm(const void* x, const void* weight, void* out, int n, float eps, int dtype,
                      nve_stream_t stream);

/* Fused silu(gate)*up -> 16-bit round -> int8 quantisation (src/gpu_layer.rs:942-946 in one launch).
 * mid_out may be NULL. */
NVE_API int nve_b200_silu_mul_quantize_q8(const void* gate, const void* up, void* mid_out, int8_t* xq, float* scales,
                                  int n, int dtype, nve_stream_t stream);

/* Fused silu(gate)*up -> 16-bit round -> [* awq] -> 16-bit fixed point per group of 32 (v = rint(x * 32767 / amax),
 * low bytes to x_lo, high bytes to x_hi, amax / 32767 to x_scales): the activation form the W4A16 GEMV multiplies
 * with, produced once here instead of by every CTA of the GEMV (nve_b200_matvec_w4a16_planes_multi consumes it).
 * No counterpart in the reference (src/gpu_layer.rs:977-980 feeds the f16 product to nve_matvec_w4a16); the
 * results are bit-identical to nve_b200_silu_mul followed by nve_b200_matvec_w4a16_multi.  mid_out and awq may
 * be NULL; n % 32 == 0. */
NVE_API int nve_b200_silu_mul_x16(const void* gate, const void* up, void* mid_out, uint8_t* x_lo, int8_t* x_hi,
                                  float* x_scales, const float* awq, int n, int dtype, nve_stream_t stream);

/* silu(gate)*up and residual add with selectable 16-bit type. */
NVE_API int nve_b200_silu_mul(void* gate, const void* up, int n, int dtype, nve_stream_t stream);

/* ---- prefill (a block of S new positions of one sequence; src/gpu_layer.rs:777-890, :1086-1160) --------------
 * The projections of a block go through nve_b200_gemm_w4a16 / _multi (M = S, in slices of 64 rows); these three
 * entry points are the glue around them.
 * nve_b200_rms_norm_rows: RMSNorm of every row of x [rows, n] with one weight vector, one launch (the reference runs
 *   its kernel once per token, src/gpu_layer.rs:137); each row is bit-identical to nve_b200_rms_norm on it.
 * nve_b200_kv_cache_write_rows: cache[kvh, start_pos + s, :] = new[s, kvh, :] for K and V (k_new / v_new
 *   [rows, num_kv_heads, head_dim], caches [num_kv_heads, max_seq_len, head_dim]); replaces the transpose + append of
 *   src/gpu_layer.rs:814-818.
 * nve_b200_attn_prefill_causal: row r of q [rows, num_heads * head_dim] attends to positions [0, start_pos + r] of the
 *   caches (which already hold the block); out has q's layout.  Replaces the unfused masked SDPA of
 *   src/gpu_layer.rs:846-885.  Blocks of fewer than 64 (row, KV head) pairs run the decode kernel with the row as
 *   second grid dimension: every row equals a nve_flash_decode_f16 call of length start_pos + r + 1 bit for bit.
 *   Larger blocks run a tensor-core kernel (one CTA per row and KV head; f16 probabilities, another summation
 *   order): equal to those calls within 5e-3 of the largest output.  head_dim 64 or 128; q and caches 16-byte
 *   aligned. */
NVE_API int nve_b200_rms_norm_rows(const void* x, const void* weight, void* out, int rows, int n, float eps, int dtype,
                                   nve_stream_t stream);
/* x[r] += delta[r] in place (nve_b200_add_inplace's arithmetic) and out[r] = RMSNorm(x[r]) for every row, one launch:
 * the residual add and the norm between two projections of a batched layer (src/gpu_layer.rs:1139-1147 runs them as
 * separate kernels per token).  Bit-identical to nve_b200_add_inplace followed by nve_b200_rms_norm_rows.  n % 8 == 0,
 * 16-byte aligned pointers. */
NVE_API int nve_b200_add_rms_norm_rows(void* x, const void* delta, const void* weight, void* out, int rows, int n,
                                       float eps, int dtype, nve_stream_t stream);
NVE_API int nve_b200_kv_cache_write_rows(const uint16_t* k_new, uint16_t* k_cache, const uint16_t* v_new,
                                         uint16_t* v_cache, int rows, int start_pos, int num_kv_heads, int head_dim,
                                         int max_seq_len, nve_stream_t stream);
NVE_API int nve_b200_attn_prefill_causal(const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache,
                                         uint16_t* out, int rows, int start_pos, int num_heads, int num_kv_heads,
                                         int head_dim, int max_seq_len, float scale, nve_stream_t stream);
NVE_API int nve_b200_add_inplace(void* dst, const void* src, int n, int dtype, nve_stream_t stream);

/* One matrix of a fused multi-matrix GEMV (all share the activation vector and K). */
typedef struct {
    const uint8_t* nibbles; /* [N, K/2]  */
    const float* scales;    /* [N, K/32] */
    void* out;              /* [N] of out_dtype */
    const void* residual;   /* NULL, or [N] of out_dtype: out = residual + y (may alias out) */
    int N;
} nve_b200_w4_matrix;

/* W4A8 GEMV over 1..3 matrices in one launch (q/k/v, or gate/up), selectable output type and optional
 * fused residual add.  Arithmetic as nve_matvec_w4a8 (cuda/nve_kernels.cu:796-878). */
NVE_API int nve_b200_matvec_w4a8_multi(const int8_t* xq, const float* xq_scales, const nve_b200_w4_matrix* mats,
                               int num_mats, int K, int out_dtype, nve_stream_t stream);

/* W4A16 GEMV over 1..3 matrices in one launch; x of x_dtype (f16/bf16), awq may be NULL (shared by all
 * matrices of the call).  Arithmetic as nve_matvec_w4a16 (cuda/nve_kernels.cu:349-370). */
NVE_API int nve_b200_matvec_w4a16_multi(const void* x, int x_dtype, const float* awq, const nve_b200_w4_matrix* mats,
                                int num_mats, int K, int out_dtype, nve_stream_t stream);

/* W4A16 GEMV over 1..3 matrices whose activations are already in the 16-bit fixed-point plane form written by
 * nve_b200_silu_mul_x16 (x_lo / x_hi [K], x_scales [K/32]; all 16-byte aligned). */
NVE_API int nve_b200_matvec_w4a16_planes_multi(const uint8_t* x_lo, const int8_t* x_hi, const float* x_scales,
                                               const nve_b200_w4_matrix* mats, int num_mats, int K, int out_dtype,
                                               nve_stream_t stream);

/* The same GEMVs with the RMSNorm of the input fused into the kernel prologue: h is the un-normalised
 * 16-bit hidden state (act_dtype f16/bf16), norm_weight its RMSNorm weight.  Every CTA recomputes the norm
 * in the library's fixed order, rounds to 16 bits and then quantises (W4A8) or stages (W4A16) exactly as the
 * separate kernels do, so results are bit-identical to nve_b200_rmsnorm_quantize_q8 / nve_b200_rms_norm
 * followed by the plain GEMV (src/gpu_layer.rs:1032-1038 + :656-672 in one launch). */
NVE_API int nve_b200_rmsnorm_matvec_w4a8_multi(const void* h, const void* norm_weight, float eps, int act_dtype,
                                               const nve_b200_w4_matrix* mats, int num_mats, int K, int out_dtype,
                                               nve_stream_t stream);
NVE_API int nve_b200_rmsnorm_matvec_w4a16_multi(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                const float* awq, const nve_b200_w4_matrix* mats, int num_mats, int K,
                                                int out_dtype, nve_stream_t stream);
/* nve_b200_rmsnorm_matvec_w4a8_multi with the AWQ multiplier folded into the quantiser (the normalised, 16-bit
 * rounded value times awq_inv[k] is what gets quantised, as nve_b200_quantize_q8_awq does). */
NVE_API int nve_b200_rmsnorm_matvec_w4a8_awq_multi(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                   const float* awq_inv, const nve_b200_w4_matrix* mats, int num_mats,
                                                   int K, int out_dtype, nve_stream_t stream);

/* RMSNorm + gate/up GEMV + SiLU*up in ONE launch (src/gpu_layer.rs:937-945 / :977-980 and the RMSNorm in front of
 * them): a warp item holds gate row i and up row i, so the epilogue writes mid[i] = 16-bit(silu(16-bit gate_i) *
 * 16-bit up_i) -- the bits of the GEMV with 16-bit outputs followed by nve_silu_mul_f16 -- and the gate / up vectors
 * never reach memory.  gate->N == up->N (a multiple of 8); the `out` / `residual` members of the two matrices are
 * ignored; mid_out [N] has the activation type.  awq_inv / awq may be NULL (see nve_b200_quantize_q8_awq for the
 * W4A8 form). */
NVE_API int nve_b200_rmsnorm_gateup_silu_w4a8(const void* h, const void* norm_weight, float eps, int act_dtype,
                                              const float* awq_inv, const nve_b200_w4_matrix* gate,
                                              const nve_b200_w4_matrix* up, void* mid_out, int K, nve_stream_t stream);
NVE_API int nve_b200_rmsnorm_gateup_silu_w4a16(const void* h, const void* norm_weight, float eps, int act_dtype,
                                               const float* awq, const nve_b200_w4_matrix* gate,
                                               const nve_b200_w4_matrix* up, void* mid_out, int K, nve_stream_t stream);
/* The same launch, which in addition leaves mid converted for the down projection, so that neither a SiLU*up
 * kernel nor a quantiser runs between the gate/up and the down GEMV (src/gpu_layer.rs:937-947 in two launches):
 *   _q8_w4a8:   mid_q [N] int8 codes + mid_scales [N/32], the bits of nve_quantize_f16_q8 on mid;
 *   _x16_w4a16: the 16-bit fixed-point planes mid_lo / mid_hi [N] + mid_scales [N/32] that
 *               nve_b200_matvec_w4a16_planes_multi reads (down_awq, optional, multiplies mid first, as the W4A16
 *               GEMV's own staging does).
 * A CTA writes a contiguous range of mid; the CTA whose store completes a 32-wide group converts that group
 * (group_counters [N/32] u32 count the values written per group: zero them once, every launch adds 32 to each; a
 * buffer belongs to one mid vector and to launches that are ordered on one stream).  N % 32 == 0; mid_out 16-byte,
 * mid_q / mid_lo / mid_hi 8-byte aligned. */
NVE_API int nve_b200_rmsnorm_gateup_silu_q8_w4a8(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                 const float* awq_inv, const nve_b200_w4_matrix* gate,
                                                 const nve_b200_w4_matrix* up, void* mid_out, int K, int8_t* mid_q,
                                                 float* mid_scales, unsigned* group_counters, nve_stream_t stream);
NVE_API int nve_b200_rmsnorm_gateup_silu_x16_w4a16(const void* h, const void* norm_weight, float eps, int act_dtype,
                                                   const float* awq, const nve_b200_w4_matrix* gate,
                                                   const nve_b200_w4_matrix* up, void* mid_out, int K, uint8_t* mid_lo,
                                                   int8_t* mid_hi, float* mid_scales, const float* down_awq,
                                                   unsigned* group_counters, nve_stream_t stream);
/* W4A8 GEMV whose int8 activation codes are produced in the kernel prologue from a 16-bit vector x (every CTA runs
 * the arithmetic of nve_b200_quantize_q8 / _awq on it): nve_quantize_f16_q8 + nve_matvec_w4a8
 * (src/gpu_layer.rs:946-947) in one launch, bit-identical to the two.  Output type = x_dtype; residual as in
 * nve_b200_matvec_w4a8_multi.  The _allreduce form is the tensor-parallel one (see below). */
NVE_API int nve_b200_quantize_matvec_w4a8_multi(const void* x, int x_dtype, const float* awq_inv,
                                                const nve_b200_w4_matrix* mats, int num_mats, int K, nve_stream_t stream);
NVE_API int nve_b200_quantize_matvec_w4a8_allreduce(const void* x, int x_dtype, const float* awq_inv,
                                                    const nve_b200_w4_matrix* mat, int K, nve_stream_t stream);

/* RoPE of q and the new k at position *d_pos, the KV-cache write of the new row and single-query GQA
 * attention over the first *d_seq_len positions, in one launch (src/gpu_layer.rs:697-735 /
 * src/decode_graph.rs:247-283).  q [nh,hd] and k_new/v_new [nkv,hd] are read, not modified; caches are
 * [nkv, max_seq_len, hd]; tables [max_seq_len, hd/2]; out [nh,hd] f16.  When out_q / out_scales are given
 * the output is also quantised to int8 per group of 32 (the call at src/gpu_layer.rs:739).  head_dim 64 or
 * 128.  Results -- cache row, output and int8 codes -- are bit-identical to the separate RoPE, KV-write,
 * flash-decode and quantise launches of this library.
 * Two attention kernels exist and nve_flash_decode_f16 / _dyn, nve_b200_attn_prefill_causal (small blocks) and this
 * entry point always run the same one: by default a tensor-core kernel (a cluster of 8 CTAs per KV head, all its
 * query heads as rows of mma.sync, f16 probabilities) when there are 1, 2, 4 or 8 query heads per KV head and the
 * pointers are 16-byte aligned; nve_b200_set_attn_decode_kernel(1) selects the CUDA-core kernel for all of them
 * (also used for other shapes; it is the arithmetic of the persistent one-kernel step), 0 restores the default.  The
 * two kernels agree within 5e-3 of the largest output.  The setting is process-wide, a captured graph keeps the
 * kernel it was recorded with; the previous setting is returned. */
NVE_API int nve_b200_attn_decode_fused(const uint16_t* q, const uint16_t* k_new, const uint16_t* v_new,
                                       uint16_t* k_cache, uint16_t* v_cache, const uint16_t* cos_tab,
                                       const uint16_t* sin_tab, const int* d_pos, const int* d_seq_len, uint16_t* out,
                                       int8_t* out_q, float* out_scales, int num_heads, int num_kv_heads,
                                       int head_dim, int max_seq_len, float scale, nve_stream_t stream);
NVE_API int nve_b200_set_attn_decode_kernel(int mode);
/* The same launch for `batch` independent sequences (batched decode; the reference has none): row b of q
 * [batch, nh*hd] and of k_new / v_new [batch, nkv*hd] belongs to sequence b, whose caches are k_cache / v_cache +
 * b * nkv * max_seq_len * hd, whose position is d_pos[b] and whose valid length is d_seq_len[b] (device arrays).
 * The cache row written is bit-identical to a single-sequence call.  Up to 63 (sequence, KV head) units the clustered
 * decode kernel that nve_b200_attn_decode_fused would launch (see nve_b200_set_attn_decode_kernel) runs with the
 * sequence as second grid dimension and row b of out [batch, nh*hd] is bit-identical too;
 * from 64 units on (and 1, 2, 4 or 8 query heads per KV head) one CTA per unit streams all positions and computes
 * q.K^T and p.V with mma.sync (probabilities rounded to f16): rows then agree with the single-sequence call to about
 * 1e-3 of their RMS.  q / k_new / v_new and the caches 16-byte aligned. */
NVE_API int nve_b200_attn_decode_fused_batch(const uint16_t* q, const uint16_t* k_new, const uint16_t* v_new,
                                             uint16_t* k_cache, uint16_t* v_cache, const uint16_t* cos_tab,
                                             const uint16_t* sin_tab, const int* d_pos, const int* d_seq_len,
                                             uint16_t* out, int batch, int num_heads, int num_kv_heads, int head_dim,
                                             int max_seq_len, float scale, nve_stream_t stream);

/* Exact per-block integer dot products I[N, K/32] (int32) of the W4A8 GEMV, for bit-level checks. */
NVE_API int nve_b200_w4a8_idot(const int8_t* xq, const uint8_t* nibbles, int32_t* I, int N, int K, nve_stream_t stream);

/* Dequantisation with selectable 16-bit output type (cuda/nve_kernels.cu:397-433 arithmetic). */
NVE_API int nve_b200_dequant_w4a16(const uint8_t* nibbles, const float* scales, const float* awq, void* out, int N,
                           int K, int out_dtype, nve_stream_t stream);

/* On-device weight preparation, bit-identical to src/quantize.rs:711-731 (quantize_block_q4) followed by
 * src/quantize.rs:437-463 (extract_for_gpu): W [N,K] f32 row-major -> nibbles, scales.  awq_scales
 * (may be NULL) multiplies each column before quantisation as src/quantize.rs:283-286 does. */
NVE_API int nve_b200_q4_quantize(const float* W, const float* awq_scales, uint8_t* nibbles, float* scales, int N, int K,
                         nve_stream_t stream);

/* Repack reference CPU blocks (20 bytes: f32 scale + 16 bytes of {2i, 2i+1} pairs) already copied to the
 * device into the device layout (src/quantize.rs:437-463). */
NVE_API int nve_b200_q4_repack_blocks(const uint8_t* cpu_blocks, uint8_t* nibbles, float* scales, int N, int K,
                              nve_stream_t stream);

/* Counter-based synthetic generator: out[i] = normal(seed, stream_id, first+i) * scale (f32), the same
 * integer recipe as the test oracle so host and device inputs agree bit for bit. */
NVE_API int nve_b200_fill_normal(float* out, long long n, unsigned long long seed, unsigned long long stream_id,
                         unsigned long long first, float scale, nve_stream_t stream);
/* Same values rounded to a 16-bit type. */
NVE_API int nve_b200_fill_normal_16(void* out, long long n, unsigned long long seed, unsigned long long stream_id,
                            unsigned long long first, float scale, int dtype, nve_stream_t stream);

/* Batched W4A16 GEMM for decode batches 1 < M <= 64 on the tensor cores: Y[M,N] = X[M,K] . W^T with the packed
 * weights read once and dequantised on the fly (replaces nve_dequant_w4a16 + dense GEMM,
 * src/gpu_layer.rs:220-239).  Above 8 rows the weights go to tensor memory and tcgen05.mma; up to 8 rows a kernel
 * that keeps them in registers and issues mma.sync is faster and is used instead (same arguments, same work split
 * and workspace, results equal up to the order of the f32 additions).  The environment variable
 * NVE_B200_GEMM_KERNEL = tc | mma, read at the first call, forces one kernel (mma: M <= 32 only).
 * X and Y are row-major; x_dtype f16 or bf16, y_dtype = x_dtype or f32; K % 64 == 0; X and nibbles 16-byte aligned,
 * scales 8-byte aligned.  Weights are rounded to f16 as (q-8)*scale like the reference's dequantisation;
 * accumulation is f32.
 * `scratch` (may be NULL for f16 activations) holds, in this order, an f16 copy of bf16 activations (exact up to
 * +-65504, saturating beyond) and f32 partial tiles: with a workspace the (tile, 256-weight K slice) units are dealt
 * to the SMs in equal contiguous runs, so that few tiles still fill all SMs and a tile count that is not a multiple
 * of the SM count is balanced; tiles that several CTAs share are summed in ascending K order by a second kernel
 * (reproducible for a given SM count).  Its size comes from nve_b200_gemm_w4a16_scratch_bytes.  bf16 activations
 * without enough scratch for their copy are refused with NVE_ERR_TOO_LARGE; a scratch too small for the partial
 * tiles only lengthens the runs (fewer CTAs), down to one whole tile per CTA, which needs none.
 * nve_b200_gemm_error returns the code latched by an expired bounded wait. */
NVE_API size_t nve_b200_gemm_w4a16_scratch_bytes(int M, int N, int K);
NVE_API int nve_b200_gemm_w4a16(const void* X, int x_dtype, const uint8_t* nibbles, const float* scales, void* Y,
                                int y_dtype, int M, int N, int K, void* scratch, size_t scratch_bytes,
                                nve_stream_t stream);
/* The same GEMM over 1..3 matrices that share X (q/k/v, gate/up) in one launch: mats[i].{nibbles, scales, out, N},
 * out [M, N_i] row-major, residual must be NULL.  Their 128-row tiles follow one another in one unit sequence and the
 * runs are chosen for the total, which is what lets the narrow k and v projections fill the GPU. */
NVE_API size_t nve_b200_gemm_w4a16_multi_scratch_bytes(int M, const int* Ns, int num_mats, int K);
NVE_API int nve_b200_gemm_w4a16_multi(const void* X, int x_dtype, const nve_b200_w4_matrix* mats, int num_mats,
                                      int y_dtype, int M, int K, void* scratch, size_t scratch_bytes,
                                      nve_stream_t stream);
NVE_API int nve_b200_gemm_error(int reset);

/* Allocation-free form of nve_b200_gemm_w4a16.  No counterpart in the reference: it exists for callers that have
 * no workspace to pass and may not allocate one -- the reference's batch > 1 call site (GpuWeight::matmul_x,
 * src/gpu_layer.rs:220-239) only receives activations and weights and can run under CUDA-graph capture, where
 * cudaMalloc is illegal; a latency-critical serving thread is in the same position.  The partial tiles go
 * to a fixed 4 MiB array inside the library image (held on every GPU that loads the library until the process
 * exits) instead of a caller buffer.  Same arguments and results as nve_b200_gemm_w4a16 otherwise.
 *   - A shape whose workspace (partial tiles, plus the f16 copy of bf16 activations) exceeds 4 MiB is
 *     refused: NVE_ERR_TOO_LARGE.
 *   - The first call on each device resolves the array's device address and caches it; make that call before
 *     any stream capture begins.
 *   - All calls share the array and it keeps the previous call's contents (nothing in it needs to start at
 *     zero); two of these GEMMs running concurrently on one GPU race on it -- keep them on one stream.
 *   - The work split is the one the workspace form would choose; it is not changed to make a shape fit, so e.g.
 *     the 8B down projection at M = 64 (138 CTAs x 2 partial tiles x 64 x 128 floats = 9 MB) is refused although
 *     longer runs would fit: use the workspace form there.
 *   - The cached address belongs to the device's current context: after cudaDeviceReset the library must be
 *     reloaded before this entry point is used again on that device. */
NVE_API int nve_b200_gemm_w4a16_noalloc(const void* X, int x_dtype, const uint8_t* nibbles, const float* scales, void* Y,
                                        int y_dtype, int M, int N, int K, nve_stream_t stream);

/* ---- whole decode step in one persistent kernel ------------------------------------------------------------
 * nve_b200_decode_step runs one token through every layer of a Llama-style W4 stack in ONE cooperative launch:
 * per layer RMSNorm -> q/k/v GEMV -> RoPE + KV write + attention -> o_proj + residual -> RMSNorm -> gate/up GEMV ->
 * SiLU*up -> down GEMV + residual, i.e. the kernel sequence of src/decode_graph.rs:206-343 (and of
 * src/gpu_layer.rs:633-997 with the W4A8 route of :1017-1025 chosen per layer by use_w4a8), optionally followed
 * by the final RMSNorm and the lm_head GEMV that the reference computes on the host (src/paged_model.rs:1424-1433).
 * The hidden state it leaves is bit-identical to the fused six-launch-per-layer sequence of this library.
 *
 *   - `layers_dev` is a DEVICE array of model->num_layers descriptors (the caller copies it there once); all
 *     pointers inside are device addresses.  Weights in the library's W4 format; norm weights f16 [hidden];
 *     caches f16 [num_kv_heads, max_seq, head_dim]; rope tables f16 [max_seq, head_dim/2].
 *   - awq[i] (may be NULL) multiplies the activations of the W4A16 route in front of q/k/v (0), o_proj (1),
 *     gate/up (2) and down_proj (3), as nve_matvec_w4a16's awq argument does.
 *   - `hidden` [hidden] f16 is updated in place; *d_pos / *d_seq_len as for nve_b200_attn_decode_fused.
 *   - `workspace`: nve_b200_decode_step_workspace_bytes(model) bytes, 256-byte aligned, zeroed once with
 *     nve_b200_decode_step_init; one workspace serves one stream of steps (steps sharing it must not overlap).
 *   - head_dim 64 or 128, an even number of query heads per KV head, hidden / ffn multiples of 32, every
 *     projection's row count a multiple of 8, hidden and num_heads*head_dim <= 8192.
 *   - The launch is cooperative (one 512-thread CTA per SM must be co-resident; otherwise NVE_ERR_CUDA and nothing
 *     runs).  Every device-wide wait inside is bounded (100 ms): if one expires the kernel finishes with an
 *     undefined hidden state and nve_b200_decode_step_error returns NVE_ERR_TIMEOUT until reset.
 *   - With lm_nibbles != NULL the kernel ends with logits[vocab] (f32) = lm_head . RMSNorm(hidden, final_norm).
 */
typedef struct {
    const uint8_t* nibbles[7]; /* q, k, v, o, gate, up, down */
    const float* scales[7];
    const float* awq[4];
    const uint16_t* input_norm;
    const uint16_t* post_attn_norm;
    uint16_t* k_cache;
    uint16_t* v_cache;
    int use_w4a8; /* 1: int8 activations (W4A8), 0: 16-bit activations (W4A16) */
    int reserved;
} nve_b200_decode_layer;

typedef struct {
    int hidden, ffn, num_heads, num_kv_heads, head_dim, max_seq, num_layers;
    float norm_eps, attn_scale;
    const uint16_t* rope_cos;
    const uint16_t* rope_sin;
    /* optional head (all NULL / 0 when unused) */
    const uint16_t* final_norm;
    const uint8_t* lm_nibbles; /* [vocab, hidden/2] */
    const float* lm_scales;    /* [vocab, hidden/32] */
    float* logits;             /* [vocab] f32 */
    int vocab;
    int lm_use_w4a8;
} nve_b200_decode_model;

NVE_API size_t nve_b200_decode_step_workspace_bytes(const nve_b200_decode_model* model);
NVE_API int nve_b200_decode_step_init(void* workspace, size_t workspace_bytes, nve_stream_t stream);
NVE_API int nve_b200_decode_step(const nve_b200_decode_model* model, const nve_b200_decode_layer* layers_dev, void* hidden,
                                 const int* d_pos, const int* d_seq_len, void* workspace, size_t workspace_bytes,
                                 nve_stream_t stream);
/* Synchronous: the latched error word of the workspace (0 = none); reset != 0 clears it and the barrier state. */
NVE_API int nve_b200_decode_step_error(void* workspace, int reset);
/* Run-ahead distance of the kernel's L2 prefetch walk, in weight items (5 KB) per warp (0 disables it, at most 64);
 * returns the previous value; a negative argument only queries. */
NVE_API int nve_b200_decode_step_set_prefetch(int items);
/* Debugging aid: when `buf` (device memory, 2 * phases * 4 u64; phases = 7 per layer + 1 with an lm_head) is set,
 * CTA 0 and the last CTA record nanosecond timestamps per phase: phase entry, barrier passed, activations staged,
 * phase done.  NULL (the default) switches it off. */
NVE_API void nve_b200_decode_step_set_trace(unsigned long long* buf);
/* Test hook for the bounded wait: a one-CTA kernel waits (at most wait_ns <= 100 ms) at the workspace's barrier
 * for an arrival that never comes; afterwards nve_b200_decode_step_error reports NVE_ERR_TIMEOUT.  Reset the
 * workspace (nve_b200_decode_step_error(ws, 1)) before using it for a step again. */
NVE_API int nve_b200_decode_step_wait_probe(void* workspace, unsigned long long wait_ns, nve_stream_t stream);

/* ---- tensor parallel (no counterpart in the reference, which is single-GPU) -------------------------------
 * One process per GPU.  nve_b200_tp_create allocates this rank's symmetric buffer (partial sums for up to
 * max_rows output rows, per-CTA launch counters) and returns its 64-byte CUDA IPC handle; after the handles of
 * all ranks have been exchanged on the host, nve_b200_tp_connect(handles[world][64], rank order) maps the
 * peers.  The *_allreduce GEMVs then compute out = [residual +] sum over ranks of (W_shard . x_shard) for a
 * K-sharded (row-parallel) projection in ONE kernel: each CTA pushes its partial rows as {value, epoch} slots
 * into every rank's buffer with plain 8-byte peer stores, then polls (bounded) its own buffer until the slots
 * of its rows carry the current epoch and adds them in rank order, so every rank holds bit-identical results.
 * All ranks must issue the same sequence of *_allreduce calls (same N in the same order on every rank; N and K may
 * differ from call to call: every all-reduce launch uses the full grid, so the per-CTA launch counters that number
 * the epochs stay in step).  nve_b200_tp_error returns 0, or 1 + the rank whose slot a bounded wait (2^22 polls,
 * >= 0.14 s) gave up on; the affected rows are then set to NaN.  Check it once per step; an eager (non-graph) caller
 * should barrier the ranks after warm-up so that first-call module loading on one rank cannot outlast the wait.
 * nve_b200_tp_destroy frees the buffer that every peer has mapped: call it only when ALL ranks are idle (no
 * all-reduce kernel in flight anywhere) and have passed a host barrier; it closes the peer mappings first. */
NVE_API int nve_b200_tp_create(int rank, int world, int max_rows, void* handle_out);
NVE_API int nve_b200_tp_connect(const void* handles);
NVE_API int nve_b200_tp_world(void);
NVE_API int nve_b200_tp_error(int reset);
NVE_API int nve_b200_tp_destroy(void);
NVE_API int nve_b200_matvec_w4a8_allreduce(const int8_t* xq, const float* xq_scales, const nve_b200_w4_matrix* mat,
                                           int K, int out_dtype, nve_stream_t stream);
NVE_API int nve_b200_matvec_w4a16_allreduce(const void* x, int x_dtype, const float* awq,
                                            const nve_b200_w4_matrix* mat, int K, int out_dtype, nve_stream_t stream);
/* The W4A16 form fed with the fixed-point planes of nve_b200_silu_mul_x16 (this rank's K shard of them). */
NVE_API int nve_b200_matvec_w4a16_planes_allreduce(const uint8_t* x_lo, const int8_t* x_hi, const float* x_scales,
                                                   const nve_b200_w4_matrix* mat, int K, int out_dtype,
                                                   nve_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* NVE_KERNELS_H */
