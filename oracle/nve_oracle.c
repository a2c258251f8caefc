/*
 * CPU oracle for the NVE quantized decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference project's
 * (genovationtech/nve) quantized decode path so that the CUDA library can be
 * checked against it.  It is never linked into, imported by, or called from
 * the product path (the CUDA library and the nve_b200 package); only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may use it.
 *
 * Every function names the reference file:line whose arithmetic it follows.
 * Reference paths are relative to the reference project's root.
 *
 * Parity status of this oracle:
 *   - W4A16 / Q4 quantizer: pinned against the reference's own unit-test cases
 *     (src/quantize.rs:2234-2252, 2274-2289, 2522-2546) which are restated in
 *     the test suite, and cross-checked against an independent numpy
 *     restatement.
 *   - Activation quantizer and W4A8 integer GEMV: the reference has no test
 *     that pins them and its CPU code has no such path; the restatement follows
 *     the reference's CUDA source and is cross-checked on a B200 against that
 *     source compiled unmodified.
 *
 * Build: see the Makefile beside this file (gcc -O2 -fno-fast-math; the timed
 * baseline entry points additionally use pthreads and, when available, AVX2).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#define ORC_HAVE_AVX2 1
#else
#define ORC_HAVE_AVX2 0
#endif

#define Q4_BLOCK 32      /* src/quantize.rs:20 */
#define Q4_BLOCK_BYTES 20 /* src/quantize.rs:22 : f32 scale + 16 packed bytes */

/* ------------------------------------------------------------------------- */
/* 16-bit float helpers (exact widening, round-to-nearest-even narrowing)     */
/* ------------------------------------------------------------------------- */

static float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | ((absx > 0x7F800000u) ? 0x200u : 0u));
    }
    if (absx >= 0x477FF000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* < 2^-25 (or exactly 2^-25 -> ties to even 0) */
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7FFFFFu) | 0x800000u;
    uint32_t shift;
    uint32_t hexp;
    if (e < -14) { /* subnormal half */
        shift = (uint32_t)(13 + (-14 - e));
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(e + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    uint32_t out;
    if (hexp == 0) {
        out = q; /* may carry into exponent 1: correct */
    } else {
        out = ((hexp - 1) << 10) + q; /* q includes the implicit bit (0x400) */
    }
    return (uint16_t)(sign | out);
}

static float bf16_to_f32(uint16_t h) {
    uint32_t bits = (uint32_t)h << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t f32_to_bf16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
    uint32_t lsb = (x >> 16) & 1u;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

void orc_f16_to_f32(const uint16_t* in, float* out, long n) {
    for (long i = 0; i < n; i++) out[i] = f16_to_f32(in[i]);
}
void orc_f32_to_f16(const float* in, uint16_t* out, long n) {
    for (long i = 0; i < n; i++) out[i] = f32_to_f16(in[i]);
}
void orc_bf16_to_f32(const uint16_t* in, float* out, long n) {
    for (long i = 0; i < n; i++) out[i] = bf16_to_f32(in[i]);
}
void orc_f32_to_bf16(const float* in, uint16_t* out, long n) {
    for (long i = 0; i < n; i++) out[i] = f32_to_bf16(in[i]);
}

static float act16_to_f32(uint16_t v, int is_bf16) {
    return is_bf16 ? bf16_to_f32(v) : f16_to_f32(v);
}
static uint16_t f32_to_act16(float v, int is_bf16) {
    return is_bf16 ? f32_to_bf16(v) : f32_to_f16(v);
}

/* ------------------------------------------------------------------------- */
/* Counter-based synthetic input generator (shared definition with the CUDA   */
/* generator and the numpy one; integer arithmetic plus one f32 multiply, so  */
/* all three agree bit for bit).                                              */
/* ------------------------------------------------------------------------- */

static uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

#define ORC_GOLDEN 0x9E3779B97F4A7C15ull
#define ORC_STREAM_MUL 0xD6E8FEB86659FD93ull
/* 1 / sqrt(8 * (65536^2 - 1) / 12): unit variance for a sum of 8 uniform u16 */
#define ORC_IH8_SCALE 0x1.3988e2p-16f

static uint64_t orc_state(uint64_t seed, uint64_t stream) {
    return mix64(seed ^ (stream * ORC_STREAM_MUL));
}

static float orc_normal_at(uint64_t st, uint64_t i) {
    uint64_t a = mix64(st + (2 * i + 1) * ORC_GOLDEN);
    uint64_t b = mix64(st + (2 * i + 2) * ORC_GOLDEN);
    int32_t s = 0;
    for (int j = 0; j < 4; j++) {
        s += (int32_t)((a >> (16 * j)) & 0xFFFFu);
        s += (int32_t)((b >> (16 * j)) & 0xFFFFu);
    }
    return (float)(s - 262140) * ORC_IH8_SCALE;
}

static float orc_uniform_at(uint64_t st, uint64_t i) {
    uint64_t a = mix64(st + (2 * i + 1) * ORC_GOLDEN);
    return (float)(a >> 40) * 5.9604644775390625e-08f; /* 2^-24 */
}

/* out[i] = normal(seed, stream, first + i) * scale */
void orc_fill_normal(float* out, long n, uint64_t seed, uint64_t stream, uint64_t first, float scale) {
    uint64_t st = orc_state(seed, stream);
    for (long i = 0; i < n; i++) out[i] = orc_normal_at(st, first + (uint64_t)i) * scale;
}

void orc_fill_uniform(float* out, long n, uint64_t seed, uint64_t stream, uint64_t first) {
    uint64_t st = orc_state(seed, stream);
    for (long i = 0; i < n; i++) out[i] = orc_uniform_at(st, first + (uint64_t)i);
}

/* ------------------------------------------------------------------------- */
/* Q4 weight quantizer                                                        */
/* ------------------------------------------------------------------------- */

/* Rust `f32::round`: half away from zero.  `as i8`: saturating, NaN -> 0. */
static int sat_i8_round_away(float v) {
    if (v != v) return 0;
    float r = roundf(v);
    if (r >= 127.0f) return 127;
    if (r <= -128.0f) return -128;
    return (int)r;
}

/* src/quantize.rs:711-731 (quantize_block_q4): 32 f32 -> 20-byte CPU block. */
void orc_quantize_block_q4(const float* v, uint8_t* out) {
    float amax = 0.0f;
    for (int i = 0; i < Q4_BLOCK; i++) {
        float a = fabsf(v[i]);
        /* f32::max semantics: NaN operands are ignored */
        if (a > amax) amax = a;
    }
    float scale = amax > 0.0f ? amax / 7.0f : 0.0f;
    float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
    memcpy(out, &scale, 4);
    for (int i = 0; i < 16; i++) {
        int q0 = sat_i8_round_away(v[2 * i] * inv);
        int q1 = sat_i8_round_away(v[2 * i + 1] * inv);
        if (q0 < -8) q0 = -8;
        if (q0 > 7) q0 = 7;
        if (q1 < -8) q1 = -8;
        if (q1 > 7) q1 = 7;
        out[4 + i] = (uint8_t)((q0 + 8) | ((q1 + 8) << 4));
    }
}

/* src/quantize.rs:347-375 (from_f32): row-major [N,K] f32 -> N*K/32 CPU blocks.
 * awq_scales (may be NULL) follows src/quantize.rs:271-304 (from_compact_awq):
 * each row is multiplied column-wise by awq_scales before quantization. */
void orc_q4_from_f32(const float* W, long N, long K, const float* awq_scales, uint8_t* blocks) {
    long nb = K / Q4_BLOCK;
    float tmp[Q4_BLOCK];
    for (long n = 0; n < N; n++) {
        for (long b = 0; b < nb; b++) {
            const float* src = W + n * K + b * Q4_BLOCK;
            if (awq_scales) {
                for (int e = 0; e < Q4_BLOCK; e++) tmp[e] = src[e] * awq_scales[b * Q4_BLOCK + e];
                src = tmp;
            }
            orc_quantize_block_q4(src, blocks + (n * nb + b) * Q4_BLOCK_BYTES);
        }
    }
}

/* src/quantize.rs:298 : inverse AWQ scales handed to the GEMV. */
void orc_awq_inverse(const float* awq_scales, long K, float* inv) {
    for (long k = 0; k < K; k++) inv[k] = fabsf(awq_scales[k]) > 1e-10f ? 1.0f / awq_scales[k] : 0.0f;
}

/* src/quantize.rs:437-463 (extract_for_gpu): CPU blocks -> device arrays.
 * nibbles[n][16b+j] = e[j] | e[j+16] << 4 ; scales[n][b] copied verbatim. */
void orc_extract_for_gpu(const uint8_t* blocks, long N, long K, uint8_t* nibbles, float* scales) {
    long nb = K / Q4_BLOCK;
    for (long n = 0; n < N; n++) {
        for (long b = 0; b < nb; b++) {
            const uint8_t* blk = blocks + (n * nb + b) * Q4_BLOCK_BYTES;
            memcpy(&scales[n * nb + b], blk, 4);
            const uint8_t* cpu = blk + 4;
            uint8_t* dst = nibbles + (n * nb + b) * 16;
            for (int j = 0; j < 16; j++) {
                int h = j >> 1;
                uint8_t ej = (j & 1) ? (uint8_t)(cpu[h] >> 4) : (uint8_t)(cpu[h] & 0x0F);
                uint8_t ej16 = (j & 1) ? (uint8_t)(cpu[h + 8] >> 4) : (uint8_t)(cpu[h + 8] & 0x0F);
                dst[j] = (uint8_t)(ej | (ej16 << 4));
            }
        }
    }
}

/* Element e (0..31) of block (n,b) as the signed 4-bit value, from device arrays
 * (cuda/nve_kernels.cu:357-361: low nibble of byte e for e<16, high nibble of byte e-16 otherwise). */
static inline int gpu_q(const uint8_t* nibbles, long n, long nb, long b, int e) {
    uint8_t bv = nibbles[(n * nb + b) * 16 + (e & 15)];
    return (int)((e < 16) ? (bv & 0xF) : (bv >> 4)) - 8;
}

/* ------------------------------------------------------------------------- */
/* W4A16: CPU reference GEMV                                                  */
/* ------------------------------------------------------------------------- */

/* src/quantize.rs:853-879 (q4_dot_row_scalar). */
static float q4_dot_row_scalar(const uint8_t* row, const float* x, long nb) {
    float total = 0.0f;
    for (long b = 0; b < nb; b++) {
        const uint8_t* blk = row + b * Q4_BLOCK_BYTES;
        float scale;
        memcpy(&scale, blk, 4);
        const uint8_t* nib = blk + 4;
        const float* xb = x + b * Q4_BLOCK;
        float block_sum = 0.0f;
        for (int i = 0; i < 16; i++) {
            int q0 = (int)(nib[i] & 0x0F) - 8;
            int q1 = (int)(nib[i] >> 4) - 8;
            block_sum += (float)q0 * xb[2 * i];
            block_sum += (float)q1 * xb[2 * i + 1];
        }
        total += block_sum * scale;
    }
    return total;
}

/* src/quantize.rs:883-938 (q4_dot_row_avx2), restated lane by lane with fmaf so that
 * it reproduces the AVX2+FMA summation order on any host. */
static float q4_dot_row_avx2order(const uint8_t* row, const float* x, long nb) {
    float total[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (long b = 0; b < nb; b++) {
        const uint8_t* blk = row + b * Q4_BLOCK_BYTES;
        float scale;
        memcpy(&scale, blk, 4);
        const uint8_t* nib = blk + 4;
        const float* xb = x + b * Q4_BLOCK;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int g = 0; g < 4; g++) {
            for (int l = 0; l < 8; l++) {
                uint8_t byte = nib[g * 4 + (l >> 1)];
                int q = (int)((l & 1) ? (byte >> 4) : (byte & 0x0F)) - 8;
                acc[l] = fmaf((float)q, xb[g * 8 + l], acc[l]);
            }
        }
        for (int l = 0; l < 8; l++) total[l] = fmaf(acc[l], scale, total[l]);
    }
    /* horizontal sum: (lo128 + hi128), then movehl, then lane 0 + lane 1 */
    float s0 = total[0] + total[4], s1 = total[1] + total[5];
    float s2 = total[2] + total[6], s3 = total[3] + total[7];
    float t0 = s0 + s2, t1 = s1 + s3;
    return t0 + t1;
}

#if ORC_HAVE_AVX2
/* Same arithmetic as q4_dot_row_avx2order, with real AVX2 instructions (timed baseline). */
static float q4_dot_row_avx2(const uint8_t* row, const float* x, long nb) {
    __m256 total = _mm256_setzero_ps();
    const __m256i eight = _mm256_set1_epi32(8);
    const __m256i shifts = _mm256_set_epi32(28, 24, 20, 16, 12, 8, 4, 0);
    const __m256i mask = _mm256_set1_epi32(0xF);
    for (long b = 0; b < nb; b++) {
        const uint8_t* blk = row + b * Q4_BLOCK_BYTES;
        float scale;
        memcpy(&scale, blk, 4);
        __m256 acc = _mm256_setzero_ps();
        for (int g = 0; g < 4; g++) {
            uint32_t w;
            memcpy(&w, blk + 4 + g * 4, 4);
            __m256i v = _mm256_and_si256(_mm256_srlv_epi32(_mm256_set1_epi32((int)w), shifts), mask);
            __m256 f = _mm256_cvtepi32_ps(_mm256_sub_epi32(v, eight));
            acc = _mm256_fmadd_ps(f, _mm256_loadu_ps(x + b * Q4_BLOCK + g * 8), acc);
        }
        total = _mm256_fmadd_ps(acc, _mm256_set1_ps(scale), total);
    }
    __m128 hi = _mm256_extractf128_ps(total, 1);
    __m128 lo = _mm256_castps256_ps128(total);
    __m128 s = _mm_add_ps(lo, hi);
    __m128 s2 = _mm_add_ps(s, _mm_movehl_ps(s, s));
    __m128 s1 = _mm_add_ss(s2, _mm_shuffle_ps(s2, s2, 1));
    return _mm_cvtss_f32(s1);
}
#endif

int orc_have_avx2(void) { return ORC_HAVE_AVX2; }

/* src/quantize.rs:466-488 (matvec_f32) + :1107-1111 (apply_awq_inv_scales).
 * order: 0 = scalar path (:853-879), 1 = AVX2 summation order (:883-938). */
void orc_q4_matvec(const uint8_t* blocks, const float* x, long N, long K, const float* awq_inv, int order,
                   float* y) {
    long nb = K / Q4_BLOCK;
    float* xe = NULL;
    if (awq_inv) {
        xe = (float*)malloc(sizeof(float) * (size_t)K);
        for (long k = 0; k < K; k++) xe[k] = x[k] * awq_inv[k];
        x = xe;
    }
    for (long n = 0; n < N; n++) {
        const uint8_t* row = blocks + n * nb * Q4_BLOCK_BYTES;
        y[n] = order ? q4_dot_row_avx2order(row, x, nb) : q4_dot_row_scalar(row, x, nb);
    }
    free(xe);
}

/* src/quantize.rs:1057-1075 (q4_linear): one matvec per row of X [M,K] -> Y [M,N]. */
void orc_q4_linear(const uint8_t* blocks, const float* X, long M, long N, long K, const float* awq_inv, int order,
                   float* Y) {
    for (long m = 0; m < M; m++) orc_q4_matvec(blocks, X + m * K, N, K, awq_inv, order, Y + m * N);
}


/* ------------------------------------------------------------------------- */
/* Minimal parallel-for over rows for the timed baselines (pthreads).         */
/* ------------------------------------------------------------------------- */

typedef void (*orc_row_fn)(void* ctx, long n0, long n1);
static int g_orc_threads = 1;
void orc_set_threads(int n) { g_orc_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
int orc_get_threads(void) { return g_orc_threads; }

/* A persistent pool (the reference's rayon keeps its workers alive between calls too): workers sleep on a condition
 * variable until a new job generation is published; the caller runs slice 0 itself and waits for the others. */
static struct {
    pthread_mutex_t mu;
    pthread_cond_t go, done;
    pthread_t th[256];
    int workers;        /* threads created so far (worker w runs slice w + 1) */
    unsigned long gen;  /* job generation */
    int active;         /* slices of the current job that run on workers */
    int pending;        /* of those, still running */
    orc_row_fn fn;
    void* ctx;
    long N;
    int T;
    int ready;
} g_pool = {PTHREAD_MUTEX_INITIALIZER, PTHREAD_COND_INITIALIZER, PTHREAD_COND_INITIALIZER, {0}, 0, 0, 0, 0, 0, 0, 0, 0, 1};

static void* orc_pool_main(void* arg) {
    long w = (long)arg;
    unsigned long seen = 0;
    pthread_mutex_lock(&g_pool.mu);
    for (;;) {
        while (g_pool.gen == seen) pthread_cond_wait(&g_pool.go, &g_pool.mu);
        seen = g_pool.gen;
        if (w + 1 >= g_pool.T) continue; /* not part of this job */
        orc_row_fn fn = g_pool.fn;
        void* ctx = g_pool.ctx;
        long N = g_pool.N;
        int T = g_pool.T;
        pthread_mutex_unlock(&g_pool.mu);
        fn(ctx, N * (w + 1) / T, N * (w + 2) / T);
        pthread_mutex_lock(&g_pool.mu);
        if (--g_pool.pending == 0) pthread_cond_signal(&g_pool.done);
    }
    return NULL;
}

static void orc_parallel_rows(orc_row_fn fn, void* ctx, long N) {
    int T = g_orc_threads;
    if (T <= 1 || N < 32) { /* src/quantize.rs:473: serial below 32 rows */
        fn(ctx, 0, N);
        return;
    }
    pthread_mutex_lock(&g_pool.mu);
    while (g_pool.workers < T - 1) {
        long w = g_pool.workers;
        if (pthread_create(&g_pool.th[w], NULL, orc_pool_main, (void*)w) != 0) break;
        g_pool.workers++;
    }
    if (T > g_pool.workers + 1) T = g_pool.workers + 1;
    g_pool.fn = fn;
    g_pool.ctx = ctx;
    g_pool.N = N;
    g_pool.T = T;
    g_pool.pending = T - 1;
    g_pool.gen++;
    pthread_cond_broadcast(&g_pool.go);
    pthread_mutex_unlock(&g_pool.mu);
    fn(ctx, 0, N / T);
    pthread_mutex_lock(&g_pool.mu);
    while (g_pool.pending > 0) pthread_cond_wait(&g_pool.done, &g_pool.mu);
    pthread_mutex_unlock(&g_pool.mu);
}

/* Threaded form of matvec_f32 for the timed CPU baseline: rows in parallel as rayon does for
 * rows >= 32 (src/quantize.rs:473-487); AVX2 inner loop when the host has it (:844-851). */
typedef struct {
    const uint8_t* blocks;
    const float* x;
    long nb;
    float* y;
} orc_q4_ctx;

static void orc_q4_rows(void* p, long n0, long n1) {
    orc_q4_ctx* c = (orc_q4_ctx*)p;
    for (long n = n0; n < n1; n++) {
        const uint8_t* row = c->blocks + n * c->nb * Q4_BLOCK_BYTES;
#if ORC_HAVE_AVX2
        c->y[n] = q4_dot_row_avx2(row, c->x, c->nb);
#else
        c->y[n] = q4_dot_row_scalar(row, c->x, c->nb);
#endif
    }
}

void orc_q4_matvec_mt(const uint8_t* blocks, const float* x, long N, long K, float* y) {
    orc_q4_ctx c = {blocks, x, K / Q4_BLOCK, y};
    orc_parallel_rows(orc_q4_rows, &c, N);
}

/* High-precision W4A16 value from the device arrays: sum_b scale * sum_e q * x in f64. */
void orc_w4a16_matvec_f64(const float* x, const uint8_t* nibbles, const float* scales, const float* awq, long N,
                          long K, double* y) {
    long nb = K / Q4_BLOCK;
    for (long n = 0; n < N; n++) {
        double tot = 0.0;
        for (long b = 0; b < nb; b++) {
            double bs = 0.0;
            for (int e = 0; e < Q4_BLOCK; e++) {
                float xi = x[b * Q4_BLOCK + e];
                if (awq) xi = xi * awq[b * Q4_BLOCK + e];
                bs += (double)gpu_q(nibbles, n, nb, b, e) * (double)xi;
            }
            tot += bs * (double)scales[n * nb + b];
        }
        y[n] = tot;
    }
}

/* cuda/nve_kernels.cu:397-433 (nve_dequant_w4a16): W[n][k] = f16((q-8)*scale [*awq[k]]). */
void orc_dequant_w4a16(const uint8_t* nibbles, const float* scales, const float* awq, long N, long K, int is_bf16,
                       uint16_t* out) {
    long nb = K / Q4_BLOCK;
    for (long n = 0; n < N; n++)
        for (long k = 0; k < K; k++) {
            float v = (float)gpu_q(nibbles, n, nb, k / Q4_BLOCK, (int)(k % Q4_BLOCK)) * scales[n * nb + k / Q4_BLOCK];
            if (awq) v = v * awq[k];
            out[n * K + k] = f32_to_act16(v, is_bf16);
        }
}

/* ------------------------------------------------------------------------- */
/* Activation quantizer and W4A8                                              */
/* ------------------------------------------------------------------------- */

/* cuda/nve_kernels.cu:712-745 (_nve_quantize_f16_q8), IEEE arithmetic:
 * scale = amax > 0 ? amax/127 : 1 ; q = clamp(rint(x * (1/scale)), -127, 127). */
void orc_quantize_q8(const uint16_t* x16, long K, int is_bf16, int8_t* xq, float* scales) {
    for (long g = 0; g < K / 32; g++) {
        float amax = 0.0f;
        for (int e = 0; e < 32; e++) amax = fmaxf(amax, fabsf(act16_to_f32(x16[g * 32 + e], is_bf16)));
        float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        scales[g] = scale;
        float inv = 1.0f / scale;
        for (int e = 0; e < 32; e++) {
            float v = act16_to_f32(x16[g * 32 + e], is_bf16) * inv;
            long q = lrintf(v); /* round half to even under the default rounding mode */
            if (q < -127) q = -127;
            if (q > 127) q = 127;
            xq[g * 32 + e] = (int8_t)q;
        }
    }
}

/* The same quantiser for activations of an AWQ pre-scaled matrix: x[k] * awq_inv[k] (one f32 product, the multiply
 * the W4A16 kernels apply per element, cuda/nve_kernels.cu:354-355; awq_inv from src/quantize.rs:1107-1111) goes
 * through the arithmetic of orc_quantize_q8.  The reference has no such W4A8 path (src/gpu_layer.rs:659 drops the
 * multiplier): this restates the library's own extension. */
void orc_quantize_q8_awq(const uint16_t* x16, const float* awq_inv, long K, int is_bf16, int8_t* xq, float* scales) {
    for (long g = 0; g < K / 32; g++) {
        float v[32];
        float amax = 0.0f;
        for (int e = 0; e < 32; e++) {
            v[e] = act16_to_f32(x16[g * 32 + e], is_bf16) * awq_inv[g * 32 + e];
            amax = fmaxf(amax, fabsf(v[e]));
        }
        float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
        scales[g] = scale;
        float inv = 1.0f / scale;
        for (int e = 0; e < 32; e++) {
            long q = lrintf(v[e] * inv);
            if (q < -127) q = -127;
            if (q > 127) q = 127;
            xq[g * 32 + e] = (int8_t)q;
        }
    }
}

/* cuda/nve_kernels.cu:817-862: exact per-block integer dot I[n][b] = sum_e (q-8)*xq. */
void orc_w4a8_idot(const int8_t* xq, const uint8_t* nibbles, long N, long K, int32_t* I) {
    long nb = K / Q4_BLOCK;
    for (long n = 0; n < N; n++)
        for (long b = 0; b < nb; b++) {
            int32_t s = 0;
            for (int e = 0; e < Q4_BLOCK; e++) s += gpu_q(nibbles, n, nb, b, e) * (int32_t)xq[b * Q4_BLOCK + e];
            I[n * nb + b] = s;
        }
}

/* W4A8 output value in f64: sum_b wsc*xsc*I (cuda/nve_kernels.cu:864-867 with an exact sum). */
void orc_w4a8_matvec_f64(const int8_t* xq, const float* xs, const uint8_t* nibbles, const float* wsc, long N, long K,
                         double* y) {
    long nb = K / Q4_BLOCK;
    for (long n = 0; n < N; n++) {
        double tot = 0.0;
        for (long b = 0; b < nb; b++) {
            int32_t s = 0;
            for (int e = 0; e < Q4_BLOCK; e++) s += gpu_q(nibbles, n, nb, b, e) * (int32_t)xq[b * Q4_BLOCK + e];
            tot += (double)wsc[n * nb + b] * (double)xs[b] * (double)s;
        }
        y[n] = tot;
    }
}

/* cuda/nve_kernels.cu:796-878 in the reference kernel's own f32 summation order:
 * 128 threads per row, thread tid owns the half-block (kbx = tid/2 + 64*it, half = tid%2);
 * per half-block acc = fma(wsc*xsc, (float)I_half, acc) (nvcc's default mul-add contraction);
 * warps 1..3 are added onto warp 0 lane-wise in order, then a xor butterfly 16,8,4,2,1. */
void orc_w4a8_matvec_reforder(const int8_t* xq, const float* xs, const uint8_t* nibbles, const float* wsc, long N,
                              long K, float* y) {
    long nb = K / Q4_BLOCK;
    for (long n = 0; n < N; n++) {
        float acc[128];
        for (int tid = 0; tid < 128; tid++) {
            float a = 0.0f;
            int half = tid & 1;
            for (long kbx = tid / 2; kbx < nb; kbx += 64) {
                /* int32 #j of the block holds elems 4j..4j+3 (low) and 16+4j..16+4j+3 (high); half h owns j = 2h, 2h+1 */
                int32_t s = 0;
                for (int j = 2 * half; j < 2 * half + 2; j++)
                    for (int t = 0; t < 4; t++) {
                        s += gpu_q(nibbles, n, nb, kbx, 4 * j + t) * (int32_t)xq[kbx * 32 + 4 * j + t];
                        s += gpu_q(nibbles, n, nb, kbx, 16 + 4 * j + t) * (int32_t)xq[kbx * 32 + 16 + 4 * j + t];
                    }
                a = fmaf(wsc[n * nb + kbx] * xs[kbx], (float)s, a);
            }
            acc[tid] = a;
        }
        float lane[32];
        for (int l = 0; l < 32; l++) {
            float a = acc[l];
            a += acc[32 + l];
            a += acc[64 + l];
            a += acc[96 + l];
            lane[l] = a;
        }
        for (int m = 16; m > 0; m >>= 1) {
            float nxt[32];
            for (int l = 0; l < 32; l++) nxt[l] = lane[l] + lane[l ^ m];
            memcpy(lane, nxt, sizeof(lane));
        }
        y[n] = lane[0];
    }
}

/* Threaded W4A8 GEMV on the CPU for the timed baseline (same arithmetic as orc_w4a8_matvec_f64 but
 * an int8 inner loop and f32 accumulation, rows in parallel). */
typedef struct {
    const int8_t* xq;
    const float* xs;
    const uint8_t* nibbles;
    const float* wsc;
    long nb;
    float* y;
} orc_w4a8_ctx;

static void orc_w4a8_rows(void* p, long n0, long n1) {
    orc_w4a8_ctx* c = (orc_w4a8_ctx*)p;
    long nb = c->nb;
    for (long n = n0; n < n1; n++) {
        float tot = 0.0f;
        const uint8_t* rown = c->nibbles + n * nb * 16;
        for (long b = 0; b < nb; b++) {
            const uint8_t* q = rown + b * 16;
            const int8_t* xb = c->xq + b * 32;
            int32_t s = 0;
            for (int j = 0; j < 16; j++) {
                s += ((int)(q[j] & 0xF) - 8) * (int)xb[j];
                s += ((int)(q[j] >> 4) - 8) * (int)xb[j + 16];
            }
            tot += c->wsc[n * nb + b] * c->xs[b] * (float)s;
        }
        c->y[n] = tot;
    }
}

void orc_w4a8_matvec_mt(const int8_t* xq, const float* xs, const uint8_t* nibbles, const float* wsc, long N, long K,
                        float* y) {
    orc_w4a8_ctx c = {xq, xs, nibbles, wsc, K / Q4_BLOCK, y};
    orc_parallel_rows(orc_w4a8_rows, &c, N);
}

/* ------------------------------------------------------------------------- */
/* Restatement of the CUDA library's own f32 summation order (bit-level checks) */
/* ------------------------------------------------------------------------- */

/* The library's summation order for one row: a column set is 32 consecutive blocks, lane l owns block l of
 * it; per lane the column sets of a group of four are added in ascending order (first term exact); the 32
 * lane values of a group are added with a xor butterfly (pairs l^16, then ^8, ^4, ^2, ^1); the groups are
 * added in ascending order. */
static float lane_tree32(const float* v) {
    float a[32];
    memcpy(a, v, sizeof(a));
    for (int m = 16; m > 0; m >>= 1)
        for (int l = 0; l < m; l++) a[l] = a[l] + a[l + m];
    return a[0];
}

/* blockval(ctx, b) returns the f32 value of block b of the current row. */
typedef float (*orc_blockval_fn)(void* ctx, long b);

static float b200_row_sum(orc_blockval_fn fn, void* ctx, long nb) {
    long S = (nb + 31) / 32;
    float tot = 0.0f;
    for (long g0 = 0; g0 < S; g0 += 4) {
        float lane[32];
        for (int l = 0; l < 32; l++) {
            float a = 0.0f;
            for (long s = g0; s < g0 + 4 && s < S; s++) {
                long b = s * 32 + l;
                float v = b < nb ? fn(ctx, b) : 0.0f;
                a = (s == g0) ? v : a + v;
            }
            lane[l] = a;
        }
        float part = lane_tree32(lane);
        tot = (g0 == 0) ? part : tot + part;
    }
    return tot;
}

typedef struct {
    const int8_t* xq;
    const float* xs;
    const uint8_t* nibbles;
    const float* wsc;
    long n, nb;
} b200_w4a8_ctx;

static float b200_w4a8_block(void* p, long b) {
    b200_w4a8_ctx* c = (b200_w4a8_ctx*)p;
    int32_t I = 0;
    for (int e = 0; e < Q4_BLOCK; e++) I += gpu_q(c->nibbles, c->n, c->nb, b, e) * (int32_t)c->xq[b * Q4_BLOCK + e];
    return (c->wsc[c->n * c->nb + b] * c->xs[b]) * (float)I;
}

/* W4A8 GEMV with the library's order: v = (wsc*xs) * (float)I per block (two roundings), summed as above.
 * The integer part is cuda/nve_kernels.cu:817-862. */
void orc_w4a8_matvec_b200(const int8_t* xq, const float* xs, const uint8_t* nibbles, const float* wsc, long N, long K,
                          float* y) {
    b200_w4a8_ctx c = {xq, xs, nibbles, wsc, 0, K / Q4_BLOCK};
    for (long n = 0; n < N; n++) {
        c.n = n;
        y[n] = b200_row_sum(b200_w4a8_block, &c, c.nb);
    }
}

/* The library's W4A16 activation staging: per 32-wide block a 16-bit fixed-point code
 *   xe = f32(x) [* awq] ; amax = max|xe| ; scale = amax > 0 ? amax/32767 : 1 ; v = clamp(rint(xe * (1/scale)), +-32767). */
void orc_x16_fixedpoint(const uint16_t* x16, long K, int is_bf16, const float* awq, int32_t* v, float* scales) {
    for (long g = 0; g < K / 32; g++) {
        float xe[32];
        float amax = 0.0f;
        for (int e = 0; e < 32; e++) {
            xe[e] = act16_to_f32(x16[g * 32 + e], is_bf16);
            if (awq) xe[e] = xe[e] * awq[g * 32 + e];
            amax = fmaxf(amax, fabsf(xe[e]));
        }
        float scale = amax > 0.0f ? amax / 32767.0f : 1.0f;
        float inv = 1.0f / scale;
        scales[g] = scale;
        for (int e = 0; e < 32; e++) {
            long q = lrintf(xe[e] * inv);
            if (q < -32767) q = -32767;
            if (q > 32767) q = 32767;
            v[g * 32 + e] = (int32_t)q;
        }
    }
}

typedef struct {
    const int32_t* v16;
    const float* xs;
    const uint8_t* nibbles;
    const float* wsc;
    long n, nb;
} b200_w4a16_ctx;

static float b200_w4a16_block(void* p, long b) {
    b200_w4a16_ctx* c = (b200_w4a16_ctx*)p;
    int64_t I = 0;
    for (int e = 0; e < Q4_BLOCK; e++) I += (int64_t)gpu_q(c->nibbles, c->n, c->nb, b, e) * c->v16[b * Q4_BLOCK + e];
    return (c->wsc[c->n * c->nb + b] * c->xs[b]) * (float)(int32_t)I;
}

/* W4A16 GEMV as the library computes it: integer dot of (q-8) with the fixed-point codes, then the same
 * scaling and summation order as orc_w4a8_matvec_b200. */
void orc_w4a16_matvec_b200(const uint16_t* x16, int is_bf16, const float* awq, const uint8_t* nibbles,
                           const float* wsc, long N, long K, float* y) {
    long nb = K / Q4_BLOCK;
    int32_t* v16 = (int32_t*)malloc(sizeof(int32_t) * (size_t)K);
    float* xs = (float*)malloc(sizeof(float) * (size_t)nb);
    orc_x16_fixedpoint(x16, K, is_bf16, awq, v16, xs);
    b200_w4a16_ctx c = {v16, xs, nibbles, wsc, 0, nb};
    for (long n = 0; n < N; n++) {
        c.n = n;
        y[n] = b200_row_sum(b200_w4a16_block, &c, nb);
    }
    free(v16);
    free(xs);
}

/* ------------------------------------------------------------------------- */
/* Decode glue (norm, activation, RoPE, attention)                            */
/* ------------------------------------------------------------------------- */

/* src/ops.rs:12-30 (rms_norm): f64 accumulation, f32 result. */
void orc_rms_norm_f64(const float* x, const float* w, long n, double eps, float* out) {
    double ss = 0.0;
    for (long i = 0; i < n; i++) ss += (double)x[i] * (double)x[i];
    double inv = 1.0 / sqrt(ss / (double)n + eps);
    for (long i = 0; i < n; i++) out[i] = (float)((double)x[i] * inv * (double)w[i]);
}

/* cuda/nve_kernels.cu:26-60 with a fixed f32 summation order -- the order the CUDA library under test
 * uses for its norm kernels, restated here so that the 16-bit result can be compared bit for bit:
 *   256 threads; thread t adds x[i]^2 (fma chain, ascending i) over the 8-element chunks t, t+256, ...;
 *   per 32-lane group a xor butterfly 16,8,4,2,1; the 8 group sums are added in ascending order;
 *   r = 1 / sqrt(sum / n + eps) with IEEE sqrt and divide;
 *   out[i] = round16((x[i] * r) * w[i]). */
void orc_rms_norm_16(const uint16_t* x16, const uint16_t* w16, long n, float eps, int is_bf16, uint16_t* out16) {
    float p[256];
    long chunks = (n + 7) / 8;
    for (int t = 0; t < 256; t++) {
        float a = 0.0f;
        for (long c = t; c < chunks; c += 256) {
            for (int e = 0; e < 8; e++) {
                long i = c * 8 + e;
                float v = i < n ? act16_to_f32(x16[i], is_bf16) : 0.0f;
                a = fmaf(v, v, a);
            }
        }
        p[t] = a;
    }
    float total = 0.0f;
    for (int w = 0; w < 8; w++) {
        float lane[32];
        memcpy(lane, p + 32 * w, sizeof(lane));
        for (int m = 16; m > 0; m >>= 1) {
            float nxt[32];
            for (int l = 0; l < 32; l++) nxt[l] = lane[l] + lane[l ^ m];
            memcpy(lane, nxt, sizeof(lane));
        }
        total = (w == 0) ? lane[0] : total + lane[0];
    }
    float r = 1.0f / sqrtf(total / (float)n + eps);
    for (long i = 0; i < n; i++) {
        float v = act16_to_f32(x16[i], is_bf16) * r;
        v = v * act16_to_f32(w16[i], is_bf16);
        out16[i] = f32_to_act16(v, is_bf16);
    }
}

/* src/ops.rs:60-64 (silu) and src/generic_model.rs:765-768 (silu(g) * u), on 16-bit inputs with one
 * rounding of the product as cuda/nve_kernels.cu:978-995 does. */
void orc_silu_mul_16(const uint16_t* g16, const uint16_t* u16, long n, int is_bf16, uint16_t* out16) {
    for (long i = 0; i < n; i++) {
        float g = act16_to_f32(g16[i], is_bf16);
        float u = act16_to_f32(u16[i], is_bf16);
        float v = g / (1.0f + expf(-g)) * u;
        out16[i] = f32_to_act16(v, is_bf16);
    }
}

/* src/main.rs:1456-1470 (bench-random RoPE tables): f32 freqs 1/theta^(2i/hd), angle = pos*freq in f32. */
void orc_rope_tables_f32(int head_dim, int max_seq, float theta, float* cos_t, float* sin_t) {
    int half = head_dim / 2;
    for (int pos = 0; pos < max_seq; pos++)
        for (int i = 0; i < half; i++) {
            float freq = 1.0f / powf(theta, 2.0f * (float)i / (float)head_dim);
            float ang = (float)pos * freq;
            cos_t[pos * half + i] = cosf(ang);
            sin_t[pos * half + i] = sinf(ang);
        }
}

/* src/ops.rs:228-250 (RopeFreqs::apply), half-split pairs (i, i+hd/2), on f32 vectors. */
void orc_rope_apply(float* v, int n_heads, int head_dim, const float* cos_row, const float* sin_row) {
    int half = head_dim / 2;
    for (int h = 0; h < n_heads; h++) {
        float* p = v + (long)h * head_dim;
        for (int i = 0; i < half; i++) {
            float a = p[i], b = p[i + half];
            p[i] = a * cos_row[i] - b * sin_row[i];
            p[i + half] = a * sin_row[i] + b * cos_row[i];
        }
    }
}

/* src/attention.rs:199-224: single-query GQA attention over a cache [nkv, stride, hd] (f32),
 * scores = q.k * scale, softmax with max subtraction (src/ops.rs softmax), weighted V sum. */
void orc_attn_decode(const float* q, const float* kc, const float* vc, int nh, int nkv, int seq_len, int stride,
                     int hd, float scale, float* out) {
    int groups = nh / nkv;
    double* sc = (double*)malloc(sizeof(double) * (size_t)(seq_len > 0 ? seq_len : 1));
    for (int h = 0; h < nh; h++) {
        int kvh = h / groups;
        const float* qh = q + (long)h * hd;
        double mx = -1e300;
        for (int t = 0; t < seq_len; t++) {
            const float* kt = kc + ((long)kvh * stride + t) * hd;
            double d = 0.0;
            for (int i = 0; i < hd; i++) d += (double)qh[i] * (double)kt[i];
            sc[t] = d * (double)scale;
            if (sc[t] > mx) mx = sc[t];
        }
        double sum = 0.0;
        for (int t = 0; t < seq_len; t++) {
            sc[t] = exp(sc[t] - mx);
            sum += sc[t];
        }
        for (int i = 0; i < hd; i++) {
            double a = 0.0;
            for (int t = 0; t < seq_len; t++) a += sc[t] * (double)vc[((long)kvh * stride + t) * hd + i];
            out[(long)h * hd + i] = (float)(sum > 0.0 ? a / sum : 0.0);
        }
    }
    free(sc);
}

/* src/tensor.rs:932-953: f32 dot with the AVX2+FMA form the reference dispatches to on x86-64 (32 floats per
 * iteration in four accumulators), scalar 8-way unrolled otherwise (:955-985). */
static float orc_dot_f32(const float* a, const float* b, int n) {
    int i = 0;
    float sum = 0.0f;
#if ORC_HAVE_AVX2
    if (n >= 32) {
        __m256 s0 = _mm256_setzero_ps(), s1 = s0, s2 = s0, s3 = s0;
        for (; i + 32 <= n; i += 32) {
            s0 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i), _mm256_loadu_ps(b + i), s0);
            s1 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 8), _mm256_loadu_ps(b + i + 8), s1);
            s2 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 16), _mm256_loadu_ps(b + i + 16), s2);
            s3 = _mm256_fmadd_ps(_mm256_loadu_ps(a + i + 24), _mm256_loadu_ps(b + i + 24), s3);
        }
        __m256 t = _mm256_add_ps(_mm256_add_ps(s0, s1), _mm256_add_ps(s2, s3));
        float lanes[8];
        _mm256_storeu_ps(lanes, t);
        sum = ((lanes[0] + lanes[1]) + (lanes[2] + lanes[3])) + ((lanes[4] + lanes[5]) + (lanes[6] + lanes[7]));
    }
#endif
    for (; i < n; i++) sum += a[i] * b[i];
    return sum;
}

/* src/attention.rs:199-224 with the reference's own types and loop order (f32 dot, f32 softmax with max
 * subtraction as src/ops.rs:152-163, t-outer / d-inner weighted V sum, one head after the other on one thread):
 * the form timed by the CPU baseline.  orc_attn_decode above accumulates in f64 and is the one parity checks use. */
void orc_attn_decode_f32(const float* q, const float* kc, const float* vc, int nh, int nkv, int seq_len, int stride,
                         int hd, float scale, float* out) {
    int groups = nh / nkv;
    float* sc = (float*)malloc(sizeof(float) * (size_t)(seq_len > 0 ? seq_len : 1));
    for (int h = 0; h < nh; h++) {
        int kvh = h / groups;
        const float* qh = q + (long)h * hd;
        float mx = -INFINITY;
        for (int t = 0; t < seq_len; t++) {
            sc[t] = orc_dot_f32(qh, kc + ((long)kvh * stride + t) * hd, hd) * scale;
            if (sc[t] > mx) mx = sc[t];
        }
        float sum = 0.0f;
        for (int t = 0; t < seq_len; t++) {
            sc[t] = expf(sc[t] - mx);
            sum += sc[t];
        }
        float inv = 1.0f / sum;
        for (int t = 0; t < seq_len; t++) sc[t] *= inv;
        float* oh = out + (long)h * hd;
        for (int i = 0; i < hd; i++) oh[i] = 0.0f;
        for (int t = 0; t < seq_len; t++) {
            const float* vt = vc + ((long)kvh * stride + t) * hd;
            const float w = sc[t];
            int i = 0;
#if ORC_HAVE_AVX2
            const __m256 wv = _mm256_set1_ps(w);
            for (; i + 8 <= hd; i += 8)
                _mm256_storeu_ps(oh + i, _mm256_add_ps(_mm256_loadu_ps(oh + i), _mm256_mul_ps(wv, _mm256_loadu_ps(vt + i))));
#endif
            for (; i < hd; i++) oh[i] += w * vt[i];
        }
    }
    free(sc);
}

/* ------------------------------------------------------------------------- */
/* Routing                                                                    */
/* ------------------------------------------------------------------------- */

/* src/main.rs:891-898: min-max normalisation of raw scores (all 0.5 when the range is <= 1e-9). */
void orc_normalize_importance(const double* scores, int n, double* out) {
    double mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < n; i++) {
        if (scores[i] < mn) mn = scores[i];
        if (scores[i] > mx) mx = scores[i];
    }
    double range = mx - mn;
    for (int i = 0; i < n; i++) out[i] = range > 1e-9 ? (scores[i] - mn) / range : 0.5;
}

/* src/gpu_layer.rs:1017-1025: use_w4a8 = !no_w4a8 && importance < threshold. */
int orc_use_w4a8(double importance, double threshold, int no_w4a8) {
    if (no_w4a8) return 0;
    return importance < threshold ? 1 : 0;
}
