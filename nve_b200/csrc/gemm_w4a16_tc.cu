// Batched W4A16 GEMM on the 5th-generation tensor cores:  Y[M,N] = X[M,K] . W^T,  M = decode batch (<= 64).
//
// Replaces the reference's batch > 1 path, which materialises the whole weight matrix as f16 in HBM
// (cuda/nve_kernels.cu:397-433, nve_dequant_w4a16) and then runs a dense GEMM on it
// (src/gpu_layer.rs:220-239): 0.625 + 2 + 2 = 4.6 bytes of HBM traffic per weight instead of 0.625.
// Here the packed weights are read once, dequantised to 16-bit in shared memory and consumed by tcgen05.mma
// with the accumulators in tensor memory.
//
// Mapping: the 128 weight rows of a tile are the MMA M dimension, the batch is the MMA N dimension
// (16 / 32 / 64), K advances 64 elements (one 128-byte swizzle row) per pipeline stage, 16 per instruction.
//   D[128 x MB] (TMEM, f32) += A[128 x 64] (dequantised f16 weights, K-major, SWIZZLE_128B)
//                            * B[MB x 64]  (f16 activations,         K-major, SWIZZLE_128B)
// Weights are always dequantised to f16, the type the reference dequantises to; bf16 activations are converted
// to f16 while the tile is staged (bf16 weights would cost 2^-8 per weight and leave no tolerance margin).
// Roles in a CTA of 288 threads:
//   warps 0-7  producers: cp.async ring of raw nibbles + scales (8 stages deep, each thread copies and later
//              reads only its own 16 + 4 bytes, so no barrier is needed on that ring); dequantise
//              (q-8)*scale with the f16/bf16 "magic number" trick (3 instructions per 2 weights) and store
//              128-bit chunks into the swizzled operand stage; load and store the activation tile;
//              fence.proxy.async; arrive on the stage's "full" mbarrier.
//   warp 8     allocates TMEM, issues tcgen05.mma (one elected lane), tcgen05.commit -> "empty" mbarrier of
//              the stage, and after the last K block -> the accumulator barrier.
//   warps 0-3  epilogue: tcgen05.ld (32 lanes x MB columns per warp), convert, store Y (or f32 split-K
//              partials to scratch, reduced in fixed order by a second small kernel).
// Inside a 64-wide K block both operands use the same fixed permutation of K inside every 8-element chunk
// ([0,2,1,3,4,6,5,7]), which is what the cheapest nibble extraction produces; a GEMM is invariant to a
// permutation of K applied to both operands.
// Every mbarrier wait is bounded; an expired wait latches an error code (nve_b200_gemm_error) and the CTA
// leaves through the normal path, freeing its TMEM columns.
#include <mutex>

#include "common.cuh"

namespace nve {

constexpr int kTileN = 128;      // weight rows per CTA = MMA M
constexpr int kKBlock = 64;      // K elements per pipeline stage (128 bytes of 16-bit)
constexpr int kRawStages = 8;    // cp.async ring depth (raw nibbles + scales)
constexpr int kOpStages = 4;     // dequantised operand stages
constexpr int kProducerThreads = 256;
constexpr int kGemmThreads = kProducerThreads + 32;
constexpr unsigned kGemmSpinLimit = 1u << 24;

__device__ int g_gemm_device_error = 0;

struct GemmParams {
    const uint16_t* X;     // [M, K] 16-bit
    const uint8_t* nib;    // [N, K/2]
    const float* sc;       // [N, K/32]
    void* Y;               // [M, N]
    float* partial;        // [ksplit, M, N] f32 when ksplit > 1
    int M, N, K;
    int nb;                // K / 32
    int kblocks;           // K / 64
    int ksplit;
};

__device__ __forceinline__ uint32_t s_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mb_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mb_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mb_wait(uint64_t* bar, unsigned parity) {
    const uint32_t addr = s_addr(bar);
    for (unsigned spin = 0; spin < kGemmSpinLimit; spin++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Shared-memory matrix descriptor, K-major, SWIZZLE_128B: start address (16-byte units), leading byte offset
// (unused for swizzled K-major, set to 1), stride byte offset = 1024 bytes between 8-row groups, descriptor
// version 1 (Blackwell), layout type 2.
__device__ __forceinline__ uint64_t make_desc_k_sw128(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_byte_addr & 0x3FFFFu) >> 4);
    d |= static_cast<uint64_t>(1) << 16;
    d |= static_cast<uint64_t>(1024 >> 4) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(2) << 61;
    return d;
}

// Instruction descriptor for kind::f16: D = f32, A and B = f16 (0) or bf16 (1), both K-major, M = 128, N = MB.
__host__ __device__ constexpr uint32_t make_idesc(int mb, bool bf16) {
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | (static_cast<uint32_t>(mb >> 3) << 17) |
           (static_cast<uint32_t>(kTileN >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(bar)) : "memory");
}

// byte offset of 16-byte chunk c (0..7) of row r inside a [rows x 128 B] SWIZZLE_128B tile
__device__ __forceinline__ uint32_t sw128_off(int r, int c) {
    return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

// (q - 8) * scale for the two nibbles selected by `pair` = 0x000N000N-masked word, as packed 16-bit floats.
template <bool BF16> __device__ __forceinline__ uint32_t dequant_pair(uint32_t masked, uint32_t scale2) {
    if constexpr (BF16) {
        // 0x4300 = 128.0 in bf16, one ulp = 1: 128 + q is exact; minus 136 gives q - 8 exactly
        masked |= 0x43004300u;
        __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&masked);
        const uint32_t c136 = 0x43084308u;
        v = __hsub2(v, *reinterpret_cast<const __nv_bfloat162*>(&c136));
        v = __hmul2(v, *reinterpret_cast<const __nv_bfloat162*>(&scale2));
        return *reinterpret_cast<uint32_t*>(&v);
    } else {
        // 0x6400 = 1024.0 in f16, one ulp = 1: 1024 + q is exact; minus 1032 gives q - 8 exactly
        masked |= 0x64006400u;
        __half2 v = *reinterpret_cast<const __half2*>(&masked);
        const uint32_t c1032 = 0x64086408u;
        v = __hsub2(v, *reinterpret_cast<const __half2*>(&c1032));
        v = __hmul2(v, *reinterpret_cast<const __half2*>(&scale2));
        return *reinterpret_cast<uint32_t*>(&v);
    }
}

// One raw word (4 bytes = elements j..j+3 in the low nibbles, j+16..j+19 in the high nibbles) -> two low pairs
// (e_j, e_j+2), (e_j+1, e_j+3) and two high pairs in the same pattern.
template <bool BF16> __device__ __forceinline__ void dequant_word(uint32_t w, uint32_t scale2, uint32_t& lo0, uint32_t& lo1,
                                                                  uint32_t& hi0, uint32_t& hi1) {
    lo0 = dequant_pair<BF16>(w & 0x000F000Fu, scale2);
    lo1 = dequant_pair<BF16>((w >> 8) & 0x000F000Fu, scale2);
    hi0 = dequant_pair<BF16>((w >> 4) & 0x000F000Fu, scale2);
    hi1 = dequant_pair<BF16>((w >> 12) & 0x000F000Fu, scale2);
}

// bf16 pair -> f16 pair.  Exact for 6.1e-5 <= |x| <= 65504 (every bf16 significand fits f16); larger magnitudes
// saturate to +-65504, smaller ones round into the f16 subnormal range.
__device__ __forceinline__ uint32_t bf16x2_to_f16x2(uint32_t v) {
    float lo = __uint_as_float(v << 16), hi = __uint_as_float(v & 0xFFFF0000u);
    lo = fminf(fmaxf(lo, -65504.0f), 65504.0f);
    hi = fminf(fmaxf(hi, -65504.0f), 65504.0f);
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Apply the chunk permutation [0,2,1,3,4,6,5,7] to 8 consecutive 16-bit activations.
__device__ __forceinline__ uint4 permute_chunk(uint4 x) {
    uint4 r;
    r.x = __byte_perm(x.x, x.y, 0x5410);  // (x0, x2)
    r.y = __byte_perm(x.x, x.y, 0x7632);  // (x1, x3)
    r.z = __byte_perm(x.z, x.w, 0x5410);  // (x4, x6)
    r.w = __byte_perm(x.z, x.w, 0x7632);  // (x5, x7)
    return r;
}

template <int MB, bool BF16, int ODT>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_w4a16_tc_kernel(const GemmParams p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // layout: A stages | B stages | raw nibbles | raw scales | barriers
    constexpr int kABytes = kTileN * 128;
    constexpr int kBBytes = MB * 128;
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = smem;
    unsigned char* sB = sA + kOpStages * kABytes;
    unsigned char* sRawN = sB + kOpStages * kBBytes;            // [kRawStages][128 rows][32 B]
    float* sRawS = reinterpret_cast<float*>(sRawN + kRawStages * kTileN * 32);  // [kRawStages][128][2]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sRawS + kRawStages * kTileN * 2);
    uint64_t* full = bars;                  // [kOpStages], 256 arrivals
    uint64_t* empty = bars + kOpStages;     // [kOpStages], 1 arrival (tcgen05.commit)
    uint64_t* accum = bars + 2 * kOpStages; // 1 arrival
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kOpStages + 1);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * kTileN;
    const int split = blockIdx.y;
    const int kb_begin = static_cast<int>(static_cast<long long>(p.kblocks) * split / p.ksplit);
    const int kb_end = static_cast<int>(static_cast<long long>(p.kblocks) * (split + 1) / p.ksplit);
    const int nkb = kb_end - kb_begin;
    constexpr int kTmemCols = MB < 32 ? 32 : MB;

    if (tid == 0) {
        for (int i = 0; i < kOpStages; i++) {
            mb_init(&full[i], kProducerThreads);
            mb_init(&empty[i], 1);
        }
        mb_init(accum, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {  // TMEM allocation is warp-wide
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp < 8) {
        // ------------------------------------------------------------------ producers
        const int r = tid & (kTileN - 1);  // weight row inside the tile
        const int h = tid >> 7;            // which 32-wide quantisation block of the K block
        const int grow = min(n0 + r, p.N - 1);
        const uint8_t* nib_row = p.nib + static_cast<long long>(grow) * (p.K / 2);
        const float* sc_row = p.sc + static_cast<long long>(grow) * p.nb;
        auto issue_raw = [&](int i) {
            if (i < nkb) {
                const int kb = kb_begin + i;
                const int st = i % kRawStages;
                cp_async_16(sRawN + (static_cast<size_t>(st) * kTileN + r) * 32 + h * 16, nib_row + kb * 32 + h * 16);
                cp_async_4(sRawS + (static_cast<size_t>(st) * kTileN + r) * 2 + h, sc_row + kb * 2 + h);
            }
            cp_async_commit();
        };
        for (int i = 0; i < kRawStages - 1; i++) issue_raw(i);

        // activation chunks owned by this thread: chunk id = j * 8 + c, ids tid and tid + 256 (MB * 8 <= 512)
        constexpr int kXChunks = MB * 8;
        auto load_x = [&](int i, int id) -> uint4 {
            uint4 v = make_uint4(0, 0, 0, 0);
            const int j = id >> 3, c = id & 7;
            if (i < nkb && id < kXChunks && j < p.M) {
                v = *reinterpret_cast<const uint4*>(p.X + static_cast<long long>(j) * p.K + (kb_begin + i) * kKBlock + c * 8);
                if constexpr (BF16) {
                    v.x = bf16x2_to_f16x2(v.x); v.y = bf16x2_to_f16x2(v.y);
                    v.z = bf16x2_to_f16x2(v.z); v.w = bf16x2_to_f16x2(v.w);
                }
            }
            return v;
        };
        pdl_wait();  // activations come from the previous kernel; weights do not
        uint4 x0 = load_x(0, tid), x1 = load_x(0, tid + 256);

        bool ok = true;
        for (int i = 0; i < nkb && ok; i++) {
            const int so = i % kOpStages;
            issue_raw(i + kRawStages - 1);
            cp_async_wait<kRawStages - 1>();  // this thread's copies for K block i have landed
            if (i >= kOpStages) {
                ok = mb_wait(&empty[so], static_cast<unsigned>(i / kOpStages - 1) & 1u);
                if (!ok || *reinterpret_cast<volatile int*>(abort_flag)) {
                    atomicCAS(&g_gemm_device_error, 0, 1);
                    atomicExch(abort_flag, 1);
                    ok = false;
                    break;
                }
            }
            // ---- dequantise this thread's 32 weights -> 4 chunks of the operand row
            const int st = i % kRawStages;
            const uint4 raw = *reinterpret_cast<const uint4*>(sRawN + (static_cast<size_t>(st) * kTileN + r) * 32 + h * 16);
            const float scale = sRawS[(static_cast<size_t>(st) * kTileN + r) * 2 + h];
            const __half2 s2 = __float2half2_rn(scale);
            const uint32_t scale2 = *reinterpret_cast<const uint32_t*>(&s2);
            uint4 c0, c1, c2, c3;  // chunks 4h .. 4h+3 of the row
            dequant_word<false>(raw.x, scale2, c0.x, c0.y, c2.x, c2.y);
            dequant_word<false>(raw.y, scale2, c0.z, c0.w, c2.z, c2.w);
            dequant_word<false>(raw.z, scale2, c1.x, c1.y, c3.x, c3.y);
            dequant_word<false>(raw.w, scale2, c1.z, c1.w, c3.z, c3.w);
            unsigned char* a_stage = sA + so * kABytes;
            *reinterpret_cast<uint4*>(a_stage + sw128_off(r, 4 * h + 0)) = c0;
            *reinterpret_cast<uint4*>(a_stage + sw128_off(r, 4 * h + 1)) = c1;
            *reinterpret_cast<uint4*>(a_stage + sw128_off(r, 4 * h + 2)) = c2;
            *reinterpret_cast<uint4*>(a_stage + sw128_off(r, 4 * h + 3)) = c3;
            // ---- activation tile (same K permutation inside every chunk)
            unsigned char* b_stage = sB + so * kBBytes;
            if (tid < kXChunks) *reinterpret_cast<uint4*>(b_stage + sw128_off(tid >> 3, tid & 7)) = permute_chunk(x0);
            if (tid + 256 < kXChunks) *reinterpret_cast<uint4*>(b_stage + sw128_off((tid + 256) >> 3, tid & 7)) = permute_chunk(x1);
            x0 = load_x(i + 1, tid);
            x1 = load_x(i + 1, tid + 256);
            // make the generic-proxy stores visible to the tensor core (async proxy), then signal
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mb_arrive(&full[so]);
        }
        cp_async_wait<0>();
        pdl_launch_dependents();

        // ------------------------------------------------------------------ epilogue (warps 0-3)
        if (warp < 4) {
            bool done = ok && mb_wait(accum, 0);
            if (!done || *reinterpret_cast<volatile int*>(abort_flag)) {
                atomicCAS(&g_gemm_device_error, 0, 3);
                atomicExch(abort_flag, 1);
                done = false;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (done) {
                const int n = n0 + warp * 32 + lane;  // this thread's output feature
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
#pragma unroll
                for (int cb = 0; cb < MB; cb += 8) {
                    uint32_t v[8];
                    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                                 : "r"(taddr + cb));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int m = cb + j;
                            if (m < p.M) {
                                const float y = __uint_as_float(v[j]);
                                if (p.ksplit > 1) p.partial[(static_cast<long long>(split) * p.M + m) * p.N + n] = y;
                                else store_out<ODT>(p.Y, static_cast<long long>(m) * p.N + n, y);
                            }
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
    } else {
        // ------------------------------------------------------------------ MMA issuer (warp 8)
        constexpr uint32_t idesc = make_idesc(MB, false);  // both operands are f16 (bf16 activations are converted)
        bool ok = true;
        for (int i = 0; i < nkb && ok; i++) {
            const int so = i % kOpStages;
            bool w = true;
            if (lane == 0) w = mb_wait(&full[so], static_cast<unsigned>(i / kOpStages) & 1u);
            w = __shfl_sync(0xffffffffu, w, 0);
            if (!w || *reinterpret_cast<volatile int*>(abort_flag)) {
                if (lane == 0) {
                    atomicCAS(&g_gemm_device_error, 0, 2);
                    atomicExch(abort_flag, 1);
                }
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint64_t adesc = make_desc_k_sw128(s_addr(sA + so * kABytes));
                const uint64_t bdesc = make_desc_k_sw128(s_addr(sB + so * kBBytes));
#pragma unroll
                for (int kk = 0; kk < kKBlock / 16; kk++) {
                    // 16 elements = 32 bytes further along K inside the swizzle row: +2 in 16-byte units
                    umma_f16(tmem_base, adesc + 2 * kk, bdesc + 2 * kk, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(&empty[so]);                 // stage reusable once these MMAs have read it
                if (i == nkb - 1) umma_commit(accum);    // accumulator complete
            }
            __syncwarp();
        }
    }

    // ---- teardown: all tensor-memory traffic is finished or abandoned; free the columns
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// Sum the split-K partials in ascending split order and convert.
template <int ODT> __global__ void gemm_splitk_reduce_kernel(const float* partial, void* Y, int ksplit, long long mn) {
    pdl_wait();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= mn) return;
    float y = partial[i];
    for (int s = 1; s < ksplit; s++) y = __fadd_rn(y, partial[static_cast<long long>(s) * mn + i]);
    store_out<ODT>(Y, i, y);
}

static size_t gemm_smem_bytes(int mb) {
    return 1024 + static_cast<size_t>(kOpStages) * (kTileN * 128 + mb * 128) + static_cast<size_t>(kRawStages) * kTileN * (32 + 8) +
           (2 * kOpStages + 1) * 8 + 16;
}

static int choose_ksplit(int N, int K, bool have_scratch) {
    if (!have_scratch) return 1;
    const int tiles = (N + kTileN - 1) / kTileN;
    int ks = sm_count() / tiles;
    const int kblocks = K / kKBlock;
    if (ks > kblocks / 8) ks = kblocks / 8;  // at least 8 K blocks (512 elements) per split
    if (ks > 8) ks = 8;
    if (ks < 1) ks = 1;
    return ks;
}

template <int MB, bool BF16, int ODT> static int launch_gemm(const GemmParams& p, cudaStream_t st) {
    auto kern = gemm_w4a16_tc_kernel<MB, BF16, ODT>;
    const size_t smem = gemm_smem_bytes(MB);
    int s = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), static_cast<int>(smem));
    if (s != NVE_OK) return s;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.N + kTileN - 1) / kTileN, p.ksplit);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    if (pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
    count_launch();
    if (e != cudaSuccess) return set_cuda_status(e);
    if (p.ksplit > 1) {
        const long long mn = static_cast<long long>(p.M) * p.N;
        gemm_splitk_reduce_kernel<ODT><<<static_cast<unsigned>((mn + 255) / 256), 256, 0, st>>>(p.partial, p.Y, p.ksplit, mn);
        count_launch();
        return check_launch();
    }
    return set_status(NVE_OK);
}

template <bool BF16, int ODT> static int gemm_mb(const GemmParams& p, cudaStream_t st) {
    if (p.M <= 16) return launch_gemm<16, BF16, ODT>(p, st);
    if (p.M <= 32) return launch_gemm<32, BF16, ODT>(p, st);
    return launch_gemm<64, BF16, ODT>(p, st);
}

}  // namespace nve

using namespace nve;

extern "C" size_t nve_b200_gemm_w4a16_scratch_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % kKBlock) != 0) return 0;
    const int ks = choose_ksplit(N, K, true);
    return ks > 1 ? static_cast<size_t>(ks) * M * N * sizeof(float) : 0;
}

extern "C" int nve_b200_gemm_w4a16(const void* X, int x_dtype, const uint8_t* nibbles, const float* scales, void* Y, int y_dtype,
                                   int M, int N, int K, void* scratch, size_t scratch_bytes, nve_stream_t stream) {
    if (!X || !nibbles || !scales || !Y) return set_status(NVE_ERR_BAD_POINTER);
    if (M < 1 || M > 64 || N < 1 || K < kKBlock || (K % kKBlock) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    if (x_dtype != NVE_DT_F16 && x_dtype != NVE_DT_BF16) return set_status(NVE_ERR_BAD_DTYPE);
    if (y_dtype != x_dtype && y_dtype != NVE_DT_F32) return set_status(NVE_ERR_BAD_DTYPE);
    if (!aligned(X, 16) || !aligned(nibbles, 16) || !aligned(scales, 4)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    GemmParams p;
    p.X = static_cast<const uint16_t*>(X);
    p.nib = nibbles;
    p.sc = scales;
    p.Y = Y;
    p.M = M; p.N = N; p.K = K;
    p.nb = K / 32;
    p.kblocks = K / kKBlock;
    int ks = choose_ksplit(N, K, scratch != nullptr);
    while (ks > 1 && static_cast<size_t>(ks) * M * N * sizeof(float) > scratch_bytes) ks--;
    p.ksplit = ks;
    p.partial = static_cast<float*>(scratch);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_dtype == NVE_DT_F16) {
        return y_dtype == NVE_DT_F32 ? gemm_mb<false, NVE_DT_F32>(p, st) : gemm_mb<false, NVE_DT_F16>(p, st);
    }
    return y_dtype == NVE_DT_F32 ? gemm_mb<true, NVE_DT_F32>(p, st) : gemm_mb<true, NVE_DT_BF16>(p, st);
}

extern "C" int nve_b200_gemm_error(int reset) {
    int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_gemm_device_error, sizeof(int));
    if (e != cudaSuccess) { set_cuda_status(e); return -1; }
    if (reset && v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_gemm_device_error, &zero, sizeof(int));
    }
    return v;
}

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant of the batched GEMM.
//
// Who needs it: the reference's batch > 1 call site (GpuWeight::matmul_x) receives only the activations and the
// weight tensors -- it has no workspace to hand down -- and it can run while a CUDA graph is being recorded,
// where cudaMalloc is illegal; a serving thread that must not touch the allocator is in the same position.
// For those callers the split-K partial sums live in a fixed array inside the library image instead of a
// caller-provided buffer.
//
// Cost and limits: the array is kStaticScratchFloats * 4 bytes (4 MiB) of device memory on every GPU that loads
// the library, until the process exits.  A call whose split-K partials (nve_b200_gemm_w4a16_scratch_bytes) exceed
// it is rejected with NVE_ERR_TOO_LARGE.  All calls share the one array: two such GEMMs that overlap on the same
// GPU (different streams) race on it; issue them on one stream.  The array keeps whatever the previous call
// left in it; nothing in it has to start at zero, because every partial a call reads was written by that same
// call's first kernel.
//
// The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
// current) and caches it; make that first call before starting any stream capture.
// ---------------------------------------------------------------------------------------------------------
namespace nve {

constexpr size_t kStaticScratchFloats = static_cast<size_t>(1) << 20;  // 1 Mi floats = 4 MiB
static __device__ __align__(256) float g_gemm_static_scratch[kStaticScratchFloats];

// Device address of g_gemm_static_scratch on the current device.  In host code the symbol itself is only a
// stand-in and must never be passed to a kernel; the address comes from the runtime, once per device.
static int static_scratch_address(float** out) {
    static std::mutex mu;
    static float* cached[64] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_cuda_status(e);
    if (dev < 0 || dev >= 64) return set_status(NVE_ERR_BAD_SHAPE);
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        float* ptr = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_gemm_static_scratch);
        if (e != cudaSuccess) return set_cuda_status(e);
        if (ptr == nullptr) return set_status(NVE_ERR_BAD_POINTER);
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return NVE_OK;
}

}  // namespace nve

extern "C" int nve_b200_gemm_w4a16_noalloc(const void* X, int x_dtype, const uint8_t* nibbles, const float* scales, void* Y,
                                           int y_dtype, int M, int N, int K, nve_stream_t stream) {
    if (!X || !nibbles || !scales || !Y) return set_status(NVE_ERR_BAD_POINTER);
    if (M < 1 || M > 64 || N < 1 || K < kKBlock || (K % kKBlock) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    if (x_dtype != NVE_DT_F16 && x_dtype != NVE_DT_BF16) return set_status(NVE_ERR_BAD_DTYPE);
    if (y_dtype != x_dtype && y_dtype != NVE_DT_F32) return set_status(NVE_ERR_BAD_DTYPE);
    if (!aligned(X, 16) || !aligned(nibbles, 16) || !aligned(scales, 4)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    const int ks = choose_ksplit(N, K, true);
    const size_t need = ks > 1 ? static_cast<size_t>(ks) * M * N : 0;  // floats
    if (need > kStaticScratchFloats) return set_status(NVE_ERR_TOO_LARGE);
    float* scratch = nullptr;
    int st = static_scratch_address(&scratch);
    if (st != NVE_OK) return st;
    GemmParams p;
    p.X = static_cast<const uint16_t*>(X);
    p.nib = nibbles;
    p.sc = scales;
    p.Y = Y;
    p.M = M; p.N = N; p.K = K;
    p.nb = K / 32;
    p.kblocks = K / kKBlock;
    p.ksplit = ks;
    p.partial = scratch;
    cudaStream_t cs = static_cast<cudaStream_t>(stream);
    if (x_dtype == NVE_DT_F16) {
        return y_dtype == NVE_DT_F32 ? gemm_mb<false, NVE_DT_F32>(p, cs) : gemm_mb<false, NVE_DT_F16>(p, cs);
    }
    return y_dtype == NVE_DT_F32 ? gemm_mb<true, NVE_DT_F32>(p, cs) : gemm_mb<true, NVE_DT_BF16>(p, cs);
}
