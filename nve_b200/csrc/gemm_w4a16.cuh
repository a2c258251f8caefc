// Shared by the two batched W4A16 GEMM kernels (tcgen05 for wide batches, mma.sync for narrow ones): the launch
// parameters, the work split over (tile, super-block) units, the nibble dequantisation and the cp.async helpers.
#pragma once

#include "common.cuh"

namespace nve {

constexpr int kTileN = 128;      // weight rows per tile
constexpr int kKBlock = 64;      // K elements per pipeline stage of the tcgen05 kernel (128 bytes of 16-bit)
constexpr int kSuper = 4;        // K blocks per super-block: 256 elements = 128 contiguous nibble bytes per row

struct GemmParams {
    const uint16_t* X;     // [M, K] f16
    const uint8_t* nib[3]; // per matrix [N_i, K/2]
    const float* sc[3];    // per matrix [N_i, K/32]
    void* Y[3];            // per matrix [M, N_i]
    int Nm[3];             // rows of each matrix
    int tile_end[3];       // cumulative 128-row tiles
    int col0[3];           // first column of each matrix in the concatenated [M, N] view
    float* partial;        // [2 * grid][M][128] f32: slot 2c = first, slot 2c + 1 = last partial tile of CTA c
    int M, N, K;           // N = sum of Nm
    int nb;                // K / 32
    int kblocks;           // K / 64
    int sb_per_tile;       // super-blocks (4 K blocks) per tile
    int units_per_cta;     // super-blocks in a CTA's contiguous run of the (tile, super-block) sequence
    int total_units;       // tiles * sb_per_tile
};

// matrix and first row (inside that matrix) of a 128-row tile of the side-by-side tile sequence
__device__ __forceinline__ void tile_locate(const GemmParams& p, int tile, int& mi, int& n0) {
    mi = tile < p.tile_end[0] ? 0 : (tile < p.tile_end[1] ? 1 : 2);
    n0 = (tile - (mi == 0 ? 0 : p.tile_end[mi - 1])) * kTileN;
}

__device__ __forceinline__ uint32_t s_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async_16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16s(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_8s(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(s_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s_addr(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Dequantisation of two nibbles.  0x6400 is 1024.0 in f16 with one ulp = 1, so OR-ing a nibble into mantissa bits
// 0-3 gives 1024 + q exactly; 0x5400 is 64.0 with one ulp = 1/16, so a nibble left in place at bits 4-7 gives
// 64 + q exactly (no shift needed).  Subtracting 1032 (72) gives q - 8 exactly, and one multiply by the f16 scale
// rounds once.  (A single-FMA form needs 1.5 * scale to be exact, which costs two bits of scale precision --
// measured at 9e-3 of the output RMS, too close to the tolerance -- so it is not used.)
struct DequantScale {
    uint32_t mul2;  // half2(s, s)
};
__device__ __forceinline__ DequantScale make_dequant_scale(float scale) {
    const __half2 m = __float2half2_rn(scale);
    DequantScale d;
    d.mul2 = *reinterpret_cast<const uint32_t*>(&m);
    return d;
}
// Masks, magic numbers and offsets live in registers that the optimiser cannot see through: with literal
// constants the compiler emitted two LOP3 per pair (one immediate per instruction); (w & mask) | magic is a
// single LOP3 when all three operands are registers.
struct DequantConsts {
    uint32_t mask_lo, magic_lo, off_lo, mask_hi, magic_hi, off_hi;
};
__device__ __forceinline__ DequantConsts make_dequant_consts() {
    DequantConsts c;
    asm volatile("mov.b32 %0, 0x000F000F;" : "=r"(c.mask_lo));
    asm volatile("mov.b32 %0, 0x64006400;" : "=r"(c.magic_lo));
    asm volatile("mov.b32 %0, 0x64086408;" : "=r"(c.off_lo));   // 1032
    asm volatile("mov.b32 %0, 0x00F000F0;" : "=r"(c.mask_hi));
    asm volatile("mov.b32 %0, 0x54005400;" : "=r"(c.magic_hi));
    asm volatile("mov.b32 %0, 0x54805480;" : "=r"(c.off_hi));   // 72
    return c;
}
template <bool HIGH> __device__ __forceinline__ uint32_t dequant_pair(uint32_t w, const DequantScale& d, const DequantConsts& c) {
    uint32_t bits;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(bits) : "r"(w), "r"(HIGH ? c.mask_hi : c.mask_lo), "r"(HIGH ? c.magic_hi : c.magic_lo));
    const uint32_t off = HIGH ? c.off_hi : c.off_lo;
    __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&bits), *reinterpret_cast<const __half2*>(&off));
    v = __hmul2(v, *reinterpret_cast<const __half2*>(&d.mul2));
    return *reinterpret_cast<const uint32_t*>(&v);
}

// One raw word (4 bytes = elements j..j+3 in the low nibbles, j+16..j+19 in the high nibbles) -> pairs in natural
// order: lo0 = (e_j, e_j+1), lo1 = (e_j+2, e_j+3), hi0 = (e_j+16, e_j+17), hi1 = (e_j+18, e_j+19).  One byte
// permute per word ([b0,b2,b1,b3]) puts the two elements of every pair 16 bits apart, where a half2 wants them.
__device__ __forceinline__ void dequant_word(uint32_t w, const DequantScale& d, const DequantConsts& c, uint32_t& lo0,
                                             uint32_t& lo1, uint32_t& hi0, uint32_t& hi1) {
    const uint32_t u = __byte_perm(w, 0, 0x3120);
    const uint32_t t = u >> 8;
    lo0 = dequant_pair<false>(u, d, c);  // b0 low nibble, b1 low nibble
    hi0 = dequant_pair<true>(u, d, c);   // b0 high, b1 high
    lo1 = dequant_pair<false>(t, d, c);  // b2 low, b3 low
    hi1 = dequant_pair<true>(t, d, c);   // b2 high, b3 high
}

// The narrow-batch kernel (gemm_w4a16_mma.cu): same parameters, same partial-tile layout, same reduce kernel.
// Returns false when it has no instantiation for this batch, else true with the launch status in `status`.
bool gemm_mma_try(const GemmParams& p, int y_dtype, cudaStream_t st, int& status);

}  // namespace nve
