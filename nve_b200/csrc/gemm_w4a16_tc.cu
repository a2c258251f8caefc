// Batched W4A16 GEMM on the 5th-generation tensor cores:  Y[M,N] = X[M,K] . W^T,  M = decode batch (<= 64).
//
// Replaces the reference's batch > 1 path, which materialises the whole weight matrix as f16 in HBM
// (cuda/nve_kernels.cu:397-433, nve_dequant_w4a16) and then runs a dense GEMM on it
// (src/gpu_layer.rs:220-239): 0.625 + 2 + 2 = 4.6 bytes of HBM traffic per weight instead of 0.625.
// Here the packed weights are read once, dequantised to f16 in registers, written straight into tensor memory
// and consumed from there by tcgen05.mma (A operand in TMEM), with the accumulators in tensor memory as well.
//
// Mapping: the 128 weight rows of a tile are the MMA M dimension (TMEM lanes), the batch is the MMA N dimension
// (16 / 32 / 64), K advances 64 elements per pipeline stage, 16 per instruction.
//   D[128 x MB] (TMEM, f32) += A[128 x 64] (dequantised f16 weights, TMEM: lane = row, 2 elements per column)
//                            * B[MB x 64]  (f16 activations, shared memory, K-major, SWIZZLE_128B, loaded by TMA)
// TMEM columns: four accumulator sets of MB columns, then 12 (MB = 64: 8) operand stages of 32 columns.  Eight to
// twelve stages (two or three super-blocks of four K blocks) decouple the dequantisers from the MMA round trip
// (arrive -> issue -> commit -> wake-up, about a microsecond).
// Weights are always dequantised to f16, the type the reference dequantises to; bf16 activations are converted
// to f16 by a small pre-pass into the caller's scratch (bf16 weights would cost 2^-8 per weight and leave no
// tolerance margin; tcgen05.mma kind::f16 takes both operands in one format).
// Work split: the K range of every 128-row tile is cut into super-blocks of 256 weights per row, and the sequence
// (tile 0, super-block 0), (tile 0, super-block 1), ... is dealt out in equal contiguous runs, one per CTA (one
// CTA per SM: a CTA owns all 512 TMEM columns).  A run may start and end inside a tile; the part of a tile that a
// CTA computes is a segment.  Whole-tile segments are stored to Y, the others as f32 partial tiles that a second
// kernel adds in ascending K order.
// Roles in a CTA of 640 threads:
//   warps 0-15 producers, two teams of eight warps that take alternate super-blocks (256 weights per row), each
//              with its own named barrier and its own cp.async ring of raw nibbles + scales (coalesced along K:
//              a warp-wide copy touches 4 cache lines; three super-stages per team).  A team is two groups of four
//              warps (thread = weight row = TMEM lane); group g dequantises K blocks 2g and 2g+1 of the team's
//              super-block: (q-8)*scale with the f16 magic-number trick (exact q-8, one rounding in the multiply),
//              tcgen05.st into the stage's columns, tcgen05.wait::st, one arrival per warp on the stage's "full"
//              mbarrier.  One lane per group issues the TMA tile load of the stage's activations, which completes
//              on the same barrier (expect_tx).  The producers run through the CTA's whole run without regard to
//              segment boundaries (only the global addresses change at a tile boundary).
//   warps 16-19 issue tcgen05.mma (one lane each): warp 16+w takes K block w of every super-block into accumulator
//              set w, tcgen05.commit -> "empty" mbarrier of the stage, and after the last K block of a segment ->
//              the accumulator barrier.  Issuing costs a thread ~70 cycles per MMA and ~150 per commit whatever the
//              shape, which is why four warps share it.  The same warps are the epilogue: tcgen05.ld (warp w reads
//              TMEM lanes 32w..32w+31, MB columns, the four sets added in ascending order), convert, store; the
//              next segment's MMAs wait until all four warps have read.  Warp 16 also allocates and frees the
//              TMEM columns.
// K order is natural in both operands: one byte permute per raw word puts the two nibbles of consecutive
// elements 16 bits apart, where a half2 wants them.
// Every mbarrier wait is bounded in time; an expired wait latches an error code (nve_b200_gemm_error) and the
// CTA leaves through the normal path, freeing its TMEM columns.
// What bounds the kernel (ncu, 28672 x 4096 at batch 16): 3.8 instructions per weight, of which 1.75 are the
// dequantisation itself (PRMT, SHF, 4 x (LOP3, HADD2, HMUL2) per 8 weights) and about a third is executed by
// waiting threads (mbarrier polling); issue slots 40 % busy, about 5 warps active per scheduler of which 0.7 are
// eligible per cycle.  A CTA needs ~6 us for start-up and tail (barrier setup, TMEM allocation, first bytes from
// DRAM, last MMAs and epilogue) and ~1 us per unit (128 rows x 256 weights) with all SMs busy, 0.8 us alone on the
// GPU -- a latency-bound pipeline at about a third of the HBM rate.  A variant with TMA-fed raw rings, dedicated
// loader warps and units issued by four warps side by side measured the same per-unit time, as did runs without
// the dequantisation arithmetic (-14 %), without the MMAs (-16 %) and without the TMEM stores (0 %).
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "gemm_w4a16.cuh"

namespace nve {

constexpr int kRawStages = 3;    // cp.async ring depth per team, in super-stages
constexpr int kStageCols = kKBlock / 2;     // TMEM columns of one A stage: two f16 per 32-bit column
constexpr int kTmemCols = 512;   // the whole tensor memory of the SM
constexpr int kMmaWarps = kSuper; // one per K block of a super-block, each with its own accumulator set
// Issuing is what bounds this kernel, not the tensor pipe: with N <= 64 an MMA is a few cycles of work, but a
// thread needs about 70 cycles per tcgen05.mma and 150 per tcgen05.commit (measured with clock64 around each),
// whatever the instruction's shape.  Four warps therefore issue in parallel, warp w taking K block w of every
// super-block into its own accumulator set; the epilogue sums the sets in ascending order.
__host__ __device__ constexpr int acc_sets(int) { return kMmaWarps; }
// super-blocks of operand stages in flight: what is left of the 512 columns, in units of 4 stages x 32 columns
__host__ __device__ constexpr int op_slots(int mb) { return (kTmemCols - acc_sets(mb) * mb) / (kSuper * kStageCols); }
constexpr int kMaxOpStages = 12;
// Barriers are indexed by the unit number modulo kBarUnits (x 4 K blocks), not by the operand slot: see the kernel.
constexpr int kBarUnits = 6;
constexpr int kBarStages = kBarUnits * kSuper;
constexpr int kTeams = 2;          // producer teams; team t takes super-blocks t, t+2, ... on its own barrier and raw ring
constexpr int kGroups = 2;         // groups of four warps per team (thread = weight row = TMEM lane)
constexpr int kBurst = kSuper / kGroups;  // K blocks a group dequantises per super-block
constexpr int kTeamThreads = 128 * kGroups;
constexpr int kProducerThreads = kTeamThreads * kTeams;
constexpr int kProducerWarps = kProducerThreads / 32;
constexpr int kGemmThreads = kProducerThreads + 32 * kMmaWarps;
constexpr unsigned long long kGemmWaitLimitNs = 50ull * 1000 * 1000;  // a legitimate wait lasts microseconds

__device__ int g_gemm_device_error = 0;

__device__ __forceinline__ void mb_init(uint64_t* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mb_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_addr(bar)) : "memory");
}
// One try_wait with a suspend-time hint: the hardware parks the thread until the phase completes or the hint
// (nanoseconds) runs out, so a waiting warp does not burn issue slots that the dequantising warps need.
__device__ __forceinline__ void mb_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_addr(bar)), "r"(bytes) : "memory");
}
// One TMA tile load (no multicast): box at element coordinates (x, y) of the tensor map -> shared memory, bytes
// counted on the mbarrier.  x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_dst), "l"(map), "r"(x), "r"(y), "r"(mbar)
                 : "memory");
}
__device__ __forceinline__ bool mb_try(uint32_t addr, unsigned parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity), "r"(20000u)
        : "memory");
    return done != 0;
}
// The same test without the suspend-time hint.
__device__ __forceinline__ bool mb_test(uint32_t addr, unsigned parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded by wall time: false after kGemmWaitLimitNs without the phase completing.  The clock is read once per 64
// tries.  A parity wait is only meaningful when the previous phase of the barrier is known to be complete; every
// wait in this kernel is made by a thread that, in program order, has already dealt with that previous phase (see
// the barrier ring in the kernel).
__device__ __forceinline__ bool mb_wait(uint64_t* bar, unsigned parity) {
    const uint32_t addr = s_addr(bar);
    for (int i = 0; i < 64; i++)
        if (mb_try(addr, parity)) return true;
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    do {
        for (int i = 0; i < 64; i++)
            if (mb_try(addr, parity)) return true;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    } while (t - t0 < kGemmWaitLimitNs);
    return false;
}
// mb_wait that polls without the hint, for the waits whose end is the critical path of the CTA (segment ends).
__device__ __forceinline__ bool mb_wait_spin(uint64_t* bar, unsigned parity) {
    const uint32_t addr = s_addr(bar);
    for (int i = 0; i < 256; i++)
        if (mb_test(addr, parity)) return true;
    unsigned long long t0, t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    do {
        for (int i = 0; i < 64; i++)
            if (mb_test(addr, parity)) return true;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    } while (t - t0 < kGemmWaitLimitNs);
    return false;
}
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
__host__ __device__ constexpr uint32_t make_idesc(int mb, bool a_bf16, bool b_bf16) {
    return (1u << 4) | ((a_bf16 ? 1u : 0u) << 7) | ((b_bf16 ? 1u : 0u) << 10) | (static_cast<uint32_t>(mb >> 3) << 17) |
           (static_cast<uint32_t>(kTileN >> 4) << 24);
}

// A operand read from tensor memory (128 lanes x 8 columns = 16 f16 per row), B through a shared-memory descriptor.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 consecutive TMEM columns of this thread's lane (lane = 32 * (warp % 4) + lane id).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(bar)) : "memory");
}

// byte offset of 16-byte chunk c (0..7) of row r inside a [rows x 128 B] SWIZZLE_128B tile
__device__ __forceinline__ uint32_t sw128_off(int r, int c) {
    return static_cast<uint32_t>((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4));
}

template <int MB, int ODT>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_w4a16_tc_kernel(const GemmParams p, const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // layout: B stages | raw nibbles | raw scales | barriers
    constexpr int kBBytes = MB * 128;
    constexpr int kAccSets = acc_sets(MB);
    constexpr int kAccCols = kAccSets * MB;     // TMEM columns [0, kAccCols): accumulators, then the operand stages
    constexpr int kSlots = op_slots(MB);
    constexpr int kOpStages = kSlots * kSuper;  // dequantised operand stages (A in TMEM, B in shared memory)
    static_assert(kAccCols + kOpStages * kStageCols <= kTmemCols && kSlots >= 2 && kOpStages <= kMaxOpStages, "TMEM budget");
    static_assert(kBarUnits % kSlots == 0 && kBarUnits % kTeams == 0, "the barrier ring must be a multiple of the operand ring and of the team count");
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sB = smem;
    unsigned char* sRawN = sB + kOpStages * kBBytes;            // [kTeams][kRawStages][128 rows][128 B], 16-byte chunks XOR-swizzled
    float* sRawS = reinterpret_cast<float*>(sRawN + kTeams * kRawStages * kTileN * 128);  // [kTeams][kRawStages][128 rows][8 scales]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sRawS + kTeams * kRawStages * kTileN * 8);
    // A parity wait is only meaningful when the waiter knows that the barrier's previous phase is complete.  The
    // operand ring has two or three slots, but units alternate between two dequantiser teams: with one barrier
    // per slot, consecutive phases of an "empty" barrier would be awaited by different teams, which are not ordered
    // with each other.  The barriers of a unit are therefore indexed by the unit number modulo kBarUnits = 6 (a
    // multiple of both ring depths and of the team count): the thread that awaits phase k of a barrier has, in
    // program order, already awaited its phase k - 1, and so has every thread that arrives on it.
    uint64_t* full = bars;                  // [kBarStages], one arrival per warp of the owning group + the activation tile's bytes
    uint64_t* empty = bars + kBarStages;    // [kBarStages], 1 arrival (tcgen05.commit)
    uint64_t* accum = bars + 2 * kBarStages; // one arrival per issuing warp: the segment's accumulators are complete
    uint64_t* accfree = accum + 1;          // one arrival per issuing warp: the segment's accumulators have been read
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfree + 1);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    // This CTA's work: units [u0, u0 + n_units) of the sequence (tile 0, super-block 0), (tile 0, super-block 1),
    // ..., (tile 1, super-block 0), ...  The tiles of the (up to three) matrices follow one another.  A maximal
    // run of units of one tile is a segment; it is whole when it covers all super-blocks of the tile.
    const int SB = p.sb_per_tile;
    const int u0 = blockIdx.x * p.units_per_cta;
    const int n_units = min(p.units_per_cta, p.total_units - u0);

    if (tid == 0) {
        for (int i = 0; i < kBarStages; i++) {
            mb_init(&full[i], 5);  // the four warps of the group that owns the stage + the TMA issuer's expect_tx
            mb_init(&empty[i], 1);
        }
        mb_init(accum, kMmaWarps);
        mb_init(accfree, kMmaWarps);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kProducerWarps) {  // TMEM allocation is warp-wide
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (warp < kProducerWarps) {
        // ------------------------------------------------------------------ producers
        // Raw loading is coalesced along K: 8 lanes copy the 128 contiguous nibble bytes (256 weights) of one row,
        // so a warp-wide cp.async touches 4 cache lines instead of 32.  16-byte chunks are XOR-swizzled by the row
        // so that the later per-row reads are bank-conflict free.  Addresses are set up once per tile; inside a
        // tile the loop only advances them (the kernel is bound by instruction issue, so loop overhead counts).
        // The chain of one super-block (copy wait -> barrier -> ring wait -> load -> convert -> store -> fences ->
        // arrive) is over a thousand cycles of mostly latency; two teams run it out of phase on alternate
        // units, each with its own named barrier and raw ring.
        const int team = tid / kTeamThreads;
        const int tt = tid - team * kTeamThreads;        // thread inside the team
        const int nsb_team = n_units > team ? (n_units - team + kTeams - 1) / kTeams : 0;  // units team, team + kTeams, ...
        constexpr int kNibPer = 1024 / kTeamThreads;  // 128 rows x 8 chunks of 16 bytes
        constexpr int kScPer = 512 / kTeamThreads;    // 128 rows x 4 K blocks x 2 scales
        constexpr uint32_t kRawNStage = kTileN * 128, kRawSStage = kTileN * 8 * 4;
        const unsigned char* teamRawN = sRawN + team * (kRawStages * kRawNStage);
        const unsigned char* teamRawS = reinterpret_cast<const unsigned char*>(sRawS) + team * (kRawStages * kRawSStage);
        const uint8_t* gn[kNibPer];
        uint32_t sn[kNibPer];
        const float* gs[kScPer];
        uint32_t ss[kScPer];
#pragma unroll
        for (int j = 0; j < kNibPer; j++) {
            const int id = tt + kTeamThreads * j;
            const int rr = id >> 3, c = id & 7;
            sn[j] = s_addr(teamRawN) + rr * 128 + ((c ^ (rr & 7)) << 4);
        }
#pragma unroll
        for (int j = 0; j < kScPer; j++) {
            const int id = tt + kTeamThreads * j;
            const int rr = id >> 2, kbi = id & 3;
            ss[j] = s_addr(teamRawS) + (rr * 8 + kbi * 2) * 4;
        }
        // global addresses of this thread's chunks of super-block sbi of a tile
        auto set_ptrs = [&](int tile, int sbi) {
            int mi, n0;
            tile_locate(p, tile, mi, n0);
            const int Nloc = p.Nm[mi];
            const uint8_t* nb0 = p.nib[mi] + sbi * (kSuper * 32);
            const float* sc0 = p.sc[mi] + sbi * (kSuper * 2);
#pragma unroll
            for (int j = 0; j < kNibPer; j++) {
                const int id = tt + kTeamThreads * j;
                const int rr = id >> 3, c = id & 7;
                const int grow = min(n0 + rr, Nloc - 1);
                gn[j] = nb0 + static_cast<long long>(grow) * (p.K / 2) + c * 16;
            }
#pragma unroll
            for (int j = 0; j < kScPer; j++) {
                const int id = tt + kTeamThreads * j;
                const int rr = id >> 2, kbi = id & 3;
                const int grow = min(n0 + rr, Nloc - 1);
                gs[j] = sc0 + static_cast<long long>(grow) * p.nb + kbi * 2;
            }
        };
        // cursor of the raw copies: the team's next unit to fetch
        int i_tile = (u0 + team) / SB;
        int i_sbi = (u0 + team) - i_tile * SB;
        int i_left = nsb_team;
        if (i_left > 0) set_ptrs(i_tile, i_sbi);
        uint32_t issue_n = 0, issue_s = 0;     // byte offsets of the raw stage to fill
        auto issue_raw = [&]() {
            if (i_left > 0) {
                const int valid = p.kblocks - i_sbi * kSuper;  // K blocks of this super-block that exist (>= 1)
#pragma unroll
                for (int j = 0; j < kNibPer; j++) {
                    const int kn = ((tt + kTeamThreads * j) & 7) >> 1;  // K block of the super-block that the chunk belongs to
                    if (kn < valid) cp_async_16s(sn[j] + issue_n, gn[j]);
                }
#pragma unroll
                for (int j = 0; j < kScPer; j++) {
                    const int ks = (tt + kTeamThreads * j) & 3;
                    if (ks < valid) cp_async_8s(ss[j] + issue_s, gs[j]);
                }
                i_left--;
                i_sbi += kTeams;
                if (i_sbi >= SB) {  // the team's next unit lies in a later tile
                    do {
                        i_sbi -= SB;
                        i_tile++;
                    } while (i_sbi >= SB);
                    if (i_left > 0) set_ptrs(i_tile, i_sbi);
                } else {
#pragma unroll
                    for (int j = 0; j < kNibPer; j++) gn[j] += kTeams * kSuper * 32;
#pragma unroll
                    for (int j = 0; j < kScPer; j++) gs[j] += kTeams * kSuper * 2;
                }
                issue_n = issue_n == (kRawStages - 1) * kRawNStage ? 0 : issue_n + kRawNStage;
                issue_s = issue_s == (kRawStages - 1) * kRawSStage ? 0 : issue_s + kRawSStage;
            }
            cp_async_commit();
        };
        issue_raw();
        issue_raw();

        // Groups of four warps; in every super-block group g dequantises K blocks kBurst*g .. kBurst*(g+1)-1 in one
        // go: the waits first, then all loads, arithmetic and stores, one round of fences, one arrival per stage.
        // The activation tile of a stage is one TMA tile load (SWIZZLE_128B, rows beyond M zero-filled), issued by
        // one lane of the group as soon as the stage is free; it completes on the stage's "full" barrier.
        const int r = tid & (kTileN - 1);  // weight row inside the tile = TMEM lane
        const int g = tt >> 7;             // group inside the team
        const uint32_t tmem_lane = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + kAccCols;
        const bool tma_lane = (warp & 3) == 0 && lane == 0;
        pdl_wait();  // activations come from the previous kernel; weights do not
        int d_sbi = (u0 + team) % SB;  // super-block (inside its tile) of the unit being dequantised

        // read offsets of this group's quantisation blocks inside a raw row / scale row
        uint32_t roff[2 * kBurst];
#pragma unroll
        for (int q = 0; q < 2 * kBurst; q++) roff[q] = r * 128 + (((2 * kBurst * g + q) ^ (r & 7)) << 4);
        const uint32_t soff = (r * 8 + 2 * kBurst * g) * 4;

        const DequantConsts dc = make_dequant_consts();
        bool ok = true;
        int slot = team % kSlots;  // operand-ring slot of the unit
        uint32_t raw_n = 0, raw_s = 0;  // byte offsets of the raw stage to read
        for (int it = 0; it < nsb_team; it++) {
            cp_async_wait<1>();                               // this thread's copies of the super-block have landed
            if (team == 0) asm volatile("bar.sync 2, %0;" ::"n"(kTeamThreads) : "memory");  // ... and the team's
            else asm volatile("bar.sync 3, %0;" ::"n"(kTeamThreads) : "memory");
            // every thread of the team has finished the previous super-block, whose raw stage is refilled now
            issue_raw();
            // K blocks of the burst that exist (fewer than kBurst only in the last super-block of a K that is not
            // a multiple of 256, which the host allows only when a CTA's run is exactly one tile)
            const int nvalid = max(0, min(kBurst, p.kblocks - d_sbi * kSuper - kBurst * g));
            const int kx = (d_sbi * kSuper + kBurst * g) * kKBlock;  // K coordinate of the burst
            const int so0 = slot * kSuper + kBurst * g;  // operand stage of the first K block of the burst
            const int jj = team + kTeams * it;           // index of the unit in the CTA's run
            const int fb0 = (jj % kBarUnits) * kSuper + kBurst * g;  // its "full" barriers
            const int pj = jj - kSlots;                  // the unit whose MMAs read these operand stages last
            // a warp that gave up keeps attending the producer barrier above (the others would wait for it for ever)
            // and does nothing else
            if (ok && nvalid > 0) {
                if (pj >= 0) {
                    // one lane polls for the warp: many threads spinning on one mbarrier word serialise
                    bool w = true;
                    const unsigned par = static_cast<unsigned>(pj / kBarUnits) & 1u;
                    const int eb0 = (pj % kBarUnits) * kSuper + kBurst * g;
                    if (lane == 0)
                        for (int b2 = 0; b2 < nvalid && w; b2++) w = mb_wait(&empty[eb0 + b2], par);
                    w = __shfl_sync(0xffffffffu, w, 0);
                    if (!w) {
                        if (lane == 0) {
                            atomicCAS(&g_gemm_device_error, 0, 1);
                            atomicExch(abort_flag, 1);
                        }
                        ok = false;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                }
                if (ok) {
                    if (tma_lane) {
                        for (int b2 = 0; b2 < nvalid; b2++) {
                            mb_expect_tx(&full[fb0 + b2], kBBytes);
                            tma_load_2d(s_addr(sB + (so0 + b2) * kBBytes), &xmap, kx + b2 * kKBlock, 0, s_addr(&full[fb0 + b2]));
                        }
                    }
                    float scv[2 * kBurst];
                    uint4 raw[2 * kBurst];
#pragma unroll
                    for (int q = 0; q < 2 * kBurst; q += 2) {
                        const float2 s2 = *reinterpret_cast<const float2*>(teamRawS + raw_s + soff + q * 4);
                        scv[q] = s2.x;
                        scv[q + 1] = s2.y;
                    }
#pragma unroll
                    for (int q = 0; q < 2 * kBurst; q++)  // this group's quantisation blocks of the super-stage row
                        raw[q] = *reinterpret_cast<const uint4*>(teamRawN + raw_n + roff[q]);
#pragma unroll
                    for (int q = 0; q < 2 * kBurst; q++) {
                        const int b2 = q >> 1, h = q & 1;
                        if (b2 < nvalid) {
                            const DequantScale ds = make_dequant_scale(scv[q]);
                            // v[c] = elements (2c, 2c+1) of the block: TMEM column c of the block's 16 columns
                            uint32_t v[16];
                            dequant_word(raw[q].x, ds, dc, v[0], v[1], v[8], v[9]);
                            dequant_word(raw[q].y, ds, dc, v[2], v[3], v[10], v[11]);
                            dequant_word(raw[q].z, ds, dc, v[4], v[5], v[12], v[13]);
                            dequant_word(raw[q].w, ds, dc, v[6], v[7], v[14], v[15]);
                            tmem_st16(tmem_lane + (so0 + b2) * kStageCols + 16 * h, v);
                        }
                    }
                    // TMEM stores complete and ordered before the arrival
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {  // one arrival per warp
                        for (int b2 = 0; b2 < nvalid; b2++) mb_arrive(&full[fb0 + b2]);
                    }
                }
            }
            d_sbi += kTeams;
            while (d_sbi >= SB) d_sbi -= SB;
            raw_n = raw_n == (kRawStages - 1) * kRawNStage ? 0 : raw_n + kRawNStage;
            raw_s = raw_s == (kRawStages - 1) * kRawSStage ? 0 : raw_s + kRawSStage;
            slot = (slot + kTeams) % kSlots;
        }
        cp_async_wait<0>();
        pdl_launch_dependents();
    } else {
        // ------------------------------------------------------------------ MMA issuers and epilogue (last four warps)
        // Warp w issues K block w of every unit into accumulator set w (one lane: waits, fences, MMAs and commits
        // are single-thread operations).  At the end of a segment the four warps wait for all four sets, and
        // warp w reads TMEM lanes 32w .. 32w+31 (the lanes a warp with this index may touch) of every set, adds
        // them in ascending order and stores the tile -- to Y when the segment is whole, else as an f32 partial
        // tile that the reduce kernel sums.  The next segment's MMAs start once all four warps have read.
        constexpr uint32_t idesc = make_idesc(MB, false, false);  // both operands f16 (bf16 activations are converted first)
        const int w = warp - kProducerWarps;
        pdl_wait();  // the stores below must not overtake the previous kernel's reads of Y / the partials
        int j = 0, seg = 0;
        int tile = u0 / SB;
        int sbi = u0 - tile * SB;
        bool ok = true;
        while (j < n_units) {
            const int seg_units = min(SB - sbi, n_units - j);
            if (lane == 0) {
                if (seg > 0) ok = mb_wait_spin(accfree, static_cast<unsigned>(seg - 1) & 1u);
                bool issued = false;
                for (int q = 0; q < seg_units && ok; q++) {
                    if ((sbi + q) * kSuper + w >= p.kblocks) break;  // K block beyond the end of a ragged K
                    const int jj = j + q;
                    const int so = (jj % kSlots) * kSuper + w;
                    const int ub = (jj % kBarUnits) * kSuper + w;  // the barriers of this K block of the unit
                    ok = mb_wait(&full[ub], static_cast<unsigned>(jj / kBarUnits) & 1u);
                    if (!ok || *reinterpret_cast<volatile int*>(abort_flag)) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_tmem = tmem_base + kAccCols + so * kStageCols;
                    const uint64_t bdesc = make_desc_k_sw128(s_addr(sB + so * kBBytes));
#pragma unroll
                    for (int kk = 0; kk < kKBlock / 16; kk++) {
                        // 16 elements further along K: 8 TMEM columns for A, 32 bytes (+2 in 16-byte units) for B
                        umma_f16_ts(tmem_base + w * MB, a_tmem + 8 * kk, bdesc + 2 * kk, idesc, (q > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[ub]);  // stage reusable once these MMAs have read it
                    issued = true;
                }
                if (ok) {
                    // this warp's accumulator set is complete (a warp without a K block of its own just arrives)
                    if (issued) umma_commit(accum);
                    else mb_arrive(accum);
                    ok = mb_wait_spin(accum, static_cast<unsigned>(seg) & 1u);
                }
                if (!ok || *reinterpret_cast<volatile int*>(abort_flag)) {
                    atomicCAS(&g_gemm_device_error, 0, 2);
                    atomicExch(abort_flag, 1);
                    ok = false;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            {
                int mi, n0;
                tile_locate(p, tile, mi, n0);
                const int Nloc = p.Nm[mi];
                const bool whole = seg_units == SB;
                const int n = n0 + w * 32 + lane;  // this thread's output feature
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(w * 32) << 16);
                const int used = min(kAccSets, min((sbi + seg_units) * kSuper, p.kblocks) - sbi * kSuper);  // sets that received an MMA
                float* part = p.partial + (static_cast<long long>(2 * blockIdx.x + (seg > 0 ? 1 : 0)) * p.M) * kTileN + w * 32 + lane;
#pragma unroll
                for (int cb = 0; cb < MB; cb += 8) {
                    // the four sets' loads go out together and are waited for once (a set that received no MMA --
                    // only when the whole K is shorter than four K blocks -- is read and ignored)
                    uint32_t v[kAccSets][8];
#pragma unroll
                    for (int a = 0; a < kAccSets; a++)
                        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                                     : "=r"(v[a][0]), "=r"(v[a][1]), "=r"(v[a][2]), "=r"(v[a][3]), "=r"(v[a][4]), "=r"(v[a][5]),
                                       "=r"(v[a][6]), "=r"(v[a][7])
                                     : "r"(taddr + a * MB + cb));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    float y[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        y[e] = __uint_as_float(v[0][e]);
#pragma unroll
                        for (int a = 1; a < kAccSets; a++)
                            if (a < used) y[e] = __fadd_rn(y[e], __uint_as_float(v[a][e]));
                    }
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const int m = cb + e;
                        if (m < p.M) {
                            if (!whole) part[m * kTileN] = y[e];
                            else if (n < Nloc) store_out<ODT>(p.Y[mi], static_cast<long long>(m) * Nloc + n, y[e]);
                        }
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mb_arrive(accfree);
            j += seg_units;
            sbi += seg_units;
            if (sbi >= SB) {
                sbi = 0;
                tile++;
            }
            seg++;
        }
        __syncwarp();
    }

    // ---- teardown: all tensor-memory traffic is finished or abandoned; free the columns
    __syncthreads();
    if (warp == kProducerWarps) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// Tiles that more than one CTA worked on: sum their partial tiles in ascending CTA (= ascending K) order, convert
// and store.  One block per tile; a tile that a single CTA covered was stored by that CTA.
template <int ODT> __global__ void __launch_bounds__(512) gemm_partial_reduce_kernel(const GemmParams p) {
    pdl_wait();
    const int t = blockIdx.x;
    const int SB = p.sb_per_tile, U = p.units_per_cta;
    const int first = (t * SB) / U, last = ((t + 1) * SB - 1) / U;
    if (first == last) return;
    int mi, n0;
    tile_locate(p, t, mi, n0);
    const int Nloc = p.Nm[mi];
    const int n = n0 + threadIdx.x;
    const int m = blockIdx.y * blockDim.y + threadIdx.y;
    if (n >= Nloc || m >= p.M) return;
    // the CTA's first segment when its run starts inside this tile, else its last one
    auto part = [&](int c) {
        const int slot = 2 * c + (c * U >= t * SB ? 0 : 1);
        return __ldcg(p.partial + (static_cast<long long>(slot) * p.M + m) * kTileN + threadIdx.x);
    };
    float y = part(first);
    int c = first + 1;
    for (; c + 3 <= last; c += 4) {  // four loads in flight, added in ascending order
        const float v0 = part(c), v1 = part(c + 1), v2 = part(c + 2), v3 = part(c + 3);
        y = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(y, v0), v1), v2), v3);
    }
    for (; c <= last; c++) y = __fadd_rn(y, part(c));
    store_out<ODT>(p.Y[mi], static_cast<long long>(m) * Nloc + n, y);
}

static size_t gemm_smem_bytes(int mb) {
    const size_t need = 1024 + static_cast<size_t>(op_slots(mb) * kSuper) * (mb * 128) + static_cast<size_t>(kTeams * kRawStages) * kTileN * (128 + 32) +
                        (2 * kBarStages + 2) * 8 + 16;
    // A CTA allocates all 512 TMEM columns, so a second CTA on the same SM would only sit in tcgen05.alloc until the
    // first one ends: ask for more than half of the SM's shared memory to keep it off the SM instead.
    const size_t half_sm = 120 * 1024;
    return need > half_sm ? need : half_sm;
}

// How the (tile, super-block) sequence is cut into one contiguous run per CTA.  With a workspace the runs are equal
// (total / SM count, rounded up; at least two super-blocks = 512 weights per row), whatever the tile count: few
// tiles are split over K so that every SM streams weights, and a tile count that is not a multiple of the SM count
// (gate/up of an 8B model: 224 tiles on 148 SMs) costs total / SMs instead of two full waves.  Runs that cut a
// tile leave f32 partial tiles in the workspace (two slots per CTA: its first and its last segment); the reduce
// kernel adds them in ascending K order, so the result is reproducible for a given SM count.  Without a workspace,
// or with K not a multiple of 256, a CTA takes exactly one tile.
struct GemmPlan {
    int sb;      // super-blocks per tile
    int U;       // units per CTA
    int grid;
    size_t partial_bytes;  // 0 when every run consists of whole tiles
};
static size_t plan_partial_bytes(int total, int sb, int U, int M) {
    if (U % sb == 0) return 0;
    const int grid = (total + U - 1) / U;
    return static_cast<size_t>(2) * grid * M * kTileN * sizeof(float);
}
static GemmPlan plan_gemm(int tiles, int K, int M, bool have_scratch, size_t avail) {
    GemmPlan g;
    const int kblocks = K / kKBlock;
    g.sb = (kblocks + kSuper - 1) / kSuper;
    const long long total = static_cast<long long>(tiles) * g.sb;
    g.U = g.sb;
    if (have_scratch && (kblocks % kSuper) == 0 && total < 0x3FFFFFFF) {
        const int sms = sm_count();
        int U = static_cast<int>((total + sms - 1) / sms);
        if (U < 2) U = g.sb < 2 ? g.sb : 2;
        // More tiles than SMs and a wide batch: the partial tiles (2 x M x 128 floats per CTA, written and read back)
        // and the longer epilogues cost more than the uneven waves do (measured at M = 64 on 224 tiles); whole tiles.
        if (M > 32 && tiles >= sms) U = g.sb;
        // a workspace too small for the partial tiles: longer runs (fewer CTAs) until they fit; whole tiles need none
        while (plan_partial_bytes(static_cast<int>(total), g.sb, U, M) > avail) U++;
        g.U = U;
    }
    g.grid = static_cast<int>((total + g.U - 1) / g.U);
    g.partial_bytes = plan_partial_bytes(static_cast<int>(total), g.sb, g.U, M);
    return g;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link-time dependency on libcuda).
// It is a pure host-side encoder: no allocation, no device work, legal during stream capture.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

// Tensor map of X [M rows, K columns] (16-bit), box = one K block x MB rows, 128-byte swizzle; rows >= M read zero.
static int make_x_map(const GemmParams& p, int mb, CUtensorMap* map) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (fn == nullptr) return set_status(NVE_ERR_CUDA);
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(p.K), static_cast<cuuint64_t>(p.M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(p.K) * 2};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kKBlock), static_cast<cuuint32_t>(mb)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                          const_cast<uint16_t*>(p.X), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NVE_OK : set_status(NVE_ERR_CUDA);
}

// the second kernel of a call whose runs cut tiles
template <int ODT> static int launch_reduce(const GemmParams& p, cudaStream_t st) {
    if (p.units_per_cta % p.sb_per_tile != 0) {
        gemm_partial_reduce_kernel<ODT><<<dim3(p.tile_end[2], (p.M + 3) / 4), dim3(kTileN, 4), 0, st>>>(p);
        count_launch();
        return check_launch();
    }
    return set_status(NVE_OK);
}

template <int MB, int ODT> static int launch_gemm(const GemmParams& p, cudaStream_t st) {
    auto kern = gemm_w4a16_tc_kernel<MB, ODT>;
    CUtensorMap xmap;
    if (int ms = make_x_map(p, MB, &xmap); ms != NVE_OK) return ms;
    const size_t smem = gemm_smem_bytes(MB);
    int s = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), static_cast<int>(smem));
    if (s != NVE_OK) return s;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.total_units + p.units_per_cta - 1) / p.units_per_cta);
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
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p, xmap);
    count_launch();
    if (e != cudaSuccess) return set_cuda_status(e);
    return launch_reduce<ODT>(p, st);
}

// Which kernel a batch goes to.  Measured on the four projection groups of an 8B model (us per call, this kernel /
// the mma.sync kernel): batch 8: qkv 13.5 / 11.3, o 10.8 / 9.0, gate+up 31.7 / 28.6, down 19.8 / 17.6; batch 16:
// 14.0 / 13.2, 11.0 / 10.1, 33.4 / 37.5, 20.3 / 21.0; batch 32: 15.9 / 17.5, 11.9 / 12.9, 38.1 / 52.6, 22.0 / 29.0 --
// every eight batch rows cost the mma.sync kernel another pass over the legacy tensor path (about 9 us on gate+up),
// whereas tcgen05 takes up to 64 rows in one instruction.  So: up to 8 rows mma.sync, above that tcgen05.
// NVE_B200_GEMM_KERNEL = "tc" or "mma" (read once) overrides the choice where the named kernel supports the batch.
static int gemm_kernel_choice() {
    static const int choice = [] {
        const char* e = std::getenv("NVE_B200_GEMM_KERNEL");
        if (e != nullptr && std::strcmp(e, "tc") == 0) return 1;
        if (e != nullptr && std::strcmp(e, "mma") == 0) return 2;
        return 0;
    }();
    return choice;
}

template <int ODT> static int gemm_mb(const GemmParams& p, cudaStream_t st) {
    if (gemm_kernel_choice() == 2 || (gemm_kernel_choice() == 0 && p.M <= 8)) {
        int status = NVE_OK;
        if (gemm_mma_try(p, ODT, st, status)) return status != NVE_OK ? status : launch_reduce<ODT>(p, st);
    }
    if (p.M <= 16) return launch_gemm<16, ODT>(p, st);
    if (p.M <= 32) return launch_gemm<32, ODT>(p, st);
    return launch_gemm<64, ODT>(p, st);
}

// bf16 -> f16, eight elements per thread.  Exact for 6.1e-5 <= |x| <= 65504 (every bf16 significand fits f16);
// larger magnitudes saturate to +-65504, smaller ones round into the f16 subnormal range.
__global__ void bf16_to_f16_kernel(const uint4* in, uint4* out, long long n8) {
    pdl_wait();
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const uint4 v = in[i];
    auto cvt = [](uint32_t w) {
        float lo = __uint_as_float(w << 16), hi = __uint_as_float(w & 0xFFFF0000u);
        lo = fminf(fmaxf(lo, -65504.0f), 65504.0f);
        hi = fminf(fmaxf(hi, -65504.0f), 65504.0f);
        const __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&h);
    };
    out[i] = make_uint4(cvt(v.x), cvt(v.y), cvt(v.z), cvt(v.w));
}

static size_t x16_region_bytes(int M, int K) { return (static_cast<size_t>(M) * K * 2 + 255) & ~static_cast<size_t>(255); }

// Shared by both entry points.  Scratch layout: [f16 copy of bf16 activations (x16_region_bytes)][partial tiles].
// bf16 activations need the first region; the partial tiles of split runs use what is left.
struct GemmMat {
    const uint8_t* nib;
    const float* sc;
    void* Y;
    int N;
};

static int run_gemm_multi(const void* X, int x_dtype, const GemmMat* mats, int num_mats, int y_dtype, int M, int K, void* scratch,
                          size_t scratch_bytes, cudaStream_t st) {
    unsigned char* sp = static_cast<unsigned char*>(scratch);
    GemmParams p;
    p.X = static_cast<const uint16_t*>(X);
    if (x_dtype == NVE_DT_BF16) {
        const size_t xb = x16_region_bytes(M, K);
        if (sp == nullptr || scratch_bytes < xb) return set_status(NVE_ERR_TOO_LARGE);
        if (!aligned(sp, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
        const long long n8 = static_cast<long long>(M) * K / 8;
        bf16_to_f16_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, st>>>(static_cast<const uint4*>(X),
                                                                                     reinterpret_cast<uint4*>(sp), n8);
        count_launch();
        if (int cs = check_launch(); cs != NVE_OK) return cs;
        p.X = reinterpret_cast<const uint16_t*>(sp);
        sp += xb;
        scratch_bytes -= xb;
    }
    int tiles = 0, cols = 0;
    for (int m = 0; m < 3; m++) {
        const GemmMat& g = mats[m < num_mats ? m : 0];
        p.nib[m] = g.nib; p.sc[m] = g.sc; p.Y[m] = g.Y;
        p.Nm[m] = m < num_mats ? g.N : 0;
        p.col0[m] = cols;
        if (m < num_mats) {
            tiles += (g.N + kTileN - 1) / kTileN;
            cols += g.N;
        }
        p.tile_end[m] = tiles;
    }
    // matrices that are not there: col0 past the last column so that the reduce kernel never selects them
    for (int m = num_mats; m < 3; m++) p.col0[m] = 0x7FFFFFFF;
    p.M = M; p.N = cols; p.K = K;
    p.nb = K / 32;
    p.kblocks = K / kKBlock;
    const GemmPlan plan = plan_gemm(tiles, K, M, sp != nullptr, sp != nullptr ? scratch_bytes : 0);
    p.sb_per_tile = plan.sb;
    p.units_per_cta = plan.U;
    p.total_units = tiles * plan.sb;
    p.partial = reinterpret_cast<float*>(sp);
    if (y_dtype == NVE_DT_F32) return gemm_mb<NVE_DT_F32>(p, st);
    return y_dtype == NVE_DT_F16 ? gemm_mb<NVE_DT_F16>(p, st) : gemm_mb<NVE_DT_BF16>(p, st);
}

static int run_gemm(const void* X, int x_dtype, const uint8_t* nibbles, const float* scales, void* Y, int y_dtype, int M, int N,
                    int K, void* scratch, size_t scratch_bytes, cudaStream_t st) {
    const GemmMat one = {nibbles, scales, Y, N};
    return run_gemm_multi(X, x_dtype, &one, 1, y_dtype, M, K, scratch, scratch_bytes, st);
}

}  // namespace nve

using namespace nve;

extern "C" size_t nve_b200_gemm_w4a16_scratch_bytes(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0 || (K % kKBlock) != 0) return 0;
    return x16_region_bytes(M, K) + plan_gemm((N + kTileN - 1) / kTileN, K, M, true, ~static_cast<size_t>(0)).partial_bytes;
}

extern "C" size_t nve_b200_gemm_w4a16_multi_scratch_bytes(int M, const int* Ns, int num_mats, int K) {
    if (M <= 0 || K <= 0 || (K % kKBlock) != 0 || Ns == nullptr || num_mats < 1 || num_mats > 3) return 0;
    long long tiles = 0, cols = 0;
    for (int m = 0; m < num_mats; m++) {
        if (Ns[m] <= 0) return 0;
        tiles += (Ns[m] + kTileN - 1) / kTileN;
        cols += Ns[m];
    }
    if (tiles > 0x00FFFFFF) return 0;
    return x16_region_bytes(M, K) + plan_gemm(static_cast<int>(tiles), K, M, true, ~static_cast<size_t>(0)).partial_bytes;
}

extern "C" int nve_b200_gemm_w4a16_multi(const void* X, int x_dtype, const nve_b200_w4_matrix* mats, int num_mats, int y_dtype,
                                         int M, int K, void* scratch, size_t scratch_bytes, nve_stream_t stream) {
    if (!X || !mats) return set_status(NVE_ERR_BAD_POINTER);
    if (num_mats < 1 || num_mats > 3 || M < 1 || M > 64 || K < kKBlock || (K % kKBlock) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    if (x_dtype != NVE_DT_F16 && x_dtype != NVE_DT_BF16) return set_status(NVE_ERR_BAD_DTYPE);
    if (y_dtype != x_dtype && y_dtype != NVE_DT_F32) return set_status(NVE_ERR_BAD_DTYPE);
    if (!aligned(X, 16)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    GemmMat g[3];
    long long cols = 0;
    for (int m = 0; m < num_mats; m++) {
        if (!mats[m].nibbles || !mats[m].scales || !mats[m].out) return set_status(NVE_ERR_BAD_POINTER);
        if (mats[m].residual != nullptr) return set_status(NVE_ERR_BAD_POINTER);  // no fused residual in the GEMM
        if (mats[m].N < 1) return set_status(NVE_ERR_BAD_SHAPE);
        if (!aligned(mats[m].nibbles, 16) || !aligned(mats[m].scales, 8)) return set_status(NVE_ERR_BAD_ALIGNMENT);
        g[m] = {mats[m].nibbles, mats[m].scales, mats[m].out, mats[m].N};
        cols += mats[m].N;
    }
    if (cols > 0x7FFFFFF0ll) return set_status(NVE_ERR_BAD_SHAPE);
    return run_gemm_multi(X, x_dtype, g, num_mats, y_dtype, M, K, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int nve_b200_gemm_w4a16(const void* X, int x_dtype, const uint8_t* nibbles, const float* scales, void* Y, int y_dtype,
                                   int M, int N, int K, void* scratch, size_t scratch_bytes, nve_stream_t stream) {
    if (!X || !nibbles || !scales || !Y) return set_status(NVE_ERR_BAD_POINTER);
    if (M < 1 || M > 64 || N < 1 || K < kKBlock || (K % kKBlock) != 0) return set_status(NVE_ERR_BAD_SHAPE);
    if (x_dtype != NVE_DT_F16 && x_dtype != NVE_DT_BF16) return set_status(NVE_ERR_BAD_DTYPE);
    if (y_dtype != x_dtype && y_dtype != NVE_DT_F32) return set_status(NVE_ERR_BAD_DTYPE);
    if (!aligned(X, 16) || !aligned(nibbles, 16) || !aligned(scales, 8)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    return run_gemm(X, x_dtype, nibbles, scales, Y, y_dtype, M, N, K, scratch, scratch_bytes, static_cast<cudaStream_t>(stream));
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
// For those callers the partial tiles of split runs live in a fixed array inside the library image instead of a
// caller-provided buffer.
//
// Cost and limits: the array is kStaticScratchFloats * 4 bytes (4 MiB) of device memory on every GPU that loads
// the library, until the process exits.  A call whose partial tiles (nve_b200_gemm_w4a16_scratch_bytes) exceed
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
    if (!aligned(X, 16) || !aligned(nibbles, 16) || !aligned(scales, 8)) return set_status(NVE_ERR_BAD_ALIGNMENT);
    const size_t need = (x_dtype == NVE_DT_BF16 ? x16_region_bytes(M, K) : 0) +
                        plan_gemm((N + kTileN - 1) / kTileN, K, M, true, ~static_cast<size_t>(0)).partial_bytes;
    if (need > kStaticScratchFloats * sizeof(float)) return set_status(NVE_ERR_TOO_LARGE);
    float* scratch = nullptr;
    int st = static_scratch_address(&scratch);
    if (st != NVE_OK) return st;
    return run_gemm(X, x_dtype, nibbles, scales, Y, y_dtype, M, N, K, scratch, kStaticScratchFloats * sizeof(float),
                    static_cast<cudaStream_t>(stream));
}
