// Prefill / ragged-batch grouped expert FFN on the 5th-generation tensor cores (tcgen05 + TMEM), sm_100a only.
//
// Replaces PrefillGroupedRoutedMoE.encodeStreamedBatched and its kernels
// (Sources/Mference/Kernels/Prefill/PrefillGroupedRoutedMoE.swift:391-466, Sources/Mference/Metal/Prefill/prefill.metal:748-820;
// tensor-unit precedent mpp_prefill_affine_threadgroup_f16): tokens sorted by expert form a ragged grouped GEMM
//     phase 1   H[pair, f] = act(X[pair,:] . Wgate[f,:]) * (X[pair,:] . Wup[f,:])      contraction over d
//     phase 2   P[pair, d] = H[pair,:] . Wdown[d,:]                                    contraction over f
// With many rows per expert this is a dense contraction, so it goes to the tensor cores.
//
// Shape of one MMA tile: M = 128 *weight rows*, N = *token rows* of one expert (up to 128 in phase 1, 256 in phase 2),
// K in chunks of 64.  The weights are the A operand: their row count is always a multiple of 128, while the ragged
// side (tokens of an expert, from a handful to thousands) rides in N, which the hardware accepts in steps of 16.
// Tensor memory (512 columns per CTA) holds the accumulators in columns [0, 256) - phase 1: gate then up - and,
// behind them, a four-stage ring of dequantised weight chunks: the A operand is read from tensor memory, so the
// weights never touch shared memory, which only stages the activations (B operand).
//
// Roles inside a CTA (448 threads in phase 1, 576 in phase 2), connected by mbarriers, every wait bounded:
//   warp 0        TMA: the activation chunk [N x 64] fp16 of the current token rows (gathered once per call into
//                 expert-major order, so a group's rows are contiguous) lands in shared memory in the 128-byte swizzle
//   warp 1        one elected thread issues tcgen05.mma (A from TMEM, B from shared memory, D in TMEM) and tcgen05.commit
//   warps 2-9     dequantise: packed 4-bit or 2-bit codes + fp16/bf16 scale and bias -> fp16 weights, stored with
//                 tcgen05.st into the ring (a warp owns the 32 rows of its TMEM lane quarter); the packed bytes and
//                 scales come from global memory eight chunks ahead, across work-item boundaries
//   warps 10-...  epilogue (4 warps in phase 1, 8 in phase 2): tcgen05.ld the accumulators (warp w reads TMEM lanes
//                 32 (w % 4) ...), apply the activation and store fp16 hidden rows (phase 1) / fp32 partial rows (phase 2)
// The K order inside each 8- or 16-element run is the one the mask-unpack of a packed word yields (4-bit: 0 4 1 5 2
// 6 3 7; 2-bit: 0 8 1 9 ...); the gather kernel and the phase-1 epilogue store activations in the same order, so
// nothing is shuffled.
#include <cuda.h>

#include <new>

#include "prefill_tc.cuh"
#include "tmap.cuh"

namespace mfb {

namespace {

constexpr uint32_t TC_M = 128;          // weight rows per tile
constexpr uint32_t TC_KC = 64;          // k elements per chunk = one 128-byte swizzle row of fp16
constexpr uint32_t TC_BOX_ROWS = 64;    // token rows per TMA box
constexpr uint32_t TC_DQ_WARPS = 8;   // eight dequantising warps measured faster than sixteen
// epilogue warps: four in phase 1 (the dequantising threads need 128 registers, which 14 warps still allow), eight in
// phase 2, whose accumulator tiles are twice as wide
__host__ __device__ constexpr uint32_t tc_epi_warps(int phase) { return phase == 1 ? 4 : 8; }
__host__ __device__ constexpr uint32_t tc_threads(int phase) { return (2 + TC_DQ_WARPS + tc_epi_warps(phase)) * 32; }
constexpr uint32_t TC_TMEM_COLS = 512;
constexpr uint32_t TC_STAGES = 4;
// token rows per MMA tile.  Phase 1 keeps gate and up of a tile (128 columns each) in ONE accumulator buffer, the
// other 256 tensor-memory columns hold the weight ring.  Phase 2 has one matrix and a weight ring of 128 columns: tiles
// of 192 rows leave room for TWO accumulator buffers, so the epilogue of an item (a third of the launch when it ran
// alone) overlaps the MMAs of the next one.
#ifndef MFB_TC_N2
#define MFB_TC_N2 192
#endif
__host__ __device__ constexpr uint32_t tc_tile_n(int phase) { return phase == 1 ? TC_TILE_N / 2 : MFB_TC_N2; }
__host__ __device__ constexpr uint32_t tc_acc_bufs(int phase) { return phase == 1 ? 1 : (2 * tc_tile_n(2) + TC_STAGES * 32 <= TC_TMEM_COLS ? 2 : 1); }
static_assert(tc_tile_n(2) <= TC_TILE_N && tc_tile_n(2) % 64 == 0, "phase-2 tile");
constexpr long long TC_WAIT_CYCLES = 400000000ll;      // ~0.2 s

struct TcParams {
    const uint8_t* pool;
    uint64_t slot_stride;
    const int16_t* slot_of;
    const uint8_t* shared_blob;
    mfb_expert_offsets routed_off, shared_off;
    uint32_t d, f, num_experts, bits, shared_bits, scale_dtype, activation;
    float limit;
    const mfb_pair* sorted;
    const mfb_group* groups;
    const uint32_t* n_groups;
    const uint32_t* tile_prefix1;  // [n_groups + 1] exclusive prefix of ceil(pair_count / 128): token tiles of phase 1
    const uint32_t* tile_prefix2;  // the same for the 256-row token tiles of phase 2
    __half* acts16;                // [rows, f] hidden activations in sorted-pair order (phase 1 out, phase 2 in)
    float* partial;                // [token * slots + rank, d]
    float* const* row_dest;        // optional: address of the result row of (token, rank) at [token * slots + rank] (NULL entry = drop)
    uint32_t slots;
    uint32_t* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait; false when the limit runs out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    const long long t0 = clock64();
    for (;;) {
        uint32_t done;
        // the hint lets the hardware park the thread until the phase completes (or ~2 us pass): a waiting warp takes
        // no issue slots from the dequantising ones and still wakes up at once
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity), "r"(2000u) : "memory");
        if (done) return true;
        if (clock64() - t0 > TC_WAIT_CYCLES) return false;
    }
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint32_t x, uint32_t y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]^T, fp16 inputs, fp32 accumulate; issued by one thread.  A sits in tensor memory:
// 128 lanes = rows, two fp16 per 32-bit column along K.
__device__ __forceinline__ void umma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// N consecutive 32-bit columns of this thread's TMEM lane, from registers.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Arrives on the mbarrier when every MMA this thread has issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory operand descriptor: K-major tile of 128-byte rows in the 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t smem_desc(const void* tile) {
    const uint64_t addr = (smem_u32(tile) & 0x3FFFFu) >> 4;
    return addr | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: fp16 A and B, both K-major, fp32 D, M = 128, N = n.
__device__ __forceinline__ uint32_t instr_desc(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((TC_M >> 4) << 24);
}

// Position of element e (0..7) of an 8-element piece in the stored order 0 4 1 5 2 6 3 7.
__host__ __device__ inline uint32_t tc_perm8(uint32_t e) { return ((e & 3u) << 1) | (e >> 2); }

__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// Eight 4-bit codes of one packed word -> eight fp16 weights q * scale + bias, as four half2 in the stored order.
__device__ __forceinline__ uint4 dequant_word4(uint32_t w, uint32_t scale2, uint32_t bias2) {
    constexpr uint32_t MAGIC = 0x64006400u, SIXTEENTH = 0x2C002C00u, M64 = 0xD400D400u;
    const uint32_t hi = w >> 8;
    uint4 o;
    o.x = h2_fma(h2_sub((w & 0x000F000Fu) | MAGIC, MAGIC), scale2, bias2);            // codes 0, 4
    o.y = h2_fma(h2_fma((w & 0x00F000F0u) | MAGIC, SIXTEENTH, M64), scale2, bias2);   // codes 1, 5
    o.z = h2_fma(h2_sub((hi & 0x000F000Fu) | MAGIC, MAGIC), scale2, bias2);           // codes 2, 6
    o.w = h2_fma(h2_fma((hi & 0x00F000F0u) | MAGIC, SIXTEENTH, M64), scale2, bias2);  // codes 3, 7
    return o;
}

// Sixteen 2-bit codes of one packed word -> sixteen fp16 weights as eight half2 (two 16-byte pieces), element i paired
// with element i + 8: stored order 0 8 1 9 ... 7 15.  (1024 + 4^k q) * 4^-k - 1024 * 4^-k = q exactly.
__device__ __forceinline__ void dequant_word2(uint32_t w, uint32_t scale2, uint32_t bias2, uint4& lo, uint4& hi) {
    constexpr uint32_t MAGIC = 0x64006400u;
    constexpr uint32_t S1 = 0x34003400u, C1 = 0xDC00DC00u;   // 1/4, -256
    constexpr uint32_t S2 = 0x2C002C00u, C2 = 0xD400D400u;   // 1/16, -64
    constexpr uint32_t S3 = 0x24002400u, C3 = 0xCC00CC00u;   // 1/64, -16
    constexpr uint32_t S4 = 0x1C001C00u, C4 = 0xC400C400u;   // 1/256, -4
    const uint32_t b = w >> 10;
    lo.x = h2_fma(h2_sub((w & 0x00030003u) | MAGIC, MAGIC), scale2, bias2);
    lo.y = h2_fma(h2_fma((w & 0x000C000Cu) | MAGIC, S1, C1), scale2, bias2);
    lo.z = h2_fma(h2_fma((w & 0x00300030u) | MAGIC, S2, C2), scale2, bias2);
    lo.w = h2_fma(h2_fma((w & 0x00C000C0u) | MAGIC, S3, C3), scale2, bias2);
    hi.x = h2_fma(h2_fma((w & 0x03000300u) | MAGIC, S4, C4), scale2, bias2);
    hi.y = h2_fma(h2_sub((b & 0x00030003u) | MAGIC, MAGIC), scale2, bias2);
    hi.z = h2_fma(h2_fma((b & 0x000C000Cu) | MAGIC, S1, C1), scale2, bias2);
    hi.w = h2_fma(h2_fma((b & 0x00300030u) | MAGIC, S2, C2), scale2, bias2);
}

// Position of element e of a 16-element run in the stored order of its code width (4-bit: per 8 elements).
__host__ __device__ inline uint32_t tc_perm(uint32_t e, uint32_t bits) {
    return bits == 4 ? (e & 8u) | tc_perm8(e & 7u) : ((e & 7u) << 1) | (e >> 3);
}

__device__ __forceinline__ uint32_t scale_pair(uint16_t bits, uint32_t dtype) {
    __half h = dtype == MFB_DT_BF16 ? __float2half_rn(__uint_as_float((uint32_t)bits << 16)) : __ushort_as_half(bits);
    const uint32_t u = __half_as_ushort(h);
    return u | (u << 16);
}

struct Item {
    const uint8_t* blob;
    mfb_expert_offsets off;
    uint32_t pair_start, count, row0, n, n_mma, ok, shared, bits;
};

// What a work item needs to know of its group, resolved once per CTA into shared memory: every role decodes every
// item, and two dependent global loads (group record, slot table) per decode stalled each of them for a couple of
// thousand cycles per item - as long as the arithmetic of a short item.
struct TcGroup {
    uint32_t pair_start, pair_count;
    int32_t slot;        // pool slot of a routed expert (-1: not resident); for the shared expert 0 / -1
    uint32_t shared;
};

// Work item `it` -> (group, token tile, weight-row tile); the same arithmetic in every role.
__device__ __forceinline__ Item decode_item(const TcParams& P, const uint32_t* tp_s, const TcGroup* grp_s, uint32_t n_groups, uint32_t it,
                                            uint32_t n_row_tiles, uint32_t tile_n) {
    Item I;
    const uint32_t tt = it / n_row_tiles;
    uint32_t lo = 0, hi = n_groups;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) / 2;
        if (tp_s[mid] <= tt) lo = mid; else hi = mid;
    }
    const TcGroup g = grp_s[lo];
    const uint32_t n0 = (tt - tp_s[lo]) * tile_n;
    I.pair_start = g.pair_start + n0;
    I.count = g.pair_count;
    I.n = min(tile_n, g.pair_count - n0);
    I.n_mma = max(16u, (I.n + 15u) & ~15u);
    I.row0 = (it % n_row_tiles) * TC_M;
    I.shared = g.shared;
    I.ok = g.slot >= 0;
    if (I.shared) {
        I.blob = P.shared_blob; I.off = P.shared_off; I.bits = P.shared_bits;
    } else {
        I.blob = P.pool + (uint64_t)(g.slot < 0 ? 0 : g.slot) * P.slot_stride;
        I.off = P.routed_off; I.bits = P.bits;
    }
    return I;
}

struct TcShared {
    uint64_t full_a[TC_STAGES], full_b[TC_STAGES], empty[TC_STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base, abort;
    uint32_t tp[MFB_MAX_EXPERTS + 2];
    TcGroup grp[MFB_MAX_EXPERTS + 1];
    float* out_ptr[TC_TILE_N];     // phase 2 with a destination table: where the result row of each token column goes
    uint32_t out_row[TC_TILE_N];   // phase 2 without one: token * slots + rank of the current item's token columns
};

template <int PHASE>   // 1: gate / up over x;  2: down over the hidden activations
__global__ void __launch_bounds__(tc_threads(PHASE), 1) tc_ffn_kernel(const TcParams P, const __grid_constant__ CUtensorMap map_b) {
    constexpr uint32_t NMAT = PHASE == 1 ? 2 : 1;
    constexpr uint32_t TILE_N = tc_tile_n(PHASE);
    constexpr uint32_t TC_EPI_WARPS = tc_epi_warps(PHASE);
    constexpr uint32_t STAGE_BYTES = TILE_N * 128;        // shared memory holds only the activation tiles
    // tensor memory: accumulators in columns [0, 256) (phase 1: gate then up, N <= 128 each), the dequantised weight
    // chunks of the ring behind them - a 64-element chunk of a matrix is 32 columns (two fp16 per column)
    constexpr uint32_t ACC_BUFS = tc_acc_bufs(PHASE), ACC_COLS = NMAT * TILE_N;   // columns of one accumulator buffer
    constexpr uint32_t A_COL0 = ACC_BUFS * ACC_COLS, A_STAGE_COLS = NMAT * 32;
    static_assert(A_COL0 + TC_STAGES * A_STAGE_COLS <= TC_TMEM_COLS, "tensor memory budget");
    constexpr uint32_t STAGES = TC_STAGES;
    extern __shared__ uint8_t smem_raw[];
    __shared__ TcShared S;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t K = PHASE == 1 ? P.d : P.f, rows = PHASE == 1 ? P.f : P.d;
    const uint32_t n_chunks = K / TC_KC, n_row_tiles = rows / TC_M;
    const uint32_t n_groups = *P.n_groups;
    for (uint32_t i = threadIdx.x; i <= n_groups; i += blockDim.x) S.tp[i] = (PHASE == 1 ? P.tile_prefix1 : P.tile_prefix2)[i];
    for (uint32_t i = threadIdx.x; i < n_groups; i += blockDim.x) {
        const mfb_group g = P.groups[i];
        TcGroup t;
        t.pair_start = g.pair_start; t.pair_count = g.pair_count;
        t.shared = g.expert >= P.num_experts ? 1u : 0u;
        if (t.shared) t.slot = P.shared_blob != nullptr ? 0 : -1;
        else t.slot = P.slot_of ? (int32_t)P.slot_of[g.expert] : (int32_t)g.expert;
        S.grp[i] = t;
    }
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; ++s) { mbar_init(&S.full_a[s], TC_DQ_WARPS); mbar_init(&S.full_b[s], 1); mbar_init(&S.empty[s], 1); }
        for (uint32_t b = 0; b < 2; ++b) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], TC_EPI_WARPS); }
        S.abort = 0;
        fence_barrier_init();
    }
    __syncthreads();
    if (warp == 0) tmem_alloc(&S.tmem_base, TC_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = S.tmem_base;
    const uint32_t total = S.tp[n_groups] * n_row_tiles;
    volatile uint32_t* abort_flag = &S.abort;
    auto fail = [&]() { *abort_flag = 1u; atomicOr(P.status, STATUS_MBAR_TIMEOUT); };
    auto stage_b = [&](uint32_t s) { return smem + s * STAGE_BYTES; };

    if (warp == 0) {
        // ---------------------------------------------------------------- activation tiles by TMA
        uint32_t seq = 0;
        for (uint32_t it = blockIdx.x; it < total && !*abort_flag; it += gridDim.x) {
            const Item I = decode_item(P, S.tp, S.grp, n_groups, it, n_row_tiles, TILE_N);
            if (!I.ok) continue;
            const uint32_t copies = (I.n_mma + TC_BOX_ROWS - 1) / TC_BOX_ROWS;
            for (uint32_t c = 0; c < n_chunks; ++c, ++seq) {
                const uint32_t s = seq % STAGES, ph = (seq / STAGES) & 1u;
                if (!mbar_wait(&S.empty[s], ph ^ 1u)) { fail(); break; }
                if (lane == 0) {
                    mbar_expect_tx(&S.full_b[s], copies * TC_BOX_ROWS * 128);
                    for (uint32_t j = 0; j < copies; ++j)
                        tma_load_2d(stage_b(s) + j * TC_BOX_ROWS * 128, &map_b, c * TC_KC, I.pair_start + j * TC_BOX_ROWS, &S.full_b[s]);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issue
        uint32_t seq = 0, item = 0;
        for (uint32_t it = blockIdx.x; it < total && !*abort_flag; it += gridDim.x) {
            const Item I = decode_item(P, S.tp, S.grp, n_groups, it, n_row_tiles, TILE_N);
            if (!I.ok) continue;
            const uint32_t buf = item % ACC_BUFS, use = (item / ACC_BUFS) & 1u;   // accumulator buffer and the parity of its uses
            if (!mbar_wait(&S.acc_empty[buf], use ^ 1u)) { fail(); break; }
            tc_fence_after();
            const uint32_t idesc = instr_desc(I.n_mma);
            bool ok = true;
            for (uint32_t c = 0; c < n_chunks && ok; ++c, ++seq) {
                const uint32_t s = seq % STAGES, ph = (seq / STAGES) & 1u;
                if (!mbar_wait(&S.full_a[s], ph)) { fail(); ok = false; break; }
                if (!mbar_wait(&S.full_b[s], ph)) { fail(); ok = false; break; }
                tc_fence_after();
                if (lane == 0) {
                    const uint64_t b_desc = smem_desc(stage_b(s));
#pragma unroll
                    for (uint32_t m = 0; m < NMAT; ++m) {
                        const uint32_t a_tmem = tmem + A_COL0 + s * A_STAGE_COLS + m * 32;
#pragma unroll
                        for (uint32_t kk = 0; kk < TC_KC / 16; ++kk)   // 16 k per MMA: 8 TMEM columns of A, 32 bytes of B's swizzled row
                            umma_f16_ta(tmem + buf * ACC_COLS + m * TILE_N, a_tmem + kk * 8, b_desc + kk * 2, idesc, (c | kk) ? 1u : 0u);
                    }
                    umma_commit(&S.empty[s]);   // frees the stage once these MMAs have read it
                }
                __syncwarp();
            }
            if (!ok) break;
            if (lane == 0) umma_commit(&S.acc_full[buf]);
            __syncwarp();
            ++item;
        }
    } else if (warp < 2 + TC_DQ_WARPS) {
        // ---------------------------------------------------------------- dequantise
        // The dequantising threads share the NMAT * 128 row chunks of a stage: a thread owns WORDS consecutive 16-byte
        // pieces of fp16 (= WORDS packed words at 4 bits, WORDS / 2 at 2 bits) of one row.
        constexpr uint32_t WORDS = NMAT * 1024 / (TC_DQ_WARPS * 32), PARTS_PER_ROW = 8 / WORDS;
        // a warp may only touch the 32 TMEM lanes of its quarter (warp index % 4), so it takes those 32 weight rows;
        // the two warps of a quarter split the matrices (phase 1) or the chunk's halves (phase 2)
        const uint32_t q = warp & 3u, part = (warp - 2) >> 2;
        const uint32_t r = 32 * q + lane;
        const uint32_t mat = part / PARTS_PER_ROW;              // 0 in phase 2
        const uint32_t word0 = (part % PARTS_PER_ROW) * WORDS;
        const uint32_t a_lane_col = ((32 * q) << 16) + A_COL0 + mat * 32 + word0 * 4;   // + stage * A_STAGE_COLS
        // Packed codes and scales are fetched eight chunks (one scale vector) ahead of their use, through a ring of
        // registers that a load cursor refills as soon as a slot has been consumed; the cursor runs on into the
        // next work item, so the memory latency is hidden across item boundaries too.
        struct RowSrc {
            const uint32_t* wrow; const uint4* srow; const uint4* brow;
            uint32_t wpc, it, blk; bool four, valid;
        };
        auto open_item = [&](uint32_t it) {   // first resident item at or after `it` in this CTA's sequence
            RowSrc R{};
            for (; it < total; it += gridDim.x) {
                const Item I = decode_item(P, S.tp, S.grp, n_groups, it, n_row_tiles, TILE_N);
                if (!I.ok) continue;
                const uint32_t w_off = PHASE == 1 ? (mat ? I.off.up_w : I.off.gate_w) : I.off.down_w;
                const uint32_t s_off = PHASE == 1 ? (mat ? I.off.up_s : I.off.gate_s) : I.off.down_s;
                const uint32_t b_off = PHASE == 1 ? (mat ? I.off.up_b : I.off.gate_b) : I.off.down_b;
                const size_t row = I.row0 + r;
                R.four = I.bits == 4;
                R.wpc = R.four ? 8u : 4u;   // packed words per 64-element chunk of a row
                R.wrow = reinterpret_cast<const uint32_t*>(I.blob + w_off + row * (K * I.bits / 8)) + (R.four ? word0 : word0 / 2);
                R.srow = reinterpret_cast<const uint4*>(I.blob + s_off + row * (K / 64) * 2);
                R.brow = reinterpret_cast<const uint4*>(I.blob + b_off + row * (K / 64) * 2);
                R.valid = true;
                break;
            }
            R.it = it; R.blk = 0;
            return R;
        };
        auto load_n = [&](const uint32_t* src, uint32_t (&dst)[WORDS], uint32_t n) {   // n = 1, 2, 4 or 8 words
            if (n >= 4) {
                const uint4 v = *reinterpret_cast<const uint4*>(src);
                dst[0] = v.x; dst[1 % WORDS] = v.y; dst[2 % WORDS] = v.z; dst[3 % WORDS] = v.w;
                if (n == 8) {
                    const uint4 u = *reinterpret_cast<const uint4*>(src + 4);
                    dst[4 % WORDS] = u.x; dst[5 % WORDS] = u.y; dst[6 % WORDS] = u.z; dst[7 % WORDS] = u.w;
                }
            } else if (n == 2) {
                const uint2 v = *reinterpret_cast<const uint2*>(src);
                dst[0] = v.x; dst[1 % WORDS] = v.y;
            } else {
                dst[0] = *src;
            }
        };
        constexpr uint32_t RING = 8;
        uint32_t ring[RING][WORDS];
        uint4 sc_nxt = make_uint4(0, 0, 0, 0), bi_nxt = make_uint4(0, 0, 0, 0);
        RowSrc Lc = open_item(blockIdx.x);   // load cursor
        auto load_block_head = [&]() {       // scales and biases of the cursor's block
            if (Lc.valid) { sc_nxt = Lc.srow[Lc.blk]; bi_nxt = Lc.brow[Lc.blk]; }
        };
        auto load_chunk = [&](uint32_t i, uint32_t (&dst)[WORDS]) {   // chunk i of the cursor's block
            if (Lc.valid) load_n(Lc.wrow + (Lc.blk * RING + i) * Lc.wpc, dst, Lc.four ? WORDS : WORDS / 2);
        };
        auto advance_block = [&]() {
            if (!Lc.valid) return;
            if (++Lc.blk * RING >= n_chunks) Lc = open_item(Lc.it + gridDim.x);
        };
        // prime the ring with the first block
        load_block_head();
#pragma unroll
        for (uint32_t i = 0; i < RING; ++i) load_chunk(i, ring[i]);
        advance_block();
        uint32_t seq = 0;
        bool ok = true;
        for (uint32_t it = blockIdx.x; it < total && !*abort_flag && ok; it += gridDim.x) {
            const Item I = decode_item(P, S.tp, S.grp, n_groups, it, n_row_tiles, TILE_N);
            if (!I.ok) continue;
            const bool four = I.bits == 4;
            for (uint32_t cb = 0; cb < n_chunks && ok; cb += RING) {   // n_chunks is a multiple of 8
                const uint4 sc8 = sc_nxt, bi8 = bi_nxt;   // fetched one block ago
                load_block_head();                        // the cursor's block: the one after this
#pragma unroll
                for (uint32_t i = 0; i < RING; ++i, ++seq) {
                    const uint32_t s = seq % STAGES, ph = (seq / STAGES) & 1u;
                    const uint32_t sw = (&sc8.x)[i >> 1], bw = (&bi8.x)[i >> 1];
                    const uint32_t s2 = scale_pair((uint16_t)((i & 1u) ? (sw >> 16) : (sw & 0xFFFFu)), P.scale_dtype);
                    const uint32_t b2 = scale_pair((uint16_t)((i & 1u) ? (bw >> 16) : (bw & 0xFFFFu)), P.scale_dtype);
                    uint32_t outw[WORDS * 4];   // WORDS * 8 fp16 weights = WORDS * 4 TMEM columns of this row
                    if (four) {
#pragma unroll
                        for (uint32_t j = 0; j < WORDS; ++j) {
                            const uint4 o = dequant_word4(ring[i][j], s2, b2);
                            outw[4 * j] = o.x; outw[4 * j + 1] = o.y; outw[4 * j + 2] = o.z; outw[4 * j + 3] = o.w;
                        }
                    } else {
#pragma unroll
                        for (uint32_t j = 0; j < WORDS / 2; ++j) {
                            uint4 lo, hi;
                            dequant_word2(ring[i][j], s2, b2, lo, hi);
                            outw[8 * j] = lo.x; outw[8 * j + 1] = lo.y; outw[8 * j + 2] = lo.z; outw[8 * j + 3] = lo.w;
                            outw[8 * j + 4] = hi.x; outw[8 * j + 5] = hi.y; outw[8 * j + 6] = hi.z; outw[8 * j + 7] = hi.w;
                        }
                    }
                    load_chunk(i, ring[i]);   // refill the slot just consumed: needed eight chunks from now
                    if (!mbar_wait(&S.empty[s], ph ^ 1u)) { fail(); ok = false; break; }
                    if (WORDS == 8) tmem_st32(tmem + a_lane_col + s * A_STAGE_COLS, reinterpret_cast<const uint32_t (&)[32]>(outw));
                    else tmem_st16(tmem + a_lane_col + s * A_STAGE_COLS, reinterpret_cast<const uint32_t (&)[16]>(outw));
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&S.full_a[s]);
                }
                advance_block();
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue: eight warps, two per TMEM lane
        // quarter, each taking every other block of 32 token columns
        const uint32_t te = threadIdx.x - (2 + TC_DQ_WARPS) * 32;   // 0..255
        const uint32_t q = warp & 3u;                               // TMEM lane quarter this warp may read
        const uint32_t col_par = (warp - (2 + TC_DQ_WARPS)) >> 2;   // which 32-column blocks this warp takes
        constexpr uint32_t COL_WAYS = TC_EPI_WARPS / 4;
        uint32_t item = 0;
        for (uint32_t it = blockIdx.x; it < total && !*abort_flag; it += gridDim.x) {
            const Item I = decode_item(P, S.tp, S.grp, n_groups, it, n_row_tiles, TILE_N);
            const uint32_t out_row = I.row0 + 32 * q + lane;
            if (PHASE == 2) {
                // where each token column of this item goes: fetched once into shared memory (a dependent global
                // load per column inside the loop below would serialise it)
                asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");   // the previous item's table is no longer read
                for (uint32_t n = te; n < I.n; n += TC_EPI_WARPS * 32) {
                    const mfb_pair pr = P.sorted[I.pair_start + n];
                    const size_t slot = (size_t)pr.token * P.slots + pr.rank;
                    if (P.row_dest) S.out_ptr[n] = P.row_dest[slot];
                    else S.out_row[n] = (uint32_t)slot;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
            }
            if (!I.ok) {
                if (PHASE == 2)   // a non-resident expert contributes nothing: clear its partial rows
                    for (uint32_t n = col_par; n < I.n; n += COL_WAYS) {
                        if (!P.row_dest) P.partial[(size_t)S.out_row[n] * P.d + out_row] = 0.0f;
                        else if (S.out_ptr[n]) S.out_ptr[n][out_row] = 0.0f;
                    }
                continue;
            }
            const uint32_t buf = item % ACC_BUFS, use = (item / ACC_BUFS) & 1u;
            if (!mbar_wait(&S.acc_full[buf], use)) { fail(); break; }
            tc_fence_after();
            const uint32_t taddr = tmem + ((32 * q) << 16) + buf * ACC_COLS;
            for (uint32_t col0 = col_par * 32; col0 < I.n; col0 += 32 * COL_WAYS) {
                float v[32];
                tmem_ld32(taddr + col0, v);
                if (PHASE == 1) {
                    float u[32];
                    tmem_ld32(taddr + TILE_N + col0, u);
                    const uint32_t fpos = (out_row & ~15u) + tc_perm(out_row & 15u, I.bits);
                    const bool clamp = !I.shared && P.limit > 0.0f;   // moe_swiglu_clamp (moe.metal:27-34), routed experts only
                    const bool silu = P.activation == MFB_ACT_SILU;
                    __half* out = P.acts16 + (size_t)(I.pair_start + col0) * P.f + fpos;
                    const uint32_t live = min(32u, I.n - col0);
                    // all 32 columns are computed as independent chains (no early exit inside: one element's clamp, exp,
                    // reciprocal and conversion depend on each other, and run one after the other they took ~130
                    // cycles per element - the epilogue held the tensor pipe idle for a quarter of the launch); the
                    // stores are predicated afterwards
                    if (silu) {
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i) {
                            const float gate = clamp ? fminf(v[i], P.limit) : v[i];
                            const float up = clamp ? fminf(fmaxf(u[i], -P.limit), P.limit) : u[i];
                            // SiLU with the fast divide (2 ulp): the result is rounded to fp16 right after
                            const float a = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                            v[i] = fminf(fmaxf(a, -65504.0f), 65504.0f);
                        }
                    } else {
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i) {
                            const float gate = clamp ? fminf(v[i], P.limit) : v[i];
                            const float up = clamp ? fminf(fmaxf(u[i], -P.limit), P.limit) : u[i];
                            const float a = hidden_act(gate, (int)P.activation) * up;
                            v[i] = fminf(fmaxf(a, -65504.0f), 65504.0f);
                        }
                    }
#pragma unroll
                    for (uint32_t i = 0; i < 32; ++i)
                        if (i < live) out[(size_t)i * P.f] = __float2half_rn(v[i]);
                } else {
                    const uint32_t live = min(32u, I.n - col0);
                    if (!P.row_dest) {
                        float* out = P.partial + out_row;
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i) {
                            if (i >= live) break;
                            out[(size_t)S.out_row[col0 + i] * P.d] = v[i];
                        }
                    } else {
#pragma unroll
                        for (uint32_t i = 0; i < 32; ++i) {
                            if (i >= live) break;
                            float* out = S.out_ptr[col0 + i];
                            if (out) out[out_row] = v[i];
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&S.acc_empty[buf]);
            ++item;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, TC_TMEM_COLS);
}

// xs16[pos, :] = fp16(x[sorted[pos].token, :]) in the stored k order, for every sorted pair.
// Rows from n_routed on belong to the shared expert's group and follow its code width.  A thread converts sixteen
// consecutive elements: two 16-byte loads, the permutation in registers, two 16-byte stores.
__global__ void tc_gather_kernel(const void* __restrict__ x, int x_dtype, uint32_t ldx, uint32_t d,
                                 const mfb_pair* __restrict__ sorted, const mfb_group* __restrict__ groups,
                                 const uint32_t* __restrict__ n_groups, uint32_t n_rows, uint32_t n_routed, uint32_t n_tokens,
                                 uint32_t bits, uint32_t shared_bits, __half* __restrict__ xs16) {
    const uint32_t pos = blockIdx.x;
    if (pos >= n_rows) return;
    {   // rows behind the last group are not part of the call (a routing table with dropped or masked entries)
        const uint32_t ng = *n_groups;
        if (ng == 0) return;
        const mfb_group last = groups[ng - 1];
        if (pos >= last.pair_start + last.pair_count) return;
    }
    const uint32_t width = pos < n_routed ? bits : shared_bits;
    const uint32_t token = sorted[pos].token;
    if (token >= n_tokens) return;   // an entry no group refers to (a caller's list shorter than n_tokens * top_k)
    const size_t src = (size_t)token * ldx;
    const bool vec = x_dtype != MFB_DT_F32 && (ldx & 7u) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
    for (uint32_t k = threadIdx.x * 16; k < d; k += blockDim.x * 16) {
        uint16_t in[16];
        if (vec) {
            const uint4 a = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + src + k);
            const uint4 b = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + src + k + 8);
            const uint32_t u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int j = 0; j < 16; ++j) in[j] = (uint16_t)((j & 1) ? (u[j >> 1] >> 16) : (u[j >> 1] & 0xFFFFu));
        }
        uint16_t out[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float v = vec ? widen16(in[j], x_dtype) : load_act(x, src + k + j, x_dtype);
            v = fminf(fmaxf(v, -65504.0f), 65504.0f);
            const uint16_t h = __half_as_ushort(__float2half_rn(v));
            // both permutations, selected by the row's width (register indices stay compile-time constants)
            const int p4 = (j & 8) | (((j & 7) & 3) << 1) | ((j & 7) >> 2), p2 = ((j & 7) << 1) | (j >> 3);
            if (width == 4) out[p4] = h; else out[p2] = h;
        }
        uint4 o0, o1;
        o0.x = out[0] | ((uint32_t)out[1] << 16); o0.y = out[2] | ((uint32_t)out[3] << 16);
        o0.z = out[4] | ((uint32_t)out[5] << 16); o0.w = out[6] | ((uint32_t)out[7] << 16);
        o1.x = out[8] | ((uint32_t)out[9] << 16); o1.y = out[10] | ((uint32_t)out[11] << 16);
        o1.z = out[12] | ((uint32_t)out[13] << 16); o1.w = out[14] | ((uint32_t)out[15] << 16);
        uint4* dst = reinterpret_cast<uint4*>(xs16 + (size_t)pos * d + k);
        dst[0] = o0;
        dst[1] = o1;
    }
}

// prefix1[g] / prefix2[g] = number of 128-row / 256-row token tiles in groups [0, g); one warp.
__global__ void tc_tile_prefix_kernel(const mfb_group* __restrict__ groups, const uint32_t* __restrict__ n_groups,
                                      uint32_t* __restrict__ prefix1, uint32_t* __restrict__ prefix2) {
    const uint32_t ng = *n_groups, lane = threadIdx.x;
    const uint32_t per = (ng + 31) / 32, g0 = lane * per;
    const uint32_t t1 = tc_tile_n(1), t2 = tc_tile_n(2);
    uint32_t l1 = 0, l2 = 0;
    for (uint32_t j = 0; j < per; ++j)
        if (g0 + j < ng) { const uint32_t c = groups[g0 + j].pair_count; l1 += (c + t1 - 1) / t1; l2 += (c + t2 - 1) / t2; }
    uint32_t i1 = l1, i2 = l2;
    for (uint32_t off = 1; off < 32; off <<= 1) {
        const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, i1, off), b = __shfl_up_sync(0xFFFFFFFFu, i2, off);
        if (lane >= off) { i1 += a; i2 += b; }
    }
    uint32_t r1 = i1 - l1, r2 = i2 - l2;
    for (uint32_t j = 0; j < per; ++j)
        if (g0 + j < ng) {
            const uint32_t c = groups[g0 + j].pair_count;
            prefix1[g0 + j] = r1; prefix2[g0 + j] = r2;
            r1 += (c + t1 - 1) / t1; r2 += (c + t2 - 1) / t2;
        }
    if (lane == 31) { prefix1[ng] = i1; prefix2[ng] = i2; }
}

struct TcState {
    CUtensorMap map_x, map_h;
    uint64_t rows_cap = 0;
    uint32_t* prefix = nullptr;   // device: two arrays of MFB_MAX_EXPERTS + 2 token-tile prefixes
    bool ready = false;
};

constexpr size_t TC_SMEM_BYTES = TC_STAGES * tc_tile_n(2) * 128 + 1024;   // activation tiles only (phase 2 is the larger)

int32_t make_map(CUtensorMap* map, void* base, uint64_t inner, uint64_t rows) {
    const uint64_t dims[2] = {inner, rows}, strides[1] = {inner * sizeof(__half)};
    const uint32_t box[2] = {TC_KC, TC_BOX_ROWS};
    return encode_tensor_map(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, base, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
}

}  // namespace

bool tc_supported(const mfb_moe_config& c) {
    // scales are fetched 8 groups (16 bytes) at a time, so both contraction lengths are multiples of 512; the
    // dequantising warps handle 4-bit and 2-bit codes (an 8-bit shared expert runs the generic kernels)
    return c.d % 512 == 0 && c.f % 512 == 0 && c.shared_bits != 8;
}

// Everything the tensor-core path needs besides its launches, built once when the handle is created: the tensor maps
// over the arena's gathered rows and hidden activations, the token-tile prefix arrays and the kernels' opt-in to
// large dynamic shared memory.  The per-call path only launches.
int32_t tc_init(mfb_moe* m) {
    const mfb_moe_config& c = m->cfg;
    Arena& a = m->a;
    if (!a.xs16 || !a.acts16 || !tc_supported(c)) return MFB_OK;
    TcState* st = new (std::nothrow) TcState();
    MFB_REQUIRE(st != nullptr, MFB_ERR_ALLOC, "out of host memory");
    m->tma = st;
    st->rows_cap = m->max_rows + TC_ROW_PAD;
    int32_t rc = make_map(&st->map_x, a.xs16, c.d, st->rows_cap);
    if (rc) return rc;
    rc = make_map(&st->map_h, a.acts16, c.f, st->rows_cap);
    if (rc) return rc;
    MFB_CUDA(cudaMalloc(&st->prefix, 2 * (MFB_MAX_EXPERTS + 2) * sizeof(uint32_t)));
    MFB_CUDA(cudaFuncSetAttribute(tc_ffn_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES));
    MFB_CUDA(cudaFuncSetAttribute(tc_ffn_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM_BYTES));
    st->ready = true;
    return MFB_OK;
}

void tc_release(mfb_moe* m) {
    if (m->tma) cudaFree(static_cast<TcState*>(m->tma)->prefix);
    delete static_cast<TcState*>(m->tma);
    m->tma = nullptr;
}

int32_t tc_grouped_ffn(mfb_moe* m, cudaStream_t s, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                       uint32_t n_tokens, const mfb_pair* sorted, const mfb_group* groups, const uint32_t* n_groups,
                       uint32_t max_groups, bool routed_only, float* partial, uint32_t slots, float* const* row_dest) {
    const mfb_moe_config& c = m->cfg;
    Arena& a = m->a;
    MFB_REQUIRE(a.xs16 && a.acts16, MFB_ERR_INVALID_ARGUMENT, "tensor-core path: the handle was created without MFB_FLAG_PREFILL_TENSOR_CORE");
    TcState* st = static_cast<TcState*>(m->tma);
    MFB_REQUIRE(st && st->ready, MFB_ERR_INVALID_ARGUMENT, "tensor-core path: the handle's tensor maps were not built");
    // the shared expert's rows follow the routed pairs only when the layer has one (the grouping appends them then)
    const bool with_shared = !routed_only && w->shared_blob != nullptr;
    const uint32_t n_rows = n_tokens * c.top_k + (with_shared ? n_tokens : 0u);
    TcParams P;
    P.pool = (const uint8_t*)w->pool; P.slot_stride = w->slot_stride; P.slot_of = w->slot_of;
    P.shared_blob = with_shared ? (const uint8_t*)w->shared_blob : nullptr;
    P.routed_off = w->routed_off; P.shared_off = w->shared_off;
    P.d = c.d; P.f = c.f; P.num_experts = c.num_experts; P.bits = c.bits; P.shared_bits = c.shared_bits;
    P.scale_dtype = c.scale_dtype; P.activation = c.activation; P.limit = c.swiglu_limit;
    P.sorted = sorted; P.groups = groups; P.n_groups = n_groups;
    P.tile_prefix1 = st->prefix; P.tile_prefix2 = st->prefix + MFB_MAX_EXPERTS + 2;
    P.acts16 = a.acts16; P.partial = partial; P.row_dest = row_dest; P.slots = slots; P.status = a.status;

    tc_tile_prefix_kernel<<<1, 32, 0, s>>>(groups, n_groups, st->prefix, st->prefix + MFB_MAX_EXPERTS + 2);
    tc_gather_kernel<<<n_rows, 128, 0, s>>>(x, (int)c.x_dtype, ldx, c.d, sorted, groups, n_groups, n_rows, n_tokens * c.top_k, n_tokens,
                                            c.bits, c.shared_bits ? c.shared_bits : c.bits, a.xs16);
    // upper bounds of the work items (the kernels read the exact counts from the prefix arrays)
    const uint32_t items1 = ((n_rows + tc_tile_n(1) - 1) / tc_tile_n(1) + max_groups) * (c.f / TC_M);
    const uint32_t items2 = ((n_rows + tc_tile_n(2) - 1) / tc_tile_n(2) + max_groups) * (c.d / TC_M);
    const uint32_t grid1 = items1 < (uint32_t)m->sm_count ? items1 : (uint32_t)m->sm_count;
    const uint32_t grid2 = items2 < (uint32_t)m->sm_count ? items2 : (uint32_t)m->sm_count;
    tc_ffn_kernel<1><<<grid1, tc_threads(1), TC_SMEM_BYTES, s>>>(P, st->map_x);
    tc_ffn_kernel<2><<<grid2, tc_threads(2), TC_SMEM_BYTES, s>>>(P, st->map_h);
    count_launches(4);
    MFB_CUDA(cudaGetLastError());
    return MFB_OK;
}

}  // namespace mfb
