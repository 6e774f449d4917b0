// Decode-time expert FFN, fast path: packed rows staged into shared memory by bulk async copies (TMA unit),
// unpacked in registers straight into tensor-core fragments, fp32 accumulation; and the fused stack kernel that
// runs every layer of a decode step in one cooperative launch.
//
// Why tensor-core fragments for a GEMV: at 4 bits per weight B200's HBM delivers ~13 T codes/s while the CUDA
// cores issue ~36 T lane-instructions/s, i.e. fewer than three instructions per code for everything (unpack,
// convert, multiply-add, scale).  A scalar fp32 multiply-add per code already spends most of that.  Feeding
// mma.sync.m16n8k16 instead costs ~1.1 instructions per code for the unpack (one logic op and one half2
// op per two codes) and nothing for the multiply-adds, and the same instruction stream serves one to eight
// token rows, so batch 1 and batch 8 per expert cost the same.  tcgen05 is the wrong tool here: its A operand
// must sit dequantised in shared memory, which at 2 bytes per weight written and read again exceeds the
// shared-memory bandwidth at HBM rate; the register-operand mma does not touch shared memory for weights
// beyond the 0.5 byte per code the copy engine deposits.
//
// Arithmetic is the reference's factored form (Sources/Mference/Metal/MoE/moe.metal:349-529, 902-1062):
// per 64-element group  acc += scale * sum(code * x) + bias * sum(x), fp32; sum(code * x) is produced by four
// k16 MMAs on exact small integers (codes) times fp16 activations with fp32 accumulation, sum(x) by four MMAs
// against an all-ones fragment.
//
// The K dimension of an MMA may be permuted freely as long as both operands agree, so packed rows are consumed
// as they lie in memory: lane (g, t) of a warp takes bytes [8t, 8t+8) of each 32-byte group of rows g and g+8
// (4-bit; 4 bytes of each 16-byte group for 2-bit) and the activations are stored once per layer in the
// matching within-16 order (see perm_pos).
#include "common.cuh"
#include "decode_mma.cuh"
#include "select.cuh"

namespace mfb {

namespace {

constexpr int CW = 16;                      // compute warps per CTA
constexpr int FAST_THREADS = (CW + 1) * 32; // + one copy-issuing warp
constexpr int KS = 8;                       // k splits of a phase-1 row tile
constexpr int RT = CW / KS;                 // 16-row tiles per phase-1 stage
constexpr int F1_STAGES = 2;
constexpr int F2_SLOTS = 10;                // ring depth of phase 2 (one slot = one (group, token tile))
constexpr uint32_t ROW_PAD = 32;            // bytes after each 8-row block of a phase-1 tile (bank stagger)
constexpr long long MBAR_WAIT_CYCLES = 400000000ll;   // bounded spin on mbarriers: ~0.2 s at 1.9 GHz
constexpr uint32_t MAX_GROUPS = MFB_MAX_EXPERTS + 1;

// ------------------------------------------------------------------------------------------ PTX helpers
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
// Bounded wait: returns false when the limit runs out (the caller records it and unwinds).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    const long long t0 = clock64();
    for (;;) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if (clock64() - t0 > MBAR_WAIT_CYCLES) return false;
        __nanosleep(32);   // a waiting warp should not take issue slots from the computing ones
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
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
// Loads that bypass L1: for buffers other CTAs write during the same launch (fused stack kernel) a line left in
// this SM's L1 by an earlier layer would be stale.  volatile keeps them from being merged across layers.
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ld_cg_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_cg_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ld_cg_f32(const void* p) { return __uint_as_float(ld_cg_u32(p)); }
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// ------------------------------------------------------------------------------------------ unpacking
// Codes of a lane's 16-element segment as eight half2 registers of exact small integers.
// 4-bit: words w0 (codes 0-7) and w1 (codes 8-15); register i holds (q[e], q[e+4]) with e following
// 0,1,2,3,8,9,10,11.  The OR with 0x6400 plants a code in the mantissa of 1024.0 (or of 1024 + 16 q for the
// high nibble), one half2 subtract / fma then leaves the code itself.
template <int BITS>
struct Unpack;

template <>
struct Unpack<4> {
    static constexpr int WORDS = 2;   // 32-bit words per lane per row per 64-element group
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t (&p)[8]) {
        constexpr uint32_t MAGIC = 0x64006400u, SIXTEENTH = 0x2C002C00u, M64 = 0xD400D400u;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t lo = w[i], hi = w[i] >> 8;
            p[4 * i + 0] = h2_sub((lo & 0x000F000Fu) | MAGIC, MAGIC);
            p[4 * i + 1] = h2_fma((lo & 0x00F000F0u) | MAGIC, SIXTEENTH, M64);
            p[4 * i + 2] = h2_sub((hi & 0x000F000Fu) | MAGIC, MAGIC);
            p[4 * i + 3] = h2_fma((hi & 0x00F000F0u) | MAGIC, SIXTEENTH, M64);
        }
    }
};

// 2-bit: one word holds the 16 codes; register i holds (q[i], q[i+8]).
template <>
struct Unpack<2> {
    static constexpr int WORDS = 1;
    __device__ static __forceinline__ void run(const uint32_t (&w)[1], uint32_t (&p)[8]) {
        constexpr uint32_t MAGIC = 0x64006400u;
        // (1024 + 4^k q) * 4^-k - 1024 * 4^-k = q, exactly
        constexpr uint32_t S1 = 0x34003400u, C1 = 0xDC00DC00u;   // 0.25, -256
        constexpr uint32_t S2 = 0x2C002C00u, C2 = 0xD400D400u;   // 1/16, -64
        constexpr uint32_t S3 = 0x24002400u, C3 = 0xCC00CC00u;   // 1/64, -16
        constexpr uint32_t S4 = 0x1C001C00u, C4 = 0xC400C400u;   // 1/256, -4
        const uint32_t a = w[0], b = w[0] >> 10;
        p[0] = h2_sub((a & 0x00030003u) | MAGIC, MAGIC);
        p[1] = h2_fma((a & 0x000C000Cu) | MAGIC, S1, C1);
        p[2] = h2_fma((a & 0x00300030u) | MAGIC, S2, C2);
        p[3] = h2_fma((a & 0x00C000C0u) | MAGIC, S3, C3);
        p[4] = h2_fma((a & 0x03000300u) | MAGIC, S4, C4);
        p[5] = h2_sub((b & 0x00030003u) | MAGIC, MAGIC);
        p[6] = h2_fma((b & 0x000C000Cu) | MAGIC, S1, C1);
        p[7] = h2_fma((b & 0x00300030u) | MAGIC, S2, C2);
    }
};

}  // namespace

// Position of element e (0..15) of a 16-element segment in the permuted activation layout.
__host__ __device__ uint32_t perm_pos(uint32_t e, uint32_t bits) {
    if (bits == 4) {
        // layout: x0 x4 x1 x5 x2 x6 x3 x7 | x8 x12 x9 x13 x10 x14 x11 x15
        const uint32_t half = e & 8u, r = e & 7u;
        return half + ((r & 3u) << 1) + (r >> 2);
    }
    // layout: x0 x8 x1 x9 ... x7 x15
    return ((e & 7u) << 1) + (e >> 3);
}

namespace {

struct GroupRef {
    const uint8_t* blob;
    mfb_expert_offsets off;
    uint32_t bits, pair_start, pair_count;
    bool shared, ok;
};

// P.groups / P.sorted may live in global memory (separate kernels) or in shared memory (fused kernel).
__device__ __forceinline__ GroupRef group_ref(const FastParams& P, uint32_t g) {
    GroupRef v;
    const mfb_group grp = P.groups[g];
    v.shared = grp.expert >= P.num_experts;
    v.pair_start = grp.pair_start;
    v.pair_count = grp.pair_count;
    v.ok = true;
    if (v.shared) {
        v.blob = P.shared_blob; v.off = P.shared_off; v.bits = P.shared_bits;
        v.ok = P.shared_blob != nullptr;
    } else {
        int64_t slot = grp.expert;
        if (P.slot_of) slot = P.slot_of[grp.expert];
        v.ok = slot >= 0;
        v.blob = P.pool + (uint64_t)(slot < 0 ? 0 : slot) * P.slot_stride;
        v.off = P.routed_off; v.bits = P.bits;
    }
    return v;
}

// sum(x) over one 64-element group for this lane's two token columns (2t, 2t+1): four MMAs against an all-ones
// A fragment leave exactly those sums in c0 and c1 - no conversions, shuffles or shared memory.
__device__ __forceinline__ float2 group_sum(const uint32_t (&bf)[8]) {
    constexpr uint32_t ONES = 0x3C003C00u;
    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) mma16816(d, ONES, ONES, ONES, ONES, bf[2 * j], bf[2 * j + 1]);
    return make_float2(d[0], d[1]);
}

// One 64-element group of rows g and g+8 of one matrix: sum(code * x) by four MMAs, then the affine factors.
template <int BITS>
__device__ __forceinline__ void group_mma(const uint8_t* row_lo, const uint8_t* row_hi, uint32_t byte_off,
                                          const uint32_t (&bf)[8], float s_lo, float b_lo, float s_hi, float b_hi,
                                          float2 sx, float (&acc)[4]) {
    constexpr int W = Unpack<BITS>::WORDS;
    uint32_t wl[W], wh[W];
    if (W == 2) {
        const uint2 a = *reinterpret_cast<const uint2*>(row_lo + byte_off);
        const uint2 b = *reinterpret_cast<const uint2*>(row_hi + byte_off);
        wl[0] = a.x; wl[W - 1] = a.y; wh[0] = b.x; wh[W - 1] = b.y;
    } else {
        wl[0] = *reinterpret_cast<const uint32_t*>(row_lo + byte_off);
        wh[0] = *reinterpret_cast<const uint32_t*>(row_hi + byte_off);
    }
    uint32_t pl[8], ph[8];
    Unpack<BITS>::run(wl, pl);
    Unpack<BITS>::run(wh, ph);
    float dsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) mma16816(dsum, pl[2 * j], ph[2 * j], pl[2 * j + 1], ph[2 * j + 1], bf[2 * j], bf[2 * j + 1]);
    acc[0] = fmaf(s_lo, dsum[0], acc[0]); acc[0] = fmaf(b_lo, sx.x, acc[0]);
    acc[1] = fmaf(s_lo, dsum[1], acc[1]); acc[1] = fmaf(b_lo, sx.y, acc[1]);
    acc[2] = fmaf(s_hi, dsum[2], acc[2]); acc[2] = fmaf(b_hi, sx.x, acc[2]);
    acc[3] = fmaf(s_hi, dsum[3], acc[3]); acc[3] = fmaf(b_hi, sx.y, acc[3]);
}

// N consecutive 16-bit scales (or biases) of one row with the widest load that fits.
template <int N>
struct ScaleRow {
    uint32_t w[(N + 1) / 2];
    __device__ __forceinline__ void load(const uint16_t* p) {
        if (N == 8) { const uint4 v = *reinterpret_cast<const uint4*>(p); w[0] = v.x; w[(N > 2) ? 1 : 0] = v.y; w[(N > 4) ? 2 : 0] = v.z; w[(N > 6) ? 3 : 0] = v.w; }
        else if (N == 4) { const uint2 v = *reinterpret_cast<const uint2*>(p); w[0] = v.x; w[(N > 2) ? 1 : 0] = v.y; }
        else if (N == 2) w[0] = *reinterpret_cast<const uint32_t*>(p);
        else w[0] = *p;
    }
    __device__ __forceinline__ float at(int i, int dtype) const {
        const uint32_t h = (i & 1) ? (w[i >> 1] >> 16) : (w[i >> 1] & 0xFFFFu);
        return widen16((uint16_t)h, dtype);
    }
};

// ------------------------------------------------------------------------------------------ work lists
// A unit of work is one (group, token tile of up to 8 rows[, 32-row tile of gate/up]).  Exclusive prefix sums of
// the units of each group, by one warp: pref1[g] counts phase-1 units, pref2[g] phase-2 units.
__device__ __forceinline__ void warp_unit_prefix(const mfb_group* groups, uint32_t n_groups, uint32_t tiles_per_group,
                                                 uint32_t* pref1, uint32_t* pref2, uint32_t lane) {
    const uint32_t per = (n_groups + 31) / 32, g0 = lane * per;
    uint32_t local = 0;
    for (uint32_t j = 0; j < per; ++j)
        if (g0 + j < n_groups) local += (groups[g0 + j].pair_count + 7) / 8;
    uint32_t incl = local;
    for (uint32_t off = 1; off < 32; off <<= 1) {
        const uint32_t n = __shfl_up_sync(0xFFFFFFFFu, incl, off);
        if (lane >= off) incl += n;
    }
    uint32_t run = incl - local;
    for (uint32_t j = 0; j < per; ++j)
        if (g0 + j < n_groups) {
            pref2[g0 + j] = run;
            pref1[g0 + j] = run * tiles_per_group;
            run += (groups[g0 + j].pair_count + 7) / 8;
        }
    const uint32_t total = __shfl_sync(0xFFFFFFFFu, incl, 31);
    if (lane == 0) { pref2[n_groups] = total; pref1[n_groups] = total * tiles_per_group; }
    __syncwarp();
}

// Optional cycle accounting of CTA 0 (attached with the phase trace): counter k of warp w at dbg[w*8 + k].
__device__ __forceinline__ void dbg_add(unsigned long long* dbg, uint32_t warp, uint32_t lane, int k, long long t0) {
    if (dbg && blockIdx.x == 0 && lane == 0) dbg[warp * 8 + k] += (unsigned long long)(clock64() - t0);
}

// Advances `g` until unit u lies in group g (units are visited in increasing order).
__device__ __forceinline__ void seek_group(const uint32_t* pref, uint32_t n_groups, uint32_t u, uint32_t& g) {
    while (g + 1 < n_groups && pref[g + 1] <= u) ++g;
}

// ------------------------------------------------------------------------------------------ phase 1
// Stage = 32 rows of gate and 32 rows of up of one expert (+ their scales and biases).  Warp w of the 16 compute
// warps owns k range [ks*d/8, (ks+1)*d/8) (ks = w % 8) of row tile rt = w / 8; the partial sums of the eight k
// splits meet in shared memory in a fixed order.  The 17th warp issues the bulk copies: one per row (padded
// destination rows), one per scale block.
struct F1Geom {
    uint32_t tile_rows, tiles_per_group, blk_stride, mat_bytes, stage_bytes, groups_per_row, k_per_warp;
};

__host__ __device__ inline F1Geom f1_geom(uint32_t d, uint32_t f, uint32_t max_bits) {
    F1Geom g;
    g.tile_rows = 16 * RT;
    g.tiles_per_group = f / g.tile_rows;
    // a matrix tile of 32 rows is staged as four blocks of eight consecutive rows, one bulk copy each (the copy
    // unit sustains only a handful of copies in flight, so copies must be kilobytes, not rows); 32 pad bytes
    // after each block put the four rows that one shared-memory load phase touches into different banks
    g.blk_stride = 8 * (d * max_bits / 8) + ROW_PAD;
    g.mat_bytes = 4 * g.blk_stride;
    g.groups_per_row = d / 64;
    g.k_per_warp = d / KS;
    g.stage_bytes = 2 * g.mat_bytes + 4 * g.tile_rows * g.groups_per_row * 2;
    return g;
}

struct Phase1Ctx {
    uint8_t* stages;
    uint64_t* full;     // [F1_STAGES]
    uint64_t* empty;    // [F1_STAGES]
    float* red;         // [2][CW*32*8]
    const uint32_t* pref1;
};

// Copy-issuing side of one unit (all 32 lanes of the issuing warp call this).
__device__ __forceinline__ bool f1_produce(const FastParams& P, const F1Geom& geo, const Phase1Ctx& C, const GroupRef& G,
                                           uint32_t tile, uint32_t seq, uint32_t lane) {
    const uint32_t s = seq % F1_STAGES, ph = (seq / F1_STAGES) & 1u;
    if (!mbar_wait(&C.empty[s], ph ^ 1u)) return false;
    if (!G.ok) {   // nothing to copy: complete the phase so the consumers move on
        if (lane == 0) mbar_arrive(&C.full[s]);
        return true;
    }
    const uint32_t row0 = tile * geo.tile_rows;
    const uint32_t row_bytes = P.d * G.bits / 8, gpr = geo.groups_per_row;
    uint8_t* st = C.stages + s * geo.stage_bytes;
    const uint32_t scale_block = geo.tile_rows * gpr * 2;
    if (lane == 0) mbar_expect_tx(&C.full[s], 2 * geo.tile_rows * row_bytes + 4 * scale_block);
    __syncwarp();
    if (lane < 8) {          // blocks 0-3 of gate, 0-3 of up: eight consecutive rows each
        const bool up = lane >= 4;
        const uint32_t b = lane & 3;
        const uint8_t* src = G.blob + (up ? G.off.up_w : G.off.gate_w) + (size_t)(row0 + 8 * b) * row_bytes;
        bulk_g2s(st + (up ? geo.mat_bytes : 0) + b * geo.blk_stride, src, 8 * row_bytes, &C.full[s]);
    } else if (lane < 12) {
        const uint32_t m = lane - 8;
        const uint32_t o = m == 0 ? G.off.gate_s : (m == 1 ? G.off.gate_b : (m == 2 ? G.off.up_s : G.off.up_b));
        bulk_g2s(st + 2 * geo.mat_bytes + m * scale_block, G.blob + o + (size_t)row0 * gpr * 2, scale_block, &C.full[s]);
    }
    return true;
}

// B fragments of this warp's k range for token column g of a token tile (registers, loaded from L2 or, in the
// single-token mode of the fused kernel, from shared memory).
template <int NGW>
__device__ __forceinline__ void f1_load_x(const FastParams& P, const GroupRef& G, uint32_t tt, uint32_t k0, uint32_t lane,
                                          uint32_t (&bf)[NGW][8]) {
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t cols = min(8u, G.pair_count - tt * 8);
    const __half* xsrc = (G.shared && P.shared_bits != P.bits) ? P.xp_shared : P.xp;
    const __half* row = nullptr;
    if (g < cols) row = xsrc + (size_t)P.sorted[G.pair_start + tt * 8 + g].token * P.d + k0 + t * 16;
#pragma unroll
    for (int gi = 0; gi < NGW; ++gi) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
        if (row) {
            if (P.x_in_smem) { lo = *reinterpret_cast<const uint4*>(row + gi * 64); hi = *reinterpret_cast<const uint4*>(row + gi * 64 + 8); }
            else { lo = ld_cg_u4(row + gi * 64); hi = ld_cg_u4(row + gi * 64 + 8); }
        }
        bf[gi][0] = lo.x; bf[gi][1] = lo.y; bf[gi][2] = lo.z; bf[gi][3] = lo.w;
        bf[gi][4] = hi.x; bf[gi][5] = hi.y; bf[gi][6] = hi.z; bf[gi][7] = hi.w;
    }
}

// Row of a 32-row stage tile that MMA row (row tile rt, lane group g, upper half hi) works on.
__device__ __forceinline__ uint32_t tile_row(uint32_t rt, uint32_t g, uint32_t hi) {
    return (g & 3) * 8 + rt * 4 + hi * 2 + (g >> 2);
}

template <int BITS, int NGW>
__device__ __forceinline__ void f1_compute(const FastParams& P, const GroupRef& G, const F1Geom& geo, const uint8_t* stage,
                                           uint32_t tile, uint32_t tt, const uint32_t (&bf)[NGW][8], float2 (&sx)[NGW],
                                           bool fresh_x, uint32_t warp, uint32_t lane, float* red, uint32_t& red_buf) {
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t ks = warp % KS, rt = warp / KS;
    const uint32_t row_bytes = P.d * BITS / 8;
    const uint32_t gpr = geo.groups_per_row;
    const uint8_t* gate_rows = stage;
    const uint8_t* up_rows = stage + geo.mat_bytes;
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(stage + 2 * geo.mat_bytes);
    const uint32_t blk = geo.tile_rows * gpr;
    // MMA row (rt, g, +8) -> row of the 32-row tile: block g % 4, then rt, upper half, g / 4 inside the block
    const uint32_t r_lo = tile_row(rt, g, 0), r_hi = tile_row(rt, g, 1);
    const uint32_t a_lo = (g & 3) * geo.blk_stride + (r_lo & 7) * row_bytes, a_hi = a_lo + 2 * row_bytes;
    constexpr uint32_t lane_bytes = BITS == 4 ? 8 : 4, group_bytes = 64 * BITS / 8;
    const int sdt = (int)P.scale_dtype;
    const uint8_t* g_lo = gate_rows + a_lo, *g_hi = gate_rows + a_hi;
    const uint8_t* u_lo = up_rows + a_lo, *u_hi = up_rows + a_hi;
    const uint32_t cols = min(8u, G.pair_count - tt * 8);

    float ag[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
    // scales and biases of this warp's NGW groups, rows r_lo / r_hi of gate_s, gate_b, up_s, up_b
    ScaleRow<NGW> sr[8];
#pragma unroll
    for (int m = 0; m < 4; ++m) {
        sr[2 * m].load(sc + m * blk + r_lo * gpr + ks * NGW);
        sr[2 * m + 1].load(sc + m * blk + r_hi * gpr + ks * NGW);
    }
#pragma unroll
    for (int gi = 0; gi < NGW; ++gi) {
        const uint32_t boff = (ks * NGW + gi) * group_bytes + t * lane_bytes;
        if (fresh_x) sx[gi] = group_sum(bf[gi]);   // the sums stay valid for every row tile of this token tile
        const float2 sxv = sx[gi];
        group_mma<BITS>(g_lo, g_hi, boff, bf[gi], sr[0].at(gi, sdt), sr[2].at(gi, sdt), sr[1].at(gi, sdt), sr[3].at(gi, sdt), sxv, ag);
        group_mma<BITS>(u_lo, u_hi, boff, bf[gi], sr[4].at(gi, sdt), sr[6].at(gi, sdt), sr[5].at(gi, sdt), sr[7].at(gi, sdt), sxv, au);
    }
    // partial sums of this warp -> shared memory, then a fixed-order sum over the k splits
    float* rb = red + red_buf * (CW * 32 * 8);
    float4* dst = reinterpret_cast<float4*>(rb + ((ks * RT + rt) * 32 + lane) * 8);
    dst[0] = make_float4(ag[0], ag[1], ag[2], ag[3]);
    dst[1] = make_float4(au[0], au[1], au[2], au[3]);
    named_barrier(1, CW * 32);
    const uint32_t o = warp * 32 + lane;
    if (o < RT * 128) {
        const uint32_t ort = o >> 7, row = (o & 127) >> 3, n = o & 7;
        const uint32_t src_lane = (row & 7) * 4 + (n >> 1), reg = (row >> 3) * 2 + (n & 1);
        float gsum = 0.0f, usum = 0.0f;
#pragma unroll
        for (uint32_t k = 0; k < KS; ++k) {
            const float* src = rb + ((k * RT + ort) * 32 + src_lane) * 8;
            gsum += src[reg];
            usum += src[4 + reg];
        }
        if (n < cols) {
            if (!G.shared && P.limit > 0.0f) {   // moe_swiglu_clamp (moe.metal:27-34), routed experts only
                gsum = fminf(gsum, P.limit);
                usum = fminf(fmaxf(usum, -P.limit), P.limit);
            }
            float a = hidden_act(gsum, (int)P.activation) * usum;
            a = fminf(fmaxf(a, -65504.0f), 65504.0f);
            const uint32_t r = tile * geo.tile_rows + tile_row(ort, row & 7, row >> 3);
            const uint32_t pos = (r & ~15u) + perm_pos(r & 15u, G.bits);
            P.actp[(size_t)(G.pair_start + tt * 8 + n) * P.f + pos] = __float2half_rn(a);
        }
    }
    red_buf ^= 1u;
}

// Runs this CTA's share of phase 1: units [first, last) of the flattened (group, token tile, row tile) list.
// `seq` is the number of units the CTA has processed since its barriers were initialised (all warps keep it).
template <int NGW>
__device__ __forceinline__ bool phase1(const FastParams& P, const F1Geom& geo, const Phase1Ctx& C, uint32_t n_groups,
                                       uint32_t first, uint32_t last, uint32_t& seq, uint32_t warp, uint32_t lane) {
    bool ok = true;
    uint32_t g = 0, local_seq = seq;
    if (warp == CW) {
        fence_proxy_async();
        for (uint32_t u = first; u < last && ok; ++u, ++local_seq) {
            seek_group(C.pref1, n_groups, u, g);
            const GroupRef G = group_ref(P, g);
            const long long t0 = clock64();
            ok = f1_produce(P, geo, C, G, (u - C.pref1[g]) % geo.tiles_per_group, local_seq, lane);
            dbg_add(P.dbg, warp, lane, 0, t0);
        }
    } else {
        uint32_t bf[NGW][8];
        float2 sx[NGW];
        uint32_t cached = 0xFFFFFFFFu, red_buf = 0;
        const uint32_t k0 = (warp % KS) * geo.k_per_warp;
        for (uint32_t u = first; u < last && ok; ++u, ++local_seq) {
            seek_group(C.pref1, n_groups, u, g);
            const GroupRef G = group_ref(P, g);
            const uint32_t local = u - C.pref1[g], tt = local / geo.tiles_per_group, tile = local % geo.tiles_per_group;
            const uint32_t key = g * 16 + tt;
            const bool fresh_x = G.ok && key != cached;
            if (fresh_x) { f1_load_x<NGW>(P, G, tt, k0, lane, bf); cached = key; }   // issued before the wait below
            const uint32_t s = local_seq % F1_STAGES, ph = (local_seq / F1_STAGES) & 1u;
            long long t0 = clock64();
            if (!mbar_wait(&C.full[s], ph)) { ok = false; break; }
            dbg_add(P.dbg, warp, lane, 0, t0);
            t0 = clock64();
            if (G.ok) {
                const uint8_t* st = C.stages + s * geo.stage_bytes;
                if (G.bits == 4) f1_compute<4, NGW>(P, G, geo, st, tile, tt, bf, sx, fresh_x, warp, lane, C.red, red_buf);
                else f1_compute<2, NGW>(P, G, geo, st, tile, tt, bf, sx, fresh_x, warp, lane, C.red, red_buf);
            }
            __syncwarp();
            dbg_add(P.dbg, warp, lane, 1, t0);
            if (lane == 0) mbar_arrive(&C.empty[s]);
        }
    }
    seq += last > first ? last - first : 0;
    return ok;
}

// ------------------------------------------------------------------------------------------ phase 2 + combine
// One CTA per block of 16 output rows (columns of the hidden state).  Units (group, token tile) flow through a
// ring of slots: the copy warp deposits the group's 16 down rows, their scales and the token tile's hidden
// activation rows; compute warp u % 16 multiplies them and leaves 16 x (tokens) results in a CTA-wide array
// indexed by (token, rank slot).  When every unit is done the CTA applies the routing weights in rank order,
// residual first, and writes its 16 columns of every token row: moe_phase2_down_reduce_k8 (moe.metal:349-404)
// without a partials buffer in global memory.
struct F2Geom {
    uint32_t row_stride_max, gpr, act_stride, scale_off, act_off, slot_bytes;
};

__host__ __device__ inline F2Geom f2_geom(uint32_t f, uint32_t max_bits) {
    F2Geom g;
    g.row_stride_max = f * max_bits / 8;   // rows stay contiguous: one warp computes a unit, so bank conflicts cost little
    g.gpr = f / 64;
    g.act_stride = f * 2;
    g.scale_off = 16 * g.row_stride_max;
    g.act_off = g.scale_off + 2 * 16 * g.gpr * 2;
    g.slot_bytes = (g.act_off + 8 * g.act_stride + 127u) & ~127u;
    return g;
}

struct Phase2Ctx {
    uint8_t* slots;
    uint64_t* full;    // [F2_SLOTS]
    uint64_t* empty;   // [F2_SLOTS]
    float* part;       // [n_tokens][top_k + 1][16]
    const uint32_t* pref2;
};

// Copy-issuing side of up to eight consecutive units at once: lanes 4j..4j+3 of the issuing warp serve unit
// first_unit + j (wait for its slot, post the byte count, then one copy per lane: the 16 contiguous rows, their
// scales, their biases, the token tile's activation rows).  Issuing is latency bound per unit, so the eight units
// of a pass overlap their waits and address arithmetic.  `g` is this lane's group cursor.
__device__ __forceinline__ bool f2_produce8(const FastParams& P, const F2Geom& geo, const Phase2Ctx& C, uint32_t n_groups,
                                            uint32_t n_units, uint32_t first_unit, uint32_t row0, uint32_t seq, uint32_t lane,
                                            uint32_t& g) {
    const uint32_t u = first_unit + (lane >> 2), role = lane & 3;
    const bool active = u < n_units;
    bool ok = true, copy = false;
    GroupRef G;
    uint32_t s = 0, tt = 0;
    if (active) {
        seek_group(C.pref2, n_groups, u, g);
        G = group_ref(P, g);
        tt = u - C.pref2[g];
        s = (seq + u) % F2_SLOTS;
        ok = mbar_wait(&C.empty[s], (((seq + u) / F2_SLOTS) & 1u) ^ 1u);
        copy = ok && G.ok;
        if (ok && role == 0) {
            if (G.ok) {
                const uint32_t cols = min(8u, G.pair_count - tt * 8);
                mbar_expect_tx(&C.full[s], 16 * (P.f * G.bits / 8) + 2 * (16 * geo.gpr * 2) + cols * P.f * 2);
            } else {
                mbar_arrive(&C.full[s]);   // nothing to copy: complete the phase so the consumer moves on
            }
        }
    }
    __syncwarp();   // every byte count is posted before any copy of this pass is issued
    if (copy) {
        const uint32_t row_bytes = P.f * G.bits / 8, scale_block = 16 * geo.gpr * 2;
        uint8_t* st = C.slots + s * geo.slot_bytes;
        if (role == 0) bulk_g2s(st, G.blob + G.off.down_w + (size_t)row0 * row_bytes, 16 * row_bytes, &C.full[s]);
        else if (role < 3)
            bulk_g2s(st + geo.scale_off + (role - 1) * scale_block,
                     G.blob + (role == 1 ? G.off.down_s : G.off.down_b) + (size_t)row0 * geo.gpr * 2, scale_block, &C.full[s]);
        else {
            const uint32_t cols = min(8u, G.pair_count - tt * 8);
            bulk_g2s(st + geo.act_off, P.actp + (size_t)(G.pair_start + tt * 8) * P.f, cols * P.f * 2, &C.full[s]);
        }
    }
    return __all_sync(0xFFFFFFFFu, ok);
}

template <int BITS, int NG>
__device__ __forceinline__ void f2_compute(const FastParams& P, const F2Geom& geo, const GroupRef& G, uint32_t tt,
                                           const uint8_t* st, uint32_t lane, float* part, uint32_t slots) {
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t row_stride = P.f * BITS / 8;
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(st + geo.scale_off);
    constexpr uint32_t lane_bytes = BITS == 4 ? 8 : 4, group_bytes = 64 * BITS / 8;
    const int sdt = (int)P.scale_dtype;
    ScaleRow<NG> s_lo, s_hi, b_lo, b_hi;
    s_lo.load(sc + g * NG); s_hi.load(sc + (g + 8) * NG);
    b_lo.load(sc + 16 * NG + g * NG); b_hi.load(sc + 16 * NG + (g + 8) * NG);
    const uint32_t cols = min(8u, G.pair_count - tt * 8);
    const uint8_t* act_row = st + geo.act_off + g * geo.act_stride + t * 32;   // columns >= cols hold stale rows: unused
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
        uint32_t bf[8];
        const uint4 lo = *reinterpret_cast<const uint4*>(act_row + gi * 128);
        const uint4 hi = *reinterpret_cast<const uint4*>(act_row + gi * 128 + 16);
        bf[0] = lo.x; bf[1] = lo.y; bf[2] = lo.z; bf[3] = lo.w; bf[4] = hi.x; bf[5] = hi.y; bf[6] = hi.z; bf[7] = hi.w;
        group_mma<BITS>(st + g * row_stride, st + (g + 8) * row_stride, gi * group_bytes + t * lane_bytes, bf,
                        s_lo.at(gi, sdt), b_lo.at(gi, sdt), s_hi.at(gi, sdt), b_hi.at(gi, sdt), group_sum(bf), acc);
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const uint32_t n = 2 * t + c;
        if (n < cols) {
            const mfb_pair pr = P.sorted[G.pair_start + tt * 8 + n];
            float* dst = part + ((size_t)pr.token * slots + pr.rank) * 16;
            dst[g] = acc[c];
            dst[g + 8] = acc[2 + c];
        }
    }
}

template <int BITS>
__device__ __forceinline__ void f2_dispatch(const FastParams& P, const F2Geom& geo, const GroupRef& G, uint32_t tt,
                                            const uint8_t* st, uint32_t lane, float* part, uint32_t slots) {
    switch (geo.gpr) {
        case 8: f2_compute<BITS, 8>(P, geo, G, tt, st, lane, part, slots); break;
        case 4: f2_compute<BITS, 4>(P, geo, G, tt, st, lane, part, slots); break;
        case 2: f2_compute<BITS, 2>(P, geo, G, tt, st, lane, part, slots); break;
        default: f2_compute<BITS, 1>(P, geo, G, tt, st, lane, part, slots); break;
    }
}

// Runs phase 2 for the 16 output rows starting at row0 over all units; `seq` as in phase1.
__device__ __forceinline__ bool phase2(const FastParams& P, const F2Geom& geo, const Phase2Ctx& C, uint32_t n_groups,
                                       uint32_t row0, uint32_t& seq, uint32_t warp, uint32_t lane) {
    const uint32_t n_units = C.pref2[n_groups], slots = P.top_k + 1;
    bool ok = true;
    uint32_t g = 0;
    if (warp == CW) {
        fence_proxy_async();
        for (uint32_t u = 0; u < n_units && ok; u += 8) {
            const long long t0 = clock64();
            ok = f2_produce8(P, geo, C, n_groups, n_units, u, row0, seq, lane, g);
            dbg_add(P.dbg, warp, lane, 2, t0);
        }
    } else if (warp < (uint32_t)F2_SLOTS) {
        // Compute warp w serves slot w only, so its waits on that slot's barriers follow each other in phase order.
        // (A parity wait is only meaningful one phase ahead: a warp that started a whole lap ahead of its slot would
        // see the not-yet-started previous phase as complete.)
        const uint32_t u0 = (warp + F2_SLOTS - seq % F2_SLOTS) % F2_SLOTS;
        for (uint32_t u = u0; u < n_units && ok; u += F2_SLOTS) {
            seek_group(C.pref2, n_groups, u, g);
            const GroupRef G = group_ref(P, g);
            const uint32_t s = (seq + u) % F2_SLOTS, ph = ((seq + u) / F2_SLOTS) & 1u;
            long long t0 = clock64();
            if (!mbar_wait(&C.full[s], ph)) { ok = false; break; }
            dbg_add(P.dbg, warp, lane, 2, t0);
            t0 = clock64();
            if (G.ok) {
                const uint8_t* st = C.slots + s * geo.slot_bytes;
                if (G.bits == 4) f2_dispatch<4>(P, geo, G, u - C.pref2[g], st, lane, C.part, slots);
                else f2_dispatch<2>(P, geo, G, u - C.pref2[g], st, lane, C.part, slots);
            }
            __syncwarp();
            dbg_add(P.dbg, warp, lane, 3, t0);
            if (lane == 0) mbar_arrive(&C.empty[s]);
        }
    }
    seq += n_units;
    return ok;
}

// Rank-ordered weighted combine of this CTA's 16 columns: residual first, shared expert, then ranks ascending.
__device__ __forceinline__ void f2_combine(const FastParams& P, const float* part, uint32_t slots, uint32_t row0, bool with_shared) {
    for (uint32_t o = threadIdx.x; o < P.n_tokens * 16; o += blockDim.x) {
        const uint32_t tok = o >> 4, r = o & 15;
        const float* pt = part + (size_t)tok * slots * 16;
        float acc = 0.0f;
        if (P.residual) acc = widen16(ld_cg_u16((const uint16_t*)P.residual + (size_t)tok * P.d + row0 + r), P.x_dtype);
        if (with_shared) acc += pt[P.top_k * 16 + r];
        for (uint32_t k = 0; k < P.top_k; ++k)
            acc = fmaf(__half2float(__ushort_as_half(P.route_w[(size_t)tok * P.top_k + k])), pt[k * 16 + r], acc);
        store_act(P.y, (size_t)tok * P.d + row0 + r, acc, P.x_dtype);
    }
}

// ------------------------------------------------------------------------------------------ separate kernels
struct FastShared {
    uint64_t full1[F1_STAGES], empty1[F1_STAGES], full2[F2_SLOTS], empty2[F2_SLOTS];
    uint32_t pref1[MAX_GROUPS + 1], pref2[MAX_GROUPS + 1];
    uint32_t flag, n_groups;
    float red[32];
};

__device__ __forceinline__ void init_barriers(FastShared& S) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < F1_STAGES; ++s) { mbar_init(&S.full1[s], 1); mbar_init(&S.empty1[s], CW); }
        for (int s = 0; s < F2_SLOTS; ++s) { mbar_init(&S.full2[s], 1); mbar_init(&S.empty2[s], 1); }
        fence_barrier_init();
    }
    __syncthreads();
}

template <int NGW>
__global__ void __launch_bounds__(FAST_THREADS, 1) ffn1_mma_kernel(const FastParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ FastShared S;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t max_bits = P.shared_blob && P.shared_bits > P.bits ? P.shared_bits : P.bits;
    const F1Geom geo = f1_geom(P.d, P.f, max_bits);
    init_barriers(S);
    const uint32_t n_groups = *P.n_groups;
    if (warp == 0) warp_unit_prefix(P.groups, n_groups, geo.tiles_per_group, S.pref1, S.pref2, lane);
    __syncthreads();
    Phase1Ctx C{smem, S.full1, S.empty1, reinterpret_cast<float*>(smem + F1_STAGES * geo.stage_bytes), S.pref1};
    const uint32_t n_units = S.pref1[n_groups];
    const uint32_t per_cta = (n_units + gridDim.x - 1) / gridDim.x;
    const uint32_t first = min(blockIdx.x * per_cta, n_units), last = min(first + per_cta, n_units);
    uint32_t seq = 0;
    if (!phase1<NGW>(P, geo, C, n_groups, first, last, seq, warp, lane)) atomicOr(P.status, STATUS_MBAR_TIMEOUT);
}

__global__ void __launch_bounds__(FAST_THREADS, 1) ffn2_mma_kernel(const FastParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ FastShared S;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t max_bits = P.shared_blob && P.shared_bits > P.bits ? P.shared_bits : P.bits;
    const F2Geom geo = f2_geom(P.f, max_bits);
    const uint32_t slots = P.top_k + 1;
    float* part = reinterpret_cast<float*>(smem + F2_SLOTS * geo.slot_bytes);
    init_barriers(S);
    const uint32_t n_groups = *P.n_groups;
    if (warp == 0) warp_unit_prefix(P.groups, n_groups, 1, S.pref1, S.pref2, lane);
    for (uint32_t i = threadIdx.x; i < P.n_tokens * slots * 16; i += blockDim.x) part[i] = 0.0f;
    __syncthreads();
    Phase2Ctx C{smem, S.full2, S.empty2, part, S.pref2};
    uint32_t seq = 0;
    if (!phase2(P, geo, C, n_groups, blockIdx.x * 16, seq, warp, lane)) atomicOr(P.status, STATUS_MBAR_TIMEOUT);
    __syncthreads();
    f2_combine(P, part, slots, blockIdx.x * 16, P.shared_blob != nullptr);
}

// ------------------------------------------------------------------------------------------ prep: RMSNorm + layouts
// Same arithmetic as rmsnorm_kernel (glue.cu), so the normalised rows are bit-identical; additionally writes the
// rows as fp16 in the permuted order the MMA fragments read (one copy per distinct code width).
__global__ void prep_kernel(const void* __restrict__ h, int dtype, const __nv_bfloat16* __restrict__ w, uint32_t d, float eps,
                            int do_norm, void* __restrict__ xn, __half* __restrict__ xp, uint32_t bits,
                            __half* __restrict__ xp2, uint32_t bits2) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    float inv = 1.0f;
    if (do_norm) {
        float ss = 0.0f;
        for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
            const float v = load_act(h, row * d + i, dtype);
            ss = fmaf(v, v, ss);
        }
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, off);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        if (threadIdx.x < 32) {
            float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0f;
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            if (threadIdx.x == 0) red[0] = v;
        }
        __syncthreads();
        inv = rsqrtf(red[0] / (float)d + eps);
    }
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        float v = load_act(h, row * d + i, dtype);
        if (do_norm) {
            const float g = w ? __bfloat162float(w[i]) : 1.0f;
            v = v * inv * g;
            store_act(xn, row * d + i, v, dtype);
            v = widen16(narrow16(v, dtype), dtype);   // the FFN consumes the rounded row, as the layer-by-layer path does
        }
        v = fminf(fmaxf(v, -65504.0f), 65504.0f);
        const __half hv = __float2half_rn(v);
        xp[row * d + (i & ~15u) + perm_pos(i & 15u, bits)] = hv;
        if (xp2) xp2[row * d + (i & ~15u) + perm_pos(i & 15u, bits2)] = hv;
    }
}

// ------------------------------------------------------------------------------------------ fused stack kernel
// All layers of a decode step in ONE cooperative launch: RMSNorm, gate GEMV, top-k, sort, phase 1, phase 2 and
// the weighted combine, with grid-wide barriers between dependent phases.  At batch 1 a layer moves 17 MB, which
// HBM delivers in under 3 us - less than a kernel launch - so the per-layer launch sequence is latency bound by
// construction; here the only serial costs left are the barriers and the memory latency behind them.
//
// Every wait is bounded: a barrier or mbarrier that does not complete within its limit sets the abort word and
// the device status, every CTA then falls through its remaining barriers and returns; nothing spins for ever.
constexpr long long GRID_WAIT_CYCLES = 1500000000ll;   // ~0.8 s at 1.9 GHz

// Arrive-and-wait over all CTAs.  `epoch` counts the arrivals this CTA expects to have been made in total.
__device__ __forceinline__ bool grid_barrier(const MegaParams& M, FastShared& S, uint32_t& epoch) {
    __syncthreads();
    if (threadIdx.x == 0) {
        epoch += gridDim.x;
        __threadfence();
        atomicAdd(M.bar_counter, 1u);
        bool ok = true;
        const long long t0 = clock64();
        while (ld_acquire_u32(M.bar_counter) < epoch) {
            if (ld_acquire_u32(M.abort) != 0u) { ok = false; break; }
            if (clock64() - t0 > GRID_WAIT_CYCLES) {
                atomicOr(M.status, STATUS_GRID_BARRIER_TIMEOUT);
                atomicExch(M.abort, 1u);
                ok = false;
                break;
            }
        }
        __threadfence();
        S.flag = ok ? 1u : 0u;
    }
    __syncthreads();
    return S.flag != 0u;
}

// RMSNorm of one row by the first 256 threads of the CTA, arithmetic and order of rmsnorm_kernel (glue.cu).
// Writes the row in the activation dtype and in the permuted fp16 layout(s); the outputs may be global or shared.
__device__ __forceinline__ void mega_norm_row(const MegaParams& M, const MegaLayer& Ly, FastShared& S, const void* h,
                                              uint32_t tok, uint16_t* xn_out, __half* xp_out, __half* xp2_out) {
    const uint32_t d = M.d, tid = threadIdx.x;
    const uint16_t* src = (const uint16_t*)h + (size_t)tok * d;
    float ss = 0.0f;
    if (tid < 256) {
#pragma unroll 8
        for (uint32_t i = tid; i < d; i += 256) {
            const float v = widen16(ld_cg_u16(src + i), M.x_dtype);
            ss = fmaf(v, v, ss);
        }
    }
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, off);
    if (tid < 256 && (tid & 31) == 0) S.red[tid >> 5] = ss;
    __syncthreads();
    if (tid < 32) {
        float v = tid < 8 ? S.red[tid] : 0.0f;
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
        if (tid == 0) S.red[8] = v;
    }
    __syncthreads();
    const float inv = rsqrtf(S.red[8] / (float)d + M.eps);
    if (tid < 256) {
#pragma unroll 8
        for (uint32_t i = tid; i < d; i += 256) {
            float v = widen16(ld_cg_u16(src + i), M.x_dtype);
            const float gw = Ly.norm_w ? __bfloat162float(Ly.norm_w[i]) : 1.0f;
            v = v * inv * gw;
            const uint16_t bits = narrow16(v, M.x_dtype);
            xn_out[i] = bits;
            v = fminf(fmaxf(widen16(bits, M.x_dtype), -65504.0f), 65504.0f);
            const __half hv = __float2half_rn(v);
            xp_out[(i & ~15u) + perm_pos(i & 15u, M.bits)] = hv;
            if (xp2_out) xp2_out[(i & ~15u) + perm_pos(i & 15u, M.shared_bits)] = hv;
        }
    }
    __syncthreads();
}

// logits[t, e] for the experts this CTA owns (e = blockIdx.x, + gridDim.x, ...), every token, in the fixed
// summation order of router_logits_kernel: lane l takes k = l, l+32, ... ascending, then a xor butterfly.
// `stage` is free shared memory: up to two gate rows as fp32, then one activation row per warp as raw 16-bit.
// With x_smem the single activation row is already in shared memory.
constexpr uint32_t MEGA_ROWS_PER_PASS = 2;

__device__ __forceinline__ void mega_logits(const MegaParams& M, const MegaLayer& Ly, uint8_t* stage, const uint16_t* x_smem) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5, d = M.d;
    float* w_rows = reinterpret_cast<float*>(stage);                                                   // [2][d]
    uint16_t* x_stage = reinterpret_cast<uint16_t*>(stage + MEGA_ROWS_PER_PASS * d * 4) + warp * d;    // [warps][d]
    for (uint32_t e0 = blockIdx.x; e0 < M.num_experts; e0 += MEGA_ROWS_PER_PASS * gridDim.x) {
        __syncthreads();
        uint32_t ne = 0;
        for (uint32_t j = 0; j < MEGA_ROWS_PER_PASS; ++j) {
            const uint32_t e = e0 + j * gridDim.x;
            if (e >= M.num_experts) break;
            ++ne;
            const uint4* src = reinterpret_cast<const uint4*>(Ly.router_w + (size_t)e * d);
            for (uint32_t i = threadIdx.x; i < d / 8; i += blockDim.x) {
                const uint4 q = src[i];
                float* dst = w_rows + j * d + i * 8;
                dst[0] = __uint_as_float(q.x << 16); dst[1] = __uint_as_float(q.x & 0xFFFF0000u);
                dst[2] = __uint_as_float(q.y << 16); dst[3] = __uint_as_float(q.y & 0xFFFF0000u);
                dst[4] = __uint_as_float(q.z << 16); dst[5] = __uint_as_float(q.z & 0xFFFF0000u);
                dst[6] = __uint_as_float(q.w << 16); dst[7] = __uint_as_float(q.w & 0xFFFF0000u);
            }
        }
        __syncthreads();
        for (uint32_t t = warp; t < M.n_tokens; t += warps) {
            const uint16_t* x_row = x_smem;
            if (!x_smem) {
                const uint16_t* x = (const uint16_t*)M.xn + (size_t)t * d;
                __syncwarp();
                for (uint32_t i = lane; i < d / 8; i += 32) *reinterpret_cast<uint4*>(x_stage + i * 8) = ld_cg_u4(x + i * 8);
                __syncwarp();
                x_row = x_stage;
            }
            float acc[MEGA_ROWS_PER_PASS] = {0.0f, 0.0f};
#pragma unroll 8
            for (uint32_t i = lane; i < d; i += 32) {
                const float xv = widen16(x_row[i], M.x_dtype);
#pragma unroll
                for (uint32_t j = 0; j < MEGA_ROWS_PER_PASS; ++j) acc[j] = fmaf(w_rows[j * d + i], xv, acc[j]);
            }
#pragma unroll
            for (uint32_t j = 0; j < MEGA_ROWS_PER_PASS; ++j) {
                float v = acc[j];
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                const uint32_t e = e0 + j * gridDim.x;
                if (lane == 0 && j < ne) {
                    if (Ly.logit_bias) v = v + Ly.logit_bias[e];
                    M.logits[(size_t)t * M.num_experts + e] = v;
                }
            }
        }
    }
    __syncthreads();
}

// Counting sort of the routing table into shared memory, identical order to group.cu / route_small_kernel; every
// CTA builds the same lists.  run_s is scratch of num_experts entries.  Warp 0 does the scans with shuffles.
__device__ __forceinline__ void mega_group(const MegaParams& M, FastShared& S, const uint32_t* idx_s, const uint16_t* w_s,
                                           uint32_t* run_s, mfb_pair* sorted_s, mfb_group* groups_s, bool shared) {
    const uint32_t n_pairs = M.n_tokens * M.top_k, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t e = threadIdx.x; e < M.num_experts; e += blockDim.x) run_s[e] = 0;
    __syncthreads();
    for (uint32_t p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&run_s[idx_s[p]], 1u);
    __syncthreads();
    if (warp == 0) {
        const uint32_t per = (M.num_experts + 31) / 32, e0 = lane * per;
        uint32_t cnt = 0, nz = 0;
        for (uint32_t j = 0; j < per; ++j)
            if (e0 + j < M.num_experts) { const uint32_t c = run_s[e0 + j]; cnt += c; nz += c ? 1u : 0u; }
        uint32_t cnt_incl = cnt, nz_incl = nz;
        for (uint32_t off = 1; off < 32; off <<= 1) {
            const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, cnt_incl, off), b = __shfl_up_sync(0xFFFFFFFFu, nz_incl, off);
            if (lane >= off) { cnt_incl += a; nz_incl += b; }
        }
        uint32_t run = cnt_incl - cnt, gi = nz_incl - nz;
        for (uint32_t j = 0; j < per; ++j)
            if (e0 + j < M.num_experts) {
                const uint32_t c = run_s[e0 + j];
                run_s[e0 + j] = run;
                if (c) { groups_s[gi].expert = e0 + j; groups_s[gi].pair_start = run; groups_s[gi].pair_count = c; ++gi; }
                run += c;
            }
        uint32_t ng = __shfl_sync(0xFFFFFFFFu, nz_incl, 31);
        if (lane == 0) {
            if (shared) { groups_s[ng].expert = M.num_experts; groups_s[ng].pair_start = n_pairs; groups_s[ng].pair_count = M.n_tokens; ++ng; }
            S.n_groups = ng;
        }
        __syncwarp();
        // ordered scatter: 32 pairs per round in (token, rank) order
        for (uint32_t p0 = 0; p0 < n_pairs; p0 += 32) {
            const uint32_t p = p0 + lane;
            const uint32_t e = p < n_pairs ? idx_s[p] : 0xFFFFFFFFu;
            const uint32_t peers = __match_any_sync(0xFFFFFFFFu, e);
            const uint32_t before = __popc(peers & ((1u << lane) - 1u));
            uint32_t pos = 0;
            if (p < n_pairs) pos = run_s[e] + before;
            __syncwarp();
            if (p < n_pairs && before == 0) run_s[e] += __popc(peers);
            __syncwarp();
            if (p < n_pairs) {
                mfb_pair out;
                out.token = p / M.top_k; out.expert = e; out.rank = p % M.top_k; out.weight_bits = w_s[p];
                sorted_s[pos] = out;
            }
        }
    } else if (shared) {
        for (uint32_t t = threadIdx.x - 32; t < M.n_tokens; t += blockDim.x - 32) {
            mfb_pair out;
            out.token = t; out.expert = M.num_experts; out.rank = M.top_k; out.weight_bits = 0x3C00u;
            sorted_s[n_pairs + t] = out;
        }
    }
    __syncthreads();
}

template <int NGW>
__global__ void __launch_bounds__(FAST_THREADS, 1) stack_mega_kernel(const MegaParams M) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ FastShared S;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t max_bits = M.shared_bits > M.bits ? M.shared_bits : M.bits;
    const F1Geom geo1 = f1_geom(M.d, M.f, max_bits);
    const F2Geom geo2 = f2_geom(M.f, max_bits);
    const uint32_t slots = M.top_k + 1, n_pairs = M.n_tokens * M.top_k;
    const bool single = M.n_tokens == 1;
    // ---- shared memory carve-up.  Region A holds the two phase-1 stages and the k-split exchange buffer; phase 2
    // reuses it for its slot ring and the per-(token, slot) partial rows.  The routing lists follow it.
    uint8_t* region_a = smem;
    const uint32_t region_a_bytes = F1_STAGES * geo1.stage_bytes + 2 * CW * 32 * 8 * 4;
    float* red = reinterpret_cast<float*>(smem + F1_STAGES * geo1.stage_bytes);
    float* part = reinterpret_cast<float*>(region_a + F2_SLOTS * geo2.slot_bytes);
    mfb_pair* sorted_s = reinterpret_cast<mfb_pair*>(smem + region_a_bytes);
    mfb_group* groups_s = reinterpret_cast<mfb_group*>(sorted_s + (n_pairs + M.n_tokens));
    uint32_t* idx_s = reinterpret_cast<uint32_t*>(groups_s + (M.num_experts + 1));
    uint16_t* w_s = reinterpret_cast<uint16_t*>(idx_s + n_pairs);
    uint32_t* run_s = reinterpret_cast<uint32_t*>(w_s + ((n_pairs + 1) & ~1u));
    // single-token mode keeps the normalised row in shared memory (16-byte aligned)
    uint16_t* xn_s = reinterpret_cast<uint16_t*>((reinterpret_cast<uintptr_t>(run_s + M.num_experts) + 15) & ~(uintptr_t)15);
    __half* xp_s = reinterpret_cast<__half*>(xn_s + M.d);
    __half* xp2_s = xp_s + M.d;

    init_barriers(S);
    uint32_t epoch = 0, seq1 = 0, seq2 = 0;
    bool alive = true;
    for (uint32_t l = 0; l < M.n_layers && alive; ++l) {
        const MegaLayer Ly = M.layers[l];
        void* h = (uint8_t*)M.hidden + (size_t)l * M.layer_stride * 2;   // 16-bit activations
        const bool shared = Ly.shared_blob != nullptr;
        uint64_t* trace = M.trace ? M.trace + (size_t)l * 8 : nullptr;
        auto stamp = [&](int slot) {
            if (trace && blockIdx.x == 0 && threadIdx.x == 0) {
                uint64_t t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                trace[slot] = t;
            }
        };
        stamp(0);
        if (single) {
            // every CTA normalises the one row itself (no barrier), computes the logits of its experts, and after
            // the barrier every CTA repeats the selection: two grid barriers fewer per layer
            mega_norm_row(M, Ly, S, h, 0, xn_s, xp_s, M.xp2 ? xp2_s : nullptr);
            stamp(1);
            mega_logits(M, Ly, region_a, xn_s);
            if (!(alive = grid_barrier(M, S, epoch))) break;
            stamp(2);
            float* lg_s = red;
            for (uint32_t e = threadIdx.x; e < M.num_experts; e += blockDim.x) lg_s[e] = ld_cg_f32(M.logits + e);
            __syncthreads();
            if (warp == 0) {
                uint32_t e = 0;
                uint16_t wgt = 0;
                select_row(lg_s, M.num_experts, M.top_k, M.router_mode, Ly.per_expert_scale, Ly.correction_bias, M.route_scale,
                           lane, e, wgt);
                if (lane < M.top_k) {
                    w_s[lane] = wgt;
                    groups_s[lane].expert = e; groups_s[lane].pair_start = lane; groups_s[lane].pair_count = 1;
                    mfb_pair pr; pr.token = 0; pr.expert = e; pr.rank = lane; pr.weight_bits = wgt;
                    sorted_s[lane] = pr;
                    if (blockIdx.x == 0) { M.idx[lane] = e; M.route_w[lane] = wgt; }
                }
                if (lane == 0) {
                    uint32_t ng = M.top_k;
                    if (shared) {
                        groups_s[ng].expert = M.num_experts; groups_s[ng].pair_start = ng; groups_s[ng].pair_count = 1;
                        mfb_pair pr; pr.token = 0; pr.expert = M.num_experts; pr.rank = M.top_k; pr.weight_bits = 0x3C00u;
                        sorted_s[ng] = pr;
                        ++ng;
                    }
                    S.n_groups = ng;
                }
            }
            __syncthreads();
            stamp(3);
        } else {
            // ---- RMSNorm, token t by CTA t % grid
            for (uint32_t t = blockIdx.x; t < M.n_tokens; t += gridDim.x)
                mega_norm_row(M, Ly, S, h, t, (uint16_t*)M.xn + (size_t)t * M.d, M.xp + (size_t)t * M.d,
                              M.xp2 ? M.xp2 + (size_t)t * M.d : nullptr);
            if (!(alive = grid_barrier(M, S, epoch))) break;
            stamp(1);
            // ---- gate logits, expert e by CTA e % grid
            mega_logits(M, Ly, region_a, nullptr);
            if (!(alive = grid_barrier(M, S, epoch))) break;
            stamp(2);
            // ---- selection, token t by warp 0 of CTA t % grid
            for (uint32_t t = blockIdx.x; t < M.n_tokens; t += gridDim.x) {
                float* lg_s = red;   // the row is copied to shared memory with L2-coherent loads first
                for (uint32_t e = threadIdx.x; e < M.num_experts; e += blockDim.x) lg_s[e] = ld_cg_f32(M.logits + (size_t)t * M.num_experts + e);
                __syncthreads();
                if (warp == 0) {
                    uint32_t e = 0;
                    uint16_t wgt = 0;
                    select_row(lg_s, M.num_experts, M.top_k, M.router_mode, Ly.per_expert_scale, Ly.correction_bias, M.route_scale,
                               lane, e, wgt);
                    if (lane < M.top_k) {
                        M.idx[(size_t)t * M.top_k + lane] = e;
                        M.route_w[(size_t)t * M.top_k + lane] = wgt;
                    }
                }
                __syncthreads();
            }
            if (!(alive = grid_barrier(M, S, epoch))) break;
            stamp(3);
            // ---- sort of the routing table, redundantly in every CTA (no barrier needed)
            for (uint32_t p = threadIdx.x; p < n_pairs; p += blockDim.x) {
                idx_s[p] = ld_cg_u32(M.idx + p);
                w_s[p] = ld_cg_u16(M.route_w + p);
            }
            __syncthreads();
            mega_group(M, S, idx_s, w_s, run_s, sorted_s, groups_s, shared);
        }
        const uint32_t n_groups = S.n_groups;
        if (warp == 0) warp_unit_prefix(groups_s, n_groups, geo1.tiles_per_group, S.pref1, S.pref2, lane);
        __syncthreads();

        FastParams P;
        P.pool = Ly.pool; P.slot_stride = Ly.slot_stride; P.slot_of = Ly.slot_of; P.shared_blob = Ly.shared_blob;
        P.routed_off = Ly.routed_off; P.shared_off = Ly.shared_off;
        P.d = M.d; P.f = M.f; P.num_experts = M.num_experts; P.top_k = M.top_k; P.bits = M.bits; P.shared_bits = M.shared_bits;
        P.scale_dtype = M.scale_dtype; P.activation = M.activation; P.limit = M.limit;
        P.sorted = sorted_s; P.groups = groups_s; P.n_groups = &S.n_groups;
        P.xp = single ? xp_s : M.xp; P.xp_shared = single ? (M.xp2 ? xp2_s : xp_s) : (M.xp2 ? M.xp2 : M.xp);
        P.x_in_smem = single ? 1 : 0;
        P.actp = M.actp; P.route_w = w_s;
        P.dbg = M.trace ? reinterpret_cast<unsigned long long*>(M.trace + (size_t)M.n_layers * 8) : nullptr;
        P.residual = h; P.y = h; P.x_dtype = M.x_dtype; P.n_tokens = M.n_tokens; P.status = M.status;
        stamp(4);

        // ---- phase 1: this CTA's contiguous share of the (group, token tile, row tile) units
        {
            Phase1Ctx C{region_a, S.full1, S.empty1, red, S.pref1};
            const uint32_t n_units = S.pref1[n_groups];
            const uint32_t per_cta = (n_units + gridDim.x - 1) / gridDim.x;
            const uint32_t first = min(blockIdx.x * per_cta, n_units), last = min(first + per_cta, n_units);
            if (!phase1<NGW>(P, geo1, C, n_groups, first, last, seq1, warp, lane)) { atomicOr(M.status, STATUS_MBAR_TIMEOUT); atomicExch(M.abort, 1u); }
        }
        fence_proxy_async();   // hidden activations written here are read by other CTAs' bulk copies after the barrier
        stamp(5);
        if (!(alive = grid_barrier(M, S, epoch))) break;
        stamp(6);

        // ---- phase 2 + combine on the CTAs that own a block of 16 output columns
        const bool p2_cta = blockIdx.x < M.d / 16;
        if (p2_cta) {
            for (uint32_t i = threadIdx.x; i < M.n_tokens * slots * 16; i += blockDim.x) part[i] = 0.0f;
            __syncthreads();
            Phase2Ctx C{region_a, S.full2, S.empty2, part, S.pref2};
            if (!phase2(P, geo2, C, n_groups, blockIdx.x * 16, seq2, warp, lane)) { atomicOr(M.status, STATUS_MBAR_TIMEOUT); atomicExch(M.abort, 1u); }
            __syncthreads();
            f2_combine(P, part, slots, blockIdx.x * 16, shared);
        }
        stamp(7);
        if (!(alive = grid_barrier(M, S, epoch))) break;
    }
}

}  // namespace

// ------------------------------------------------------------------------------------------ host side
static uint32_t cfg_max_bits(const mfb_moe_config& c) { return c.shared_bits > c.bits ? c.shared_bits : c.bits; }

bool fast_supported(const mfb_moe_config& c) {
    if (!(c.d == 512 || c.d == 1024 || c.d == 2048)) return false;   // 1, 2 or 4 groups per warp in phase 1
    const uint32_t ng = c.f / 64;
    if (c.f % 64 || !(ng == 1 || ng == 2 || ng == 4 || ng == 8)) return false;
    if (c.f % (16 * RT)) return false;
    if (c.top_k + 1 > 32) return false;
    return true;
}

size_t fast_smem1(const mfb_moe_config& c) {
    const F1Geom g = f1_geom(c.d, c.f, cfg_max_bits(c));
    return (size_t)F1_STAGES * g.stage_bytes + 2 * CW * 32 * 8 * sizeof(float);
}

size_t fast_smem2(const mfb_moe_config& c, uint32_t n_tokens) {
    const F2Geom g = f2_geom(c.f, cfg_max_bits(c));
    return (size_t)F2_SLOTS * g.slot_bytes + (size_t)n_tokens * (c.top_k + 1) * 16 * sizeof(float);
}

size_t fast_smem_stack(const mfb_moe_config& c, uint32_t n_tokens) {
    const size_t pairs = (size_t)n_tokens * c.top_k;
    const size_t lists = (pairs + n_tokens) * sizeof(mfb_pair) + (c.num_experts + 1) * sizeof(mfb_group) + pairs * 4 +
                         ((pairs + 1) & ~(size_t)1) * 2 + c.num_experts * 4 + 16 + (n_tokens == 1 ? (size_t)c.d * 6 : 0);
    const size_t region_a = fast_smem1(c);
    if (fast_smem2(c, n_tokens) > region_a || (size_t)c.d * (MEGA_ROWS_PER_PASS * 4 + (CW + 1) * 2) > region_a)
        return (size_t)1 << 30;   // does not fit: the caller falls back to the per-layer launches
    return region_a + lists + 64;
}

template <int NGW>
static cudaError_t fast_init_ngw() {
    cudaError_t e = cudaFuncSetAttribute(ffn1_mma_kernel<NGW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_mega_kernel<NGW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    return e;
}

// One-time opt-in to large dynamic shared memory for the fast kernels (called when a handle is created, so that no
// attribute call happens while a caller captures a CUDA graph).
cudaError_t fast_init() {
    cudaError_t e = cudaFuncSetAttribute(ffn2_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    if (e == cudaSuccess) e = fast_init_ngw<1>();
    if (e == cudaSuccess) e = fast_init_ngw<2>();
    if (e == cudaSuccess) e = fast_init_ngw<4>();
    return e;
}

cudaError_t launch_fast_prep(cudaStream_t s, const void* h, int dtype, const __nv_bfloat16* w, uint32_t n_tokens, uint32_t d,
                             float eps, bool do_norm, void* xn, __half* xp, uint32_t bits, __half* xp2, uint32_t bits2) {
    if (n_tokens == 0) return cudaSuccess;
    prep_kernel<<<n_tokens, 256, 0, s>>>(h, dtype, w, d, eps, do_norm ? 1 : 0, xn, xp, bits, xp2, bits2);
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_fast_ffn(cudaStream_t s, const FastParams& P, const mfb_moe_config& c, int sm_count, uint32_t max_groups) {
    const F1Geom g = f1_geom(c.d, c.f, cfg_max_bits(c));
    const uint32_t max_units = max_groups * g.tiles_per_group * ((P.n_tokens + 7) / 8);
    const uint32_t grid = max_units < (uint32_t)sm_count ? max_units : (uint32_t)sm_count;
    switch (c.d / (64 * KS)) {
        case 1: ffn1_mma_kernel<1><<<grid, FAST_THREADS, fast_smem1(c), s>>>(P); break;
        case 2: ffn1_mma_kernel<2><<<grid, FAST_THREADS, fast_smem1(c), s>>>(P); break;
        case 4: ffn1_mma_kernel<4><<<grid, FAST_THREADS, fast_smem1(c), s>>>(P); break;
        default: return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ffn2_mma_kernel<<<P.d / 16, FAST_THREADS, fast_smem2(c, P.n_tokens), s>>>(P);
    count_launches(2);
    return cudaGetLastError();
}

cudaError_t launch_stack_mega(cudaStream_t s, const MegaParams& M, const mfb_moe_config& c, int sm_count) {
    cudaError_t e = cudaMemsetAsync(M.bar_counter, 0, 2 * sizeof(uint32_t), s);   // barrier counter and abort word are adjacent
    if (e != cudaSuccess) return e;
    MegaParams copy = M;
    void* args[] = {&copy};
    const void* fn = nullptr;
    switch (c.d / (64 * KS)) {
        case 1: fn = (const void*)stack_mega_kernel<1>; break;
        case 2: fn = (const void*)stack_mega_kernel<2>; break;
        case 4: fn = (const void*)stack_mega_kernel<4>; break;
        default: return cudaErrorInvalidValue;
    }
    e = cudaLaunchCooperativeKernel(fn, dim3((unsigned)sm_count), dim3(FAST_THREADS), args, fast_smem_stack(c, M.n_tokens), s);
    count_launches(1);
    return e;
}

}  // namespace mfb
