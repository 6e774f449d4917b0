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
// k16 MMAs on the codes (exact, as fp16 subnormals masked straight out of the packed words) times fp16
// activations with fp32 accumulation, sum(x) by four MMAs against a constant fragment.
//
// The K dimension of an MMA may be permuted freely as long as both operands agree, so packed rows are consumed
// as they lie in memory: lane (g, t) of a warp takes bytes [8t, 8t+8) of each 32-byte group of rows g and g+8
// (4-bit; 4 bytes of each 16-byte group for 2-bit) and the activations are stored once per layer in the
// matching within-16 order (see perm_pos).
#include "common.cuh"
#include "decode_mma.cuh"
#include "select.cuh"
#include "tmap.cuh"

#include <cstring>

namespace mfb {

namespace {

constexpr int CW = 8;                       // compute warps per CTA
constexpr int FAST_THREADS = (CW + 1) * 32; // + one copy-issuing warp
constexpr int MAX_STAGES = 4;               // ring depth limit of a phase
constexpr uint32_t RING_BYTES = 150 * 1024; // shared memory of the stage ring (both phases use the same region)
constexpr uint32_t RED_BYTES = 2 * CW * 2 * 2 * 128 * 4;   // two exchange buffers for the k-split partial sums
constexpr uint32_t ROW_PAD = 32;            // bytes after each block of staged rows (bank stagger)
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long limit = MBAR_WAIT_CYCLES) {
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
        if (clock64() - t0 > limit) return false;
        __nanosleep(32);   // a waiting warp should not take issue slots from the computing ones
    }
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {   // L2-coherent (.cg): sees other CTAs' writes
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
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
// Codes of a lane's 16-element segment as eight half2 registers, with no arithmetic at all: a code masked in place
// inside a 16-bit lane IS an fp16 number - a subnormal, code * 2^(shift - 24) for a code whose lowest bit sits at
// bit `shift` (all fields used here lie in the ten mantissa bits).  The tensor core multiplies subnormals exactly.
// The per-register factor 2^shift is taken out again on the activation side (perm_scale: the activation that
// meets a code at bit `shift` is stored divided by 2^shift), the common 2^-24 in the epilogue of a phase.
// 4-bit: words w0 (codes 0-7) and w1 (codes 8-15); register i holds (q[e], q[e+4]) with e following
// 0,1,2,3,8,9,10,11; odd e are high nibbles (shift 4).
constexpr float CODE_UNSCALE = 16777216.0f;   // 2^24

template <int BITS>
struct Unpack;

template <>
struct Unpack<4> {
    static constexpr int WORDS = 2;   // 32-bit words per lane per row per 64-element group
    __device__ static __forceinline__ void run(const uint32_t (&w)[2], uint32_t (&p)[8]) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t lo = w[i], hi = w[i] >> 8;
            p[4 * i + 0] = lo & 0x000F000Fu;
            p[4 * i + 1] = lo & 0x00F000F0u;
            p[4 * i + 2] = hi & 0x000F000Fu;
            p[4 * i + 3] = hi & 0x00F000F0u;
        }
    }
    // all-ones counterpart of register i: the factor its activations were divided by
    __device__ static __forceinline__ uint32_t unit(int i) { return (i & 1) ? 0x4C004C00u : 0x3C003C00u; }   // 16, 1
};

// 2-bit: one word holds the 16 codes; register i holds (q[i], q[i+8]); registers 0-4 come from the word itself
// (shifts 0, 2, 4, 6, 8), registers 5-7 from the word shifted right by ten (shifts 0, 2, 4).
template <>
struct Unpack<2> {
    static constexpr int WORDS = 1;
    __device__ static __forceinline__ void run(const uint32_t (&w)[1], uint32_t (&p)[8]) {
        const uint32_t a = w[0], b = w[0] >> 10;
        p[0] = a & 0x00030003u;
        p[1] = a & 0x000C000Cu;
        p[2] = a & 0x00300030u;
        p[3] = a & 0x00C000C0u;
        p[4] = a & 0x03000300u;
        p[5] = b & 0x00030003u;
        p[6] = b & 0x000C000Cu;
        p[7] = b & 0x00300030u;
    }
    __device__ static __forceinline__ uint32_t unit(int i) {
        const int k = i < 5 ? i : i - 5;   // 4^k as fp16 pairs
        return k == 0 ? 0x3C003C00u : k == 1 ? 0x44004400u : k == 2 ? 0x4C004C00u : k == 3 ? 0x54005400u : 0x5C005C00u;
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

// Factor the activation of element e (0..15) of a 16-element segment is stored with: 2^-shift of the code it meets
// (see Unpack).  Powers of two, so the only rounding is that of values pushed into the fp16 subnormal range.
__host__ __device__ float perm_scale(uint32_t e, uint32_t bits) {
    if (bits == 4) return (e & 1u) ? 0.0625f : 1.0f;
    const uint32_t i = e & 7u, k = i < 5u ? i : i - 5u;
    return 1.0f / (float)(1u << (2u * k));
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

// sum(x) * 2^-24 over one 64-element group for this lane's two token columns (2t, 2t+1): four MMAs against a
// constant A fragment that undoes the per-register storage factor leave the sums in c0 and c1 - no conversions,
// shuffles or shared memory.  The 2^-24 matches the scale of the code sums (see Unpack).
template <int BITS>
__device__ __forceinline__ float2 group_sum(const uint32_t (&bf)[8]) {
    float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t u0 = Unpack<BITS>::unit(2 * j), u1 = Unpack<BITS>::unit(2 * j + 1);
        mma16816(d, u0, u0, u1, u1, bf[2 * j], bf[2 * j + 1]);
    }
    return make_float2(d[0] * (1.0f / CODE_UNSCALE), d[1] * (1.0f / CODE_UNSCALE));
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
    template <int SDT>
    __device__ __forceinline__ float at(int i) const {
        const uint32_t v = w[i >> 1];
        if (SDT == MFB_DT_BF16) return __uint_as_float((i & 1) ? (v & 0xFFFF0000u) : (v << 16));
        const __half2 h = *reinterpret_cast<const __half2*>(&v);
        return (i & 1) ? __high2float(h) : __low2float(h);
    }
};

// ------------------------------------------------------------------------------------------ work lists
// A unit of work is one (group, token tile of up to 8 rows[, 32-row tile of gate/up]).  Exclusive prefix sums of
// the units of each group, by one warp: pref1[g] counts phase-1 units, pref2[g] phase-2 units.
//
// Units do not cost the same: the MMA work of a unit is fixed, its epilogue grows with the token columns in use.
// wpref1[g] / wpref2[g] are the exclusive prefixes of the groups' weights in phase 1 / phase 2, a token tile with c
// columns weighing base + c (per row tile); the CTAs cut the unit list at equal weight rather than at equal count.
// The bases are the measured ratios of a unit's fixed cost to its cost per token column (SM cycles in the running
// pipeline: phase 1 about 4330 + 154 c, phase 2 about 2360 + 195 c).
// With only a handful of units per CTA (small batches) the cut points matter less than their granularity, and
// the flatter weights measured slower there: those launches keep a base of 6 for both phases.
struct UnitBases { uint32_t b1, b2; };
__device__ __forceinline__ UnitBases unit_bases(bool large_batch) { return large_batch ? UnitBases{28u, 12u} : UnitBases{6u, 6u}; }

__device__ __forceinline__ uint32_t group_weight(uint32_t pair_count, uint32_t base) {
    const uint32_t full = pair_count / 8, rem = pair_count % 8;
    return full * (base + 8) + (rem ? base + rem : 0);
}

template <bool TWO>   // TWO = false: one weight model for both phases (b1), wpref2 is not written
__device__ __forceinline__ void warp_unit_prefix2(const mfb_group* groups, uint32_t n_groups, uint32_t tiles1, uint32_t tiles2,
                                                  uint32_t* pref1, uint32_t* pref2, uint32_t* wpref1, uint32_t* wpref2,
                                                  UnitBases ub, uint32_t lane) {
    const uint32_t per = (n_groups + 31) / 32, g0 = lane * per;
    uint32_t local = 0, w1local = 0, w2local = 0;
    for (uint32_t j = 0; j < per; ++j)
        if (g0 + j < n_groups) {
            const uint32_t c = groups[g0 + j].pair_count;
            local += (c + 7) / 8;
            w1local += group_weight(c, ub.b1);
            if (TWO) w2local += group_weight(c, ub.b2);
        }
    uint32_t incl = local, w1incl = w1local, w2incl = w2local;
    for (uint32_t off = 1; off < 32; off <<= 1) {
        const uint32_t n = __shfl_up_sync(0xFFFFFFFFu, incl, off), a = __shfl_up_sync(0xFFFFFFFFu, w1incl, off);
        if (lane >= off) { incl += n; w1incl += a; }
        if (TWO) {
            const uint32_t b = __shfl_up_sync(0xFFFFFFFFu, w2incl, off);
            if (lane >= off) w2incl += b;
        }
    }
    uint32_t run = incl - local, w1run = w1incl - w1local, w2run = w2incl - w2local;
    for (uint32_t j = 0; j < per; ++j)
        if (g0 + j < n_groups) {
            const uint32_t c = groups[g0 + j].pair_count;
            pref1[g0 + j] = run * tiles1;
            pref2[g0 + j] = run * tiles2;
            wpref1[g0 + j] = w1run;
            if (TWO) wpref2[g0 + j] = w2run;
            run += (c + 7) / 8;
            w1run += group_weight(c, ub.b1);
            if (TWO) w2run += group_weight(c, ub.b2);
        }
    const uint32_t total = __shfl_sync(0xFFFFFFFFu, incl, 31), w1total = __shfl_sync(0xFFFFFFFFu, w1incl, 31);
    if (lane == 0) { pref1[n_groups] = total * tiles1; pref2[n_groups] = total * tiles2; wpref1[n_groups] = w1total; }
    if (TWO) {
        const uint32_t w2total = __shfl_sync(0xFFFFFFFFu, w2incl, 31);
        if (lane == 0) wpref2[n_groups] = w2total;
    }
    __syncwarp();
}

// First unit at or after weight position `cut` of `parts` equal cuts of the phase's total weight.  32-bit arithmetic
// suffices: at most 64 tokens x (top_k + 1) pairs of weight <= base + 1 each, times tiles, times parts.
__device__ __forceinline__ uint32_t unit_at_cut(const mfb_group* groups, uint32_t n_groups, const uint32_t* pref,
                                                const uint32_t* wpref, uint32_t tiles, uint32_t base, uint32_t cut,
                                                uint32_t parts) {
    if (cut >= parts) return pref[n_groups];
    const uint32_t target = wpref[n_groups] * tiles * cut / parts;   // weight in front of the unit looked for
    uint32_t lo = 0, hi = n_groups;   // last group whose prefix (times tiles) is <= target
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) / 2;
        if (wpref[mid] * tiles <= target) lo = mid; else hi = mid;
    }
    uint32_t rem = target - wpref[lo] * tiles;
    const uint32_t count = groups[lo].pair_count, full = count / 8, r = count % 8;
    const uint32_t full_block = tiles * (base + 8);
    const uint32_t tt = min(full, rem / full_block);
    rem -= tt * full_block;
    const uint32_t w = tt < full ? base + 8 : base + r;
    return pref[lo] + tt * tiles + min(rem / w, tiles - 1);
}

// Optional cycle accounting of one CTA (attached with the phase trace): counter k of warp w at dbg[w*8 + k].  The
// CTA is number 1 where there is one: with a single token CTA 0 can be left without a unit.
__device__ __forceinline__ void dbg_add(unsigned long long* dbg, uint32_t warp, uint32_t lane, int k, long long t0) {
    if (dbg && blockIdx.x == (gridDim.x > 1 ? 1u : 0u) && lane == 0) atomicAdd(&dbg[warp * 8 + k], (unsigned long long)(clock64() - t0));   // no result: does not stall
}

// Advances `g` until unit u lies in group g (units are visited in increasing order).
__device__ __forceinline__ void seek_group(const uint32_t* pref, uint32_t n_groups, uint32_t u, uint32_t& g) {
    while (g + 1 < n_groups && pref[g + 1] <= u) ++g;
}

// ------------------------------------------------------------------------------------------ one FFN phase
// Both matrix phases of the expert FFN run through the same machinery:
//   phase 1  NMAT = 2 (gate, up), contraction over d, rows = f, epilogue act(gate) * up -> fp16 hidden activations
//   phase 2  NMAT = 1 (down),     contraction over f, rows = d, epilogue -> fp32 rows of the (token, slot) partials
// A unit of work is one (group, token tile of <= 8 rows, tile of `tile_rows` matrix rows).  The copy warp stages the
// tile: each matrix as four blocks of consecutive rows, one bulk copy per block (kilobytes each: the copy unit
// sustains only a few copies in flight), 32 pad bytes after a block so that the four rows one shared-memory load
// phase touches fall into different banks; plus one copy per scale / bias block.  The eight compute warps split
// the tile as (k split) x (row group); every warp works on RPW = 2 sixteen-row MMA tiles with the same activation
// fragments, which gives the scheduler independent MMA chains to interleave.  Partial sums of the k splits meet
// in shared memory and are added in a fixed order.
constexpr int RPW = 2;   // 16-row MMA tiles per warp

struct PhaseGeom {
    uint32_t k, n_rows, ksplit, row_groups, tile_rows, tiles, blk_rows, blk_stride, mat_bytes, gpr, scale_block,
        stage_bytes, k_per_warp, n_stages, tile_shift, blk_shift;   // tile_rows and blk_rows are powers of two
};

__host__ __device__ inline PhaseGeom phase_geom(uint32_t nmat, uint32_t k, uint32_t n_rows, uint32_t ngw, uint32_t max_bits,
                                                uint32_t ring_bytes) {
    PhaseGeom g;
    g.k = k; g.n_rows = n_rows;
    g.gpr = k / 64;
    g.ksplit = g.gpr / ngw;
    g.row_groups = CW / g.ksplit;
    g.tile_rows = 16 * RPW * g.row_groups;
    g.tiles = n_rows / g.tile_rows;
    g.blk_rows = g.tile_rows / 4;
    g.tile_shift = 0;
    while ((1u << g.tile_shift) < g.tile_rows) ++g.tile_shift;
    g.blk_shift = g.tile_shift - 2;
    g.blk_stride = g.blk_rows * (k * max_bits / 8) + ROW_PAD;
    g.mat_bytes = 4 * g.blk_stride;
    g.scale_block = g.tile_rows * g.gpr * 2;
    g.stage_bytes = nmat * g.mat_bytes + 2 * nmat * g.scale_block;
    g.k_per_warp = ngw * 64;
    const uint32_t fit = ring_bytes / g.stage_bytes;
    g.n_stages = fit > MAX_STAGES ? MAX_STAGES : fit;
    return g;
}

struct PhaseCtx {
    uint8_t* ring;       // n_stages * stage_bytes
    uint64_t* full;      // [MAX_STAGES]
    uint64_t* empty;     // [MAX_STAGES]
    float* red;          // [2][CW * RPW * 2 * 128]
    const uint32_t* pref;   // exclusive prefix of units per group, pref[n_groups] = total
};

// Row of a stage tile that MMA row (row tile rtile of the stage, lane group g, upper half hi) works on:
// block g % 4, then four rows per row tile inside the block.
__device__ __forceinline__ uint32_t tile_row(uint32_t blk_rows, uint32_t rtile, uint32_t g, uint32_t hi) {
    return (g & 3) * blk_rows + rtile * 4 + hi * 2 + (g >> 2);
}

// Copy-issuing side of one unit (all 32 lanes of the issuing warp call this).
template <int NMAT>
__device__ __forceinline__ bool phase_produce(const FastParams& P, const PhaseGeom& geo, const PhaseCtx& C, const GroupRef& G,
                                              uint32_t tile, uint32_t s, uint32_t ph, uint32_t lane) {
    if (!mbar_wait(&C.empty[s], ph ^ 1u)) return false;
    if (!G.ok) {   // nothing to copy: complete the phase so the consumers move on
        if (lane == 0) mbar_arrive(&C.full[s]);
        return true;
    }
    const uint32_t row0 = tile * geo.tile_rows, row_bytes = geo.k * G.bits / 8;
    uint8_t* st = C.ring + s * geo.stage_bytes;
    if (lane == 0) mbar_expect_tx(&C.full[s], NMAT * geo.tile_rows * row_bytes + 2 * NMAT * geo.scale_block);
    __syncwarp();
    const uint32_t* off = &G.off.gate_w;   // gate W,S,B, up W,S,B, down W,S,B
    if (lane < 4 * NMAT) {
        const uint32_t m = lane >> 2, b = lane & 3;
        const uint32_t w_off = NMAT == 2 ? off[3 * m] : off[6];
        bulk_g2s(st + m * geo.mat_bytes + b * geo.blk_stride, G.blob + w_off + (size_t)(row0 + b * geo.blk_rows) * row_bytes,
                 geo.blk_rows * row_bytes, &C.full[s]);
    } else if (lane < 6 * NMAT) {
        const uint32_t i = lane - 4 * NMAT, m = i >> 1, sb = i & 1;    // scale / bias of matrix m
        const uint32_t s_off = NMAT == 2 ? off[3 * m + 1 + sb] : off[7 + sb];
        bulk_g2s(st + NMAT * geo.mat_bytes + i * geo.scale_block, G.blob + s_off + (size_t)row0 * geo.gpr * 2, geo.scale_block,
                 &C.full[s]);
    }
    return true;
}

// Single-token mode of the fused kernel: asks L2 for the bytes of one unit of the NEXT phase while this phase still
// runs (the whole layer's traffic is a fraction of L2 there, and the phase after the grid barrier then starts from
// L2 hits instead of DRAM latency).  Mirrors phase_produce.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
template <int NMAT>
__device__ __forceinline__ void phase_prefetch_l2(const PhaseGeom& geo, const GroupRef& G, uint32_t tile, uint32_t lane) {
    if (!G.ok) return;
    const uint32_t row0 = tile * geo.tile_rows, row_bytes = geo.k * G.bits / 8;
    const uint32_t* off = &G.off.gate_w;
    if (lane < NMAT) {
        const uint32_t w_off = NMAT == 2 ? off[3 * lane] : off[6];
        bulk_prefetch_l2(G.blob + w_off + (size_t)row0 * row_bytes, geo.tile_rows * row_bytes);
    } else if (lane < 3 * NMAT) {
        const uint32_t i = lane - NMAT, m = i >> 1, sb = i & 1;
        const uint32_t s_off = NMAT == 2 ? off[3 * m + 1 + sb] : off[7 + sb];
        bulk_prefetch_l2(G.blob + s_off + (size_t)row0 * geo.gpr * 2, geo.scale_block);
    }
}

// B fragments of this warp's k range for token column g of a token tile: registers, loaded from L2 (or from shared
// memory in the single-token mode of the fused kernel).  Phase 1 reads the permuted activations of the group's
// tokens, phase 2 the hidden activations phase 1 left for the group's sorted pairs.
template <int NMAT, int NGW>
__device__ __forceinline__ void phase_load_x(const FastParams& P, const GroupRef& G, uint32_t tt, uint32_t k0, uint32_t lane,
                                             uint32_t (&bf)[NGW][8]) {
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t cols = min(8u, G.pair_count - tt * 8);
    const __half* row = nullptr;
    bool smem_src = false;
    if (g < cols) {
        if (NMAT == 2) {
            const __half* xsrc = (G.shared && P.shared_bits != P.bits) ? P.xp_shared : P.xp;
            row = xsrc + (size_t)P.sorted[G.pair_start + tt * 8 + g].token * P.d + k0 + t * 16;
            smem_src = P.x_in_smem != 0;
        } else {
            row = P.actp + (size_t)(G.pair_start + tt * 8 + g) * P.f + k0 + t * 16;
        }
    }
#pragma unroll
    for (int gi = 0; gi < NGW; ++gi) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
        if (row) {
            if (smem_src) { lo = *reinterpret_cast<const uint4*>(row + gi * 64); hi = *reinterpret_cast<const uint4*>(row + gi * 64 + 8); }
            else { lo = ld_cg_u4(row + gi * 64); hi = ld_cg_u4(row + gi * 64 + 8); }
        }
        bf[gi][0] = lo.x; bf[gi][1] = lo.y; bf[gi][2] = lo.z; bf[gi][3] = lo.w;
        bf[gi][4] = hi.x; bf[gi][5] = hi.y; bf[gi][6] = hi.z; bf[gi][7] = hi.w;
    }
}

// Compute side of one unit by one warp: RPW row tiles x NMAT matrices x NGW groups of this warp's k range, then the
// exchange of the k-split partial sums and the epilogue.
template <int NMAT, int NGW, int BITS, int SDT>
__device__ __forceinline__ void phase_compute(const FastParams& P, const GroupRef& G, const PhaseGeom& geo, const uint8_t* stage,
                                              uint32_t tile, uint32_t tt, const uint32_t (&bf)[NGW][8], float2 (&sx)[NGW],
                                              bool fresh_x, uint32_t warp, uint32_t lane, float* red, uint32_t& red_buf) {
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t ksi = warp % geo.ksplit, rg = warp / geo.ksplit;
    const uint32_t row_bytes = geo.k * BITS / 8, gpr = geo.gpr;
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(stage + NMAT * geo.mat_bytes);
    const uint32_t sblk = geo.tile_rows * gpr;
    constexpr uint32_t lane_bytes = BITS == 4 ? 8 : 4, group_bytes = 64 * BITS / 8;
    const uint32_t cols = min(8u, G.pair_count - tt * 8);

    if (fresh_x) {
#pragma unroll
        for (int gi = 0; gi < NGW; ++gi) sx[gi] = group_sum<BITS>(bf[gi]);   // valid for every row tile of this token tile
    }
    float acc[RPW][NMAT][4];
#pragma unroll
    for (int j = 0; j < RPW; ++j) {
        const uint32_t rtile = rg * RPW + j;
        const uint32_t r_lo = tile_row(geo.blk_rows, rtile, g, 0), r_hi = r_lo + 2;
        const uint32_t a_lo = (g & 3) * geo.blk_stride + (r_lo - (g & 3) * geo.blk_rows) * row_bytes, a_hi = a_lo + 2 * row_bytes;
        ScaleRow<NGW> sr[NMAT][4];   // [matrix][scale lo, scale hi, bias lo, bias hi] for this warp's groups
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
            sr[m][0].load(sc + (2 * m) * sblk + r_lo * gpr + ksi * NGW);
            sr[m][1].load(sc + (2 * m) * sblk + r_hi * gpr + ksi * NGW);
            sr[m][2].load(sc + (2 * m + 1) * sblk + r_lo * gpr + ksi * NGW);
            sr[m][3].load(sc + (2 * m + 1) * sblk + r_hi * gpr + ksi * NGW);
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[j][m][c] = 0.0f;
        }
#pragma unroll
        for (int gi = 0; gi < NGW; ++gi) {
            const uint32_t boff = (ksi * NGW + gi) * group_bytes + t * lane_bytes;
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
                group_mma<BITS>(stage + m * geo.mat_bytes + a_lo, stage + m * geo.mat_bytes + a_hi, boff, bf[gi],
                                sr[m][0].template at<SDT>(gi), sr[m][2].template at<SDT>(gi), sr[m][1].template at<SDT>(gi),
                                sr[m][3].template at<SDT>(gi), sx[gi],
                                acc[j][m]);
        }
    }
    // partial sums of this warp -> shared memory; fixed-order sum over the k splits by whoever owns the output
    constexpr uint32_t PER_TILE = NMAT * 128;    // floats one (k split, row tile) leaves: [matrix][lane][4]
    const uint32_t n_rtiles = geo.row_groups * RPW;
    float* rb = red + red_buf * (CW * RPW * 2 * 128);
#pragma unroll
    for (int j = 0; j < RPW; ++j)
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
            *reinterpret_cast<float4*>(rb + ((ksi * n_rtiles + rg * RPW + j) * PER_TILE) + m * 128 + lane * 4) =
                make_float4(acc[j][m][0], acc[j][m][1], acc[j][m][2], acc[j][m][3]);
    named_barrier(1, CW * 32);
    // Fixed-order sum over the k splits and the phase's epilogue.  A thread keeps one row of the stage tile and steps
    // through the token columns (tile_rows divides the CW * 32 threads or is a multiple of them), so everything that
    // depends on the row is computed once, and consecutive threads store consecutive matrix rows of one column.
    const uint32_t et = warp * 32 + lane;
    for (uint32_t rl0 = 0; rl0 < geo.tile_rows; rl0 += CW * 32) {   // one pass unless the tile has more rows than threads
        const uint32_t rl = rl0 + (et & (geo.tile_rows - 1)), n0 = et >> geo.tile_shift;
        const uint32_t n_step = geo.tile_rows >= CW * 32 ? 1u : (CW * 32) >> geo.tile_shift;
        // inverse of tile_row: block b = lane group % 4, then rtile * 4 + hi * 2 + (lane group / 4)
        const uint32_t b = rl >> geo.blk_shift, q = rl & (geo.blk_rows - 1);
        const uint32_t rtile = q >> 2, hi = (q >> 1) & 1u, gq = b + 4u * (q & 1u);
        const float* rrow = rb + rtile * PER_TILE + gq * 16 + hi * 2;   // + k * n_rtiles * PER_TILE + m * 128 + (n / 2) * 4 + (n & 1)
        const uint32_t r = tile * geo.tile_rows + rl;
        const uint32_t pair0 = G.pair_start + tt * 8;
        const uint32_t act_col = (r & ~15u) + perm_pos(r & 15u, G.bits);
        const float act_scale = perm_scale(r & 15u, G.bits);
        const bool clamp = !G.shared && P.limit > 0.0f;   // moe_swiglu_clamp (moe.metal:27-34), routed experts only
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j) {
            const uint32_t n = n0 + j * n_step;
            if (n >= cols) break;
            float v[NMAT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) v[m] = 0.0f;
            const float* src = rrow + (n >> 1) * 4 + (n & 1);
            for (uint32_t k = 0; k < geo.ksplit; ++k)
#pragma unroll
                for (int m = 0; m < NMAT; ++m) v[m] += src[k * n_rtiles * PER_TILE + m * 128];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) v[m] *= CODE_UNSCALE;
            if (NMAT == 2) {
                float gate = v[0], up = v[NMAT - 1];
                if (clamp) {
                    gate = fminf(gate, P.limit);
                    up = fminf(fmaxf(up, -P.limit), P.limit);
                }
                float a = hidden_act(gate, (int)P.activation) * up;
                a = fminf(fmaxf(a, -65504.0f), 65504.0f);
                P.actp[(size_t)(pair0 + n) * P.f + act_col] = __float2half_rn(a * act_scale);
            } else {
                const mfb_pair pr = P.sorted[pair0 + n];
                P.partial[((size_t)pr.token * (P.top_k + 1) + pr.rank) * P.d + r] = v[0];
            }
        }
    }
    red_buf ^= 1u;
}

// Runs this CTA's share of one phase: units [first, last) of the flattened (group, token tile, row tile) list.
// `seq` counts the units the CTA has pushed through this ring since its barriers were initialised.
template <int NMAT, int NGW>
__device__ __forceinline__ bool run_phase(const FastParams& P, const PhaseGeom& geo, const PhaseCtx& C, uint32_t n_groups,
                                          uint32_t first, uint32_t last, uint32_t& seq, uint32_t warp, uint32_t lane) {
    bool ok = true;
    if (first >= last) return true;
    // cursors advanced by one unit per iteration: (group, token tile, row tile) and (ring stage, parity) - no
    // divisions in the loop
    uint32_t g = 0;
    seek_group(C.pref, n_groups, first, g);
    uint32_t tt = (first - C.pref[g]) / geo.tiles, tile = (first - C.pref[g]) % geo.tiles;
    uint32_t st_i = seq % geo.n_stages, ph = (seq / geo.n_stages) & 1u;
    GroupRef G = group_ref(P, g);   // the slot lookup is a dependent global load: once per group
#define MFB_ADVANCE_UNIT()                                                                              \
    do {                                                                                                \
        if (++st_i == geo.n_stages) { st_i = 0; ph ^= 1u; }                                             \
        if (++tile == geo.tiles) {                                                                      \
            tile = 0; ++tt;                                                                             \
            if (tt * 8 >= G.pair_count && g + 1 < n_groups) { ++g; tt = 0; G = group_ref(P, g); }       \
        }                                                                                               \
    } while (0)
    constexpr int DBG = NMAT == 2 ? 0 : 2;
    if (warp == CW) {
        fence_proxy_async();
        for (uint32_t u = first; u < last && ok; ++u) {
            const long long t0 = clock64();
            ok = phase_produce<NMAT>(P, geo, C, G, tile, st_i, ph, lane);
            dbg_add(P.dbg, warp, lane, DBG, t0);
            MFB_ADVANCE_UNIT();
        }
    } else {
        uint32_t bf[NGW][8];
        float2 sx[NGW];
        uint32_t cached = 0xFFFFFFFFu, red_buf = 0;
        const uint32_t k0 = (warp % geo.ksplit) * geo.k_per_warp;
        const long long t_phase = clock64();
        for (uint32_t u = first; u < last && ok; ++u) {
            const long long t_top = clock64();
            const uint32_t key = g * 16 + tt;
            const bool fresh_x = G.ok && key != cached;
            if (fresh_x) { phase_load_x<NMAT, NGW>(P, G, tt, k0, lane, bf); cached = key; }   // issued before the wait below
            dbg_add(P.dbg, warp, lane, 4 + DBG, t_top);
            long long t0 = clock64();
            if (!mbar_wait(&C.full[st_i], ph)) { ok = false; break; }
            dbg_add(P.dbg, warp, lane, DBG, t0);
            t0 = clock64();
            if (G.ok) {
                const uint8_t* st = C.ring + st_i * geo.stage_bytes;
                const bool bf16_scales = P.scale_dtype == MFB_DT_BF16;
                if (G.bits == 4) {
                    if (bf16_scales) phase_compute<NMAT, NGW, 4, MFB_DT_BF16>(P, G, geo, st, tile, tt, bf, sx, fresh_x, warp, lane, C.red, red_buf);
                    else phase_compute<NMAT, NGW, 4, MFB_DT_F16>(P, G, geo, st, tile, tt, bf, sx, fresh_x, warp, lane, C.red, red_buf);
                } else {
                    if (bf16_scales) phase_compute<NMAT, NGW, 2, MFB_DT_BF16>(P, G, geo, st, tile, tt, bf, sx, fresh_x, warp, lane, C.red, red_buf);
                    else phase_compute<NMAT, NGW, 2, MFB_DT_F16>(P, G, geo, st, tile, tt, bf, sx, fresh_x, warp, lane, C.red, red_buf);
                }
            } else if (NMAT == 1) {
                // an expert that is not resident contributes nothing: its rows of the partials are cleared
                const uint32_t cols = min(8u, G.pair_count - tt * 8);
                for (uint32_t o = warp * 32 + lane; o < geo.tile_rows * cols; o += CW * 32) {
                    const mfb_pair pr = P.sorted[G.pair_start + tt * 8 + o / geo.tile_rows];
                    P.partial[((size_t)pr.token * (P.top_k + 1) + pr.rank) * P.d + tile * geo.tile_rows + o % geo.tile_rows] = 0.0f;
                }
            }
            __syncwarp();
            dbg_add(P.dbg, warp, lane, DBG + 1, t0);
            if (lane == 0) mbar_arrive(&C.empty[st_i]);
            MFB_ADVANCE_UNIT();
        }
        dbg_add(P.dbg, warp, lane, 5 + DBG, t_phase);
    }
#undef MFB_ADVANCE_UNIT
    seq += last - first;
    return ok;
}

// ------------------------------------------------------------------------------------------ one FFN phase, row-stationary form
// Used for batches above 16 rows.  The k-split form above hands every warp a slice of the contraction and pays for
// it per unit with an exchange of partial sums through shared memory, a barrier and a separate epilogue; with
// hundreds of units per CTA that serial tail costs as much as the arithmetic.  Here a warp owns sixteen matrix rows
// for the WHOLE contraction: its accumulators hold finished sums, the epilogue runs on registers, and nothing is
// exchanged.  The price is that a stage must hold a k-slice of 128 rows, i.e. row pieces that are not contiguous in
// memory - which is what tiled TMA is for:
//   stage     two tiles of [128 rows x 128 bytes of codes] (phase 1: gate and up rows of one row block; phase 2: two
//             consecutive row blocks of down), each one cp.async.bulk.tensor.3d over (row bytes, rows, pool slot) in
//             the 128-byte swizzle, plus the matching 256-element slice of the unit's (up to eight) activation rows,
//             one bulk copy per row.  Four stages.
//   scales    per sixteen groups of the contraction: scale and bias of both tiles as four tensor copies of
//             [128 rows x 32 bytes] (32-byte swizzle; 16-byte rows unswizzled when a row has eight groups),
//             double-buffered beside the ring with barriers of their own.
// Bank conflicts: MMA row g of a warp's sixteen is tile row 2g (g < 4) or 2(g-4)+1, so the four lane groups of a
// half warp read rows whose swizzle patterns differ in the upper two bits: every 8-byte load of the codes and of the
// scales falls into distinct banks.  Activation rows sit 528 bytes apart (16 bytes of stagger).
namespace wide {

constexpr uint32_t TILE_ROWS = 128, TILE_ROW_BYTES = 128, TILE_BYTES = TILE_ROWS * TILE_ROW_BYTES;
constexpr uint32_t NT = 2;                        // tiles per stage
constexpr uint32_t KC = 256;                      // codes per k chunk: 128 bytes of 4-bit codes
constexpr uint32_t GPC = KC / 64;                 // 64-element groups per chunk
constexpr uint32_t X_STRIDE = KC * 2 + 16;        // bytes between the activation rows of a stage
constexpr uint32_t STAGE_BYTES = 37 * 1024;       // NT tiles + 8 activation rows, rounded up to the swizzle alignment
constexpr uint32_t STAGES = 4;
constexpr uint32_t SCALE_BUF_BYTES = 16 * 1024;   // scale and bias of both tiles for sixteen groups
constexpr uint32_t RING_BYTES = STAGES * STAGE_BYTES + 2 * SCALE_BUF_BYTES;
static_assert(NT * TILE_BYTES + 8 * X_STRIDE <= STAGE_BYTES, "stage layout");

struct Geom {
    uint32_t k, rows, tiles, nkc, sbg, nsb, kc_per_sb, srb;
};

// PHASE 1: contraction over d, 128-row blocks of f (gate and up of the same rows);
// PHASE 2: contraction over f, 256-row blocks of d.
__host__ __device__ inline Geom geom(int phase, uint32_t d, uint32_t f) {
    Geom g;
    g.k = phase == 1 ? d : f;
    g.rows = phase == 1 ? f : d;
    g.tiles = phase == 1 ? f / TILE_ROWS : d / (NT * TILE_ROWS);
    g.nkc = g.k / KC;
    const uint32_t gpr = g.k / 64;
    g.sbg = gpr < 16 ? gpr : 16;
    g.nsb = gpr / g.sbg;
    g.kc_per_sb = g.sbg / GPC;
    g.srb = g.sbg * 2;
    return g;
}

struct Ctx {
    uint8_t* ring;        // STAGES stages, then the two scale buffers; 1024-byte aligned
    uint64_t* full;       // [STAGES]
    uint64_t* empty;      // [STAGES]
    uint64_t* sfull;      // [2]
    uint64_t* sempty;     // [2]
    const uint32_t* pref; // exclusive prefix of units per group
    const uint32_t* pref_dep;   // phase 2 with P.ready: the phase-1 prefix (units of a group that must have finished)
};

__device__ __forceinline__ void red_release_add(uint32_t* p, uint32_t v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint32_t c0, uint32_t c1, uint32_t c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)) : "memory");
}

// Makes a tensor map that the host rewrote since an earlier launch (a recycled slot of the handle's map array)
// visible to the tensor copies of this thread's CTA.
__device__ __forceinline__ void tensormap_acquire(const CUtensorMap* map) {
    asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

struct UnitRef {
    const CUtensorMap* maps;   // the nine maps of the unit's weights (routed pool or shared blob)
    uint32_t slot, pair_start, pair_count;
    bool shared, ok;
};

__device__ __forceinline__ UnitRef unit_ref(const FastParams& P, uint32_t g) {
    UnitRef v;
    const mfb_group grp = P.groups[g];
    v.shared = grp.expert >= P.num_experts;
    v.pair_start = grp.pair_start;
    v.pair_count = grp.pair_count;
    v.ok = true;
    v.slot = 0;
    if (v.shared) {
        v.maps = P.maps->m[1];
        v.ok = P.shared_blob != nullptr;
    } else {
        int32_t slot = (int32_t)grp.expert;
        if (P.slot_of) slot = P.slot_of[grp.expert];
        v.ok = slot >= 0;
        v.slot = slot < 0 ? 0u : (uint32_t)slot;
        v.maps = P.maps->m[0];
    }
    return v;
}

// Runs this CTA's share [first, last) of one phase.  `seq` / `sseq` count the stages / scale blocks this CTA has
// pushed through the ring since its barriers were initialised (both phases and all layers share ring and barriers).
template <int PHASE, int SDT>
__device__ __forceinline__ bool run(const FastParams& P, const Geom& geo, const Ctx& C, uint32_t n_groups, uint32_t first,
                                    uint32_t last, uint32_t& seq, uint32_t& sseq, uint32_t warp, uint32_t lane) {
    if (first >= last) return true;
    bool ok = true;
    uint32_t g = 0;
    seek_group(C.pref, n_groups, first, g);
    uint32_t tt = (first - C.pref[g]) / geo.tiles, tile = (first - C.pref[g]) % geo.tiles;
    UnitRef G = unit_ref(P, g);
    uint8_t* const sbufs = C.ring + STAGES * STAGE_BYTES;
    uint32_t my_seq = seq, my_sseq = sseq, ok_units = 0;
    constexpr int DBG = PHASE == 1 ? 0 : 2;
#define MFB_ADVANCE_UNIT()                                                                              \
    do {                                                                                                \
        if (++tile == geo.tiles) {                                                                      \
            tile = 0; ++tt;                                                                             \
            if (tt * 8 >= G.pair_count && g + 1 < n_groups) { ++g; tt = 0; G = unit_ref(P, g); }        \
        }                                                                                               \
    } while (0)
    if (warp == CW) {
        // ------------------------------------------------------------ copy-issuing warp
        fence_proxy_async();   // activation rows written through the generic proxy by other CTAs before the grid barrier
        if (lane < 18) tensormap_acquire(&P.maps->m[lane / 9][lane % 9]);
        __syncwarp();
        uint32_t checked = 0xFFFFFFFFu;
        for (uint32_t u = first; u < last && ok; ++u) {
            if (G.ok) {
                ++ok_units;
                if (PHASE == 2 && P.ready && g != checked) {
                    // no grid barrier in front of this phase: the hidden activations of group g are complete once every
                    // computing warp of every phase-1 unit of the group has counted itself in
                    const uint32_t need = (C.pref_dep[g + 1] - C.pref_dep[g]) * CW;
                    uint32_t good = 1;
                    if (lane == 0) {
                        const long long t0 = clock64();
                        while (ld_acquire_u32(P.ready + g) < need)
                            if (clock64() - t0 > MBAR_WAIT_CYCLES) { good = 0; break; }
                    }
                    good = __shfl_sync(0xFFFFFFFFu, good, 0);
                    if (!good) { ok = false; break; }
                    fence_proxy_async();
                    checked = g;
                }
                const uint32_t cols = min(8u, G.pair_count - tt * 8), pair0 = G.pair_start + tt * 8;
                const uint32_t row0 = PHASE == 1 ? tile * TILE_ROWS : tile * NT * TILE_ROWS;
                // source of this lane's activation row (lanes 2 .. 2 + cols)
                const uint8_t* xsrc = nullptr;
                if (lane >= 2 && lane - 2 < cols) {
                    if (PHASE == 1) xsrc = reinterpret_cast<const uint8_t*>(P.xp + (size_t)P.sorted[pair0 + lane - 2].token * P.d);
                    else xsrc = reinterpret_cast<const uint8_t*>(P.actp + (size_t)(pair0 + lane - 2) * P.f);
                }
                for (uint32_t sb = 0; sb < geo.nsb && ok; ++sb) {
                    const long long t0 = P.dbg ? clock64() : 0;
                    const uint32_t sbuf = my_sseq & 1u, sph = (my_sseq >> 1) & 1u;
                    if (!mbar_wait(&C.sempty[sbuf], sph ^ 1u)) { ok = false; break; }
                    if (lane == 0) mbar_expect_tx(&C.sfull[sbuf], 2 * NT * TILE_ROWS * geo.srb);
                    __syncwarp();
                    if (lane < 2 * NT) {
                        const uint32_t tl = lane >> 1, arr = lane & 1u;
                        const CUtensorMap* map = G.maps + (PHASE == 1 ? 3 + 2 * tl + arr : 7 + arr);
                        tma_load_3d(sbufs + sbuf * SCALE_BUF_BYTES + lane * TILE_ROWS * geo.srb, map, sb * geo.srb,
                                    PHASE == 1 ? row0 : row0 + tl * TILE_ROWS, G.slot, &C.sfull[sbuf]);
                    }
                    ++my_sseq;
                    for (uint32_t kc = sb * geo.kc_per_sb; kc < (sb + 1) * geo.kc_per_sb; ++kc) {
                        const uint32_t s = my_seq % STAGES, ph = (my_seq / STAGES) & 1u;
                        if (!mbar_wait(&C.empty[s], ph ^ 1u)) { ok = false; break; }
                        uint8_t* st = C.ring + s * STAGE_BYTES;
                        if (lane == 0) mbar_expect_tx(&C.full[s], NT * TILE_BYTES + cols * KC * 2);
                        __syncwarp();
                        if (lane < NT) {
                            const CUtensorMap* map = G.maps + (PHASE == 1 ? lane : 2);
                            tma_load_3d(st + lane * TILE_BYTES, map, kc * TILE_ROW_BYTES, PHASE == 1 ? row0 : row0 + lane * TILE_ROWS,
                                        G.slot, &C.full[s]);
                        } else if (xsrc) {
                            bulk_g2s(st + NT * TILE_BYTES + (lane - 2) * X_STRIDE, xsrc + (size_t)kc * KC * 2, KC * 2, &C.full[s]);
                        }
                        ++my_seq;
                    }
                    if (P.dbg) dbg_add(P.dbg, warp, lane, DBG, t0);
                }
            }
            MFB_ADVANCE_UNIT();
        }
    } else {
        // ------------------------------------------------------------ eight computing warps, sixteen rows each
        const uint32_t gq = lane >> 2, t = lane & 3;
        const uint32_t rho = gq < 4 ? 2 * gq : 2 * (gq - 4) + 1;
        const uint32_t row_lo = 16 * warp + rho;                                   // tile-local; the upper MMA row is row_lo + 8
        const uint32_t wbase = row_lo * TILE_ROW_BYTES + ((((t >> 1) ^ (rho & 1u)) << 4) | ((t & 1u) << 3));
        const uint32_t swz = (rho & 6u) << 4;
        const uint32_t xoff = NT * TILE_BYTES + gq * X_STRIDE + t * 32;
        const long long t_phase = P.dbg ? clock64() : 0;
        for (uint32_t u = first; u < last && ok; ++u) {
            const uint32_t cols = min(8u, G.pair_count - tt * 8), pair0 = G.pair_start + tt * 8;
            if (G.ok) {
                ++ok_units;
                float acc[NT][4];
#pragma unroll
                for (int tl = 0; tl < (int)NT; ++tl)
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[tl][c] = 0.0f;
                for (uint32_t sb = 0; sb < geo.nsb && ok; ++sb) {
                    const uint32_t sbuf = my_sseq & 1u, sph = (my_sseq >> 1) & 1u;
                    if (!mbar_wait(&C.sfull[sbuf], sph)) { ok = false; break; }
                    const uint8_t* sbase = sbufs + sbuf * SCALE_BUF_BYTES;
                    for (uint32_t kci = 0; kci < geo.kc_per_sb; ++kci) {
                        const uint32_t s = my_seq % STAGES, ph = (my_seq / STAGES) & 1u;
                        long long t0 = P.dbg ? clock64() : 0;
                        if (!mbar_wait(&C.full[s], ph)) { ok = false; break; }
                        if (P.dbg) { dbg_add(P.dbg, warp, lane, DBG, t0); t0 = clock64(); }
                        const uint8_t* st = C.ring + s * STAGE_BYTES;
                        // scale and bias of this chunk's four groups for the lane's two rows of both tiles
                        const uint32_t jj = kci * GPC;
                        const uint32_t soff = geo.srb == 32 ? row_lo * 32 + ((((jj >> 3) ^ (row_lo >> 2)) & 1u) << 4) + (jj & 7u) * 2
                                                            : row_lo * 16 + jj * 2;
                        ScaleRow<GPC> sr[NT][4];   // [tile][scale lo, scale hi, bias lo, bias hi]
#pragma unroll
                        for (int tl = 0; tl < (int)NT; ++tl) {
                            const uint8_t* sa = sbase + (2 * tl) * TILE_ROWS * geo.srb + soff;
                            const uint8_t* ba = sa + TILE_ROWS * geo.srb;
                            sr[tl][0].load(reinterpret_cast<const uint16_t*>(sa));
                            sr[tl][1].load(reinterpret_cast<const uint16_t*>(sa + 8 * geo.srb));
                            sr[tl][2].load(reinterpret_cast<const uint16_t*>(ba));
                            sr[tl][3].load(reinterpret_cast<const uint16_t*>(ba + 8 * geo.srb));
                        }
#pragma unroll
                        for (int j = 0; j < (int)GPC; ++j) {
                            uint32_t bf[8];
                            {
                                const uint4 lo = *reinterpret_cast<const uint4*>(st + xoff + j * 128);
                                const uint4 hi = *reinterpret_cast<const uint4*>(st + xoff + j * 128 + 16);
                                bf[0] = lo.x; bf[1] = lo.y; bf[2] = lo.z; bf[3] = lo.w;
                                bf[4] = hi.x; bf[5] = hi.y; bf[6] = hi.z; bf[7] = hi.w;
                            }
                            const float2 sx = group_sum<4>(bf);
                            const uint32_t woff = wbase + ((32u * j) ^ swz);
#pragma unroll
                            for (int tl = 0; tl < (int)NT; ++tl) {
                                const uint2 a = *reinterpret_cast<const uint2*>(st + tl * TILE_BYTES + woff);
                                const uint2 b = *reinterpret_cast<const uint2*>(st + tl * TILE_BYTES + woff + 8 * TILE_ROW_BYTES);
                                const uint32_t wl[2] = {a.x, a.y}, wh[2] = {b.x, b.y};
                                uint32_t pl[8], phh[8];
                                Unpack<4>::run(wl, pl);
                                Unpack<4>::run(wh, phh);
                                float dsum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    mma16816(dsum, pl[2 * q], phh[2 * q], pl[2 * q + 1], phh[2 * q + 1], bf[2 * q], bf[2 * q + 1]);
                                const float s_lo = sr[tl][0].template at<SDT>(j), s_hi = sr[tl][1].template at<SDT>(j);
                                const float b_lo = sr[tl][2].template at<SDT>(j), b_hi = sr[tl][3].template at<SDT>(j);
                                acc[tl][0] = fmaf(s_lo, dsum[0], acc[tl][0]); acc[tl][0] = fmaf(b_lo, sx.x, acc[tl][0]);
                                acc[tl][1] = fmaf(s_lo, dsum[1], acc[tl][1]); acc[tl][1] = fmaf(b_lo, sx.y, acc[tl][1]);
                                acc[tl][2] = fmaf(s_hi, dsum[2], acc[tl][2]); acc[tl][2] = fmaf(b_hi, sx.x, acc[tl][2]);
                                acc[tl][3] = fmaf(s_hi, dsum[3], acc[tl][3]); acc[tl][3] = fmaf(b_hi, sx.y, acc[tl][3]);
                            }
                        }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&C.empty[s]);
                        ++my_seq;
                        if (P.dbg) dbg_add(P.dbg, warp, lane, DBG + 1, t0);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&C.sempty[sbuf]);
                    ++my_sseq;
                }
                if (!ok) break;
                // ---- epilogue on registers: the lane holds rows (row_lo, row_lo + 8) x token columns (2t, 2t + 1)
                if (PHASE == 1) {
                    const bool clamp = !G.shared && P.limit > 0.0f;   // moe_swiglu_clamp (moe.metal:27-34), routed experts only
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t r = tile * TILE_ROWS + row_lo + 8 * h;
                        const uint32_t act_col = (r & ~15u) + perm_pos(r & 15u, 4);
                        const float act_scale = perm_scale(r & 15u, 4);
#pragma unroll
                        for (int c = 0; c < 2; ++c) {
                            const uint32_t n = 2 * t + c;
                            if (n >= cols) continue;
                            float gate = acc[0][2 * h + c] * CODE_UNSCALE, up = acc[1][2 * h + c] * CODE_UNSCALE;
                            if (clamp) {
                                gate = fminf(gate, P.limit);
                                up = fminf(fmaxf(up, -P.limit), P.limit);
                            }
                            float a = hidden_act(gate, (int)P.activation) * up;
                            a = fminf(fmaxf(a, -65504.0f), 65504.0f);
                            P.actp[(size_t)(pair0 + n) * P.f + act_col] = __float2half_rn(a * act_scale);
                        }
                    }
                    if (P.ready) {   // this warp's rows of the unit are written: count it in (release, cumulative over the warp)
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0) red_release_add(P.ready + g, 1u);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        const uint32_t n = 2 * t + c;
                        if (n >= cols) continue;
                        const mfb_pair pr = P.sorted[pair0 + n];
                        float* out = P.partial + ((size_t)pr.token * (P.top_k + 1) + pr.rank) * P.d + tile * NT * TILE_ROWS + row_lo;
#pragma unroll
                        for (int tl = 0; tl < (int)NT; ++tl) {
                            out[tl * TILE_ROWS] = acc[tl][c] * CODE_UNSCALE;
                            out[tl * TILE_ROWS + 8] = acc[tl][2 + c] * CODE_UNSCALE;
                        }
                    }
                }
            } else if (PHASE == 2) {
                // an expert that is not resident contributes nothing: its rows of the partials are cleared
                for (uint32_t o = warp * 32 + lane; o < NT * TILE_ROWS * cols; o += CW * 32) {
                    const mfb_pair pr = P.sorted[pair0 + o / (NT * TILE_ROWS)];
                    P.partial[((size_t)pr.token * (P.top_k + 1) + pr.rank) * P.d + tile * NT * TILE_ROWS + o % (NT * TILE_ROWS)] = 0.0f;
                }
            }
            MFB_ADVANCE_UNIT();
        }
        if (PHASE == 1) fence_proxy_async();   // the hidden activations are read by bulk copies in phase 2
        if (P.dbg) dbg_add(P.dbg, warp, lane, 5 + DBG, t_phase);
    }
#undef MFB_ADVANCE_UNIT
    // every warp walks the same unit list, so the counters agree; on an abort they no longer matter
    seq += ok_units * geo.nkc;
    sseq += ok_units * geo.nsb;
    return ok;
}

}  // namespace wide

// Rank-ordered weighted combine of a slice of (token, column) outputs from the fp32 partial rows: residual first,
// shared expert, then ranks ascending (moe_phase2_down_reduce_k8, moe.metal:349-404; same order as combine_kernel).
__device__ __forceinline__ void combine_slice(const FastParams& P, uint32_t begin, uint32_t end, bool with_shared) {
    const uint32_t slots = P.top_k + 1;
    for (uint32_t o = begin + threadIdx.x; o < end; o += blockDim.x) {
        const uint32_t tok = o / P.d, c = o % P.d;
        const float* pt = P.partial + (size_t)tok * slots * P.d + c;
        float acc = 0.0f;
        if (P.residual) acc = widen16(ld_cg_u16((const uint16_t*)P.residual + o), P.x_dtype);
        if (with_shared) acc += ld_cg_f32(pt + (size_t)P.top_k * P.d);
        for (uint32_t k = 0; k < P.top_k; ++k)
            acc = fmaf(__half2float(__ushort_as_half(P.route_w[(size_t)tok * P.top_k + k])), ld_cg_f32(pt + (size_t)k * P.d), acc);
        store_act(P.y, o, acc, P.x_dtype);
    }
}

// ------------------------------------------------------------------------------------------ separate kernels
struct FastShared {
    uint64_t full1[MAX_STAGES], empty1[MAX_STAGES], full2[MAX_STAGES], empty2[MAX_STAGES];
    uint64_t wfull[wide::STAGES], wempty[wide::STAGES], sfull[2], sempty[2];   // row-stationary form
    uint32_t pref1[MAX_GROUPS + 1], pref2[MAX_GROUPS + 1], wpref1[MAX_GROUPS + 1];
    uint32_t range[4];   // this CTA's [first, last) units of phase 1 and of phase 2
    uint32_t flag, n_groups;
    float red[32];
};

__device__ __forceinline__ void init_barriers(FastShared& S) {
    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(&S.full1[s], 1); mbar_init(&S.empty1[s], CW);
            mbar_init(&S.full2[s], 1); mbar_init(&S.empty2[s], CW);
        }
        for (uint32_t s = 0; s < wide::STAGES; ++s) { mbar_init(&S.wfull[s], 1); mbar_init(&S.wempty[s], CW); }
        for (int b = 0; b < 2; ++b) { mbar_init(&S.sfull[b], 1); mbar_init(&S.sempty[b], CW); }
        fence_barrier_init();
    }
    __syncthreads();
}

// This CTA's contiguous share of each phase's units: cuts at equal weight (see warp_unit_prefix2).  Called by warp 0
// right after the prefix sums; lanes 0..3 each find one of the four cut points.
template <bool TWO>   // wpref2: scratch of MAX_GROUPS + 1 entries, dead once the ranges are found (used when TWO)
__device__ __forceinline__ void warp_unit_ranges(FastShared& S, const mfb_group* groups, uint32_t n_groups, uint32_t tiles1,
                                                 uint32_t tiles2, UnitBases ub, const uint32_t* wpref2, uint32_t lane) {
    if (lane < 4)
        S.range[lane] = unit_at_cut(groups, n_groups, lane < 2 ? S.pref1 : S.pref2, (lane < 2 || !TWO) ? S.wpref1 : wpref2,
                                    lane < 2 ? tiles1 : tiles2, (lane < 2 || !TWO) ? ub.b1 : ub.b2, blockIdx.x + (lane & 1u),
                                    gridDim.x);
}

// Phase 1 (NMAT = 2) or phase 2 (NMAT = 1) over the groups of one layer call, as a kernel of its own.
template <int NMAT, int NGW>
__global__ void __launch_bounds__(FAST_THREADS, 1) ffn_phase_kernel(const FastParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ FastShared S;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t max_bits = P.shared_blob && P.shared_bits > P.bits ? P.shared_bits : P.bits;
    const PhaseGeom geo = NMAT == 2 ? phase_geom(2, P.d, P.f, NGW, max_bits, RING_BYTES)
                                    : phase_geom(1, P.f, P.d, NGW, max_bits, RING_BYTES);
    init_barriers(S);
    const uint32_t n_groups = *P.n_groups;
    if (warp == 0) {
        const UnitBases ub = unit_bases(P.n_tokens > 16);
        uint32_t* wpref2 = reinterpret_cast<uint32_t*>(smem);   // the stage ring is not in use yet
        warp_unit_prefix2<true>(P.groups, n_groups, geo.tiles, geo.tiles, S.pref1, S.pref2, S.wpref1, wpref2, ub, lane);
        warp_unit_ranges<true>(S, P.groups, n_groups, geo.tiles, geo.tiles, ub, wpref2, lane);
    }
    __syncthreads();
    PhaseCtx C{smem, S.full1, S.empty1, reinterpret_cast<float*>(smem + RING_BYTES), S.pref1};
    uint32_t seq = 0;
    const uint32_t first = S.range[NMAT == 2 ? 0 : 2], last = S.range[NMAT == 2 ? 1 : 3];   // cut with this phase's weights
    if (!run_phase<NMAT, NGW>(P, geo, C, n_groups, first, last, seq, warp, lane)) atomicOr(P.status, STATUS_MBAR_TIMEOUT);
}

// Unit weights of the row-stationary form: a unit's cost is its k loop, the token columns in use add next to nothing.
__device__ __forceinline__ UnitBases wide_unit_bases() { return UnitBases{64u, 64u}; }
// relative time of a phase-1 and of a phase-2 unit of the row-stationary form (measured: ~10 us and ~3.7 us)
#ifndef MFB_WIDE_T1
#define MFB_WIDE_T1 10
#endif
constexpr uint64_t WIDE_T1 = MFB_WIDE_T1, WIDE_T2 = 4;

__device__ __forceinline__ uint8_t* align_1k(uint8_t* p) {
    return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~(uintptr_t)1023);
}

// Phase 1 or phase 2 in the row-stationary form, as a kernel of its own (batches above 16 rows).
template <int PHASE>
__global__ void __launch_bounds__(FAST_THREADS, 1) ffn_wide_kernel(const FastParams P) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ FastShared S;
    uint8_t* smem = align_1k(smem_raw);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const wide::Geom geo = wide::geom(PHASE, P.d, P.f);
    init_barriers(S);
    const uint32_t n_groups = *P.n_groups;
    if (warp == 0) {
        const UnitBases ub = wide_unit_bases();
        uint32_t* wpref2 = reinterpret_cast<uint32_t*>(smem);   // the stage ring is not in use yet
        warp_unit_prefix2<true>(P.groups, n_groups, geo.tiles, geo.tiles, S.pref1, S.pref2, S.wpref1, wpref2, ub, lane);
        warp_unit_ranges<true>(S, P.groups, n_groups, geo.tiles, geo.tiles, ub, wpref2, lane);
    }
    __syncthreads();
    const wide::Ctx C{smem, S.wfull, S.wempty, S.sfull, S.sempty, S.pref1, nullptr};
    uint32_t seq = 0, sseq = 0;
    const uint32_t first = S.range[0], last = S.range[1];
    const bool ok = P.scale_dtype == MFB_DT_BF16 ? wide::run<PHASE, MFB_DT_BF16>(P, geo, C, n_groups, first, last, seq, sseq, warp, lane)
                                                 : wide::run<PHASE, MFB_DT_F16>(P, geo, C, n_groups, first, last, seq, sseq, warp, lane);
    if (!ok) atomicOr(P.status, STATUS_MBAR_TIMEOUT);
}

// Self-test of the bounded wait every pipeline above relies on: one CTA, one mbarrier that nothing ever arrives at.
// The wait gives up after `limit` SM cycles, the kernel records it in the status word and returns normally.
__global__ void wait_selftest_kernel(uint32_t* status, long long limit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait(&bar, 0u, limit)) atomicOr(status, STATUS_MBAR_TIMEOUT);
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
        xp[row * d + (i & ~15u) + perm_pos(i & 15u, bits)] = __float2half_rn(v * perm_scale(i & 15u, bits));
        if (xp2) xp2[row * d + (i & ~15u) + perm_pos(i & 15u, bits2)] = __float2half_rn(v * perm_scale(i & 15u, bits2));
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
        // release at GPU scope: cumulative over what the CTA's threads wrote before the __syncthreads above; the acquire
        // load of the poll below is its counterpart, so no separate fences
        asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(M.bar_counter), "r"(1u) : "memory");
        bool ok = true;
        const long long t0 = clock64();
        // one L2 round trip per poll: the abort word and the clock are looked at every sixteenth poll only
        for (uint32_t polls = 1; ld_acquire_u32(M.bar_counter) < epoch; ++polls) {
            if (polls & 15u) continue;
            if (ld_acquire_u32(M.abort) != 0u) { ok = false; break; }
            if (clock64() - t0 > GRID_WAIT_CYCLES) {
                atomicOr(M.status, STATUS_GRID_BARRIER_TIMEOUT);
                atomicExch(M.abort, 1u);
                ok = false;
                break;
            }
        }
        S.flag = ok ? 1u : 0u;
    }
    __syncthreads();
    return S.flag != 0u;
}

// RMSNorm of one row by the first 256 threads of the CTA, arithmetic and order of rmsnorm_kernel (glue.cu).
// Writes the row in the activation dtype and in the permuted fp16 layout(s); the outputs may be global or shared.
// With row_smem the row is read from shared memory (the single-token mode keeps the residual stream there).
__device__ __forceinline__ void mega_norm_row(const MegaParams& M, const MegaLayer& Ly, FastShared& S, const void* h,
                                              uint32_t tok, uint16_t* xn_out, __half* xp_out, __half* xp2_out,
                                              const uint16_t* row_smem = nullptr) {
    const uint32_t d = M.d, tid = threadIdx.x;
    const uint16_t* src = (const uint16_t*)h + (size_t)tok * d;
    // the gain of this thread's first eight columns is requested now, so that its latency runs beside the reductions
    constexpr uint32_t GAIN_REGS = 8;
    float gain[GAIN_REGS];
#pragma unroll
    for (uint32_t j = 0; j < GAIN_REGS; ++j) {
        const uint32_t i = tid + 256 * j;
        gain[j] = (tid < 256 && i < d && Ly.norm_w) ? __bfloat162float(Ly.norm_w[i]) : 1.0f;
    }
    float ss = 0.0f;
    if (tid < 256) {
#pragma unroll 8
        for (uint32_t i = tid; i < d; i += 256) {
            const float v = widen16(row_smem ? row_smem[i] : ld_cg_u16(src + i), M.x_dtype);
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
#pragma unroll
        for (uint32_t j = 0; j < GAIN_REGS; ++j) {
            const uint32_t i = tid + 256 * j;
            if (i >= d) break;
            float v = widen16(row_smem ? row_smem[i] : ld_cg_u16(src + i), M.x_dtype);
            v = v * inv * gain[j];
            const uint16_t bits = narrow16(v, M.x_dtype);
            xn_out[i] = bits;
            v = fminf(fmaxf(widen16(bits, M.x_dtype), -65504.0f), 65504.0f);
            xp_out[(i & ~15u) + perm_pos(i & 15u, M.bits)] = __float2half_rn(v * perm_scale(i & 15u, M.bits));
            if (xp2_out) xp2_out[(i & ~15u) + perm_pos(i & 15u, M.shared_bits)] = __float2half_rn(v * perm_scale(i & 15u, M.shared_bits));
        }
        for (uint32_t i = tid + 256 * GAIN_REGS; i < d; i += 256) {
            float v = widen16(row_smem ? row_smem[i] : ld_cg_u16(src + i), M.x_dtype);
            const float gw = Ly.norm_w ? __bfloat162float(Ly.norm_w[i]) : 1.0f;
            v = v * inv * gw;
            const uint16_t bits = narrow16(v, M.x_dtype);
            xn_out[i] = bits;
            v = fminf(fmaxf(widen16(bits, M.x_dtype), -65504.0f), 65504.0f);
            xp_out[(i & ~15u) + perm_pos(i & 15u, M.bits)] = __float2half_rn(v * perm_scale(i & 15u, M.bits));
            if (xp2_out) xp2_out[(i & ~15u) + perm_pos(i & 15u, M.shared_bits)] = __float2half_rn(v * perm_scale(i & 15u, M.shared_bits));
        }
        fence_proxy_async();   // the row-stationary phases fetch these rows with bulk copies
    }
    __syncthreads();
}

// logits[t, e] in the fixed summation order of router_logits_kernel: lane l takes k = l, l+32, ... ascending, then
// a xor butterfly, the bias last.  The (expert, token) plane is cut into tasks of EB consecutive experts x
// (warps x TT) tokens, dealt round-robin to the CTAs.  A CTA stages the EB gate rows as fp32 in `stage`; each
// warp fetches its TT token rows into shared memory with asynchronous 16-byte copies (in flight while the gate
// rows are converted) and then forms the EB x TT dot products together, so that every shared-memory load feeds
// several multiply-adds.  With x_smem the single activation row is already in shared memory.
constexpr uint32_t MEGA_MAX_EB = 4, MEGA_MAX_TT = 4;

template <uint32_t EB, uint32_t TT>
__device__ __forceinline__ void mega_logits_run(const MegaParams& M, const MegaLayer& Ly, uint8_t* stage, const uint16_t* x_smem) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5, d = M.d;
    float* w_rows = reinterpret_cast<float*>(stage);                                                       // [EB][d]
    uint16_t* x_stage = reinterpret_cast<uint16_t*>(stage + MEGA_MAX_EB * d * 4) + warp * MEGA_MAX_TT * d; // [warps][TT][d]
    const uint32_t tb = warps * TT;
    const uint32_t n_eb = (M.num_experts + EB - 1) / EB, n_tb = (M.n_tokens + tb - 1) / tb;
    for (uint32_t task = blockIdx.x; task < n_eb * n_tb; task += gridDim.x) {
        const uint32_t e0 = (task % n_eb) * EB, t0 = (task / n_eb) * tb + warp * TT;
        const uint32_t ne = min(EB, M.num_experts - e0);
        const uint32_t nt = t0 < M.n_tokens ? min(TT, M.n_tokens - t0) : 0;
        __syncthreads();
        if (!x_smem) {
            for (uint32_t r = 0; r < nt; ++r) {
                const uint16_t* x = (const uint16_t*)M.xn + (size_t)(t0 + r) * d;
                for (uint32_t i = lane; i < d / 8; i += 32) cp_async16(x_stage + r * d + i * 8, x + i * 8);
            }
            cp_async_commit();
        }
        for (uint32_t j = 0; j < ne; ++j)
        for (uint32_t c = threadIdx.x; c < d / 8; c += blockDim.x) {
            const uint4 q = *reinterpret_cast<const uint4*>(Ly.router_w + (size_t)(e0 + j) * d + c * 8);
            float* dst = w_rows + j * d + c * 8;
            *reinterpret_cast<float4*>(dst) = make_float4(__uint_as_float(q.x << 16), __uint_as_float(q.x & 0xFFFF0000u),
                                                          __uint_as_float(q.y << 16), __uint_as_float(q.y & 0xFFFF0000u));
            *reinterpret_cast<float4*>(dst + 4) = make_float4(__uint_as_float(q.z << 16), __uint_as_float(q.z & 0xFFFF0000u),
                                                              __uint_as_float(q.w << 16), __uint_as_float(q.w & 0xFFFF0000u));
        }
        cp_async_wait_all();
        __syncthreads();
        if (nt == 0) continue;
        const uint16_t* xr = x_smem ? x_smem : x_stage;
        float acc[EB][TT];
#pragma unroll
        for (uint32_t j = 0; j < EB; ++j)
#pragma unroll
            for (uint32_t r = 0; r < TT; ++r) acc[j][r] = 0.0f;
#pragma unroll 2
        for (uint32_t i = lane; i < d; i += 32) {
            float xv[TT], wv[EB];
#pragma unroll
            for (uint32_t r = 0; r < TT; ++r) xv[r] = r < nt ? widen16(xr[r * d + i], M.x_dtype) : 0.0f;
#pragma unroll
            for (uint32_t j = 0; j < EB; ++j) wv[j] = w_rows[j * d + i];
#pragma unroll
            for (uint32_t j = 0; j < EB; ++j)
#pragma unroll
                for (uint32_t r = 0; r < TT; ++r) acc[j][r] = fmaf(wv[j], xv[r], acc[j][r]);
        }
#pragma unroll
        for (uint32_t j = 0; j < EB; ++j)
#pragma unroll
            for (uint32_t r = 0; r < TT; ++r) {
                float v = acc[j][r];
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                if (lane == 0 && j < ne && r < nt) {
                    if (Ly.logit_bias) v = v + Ly.logit_bias[e0 + j];
                    M.logits[(size_t)(t0 + r) * M.num_experts + e0 + j] = v;
                }
            }
    }
    __syncthreads();
}

__device__ __forceinline__ void mega_logits(const MegaParams& M, const MegaLayer& Ly, uint8_t* stage, const uint16_t* x_smem) {
    const uint32_t warps = blockDim.x >> 5;
    if (M.n_tokens <= warps) {   // one token per warp; two experts per task give 128 tasks for 256 experts
        mega_logits_run<2, 1>(M, Ly, stage, x_smem);
    } else {
        const uint32_t n_tb = (M.n_tokens + warps * 4 - 1) / (warps * 4);
        if (((M.num_experts + 3) / 4) * n_tb * 4 >= gridDim.x * 3) mega_logits_run<4, 4>(M, Ly, stage, x_smem);
        else mega_logits_run<2, 4>(M, Ly, stage, x_smem);
    }
}

// Counting sort of the routing table into shared memory, identical order to group.cu / route_small_kernel; every
// CTA builds the same lists.  run_s (u32) and mask_s (u64) are scratch of num_experts entries; warp 0 does the scans.
// Two forms with the same result.  The scan form places 32 pairs per round with one warp (cheap for a few dozen
// pairs); the mask form places all pairs at once (several hundred pairs).  The kernel is instantiated once per form
// (LARGE_BATCH) so that neither changes the other's code.
__device__ __forceinline__ void mega_group_scan(const MegaParams& M, FastShared& S, const uint32_t* idx_s, const uint16_t* w_s,
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

__device__ __forceinline__ void mega_group_mask(const MegaParams& M, FastShared& S, const uint32_t* idx_s, const uint16_t* w_s,
                                           uint32_t* run_s, unsigned long long* mask_s, mfb_pair* sorted_s, mfb_group* groups_s,
                                           bool shared) {
    // A token selects an expert at most once and there are at most 64 tokens, so the rows of a group are a 64-bit
    // token mask per expert: the count is its population count, a pair's place inside its group the number of set
    // bits below its token.  That is the (token, rank) order of the stable sort, found without any serial scan.
    const uint32_t n_pairs = M.n_tokens * M.top_k, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t e = threadIdx.x; e < M.num_experts; e += blockDim.x) mask_s[e] = 0ull;
    __syncthreads();
    for (uint32_t p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicOr(&mask_s[idx_s[p]], 1ull << (p / M.top_k));
    __syncthreads();
    if (warp == 0) {
        const uint32_t per = (M.num_experts + 31) / 32, e0 = lane * per;
        uint32_t cnt = 0, nz = 0;
        for (uint32_t j = 0; j < per; ++j)
            if (e0 + j < M.num_experts) { const uint32_t c = __popcll(mask_s[e0 + j]); cnt += c; nz += c ? 1u : 0u; }
        uint32_t cnt_incl = cnt, nz_incl = nz;
        for (uint32_t off = 1; off < 32; off <<= 1) {
            const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, cnt_incl, off), b = __shfl_up_sync(0xFFFFFFFFu, nz_incl, off);
            if (lane >= off) { cnt_incl += a; nz_incl += b; }
        }
        uint32_t run = cnt_incl - cnt, gi = nz_incl - nz;
        for (uint32_t j = 0; j < per; ++j)
            if (e0 + j < M.num_experts) {
                const uint32_t c = __popcll(mask_s[e0 + j]);
                run_s[e0 + j] = run;
                if (c) { groups_s[gi].expert = e0 + j; groups_s[gi].pair_start = run; groups_s[gi].pair_count = c; ++gi; }
                run += c;
            }
        uint32_t ng = __shfl_sync(0xFFFFFFFFu, nz_incl, 31);
        if (lane == 0) {
            if (shared) { groups_s[ng].expert = M.num_experts; groups_s[ng].pair_start = n_pairs; groups_s[ng].pair_count = M.n_tokens; ++ng; }
            S.n_groups = ng;
        }
    } else if (shared) {
        for (uint32_t t = threadIdx.x - 32; t < M.n_tokens; t += blockDim.x - 32) {
            mfb_pair out;
            out.token = t; out.expert = M.num_experts; out.rank = M.top_k; out.weight_bits = 0x3C00u;
            sorted_s[n_pairs + t] = out;
        }
    }
    __syncthreads();
    for (uint32_t p = threadIdx.x; p < n_pairs; p += blockDim.x) {
        const uint32_t e = idx_s[p], t = p / M.top_k;
        mfb_pair out;
        out.token = t; out.expert = e; out.rank = p - t * M.top_k; out.weight_bits = w_s[p];
        sorted_s[run_s[e] + __popcll(mask_s[e] & ((1ull << t) - 1ull))] = out;
    }
    __syncthreads();
}

// Single-token mode, gate logits: one warp per expert (expert e by warp e / grid of CTA e % grid).  The gate row does
// not depend on the activations: its asynchronous copy into the warp's shared-memory row starts at the top of the layer
// and lands while the norm runs.  Same summation order as router_logits_kernel.
__device__ __forceinline__ void single_fetch_gate_row(const MegaParams& M, const MegaLayer& Ly, uint32_t e, uint32_t lane, uint16_t* wrow) {
    if (e < M.num_experts)
        for (uint32_t c = lane; c < M.d / 8; c += 32) cp_async16(wrow + c * 8, Ly.router_w + (size_t)e * M.d + c * 8);
    cp_async_commit();
}

__device__ __forceinline__ void single_logit(const MegaParams& M, const MegaLayer& Ly, uint32_t e, uint32_t lane, const uint16_t* wrow,
                                             const uint16_t* xn_s) {
    cp_async_wait_all();
    __syncwarp();
    if (e >= M.num_experts) return;
    float acc = 0.0f;
#pragma unroll 8
    for (uint32_t i = lane; i < M.d; i += 32) acc = fmaf(__uint_as_float((uint32_t)wrow[i] << 16), widen16(xn_s[i], M.x_dtype), acc);
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0) {
        if (Ly.logit_bias) acc = acc + Ly.logit_bias[e];
        M.logits[e] = acc;
    }
}

__device__ __forceinline__ float4 ld_cg_f4(const float* p) {
    float4 v;
    asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// Single-token mode, combine: every CTA forms the whole new row itself from the fp32 partial rows (rank order, as
// combine_slice) and keeps it in shared memory as the next layer's input; CTA 0 also stores it.  Four columns per
// thread, the loads of up to eight ranks in flight together.
__device__ __forceinline__ void single_combine(const MegaParams& M, const uint16_t* w_s, bool with_shared, uint16_t* h_s, void* h_out) {
    const uint32_t d = M.d;
    for (uint32_t c = threadIdx.x * 4; c < d; c += blockDim.x * 4) {
        const float* pt = M.partial + c;
        const uint2 hb = *reinterpret_cast<const uint2*>(h_s + c);
        float acc[4] = {widen16((uint16_t)(hb.x & 0xFFFFu), M.x_dtype), widen16((uint16_t)(hb.x >> 16), M.x_dtype),
                        widen16((uint16_t)(hb.y & 0xFFFFu), M.x_dtype), widen16((uint16_t)(hb.y >> 16), M.x_dtype)};
        if (with_shared) {
            const float4 sh = ld_cg_f4(pt + (size_t)M.top_k * d);
            acc[0] += sh.x; acc[1] += sh.y; acc[2] += sh.z; acc[3] += sh.w;
        }
        for (uint32_t k0 = 0; k0 < M.top_k; k0 += 8) {
            float4 v[8];
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) v[j] = k0 + j < M.top_k ? ld_cg_f4(pt + (size_t)(k0 + j) * d) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) {
                if (k0 + j < M.top_k) {
                    const float w = __half2float(__ushort_as_half(w_s[k0 + j]));
                    acc[0] = fmaf(w, v[j].x, acc[0]); acc[1] = fmaf(w, v[j].y, acc[1]);
                    acc[2] = fmaf(w, v[j].z, acc[2]); acc[3] = fmaf(w, v[j].w, acc[3]);
                }
            }
        }
        uint2 ob;
        ob.x = (uint32_t)narrow16(acc[0], M.x_dtype) | ((uint32_t)narrow16(acc[1], M.x_dtype) << 16);
        ob.y = (uint32_t)narrow16(acc[2], M.x_dtype) | ((uint32_t)narrow16(acc[3], M.x_dtype) << 16);
        *reinterpret_cast<uint2*>(h_s + c) = ob;
        if (blockIdx.x == 0) *reinterpret_cast<uint2*>((uint16_t*)h_out + c) = ob;
    }
    __syncthreads();
}

// MODE 0: at most 16 rows (one-warp scan for the sort, flat unit weights); 1: more rows, k-split FFN phases;
// 2: more rows, row-stationary FFN phases (every layer carries tensor maps).
template <int NGW, int MODE>
__global__ void __launch_bounds__(FAST_THREADS, 1) stack_mega_kernel(const MegaParams M) {
    constexpr bool LARGE_BATCH = MODE >= 1, WIDE = MODE == 2;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ FastShared S;
    // the tensor copies of the row-stationary form want their tiles on a 1 KB boundary; the other instantiations keep
    // the array itself as the base (a run-time base pointer costs them registers they do not have)
    uint8_t* const smem = WIDE ? align_1k(smem_raw) : smem_raw;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t max_bits = M.shared_bits > M.bits ? M.shared_bits : M.bits;
    const PhaseGeom geo1 = phase_geom(2, M.d, M.f, NGW, max_bits, RING_BYTES);
    const PhaseGeom geo2 = phase_geom(1, M.f, M.d, 4, max_bits, RING_BYTES);
    const uint32_t n_pairs = M.n_tokens * M.top_k;
    const bool single = MODE == 0 && M.n_tokens == 1;   // compiled out of the large-batch forms
    // ---- shared memory carve-up.  Region A holds the stage ring of whichever phase runs plus the k-split exchange
    // buffers; during the router phase it stages gate rows.  The routing lists follow it.
    uint8_t* region_a = smem;
    const uint32_t region_a_bytes = WIDE ? wide::RING_BYTES : RING_BYTES + RED_BYTES;
    float* red = reinterpret_cast<float*>(smem + RING_BYTES);
    const wide::Geom wgeo1 = wide::geom(1, M.d, M.f), wgeo2 = wide::geom(2, M.d, M.f);
    const uint32_t tiles1 = WIDE ? wgeo1.tiles : geo1.tiles, tiles2 = WIDE ? wgeo2.tiles : geo2.tiles;
    mfb_pair* sorted_s = reinterpret_cast<mfb_pair*>(smem + region_a_bytes);
    mfb_group* groups_s = reinterpret_cast<mfb_group*>(sorted_s + (n_pairs + M.n_tokens));
    uint32_t* idx_s = reinterpret_cast<uint32_t*>(groups_s + (M.num_experts + 1));
    uint16_t* w_s = reinterpret_cast<uint16_t*>(idx_s + n_pairs);
    uint32_t* run_s = reinterpret_cast<uint32_t*>(w_s + ((n_pairs + 1) & ~1u));
    // single-token mode keeps the normalised row in shared memory (16-byte aligned)
    uint16_t* xn_s = reinterpret_cast<uint16_t*>((reinterpret_cast<uintptr_t>(run_s + M.num_experts) + 15) & ~(uintptr_t)15);
    __half* xp_s = reinterpret_cast<__half*>(xn_s + M.d);
    __half* xp2_s = xp_s + M.d;
    uint16_t* h_s = reinterpret_cast<uint16_t*>(xp2_s + M.d);   // single-token mode: the residual stream's row

    init_barriers(S);
    uint32_t split_groups = 0;
    uint32_t epoch = 0, seq1 = 0, seq2 = 0;   // row-stationary form: seq1 counts stages, seq2 scale blocks
    bool alive = true;
    // SM clock against the global timer over the whole launch (row 16 of the cycle counters): cycles per ns
    auto clock_pair = [&](int slot) {
        if (M.trace && blockIdx.x == 0 && threadIdx.x == 0) {
            uint64_t t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            uint64_t* row = M.trace + (size_t)M.n_layers * 8 + 16 * 8;
            row[4 + slot] = (uint64_t)clock64();
            row[6 + slot] = t;
        }
    };
    clock_pair(0);
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
            // every CTA keeps the row in shared memory and normalises it itself (no barrier), computes the logits of
            // its experts, and after the barrier every CTA repeats the selection: two grid barriers fewer per layer.
            // The gate rows do not depend on the row: they are requested first.
            const uint32_t e_w = blockIdx.x + warp * gridDim.x;
            uint16_t* gate_row = reinterpret_cast<uint16_t*>(region_a) + (size_t)warp * M.d;
            single_fetch_gate_row(M, Ly, e_w, lane, gate_row);
            if (l == 0 || M.layer_stride != 0) {
                for (uint32_t i = threadIdx.x; i < M.d; i += blockDim.x) h_s[i] = ld_cg_u16((const uint16_t*)h + i);
                __syncthreads();
            }
            mega_norm_row(M, Ly, S, h, 0, xn_s, xp_s, M.xp2 ? xp2_s : nullptr, h_s);
            stamp(1);
            single_logit(M, Ly, e_w, lane, gate_row, xn_s);
            for (uint32_t e = e_w + (blockDim.x >> 5) * gridDim.x; e < M.num_experts; e += (blockDim.x >> 5) * gridDim.x) {
                single_fetch_gate_row(M, Ly, e, lane, gate_row);   // more experts than warps in the grid: further rounds
                single_logit(M, Ly, e, lane, gate_row, xn_s);
            }
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
            if (LARGE_BATCH) mega_group_mask(M, S, idx_s, w_s, run_s, reinterpret_cast<unsigned long long*>(region_a), sorted_s, groups_s, shared);
            else mega_group_scan(M, S, idx_s, w_s, run_s, sorted_s, groups_s, shared);
        }
        const uint32_t n_groups = S.n_groups;
        // one token: every group holds one pair, so the split of the units over the CTAs is that of the first layer
        // as long as the group count (shared expert or not) stays what it was
        const bool same_split = single && l > 0 && n_groups == split_groups;
        split_groups = n_groups;
        if (warp == 0 && !same_split) {
            const UnitBases ub = WIDE ? wide_unit_bases() : unit_bases(LARGE_BATCH);
            uint32_t* wpref2 = reinterpret_cast<uint32_t*>(region_a);   // the stage ring is not in use yet
            warp_unit_prefix2<LARGE_BATCH>(groups_s, n_groups, tiles1, tiles2, S.pref1, S.pref2, S.wpref1, wpref2, ub, lane);
            warp_unit_ranges<LARGE_BATCH>(S, groups_s, n_groups, tiles1, tiles2, ub, wpref2, lane);
            if (WIDE && M.ready && lane == 0) {
                // Without a barrier between the phases a CTA's time is the sum of its two shares, so phase 2 is cut to
                // even out what the whole-unit cuts of phase 1 left uneven (six or seven units of ~10 us each): CTA k
                // starts phase 2 at the unit where k / n of the total time, less the phase-1 time in front of its
                // phase-1 cut, is spent.  Depends only on k and cut k, so neighbours agree on their common boundary.
                const uint64_t u1 = S.pref1[n_groups], u2 = S.pref2[n_groups], n = gridDim.x;
                const uint64_t total = WIDE_T1 * u1 + WIDE_T2 * u2;
                auto cut2 = [&](uint64_t k, uint64_t cut1) -> uint32_t {
                    if (k >= n) return (uint32_t)u2;
                    const long long v = ((long long)(k * total / n) - (long long)(WIDE_T1 * cut1)) / (long long)WIDE_T2;
                    return (uint32_t)(v < 0 ? 0 : (v > (long long)u2 ? (long long)u2 : v));
                };
                S.range[2] = cut2(blockIdx.x, S.range[0]);
                S.range[3] = cut2(blockIdx.x + 1, S.range[1]);
            }
        }
        __syncthreads();

        FastParams P;
        P.pool = Ly.pool; P.slot_stride = Ly.slot_stride; P.slot_of = Ly.slot_of; P.shared_blob = Ly.shared_blob;
        P.routed_off = Ly.routed_off; P.shared_off = Ly.shared_off;
        P.d = M.d; P.f = M.f; P.num_experts = M.num_experts; P.top_k = M.top_k; P.bits = M.bits; P.shared_bits = M.shared_bits;
        P.scale_dtype = M.scale_dtype; P.activation = M.activation; P.limit = M.limit;
        P.sorted = sorted_s; P.groups = groups_s; P.n_groups = &S.n_groups;
        P.xp = single ? xp_s : M.xp; P.xp_shared = single ? (M.xp2 ? xp2_s : xp_s) : (M.xp2 ? M.xp2 : M.xp);
        P.x_in_smem = single ? 1 : 0;
        P.actp = M.actp; P.partial = M.partial; P.route_w = w_s;
        P.dbg = M.trace ? reinterpret_cast<unsigned long long*>(M.trace + (size_t)M.n_layers * 8) : nullptr;
        P.residual = h; P.y = h; P.x_dtype = M.x_dtype; P.n_tokens = M.n_tokens; P.status = M.status;
        P.maps = Ly.maps;
        // row-stationary form: no grid barrier between the FFN phases - a phase-2 unit waits for the phase-1 units of its
        // own group only (per-group counters, one array per layer parity)
        P.ready = (WIDE && M.ready) ? M.ready + (l & 1u) * MEGA_READY_WORDS : nullptr;
        if (WIDE && M.ready && blockIdx.x == 0)   // the other parity's counters were last read before the previous layer's final barrier
            for (uint32_t i = threadIdx.x; i < MEGA_READY_WORDS; i += blockDim.x) M.ready[((l + 1) & 1u) * MEGA_READY_WORDS + i] = 0u;
        stamp(4);

        // ---- phase 1: this CTA's contiguous share of the (group, token tile, row tile) units
        if constexpr (WIDE) {
            const wide::Ctx C{region_a, S.wfull, S.wempty, S.sfull, S.sempty, S.pref1, nullptr};
            const uint32_t first = S.range[0], last = S.range[1];
            const bool ok = M.scale_dtype == MFB_DT_BF16 ? wide::run<1, MFB_DT_BF16>(P, wgeo1, C, n_groups, first, last, seq1, seq2, warp, lane)
                                                         : wide::run<1, MFB_DT_F16>(P, wgeo1, C, n_groups, first, last, seq1, seq2, warp, lane);
            if (!ok) { atomicOr(M.status, STATUS_MBAR_TIMEOUT); atomicExch(M.abort, 1u); }
        } else {
            PhaseCtx C{region_a, S.full1, S.empty1, red, S.pref1};
            const uint32_t first = S.range[0], last = S.range[1];
            if (!run_phase<2, NGW>(P, geo1, C, n_groups, first, last, seq1, warp, lane)) { atomicOr(M.status, STATUS_MBAR_TIMEOUT); atomicExch(M.abort, 1u); }
            if (single && warp == CW) {   // this CTA's phase-2 units, requested into L2 ahead of the barrier
                uint32_t g2 = 0;
                const uint32_t f2 = S.range[2], l2 = S.range[3];
                for (uint32_t u = f2; u < l2; ++u) {
                    seek_group(S.pref2, n_groups, u, g2);
                    phase_prefetch_l2<1>(geo2, group_ref(P, g2), (u - S.pref2[g2]) % geo2.tiles, lane);
                }
            }
        }
        stamp(5);
        if (!(WIDE && M.ready) && !(alive = grid_barrier(M, S, epoch))) break;
        stamp(6);
        // ---- phase 2: down projections of every (group, token tile, 128-row block) into the fp32 partial rows
        if constexpr (WIDE) {
            const wide::Ctx C{region_a, S.wfull, S.wempty, S.sfull, S.sempty, S.pref2, S.pref1};
            const uint32_t first = S.range[2], last = S.range[3];
            const bool ok = M.scale_dtype == MFB_DT_BF16 ? wide::run<2, MFB_DT_BF16>(P, wgeo2, C, n_groups, first, last, seq1, seq2, warp, lane)
                                                         : wide::run<2, MFB_DT_F16>(P, wgeo2, C, n_groups, first, last, seq1, seq2, warp, lane);
            if (!ok) { atomicOr(M.status, STATUS_MBAR_TIMEOUT); atomicExch(M.abort, 1u); }
        } else {
            PhaseCtx C{region_a, S.full2, S.empty2, red, S.pref2};
            const uint32_t first = S.range[2], last = S.range[3];
            if (!run_phase<1, 4>(P, geo2, C, n_groups, first, last, seq2, warp, lane)) { atomicOr(M.status, STATUS_MBAR_TIMEOUT); atomicExch(M.abort, 1u); }
        }
        if (!(alive = grid_barrier(M, S, epoch))) break;
        stamp(7);
        // ---- rank-ordered weighted combine, a contiguous slice of (token, column) outputs per CTA
        if (single) {
            // no barrier behind it: the next layer reads the row from this CTA's shared memory, and the partial rows are
            // not written again before two more barriers
            single_combine(M, w_s, shared, h_s, h);
        } else {
            const uint32_t total = M.n_tokens * M.d, per = (total + gridDim.x - 1) / gridDim.x;
            const uint32_t begin = min(blockIdx.x * per, total);
            combine_slice(P, begin, min(begin + per, total), shared);
            // rows of independent layers need no barrier here: the buffers the next layer writes first are not read by
            // this combine, and the partial rows are not written again before three more barriers
            if (M.layer_stride == 0 && !(alive = grid_barrier(M, S, epoch))) break;
        }
    }
    clock_pair(1);
}

}  // namespace

// ------------------------------------------------------------------------------------------ host side
static uint32_t cfg_max_bits(const mfb_moe_config& c) { return c.shared_bits > c.bits ? c.shared_bits : c.bits; }

bool fast_supported(const mfb_moe_config& c) {
    if (c.shared_bits == 8) return false;                             // 8-bit shared expert: generic kernels
    if (!(c.d == 512 || c.d == 1024 || c.d == 2048)) return false;   // 1, 2 or 4 groups per warp in phase 1 (k split 8)
    if (!(c.f == 256 || c.f == 512)) return false;                   // 4 groups per warp in phase 2 (k split 1 or 2)
    if (c.top_k + 1 > 32) return false;
    const PhaseGeom g1 = phase_geom(2, c.d, c.f, c.d / 512, cfg_max_bits(c), RING_BYTES);
    const PhaseGeom g2 = phase_geom(1, c.f, c.d, 4, cfg_max_bits(c), RING_BYTES);
    if (c.f % g1.tile_rows || c.d % g2.tile_rows) return false;
    return g1.n_stages >= 2 && g2.n_stages >= 2;
}

bool wide_supported(const mfb_moe_config& c) {
    if (!fast_supported(c)) return false;   // the small-batch instantiations and the router steps come from the same kernel
    if (c.bits != 4 || !(c.shared_bits == 0 || c.shared_bits == 4)) return false;
    return c.d % 1024 == 0 && (c.f == 512 || c.f % 1024 == 0);
}

int32_t wide_encode_maps(const mfb_moe_config& c, const mfb_layer_weights& w, WideMaps* out) {
    memset(out, 0, sizeof *out);
    for (int sh = 0; sh < 2; ++sh) {
        const uint8_t* base = sh ? w.shared_blob : w.pool;
        if (!base) continue;
        const mfb_expert_offsets& off = sh ? w.shared_off : w.routed_off;
        const uint32_t* o = &off.gate_w;
        // the third coordinate is the pool slot; a slot table may name any int16 slot, the identity mapping names experts
        const uint64_t slots = sh ? 1 : (w.slot_of ? 32768ull : (uint64_t)c.num_experts);
        const uint64_t blob_stride = w.slot_stride;
        for (int m = 0; m < 3; ++m) {   // gate, up: [f rows, d codes]; down: [d rows, f codes]
            const uint64_t k = m < 2 ? c.d : c.f, rows = m < 2 ? c.f : c.d, gpr = k / 64;
            const uint64_t row_bytes = k / 2, srow_bytes = gpr * 2;
            const uint32_t srb = (uint32_t)(gpr < 16 ? gpr : 16) * 2;
            {
                const uint64_t dims[3] = {row_bytes, rows, slots}, strides[2] = {row_bytes, sh ? rows * row_bytes : blob_stride};
                const uint32_t box[3] = {wide::TILE_ROW_BYTES, wide::TILE_ROWS, 1};
                const int32_t rc = encode_tensor_map(&out->m[sh][m], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base + o[3 * m], dims, strides,
                                                     box, CU_TENSOR_MAP_SWIZZLE_128B);
                if (rc) return rc;
            }
            for (int a = 0; a < 2; ++a) {
                const uint64_t dims[3] = {srow_bytes, rows, slots}, strides[2] = {srow_bytes, sh ? rows * srow_bytes : blob_stride};
                const uint32_t box[3] = {srb, wide::TILE_ROWS, 1};
                const int32_t rc = encode_tensor_map(&out->m[sh][3 + 2 * m + a], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, base + o[3 * m + 1 + a],
                                                     dims, strides, box, srb == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE);
                if (rc) return rc;
            }
        }
    }
    return MFB_OK;
}

size_t fast_smem1(const mfb_moe_config&) { return (size_t)RING_BYTES + RED_BYTES; }
size_t fast_smem2(const mfb_moe_config&, uint32_t) { return (size_t)RING_BYTES + RED_BYTES; }

size_t fast_smem_stack(const mfb_moe_config& c, uint32_t n_tokens, bool wide_form) {
    const size_t pairs = (size_t)n_tokens * c.top_k;
    const size_t lists = (pairs + n_tokens) * sizeof(mfb_pair) + (c.num_experts + 1) * sizeof(mfb_group) + pairs * 4 +
                         ((pairs + 1) & ~(size_t)1) * 2 + c.num_experts * 4 + 16 + (n_tokens == 1 ? (size_t)c.d * 8 : 0);
    const size_t region_a = wide_form && n_tokens > 16 ? (size_t)wide::RING_BYTES : (size_t)RING_BYTES + RED_BYTES;
    if ((size_t)c.d * (MEGA_MAX_EB * 4 + (CW + 1) * MEGA_MAX_TT * 2) > region_a)
        return (size_t)1 << 30;   // the router staging does not fit: the caller falls back to the per-layer launches
    return region_a + lists + 64 + 1024;   // + slack for the 1 KB alignment of the ring
}

template <int NGW>
static cudaError_t fast_init_ngw() {
    cudaError_t e = cudaFuncSetAttribute(ffn_phase_kernel<2, NGW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_mega_kernel<NGW, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(stack_mega_kernel<NGW, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    if (e == cudaSuccess && NGW >= 2) e = cudaFuncSetAttribute(stack_mega_kernel<(NGW >= 2 ? NGW : 2), 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    return e;
}

// One-time opt-in to large dynamic shared memory for the fast kernels (called when a handle is created, so that no
// attribute call happens while a caller captures a CUDA graph).
cudaError_t fast_init() {
    cudaError_t e = cudaFuncSetAttribute(ffn_phase_kernel<1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(ffn_wide_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(ffn_wide_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FAST_SMEM_LIMIT);
    if (e == cudaSuccess) e = fast_init_ngw<1>();
    if (e == cudaSuccess) e = fast_init_ngw<2>();
    if (e == cudaSuccess) e = fast_init_ngw<4>();
    return e;
}

// Whether `blocks` CTAs of the fused kernel can be co-resident on the current device with `smem` bytes of dynamic
// shared memory each (a cooperative launch needs all of them resident at once).
bool stack_mega_fits(const mfb_moe_config& c, int sm_count, size_t smem) {
    int per_sm = 0;
    const void* fn = c.d / 512 == 1 ? (const void*)stack_mega_kernel<1, 0> : c.d / 512 == 2 ? (const void*)stack_mega_kernel<2, 0>
                                                                                            : (const void*)stack_mega_kernel<4, 0>;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, FAST_THREADS, smem) != cudaSuccess) return false;
    return per_sm >= 1 && sm_count >= 1;
}

cudaError_t launch_wait_selftest(cudaStream_t s, uint32_t* status, long long limit_cycles) {
    wait_selftest_kernel<<<1, 32, 0, s>>>(status, limit_cycles);
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_fast_prep(cudaStream_t s, const void* h, int dtype, const __nv_bfloat16* w, uint32_t n_tokens, uint32_t d,
                             float eps, bool do_norm, void* xn, __half* xp, uint32_t bits, __half* xp2, uint32_t bits2) {
    if (n_tokens == 0) return cudaSuccess;
    prep_kernel<<<n_tokens, 256, 0, s>>>(h, dtype, w, d, eps, do_norm ? 1 : 0, xn, xp, bits, xp2, bits2);
    count_launches(1);
    return cudaGetLastError();
}

// Phase 1 and phase 2 as two launches; the caller follows with the combine kernel over P.partial.  Batches above 16
// rows whose layer carries tensor maps (P.maps) take the row-stationary kernels, like the fused kernel does.
cudaError_t launch_fast_ffn(cudaStream_t s, const FastParams& P, const mfb_moe_config& c, int sm_count, uint32_t max_groups) {
    const uint32_t max_bits = cfg_max_bits(c), tts = (P.n_tokens + 7) / 8;
    if (P.maps && P.n_tokens > 16) {
        const wide::Geom g1 = wide::geom(1, c.d, c.f), g2 = wide::geom(2, c.d, c.f);
        const size_t smem = (size_t)wide::RING_BYTES + 1024;
        const uint32_t u1 = max_groups * g1.tiles * tts, u2 = max_groups * g2.tiles * tts;
        const uint32_t grid1 = u1 < (uint32_t)sm_count ? u1 : (uint32_t)sm_count, grid2 = u2 < (uint32_t)sm_count ? u2 : (uint32_t)sm_count;
        ffn_wide_kernel<1><<<grid1, FAST_THREADS, smem, s>>>(P);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        ffn_wide_kernel<2><<<grid2, FAST_THREADS, smem, s>>>(P);
        count_launches(2);
        return cudaGetLastError();
    }
    const PhaseGeom g1 = phase_geom(2, c.d, c.f, c.d / 512, max_bits, RING_BYTES);
    const PhaseGeom g2 = phase_geom(1, c.f, c.d, 4, max_bits, RING_BYTES);
    const size_t smem = (size_t)RING_BYTES + RED_BYTES;
    const uint32_t u1 = max_groups * g1.tiles * tts, u2 = max_groups * g2.tiles * tts;
    const uint32_t grid1 = u1 < (uint32_t)sm_count ? u1 : (uint32_t)sm_count, grid2 = u2 < (uint32_t)sm_count ? u2 : (uint32_t)sm_count;
    switch (c.d / 512) {
        case 1: ffn_phase_kernel<2, 1><<<grid1, FAST_THREADS, smem, s>>>(P); break;
        case 2: ffn_phase_kernel<2, 2><<<grid1, FAST_THREADS, smem, s>>>(P); break;
        case 4: ffn_phase_kernel<2, 4><<<grid1, FAST_THREADS, smem, s>>>(P); break;
        default: return cudaErrorInvalidValue;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    ffn_phase_kernel<1, 4><<<grid2, FAST_THREADS, smem, s>>>(P);
    count_launches(2);
    return cudaGetLastError();
}

cudaError_t launch_stack_mega(cudaStream_t s, const MegaParams& M, const mfb_moe_config& c, int sm_count) {
    cudaError_t e = cudaMemsetAsync(M.bar_counter, 0, MEGA_BAR_WORDS * sizeof(uint32_t), s);   // barrier counter, abort word, group counters
    if (e != cudaSuccess) return e;
    MegaParams copy = M;
    void* args[] = {&copy};
    const void* fn = nullptr;
    // above 16 rows: the all-threads form of the routing-table sort (several rounds of the one-warp scan cost more) and
    // per-phase unit weights; with tensor maps on every layer additionally the row-stationary FFN phases
    const int mode = M.n_tokens > 16 ? (M.wide ? 2 : 1) : 0;
    switch (c.d / 512) {
        case 1: fn = mode ? (const void*)stack_mega_kernel<1, 1> : (const void*)stack_mega_kernel<1, 0>; break;
        case 2: fn = mode == 2 ? (const void*)stack_mega_kernel<2, 2> : mode ? (const void*)stack_mega_kernel<2, 1> : (const void*)stack_mega_kernel<2, 0>; break;
        case 4: fn = mode == 2 ? (const void*)stack_mega_kernel<4, 2> : mode ? (const void*)stack_mega_kernel<4, 1> : (const void*)stack_mega_kernel<4, 0>; break;
        default: return cudaErrorInvalidValue;
    }
    e = cudaLaunchCooperativeKernel(fn, dim3((unsigned)sm_count), dim3(FAST_THREADS), args, fast_smem_stack(c, M.n_tokens, mode == 2), s);
    count_launches(1);
    return e;
}

}  // namespace mfb
