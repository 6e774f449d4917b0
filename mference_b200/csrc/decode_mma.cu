// Decode-time expert FFN, fast path: packed rows staged into shared memory by bulk async copies (TMA unit),
// unpacked in registers straight into tensor-core fragments, fp32 accumulation.
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
// k16 MMAs on exact small integers (codes) times fp16 activations with fp32 accumulation.
//
// The K dimension of an MMA may be permuted freely as long as both operands agree, so packed rows are consumed
// as they lie in memory: lane (g, t) of a warp takes bytes [8t, 8t+8) of each 32-byte group of rows g and g+8
// (4-bit; 4 bytes of each 16-byte group for 2-bit) and the activations are stored once per layer in the
// matching within-16 order (see perm_pos).
#include "common.cuh"
#include "decode_mma.cuh"

namespace mfb {

namespace {

constexpr int CW = 8;                       // compute warps per CTA
constexpr int F1_THREADS = (CW + 1) * 32;   // + one copy-issuing warp
constexpr int F1_STAGES = 2;
constexpr uint32_t ROW_PAD = 32;            // bytes added to each staged row: keeps 8-byte fragment loads conflict free
constexpr uint32_t WAIT_LIMIT = 1u << 24;   // bounded spin on mbarriers

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
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
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
        constexpr uint32_t MAGIC = 0x64006400u, K1024 = 0x64006400u, SIXTEENTH = 0x2C002C00u, M64 = 0xD400D400u;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t lo = w[i], hi = w[i] >> 8;
            p[4 * i + 0] = h2_sub((lo & 0x000F000Fu) | MAGIC, K1024);
            p[4 * i + 1] = h2_fma((lo & 0x00F000F0u) | MAGIC, SIXTEENTH, M64);
            p[4 * i + 2] = h2_sub((hi & 0x000F000Fu) | MAGIC, K1024);
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

// Loads the B fragments (activations of token column g of the tile, this warp's k range) and leaves the
// per-group activation sums of the eight token columns in sx[group][column].
template <int NG>
__device__ __forceinline__ void load_bfrags(const __half* row_ptr /* nullptr: column unused */, uint32_t k0, uint32_t lane,
                                            uint32_t (&bf)[NG][8], float* sx /* [NG][8] */) {
    const uint32_t g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
        uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
        if (row_ptr) {
            const uint4* src = reinterpret_cast<const uint4*>(row_ptr + k0 + gi * 64 + t * 16);
            lo = src[0]; hi = src[1];
        }
        bf[gi][0] = lo.x; bf[gi][1] = lo.y; bf[gi][2] = lo.z; bf[gi][3] = lo.w;
        bf[gi][4] = hi.x; bf[gi][5] = hi.y; bf[gi][6] = hi.z; bf[gi][7] = hi.w;
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&bf[gi][i]));
            s += v.x + v.y;
        }
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
        s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
        if (t == 0) sx[gi * 8 + g] = s;
    }
    __syncwarp();
}

// One 64-element group of rows g and g+8 of one matrix: sum(code * x) by four MMAs, then the affine factors.
template <int BITS>
__device__ __forceinline__ void group_mma(const uint8_t* row_lo, const uint8_t* row_hi, uint32_t byte_off,
                                          const uint32_t (&bf)[8], float s_lo, float b_lo, float s_hi, float b_hi,
                                          float sx0, float sx1, float (&acc)[4]) {
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
    acc[0] = fmaf(s_lo, dsum[0], acc[0]); acc[0] = fmaf(b_lo, sx0, acc[0]);
    acc[1] = fmaf(s_lo, dsum[1], acc[1]); acc[1] = fmaf(b_lo, sx1, acc[1]);
    acc[2] = fmaf(s_hi, dsum[2], acc[2]); acc[2] = fmaf(b_hi, sx0, acc[2]);
    acc[3] = fmaf(s_hi, dsum[3], acc[3]); acc[3] = fmaf(b_hi, sx1, acc[3]);
}

// ------------------------------------------------------------------------------------------ phase 1
// Work item = (group, tile of TILE_ROWS rows of gate and up).  Warp w of the 8 compute warps owns k range
// [ks*512, ks*512+512) (ks = w % KS) of row tile rt = w / KS; partial sums of the KS warps of a row tile meet in
// shared memory.  Warp 8 issues the bulk copies: one per row (padded destination rows), one per scale block.
struct F1Geom {
    uint32_t ks_count, rt_count, tile_rows, tiles_per_group, row_stride_max, stage_bytes, groups_per_row;
};

__host__ __device__ inline F1Geom f1_geom(uint32_t d, uint32_t f, uint32_t max_bits) {
    F1Geom g;
    g.ks_count = d / 512;
    g.rt_count = CW / g.ks_count;
    g.tile_rows = 16 * g.rt_count;
    g.tiles_per_group = f / g.tile_rows;
    g.row_stride_max = d * max_bits / 8 + ROW_PAD;
    g.groups_per_row = d / 64;
    g.stage_bytes = 2 * g.tile_rows * g.row_stride_max + 4 * g.tile_rows * g.groups_per_row * 2;
    return g;
}

template <int BITS>
__device__ __forceinline__ void f1_compute(const FastParams& P, const GroupRef& G, const F1Geom& geo, const uint8_t* stage,
                                           uint32_t tile, uint32_t warp, uint32_t lane, float* sx_w, float* red,
                                           uint32_t& red_buf) {
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t ks = warp % geo.ks_count, rt = warp / geo.ks_count;
    const uint32_t row_bytes = P.d * BITS / 8, row_stride = row_bytes + ROW_PAD;
    const uint32_t gpr = geo.groups_per_row;
    const uint8_t* gate_rows = stage;
    const uint8_t* up_rows = stage + geo.tile_rows * geo.row_stride_max;
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(stage + 2 * geo.tile_rows * geo.row_stride_max);
    const uint16_t* gs = sc, *gb = sc + geo.tile_rows * gpr, *us = gb + geo.tile_rows * gpr, *ub = us + geo.tile_rows * gpr;
    const uint32_t r_lo = rt * 16 + g, r_hi = r_lo + 8;
    const uint32_t lane_bytes = BITS == 4 ? 8 : 4, group_bytes = 64 * BITS / 8;
    const __half* xsrc = (G.shared && P.shared_bits != P.bits) ? P.xp_shared : P.xp;
    const int sdt = (int)P.scale_dtype;

    for (uint32_t tt = 0; tt < G.pair_count; tt += 8) {
        const uint32_t cols = min(8u, G.pair_count - tt);
        const __half* row_ptr = nullptr;
        if (g < cols) row_ptr = xsrc + (size_t)P.sorted[G.pair_start + tt + g].token * P.d;
        uint32_t bf[8][8];
        load_bfrags<8>(row_ptr, ks * 512, lane, bf, sx_w);
        float ag[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int gi = 0; gi < 8; ++gi) {
            const uint32_t grp = ks * 8 + gi;
            const uint32_t boff = grp * group_bytes + t * lane_bytes;
            const float2 sxv = *reinterpret_cast<const float2*>(sx_w + gi * 8 + 2 * t);
            group_mma<BITS>(gate_rows + r_lo * row_stride, gate_rows + r_hi * row_stride, boff, bf[gi],
                            widen16(gs[r_lo * gpr + grp], sdt), widen16(gb[r_lo * gpr + grp], sdt),
                            widen16(gs[r_hi * gpr + grp], sdt), widen16(gb[r_hi * gpr + grp], sdt), sxv.x, sxv.y, ag);
            group_mma<BITS>(up_rows + r_lo * row_stride, up_rows + r_hi * row_stride, boff, bf[gi],
                            widen16(us[r_lo * gpr + grp], sdt), widen16(ub[r_lo * gpr + grp], sdt),
                            widen16(us[r_hi * gpr + grp], sdt), widen16(ub[r_hi * gpr + grp], sdt), sxv.x, sxv.y, au);
        }
        // partial sums of this warp -> shared memory, then a fixed-order sum over the k splits
        float* rb = red + red_buf * (CW * 32 * 8);
        float4* dst = reinterpret_cast<float4*>(rb + ((ks * geo.rt_count + rt) * 32 + lane) * 8);
        dst[0] = make_float4(ag[0], ag[1], ag[2], ag[3]);
        dst[1] = make_float4(au[0], au[1], au[2], au[3]);
        named_barrier(1, CW * 32);
        const uint32_t tid = warp * 32 + lane;
        for (uint32_t o = tid; o < geo.rt_count * 128; o += CW * 32) {
            const uint32_t ort = o >> 7, row = (o & 127) >> 3, n = o & 7;
            const uint32_t src_lane = (row & 7) * 4 + (n >> 1), reg = (row >> 3) * 2 + (n & 1);
            float gsum = 0.0f, usum = 0.0f;
            for (uint32_t k = 0; k < geo.ks_count; ++k) {
                const float* src = rb + ((k * geo.rt_count + ort) * 32 + src_lane) * 8;
                gsum += src[reg];
                usum += src[4 + reg];
            }
            if (n < cols) {
                if (!G.shared && P.limit > 0.0f) {
                    gsum = fminf(gsum, P.limit);
                    usum = fminf(fmaxf(usum, -P.limit), P.limit);
                }
                float a = hidden_act(gsum, (int)P.activation) * usum;
                a = fminf(fmaxf(a, -65504.0f), 65504.0f);
                const uint32_t r = tile * geo.tile_rows + ort * 16 + row;
                const uint32_t pos = (r & ~15u) + perm_pos(r & 15u, G.bits);
                P.actp[(size_t)(G.pair_start + tt + n) * P.f + pos] = __float2half_rn(a);
            }
        }
        red_buf ^= 1u;
    }
}

__global__ void __launch_bounds__(F1_THREADS, 1) ffn1_mma_kernel(const FastParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_bar[F1_STAGES], empty_bar[F1_STAGES];
    __shared__ uint32_t abort_flag;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t max_bits = P.shared_blob && P.shared_bits > P.bits ? P.shared_bits : P.bits;
    const F1Geom geo = f1_geom(P.d, P.f, max_bits);
    uint8_t* stages = smem;
    float* red = reinterpret_cast<float*>(smem + F1_STAGES * geo.stage_bytes);
    float* sx = red + 2 * CW * 32 * 8;
    if (threadIdx.x == 0) {
        for (int s = 0; s < F1_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], CW); }
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    const uint32_t n_groups = *P.n_groups;
    const uint32_t n_items = n_groups * geo.tiles_per_group;
    const uint32_t per_cta = (n_items + gridDim.x - 1) / gridDim.x;
    const uint32_t first = blockIdx.x * per_cta, last = min(first + per_cta, n_items);

    if (warp == CW) {
        // ---- copy-issuing warp
        uint32_t issued = 0;
        for (uint32_t item = first; item < last; ++item, ++issued) {
            const uint32_t s = issued % F1_STAGES, ph = (issued / F1_STAGES) & 1u;
            const GroupRef G = group_ref(P, item / geo.tiles_per_group);
            if (!mbar_wait(&empty_bar[s], ph ^ 1u)) { atomicOr(P.status, STATUS_MBAR_TIMEOUT); abort_flag = 1; break; }
            if (!G.ok) {   // nothing to copy: complete the phase so the consumers move on
                if (lane == 0) mbar_arrive(&full_bar[s]);
                continue;
            }
            const uint32_t tile = item % geo.tiles_per_group, row0 = tile * geo.tile_rows;
            const uint32_t row_bytes = P.d * G.bits / 8, row_stride = row_bytes + ROW_PAD, gpr = geo.groups_per_row;
            uint8_t* st = stages + s * geo.stage_bytes;
            const uint32_t scale_block = geo.tile_rows * gpr * 2;
            if (lane == 0) mbar_expect_tx(&full_bar[s], 2 * geo.tile_rows * row_bytes + 4 * scale_block);
            __syncwarp();
            for (uint32_t r = lane; r < 2 * geo.tile_rows; r += 32) {
                const bool up = r >= geo.tile_rows;
                const uint32_t rr = up ? r - geo.tile_rows : r;
                const uint8_t* src = G.blob + (up ? G.off.up_w : G.off.gate_w) + (size_t)(row0 + rr) * row_bytes;
                bulk_g2s(st + (up ? geo.tile_rows * geo.row_stride_max : 0) + rr * row_stride, src, row_bytes, &full_bar[s]);
            }
            if (lane < 4) {
                const uint32_t o = lane == 0 ? G.off.gate_s : (lane == 1 ? G.off.gate_b : (lane == 2 ? G.off.up_s : G.off.up_b));
                bulk_g2s(st + 2 * geo.tile_rows * geo.row_stride_max + lane * scale_block,
                         G.blob + o + (size_t)row0 * gpr * 2, scale_block, &full_bar[s]);
            }
        }
        return;
    }

    // ---- compute warps
    float* sx_w = sx + warp * 64;
    uint32_t red_buf = 0, done = 0;
    for (uint32_t item = first; item < last; ++item, ++done) {
        const uint32_t s = done % F1_STAGES, ph = (done / F1_STAGES) & 1u;
        const GroupRef G = group_ref(P, item / geo.tiles_per_group);
        if (!mbar_wait(&full_bar[s], ph)) { atomicOr(P.status, STATUS_MBAR_TIMEOUT); break; }
        if (G.ok) {
            const uint8_t* st = stages + s * geo.stage_bytes;
            if (G.bits == 4) f1_compute<4>(P, G, geo, st, item % geo.tiles_per_group, warp, lane, sx_w, red, red_buf);
            else f1_compute<2>(P, G, geo, st, item % geo.tiles_per_group, warp, lane, sx_w, red, red_buf);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
}

// ------------------------------------------------------------------------------------------ phase 2 + combine
// One CTA per block of 16 output rows (columns of the hidden state).  Warp w walks groups w, w+8, ...: the group's
// 16 down-projection rows are copied into a warp-private ring of stages, multiplied against the group's hidden
// activations, and the 16 x (tokens) results land in a CTA-wide array indexed by (token, rank slot).  When every
// group is done the CTA applies the routing weights in rank order, residual first, and writes its 16 columns of
// every token row:  moe_phase2_down_reduce_k8 (moe.metal:349-404) without a partials buffer in global memory.
constexpr int F2_STAGES = 3;
constexpr int F2_THREADS = CW * 32;

template <int BITS, int NG>
__device__ __forceinline__ void f2_compute(const FastParams& P, const GroupRef& G, const uint8_t* st, uint32_t row_stride_max,
                                           uint32_t lane, float* sx_w, float* part, uint32_t slots) {
    const uint32_t g = lane >> 2, t = lane & 3;
    const uint32_t row_stride = P.f * BITS / 8 + ROW_PAD, gpr = P.f / 64;
    const uint16_t* sc = reinterpret_cast<const uint16_t*>(st + 16 * row_stride_max);
    const uint16_t* ds = sc, *db = sc + 16 * gpr;
    const uint32_t lane_bytes = BITS == 4 ? 8 : 4, group_bytes = 64 * BITS / 8;
    const int sdt = (int)P.scale_dtype;
    for (uint32_t tt = 0; tt < G.pair_count; tt += 8) {
        const uint32_t cols = min(8u, G.pair_count - tt);
        const __half* row_ptr = g < cols ? P.actp + (size_t)(G.pair_start + tt + g) * P.f : nullptr;
        uint32_t bf[NG][8];
        load_bfrags<NG>(row_ptr, 0, lane, bf, sx_w);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
            const float2 sxv = *reinterpret_cast<const float2*>(sx_w + gi * 8 + 2 * t);
            group_mma<BITS>(st + g * row_stride, st + (g + 8) * row_stride, gi * group_bytes + t * lane_bytes, bf[gi],
                            widen16(ds[g * gpr + gi], sdt), widen16(db[g * gpr + gi], sdt),
                            widen16(ds[(g + 8) * gpr + gi], sdt), widen16(db[(g + 8) * gpr + gi], sdt), sxv.x, sxv.y, acc);
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const uint32_t n = 2 * t + c;
            if (n < cols) {
                const mfb_pair pr = P.sorted[G.pair_start + tt + n];
                float* dst = part + ((size_t)pr.token * slots + pr.rank) * 16;
                dst[g] = acc[c];
                dst[g + 8] = acc[2 + c];
            }
        }
        __syncwarp();
    }
}

template <int NG>
__global__ void __launch_bounds__(F2_THREADS, 1) ffn2_mma_kernel(const FastParams P) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_bar[CW][F2_STAGES];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t max_bits = P.shared_blob && P.shared_bits > P.bits ? P.shared_bits : P.bits;
    const uint32_t row_stride_max = P.f * max_bits / 8 + ROW_PAD, gpr = P.f / 64;
    const uint32_t stage_bytes = 16 * row_stride_max + 2 * 16 * gpr * 2;
    const uint32_t slots = P.top_k + 1;
    uint8_t* my_stages = smem + warp * F2_STAGES * stage_bytes;
    float* part = reinterpret_cast<float*>(smem + CW * F2_STAGES * stage_bytes);
    float* sx = part + (size_t)P.n_tokens * slots * 16;
    float* sx_w = sx + warp * (NG * 8);
    const uint32_t row0 = blockIdx.x * 16;

    if (lane == 0) {
        for (int s = 0; s < F2_STAGES; ++s) mbar_init(&full_bar[warp][s], 1);
        fence_barrier_init();
    }
    for (uint32_t i = threadIdx.x; i < P.n_tokens * slots * 16; i += F2_THREADS) part[i] = 0.0f;
    __syncthreads();

    const uint32_t n_groups = *P.n_groups;
    auto issue = [&](uint32_t gidx, uint32_t s) {
        const GroupRef G = group_ref(P, gidx);
        if (!G.ok) { if (lane == 0) mbar_arrive(&full_bar[warp][s]); return; }
        const uint32_t row_bytes = P.f * G.bits / 8, row_stride = row_bytes + ROW_PAD, scale_block = 16 * gpr * 2;
        uint8_t* st = my_stages + s * stage_bytes;
        fence_proxy_async();
        if (lane == 0) mbar_expect_tx(&full_bar[warp][s], 16 * row_bytes + 2 * scale_block);
        __syncwarp();
        if (lane < 16) bulk_g2s(st + lane * row_stride, G.blob + G.off.down_w + (size_t)(row0 + lane) * row_bytes, row_bytes, &full_bar[warp][s]);
        else if (lane < 18) bulk_g2s(st + 16 * row_stride_max + (lane - 16) * scale_block,
                                     G.blob + (lane == 16 ? G.off.down_s : G.off.down_b) + (size_t)row0 * gpr * 2, scale_block, &full_bar[warp][s]);
    };
    uint32_t n_mine = 0;
    for (uint32_t gidx = warp; gidx < n_groups; gidx += CW) ++n_mine;
    for (uint32_t i = 0; i < n_mine && i < (uint32_t)F2_STAGES; ++i) issue(warp + i * CW, i);
    for (uint32_t i = 0; i < n_mine; ++i) {
        const uint32_t s = i % F2_STAGES, ph = (i / F2_STAGES) & 1u;
        const uint32_t gidx = warp + i * CW;
        const GroupRef G = group_ref(P, gidx);
        if (!mbar_wait(&full_bar[warp][s], ph)) { atomicOr(P.status, STATUS_MBAR_TIMEOUT); break; }
        if (G.ok) {
            const uint8_t* st = my_stages + s * stage_bytes;
            if (G.bits == 4) f2_compute<4, NG>(P, G, st, row_stride_max, lane, sx_w, part, slots);
            else f2_compute<2, NG>(P, G, st, row_stride_max, lane, sx_w, part, slots);
        }
        __syncwarp();
        if (i + F2_STAGES < n_mine) issue(warp + (i + F2_STAGES) * CW, s);
    }
    __syncthreads();
    // rank-ordered weighted combine of this CTA's 16 columns
    const bool with_shared = P.shared_blob != nullptr;
    for (uint32_t o = threadIdx.x; o < P.n_tokens * 16; o += F2_THREADS) {
        const uint32_t tok = o >> 4, r = o & 15;
        const float* pt = part + (size_t)tok * slots * 16;
        float acc = P.residual ? load_act(P.residual, (size_t)tok * P.d + row0 + r, P.x_dtype) : 0.0f;
        if (with_shared) acc += pt[P.top_k * 16 + r];
        for (uint32_t k = 0; k < P.top_k; ++k)
            acc = fmaf(__half2float(__ushort_as_half(P.route_w[(size_t)tok * P.top_k + k])), pt[k * 16 + r], acc);
        store_act(P.y, (size_t)tok * P.d + row0 + r, acc, P.x_dtype);
    }
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

}  // namespace

// ------------------------------------------------------------------------------------------ host side
bool fast_supported(const mfb_moe_config& c) {
    const uint32_t ks = c.d / 512;
    if (c.d % 512 || !(ks == 1 || ks == 2 || ks == 4 || ks == 8)) return false;
    if (c.f % 64 || c.f > 512) return false;            // phase 2 keeps a whole row's activations in registers
    const uint32_t tile_rows = 16 * (CW / ks);
    if (c.f % tile_rows || c.d % 16) return false;
    if (c.top_k + 1 > 32) return false;
    return true;
}

size_t fast_smem1(const mfb_moe_config& c) {
    const uint32_t max_bits = c.shared_bits > c.bits ? c.shared_bits : c.bits;
    const F1Geom g = f1_geom(c.d, c.f, max_bits);
    return (size_t)F1_STAGES * g.stage_bytes + 2 * CW * 32 * 8 * sizeof(float) + CW * 64 * sizeof(float);
}

size_t fast_smem2(const mfb_moe_config& c, uint32_t n_tokens) {
    const uint32_t max_bits = c.shared_bits > c.bits ? c.shared_bits : c.bits;
    const uint32_t row_stride_max = c.f * max_bits / 8 + ROW_PAD, gpr = c.f / 64;
    const size_t stage_bytes = 16 * row_stride_max + 2 * 16 * gpr * 2;
    return (size_t)CW * F2_STAGES * stage_bytes + (size_t)n_tokens * (c.top_k + 1) * 16 * sizeof(float) + CW * (c.f / 64) * 8 * sizeof(float);
}

template <int NG>
static cudaError_t launch_f2(cudaStream_t s, const FastParams& P, size_t smem) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(ffn2_mma_kernel<NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    ffn2_mma_kernel<NG><<<P.d / 16, F2_THREADS, smem, s>>>(P);
    return cudaGetLastError();
}

cudaError_t launch_fast_prep(cudaStream_t s, const void* h, int dtype, const __nv_bfloat16* w, uint32_t n_tokens, uint32_t d,
                             float eps, bool do_norm, void* xn, __half* xp, uint32_t bits, __half* xp2, uint32_t bits2) {
    if (n_tokens == 0) return cudaSuccess;
    prep_kernel<<<n_tokens, 256, 0, s>>>(h, dtype, w, d, eps, do_norm ? 1 : 0, xn, xp, bits, xp2, bits2);
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_fast_ffn(cudaStream_t s, const FastParams& P, const mfb_moe_config& c, int sm_count, uint32_t max_groups) {
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(ffn1_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    const uint32_t max_bits = c.shared_bits > c.bits ? c.shared_bits : c.bits;
    const F1Geom g = f1_geom(c.d, c.f, max_bits);
    const uint32_t max_items = max_groups * g.tiles_per_group;
    const uint32_t grid = max_items < (uint32_t)sm_count ? max_items : (uint32_t)sm_count;
    ffn1_mma_kernel<<<grid, F1_THREADS, fast_smem1(c), s>>>(P);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const size_t smem2 = fast_smem2(c, P.n_tokens);
    switch (c.f / 64) {
        case 1: e = launch_f2<1>(s, P, smem2); break;
        case 2: e = launch_f2<2>(s, P, smem2); break;
        case 4: e = launch_f2<4>(s, P, smem2); break;
        case 8: e = launch_f2<8>(s, P, smem2); break;
        default: return cudaErrorInvalidValue;
    }
    count_launches(2);
    return e;
}

}  // namespace mfb
