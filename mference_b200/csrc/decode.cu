// Decode-time quantised expert FFN: expert-major GEMV over affine group-quantised rows.
//
// Work is organised by distinct expert, not by token: the routing table of the batch is sorted by expert
// (group.cu) and every (expert, row block) is visited once, its packed rows applied to all token rows routed
// to that expert, so each expert's bytes leave HBM once per layer whatever the batch size.  The shared expert
// is one more group that owns every token.
//
//   phase 1  acts[p, r]     = act(gate_e[r,:] . x_t) * (up_e[r,:] . x_t)        p = sorted pair (t, e)
//   phase 2  partial[t,s,c] = down_e[c,:] . acts[p,:]                           s = rank slot (top_k = shared)
//
// Arithmetic follows moe_int4_gate_up_rows_simd_dev_vec_u16load / moe_int4_gemv_row_simd_dev_vec and their
// 2-bit siblings (Sources/Mference/Metal/MoE/moe.metal:349-529, 902-1062): per 64-element group the dot
// product is factored as scale * sum(code * x) + bias * sum(x), accumulated in fp32; a row is spread over the
// lanes of a warp in 16-byte pieces (128-bit coalesced loads of the packed codes) and reduced with shuffles.
// Activations are staged in shared memory once per block together with their per-32-element sums.
#include "common.cuh"

namespace mfb {

namespace {

constexpr int FFN_WARPS = 4;
constexpr int FFN_THREADS = FFN_WARPS * 32;
constexpr int FFN_SETS_PER_WARP = 2;

struct FfnParams {
    const uint8_t* pool;
    uint64_t slot_stride;
    const int16_t* slot_of;
    const uint8_t* shared_blob;
    mfb_expert_offsets routed_off, shared_off;
    uint32_t d, f, num_experts, top_k, bits, shared_bits, scale_dtype, activation;
    float limit;
    const void* x;
    int x_dtype;
    uint32_t ldx;
    const mfb_pair* sorted;
    const mfb_group* groups;
    const uint32_t* n_groups;
    float* acts;
    float* partial;
    uint32_t slots;
    uint32_t gate32;   // routed experts' gate_proj carries one scale and bias per 32 elements (DeepSeek V4)
    uint32_t round16;  // gate, up and their activation product rounded to fp16 (the Inkling batched expert kernels)
};

// Shared-memory layout of one staged activation row: every 32 elements are followed by 4 pad floats, the
// first of which holds the sum of those 32 elements.  The pad also staggers the banks so that lanes reading
// consecutive 32-element pieces with 16-byte loads do not collide.
__host__ __device__ __forceinline__ uint32_t padded(uint32_t e) { return e + (e >> 5) * 4u; }

__device__ __forceinline__ uint4 ldg_stream(const uint8_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// exact small-integer to float without a convert instruction
__device__ __forceinline__ float code_f32(uint32_t c) { return __uint_as_float(0x4B000000u | c) - 8388608.0f; }

// Stage NT rows of `cols` values (from `src`, row r at src_row[r]) into shared memory with chunk sums.
template <int NT>
__device__ __forceinline__ void stage_rows(const void* src, int dtype, const size_t (&row_elem0)[NT], uint32_t n_valid,
                                           uint32_t cols, float* xs, uint32_t xstride) {
    const uint32_t tid = threadIdx.x;
    for (uint32_t t = 0; t < (uint32_t)NT; ++t) {
        // uniform trip count: every lane takes part in the shuffles below (cols is a multiple of 32, so the
        // eight lanes that share a 32-element piece are in range together)
        for (uint32_t base = 0; base < cols; base += FFN_THREADS * 4) {
            const uint32_t e0 = base + tid * 4;
            const bool in_range = e0 < cols;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (t < n_valid && in_range) {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = load_act(src, row_elem0[t] + e0 + j, dtype);
            }
            if (in_range) {
                float* dst = xs + t * xstride + padded(e0);
                dst[0] = v[0]; dst[1] = v[1]; dst[2] = v[2]; dst[3] = v[3];
            }
            float s = (v[0] + v[1]) + (v[2] + v[3]);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 1);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 2);
            s += __shfl_xor_sync(0xFFFFFFFFu, s, 4);
            if (in_range && (tid & 7) == 0) xs[t * xstride + padded(e0 & ~31u) + 32] = s;
        }
    }
}

// Dot products of one row (of NMAT matrices sharing the activations) against NT staged activation rows.
// Lane `sl` of a sub-warp of width `sw` owns 16-byte pieces sl, sl+sw, ... of the row.
template <int BITS, int NT, int NMAT>
__device__ __forceinline__ void row_dot(const uint8_t* const (&wrow)[NMAT], const uint16_t* const (&srow)[NMAT],
                                        const uint16_t* const (&brow)[NMAT], int scale_dtype, bool row_ok,
                                        uint32_t pieces, uint32_t sw, uint32_t sl, const float* xs, uint32_t xstride,
                                        float (&acc)[NMAT][NT], bool gate32 = false) {
    constexpr uint32_t CPP = 128 / BITS;   // codes per 16-byte piece
    constexpr uint32_t CPW = 32 / BITS;    // codes per 32-bit word
    constexpr uint32_t MASK = (1u << BITS) - 1u;
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[m][t] = 0.0f;
    if (row_ok) {
        for (uint32_t pc = sl; pc < pieces; pc += sw) {
            const uint32_t elem0 = pc * CPP;
            uint4 q[NMAT];
            float sc[NMAT], bi[NMAT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
                q[m] = ldg_stream(wrow[m] + (size_t)pc * 16);
                const uint32_t gidx = (gate32 && m == 0) ? elem0 >> 5 : elem0 >> 6;   // matrix 0 is gate where gate32 applies
                sc[m] = widen16(srow[m][gidx], scale_dtype);
                bi[m] = widen16(brow[m][gidx], scale_dtype);
            }
            // 2-bit pieces hold 64 codes: with 32-element gate groups the piece's second half has a scale of its own
            const bool split = gate32 && CPP == 64;
            float sc_hi = 0.0f, bi_hi = 0.0f, dot_hi[NT];
            if (split) {
                sc_hi = widen16(srow[0][(elem0 >> 5) + 1], scale_dtype);
                bi_hi = widen16(brow[0][(elem0 >> 5) + 1], scale_dtype);
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) dot_hi[t] = 0.0f;
            float dot[NMAT][NT];
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
                for (int t = 0; t < NT; ++t) dot[m][t] = 0.0f;
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                const uint32_t eo = padded(elem0 + wi * CPW);
#pragma unroll
                for (uint32_t j0 = 0; j0 < CPW; j0 += 4) {
                    float4 xv[NT];
#pragma unroll
                    for (int t = 0; t < NT; ++t) xv[t] = *reinterpret_cast<const float4*>(xs + t * xstride + eo + j0);
#pragma unroll
                    for (int m = 0; m < NMAT; ++m) {
                        const uint32_t word = wi == 0 ? q[m].x : (wi == 1 ? q[m].y : (wi == 2 ? q[m].z : q[m].w));
                        const float c0 = code_f32((word >> ((j0 + 0) * BITS)) & MASK);
                        const float c1 = code_f32((word >> ((j0 + 1) * BITS)) & MASK);
                        const float c2 = code_f32((word >> ((j0 + 2) * BITS)) & MASK);
                        const float c3 = code_f32((word >> ((j0 + 3) * BITS)) & MASK);
                        if (split && m == 0 && wi >= 2) {
#pragma unroll
                            for (int t = 0; t < NT; ++t) {
                                dot_hi[t] = fmaf(c0, xv[t].x, dot_hi[t]);
                                dot_hi[t] = fmaf(c1, xv[t].y, dot_hi[t]);
                                dot_hi[t] = fmaf(c2, xv[t].z, dot_hi[t]);
                                dot_hi[t] = fmaf(c3, xv[t].w, dot_hi[t]);
                            }
                        } else {
#pragma unroll
                            for (int t = 0; t < NT; ++t) {
                                dot[m][t] = fmaf(c0, xv[t].x, dot[m][t]);
                                dot[m][t] = fmaf(c1, xv[t].y, dot[m][t]);
                                dot[m][t] = fmaf(c2, xv[t].z, dot[m][t]);
                                dot[m][t] = fmaf(c3, xv[t].w, dot[m][t]);
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < NT; ++t) {
                const float xsum_lo = xs[t * xstride + padded(elem0 & ~31u) + 32];
                const float xsum_hi = CPP == 64 ? xs[t * xstride + padded((elem0 & ~31u) + 32) + 32] : 0.0f;
                float xsum = xsum_lo + xsum_hi;
                if (CPP == 16 && (pc & 1u)) xsum = 0.0f;   // 8-bit codes: the 32-element sum goes with the block's first piece
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                    if (split && m == 0) {
                        acc[m][t] = fmaf(sc[m], dot[m][t], acc[m][t]);
                        acc[m][t] = fmaf(bi[m], xsum_lo, acc[m][t]);
                        acc[m][t] = fmaf(sc_hi, dot_hi[t], acc[m][t]);
                        acc[m][t] = fmaf(bi_hi, xsum_hi, acc[m][t]);
                    } else {
                        acc[m][t] = fmaf(sc[m], dot[m][t], acc[m][t]);
                        acc[m][t] = fmaf(bi[m], xsum, acc[m][t]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
        for (int t = 0; t < NT; ++t)
            for (uint32_t off = sw >> 1; off > 0; off >>= 1) acc[m][t] += __shfl_xor_sync(0xFFFFFFFFu, acc[m][t], off);
}

struct GroupView {
    const uint8_t* blob;
    mfb_expert_offsets off;
    uint32_t bits;
    uint32_t pair_start, pair_count;
    bool shared, ok;
};

__device__ __forceinline__ GroupView view_group(const FfnParams& P, uint32_t g) {
    GroupView v;
    v.ok = g < *P.n_groups;
    if (!v.ok) return v;
    const mfb_group grp = P.groups[g];
    v.shared = grp.expert >= P.num_experts;
    v.pair_start = grp.pair_start;
    v.pair_count = grp.pair_count;
    if (v.shared) {
        v.blob = P.shared_blob; v.off = P.shared_off; v.bits = P.shared_bits;
        v.ok = P.shared_blob != nullptr;
    } else {
        int64_t slot = grp.expert;
        if (P.slot_of) slot = P.slot_of[grp.expert];
        v.ok = slot >= 0;   // an expert that is not resident is a visible no-op, never an out-of-bounds read
        v.blob = P.pool + (uint64_t)(slot < 0 ? 0 : slot) * P.slot_stride;
        v.off = P.routed_off; v.bits = P.bits;
    }
    return v;
}

template <int BITS, int NT>
__device__ void phase1_body(const FfnParams& P, const GroupView& G, float* xs) {
    const uint32_t d = P.d, f = P.f;
    const uint32_t pieces = d * BITS / 128, sw = pieces >= 32 ? 32u : pieces;
    const uint32_t rows_per_set = 32 / sw, rows_per_block = FFN_WARPS * FFN_SETS_PER_WARP * rows_per_set;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sl = lane % sw, sub = lane / sw;
    const uint32_t row_bytes = d * BITS / 8, groups_per_row = d / 64, xstride = padded(d);
    const bool gate32 = P.gate32 && !G.shared;                       // 32-element groups: routed experts' gate_proj only
    const uint32_t gate_groups_per_row = gate32 ? d / 32 : d / 64;
    const uint32_t r_begin = blockIdx.x * rows_per_block;
    for (uint32_t t0 = 0; t0 < G.pair_count; t0 += NT) {
        const uint32_t nv = min((uint32_t)NT, G.pair_count - t0);
        size_t row0[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t)
            row0[t] = (uint32_t)t < nv ? (size_t)P.sorted[G.pair_start + t0 + t].token * P.ldx : 0;
        __syncthreads();
        stage_rows<NT>(P.x, P.x_dtype, row0, nv, d, xs, xstride);
        __syncthreads();
#pragma unroll
        for (int set = 0; set < FFN_SETS_PER_WARP; ++set) {
            const uint32_t r = r_begin + (warp * FFN_SETS_PER_WARP + set) * rows_per_set + sub;
            const bool ok = r < f;
            const uint8_t* const wr[2] = {G.blob + G.off.gate_w + (size_t)r * row_bytes, G.blob + G.off.up_w + (size_t)r * row_bytes};
            const uint16_t* const sr[2] = {(const uint16_t*)(G.blob + G.off.gate_s) + (size_t)r * gate_groups_per_row,
                                           (const uint16_t*)(G.blob + G.off.up_s) + (size_t)r * groups_per_row};
            const uint16_t* const br[2] = {(const uint16_t*)(G.blob + G.off.gate_b) + (size_t)r * gate_groups_per_row,
                                           (const uint16_t*)(G.blob + G.off.up_b) + (size_t)r * groups_per_row};
            float acc[2][NT];
            row_dot<BITS, NT, 2>(wr, sr, br, (int)P.scale_dtype, ok, pieces, sw, sl, xs, xstride, acc, gate32);
            if (ok && sl == 0) {
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    if ((uint32_t)t < nv) {
                        float g = acc[0][t], u = acc[1][t];
                        if (!G.shared && P.limit > 0.0f) {   // moe_swiglu_clamp, moe.metal:27-34 (routed experts only)
                            g = fminf(g, P.limit);
                            u = fminf(fmaxf(u, -P.limit), P.limit);
                        }
                        if (P.round16) {   // prefill.metal:714-721: the two GEMV results pass through fp16 before they are combined
                            g = __half2float(__float2half_rn(g));
                            u = __half2float(__float2half_rn(u));
                        }
                        float a = hidden_act(g, (int)P.activation) * u;
                        if (P.round16) a = __half2float(__float2half_rn(a));
                        P.acts[(size_t)(G.pair_start + t0 + t) * f + r] = a;
                    }
                }
            }
        }
    }
}

template <int BITS, int NT>
__device__ void phase2_body(const FfnParams& P, const GroupView& G, float* xs) {
    const uint32_t d = P.d, f = P.f;
    const uint32_t pieces = f * BITS / 128, sw = pieces >= 32 ? 32u : pieces;
    const uint32_t rows_per_set = 32 / sw, rows_per_block = FFN_WARPS * FFN_SETS_PER_WARP * rows_per_set;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sl = lane % sw, sub = lane / sw;
    const uint32_t row_bytes = f * BITS / 8, groups_per_row = f / 64, xstride = padded(f);
    const uint32_t r_begin = blockIdx.x * rows_per_block;
    for (uint32_t t0 = 0; t0 < G.pair_count; t0 += NT) {
        const uint32_t nv = min((uint32_t)NT, G.pair_count - t0);
        size_t row0[NT];
        size_t out_row[NT];
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            row0[t] = (size_t)(G.pair_start + t0 + t) * f;
            out_row[t] = 0;
            if ((uint32_t)t < nv) {
                const mfb_pair pr = P.sorted[G.pair_start + t0 + t];
                out_row[t] = ((size_t)pr.token * P.slots + pr.rank) * d;
            }
        }
        __syncthreads();
        stage_rows<NT>(P.acts, MFB_DT_F32, row0, nv, f, xs, xstride);
        __syncthreads();
#pragma unroll
        for (int set = 0; set < FFN_SETS_PER_WARP; ++set) {
            const uint32_t r = r_begin + (warp * FFN_SETS_PER_WARP + set) * rows_per_set + sub;
            const bool ok = r < d;
            const uint8_t* const wr[1] = {G.blob + G.off.down_w + (size_t)r * row_bytes};
            const uint16_t* const sr[1] = {(const uint16_t*)(G.blob + G.off.down_s) + (size_t)r * groups_per_row};
            const uint16_t* const br[1] = {(const uint16_t*)(G.blob + G.off.down_b) + (size_t)r * groups_per_row};
            float acc[1][NT];
            row_dot<BITS, NT, 1>(wr, sr, br, (int)P.scale_dtype, ok, pieces, sw, sl, xs, xstride, acc);
            if (ok && sl == 0) {
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    if ((uint32_t)t < nv) P.partial[out_row[t] + r] = acc[0][t];
            }
        }
    }
}

template <int NT>
__global__ void __launch_bounds__(FFN_THREADS) ffn_phase1_kernel(const FfnParams P) {
    extern __shared__ __align__(16) float xs[];
    const GroupView G = view_group(P, blockIdx.y);
    if (!G.ok) return;
    if (G.bits == 4) phase1_body<4, NT>(P, G, xs);
    else if (G.bits == 8) phase1_body<8, NT>(P, G, xs);
    else phase1_body<2, NT>(P, G, xs);
}

template <int NT>
__global__ void __launch_bounds__(FFN_THREADS) ffn_phase2_kernel(const FfnParams P) {
    extern __shared__ __align__(16) float xs[];
    const GroupView G = view_group(P, blockIdx.y);
    if (!G.ok) return;
    if (G.bits == 4) phase2_body<4, NT>(P, G, xs);
    else if (G.bits == 8) phase2_body<8, NT>(P, G, xs);
    else phase2_body<2, NT>(P, G, xs);
}

uint32_t rows_per_block(uint32_t cols, uint32_t bits) {
    const uint32_t pieces = cols * bits / 128, sw = pieces >= 32 ? 32u : pieces;
    return FFN_WARPS * FFN_SETS_PER_WARP * (32 / sw);
}

template <int NT>
cudaError_t launch_nt(cudaStream_t s, const FfnParams& P, uint32_t max_groups) {
    const uint32_t min_bits = P.shared_blob ? (P.bits < P.shared_bits ? P.bits : P.shared_bits) : P.bits;
    const uint32_t max_bits = P.shared_blob ? (P.bits > P.shared_bits ? P.bits : P.shared_bits) : P.bits;
    // the narrower code width has the wider sub-warp, hence the fewer rows per block: size the grid for it
    const uint32_t rpb1 = rows_per_block(P.d, max_bits), rpb2 = rows_per_block(P.f, max_bits);
    (void)min_bits;
    const size_t smem1 = (size_t)NT * padded(P.d) * sizeof(float), smem2 = (size_t)NT * padded(P.f) * sizeof(float);
    cudaError_t e;
    e = cudaFuncSetAttribute(ffn_phase1_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(ffn_phase2_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    if (e != cudaSuccess) return e;
    dim3 g1((P.f + rpb1 - 1) / rpb1, max_groups), g2((P.d + rpb2 - 1) / rpb2, max_groups);
    ffn_phase1_kernel<NT><<<g1, FFN_THREADS, smem1, s>>>(P);
    ffn_phase2_kernel<NT><<<g2, FFN_THREADS, smem2, s>>>(P);
    count_launches(2);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_decode_ffn(cudaStream_t s, const DecodeArgs& a) {
    FfnParams P;
    P.pool = a.w->pool; P.slot_stride = a.w->slot_stride; P.slot_of = a.w->slot_of; P.shared_blob = a.w->shared_blob;
    P.routed_off = a.w->routed_off; P.shared_off = a.w->shared_off;
    P.d = a.d; P.f = a.f; P.num_experts = a.num_experts; P.top_k = a.top_k; P.bits = a.bits;
    P.shared_bits = a.shared_bits; P.scale_dtype = a.scale_dtype; P.activation = a.activation; P.limit = a.swiglu_limit;
    P.x = a.x; P.x_dtype = a.x_dtype; P.ldx = a.ldx; P.sorted = a.sorted; P.groups = a.groups; P.n_groups = a.n_groups;
    P.acts = a.acts; P.partial = a.partial; P.slots = a.slots;
    P.gate32 = a.w->gate_group_size == 32 ? 1u : 0u;
    P.round16 = a.round16;
    if (a.max_groups == 0) return cudaSuccess;
    // rows of one expert are applied to NT token rows per pass over its codes
    if (a.max_groups <= a.top_k + 1) return launch_nt<1>(s, P, a.max_groups);   // single token
    return launch_nt<4>(s, P, a.max_groups);
}

}  // namespace mfb
