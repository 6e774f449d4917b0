// Router: gate GEMV over a bf16 gate, top-k selection with routing weights, slot lookup.
//
// The logits feed an exact comparison (top-k with ties to the lower index), so their summation order is
// part of the contract: for every (token, expert) lane l of a 32-lane group accumulates elements
// l, l+32, l+64, ... with fused multiply-adds in ascending order, then the 32 partial sums are combined by a
// xor butterfly (16, 8, 4, 2, 1), and an optional per-expert bias is added last.  That is the structure of
// router_gemv_bf16_r4 (Sources/Mference/Metal/MoE/moe.metal:162-185) with its lane sum made concrete, and it
// makes a block of B token rows bit-identical to B single-row calls.
#include <algorithm>

#include "common.cuh"
#include "decode_mma.cuh"
#include "select.cuh"

namespace mfb {

namespace {

constexpr int RT_WARPS = 8;     // warps per block
constexpr int RT_KC = 256;      // k elements staged per step (8 per lane)

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xFFFF0000u); }

// Block tile: TM token rows x (RT_WARPS * TE) experts.  Each warp owns TE experts for all TM rows; lane l
// owns k = l (mod 32).  The staged tiles are stored "lane-major" in shared memory — the RT_KC/32 = 8 values a
// lane needs from a row are contiguous — so one 16-byte (bf16) or two 16-byte (fp32) loads fetch them.
template <int TM, int TE>
__global__ void __launch_bounds__(RT_WARPS * 32)
router_logits_kernel(const void* __restrict__ x, int x_dtype, uint32_t ldx, uint32_t n_tokens,
                     const __nv_bfloat16* __restrict__ w, uint32_t num_experts, uint32_t d,
                     const float* __restrict__ logit_bias, float* __restrict__ logits) {
    constexpr int BE = RT_WARPS * TE;
    __shared__ __align__(16) float xs[TM][RT_KC];          // [row][lane*8 + j]  <- element k = j*32 + lane
    __shared__ __align__(16) uint16_t ws[BE][RT_KC];       // same permutation, raw bf16 bits
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t t0 = blockIdx.y * TM, e0 = blockIdx.x * BE;
    float acc[TM][TE];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TE; ++j) acc[i][j] = 0.0f;

    // 16-byte loads of eight consecutive k when rows are 16-bit and aligned; element by element otherwise
    const bool vec = x_dtype != MFB_DT_F32 && (ldx & 7u) == 0 && (d & 7u) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15u) == 0;
    for (uint32_t k0 = 0; k0 < d; k0 += RT_KC) {
        __syncthreads();
        if (vec) {
            // A thread takes columns c*8 .. c*8+7 of all eight 32-column blocks of one row: eight 16-byte loads form
            // an 8 x 8 block whose transpose is, per column, the eight values one lane slot holds - contiguous in
            // the lane-major tile, so they leave as whole 16-byte stores.
            for (uint32_t i = tid; i < (TM + BE) * 4; i += RT_WARPS * 32) {
                const bool is_x = i < TM * 4;
                const uint32_t r = (is_x ? i : i - TM * 4) >> 2, c = i & 3u;
                const bool live = is_x ? (t0 + r < n_tokens) : (e0 + r < num_experts);
                const uint16_t* src = is_x ? reinterpret_cast<const uint16_t*>(x) + (size_t)(t0 + r) * ldx
                                           : reinterpret_cast<const uint16_t*>(w) + (size_t)(e0 + r) * d;
                uint32_t blk[8][4];
#pragma unroll
                for (int jb = 0; jb < 8; ++jb) {
                    const uint32_t k = k0 + jb * 32 + c * 8;
                    uint4 q = make_uint4(0, 0, 0, 0);
                    if (live && k < d) q = *reinterpret_cast<const uint4*>(src + k);
                    blk[jb][0] = q.x; blk[jb][1] = q.y; blk[jb][2] = q.z; blk[jb][3] = q.w;
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {   // column c*8 + j = lane slot, values of the eight blocks in k order
                    uint16_t h[8];
#pragma unroll
                    for (int jb = 0; jb < 8; ++jb)
                        h[jb] = (uint16_t)((j & 1) ? (blk[jb][j >> 1] >> 16) : (blk[jb][j >> 1] & 0xFFFFu));
                    const uint32_t slot = (c * 8 + j) * 8;
                    if (is_x) {
                        *reinterpret_cast<float4*>(&xs[r][slot]) = make_float4(widen16(h[0], x_dtype), widen16(h[1], x_dtype),
                                                                                widen16(h[2], x_dtype), widen16(h[3], x_dtype));
                        *reinterpret_cast<float4*>(&xs[r][slot + 4]) = make_float4(widen16(h[4], x_dtype), widen16(h[5], x_dtype),
                                                                                    widen16(h[6], x_dtype), widen16(h[7], x_dtype));
                    } else {
                        *reinterpret_cast<uint4*>(&ws[r][slot]) = make_uint4(h[0] | ((uint32_t)h[1] << 16), h[2] | ((uint32_t)h[3] << 16),
                                                                             h[4] | ((uint32_t)h[5] << 16), h[6] | ((uint32_t)h[7] << 16));
                    }
                }
            }
        } else {
            for (uint32_t i = tid; i < TM * RT_KC; i += RT_WARPS * 32) {
                const uint32_t r = i / RT_KC, k = i % RT_KC;
                float v = 0.0f;
                if (t0 + r < n_tokens && k0 + k < d) v = load_act(x, (size_t)(t0 + r) * ldx + k0 + k, x_dtype);
                xs[r][(k & 31) * 8 + (k >> 5)] = v;
            }
            for (uint32_t i = tid; i < BE * RT_KC; i += RT_WARPS * 32) {
                const uint32_t r = i / RT_KC, k = i % RT_KC;
                uint16_t v = 0;
                if (e0 + r < num_experts && k0 + k < d) v = __bfloat16_as_ushort(w[(size_t)(e0 + r) * d + k0 + k]);
                ws[r][(k & 31) * 8 + (k >> 5)] = v;
            }
        }
        __syncthreads();
        float xv[TM][8];
#pragma unroll
        for (int i = 0; i < TM; ++i) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[i][lane * 8]);
            const float4 b = *reinterpret_cast<const float4*>(&xs[i][lane * 8 + 4]);
            xv[i][0] = a.x; xv[i][1] = a.y; xv[i][2] = a.z; xv[i][3] = a.w;
            xv[i][4] = b.x; xv[i][5] = b.y; xv[i][6] = b.z; xv[i][7] = b.w;
        }
#pragma unroll
        for (int j = 0; j < TE; ++j) {
            const uint4 q = *reinterpret_cast<const uint4*>(&ws[warp * TE + j][lane * 8]);
            const float wv[8] = {bf16_lo(q.x), bf16_hi(q.x), bf16_lo(q.y), bf16_hi(q.y),
                                 bf16_lo(q.z), bf16_hi(q.z), bf16_lo(q.w), bf16_hi(q.w)};
#pragma unroll
            for (int s = 0; s < 8; ++s)   // ascending k for this lane: k0 + s*32 + lane
#pragma unroll
                for (int i = 0; i < TM; ++i) acc[i][j] = fmaf(wv[s], xv[i][s], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TE; ++j) {
            float v = acc[i][j];
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            const uint32_t e = e0 + warp * TE + j, t = t0 + i;
            if (lane == 0 && e < num_experts && t < n_tokens) {
                if (logit_bias) v = v + logit_bias[e];
                logits[(size_t)t * num_experts + e] = v;
            }
        }
}

// Large batches (prefill): block tile 32 token rows x 16 experts, eight warps as 4 x 2, each warp 8 x 8 dot products
// held as 64 accumulators per lane.  The staged tiles keep the natural k order (fp32 activations, raw bf16 gate
// rows): lane l reads element s*32 + l of a row at sub-step s - exactly its k subset - so no transposition is needed
// and every shared-memory read is conflict-free.  Summation order per dot product is the same as above: lane l adds
// k = l, l+32, ... ascending with fma, then the xor butterfly, the bias last.
constexpr int RL_TM = 32, RL_TE = 16;

__global__ void __launch_bounds__(256, 2)
router_logits_tile_kernel(const void* __restrict__ x, int x_dtype, uint32_t ldx, uint32_t n_tokens,
                          const __nv_bfloat16* __restrict__ w, uint32_t num_experts, uint32_t d,
                          const float* __restrict__ logit_bias, float* __restrict__ logits) {
    __shared__ __align__(16) float xs[RL_TM][RT_KC];
    __shared__ __align__(16) uint16_t ws[RL_TE][RT_KC];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t t0 = blockIdx.y * RL_TM, e0 = blockIdx.x * RL_TE;
    const uint32_t wt = (warp & 3u) * 8, we = (warp >> 2) * 8;   // this warp's rows of the two tiles
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;
    const bool vec = x_dtype != MFB_DT_F32 && (ldx & 7u) == 0 && (d & 7u) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15u) == 0;
    for (uint32_t k0 = 0; k0 < d; k0 += RT_KC) {
        __syncthreads();
        if (vec) {
            for (uint32_t i = tid; i < RL_TM * (RT_KC / 8); i += 256) {
                const uint32_t r = i / (RT_KC / 8), k = (i % (RT_KC / 8)) * 8;
                uint4 q = make_uint4(0, 0, 0, 0);
                if (t0 + r < n_tokens && k0 + k < d)
                    q = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + (size_t)(t0 + r) * ldx + k0 + k);
                const uint32_t u[4] = {q.x, q.y, q.z, q.w};
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    f[j] = widen16((uint16_t)((j & 1) ? (u[j >> 1] >> 16) : (u[j >> 1] & 0xFFFFu)), x_dtype);
                *reinterpret_cast<float4*>(&xs[r][k]) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(&xs[r][k + 4]) = make_float4(f[4], f[5], f[6], f[7]);
            }
            for (uint32_t i = tid; i < RL_TE * (RT_KC / 8); i += 256) {
                const uint32_t r = i / (RT_KC / 8), k = (i % (RT_KC / 8)) * 8;
                uint4 q = make_uint4(0, 0, 0, 0);
                if (e0 + r < num_experts && k0 + k < d)
                    q = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(w) + (size_t)(e0 + r) * d + k0 + k);
                *reinterpret_cast<uint4*>(&ws[r][k]) = q;
            }
        } else {
            for (uint32_t i = tid; i < RL_TM * RT_KC; i += 256) {
                const uint32_t r = i / RT_KC, k = i % RT_KC;
                xs[r][k] = (t0 + r < n_tokens && k0 + k < d) ? load_act(x, (size_t)(t0 + r) * ldx + k0 + k, x_dtype) : 0.0f;
            }
            for (uint32_t i = tid; i < RL_TE * RT_KC; i += 256) {
                const uint32_t r = i / RT_KC, k = i % RT_KC;
                ws[r][k] = (e0 + r < num_experts && k0 + k < d) ? __bfloat16_as_ushort(w[(size_t)(e0 + r) * d + k0 + k]) : (uint16_t)0;
            }
        }
        __syncthreads();
#pragma unroll
        for (int s = 0; s < RT_KC / 32; ++s) {   // ascending k for this lane: k0 + s*32 + lane
            float xv[8], wv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) xv[i] = xs[wt + i][s * 32 + lane];
#pragma unroll
            for (int j = 0; j < 8; ++j) wv[j] = __uint_as_float((uint32_t)ws[we + j][s * 32 + lane] << 16);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(wv[j], xv[i], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float v = acc[i][j];
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
            const uint32_t e = e0 + we + j, t = t0 + wt + i;
            if (lane == ((i * 8 + j) & 31) && e < num_experts && t < n_tokens) {   // every lane holds the sum: spread the stores
                if (logit_bias) v = v + logit_bias[e];
                logits[(size_t)t * num_experts + e] = v;
            }
        }
}

// ---------------------------------------------------------------------------------------------- prefill-size gate
// Thousands of token rows: the same sums in the same order, arranged so that the multiply-adds are nearly the only
// instructions issued.  A first pass (router_lane_major_kernel) widens the activations and the gate to fp32 and stores
// every 128-element chunk of a row lane-major: position 4*l + s of a chunk holds element 32*s + l, i.e. the four
// elements lane l adds, in the order it adds them.  The tile kernel then needs no conversion and no address
// arithmetic: 16-byte asynchronous copies bring [32 token rows + 32 gate rows] x 128 floats per stage into a
// four-stage ring, and lane l reads its four values of a row with ONE conflict-free 16-byte shared-memory load
// (consecutive lanes, consecutive 16 bytes).  Sixteen warps as 4 x 4, a warp holds 8 tokens x 8 experts as 64
// accumulators; per stage it issues 16 loads for 256 multiply-adds.  The 32 lane sums of each dot product are
// combined by a butterfly in which every step halves the number of values a lane still carries (lanes whose bit
// `off` is clear keep the lower half of the values, the others the upper half): each value goes through the additions
// of the xor butterfly 16, 8, 4, 2, 1 with the same partners, and since a + b == b + a in IEEE arithmetic the result
// is bit-identical to it with 62 instead of 320 shuffles.
constexpr uint32_t RQ_TM = 32, RQ_TE = 32, RQ_KC = 128, RQ_STAGES = 4;
#ifndef MFB_RQ_NW
#define MFB_RQ_NW 8
#endif
constexpr int RQ_NW = MFB_RQ_NW, RQ_EW = 128 / RQ_NW;
constexpr uint32_t RQ_STAGE_FLOATS = (RQ_TM + RQ_TE) * RQ_KC;
constexpr uint32_t RQ_SMEM_BYTES = RQ_STAGES * RQ_STAGE_FLOATS * 4;

__global__ void router_lane_major_kernel(const void* __restrict__ src, int dtype, uint32_t ld, uint32_t rows, uint32_t d,
                                         float* __restrict__ dst) {
    const uint32_t per_row = d / 4;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * per_row) return;
    const uint32_t row = (uint32_t)(i / per_row), q = (uint32_t)(i % per_row), c = q / 32, l = q % 32;
    const size_t base = (size_t)row * ld + c * RQ_KC + l;
    reinterpret_cast<float4*>(dst)[i] = make_float4(load_act(src, base, dtype), load_act(src, base + 32, dtype),
                                                    load_act(src, base + 64, dtype), load_act(src, base + 96, dtype));
}

__device__ __forceinline__ void rq_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}

template <int N, int OFF>   // one step of the halving butterfly over v[0, N)
__device__ __forceinline__ void rq_halve(float* v, uint32_t lane) {
    const bool upper = (lane & OFF) != 0;
#pragma unroll
    for (int a = 0; a < N / 2; ++a) {
        const float keep = upper ? v[a + N / 2] : v[a], send = upper ? v[a] : v[a + N / 2];
        v[a] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, OFF);
    }
}

template <int NW, int EW>   // warps per block (4 token groups x NW/4 expert groups), experts per warp: NW/4 * EW = 32
__global__ void __launch_bounds__(NW * 32, 1)
router_logits_lane_major_kernel(const float* __restrict__ xq, uint32_t n_tokens, const float* __restrict__ wq, uint32_t num_experts,
                                uint32_t d, const float* __restrict__ logit_bias, float* __restrict__ logits) {
    static_assert((NW / 4) * EW == (int)RQ_TE, "tile shape");
    constexpr uint32_t THREADS = NW * 32, COPIES = (RQ_TM + RQ_TE) * (RQ_KC / 4) / THREADS, NV = 8 * EW;
    extern __shared__ __align__(16) float rq_smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t t0 = blockIdx.y * RQ_TM, e0 = blockIdx.x * RQ_TE;
    const uint32_t wt = (warp & 3u) * 8, we = (warp >> 2) * EW;
    const uint32_t n_chunks = d / RQ_KC;
    // copies of one stage: 64 rows x 32 pieces of 16 bytes; rows past the end repeat the last one (their sums are
    // computed and dropped)
    const float* src_row[COPIES];
    uint32_t dst_off[COPIES];
#pragma unroll
    for (uint32_t j = 0; j < COPIES; ++j) {
        const uint32_t piece = tid + j * THREADS, r = piece / 32, p = piece % 32;
        src_row[j] = r < RQ_TM ? xq + (size_t)min(t0 + r, n_tokens - 1) * d + p * 4
                               : wq + (size_t)min(e0 + r - RQ_TM, num_experts - 1) * d + p * 4;
        dst_off[j] = r * RQ_KC + p * 4;
    }
    auto issue = [&](uint32_t c) {
        if (c < n_chunks) {
            float* st = rq_smem + (c % RQ_STAGES) * RQ_STAGE_FLOATS;
#pragma unroll
            for (uint32_t j = 0; j < COPIES; ++j) rq_cp_async16(st + dst_off[j], src_row[j] + (size_t)c * RQ_KC);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[8][EW];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < EW; ++j) acc[i][j] = 0.0f;
    for (uint32_t c = 0; c + 1 < RQ_STAGES; ++c) issue(c);
    for (uint32_t c = 0; c < n_chunks; ++c) {
        asm volatile("cp.async.wait_group %0;" ::"n"(RQ_STAGES - 2) : "memory");
        __syncthreads();                 // chunk c has landed for every thread, and chunk c - 1 has been read by every warp
        issue(c + RQ_STAGES - 1);        // into the stage chunk c - 1 used
        const float4* st = reinterpret_cast<const float4*>(rq_smem + (c % RQ_STAGES) * RQ_STAGE_FLOATS);
        float4 xv[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) xv[i] = st[(wt + i) * (RQ_KC / 4) + lane];
#pragma unroll
        for (int j = 0; j < EW; ++j) {
            const float4 wv = st[(RQ_TM + we + j) * (RQ_KC / 4) + lane];
#pragma unroll
            for (int i = 0; i < 8; ++i) {   // ascending k for this lane: c*128 + lane, + 32, + 64, + 96
                acc[i][j] = fmaf(wv.x, xv[i].x, acc[i][j]);
                acc[i][j] = fmaf(wv.y, xv[i].y, acc[i][j]);
                acc[i][j] = fmaf(wv.z, xv[i].z, acc[i][j]);
                acc[i][j] = fmaf(wv.w, xv[i].w, acc[i][j]);
            }
        }
    }
    // halving butterfly over the NV values (index a = EW i + j): after the step with offset `off` a lane keeps the half
    // of its values selected by its bit `off`; at the end lane l holds values (NV/32) l ... (NV/32) l + NV/32 - 1
    float (&v)[NV] = reinterpret_cast<float (&)[NV]>(acc);
    rq_halve<NV, 16>(v, lane);
    rq_halve<NV / 2, 8>(v, lane);
    rq_halve<NV / 4, 4>(v, lane);
    rq_halve<NV / 8, 2>(v, lane);
    rq_halve<NV / 16, 1>(v, lane);
    constexpr uint32_t PER = NV / 32, LPR = EW / PER;   // values per lane; lanes per token row
    const uint32_t t = t0 + wt + lane / LPR, e = e0 + we + PER * (lane % LPR);
    if (t < n_tokens) {
#pragma unroll
        for (uint32_t j = 0; j < PER; ++j)
            if (e + j < num_experts) logits[(size_t)t * num_experts + e + j] = logit_bias ? v[j] + logit_bias[e + j] : v[j];
    }
}

__global__ void router_select_kernel(const float* __restrict__ logits, uint32_t n_tokens, uint32_t num_experts,
                                     uint32_t top_k, int mode, const __nv_bfloat16* __restrict__ per_expert_scale,
                                     const float* __restrict__ correction_bias, float route_scale,
                                     uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n_tokens) return;
    uint32_t e = 0;
    uint16_t w = 0;
    select_row(logits + (size_t)t * num_experts, num_experts, top_k, mode, per_expert_scale, correction_bias, route_scale,
               lane, e, w);
    if (lane < top_k) {
        out_idx[(size_t)t * top_k + lane] = e;
        out_w[(size_t)t * top_k + lane] = w;
    }
}

// Small batches (decode): selection for every row and the sort of the routing table by (expert, token, rank) in
// one CTA, so a decode layer spends one launch on routing.  Same outputs as router_select_kernel followed by the
// counting sort of group.cu.
constexpr uint32_t ROUTE_SMALL_MAX_PAIRS = 1024;

__global__ void __launch_bounds__(256) route_small_kernel(
    const float* __restrict__ logits, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k, int mode,
    const __nv_bfloat16* __restrict__ per_expert_scale, const float* __restrict__ correction_bias, float route_scale,
    int append_shared, uint32_t* __restrict__ out_idx, uint16_t* __restrict__ out_w, mfb_pair* __restrict__ sorted,
    mfb_group* __restrict__ groups, uint32_t* __restrict__ n_groups) {
    __shared__ uint32_t s_idx[ROUTE_SMALL_MAX_PAIRS];
    __shared__ uint16_t s_w[ROUTE_SMALL_MAX_PAIRS];
    __shared__ uint32_t s_run[MFB_MAX_EXPERTS];
    __shared__ uint32_t s_total;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_pairs = n_tokens * top_k;
    for (uint32_t e = threadIdx.x; e < num_experts; e += blockDim.x) s_run[e] = 0;
    for (uint32_t t = warp; t < n_tokens; t += blockDim.x >> 5) {
        uint32_t e = 0;
        uint16_t w = 0;
        select_row(logits + (size_t)t * num_experts, num_experts, top_k, mode, per_expert_scale, correction_bias,
                   route_scale, lane, e, w);
        if (lane < top_k) {
            s_idx[t * top_k + lane] = e;
            s_w[t * top_k + lane] = w;
            out_idx[(size_t)t * top_k + lane] = e;
            out_w[(size_t)t * top_k + lane] = w;
        }
    }
    __syncthreads();
    for (uint32_t p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&s_run[s_idx[p]], 1u);
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t run = 0, ng = 0;
        for (uint32_t e = 0; e < num_experts; ++e) {
            const uint32_t c = s_run[e];
            s_run[e] = run;
            if (c) { groups[ng].expert = e; groups[ng].pair_start = run; groups[ng].pair_count = c; ++ng; }
            run += c;
        }
        if (append_shared) { groups[ng].expert = num_experts; groups[ng].pair_start = run; groups[ng].pair_count = n_tokens; ++ng; }
        *n_groups = ng;
        s_total = run;
    }
    __syncthreads();
    if (warp == 0) {
        // ordered scatter: 32 pairs per round in (token, rank) order
        for (uint32_t p0 = 0; p0 < n_pairs; p0 += 32) {
            const uint32_t p = p0 + lane;
            const uint32_t e = p < n_pairs ? s_idx[p] : 0xFFFFFFFFu;
            const uint32_t peers = __match_any_sync(0xFFFFFFFFu, e);
            const uint32_t before = __popc(peers & ((1u << lane) - 1u));
            uint32_t pos = 0;
            if (p < n_pairs) pos = s_run[e] + before;
            __syncwarp();
            if (p < n_pairs && before == 0) s_run[e] += __popc(peers);
            __syncwarp();
            if (p < n_pairs) {
                mfb_pair out;
                out.token = p / top_k; out.expert = e; out.rank = p % top_k; out.weight_bits = s_w[p];
                sorted[pos] = out;
            }
        }
    } else if (append_shared) {
        for (uint32_t t = threadIdx.x - 32; t < n_tokens; t += blockDim.x - 32) {
            mfb_pair out;
            out.token = t; out.expert = num_experts; out.rank = top_k; out.weight_bits = 0x3C00u;
            sorted[s_total + t] = out;
        }
    }
}

// router_slot_lookup_k8 (moe.metal:594-617) for a block of rows and 64-bit offsets.
__global__ void slot_lookup_kernel(const uint32_t* __restrict__ idx, uint32_t n_tokens, uint32_t top_k,
                                   uint32_t num_experts, const int16_t* __restrict__ slot_of, uint64_t slot_stride,
                                   uint64_t* __restrict__ out_offsets, uint32_t* __restrict__ out_all_hit) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_tokens) return;
    uint32_t all_hit = 1u;
    for (uint32_t k = 0; k < top_k; ++k) {
        const uint32_t e = min(idx[(size_t)t * top_k + k], num_experts - 1u);
        const int16_t slot = slot_of[e];
        if (slot < 0) { all_hit = 0u; out_offsets[(size_t)t * top_k + k] = 0ull; }
        else out_offsets[(size_t)t * top_k + k] = (uint64_t)slot * slot_stride;
    }
    out_all_hit[t] = all_hit;
}

}  // namespace

// Set by router_init(): the prefill-size kernel's shared-memory attribute is in place (done when a handle is created, so
// that no later call changes function attributes).
static bool g_router_ready = false;

cudaError_t router_init() {
    const cudaError_t e = cudaFuncSetAttribute(router_logits_lane_major_kernel<RQ_NW, RQ_EW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RQ_SMEM_BYTES);
    if (e == cudaSuccess) g_router_ready = true;
    return e;
}

size_t router_workspace_floats(uint32_t max_tokens, uint32_t num_experts, uint32_t d) {
    if (max_tokens <= 64 || d % RQ_KC != 0) return 0;
    const uint64_t rows = max_tokens < ROUTER_WS_MAX_ROWS ? max_tokens : ROUTER_WS_MAX_ROWS;
    return (size_t)((rows + num_experts) * d);
}

cudaError_t launch_router_logits(cudaStream_t s, const void* x, int x_dtype, uint32_t ldx, uint32_t n_tokens,
                                 const __nv_bfloat16* w, uint32_t num_experts, uint32_t d, const float* logit_bias,
                                 float* logits, float* workspace, size_t workspace_floats) {
    if (n_tokens == 0) return cudaSuccess;
    if (n_tokens <= 2) {
        // decode: one expert per warp keeps 64 blocks busy on a 256-expert gate
        dim3 grid((num_experts + RT_WARPS - 1) / RT_WARPS, (n_tokens + 1) / 2);
        if (n_tokens == 1) { grid.y = 1; router_logits_kernel<1, 1><<<grid, RT_WARPS * 32, 0, s>>>(x, x_dtype, ldx, n_tokens, w, num_experts, d, logit_bias, logits); }
        else router_logits_kernel<2, 1><<<grid, RT_WARPS * 32, 0, s>>>(x, x_dtype, ldx, n_tokens, w, num_experts, d, logit_bias, logits);
    } else if (n_tokens <= 64) {
        dim3 grid((num_experts + RT_WARPS - 1) / RT_WARPS, (n_tokens + 7) / 8);
        router_logits_kernel<8, 1><<<grid, RT_WARPS * 32, 0, s>>>(x, x_dtype, ldx, n_tokens, w, num_experts, d, logit_bias, logits);
    } else if (g_router_ready && workspace && d % RQ_KC == 0 && workspace_floats >= (size_t)(num_experts + 1) * d) {
        // lane-major fp32 copies of the gate and of as many token rows as the workspace holds at a time
        float* wq = workspace;
        float* xq = workspace + (size_t)num_experts * d;
        const uint32_t cap = (uint32_t)std::min<size_t>((workspace_floats - (size_t)num_experts * d) / d, n_tokens);
        const uint32_t per_row = d / 4;
        router_lane_major_kernel<<<(uint32_t)(((size_t)num_experts * per_row + 255) / 256), 256, 0, s>>>(w, MFB_DT_BF16, d, num_experts, d, wq);
        for (uint32_t t0 = 0; t0 < n_tokens; t0 += cap) {
            const uint32_t n = std::min(cap, n_tokens - t0);
            const void* xs = (const uint8_t*)x + (size_t)t0 * ldx * (x_dtype == MFB_DT_F32 ? 4 : 2);
            router_lane_major_kernel<<<(uint32_t)(((size_t)n * per_row + 255) / 256), 256, 0, s>>>(xs, x_dtype, ldx, n, d, xq);
            dim3 grid((num_experts + RQ_TE - 1) / RQ_TE, (n + RQ_TM - 1) / RQ_TM);
            router_logits_lane_major_kernel<RQ_NW, RQ_EW><<<grid, RQ_NW * 32, RQ_SMEM_BYTES, s>>>(xq, n, wq, num_experts, d, logit_bias,
                                                                                                   logits + (size_t)t0 * num_experts);
            count_launches(2);
        }
    } else {
        dim3 grid((num_experts + RL_TE - 1) / RL_TE, (n_tokens + RL_TM - 1) / RL_TM);
        router_logits_tile_kernel<<<grid, 256, 0, s>>>(x, x_dtype, ldx, n_tokens, w, num_experts, d, logit_bias, logits);
    }
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_router_select(cudaStream_t s, const float* logits, uint32_t n_tokens, uint32_t num_experts,
                                 uint32_t top_k, int mode, const __nv_bfloat16* per_expert_scale,
                                 const float* correction_bias, float route_scale, uint32_t* out_idx, uint16_t* out_w) {
    if (n_tokens == 0) return cudaSuccess;
    const uint32_t warps = n_tokens >= 4 ? 4 : 1;
    router_select_kernel<<<(n_tokens + warps - 1) / warps, warps * 32, 0, s>>>(
        logits, n_tokens, num_experts, top_k, mode, per_expert_scale, correction_bias, route_scale, out_idx, out_w);
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_route_small(cudaStream_t s, const float* logits, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k,
                               int mode, const __nv_bfloat16* per_expert_scale, const float* correction_bias,
                               float route_scale, int append_shared, uint32_t* out_idx, uint16_t* out_w,
                               mfb_pair* sorted, mfb_group* groups, uint32_t* n_groups) {
    if (n_tokens == 0) return cudaSuccess;
    if (n_tokens * top_k > ROUTE_SMALL_MAX_PAIRS) return cudaErrorInvalidValue;
    route_small_kernel<<<1, 256, 0, s>>>(logits, n_tokens, num_experts, top_k, mode, per_expert_scale, correction_bias,
                                         route_scale, append_shared, out_idx, out_w, sorted, groups, n_groups);
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_slot_lookup(cudaStream_t s, const uint32_t* idx, uint32_t n_tokens, uint32_t top_k,
                               uint32_t num_experts, const int16_t* slot_of, uint64_t slot_stride,
                               uint64_t* out_offsets, uint32_t* out_all_hit) {
    if (n_tokens == 0) return cudaSuccess;
    slot_lookup_kernel<<<(n_tokens + 127) / 128, 128, 0, s>>>(idx, n_tokens, top_k, num_experts, slot_of, slot_stride,
                                                              out_offsets, out_all_hit);
    count_launches(1);
    return cudaGetLastError();
}

}  // namespace mfb
