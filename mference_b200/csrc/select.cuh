// Top-k selection of one row of router scores by one warp; shared by the router kernels and the fused decode kernel.
#pragma once

#include "common.cuh"

namespace mfb {

// sqrt(softplus(x)) in the numerically safe form of moe.metal:737-741.
__device__ __forceinline__ float sqrtsoftplus(float x) {
    const float sp = fmaxf(x, 0.0f) + logf(1.0f + expf(-fabsf(x)));
    return sqrtf(sp);
}

// One warp per token row.  Blocked ownership as in router_topk_select_k8_par (moe.metal:262-345): lane L owns
// experts [L*per, L*per + per); every round takes a lane-local strict-greater ascending maximum and a
// shuffle argmax that prefers the lower index on equal scores, which reproduces the serial insertion scan
// (strictly greater wins, equal keeps the earlier expert).  The weight tail runs on lane 0 in the serial order.
constexpr int SEL_MAX_PER_LANE = MFB_MAX_EXPERTS / 32;
constexpr uint32_t SEL_NONE = 0xFFFFFFFFu;

// Selection for one row by one warp; lane r < top_k returns the rank-r expert and its fp16 weight bits.
__device__ __forceinline__ void select_row(const float* __restrict__ lg, uint32_t num_experts, uint32_t top_k, int mode,
                                           const __nv_bfloat16* __restrict__ per_expert_scale,
                                           const float* __restrict__ correction_bias, float route_scale, uint32_t lane,
                                           uint32_t& out_expert, uint16_t& out_weight) {
    const uint32_t per = (num_experts + 31) / 32, base = lane * per;
    float ch[SEL_MAX_PER_LANE];
#pragma unroll
    for (int j = 0; j < SEL_MAX_PER_LANE; ++j) {
        const uint32_t e = base + j;
        float v = -INFINITY;
        if ((uint32_t)j < per && e < num_experts) {
            v = lg[e];
            if (mode == MFB_ROUTER_SQRTSOFTPLUS) v = sqrtsoftplus(v) + (correction_bias ? correction_bias[e] : 0.0f);
        }
        ch[j] = v;
    }
    uint32_t taken = 0;
    uint32_t my_idx = 0;     // lane r keeps the winner of round r
    float my_score = -INFINITY;
    for (uint32_t r = 0; r < top_k; ++r) {
        float bv = -INFINITY;
        uint32_t bi = SEL_NONE;
#pragma unroll
        for (int j = 0; j < SEL_MAX_PER_LANE; ++j)
            if (!(taken & (1u << j)) && ch[j] > bv) { bv = ch[j]; bi = base + j; }
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_down_sync(0xFFFFFFFFu, bv, off);
            const uint32_t oi = __shfl_down_sync(0xFFFFFFFFu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        bi = __shfl_sync(0xFFFFFFFFu, bi, 0);
        bv = __shfl_sync(0xFFFFFFFFu, bv, 0);
        if (bi != SEL_NONE && bi >= base && bi < base + per) taken |= 1u << (bi - base);
        if (lane == r) {
            // fewer experts than top_k: the serial scan leaves index 0 with score -inf (moe.metal:321-330)
            my_idx = bi == SEL_NONE ? 0u : bi;
            my_score = bi == SEL_NONE ? -INFINITY : bv;
        }
    }
    // weight tail, serial order on values gathered to lane 0 (top_k <= 16 < 32)
    float score = my_score;
    if (mode == MFB_ROUTER_SQRTSOFTPLUS) score = lane < top_k ? sqrtsoftplus(lg[my_idx]) : 0.0f;
    const float max_s = __shfl_sync(0xFFFFFFFFu, score, 0);
    float term = 0.0f;
    if (lane < top_k) term = mode == MFB_ROUTER_SQRTSOFTPLUS ? score : expf(score - max_s);
    float sum = 0.0f;
    for (uint32_t r = 0; r < top_k; ++r) sum += __shfl_sync(0xFFFFFFFFu, term, r);  // rank order, same on every lane
    if (lane < top_k) {
        float wgt;
        if (mode == MFB_ROUTER_SQRTSOFTPLUS) {
            const float inv = route_scale / (sum + 1e-20f);
            wgt = term * inv;
        } else {
            const float gain = per_expert_scale ? __bfloat162float(per_expert_scale[my_idx]) : 1.0f;
            wgt = term / sum * gain;
        }
        out_expert = my_idx;
        out_weight = __half_as_ushort(__float2half_rn(wgt));
    }
}

}  // namespace mfb
