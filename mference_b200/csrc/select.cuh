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
// experts [L*per, L*per + per); every round takes a lane-local strict-greater ascending maximum (the lowest index
// among equal scores of the lane) and a warp-wide maximum that prefers the lower index on equal scores, which
// reproduces the serial insertion scan (strictly greater wins, equal keeps the earlier expert).  The warp-wide step
// is two hardware reductions: the maximum of an order-preserving integer image of the scores, then the minimum
// expert index among the lanes that hold it.  The weight tail runs in the serial rank order.
constexpr int SEL_MAX_PER_LANE = MFB_MAX_EXPERTS / 32;
constexpr uint32_t SEL_NONE = 0xFFFFFFFFu;

// Order-preserving map of fp32 (no NaN) onto uint32: a < b  <=>  key(a) < key(b); -0 and +0 differ, which the
// equality test below must not see, so -0 is folded onto +0 first.
__device__ __forceinline__ uint32_t sel_key(float v) {
    const uint32_t b = __float_as_uint(v + 0.0f);   // -0 + 0 = +0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

template <int PER>
__device__ __forceinline__ void select_row_per(const float* __restrict__ lg, uint32_t num_experts, uint32_t top_k, int mode,
                                               const __nv_bfloat16* __restrict__ per_expert_scale,
                                               const float* __restrict__ correction_bias, float route_scale, uint32_t lane,
                                               uint32_t& out_expert, uint16_t& out_weight) {
    const uint32_t base = lane * PER;
    float ch[PER];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
        const uint32_t e = base + j;
        float v = -INFINITY;
        if (e < num_experts) {
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
        for (int j = 0; j < PER; ++j)
            if (!(taken & (1u << j)) && ch[j] > bv) { bv = ch[j]; bi = base + j; }
        const uint32_t best_key = __reduce_max_sync(0xFFFFFFFFu, bi == SEL_NONE ? 0u : sel_key(bv));
        const uint32_t win = __reduce_min_sync(0xFFFFFFFFu, (bi != SEL_NONE && sel_key(bv) == best_key) ? bi : SEL_NONE);
        if (win != SEL_NONE && win >= base && win < base + PER) taken |= 1u << (win - base);
        if (lane == r) {
            // fewer experts than top_k: the serial scan leaves index 0 with score -inf (moe.metal:321-330)
            my_idx = win == SEL_NONE ? 0u : win;
            const uint32_t kb = (best_key & 0x80000000u) ? (best_key & 0x7FFFFFFFu) : ~best_key;
            my_score = win == SEL_NONE ? -INFINITY : __uint_as_float(kb);
        }
    }
    // weight tail, serial order on values gathered from the rank lanes (top_k <= 16 < 32)
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

// Selection for one row by one warp; lane r < top_k returns the rank-r expert and its fp16 weight bits.
__device__ __forceinline__ void select_row(const float* __restrict__ lg, uint32_t num_experts, uint32_t top_k, int mode,
                                           const __nv_bfloat16* __restrict__ per_expert_scale,
                                           const float* __restrict__ correction_bias, float route_scale, uint32_t lane,
                                           uint32_t& out_expert, uint16_t& out_weight) {
    const uint32_t per = (num_experts + 31) / 32;
    if (per <= 4) select_row_per<4>(lg, num_experts, top_k, mode, per_expert_scale, correction_bias, route_scale, lane, out_expert, out_weight);
    else if (per <= 8) select_row_per<8>(lg, num_experts, top_k, mode, per_expert_scale, correction_bias, route_scale, lane, out_expert, out_weight);
    else select_row_per<SEL_MAX_PER_LANE>(lg, num_experts, top_k, mode, per_expert_scale, correction_bias, route_scale, lane, out_expert, out_weight);
}

}  // namespace mfb
