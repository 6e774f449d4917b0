// Layer glue: RMSNorm, residual add and the rank-ordered weighted combine.
#include "common.cuh"

namespace mfb {

namespace {

// rmsnorm_bf16w (Sources/Mference/Metal/Primitives/rmsnorm.metal:32-93): inv = rsqrt(mean(x^2) + eps),
// out = dtype(x * inv * w).  One block per row, fp32 throughout.
__global__ void rmsnorm_kernel(const void* __restrict__ x, int in_dtype, const __nv_bfloat16* __restrict__ w,
                               uint32_t d, float eps, void* __restrict__ out, int out_dtype) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = load_act(x, row * d + i, in_dtype);
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
    const float inv = rsqrtf(red[0] / (float)d + eps);
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = load_act(x, row * d + i, in_dtype);
        const float g = w ? __bfloat162float(w[i]) : 1.0f;
        store_act(out, row * d + i, v * inv * g, out_dtype);
    }
}

// The same arithmetic in the same order for 16-bit rows whose length is a multiple of eight: the row crosses global
// memory once each way in 16-byte pieces and is kept in shared memory between the two passes (the element-wise form
// above moves 64 bytes per warp instruction and reads the row twice: 27 us for 4096 x 2048 against 9 us of traffic).
__global__ void rmsnorm_rows16_kernel(const uint16_t* __restrict__ x, int in_dtype, const __nv_bfloat16* __restrict__ w,
                                      uint32_t d, float eps, uint16_t* __restrict__ out, int out_dtype) {
    extern __shared__ __align__(16) uint16_t row_s[];
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(x + row * d);
    for (uint32_t p = threadIdx.x; p < d / 8; p += blockDim.x) reinterpret_cast<uint4*>(row_s)[p] = src[p];
    __syncthreads();
    float ss = 0.0f;
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = widen16(row_s[i], in_dtype);
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
    const float inv = rsqrtf(red[0] / (float)d + eps);
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x) {   // element i is read and rewritten by the same thread
        const float v = widen16(row_s[i], in_dtype);
        const float g = w ? __bfloat162float(w[i]) : 1.0f;
        row_s[i] = narrow16(v * inv * g, out_dtype);
    }
    __syncthreads();
    uint4* dst = reinterpret_cast<uint4*>(out + row * d);
    for (uint32_t p = threadIdx.x; p < d / 8; p += blockDim.x) dst[p] = reinterpret_cast<const uint4*>(row_s)[p];
}

// residual_add_fp16 (Sources/Mference/Metal/Primitives/utility.metal:83-92) in the activation dtype.
__global__ void residual_add_kernel(const void* __restrict__ a, const void* __restrict__ b, uint64_t n,
                                    void* __restrict__ out, int dtype) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) store_act(out, i, load_act(a, i, dtype) + load_act(b, i, dtype), dtype);
}

// y[t,i] = dtype( residual[t,i] + partial[t,top_k,i] (shared expert, weight 1) + sum_r w[t,r] * partial[t,r,i] )
// in fp32, residual first, ranks in ascending order: the order of moe_phase2_down_reduce_k8
// (Sources/Mference/Metal/MoE/moe.metal:349-404) and of prefill_moe_reduce_token_major
// (Sources/Mference/Metal/Prefill/prefill.metal:631-652).  Four elements per thread.
__global__ void combine_kernel(const float* __restrict__ partial, const uint16_t* __restrict__ route_w,
                               uint32_t n_tokens, uint32_t top_k, uint32_t slots, uint32_t d, uint32_t slot_mask,
                               int with_shared, const void* __restrict__ residual, void* __restrict__ y, int dtype) {
    const uint32_t quads = d / 4;
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)n_tokens * quads) return;
    const uint32_t t = (uint32_t)(i / quads), c = (uint32_t)(i % quads) * 4;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (residual) {
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = load_act(residual, (size_t)t * d + c + j, dtype);
    }
    const float* base = partial + (size_t)t * slots * d + c;
    if (with_shared) {
        const float4 v = *reinterpret_cast<const float4*>(base + (size_t)top_k * d);
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
    }
    for (uint32_t r = 0; r < top_k; ++r) {
        if (!((slot_mask >> r) & 1u)) continue;
        const float wr = __half2float(__ushort_as_half(route_w[(size_t)t * top_k + r]));
        const float4 v = *reinterpret_cast<const float4*>(base + (size_t)r * d);
        acc[0] = fmaf(wr, v.x, acc[0]); acc[1] = fmaf(wr, v.y, acc[1]);
        acc[2] = fmaf(wr, v.z, acc[2]); acc[3] = fmaf(wr, v.w, acc[3]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) store_act(y, (size_t)t * d + c + j, acc[j], dtype);
}

}  // namespace

// Expert id of every (token, rank) from the expert-major pair list; pairs that are not in the list keep 0xFFFFFFFF.
__global__ void pair_expert_table_kernel(const mfb_pair* __restrict__ sorted, const mfb_group* __restrict__ groups,
                                         const uint32_t* __restrict__ n_groups, uint32_t top_k, uint32_t num_slots,
                                         uint32_t* __restrict__ tok_expert) {
    const uint32_t ng = *n_groups;
    if (ng == 0) return;
    const mfb_group last = groups[ng - 1];
    const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= last.pair_start + last.pair_count) return;
    const mfb_pair pr = sorted[p];
    if (pr.rank < top_k && pr.token * top_k + pr.rank < num_slots) tok_expert[pr.token * top_k + pr.rank] = pr.expert;
}

// inkling_prefill_expert_down_accum (Sources/Mference/Metal/Prefill/prefill.metal:723-744) applied expert by expert in
// the order its host loop dispatches them (ascending expert id): for token t the ranks are visited in ascending expert
// order and acc = fma(weight, row, acc) in fp32.  One thread per (token, column); no atomics.
__global__ void accumulate_expert_order_kernel(const float* __restrict__ partial, const float* __restrict__ pair_weights,
                                               const uint32_t* __restrict__ tok_expert, uint32_t n_tokens, uint32_t top_k,
                                               uint32_t d, float* __restrict__ acc) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (uint64_t)n_tokens * d) return;
    const uint32_t t = (uint32_t)(i / d), c = (uint32_t)(i % d);
    float a = acc[i];
    uint32_t done = 0;   // bit r: rank r has been applied
    for (uint32_t step = 0; step < top_k; ++step) {
        uint32_t best = 0xFFFFFFFFu, best_r = 0;
        for (uint32_t r = 0; r < top_k; ++r) {
            const uint32_t e = tok_expert[t * top_k + r];
            if (!((done >> r) & 1u) && e < best) { best = e; best_r = r; }
        }
        if (best == 0xFFFFFFFFu) break;   // the remaining ranks are not in the pair list
        done |= 1u << best_r;
        a = fmaf(pair_weights[t * top_k + best_r], partial[((size_t)t * top_k + best_r) * d + c], a);
    }
    acc[i] = a;
}

cudaError_t launch_accumulate_expert_order(cudaStream_t s, const mfb_pair* sorted, const mfb_group* groups, const uint32_t* n_groups,
                                           uint32_t n_tokens, uint32_t top_k, uint32_t d, const float* partial,
                                           const float* pair_weights, uint32_t* tok_expert, float* acc) {
    if (n_tokens == 0) return cudaSuccess;
    const uint32_t slots = n_tokens * top_k;
    cudaError_t e = cudaMemsetAsync(tok_expert, 0xFF, (size_t)slots * sizeof(uint32_t), s);
    if (e != cudaSuccess) return e;
    pair_expert_table_kernel<<<(slots + 255) / 256, 256, 0, s>>>(sorted, groups, n_groups, top_k, slots, tok_expert);
    const uint64_t n = (uint64_t)n_tokens * d;
    accumulate_expert_order_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(partial, pair_weights, tok_expert, n_tokens, top_k, d, acc);
    count_launches(2);
    return cudaGetLastError();
}

cudaError_t launch_rmsnorm(cudaStream_t s, const void* x, int in_dtype, const __nv_bfloat16* w, uint32_t n_rows,
                           uint32_t d, float eps, void* out, int out_dtype) {
    if (n_rows == 0) return cudaSuccess;
    const bool rows16 = in_dtype != MFB_DT_F32 && out_dtype != MFB_DT_F32 && d % 8 == 0 && d * 2 <= 48 * 1024 &&
                        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    if (rows16)
        rmsnorm_rows16_kernel<<<n_rows, 256, d * 2, s>>>((const uint16_t*)x, in_dtype, w, d, eps, (uint16_t*)out, out_dtype);
    else
        rmsnorm_kernel<<<n_rows, 256, 0, s>>>(x, in_dtype, w, d, eps, out, out_dtype);
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_residual_add(cudaStream_t s, const void* a, const void* b, uint64_t n, void* out, int dtype) {
    if (n == 0) return cudaSuccess;
    residual_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, b, n, out, dtype);
    count_launches(1);
    return cudaGetLastError();
}

cudaError_t launch_combine(cudaStream_t s, const float* partial, const uint16_t* route_w, uint32_t n_tokens,
                           uint32_t top_k, uint32_t slots, uint32_t d, uint32_t slot_mask, int with_shared,
                           const void* residual, void* y, int dtype) {
    if (n_tokens == 0) return cudaSuccess;
    const uint64_t n = (uint64_t)n_tokens * (d / 4);
    combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(partial, route_w, n_tokens, top_k, slots, d, slot_mask,
                                                               with_shared, residual, y, dtype);
    count_launches(1);
    return cudaGetLastError();
}

}  // namespace mfb
