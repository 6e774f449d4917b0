// Expert-parallel dispatch / combine kernels (batched and prefill workloads over 2, 4 or 8 GPUs of one box).
//
// Experts are block-sharded: rank g owns experts [g * E/G, (g+1) * E/G); tokens stay data-parallel.  One exchange
// each way per layer: the activation row of every (token, rank slot) pair travels to the rank that owns the pair's
// expert, the expert's down-projection row travels back, and the home rank applies the routing weights in rank
// order - the same order, with the same fp32 fused multiply-adds, as the single-GPU combine, so the two agree bit
// for bit.  The exchanges themselves are NCCL all-to-all calls made by the host layer (mference_b200/ep.py); the
// kernels here build the send order, pack the rows, and fuse "receive + weighted reduce + shared expert + residual".
// The reference has no multi-GPU code; the single-device semantics being preserved are those of
// prefill_moe_reduce_token_major (Sources/Mference/Metal/Prefill/prefill.metal:631-652).
#include "common.cuh"

namespace mfb {
namespace {

constexpr int EP_MAX_WORLD = 8;

// One block.  Stable counting sort of the T*K pairs by destination rank: send order = (dest, token, rank slot).
// perm[pos] = pair id (token * K + slot) at send position pos; inv[pair] = pos; counts[g] = pairs bound for rank g;
// local_expert[pos] = expert id relative to the destination's first expert.
__global__ void ep_plan_kernel(const uint32_t* __restrict__ idx, uint32_t n_pairs, uint32_t experts_per_rank, uint32_t world,
                               uint32_t* __restrict__ perm, uint32_t* __restrict__ inv, int32_t* __restrict__ counts,
                               int32_t* __restrict__ local_expert) {
    __shared__ uint32_t hist[EP_MAX_WORLD], run[EP_MAX_WORLD];
    if (threadIdx.x < EP_MAX_WORLD) hist[threadIdx.x] = 0;
    __syncthreads();
    for (uint32_t p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&hist[min(idx[p] / experts_per_rank, world - 1)], 1u);
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t acc = 0;
        for (uint32_t g = 0; g < world; ++g) { run[g] = acc; counts[g] = (int32_t)hist[g]; acc += hist[g]; }
    }
    __syncthreads();
    // ordered scatter by warp 0, 32 pairs per round in pair order (the same scheme as the grouping kernels)
    if (threadIdx.x < 32) {
        const uint32_t lane = threadIdx.x;
        for (uint32_t p0 = 0; p0 < n_pairs; p0 += 32) {
            const uint32_t p = p0 + lane;
            const uint32_t e = p < n_pairs ? idx[p] : 0u;
            const uint32_t g = p < n_pairs ? min(e / experts_per_rank, world - 1) : 0xFFFFFFFFu;
            const uint32_t peers = __match_any_sync(0xFFFFFFFFu, g);
            const uint32_t before = __popc(peers & ((1u << lane) - 1u));
            uint32_t pos = 0;
            if (p < n_pairs) pos = run[g] + before;
            __syncwarp();
            if (p < n_pairs && before == 0) run[g] += __popc(peers);
            __syncwarp();
            if (p < n_pairs) {
                perm[pos] = p;
                inv[p] = pos;
                local_expert[pos] = (int32_t)(e - g * experts_per_rank);
            }
        }
    }
}

// rows[pos, :] = x[perm[pos] / K, :]   (16-bit rows, 16-byte pieces)
__global__ void ep_pack_kernel(const uint16_t* __restrict__ x, uint32_t ldx, uint32_t d, const uint32_t* __restrict__ perm,
                               uint32_t n_pairs, uint32_t top_k, uint16_t* __restrict__ rows) {
    const uint32_t pos = blockIdx.x;
    if (pos >= n_pairs) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(perm[pos] / top_k) * ldx);
    uint4* dst = reinterpret_cast<uint4*>(rows + (size_t)pos * d);
    for (uint32_t i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}

// y[t, c] = dtype( residual + shared + sum_k fma(w[t,k], recv[inv[t*K+k], c]) ), ranks ascending.
__global__ void ep_combine_kernel(const float* __restrict__ recv, const uint32_t* __restrict__ inv, const uint16_t* __restrict__ route_w,
                                  const float* __restrict__ shared_partial, const void* __restrict__ residual, void* __restrict__ y,
                                  uint32_t n_tokens, uint32_t top_k, uint32_t d, int x_dtype) {
    const uint32_t t = blockIdx.x;
    if (t >= n_tokens) return;
    for (uint32_t c = threadIdx.x; c < d; c += blockDim.x) {
        float acc = residual ? load_act(residual, (size_t)t * d + c, x_dtype) : 0.0f;
        if (shared_partial) acc += shared_partial[(size_t)t * d + c];
        for (uint32_t k = 0; k < top_k; ++k) {
            const float w = __half2float(__ushort_as_half(route_w[(size_t)t * top_k + k]));
            acc = fmaf(w, recv[(size_t)inv[(size_t)t * top_k + k] * d + c], acc);
        }
        store_act(y, (size_t)t * d + c, acc, x_dtype);
    }
}

}  // namespace
}  // namespace mfb

using namespace mfb;

extern "C" int32_t mfb_ep_plan(void* stream, const uint32_t* idx, uint32_t n_tokens, uint32_t top_k, uint32_t num_experts,
                               uint32_t world, uint32_t* perm, uint32_t* inv, int32_t* counts, int32_t* local_expert) {
    MFB_REQUIRE(idx && perm && inv && counts && local_expert, MFB_ERR_INVALID_ARGUMENT, "ep_plan: NULL argument");
    MFB_REQUIRE(world >= 1 && world <= (uint32_t)EP_MAX_WORLD && num_experts % world == 0, MFB_ERR_INVALID_ARGUMENT,
                "ep_plan: world must be in 1..%d and divide num_experts", EP_MAX_WORLD);
    if (n_tokens == 0) {
        MFB_CUDA(cudaMemsetAsync(counts, 0, world * sizeof(int32_t), (cudaStream_t)stream));
        return MFB_OK;
    }
    ep_plan_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(idx, n_tokens * top_k, num_experts / world, world, perm, inv, counts, local_expert);
    count_launches(1);
    MFB_CUDA(cudaGetLastError());
    return MFB_OK;
}

extern "C" int32_t mfb_ep_pack(void* stream, const void* x, uint32_t ldx, uint32_t d, const uint32_t* perm, uint32_t n_pairs,
                               uint32_t top_k, void* rows) {
    MFB_REQUIRE(x && perm && rows, MFB_ERR_INVALID_ARGUMENT, "ep_pack: NULL argument");
    MFB_REQUIRE(d % 8 == 0 && ldx % 8 == 0 && top_k >= 1, MFB_ERR_INVALID_ARGUMENT, "ep_pack: d and the row stride must be multiples of 8");
    if (n_pairs == 0) return MFB_OK;
    ep_pack_kernel<<<n_pairs, 128, 0, (cudaStream_t)stream>>>((const uint16_t*)x, ldx, d, perm, n_pairs, top_k, (uint16_t*)rows);
    count_launches(1);
    MFB_CUDA(cudaGetLastError());
    return MFB_OK;
}

extern "C" int32_t mfb_ep_combine(void* stream, const float* recv, const uint32_t* inv, const uint16_t* route_w,
                                  const float* shared_partial, const void* residual, void* y, uint32_t n_tokens, uint32_t top_k,
                                  uint32_t d, uint32_t x_dtype) {
    MFB_REQUIRE(recv && inv && route_w && y, MFB_ERR_INVALID_ARGUMENT, "ep_combine: NULL argument");
    MFB_REQUIRE(x_dtype == MFB_DT_BF16 || x_dtype == MFB_DT_F16, MFB_ERR_INVALID_ARGUMENT, "ep_combine: activation dtype must be fp16 or bf16");
    if (n_tokens == 0) return MFB_OK;
    ep_combine_kernel<<<n_tokens, 256, 0, (cudaStream_t)stream>>>(recv, inv, route_w, shared_partial, residual, y, n_tokens, top_k, d, (int)x_dtype);
    count_launches(1);
    MFB_CUDA(cudaGetLastError());
    return MFB_OK;
}
