// Router top-k for callers that cannot allocate: the logits scratch is a fixed array inside this library's device
// image instead of a handle's arena.
//
// Why it exists: mfb_router_topk needs a handle, and creating a handle allocates device memory.  A host that has
// handed the whole GPU memory budget to its own allocator (an inference server with a pre-sized pool, a process
// running under a memory cap, code inside a region where allocation calls are forbidden) can still route a decode
// batch with this entry point: nothing here calls an allocator, directly or through a library.
#include <mutex>

#include "common.cuh"

namespace mfb {
namespace {

constexpr int MAX_DEVICES = 64;

// [MFB_STATIC_ROUTER_MAX_TOKENS][MFB_MAX_EXPERTS] fp32 logits, 128 KiB of the module's global memory per device.
// Every element a call reads it has written before (the logits kernel fills rows [0, n_tokens) x [0, num_experts)
// that the selection kernel then reads), so nothing has to start at zero.
static __device__ __align__(256) float g_router_logits[MFB_STATIC_ROUTER_MAX_TOKENS * MFB_MAX_EXPERTS];

std::mutex g_mutex;
float* g_scratch[MAX_DEVICES] = {};   // device address of g_router_logits on each device, resolved once

// Resolves the scratch address for the current device (the array name is a host-side handle, not a device pointer).
int32_t scratch_for_current_device(float** out) {
    int dev = -1;
    MFB_CUDA(cudaGetDevice(&dev));
    MFB_REQUIRE(dev >= 0 && dev < MAX_DEVICES, MFB_ERR_CUDA, "router_topk_static: device ordinal %d not supported", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    if (!g_scratch[dev]) {
        void* p = nullptr;
        MFB_CUDA(cudaGetSymbolAddress(&p, g_router_logits));
        MFB_REQUIRE(p != nullptr, MFB_ERR_CUDA, "router_topk_static: scratch symbol has no address on device %d", dev);
        g_scratch[dev] = static_cast<float*>(p);
    }
    *out = g_scratch[dev];
    return MFB_OK;
}

}  // namespace
}  // namespace mfb

using namespace mfb;

extern "C" int32_t mfb_router_topk_static(void* stream, const void* x, uint32_t x_dtype, uint32_t ldx, uint32_t n_tokens,
                                          uint32_t d, const void* router_w, const float* logit_bias, uint32_t num_experts,
                                          uint32_t top_k, uint32_t router_mode, const void* per_expert_scale,
                                          const float* correction_bias, float route_scale, uint32_t* out_idx,
                                          uint16_t* out_w) {
    MFB_REQUIRE(x && router_w && out_idx && out_w, MFB_ERR_INVALID_ARGUMENT, "router_topk_static: NULL argument");
    MFB_REQUIRE(n_tokens <= MFB_STATIC_ROUTER_MAX_TOKENS, MFB_ERR_CAPACITY,
                "router_topk_static: %u token rows exceed the fixed scratch of %d rows; use mfb_router_topk with a handle",
                n_tokens, MFB_STATIC_ROUTER_MAX_TOKENS);
    MFB_REQUIRE(num_experts >= 1 && num_experts <= MFB_MAX_EXPERTS, MFB_ERR_UNSUPPORTED_SHAPE,
                "router_topk_static: num_experts must be in 1..%d", MFB_MAX_EXPERTS);
    MFB_REQUIRE(top_k >= 1 && top_k <= MFB_MAX_TOP_K && top_k <= num_experts, MFB_ERR_UNSUPPORTED_SHAPE,
                "router_topk_static: top_k must be in 1..%d and at most num_experts", MFB_MAX_TOP_K);
    MFB_REQUIRE(d >= 1 && ldx >= d, MFB_ERR_INVALID_ARGUMENT, "router_topk_static: row stride smaller than d");
    MFB_REQUIRE(x_dtype == MFB_DT_F16 || x_dtype == MFB_DT_BF16, MFB_ERR_INVALID_ARGUMENT,
                "router_topk_static: activation dtype must be fp16 or bf16");
    MFB_REQUIRE(router_mode <= MFB_ROUTER_SQRTSOFTPLUS, MFB_ERR_INVALID_ARGUMENT, "router_topk_static: router mode");
    float* logits = nullptr;
    const int32_t rc = scratch_for_current_device(&logits);
    if (rc) return rc;
    if (n_tokens == 0) return MFB_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MFB_CUDA(launch_router_logits(s, x, (int)x_dtype, ldx, n_tokens, (const __nv_bfloat16*)router_w, num_experts, d, logit_bias,
                                  logits));
    MFB_CUDA(launch_router_select(s, logits, n_tokens, num_experts, top_k, (int)router_mode,
                                  (const __nv_bfloat16*)per_expert_scale, correction_bias, route_scale, out_idx, out_w));
    return MFB_OK;
}
