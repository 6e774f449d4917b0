// Shared declarations of the sm_100a MoE feed-forward library: the handle, the scratch arena, dtype
// helpers and the launch prototypes each translation unit exports to api.cu.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mfb200.h"

namespace mfb {

// ---- error plumbing -------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
void count_launches(uint64_t n);   // bookkeeping behind mfb_launch_count()
int32_t cuda_fail(cudaError_t e, const char* what);

#define MFB_CUDA(call)                                                    \
    do {                                                                  \
        cudaError_t e__ = (call);                                         \
        if (e__ != cudaSuccess) return ::mfb::cuda_fail(e__, #call);      \
    } while (0)

#define MFB_REQUIRE(cond, code, ...)                                      \
    do {                                                                  \
        if (!(cond)) {                                                    \
            ::mfb::set_error(__VA_ARGS__);                                \
            return (code);                                                \
        }                                                                 \
    } while (0)

// ---- device-side status word ----------------------------------------------------------------------------
// Kernels with bounded waits OR a reason code in here instead of spinning for ever or trapping.
enum : uint32_t {
    STATUS_MBAR_TIMEOUT = 1u,
    STATUS_GRID_BARRIER_TIMEOUT = 2u,
    STATUS_SELF_CHECK = 4u,
};

// ---- scratch arena owned by a handle --------------------------------------------------------------------
struct Arena {
    // router
    float* logits = nullptr;        // [max_tokens, E]
    uint32_t* idx = nullptr;        // [max_tokens, K]
    uint16_t* route_w = nullptr;    // [max_tokens, K] fp16 bits
    float* router_ws = nullptr;     // fp32 lane-major copies for the prefill-size gate kernel (router_workspace_floats)
    size_t router_ws_floats = 0;
    // normalised activations of a layer call, in x_dtype
    void* xn = nullptr;             // [max_tokens, d]
    // grouping
    mfb_pair* sorted = nullptr;     // [max_tokens*K + max_tokens]  (routed pairs, then one shared pair per token)
    uint32_t* chunk_hist = nullptr; // [n_chunks, E]
    uint32_t* offsets = nullptr;    // [E]
    uint32_t* counts = nullptr;     // [E]
    mfb_group* groups = nullptr;    // [E + 1]
    uint32_t* n_groups = nullptr;   // [1]
    uint32_t* tile_prefix = nullptr;// [E + 2] prefix of per-group tile counts for the grouped GEMM
    // expert FFN intermediates
    float* acts = nullptr;          // [max_tokens*(K+1), f]   decode path (fp32)
    float* partial = nullptr;       // [max_tokens*(K+1), d]   per-(token, slot) down-projection rows
    __half* xs16 = nullptr;         // [max_tokens*(K+1) (+pad), d] gathered fp16 activations (tensor-core path)
    __half* acts16 = nullptr;       // [max_tokens*(K+1) (+pad), f] fp16 activations (tensor-core path)
    // fast decode path: fp16 activations in the fragment order of the code width(s), fp16 hidden activations
    __half* xp = nullptr;           // [max_tokens, d]
    __half* xp2 = nullptr;          // [max_tokens, d] second permutation when shared_bits != bits
    __half* actp = nullptr;         // [max_tokens*(K+1), f]
    uint32_t* status = nullptr;     // device status word
    uint32_t n_chunks = 0;
};

}  // namespace mfb

struct mfb_moe {
    mfb_moe_config cfg;
    mfb::Arena a;
    int device = 0;
    int sm_count = 0;
    uint64_t max_pairs = 0;   // max_tokens * top_k
    uint64_t max_rows = 0;    // max_tokens * (top_k + 1)
    void* tma = nullptr;      // tensor-map cache of the tcgen05 path (opaque here)
    bool force_generic = false;  // route every call through the generic SIMT kernels (mfb_moe_set_generic)
    bool no_fused = false;       // keep the fast kernels but launch them layer by layer, phase by phase
    // fused stack kernel: device copy of the per-layer weight table, its host mirror (to skip identical uploads),
    // the barrier words, and whether the device supports cooperative launches
    void* mega_dev = nullptr;
    void* mega_host = nullptr;
    uint32_t mega_cap = 0, mega_count = 0;
    uint32_t* mega_bar = nullptr;
    bool coop = false;
    void* wide_cache = nullptr;  // tensor maps of the layers this handle has seen (row-stationary decode phases; opaque here)
    uint64_t* trace = nullptr;   // device buffer for phase time stamps (mfb_moe_set_trace), not owned
};

namespace mfb {

constexpr int GROUP_CHUNK = 256;  // pairs per warp in the counting sort

// ---- dtype helpers --------------------------------------------------------------------------------------
__device__ __forceinline__ float widen16(uint16_t v, int dtype) {
    return dtype == MFB_DT_BF16 ? __uint_as_float((uint32_t)v << 16) : __half2float(__ushort_as_half(v));
}
__device__ __forceinline__ uint16_t narrow16(float v, int dtype) {
    return dtype == MFB_DT_BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}
__device__ __forceinline__ float load_act(const void* p, size_t i, int dtype) {
    if (dtype == MFB_DT_F32) return ((const float*)p)[i];
    return widen16(((const uint16_t*)p)[i], dtype);
}
__device__ __forceinline__ void store_act(void* p, size_t i, float v, int dtype) {
    if (dtype == MFB_DT_F32) ((float*)p)[i] = v;
    else ((uint16_t*)p)[i] = narrow16(v, dtype);
}

// Hidden activation of the expert FFN (Sources/Mference/Metal/MoE/moe.metal:71-84).
__device__ __forceinline__ float hidden_act(float g, int act) {
    if (act == MFB_ACT_SILU) return g / (1.0f + __expf(-g));
    float inner = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    inner = fminf(fmaxf(inner, -20.0f), 20.0f);
    return 0.5f * g * (1.0f + tanhf(inner));
}

// ---- launch prototypes ----------------------------------------------------------------------------------
// router.cu
// `workspace` (optional, router_workspace_floats() floats for a given row capacity): scratch for the fp32 lane-major
// copies the prefill-size kernel reads; without it batches above 64 rows take the slower self-contained kernel.
constexpr uint32_t ROUTER_WS_MAX_ROWS = 8192;   // token rows converted at a time
size_t router_workspace_floats(uint32_t max_tokens, uint32_t num_experts, uint32_t d);
cudaError_t router_init();   // once per process, from mfb_moe_create
cudaError_t launch_router_logits(cudaStream_t s, const void* x, int x_dtype, uint32_t ldx, uint32_t n_tokens,
                                 const __nv_bfloat16* w, uint32_t num_experts, uint32_t d, const float* logit_bias,
                                 float* logits, float* workspace = nullptr, size_t workspace_floats = 0);
cudaError_t launch_router_select(cudaStream_t s, const float* logits, uint32_t n_tokens, uint32_t num_experts,
                                 uint32_t top_k, int mode, const __nv_bfloat16* per_expert_scale,
                                 const float* correction_bias, float route_scale, uint32_t* out_idx, uint16_t* out_w);
cudaError_t launch_slot_lookup(cudaStream_t s, const uint32_t* idx, uint32_t n_tokens, uint32_t top_k,
                               uint32_t num_experts, const int16_t* slot_of, uint64_t slot_stride,
                               uint64_t* out_offsets, uint32_t* out_all_hit);
// quant_gemv.cu
cudaError_t launch_gemv_int8(cudaStream_t s, const uint8_t* W, const void* scales, const void* biases, const void* x, int x_dtype,
                             uint32_t ldx, uint32_t n_tokens, const void* effective_scale, uint32_t M, uint32_t N, float* y);
cudaError_t launch_shared_gate_scale(cudaStream_t s, const float* gate, float* rows, uint64_t row_stride, uint32_t n_tokens, uint32_t d);
// glue.cu
cudaError_t launch_rmsnorm(cudaStream_t s, const void* x, int in_dtype, const __nv_bfloat16* w, uint32_t n_rows,
                           uint32_t d, float eps, void* out, int out_dtype);
cudaError_t launch_residual_add(cudaStream_t s, const void* a, const void* b, uint64_t n, void* out, int dtype);
cudaError_t launch_combine(cudaStream_t s, const float* partial, const uint16_t* route_w, uint32_t n_tokens,
                           uint32_t top_k, uint32_t slots, uint32_t d, uint32_t slot_mask, int with_shared,
                           const void* residual, void* y, int dtype);
// group.cu
cudaError_t launch_group(cudaStream_t s, const uint32_t* idx, const uint16_t* route_w, uint32_t n_tokens,
                         uint32_t top_k, uint32_t num_experts, uint32_t slot_mask, int append_shared,
                         uint32_t tile_rows, Arena& a, mfb_pair* out_sorted, uint32_t* out_offsets,
                         uint32_t* out_counts, mfb_group* out_groups, uint32_t* out_n_groups, uint32_t* tile_prefix);
// decode.cu
struct DecodeArgs {
    const mfb_layer_weights* w;  // host copy
    uint32_t d, f, num_experts, top_k, bits, shared_bits, scale_dtype, activation;
    float swiglu_limit;
    const void* x;
    int x_dtype;
    uint32_t ldx;
    const mfb_pair* sorted;
    const mfb_group* groups;
    const uint32_t* n_groups;
    uint32_t max_groups;
    float* acts;     // [rows, f]
    float* partial;  // [rows, d]
    uint32_t slots;  // top_k + 1
    uint32_t round16 = 0;   // gate, up and the activation product rounded to fp16 (inkling_prefill_expert_act, prefill.metal:695-721)
};
cudaError_t launch_decode_ffn(cudaStream_t s, const DecodeArgs& a);
// acc[t, :] = fma(w[t, r], partial[t * top_k + r, :], acc[t, :]) over the ranks of token t in ascending expert order
cudaError_t launch_accumulate_expert_order(cudaStream_t s, const mfb_pair* sorted, const mfb_group* groups, const uint32_t* n_groups,
                                           uint32_t n_tokens, uint32_t top_k, uint32_t d, const float* partial,
                                           const float* pair_weights, uint32_t* tok_expert, float* acc);
// synth.cu
cudaError_t launch_synth_pool(cudaStream_t s, const uint64_t* seeds_dev, uint32_t n_experts, uint32_t bits,
                              uint32_t scale_dtype, uint32_t d, uint32_t f, uint8_t* pool, uint64_t slot_stride,
                              mfb_expert_offsets off);
cudaError_t launch_synth_normal(cudaStream_t s, uint64_t seed, uint64_t n, double mean, double std, int absolute,
                                uint32_t dtype, void* out);

}  // namespace mfb
