// Fast decode path (tensor-core fragments fed from TMA-staged packed rows): interface used by api.cu.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace mfb {

// Tensor maps over one layer's weights for the row-stationary FFN phases: [0] the routed pool (third coordinate =
// pool slot), [1] the shared expert's blob; in each: gate W, up W, down W (codes, boxes of 128 rows x 128 bytes,
// 128-byte swizzle), then gate S, gate B, up S, up B, down S, down B (scales and biases, boxes of 128 rows x 32 or 16
// bytes).  Lives in device memory owned by the handle.
struct WideMaps {
    CUtensorMap m[2][9];
};

struct FastParams {
    const uint8_t* pool;
    uint64_t slot_stride;
    const int16_t* slot_of;
    const uint8_t* shared_blob;
    mfb_expert_offsets routed_off, shared_off;
    uint32_t d, f, num_experts, top_k, bits, shared_bits, scale_dtype, activation;
    float limit;
    const mfb_pair* sorted;
    const mfb_group* groups;
    const uint32_t* n_groups;
    const __half* xp;         // [tokens, d] fp16 activations, permuted for `bits`
    const __half* xp_shared;  // the same permuted for `shared_bits` (== xp when the widths agree)
    int x_in_smem;            // xp / xp_shared point into shared memory (single-token mode of the fused kernel)
    __half* actp;             // [sorted pairs (+ tokens), f] fp16 hidden activations, permuted per group width
    float* partial;           // [tokens, top_k + 1, d] fp32 down-projection rows per (token, rank slot)
    const uint16_t* route_w;  // [tokens, top_k] fp16 bits
    const void* residual;     // [tokens, d] or NULL
    void* y;                  // [tokens, d]
    int x_dtype;
    uint32_t n_tokens;
    uint32_t* status;
    unsigned long long* dbg;  // optional cycle counters of CTA 0: [17 warps][8] (wait / compute per phase), or NULL
    const WideMaps* maps;     // tensor maps of the layer (row-stationary phases, batches above 16 rows), or NULL
    uint32_t* ready;          // fused kernel, row-stationary form: per-group count of finished phase-1 units (x CW warps), or NULL
};

// Per-layer weights as the fused stack kernel reads them (device array, one entry per layer).
struct MegaLayer {
    const __nv_bfloat16* router_w;
    const float* logit_bias;
    const __nv_bfloat16* per_expert_scale;
    const float* correction_bias;
    const __nv_bfloat16* norm_w;
    const uint8_t* pool;
    uint64_t slot_stride;
    const int16_t* slot_of;
    const uint8_t* shared_blob;
    mfb_expert_offsets routed_off, shared_off;
    const WideMaps* maps;     // device pointer, or NULL when the shape has no row-stationary form
};

struct MegaParams {
    const MegaLayer* layers;
    uint32_t n_layers;
    uint32_t d, f, num_experts, top_k, bits, shared_bits, scale_dtype, activation;
    int router_mode, x_dtype;
    float limit, route_scale, eps;
    void* hidden;             // [n_tokens, d] (layer_stride == 0: the residual stream is carried through the layers)
    uint64_t layer_stride;    // elements between the rows of consecutive layers, or 0
    uint32_t n_tokens;
    void* xn;                 // scratch, all device memory owned by the handle
    __half* xp;
    __half* xp2;
    float* logits;
    uint32_t* idx;
    uint16_t* route_w;
    __half* actp;
    float* partial;
    uint32_t* bar_counter;    // [2]: arrivals, abort word (zeroed before every launch)
    uint32_t* ready;          // [2][MEGA_READY_WORDS] finished phase-1 units per expert group, by layer parity (zeroed before
                              // every launch and by the kernel one layer ahead), or NULL: a grid barrier between the FFN phases
    uint32_t* abort;
    uint32_t* status;
    int wide;                 // every layer carries tensor maps: batches above 16 rows run the row-stationary phases
    uint64_t* trace;          // optional [n_layers][8] global-timer stamps of the phase boundaries (CTA 0), followed by
                              // [17][8] cycle counters (per warp of CTA 0: phase-1 wait, phase-1 compute, phase-2 wait, phase-2 compute)
};

constexpr uint32_t MEGA_READY_WORDS = MFB_MAX_EXPERTS + 1;
constexpr uint32_t MEGA_BAR_WORDS = 2 + 2 * MEGA_READY_WORDS;   // what the handle allocates behind bar_counter
constexpr size_t FAST_SMEM_LIMIT = 220 * 1024;   // dynamic shared memory the fast kernels may ask for (static use on top)
constexpr uint32_t FAST_MAX_TOKENS = 64;   // phase 2 keeps (token, slot) x 16 partial rows in shared memory

__host__ __device__ uint32_t perm_pos(uint32_t e, uint32_t bits);
bool fast_supported(const mfb_moe_config& c);
// Shapes the row-stationary phases handle: 4-bit codes throughout, d a multiple of 1024, f = 512 or a multiple of 1024.
bool wide_supported(const mfb_moe_config& c);
// Fills the eighteen tensor maps of one layer (host memory; the caller copies them to the device).
int32_t wide_encode_maps(const mfb_moe_config& c, const mfb_layer_weights& w, WideMaps* out);
size_t fast_smem1(const mfb_moe_config& c);
size_t fast_smem2(const mfb_moe_config& c, uint32_t n_tokens);
cudaError_t launch_fast_prep(cudaStream_t s, const void* h, int dtype, const __nv_bfloat16* w, uint32_t n_tokens, uint32_t d,
                             float eps, bool do_norm, void* xn, __half* xp, uint32_t bits, __half* xp2, uint32_t bits2);
cudaError_t launch_fast_ffn(cudaStream_t s, const FastParams& P, const mfb_moe_config& c, int sm_count, uint32_t max_groups);
size_t fast_smem_stack(const mfb_moe_config& c, uint32_t n_tokens, bool wide_form);
bool stack_mega_fits(const mfb_moe_config& c, int sm_count, size_t smem);
cudaError_t fast_init();
// One CTA waits on an mbarrier nobody arrives at and reports STATUS_MBAR_TIMEOUT after limit_cycles SM cycles.
cudaError_t launch_wait_selftest(cudaStream_t s, uint32_t* status, long long limit_cycles);
// All layers of a decode step in one cooperative launch (norm, router, sort, both FFN phases, combine).
cudaError_t launch_stack_mega(cudaStream_t s, const MegaParams& M, const mfb_moe_config& c, int sm_count);
// select + sort of a small batch in one CTA (router.cu)
cudaError_t launch_route_small(cudaStream_t s, const float* logits, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k,
                               int mode, const __nv_bfloat16* per_expert_scale, const float* correction_bias,
                               float route_scale, int append_shared, uint32_t* out_idx, uint16_t* out_w,
                               mfb_pair* sorted, mfb_group* groups, uint32_t* n_groups);

}  // namespace mfb
