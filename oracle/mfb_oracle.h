/*
 * mfb_oracle.h — CPU restatement of the reference's MoE feed-forward arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or calls
 * this code; it exists so that tests, the smoke check and the benchmark's CPU
 * baseline leg can compare the CUDA path against an independent statement of the
 * same mathematics.
 *
 * Parity status: the reference (Swift + Metal) cannot be compiled or run on this
 * platform and its tests hold no golden output vectors for this path, so output
 * parity is pinned only through the structural fixtures restated under
 * tests/golden (sort order, tie-breaks, nibble order, struct layouts) and through
 * the semantics of the reference files cited beside each function.  The 2-bit
 * path has no CPU reference in the upstream tests at all: "parity unpinned" for
 * 2-bit beyond self-consistency.
 *
 * Every function cites the reference file:line it follows (paths are relative to
 * the reference project root).
 */
#ifndef MFB_ORACLE_H
#define MFB_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* dtype tags shared with include/mfb200.h */
#define MFBO_DT_BF16 0
#define MFBO_DT_F16 1
#define MFBO_DT_F32 2

#define MFBO_ACT_SILU 0
#define MFBO_ACT_GELU_TANH 1

/* Nine sub-tensor byte offsets inside one expert blob (Sources/Mference/Kernels/MoE/MoE.swift:4-15). */
typedef struct mfbo_expert_offsets {
    uint32_t gate_w, gate_s, gate_b;
    uint32_t up_w, up_s, up_b;
    uint32_t down_w, down_s, down_b;
} mfbo_expert_offsets;

/* 16-byte token/expert pair (Sources/Mference/Kernels/Prefill/MoE/PrefillRouter.swift:4-28). */
typedef struct mfbo_pair {
    uint32_t token, expert, rank, weight_bits;
} mfbo_pair;

typedef struct mfbo_group {
    uint32_t expert, pair_start, pair_count;
} mfbo_group;

typedef struct mfbo_tile {
    uint32_t group_start, group_count, pair_start, pair_count;
} mfbo_tile;

/* ---- PRNG (Sources/MferenceValidation/Support/PRNG/SplitMix64.swift:4-24, SeedTree.swift:12-19) ---- */
uint64_t mfbo_splitmix_at(uint64_t seed, uint64_t index);              /* index-th draw, 0-based */
uint64_t mfbo_seed_for_label(uint64_t root, const char* label);        /* root ^ FNV-1a(label) */
float mfbo_uniform_at(uint64_t seed, uint64_t index, float lo, float hi); /* SplitMix64.uniform */
void mfbo_fill_raw(uint64_t seed, uint64_t first_draw, uint64_t n_draws, uint64_t* out);
void mfbo_fill_normal(uint64_t seed, uint64_t first_value, uint64_t n, double mean, double std,
                      int absolute, int dtype, void* out);

/* ---- synthetic layer weights: one labelled stream per tensor, root seed chosen by the caller.
 * Labels: "L{layer}.e{expert}.{gate|up|down}.{q|s|b}", "L{layer}.shared.…", "L{layer}.router".
 * Codes are the raw little-endian draw stream (uniform nibbles / crumbs), scales are |N(0,0.02)| and biases
 * N(0,0.01) rounded to the 16-bit scale dtype, router weights are N(0,0.02) in bf16. ---- */
void mfbo_make_offsets(int bits, uint32_t d, uint32_t f, mfbo_expert_offsets* off, uint64_t* blob_bytes);
/* the same with gate_proj scales and biases per `gate_group` elements (32 or 64) */
void mfbo_make_offsets_gate(int bits, uint32_t d, uint32_t f, uint32_t gate_group, mfbo_expert_offsets* off, uint64_t* blob_bytes);
void mfbo_synth_expert(uint64_t root, uint32_t layer, int32_t expert, int bits, int scale_dtype, uint32_t d,
                       uint32_t f, uint8_t* blob);
void mfbo_synth_expert_gate(uint64_t root, uint32_t layer, int32_t expert, int bits, int scale_dtype, uint32_t d,
                            uint32_t f, uint32_t gate_group, uint8_t* blob);
void mfbo_synth_router(uint64_t root, uint32_t layer, uint32_t num_experts, uint32_t d, uint16_t* w_bf16);

/* ---- scalar conversions (Sources/Mference/Infrastructure/ModelIO/Quantization.swift:16-28) ---- */
uint16_t mfbo_f32_to_bf16(float x);
float mfbo_bf16_to_f32(uint16_t b);
uint16_t mfbo_f32_to_f16(float x);
float mfbo_f16_to_f32(uint16_t h);

/* ---- affine group quantisation (Quantization.swift:32-119; 2-bit Sources/Mference/Metal/MoE/moe.metal:902-960) ---- */
void mfbo_dequant_rows(const uint8_t* codes, const uint16_t* scales, const uint16_t* biases, int bits,
                       int group_size, int scale_dtype, uint32_t rows, uint32_t cols, float* out);
void mfbo_quantize_int4_row(const float* row, uint32_t n, uint8_t* packed, uint16_t* scales_bf16,
                            uint16_t* biases_bf16);

/* ---- router (moe.metal:162-185 gate GEMV; 190-240 top-k softmax; 737-793 sqrt-softplus) ---- */
void mfbo_router_logits(const uint16_t* x, int x_dtype, uint32_t ldx, uint32_t n_tokens, const uint16_t* w_bf16,
                        uint32_t num_experts, uint32_t d, const float* logit_bias, int exact_f64, float* logits);
void mfbo_topk_softmax(const float* logits, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k,
                       const uint16_t* per_expert_scale_bf16, uint32_t* out_idx, uint16_t* out_w_f16);
void mfbo_topk_sqrtsoftplus(const float* logits, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k,
                            const float* correction_bias, float route_scale, uint32_t* out_idx,
                            uint16_t* out_w_f16);
/* minimum gap between consecutive selection scores among the best top_k+1, per token (test aid) */
void mfbo_topk_margin(const float* scores, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k, float* margin);

/* ---- expert FFN and the layer (Sources/MferenceValidation/Support/Reference/MoE/Moe.swift:31-88) ---- */
typedef struct mfbo_layer {
    uint32_t d, f, num_experts, top_k;
    uint32_t bits, shared_bits, group_size, scale_dtype;
    uint32_t activation;
    float swiglu_limit;
    const uint8_t* pool;        /* expert e at pool + e * expert_stride */
    uint64_t expert_stride;
    const uint8_t* shared_blob; /* may be NULL */
    mfbo_expert_offsets routed_off, shared_off;
    uint32_t gate_group_size;   /* routed experts' gate_proj: 0 = group_size, or 32 (DeepSeek V4: ModelExpertIO.swift:118-135) */
} mfbo_layer;

void mfbo_expert_ffn(const uint8_t* blob, const mfbo_expert_offsets* off, int bits, int group_size,
                     int scale_dtype, uint32_t d, uint32_t f, int activation, float swiglu_limit,
                     const float* x, double* out);
/* y[t,:] = residual[t,:] + shared(x_t) + sum_r w[t,r] * ffn_{idx[t,r]}(x_t), rank order, double accumulation */
void mfbo_moe_layer(const mfbo_layer* L, const uint16_t* x, int x_dtype, uint32_t ldx, uint32_t n_tokens,
                    const uint32_t* idx, const uint16_t* w_f16, const float* residual, float* y);
/* per-pair partial rows: partial[p,:] = ffn_{pairs[p].expert}(x_{pairs[p].token}) */
void mfbo_pair_partials(const mfbo_layer* L, const uint16_t* x, int x_dtype, uint32_t ldx, const mfbo_pair* pairs,
                        uint32_t n_pairs, float* partial);

/* ---- prefill grouping (Sources/Mference/Kernels/Prefill/MoE/PrefillMoEGrouping.swift:90-192) ---- */
#define MFBO_GROUP_OK 0
#define MFBO_GROUP_INVALID_QUERY_COUNT 1
#define MFBO_GROUP_INVALID_TOP_K 2
#define MFBO_GROUP_INVALID_NUM_EXPERTS 3
#define MFBO_GROUP_INVALID_TILE_EXPERT_COUNT 4
#define MFBO_GROUP_PAIR_COUNT_MISMATCH 5
#define MFBO_GROUP_TOKEN_OUT_OF_RANGE 6
#define MFBO_GROUP_RANK_OUT_OF_RANGE 7
#define MFBO_GROUP_EXPERT_OUT_OF_RANGE 8
#define MFBO_GROUP_DUPLICATE_TOKEN_RANK 9
#define MFBO_GROUP_SORT_KEY_COUNT_MISMATCH 10
int mfbo_group_pairs(const mfbo_pair* pairs, int64_t n_pairs, int64_t query_count, int64_t top_k,
                     int64_t num_experts, int64_t tile_expert_count, const uint64_t* sort_keys,
                     int64_t n_sort_keys, mfbo_pair* sorted, uint32_t* offsets, uint32_t* counts,
                     mfbo_group* groups, uint32_t* n_groups, mfbo_tile* tiles, uint32_t* n_tiles,
                     uint32_t* err_a, uint32_t* err_b);

/* ---- weighted reduce (Sources/Mference/Metal/Prefill/prefill.metal:631-652) ---- */
void mfbo_reduce_token_major(const float* partial, const uint16_t* w_f16, uint32_t n_tokens, uint32_t top_k,
                             uint32_t d, float* h2);

/* ---- glue (Sources/Mference/Metal/Primitives/rmsnorm.metal:32-93) ---- */
void mfbo_rmsnorm(const float* x, const uint16_t* w_bf16, uint32_t n_rows, uint32_t d, float eps, float* out);

/* ---- timed CPU baseline: the reference's scalar decode arithmetic in fp32 with the affine factoring
 * s*sum(q*x) + b*sum(x) per group (moe.metal:349-404, 408-529), threaded over rows with OpenMP ---- */
void mfbo_ref_moe_layer_f32(const mfbo_layer* L, const float* x, uint32_t n_tokens, const uint32_t* idx,
                            const uint16_t* w_f16, const float* residual, float* y);
/* quantised gate / projections (hash-routed weights, INT8 gate GEMV in the reference kernels' order, INT4 GEMV in fp32) */
void mfbo_hash_weights(const float* logits, const uint32_t* idx, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k,
                       float route_scale, uint16_t* out_w_f16);
void mfbo_gemv_int8(const uint8_t* W, const uint16_t* s_bf16, const uint16_t* b_bf16, const uint16_t* x, int x_dtype,
                    uint32_t ldx, uint32_t n_tokens, const uint16_t* effective_scale_bf16, uint32_t M, uint32_t N, float* y);
void mfbo_gemv_int4(const uint8_t* W, const uint16_t* scales, const uint16_t* biases, int scale_dtype, const uint16_t* x,
                    int x_dtype, uint32_t ldx, uint32_t n_tokens, uint32_t M, uint32_t N, float* y);
int mfbo_num_threads(void);
void mfbo_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
