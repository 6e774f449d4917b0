/*
 * mfb200.h — C ABI of the B200-native MoE feed-forward path.
 *
 * The reference engine (Swift + Metal) has no plugin or FFI surface; its MoE path sits behind Swift
 * classes whose methods encode GPU work into a caller-owned command buffer.  Each entry point below
 * replaces one of those encode methods (cited per function, paths relative to the reference project
 * root).  Conventions, all taken from that surface:
 *   - every buffer is caller-owned device memory passed as a plain pointer (the reference passes
 *     MTLBuffer + byte offset); kernels never allocate.  A handle owns only its scratch arena;
 *   - work is enqueued on the caller's stream (`stream` is a cudaStream_t passed as void*; the
 *     reference's MTLCommandBuffer) and is asynchronous; nothing here synchronises the device;
 *   - every call returns an int32 status, 0 = MFB_OK; nothing throws or aborts.  The text of the last
 *     failure on the calling thread is available from mfb_last_error();
 *   - handles are thread-compatible, not thread-safe, like the reference's wrappers;
 *   - there is no CPU fallback and no backend dispatch behind this ABI: without a CUDA device every
 *     compute call fails with MFB_ERR_CUDA.
 */
#ifndef MFB200_H
#define MFB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MFB_OK 0
#define MFB_ERR_INVALID_ARGUMENT 1   /* contract violation (the reference traps with precondition) */
#define MFB_ERR_UNSUPPORTED_SHAPE 2  /* shape outside what the kernels handle */
#define MFB_ERR_CUDA 3               /* CUDA runtime error; text in mfb_last_error() */
#define MFB_ERR_CAPACITY 4           /* more tokens than the handle's scratch arena was created for */
#define MFB_ERR_ALLOC 5
#define MFB_ERR_DEVICE_STATUS 6      /* a kernel reported a bounded wait that ran out or a failed self-check */
#define MFB_ERR_IO 7                 /* staging source too short / unreadable (StreamerError.sizeMismatch) */
#define MFB_ERR_NO_SLOT 8            /* expert cache cannot place the requested misses */
/* grouping validation, one code per PrefillMoEGroupingError case
 * (Sources/Mference/Kernels/Prefill/MoE/PrefillMoEGrouping.swift:52-63) */
#define MFB_ERR_GROUP_INVALID_QUERY_COUNT 101
#define MFB_ERR_GROUP_INVALID_TOP_K 102
#define MFB_ERR_GROUP_INVALID_NUM_EXPERTS 103
#define MFB_ERR_GROUP_INVALID_TILE_EXPERT_COUNT 104
#define MFB_ERR_GROUP_PAIR_COUNT_MISMATCH 105
#define MFB_ERR_GROUP_TOKEN_OUT_OF_RANGE 106
#define MFB_ERR_GROUP_RANK_OUT_OF_RANGE 107
#define MFB_ERR_GROUP_EXPERT_OUT_OF_RANGE 108
#define MFB_ERR_GROUP_DUPLICATE_TOKEN_RANK 109
#define MFB_ERR_GROUP_SORT_KEY_COUNT_MISMATCH 110

#define MFB_DT_BF16 0
#define MFB_DT_F16 1
#define MFB_DT_F32 2

#define MFB_ACT_SILU 0       /* Qwen SwiGLU (moe.metal function constant 4) */
#define MFB_ACT_GELU_TANH 1  /* Gemma gelu_pytorch_tanh */

#define MFB_ROUTER_SOFTMAX_TOPK 0   /* Sources/Mference/Metal/MoE/moe.metal:190-345 */
#define MFB_ROUTER_SQRTSOFTPLUS 1   /* moe.metal:737-845 */

#define MFB_MAX_TOP_K 16
#define MFB_MAX_EXPERTS 512

/* Nine sub-tensor byte offsets inside one expert blob, common to every expert of a layer.
 * Replaces MoEExpertOffsets (Sources/Mference/Kernels/MoE/MoE.swift:4-29); same field order, 36 bytes.
 * This implementation additionally requires every offset to be a multiple of 16 bytes. */
typedef struct mfb_expert_offsets {
    uint32_t gate_w, gate_s, gate_b;
    uint32_t up_w, up_s, up_b;
    uint32_t down_w, down_s, down_b;
} mfb_expert_offsets;

/* One (token, expert, rank, weight) route.  Replaces PrefillTokenExpertPair
 * (Sources/Mference/Kernels/Prefill/MoE/PrefillRouter.swift:4-28); 16 bytes, the fp16 weight bits sit in
 * the low half of weight_bits. */
typedef struct mfb_pair {
    uint32_t token, expert, rank, weight_bits;
} mfb_pair;

/* PrefillMoEGroup / PrefillMoETile (PrefillMoEGrouping.swift:3-29). */
typedef struct mfb_group {
    uint32_t expert, pair_start, pair_count;
} mfb_group;
typedef struct mfb_tile {
    uint32_t group_start, group_count, pair_start, pair_count;
} mfb_tile;

/* Shape and numerics of one MoE layer family.  Plays the part of MoE.init's specialisation arguments
 * (MoE.swift:65-70) and of the Metal function constants 0-5 / 40-43 (moe.metal:9-25). */
typedef struct mfb_moe_config {
    uint32_t d;             /* hidden size, multiple of 64 */
    uint32_t f;             /* expert intermediate size, multiple of 64 */
    uint32_t num_experts;   /* <= MFB_MAX_EXPERTS */
    uint32_t top_k;         /* <= MFB_MAX_TOP_K */
    uint32_t bits;          /* routed expert code width: 4 or 2 */
    uint32_t shared_bits;   /* shared expert code width: 4, 2 or 8 (SharedExpertInt8, Sources/Mference/Kernels/MoE/
                               SharedExpertInt8.swift: generic kernels only); 0 = the layer has no shared expert */
    uint32_t group_size;    /* 64 */
    uint32_t scale_dtype;   /* MFB_DT_F16 (MLX files) or MFB_DT_BF16 (reference .gturbo files) */
    uint32_t x_dtype;       /* activation dtype in and out: MFB_DT_BF16 or MFB_DT_F16 */
    uint32_t activation;    /* MFB_ACT_* */
    uint32_t router_mode;   /* MFB_ROUTER_* */
    float swiglu_limit;     /* > 0: clamp gate <= limit, up in [-limit, limit] before the activation */
    float route_scale;      /* sqrt-softplus mode only */
    float rms_eps;          /* 1e-6 in the reference (RealForwardRunner.swift:2583) */
    uint32_t max_tokens;    /* scratch arena capacity in token rows per call */
    uint32_t flags;         /* MFB_FLAG_* */
    uint32_t max_layers;    /* most layers one mfb_moe_stack / mfb_moe_stack_rows call may be given, and the number of
                               distinct layers whose tensor maps the handle keeps; 0 = 64 */
} mfb_moe_config;

#define MFB_FLAG_PREFILL_TENSOR_CORE 1u /* allocate the arena of the tcgen05 grouped-GEMM path */

/* Device-resident weights of one layer. */
typedef struct mfb_layer_weights {
    const void* router_w;          /* bf16 [num_experts, d] */
    const float* logit_bias;       /* optional f32 [num_experts], added to the logits */
    const void* per_expert_scale;  /* optional bf16 [num_experts] (softmax mode) */
    const float* correction_bias;  /* optional f32 [num_experts] (sqrt-softplus mode, selection only) */
    const void* norm_w;            /* optional bf16 [d]; NULL = weight 1 */
    const uint8_t* pool;           /* slab of expert slots */
    uint64_t slot_stride;          /* bytes between slots */
    const int16_t* slot_of;        /* optional device table expert -> slot (-1 = not resident); NULL = identity */
    const uint8_t* shared_blob;    /* shared expert blob, or NULL */
    mfb_expert_offsets routed_off;
    mfb_expert_offsets shared_off;
    /* INT8 affine group-64 gate, as Qwen 3.6 files carry it (Sources/Mference/Metal/MoE/moe.metal:102-157): when
     * router_scales is non-NULL, router_w holds unsigned byte codes [num_experts, d] and router_scales / router_biases
     * bf16 [num_experts, d/64]; router_effective_scale (bf16 [d], may be NULL = 1) multiplies the activations first. */
    const void* router_scales;
    const void* router_biases;
    const void* router_effective_scale;
    /* Qwen shared-expert scalar gate (RealForwardRunner.swift:2925-2941, prefill.metal:37-80): when shared_gate_w is
     * non-NULL (byte codes [d], bf16 scales / biases [d/64]) the shared expert's output row of every token is multiplied
     * by sigmoid(fp16(g . x)) before the combine. */
    const void* shared_gate_w;
    const void* shared_gate_s;
    const void* shared_gate_b;
    /* Scale group of the routed experts' gate_proj: 0 or 64 = the handle's group size; 32 = DeepSeek V4's conversion on
     * most layers (routedGateGroupSize, Sources/Mference/Runtime/Inference/ModelExpertIO.swift:118-135; kernels
     * moe.metal:962-1062): gate_s / gate_b then hold d/32 entries per row.  Such a layer runs the generic kernels. */
    uint32_t gate_group_size;
} mfb_layer_weights;

typedef struct mfb_moe mfb_moe;

const char* mfb_last_error(void);
int32_t mfb_version(void);
/* Number of GPU kernels this library has launched in the calling process so far (monotonic). */
uint64_t mfb_launch_count(void);
/* Fills the offsets of the canonical blob layout (gate W,S,B · up W,S,B · down W,S,B, row-major). */
int32_t mfb_expert_layout(uint32_t bits, uint32_t d, uint32_t f, mfb_expert_offsets* off, uint64_t* blob_bytes);
/* The same with gate_proj's scales and biases per `gate_group_size` (32 or 64) elements. */
int32_t mfb_expert_layout_gate(uint32_t bits, uint32_t d, uint32_t f, uint32_t gate_group_size, mfb_expert_offsets* off,
                               uint64_t* blob_bytes);

/* MoE.init / deinit (MoE.swift:65-151): builds the handle and its scratch arena. */
int32_t mfb_moe_create(const mfb_moe_config* cfg, mfb_moe** out);
int32_t mfb_moe_destroy(mfb_moe* moe);
/* on == 1: run every call of this handle through the generic kernels (any supported shape, any slot subset)
 * instead of the shape-specialised fast kernels; the two agree within the documented tolerance.  Plays the part of
 * the reference's generic vs. specialised pipeline states (MoE.swift:77-135).
 * on == 2: keep the fast kernels but launch a stack layer by layer and phase by phase instead of as one fused
 * cooperative kernel (same results bit for bit; for profiling one phase alone).  on == 0: default selection. */
int32_t mfb_moe_set_generic(mfb_moe* moe, int32_t on);
/* Phase tracing of the fused stack kernel (the reference's MFERENCE_PHASES counters,
 * Sources/Mference/Runtime/Inference/RealForwardRunner.swift:395-398, 5478-5529): while a device buffer of
 * (n_layers + 17) x 8 uint64 is attached, mfb_moe_stack / mfb_moe_stack_rows record in its first n_layers rows the
 * GPU global timer (ns) at the eight phase boundaries of every layer - norm, logits, select, sort, phase 1, barrier,
 * phase 2, end - and in the 17 rows behind them SM-cycle counters of CTA 0: one row per warp (wait and compute cycles
 * of the two FFN phases), and in the last row the SM clock and the global timer at the start and end of the launch
 * (cycles per ns).  The caller zeroes the buffer; NULL detaches. */
int32_t mfb_moe_set_trace(mfb_moe* moe, uint64_t* device_stamps);
/* Reads and clears the device status word that kernels set when a bounded wait runs out. Synchronises `stream`. */
int32_t mfb_moe_device_status(mfb_moe* moe, void* stream, uint32_t* status);

/* Device pointer to the handle's fp32 down-projection rows [max_tokens, top_k + 1, d] (slot top_k = shared expert)
 * as the last mfb_moe_experts / mfb_moe_decode / mfb_moe_layer / mfb_moe_stack call left them: what the reference's
 * phase-2 kernels hold before the weighted reduce (Sources/Mference/Metal/MoE/moe.metal:349-404).  Lets a caller
 * (and the parity tests) look at the unrounded partial sums.  Owned by the handle. */
int32_t mfb_moe_partial_rows(mfb_moe* moe, const float** rows);
/* Self-test of the bounded waits (no counterpart in the reference): launches one CTA that waits on a barrier nothing
 * arrives at; after limit_cycles SM cycles (1 .. 20,000,000) the wait gives up, the kernel sets the device status
 * word and returns.  mfb_moe_device_status then reports MFB_ERR_DEVICE_STATUS once, and the handle stays usable. */
int32_t mfb_moe_selftest_wait(mfb_moe* moe, void* stream, uint64_t limit_cycles);

/* ---- router -------------------------------------------------------------------------------------------- */

/* Gate GEMV over an unquantised bf16 gate: logits[t,e] = sum_i w[e,i] * x[t,i] (+ bias[e]).
 * Replaces router_gemv_bf16_r4 as driven by MoEDeepseekV4.encodeRouterGemv
 * (Sources/Mference/Kernels/MoE/MoEDeepseekV4.swift:153-173; kernel moe.metal:162-185). */
int32_t mfb_router_logits(mfb_moe* moe, void* stream, const void* x, uint32_t ldx, uint32_t n_tokens,
                          const void* router_w, const float* logit_bias, float* logits);
/* Top-k select + routing weights for n_tokens rows of logits.  Ties go to the lower expert index.
 * Replaces router_topk_select_k8(_par) / router_topk_select_sqrtsoftplus_k6(_par) (moe.metal:190-345,
 * 737-845) and the selection tail of prefill_router_gemma4_block (Sources/Mference/Metal/Prefill/prefill.metal:586-628). */
int32_t mfb_router_select(mfb_moe* moe, void* stream, const float* logits, uint32_t n_tokens,
                          const void* per_expert_scale, const float* correction_bias, uint32_t* out_idx,
                          uint16_t* out_w);
/* Both steps.  Replaces MoE.encodeRouterGemma4 (MoE.swift:153-203) for one row and
 * PrefillRouter.encodeGemma4Block (PrefillRouter.swift:37-89) for a block of rows. */
int32_t mfb_router_topk(mfb_moe* moe, void* stream, const void* x, uint32_t ldx, uint32_t n_tokens,
                        const mfb_layer_weights* w, uint32_t* out_idx, uint16_t* out_w);
/* Expert id -> slot byte offset through the device-resident slot table, plus an all-hit flag per token row.
 * Replaces MoE.encodeSlotLookup (MoE.swift:302-330; kernel router_slot_lookup_k8, moe.metal:594-617). */
int32_t mfb_slot_lookup(mfb_moe* moe, void* stream, const uint32_t* idx, uint32_t n_tokens,
                        const int16_t* slot_of, uint64_t slot_stride, uint64_t* out_offsets, uint32_t* out_all_hit);

/* Router top-k without a handle and without any allocation (no counterpart in the reference, whose wrappers are
 * handed a pre-allocated logits buffer by their caller, MoE.swift:136-150): same kernels and the same results, bit
 * for bit, as mfb_router_topk, but the fp32 logits scratch is a fixed array inside the library's device image, so
 * that a host which may not allocate device memory - its whole budget lives in its own pool, it runs under a
 * memory cap, or it is inside a region where allocation calls are not allowed - can still route a decode batch.
 *  - Limit: n_tokens <= MFB_STATIC_ROUTER_MAX_TOKENS and num_experts <= MFB_MAX_EXPERTS; more rows return
 *    MFB_ERR_CAPACITY (use mfb_router_topk with a handle for those).
 *  - The first call on each device (with that device current) looks up the scratch array's device address; make
 *    that first call before starting a stream capture.  Later calls only launch the two kernels.
 *  - The scratch is one array per device shared by all callers: two calls that may overlap in time (different
 *    streams, different threads) race on it.  Serialise them on one stream or with events.
 *  - Nothing needs zeroing between calls: each call overwrites the part of the scratch it reads.
 * x: [n_tokens, ldx] activations of x_dtype (MFB_DT_BF16 / MFB_DT_F16); router_w: bf16 [num_experts, d]; the other
 * arguments have the meaning of the same-named fields of mfb_moe_config and mfb_layer_weights. */
#define MFB_STATIC_ROUTER_MAX_TOKENS 64
int32_t mfb_router_topk_static(void* stream, const void* x, uint32_t x_dtype, uint32_t ldx, uint32_t n_tokens, uint32_t d,
                               const void* router_w, const float* logit_bias, uint32_t num_experts, uint32_t top_k,
                               uint32_t router_mode, const void* per_expert_scale, const float* correction_bias,
                               float route_scale, uint32_t* out_idx, uint16_t* out_w);

/* Routing weights of hash-routed layers: the expert indices are given (a frozen token-id table in the reference), the
 * weights are sqrt(softplus(logit)) of exactly those experts, normalised over them in rank order and scaled.
 * Replaces router_hash_weights_k6(_par) (moe.metal:852-896) for any top_k <= MFB_MAX_TOP_K. */
int32_t mfb_router_hash_weights(void* stream, const float* logits, const uint32_t* idx, uint32_t n_tokens, uint32_t num_experts,
                                uint32_t top_k, float route_scale, uint16_t* out_w);
/* INT8 affine group-64 GEMV y[t, r] = sum_i (q[r,i] * s[r,i/64] + b[r,i/64]) * x[t,i] in the summation order of
 * router_gemv_gemma4_r4 (moe.metal:102-157; host MoE.encodeRouterGemma4, MoE.swift:153-188): the Qwen router's logits
 * (M = num_experts) and the shared-expert scalar gate (M = 1).  y is f32 [n_tokens, M]. */
int32_t mfb_gemv_int8(void* stream, const uint8_t* W, const void* scales_bf16, const void* biases_bf16, const void* x,
                      uint32_t x_dtype, uint32_t ldx, uint32_t n_tokens, const void* effective_scale_bf16, uint32_t M,
                      uint32_t N, float* y);
/* INT4 affine group-64 GEMV of a resident projection, up to 8 activation rows per weight read: y[t, r] f32 [n_tokens, M].
 * Replaces DequantInt4GEMV.encode and its multi-row form (Sources/Mference/Kernels/Quant/DequantInt4GEMV.swift:1-104;
 * kernels Sources/Mference/Metal/Quant/dequant_int4.metal:248-288, 343-446).  W: [M, N/2] bytes, low nibble = even
 * element; scales / biases 16-bit [M, N/64] of scale_dtype. */
int32_t mfb_gemv_int4(void* stream, const uint8_t* W, const void* scales, const void* biases, uint32_t scale_dtype,
                      const void* x, uint32_t x_dtype, uint32_t ldx, uint32_t n_tokens, uint32_t M, uint32_t N, float* y);

/* ---- decode -------------------------------------------------------------------------------------------- */

/* Routed + shared expert FFN with the weighted combine for n_tokens rows:
 *   y[t] = dtype( residual[t] + shared(x[t]) + sum_r w[t,r] * ffn_{idx[t,r]}(x[t]) ), fp32, rank order.
 * Each distinct expert's weights are read once for all rows routed to it.  Replaces
 * MoE.encodeRoutedPersistentPhase1U16Load + encodeRoutedPersistentPhase2Reduce (MoE.swift:220-253, 400-440),
 * the slot-map form MoE.encodeSlotMapGuardedFFN (MoE.swift:332-398) when w->slot_of is given, and
 * SharedExpertRuntime.encode (Sources/Mference/Kernels/MoE/SharedExpertInt4.swift:193-222).
 * residual may be NULL; y may alias residual. */
int32_t mfb_moe_decode(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                       uint32_t n_tokens, const uint32_t* idx, const uint16_t* route_w, const void* residual,
                       void* y);
/* The two halves of mfb_moe_decode, for callers that run cache-hit experts first and the misses after their
 * fill.  mfb_moe_experts computes the down-projection rows of the listed rank slots (host array; NULL = all
 * top_k slots) and, when with_shared != 0, of the shared expert, into the handle's arena; mfb_moe_combine then
 * reduces every slot in rank order.  A hit/miss split gives bit-identical results to one full call.
 * Replaces MoE.encodeRoutedPersistentPhase1SubsetU16Load (MoE.swift:255-298) followed by
 * MoE.encodeRoutedPersistentPhase2Reduce (MoE.swift:400-440). */
int32_t mfb_moe_experts(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                        uint32_t n_tokens, const uint32_t* idx, const uint16_t* route_w,
                        const uint32_t* active_slots, uint32_t active_count, int32_t with_shared);
int32_t mfb_moe_combine(mfb_moe* moe, void* stream, uint32_t n_tokens, const uint16_t* route_w, int32_t with_shared,
                        const void* residual, void* y);
/* One whole layer on the residual stream: h_out = h_in + MoE(RMSNorm(h_in)), router included.
 * Mirrors the MoE section of RealForwardRunner.produceToken
 * (Sources/Mference/Runtime/Inference/RealForwardRunner.swift:2811-3253) with every expert resident. */
int32_t mfb_moe_layer(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* h_in, void* h_out,
                      uint32_t n_tokens);
/* n_layers of the above back to back (the per-layer loop RealForwardRunner.swift:2646). */
int32_t mfb_moe_stack(mfb_moe* moe, void* stream, const mfb_layer_weights* layers, uint32_t n_layers,
                      void* hidden, uint32_t n_tokens);

/* The same loop over separate row blocks: layer l reads and rewrites the n_tokens rows at rows + l * layer_stride
 * elements (layer_stride = 0 is mfb_moe_stack).  Layers still run strictly one after the other.  Serves callers
 * that interleave independent micro-batches through the layers. */
int32_t mfb_moe_stack_rows(mfb_moe* moe, void* stream, const mfb_layer_weights* layers, uint32_t n_layers,
                           void* rows, uint64_t layer_stride, uint32_t n_tokens);

/* ---- prefill / ragged batch ---------------------------------------------------------------------------- */

/* Device-side sort of the routing table by (expert, token, rank): sorted pairs, per-expert offsets
 * (0xFFFFFFFF = absent) and counts, the compacted group list and its length.  Same order as
 * PrefillMoEGrouping.groupTokenExpertPairs (PrefillMoEGrouping.swift:90-192) without sort keys.
 * All outputs are device pointers; out_groups holds up to num_experts entries. */
int32_t mfb_moe_group(mfb_moe* moe, void* stream, const uint32_t* idx, const uint16_t* route_w, uint32_t n_tokens,
                      mfb_pair* out_sorted, uint32_t* out_offsets, uint32_t* out_counts, mfb_group* out_groups,
                      uint32_t* out_n_groups);
/* Host-side grouping with the reference's validation, optional expert sort keys and tiles; plain host
 * arrays in and out.  Replaces PrefillMoEGrouping.groupTokenExpertPairs for callers that hold the table on
 * the host (RealForwardRunner.swift:2276-2297). err_a / err_b carry the offending values. */
int32_t mfb_moe_group_host(const mfb_pair* pairs, int64_t n_pairs, int64_t query_count, int64_t top_k,
                           int64_t num_experts, int64_t tile_expert_count, const uint64_t* expert_sort_keys,
                           int64_t n_sort_keys, mfb_pair* out_sorted, uint32_t* out_offsets, uint32_t* out_counts,
                           mfb_group* out_groups, uint32_t* out_n_groups, mfb_tile* out_tiles,
                           uint32_t* out_n_tiles, uint32_t* err_a, uint32_t* err_b);
/* Grouped routed FFN over sorted pairs ("gather-QMM"): partial[(token*top_k + rank), :] = ffn_expert(x[token]).
 * partial is f32 [n_tokens*top_k, d].  Replaces PrefillGroupedRoutedMoE.encodeStreamedBatched
 * (Sources/Mference/Kernels/Prefill/MoE/PrefillGroupedRoutedMoE.swift:391-466; kernels prefill.metal:748-820). */
int32_t mfb_moe_prefill_grouped(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                                uint32_t n_tokens, const mfb_pair* sorted, const mfb_group* groups,
                                const uint32_t* n_groups, float* partial);
/* The same grouped FFN with one destination address per result row instead of a dense array: the row of (token, rank)
 * is written to row_dest[token * top_k + rank] (device array of device-visible addresses, e.g. a peer GPU's buffer
 * mapped with CUDA IPC; a NULL entry drops the row).  Entries of `sorted` behind the last group are ignored.  Used by
 * the expert-parallel layer, whose results go straight to the home rank; tensor-core path only.  No counterpart in the
 * reference (single device); the per-row arithmetic is that of PrefillGroupedRoutedMoE.encodeStreamedBatched. */
int32_t mfb_moe_prefill_grouped_rows(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                                     uint32_t n_tokens, const mfb_pair* sorted, const mfb_group* groups,
                                     const uint32_t* n_groups, float* const* row_dest);
/* The Inkling batched expert application (inkling_prefill_expert_act + inkling_prefill_expert_down_accum,
 * Sources/Mference/Metal/Prefill/prefill.metal:654-746): the grouped expert FFN with gate and up rounded to fp16
 * before the activation and the product stored as fp16, accumulated expert by expert - ascending expert id, the order
 * the reference's host loop dispatches them - into an fp32 accumulator with fp32 pair weights:
 * acc[t,:] = fma(pair_weights[t*top_k + rank], down_row, acc[t,:]).  acc is f32 [n_tokens, d], read and written
 * (the caller zeroes it, or leaves the shared expert's contribution in it); routed experts only; generic kernels. */
int32_t mfb_moe_prefill_accumulate_f32(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                                       uint32_t n_tokens, const mfb_pair* sorted, const mfb_group* groups,
                                       const uint32_t* n_groups, const float* pair_weights, float* acc);
/* h2[t,:] = sum_r w[t,r] * partial[t,r,:] in rank order (+ residual).  Replaces
 * PrefillMoE.encodeReduceTokenMajor (Sources/Mference/Kernels/Prefill/MoE/PrefillMoE.swift:11-38). */
int32_t mfb_moe_reduce(mfb_moe* moe, void* stream, const float* partial, const uint16_t* route_w, uint32_t n_tokens,
                       const void* residual, void* y);
/* Whole prefill layer for a block of rows: h_out = h_in + MoE(RMSNorm(h_in)); router, sort, grouped FFN,
 * shared expert and reduce.  Mirrors RealForwardRunner.executePrefillChunk's MoE section
 * (RealForwardRunner.swift:2173-2498). */
int32_t mfb_moe_layer_prefill(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* h_in, void* h_out,
                              uint32_t n_tokens);

/* ---- expert-slot cache over an HBM-resident pool ------------------------------------------------------ */

/* Replaces PreadExpertStreamer (Sources/Mference/Infrastructure/Streaming/PreadExpertStreamer.swift:57-580): a slab of
 * `slot_count` slots in HBM, an expert -> slot table (int16, -1 = not resident) on the device for the FFN kernels
 * (mfb_layer_weights.pool / slot_stride / slot_of), and the same cache planning on the host.  One pool per layer.
 * The reference reads missing experts from SSD with pread; here they are copied from pinned host memory. */
typedef struct mfb_pool mfb_pool;
#define MFB_POOL_LFU 0u        /* least frequently used expert first, recency as tie break (the reference's default) */
#define MFB_POOL_LRU 1u
#define MFB_POOL_HOST_ONLY 1u  /* flag: planning bookkeeping only, no device memory */
int32_t mfb_pool_create(uint32_t num_experts, uint64_t slot_bytes, uint32_t slot_count, uint32_t policy, uint32_t flags,
                        mfb_pool** out);
int32_t mfb_pool_destroy(mfb_pool* pool);
/* Device slab, bytes between slots, device slot table: the three fields of mfb_layer_weights. */
int32_t mfb_pool_info(const mfb_pool* pool, void** slab, uint64_t* slot_stride, const int16_t** slot_of_device);
/* planExpertsCachedIfPossible (PreadExpertStreamer.swift:197-269): out_slots[i] = slot of experts[i], out_miss[i] = 1
 * if it has to be filled.  Hits keep their slots; `avoid_slots` (slots queued GPU work still reads) are never chosen
 * as victims; MFB_ERR_NO_SLOT when the misses cannot be placed (nothing is changed then). */
int32_t mfb_pool_plan(mfb_pool* pool, const int32_t* experts, uint32_t n, const int32_t* avoid_slots, uint32_t n_avoid,
                      int32_t* out_slots, uint8_t* out_miss, uint32_t* out_hits);
/* executeExpertCachePlan, first half (PreadExpertStreamer.swift:271-302): one asynchronous copy per miss from
 * host_blobs[i] (pinned host memory, blob_bytes each) into its slot, on `stream`; the device table is refreshed
 * first so that the victims read -1 before their bytes change.  MFB_ERR_IO for a missing or oversized source. */
int32_t mfb_pool_fill_async(mfb_pool* pool, void* stream, const int32_t* experts, const int32_t* slots, const uint8_t* miss,
                            uint32_t n, const void* const* host_blobs, uint64_t blob_bytes);
/* executeExpertCachePlan, second half: the filled slots become hits on the host and, in stream order, on the device. */
int32_t mfb_pool_publish(mfb_pool* pool, void* stream, const int32_t* experts, const int32_t* slots, const uint8_t* miss,
                         uint32_t n);
/* reserveSpeculativeSlots (PreadExpertStreamer.swift:344-372): slots for a speculative read of `experts` (already
 * filtered to the non-resident ones by the caller).  Slots that hold one of the predicted experts or that another
 * read is filling are never victims; `keep_evictable` evictable slots are left alone so that the real plan which
 * follows can always place its own misses.  Victims come in the normal eviction order, but no use count and no clock
 * is written.  Reserved slots are marked in flight and read -1 until the reservation is finished; out_n entries of
 * (out_experts, out_slots) are the reservation (possibly fewer than n, possibly none). */
int32_t mfb_pool_reserve_speculative(mfb_pool* pool, const int32_t* experts, uint32_t n, uint32_t keep_evictable,
                                     int32_t* out_experts, int32_t* out_slots, uint32_t* out_n);
/* beginAsyncFill, first step (PreadExpertStreamer.swift:452-462): marks a plan's miss slots in flight, so that plans made
 * while the eager fill runs keep away from them exactly as from speculative reads. */
int32_t mfb_pool_mark_in_flight(mfb_pool* pool, const int32_t* slots, uint32_t n);
/* executeSpeculativeReservation, second half (PreadExpertStreamer.swift:374-402) and the completion of beginAsyncFill:
 * slots whose read landed (loaded[i] != 0) become hits, slots whose read failed stay empty, every in-flight mark is
 * cleared; the device table follows in stream order (after the copies enqueued with mfb_pool_fill_async). */
int32_t mfb_pool_finish_speculative(mfb_pool* pool, void* stream, const int32_t* experts, const int32_t* slots,
                                    const uint8_t* loaded, uint32_t n);
/* noteAllHitUse (PreadExpertStreamer.swift:427-440): usage accounting when the device-side lookup found every expert. */
int32_t mfb_pool_note_all_hit(mfb_pool* pool, const int32_t* experts, uint32_t n);
/* Host mirror of the slot table (num_experts entries). */
int32_t mfb_pool_slot_of_host(mfb_pool* pool, int16_t* out);

/* ---- expert parallelism (2, 4 or 8 GPUs of one box; batched / prefill workloads) ------------------------- */

/* No counterpart in the reference (single device).  Experts are block-sharded, rank g owns experts
 * [g * E/G, (g+1) * E/G); tokens stay on their home rank.  Per layer the host layer (mference_b200/ep.py) calls
 * mfb_ep_plan + mfb_ep_pack, exchanges rows with an NCCL all-to-all, runs the grouped expert FFN on the received
 * rows, exchanges the fp32 result rows back and calls mfb_ep_combine, which is bit-identical to the single-GPU
 * weighted reduce (prefill_moe_reduce_token_major, prefill.metal:631-652: ranks ascending, fused multiply-add). */
/* Send order of the n_tokens * top_k pairs: by (destination rank, token, rank slot).  perm[pos] = token * top_k + slot;
 * inv = inverse of perm; counts[g] = pairs bound for rank g; local_expert[pos] = expert id relative to rank g's first. */
int32_t mfb_ep_plan(void* stream, const uint32_t* idx, uint32_t n_tokens, uint32_t top_k, uint32_t num_experts, uint32_t world,
                    uint32_t* perm, uint32_t* inv, int32_t* counts, int32_t* local_expert);
/* rows[pos, :] = x[perm[pos] / top_k, :] for 16-bit activations (the dispatch send buffer). */
int32_t mfb_ep_pack(void* stream, const void* x, uint32_t ldx, uint32_t d, const uint32_t* perm, uint32_t n_pairs,
                    uint32_t top_k, void* rows);
/* y[t,:] = dtype(residual[t,:] + shared_partial[t,:] + sum_k w[t,k] * recv[inv[t*top_k+k],:]); recv = the fp32 rows that
 * came back, in send order; shared_partial and residual may be NULL. */
int32_t mfb_ep_combine(void* stream, const float* recv, const uint32_t* inv, const uint16_t* route_w,
                       const float* shared_partial, const void* residual, void* y, uint32_t n_tokens, uint32_t top_k,
                       uint32_t d, uint32_t x_dtype);

/* One-sided exchange over peer memory (NVLink) instead of a collective library: every rank's receive and result
 * buffers are plain device allocations exported with CUDA IPC; dispatch stores the packed rows straight into the
 * destination ranks' buffers, the expert side's grouped FFN stores each result row straight into the home rank's
 * buffer (mfb_moe_prefill_grouped_rows), and arrival is signalled by epoch-valued flags that the other side polls
 * with a clock limit (a time-out sets the status word read by mfb_ep_status; nothing hangs).  No host
 * synchronisation and no collective on the data path.  max_pairs = tokens per rank * top_k, equal on all ranks.
 * Set-up: mfb_ep_create on every rank, mfb_ep_export (4 IPC handles of 64 bytes), all-gather the handles by any
 * means, mfb_ep_import (world * 4 handles, rank-major).  Per layer, on one stream:
 *   mfb_ep_dispatch   plan by destination, pack, peer stores, flags; inv[token * top_k + slot] = send position
 *   mfb_ep_receive    waits for every source; returns the received rows [world * max_pairs, d], their expert ids relative
 *                     to this rank's first expert (0xFFFFFFFF = no row) and the destination address of each result row
 *   ... mfb_moe_group + mfb_moe_prefill_grouped_rows on the received rows (top_k = 1) ...
 *   mfb_ep_return     tells every home rank that its results are in place
 *   mfb_ep_results    waits for every expert side; returns this rank's fp32 result rows in send order for mfb_ep_combine
 * One call sequence at a time per handle; the next dispatch may be enqueued right after mfb_ep_combine. */
typedef struct mfb_ep mfb_ep;
#define MFB_EP_HANDLE_BYTES 256   /* what mfb_ep_export writes: 4 IPC handles */
int32_t mfb_ep_create(uint32_t rank, uint32_t world, uint32_t d, uint32_t max_pairs, mfb_ep** out);
int32_t mfb_ep_destroy(mfb_ep* ep);
int32_t mfb_ep_export(mfb_ep* ep, void* handles);
int32_t mfb_ep_import(mfb_ep* ep, const void* all_handles);
int32_t mfb_ep_dispatch(mfb_ep* ep, void* stream, const void* x, uint32_t ldx, const uint32_t* idx, uint32_t n_tokens,
                        uint32_t top_k, uint32_t num_experts, uint32_t* inv);
int32_t mfb_ep_receive(mfb_ep* ep, void* stream, const void** rows, const uint32_t** row_expert, float* const** row_dest,
                       uint32_t* n_rows);
int32_t mfb_ep_return(mfb_ep* ep, void* stream);
int32_t mfb_ep_results(mfb_ep* ep, void* stream, const float** ret);
/* Reads and clears the exchange's status word (synchronises the stream); counts_host (optional, world entries) receives
 * the number of rows each source rank sent in the last call. */
int32_t mfb_ep_status(mfb_ep* ep, void* stream, uint32_t* status, int32_t* counts_host);

/* ---- glue ---------------------------------------------------------------------------------------------- */

/* out = dtype(x * rsqrt(mean(x^2) + eps) * w).  Replaces rmsnorm_bf16w
 * (Sources/Mference/Metal/Primitives/rmsnorm.metal:32-93). */
int32_t mfb_rmsnorm(mfb_moe* moe, void* stream, const void* x, const void* w_bf16, uint32_t n_rows, void* out);
/* out = dtype(a + b).  Replaces residual_add_fp16 (Sources/Mference/Metal/Primitives/utility.metal:83-92). */
int32_t mfb_residual_add(mfb_moe* moe, void* stream, const void* a, const void* b, uint64_t n, void* out);

/* ---- synthetic weights (benchmark and test support) ---------------------------------------------------- */

/* Fills device memory with the labelled SplitMix64 streams the benchmark configurations are defined on:
 * uniform codes, |N(0,0.02)| scales, N(0,0.01) biases, N(0,0.02) bf16 router rows, N(0,1) activations.
 * Stream labels follow Sources/MferenceValidation/Support/PRNG/SeedTree.swift:12-19. */
int32_t mfb_synth_expert_pool(void* stream, uint64_t root_seed, uint32_t layer, uint32_t first_expert,
                              uint32_t n_experts, int32_t shared, uint32_t bits, uint32_t scale_dtype, uint32_t d,
                              uint32_t f, uint8_t* pool, uint64_t slot_stride);
int32_t mfb_synth_normal(void* stream, uint64_t root_seed, const char* label, uint64_t n, double mean, double std,
                         int32_t absolute, uint32_t dtype, void* out);

#ifdef __cplusplus
}
#endif
#endif /* MFB200_H */
