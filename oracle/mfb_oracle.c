/*
 * mfb_oracle.c — CPU restatement of the reference's MoE feed-forward arithmetic.
 * TEST INFRASTRUCTURE ONLY; see mfb_oracle.h for the rules and the parity status.
 *
 * Numerical definition of the grading reference: weights are dequantised to fp32
 * exactly as the reference decodes them (float(code) * scale + bias, one rounding
 * after the multiply and one after the add), activations and scales are widened
 * exactly, and every dot product is accumulated in double so that the target does
 * not depend on a summation order.  The router logits are the one exception: they
 * feed an exact integer comparison (top-k), so they are defined in fp32 with one
 * fixed summation order (32 strided partial sums, then a xor butterfly) that a
 * 32-lane warp reproduces bit for bit.
 *
 * Build: gcc -O3 -fopenmp -ffp-contract=off (see oracle/Makefile).
 */
#include "mfb_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------ PRNG */

static inline uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* SplitMix64.swift:11-17: state += gamma, output = mix(state); so draw i is mix(seed + (i+1)*gamma). */
uint64_t mfbo_splitmix_at(uint64_t seed, uint64_t index) {
    return mix64(seed + (index + 1ull) * 0x9E3779B97F4A7C15ull);
}

/* SeedTree.swift:12-19. */
uint64_t mfbo_seed_for_label(uint64_t root, const char* label) {
    uint64_t h = 0xCBF29CE484222325ull;
    for (const unsigned char* p = (const unsigned char*)label; *p; ++p) {
        h ^= (uint64_t)*p;
        h *= 0x100000001B3ull;
    }
    return root ^ h;
}

/* SplitMix64.swift:20-23: 24-bit mantissa uniform in [lo, hi). */
float mfbo_uniform_at(uint64_t seed, uint64_t index, float lo, float hi) {
    float u = (float)(mfbo_splitmix_at(seed, index) >> 40) / (float)(1 << 24);
    return lo + (hi - lo) * u;
}

void mfbo_fill_raw(uint64_t seed, uint64_t first_draw, uint64_t n_draws, uint64_t* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n_draws; ++i) out[i] = mfbo_splitmix_at(seed, first_draw + (uint64_t)i);
}

/* Box-Muller in double; value i consumes draws 2i and 2i+1 so any value can be produced on its own. */
static inline double normal_at(uint64_t seed, uint64_t i) {
    const uint64_t a = mfbo_splitmix_at(seed, 2 * i), b = mfbo_splitmix_at(seed, 2 * i + 1);
    const double u1 = (double)((a >> 11) + 1ull) * (1.0 / 9007199254740992.0);
    const double u2 = (double)(b >> 11) * (1.0 / 9007199254740992.0);
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925286766559 * u2);
}

void mfbo_fill_normal(uint64_t seed, uint64_t first_value, uint64_t n, double mean, double std, int absolute,
                      int dtype, void* out) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        double z = normal_at(seed, first_value + (uint64_t)i) * std;
        if (absolute) z = fabs(z);
        const float v = (float)(mean + z);
        if (dtype == MFBO_DT_BF16) ((uint16_t*)out)[i] = mfbo_f32_to_bf16(v);
        else if (dtype == MFBO_DT_F16) ((uint16_t*)out)[i] = mfbo_f32_to_f16(v);
        else ((float*)out)[i] = v;
    }
}

/* ------------------------------------------------------------------ synthetic weights */

/* Blob layout of Sources/Mference/Kernels/MoE/MoE.swift:4-29: gate W,S,B then up W,S,B then down W,S,B,
 * each sub-tensor row-major; gate/up are [f, d], down is [d, f]; 64 elements per scale group. */
void mfbo_make_offsets(int bits, uint32_t d, uint32_t f, mfbo_expert_offsets* off, uint64_t* blob_bytes) {
    mfbo_make_offsets_gate(bits, d, f, 64u, off, blob_bytes);
}

/* DeepSeek V4 ships most layers' gate_proj at group 32 (ModelExpertIO.swift:118-135, moe.metal:962-965): only the
 * scale / bias row stride of gate changes. */
void mfbo_make_offsets_gate(int bits, uint32_t d, uint32_t f, uint32_t gate_group, mfbo_expert_offsets* off, uint64_t* blob_bytes) {
    const uint32_t wbytes = (uint32_t)((uint64_t)d * f * (uint32_t)bits / 8u);
    const uint32_t sbytes = d * f / 64u * 2u, gbytes = d * f / gate_group * 2u;
    uint32_t o = 0;
    off->gate_w = o; o += wbytes; off->gate_s = o; o += gbytes; off->gate_b = o; o += gbytes;
    off->up_w = o; o += wbytes; off->up_s = o; o += sbytes; off->up_b = o; o += sbytes;
    off->down_w = o; o += wbytes; off->down_s = o; o += sbytes; off->down_b = o; o += sbytes;
    *blob_bytes = o;
}

void mfbo_synth_expert(uint64_t root, uint32_t layer, int32_t expert, int bits, int scale_dtype, uint32_t d,
                       uint32_t f, uint8_t* blob) {
    mfbo_synth_expert_gate(root, layer, expert, bits, scale_dtype, d, f, 64u, blob);
}

void mfbo_synth_expert_gate(uint64_t root, uint32_t layer, int32_t expert, int bits, int scale_dtype, uint32_t d,
                            uint32_t f, uint32_t gate_group, uint8_t* blob) {
    static const char* proj[3] = {"gate", "up", "down"};
    mfbo_expert_offsets off;
    uint64_t total;
    mfbo_make_offsets_gate(bits, d, f, gate_group, &off, &total);
    const uint32_t* o = &off.gate_w;
    const uint64_t wbytes = (uint64_t)d * f * (uint32_t)bits / 8u;
    char who[48], label[96];
    if (expert < 0) snprintf(who, sizeof who, "L%u.shared", layer);
    else snprintf(who, sizeof who, "L%u.e%d", layer, expert);
    for (int p = 0; p < 3; ++p) {
        const uint64_t n_groups = (uint64_t)d * f / (p == 0 ? gate_group : 64u);
        snprintf(label, sizeof label, "%s.%s.q", who, proj[p]);
        mfbo_fill_raw(mfbo_seed_for_label(root, label), 0, wbytes / 8u, (uint64_t*)(blob + o[3 * p]));
        snprintf(label, sizeof label, "%s.%s.s", who, proj[p]);
        mfbo_fill_normal(mfbo_seed_for_label(root, label), 0, n_groups, 0.0, 0.02, 1, scale_dtype, blob + o[3 * p + 1]);
        snprintf(label, sizeof label, "%s.%s.b", who, proj[p]);
        mfbo_fill_normal(mfbo_seed_for_label(root, label), 0, n_groups, 0.0, 0.01, 0, scale_dtype, blob + o[3 * p + 2]);
    }
}

void mfbo_synth_router(uint64_t root, uint32_t layer, uint32_t num_experts, uint32_t d, uint16_t* w_bf16) {
    char label[48];
    snprintf(label, sizeof label, "L%u.router", layer);
    mfbo_fill_normal(mfbo_seed_for_label(root, label), 0, (uint64_t)num_experts * d, 0.0, 0.02, 0, MFBO_DT_BF16, w_bf16);
}

/* ------------------------------------------------------------------ conversions */

/* Quantization.swift:16-23 (round half to even on the dropped 16 bits). */
uint16_t mfbo_f32_to_bf16(float x) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    const uint32_t lsb = (bits >> 16) & 1u;
    return (uint16_t)((bits + 0x7FFFu + lsb) >> 16);
}

float mfbo_bf16_to_f32(uint16_t b) {
    uint32_t bits = (uint32_t)b << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t mfbo_f32_to_f16(float x) {
    _Float16 h = (_Float16)x; /* IEEE round-to-nearest-even */
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}

float mfbo_f16_to_f32(uint16_t u) {
    _Float16 h;
    memcpy(&h, &u, 2);
    return (float)h;
}

static inline float widen16(uint16_t v, int dtype) {
    return dtype == MFBO_DT_BF16 ? mfbo_bf16_to_f32(v) : mfbo_f16_to_f32(v);
}

/* ------------------------------------------------------------------ quantisation */

/* Code j of a row: 4-bit — byte j/2, low nibble is the even element (Quantization.swift:36,104-119);
 * 2-bit — byte j/4, element j at bit 2*(j%4) (moe.metal:948-950). */
static inline uint32_t code_at(const uint8_t* row, int bits, uint32_t j) {
    if (bits == 4) return (row[j >> 1] >> ((j & 1u) * 4u)) & 0xFu;
    if (bits == 2) return (row[j >> 2] >> ((j & 3u) * 2u)) & 0x3u;
    return row[j]; /* 8-bit: one unsigned byte per element (Quantization.swift:121-135) */
}

/* Quantization.swift:104-119: out = Float(code) * scale + bias (two roundings; no fused multiply-add). */
void mfbo_dequant_rows(const uint8_t* codes, const uint16_t* scales, const uint16_t* biases, int bits,
                       int group_size, int scale_dtype, uint32_t rows, uint32_t cols, float* out) {
    const uint32_t groups = cols / (uint32_t)group_size;
    const uint64_t row_bytes = (uint64_t)cols * (uint64_t)bits / 8u;
    for (uint32_t r = 0; r < rows; ++r) {
        const uint8_t* crow = codes + r * row_bytes;
        for (uint32_t g = 0; g < groups; ++g) {
            const float s = widen16(scales[(uint64_t)r * groups + g], scale_dtype);
            const float b = widen16(biases[(uint64_t)r * groups + g], scale_dtype);
            for (uint32_t k = 0; k < (uint32_t)group_size; ++k) {
                const uint32_t j = g * (uint32_t)group_size + k;
                const float prod = (float)code_at(crow, bits, j) * s;
                out[(uint64_t)r * cols + j] = prod + b;
            }
        }
    }
}

/* Quantization.swift:49-102: per-group min/max, scale = (max-min)/15, bias = min, both rounded through
 * bf16 before the codes are chosen; a constant group encodes as scale 1, bias value. */
void mfbo_quantize_int4_row(const float* row, uint32_t n, uint8_t* packed, uint16_t* scales_bf16,
                            uint16_t* biases_bf16) {
    memset(packed, 0, n / 2);
    for (uint32_t g = 0; g < n / 64; ++g) {
        float wmin = INFINITY, wmax = -INFINITY;
        for (uint32_t k = 0; k < 64; ++k) {
            const float w = row[g * 64 + k];
            if (w < wmin) wmin = w;
            if (w > wmax) wmax = w;
        }
        float sf, bf;
        if (wmax == wmin) { sf = 1.0f; bf = wmin; }
        else { sf = (wmax - wmin) / 15.0f; bf = wmin; }
        scales_bf16[g] = mfbo_f32_to_bf16(sf);
        biases_bf16[g] = mfbo_f32_to_bf16(bf);
        const float scale = mfbo_bf16_to_f32(scales_bf16[g]), bias = mfbo_bf16_to_f32(biases_bf16[g]);
        const float inv = scale == 0.0f ? 0.0f : 1.0f / scale;
        for (uint32_t k = 0; k < 64; ++k) {
            /* Swift's .rounded() is round-half-away-from-zero, as roundf is. */
            int q = (int)roundf((row[g * 64 + k] - bias) * inv);
            q = q < 0 ? 0 : (q > 15 ? 15 : q);
            const uint32_t byte = g * 32 + k / 2;
            if ((k & 1u) == 0) packed[byte] = (uint8_t)((packed[byte] & 0xF0) | (uint8_t)q);
            else packed[byte] = (uint8_t)((packed[byte] & 0x0F) | (uint8_t)(q << 4));
        }
    }
}

/* ------------------------------------------------------------------ router */

/* moe.metal:162-185 (router_gemv_bf16_r4): one 32-lane group per expert row, lane l accumulates elements
 * l, l+32, ... with fma, then the lanes are summed.  The reference leaves the lane-sum order to the
 * hardware; here it is fixed to a xor butterfly (16, 8, 4, 2, 1).  effective_scale is 1 for the model
 * families in scope (Sources/Mference/Runtime/Inference/RealForwardRunner.swift:950-959).  An optional
 * per-expert additive bias (used to skew routing in synthetic workloads) is added last, in fp32. */
void mfbo_router_logits(const uint16_t* x, int x_dtype, uint32_t ldx, uint32_t n_tokens, const uint16_t* w_bf16,
                        uint32_t num_experts, uint32_t d, const float* logit_bias, int exact_f64, float* logits) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < (int64_t)n_tokens; ++t) {
        float* xf = (float*)malloc(sizeof(float) * d);
        for (uint32_t i = 0; i < d; ++i) xf[i] = widen16(x[(uint64_t)t * ldx + i], x_dtype);
        for (uint32_t e = 0; e < num_experts; ++e) {
            const uint16_t* wr = w_bf16 + (uint64_t)e * d;
            float v;
            if (exact_f64) {
                double acc = 0.0;
                for (uint32_t i = 0; i < d; ++i) acc += (double)mfbo_bf16_to_f32(wr[i]) * (double)xf[i];
                v = (float)acc;
            } else {
                float lane[32];
                for (uint32_t l = 0; l < 32; ++l) {
                    float acc = 0.0f;
                    for (uint32_t i = l; i < d; i += 32) acc = fmaf(mfbo_bf16_to_f32(wr[i]), xf[i], acc);
                    lane[l] = acc;
                }
                for (uint32_t off = 16; off > 0; off >>= 1) {
                    float nxt[32];
                    for (uint32_t l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ off];
                    memcpy(lane, nxt, sizeof(lane));
                }
                v = lane[0];
            }
            if (logit_bias) v = v + logit_bias[e];
            logits[(uint64_t)t * num_experts + e] = v;
        }
        free(xf);
    }
}

/* Insertion scan shared by both selectors: a strictly greater score wins, an equal score keeps the lower
 * expert index (moe.metal:206-222).  Unfilled slots stay at index 0 with score -inf. */
static void select_topk(const float* score, uint32_t num_experts, uint32_t top_k, uint32_t* top_idx,
                        float* top_score) {
    for (uint32_t i = 0; i < top_k; ++i) { top_idx[i] = 0; top_score[i] = -INFINITY; }
    for (uint32_t e = 0; e < num_experts; ++e) {
        const float s = score[e];
        if (s <= top_score[top_k - 1]) continue;
        uint32_t pos = top_k;
        for (uint32_t i = 0; i < top_k; ++i) {
            if (s > top_score[i] || (s == top_score[i] && e < top_idx[i])) { pos = i; break; }
        }
        if (pos >= top_k) continue;
        for (uint32_t i = top_k - 1; i > pos; --i) { top_idx[i] = top_idx[i - 1]; top_score[i] = top_score[i - 1]; }
        top_idx[pos] = e;
        top_score[pos] = s;
    }
}

/* moe.metal:190-240 / prefill.metal:586-628: weights are the softmax over the selected logits only,
 * times an optional per-expert scale, rounded to fp16. */
void mfbo_topk_softmax(const float* logits, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k,
                       const uint16_t* per_expert_scale_bf16, uint32_t* out_idx, uint16_t* out_w_f16) {
    for (uint32_t t = 0; t < n_tokens; ++t) {
        uint32_t ti[64];
        float ts[64], ex[64];
        select_topk(logits + (uint64_t)t * num_experts, num_experts, top_k, ti, ts);
        const float max_s = ts[0];
        float sum = 0.0f;
        for (uint32_t i = 0; i < top_k; ++i) { ex[i] = expf(ts[i] - max_s); sum += ex[i]; }
        for (uint32_t i = 0; i < top_k; ++i) {
            const float gain = per_expert_scale_bf16 ? mfbo_bf16_to_f32(per_expert_scale_bf16[ti[i]]) : 1.0f;
            out_idx[(uint64_t)t * top_k + i] = ti[i];
            out_w_f16[(uint64_t)t * top_k + i] = mfbo_f32_to_f16(ex[i] / sum * gain);
        }
    }
}

/* moe.metal:737-741. */
static inline float sqrtsoftplus(float x) {
    const float sp = fmaxf(x, 0.0f) + logf(1.0f + expf(-fabsf(x)));
    return sqrtf(sp);
}

/* moe.metal:745-793: selection on sqrtsoftplus(logit) + correction bias; weights from the raw scores of
 * the selected experts, normalised over them and scaled by route_scale. */
void mfbo_topk_sqrtsoftplus(const float* logits, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k,
                            const float* correction_bias, float route_scale, uint32_t* out_idx,
                            uint16_t* out_w_f16) {
    float* sel = (float*)malloc(sizeof(float) * num_experts);
    for (uint32_t t = 0; t < n_tokens; ++t) {
        const float* lg = logits + (uint64_t)t * num_experts;
        for (uint32_t e = 0; e < num_experts; ++e)
            sel[e] = sqrtsoftplus(lg[e]) + (correction_bias ? correction_bias[e] : 0.0f);
        uint32_t ti[64];
        float ts[64], sc[64];
        select_topk(sel, num_experts, top_k, ti, ts);
        float sum = 0.0f;
        for (uint32_t i = 0; i < top_k; ++i) { sc[i] = sqrtsoftplus(lg[ti[i]]); sum += sc[i]; }
        const float inv = route_scale / (sum + 1e-20f);
        for (uint32_t i = 0; i < top_k; ++i) {
            out_idx[(uint64_t)t * top_k + i] = ti[i];
            out_w_f16[(uint64_t)t * top_k + i] = mfbo_f32_to_f16(sc[i] * inv);
        }
    }
    free(sel);
}

void mfbo_topk_margin(const float* scores, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k, float* margin) {
    for (uint32_t t = 0; t < n_tokens; ++t) {
        uint32_t ti[65];
        float ts[65];
        const uint32_t kk = top_k + 1 <= num_experts ? top_k + 1 : num_experts;
        select_topk(scores + (uint64_t)t * num_experts, num_experts, kk, ti, ts);
        float m = INFINITY;
        for (uint32_t i = 0; i + 1 < kk; ++i) m = fminf(m, ts[i] - ts[i + 1]);
        margin[t] = m;
    }
}

/* ------------------------------------------------------------------ expert FFN */

/* moe.metal:71-84 (gelu_pytorch_tanh with its clamp; silu = x / (1 + exp(-x))). */
static inline double activation(double g, int act) {
    if (act == MFBO_ACT_SILU) return g / (1.0 + exp(-g));
    double inner = 0.7978845608028654 * (g + 0.044715 * g * g * g);
    if (inner > 20.0) inner = 20.0;
    if (inner < -20.0) inner = -20.0;
    return 0.5 * g * (1.0 + tanh(inner));
}

static inline double dotd(const float* a, const float* b, uint32_t n) {
    double s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    uint32_t i = 0;
    for (; i + 4 <= n; i += 4) {
        s0 += (double)a[i] * (double)b[i];
        s1 += (double)a[i + 1] * (double)b[i + 1];
        s2 += (double)a[i + 2] * (double)b[i + 2];
        s3 += (double)a[i + 3] * (double)b[i + 3];
    }
    for (; i < n; ++i) s0 += (double)a[i] * (double)b[i];
    return (s0 + s1) + (s2 + s3);
}

typedef struct expert_f32 {
    float *gate, *up, *down; /* [f,d], [f,d], [d,f] */
} expert_f32;

static void expert_dequant_gate(const uint8_t* blob, const mfbo_expert_offsets* off, int bits, int group_size, int gate_group,
                                int scale_dtype, uint32_t d, uint32_t f, expert_f32* w);
static void expert_dequant(const uint8_t* blob, const mfbo_expert_offsets* off, int bits, int group_size,
                           int scale_dtype, uint32_t d, uint32_t f, expert_f32* w) {
    expert_dequant_gate(blob, off, bits, group_size, group_size, scale_dtype, d, f, w);
}
static void expert_dequant_gate(const uint8_t* blob, const mfbo_expert_offsets* off, int bits, int group_size, int gate_group,
                                int scale_dtype, uint32_t d, uint32_t f, expert_f32* w) {
    w->gate = (float*)malloc(sizeof(float) * (size_t)d * f);
    w->up = (float*)malloc(sizeof(float) * (size_t)d * f);
    w->down = (float*)malloc(sizeof(float) * (size_t)d * f);
    mfbo_dequant_rows(blob + off->gate_w, (const uint16_t*)(blob + off->gate_s), (const uint16_t*)(blob + off->gate_b),
                      bits, gate_group, scale_dtype, f, d, w->gate);
    mfbo_dequant_rows(blob + off->up_w, (const uint16_t*)(blob + off->up_s), (const uint16_t*)(blob + off->up_b),
                      bits, group_size, scale_dtype, f, d, w->up);
    mfbo_dequant_rows(blob + off->down_w, (const uint16_t*)(blob + off->down_s), (const uint16_t*)(blob + off->down_b),
                      bits, group_size, scale_dtype, d, f, w->down);
}

static void expert_free(expert_f32* w) { free(w->gate); free(w->up); free(w->down); }

/* Moe.swift:31-53 (runFFN): down( act(gate x) * (up x) ); clamp of moe.metal:27-34 before the activation. */
static void expert_apply(const expert_f32* w, uint32_t d, uint32_t f, int act, float limit, const float* x,
                         double* out) {
    float* h = (float*)malloc(sizeof(float) * f);
    for (uint32_t r = 0; r < f; ++r) {
        double g = dotd(w->gate + (size_t)r * d, x, d);
        double u = dotd(w->up + (size_t)r * d, x, d);
        if (limit > 0.0f) {
            if (g > limit) g = limit;
            if (u > limit) u = limit;
            if (u < -limit) u = -limit;
        }
        h[r] = (float)(activation(g, act) * u);
    }
    for (uint32_t r = 0; r < d; ++r) out[r] = dotd(w->down + (size_t)r * f, h, f);
    free(h);
}

void mfbo_expert_ffn(const uint8_t* blob, const mfbo_expert_offsets* off, int bits, int group_size,
                     int scale_dtype, uint32_t d, uint32_t f, int act, float swiglu_limit, const float* x,
                     double* out) {
    expert_f32 w;
    expert_dequant(blob, off, bits, group_size, scale_dtype, d, f, &w);
    expert_apply(&w, d, f, act, swiglu_limit, x, out);
    expert_free(&w);
}

/* Moe.swift:59-88 (applyStreamedRouted): y = residual + sum over slots in rank order of w * ffn(x); the
 * always-on shared expert is added to the residual first (RealForwardRunner.swift:3211 passes the shared
 * output as the residual of the weighted reduce). */
void mfbo_moe_layer(const mfbo_layer* L, const uint16_t* x, int x_dtype, uint32_t ldx, uint32_t n_tokens,
                    const uint32_t* idx, const uint16_t* w_f16, const float* residual, float* y) {
    const uint32_t d = L->d, f = L->f, K = L->top_k, E = L->num_experts;
    const size_t slots = (size_t)K + 1;
    float* xf = (float*)malloc(sizeof(float) * (size_t)n_tokens * d);
    for (uint32_t t = 0; t < n_tokens; ++t)
        for (uint32_t i = 0; i < d; ++i) xf[(size_t)t * d + i] = widen16(x[(size_t)t * ldx + i], x_dtype);
    double* part = (double*)calloc((size_t)n_tokens * slots * d, sizeof(double));
    const int n_units = (int)E + 1;
#pragma omp parallel for schedule(dynamic, 1)
    for (int e = 0; e < n_units; ++e) {
        const int shared = (e == (int)E);
        if (shared && !L->shared_blob) continue;
        int any = shared;
        for (size_t p = 0; !any && p < (size_t)n_tokens * K; ++p) any = (idx[p] == (uint32_t)e);
        if (!any) continue;
        expert_f32 w;
        if (shared) expert_dequant(L->shared_blob, &L->shared_off, (int)L->shared_bits, (int)L->group_size,
                                   (int)L->scale_dtype, d, f, &w);
        else expert_dequant_gate(L->pool + (uint64_t)e * L->expert_stride, &L->routed_off, (int)L->bits, (int)L->group_size,
                                 (int)(L->gate_group_size ? L->gate_group_size : L->group_size), (int)L->scale_dtype, d, f, &w);
        for (uint32_t t = 0; t < n_tokens; ++t) {
            if (shared) {
                expert_apply(&w, d, f, (int)L->activation, 0.0f, xf + (size_t)t * d, part + ((size_t)t * slots + K) * d);
            } else {
                for (uint32_t r = 0; r < K; ++r)
                    if (idx[(size_t)t * K + r] == (uint32_t)e)
                        expert_apply(&w, d, f, (int)L->activation, L->swiglu_limit, xf + (size_t)t * d,
                                     part + ((size_t)t * slots + r) * d);
            }
        }
        expert_free(&w);
    }
    for (uint32_t t = 0; t < n_tokens; ++t) {
        for (uint32_t i = 0; i < d; ++i) {
            double acc = residual ? (double)residual[(size_t)t * d + i] : 0.0;
            if (L->shared_blob) acc += part[((size_t)t * slots + K) * d + i];
            for (uint32_t r = 0; r < K; ++r)
                acc += (double)mfbo_f16_to_f32(w_f16[(size_t)t * K + r]) * part[((size_t)t * slots + r) * d + i];
            y[(size_t)t * d + i] = (float)acc;
        }
    }
    free(part);
    free(xf);
}

/* Sources/Mference/Metal/Prefill/prefill.metal:748-820: one FFN result row per sorted (token, expert) pair. */
void mfbo_pair_partials(const mfbo_layer* L, const uint16_t* x, int x_dtype, uint32_t ldx, const mfbo_pair* pairs,
                        uint32_t n_pairs, float* partial) {
    const uint32_t d = L->d, f = L->f;
#pragma omp parallel for schedule(dynamic, 1)
    for (int e = 0; e < (int)L->num_experts; ++e) {
        int any = 0;
        for (uint32_t p = 0; !any && p < n_pairs; ++p) any = (pairs[p].expert == (uint32_t)e);
        if (!any) continue;
        expert_f32 w;
        expert_dequant_gate(L->pool + (uint64_t)e * L->expert_stride, &L->routed_off, (int)L->bits, (int)L->group_size,
                       (int)(L->gate_group_size ? L->gate_group_size : L->group_size),
                       (int)L->scale_dtype, d, f, &w);
        float* xf = (float*)malloc(sizeof(float) * d);
        double* out = (double*)malloc(sizeof(double) * d);
        for (uint32_t p = 0; p < n_pairs; ++p) {
            if (pairs[p].expert != (uint32_t)e) continue;
            for (uint32_t i = 0; i < d; ++i) xf[i] = widen16(x[(size_t)pairs[p].token * ldx + i], x_dtype);
            expert_apply(&w, d, f, (int)L->activation, L->swiglu_limit, xf, out);
            for (uint32_t i = 0; i < d; ++i) partial[(size_t)p * d + i] = (float)out[i];
        }
        free(out);
        free(xf);
        expert_free(&w);
    }
}

/* ------------------------------------------------------------------ grouping */

typedef struct sort_item {
    uint64_t key;
    mfbo_pair pair;
    int has_key;
} sort_item;

static int cmp_items(const void* pa, const void* pb) {
    const sort_item* a = (const sort_item*)pa;
    const sort_item* b = (const sort_item*)pb;
    if (a->has_key && a->key != b->key) return a->key < b->key ? -1 : 1;
    if (a->pair.expert != b->pair.expert) return a->pair.expert < b->pair.expert ? -1 : 1;
    if (a->pair.token != b->pair.token) return a->pair.token < b->pair.token ? -1 : 1;
    if (a->pair.rank != b->pair.rank) return a->pair.rank < b->pair.rank ? -1 : 1;
    return 0;
}

static int cmp_u64(const void* a, const void* b) {
    const uint64_t x = *(const uint64_t*)a, y = *(const uint64_t*)b;
    return x < y ? -1 : (x > y ? 1 : 0);
}

/* PrefillMoEGrouping.swift:90-192.  Validation order and error cases follow the reference; err_a/err_b carry
 * the offending values.  The comparison is a total order once (token, rank) is unique, so qsort's instability
 * cannot show. */
int mfbo_group_pairs(const mfbo_pair* pairs, int64_t n_pairs, int64_t query_count, int64_t top_k,
                     int64_t num_experts, int64_t tile_expert_count, const uint64_t* sort_keys,
                     int64_t n_sort_keys, mfbo_pair* sorted, uint32_t* offsets, uint32_t* counts,
                     mfbo_group* groups, uint32_t* n_groups, mfbo_tile* tiles, uint32_t* n_tiles,
                     uint32_t* err_a, uint32_t* err_b) {
    *err_a = 0; *err_b = 0; *n_groups = 0; *n_tiles = 0;
    if (query_count < 0) { *err_a = (uint32_t)query_count; return MFBO_GROUP_INVALID_QUERY_COUNT; }
    if (top_k <= 0) { *err_a = (uint32_t)top_k; return MFBO_GROUP_INVALID_TOP_K; }
    if (num_experts <= 0) { *err_a = (uint32_t)num_experts; return MFBO_GROUP_INVALID_NUM_EXPERTS; }
    if (tile_expert_count < 1 || tile_expert_count > 16) {
        *err_a = (uint32_t)tile_expert_count;
        return MFBO_GROUP_INVALID_TILE_EXPERT_COUNT;
    }
    if (sort_keys && n_sort_keys != num_experts) {
        *err_a = (uint32_t)num_experts; *err_b = (uint32_t)n_sort_keys;
        return MFBO_GROUP_SORT_KEY_COUNT_MISMATCH;
    }
    if (n_pairs != query_count * top_k) {
        *err_a = (uint32_t)(query_count * top_k); *err_b = (uint32_t)n_pairs;
        return MFBO_GROUP_PAIR_COUNT_MISMATCH;
    }
    uint64_t* seen = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n_pairs ? n_pairs : 1));
    for (int64_t i = 0; i < n_pairs; ++i) {
        const mfbo_pair* p = &pairs[i];
        int rc = 0;
        if (p->token >= (uint32_t)query_count) { *err_a = p->token; rc = MFBO_GROUP_TOKEN_OUT_OF_RANGE; }
        else if (p->rank >= (uint32_t)top_k) { *err_a = p->rank; rc = MFBO_GROUP_RANK_OUT_OF_RANGE; }
        else if (p->expert >= (uint32_t)num_experts) { *err_a = p->expert; rc = MFBO_GROUP_EXPERT_OUT_OF_RANGE; }
        if (rc) { free(seen); return rc; }
        seen[i] = ((uint64_t)p->token << 32) | p->rank;
        /* the reference reports the first repeated (token, rank) in input order */
        for (int64_t j = 0; n_pairs <= 4096 && j < i; ++j)
            if (seen[j] == seen[i]) { *err_a = p->token; *err_b = p->rank; free(seen); return MFBO_GROUP_DUPLICATE_TOKEN_RANK; }
    }
    if (n_pairs > 4096) {
        qsort(seen, (size_t)n_pairs, sizeof(uint64_t), cmp_u64);
        for (int64_t i = 1; i < n_pairs; ++i)
            if (seen[i] == seen[i - 1]) {
                *err_a = (uint32_t)(seen[i] >> 32); *err_b = (uint32_t)seen[i];
                free(seen);
                return MFBO_GROUP_DUPLICATE_TOKEN_RANK;
            }
    }
    free(seen);

    sort_item* items = (sort_item*)malloc(sizeof(sort_item) * (size_t)(n_pairs ? n_pairs : 1));
    for (int64_t i = 0; i < n_pairs; ++i) {
        items[i].pair = pairs[i];
        items[i].has_key = sort_keys != NULL;
        items[i].key = sort_keys ? sort_keys[pairs[i].expert] : 0;
    }
    qsort(items, (size_t)n_pairs, sizeof(sort_item), cmp_items);
    for (int64_t i = 0; i < n_pairs; ++i) sorted[i] = items[i].pair;
    free(items);

    for (int64_t e = 0; e < num_experts; ++e) { offsets[e] = 0xFFFFFFFFu; counts[e] = 0; }
    uint32_t ng = 0;
    int64_t i = 0;
    while (i < n_pairs) {
        const uint32_t expert = sorted[i].expert;
        const int64_t start = i;
        while (i < n_pairs && sorted[i].expert == expert) ++i;
        offsets[expert] = (uint32_t)start;
        counts[expert] = (uint32_t)(i - start);
        groups[ng].expert = expert;
        groups[ng].pair_start = (uint32_t)start;
        groups[ng].pair_count = (uint32_t)(i - start);
        ++ng;
    }
    uint32_t nt = 0;
    for (uint32_t gs = 0; gs < ng;) {
        const uint32_t ge = gs + (uint32_t)tile_expert_count < ng ? gs + (uint32_t)tile_expert_count : ng;
        tiles[nt].group_start = gs;
        tiles[nt].group_count = ge - gs;
        tiles[nt].pair_start = groups[gs].pair_start;
        tiles[nt].pair_count = groups[ge - 1].pair_start + groups[ge - 1].pair_count - groups[gs].pair_start;
        ++nt;
        gs = ge;
    }
    *n_groups = ng;
    *n_tiles = nt;
    return MFBO_GROUP_OK;
}

/* ------------------------------------------------------------------ reduce, rmsnorm */

/* prefill.metal:631-652: h2[t,d] = sum over ranks, in rank order, of w[t,r] * partial[t,r,d] (double here). */
void mfbo_reduce_token_major(const float* partial, const uint16_t* w_f16, uint32_t n_tokens, uint32_t top_k,
                             uint32_t d, float* h2) {
    for (uint32_t t = 0; t < n_tokens; ++t)
        for (uint32_t i = 0; i < d; ++i) {
            double acc = 0.0;
            for (uint32_t r = 0; r < top_k; ++r)
                acc += (double)mfbo_f16_to_f32(w_f16[(size_t)t * top_k + r]) *
                       (double)partial[((size_t)t * top_k + r) * d + i];
            h2[(size_t)t * d + i] = (float)acc;
        }
}

/* rmsnorm.metal:32-93 / Support/Reference/Primitives/RmsNorm.swift:13-45: inv = 1/sqrt(mean(x^2)+eps),
 * out = x * inv * w (bf16 weight); the caller rounds to its storage dtype. */
void mfbo_rmsnorm(const float* x, const uint16_t* w_bf16, uint32_t n_rows, uint32_t d, float eps, float* out) {
    for (uint32_t r = 0; r < n_rows; ++r) {
        double ss = 0.0;
        for (uint32_t i = 0; i < d; ++i) ss += (double)x[(size_t)r * d + i] * (double)x[(size_t)r * d + i];
        const double inv = 1.0 / sqrt(ss / (double)d + (double)eps);
        for (uint32_t i = 0; i < d; ++i)
            out[(size_t)r * d + i] = (float)((double)x[(size_t)r * d + i] * inv *
                                             (w_bf16 ? (double)mfbo_bf16_to_f32(w_bf16[i]) : 1.0));
    }
}

/* ------------------------------------------------------------------ timed CPU baseline (fp32, fused dequant) */

/* One affine row dot in the reference's factored form (moe.metal:349-404): per group
 * acc = fma(s, sum(q*x), acc); acc = fma(b, sum(x), acc). */
static inline float row_dot_f32(const uint8_t* crow, const uint16_t* s, const uint16_t* b, int bits, int sdt,
                                uint32_t cols, const float* x, const float* xsum) {
    float acc = 0.0f;
    for (uint32_t g = 0; g < cols / 64; ++g) {
        float dot = 0.0f;
        const float* xg = x + g * 64;
        if (bits == 4) {
            const uint8_t* cg = crow + g * 32;
            for (uint32_t k = 0; k < 32; ++k) {
                dot += (float)(cg[k] & 0xF) * xg[2 * k];
                dot += (float)(cg[k] >> 4) * xg[2 * k + 1];
            }
        } else if (bits == 8) {
            const uint8_t* cg = crow + g * 64;
            for (uint32_t k = 0; k < 64; ++k) dot += (float)cg[k] * xg[k];
        } else {
            const uint8_t* cg = crow + g * 16;
            for (uint32_t k = 0; k < 16; ++k) {
                dot += (float)(cg[k] & 3) * xg[4 * k];
                dot += (float)((cg[k] >> 2) & 3) * xg[4 * k + 1];
                dot += (float)((cg[k] >> 4) & 3) * xg[4 * k + 2];
                dot += (float)(cg[k] >> 6) * xg[4 * k + 3];
            }
        }
        acc += widen16(s[g], sdt) * dot;
        acc += widen16(b[g], sdt) * xsum[g];
    }
    return acc;
}

static void group_sums(const float* x, uint32_t n, float* out) {
    for (uint32_t g = 0; g < n / 64; ++g) {
        float s = 0.0f;
        for (uint32_t k = 0; k < 64; ++k) s += x[g * 64 + k];
        out[g] = s;
    }
}

/* The reference's decode sequence for one layer (RealForwardRunner.swift:2910-2918, 3188-3218): shared
 * expert, phase 1 (gate/up + activation, fp16 store), phase 2 (down + weighted reduce, residual first, rank
 * order).  Rows are spread over the host threads. */
void mfbo_ref_moe_layer_f32(const mfbo_layer* L, const float* x, uint32_t n_tokens, const uint32_t* idx,
                            const uint16_t* w_f16, const float* residual, float* y) {
    const uint32_t d = L->d, f = L->f, K = L->top_k;
    const uint32_t units = K + (L->shared_blob ? 1u : 0u);
    float* acts = (float*)malloc(sizeof(float) * (size_t)units * f);
    float* xs = (float*)malloc(sizeof(float) * (d / 64));
    float* as = (float*)malloc(sizeof(float) * (size_t)units * (f / 64));
    const int sdt = (int)L->scale_dtype;
    for (uint32_t t = 0; t < n_tokens; ++t) {
        const float* xt = x + (size_t)t * d;
        group_sums(xt, d, xs);
#pragma omp parallel for schedule(static)
        for (int64_t row = 0; row < (int64_t)units * f; ++row) {
            const uint32_t u = (uint32_t)(row / f), r = (uint32_t)(row % f);
            const int shared = (u == K);
            const uint8_t* blob = shared ? L->shared_blob : L->pool + (uint64_t)idx[(size_t)t * K + u] * L->expert_stride;
            const mfbo_expert_offsets* o = shared ? &L->shared_off : &L->routed_off;
            const int bits = shared ? (int)L->shared_bits : (int)L->bits;
            const uint64_t rb = (uint64_t)d * (uint64_t)bits / 8u;
            float g = row_dot_f32(blob + o->gate_w + r * rb, (const uint16_t*)(blob + o->gate_s) + (size_t)r * (d / 64),
                                  (const uint16_t*)(blob + o->gate_b) + (size_t)r * (d / 64), bits, sdt, d, xt, xs);
            float v = row_dot_f32(blob + o->up_w + r * rb, (const uint16_t*)(blob + o->up_s) + (size_t)r * (d / 64),
                                  (const uint16_t*)(blob + o->up_b) + (size_t)r * (d / 64), bits, sdt, d, xt, xs);
            if (!shared && L->swiglu_limit > 0.0f) {
                g = fminf(g, L->swiglu_limit);
                v = fmaxf(fminf(v, L->swiglu_limit), -L->swiglu_limit);
            }
            const float a = L->activation == MFBO_ACT_SILU ? g / (1.0f + expf(-g)) : (float)activation(g, MFBO_ACT_GELU_TANH);
            acts[(size_t)u * f + r] = mfbo_f16_to_f32(mfbo_f32_to_f16(a * v));
        }
        for (uint32_t u = 0; u < units; ++u) group_sums(acts + (size_t)u * f, f, as + (size_t)u * (f / 64));
#pragma omp parallel for schedule(static)
        for (int64_t row = 0; row < (int64_t)d; ++row) {
            float acc = residual ? residual[(size_t)t * d + row] : 0.0f;
            for (uint32_t uu = 0; uu < units; ++uu) {
                const uint32_t u = (uu == 0 && L->shared_blob) ? K : (L->shared_blob ? uu - 1 : uu);
                const int shared = (u == K);
                const uint8_t* blob = shared ? L->shared_blob : L->pool + (uint64_t)idx[(size_t)t * K + u] * L->expert_stride;
                const mfbo_expert_offsets* o = shared ? &L->shared_off : &L->routed_off;
                const int bits = shared ? (int)L->shared_bits : (int)L->bits;
                const uint64_t rb = (uint64_t)f * (uint64_t)bits / 8u;
                const float v = row_dot_f32(blob + o->down_w + (uint64_t)row * rb,
                                            (const uint16_t*)(blob + o->down_s) + (size_t)row * (f / 64),
                                            (const uint16_t*)(blob + o->down_b) + (size_t)row * (f / 64), bits, sdt, f,
                                            acts + (size_t)u * f, as + (size_t)u * (f / 64));
                const float wgt = shared ? 1.0f : mfbo_f16_to_f32(w_f16[(size_t)t * K + u]);
                acc += wgt * v;
            }
            y[(size_t)t * d + row] = acc;
        }
    }
    free(as);
    free(xs);
    free(acts);
}

int mfbo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* ------------------------------------------------------------------ quantised gate / projections */

/* Weights of hash-routed layers (moe.metal:852-896, router_hash_weights_k6): the expert indices are given (a frozen
 * token-id table in the reference); the weights are sqrt(softplus(logit)) of exactly those experts, summed in rank
 * order, normalised and scaled by route_scale. */
void mfbo_hash_weights(const float* logits, const uint32_t* idx, uint32_t n_tokens, uint32_t num_experts, uint32_t top_k,
                       float route_scale, uint16_t* out_w_f16) {
    for (uint32_t t = 0; t < n_tokens; ++t) {
        float sc[64], sum = 0.0f;
        for (uint32_t i = 0; i < top_k; ++i) {
            sc[i] = sqrtsoftplus(logits[(uint64_t)t * num_experts + idx[(uint64_t)t * top_k + i]]);
            sum += sc[i];
        }
        const float inv = route_scale / (sum + 1e-20f);
        for (uint32_t i = 0; i < top_k; ++i) out_w_f16[(uint64_t)t * top_k + i] = mfbo_f32_to_f16(sc[i] * inv);
    }
}

/* INT8 affine group-64 GEMV in the order of router_gemv_gemma4_r4 (moe.metal:102-157) and of the shared-expert scalar
 * gate (prefill.metal:37-80): one 32-lane group per output row; for every 64-element group lane l takes elements
 * 2l and 2l+1:  acc = fma(s, q0*x0 + q1*x1, acc); acc = fma(b, x0 + x1, acc)  with every product and sum rounded to
 * fp32; the lane sums meet in the xor butterfly fixed for the bf16 gate above.  Codes are unsigned bytes, scales and
 * biases bf16 per (row, group).  effective_scale (bf16 per element, may be NULL = 1) multiplies the activation first. */
void mfbo_gemv_int8(const uint8_t* W, const uint16_t* s_bf16, const uint16_t* b_bf16, const uint16_t* x, int x_dtype,
                    uint32_t ldx, uint32_t n_tokens, const uint16_t* effective_scale_bf16, uint32_t M, uint32_t N, float* y) {
    const uint32_t groups = N / 64;
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < (int64_t)n_tokens; ++t) {
        float* xf = (float*)malloc(sizeof(float) * N);
        for (uint32_t i = 0; i < N; ++i) {
            float v = widen16(x[(uint64_t)t * ldx + i], x_dtype);
            if (effective_scale_bf16) v = v * mfbo_bf16_to_f32(effective_scale_bf16[i]);
            xf[i] = v;
        }
        for (uint32_t r = 0; r < M; ++r) {
            float lane[32];
            for (uint32_t l = 0; l < 32; ++l) {
                float acc = 0.0f;
                for (uint32_t g = 0; g < groups; ++g) {
                    const float s = mfbo_bf16_to_f32(s_bf16[(uint64_t)r * groups + g]);
                    const float b = mfbo_bf16_to_f32(b_bf16[(uint64_t)r * groups + g]);
                    const uint32_t i0 = g * 64 + 2 * l;
                    const float q0 = (float)W[(uint64_t)r * N + i0], q1 = (float)W[(uint64_t)r * N + i0 + 1];
                    const float p0 = q0 * xf[i0], p1 = q1 * xf[i0 + 1];
                    const float dot = p0 + p1, sx = xf[i0] + xf[i0 + 1];
                    acc = fmaf(s, dot, acc);
                    acc = fmaf(b, sx, acc);
                }
                lane[l] = acc;
            }
            for (uint32_t off = 16; off > 0; off >>= 1) {
                float nxt[32];
                for (uint32_t l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ off];
                memcpy(lane, nxt, sizeof(lane));
            }
            y[(uint64_t)t * M + r] = lane[0];
        }
        free(xf);
    }
}

/* fp32 reference of the INT4 affine group-64 GEMV y = W x (DequantInt4Gemv.swift:13-42: every row dequantised to
 * fp32 as Quantization.dequantizeInt4Affine does, then a dot product; accumulated in double here). */
void mfbo_gemv_int4(const uint8_t* W, const uint16_t* scales, const uint16_t* biases, int scale_dtype, const uint16_t* x,
                    int x_dtype, uint32_t ldx, uint32_t n_tokens, uint32_t M, uint32_t N, float* y) {
    const uint32_t groups = N / 64;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)M; ++r) {
        float* wr = (float*)malloc(sizeof(float) * N);
        for (uint32_t i = 0; i < N; ++i) {
            const uint8_t byte = W[(uint64_t)r * (N / 2) + i / 2];
            const float q = (float)((i & 1) ? (byte >> 4) : (byte & 15));
            wr[i] = q * widen16(scales[(uint64_t)r * groups + i / 64], scale_dtype) + widen16(biases[(uint64_t)r * groups + i / 64], scale_dtype);
        }
        for (uint32_t t = 0; t < n_tokens; ++t) {
            double acc = 0.0;
            for (uint32_t i = 0; i < N; ++i) acc += (double)wr[i] * (double)widen16(x[(uint64_t)t * ldx + i], x_dtype);
            y[(uint64_t)t * M + r] = (float)acc;
        }
        free(wr);
    }
}

/* Number of threads of the following parallel loops (the timed CPU baseline uses every host core even when the
 * launcher exported OMP_NUM_THREADS=1 for its ranks). */
void mfbo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
