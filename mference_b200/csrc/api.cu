// C ABI entry points: argument validation, the handle and its scratch arena, and the launch sequences.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"
#include "decode_mma.cuh"
#include "prefill_tc.cuh"

namespace mfb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

static std::atomic<uint64_t> g_launches{0};
void count_launches(uint64_t n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int32_t cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return MFB_ERR_CUDA;
}

namespace {

bool pow2_or_wide(uint32_t cols, uint32_t bits) {
    const uint32_t pieces = cols * bits / 128;
    if (pieces == 0) return false;
    return pieces >= 32 || (pieces & (pieces - 1)) == 0;
}

bool offsets_aligned(const mfb_expert_offsets& o) {
    const uint32_t* p = &o.gate_w;
    for (int i = 0; i < 9; ++i)
        if (p[i] % 16) return false;
    return true;
}

template <typename T>
cudaError_t dev_alloc(T*& p, size_t count) {
    return cudaMalloc((void**)&p, (count ? count : 1) * sizeof(T));
}

void free_arena(Arena& a) {
    cudaFree(a.logits); cudaFree(a.router_ws); cudaFree(a.idx); cudaFree(a.route_w); cudaFree(a.xn); cudaFree(a.sorted);
    cudaFree(a.chunk_hist); cudaFree(a.offsets); cudaFree(a.counts); cudaFree(a.groups); cudaFree(a.n_groups);
    cudaFree(a.tile_prefix); cudaFree(a.acts); cudaFree(a.partial); cudaFree(a.xs16); cudaFree(a.acts16); cudaFree(a.xp); cudaFree(a.xp2); cudaFree(a.actp);
    cudaFree(a.status);
    a = Arena();
}

int32_t check_handle(const mfb_moe* m, uint32_t n_tokens) {
    MFB_REQUIRE(m != nullptr, MFB_ERR_INVALID_ARGUMENT, "handle is NULL");
    MFB_REQUIRE(n_tokens <= m->cfg.max_tokens, MFB_ERR_CAPACITY, "%u tokens exceed the arena capacity of %u", n_tokens,
                m->cfg.max_tokens);
    return MFB_OK;
}

int32_t check_weights(const mfb_moe* m, const mfb_layer_weights* w, bool need_router) {
    MFB_REQUIRE(w != nullptr, MFB_ERR_INVALID_ARGUMENT, "layer weights are NULL");
    MFB_REQUIRE(!need_router || w->router_w != nullptr, MFB_ERR_INVALID_ARGUMENT, "router weights are NULL");
    MFB_REQUIRE(w->pool != nullptr, MFB_ERR_INVALID_ARGUMENT, "expert pool is NULL");
    MFB_REQUIRE(((uintptr_t)w->pool % 16) == 0 && (w->slot_stride % 16) == 0, MFB_ERR_INVALID_ARGUMENT,
                "pool base and slot stride must be multiples of 16 bytes");
    MFB_REQUIRE(offsets_aligned(w->routed_off), MFB_ERR_INVALID_ARGUMENT, "routed expert offsets must be multiples of 16 bytes");
    MFB_REQUIRE((w->router_scales == nullptr) == (w->router_biases == nullptr), MFB_ERR_INVALID_ARGUMENT,
                "an INT8 gate needs both router_scales and router_biases");
    MFB_REQUIRE(!w->router_scales || !w->logit_bias, MFB_ERR_INVALID_ARGUMENT, "logit_bias is not supported with an INT8 gate");
    MFB_REQUIRE(!w->shared_gate_w || (w->shared_gate_s && w->shared_gate_b), MFB_ERR_INVALID_ARGUMENT,
                "the shared-expert gate needs its scales and biases");
    MFB_REQUIRE(w->gate_group_size == 0 || w->gate_group_size == 64 || w->gate_group_size == 32, MFB_ERR_INVALID_ARGUMENT,
                "gate_group_size must be 0, 32 or 64");
    if (w->shared_blob) {
        MFB_REQUIRE(m->cfg.shared_bits != 0, MFB_ERR_INVALID_ARGUMENT, "shared blob given but the handle has shared_bits = 0");
        MFB_REQUIRE(((uintptr_t)w->shared_blob % 16) == 0 && offsets_aligned(w->shared_off), MFB_ERR_INVALID_ARGUMENT,
                    "shared expert blob and offsets must be multiples of 16 bytes");
    }
    return MFB_OK;
}

uint32_t all_slots(const mfb_moe* m) { return (1u << m->cfg.top_k) - 1u; }

// A layer whose routed gate_proj uses 32-element scale groups takes the generic kernels.
bool gate64(const mfb_layer_weights* w) { return w->gate_group_size == 0 || w->gate_group_size == 64; }

bool use_fast(const mfb_moe* m, uint32_t n_tokens) {
    return m->a.xp != nullptr && n_tokens <= FAST_MAX_TOKENS && (uint64_t)n_tokens * m->cfg.top_k <= 1024 &&
           !m->force_generic && fast_smem2(m->cfg, n_tokens) <= FAST_SMEM_LIMIT && fast_smem1(m->cfg) <= FAST_SMEM_LIMIT;
}

FastParams fast_params(mfb_moe* m, const mfb_layer_weights* w, uint32_t n_tokens, const uint16_t* route_w,
                       const void* residual, void* y, const WideMaps* maps) {
    const mfb_moe_config& c = m->cfg;
    Arena& a = m->a;
    FastParams P;
    P.pool = w->pool; P.slot_stride = w->slot_stride; P.slot_of = w->slot_of; P.shared_blob = w->shared_blob;
    P.routed_off = w->routed_off; P.shared_off = w->shared_off;
    P.d = c.d; P.f = c.f; P.num_experts = c.num_experts; P.top_k = c.top_k; P.bits = c.bits; P.shared_bits = c.shared_bits;
    P.scale_dtype = c.scale_dtype; P.activation = c.activation; P.limit = c.swiglu_limit;
    P.sorted = a.sorted; P.groups = a.groups; P.n_groups = a.n_groups;
    P.xp = a.xp; P.xp_shared = a.xp2 ? a.xp2 : a.xp; P.x_in_smem = 0; P.dbg = nullptr; P.actp = a.actp; P.partial = a.partial; P.route_w = route_w;
    P.residual = residual; P.y = y; P.x_dtype = (int)c.x_dtype; P.n_tokens = n_tokens; P.status = a.status;
    P.maps = maps;
    P.ready = nullptr;   // separate launches are ordered by the stream
    return P;
}

// Tensor maps of the layers a handle has been given, for the row-stationary decode phases.  A layer is recognised by
// the fields the maps are built from; its maps live in one slot of a device array allocated when the handle is
// created.  Slots are recycled oldest first, never one that the current call already uses.
struct WideKey {
    const void* pool; uint64_t slot_stride; const void* shared_blob; uint32_t has_table;
    mfb_expert_offsets routed_off, shared_off;
};
struct WideCache {
    WideMaps* dev = nullptr;
    std::vector<WideKey> keys;
    std::vector<uint64_t> stamp;   // call counter of the last use, 0 = empty
    uint64_t call = 0;
    uint32_t cap = 0;
};

WideKey wide_key(const mfb_layer_weights* w) {
    WideKey k;
    memset(&k, 0, sizeof k);
    k.pool = w->pool; k.slot_stride = w->slot_stride; k.shared_blob = w->shared_blob; k.has_table = w->slot_of != nullptr;
    k.routed_off = w->routed_off;
    if (w->shared_blob) k.shared_off = w->shared_off;
    return k;
}

// Device pointer to the maps of layer `w` (built and uploaded on `s` when the layer is new); *out = NULL when the
// handle has no row-stationary form.  Calls of one mfb_* entry share one `call` number (begin_wide_call).
int32_t wide_maps_for(mfb_moe* m, cudaStream_t s, const mfb_layer_weights* w, const WideMaps** out) {
    *out = nullptr;
    WideCache* wc = static_cast<WideCache*>(m->wide_cache);
    if (!wc) return MFB_OK;
    const WideKey k = wide_key(w);
    uint32_t victim = 0;
    uint64_t oldest = ~0ull;
    for (uint32_t i = 0; i < wc->cap; ++i) {
        if (wc->stamp[i] && memcmp(&wc->keys[i], &k, sizeof k) == 0) {
            wc->stamp[i] = wc->call;
            *out = wc->dev + i;
            return MFB_OK;
        }
        if (wc->stamp[i] < oldest) { oldest = wc->stamp[i]; victim = i; }
    }
    MFB_REQUIRE(oldest < wc->call, MFB_ERR_CAPACITY, "more than %u distinct layers in one call (mfb_moe_config.max_layers)", wc->cap);
    WideMaps host;
    const int32_t rc = wide_encode_maps(m->cfg, *w, &host);
    if (rc) return rc;
    // pageable source: the runtime stages it before returning
    MFB_CUDA(cudaMemcpyAsync(wc->dev + victim, &host, sizeof host, cudaMemcpyHostToDevice, s));
    wc->keys[victim] = k;
    wc->stamp[victim] = wc->call;
    *out = wc->dev + victim;
    return MFB_OK;
}

void begin_wide_call(mfb_moe* m) {
    if (m->wide_cache) ++static_cast<WideCache*>(m->wide_cache)->call;
}

// Gate logits of a layer into `logits`: the bf16 gate, or the INT8 affine gate when the layer carries one.
cudaError_t layer_logits(mfb_moe* m, cudaStream_t s, const mfb_layer_weights* w, const void* x, uint32_t ldx, uint32_t n_tokens,
                         float* logits) {
    const mfb_moe_config& c = m->cfg;
    if (w->router_scales)
        return launch_gemv_int8(s, (const uint8_t*)w->router_w, w->router_scales, w->router_biases, x, (int)c.x_dtype, ldx, n_tokens,
                                w->router_effective_scale, c.num_experts, c.d, logits);
    return launch_router_logits(s, x, (int)c.x_dtype, ldx, n_tokens, (const __nv_bfloat16*)w->router_w, c.num_experts, c.d,
                                w->logit_bias, logits, m->a.router_ws, m->a.router_ws_floats);
}

// Qwen shared-expert scalar gate: the shared expert's fp32 row of every token (rank slot top_k of `partial`) times
// sigmoid(fp16(g . x)).  The gate logits use the head of the logits scratch, which the router no longer needs.
cudaError_t apply_shared_gate(mfb_moe* m, cudaStream_t s, const mfb_layer_weights* w, const void* x, uint32_t ldx, uint32_t n_tokens,
                              float* partial, uint32_t slots) {
    if (!w->shared_gate_w || !w->shared_blob || n_tokens == 0) return cudaSuccess;
    const mfb_moe_config& c = m->cfg;
    cudaError_t e = launch_gemv_int8(s, (const uint8_t*)w->shared_gate_w, w->shared_gate_s, w->shared_gate_b, x, (int)c.x_dtype, ldx,
                                     n_tokens, nullptr, 1, c.d, m->a.logits);
    if (e != cudaSuccess) return e;
    return launch_shared_gate_scale(s, m->a.logits, partial + (size_t)c.top_k * c.d, (uint64_t)slots * c.d, n_tokens, c.d);
}

uint32_t max_groups_for(const mfb_moe* m, uint32_t n_tokens, bool shared) {
    const uint64_t pairs = (uint64_t)n_tokens * m->cfg.top_k;
    return (uint32_t)(pairs < m->cfg.num_experts ? pairs : m->cfg.num_experts) + (shared ? 1u : 0u);
}

int32_t run_experts(mfb_moe* m, cudaStream_t s, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                    uint32_t n_tokens, const uint32_t* idx, const uint16_t* route_w, uint32_t slot_mask, bool with_shared) {
    const mfb_moe_config& c = m->cfg;
    Arena& a = m->a;
    const bool shared = with_shared && w->shared_blob != nullptr;
    MFB_CUDA(launch_group(s, idx, route_w, n_tokens, c.top_k, c.num_experts, slot_mask, shared ? 1 : 0, 0, a, a.sorted,
                          a.offsets, a.counts, a.groups, a.n_groups, nullptr));
    DecodeArgs d;
    d.w = w; d.d = c.d; d.f = c.f; d.num_experts = c.num_experts; d.top_k = c.top_k; d.bits = c.bits;
    d.shared_bits = c.shared_bits; d.scale_dtype = c.scale_dtype; d.activation = c.activation;
    d.swiglu_limit = c.swiglu_limit; d.x = x; d.x_dtype = (int)c.x_dtype; d.ldx = ldx; d.sorted = a.sorted;
    d.groups = a.groups; d.n_groups = a.n_groups;
    const uint64_t pairs = (uint64_t)n_tokens * c.top_k;
    d.max_groups = (uint32_t)(pairs < c.num_experts ? pairs : c.num_experts) + (shared ? 1u : 0u);
    d.acts = a.acts; d.partial = a.partial; d.slots = c.top_k + 1;
    MFB_CUDA(launch_decode_ffn(s, d));
    return MFB_OK;
}

}  // namespace
}  // namespace mfb

using namespace mfb;

extern "C" const char* mfb_last_error(void) { return g_error; }
extern "C" int32_t mfb_version(void) { return 100; }
extern "C" uint64_t mfb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int32_t mfb_expert_layout(uint32_t bits, uint32_t d, uint32_t f, mfb_expert_offsets* off, uint64_t* blob_bytes) {
    return mfb_expert_layout_gate(bits, d, f, 64, off, blob_bytes);
}

extern "C" int32_t mfb_expert_layout_gate(uint32_t bits, uint32_t d, uint32_t f, uint32_t gate_group_size, mfb_expert_offsets* off,
                                          uint64_t* blob_bytes) {
    MFB_REQUIRE(off && blob_bytes, MFB_ERR_INVALID_ARGUMENT, "layout: NULL output");
    MFB_REQUIRE(gate_group_size == 64 || gate_group_size == 32, MFB_ERR_INVALID_ARGUMENT, "layout: gate group size must be 32 or 64");
    MFB_REQUIRE(bits == 4 || bits == 2 || bits == 8, MFB_ERR_INVALID_ARGUMENT, "layout: bits must be 2, 4 or 8");
    MFB_REQUIRE(d && f && d % 64 == 0 && f % 64 == 0, MFB_ERR_INVALID_ARGUMENT, "layout: d and f must be multiples of 64");
    const uint64_t wbytes = (uint64_t)d * f * bits / 8, sbytes = (uint64_t)d * f / 64 * 2, gbytes = (uint64_t)d * f / gate_group_size * 2;
    MFB_REQUIRE(3 * (wbytes + 2 * sbytes) + 2 * (gbytes - sbytes) <= 0xFFFFFFFFull, MFB_ERR_UNSUPPORTED_SHAPE, "layout: blob exceeds 4 GiB");
    uint32_t o = 0;
    uint32_t* p = &off->gate_w;
    for (int i = 0; i < 9; ++i) { p[i] = o; o += (uint32_t)(i % 3 == 0 ? wbytes : (i < 3 ? gbytes : sbytes)); }
    *blob_bytes = o;
    return MFB_OK;
}

extern "C" int32_t mfb_moe_create(const mfb_moe_config* cfg, mfb_moe** out) {
    MFB_REQUIRE(cfg && out, MFB_ERR_INVALID_ARGUMENT, "create: NULL argument");
    *out = nullptr;
    const mfb_moe_config& c = *cfg;
    MFB_REQUIRE(c.d && c.f && c.d % 64 == 0 && c.f % 64 == 0, MFB_ERR_INVALID_ARGUMENT, "d and f must be multiples of 64");
    MFB_REQUIRE(c.group_size == 64, MFB_ERR_UNSUPPORTED_SHAPE, "group size must be 64");
    MFB_REQUIRE(c.bits == 4 || c.bits == 2, MFB_ERR_INVALID_ARGUMENT, "bits must be 4 or 2");
    // 8-bit codes for the shared expert only (SharedExpertInt8, Sources/Mference/Kernels/MoE/SharedExpertInt8.swift): such
    // a handle runs the generic kernels
    MFB_REQUIRE(c.shared_bits == 0 || c.shared_bits == 4 || c.shared_bits == 2 || c.shared_bits == 8, MFB_ERR_INVALID_ARGUMENT,
                "shared_bits must be 0, 2, 4 or 8");
    MFB_REQUIRE(c.num_experts >= 1 && c.num_experts <= MFB_MAX_EXPERTS, MFB_ERR_UNSUPPORTED_SHAPE, "num_experts must be in 1..%d", MFB_MAX_EXPERTS);
    MFB_REQUIRE(c.top_k >= 1 && c.top_k <= MFB_MAX_TOP_K, MFB_ERR_UNSUPPORTED_SHAPE, "top_k must be in 1..%d", MFB_MAX_TOP_K);
    MFB_REQUIRE(c.scale_dtype == MFB_DT_F16 || c.scale_dtype == MFB_DT_BF16, MFB_ERR_INVALID_ARGUMENT, "scale dtype must be fp16 or bf16");
    MFB_REQUIRE(c.x_dtype == MFB_DT_F16 || c.x_dtype == MFB_DT_BF16, MFB_ERR_INVALID_ARGUMENT, "activation dtype must be fp16 or bf16");
    MFB_REQUIRE(c.activation <= MFB_ACT_GELU_TANH && c.router_mode <= MFB_ROUTER_SQRTSOFTPLUS, MFB_ERR_INVALID_ARGUMENT, "activation / router mode");
    MFB_REQUIRE(c.max_tokens >= 1, MFB_ERR_INVALID_ARGUMENT, "max_tokens must be positive");
    const uint32_t widths[2] = {c.bits, c.shared_bits};
    for (uint32_t b : widths) {
        if (!b) continue;
        MFB_REQUIRE(pow2_or_wide(c.d, b) && pow2_or_wide(c.f, b), MFB_ERR_UNSUPPORTED_SHAPE,
                    "a row of d or f codes must span a power-of-two number of 16-byte pieces, or at least 32");
    }
    int count = 0;
    MFB_CUDA(cudaGetDeviceCount(&count));
    MFB_REQUIRE(count > 0, MFB_ERR_CUDA, "no CUDA device");

    mfb_moe* m = new (std::nothrow) mfb_moe();
    MFB_REQUIRE(m != nullptr, MFB_ERR_ALLOC, "out of host memory");
    m->cfg = c;
    if (m->cfg.rms_eps <= 0.0f) m->cfg.rms_eps = 1e-6f;
    if (m->cfg.max_layers == 0) m->cfg.max_layers = 64;
    cudaGetDevice(&m->device);
    cudaDeviceGetAttribute(&m->sm_count, cudaDevAttrMultiProcessorCount, m->device);
    const uint64_t T = c.max_tokens, K = c.top_k, E = c.num_experts;
    m->max_pairs = T * K;
    m->max_rows = T * (K + 1);
    Arena& a = m->a;
    a.n_chunks = (uint32_t)((m->max_pairs + GROUP_CHUNK - 1) / GROUP_CHUNK);
    cudaError_t e = cudaSuccess;
    auto ok = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    ok(dev_alloc(a.logits, T * E));
    a.router_ws_floats = router_workspace_floats(c.max_tokens, c.num_experts, c.d);
    if (a.router_ws_floats) { ok(dev_alloc(a.router_ws, a.router_ws_floats)); ok(router_init()); }
    ok(dev_alloc(a.idx, T * K));
    ok(dev_alloc(a.route_w, T * K));
    { uint16_t* p = nullptr; ok(dev_alloc(p, T * c.d)); a.xn = p; }
    ok(dev_alloc(a.sorted, m->max_rows));
    ok(dev_alloc(a.chunk_hist, (uint64_t)a.n_chunks * E));
    ok(dev_alloc(a.offsets, E));
    ok(dev_alloc(a.counts, E));
    ok(dev_alloc(a.groups, E + 1));
    ok(dev_alloc(a.n_groups, 1));
    ok(dev_alloc(a.tile_prefix, E + 2));
    ok(dev_alloc(a.acts, m->max_rows * c.f));
    ok(dev_alloc(a.partial, m->max_rows * c.d));
    ok(dev_alloc(a.status, 1));
    if (fast_supported(c)) {
        int coop = 0;
        cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, m->device);
        m->coop = coop != 0;
        ok(fast_init());
        ok(dev_alloc(m->mega_bar, MEGA_BAR_WORDS));
        const uint64_t ft = T < FAST_MAX_TOKENS ? T : FAST_MAX_TOKENS;
        ok(dev_alloc(a.xp, ft * c.d));
        if (c.shared_bits && c.shared_bits != c.bits) ok(dev_alloc(a.xp2, ft * c.d));
        ok(dev_alloc(a.actp, ft * (K + 1) * c.f));
        // everything a stack call needs is allocated here, so that no later call allocates: the per-layer weight
        // table of the fused kernel and, for shapes with a row-stationary form, the tensor maps of max_layers layers
        const uint32_t cap = m->cfg.max_layers;
        { MegaLayer* p = nullptr; ok(dev_alloc(p, cap)); m->mega_dev = p; }
        m->mega_host = calloc(cap, sizeof(MegaLayer));
        if (!m->mega_host) ok(cudaErrorMemoryAllocation);
        m->mega_cap = cap;
        if (wide_supported(c)) {
            WideCache* wc = new (std::nothrow) WideCache();
            if (!wc) ok(cudaErrorMemoryAllocation);
            else {
                m->wide_cache = wc;
                wc->cap = cap;
                wc->keys.resize(cap);
                wc->stamp.assign(cap, 0);
                ok(dev_alloc(wc->dev, cap));
            }
        }
        // a cooperative launch needs one CTA per SM resident at once: otherwise stacks run layer by layer
        if (m->coop && e == cudaSuccess && !stack_mega_fits(c, m->sm_count, fast_smem_stack(c, (uint32_t)ft, m->wide_cache != nullptr))) m->coop = false;
    }
    if (c.flags & MFB_FLAG_PREFILL_TENSOR_CORE) {
        const uint64_t rows = m->max_rows + TC_ROW_PAD;
        ok(dev_alloc(a.xs16, rows * c.d));
        ok(dev_alloc(a.acts16, rows * c.f));
    }
    if (e == cudaSuccess) e = cudaMemset(a.status, 0, sizeof(uint32_t));
    if (e == cudaSuccess && a.xs16) e = cudaMemset(a.xs16, 0, (m->max_rows + TC_ROW_PAD) * c.d * sizeof(__half));
    if (e == cudaSuccess && a.acts16) e = cudaMemset(a.acts16, 0, (m->max_rows + TC_ROW_PAD) * c.f * sizeof(__half));
    if (e != cudaSuccess) {
        set_error("arena allocation failed: %s", cudaGetErrorString(e));
        mfb_moe_destroy(m);
        return e == cudaErrorMemoryAllocation ? MFB_ERR_ALLOC : MFB_ERR_CUDA;
    }
    if (c.flags & MFB_FLAG_PREFILL_TENSOR_CORE) {
        const int32_t rc = tc_init(m);
        if (rc) { mfb_moe_destroy(m); return rc; }
    }
    *out = m;
    return MFB_OK;
}

extern "C" int32_t mfb_moe_destroy(mfb_moe* moe) {
    if (!moe) return MFB_OK;
    tc_release(moe);
    free_arena(moe->a);
    if (moe->wide_cache) {
        WideCache* wc = static_cast<WideCache*>(moe->wide_cache);
        cudaFree(wc->dev);
        delete wc;
    }
    cudaFree(moe->mega_dev);
    cudaFree(moe->mega_bar);
    free(moe->mega_host);
    delete moe;
    return MFB_OK;
}

extern "C" int32_t mfb_moe_set_generic(mfb_moe* moe, int32_t on) {
    MFB_REQUIRE(moe != nullptr, MFB_ERR_INVALID_ARGUMENT, "handle is NULL");
    moe->force_generic = on == 1;
    moe->no_fused = on == 2;
    return MFB_OK;
}

extern "C" int32_t mfb_moe_set_trace(mfb_moe* moe, uint64_t* device_stamps) {
    MFB_REQUIRE(moe != nullptr, MFB_ERR_INVALID_ARGUMENT, "handle is NULL");
    moe->trace = device_stamps;
    return MFB_OK;
}

extern "C" int32_t mfb_moe_device_status(mfb_moe* moe, void* stream, uint32_t* status) {
    MFB_REQUIRE(moe && status, MFB_ERR_INVALID_ARGUMENT, "device_status: NULL argument");
    MFB_CUDA(cudaMemcpyAsync(status, moe->a.status, sizeof(uint32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    MFB_CUDA(cudaMemsetAsync(moe->a.status, 0, sizeof(uint32_t), (cudaStream_t)stream));
    MFB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    if (*status) { set_error("device status word = 0x%x", *status); return MFB_ERR_DEVICE_STATUS; }
    return MFB_OK;
}

extern "C" int32_t mfb_moe_partial_rows(mfb_moe* moe, const float** rows) {
    MFB_REQUIRE(moe && rows, MFB_ERR_INVALID_ARGUMENT, "partial_rows: NULL argument");
    *rows = moe->a.partial;
    return MFB_OK;
}

extern "C" int32_t mfb_moe_selftest_wait(mfb_moe* moe, void* stream, uint64_t limit_cycles) {
    MFB_REQUIRE(moe != nullptr, MFB_ERR_INVALID_ARGUMENT, "handle is NULL");
    MFB_REQUIRE(limit_cycles >= 1 && limit_cycles <= 20000000ull, MFB_ERR_INVALID_ARGUMENT,
                "selftest_wait: limit must be 1..20,000,000 cycles (about 10 ms)");
    MFB_CUDA(launch_wait_selftest((cudaStream_t)stream, moe->a.status, (long long)limit_cycles));
    return MFB_OK;
}

// ------------------------------------------------------------------------------------------------- router

extern "C" int32_t mfb_router_logits(mfb_moe* moe, void* stream, const void* x, uint32_t ldx, uint32_t n_tokens,
                                     const void* router_w, const float* logit_bias, float* logits) {
    int32_t rc = check_handle(moe, 0);
    if (rc) return rc;
    MFB_REQUIRE(x && router_w && logits, MFB_ERR_INVALID_ARGUMENT, "router_logits: NULL argument");
    MFB_REQUIRE(ldx >= moe->cfg.d, MFB_ERR_INVALID_ARGUMENT, "router_logits: row stride smaller than d");
    MFB_CUDA(launch_router_logits((cudaStream_t)stream, x, (int)moe->cfg.x_dtype, ldx, n_tokens,
                                  (const __nv_bfloat16*)router_w, moe->cfg.num_experts, moe->cfg.d, logit_bias, logits,
                                  moe->a.router_ws, moe->a.router_ws_floats));
    return MFB_OK;
}

extern "C" int32_t mfb_router_select(mfb_moe* moe, void* stream, const float* logits, uint32_t n_tokens,
                                     const void* per_expert_scale, const float* correction_bias, uint32_t* out_idx,
                                     uint16_t* out_w) {
    int32_t rc = check_handle(moe, 0);
    if (rc) return rc;
    MFB_REQUIRE(logits && out_idx && out_w, MFB_ERR_INVALID_ARGUMENT, "router_select: NULL argument");
    const mfb_moe_config& c = moe->cfg;
    MFB_CUDA(launch_router_select((cudaStream_t)stream, logits, n_tokens, c.num_experts, c.top_k, (int)c.router_mode,
                                  (const __nv_bfloat16*)per_expert_scale, correction_bias, c.route_scale, out_idx, out_w));
    return MFB_OK;
}

extern "C" int32_t mfb_router_topk(mfb_moe* moe, void* stream, const void* x, uint32_t ldx, uint32_t n_tokens,
                                   const mfb_layer_weights* w, uint32_t* out_idx, uint16_t* out_w) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    MFB_REQUIRE(w && w->router_w && x && out_idx && out_w, MFB_ERR_INVALID_ARGUMENT, "router_topk: NULL argument");
    MFB_REQUIRE(ldx >= moe->cfg.d, MFB_ERR_INVALID_ARGUMENT, "router_topk: row stride smaller than d");
    MFB_REQUIRE((w->router_scales == nullptr) == (w->router_biases == nullptr) && !(w->router_scales && w->logit_bias),
                MFB_ERR_INVALID_ARGUMENT, "router_topk: an INT8 gate needs scales and biases and takes no logit bias");
    MFB_CUDA(layer_logits(moe, (cudaStream_t)stream, w, x, ldx, n_tokens, moe->a.logits));
    return mfb_router_select(moe, stream, moe->a.logits, n_tokens, w->per_expert_scale, w->correction_bias, out_idx, out_w);
}

extern "C" int32_t mfb_slot_lookup(mfb_moe* moe, void* stream, const uint32_t* idx, uint32_t n_tokens,
                                   const int16_t* slot_of, uint64_t slot_stride, uint64_t* out_offsets,
                                   uint32_t* out_all_hit) {
    int32_t rc = check_handle(moe, 0);
    if (rc) return rc;
    MFB_REQUIRE(idx && slot_of && out_offsets && out_all_hit, MFB_ERR_INVALID_ARGUMENT, "slot_lookup: NULL argument");
    MFB_CUDA(launch_slot_lookup((cudaStream_t)stream, idx, n_tokens, moe->cfg.top_k, moe->cfg.num_experts, slot_of,
                                slot_stride, out_offsets, out_all_hit));
    return MFB_OK;
}

// ------------------------------------------------------------------------------------------------- decode

extern "C" int32_t mfb_moe_experts(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                                   uint32_t n_tokens, const uint32_t* idx, const uint16_t* route_w,
                                   const uint32_t* active_slots, uint32_t active_count, int32_t with_shared) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    rc = check_weights(moe, w, false);
    if (rc) return rc;
    MFB_REQUIRE(x && idx && route_w, MFB_ERR_INVALID_ARGUMENT, "experts: NULL argument");
    MFB_REQUIRE(ldx >= moe->cfg.d, MFB_ERR_INVALID_ARGUMENT, "experts: row stride smaller than d");
    uint32_t mask = all_slots(moe);
    if (active_slots) {
        mask = 0;
        for (uint32_t i = 0; i < active_count; ++i) {
            MFB_REQUIRE(active_slots[i] < moe->cfg.top_k, MFB_ERR_INVALID_ARGUMENT, "experts: active slot %u out of range", active_slots[i]);
            mask |= 1u << active_slots[i];
        }
    }
    if (n_tokens == 0) return MFB_OK;
    rc = run_experts(moe, (cudaStream_t)stream, w, x, ldx, n_tokens, idx, route_w, mask, with_shared != 0);
    if (rc) return rc;
    if (with_shared) MFB_CUDA(apply_shared_gate(moe, (cudaStream_t)stream, w, x, ldx, n_tokens, moe->a.partial, moe->cfg.top_k + 1));
    return MFB_OK;
}

extern "C" int32_t mfb_moe_combine(mfb_moe* moe, void* stream, uint32_t n_tokens, const uint16_t* route_w,
                                   int32_t with_shared, const void* residual, void* y) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    MFB_REQUIRE(route_w && y, MFB_ERR_INVALID_ARGUMENT, "combine: NULL argument");
    const mfb_moe_config& c = moe->cfg;
    MFB_CUDA(launch_combine((cudaStream_t)stream, moe->a.partial, route_w, n_tokens, c.top_k, c.top_k + 1, c.d,
                            all_slots(moe), with_shared != 0, residual, y, (int)c.x_dtype));
    return MFB_OK;
}

extern "C" int32_t mfb_moe_decode(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                                  uint32_t n_tokens, const uint32_t* idx, const uint16_t* route_w, const void* residual,
                                  void* y) {
    int32_t rc = check_handle(moe, n_tokens);   // capacity first: the fast path below writes n_tokens rows of the arena
    if (rc) return rc;
    if (w && x && idx && route_w && y && n_tokens && use_fast(moe, n_tokens) && gate64(w) && ldx == moe->cfg.d) {
        rc = check_weights(moe, w, false);
        if (rc) return rc;
        const mfb_moe_config& c = moe->cfg;
        Arena& a = moe->a;
        cudaStream_t s = (cudaStream_t)stream;
        const bool shared = w->shared_blob != nullptr;
        MFB_CUDA(launch_fast_prep(s, x, (int)c.x_dtype, nullptr, n_tokens, c.d, c.rms_eps, false, nullptr, a.xp, c.bits, a.xp2, c.shared_bits));
        MFB_CUDA(launch_group(s, idx, route_w, n_tokens, c.top_k, c.num_experts, all_slots(moe), shared ? 1 : 0, 0, a, a.sorted,
                              a.offsets, a.counts, a.groups, a.n_groups, nullptr));
        const WideMaps* maps = nullptr;
        begin_wide_call(moe);
        if (n_tokens > 16 && (rc = wide_maps_for(moe, s, w, &maps)) != MFB_OK) return rc;
        const FastParams P = fast_params(moe, w, n_tokens, route_w, residual, y, maps);
        MFB_CUDA(launch_fast_ffn(s, P, c, moe->sm_count, max_groups_for(moe, n_tokens, shared)));
        MFB_CUDA(apply_shared_gate(moe, s, w, x, ldx, n_tokens, a.partial, c.top_k + 1));
        MFB_CUDA(launch_combine(s, a.partial, route_w, n_tokens, c.top_k, c.top_k + 1, c.d, all_slots(moe), shared, residual, y,
                                (int)c.x_dtype));
        return MFB_OK;
    }
    rc = mfb_moe_experts(moe, stream, w, x, ldx, n_tokens, idx, route_w, nullptr, 0, 1);
    if (rc) return rc;
    return mfb_moe_combine(moe, stream, n_tokens, route_w, w->shared_blob != nullptr, residual, y);
}

extern "C" int32_t mfb_moe_layer(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* h_in, void* h_out,
                                 uint32_t n_tokens) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    rc = check_weights(moe, w, true);
    if (rc) return rc;
    MFB_REQUIRE(h_in && h_out, MFB_ERR_INVALID_ARGUMENT, "layer: NULL argument");
    if (n_tokens == 0) return MFB_OK;
    const mfb_moe_config& c = moe->cfg;
    Arena& a = moe->a;
    cudaStream_t s = (cudaStream_t)stream;
    if (use_fast(moe, n_tokens) && gate64(w)) {
        const bool shared = w->shared_blob != nullptr;
        MFB_CUDA(launch_fast_prep(s, h_in, (int)c.x_dtype, (const __nv_bfloat16*)w->norm_w, n_tokens, c.d, c.rms_eps, true, a.xn,
                                  a.xp, c.bits, a.xp2, c.shared_bits));
        MFB_CUDA(layer_logits(moe, s, w, a.xn, c.d, n_tokens, a.logits));
        MFB_CUDA(launch_route_small(s, a.logits, n_tokens, c.num_experts, c.top_k, (int)c.router_mode,
                                    (const __nv_bfloat16*)w->per_expert_scale, w->correction_bias, c.route_scale, shared ? 1 : 0,
                                    a.idx, a.route_w, a.sorted, a.groups, a.n_groups));
        const WideMaps* maps = nullptr;
        begin_wide_call(moe);
        if (n_tokens > 16 && (rc = wide_maps_for(moe, s, w, &maps)) != MFB_OK) return rc;
        const FastParams P = fast_params(moe, w, n_tokens, a.route_w, h_in, h_out, maps);
        MFB_CUDA(launch_fast_ffn(s, P, c, moe->sm_count, max_groups_for(moe, n_tokens, shared)));
        MFB_CUDA(apply_shared_gate(moe, s, w, a.xn, c.d, n_tokens, a.partial, c.top_k + 1));
        MFB_CUDA(launch_combine(s, a.partial, a.route_w, n_tokens, c.top_k, c.top_k + 1, c.d, all_slots(moe), shared, h_in, h_out,
                                (int)c.x_dtype));
        return MFB_OK;
    }
    MFB_CUDA(launch_rmsnorm(s, h_in, (int)c.x_dtype, (const __nv_bfloat16*)w->norm_w, n_tokens, c.d, c.rms_eps, a.xn, (int)c.x_dtype));
    rc = mfb_router_topk(moe, stream, a.xn, c.d, n_tokens, w, a.idx, a.route_w);
    if (rc) return rc;
    return mfb_moe_decode(moe, stream, w, a.xn, c.d, n_tokens, a.idx, a.route_w, h_in, h_out);
}

// Builds (or reuses) the device table of per-layer weights for the fused stack kernel.  *all_maps: every layer has
// tensor maps (the row-stationary phases may run).
static int32_t upload_layer_table(mfb_moe* m, cudaStream_t s, const mfb_layer_weights* layers, uint32_t n_layers, bool want_maps,
                                  bool* all_maps) {
    MFB_REQUIRE(n_layers <= m->mega_cap, MFB_ERR_CAPACITY, "%u layers exceed mfb_moe_config.max_layers = %u", n_layers, m->mega_cap);
    std::vector<MegaLayer> host(n_layers);
    *all_maps = want_maps && m->wide_cache != nullptr;
    begin_wide_call(m);
    for (uint32_t l = 0; l < n_layers; ++l) {
        const mfb_layer_weights& w = layers[l];
        MegaLayer& o = host[l];
        memset(&o, 0, sizeof o);
        o.router_w = (const __nv_bfloat16*)w.router_w; o.logit_bias = w.logit_bias;
        o.per_expert_scale = (const __nv_bfloat16*)w.per_expert_scale; o.correction_bias = w.correction_bias;
        o.norm_w = (const __nv_bfloat16*)w.norm_w; o.pool = w.pool; o.slot_stride = w.slot_stride; o.slot_of = w.slot_of;
        o.shared_blob = w.shared_blob; o.routed_off = w.routed_off; o.shared_off = w.shared_off;
        if (*all_maps) {
            const int32_t rc = wide_maps_for(m, s, &w, &o.maps);
            if (rc) return rc;
        }
    }
    const size_t bytes = (size_t)n_layers * sizeof(MegaLayer);
    if (m->mega_count == n_layers && memcmp(m->mega_host, host.data(), bytes) == 0) return MFB_OK;
    memcpy(m->mega_host, host.data(), bytes);
    m->mega_count = n_layers;
    // the source is pageable host memory: the runtime stages it before returning, so reusing mega_host is safe
    MFB_CUDA(cudaMemcpyAsync(m->mega_dev, m->mega_host, bytes, cudaMemcpyHostToDevice, s));
    return MFB_OK;
}

extern "C" int32_t mfb_moe_stack_rows(mfb_moe* moe, void* stream, const mfb_layer_weights* layers, uint32_t n_layers,
                                      void* rows, uint64_t layer_stride, uint32_t n_tokens) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    MFB_REQUIRE(layers != nullptr || n_layers == 0, MFB_ERR_INVALID_ARGUMENT, "stack: layers is NULL");
    MFB_REQUIRE(rows != nullptr, MFB_ERR_INVALID_ARGUMENT, "stack: rows is NULL");
    MFB_REQUIRE(layer_stride == 0 || layer_stride >= (uint64_t)n_tokens * moe->cfg.d, MFB_ERR_INVALID_ARGUMENT,
                "stack: layer stride smaller than one layer's rows");
    if (n_layers == 0 || n_tokens == 0) return MFB_OK;
    const mfb_moe_config& c = moe->cfg;
    cudaStream_t s = (cudaStream_t)stream;
    const bool want_maps = n_tokens > 16 && moe->wide_cache != nullptr;
    bool plain = true;   // the fused kernel computes the bf16 gate itself and has no scalar gate on the shared expert
    for (uint32_t l = 0; l < n_layers; ++l) plain = plain && !layers[l].router_scales && !layers[l].shared_gate_w && gate64(&layers[l]);
    if (plain && use_fast(moe, n_tokens) && moe->coop && !moe->no_fused && fast_smem_stack(c, n_tokens, want_maps) <= FAST_SMEM_LIMIT) {
        for (uint32_t l = 0; l < n_layers; ++l) {
            rc = check_weights(moe, &layers[l], true);
            if (rc) return rc;
        }
        bool all_maps = false;
        rc = upload_layer_table(moe, s, layers, n_layers, want_maps, &all_maps);
        if (rc) return rc;
        Arena& a = moe->a;
        MegaParams M;
        M.layers = (const MegaLayer*)moe->mega_dev; M.n_layers = n_layers;
        M.d = c.d; M.f = c.f; M.num_experts = c.num_experts; M.top_k = c.top_k; M.bits = c.bits; M.shared_bits = c.shared_bits;
        M.scale_dtype = c.scale_dtype; M.activation = c.activation; M.router_mode = (int)c.router_mode; M.x_dtype = (int)c.x_dtype;
        M.limit = c.swiglu_limit; M.route_scale = c.route_scale; M.eps = c.rms_eps;
        M.hidden = rows; M.layer_stride = layer_stride; M.n_tokens = n_tokens;
        M.xn = a.xn; M.xp = a.xp; M.xp2 = a.xp2; M.logits = a.logits; M.idx = a.idx; M.route_w = a.route_w; M.actp = a.actp; M.partial = a.partial;
        M.bar_counter = moe->mega_bar; M.abort = moe->mega_bar + 1; M.ready = moe->mega_bar + 2; M.status = a.status; M.trace = moe->trace;
        M.wide = all_maps ? 1 : 0;
        MFB_CUDA(launch_stack_mega(s, M, c, moe->sm_count));
        return MFB_OK;
    }
    for (uint32_t l = 0; l < n_layers; ++l) {
        void* h = (uint8_t*)rows + (size_t)l * layer_stride * 2;
        rc = mfb_moe_layer(moe, stream, &layers[l], h, h, n_tokens);
        if (rc) return rc;
    }
    return MFB_OK;
}

extern "C" int32_t mfb_moe_stack(mfb_moe* moe, void* stream, const mfb_layer_weights* layers, uint32_t n_layers,
                                 void* hidden, uint32_t n_tokens) {
    return mfb_moe_stack_rows(moe, stream, layers, n_layers, hidden, 0, n_tokens);
}

// ------------------------------------------------------------------------------------------------- prefill

extern "C" int32_t mfb_moe_group(mfb_moe* moe, void* stream, const uint32_t* idx, const uint16_t* route_w,
                                 uint32_t n_tokens, mfb_pair* out_sorted, uint32_t* out_offsets, uint32_t* out_counts,
                                 mfb_group* out_groups, uint32_t* out_n_groups) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    MFB_REQUIRE(idx && out_sorted && out_offsets && out_counts && out_groups && out_n_groups, MFB_ERR_INVALID_ARGUMENT,
                "group: NULL argument");
    MFB_CUDA(launch_group((cudaStream_t)stream, idx, route_w, n_tokens, moe->cfg.top_k, moe->cfg.num_experts,
                          all_slots(moe), 0, 0, moe->a, out_sorted, out_offsets, out_counts, out_groups, out_n_groups, nullptr));
    return MFB_OK;
}

extern "C" int32_t mfb_moe_prefill_grouped(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x,
                                           uint32_t ldx, uint32_t n_tokens, const mfb_pair* sorted,
                                           const mfb_group* groups, const uint32_t* n_groups, float* partial) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    rc = check_weights(moe, w, false);
    if (rc) return rc;
    MFB_REQUIRE(x && sorted && groups && n_groups && partial, MFB_ERR_INVALID_ARGUMENT, "prefill_grouped: NULL argument");
    MFB_REQUIRE(ldx >= moe->cfg.d, MFB_ERR_INVALID_ARGUMENT, "prefill_grouped: row stride smaller than d");
    if (n_tokens == 0) return MFB_OK;
    const mfb_moe_config& c = moe->cfg;
    const uint64_t pairs = (uint64_t)n_tokens * c.top_k;
    const uint32_t max_groups = (uint32_t)(pairs < c.num_experts ? pairs : c.num_experts);
    if ((c.flags & MFB_FLAG_PREFILL_TENSOR_CORE) && tc_supported(c) && gate64(w))
        return tc_grouped_ffn(moe, (cudaStream_t)stream, w, x, ldx, n_tokens, sorted, groups, n_groups, max_groups,
                              /*routed_only=*/true, partial, c.top_k);
    DecodeArgs d;
    mfb_layer_weights routed_only = *w;
    routed_only.shared_blob = nullptr;
    d.w = &routed_only; d.d = c.d; d.f = c.f; d.num_experts = c.num_experts; d.top_k = c.top_k; d.bits = c.bits;
    d.shared_bits = c.shared_bits; d.scale_dtype = c.scale_dtype; d.activation = c.activation;
    d.swiglu_limit = c.swiglu_limit; d.x = x; d.x_dtype = (int)c.x_dtype; d.ldx = ldx; d.sorted = sorted;
    d.groups = groups; d.n_groups = n_groups; d.max_groups = max_groups;
    d.acts = moe->a.acts; d.partial = partial; d.slots = c.top_k;
    MFB_CUDA(launch_decode_ffn((cudaStream_t)stream, d));
    return MFB_OK;
}

extern "C" int32_t mfb_moe_prefill_grouped_rows(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x,
                                                uint32_t ldx, uint32_t n_tokens, const mfb_pair* sorted, const mfb_group* groups,
                                                const uint32_t* n_groups, float* const* row_dest) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    rc = check_weights(moe, w, false);
    if (rc) return rc;
    MFB_REQUIRE(x && sorted && groups && n_groups && row_dest, MFB_ERR_INVALID_ARGUMENT, "prefill_grouped_rows: NULL argument");
    MFB_REQUIRE(ldx >= moe->cfg.d, MFB_ERR_INVALID_ARGUMENT, "prefill_grouped_rows: row stride smaller than d");
    const mfb_moe_config& c = moe->cfg;
    MFB_REQUIRE((c.flags & MFB_FLAG_PREFILL_TENSOR_CORE) && tc_supported(c) && gate64(w), MFB_ERR_UNSUPPORTED_SHAPE,
                "prefill_grouped_rows needs the tensor-core path (MFB_FLAG_PREFILL_TENSOR_CORE, d and f multiples of 512, gate group 64)");
    if (n_tokens == 0) return MFB_OK;
    const uint64_t pairs = (uint64_t)n_tokens * c.top_k;
    const uint32_t max_groups = (uint32_t)(pairs < c.num_experts ? pairs : c.num_experts);
    return tc_grouped_ffn(moe, (cudaStream_t)stream, w, x, ldx, n_tokens, sorted, groups, n_groups, max_groups, /*routed_only=*/true,
                          nullptr, c.top_k, row_dest);
}

extern "C" int32_t mfb_moe_prefill_accumulate_f32(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                                                  uint32_t n_tokens, const mfb_pair* sorted, const mfb_group* groups,
                                                  const uint32_t* n_groups, const float* pair_weights, float* acc) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    rc = check_weights(moe, w, false);
    if (rc) return rc;
    MFB_REQUIRE(x && sorted && groups && n_groups && pair_weights && acc, MFB_ERR_INVALID_ARGUMENT, "prefill_accumulate_f32: NULL argument");
    MFB_REQUIRE(ldx >= moe->cfg.d, MFB_ERR_INVALID_ARGUMENT, "prefill_accumulate_f32: row stride smaller than d");
    if (n_tokens == 0) return MFB_OK;
    const mfb_moe_config& c = moe->cfg;
    Arena& a = moe->a;
    const uint64_t pairs = (uint64_t)n_tokens * c.top_k;
    DecodeArgs d;
    mfb_layer_weights routed_only = *w;
    routed_only.shared_blob = nullptr;
    d.w = &routed_only; d.d = c.d; d.f = c.f; d.num_experts = c.num_experts; d.top_k = c.top_k; d.bits = c.bits;
    d.shared_bits = c.shared_bits; d.scale_dtype = c.scale_dtype; d.activation = c.activation;
    d.swiglu_limit = c.swiglu_limit; d.x = x; d.x_dtype = (int)c.x_dtype; d.ldx = ldx; d.sorted = sorted;
    d.groups = groups; d.n_groups = n_groups; d.max_groups = (uint32_t)(pairs < c.num_experts ? pairs : c.num_experts);
    d.acts = a.acts; d.partial = a.partial; d.slots = c.top_k; d.round16 = 1;
    MFB_CUDA(launch_decode_ffn((cudaStream_t)stream, d));
    // the (token, rank) -> expert table lives in the index scratch of the router, which this call does not use
    MFB_CUDA(launch_accumulate_expert_order((cudaStream_t)stream, sorted, groups, n_groups, n_tokens, c.top_k, c.d, a.partial,
                                            pair_weights, a.idx, acc));
    return MFB_OK;
}

extern "C" int32_t mfb_moe_reduce(mfb_moe* moe, void* stream, const float* partial, const uint16_t* route_w,
                                  uint32_t n_tokens, const void* residual, void* y) {
    int32_t rc = check_handle(moe, 0);
    if (rc) return rc;
    MFB_REQUIRE(partial && route_w && y, MFB_ERR_INVALID_ARGUMENT, "reduce: NULL argument");
    const mfb_moe_config& c = moe->cfg;
    MFB_CUDA(launch_combine((cudaStream_t)stream, partial, route_w, n_tokens, c.top_k, c.top_k, c.d, all_slots(moe), 0,
                            residual, y, (int)c.x_dtype));
    return MFB_OK;
}

extern "C" int32_t mfb_moe_layer_prefill(mfb_moe* moe, void* stream, const mfb_layer_weights* w, const void* h_in,
                                         void* h_out, uint32_t n_tokens) {
    int32_t rc = check_handle(moe, n_tokens);
    if (rc) return rc;
    rc = check_weights(moe, w, true);
    if (rc) return rc;
    MFB_REQUIRE(h_in && h_out, MFB_ERR_INVALID_ARGUMENT, "layer_prefill: NULL argument");
    if (n_tokens == 0) return MFB_OK;
    const mfb_moe_config& c = moe->cfg;
    if (!((c.flags & MFB_FLAG_PREFILL_TENSOR_CORE) && tc_supported(c) && gate64(w))) return mfb_moe_layer(moe, stream, w, h_in, h_out, n_tokens);
    Arena& a = moe->a;
    cudaStream_t s = (cudaStream_t)stream;
    MFB_CUDA(launch_rmsnorm(s, h_in, (int)c.x_dtype, (const __nv_bfloat16*)w->norm_w, n_tokens, c.d, c.rms_eps, a.xn, (int)c.x_dtype));
    rc = mfb_router_topk(moe, stream, a.xn, c.d, n_tokens, w, a.idx, a.route_w);
    if (rc) return rc;
    const bool shared = w->shared_blob != nullptr;
    MFB_CUDA(launch_group(s, a.idx, a.route_w, n_tokens, c.top_k, c.num_experts, all_slots(moe), shared ? 1 : 0, TC_TILE_N, a,
                          a.sorted, a.offsets, a.counts, a.groups, a.n_groups, a.tile_prefix));
    const uint64_t pairs = (uint64_t)n_tokens * c.top_k;
    const uint32_t max_groups = (uint32_t)(pairs < c.num_experts ? pairs : c.num_experts) + (shared ? 1u : 0u);
    rc = tc_grouped_ffn(moe, s, w, a.xn, c.d, n_tokens, a.sorted, a.groups, a.n_groups, max_groups, /*routed_only=*/false,
                        a.partial, c.top_k + 1);
    if (rc) return rc;
    MFB_CUDA(apply_shared_gate(moe, s, w, a.xn, c.d, n_tokens, a.partial, c.top_k + 1));
    MFB_CUDA(launch_combine(s, a.partial, a.route_w, n_tokens, c.top_k, c.top_k + 1, c.d, all_slots(moe), shared, h_in, h_out,
                            (int)c.x_dtype));
    return MFB_OK;
}

// ------------------------------------------------------------------------------------------------- glue

extern "C" int32_t mfb_rmsnorm(mfb_moe* moe, void* stream, const void* x, const void* w_bf16, uint32_t n_rows, void* out) {
    int32_t rc = check_handle(moe, 0);
    if (rc) return rc;
    MFB_REQUIRE(x && out, MFB_ERR_INVALID_ARGUMENT, "rmsnorm: NULL argument");
    const mfb_moe_config& c = moe->cfg;
    MFB_CUDA(launch_rmsnorm((cudaStream_t)stream, x, (int)c.x_dtype, (const __nv_bfloat16*)w_bf16, n_rows, c.d, c.rms_eps, out, (int)c.x_dtype));
    return MFB_OK;
}

extern "C" int32_t mfb_residual_add(mfb_moe* moe, void* stream, const void* a, const void* b, uint64_t n, void* out) {
    int32_t rc = check_handle(moe, 0);
    if (rc) return rc;
    MFB_REQUIRE(a && b && out, MFB_ERR_INVALID_ARGUMENT, "residual_add: NULL argument");
    MFB_CUDA(launch_residual_add((cudaStream_t)stream, a, b, n, out, (int)moe->cfg.x_dtype));
    return MFB_OK;
}
