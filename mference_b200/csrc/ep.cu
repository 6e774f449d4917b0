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
#include <new>

#include "common.cuh"

namespace mfb {
namespace {

constexpr int EP_MAX_WORLD = 8;

// One block of EP_PLAN_WARPS warps.  Stable counting sort of the T*K pairs by destination rank: send order =
// (dest, token, rank slot).  perm[pos] = pair id (token * K + slot) at send position pos; inv[pair] = pos; counts[g] =
// pairs bound for rank g; starts[g] = first send position of rank g's block (optional); local_expert[pos] = expert
// id relative to the destination's first expert.  Every warp owns a contiguous chunk of the pairs: per-warp counts,
// a scan over (rank, warp), then an ordered scatter of the chunk 32 pairs at a time - no atomics decide an order.
constexpr int EP_PLAN_WARPS = 32;

__global__ void __launch_bounds__(EP_PLAN_WARPS * 32) ep_plan_kernel(const uint32_t* __restrict__ idx, uint32_t n_pairs,
                                                                      uint32_t experts_per_rank, uint32_t world,
                                                                      uint32_t* __restrict__ perm, uint32_t* __restrict__ inv,
                                                                      int32_t* __restrict__ counts, int32_t* __restrict__ starts,
                                                                      int32_t* __restrict__ local_expert) {
    __shared__ uint32_t cnt[EP_PLAN_WARPS][EP_MAX_WORLD], start[EP_PLAN_WARPS][EP_MAX_WORLD];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t chunk = ((n_pairs + EP_PLAN_WARPS - 1) / EP_PLAN_WARPS + 31) & ~31u;
    const uint32_t p_begin = min(warp * chunk, n_pairs), p_end = min(p_begin + chunk, n_pairs);
    uint32_t mine[EP_MAX_WORLD];
#pragma unroll
    for (int g = 0; g < EP_MAX_WORLD; ++g) mine[g] = 0;
    for (uint32_t p0 = p_begin; p0 < p_end; p0 += 32) {
        const uint32_t p = p0 + lane;
        const uint32_t g = p < p_end ? min(idx[p] / experts_per_rank, world - 1) : 0xFFFFFFFFu;
#pragma unroll
        for (int q = 0; q < EP_MAX_WORLD; ++q) mine[q] += __popc(__ballot_sync(0xFFFFFFFFu, g == (uint32_t)q));
    }
    if (lane == 0)
        for (int g = 0; g < EP_MAX_WORLD; ++g) cnt[warp][g] = mine[g];
    __syncthreads();
    if (threadIdx.x < world) {
        const uint32_t g = threadIdx.x;
        uint32_t base = 0;
        for (uint32_t q = 0; q < g; ++q)
            for (int w = 0; w < EP_PLAN_WARPS; ++w) base += cnt[w][q];
        if (starts) starts[g] = (int32_t)base;
        uint32_t run = base;
        for (int w = 0; w < EP_PLAN_WARPS; ++w) { start[w][g] = run; run += cnt[w][g]; }
        counts[g] = (int32_t)(run - base);
    }
    __syncthreads();
    uint32_t run[EP_MAX_WORLD];
#pragma unroll
    for (int g = 0; g < EP_MAX_WORLD; ++g) run[g] = (uint32_t)g < world ? start[warp][g] : 0u;
    for (uint32_t p0 = p_begin; p0 < p_end; p0 += 32) {
        const uint32_t p = p0 + lane;
        const uint32_t e = p < p_end ? idx[p] : 0u;
        const uint32_t g = p < p_end ? min(e / experts_per_rank, world - 1) : 0xFFFFFFFFu;
        uint32_t pos = 0;
#pragma unroll
        for (int q = 0; q < EP_MAX_WORLD; ++q) {
            const uint32_t peers = __ballot_sync(0xFFFFFFFFu, g == (uint32_t)q);
            if (g == (uint32_t)q) pos = run[q] + __popc(peers & ((1u << lane) - 1u));
            run[q] += __popc(peers);
        }
        if (p < p_end) {
            perm[pos] = p;
            inv[p] = pos;
            local_expert[pos] = (int32_t)(e - g * experts_per_rank);
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
    ep_plan_kernel<<<1, EP_PLAN_WARPS * 32, 0, (cudaStream_t)stream>>>(idx, n_tokens * top_k, num_experts / world, world, perm, inv, counts,
                                                                       nullptr, local_expert);
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

// ---------------------------------------------------------------------------------------------------------------
// Dispatch and combine over peer memory (NVLink), no collective library and no host synchronisation on the data path.
//
// Every rank owns, in plain device memory exported with CUDA IPC and mapped by all peers:
//   recv_x   [world][cap][d]  16-bit activation rows received from each source rank
//   recv_e   [world][cap]     expert id (relative to this rank's first expert) of each received row
//   ctrl     [world][4]       per source rank: row count, the source's send position of its first row, arrival flag,
//                             and (written by the expert side) the flag "your results are back"
//   ret      [cap][d]         fp32 result rows of this rank's own pairs, in its send order
// cap = tokens per rank x top_k, the most one rank can send.  A layer is two one-sided exchanges:
//   dispatch  one kernel packs the rows by destination and stores them straight into the destinations' recv_x / recv_e
//             (plain peer stores); the last block to finish publishes count, base position and the arrival flag on
//             every destination (system-scope fence before the flags);
//   combine   the expert side's down-projection epilogue stores each result row straight into the home rank's `ret`
//             (the grouped kernel is given one destination pointer per row); a small kernel then raises the
//             "results are back" flag on every home rank.
// Flags carry the epoch of the call (a counter that only grows), so nothing is ever reset.  Waiting is a one-warp
// kernel that polls its own memory with a clock limit and reports a time-out in the status word instead of hanging.
// A rank starts the next dispatch only after its own combine, which waits for every expert side, so one set of
// buffers is enough.  The reduce on the home rank is mfb_ep_combine: ranks ascending, fused multiply-add - the
// single-GPU order (prefill_moe_reduce_token_major, Sources/Mference/Metal/Prefill/prefill.metal:631-652).

struct mfb_ep {
    uint32_t rank = 0, world = 1, d = 0, cap = 0;
    uint32_t* epoch_dev = nullptr;   // the call's epoch lives on the device (bumped by a kernel at the start of a dispatch), so
                                     // that a layer captured into a CUDA graph advances it at every replay
    // own buffers
    uint16_t* recv_x = nullptr;
    int32_t* recv_e = nullptr;
    uint32_t* ctrl = nullptr;     // [world][4]: count, base, arrived, returned
    float* ret = nullptr;
    // peers' buffers (device arrays of `world` pointers; entry `rank` is the own buffer)
    uint16_t** peer_recv_x = nullptr;
    int32_t** peer_recv_e = nullptr;
    uint32_t** peer_ctrl = nullptr;
    float** peer_ret = nullptr;
    void* opened[4 * 8] = {};     // IPC mappings to close
    // scratch of a layer call
    uint32_t *perm = nullptr, *inv_scratch = nullptr, *done = nullptr, *status = nullptr;
    int32_t *counts = nullptr, *starts = nullptr, *local_expert = nullptr;
    uint32_t* row_expert = nullptr;   // [world * cap] expert id per received row, 0xFFFFFFFF beyond the counts
    float** row_dest = nullptr;       // [world * cap] where the result row of each received row goes
};

namespace mfb {
namespace {

constexpr long long EP_WAIT_CYCLES = 4000000000ll;   // ~2 s: a peer that never arrives is reported, not waited for

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// One block per send position: the pair's activation row goes to its destination rank's receive buffer.
__global__ void ep_dispatch_kernel(const uint16_t* __restrict__ x, uint32_t ldx, uint32_t d, const uint32_t* __restrict__ perm,
                                   const int32_t* __restrict__ local_expert, const int32_t* __restrict__ counts,
                                   const int32_t* __restrict__ starts, uint32_t n_pairs, uint32_t top_k, uint32_t world,
                                   uint32_t rank, uint32_t cap, uint16_t* const* __restrict__ peer_recv_x,
                                   int32_t* const* __restrict__ peer_recv_e, uint32_t* const* __restrict__ peer_ctrl,
                                   uint32_t* __restrict__ done, const uint32_t* __restrict__ epoch_p) {
    __shared__ uint32_t s_last;
    for (uint32_t pos = blockIdx.x; pos < n_pairs; pos += gridDim.x) {
        uint32_t g = 0;
        while (g + 1 < world && pos >= (uint32_t)starts[g + 1]) ++g;
        const uint32_t slot = pos - (uint32_t)starts[g];
        const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(perm[pos] / top_k) * ldx);
        uint4* dst = reinterpret_cast<uint4*>(peer_recv_x[g] + ((size_t)rank * cap + slot) * d);
        for (uint32_t i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
        if (threadIdx.x == 0) peer_recv_e[g][(size_t)rank * cap + slot] = local_expert[pos];
    }
    // the block that finishes last publishes the counts and raises the arrival flags
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(done, 1u) == gridDim.x - 1 ? 1u : 0u;
    __syncthreads();
    if (s_last) {
        __threadfence_system();
        if (threadIdx.x < world) {
            uint32_t* c = peer_ctrl[threadIdx.x] + rank * 4;
            c[0] = (uint32_t)counts[threadIdx.x];
            c[1] = (uint32_t)starts[threadIdx.x];
            __threadfence_system();
            st_release_sys(c + 2, *epoch_p);
        }
        if (threadIdx.x == 0) *done = 0;
    }
}

// One warp: lane s waits until source rank s has raised flag `which` (2 = rows arrived, 3 = results returned) to `epoch`.
__global__ void ep_wait_kernel(const uint32_t* __restrict__ ctrl, uint32_t world, uint32_t which, const uint32_t* __restrict__ epoch_p,
                               uint32_t* __restrict__ status) {
    const uint32_t s = threadIdx.x;
    if (s >= world) return;
    const uint32_t epoch = *epoch_p;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(ctrl + s * 4 + which) - epoch) < 0) {
        if (clock64() - t0 > EP_WAIT_CYCLES) { atomicOr(status, STATUS_MBAR_TIMEOUT); return; }
        __nanosleep(200);
    }
}

// Expert side, after the arrival flags: expert id of every received row (0xFFFFFFFF beyond a source's count) and the
// address its result row goes to - the source's `ret` at that pair's send position.
__global__ void ep_rows_kernel(const uint32_t* __restrict__ ctrl, const int32_t* __restrict__ recv_e, float* const* __restrict__ peer_ret,
                               uint32_t world, uint32_t cap, uint32_t d, uint32_t* __restrict__ row_expert,
                               float** __restrict__ row_dest) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= world * cap) return;
    const uint32_t s = i / cap, k = i % cap;
    const uint32_t count = ctrl[s * 4], base = ctrl[s * 4 + 1];
    const bool live = k < count && base + k < cap;
    row_expert[i] = live ? (uint32_t)recv_e[i] : 0xFFFFFFFFu;
    row_dest[i] = live ? peer_ret[s] + (size_t)(base + k) * d : nullptr;
}

// Expert side, after the grouped FFN: tells every home rank that its result rows are in place.
__global__ void ep_signal_kernel(uint32_t* const* __restrict__ peer_ctrl, uint32_t world, uint32_t rank, const uint32_t* __restrict__ epoch_p) {
    __threadfence_system();
    if (threadIdx.x < world) st_release_sys(peer_ctrl[threadIdx.x] + rank * 4 + 3, *epoch_p);
}

// First kernel of a dispatch: the next epoch (every rank makes the same number of calls, so the epochs agree).
__global__ void ep_epoch_kernel(uint32_t* epoch_p) { *epoch_p += 1u; }

template <typename T>
cudaError_t ep_alloc(T*& p, size_t n) { return cudaMalloc((void**)&p, (n ? n : 1) * sizeof(T)); }

}  // namespace
}  // namespace mfb

extern "C" int32_t mfb_ep_destroy(mfb_ep* ep) {
    if (!ep) return MFB_OK;
    for (void* p : ep->opened)
        if (p) cudaIpcCloseMemHandle(p);
    cudaFree(ep->recv_x); cudaFree(ep->recv_e); cudaFree(ep->ctrl); cudaFree(ep->ret);
    cudaFree(ep->peer_recv_x); cudaFree(ep->peer_recv_e); cudaFree(ep->peer_ctrl); cudaFree(ep->peer_ret);
    cudaFree(ep->perm); cudaFree(ep->inv_scratch); cudaFree(ep->done); cudaFree(ep->status); cudaFree(ep->epoch_dev);
    cudaFree(ep->counts); cudaFree(ep->starts); cudaFree(ep->local_expert); cudaFree(ep->row_expert); cudaFree(ep->row_dest);
    delete ep;
    return MFB_OK;
}

extern "C" int32_t mfb_ep_create(uint32_t rank, uint32_t world, uint32_t d, uint32_t max_pairs, mfb_ep** out) {
    MFB_REQUIRE(out != nullptr, MFB_ERR_INVALID_ARGUMENT, "ep_create: NULL output");
    *out = nullptr;
    MFB_REQUIRE(world >= 1 && world <= (uint32_t)EP_MAX_WORLD && rank < world, MFB_ERR_INVALID_ARGUMENT, "ep_create: rank / world out of range");
    MFB_REQUIRE(d % 8 == 0 && d > 0 && max_pairs > 0, MFB_ERR_INVALID_ARGUMENT, "ep_create: d must be a positive multiple of 8, max_pairs positive");
    mfb_ep* ep = new (std::nothrow) mfb_ep();
    MFB_REQUIRE(ep != nullptr, MFB_ERR_ALLOC, "out of host memory");
    ep->rank = rank; ep->world = world; ep->d = d; ep->cap = max_pairs;
    const size_t rows = (size_t)world * max_pairs;
    cudaError_t e = cudaSuccess;
    auto ok = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
    ok(ep_alloc(ep->recv_x, rows * d));
    ok(ep_alloc(ep->recv_e, rows));
    ok(ep_alloc(ep->ctrl, (size_t)world * 4));
    ok(ep_alloc(ep->ret, (size_t)max_pairs * d));
    ok(ep_alloc(ep->peer_recv_x, world)); ok(ep_alloc(ep->peer_recv_e, world)); ok(ep_alloc(ep->peer_ctrl, world)); ok(ep_alloc(ep->peer_ret, world));
    ok(ep_alloc(ep->perm, max_pairs)); ok(ep_alloc(ep->inv_scratch, max_pairs)); ok(ep_alloc(ep->done, 1)); ok(ep_alloc(ep->status, 1)); ok(ep_alloc(ep->epoch_dev, 1));
    ok(ep_alloc(ep->counts, world)); ok(ep_alloc(ep->starts, world)); ok(ep_alloc(ep->local_expert, max_pairs));
    ok(ep_alloc(ep->row_expert, rows)); ok(ep_alloc(ep->row_dest, rows));
    if (e == cudaSuccess) e = cudaMemset(ep->ctrl, 0, (size_t)world * 4 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ep->done, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ep->status, 0, sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ep->epoch_dev, 0, sizeof(uint32_t));
    if (e != cudaSuccess) {
        set_error("ep_create: %s", cudaGetErrorString(e));
        mfb_ep_destroy(ep);
        return e == cudaErrorMemoryAllocation ? MFB_ERR_ALLOC : MFB_ERR_CUDA;
    }
    *out = ep;
    return MFB_OK;
}

extern "C" int32_t mfb_ep_export(mfb_ep* ep, void* handles) {
    MFB_REQUIRE(ep && handles, MFB_ERR_INVALID_ARGUMENT, "ep_export: NULL argument");
    cudaIpcMemHandle_t* h = static_cast<cudaIpcMemHandle_t*>(handles);
    MFB_CUDA(cudaIpcGetMemHandle(&h[0], ep->recv_x));
    MFB_CUDA(cudaIpcGetMemHandle(&h[1], ep->recv_e));
    MFB_CUDA(cudaIpcGetMemHandle(&h[2], ep->ctrl));
    MFB_CUDA(cudaIpcGetMemHandle(&h[3], ep->ret));
    return MFB_OK;
}

extern "C" int32_t mfb_ep_import(mfb_ep* ep, const void* all_handles) {
    MFB_REQUIRE(ep && all_handles, MFB_ERR_INVALID_ARGUMENT, "ep_import: NULL argument");
    const cudaIpcMemHandle_t* h = static_cast<const cudaIpcMemHandle_t*>(all_handles);
    void* ptrs[4][EP_MAX_WORLD];
    void* own[4] = {ep->recv_x, ep->recv_e, ep->ctrl, ep->ret};
    for (uint32_t g = 0; g < ep->world; ++g)
        for (int b = 0; b < 4; ++b) {
            if (g == ep->rank) { ptrs[b][g] = own[b]; continue; }
            void* p = nullptr;
            MFB_CUDA(cudaIpcOpenMemHandle(&p, h[g * 4 + b], cudaIpcMemLazyEnablePeerAccess));
            ep->opened[g * 4 + b] = p;
            ptrs[b][g] = p;
        }
    MFB_CUDA(cudaMemcpy(ep->peer_recv_x, ptrs[0], ep->world * sizeof(void*), cudaMemcpyHostToDevice));
    MFB_CUDA(cudaMemcpy(ep->peer_recv_e, ptrs[1], ep->world * sizeof(void*), cudaMemcpyHostToDevice));
    MFB_CUDA(cudaMemcpy(ep->peer_ctrl, ptrs[2], ep->world * sizeof(void*), cudaMemcpyHostToDevice));
    MFB_CUDA(cudaMemcpy(ep->peer_ret, ptrs[3], ep->world * sizeof(void*), cudaMemcpyHostToDevice));
    return MFB_OK;
}

extern "C" int32_t mfb_ep_dispatch(mfb_ep* ep, void* stream, const void* x, uint32_t ldx, const uint32_t* idx, uint32_t n_tokens,
                                   uint32_t top_k, uint32_t num_experts, uint32_t* inv) {
    MFB_REQUIRE(ep && x && idx && inv, MFB_ERR_INVALID_ARGUMENT, "ep_dispatch: NULL argument");
    MFB_REQUIRE(ep->peer_recv_x != nullptr && num_experts % ep->world == 0 && ldx % 8 == 0 && ldx >= ep->d, MFB_ERR_INVALID_ARGUMENT,
                "ep_dispatch: world must divide num_experts, the row stride must be a multiple of 8 and at least d");
    const uint32_t n_pairs = n_tokens * top_k;
    MFB_REQUIRE(n_pairs <= ep->cap, MFB_ERR_CAPACITY, "ep_dispatch: %u pairs exceed the capacity of %u", n_pairs, ep->cap);
    cudaStream_t s = (cudaStream_t)stream;
    ep_epoch_kernel<<<1, 1, 0, s>>>(ep->epoch_dev);
    ep_plan_kernel<<<1, EP_PLAN_WARPS * 32, 0, s>>>(idx, n_pairs, num_experts / ep->world, ep->world, ep->perm, inv, ep->counts, ep->starts,
                                                    ep->local_expert);
    const uint32_t grid = n_pairs ? n_pairs : 1;
    ep_dispatch_kernel<<<grid, 128, 0, s>>>((const uint16_t*)x, ldx, ep->d, ep->perm, ep->local_expert, ep->counts, ep->starts, n_pairs,
                                            top_k, ep->world, ep->rank, ep->cap, ep->peer_recv_x, ep->peer_recv_e, ep->peer_ctrl, ep->done,
                                            ep->epoch_dev);
    count_launches(3);
    MFB_CUDA(cudaGetLastError());
    return MFB_OK;
}

extern "C" int32_t mfb_ep_receive(mfb_ep* ep, void* stream, const void** rows, const uint32_t** row_expert, float* const** row_dest,
                                  uint32_t* n_rows) {
    MFB_REQUIRE(ep && rows && row_expert && row_dest && n_rows, MFB_ERR_INVALID_ARGUMENT, "ep_receive: NULL argument");
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t total = ep->world * ep->cap;
    ep_wait_kernel<<<1, 32, 0, s>>>(ep->ctrl, ep->world, 2, ep->epoch_dev, ep->status);
    ep_rows_kernel<<<(total + 255) / 256, 256, 0, s>>>(ep->ctrl, ep->recv_e, ep->peer_ret, ep->world, ep->cap, ep->d, ep->row_expert, ep->row_dest);
    count_launches(2);
    MFB_CUDA(cudaGetLastError());
    *rows = ep->recv_x; *row_expert = ep->row_expert; *row_dest = ep->row_dest; *n_rows = total;
    return MFB_OK;
}

extern "C" int32_t mfb_ep_return(mfb_ep* ep, void* stream) {
    MFB_REQUIRE(ep != nullptr, MFB_ERR_INVALID_ARGUMENT, "ep_return: NULL argument");
    ep_signal_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ep->peer_ctrl, ep->world, ep->rank, ep->epoch_dev);
    count_launches(1);
    MFB_CUDA(cudaGetLastError());
    return MFB_OK;
}

extern "C" int32_t mfb_ep_results(mfb_ep* ep, void* stream, const float** ret) {
    MFB_REQUIRE(ep && ret, MFB_ERR_INVALID_ARGUMENT, "ep_results: NULL argument");
    ep_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(ep->ctrl, ep->world, 3, ep->epoch_dev, ep->status);
    count_launches(1);
    MFB_CUDA(cudaGetLastError());
    *ret = ep->ret;
    return MFB_OK;
}

extern "C" int32_t mfb_ep_status(mfb_ep* ep, void* stream, uint32_t* status, int32_t* counts_host) {
    MFB_REQUIRE(ep && status, MFB_ERR_INVALID_ARGUMENT, "ep_status: NULL argument");
    cudaStream_t s = (cudaStream_t)stream;
    MFB_CUDA(cudaMemcpyAsync(status, ep->status, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    if (counts_host) {   // rows received from each source rank in the last call (count word of every ctrl entry)
        uint32_t tmp[4 * EP_MAX_WORLD];
        MFB_CUDA(cudaMemcpyAsync(tmp, ep->ctrl, ep->world * 4 * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
        MFB_CUDA(cudaStreamSynchronize(s));
        for (uint32_t g = 0; g < ep->world; ++g) counts_host[g] = (int32_t)tmp[g * 4];
    }
    MFB_CUDA(cudaMemsetAsync(ep->status, 0, sizeof(uint32_t), s));
    MFB_CUDA(cudaStreamSynchronize(s));
    if (*status) { set_error("expert-parallel exchange: device status word = 0x%x", *status); return MFB_ERR_DEVICE_STATUS; }
    return MFB_OK;
}
