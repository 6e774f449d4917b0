// Device-side sort of a routing table by (expert, token, rank) and the host-side grouping with the
// reference's validation.  Order and outputs follow PrefillMoEGrouping.groupTokenExpertPairs
// (Sources/Mference/Kernels/Prefill/MoE/PrefillMoEGrouping.swift:90-192): the reference sorts on the CPU
// after reading the whole table back; here a counting sort (per-chunk histogram, column scan, ordered
// scatter) produces the identical order without leaving the device and without atomics on global memory,
// so the result is deterministic.
#include <algorithm>
#include <unordered_set>
#include <vector>

#include "common.cuh"

namespace mfb {

namespace {

constexpr uint32_t kNoExpert = 0xFFFFFFFFu;

__device__ __forceinline__ uint32_t pair_expert(const uint32_t* idx, uint32_t p, uint32_t n_pairs, uint32_t top_k,
                                                uint32_t slot_mask, uint32_t num_experts) {
    if (p >= n_pairs) return kNoExpert;
    if (!((slot_mask >> (p % top_k)) & 1u)) return kNoExpert;
    const uint32_t e = idx[p];
    return e < num_experts ? e : kNoExpert;
}

// One warp per chunk of GROUP_CHUNK consecutive (token-major) pairs: per-expert counts of the chunk.
__global__ void group_hist_kernel(const uint32_t* __restrict__ idx, uint32_t n_pairs, uint32_t top_k,
                                  uint32_t num_experts, uint32_t slot_mask, uint32_t n_chunks,
                                  uint32_t* __restrict__ chunk_hist) {
    extern __shared__ uint32_t sh[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t chunk = blockIdx.x * (blockDim.x >> 5) + warp;
    uint32_t* h = sh + warp * num_experts;
    for (uint32_t e = lane; e < num_experts; e += 32) h[e] = 0;
    __syncwarp();
    if (chunk < n_chunks) {
        for (uint32_t i = 0; i < GROUP_CHUNK / 32; ++i) {
            const uint32_t p = chunk * GROUP_CHUNK + i * 32 + lane;
            const uint32_t e = pair_expert(idx, p, n_pairs, top_k, slot_mask, num_experts);
            if (e != kNoExpert) atomicAdd(&h[e], 1u);
        }
        __syncwarp();
        for (uint32_t e = lane; e < num_experts; e += 32) chunk_hist[(size_t)chunk * num_experts + e] = h[e];
    }
}

// One block per expert: exclusive scan of that expert's column of chunk_hist over the chunks; total -> counts.
__global__ void group_colscan_kernel(uint32_t* __restrict__ chunk_hist, uint32_t n_chunks, uint32_t num_experts,
                                     uint32_t* __restrict__ counts) {
    __shared__ uint32_t warp_sums[8];
    __shared__ uint32_t carry_s;
    const uint32_t e = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) carry_s = 0;
    __syncthreads();
    for (uint32_t base = 0; base < n_chunks; base += blockDim.x) {
        const uint32_t c = base + tid;
        const uint32_t v = c < n_chunks ? chunk_hist[(size_t)c * num_experts + e] : 0u;
        uint32_t incl = v;
        for (uint32_t off = 1; off < 32; off <<= 1) {
            const uint32_t n = __shfl_up_sync(0xFFFFFFFFu, incl, off);
            if (lane >= off) incl += n;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        uint32_t warp_base = 0;
        for (uint32_t w = 0; w < warp; ++w) warp_base += warp_sums[w];
        const uint32_t carry = carry_s;
        if (c < n_chunks) chunk_hist[(size_t)c * num_experts + e] = carry + warp_base + incl - v;
        __syncthreads();
        if (tid == blockDim.x - 1) carry_s = carry + warp_base + incl;
        __syncthreads();
    }
    if (tid == 0) counts[e] = carry_s;
}

// One block: expert offsets (exclusive scan of counts in expert order, absent experts marked), the compacted
// group list, the optional shared-expert group over all tokens, and the tile prefix of the grouped GEMM.
__global__ void group_finalize_kernel(const uint32_t* __restrict__ counts, uint32_t num_experts, uint32_t n_tokens,
                                      uint32_t top_k, int append_shared, uint32_t tile_rows,
                                      uint32_t* __restrict__ offsets, mfb_group* __restrict__ groups,
                                      uint32_t* __restrict__ n_groups, uint32_t* __restrict__ tile_prefix,
                                      mfb_pair* __restrict__ sorted) {
    __shared__ uint32_t s_total;
    __shared__ uint32_t s_cnt[MFB_MAX_EXPERTS];
    for (uint32_t e = threadIdx.x; e < num_experts; e += blockDim.x) s_cnt[e] = counts[e];
    __syncthreads();
    if (threadIdx.x < 32) {
        // one warp, 32 experts per round: exclusive prefixes of the pair counts, of the non-empty flags (group index)
        // and of the tile counts by shuffles, carried from round to round
        const uint32_t lane = threadIdx.x;
        uint32_t run = 0, ng = 0, tiles = 0;
        for (uint32_t base = 0; base < num_experts; base += 32) {
            const uint32_t e = base + lane;
            const uint32_t c = e < num_experts ? s_cnt[e] : 0u;
            const uint32_t t = tile_prefix ? (c + tile_rows - 1) / tile_rows : 0u;
            uint32_t ic = c, it = t;
            for (uint32_t off = 1; off < 32; off <<= 1) {
                const uint32_t a = __shfl_up_sync(0xFFFFFFFFu, ic, off), b2 = __shfl_up_sync(0xFFFFFFFFu, it, off);
                if (lane >= off) { ic += a; it += b2; }
            }
            const uint32_t live = __ballot_sync(0xFFFFFFFFu, c != 0u);
            const uint32_t g = ng + __popc(live & ((1u << lane) - 1u));
            if (e < num_experts) {
                offsets[e] = c ? run + ic - c : 0xFFFFFFFFu;
                if (c) {
                    groups[g].expert = e;
                    groups[g].pair_start = run + ic - c;
                    groups[g].pair_count = c;
                    if (tile_prefix) tile_prefix[g] = tiles + it - t;
                }
            }
            run += __shfl_sync(0xFFFFFFFFu, ic, 31);
            tiles += __shfl_sync(0xFFFFFFFFu, it, 31);
            ng += __popc(live);
        }
        if (lane == 0) {
            if (append_shared) {
                groups[ng].expert = num_experts;
                groups[ng].pair_start = run;
                groups[ng].pair_count = n_tokens;
                if (tile_prefix) { tile_prefix[ng] = tiles; tiles += (n_tokens + tile_rows - 1) / tile_rows; }
                ++ng;
            }
            if (tile_prefix) tile_prefix[ng] = tiles;
            *n_groups = ng;
            s_total = run;
        }
    }
    __syncthreads();
    if (append_shared) {
        const uint32_t base = s_total;
        for (uint32_t t = threadIdx.x; t < n_tokens; t += blockDim.x) {
            mfb_pair p;
            p.token = t; p.expert = num_experts; p.rank = top_k; p.weight_bits = 0x3C00u; /* fp16 1.0 */
            sorted[base + t] = p;
        }
    }
}

// One warp per chunk again: walk the chunk in order, 32 pairs per round; a pair's slot is its expert's
// offset + pairs of that expert in earlier chunks + earlier in this chunk.
__global__ void group_scatter_kernel(const uint32_t* __restrict__ idx, const uint16_t* __restrict__ route_w,
                                     uint32_t n_pairs, uint32_t top_k, uint32_t num_experts, uint32_t slot_mask,
                                     uint32_t n_chunks, const uint32_t* __restrict__ chunk_hist,
                                     const uint32_t* __restrict__ offsets, mfb_pair* __restrict__ sorted) {
    extern __shared__ uint32_t sh[];
    uint32_t* s_off = sh;  // [num_experts] expert offsets, shared by the block
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    uint32_t* run = sh + num_experts + warp * num_experts;
    for (uint32_t e = threadIdx.x; e < num_experts; e += blockDim.x) s_off[e] = offsets[e];   // unused where the expert has no pair
    __syncthreads();
    const uint32_t chunk = blockIdx.x * warps + warp;
    if (chunk >= n_chunks) return;
    for (uint32_t e = lane; e < num_experts; e += 32) run[e] = s_off[e] + chunk_hist[(size_t)chunk * num_experts + e];
    __syncwarp();
    for (uint32_t i = 0; i < GROUP_CHUNK / 32; ++i) {
        const uint32_t p = chunk * GROUP_CHUNK + i * 32 + lane;
        const uint32_t e = pair_expert(idx, p, n_pairs, top_k, slot_mask, num_experts);
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, e);
        const uint32_t before = __popc(peers & ((1u << lane) - 1u));
        uint32_t pos = 0;
        if (e != kNoExpert) pos = run[e] + before;
        __syncwarp();
        if (e != kNoExpert && before == 0) run[e] += __popc(peers);
        __syncwarp();
        if (e != kNoExpert) {
            mfb_pair out;
            out.token = p / top_k; out.expert = e; out.rank = p % top_k;
            out.weight_bits = route_w ? (uint32_t)route_w[p] : 0u;
            sorted[pos] = out;
        }
    }
}

}  // namespace

cudaError_t launch_group(cudaStream_t s, const uint32_t* idx, const uint16_t* route_w, uint32_t n_tokens,
                         uint32_t top_k, uint32_t num_experts, uint32_t slot_mask, int append_shared,
                         uint32_t tile_rows, Arena& a, mfb_pair* out_sorted, uint32_t* out_offsets,
                         uint32_t* out_counts, mfb_group* out_groups, uint32_t* out_n_groups, uint32_t* tile_prefix) {
    const uint32_t n_pairs = n_tokens * top_k;
    const uint32_t n_chunks = (n_pairs + GROUP_CHUNK - 1) / GROUP_CHUNK;
    const uint32_t warps = 4;
    const uint32_t blocks = (n_chunks + warps - 1) / warps;
    if (n_chunks > 0) {
        group_hist_kernel<<<blocks, warps * 32, warps * num_experts * sizeof(uint32_t), s>>>(
            idx, n_pairs, top_k, num_experts, slot_mask, n_chunks, a.chunk_hist);
        count_launches(1);
    }
    if (n_chunks > 0) {
        group_colscan_kernel<<<num_experts, 256, 0, s>>>(a.chunk_hist, n_chunks, num_experts, out_counts);
        count_launches(1);
    } else {
        cudaError_t e = cudaMemsetAsync(out_counts, 0, num_experts * sizeof(uint32_t), s);
        if (e != cudaSuccess) return e;
    }
    group_finalize_kernel<<<1, 256, 0, s>>>(out_counts, num_experts, n_tokens, top_k, append_shared,
                                            tile_rows ? tile_rows : 1u, out_offsets, out_groups, out_n_groups,
                                            tile_prefix, out_sorted);
    count_launches(1);
    if (n_chunks > 0) {
        group_scatter_kernel<<<blocks, warps * 32, (warps + 1) * num_experts * sizeof(uint32_t), s>>>(
            idx, route_w, n_pairs, top_k, num_experts, slot_mask, n_chunks, a.chunk_hist, out_offsets, out_sorted);
        count_launches(1);
    }
    return cudaGetLastError();
}

}  // namespace mfb

// ---------------------------------------------------------------------------------------------------------
// Host-side grouping (validation, sort keys, tiles) for callers that hold the routing table on the host.

extern "C" int32_t mfb_moe_group_host(const mfb_pair* pairs, int64_t n_pairs, int64_t query_count, int64_t top_k,
                                      int64_t num_experts, int64_t tile_expert_count, const uint64_t* expert_sort_keys,
                                      int64_t n_sort_keys, mfb_pair* out_sorted, uint32_t* out_offsets,
                                      uint32_t* out_counts, mfb_group* out_groups, uint32_t* out_n_groups,
                                      mfb_tile* out_tiles, uint32_t* out_n_tiles, uint32_t* err_a, uint32_t* err_b) {
    uint32_t dummy_a = 0, dummy_b = 0;
    if (!err_a) err_a = &dummy_a;
    if (!err_b) err_b = &dummy_b;
    *err_a = *err_b = 0;
    if (out_n_groups) *out_n_groups = 0;
    if (out_n_tiles) *out_n_tiles = 0;
    auto fail = [&](int32_t code, uint32_t a, uint32_t b, const char* what) {
        *err_a = a; *err_b = b;
        mfb::set_error("grouping: %s (%u, %u)", what, a, b);
        return code;
    };
    if (query_count < 0) return fail(MFB_ERR_GROUP_INVALID_QUERY_COUNT, (uint32_t)query_count, 0, "queryCount must be non-negative");
    if (top_k <= 0) return fail(MFB_ERR_GROUP_INVALID_TOP_K, (uint32_t)top_k, 0, "topK must be positive");
    if (num_experts <= 0) return fail(MFB_ERR_GROUP_INVALID_NUM_EXPERTS, (uint32_t)num_experts, 0, "numExperts must be positive");
    if (tile_expert_count < 1 || tile_expert_count > 16)
        return fail(MFB_ERR_GROUP_INVALID_TILE_EXPERT_COUNT, (uint32_t)tile_expert_count, 0, "tileExpertCount must be in 1...16");
    if (expert_sort_keys && n_sort_keys != num_experts)
        return fail(MFB_ERR_GROUP_SORT_KEY_COUNT_MISMATCH, (uint32_t)num_experts, (uint32_t)n_sort_keys, "expert sort key count");
    if (n_pairs != query_count * top_k)
        return fail(MFB_ERR_GROUP_PAIR_COUNT_MISMATCH, (uint32_t)(query_count * top_k), (uint32_t)n_pairs, "route pair count");
    if (!pairs && n_pairs > 0) return fail(MFB_ERR_INVALID_ARGUMENT, 0, 0, "pairs is NULL");

    std::unordered_set<uint64_t> seen;
    seen.reserve((size_t)n_pairs * 2 + 1);
    for (int64_t i = 0; i < n_pairs; ++i) {
        const mfb_pair& p = pairs[i];
        if (p.token >= (uint32_t)query_count) return fail(MFB_ERR_GROUP_TOKEN_OUT_OF_RANGE, p.token, 0, "route token out of range");
        if (p.rank >= (uint32_t)top_k) return fail(MFB_ERR_GROUP_RANK_OUT_OF_RANGE, p.rank, 0, "route rank out of range");
        if (p.expert >= (uint32_t)num_experts) return fail(MFB_ERR_GROUP_EXPERT_OUT_OF_RANGE, p.expert, 0, "route expert out of range");
        if (!seen.insert(((uint64_t)p.token << 32) | p.rank).second)
            return fail(MFB_ERR_GROUP_DUPLICATE_TOKEN_RANK, p.token, p.rank, "duplicate route pair");
    }
    std::vector<mfb_pair> v(pairs, pairs + n_pairs);
    std::sort(v.begin(), v.end(), [&](const mfb_pair& l, const mfb_pair& r) {
        if (expert_sort_keys) {
            const uint64_t lk = expert_sort_keys[l.expert], rk = expert_sort_keys[r.expert];
            if (lk != rk) return lk < rk;
        }
        if (l.expert != r.expert) return l.expert < r.expert;
        if (l.token != r.token) return l.token < r.token;
        return l.rank < r.rank;
    });
    for (int64_t e = 0; e < num_experts; ++e) { out_offsets[e] = 0xFFFFFFFFu; out_counts[e] = 0; }
    uint32_t ng = 0;
    for (size_t i = 0; i < v.size();) {
        const uint32_t e = v[i].expert;
        const size_t start = i;
        while (i < v.size() && v[i].expert == e) ++i;
        out_offsets[e] = (uint32_t)start;
        out_counts[e] = (uint32_t)(i - start);
        out_groups[ng++] = mfb_group{e, (uint32_t)start, (uint32_t)(i - start)};
    }
    uint32_t nt = 0;
    for (uint32_t gs = 0; gs < ng;) {
        const uint32_t ge = std::min<uint32_t>(ng, gs + (uint32_t)tile_expert_count);
        if (out_tiles) {
            out_tiles[nt] = mfb_tile{gs, ge - gs, out_groups[gs].pair_start,
                                     out_groups[ge - 1].pair_start + out_groups[ge - 1].pair_count - out_groups[gs].pair_start};
        }
        ++nt;
        gs = ge;
    }
    for (size_t i = 0; i < v.size(); ++i) out_sorted[i] = v[i];
    if (out_n_groups) *out_n_groups = ng;
    if (out_n_tiles) *out_n_tiles = nt;
    return MFB_OK;
}
