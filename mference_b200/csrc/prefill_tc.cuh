// Tensor-core (tcgen05 / TMEM) grouped expert FFN for prefill and ragged batches: interface used by api.cu.
#pragma once

#include "common.cuh"

namespace mfb {

constexpr uint32_t TC_TILE_N = 256;   // token rows per tile of the grouped GEMM (the N of one tcgen05.mma)
constexpr uint32_t TC_ROW_PAD = 256;  // spare rows behind the gathered activations so a tile may over-read

bool tc_supported(const mfb_moe_config& c);
// Builds the tensor maps, prefix arrays and kernel attributes of the path (called once by mfb_moe_create).
int32_t tc_init(mfb_moe* m);
void tc_release(mfb_moe* m);
// partial[(token*slots + rank), :] = ffn_expert(x[token]) for every sorted pair of every group; with row_dest the row
// of (token, rank) goes to row_dest[token*slots + rank] instead (any device-visible address, a NULL entry drops it).
int32_t tc_grouped_ffn(mfb_moe* m, cudaStream_t s, const mfb_layer_weights* w, const void* x, uint32_t ldx,
                       uint32_t n_tokens, const mfb_pair* sorted, const mfb_group* groups, const uint32_t* n_groups,
                       uint32_t max_groups, bool routed_only, float* partial, uint32_t slots, float* const* row_dest = nullptr);

}  // namespace mfb
