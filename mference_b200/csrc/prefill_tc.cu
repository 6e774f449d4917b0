#include "prefill_tc.cuh"

namespace mfb {

bool tc_supported(const mfb_moe_config&) { return false; }
void tc_release(mfb_moe*) {}
int32_t tc_grouped_ffn(mfb_moe*, cudaStream_t, const mfb_layer_weights*, const void*, uint32_t, uint32_t,
                       const mfb_pair*, const mfb_group*, const uint32_t*, uint32_t, bool, float*, uint32_t) {
    set_error("tensor-core grouped FFN is not built");
    return MFB_ERR_UNSUPPORTED_SHAPE;
}

}  // namespace mfb
