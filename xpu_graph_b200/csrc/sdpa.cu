// Fused scaled-dot-product attention (placeholder until the flash kernel lands).
#include "common.cuh"

extern "C" int xg_sdpa_fwd(const void* q, const void* k, const void* v, const void* mask, void* out, int64_t B, int64_t H,
                           int64_t Sq, int64_t Skv, int64_t D, const int64_t* q_strides3, const int64_t* k_strides3,
                           const int64_t* v_strides3, const int64_t* o_strides3, const int64_t* mask_strides4, float scale,
                           int causal, int dtype, void* stream) {
    return xg::fail(XG_ERR_UNSUPPORTED, "xg_sdpa_fwd: not built yet");
}
