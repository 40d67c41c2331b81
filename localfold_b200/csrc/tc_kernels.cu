#include "tc_kernels.cuh"

namespace tc {

void configure_once() {}
lf_status prepare_weights(lf_context*, lf_weights*) { return LF_OK; }
bool triangle_supported(int, int, int) { return false; }
lf_status triangle_run(lf_context* ctx, ArenaCursor&, int, int, int, int, int, float, int, int, int, const void*,
                       const float*, void*, const lf_weights*) {
  return lf_fail(ctx, LF_ERR_UNSUPPORTED, "tensor-core triangle path not built");
}
bool attention_supported(int, int, int, int, int, int) { return false; }
lf_status attention_run(lf_context* ctx, ArenaCursor&, int, int, int, int, int, int, int, float, int, int, int, int, int,
                        int, const void*, const float*, void*, const lf_weights*) {
  return lf_fail(ctx, LF_ERR_UNSUPPORTED, "tensor-core attention path not built");
}
bool transition_supported(int, int, int) { return false; }
lf_status transition_run(lf_context* ctx, ArenaCursor&, int64_t, int, int, int, int, float, int, int, const void*, void*,
                         const lf_weights*) {
  return lf_fail(ctx, LF_ERR_UNSUPPORTED, "tensor-core transition path not built");
}

}  // namespace tc
