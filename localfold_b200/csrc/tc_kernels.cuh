// Tensor-core (tcgen05 / TMEM / TMA) kernels for sm_100a: interface used by api.cu.
// Each *_supported() says whether the fused kernels cover a shape; api.cu routes
// everything else to the float32 SIMT kernels.
#pragma once

#include "common.cuh"

namespace tc {

void configure_once();
lf_status prepare_weights(lf_context* ctx, lf_weights* w);

bool triangle_supported(int n, int cz, int c);
lf_status triangle_run(lf_context* ctx, ArenaCursor& cur, int n, int cz, int c, int incoming, int variance, float eps,
                       int residual, int divide, int act_dtype, const void* z, const float* mask, void* out,
                       const lf_weights* w);

bool attention_supported(int batch, int Q, int ch, int heads, int d, int bias_mode);
lf_status attention_run(lf_context* ctx, ArenaCursor& cur, int batch, int Q, int ch, int heads, int d, int transpose,
                        int variance, float eps, int residual, int bias_mode, int bias_swap, int mask_mode, int clamp,
                        int act_dtype, const void* act, const float* mask, void* out, const lf_weights* w);

bool transition_supported(int ch, int hidden, int swiglu);
lf_status transition_run(lf_context* ctx, ArenaCursor& cur, int64_t rows, int ch, int hidden, int swiglu, int variance,
                         float eps, int residual, int act_dtype, const void* act, void* out, const lf_weights* w);

}  // namespace tc
