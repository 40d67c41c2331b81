// Tensor-core (tcgen05 / TMEM / TMA) kernels for sm_100a: launchers used by api.cu.
// Each *_supported() says whether a kernel covers a shape; api.cu routes
// everything else to the float32 SIMT kernels.
#pragma once

#include "common.cuh"

namespace tc {

void configure_once();
lf_status prepare_weights(lf_context* ctx, lf_weights* w);
// Reads the device status word; LF_ERR_TIMEOUT if a bounded wait expired in a kernel.
lf_status check_status(lf_context* ctx);

// Triangle contraction, batched over the c channels of channel-major fp16
// operands a, b [c][n][ld] (ld a multiple of 8, elements past n never read):
//   outgoing: x[h][i][j] = scale * sum_k a[h][i][k] * b[h][j][k]
//   incoming: x[h][i][j] = scale * sum_k a[h][k][j] * b[h][k][i]
bool contract_supported(int n, int c);
lf_status contract(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, op16* x, int n, int ld, int c,
                   int incoming, float scale);

}  // namespace tc
