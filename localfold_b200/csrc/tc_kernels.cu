// tcgen05 / TMEM / TMA kernels for sm_100a.
#include "tc_kernels.cuh"

#include <cuda.h>
#include <cuda_fp16.h>

#include <cmath>
#include <mutex>
#include <vector>

#include "tc05.cuh"

namespace tc {

using namespace tc05;

// ---------------------------------------------------------------------------
// host helpers

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;
static std::once_flag g_once;

void configure_once();

lf_status make_map_f16_3d_box(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2) {
  if (!g_encode) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return LF_OK;
}

static lf_status make_map_f16_3d(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1,
                                 uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1) {
  return make_map_f16_3d_box(ctx, map, base, d0, d1, d2, stride1_bytes, stride2_bytes, b0, b1, 1);
}

lf_status make_map_f16_3d_ext(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1) {
  return make_map_f16_3d(ctx, map, base, d0, d1, d2, stride1_bytes, stride2_bytes, b0, b1);
}

// Attention activations q, k, v, gate, o: fp16 [batch][ldq][128] stored as 8-row x 8-channel pieces of 128
// contiguous bytes (element (b, q, c) at b*ldq*128 + (q/8)*1024 + (c/8)*64 + (q%8)*8 + c%8).  A warp whose
// threads own consecutive rows then writes whole 128-byte lines with 16-byte stores, and a piece is exactly
// one core matrix of the tensor core's unswizzled operand format.  The map's dimensions are (channel in
// piece, row in piece, piece along channels, piece along rows, batch row) - strides increasing - and a
// box of `rows` rows x 64 channels lands in shared memory as [rows/8][8 pieces][8 rows][16 B].
lf_status make_map_tiled_act(lf_context* ctx, CUtensorMap* map, const void* base, int ldq, int batch, int rows) {
  if (!g_encode) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[5] = {8, 8, 16, (cuuint64_t)(ldq / 8), (cuuint64_t)batch};
  cuuint64_t strides[4] = {16, 128, 2048, (cuuint64_t)ldq * 256};
  cuuint32_t box[5] = {8, 8, 8, (cuuint32_t)(rows / 8), 1};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled (5-d) failed with code %d", (int)r);
  return LF_OK;
}

// float32 rows of 128 channels seen as (channel, d1, d2); boxes of 32 channels (one 128-byte swizzled row) x b1 x b2
lf_status make_map_f32_rows(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                            uint64_t stride2_bytes, uint32_t b1, uint32_t b2) {
  if (!g_encode) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {128, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {32, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled (float32 rows) failed with code %d", (int)r);
  return LF_OK;
}

// the same with boxes of 16 channels (64-byte rows, 64-byte swizzle): the staging tiles of the triangle output
lf_status make_map_f32_rows_half(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                                 uint64_t stride2_bytes, uint32_t b1, uint32_t b2) {
  if (!g_encode) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {128, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {16, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled (float32 rows, 16 channels, 3-d) failed with code %d", (int)r);
  return LF_OK;
}

// float32 rows of 128 channels as a 2-d map (channel, row) with boxes of 16 channels x 32 rows (64-byte rows,
// 64-byte swizzle): the staging tiles of the transition's output
lf_status make_map_f32_rows16(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t rows) {
  if (!g_encode) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {128, rows};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {16, 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled (float32 rows, 16 channels) failed with code %d", (int)r);
  return LF_OK;
}

// fp16 operand planes [planes][plane_rows][ld] seen as (k, i, plane); boxes of 64 k (128 bytes, 128-byte swizzle) x 1 x box_h
// planes: what four epilogue warps of the triangle projection store per pass
lf_status make_map_plane_runs(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t n, uint64_t plane_rows, uint64_t planes,
                              uint64_t ld, uint32_t box_h) {
  if (!g_encode) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {n, plane_rows, planes};
  cuuint64_t strides[2] = {ld * 2, plane_rows * ld * 2};
  cuuint32_t box[3] = {64, 1, box_h};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return lf_fail(ctx, LF_ERR_CUDA, "cuTensorMapEncodeTiled (operand planes) failed with code %d", (int)r);
  return LF_OK;
}

lf_status check_status(lf_context* ctx) {
  if (!ctx->tc_status) return LF_OK;
  Status st;
  if (cudaMemcpy(&st, ctx->tc_status, sizeof st, cudaMemcpyDeviceToHost) != cudaSuccess)
    return lf_fail(ctx, LF_ERR_CUDA, "reading the kernel status word failed: %s", cudaGetErrorString(cudaGetLastError()));
  if (st.code != 0) {
    cudaMemset(ctx->tc_status, 0, sizeof st);
    return lf_fail(ctx, LF_ERR_TIMEOUT, "a bounded wait expired in a tensor-core kernel (wait %u, block %u)", st.where, st.block);
  }
  return LF_OK;
}

bool ln_gemm_supported(const lf_weights* w) { return w && !w->h.empty() && w->h[0] != nullptr; }
bool pair_bias_supported(const lf_weights* w) { return w && w->h.size() >= 6 && w->h[4] != nullptr; }

// The centre LayerNorm folded into the output projection: W' = diag(gain) Wz, s1[c] = sum_h fp16(W'[h][c]) (what the
// tensor core will multiply the mean by), t[c] = bz[c] + sum_h offset[h] Wz[h][c]; fold = (s1 | t | bg + input offset through Wg).
__global__ void triangle_fold_kernel(const float* __restrict__ wz, const float* __restrict__ gain, const float* __restrict__ offset,
                                     const float* __restrict__ bz, const float* __restrict__ bg, const float* __restrict__ wg,
                                     const float* __restrict__ in_offset, float* __restrict__ wfold, float* __restrict__ fold) {
  const int c = threadIdx.x;
  double s1 = 0.0, t = bz[c], g = bg[c];
  for (int h = 0; h < 128; ++h) {
    const float wf = gain[h] * wz[h * 128 + c];
    wfold[h * 128 + c] = wf;
    s1 += (double)__half2float(__float2half_rn(wf));
    t += (double)offset[h] * wz[h * 128 + c];
    g += (double)in_offset[h] * wg[h * 128 + c];      // the input LayerNorm's offset through the output gate
  }
  fold[c] = (float)s1;
  fold[128 + c] = (float)t;
  fold[256 + c] = (float)g;
}

// bf16/fp16 repacks for the tensor-core kernels: h[0] = swizzled fp16 image of the fused
// projection W^T (plus the pair-bias projection rows for attention), h[1] = its bias vector.
// weights w [K][ldw] float32, columns col0 .. col0+N-1 -> fp16 [N][K] (the plain GEMM wants k contiguous in both operands)
__global__ void gemm_operand_kernel(const float* __restrict__ w, int K, int ldw, int col0, int N, op16* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)N * K) return;
  int n = (int)(idx / K), k = (int)(idx % K);
  out[idx] = __float2half_rn(w[(int64_t)k * ldw + col0 + n]);
}

// ... with 16 more k columns: the bias in the first, zeros after it (the activations carry a column of ones there, so the
// GEMM adds the bias)
__global__ void gemm_operand_bias_kernel(const float* __restrict__ w, int K, int ldw, int N, const float* __restrict__ bias,
                                         op16* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int K2 = K + 16;
  if (idx >= (int64_t)N * K2) return;
  int n = (int)(idx / K2), k = (int)(idx % K2);
  out[idx] = __float2half_rn(k < K ? w[(int64_t)k * ldw + n] : k == K ? bias[n] : 0.f);
}

lf_status prepare_weights(lf_context* ctx, lf_weights* w) {
  const bool tri = w->kind == LF_WEIGHTS_TRIANGLE_AF2 || w->kind == LF_WEIGHTS_TRIANGLE_AF3;
  const bool att = w->kind == LF_WEIGHTS_ATTENTION_AF2 || w->kind == LF_WEIGHTS_GRID_ATTENTION_AF3;
  if (tri && w->dims.channels == 128 && w->dims.hidden == 128) {
    op16* img = nullptr;
    LF_CUDA(ctx, cudaMalloc(&img, 512 * 256));
    w->owned.push_back(img);
    LF_CUDA(ctx, cudaMemsetAsync(img, 0, 512 * 256, ctx->stream));
    // the input LayerNorm's gain goes into the rows of the images, its offset into the biases: the kernels' producers
    // hand the tensor core (x - mean) / std
    pack_weight_image(ctx, w->f[TRI_W4], 128, 512, 512, 0, 512, img, 0, 1.0f, w->f[TRI_LN_G]);
    float* b4 = nullptr;
    LF_CUDA(ctx, cudaMalloc(&b4, 512 * sizeof(float))); w->owned.push_back(b4);
    fold_bias(ctx, w->f[TRI_W4], 128, 512, 0, 512, w->f[TRI_LN_B], w->f[TRI_B4], 1.0f, b4);
    w->h.assign(4, nullptr);
    w->h[0] = img;
    w->h[1] = b4;
    // output kernel: rows 0..127 = (diag(gain) Wz)^T, rows 128..255 = Wg^T, plus the folded vectors
    float* dfold = nullptr; float* dw = nullptr; op16* img2 = nullptr;
    LF_CUDA(ctx, cudaMalloc(&dfold, 384 * 4)); w->owned.push_back(dfold);
    LF_CUDA(ctx, cudaMalloc(&dw, 128 * 128 * 4)); w->owned.push_back(dw);
    LF_CUDA(ctx, cudaMalloc(&img2, 256 * 256)); w->owned.push_back(img2);
    triangle_fold_kernel<<<1, 128, 0, ctx->stream>>>(w->f[TRI_WZ], w->f[TRI_LNO_G], w->f[TRI_LNO_B], w->f[TRI_BZ], w->f[TRI_BG], w->f[TRI_WG],
                                                     w->f[TRI_LN_B], dw, dfold);
    pack_weight_image(ctx, dw, 128, 128, 256, 0, 128, img2, 0, 1.0f);
    pack_weight_image(ctx, w->f[TRI_WG], 128, 128, 256, 0, 128, img2, 128, 1.0f, w->f[TRI_LN_G]);
    LF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    w->h[2] = img2;
    w->h[3] = dfold;
  } else if (att && w->dims.channels == 128 && w->dims.heads * w->dims.head_dim == 128 && w->dims.heads <= 16 &&
             !w->has_pair_norm) {
    op16* img = nullptr;
    float* bias = nullptr;
    LF_CUDA(ctx, cudaMalloc(&img, 528 * 256));
    w->owned.push_back(img);
    LF_CUDA(ctx, cudaMalloc(&bias, 528 * sizeof(float)));
    w->owned.push_back(bias);
    LF_CUDA(ctx, cudaMemsetAsync(img, 0, 528 * 256, ctx->stream));
    LF_CUDA(ctx, cudaMemsetAsync(bias, 0, 528 * sizeof(float), ctx->stream));
    // the query columns carry the head_dim^-1/2 logit scale
    const float qs = 1.0f / sqrtf((float)w->dims.head_dim);
    // the LayerNorm's gain goes into the rows of the image, its offset into the bias vector
    pack_weight_image(ctx, w->f[ATT_W4], 128, 128, 528, 0, 512, img, 0, qs, w->f[ATT_LN_G]);
    pack_weight_image(ctx, w->f[ATT_W4], 128, 384, 528, 128, 512, img, 128, 1.0f, w->f[ATT_LN_G]);
    fold_bias(ctx, w->f[ATT_W4], 128, 128, 0, 512, w->f[ATT_LN_B], w->f[ATT_B4], qs, bias);
    fold_bias(ctx, w->f[ATT_W4], 128, 384, 128, 512, w->f[ATT_LN_B], w->f[ATT_B4] + 128, 1.0f, bias + 128);
    if (w->has_pair_proj) {
      pack_weight_image(ctx, w->f[ATT_WB], 128, w->dims.heads, 528, 0, w->dims.heads, img, 512, 1.0f, w->f[ATT_LN_G]);
      fold_bias(ctx, w->f[ATT_WB], 128, w->dims.heads, 0, w->dims.heads, w->f[ATT_LN_B], nullptr, 1.0f, bias + 512);
    }
    {
      // which 128-column groups have a bias at all (the epilogue skips the others): 2 KiB read back once
      std::vector<float> hb(512);
      LF_CUDA(ctx, cudaMemcpyAsync(hb.data(), bias, 512 * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
      LF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      w->bias_flags = 0;
      for (int grp = 0; grp < 4; ++grp)
        for (int i = 0; i < 128; ++i)
          if (hb[grp * 128 + i] != 0.f) { w->bias_flags |= 1 << grp; break; }
    }
    w->h.assign(4, nullptr);
    w->h[0] = img;
    w->h[1] = bias;
    op16* img2 = nullptr;
    LF_CUDA(ctx, cudaMalloc(&img2, 128 * 256)); w->owned.push_back(img2);
    pack_weight_image(ctx, w->f[ATT_WO], 128, 128, 128, 0, 128, img2, 0, 1.0f);
    w->h[2] = img2;
  }
  if (w->has_pair_norm && w->has_pair_proj && w->dims.pair_channels == 128 && w->dims.heads <= 16 &&
      (w->kind == LF_WEIGHTS_ATTENTION_AF2 || w->kind == LF_WEIGHTS_SINGLE_ATTENTION_AF3 || w->kind == LF_WEIGHTS_MSA_ATTENTION_AF3)) {
    // pair bias from a 128-channel pair with a LayerNorm of its own: a 16-row image of the projection (gain in its
    // rows, the offset's share as a bias) for the tensor-core projection kernel run with the bias chunk alone
    op16* img = nullptr;
    float* pb = nullptr;
    LF_CUDA(ctx, cudaMalloc(&img, 16 * 256)); w->owned.push_back(img);
    LF_CUDA(ctx, cudaMalloc(&pb, 16 * sizeof(float))); w->owned.push_back(pb);
    LF_CUDA(ctx, cudaMemsetAsync(img, 0, 16 * 256, ctx->stream));
    LF_CUDA(ctx, cudaMemsetAsync(pb, 0, 16 * sizeof(float), ctx->stream));
    pack_weight_image(ctx, w->f[ATT_WB], 128, w->dims.heads, 16, 0, w->dims.heads, img, 0, 1.0f, w->f[ATT_PLN_G]);
    fold_bias(ctx, w->f[ATT_WB], 128, w->dims.heads, 0, w->dims.heads, w->f[ATT_PLN_B], nullptr, 1.0f, pb);
    if (w->h.size() < 6) w->h.resize(6, nullptr);
    w->h[4] = img;
    w->h[5] = pb;
  }
  if (w->kind == LF_WEIGHTS_TRANSITION_AF2 && w->dims.channels == 128 && w->dims.hidden == 512) {
    // per 128-wide hidden chunk: W1 slice image (rows = hidden columns, K = 128 inputs), then W2 slice
    // image (rows = 128 outputs, K = the chunk's 128 hidden channels)
    op16* img = nullptr;
    LF_CUDA(ctx, cudaMalloc(&img, 4 * 65536));
    w->owned.push_back(img);
    for (int cidx = 0; cidx < 4; ++cidx) {
      pack_weight_image(ctx, w->f[TRN_W1], 128, 128, 128, cidx * 128, 512, img + cidx * 32768, 0, 1.0f, w->f[TRN_LN_G]);
      pack_weight_image(ctx, w->f[TRN_W2] + (size_t)cidx * 128 * 128, 128, 128, 128, 0, 128, img + cidx * 32768 + 16384, 0, 1.0f);
    }
    float* b1 = nullptr;
    LF_CUDA(ctx, cudaMalloc(&b1, 512 * sizeof(float))); w->owned.push_back(b1);
    fold_bias(ctx, w->f[TRN_W1], 128, 512, 0, 512, w->f[TRN_LN_B], w->f[TRN_B1], 1.0f, b1);
    w->h.assign(2, nullptr);
    w->h[0] = img;
    w->h[1] = b1;
  }
  if (w->kind == LF_WEIGHTS_TRANSITION_AF3 && w->dims.channels == 128 && w->dims.hidden == 512) {
    // per 64-wide hidden chunk: W1 slice image of 128 rows (64 gate columns, then the matching 64 value
    // columns; K = 128 inputs: 32 KiB), then W2 slice image (rows = 128 outputs, K = 64 hidden: 16 KiB)
    op16* img = nullptr;
    LF_CUDA(ctx, cudaMalloc(&img, 8 * 49152));
    w->owned.push_back(img);
    for (int cidx = 0; cidx < 8; ++cidx) {
      op16* base = img + (size_t)cidx * 24576;
      pack_weight_image(ctx, w->f[TRN_W1], 128, 64, 128, cidx * 64, 1024, base, 0, 1.0f, w->f[TRN_LN_G]);
      pack_weight_image(ctx, w->f[TRN_W1], 128, 64, 128, 512 + cidx * 64, 1024, base, 64, 1.0f, w->f[TRN_LN_G]);
      pack_weight_image(ctx, w->f[TRN_W2] + (size_t)cidx * 64 * 128, 64, 128, 128, 0, 128, base + 16384, 0, 1.0f);
    }
    float* b1 = nullptr;
    LF_CUDA(ctx, cudaMalloc(&b1, 1024 * sizeof(float))); w->owned.push_back(b1);
    fold_bias(ctx, w->f[TRN_W1], 128, 1024, 0, 1024, w->f[TRN_LN_B], w->f[TRN_B1], 1.0f, b1);
    w->h.assign(2, nullptr);
    w->h[0] = img;
    w->h[1] = b1;
  }
  // Operands of the plain fp16 GEMM for the widths the fused kernels do not take: weights [k][n] -> fp16 [n][k]
  auto operand = [&](const float* src, int K, int ldw, int col0, int N, op16* dst) {
    gemm_operand_kernel<<<(unsigned)(((int64_t)N * K + 255) / 256), 256, 0, ctx->stream>>>(src, K, ldw, col0, N, dst);
  };
  auto alloc16 = [&](int64_t count, op16** out) -> lf_status {
    LF_CUDA(ctx, cudaMalloc(out, (size_t)count * sizeof(op16)));
    w->owned.push_back(*out);
    return LF_OK;
  };
  if (w->kind == LF_WEIGHTS_ATTENTION_AF2 && (w->h.empty() || !w->h[0]) && w->dims.heads > 0 && w->dims.channels % w->dims.heads == 0 &&
      w->dims.channels % 8 == 0) {
    const int c = w->dims.channels, HD = c;          // heads * (channels / heads)
    op16 *w4 = nullptr, *wo = nullptr;
    LF_TRY(alloc16((int64_t)4 * HD * c, &w4));
    LF_TRY(alloc16((int64_t)c * HD, &wo));
    operand(w->f[ATT_W4], c, 4 * HD, 0, 4 * HD, w4);
    operand(w->f[ATT_WO], HD, c, 0, c, wo);
    w->g = {w4, wo};
  }
  if ((w->kind == LF_WEIGHTS_TRANSITION_AF2 || w->kind == LF_WEIGHTS_TRANSITION_AF3) && w->h.empty() &&
      w->dims.channels % 8 == 0 && w->dims.hidden % 8 == 0) {
    const int c = w->dims.channels, hd = w->dims.hidden, wide = w->kind == LF_WEIGHTS_TRANSITION_AF3 ? 2 * hd : hd;
    op16 *w1 = nullptr, *w2 = nullptr;
    LF_TRY(alloc16((int64_t)wide * (c + 16), &w1));      // first projection: [wide][c + 16], its bias in column c
    LF_TRY(alloc16((int64_t)c * hd, &w2));
    gemm_operand_bias_kernel<<<(unsigned)(((int64_t)wide * (c + 16) + 255) / 256), 256, 0, ctx->stream>>>(w->f[TRN_W1], c, wide, wide,
                                                                                                       w->f[TRN_B1], w1);
    operand(w->f[TRN_W2], hd, c, 0, c, w2);
    w->g = {w1, w2};
  }
  if (w->kind == LF_WEIGHTS_OPM_AF2 && w->dims.channels % 8 == 0 && w->dims.hidden % 8 == 0 && w->dims.out_channels % 8 == 0) {
    const int cm = w->dims.channels, c = w->dims.hidden, cz = w->dims.out_channels;
    op16 *wlr = nullptr, *wout = nullptr;
    LF_TRY(alloc16((int64_t)2 * c * cm, &wlr));
    LF_TRY(alloc16((int64_t)cz * c * c, &wout));
    operand(w->f[OPM_WL], cm, c, 0, c, wlr);
    operand(w->f[OPM_WR], cm, c, 0, c, wlr + (int64_t)c * cm);
    operand(w->f[OPM_WOUT], c * c, cz, 0, cz, wout);
    w->g = {wlr, wout};
  }
  LF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return LF_OK;
}

// ---------------------------------------------------------------------------
// Triangle contraction.
//
// One 128 x 256 output tile of one channel per work item, K stepped by 64 through
// a 4-stage TMA ring, float32 accumulators double-buffered in TMEM (2 x 256
// columns) so the epilogue of a tile overlaps the main loop of the next.
// Warp roles: 0 = TMA producer, 1 = MMA issuer (owns TMEM), 2..5 = epilogue.
// MAJOR 0: both operands K-major (outgoing).  MAJOR 1: both MN-major (incoming),
// fetched as 64 x 64 boxes whose rows are k.

constexpr int CT_BM = 128, CT_BN = 256, CT_BK = 64, CT_STAGES = 4;
constexpr int CT_A_BYTES = CT_BM * CT_BK * 2;   // 16 KiB
constexpr int CT_B_BYTES = CT_BN * CT_BK * 2;   // 32 KiB
constexpr int CT_STAGE_BYTES = CT_A_BYTES + CT_B_BYTES;
constexpr int CT_OUT_STAGE = 32 * 256;          // per epilogue warp: 32 rows x 128 fp16 columns, for stores into a peer's memory
// EW epilogue warps: 4 for the triangle contraction (long k loops hide the epilogue), 8 for the plain GEMMs, whose k
// loop of 4 to 16 blocks is shorter than a 4-warp epilogue of the 128 x 256 tile; the 8-warp form gives a stage
// of the operand ring to the four extra staging areas.
constexpr int ct_stages(int ew) { return ew == 8 ? 3 : CT_STAGES; }
constexpr int ct_smem(int ew) { return ct_stages(ew) * CT_STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/ + ew * CT_OUT_STAGE; }
constexpr int ct_threads(int ew) { return 64 + 32 * ew; }

// Extras of the plain-GEMM uses of the kernel (local stores): a bias per output column and a ReLU in the epilogue;
// `group_c` > 0: rows are (i, a) and columns (j, b) with a, b < group_c, and element (i, a, j, b) is stored at
// ((i * group_n + j) * group_c + a) * group_c + b - the outer product mean's sums grouped per pair (i, j), which a
// warp writes as whole 2 * group_c^2-byte runs.  `staged`: local rows leave in 256-byte runs through the staging
// rows, as rows bound for a peer do (a GEMM with a short k loop is bound by its stores otherwise).
struct ContractExtra { const float* bias; int relu; int group_c; int group_n; int staged; };

__device__ __forceinline__ uint32_t relu_half2(uint32_t v) {      // max(v, 0) on two packed fp16 values
  const __half2 r = __hmax2(*reinterpret_cast<const __half2*>(&v), __float2half2_rn(0.f));
  return *reinterpret_cast<const uint32_t*>(&r);
}

template <int MAJOR, int EW = 4>
__global__ void __launch_bounds__(ct_threads(EW), 1)
contract_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                op16* __restrict__ x, int m_rows, int n_rows, int k_len, int ldx, int64_t x_plane, int col0, int c,
                float scale, Status* status, const __grid_constant__ PeerPtrs xpeer, int rows_per_rank, int ch0,
                const ContractExtra ex) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  constexpr int ST = EW == 8 ? 3 : CT_STAGES;      // = ct_stages(EW)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ST * CT_STAGE_BYTES);
  uint64_t* full = bars;                       // [STAGES]
  uint64_t* empty = bars + ST;                 // [STAGES]
  uint64_t* tmem_full = bars + 2 * ST;         // [2]
  uint64_t* tmem_empty = tmem_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* out_stage = smem + ST * CT_STAGE_BYTES + 256;     // [EW epilogue warps][CT_OUT_STAGE]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // x[h][i][col0 + j] for i < m_rows, j < n_rows; the contraction index runs over k_len
  const int tiles_m = (m_rows + CT_BM - 1) / CT_BM, tiles_n = (n_rows + CT_BN - 1) / CT_BN;
  const int tiles_per_h = tiles_m * tiles_n;
  const int total = c * tiles_per_h;
  const int kblocks = (k_len + CT_BK - 1) / CT_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&tmem_full[b], 1); mbar_init(&tmem_empty[b], EW); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&mapA);
      prefetch_tensormap(&mapB);
      int stage = 0; uint32_t phase = 0;
      for (int t = blockIdx.x; t < total; t += gridDim.x) {
        const int h = t / tiles_per_h, rem = t % tiles_per_h, mi = rem / tiles_n, nj = rem % tiles_n;
        bool ok = true;
        for (int kb = 0; kb < kblocks && ok; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, status, 1)) { ok = false; break; }
          uint8_t* sA = smem + stage * CT_STAGE_BYTES;
          uint8_t* sB = sA + CT_A_BYTES;
          mbar_expect_tx(&full[stage], CT_STAGE_BYTES);
          if (MAJOR == 0) {
            tma_load_3d(sA, &mapA, &full[stage], kb * CT_BK, mi * CT_BM, h);
            tma_load_3d(sB, &mapB, &full[stage], kb * CT_BK, nj * CT_BN, h);
          } else {
#pragma unroll
            for (int q = 0; q < CT_BM / 64; ++q) tma_load_3d(sA + q * 8192, &mapA, &full[stage], mi * CT_BM + q * 64, kb * CT_BK, h);
#pragma unroll
            for (int q = 0; q < CT_BN / 64; ++q) tma_load_3d(sB + q * 8192, &mapB, &full[stage], nj * CT_BN + q * 64, kb * CT_BK, h);
          }
          if (++stage == ST) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(CT_BM, CT_BN, MAJOR, MAJOR);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      for (int t = blockIdx.x; t < total; t += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(&tmem_empty[buf], ((it >> 1) & 1) ^ 1, abort_flag, status, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * CT_BN;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!mbar_wait(&full[stage], phase, abort_flag, status, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * CT_STAGE_BYTES);
          const uint32_t b_addr = a_addr + CT_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < CT_BK / 16; ++kk) {
            uint64_t adesc, bdesc;
            if (MAJOR == 0) {
              adesc = make_smem_desc(a_addr + kk * 32, 16, 1024);
              bdesc = make_smem_desc(b_addr + kk * 32, 16, 1024);
            } else {
              adesc = make_smem_desc(a_addr + kk * 2048, 8192, 1024);
              bdesc = make_smem_desc(b_addr + kk * 2048, 8192, 1024);
            }
            umma_f16(d_tmem, adesc, bdesc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);
          if (++stage == ST) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tmem_full[buf]);
      }
    }
  } else {
    const int q = warp & 3;                 // TMEM lane quadrant this warp may read
    const int chalf = (warp - 2) >> 2;      // EW == 8: the half of the tile's 256 columns this warp takes
    const int row = q * 32 + lane;
    int it = 0;
    for (int t = blockIdx.x; t < total; t += gridDim.x, ++it) {
      const int h = t / tiles_per_h, rem = t % tiles_per_h, mi = rem / tiles_n, nj = rem % tiles_n;
      const int buf = it & 1;
      if (!mbar_wait(&tmem_full[buf], (it >> 1) & 1, abort_flag, status, 4)) break;
      tc_fence_after();
      const int gi = mi * CT_BM + row;
      op16* dst_row;
      if (rows_per_rank > 0) {
        // row gi of the product belongs to rank gi / rows_per_rank: stored into that rank's
        // [channels][rows_per_rank][ldx] buffer (x_plane = rows_per_rank * ldx)
        int owner = gi / rows_per_rank;
        if (gi >= m_rows) owner = 0;      // not stored
        dst_row = reinterpret_cast<op16*>(xpeer.p[owner]) + (int64_t)(ch0 + h) * x_plane + (int64_t)(gi - owner * rows_per_rank) * ldx + col0;
      } else {
        dst_row = x + (int64_t)h * x_plane + (int64_t)gi * ldx + col0;
      }
      const int col_limit = (n_rows + 15) / 16 * 16 < ldx - col0 ? (n_rows + 15) / 16 * 16 : ldx - col0;
      if (rows_per_rank > 0 || ex.staged) {
        // Rows bound for another GPU leave in 256-byte runs: a thread holds a row of the accumulator, so its
        // own stores would be 16-byte pieces 32 rows apart, which NVLink carries as 32 small packets.  The
        // warp's 32 rows x 128 columns are turned round in shared memory (16-byte pieces swizzled by row)
        // and written two rows per instruction, 16 lanes x 16 bytes each.
        uint8_t* stage = out_stage + (warp - 2) * CT_OUT_STAGE;
        const int g_row0 = mi * CT_BM + q * 32;            // the warp's rows share an owner: rows_per_rank % 128 == 0
        const int owner = rows_per_rank > 0 && g_row0 < m_rows ? g_row0 / rows_per_rank : 0;
        op16* owner_base = rows_per_rank > 0 ? reinterpret_cast<op16*>(xpeer.p[owner]) + (int64_t)(ch0 + h) * x_plane + col0
                                             : x + (int64_t)h * x_plane + col0;
#pragma unroll 1
        for (int half = (EW == 8 ? chalf : 0); half < (EW == 8 ? chalf + 1 : 2); ++half) {
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            uint32_t r[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * CT_BN + half * 128 + cc * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(r[v * 8 + e]) * scale;
              if (ex.bias) {
                const int gj = nj * CT_BN + half * 128 + (cc * 4 + v) * 8;
                if (gj + 8 <= n_rows) {      // bias is 16-byte aligned and gj a multiple of 8
                  const float4 b0 = __ldg(reinterpret_cast<const float4*>(ex.bias + gj));
                  const float4 b1 = __ldg(reinterpret_cast<const float4*>(ex.bias + gj + 4));
                  o[0] += b0.x; o[1] += b0.y; o[2] += b0.z; o[3] += b0.w;
                  o[4] += b1.x; o[5] += b1.y; o[6] += b1.z; o[7] += b1.w;
                } else {
#pragma unroll
                  for (int e = 0; e < 8; ++e) o[e] += gj + e < n_rows ? __ldg(ex.bias + gj + e) : 0.f;
                }
              }
              uint4 pk;
              pk.x = pack_half2(o[0], o[1]);
              pk.y = pack_half2(o[2], o[3]);
              pk.z = pack_half2(o[4], o[5]);
              pk.w = pack_half2(o[6], o[7]);
              if (ex.relu) { pk.x = relu_half2(pk.x); pk.y = relu_half2(pk.y); pk.z = relu_half2(pk.z); pk.w = relu_half2(pk.w); }
              *reinterpret_cast<uint4*>(stage + lane * 256 + (((cc * 4 + v) ^ (lane & 15)) << 4)) = pk;
            }
          }
          __syncwarp();
#pragma unroll 4
          for (int rr = 0; rr < 16; ++rr) {
            const int srow = rr * 2 + (lane >> 4), piece = lane & 15;
            const uint4 pk = *reinterpret_cast<const uint4*>(stage + srow * 256 + ((piece ^ (srow & 15)) << 4));
            const int grow = g_row0 + srow, gj = nj * CT_BN + half * 128 + piece * 8;
            if (grow < m_rows && gj < col_limit)
              *reinterpret_cast<uint4*>(owner_base + (int64_t)(grow - owner * rows_per_rank) * ldx + gj) = pk;
          }
          __syncwarp();
        }
      } else
#pragma unroll 1
      for (int cc = (EW == 8 ? chalf * 4 : 0); cc < (EW == 8 ? chalf * 4 + 4 : CT_BN / 32); ++cc) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * CT_BN + cc * 32, r);
        tmem_ld_wait();
        const int gj0 = nj * CT_BN + cc * 32;   // column inside the window
        if (gi < m_rows) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int gj = gj0 + v * 8;
            if (gj < col_limit) {
              float o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(r[v * 8 + e]) * scale;
              if (ex.bias) {
                if (gj + 8 <= n_rows) {      // bias is 16-byte aligned and gj a multiple of 8
                  const float4 b0 = __ldg(reinterpret_cast<const float4*>(ex.bias + gj));
                  const float4 b1 = __ldg(reinterpret_cast<const float4*>(ex.bias + gj + 4));
                  o[0] += b0.x; o[1] += b0.y; o[2] += b0.z; o[3] += b0.w;
                  o[4] += b1.x; o[5] += b1.y; o[6] += b1.z; o[7] += b1.w;
                } else {
#pragma unroll
                  for (int e = 0; e < 8; ++e) o[e] += gj + e < n_rows ? __ldg(ex.bias + gj + e) : 0.f;
                }
              }
              uint4 pk;
              pk.x = pack_half2(o[0], o[1]);
              pk.y = pack_half2(o[2], o[3]);
              pk.z = pack_half2(o[4], o[5]);
              pk.w = pack_half2(o[6], o[7]);
              if (ex.relu) { pk.x = relu_half2(pk.x); pk.y = relu_half2(pk.y); pk.z = relu_half2(pk.z); pk.w = relu_half2(pk.w); }
              if (ex.group_c) {
                const int gc = ex.group_c;
                *reinterpret_cast<uint4*>(x + ((((int64_t)(gi / gc) * ex.group_n + gj / gc) * gc + gi % gc) * gc + gj % gc)) = pk;
              } else {
                *reinterpret_cast<uint4*>(dst_row + gj) = pk;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) drain_after_abort();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// Kernel attributes belong to a device (context), the driver entry point to the process.
void configure_once() {
  std::call_once(g_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    else
      cudaGetLastError();
  });
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return; }
  static std::once_flag per_device[64];
  std::call_once(per_device[dev], [] {
    cudaFuncSetAttribute(contract_kernel<0, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, ct_smem(4));
    cudaFuncSetAttribute(contract_kernel<1, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, ct_smem(4));
    cudaFuncSetAttribute(contract_kernel<0, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, ct_smem(8));
    cudaFuncSetAttribute(contract_kernel<1, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, ct_smem(8));
    configure_ln_gemm();
    configure_attention();
    configure_transition();
    cudaGetLastError();
  });
}

bool contract_supported(int n, int c) { return n >= 1 && c >= 1 && g_encode != nullptr; }

static lf_status contract_impl(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, op16* x, int m_rows, int n_rows,
                               int k_len, int ld_ab, int ldx, int64_t x_plane, int col0, int c, int incoming, float scale,
                               const PeerPtrs* peers, int rows_per_rank, int ch0,
                               ContractExtra ex = ContractExtra{nullptr, 0, 0, 0, 0});

lf_status contract_rect(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, op16* x, int m_rows, int n_rows,
                        int k_len, int ld_ab, int ldx, int64_t x_plane, int col0, int c, int incoming, float scale) {
  return contract_impl(ctx, cur, a, b, x, m_rows, n_rows, k_len, ld_ab, ldx, x_plane, col0, c, incoming, scale, nullptr, 0, 0);
}

lf_status contract_scatter(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, int n, int ld, int c, int incoming,
                           float scale, const PeerPtrs& x_peers, int rows_per_rank, int total_channels, int ch0) {
  (void)total_channels;
  // the product's planes at the row owners hold rows_per_rank rows of ld elements
  return contract_impl(ctx, cur, a, b, nullptr, n, n, n, ld, ld, (int64_t)rows_per_rank * ld, 0, c, incoming, scale, &x_peers,
                       rows_per_rank, ch0);
}

lf_status contract_gemm(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* w, op16* out, int m_rows, int n_out,
                        int k_len, const float* bias, int relu) {
  return contract_impl(ctx, cur, a, w, out, m_rows, n_out, k_len, k_len, n_out, 0, 0, 1, 0, 1.0f, nullptr, 0, 0,
                       ContractExtra{bias, relu, 0, 0, 1});
}

lf_status contract_outer(lf_context* ctx, ArenaCursor& cur, const op16* left, const op16* right, op16* out, int cnt, int n, int c,
                         int k_len, float scale) {
  if (c % 8 != 0) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "the grouped outer product needs c in whole groups of 8");
  // x[(i, a)][(j, b)] = scale * sum_s left[s][(i, a)] right[s][(j, b)]: both operands MN-major, the kernel's "b" is its M operand
  return contract_impl(ctx, cur, right, left, out, cnt * c, n * c, k_len, n * c, n * c, 0, 0, 1, 1, scale, nullptr, 0, 0,
                       ContractExtra{nullptr, 0, c, n, 0});
}

static lf_status contract_impl(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, op16* x, int m_rows, int n_rows,
                               int k_len, int ld_ab, int ldx, int64_t x_plane, int col0, int c, int incoming, float scale,
                               const PeerPtrs* peers, int rows_per_rank, int ch0, ContractExtra ex) {
  if (cur.dry) return LF_OK;
  // a row of an operand holds k (K-major form) or the M / N index (MN-major form)
  const int row_len = incoming ? (m_rows > n_rows ? m_rows : n_rows) : k_len;
  if (ld_ab % 8 != 0 || ld_ab < row_len || ldx % 8 != 0 || col0 % 8 != 0)
    return lf_fail(ctx, LF_ERR_ARGUMENT, "contraction strides must be multiples of 8 and cover the row");
  CUtensorMap mapA, mapB;
  const uint64_t row_bytes = (uint64_t)ld_ab * 2;
  if (!incoming) {
    LF_TRY(make_map_f16_3d(ctx, &mapA, a, k_len, m_rows, c, row_bytes, (uint64_t)m_rows * row_bytes, CT_BK, CT_BM));
    LF_TRY(make_map_f16_3d(ctx, &mapB, b, k_len, n_rows, c, row_bytes, (uint64_t)n_rows * row_bytes, CT_BK, CT_BN));
  } else {
    // A(i,k) = b[h][k][i], B(j,k) = a[h][k][j]: boxes of 64 (i or j) x 64 (k)
    LF_TRY(make_map_f16_3d(ctx, &mapA, b, m_rows, k_len, c, row_bytes, (uint64_t)k_len * row_bytes, 64, CT_BK));
    LF_TRY(make_map_f16_3d(ctx, &mapB, a, n_rows, k_len, c, row_bytes, (uint64_t)k_len * row_bytes, 64, CT_BK));
  }
  const int tiles = c * ((m_rows + CT_BM - 1) / CT_BM) * ((n_rows + CT_BN - 1) / CT_BN);
  const int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
  lf_prof_begin(ctx, LF_KERNEL_TRIANGLE_CONTRACT);
#define CT_LAUNCH(MAJ, EWN) \
  contract_kernel<MAJ, EWN><<<grid, ct_threads(EWN), ct_smem(EWN), ctx->stream>>>(mapA, mapB, x, m_rows, n_rows, k_len, ldx, x_plane, col0, c, \
      scale, (Status*)ctx->tc_status, peers ? *peers : PeerPtrs{}, rows_per_rank, ch0, ex)
  const bool wide_epilogue = (ex.staged || ex.group_c) && !peers;      // the plain-GEMM uses
  if (!incoming) { if (wide_epilogue) CT_LAUNCH(0, 8); else CT_LAUNCH(0, 4); }
  else { if (wide_epilogue) CT_LAUNCH(1, 8); else CT_LAUNCH(1, 4); }
#undef CT_LAUNCH
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

lf_status contract(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, op16* x, int n, int ld, int c,
                   int incoming, float scale) {
  return contract_rect(ctx, cur, a, b, x, n, n, n, ld, ld, (int64_t)n * ld, 0, c, incoming, scale);
}

}  // namespace tc
