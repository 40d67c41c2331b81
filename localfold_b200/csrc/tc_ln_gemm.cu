// LayerNorm -> projection kernels on tcgen05 for 128-channel activations.
//
// One persistent CTA per SM.  The projection weights (W^T, fp16, up to 528 x 128)
// stay resident in shared memory in the 128-byte-swizzled K-major layout the
// tensor core reads; each 128-row tile of the activation is normalised in
// registers by four producer warps (one row per warp-wide load, statistics by
// warp shuffle), written as the fp16 A operand straight into swizzled shared
// memory, multiplied in chunks of up to 256 output columns into double-buffered
// TMEM accumulators, and finished by eight epilogue warps (bias, sigmoid gates,
// mask, layout change) while the next chunk's MMAs run.
//
// Warp roles: 0..7 epilogue (TMEM lane quadrant = warp % 4, column half = warp / 4),
// 8..11 LayerNorm producers, 12 MMA issuer and TMEM owner.
#include <cuda.h>

#include "tc05.cuh"
#include "tc_kernels.cuh"

namespace tc {

using namespace tc05;

constexpr int LG_THREADS = 13 * 32;
constexpr int LG_ROWS = 128;
constexpr int LG_K = 128;
constexpr int LG_A_BYTES = LG_ROWS * LG_K * 2;          // 32 KiB per stage, two 16 KiB k-atoms
constexpr int LG_MAX_CHUNKS = 3;

struct LnGemmParams {
  const void* act;          // [rows][128] f32 or bf16, memory order
  int act_bf16;
  int64_t rows;             // logical rows
  int transpose, batch, Q;  // logical row (b, i) reads memory row i*batch + b when transpose
  const float* gamma;
  const float* beta;
  float eps;
  int variance;             // 1 two-pass, 2 fast
  const uint8_t* wimg;      // swizzled fp16 image of W^T: [2 atoms][n_pad rows][128 B]
  int n_pad;
  const float* bias;        // [n_pad]
  int n_chunks;
  int chunk_n[LG_MAX_CHUNKS];
  int chunk_row0[LG_MAX_CHUNKS];
  // triangle projection epilogue
  const float* mask;        // [rows]
  op16* out_a;              // [c][n][ld]
  op16* out_b;
  int n, ld;
  // attention projection epilogue
  op16* out_q; op16* out_k; op16* out_v; op16* out_g;   // [rows][128] logical order
  float* out_bias;          // [heads][Q][Q]
  int heads, bias_swap;
  float q_scale;
  Status* status;
};

enum { LG_EPI_TRIANGLE = 0, LG_EPI_ATTENTION = 1 };

__device__ __forceinline__ float sigmoid_fast(float v) { return __frcp_rn(1.0f + __expf(-v)); }

template <int EPI>
__global__ void __launch_bounds__(LG_THREADS, 1) ln_gemm_kernel(const LnGemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int w_bytes = p.n_pad * 256;
  uint8_t* sW = smem;
  uint8_t* sA = smem + w_bytes;                       // 2 stages (w_bytes is a multiple of 1024: n_pad % 8 == 0... x256)
  float* sBias = reinterpret_cast<float*>(sA + 2 * LG_A_BYTES);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sBias + 544);
  uint64_t* a_full = bars;          // [2]
  uint64_t* a_empty = bars + 2;     // [2]
  uint64_t* acc_full = bars + 4;    // [2]
  uint64_t* acc_empty = bars + 6;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tiles = (p.rows + LG_ROWS - 1) / LG_ROWS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&a_full[s], 4);
      mbar_init(&a_empty[s], 1);
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  // resident weights: straight copy of the pre-swizzled image
  {
    const uint4* src = reinterpret_cast<const uint4*>(p.wimg);
    uint4* dst = reinterpret_cast<uint4*>(sW);
    for (int i = threadIdx.x; i < w_bytes / 16; i += LG_THREADS) dst[i] = src[i];
    for (int i = threadIdx.x; i < p.n_pad; i += LG_THREADS) sBias[i] = p.bias[i];
    fence_async_smem();
  }
  if (warp == 12) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 8 && warp < 12) {
    // ---------------- LayerNorm producers ----------------
    const int pw = warp - 8;
    const float4 g4 = reinterpret_cast<const float4*>(p.gamma)[lane];
    const float4 b4 = reinterpret_cast<const float4*>(p.beta)[lane];
    int it = 0;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x, ++it) {
      const int s = it & 1;
      if (!mbar_wait(&a_empty[s], ((it >> 1) & 1) ^ 1, abort_flag, p.status, 10)) break;
      uint8_t* tile = sA + s * LG_A_BYTES;
      // 16 rows per batch: all loads of a batch are issued before any is consumed, which
      // keeps 64 rows (32 KiB) in flight per SM across the four producer warps
#pragma unroll 1
      for (int r0 = 0; r0 < 32; r0 += 16) {
        float4 vals[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int64_t r = t * LG_ROWS + pw * 32 + r0 + u;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (r < p.rows) {
            int64_t src = r;
            if (p.transpose) { int64_t b = r / p.Q, i = r % p.Q; src = i * p.batch + b; }
            if (p.act_bf16) {
              const uint2 raw = reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p.act) + src * LG_K)[lane];
              const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
              const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
              v = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
            } else {
              v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.act) + src * LG_K)[lane];
            }
          }
          vals[u] = v;
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int row = pw * 32 + r0 + u;
          const bool valid = t * LG_ROWS + row < p.rows;
          const float4 v = vals[u];
          float sum = v.x + v.y + v.z + v.w;
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
          const float mean = sum * (1.0f / LG_K);
          float var;
          if (p.variance == 2) {
            float sq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            var = sq * (1.0f / LG_K) - mean * mean;
          } else {
            const float dx = v.x - mean, dy = v.y - mean, dz = v.z - mean, dw = v.w - mean;
            float sq = dx * dx + dy * dy + dz * dz + dw * dw;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            var = sq * (1.0f / LG_K);
          }
          float inv = rsqrtf(var + p.eps);
          inv = inv * (1.5f - 0.5f * (var + p.eps) * inv * inv);
          uint2 packed = make_uint2(0u, 0u);
          if (valid) {
            packed.x = pack_half2((v.x - mean) * inv * g4.x + b4.x, (v.y - mean) * inv * g4.y + b4.y);
            packed.y = pack_half2((v.z - mean) * inv * g4.z + b4.z, (v.w - mean) * inv * g4.w + b4.w);
          }
          // channels 4*lane .. 4*lane+3: k-atom lane/16, 16-byte chunk (lane%16)/2, 8-byte half lane%2
          const uint32_t off = (uint32_t)(lane >> 4) * (LG_ROWS * 128) +
                               swizzle128_offset((uint32_t)row, (uint32_t)((lane & 15) >> 1)) + (uint32_t)(lane & 1) * 8u;
          *reinterpret_cast<uint2*>(tile + off) = packed;
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[s]);
    }
  } else if (warp == 12) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int it = 0;
      uint32_t g = 0;
      for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x, ++it) {
        const int s = it & 1;
        if (!mbar_wait(&a_full[s], (it >> 1) & 1, abort_flag, p.status, 11)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + s * LG_A_BYTES);
        bool ok = true;
        for (int j = 0; j < p.n_chunks; ++j, ++g) {
          const int b = g & 1;
          if (!mbar_wait(&acc_empty[b], ((g >> 1) & 1) ^ 1, abort_flag, p.status, 12)) { ok = false; break; }
          tc_fence_after();
          const uint32_t idesc = make_idesc_f16(LG_ROWS, p.chunk_n[j], 0, 0);
          const uint32_t w_addr = smem_u32(sW) + p.chunk_row0[j] * 128;
#pragma unroll
          for (int kk = 0; kk < LG_K / 16; ++kk) {
            const uint64_t adesc = make_smem_desc(a_addr + (kk >> 2) * (LG_ROWS * 128) + (kk & 3) * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc(w_addr + (kk >> 2) * (p.n_pad * 128) + (kk & 3) * 32, 16, 1024);
            umma_f16(tmem_base + b * 256, adesc, bdesc, idesc, kk != 0 ? 1u : 0u);
          }
          umma_commit(&acc_full[b]);
        }
        if (!ok) break;
        umma_commit(&a_empty[s]);
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3, half = warp >> 2;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    uint32_t g = 0;
    bool ok = true;
    for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
      const int64_t r = t * LG_ROWS + row;
      const bool valid = r < p.rows;
      for (int j = 0; j < p.n_chunks; ++j, ++g) {
        const int b = g & 1;
        if (!mbar_wait(&acc_full[b], (g >> 1) & 1, abort_flag, p.status, 13)) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + lane_addr + b * 256;
        if (EPI == LG_EPI_TRIANGLE) {
          // chunk j = (projection h 0..127 | gate h 0..127) of operand j (0 = a, 1 = b)
          const float m = valid ? p.mask[r] : 0.f;
          const int64_t i = valid ? r / p.n : 0, k = valid ? r % p.n : 0;
          op16* dst = (j == 0 ? p.out_a : p.out_b) + i * p.ld + k;
          const int64_t plane = (int64_t)p.n * p.ld;
          const float* bias = sBias + j * 256;
#pragma unroll 1
          for (int h0 = half * 64; h0 < half * 64 + 64; h0 += 32) {
            uint32_t pv[32], gv[32];
            tmem_ld32(acc + h0, pv);
            tmem_ld32(acc + 128 + h0, gv);
            tmem_ld_wait();
            if (valid) {
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                const int h = h0 + e;
                const float val = m * (__uint_as_float(pv[e]) + bias[h]) * sigmoid_fast(__uint_as_float(gv[e]) + bias[128 + h]);
                dst[h * plane] = __float2half_rn(val);
              }
            }
          }
        } else {
          if (j < 2) {
            // chunk 0 = (q | k), chunk 1 = (v | gate); this warp's half picks the tensor
            op16* out = j == 0 ? (half == 0 ? p.out_q : p.out_k) : (half == 0 ? p.out_v : p.out_g);
            const float* bias = sBias + j * 256 + half * 128;
            const float mul = (j == 0 && half == 0) ? p.q_scale : 1.0f;
            const bool gate = (j == 1 && half == 1);
#pragma unroll 1
            for (int c0 = 0; c0 < 128; c0 += 32) {
              uint32_t v[32];
              tmem_ld32(acc + half * 128 + c0, v);
              tmem_ld_wait();
              if (valid) {
                uint4* dst = reinterpret_cast<uint4*>(out + r * 128 + c0);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  float f[8];
#pragma unroll
                  for (int u = 0; u < 8; ++u) {
                    float x = __uint_as_float(v[e * 8 + u]) + bias[c0 + e * 8 + u];
                    f[u] = gate ? sigmoid_fast(x) : x * mul;
                  }
                  uint4 pk;
                  pk.x = pack_half2(f[0], f[1]); pk.y = pack_half2(f[2], f[3]);
                  pk.z = pack_half2(f[4], f[5]); pk.w = pack_half2(f[6], f[7]);
                  dst[e] = pk;
                }
              }
            }
          } else if (half == 0) {
            // chunk 2: pair bias, one column per head; logical row r = (q index, k index)
            uint32_t v[16];
            tmem_ld16(acc, v);
            tmem_ld_wait();
            if (valid) {
              const int64_t qi = r / p.Q, ki = r % p.Q;
              const int64_t dst = p.bias_swap ? ki * p.Q + qi : r;
              const int64_t qq = (int64_t)p.Q * p.Q;
#pragma unroll
              for (int h = 0; h < 16; ++h)
                if (h < p.heads) p.out_bias[h * qq + dst] = __uint_as_float(v[h]);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[b]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) drain_after_abort();
  if (warp == 12) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// W (in,out) float32 [K][n_out] -> fp16 image of W^T in the swizzled K-major layout
// ([K/64 atoms][n_pad rows][128 B]); rows >= n_out are zero.
__global__ void pack_weight_image_kernel(const float* __restrict__ w, int K, int n_out, int n_pad, int col0, int ld,
                                         op16* __restrict__ img, int row0) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_out * K) return;
  int n = idx / K, k = idx % K;
  int row = row0 + n;
  size_t off = (size_t)(k >> 6) * ((size_t)n_pad * 128) + (size_t)row * 128 + ((((k & 63) >> 3) ^ (row & 7)) << 4) + (k & 7) * 2;
  img[off / 2] = __float2half_rn(w[(size_t)k * ld + col0 + n]);
}

void pack_weight_image(lf_context* ctx, const float* w, int K, int n_out, int n_pad, int col0, int ld, op16* img, int row0) {
  int total = n_out * K;
  pack_weight_image_kernel<<<(total + 255) / 256, 256, 0, ctx->stream>>>(w, K, n_out, n_pad, col0, ld, img, row0);
}

static int ln_gemm_smem(int n_pad) { return n_pad * 256 + 2 * LG_A_BYTES + 544 * 4 + 128 + 1024; }

void configure_ln_gemm() {
  cudaFuncSetAttribute(ln_gemm_kernel<LG_EPI_TRIANGLE>, cudaFuncAttributeMaxDynamicSharedMemorySize, ln_gemm_smem(512));
  cudaFuncSetAttribute(ln_gemm_kernel<LG_EPI_ATTENTION>, cudaFuncAttributeMaxDynamicSharedMemorySize, ln_gemm_smem(528));
  cudaGetLastError();
}

lf_status triangle_project(lf_context* ctx, ArenaCursor& cur, const void* z, int act_dtype, const float* mask, int n,
                           int ld, int variance, float eps, const lf_weights* w, op16* a, op16* b) {
  if (cur.dry) return LF_OK;
  LnGemmParams p{};
  p.act = z; p.act_bf16 = act_dtype == LF_DTYPE_BF16; p.rows = (int64_t)n * n; p.transpose = 0; p.batch = 1; p.Q = 1;
  p.gamma = w->f[TRI_LN_G]; p.beta = w->f[TRI_LN_B]; p.eps = eps; p.variance = variance;
  p.wimg = (const uint8_t*)w->h[0]; p.n_pad = 512; p.bias = w->f[TRI_B4];
  p.n_chunks = 2; p.chunk_n[0] = 256; p.chunk_n[1] = 256; p.chunk_row0[0] = 0; p.chunk_row0[1] = 256;
  p.mask = mask; p.out_a = a; p.out_b = b; p.n = n; p.ld = ld; p.status = (Status*)ctx->tc_status;
  const int64_t tiles = (p.rows + LG_ROWS - 1) / LG_ROWS;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_LN_GEMM);
  ln_gemm_kernel<LG_EPI_TRIANGLE><<<grid, LG_THREADS, ln_gemm_smem(512), ctx->stream>>>(p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

lf_status attention_project(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int batch, int Q,
                            int transpose, int variance, float eps, int heads, int head_dim, int bias_swap,
                            const lf_weights* w, op16* q, op16* k, op16* v, op16* g, float* bias) {
  if (cur.dry) return LF_OK;
  LnGemmParams p{};
  p.act = act; p.act_bf16 = act_dtype == LF_DTYPE_BF16; p.rows = (int64_t)batch * Q; p.transpose = transpose; p.batch = batch; p.Q = Q;
  p.gamma = w->f[ATT_LN_G]; p.beta = w->f[ATT_LN_B]; p.eps = eps; p.variance = variance;
  p.wimg = (const uint8_t*)w->h[0]; p.n_pad = 528; p.bias = (const float*)w->h[1];
  p.n_chunks = bias ? 3 : 2;
  p.chunk_n[0] = 256; p.chunk_n[1] = 256; p.chunk_n[2] = 16;
  p.chunk_row0[0] = 0; p.chunk_row0[1] = 256; p.chunk_row0[2] = 512;
  p.out_q = q; p.out_k = k; p.out_v = v; p.out_g = g; p.out_bias = bias; p.heads = heads; p.bias_swap = bias_swap;
  p.q_scale = 1.0f / sqrtf((float)head_dim);
  p.status = (Status*)ctx->tc_status;
  const int64_t tiles = (p.rows + LG_ROWS - 1) / LG_ROWS;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_LN_GEMM);
  ln_gemm_kernel<LG_EPI_ATTENTION><<<grid, LG_THREADS, ln_gemm_smem(528), ctx->stream>>>(p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

}  // namespace tc
