// Fused pair transition on tcgen05 for 128-channel activations, 512 hidden:
//   AF2 form:  out = resid + relu(LN(x) W1 + b1) W2 + b2              (hidden chunks of 128)
//   AF3 form:  out = resid + (swish(u_gate) * u_value) W2, u = LN(x) W1, W1 = (gate half | value half)
//              (hidden chunks of 64: each first-GEMM chunk is 64 gate + 64 value columns)
// The 4x-wide hidden never leaves the SM: it is produced 128 columns at a time into TMEM,
// passed through bias + ReLU into a swizzled fp16 shared-memory tile, and consumed at once by
// the second GEMM, whose float32 accumulator stays in TMEM across the four chunks.  The weights
// (256 KiB as fp16) do not fit beside the tiles, so each chunk's W1/W2 slices (64 KiB, pre-swizzled
// images) stream from L2 through a two-stage bulk-copy ring.
//
// Warp roles: 0..15 epilogue (TMEM lane quadrant = warp % 4, 32 of 128 columns = warp / 4),
// 16..23 LayerNorm producers, 24 MMA issuer and TMEM owner, 25 weight streamer.
#include <cuda.h>

#include "tc05.cuh"
#include "tc_kernels.cuh"

namespace tc {

using namespace tc05;

constexpr int TR_THREADS = 26 * 32;
constexpr int TR_ROWS = 128;
constexpr int TR_TILE_BYTES = TR_ROWS * 128 * 2;   // 32 KiB: 128 rows x 128 fp16, two k-atoms
constexpr int TR_W_STAGE = 2 * TR_TILE_BYTES;      // AF2: W1 slice (32 KiB) + W2 slice (32 KiB); AF3: 32 KiB + 16 KiB
constexpr int TR_SMEM = 2 * TR_W_STAGE + 2 * TR_TILE_BYTES + (1024 + 128 + 256) * 4 + 256 + 1024;
constexpr int TR_OUT_STAGE = 32 * 64;              // per epilogue warp: 32 rows x 16 float32 channels of the pair

struct TransitionParams {
  const void* act;
  int act_bf16;
  int64_t rows;
  float eps; int variance;
  const uint8_t* wimg;      // per chunk: W1 slice image, then W2 slice image
  const float* b1;          // [512] (AF2) or [1024] = gate half | value half (AF3)
  const float* b2;          // [128]
  const void* resid;
  void* out;
  int tma_out;              // float32 pair updated in place (or no residual): the pair tile travels by TMA through staging rows
  Status* status;
};

__device__ __forceinline__ float sigmoid_tanh(float v) {   // one MUFU: 0.5 + 0.5 tanh(v/2)
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * v));
  return fmaf(0.5f, t, 0.5f);
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

template <bool SWIGLU>
__global__ void __launch_bounds__(TR_THREADS, 1) transition_kernel(const __grid_constant__ CUtensorMap mapO, const TransitionParams p) {
  constexpr int TR_CHUNKS = SWIGLU ? 8 : 4;                 // hidden chunks per tile
  constexpr int HK = SWIGLU ? 64 : 128;                     // hidden channels per chunk = K of the second GEMM
  constexpr uint32_t W_BYTES = SWIGLU ? 3 * TR_TILE_BYTES / 2 : 2 * TR_TILE_BYTES;   // bytes streamed per chunk
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sW = smem;                              // [2 stages][W1 slice | W2 slice]
  uint8_t* sA = sW + 2 * TR_W_STAGE;               // normalised activations (A of GEMM 1)
  uint8_t* sH = sA + TR_TILE_BYTES;                // hidden chunk (A of GEMM 2)
  float* sB1 = reinterpret_cast<float*>(sH + TR_TILE_BYTES);   // [512]
  float* sB2 = sB1 + 1024;                         // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB2 + 128 + 256);
  uint64_t* a_full = bars;            // count 8 producer warps
  uint64_t* a_empty = bars + 1;       // MMA commit
  // the two weight slices of a chunk travel through rings of their own: a first-GEMM slice is released when its GEMM
  // has completed, two chunks before the second-GEMM slice beside it, and is refilled at once
  uint64_t* w1_full = bars + 2;       // [2] bulk bytes
  uint64_t* w1_empty = bars + 4;      // [2] MMA commit
  uint64_t* hacc_full = bars + 6;     // [2] MMA commit
  uint64_t* hacc_empty = bars + 8;    // [2] count 16
  uint64_t* h_full = bars + 10;       // count 16: hidden tile written
  uint64_t* h_empty = bars + 11;      // MMA commit: GEMM 2 has read the hidden tile
  uint64_t* out_full = bars + 12;     // MMA commit
  uint64_t* out_empty = bars + 13;    // count 16
  uint64_t* stage_free = bars + 14;   // count 16: every warp's output copy has finished reading the staging rows
  uint64_t* w2_full = bars + 15;      // [2] bulk bytes
  uint64_t* w2_empty = bars + 17;     // [2] MMA commit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tiles = (p.rows + TR_ROWS - 1) / TR_ROWS;

  if (threadIdx.x == 0) {
    mbar_init(a_full, 8); mbar_init(a_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&w1_full[s], 1); mbar_init(&w1_empty[s], 1); mbar_init(&w2_full[s], 1); mbar_init(&w2_empty[s], 1);
      mbar_init(&hacc_full[s], 1); mbar_init(&hacc_empty[s], 16);
    }
    mbar_init(h_full, 16); mbar_init(h_empty, 1); mbar_init(out_full, 1); mbar_init(out_empty, 16);
    mbar_init(stage_free, 16);
    *abort_flag = 0;
    fence_barrier_init();
  }
  for (int i = threadIdx.x; i < (SWIGLU ? 1024 : 512); i += TR_THREADS) sB1[i] = p.b1[i];
  if (threadIdx.x < 128) sB2[threadIdx.x] = p.b2[threadIdx.x];
  if (warp == 24) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // TMEM columns: hidden accumulators at 0 and 128, output accumulator at 256

  if (warp == 25) {
    // ---------------- weight streamer ----------------
    // lane 0 feeds the first-GEMM slices, lane 1 the second-GEMM slices
    if (lane < 2) {
      uint64_t* full = lane == 0 ? w1_full : w2_full;
      uint64_t* empty = lane == 0 ? w1_empty : w2_empty;
      const uint32_t offset = lane == 0 ? 0u : (uint32_t)TR_TILE_BYTES;
      const uint32_t bytes = lane == 0 ? (uint32_t)TR_TILE_BYTES : W_BYTES - (uint32_t)TR_TILE_BYTES;
      uint32_t g = 0;
      bool ok = true;
      for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
        for (int c = 0; c < TR_CHUNKS; ++c, ++g) {
          const int s = g & 1;
          if (!mbar_wait(&empty[s], ((g >> 1) & 1) ^ 1, abort_flag, p.status, 50)) { ok = false; break; }
          mbar_expect_tx(&full[s], bytes);
          bulk_load(sW + s * TR_W_STAGE + offset, p.wimg + (size_t)c * W_BYTES + offset, bytes, &full[s]);
        }
      }
    }
  } else if (warp >= 16 && warp < 24) {
    // ---------------- LayerNorm producers (8 lanes per row) ----------------
    const int pw = warp - 16;
    const int sub = lane >> 3, j = lane & 7;
    int it = 0;
    const uint32_t row_bytes = p.act_bf16 ? 256u : 512u;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x, ++it) {
      if (pw == 0 && lane == 0 && t + gridDim.x < tiles) {
        // ask for the next tile's rows now: they arrive in L2 while this tile is normalised and multiplied
        const int64_t r0 = (t + gridDim.x) * TR_ROWS;
        const int64_t nrows = p.rows - r0 < TR_ROWS ? p.rows - r0 : TR_ROWS;
        bulk_prefetch_l2(reinterpret_cast<const uint8_t*>(p.act) + r0 * row_bytes, (uint32_t)nrows * row_bytes);
      }
      // The single operand stage is still being read by the previous tile's first GEMMs while this tile is loaded and
      // normalised into registers (both halves): only the stores wait for it.
      uint32_t packed[4][8];
#pragma unroll
      for (int grp = 0; grp < 2; ++grp) {
        float v[2][16];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int row = pw * 16 + (grp * 2 + u) * 4 + sub;
          const int64_t r = t * TR_ROWS + row;
          if (r < p.rows) {
            if (p.act_bf16) {
              // a lane's channels interleave with its neighbours' so that a load reads 128 contiguous bytes
              // per row: 16-bit input, element e is channel 64 (e / 8) + 8 j + e % 8; float, 32 (e / 4) + 4 j + e % 4
              const uint4* g = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.act) + r * 128 + 8 * j);
#pragma unroll
              for (int w4 = 0; w4 < 2; ++w4) {
                const uint4 raw = g[w4 * 8];
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&words[e]);
                  v[u][w4 * 8 + e * 2] = __low2float(h2);
                  v[u][w4 * 8 + e * 2 + 1] = __high2float(h2);
                }
              }
            } else {
              const float4* g = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.act) + r * 128 + 4 * j);
#pragma unroll
              for (int w4 = 0; w4 < 4; ++w4) {
                const float4 f = g[w4 * 8];
                v[u][w4 * 4] = f.x; v[u][w4 * 4 + 1] = f.y; v[u][w4 * 4 + 2] = f.z; v[u][w4 * 4 + 3] = f.w;
              }
            }
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[u][e] = 0.f;
          }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int row = pw * 16 + (grp * 2 + u) * 4 + sub;
          const bool valid = t * TR_ROWS + row < p.rows;
          float s4[4] = {0.f, 0.f, 0.f, 0.f};      // four chains instead of one of 16 dependent additions
#pragma unroll
          for (int e = 0; e < 16; ++e) s4[e & 3] += v[u][e];
          float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          sum += __shfl_xor_sync(0xffffffffu, sum, 4);
          const float mean = sum * (1.0f / 128.0f);
          float q4[4] = {0.f, 0.f, 0.f, 0.f};
          if (p.variance == 2) {
#pragma unroll
            for (int e = 0; e < 16; ++e) q4[e & 3] = fmaf(v[u][e], v[u][e], q4[e & 3]);
          } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) { const float d = v[u][e] - mean; q4[e & 3] = fmaf(d, d, q4[e & 3]); }
          }
          float sq = (q4[0] + q4[1]) + (q4[2] + q4[3]);
          sq += __shfl_xor_sync(0xffffffffu, sq, 1);
          sq += __shfl_xor_sync(0xffffffffu, sq, 2);
          sq += __shfl_xor_sync(0xffffffffu, sq, 4);
          const float var = p.variance == 2 ? sq * (1.0f / 128.0f) - mean * mean : sq * (1.0f / 128.0f);
          float inv = rsqrtf(var + p.eps);
          inv = inv * (1.5f - 0.5f * (var + p.eps) * inv * inv);
          // the LayerNorm's gain and offset live in the first weight image and its bias: the operand is (x - mean) / std
          const float shift = -mean * inv;
#pragma unroll
          for (int e = 0; e < 8; ++e)
            packed[grp * 2 + u][e] = valid ? pack_half2(fmaf(v[u][2 * e], inv, shift), fmaf(v[u][2 * e + 1], inv, shift)) : 0u;
        }
      }
      if (!mbar_wait(a_empty, (it & 1) ^ 1, abort_flag, p.status, 51)) break;
      {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int row = pw * 16 + u * 4 + sub;
          if (p.act_bf16) {
            // channels 64 w + 8 j .. + 7: k-atom w, 16-byte chunk j of the row
#pragma unroll
            for (int w2 = 0; w2 < 2; ++w2)
              *reinterpret_cast<uint4*>(sA + (uint32_t)w2 * (TR_ROWS * 128) + swizzle128_offset((uint32_t)row, (uint32_t)j)) =
                  make_uint4(packed[u][w2 * 4], packed[u][w2 * 4 + 1], packed[u][w2 * 4 + 2], packed[u][w2 * 4 + 3]);
          } else {
            // channels 32 w + 4 j .. + 3: k-atom w / 2, 16-byte chunk 4 (w % 2) + j / 2, its half j % 2
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4)
              *reinterpret_cast<uint2*>(sA + (uint32_t)(w4 >> 1) * (TR_ROWS * 128) +
                                        swizzle128_offset((uint32_t)row, (uint32_t)((w4 & 1) * 4 + (j >> 1))) + (j & 1) * 8) =
                  make_uint2(packed[u][w4 * 2], packed[u][w4 * 2 + 1]);
          }
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(a_full);
    }
  } else if (warp == 24) {
    // ---------------- MMA issuer ----------------
    // The whole warp runs the loop (uniform control flow and operand values, so the operands of the
    // MMA instructions stay in uniform registers); one elected lane issues.
    {
      constexpr uint32_t idesc = make_idesc_f16(TR_ROWS, 128, 0, 0);
      const uint32_t a_addr = smem_u32(sA), h_addr = smem_u32(sH);
      uint32_t g = 0;      // chunk counter across tiles
      int it = 0;
      bool ok = true;
      auto gemm2 = [&](uint32_t gc, int c) {   // out += hidden chunk x W2 slice of chunk counter gc (elected lane)
        const uint32_t w2 = smem_u32(sW + (gc & 1) * TR_W_STAGE + TR_TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < HK / 16; ++kk) {
          const uint64_t adesc = make_smem_desc(h_addr + (kk >> 2) * (TR_ROWS * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(w2 + (kk >> 2) * (128 * 128) + (kk & 3) * 32, 16, 1024);
          umma_f16(tmem_base + 256, adesc, bdesc, idesc, (c | kk) != 0 ? 1u : 0u);
        }
      };
      for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
        if (!mbar_wait(a_full, it & 1, abort_flag, p.status, 52)) break;
        tc_fence_after();
        for (int c = 0; c < TR_CHUNKS; ++c, ++g) {
          const int s = g & 1;
          if (!mbar_wait(&w1_full[s], (g >> 1) & 1, abort_flag, p.status, 54) ||
              !mbar_wait(&hacc_empty[s], ((g >> 1) & 1) ^ 1, abort_flag, p.status, 55)) { ok = false; break; }
          tc_fence_after();
          const uint32_t w1 = smem_u32(sW + s * TR_W_STAGE);
          if (elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t adesc = make_smem_desc(a_addr + (kk >> 2) * (TR_ROWS * 128) + (kk & 3) * 32, 16, 1024);
              const uint64_t bdesc = make_smem_desc(w1 + (kk >> 2) * (128 * 128) + (kk & 3) * 32, 16, 1024);
              umma_f16(tmem_base + s * 128, adesc, bdesc, idesc, kk != 0 ? 1u : 0u);
            }
            umma_commit(&hacc_full[s]);
            umma_commit(&w1_empty[s]);
            if (c == TR_CHUNKS - 1) umma_commit(a_empty);
          }
          __syncwarp();
          if (c >= 1) {
            // second GEMM of the previous chunk, once its hidden tile is in shared memory
            if (!mbar_wait(h_full, (g - 1) & 1, abort_flag, p.status, 56)) { ok = false; break; }
            // the tile's first write of the output accumulator: the previous tile's must have been read
            if (c == 1 && !mbar_wait(out_empty, (it & 1) ^ 1, abort_flag, p.status, 53)) { ok = false; break; }
            if (!mbar_wait(&w2_full[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag, p.status, 63)) { ok = false; break; }
            tc_fence_after();
            if (elect_one()) {
              gemm2(g - 1, c - 1);
              umma_commit(h_empty);
              umma_commit(&w2_empty[(g - 1) & 1]);
            }
            __syncwarp();
          }
        }
        if (!ok) break;
        if (!mbar_wait(h_full, (g - 1) & 1, abort_flag, p.status, 57)) break;
        if (!mbar_wait(&w2_full[(g - 1) & 1], ((g - 1) >> 1) & 1, abort_flag, p.status, 64)) break;
        tc_fence_after();
        if (elect_one()) {
          gemm2(g - 1, TR_CHUNKS - 1);
          umma_commit(h_empty);
          umma_commit(&w2_empty[(g - 1) & 1]);
          umma_commit(out_full);
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3, part = warp >> 2;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const bool out_bf16 = p.act_bf16 != 0;
    uint32_t g = 0;
    int it = 0;
    bool ok = true;
    for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
      const int64_t r = t * TR_ROWS + row;
      const bool valid = r < p.rows;
      for (int c = 0; c < TR_CHUNKS; ++c, ++g) {
        const int s = g & 1;
        if (!mbar_wait(&hacc_full[s], (g >> 1) & 1, abort_flag, p.status, 58)) { ok = false; break; }
        tc_fence_after();
        uint32_t pk[16];
        if (SWIGLU) {
          // hidden channels part*16 .. +15 of the chunk: gate at column j, value at column 64 + j
          uint32_t gt[16], vl[16];
          tmem_ld16(tmem_base + lane_addr + s * 128 + part * 16, gt);
          tmem_ld16(tmem_base + lane_addr + s * 128 + 64 + part * 16, vl);
          tmem_ld_wait();
          // the biases are the same for every lane: read as four 16-byte broadcasts, not sixteen scalars
          float bg[16], bv[16];
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            *reinterpret_cast<float4*>(bg + e4 * 4) = *reinterpret_cast<const float4*>(sB1 + c * 64 + part * 16 + e4 * 4);
            *reinterpret_cast<float4*>(bv + e4 * 4) = *reinterpret_cast<const float4*>(sB1 + 512 + c * 64 + part * 16 + e4 * 4);
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float g0 = __uint_as_float(gt[2 * e]) + bg[2 * e], g1 = __uint_as_float(gt[2 * e + 1]) + bg[2 * e + 1];
            const float v0 = __uint_as_float(vl[2 * e]) + bv[2 * e], v1 = __uint_as_float(vl[2 * e + 1]) + bv[2 * e + 1];
            pk[e] = pack_half2(g0 * sigmoid_tanh(g0) * v0, g1 * sigmoid_tanh(g1) * v1);
          }
        } else {
#pragma unroll
          for (int half16 = 0; half16 < 2; ++half16) {
            uint32_t v[16];
            tmem_ld16(tmem_base + lane_addr + s * 128 + part * 32 + half16 * 16, v);
            tmem_ld_wait();
            float b1[16];
#pragma unroll
            for (int e4 = 0; e4 < 4; ++e4)
              *reinterpret_cast<float4*>(b1 + e4 * 4) = *reinterpret_cast<const float4*>(sB1 + c * 128 + part * 32 + half16 * 16 + e4 * 4);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              pk[half16 * 8 + e] = pack_half2(fmaxf(__uint_as_float(v[2 * e]) + b1[2 * e], 0.f),
                                              fmaxf(__uint_as_float(v[2 * e + 1]) + b1[2 * e + 1], 0.f));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&hacc_empty[s]);
        // the hidden tile is single-buffered: the previous chunk's second GEMM must have read it
        if (!mbar_wait(h_empty, (g & 1) ^ 1, abort_flag, p.status, 59)) { ok = false; break; }
        // ... and it doubles as the staging rows of the previous tile's output: those stores must have read it
        if (p.tma_out && c == 0 && it > 0) {
          // this warp's output copies of the previous tile have had a whole hidden chunk's time to read their rows
          if (lane == 0) { bulk_wait_read(); mbar_arrive(stage_free); }
          __syncwarp();
          if (!mbar_wait(stage_free, (it - 1) & 1, abort_flag, p.status, 61)) { ok = false; break; }
        }
        if (SWIGLU) {
          // 16 hidden channels = chunks 2*part, 2*part+1 of the row's single 64-wide k-atom
#pragma unroll
          for (int ch = 0; ch < 2; ++ch)
            *reinterpret_cast<uint4*>(sH + swizzle128_offset((uint32_t)row, (uint32_t)(part * 2 + ch))) =
                make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        } else {
          // hidden columns part*32 .. +31 of this row: k-atom part/2, chunks 4*(part%2) .. +3
          uint8_t* hb = sH + (uint32_t)(part >> 1) * (TR_ROWS * 128);
#pragma unroll
          for (int ch = 0; ch < 4; ++ch)
            *reinterpret_cast<uint4*>(hb + swizzle128_offset((uint32_t)row, (uint32_t)((part & 1) * 4 + ch))) =
                make_uint4(pk[ch * 4], pk[ch * 4 + 1], pk[ch * 4 + 2], pk[ch * 4 + 3]);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(h_full);
      }
      if (!ok) break;
      if (!mbar_wait(out_full, it & 1, abort_flag, p.status, 60)) break;
      tc_fence_after();
      if (p.tma_out) {
        // The pair tile leaves by TMA from this warp's staging rows (32 rows x 16 channels, twice), which live in
        // the hidden tile's shared memory: it is free once the tile's last second GEMM has completed (out_full).
        // An update in place is a reduce-add of (accumulator + bias) into the rows, so the residual is not read
        // here at all.  A thread owning a row would otherwise touch 32 lines per 32-byte access.
        uint8_t* stage = sH + warp * TR_OUT_STAGE;
        const int64_t row0 = t * TR_ROWS + q * 32;
        const bool any_row = row0 < p.rows;
        uint32_t v[2][16];
        tmem_ld16(tmem_base + lane_addr + 256 + part * 32, v[0]);
        tmem_ld16(tmem_base + lane_addr + 256 + part * 32 + 16, v[1]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(out_empty);     // the accumulator is in registers: the next tile may overwrite it
        if (any_row) {
#pragma unroll
          for (int pass = 0; pass < 2; ++pass) {
            const int c0 = part * 32 + pass * 16;
            if (pass == 1) {                        // the first pass's copy has finished reading the rows
              if (lane == 0) bulk_wait_read();
              __syncwarp();
            }
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              const float4 bb = *reinterpret_cast<const float4*>(sB2 + c0 + k4 * 4);
              *reinterpret_cast<float4*>(stage + lane * 64 + ((uint32_t)(k4 ^ ((lane >> 1) & 3)) << 4)) =
                  make_float4(__uint_as_float(v[pass][k4 * 4]) + bb.x, __uint_as_float(v[pass][k4 * 4 + 1]) + bb.y,
                              __uint_as_float(v[pass][k4 * 4 + 2]) + bb.z, __uint_as_float(v[pass][k4 * 4 + 3]) + bb.w);
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
              if (p.resid) tma_reduce_add_2d(&mapO, stage, c0, (int)row0);
              else tma_store_2d(&mapO, stage, c0, (int)row0);
              bulk_commit();
            }
          }
        }
        __syncwarp();
        continue;      // (the staging rows are handed back before the next tile's first hidden write, below)
      } else
#pragma unroll 1
      for (int c0 = part * 32; c0 < part * 32 + 32; c0 += 16) {
        uint32_t v[16];
        tmem_ld16(tmem_base + lane_addr + 256 + c0, v);
        tmem_ld_wait();
        if (valid) {
          float o[16];
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            const float4 bb = *reinterpret_cast<const float4*>(sB2 + c0 + e4 * 4);
            o[e4 * 4] = __uint_as_float(v[e4 * 4]) + bb.x; o[e4 * 4 + 1] = __uint_as_float(v[e4 * 4 + 1]) + bb.y;
            o[e4 * 4 + 2] = __uint_as_float(v[e4 * 4 + 2]) + bb.z; o[e4 * 4 + 3] = __uint_as_float(v[e4 * 4 + 3]) + bb.w;
          }
          if (out_bf16) {
            if (p.resid) {
              uint32_t words[8];
              ld_global_v8(reinterpret_cast<const bf16*>(p.resid) + r * 128 + c0, words);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&words[e]);
                o[e * 2] += __low2float(h2);
                o[e * 2 + 1] += __high2float(h2);
              }
            }
            uint32_t ob[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const __nv_bfloat162 h2 = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
              ob[e] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            st_global_v8(reinterpret_cast<bf16*>(p.out) + r * 128 + c0, ob);
          } else {
            if (p.resid) {   // 32 bytes per load: half the L1 wavefronts of 16-byte loads for a row-per-thread access
              const float* rp = reinterpret_cast<const float*>(p.resid) + r * 128 + c0;
#pragma unroll
              for (int w8 = 0; w8 < 2; ++w8) {
                uint32_t f[8];
                ld_global_v8(rp + w8 * 8, f);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[w8 * 8 + e] += __uint_as_float(f[e]);
              }
            }
            uint32_t ob[8];
#pragma unroll
            for (int half8 = 0; half8 < 2; ++half8) {
#pragma unroll
              for (int e = 0; e < 8; ++e) ob[e] = __float_as_uint(o[half8 * 8 + e]);
              st_global_v8(reinterpret_cast<float*>(p.out) + r * 128 + c0 + half8 * 8, ob);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(out_empty);
    }
  }

  if (p.tma_out && warp < 16 && lane == 0) bulk_wait_all();     // this thread's stores have landed
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) drain_after_abort();
  if (warp == 24) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

lf_status make_map_f32_rows16(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t rows);

void configure_transition() {
  cudaFuncSetAttribute(transition_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TR_SMEM);
  cudaFuncSetAttribute(transition_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TR_SMEM);
  cudaGetLastError();
}

bool transition_supported(const lf_weights* w) { return w && w->h.size() >= 1 && w->h[0] != nullptr; }

lf_status transition_run(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int64_t rows, int variance,
                         float eps, const lf_weights* w, const void* resid, void* out) {
  if (cur.dry) return LF_OK;
  TransitionParams p{};
  p.act = act; p.act_bf16 = act_dtype == LF_DTYPE_BF16; p.rows = rows;
  p.eps = eps; p.variance = variance;
  p.wimg = (const uint8_t*)w->h[0]; p.b1 = (const float*)w->h[1]; p.b2 = w->f[TRN_B2];
  p.resid = resid; p.out = out; p.status = (Status*)ctx->tc_status;
  // float32 rows updated in place (or written without a residual): the pair tile travels by TMA
  CUtensorMap mo{};
  p.tma_out = (!p.act_bf16 && (resid == nullptr || resid == out) && rows < ((int64_t)1 << 31)) ? 1 : 0;
  if (p.tma_out) LF_TRY(make_map_f32_rows16(ctx, &mo, out, (uint64_t)rows));
  const int64_t tiles = (rows + TR_ROWS - 1) / TR_ROWS;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_TRANSITION);
  if (w->kind == LF_WEIGHTS_TRANSITION_AF3)
    transition_kernel<true><<<grid, TR_THREADS, TR_SMEM, ctx->stream>>>(mo, p);
  else
    transition_kernel<false><<<grid, TR_THREADS, TR_SMEM, ctx->stream>>>(mo, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

}  // namespace tc
