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
// Warp roles: 0..15 epilogue (TMEM lane quadrant = warp % 4, quarter of the columns =
// warp / 4), 16..23 LayerNorm producers, 24 MMA issuer and TMEM owner.  The many warps are
// there to hide arithmetic latency: each role's per-element work is a short dependent chain.
#include <cuda.h>

#include "tc05.cuh"
#include "tc_kernels.cuh"

namespace tc {

using namespace tc05;

constexpr int LG_THREADS = 25 * 32;
constexpr int LG_EPI_WARPS = 16, LG_PROD_WARPS = 8, LG_MMA_WARP = 24;
constexpr int LG_ROWS = 128;
constexpr int LG_K = 128;
constexpr int LG_A_BYTES = LG_ROWS * LG_K * 2;          // 32 KiB per stage, two 16 KiB k-atoms
constexpr int LG_MAX_CHUNKS = 3;

struct LnGemmParams {
  const void* act;          // [rows][128] f32 or bf16, memory order
  int act_bf16;
  int64_t rows;             // logical rows
  int transpose, batch, Q;  // logical row (b, i) reads memory row i*batch + b when transpose
  float eps;                // (the LayerNorm's gain and offset are folded into wimg and bias when the weights are prepared)
  int variance;             // 1 two-pass, 2 fast
  const uint8_t* wimg;      // swizzled fp16 image of W^T: [2 atoms][n_pad rows][128 B]
  int n_pad;
  const float* bias;        // [n_bias]
  int n_bias;
  int n_chunks;
  int first_chunk;          // attention projection: role of chunk 0 (0 = q|k, 1 = v|gate, 2 = pair bias); 2 with one chunk = bias only
  int bias_col0;            // attention projection: where the pair-bias chunk's bias values start in `bias`
  int chunk_n[LG_MAX_CHUNKS];
  int chunk_row0[LG_MAX_CHUNKS];
  // triangle projection epilogue
  const float* mask;        // [rows]
  op16* out_a;              // [c][n][ld]
  op16* out_b;
  int n, ld;                // pair row length and operand row stride
  int plane_rows;           // pair rows held (n for a whole pair, fewer for a row shard)
  // channel-sharded destinations (peer_ranks >= 1; one rank = rows inside whole planes of this device): channel h goes to rank h / ch_per_rank, plane h % ch_per_rank of
  // its [ch_per_rank][peer_plane_rows][ld] buffer, at rows peer_row0 + local row; stores go to the peers' memory
  int peer_ranks, ch_per_rank, peer_plane_rows, peer_row0;
  PeerPtrs peer_a, peer_b;
  const float* mask_pad;    // tiles along the pair rows (tile_per_row): the mask with rows zero-padded to mask_ld
  int mask_ld;
  int plane_tma;            // the planes are written by TMA from staging rows (maps in PlaneMaps), plane_box_h planes per copy
  int plane_box_h;
  // attention projection epilogue
  op16* out_q; op16* out_k; op16* out_v; op16* out_g;   // logical rows, stored in 8 x 8 pieces (see ldq)
  op16* out_bias;           // fp16 [heads][batch rows][ldb] (head, query, key)
  int ldb;
  int bias_ranks, bias_rows, bias_row0;   // bias_ranks > 0: the bias rows go to every rank's [heads][bias_rows][ldb] at bias_row0 + query row
  PeerPtrs peer_bias;
  int ldq;                  // attention activations (q, k, v, gate, o) are stored in 8-row x 8-channel pieces: element (b, q, c)
                            // of a [batch][Q][128] tensor sits at b*ldq*128 + (q/8)*1024 + (c/8)*64 + (q%8)*8 + c%8, ldq = Q rounded up to 16
  int heads, bias_swap;
  int bias_flags;           // bit (2*chunk + half): that 128-column group has a non-zero bias
  // output epilogues (attention output projection, triangle output): out = resid + f(acc)
  int a_is_op16;            // the A operand is an fp16 tensor of logical rows in 8 x 8 pieces (see ldq), copied as is (no LayerNorm)
  const void* resid;        // pair rows (memory order) to add, or null
  void* out;                // pair rows written in the same memory order
  int out_bf16;
  int tma_out;              // attention output only: the residual tile comes in and the result goes out through the tensor map
                            // (one map for both: the residual is the output tensor or absent), per warp 32 rows x 32 channels
  // triangle output: tiles follow pair rows (i, 128 k's); x is fetched by TMA as an MN-major operand
  int tile_per_row;         // tiles per pair row i (0 = rows are tiled linearly)
  float x_eps;              // epsilon of the centre LayerNorm in the units x is stored in
  Status* status;
};

// Tensor maps of the triangle projection's destinations: entry 2 * owner + (0 for a, 1 for b) covers that rank's
// [ch_per_rank][plane rows][ld] buffer (one owner = this device's whole planes).
constexpr int LG_MAX_PLANE_OWNERS = 8;
struct PlaneMaps { CUtensorMap m[2 * LG_MAX_PLANE_OWNERS]; };

enum { LG_EPI_TRIANGLE = 0, LG_EPI_ATTENTION = 1, LG_EPI_OUTPUT = 2, LG_EPI_TRI_OUT = 3 };

// sigmoid(v) = 0.5 + 0.5 * tanh(v / 2): one MUFU operation.  tanh.approx.f32 has a relative
// error of 2^-11, so the gate is good to about 2.4e-4 absolute - the precision of the fp16
// operand it multiplies.
__device__ __forceinline__ float sigmoid_fast(float v) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * v));
  return fmaf(0.5f, t, 0.5f);
}

// Rows of tile t: linear tiling, or (i, k-tile) tiles that never straddle a pair row.
__device__ __forceinline__ void tile_rows(const LnGemmParams& p, int64_t t, int64_t& base, int& count) {
  if (p.tile_per_row) {
    const int64_t i = t / p.tile_per_row;
    const int kt = (int)(t % p.tile_per_row);
    base = i * p.n + (int64_t)kt * LG_ROWS;
    const int left = p.n - kt * LG_ROWS;
    count = left < LG_ROWS ? left : LG_ROWS;
  } else {
    base = t * LG_ROWS;
    const int64_t left = p.rows - base;
    count = left < LG_ROWS ? (int)left : LG_ROWS;
  }
}


template <int EPI>
__global__ void __launch_bounds__(LG_THREADS, 1)
ln_gemm_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapO, const __grid_constant__ PlaneMaps planes,
               const __grid_constant__ LnGemmParams p) {
  // two operand stages everywhere; the triangle output also keeps two raw x tiles, and the epilogue of a tile stages its
  // output rows in that tile's x buffer, which its MMAs have finished with by then
  constexpr int NS = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int w_bytes = p.n_pad * 256;
  uint8_t* sW = smem;
  uint8_t* sA = smem + w_bytes;                       // 2 stages (w_bytes is a multiple of 1024: n_pad % 8 == 0... x256)
  uint8_t* sX = sA + NS * LG_A_BYTES;                 // triangle output only: the raw x tile
  uint8_t* sStage = sX + (EPI == LG_EPI_TRI_OUT ? NS * LG_A_BYTES : 0);   // attention output: per epilogue warp 32 rows x 128 B of the pair
  // (triangle projection: per group of four epilogue warps 32 channels x 128 B of an operand plane)
  float* sBias = reinterpret_cast<float*>(sStage + (EPI == LG_EPI_OUTPUT ? LG_EPI_WARPS * 4096
                                                    : EPI == LG_EPI_TRIANGLE ? 4 * 4096 : 0));
  float* sStat = sBias + 544 + 256;                   // [2 stages][2][128]: inverse std, inverse std * mean
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 512);
  uint64_t* a_full = bars;          // [2]
  uint64_t* a_empty = bars + 2;     // [2]
  uint64_t* acc_full = bars + 4;    // [2]
  uint64_t* acc_empty = bars + 6;   // [2]
  uint64_t* x_full = bars + 8;      // [2] TMA bytes of the x tile
  uint64_t* stat_full = bars + 10;  // [2] row statistics of the x tile written
  uint64_t* stage_bar = bars + 12;  // [16] hand-over of staging rows: triangle projection 0..3 slices written (count 4), 4..7 rows read;
                                    // triangle output 8..9: the epilogue warps (count 16) are done with the x buffer of that stage
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12 + LG_EPI_WARPS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t tiles = p.tile_per_row ? (int64_t)p.plane_rows * p.tile_per_row : (p.rows + LG_ROWS - 1) / LG_ROWS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&x_full[s], 1);
      mbar_init(&stat_full[s], LG_PROD_WARPS);
      mbar_init(&a_full[s], LG_PROD_WARPS);
      mbar_init(&a_empty[s], 1);
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], LG_EPI_WARPS);
    }
    for (int i = 0; i < LG_EPI_WARPS; ++i)
      mbar_init(&stage_bar[i], (EPI == LG_EPI_TRIANGLE && i < 4) ? 4 : (EPI == LG_EPI_TRI_OUT && (i == 8 || i == 9)) ? LG_EPI_WARPS : 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // resident weights: straight copy of the pre-swizzled image
  {
    const uint4* src = reinterpret_cast<const uint4*>(p.wimg);
    uint4* dst = reinterpret_cast<uint4*>(sW);
    for (int i = threadIdx.x; i < w_bytes / 16; i += LG_THREADS) dst[i] = src[i];
    for (int i = threadIdx.x; i < p.n_bias; i += LG_THREADS) sBias[i] = p.bias[i];
    fence_async_smem();
  }
  if (warp == LG_MMA_WARP) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= LG_EPI_WARPS && warp < LG_MMA_WARP) {
    // ---------------- LayerNorm producers ----------------
    // Eight lanes share a row, so one warp instruction covers four rows and a row statistic needs
    // three shuffle steps.  A lane's 16 channels are interleaved with its neighbours' so that every
    // load instruction reads 128 contiguous bytes per row: float input, element e is channel
    // 32 (e / 4) + 4 j + e % 4; 16-bit input, channel 64 (e / 8) + 8 j + e % 8.  Each warp owns 16 rows of the tile, handled as two
    // groups of two row-quads; the loads of a group are all issued before any is consumed.
    const int pw = warp - LG_EPI_WARPS;
    const int sub = lane >> 3, j = lane & 7;
    int it = 0;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x, ++it) {
      const int s = it % NS;
      const uint32_t ph = (uint32_t)(it / NS) & 1u;
      if (pw == 0 && lane == 0 && !p.a_is_op16 && !p.transpose && t + gridDim.x < tiles) {
        // rows of a tile are contiguous: ask for this CTA's next tile now, so that its loads find the rows in L2
        int64_t nb;
        int nc;
        tile_rows(p, t + gridDim.x, nb, nc);
        const uint32_t row_bytes = p.act_bf16 ? LG_K * 2u : LG_K * 4u;
        bulk_prefetch_l2(reinterpret_cast<const uint8_t*>(p.act) + nb * row_bytes, (uint32_t)nc * row_bytes);
      }
      if (!mbar_wait(&a_empty[s], ph ^ 1, abort_flag, p.status, 10)) break;
      uint8_t* tile = sA + s * LG_A_BYTES;
      int64_t row_base;
      int row_count;
      tile_rows(p, t, row_base, row_count);
      if (EPI == LG_EPI_TRI_OUT && pw == 0) {
        // the x buffer of this stage doubled as the staging rows of the tile two back: its copies must have read them
        if (!mbar_wait(&stage_bar[8 + s], ph ^ 1, abort_flag, p.status, 21)) break;
        if (lane == 0) {
          // x[h][i][k0 .. k0+127] for all 128 channels: two boxes of 64 pairs x 128 channels
          const int i = (int)(t / p.tile_per_row), k0 = (int)(t % p.tile_per_row) * LG_ROWS;
          mbar_expect_tx(&x_full[s], LG_A_BYTES);
          tma_load_3d(sX + s * LG_A_BYTES, &mapX, &x_full[s], k0, i, 0);
          tma_load_3d(sX + s * LG_A_BYTES + LG_A_BYTES / 2, &mapX, &x_full[s], k0 + 64, i, 0);
        }
      }
#pragma unroll 1
      for (int grp = 0; grp < 2; ++grp) {
        float v[2][16];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int row = pw * 16 + (grp * 2 + u) * 4 + sub;
          const int64_t r = row_base + row;
          if (row < row_count) {
            int64_t src = r;
            if (p.transpose && !p.a_is_op16) { const uint32_t ur = (uint32_t)r, uq = (uint32_t)p.Q; src = (int64_t)(ur % uq) * p.batch + ur / uq; }
            if (p.a_is_op16) {
              // rows in 8 x 8 pieces: channels 8 j .. + 7 are piece j of the row, channels 64 + 8 j .. piece 8 + j
              const uint32_t ur = (uint32_t)r, uq = (uint32_t)p.Q, rb = ur / uq, rq = ur % uq;
              const uint4* g = reinterpret_cast<const uint4*>(reinterpret_cast<const op16*>(p.act) + (int64_t)rb * p.ldq * 128 +
                                                              (int64_t)(rq >> 3) * 1024 + j * 64 + (rq & 7) * 8);
#pragma unroll
              for (int w4 = 0; w4 < 2; ++w4) {
                const uint4 raw = g[w4 * 64];
                const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&words[e]));
                  v[u][w4 * 8 + e * 2] = f2.x;
                  v[u][w4 * 8 + e * 2 + 1] = f2.y;
                }
              }
            } else if (p.act_bf16) {
              const uint4* g = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.act) + src * LG_K + 8 * j);
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
              const float4* g = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.act) + src * LG_K + 4 * j);
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
          const bool valid = row < row_count;
          uint32_t packed[8];
          if (p.a_is_op16) {
#pragma unroll
            for (int e = 0; e < 8; ++e) packed[e] = pack_half2(v[u][2 * e], v[u][2 * e + 1]);
          } else {
          float s4[4] = {0.f, 0.f, 0.f, 0.f};      // four chains instead of one of 16 dependent additions
#pragma unroll
          for (int e = 0; e < 16; ++e) s4[e & 3] += v[u][e];
          float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
          sum += __shfl_xor_sync(0xffffffffu, sum, 1);
          sum += __shfl_xor_sync(0xffffffffu, sum, 2);
          sum += __shfl_xor_sync(0xffffffffu, sum, 4);
          const float mean = sum * (1.0f / LG_K);
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
          const float var = p.variance == 2 ? sq * (1.0f / LG_K) - mean * mean : sq * (1.0f / LG_K);
          float inv = rsqrtf(var + p.eps);
          inv = inv * (1.5f - 0.5f * (var + p.eps) * inv * inv);
          // the gain and offset of the LayerNorm live in the weight image and the bias: the operand is (x - mean) / std
          const float shift = -mean * inv;
#pragma unroll
          for (int e = 0; e < 8; ++e)
            packed[e] = valid ? pack_half2(fmaf(v[u][2 * e], inv, shift), fmaf(v[u][2 * e + 1], inv, shift)) : 0u;
          }
          if (p.a_is_op16 || p.act_bf16) {
            // channels 64 w + 8 j .. + 7: k-atom w, 16-byte chunk j of the row
#pragma unroll
            for (int w2 = 0; w2 < 2; ++w2)
              *reinterpret_cast<uint4*>(tile + (uint32_t)w2 * (LG_ROWS * 128) + swizzle128_offset((uint32_t)row, (uint32_t)j)) =
                  make_uint4(packed[w2 * 4], packed[w2 * 4 + 1], packed[w2 * 4 + 2], packed[w2 * 4 + 3]);
          } else {
            // channels 32 w + 4 j .. + 3: k-atom w / 2, 16-byte chunk 4 (w % 2) + j / 2, its half j % 2
#pragma unroll
            for (int w4 = 0; w4 < 4; ++w4)
              *reinterpret_cast<uint2*>(tile + (uint32_t)(w4 >> 1) * (LG_ROWS * 128) +
                                        swizzle128_offset((uint32_t)row, (uint32_t)((w4 & 1) * 4 + (j >> 1))) + (j & 1) * 8) =
                  make_uint2(packed[w4 * 2], packed[w4 * 2 + 1]);
          }
        }
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[s]);
      if (EPI == LG_EPI_TRI_OUT) {
        // Statistics of the centre LayerNorm over the raw x tile (row h of a box = 128 bytes of 64 pairs, 128-byte
        // swizzled).  A warp owns 16 pairs; a lane reads 8 pairs (one 16-byte piece) of 8 channel rows, so the tile is
        // read once with 16-byte loads, and the 16 lanes that share a piece add up by a halving exchange: after four
        // steps lane group v holds value v of (8 sums, 8 sums of squares).
        if (!mbar_wait(&x_full[s], ph, abort_flag, p.status, 14)) break;
        const int cg = pw * 2 + (lane & 1);          // pairs 8 cg .. 8 cg + 7 of the tile
        const int hgl = lane >> 1;                   // channel rows 8 hgl .. 8 hgl + 7
        const uint8_t* xb = sX + s * LG_A_BYTES + (cg >> 3) * (LG_A_BYTES / 2);
        const uint32_t piece = (uint32_t)cg & 7u;
        float acc[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] = 0.f;
#pragma unroll
        for (int hh = 0; hh < 8; ++hh) {
          // the rows are taken in an order that differs from lane to lane, so that a warp's loads spread over the banks
          const uint32_t h = (uint32_t)hgl * 8u + (((uint32_t)hh + 2u * (uint32_t)hgl) & 7u);
          const uint4 raw = *reinterpret_cast<const uint4*>(xb + h * 128u + ((piece ^ (h & 7u)) << 4));
          const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&words[e]));
            acc[2 * e] += f2.x; acc[2 * e + 1] += f2.y;
            acc[8 + 2 * e] = fmaf(f2.x, f2.x, acc[8 + 2 * e]); acc[8 + 2 * e + 1] = fmaf(f2.y, f2.y, acc[8 + 2 * e + 1]);
          }
        }
#pragma unroll
        for (int step = 0; step < 4; ++step) {
          const int width = 8 >> step;               // values kept after this step
          const uint32_t bit = 16u >> step;          // lane bit that picks the half
          const bool upper = ((uint32_t)lane & bit) != 0u;
#pragma unroll
          for (int e = 0; e < width; ++e) {
            const float keep = upper ? acc[e + width] : acc[e];
            const float send = upper ? acc[e] : acc[e + width];
            acc[e] = keep + __shfl_xor_sync(0xffffffffu, send, (int)bit);
          }
        }
        const float sq = __shfl_down_sync(0xffffffffu, acc[0], 16);
        if (lane < 16) {
          const int pr = cg * 8 + hgl;
          const float mean = acc[0] * (1.0f / 128.0f);
          float var = sq * (1.0f / 128.0f) - mean * mean;
          if (p.variance != 2) var = fmaxf(var, 0.f);
          float inv = rsqrtf(var + p.x_eps);
          inv = inv * (1.5f - 0.5f * (var + p.x_eps) * inv * inv);
          sStat[(it & 1) * 256 + pr] = inv;            // two sets: the epilogue of the previous tile may still read its own
          sStat[(it & 1) * 256 + 128 + pr] = inv * mean;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&stat_full[s]);
      }
    }
  } else if (warp == LG_MMA_WARP) {
    // ---------------- MMA issuer ----------------
    // The whole warp runs the loop (uniform control flow and operand values, so the operands of the
    // MMA instructions stay in uniform registers); one elected lane issues.
    {
      int it = 0;
      uint32_t g = 0;
      for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x, ++it) {
        const int s = it % NS;
        const uint32_t ph = (uint32_t)(it / NS) & 1u;
        if (!mbar_wait(&a_full[s], ph, abort_flag, p.status, 11)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(sA + s * LG_A_BYTES);
        bool ok = true;
        for (int j = 0; j < p.n_chunks; ++j, ++g) {
          const int b = g & 1;
          if (!mbar_wait(&acc_empty[b], ((g >> 1) & 1) ^ 1, abort_flag, p.status, 12)) { ok = false; break; }
          tc_fence_after();
          if (EPI == LG_EPI_TRI_OUT) {
            if (!mbar_wait(&x_full[s], ph, abort_flag, p.status, 15) ||
                !mbar_wait(&stat_full[s], ph, abort_flag, p.status, 16)) { ok = false; break; }
            tc_fence_after();
          }
          if (elect_one()) {
          if (EPI == LG_EPI_TRIANGLE) {
            // D[channel][pair row]: weights are the A operand (128 projection rows, then 128 gate
            // rows of operand j), the normalised tile is the B operand (N = 128 pair rows)
            const uint32_t idesc = make_idesc_f16(128, LG_ROWS, 0, 0);
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
              const uint32_t w_addr = smem_u32(sW) + (j * 256 + grp * 128) * 128;
#pragma unroll
              for (int kk = 0; kk < LG_K / 16; ++kk) {
                const uint64_t wdesc = make_smem_desc(w_addr + (kk >> 2) * (p.n_pad * 128) + (kk & 3) * 32, 16, 1024);
                const uint64_t xdesc = make_smem_desc(a_addr + (kk >> 2) * (LG_ROWS * 128) + (kk & 3) * 32, 16, 1024);
                umma_f16(tmem_base + b * 256 + grp * 128, wdesc, xdesc, idesc, kk != 0 ? 1u : 0u);
              }
            }
          } else if (EPI == LG_EPI_TRI_OUT) {
            // columns 0..127: x tile (MN-major A, raw) times the gain-folded output projection;
            // columns 128..255: normalised pair tile (K-major A) times the output gate weights
            const uint32_t x_addr = smem_u32(sX + s * LG_A_BYTES);
            const uint32_t w_addr = smem_u32(sW);
            const uint32_t idesc_x = make_idesc_f16(LG_ROWS, 128, 1, 0);
            const uint32_t idesc_z = make_idesc_f16(LG_ROWS, 128, 0, 0);
#pragma unroll
            for (int kk = 0; kk < LG_K / 16; ++kk) {
              const uint64_t adesc = make_smem_desc(x_addr + kk * 2048, LG_A_BYTES / 2, 1024);
              const uint64_t bdesc = make_smem_desc(w_addr + (kk >> 2) * (p.n_pad * 128) + (kk & 3) * 32, 16, 1024);
              umma_f16(tmem_base + b * 256, adesc, bdesc, idesc_x, kk != 0 ? 1u : 0u);
            }
#pragma unroll
            for (int kk = 0; kk < LG_K / 16; ++kk) {
              const uint64_t adesc = make_smem_desc(a_addr + (kk >> 2) * (LG_ROWS * 128) + (kk & 3) * 32, 16, 1024);
              const uint64_t bdesc = make_smem_desc(w_addr + 128 * 128 + (kk >> 2) * (p.n_pad * 128) + (kk & 3) * 32, 16, 1024);
              umma_f16(tmem_base + b * 256 + 128, adesc, bdesc, idesc_z, kk != 0 ? 1u : 0u);
            }
          } else {
            const uint32_t idesc = make_idesc_f16(LG_ROWS, p.chunk_n[j], 0, 0);
            const uint32_t w_addr = smem_u32(sW) + p.chunk_row0[j] * 128;
#pragma unroll
            for (int kk = 0; kk < LG_K / 16; ++kk) {
              const uint64_t adesc = make_smem_desc(a_addr + (kk >> 2) * (LG_ROWS * 128) + (kk & 3) * 32, 16, 1024);
              const uint64_t bdesc = make_smem_desc(w_addr + (kk >> 2) * (p.n_pad * 128) + (kk & 3) * 32, 16, 1024);
              umma_f16(tmem_base + b * 256, adesc, bdesc, idesc, kk != 0 ? 1u : 0u);
            }
          }
          umma_commit(&acc_full[b]);
          if (j == p.n_chunks - 1) umma_commit(&a_empty[s]);
          }
          __syncwarp();
        }
        if (!ok) break;
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int q = warp & 3, part = warp >> 2;   // part: which quarter of the chunk's columns
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    uint32_t g = 0, staged = 0;
    bool ok = true;
    int it = 0;
    for (int64_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ++it) {
      int64_t row_base;
      int row_count;
      tile_rows(p, t, row_base, row_count);
      const int64_t r = row_base + row;
      const bool valid = row < row_count;
      // attention output through the tensor map: this warp's 32 rows x 32 channels of the pair
      const bool tma_tile = (EPI == LG_EPI_OUTPUT || EPI == LG_EPI_TRI_OUT) && p.tma_out && q * 32 < row_count;
      int tx = 0, ty = 0, tz = 0;
      if (tma_tile) {
        const int64_t r0 = row_base + q * 32;
        tx = part * 32;
        if (EPI == LG_EPI_TRI_OUT) {
          // (its staging rows hold 16 channels at a time: see below)
          // tiles lie inside one pair row i: the map is (channel, k, i), so a ragged last tile of a row is clipped at k = n
          tz = (int)(t / p.tile_per_row);
          ty = (int)(t % p.tile_per_row) * LG_ROWS + q * 32;
        } else if (p.transpose) { const uint32_t u0 = (uint32_t)r0, uq = (uint32_t)p.Q; ty = (int)(u0 / uq); tz = (int)(u0 % uq); }
        else ty = (int)r0;
        if (EPI == LG_EPI_OUTPUT) {
          if (lane == 0) bulk_wait_read();      // the previous tile's copy has finished reading the staging rows
          __syncwarp();
        }
      }
      for (int j = 0; j < p.n_chunks; ++j, ++g) {
        const int b = g & 1;
        if (!mbar_wait(&acc_full[b], (g >> 1) & 1, abort_flag, p.status, 13)) { ok = false; break; }
        tc_fence_after();
        const uint32_t acc = tmem_base + lane_addr + b * 256;
        if (EPI == LG_EPI_TRIANGLE) {
          // TMEM lane = hidden channel h, columns = the tile's pair rows (projection at 0..127,
          // gate at 128..255).  Each thread owns one channel and writes runs of consecutive k.
          const int h = row;
          const float bias_p = sBias[j * 256 + h], bias_g = sBias[j * 256 + 128 + h];
          op16* plane_base;
          if (p.peer_ranks >= 1) {
            const int owner = h / p.ch_per_rank;
            plane_base = reinterpret_cast<op16*>(j == 0 ? p.peer_a.p[owner] : p.peer_b.p[owner]) +
                         ((int64_t)(h - owner * p.ch_per_rank) * p.peer_plane_rows + p.peer_row0) * p.ld;
          } else {
            plane_base = (j == 0 ? p.out_a : p.out_b) + (int64_t)h * p.plane_rows * p.ld;
          }
          const bool vec = (p.n & 15) == 0;
          const uint32_t un = (uint32_t)p.n;
          // rows of this warp's quarter: r0 .. r0+31, as (i, k) with 32-bit arithmetic
          const uint32_t r0 = (uint32_t)(t * LG_ROWS) + part * 32;
          uint32_t ii = r0 / un, kk0 = r0 % un;
          if (p.plane_tma && !p.tile_per_row) {
            // The four warps that share this warp's 32 channels fill staging rows of 64 k (128 bytes, 128-byte swizzle),
            // 16 k each, twice per chunk; one of them sends the rows off as one copy per owner.  A request to the L2
            // then carries 128 bytes: with a thread's own 32-byte stores (one line in each of 32 planes per
            // instruction) the request rate, not the bytes, bounded this kernel.
            uint8_t* stage = sStage + q * 4096;
            uint64_t* grp_full = &stage_bar[q];        // count 4: the warps' slices are written
            uint64_t* grp_free = &stage_bar[4 + q];    // count 1: the copy has finished reading the rows
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {
              const int c0 = pass * 64 + part * 16;
              uint32_t pv[16], gv[16];
              tmem_ld16(acc + c0, pv);
              tmem_ld16(acc + 128 + c0, gv);
              tmem_ld_wait();
              const int64_t r64 = t * LG_ROWS + pass * 64;     // n is a multiple of 64: a run lies inside one pair row and
              if (r64 >= p.rows) break;                        // is in range or out of it as a whole, for all four warps alike
              const float4* m4 = reinterpret_cast<const float4*>(p.mask + r64 + part * 16);
              uint32_t pk[8];
#pragma unroll
              for (int g4 = 0; g4 < 4; ++g4) {
                const float4 m = __ldg(m4 + g4);
                const float mm[4] = {m.x, m.y, m.z, m.w};
                float val[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  val[e] = mm[e] * (__uint_as_float(pv[g4 * 4 + e]) + bias_p) * sigmoid_fast(__uint_as_float(gv[g4 * 4 + e]) + bias_g);
                pk[g4 * 2] = pack_half2(val[0], val[1]);
                pk[g4 * 2 + 1] = pack_half2(val[2], val[3]);
              }
              if (part == 0 && staged > 0) {
                if (lane == 0) { bulk_wait_read(); mbar_arrive(grp_free); }
                __syncwarp();
              }
              if (!mbar_wait(grp_free, (staged & 1u) ^ 1u, abort_flag, p.status, 19)) { ok = false; break; }
              const uint32_t sw = (uint32_t)lane & 7u;
              *reinterpret_cast<uint4*>(stage + lane * 128 + (((uint32_t)(part * 2) ^ sw) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              *reinterpret_cast<uint4*>(stage + lane * 128 + (((uint32_t)(part * 2 + 1) ^ sw) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
              fence_async_smem();
              __syncwarp();
              if (lane == 0) mbar_arrive(grp_full);
              if (part == 0) {
                if (!mbar_wait(grp_full, staged & 1u, abort_flag, p.status, 20)) { ok = false; break; }
                if (lane == 0) {
                  const uint32_t u64 = (uint32_t)r64;
                  const int ti = (int)(u64 / un), tk = (int)(u64 % un);
                  for (int h0 = 0; h0 < 32; h0 += p.plane_box_h) {
                    const int hh = q * 32 + h0, owner = hh / p.ch_per_rank;
                    tma_store_3d(&planes.m[2 * owner + j], stage + h0 * 128, tk, p.peer_row0 + ti, hh - owner * p.ch_per_rank);
                  }
                  bulk_commit();
                }
                __syncwarp();
              }
              ++staged;
            }
            if (!ok) break;
          } else if (p.plane_tma) {
            // The same for a length that is not a multiple of 64: the tiles lie along the pair rows, a row's last run is
            // clipped by the copy, the mask comes from its padded copy (or element by element).  Kept apart from the
            // aligned form above, which measured 18 % slower per launch with these cases folded into it.
            uint8_t* stage = sStage + q * 4096;
            uint64_t* grp_full = &stage_bar[q];        // count 4: the warps' slices are written
            uint64_t* grp_free = &stage_bar[4 + q];    // count 1: the copy has finished reading the rows
#pragma unroll 1
            for (int pass = 0; pass < 2; ++pass) {
              const int c0 = pass * 64 + part * 16;
              // A run of 64 k lies inside one pair row: n is a multiple of 64, or the tiles are laid along the pair rows
              // (tile_per_row) and the run past a row's end is clipped by the copy.  It is in range or out of it as a
              // whole, for all four warps alike.
              const int64_t r64 = row_base + pass * 64;
              if (pass * 64 >= row_count) break;
              // (tiles along the pair rows read a copy of the mask whose rows are padded with zeros to whole tiles)
              const float4* m4 = reinterpret_cast<const float4*>(
                  p.tile_per_row ? p.mask_pad + (t / p.tile_per_row) * p.mask_ld + (t % p.tile_per_row) * LG_ROWS + pass * 64 + part * 16
                                 : p.mask + r64 + part * 16);
              // the pass's 16 mask values first, all loads in flight together
              float mv[16];
              if (p.tile_per_row && !p.mask_pad) {   // ragged rows of the flat mask: no alignment, nothing read past the row's end
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                  const int in_tile = pass * 64 + part * 16 + e;
                  mv[e] = in_tile < row_count ? __ldg(p.mask + row_base + in_tile) : 0.f;
                }
              } else {
#pragma unroll
                for (int g4 = 0; g4 < 4; ++g4) {
                  const float4 m = __ldg(m4 + g4);
                  mv[g4 * 4] = m.x; mv[g4 * 4 + 1] = m.y; mv[g4 * 4 + 2] = m.z; mv[g4 * 4 + 3] = m.w;
                }
              }
              // (the mask loads above are in flight while the accumulator columns come out of tensor memory)
              uint32_t pv[16], gv[16];
              tmem_ld16(acc + c0, pv);
              tmem_ld16(acc + 128 + c0, gv);
              tmem_ld_wait();
              uint32_t pk[8];
#pragma unroll
              for (int g4 = 0; g4 < 4; ++g4) {
                const float mm[4] = {mv[g4 * 4], mv[g4 * 4 + 1], mv[g4 * 4 + 2], mv[g4 * 4 + 3]};
                float val[4];
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  val[e] = mm[e] * (__uint_as_float(pv[g4 * 4 + e]) + bias_p) * sigmoid_fast(__uint_as_float(gv[g4 * 4 + e]) + bias_g);
                pk[g4 * 2] = pack_half2(val[0], val[1]);
                pk[g4 * 2 + 1] = pack_half2(val[2], val[3]);
              }
              if (part == 0 && staged > 0) {
                if (lane == 0) { bulk_wait_read(); mbar_arrive(grp_free); }
                __syncwarp();
              }
              if (!mbar_wait(grp_free, (staged & 1u) ^ 1u, abort_flag, p.status, 19)) { ok = false; break; }
              const uint32_t sw = (uint32_t)lane & 7u;
              *reinterpret_cast<uint4*>(stage + lane * 128 + (((uint32_t)(part * 2) ^ sw) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
              *reinterpret_cast<uint4*>(stage + lane * 128 + (((uint32_t)(part * 2 + 1) ^ sw) << 4)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
              fence_async_smem();
              __syncwarp();
              if (lane == 0) mbar_arrive(grp_full);
              if (part == 0) {
                if (!mbar_wait(grp_full, staged & 1u, abort_flag, p.status, 20)) { ok = false; break; }
                if (lane == 0) {
                  const uint32_t u64 = (uint32_t)r64;
                  int ti, tk;
                  if (p.tile_per_row) { ti = (int)(t / p.tile_per_row); tk = (int)(t % p.tile_per_row) * LG_ROWS + pass * 64; }
                  else { ti = (int)(u64 / un); tk = (int)(u64 % un); }
                  for (int h0 = 0; h0 < 32; h0 += p.plane_box_h) {
                    const int hh = q * 32 + h0, owner = hh / p.ch_per_rank;
                    tma_store_3d(&planes.m[2 * owner + j], stage + h0 * 128, tk, p.peer_row0 + ti, hh - owner * p.ch_per_rank);
                  }
                  bulk_commit();
                }
                __syncwarp();
              }
              ++staged;
            }
            if (!ok) break;
          } else
#pragma unroll 1
          for (int c0 = part * 32; c0 < part * 32 + 32; c0 += 16) {
            uint32_t pv[16], gv[16];
            tmem_ld16(acc + c0, pv);
            tmem_ld16(acc + 128 + c0, gv);
            tmem_ld_wait();
            const int64_t r16 = t * LG_ROWS + c0;
            if (r16 < p.rows) {
              if (vec) {
                const float4* m4 = reinterpret_cast<const float4*>(p.mask + r16);
                uint32_t pk[8];
#pragma unroll
                for (int g4 = 0; g4 < 4; ++g4) {
                  const float4 m = __ldg(m4 + g4);
                  const float mm[4] = {m.x, m.y, m.z, m.w};
                  float val[4];
#pragma unroll
                  for (int e = 0; e < 4; ++e)
                    val[e] = mm[e] * (__uint_as_float(pv[g4 * 4 + e]) + bias_p) * sigmoid_fast(__uint_as_float(gv[g4 * 4 + e]) + bias_g);
                  pk[g4 * 2] = pack_half2(val[0], val[1]);
                  pk[g4 * 2 + 1] = pack_half2(val[2], val[3]);
                }
                st_global_v8(plane_base + (int64_t)ii * p.ld + kk0, pk);
              } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                  const int64_t r = r16 + e;
                  if (r < p.rows) {
                    const uint32_t ur = (uint32_t)r;
                    const float v1 = __ldg(p.mask + r) * (__uint_as_float(pv[e]) + bias_p) * sigmoid_fast(__uint_as_float(gv[e]) + bias_g);
                    plane_base[(int64_t)(ur / un) * p.ld + ur % un] = __float2half_rn(v1);
                  }
                }
              }
            }
            kk0 += 16;
            if (kk0 >= un) { kk0 -= un; ++ii; }
          }
        } else if ((EPI == LG_EPI_OUTPUT || EPI == LG_EPI_TRI_OUT) && p.tma_out) {
          // thread = pair row; the warp's 32 rows x 32 channels are written to its staging rows (128 B each,
          // 16-byte pieces swizzled by row so that the row-per-thread accesses spread over the banks) and leave
          // as one TMA copy (a reduce-add when the pair is updated in place): no global load or store
          // instruction touches the pair here
          if (tma_tile) {
            // attention output: 32 channels per row (128 B, 128-byte swizzle), one copy per tile; triangle output: 16
            // channels per row (64 B, 64-byte swizzle) in this tile's x buffer, one copy per half
            uint8_t* stage = EPI == LG_EPI_TRI_OUT ? sX + (it % NS) * LG_A_BYTES + warp * 2048 + lane * 64 : sStage + warp * 4096 + lane * 128;
            float rs = 0.f, rm = 0.f;
            if (EPI == LG_EPI_TRI_OUT) {
              if (!mbar_wait(&stat_full[it % NS], (uint32_t)(it / NS) & 1u, abort_flag, p.status, 17)) { ok = false; break; }
              rs = sStat[(it & 1) * 256 + row];
              rm = sStat[(it & 1) * 256 + 128 + row];
            }
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
              const int c0 = part * 32 + half * 16;
              uint32_t v1[16], v2[16];
              tmem_ld16(acc + c0, v1);
              if (EPI == LG_EPI_TRI_OUT) tmem_ld16(acc + 128 + c0, v2);
              tmem_ld_wait();
              if (EPI == LG_EPI_TRI_OUT && half == 1) {     // the first half's copy has finished reading the rows
                if (lane == 0) bulk_wait_read();
                __syncwarp();
              }
#pragma unroll
              for (int k4 = 0; k4 < 4; ++k4) {
                float4* cell = reinterpret_cast<float4*>(
                    stage + (EPI == LG_EPI_TRI_OUT ? ((uint32_t)(k4 ^ ((lane >> 1) & 3)) << 4) : ((uint32_t)((half * 4 + k4) ^ (lane & 7)) << 4)));
                // per-channel vectors are the same for every lane: 16-byte broadcasts, not scalar reads
                const float4 b0v = *reinterpret_cast<const float4*>(sBias + c0 + k4 * 4);
                const float b0[4] = {b0v.x, b0v.y, b0v.z, b0v.w};
                float e4[4];
                if (EPI == LG_EPI_TRI_OUT) {
                  const float4 b1v = *reinterpret_cast<const float4*>(sBias + 128 + c0 + k4 * 4);
                  const float4 b2v = *reinterpret_cast<const float4*>(sBias + 256 + c0 + k4 * 4);
                  const float b1[4] = {b1v.x, b1v.y, b1v.z, b1v.w}, b2[4] = {b2v.x, b2v.y, b2v.z, b2v.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    // (x - mean) * inv folded: inv * acc - inv*mean * s1[c] + t[c], gated
                    const float lin = fmaf(rs, __uint_as_float(v1[k4 * 4 + e]), fmaf(-rm, b0[e], b1[e]));
                    e4[e] = lin * sigmoid_fast(__uint_as_float(v2[k4 * 4 + e]) + b2[e]);
                  }
                } else {
#pragma unroll
                  for (int e = 0; e < 4; ++e) e4[e] = __uint_as_float(v1[k4 * 4 + e]) + b0[e];
                }
                *cell = make_float4(e4[0], e4[1], e4[2], e4[3]);
              }
              if (EPI == LG_EPI_TRI_OUT) {
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                  const uint8_t* rows = sX + (it % NS) * LG_A_BYTES + warp * 2048;
                  if (p.resid) tma_reduce_add_3d(&mapO, rows, c0, ty, tz);
                  else tma_store_3d(&mapO, rows, c0, ty, tz);
                  bulk_commit();
                }
              }
            }
            if (EPI == LG_EPI_OUTPUT) {
              fence_async_smem();
              __syncwarp();
              if (lane == 0) {
                // in place: the update is added to the rows where they live, so the residual is never read here
                if (p.resid) tma_reduce_add_3d(&mapO, sStage + warp * 4096, tx, ty, tz);
                else tma_store_3d(&mapO, sStage + warp * 4096, tx, ty, tz);
                bulk_commit();
              }
            }
          }
        } else if (EPI == LG_EPI_OUTPUT || EPI == LG_EPI_TRI_OUT) {
          // thread = pair row; this warp's quarter = 32 output channels, two runs of 16
          int64_t dst = r;
          if (EPI == LG_EPI_OUTPUT && p.transpose && valid) {
            const uint32_t ur = (uint32_t)r, uq = (uint32_t)p.Q;
            dst = (int64_t)(ur % uq) * p.batch + ur / uq;
          }
          float rs = 0.f, rm = 0.f;
          if (EPI == LG_EPI_TRI_OUT) {
            if (!mbar_wait(&stat_full[it % NS], (uint32_t)(it / NS) & 1u, abort_flag, p.status, 17)) { ok = false; break; }
            rs = sStat[(it & 1) * 256 + row];
            rm = sStat[(it & 1) * 256 + 128 + row];
          }
#pragma unroll 1
          for (int c0 = part * 32; c0 < part * 32 + 32; c0 += 16) {
            uint32_t v1[16], v2[16];
            tmem_ld16(acc + c0, v1);
            if (EPI == LG_EPI_TRI_OUT) tmem_ld16(acc + 128 + c0, v2);
            tmem_ld_wait();
            if (valid) {
              float o[16];
              float b0[16];
#pragma unroll
              for (int e4 = 0; e4 < 4; ++e4) *reinterpret_cast<float4*>(b0 + e4 * 4) = *reinterpret_cast<const float4*>(sBias + c0 + e4 * 4);
              if (EPI == LG_EPI_TRI_OUT) {
                float b1[16], b2[16];
#pragma unroll
                for (int e4 = 0; e4 < 4; ++e4) {
                  *reinterpret_cast<float4*>(b1 + e4 * 4) = *reinterpret_cast<const float4*>(sBias + 128 + c0 + e4 * 4);
                  *reinterpret_cast<float4*>(b2 + e4 * 4) = *reinterpret_cast<const float4*>(sBias + 256 + c0 + e4 * 4);
                }
                // (x - mean) * inv folded: inv * acc - inv*mean * s1[c] + t[c], gated
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                  const float lin = fmaf(rs, __uint_as_float(v1[e]), fmaf(-rm, b0[e], b1[e]));
                  o[e] = lin * sigmoid_fast(__uint_as_float(v2[e]) + b2[e]);
                }
              } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) o[e] = __uint_as_float(v1[e]) + b0[e];
              }
              if (p.out_bf16) {
                bf16* op = reinterpret_cast<bf16*>(p.out) + dst * 128 + c0;
                if (p.resid) {
                  uint32_t words[8];
                  ld_global_v8(reinterpret_cast<const bf16*>(p.resid) + dst * 128 + c0, words);
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const __nv_bfloat162 h2 = *reinterpret_cast<const __nv_bfloat162*>(&words[e]);
                    o[e * 2] += __low2float(h2);
                    o[e * 2 + 1] += __high2float(h2);
                  }
                }
                uint32_t pk[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const __nv_bfloat162 h2 = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
                  pk[e] = *reinterpret_cast<const uint32_t*>(&h2);
                }
                st_global_v8(op, pk);
              } else {
                float* op = reinterpret_cast<float*>(p.out) + dst * 128 + c0;
                if (p.resid) {   // 32 bytes per load: half the L1 wavefronts of 16-byte loads for a row-per-thread access
                  const float* rp = reinterpret_cast<const float*>(p.resid) + dst * 128 + c0;
#pragma unroll
                  for (int w8 = 0; w8 < 2; ++w8) {
                    uint32_t f[8];
                    ld_global_v8(rp + w8 * 8, f);
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[w8 * 8 + e] += __uint_as_float(f[e]);
                  }
                }
                uint32_t pk[8];
#pragma unroll
                for (int half8 = 0; half8 < 2; ++half8) {
#pragma unroll
                  for (int e = 0; e < 8; ++e) pk[e] = __float_as_uint(o[half8 * 8 + e]);
                  st_global_v8(op + half8 * 8, pk);
                }
              }
            }
          }
        } else {
          const int jr = j + p.first_chunk;
          if (jr < 2) {
            // chunk 0 = (q | k), chunk 1 = (v | gate): parts 0,1 take the first tensor, 2,3 the second
            const int second = part >> 1, col0 = (part & 1) * 64;
            op16* out = jr == 0 ? (second ? p.out_k : p.out_q) : (second ? p.out_g : p.out_v);
            const float4* bias4 = reinterpret_cast<const float4*>(sBias + jr * 256 + second * 128 + col0);
            const bool gate = (jr == 1 && second == 1);
            const bool has_bias = (p.bias_flags >> (jr * 2 + second)) & 1;
            // destination of this row in the 8 x 8-piece layout: pieces along channels are 64 elements apart
            const uint32_t ur = (uint32_t)(valid ? r : 0), uq = (uint32_t)p.Q, rb = ur / uq, rq = ur % uq;
            op16* out_row = out + (int64_t)rb * p.ldq * 128 + (int64_t)(rq >> 3) * 1024 + (rq & 7) * 8;
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 16) {
              uint32_t v[16];
              tmem_ld16(acc + second * 128 + col0 + c0, v);
              tmem_ld_wait();
              if (valid) {
                float f[16];
#pragma unroll
                for (int u = 0; u < 16; ++u) f[u] = __uint_as_float(v[u]);
                if (has_bias) {
#pragma unroll
                  for (int u4 = 0; u4 < 4; ++u4) {
                    const float4 bb = bias4[(c0 >> 2) + u4];
                    f[u4 * 4] += bb.x; f[u4 * 4 + 1] += bb.y; f[u4 * 4 + 2] += bb.z; f[u4 * 4 + 3] += bb.w;
                  }
                }
                if (gate) {
#pragma unroll
                  for (int u = 0; u < 16; ++u) f[u] = sigmoid_fast(f[u]);
                }
                uint32_t pk[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) pk[u] = pack_half2(f[2 * u], f[2 * u + 1]);
                // two 16-byte pieces: 32 consecutive rows of a warp fill four whole 128-byte lines per store
                op16* dst = out_row + ((col0 + c0) >> 3) * 64;
                *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(dst + 64) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
              }
            }
          } else if (part == 0) {
            // chunk 2: pair bias, one column per head; logical row r = (q index, k index)
            uint32_t v[16];
            tmem_ld16(acc, v);
            tmem_ld_wait();
            if (valid) {
              const uint32_t ur = (uint32_t)r, uq = (uint32_t)p.Q;
              const int64_t qi = ur / uq, ki = ur % uq;
              const int64_t bq = p.bias_swap ? ki : qi, bk = p.bias_swap ? qi : ki;   // bias[h][bq][bk]
              // row-major per head: [head][batch rows][ldb]
              const int64_t dst = bq * p.ldb + bk;
              const int64_t qq = (int64_t)p.batch * p.ldb;
              if (p.bias_ranks > 0) {
                // every rank keeps the bias of all query rows: this shard's rows go to each of them
                const int64_t pq = (int64_t)p.bias_rows * p.ldb, pdst = (p.bias_row0 + bq) * p.ldb + bk;
                for (int g2 = 0; g2 < p.bias_ranks; ++g2) {
                  op16* ob = reinterpret_cast<op16*>(p.peer_bias.p[g2]);
#pragma unroll
                  for (int h = 0; h < 16; ++h)
                    if (h < p.heads) ob[h * pq + pdst] = __float2half_rn(__uint_as_float(v[h]) + sBias[p.bias_col0 + h]);
                }
              } else {
#pragma unroll
                for (int h = 0; h < 16; ++h)
                  if (h < p.heads) p.out_bias[h * qq + dst] = __float2half_rn(__uint_as_float(v[h]) + sBias[p.bias_col0 + h]);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[b]);
      }
      if (EPI == LG_EPI_TRI_OUT && ok) {
        // this warp is done with the stage's x buffer once its copies have read their rows
        if (lane == 0) { bulk_wait_read(); mbar_arrive(&stage_bar[8 + it % NS]); }
        __syncwarp();
      }
    }
  }

  if ((((EPI == LG_EPI_OUTPUT || EPI == LG_EPI_TRI_OUT) && p.tma_out) || (EPI == LG_EPI_TRIANGLE && p.plane_tma)) && warp < LG_EPI_WARPS &&
      lane == 0)
    bulk_wait_all();   // this thread's stores have landed
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) drain_after_abort();
  if (warp == LG_MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// W (in,out) float32 [K][n_out] -> fp16 image of W^T in the swizzled K-major layout
// ([K/64 atoms][n_pad rows][128 B]); rows >= n_out are zero.
__global__ void pack_weight_image_kernel(const float* __restrict__ w, int K, int n_out, int n_pad, int col0, int ld,
                                         op16* __restrict__ img, int row0, float scale, const float* __restrict__ kscale) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_out * K) return;
  int n = idx / K, k = idx % K;
  int row = row0 + n;
  size_t off = (size_t)(k >> 6) * ((size_t)n_pad * 128) + (size_t)row * 128 + ((((k & 63) >> 3) ^ (row & 7)) << 4) + (k & 7) * 2;
  img[off / 2] = __float2half_rn(w[(size_t)k * ld + col0 + n] * scale * (kscale ? kscale[k] : 1.0f));
}

// kscale (optional, [K]): a LayerNorm gain folded into the rows of W, so that the kernel's producers only standardise
void pack_weight_image(lf_context* ctx, const float* w, int K, int n_out, int n_pad, int col0, int ld, op16* img, int row0,
                       float scale, const float* kscale) {
  int total = n_out * K;
  pack_weight_image_kernel<<<(total + 255) / 256, 256, 0, ctx->stream>>>(w, K, n_out, n_pad, col0, ld, img, row0, scale, kscale);
}

// The LayerNorm offset folded into a bias: b_out[c] = scale * (b_in[c] + sum_k offset[k] W[k][col0 + c]) (b_in optional)
__global__ void fold_bias_kernel(const float* __restrict__ w, int K, int n_out, int col0, int ld, const float* __restrict__ offset,
                                 const float* __restrict__ b_in, float scale, float* __restrict__ b_out) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_out) return;
  double acc = b_in ? (double)b_in[c] : 0.0;
  for (int k = 0; k < K; ++k) acc += (double)offset[k] * (double)w[(size_t)k * ld + col0 + c];
  b_out[c] = (float)(acc * scale);
}

void fold_bias(lf_context* ctx, const float* w, int K, int n_out, int col0, int ld, const float* offset, const float* b_in, float scale,
               float* b_out) {
  fold_bias_kernel<<<(n_out + 127) / 128, 128, 0, ctx->stream>>>(w, K, n_out, col0, ld, offset, b_in, scale, b_out);
}

lf_status make_map_f32_rows(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                            uint64_t stride2_bytes, uint32_t b1, uint32_t b2);

lf_status make_map_f32_rows_half(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                                 uint64_t stride2_bytes, uint32_t b1, uint32_t b2);

static int ln_gemm_smem(int n_pad, bool tri_out = false, bool staged_out = false, bool plane_stage = false) {
  return n_pad * 256 + (tri_out ? 4 : 2) * LG_A_BYTES + (staged_out ? LG_EPI_WARPS * 4096 : 0) + (plane_stage ? 4 * 4096 : 0) +
         (544 + 256 + 512) * 4 + 512 + 1024;
}

void configure_ln_gemm() {
  cudaFuncSetAttribute(ln_gemm_kernel<LG_EPI_TRIANGLE>, cudaFuncAttributeMaxDynamicSharedMemorySize, ln_gemm_smem(512, false, false, true));
  cudaFuncSetAttribute(ln_gemm_kernel<LG_EPI_ATTENTION>, cudaFuncAttributeMaxDynamicSharedMemorySize, ln_gemm_smem(528));
  cudaFuncSetAttribute(ln_gemm_kernel<LG_EPI_OUTPUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, ln_gemm_smem(128, false, true));
  cudaFuncSetAttribute(ln_gemm_kernel<LG_EPI_TRI_OUT>, cudaFuncAttributeMaxDynamicSharedMemorySize, ln_gemm_smem(256, true, false));
  cudaGetLastError();
}

lf_status make_map_plane_runs(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t n, uint64_t plane_rows, uint64_t planes,
                              uint64_t ld, uint32_t box_h);

// Destinations of the triangle projection as tensor maps, when the shape allows the staged copies (at most
// LG_MAX_PLANE_OWNERS owners); otherwise the kernel stores with its own threads.
static lf_status plane_maps(lf_context* ctx, LnGemmParams& p, PlaneMaps& pm, const PeerPtrs& a, const PeerPtrs& b, int owners,
                            int plane_rows) {
  p.plane_tma = 0;
  if (owners > LG_MAX_PLANE_OWNERS || 128 % owners != 0 || p.ld % 8 != 0) return LF_OK;
  // a length that is not a multiple of 64: tiles along the pair rows, so that a run never straddles two of them
  if ((p.n & 63) != 0) p.tile_per_row = (p.n + LG_ROWS - 1) / LG_ROWS;
  p.ch_per_rank = 128 / owners;
  p.plane_box_h = p.ch_per_rank < 32 ? p.ch_per_rank : 32;
  for (int o = 0; o < owners; ++o) {
    LF_TRY(make_map_plane_runs(ctx, &pm.m[2 * o], a.p[o], (uint64_t)p.n, (uint64_t)plane_rows, (uint64_t)p.ch_per_rank, (uint64_t)p.ld,
                               (uint32_t)p.plane_box_h));
    LF_TRY(make_map_plane_runs(ctx, &pm.m[2 * o + 1], b.p[o], (uint64_t)p.n, (uint64_t)plane_rows, (uint64_t)p.ch_per_rank, (uint64_t)p.ld,
                               (uint32_t)p.plane_box_h));
  }
  p.plane_tma = 1;
  return LF_OK;
}

// mask [rows][n] -> [rows][mld], zeros past n
__global__ void pad_mask_kernel(const float* __restrict__ mask, int rows, int n, int mld, float* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * mld) return;
  const int i = (int)(idx / mld), k = (int)(idx % mld);
  out[idx] = k < n ? mask[(int64_t)i * n + k] : 0.f;
}

// A length that is not a multiple of 64 runs the projection with tiles along the pair rows; they read the mask from a
// copy padded to whole tiles when the call's arena has room planned for one (taken in the sizing pass too), and
// element by element otherwise.
static const float* padded_mask(lf_context* ctx, ArenaCursor& cur, const float* mask, int rows, int n, int& mld) {
  mld = (n & 63) && cur.sized_by_dry_pass ? (n + LG_ROWS - 1) / LG_ROWS * LG_ROWS : 0;
  if (!mld) return nullptr;
  float* out = cur.take<float>((int64_t)rows * mld);
  if (!cur.dry) {
    pad_mask_kernel<<<(unsigned)(((int64_t)rows * mld + 255) / 256), 256, 0, ctx->stream>>>(mask, rows, n, mld, out);
    ctx->launches++;
  }
  return out;
}

lf_status triangle_project(lf_context* ctx, ArenaCursor& cur, const void* z, int act_dtype, const float* mask, int rows,
                           int n, int ld, int variance, float eps, const lf_weights* w, op16* a, op16* b) {
  int mld = 0;
  const float* mask_pad = padded_mask(ctx, cur, mask, rows, n, mld);
  if (cur.dry) return LF_OK;
  LnGemmParams p{};
  p.mask_pad = mask_pad; p.mask_ld = mld;
  p.act = z; p.act_bf16 = act_dtype == LF_DTYPE_BF16; p.rows = (int64_t)rows * n; p.transpose = 0; p.batch = 1; p.Q = 1;
  p.plane_rows = rows;
  p.eps = eps; p.variance = variance;
  p.wimg = (const uint8_t*)w->h[0]; p.n_pad = 512; p.bias = (const float*)w->h[1]; p.n_bias = 512;
  p.n_chunks = 2; p.chunk_n[0] = 256; p.chunk_n[1] = 256; p.chunk_row0[0] = 0; p.chunk_row0[1] = 256;
  p.mask = mask; p.out_a = a; p.out_b = b; p.n = n; p.ld = ld; p.status = (Status*)ctx->tc_status;
  PlaneMaps pm{};
  PeerPtrs pa{}, pb{};
  pa.p[0] = a; pb.p[0] = b;
  LF_TRY(plane_maps(ctx, p, pm, pa, pb, 1, rows));
  const int64_t tiles = (p.rows + LG_ROWS - 1) / LG_ROWS;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_LN_GEMM);
  ln_gemm_kernel<LG_EPI_TRIANGLE><<<grid, LG_THREADS, ln_gemm_smem(512, false, false, true), ctx->stream>>>(CUtensorMap{}, CUtensorMap{}, pm, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

lf_status triangle_project_scatter(lf_context* ctx, ArenaCursor& cur, const void* z, int act_dtype, const float* mask, int rows,
                                   int n, int ld, int variance, float eps, const lf_weights* w, const PeerPtrs& a_peers,
                                   const PeerPtrs& b_peers, int ranks, int row0) {
  int mld = 0;
  const float* mask_pad = padded_mask(ctx, cur, mask, rows, n, mld);
  if (cur.dry) return LF_OK;
  LnGemmParams p{};
  p.mask_pad = mask_pad; p.mask_ld = mld;
  p.act = z; p.act_bf16 = act_dtype == LF_DTYPE_BF16; p.rows = (int64_t)rows * n; p.transpose = 0; p.batch = 1; p.Q = 1;
  p.plane_rows = rows;
  p.eps = eps; p.variance = variance;
  p.wimg = (const uint8_t*)w->h[0]; p.n_pad = 512; p.bias = (const float*)w->h[1]; p.n_bias = 512;
  p.n_chunks = 2; p.chunk_n[0] = 256; p.chunk_n[1] = 256; p.chunk_row0[0] = 0; p.chunk_row0[1] = 256;
  p.mask = mask; p.n = n; p.ld = ld; p.status = (Status*)ctx->tc_status;
  p.peer_ranks = ranks; p.ch_per_rank = 128 / ranks; p.peer_plane_rows = n; p.peer_row0 = row0;
  p.peer_a = a_peers; p.peer_b = b_peers;
  p.out_a = (op16*)a_peers.p[0]; p.out_b = (op16*)b_peers.p[0];      // ranks == 1: plain form
  PlaneMaps pm{};
  LF_TRY(plane_maps(ctx, p, pm, a_peers, b_peers, ranks, n));
  const int64_t tiles = (p.rows + LG_ROWS - 1) / LG_ROWS;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_LN_GEMM);
  ln_gemm_kernel<LG_EPI_TRIANGLE><<<grid, LG_THREADS, ln_gemm_smem(512, false, false, true), ctx->stream>>>(CUtensorMap{}, CUtensorMap{}, pm, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

static lf_status attention_project_impl(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int batch, int Q,
                                        int transpose, int variance, float eps, int heads, int bias_swap, const lf_weights* w,
                                        op16* q, op16* k, op16* v, op16* g, op16* bias, int ldb, const PeerPtrs* bias_peers,
                                        int ranks, int bias_rows, int row0);

lf_status attention_project(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int batch, int Q,
                            int transpose, int variance, float eps, int heads, int head_dim, int bias_swap,
                            const lf_weights* w, op16* q, op16* k, op16* v, op16* g, op16* bias, int ldb) {
  (void)head_dim;
  return attention_project_impl(ctx, cur, act, act_dtype, batch, Q, transpose, variance, eps, heads, bias_swap, w, q, k, v, g,
                                bias, ldb, nullptr, 0, 0, 0);
}

lf_status attention_project_scatter(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int batch, int Q,
                                    int variance, float eps, int heads, const lf_weights* w, op16* q, op16* k, op16* v,
                                    op16* g, const PeerPtrs& bias_peers, int ranks, int bias_rows, int row0, int ldb,
                                    int transpose) {
  return attention_project_impl(ctx, cur, act, act_dtype, batch, Q, transpose, variance, eps, heads, 0, w, q, k, v, g,
                                (op16*)bias_peers.p[0], ldb, &bias_peers, ranks, bias_rows, row0);
}

static lf_status attention_project_impl(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int batch, int Q,
                                        int transpose, int variance, float eps, int heads, int bias_swap, const lf_weights* w,
                                        op16* q, op16* k, op16* v, op16* g, op16* bias, int ldb, const PeerPtrs* bias_peers,
                                        int ranks, int bias_rows, int row0) {
  if (cur.dry) return LF_OK;
  LnGemmParams p{};
  if (bias_peers) { p.bias_ranks = ranks; p.bias_rows = bias_rows; p.bias_row0 = row0; p.peer_bias = *bias_peers; }
  p.act = act; p.act_bf16 = act_dtype == LF_DTYPE_BF16; p.rows = (int64_t)batch * Q; p.transpose = transpose; p.batch = batch; p.Q = Q;
  p.eps = eps; p.variance = variance;
  p.wimg = (const uint8_t*)w->h[0]; p.n_pad = 528; p.bias = (const float*)w->h[1]; p.n_bias = 528;
  p.n_chunks = bias ? 3 : 2;
  p.first_chunk = 0; p.bias_col0 = 512;
  p.chunk_n[0] = 256; p.chunk_n[1] = 256; p.chunk_n[2] = 16;
  p.chunk_row0[0] = 0; p.chunk_row0[1] = 256; p.chunk_row0[2] = 512;
  p.out_q = q; p.out_k = k; p.out_v = v; p.out_g = g; p.out_bias = bias; p.ldb = ldb; p.heads = heads; p.bias_swap = bias_swap;
  p.ldq = (Q + 15) / 16 * 16;
  p.bias_flags = w->bias_flags;
  p.status = (Status*)ctx->tc_status;
  const int64_t tiles = (p.rows + LG_ROWS - 1) / LG_ROWS;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_LN_GEMM);
  ln_gemm_kernel<LG_EPI_ATTENTION><<<grid, LG_THREADS, ln_gemm_smem(528), ctx->stream>>>(CUtensorMap{}, CUtensorMap{}, PlaneMaps{}, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

lf_status make_map_f16_3d_box(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1, uint32_t b2);

// Pair bias from a pair tensor with a LayerNorm of its own (MSA row attention with pair bias, AF3 single attention,
// AF3 MSA pair-weighted averaging): bias[h][q][k] = LN(pair)[q][k] . W[:, h] as fp16 [heads][Q][ldb], by the
// projection kernel with the pair-bias chunk alone (image w->h[4]: 16 rows, gain folded; w->h[5]: the offset's share).
lf_status pair_bias_project(lf_context* ctx, ArenaCursor& cur, const void* pair, int pair_dtype, int Q, int variance, float eps,
                            int heads, const lf_weights* w, op16* bias, int ldb) {
  if (cur.dry) return LF_OK;
  LnGemmParams p{};
  p.act = pair; p.act_bf16 = pair_dtype == LF_DTYPE_BF16; p.rows = (int64_t)Q * Q; p.transpose = 0; p.batch = Q; p.Q = Q;
  p.eps = eps; p.variance = variance;
  p.wimg = (const uint8_t*)w->h[4]; p.n_pad = 16; p.bias = (const float*)w->h[5]; p.n_bias = 16;
  p.n_chunks = 1; p.chunk_n[0] = 16; p.chunk_row0[0] = 0; p.first_chunk = 2; p.bias_col0 = 0;
  p.out_bias = bias; p.ldb = ldb; p.heads = heads; p.bias_swap = 0; p.ldq = (Q + 15) / 16 * 16;
  p.status = (Status*)ctx->tc_status;
  const int64_t tiles = (p.rows + LG_ROWS - 1) / LG_ROWS;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_LN_GEMM);
  ln_gemm_kernel<LG_EPI_ATTENTION><<<grid, LG_THREADS, ln_gemm_smem(16), ctx->stream>>>(CUtensorMap{}, CUtensorMap{}, PlaneMaps{}, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

// out[dst(r)] = resid[dst(r)] + o[r] Wo + bo, r in logical order, dst the transposed-orientation rule
lf_status attention_output(lf_context* ctx, ArenaCursor& cur, const op16* o, int batch, int Q, int transpose,
                           const lf_weights* w, const void* resid, void* out, int act_dtype) {
  if (cur.dry) return LF_OK;
  LnGemmParams p{};
  p.act = o; p.a_is_op16 = 1; p.rows = (int64_t)batch * Q; p.transpose = transpose; p.batch = batch; p.Q = Q;
  p.ldq = (Q + 15) / 16 * 16;
  p.eps = 1e-5f; p.variance = 1;
  p.wimg = (const uint8_t*)w->h[2]; p.n_pad = 128; p.bias = w->f[ATT_BO]; p.n_bias = 128;
  p.n_chunks = 1; p.chunk_n[0] = 128; p.chunk_row0[0] = 0;
  p.resid = resid; p.out = out; p.out_bf16 = act_dtype == LF_DTYPE_BF16;
  p.status = (Status*)ctx->tc_status;
  // float32 pair, updated in place (or no residual): the residual tile and the result travel by TMA.  Logical
  // rows (b, q) sit at pair row b*Q + q, or q*batch + b for the transposed orientation, where a warp's 32
  // consecutive q must share b.
  CUtensorMap mo{};
  p.tma_out = (!p.out_bf16 && (resid == nullptr || resid == out)) ? 1 : 0;
  if (p.tma_out) {
    if (transpose) {
      LF_TRY(make_map_f32_rows(ctx, &mo, out, (uint64_t)batch, (uint64_t)Q, 512, (uint64_t)batch * 512, 1, 32));
      // a query length that is not a multiple of 32: tiles along the batch rows, so that a warp's 32 queries share
      // their batch row; the copy clips the last tile of a row at Q
      if (Q % 32 != 0) { p.tile_per_row = (Q + LG_ROWS - 1) / LG_ROWS; p.n = Q; p.plane_rows = batch; }
    } else {
      LF_TRY(make_map_f32_rows(ctx, &mo, out, (uint64_t)p.rows, 1, 512, (uint64_t)p.rows * 512, 32, 1));
    }
  }
  const int64_t tiles = p.tile_per_row ? (int64_t)batch * p.tile_per_row : (p.rows + LG_ROWS - 1) / LG_ROWS;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_LN_GEMM);
  // the fp16 rows are in logical order; the transposed scatter happens in the epilogue (or in the tensor map)
  ln_gemm_kernel<LG_EPI_OUTPUT><<<grid, LG_THREADS, ln_gemm_smem(128, false, true), ctx->stream>>>(CUtensorMap{}, mo, PlaneMaps{}, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

// out = resid + (LN_c(x) Wz + bz) * sigmoid(LN(z) Wg + bg); x is [128][n][ld] fp16 stored scaled by xscale
lf_status triangle_output(lf_context* ctx, ArenaCursor& cur, const op16* x, int rows, int n, int ld, float x_eps,
                          const void* z, int act_dtype, int variance, float eps, const lf_weights* w, const void* resid,
                          void* out, int64_t x_plane_elems) {
  if (cur.dry) return LF_OK;
  CUtensorMap mapX;
  LF_TRY(make_map_f16_3d_box(ctx, &mapX, x, n, rows, 128, (uint64_t)ld * 2,
                             (uint64_t)(x_plane_elems ? x_plane_elems : (int64_t)rows * ld) * 2, 64, 1, 128));
  LnGemmParams p{};
  p.act = z; p.act_bf16 = act_dtype == LF_DTYPE_BF16; p.rows = (int64_t)rows * n; p.transpose = 0; p.batch = 1; p.Q = 1;
  p.plane_rows = rows;
  p.eps = eps; p.variance = variance;
  p.wimg = (const uint8_t*)w->h[2]; p.n_pad = 256; p.bias = (const float*)w->h[3]; p.n_bias = 384;
  p.n_chunks = 1; p.chunk_n[0] = 256; p.chunk_row0[0] = 0;
  p.n = n; p.ld = ld; p.tile_per_row = (n + LG_ROWS - 1) / LG_ROWS; p.x_eps = x_eps;
  p.resid = resid; p.out = out; p.out_bf16 = act_dtype == LF_DTYPE_BF16;
  p.status = (Status*)ctx->tc_status;
  const int64_t tiles = (int64_t)rows * p.tile_per_row;
  const int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
  // float32 pair updated in place (or no residual): the residual tile and the result travel by TMA; the map is
  // (channel, k, i) so that the last tile of a pair row is clipped at k = n
  CUtensorMap mo{};
  p.tma_out = (!p.out_bf16 && (resid == nullptr || resid == out)) ? 1 : 0;
  if (p.tma_out) LF_TRY(make_map_f32_rows_half(ctx, &mo, out, (uint64_t)n, (uint64_t)rows, 512, (uint64_t)n * 512, 32, 1));
  lf_prof_begin(ctx, LF_KERNEL_TRIANGLE_OUTPUT);
  ln_gemm_kernel<LG_EPI_TRI_OUT><<<grid, LG_THREADS, ln_gemm_smem(256, true, false), ctx->stream>>>(mapX, mo, PlaneMaps{}, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

}  // namespace tc
