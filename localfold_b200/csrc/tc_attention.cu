// Gated attention core on tcgen05 for 4 heads x 32 (128-channel) activations.
//
// Work item = (batch row b, tile of 128 queries, pair of heads).  K and V tiles of 128
// keys stream through a two-stage TMA ring (both heads of the pair share a 128-byte
// swizzled row: 64 B per head).  Per key tile and head: S = Q K^T on the tensor core
// into TMEM; eight softmax warps (one thread per query row and head, so every row
// reduction is thread-local) add the pair bias and the key mask, keep the running
// maximum and sum, and write P as fp16 into swizzled shared memory; P V runs on the
// tensor core into the TMEM columns S just vacated, and the row's output accumulator
// lives in registers.  The full N x N x N logits never exist in memory.
//
// Warp roles: 0..3 softmax of head 0, 4..7 softmax of head 1 (TMEM lane quadrant =
// warp % 4), 8 TMA producer + mask terms, 9 MMA issuer and TMEM owner.
#include <cuda.h>

#include "tc05.cuh"
#include "tc_kernels.cuh"

namespace tc {

using namespace tc05;

constexpr int FA_THREADS = 10 * 32;
constexpr int FA_TILE = 128;
constexpr int FA_Q_BYTES = FA_TILE * 128;          // 128 rows x (2 heads x 32 x 2 B)
constexpr int FA_KV_BYTES = FA_TILE * 128;
constexpr int FA_P_BYTES = FA_TILE * FA_TILE * 2;  // per head: two 16 KiB k-atoms
constexpr int FA_SMEM = FA_Q_BYTES + 2 * 2 * FA_KV_BYTES + 2 * FA_P_BYTES + 2 * FA_TILE * 4 + 256 + 1024;

struct FlashParams {
  int batch, Q, qtiles, ktiles;
  int transpose, mask_mode, clamp;
  const float* mask;       // b*Q + j, or j*batch + b when transpose
  const op16* bias;        // [4][Q][ldb] fp16 or null
  int ldb;
  const op16* gate;        // [batch*Q][128] sigmoid(gate)
  op16* out;               // [batch*Q][128]
  Status* status;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
             const __grid_constant__ CUtensorMap mapV, const FlashParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + FA_Q_BYTES;                 // [2 stages]
  uint8_t* sV = sK + 2 * FA_KV_BYTES;            // [2 stages]
  uint8_t* sP = sV + 2 * FA_KV_BYTES;            // [2 heads]
  float* sMask = reinterpret_cast<float*>(sP + 2 * FA_P_BYTES);   // [2 stages][128] additive terms
  uint64_t* bars = reinterpret_cast<uint64_t*>(sMask + 2 * FA_TILE);
  uint64_t* q_full = bars;           // 1
  uint64_t* q_empty = bars + 1;      // 1
  uint64_t* kv_full = bars + 2;      // [2] count 2: TMA bytes + mask terms
  uint64_t* kv_empty = bars + 4;     // [2]
  uint64_t* s_full = bars + 6;       // [head][buf]
  uint64_t* s_free = bars + 10;      // [head][buf] count 4
  uint64_t* p_full = bars + 14;      // [head] count 4
  uint64_t* o_full = bars + 16;      // [head][buf]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* mask_flag = abort_flag + 1;      // [2 stages]: the stage has a non-zero term

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t items = (int64_t)p.batch * p.qtiles * 2;
  const int T = p.ktiles;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 2); mbar_init(&kv_empty[s], 1); mbar_init(&p_full[s], 4); }
    for (int i = 0; i < 4; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4); mbar_init(&o_full[i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ---------------- TMA producer + mask terms ----------------
    if (lane == 0) { prefetch_tensormap(&mapQ); prefetch_tensormap(&mapK); prefetch_tensormap(&mapV); }
    uint32_t n_item = 0, n_kv = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x, ++n_item) {
      const int hp = (int)(item & 1);
      const int qt = (int)((item >> 1) % p.qtiles);
      const int b = (int)((item >> 1) / p.qtiles);
      if (lane == 0) {
        if (!mbar_wait(q_empty, (n_item & 1) ^ 1, abort_flag, p.status, 20)) ok = false;
        else {
          mbar_expect_tx(q_full, FA_Q_BYTES);
          tma_load_3d(sQ, &mapQ, q_full, hp * 64, qt * FA_TILE, b);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      for (int t = 0; t < T && ok; ++t, ++n_kv) {
        const int st = n_kv & 1;
        if (lane == 0) {
          if (!mbar_wait(&kv_empty[st], ((n_kv >> 1) & 1) ^ 1, abort_flag, p.status, 21)) ok = false;
          else {
            mbar_expect_tx(&kv_full[st], 2 * FA_KV_BYTES);
            tma_load_3d(sK + st * FA_KV_BYTES, &mapK, &kv_full[st], hp * 64, t * FA_TILE, b);
            tma_load_3d(sV + st * FA_KV_BYTES, &mapV, &kv_full[st], hp * 64, t * FA_TILE, b);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        // additive key terms for this tile: 4 keys per lane
        bool any = false;
        float term[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = t * FA_TILE + lane * 4 + e;
          float v = -INFINITY;
          if (j < p.Q) {
            const float m = p.mask[p.transpose ? (int64_t)j * p.batch + b : (int64_t)b * p.Q + j];
            v = p.mask_mode == 0 ? 1e9f * (m - 1.0f) : (m > 0.f ? 0.f : -1e9f);
          }
          term[e] = v;
          any = any || v != 0.f;
        }
        *reinterpret_cast<float4*>(sMask + st * FA_TILE + lane * 4) = make_float4(term[0], term[1], term[2], term[3]);
        const unsigned ballot = __ballot_sync(0xffffffffu, any);
        __syncwarp();   // orders every lane's term stores before the publishing arrive
        if (lane == 0) { mask_flag[st] = ballot != 0; mbar_arrive(&kv_full[st]); }
      }
    }
  } else if (warp == 9) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(FA_TILE, FA_TILE, 0, 0);   // S[q][k], both K-major
      constexpr uint32_t idesc_pv = make_idesc_f16(FA_TILE, 32, 0, 1);        // O[q][d]: P K-major, V MN-major
      uint32_t n_item = 0, n_kv = 0, n_tile[2] = {0, 0};
      bool ok = true;
      const uint32_t q_addr = smem_u32(sQ);
      auto issue_pv = [&](int h, int st, int buf) {
        const uint32_t p_addr = smem_u32(sP + h * FA_P_BYTES);
        const uint32_t v_addr = smem_u32(sV + st * FA_KV_BYTES) + h * 64;
        const uint32_t d = tmem_base + (h * 2 + buf) * FA_TILE;
#pragma unroll
        for (int kk = 0; kk < FA_TILE / 16; ++kk) {
          const uint64_t adesc = make_smem_desc(p_addr + (kk >> 2) * (FA_TILE * 128) + (kk & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(v_addr + kk * 2048, 8192, 1024);
          umma_f16(d, adesc, bdesc, idesc_pv, kk != 0 ? 1u : 0u);
        }
      };
      for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x, ++n_item) {
        if (!mbar_wait(q_full, n_item & 1, abort_flag, p.status, 30)) break;
        tc_fence_after();
        for (int t = 0; t < T && ok; ++t, ++n_kv) {
          const int st = n_kv & 1;
          if (!mbar_wait(&kv_full[st], (n_kv >> 1) & 1, abort_flag, p.status, 31)) { ok = false; break; }
          tc_fence_after();
          const uint32_t k_addr = smem_u32(sK + st * FA_KV_BYTES);
          for (int h = 0; h < 2; ++h) {
            const uint32_t u = n_tile[h];        // tiles issued so far for this head
            const int buf = u & 1;
            if (!mbar_wait(&s_free[h * 2 + buf], ((u >> 1) & 1) ^ 1, abort_flag, p.status, 32)) { ok = false; break; }
            tc_fence_after();
            const uint32_t d = tmem_base + (h * 2 + buf) * FA_TILE;
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
              const uint64_t adesc = make_smem_desc(q_addr + h * 64 + kk * 32, 16, 1024);
              const uint64_t bdesc = make_smem_desc(k_addr + h * 64 + kk * 32, 16, 1024);
              umma_f16(d, adesc, bdesc, idesc_qk, kk);
            }
            umma_commit(&s_full[h * 2 + buf]);
          }
          if (!ok) break;
          if (t == T - 1) umma_commit(q_empty);
          if (t >= 1) {
            // P V of the previous tile
            const int pst = (n_kv - 1) & 1;
            for (int h = 0; h < 2; ++h) {
              const uint32_t u = n_tile[h] - 1;
              if (!mbar_wait(&p_full[h], u & 1, abort_flag, p.status, 33)) { ok = false; break; }
              tc_fence_after();
              issue_pv(h, pst, u & 1);
              umma_commit(&o_full[h * 2 + (u & 1)]);
            }
            if (!ok) break;
            umma_commit(&kv_empty[pst]);
          }
          n_tile[0]++; n_tile[1]++;
        }
        if (!ok) break;
        // P V of the item's last tile
        const int pst = (n_kv - 1) & 1;
        for (int h = 0; h < 2; ++h) {
          const uint32_t u = n_tile[h] - 1;
          if (!mbar_wait(&p_full[h], u & 1, abort_flag, p.status, 34)) { ok = false; break; }
          tc_fence_after();
          issue_pv(h, pst, u & 1);
          umma_commit(&o_full[h * 2 + (u & 1)]);
        }
        if (!ok) break;
        umma_commit(&kv_empty[pst]);
      }
    }
  } else {
    // ---------------- softmax: one thread per (query row, head) ----------------
    const int h = warp >> 2, q = warp & 3;
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const float L2E = 1.4426950408889634f;
    uint32_t n_kv = 0, n_tile = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int hp = (int)(item & 1);
      const int qt = (int)((item >> 1) % p.qtiles);
      const int b = (int)((item >> 1) / p.qtiles);
      const int head = hp * 2 + h;
      const int qi = qt * FA_TILE + row;
      const bool qvalid = qi < p.Q;
      const op16* bias_row = p.bias ? p.bias + ((int64_t)head * p.Q + (qvalid ? qi : 0)) * p.ldb : nullptr;
      float m_run = -INFINITY, l_run = 0.f, corr_prev = 0.f;
      float O[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) O[e] = 0.f;
      for (int t = 0; t < T && ok; ++t, ++n_kv, ++n_tile) {
        const int st = n_kv & 1, buf = n_tile & 1;
        if (!mbar_wait(&s_full[h * 2 + buf], (n_tile >> 1) & 1, abort_flag, p.status, 40)) { ok = false; break; }
        tc_fence_after();
        float s[FA_TILE];
        {
          const uint32_t acc = tmem_base + lane_addr + (h * 2 + buf) * FA_TILE;
          uint32_t* su = reinterpret_cast<uint32_t*>(s);
          tmem_ld32(acc, *reinterpret_cast<uint32_t(*)[32]>(su));
          tmem_ld32(acc + 32, *reinterpret_cast<uint32_t(*)[32]>(su + 32));
          tmem_ld32(acc + 64, *reinterpret_cast<uint32_t(*)[32]>(su + 64));
          tmem_ld32(acc + 96, *reinterpret_cast<uint32_t(*)[32]>(su + 96));
          tmem_ld_wait();
        }
        // key terms of this stage were published through kv_full
        if (!mbar_wait(&kv_full[st], (n_kv >> 1) & 1, abort_flag, p.status, 41)) { ok = false; break; }
        const bool masked = mask_flag[st] != 0;
        if (masked) {
          const float4* mt = reinterpret_cast<const float4*>(sMask + st * FA_TILE);
#pragma unroll
          for (int j4 = 0; j4 < FA_TILE / 4; ++j4) {
            const float4 m = mt[j4];
            s[j4 * 4] += m.x; s[j4 * 4 + 1] += m.y; s[j4 * 4 + 2] += m.z; s[j4 * 4 + 3] += m.w;
          }
        }
        if (bias_row) {
          const int k0 = t * FA_TILE;
#pragma unroll
          for (int g8 = 0; g8 < FA_TILE / 8; ++g8) {
            if (k0 + g8 * 8 < p.ldb) {
              const uint4 raw = __ldg(reinterpret_cast<const uint4*>(bias_row + k0 + g8 * 8));
              const uint32_t wv[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&wv[e]));
                s[g8 * 8 + e * 2] += f.x;
                s[g8 * 8 + e * 2 + 1] += f.y;
              }
            }
          }
        }
        if (masked && p.clamp) {
#pragma unroll
          for (int j = 0; j < FA_TILE; ++j)   // keys past the end stay at -inf: they are not keys at all
            s[j] = s[j] == -INFINITY ? s[j] : fminf(fmaxf(s[j], -1e8f), 1e8f);
        }
        float mx = s[0];
#pragma unroll
        for (int j = 1; j < FA_TILE; ++j) mx = fmaxf(mx, s[j]);
        const float m_new = fmaxf(m_run, mx);
        const float corr = ex2f((m_run - m_new) * L2E);
        const float neg = -m_new * L2E;
        float sum = 0.f;
        uint32_t pk[FA_TILE / 2];
#pragma unroll
        for (int j = 0; j < FA_TILE; j += 2) {
          const float p0 = ex2f(fmaf(s[j], L2E, neg)), p1 = ex2f(fmaf(s[j + 1], L2E, neg));
          // the sum uses the values the tensor core will see
          const __half2 hp2 = __floats2half2_rn(p0, p1);
          const float2 back = __half22float2(hp2);
          sum += back.x + back.y;
          pk[j >> 1] = *reinterpret_cast<const uint32_t*>(&hp2);
        }
        l_run = l_run * corr + sum;
        m_run = m_new;
        if (t > 0) {
          // fold in P V of the previous tile (this also frees the P tile and that S buffer)
          const int pbuf = buf ^ 1;
          if (!mbar_wait(&o_full[h * 2 + pbuf], ((n_tile - 1) >> 1) & 1, abort_flag, p.status, 42)) { ok = false; break; }
          tc_fence_after();
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_addr + (h * 2 + pbuf) * FA_TILE, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) O[e] = fmaf(O[e], corr_prev, __uint_as_float(o[e]));
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_free[h * 2 + pbuf]);
        }
        corr_prev = corr;
        // P as the K-major A operand of P V: row `row`, 128 keys = 2 k-atoms x 8 chunks of 16 B
        {
          uint8_t* pt = sP + h * FA_P_BYTES;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            uint8_t* dst = pt + (c >> 3) * (FA_TILE * 128) + swizzle128_offset((uint32_t)row, (uint32_t)(c & 7));
            *reinterpret_cast<uint4*>(dst) = make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
          }
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[h]);
      }
      if (!ok) break;
      {
        const int lbuf = (n_tile - 1) & 1;
        if (!mbar_wait(&o_full[h * 2 + lbuf], ((n_tile - 1) >> 1) & 1, abort_flag, p.status, 43)) { ok = false; break; }
        tc_fence_after();
        uint32_t o[32];
        tmem_ld32(tmem_base + lane_addr + (h * 2 + lbuf) * FA_TILE, o);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) O[e] = fmaf(O[e], corr_prev, __uint_as_float(o[e]));
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[h * 2 + lbuf]);
      }
      if (qvalid) {
        const int64_t r = (int64_t)b * p.Q + qi;
        const float inv = 1.0f / l_run;
        const uint4* g4 = reinterpret_cast<const uint4*>(p.gate + r * 128 + head * 32);
        op16* dst = p.out + r * 128 + head * 32;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[8];
          const uint4 ga = g4[c * 2], gb = g4[c * 2 + 1];
          const uint32_t gw[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&gw[e]));
            pk[e] = pack_half2(O[c * 16 + e * 2] * inv * gf.x, O[c * 16 + e * 2 + 1] * inv * gf.y);
          }
          st_global_v8(dst + c * 16, pk);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) drain_after_abort();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

void configure_attention() {
  cudaFuncSetAttribute(flash_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM);
  cudaGetLastError();
}

lf_status make_map_f16_3d_ext(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1);

lf_status attention_core(lf_context* ctx, ArenaCursor& cur, const op16* q, const op16* k, const op16* v, const op16* g,
                         const op16* bias, int ldb, const float* mask, int batch, int Q, int transpose, int mask_mode,
                         int clamp, op16* out) {
  if (cur.dry) return LF_OK;
  CUtensorMap mq, mk, mv;
  const uint64_t row = 256, plane = (uint64_t)Q * 256;
  LF_TRY(make_map_f16_3d_ext(ctx, &mq, q, 128, Q, batch, row, plane, 64, FA_TILE));
  LF_TRY(make_map_f16_3d_ext(ctx, &mk, k, 128, Q, batch, row, plane, 64, FA_TILE));
  LF_TRY(make_map_f16_3d_ext(ctx, &mv, v, 128, Q, batch, row, plane, 64, FA_TILE));
  FlashParams p{};
  p.batch = batch; p.Q = Q; p.qtiles = (Q + FA_TILE - 1) / FA_TILE; p.ktiles = p.qtiles;
  p.transpose = transpose; p.mask_mode = mask_mode; p.clamp = clamp; p.mask = mask; p.bias = bias; p.ldb = ldb;
  p.gate = g; p.out = out; p.status = (Status*)ctx->tc_status;
  const int64_t items = (int64_t)batch * p.qtiles * 2;
  const int grid = (int)(items < ctx->sm_count ? items : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_ATTENTION);
  flash_kernel<<<grid, FA_THREADS, FA_SMEM, ctx->stream>>>(mq, mk, mv, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

}  // namespace tc
