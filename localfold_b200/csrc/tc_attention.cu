// Gated attention core on tcgen05 for 4 heads x 32 (128-channel) activations.
//
// Work item = (batch row b, pair of 128-query tiles, pair of heads): four independent streams
// (query tile g, head h) that share the K and V tiles of the head pair, which stream through a
// two-stage TMA ring (both heads of the pair share a 128-byte swizzled row: 64 B per head).
// Per key tile and stream: S = Q K^T on the tensor core into the stream's 128 TMEM columns;
// the stream's four softmax warps (one thread per query row, so every row reduction is
// thread-local) read S once in 16-column pieces, add the pair bias and the key mask,
// exponentiate against a reference maximum known in advance (raised, with an in-place rescale of
// what was written, in the rare tile where a logit outruns it) and write P as packed fp16 back
// into the TMEM columns of S already consumed; P V then runs on the tensor core with P as the A
// operand straight from tensor memory, into TMEM columns S has vacated, and is folded into the
// row's register accumulator.  P never touches shared memory.  Sixteen softmax warps (four per scheduler)
// hide each other's memory and MMA latency at under 100 registers per thread.  The N x N x N
// logits never exist in memory.
//
// Warp roles: warp w < 16: softmax of stream w / 4 (TMEM lane quadrant = w % 4);
// 16: TMA producer + mask terms; 17: MMA issuer and TMEM owner.
#include <cuda.h>

#include "tc05.cuh"
#include "tc_kernels.cuh"

namespace tc {

using namespace tc05;

constexpr int FA_THREADS = 19 * 32;
constexpr int FA_TILE = 128;
constexpr int FA_Q_BYTES = FA_TILE * 128;          // per query tile: 128 rows x (2 heads x 32 x 2 B)
constexpr int FA_KV_BYTES = FA_TILE * 128;
constexpr int FA_BIAS_BYTES = FA_TILE * FA_TILE * 2;   // one stream's bias tile: 128 queries x 128 keys, fp16
constexpr int FA_BIAS_SLOTS = 3;
constexpr int FA_IDENT_BYTES = 2048;                    // 16 x 16 identity, 128-byte swizzled rows
constexpr int FA_SMEM = 2 * FA_Q_BYTES + 2 * 2 * FA_KV_BYTES + FA_BIAS_SLOTS * FA_BIAS_BYTES + FA_IDENT_BYTES +
                        2 * FA_TILE * 4 + 512 + 1024;

struct FlashParams {
  int batch, Q, qtiles, qpairs, ktiles;
  int transpose, mask_mode, clamp;
  const float* mask;       // b*Q + j, or j*batch + b when transpose
  int has_bias, ldb;       // the bias [4][Q][ldb] fp16 arrives through its tensor map
  const op16* gate;        // [batch*Q][128] sigmoid(gate)
  op16* out;               // [batch*Q][128]
  Status* status;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#ifdef LF_FLASH_TRACE
// Development aid, compiled only on request: clock stamps of CTA 0's first 24 tiles per stream.
__device__ long long lf_flash_trace[24 * 4 * 10];
#define FA_TRACE(stream_, tile_, ev_) \
  do { if (blockIdx.x == 0 && (tile_) < 24u) lf_flash_trace[(((stream_) * 24 + (tile_)) * 10) + (ev_)] = clock64(); } while (0)
#else
#define FA_TRACE(stream_, tile_, ev_) do {} while (0)
#endif

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
             const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapB, const FlashParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                            // [2 query tiles]
  uint8_t* sK = sQ + 2 * FA_Q_BYTES;             // [2 stages]
  uint8_t* sV = sK + 2 * FA_KV_BYTES;            // [2 stages]
  uint8_t* sBias = sV + 2 * FA_KV_BYTES;         // [3 slots] one stream's tile each
  uint8_t* sIdent = sBias + FA_BIAS_SLOTS * FA_BIAS_BYTES;
  float* sMask = reinterpret_cast<float*>(sIdent + FA_IDENT_BYTES);   // [2 stages][128] additive terms
  uint64_t* bars = reinterpret_cast<uint64_t*>(sMask + 2 * FA_TILE);
  uint64_t* q_full = bars;           // 1
  uint64_t* q_empty = bars + 1;      // 1
  uint64_t* kv_full = bars + 2;      // [2] count 2: TMA bytes + mask terms
  uint64_t* kv_empty = bars + 4;     // [2]
  uint64_t* s_full = bars + 6;       // [stream]
  uint64_t* s_free = bars + 10;      // [stream] count 4
  uint64_t* p_full = bars + 14;      // [stream] count 4
  uint64_t* o_full = bars + 18;      // [stream]
  uint64_t* b_full = bars + 22;      // [slot]
  uint64_t* b_empty = bars + 25;     // [slot]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 28);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* mask_flag = abort_flag + 1;      // [2 stages]: the stage has a non-zero term

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t items = (int64_t)p.batch * p.qpairs * 2;
  const int T = p.ktiles;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 2); mbar_init(&kv_empty[s], 1); }
    for (int i = 0; i < 4; ++i) { mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4); mbar_init(&p_full[i], 4); mbar_init(&o_full[i], 1); }
    for (int i = 0; i < FA_BIAS_SLOTS; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 17) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  // 16 x 16 identity (K-major, 128-byte swizzled rows of which the first 32 bytes are used): the
  // B operand that adds a bias tile onto S through the tensor core
  for (int i = threadIdx.x; i < FA_IDENT_BYTES / 4; i += FA_THREADS) reinterpret_cast<uint32_t*>(sIdent)[i] = 0u;
  __syncthreads();
  if (threadIdx.x < 16)
    *reinterpret_cast<__half*>(sIdent + swizzle128_offset(threadIdx.x, threadIdx.x >> 3) + (threadIdx.x & 7) * 2) = __float2half(1.0f);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 16) {
    // ---------------- TMA producer + mask terms ----------------
    if (lane == 0) { prefetch_tensormap(&mapQ); prefetch_tensormap(&mapK); prefetch_tensormap(&mapV); }
    uint32_t n_item = 0, n_kv = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x, ++n_item) {
      const int hp = (int)(item & 1);
      const int qp = (int)((item >> 1) % p.qpairs);
      const int b = (int)((item >> 1) / p.qpairs);
      if (lane == 0) {
        if (!mbar_wait(q_empty, (n_item & 1) ^ 1, abort_flag, p.status, 20)) ok = false;
        else {
          mbar_expect_tx(q_full, 2 * FA_Q_BYTES);
          tma_load_3d(sQ, &mapQ, q_full, hp * 64, (2 * qp) * FA_TILE, b);
          tma_load_3d(sQ + FA_Q_BYTES, &mapQ, q_full, hp * 64, (2 * qp + 1) * FA_TILE, b);
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
  } else if (warp == 18) {
    // ---------------- bias tiles: one per stream and key tile, in the order (key tile, stream) ----------------
    if (lane == 0 && p.has_bias) {
      prefetch_tensormap(&mapB);
      uint32_t n = 0;
      bool ok = true;
      for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int hp = (int)(item & 1);
        const int qp = (int)((item >> 1) % p.qpairs);
        for (int t = 0; t < T && ok; ++t) {
          for (int sidx = 0; sidx < 4 && ok; ++sidx, ++n) {
            const uint32_t slot = n % FA_BIAS_SLOTS, use = n / FA_BIAS_SLOTS;
            if (!mbar_wait(&b_empty[slot], (use & 1) ^ 1, abort_flag, p.status, 22)) { ok = false; break; }
            uint8_t* dst = sBias + slot * FA_BIAS_BYTES;
            const int q0 = (2 * qp + (sidx >> 1)) * FA_TILE, head = hp * 2 + (sidx & 1);
            // no copy starts outside the tensor: a half tile past the last key or a query tile past
            // the last row is not fetched, and the issuer leaves the matching steps out
            const bool first = q0 < p.Q, second = first && t * FA_TILE + 64 < p.ldb;
            if (!first) { mbar_arrive(&b_full[slot]); continue; }
            mbar_expect_tx(&b_full[slot], second ? FA_BIAS_BYTES : FA_BIAS_BYTES / 2);
            tma_load_3d(dst, &mapB, &b_full[slot], t * FA_TILE, q0, head);
            if (second) tma_load_3d(dst + FA_BIAS_BYTES / 2, &mapB, &b_full[slot], t * FA_TILE + 64, q0, head);
          }
        }
      }
    }
  } else if (warp == 17) {
    // ---------------- MMA issuer ----------------
    // Event driven: the four streams advance at their own pace.  The thread polls, per stream, for
    // "P of tile u is written" (then issues P V) and for "the stream's columns are free, K/V of tile
    // u+1 and the item's Q have landed" (then issues Q K^T), so one stream's softmax overlaps the
    // tensor-core latency of the others.  Streams stay within two tiles of each other (K/V ring).
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(FA_TILE, FA_TILE, 0, 0);   // S[q][k], both K-major
      constexpr uint32_t idesc_pv = make_idesc_f16(FA_TILE, 32, 0, 1);        // O[q][d]: P K-major, V MN-major
      constexpr uint32_t idesc_b = make_idesc_f16(FA_TILE, 16, 0, 0);         // S[:, 16 keys] += bias[:, 16 keys] I
      const uint64_t ident_desc = make_smem_desc(smem_u32(sIdent), 16, 1024);
      uint32_t my_items = 0;
      for (int64_t item = blockIdx.x; item < items; item += gridDim.x) ++my_items;
      const uint32_t U = my_items * (uint32_t)T;      // key tiles this CTA walks through, all items
      uint32_t qk_u[4] = {0, 0, 0, 0}, pv_u[4] = {0, 0, 0, 0};
      uint32_t pv_cnt[2] = {0, 0}, last_qk_cnt = 0, done = 0, b_next = 0;
      uint64_t idle_since = 0;
      uint32_t idle_polls = 0;
#ifdef LF_FLASH_TRACE
      uint32_t seen_a[4] = {0, 0, 0, 0}, seen_b[4] = {0, 0, 0, 0};
#endif
      while (done < 4) {
        bool progress = false;
#pragma unroll
        for (int sidx = 0; sidx < 4; ++sidx) {
          const int g = sidx >> 1, h = sidx & 1;
          const uint32_t d = tmem_base + sidx * FA_TILE;
          if (pv_u[sidx] < qk_u[sidx]) {
            const uint32_t u = pv_u[sidx];
            if (mbar_test(&p_full[sidx], u & 1)) {
              tc_fence_after();
              FA_TRACE(sidx, u, 6);
              const int st = u & 1;
              // P is the A operand straight from tensor memory: 16 keys per step = 8 packed columns;
              // the product lands in columns 64..95 of the stream's region (S there is dead by now)
              const uint32_t v_addr = smem_u32(sV + st * FA_KV_BYTES);
#pragma unroll
              for (int kk = 0; kk < FA_TILE / 16; ++kk) {
                const uint64_t bdesc = make_smem_desc(v_addr + h * 64 + kk * 2048, 8192, 1024);
                umma_f16_ts(d + 64, d + kk * 8, bdesc, idesc_pv, kk != 0 ? 1u : 0u);
              }
              umma_commit(&o_full[sidx]);
              FA_TRACE(sidx, u, 5);
              if (++pv_cnt[st] == 4) { pv_cnt[st] = 0; umma_commit(&kv_empty[st]); }
              pv_u[sidx] = u + 1;
              if (u + 1 == U) ++done;
              progress = true;
            }
          } else if (qk_u[sidx] < U) {
            const uint32_t u = qk_u[sidx];
            const uint32_t it_idx = u / (uint32_t)T, t = u % (uint32_t)T;
            const int st = u & 1;
            const uint32_t bn = u * 4 + sidx, bslot = bn % FA_BIAS_SLOTS;
#ifdef LF_FLASH_TRACE
            if (mbar_test(&s_free[sidx], (u & 1) ^ 1) && seen_a[sidx] != u + 1) { seen_a[sidx] = u + 1; FA_TRACE(sidx, u, 8); }
            if (mbar_test(&kv_full[st], (u >> 1) & 1) && seen_b[sidx] != u + 1) { seen_b[sidx] = u + 1; FA_TRACE(sidx, u, 9); }
#endif
            // bias tiles sit in one ring filled in the order (key tile, stream), so with a bias the
            // streams take their Q K^T turns in that order too
            if (mbar_test(&s_free[sidx], (u & 1) ^ 1) && mbar_test(&kv_full[st], (u >> 1) & 1) && mbar_test(q_full, it_idx & 1) &&
                (!p.has_bias || (bn == b_next && mbar_test(&b_full[bslot], (bn / FA_BIAS_SLOTS) & 1)))) {
              tc_fence_after();
              FA_TRACE(sidx, u, 7);
              const uint32_t q_addr = smem_u32(sQ + g * FA_Q_BYTES);
              const uint32_t k_addr = smem_u32(sK + st * FA_KV_BYTES);
#pragma unroll
              for (int kk = 0; kk < 2; ++kk) {
                const uint64_t adesc = make_smem_desc(q_addr + h * 64 + kk * 32, 16, 1024);
                const uint64_t bdesc = make_smem_desc(k_addr + h * 64 + kk * 32, 16, 1024);
                umma_f16(d, adesc, bdesc, idesc_qk, kk);
              }
              if (p.has_bias) {
                // the tile's bias is added by the tensor core: 16 keys per step against the identity
                // (key groups past the padded row and query tiles past the last row were not fetched)
                const uint32_t b_addr = smem_u32(sBias + bslot * FA_BIAS_BYTES);
                const int it_qp = (int)(((blockIdx.x + (int64_t)it_idx * gridDim.x) >> 1) % p.qpairs);
                const int groups = (2 * it_qp + g) * FA_TILE < p.Q ? min(FA_TILE / 16, (p.ldb - (int)t * FA_TILE) >> 4) : 0;
#pragma unroll
                for (int kk = 0; kk < FA_TILE / 16; ++kk) {
                  if (kk >= groups) break;
                  const uint64_t adesc = make_smem_desc(b_addr + (kk >> 2) * (FA_BIAS_BYTES / 2) + (kk & 3) * 32, 16, 1024);
                  umma_f16(d + kk * 16, adesc, ident_desc, idesc_b, 1);
                }
                umma_commit(&b_empty[bslot]);
                ++b_next;
              }
              umma_commit(&s_full[sidx]);
              FA_TRACE(sidx, u, 4);
              if (t == (uint32_t)T - 1 && ++last_qk_cnt == 4) { last_qk_cnt = 0; umma_commit(q_empty); }
              qk_u[sidx] = u + 1;
              progress = true;
            }
          }
        }
        if (progress) { idle_polls = 0; idle_since = 0; }
        else if ((++idle_polls & 1023u) == 0) {
          if (*abort_flag) break;
          const uint64_t now = global_timer_ns();
          if (idle_since == 0) idle_since = now;
          else if (now - idle_since > kWaitLimitNs) {
            *abort_flag = 1;
            if (p.status && atomicCAS(&p.status->code, 0u, 1u) == 0u) { p.status->where = 35; p.status->block = blockIdx.x; }
            break;
          }
        }
      }
    }
  } else {
    // ---------------- softmax: one thread per query row of one stream ----------------
    const int sidx = warp >> 2, q = warp & 3;
    const int g = sidx >> 1, h = sidx & 1;
    const int row = q * 32 + lane;
    const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + sidx * FA_TILE;
    const float L2E = 1.4426950408889634f;
    uint32_t n_kv = 0, n_tile = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int hp = (int)(item & 1);
      const int qp = (int)((item >> 1) % p.qpairs);
      const int b = (int)((item >> 1) / p.qpairs);
      const int head = hp * 2 + h;
      const int qi = (2 * qp + g) * FA_TILE + row;
      const bool qvalid = qi < p.Q;
      float m_run = -INFINITY, l_run = 0.f;
      float O[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) O[e] = 0.f;
      for (int t = 0; t < T && ok; ++t, ++n_kv, ++n_tile) {
        const int st = n_kv & 1;
        if (!mbar_wait(&s_full[sidx], n_tile & 1, abort_flag, p.status, 40)) { ok = false; break; }
        // key terms of this stage were published through kv_full
        if (!mbar_wait(&kv_full[st], (n_kv >> 1) & 1, abort_flag, p.status, 41)) { ok = false; break; }
        tc_fence_after();
        if (q == 0 && lane == 0) FA_TRACE(sidx, n_tile, 0);
        const bool masked = mask_flag[st] != 0;
        // One pass: exponentials are taken against a reference known before the tile is read - the
        // running reference, raised to the maximum of the tile's first 16 logits - and P (fp16, two keys
        // per 32-bit column) overwrites the S columns already consumed.  A logit may exceed the reference
        // by up to kSlack (e^8 < 3000 fits fp16 and float32 sums easily); when a later piece outruns it,
        // the reference is raised and the P columns already written are rescaled in place.
        constexpr float kSlack = 8.0f;
        float m_ref = m_run, neg = 0.f, sum = 0.f;
        // software pipeline: the S columns of piece c+1 are requested before piece c is worked on
        uint32_t su[16];
        tmem_ld16(acc, su);
#pragma unroll 1
        for (int c = 0; c < FA_TILE / 16; ++c) {
          tmem_ld_wait();
          float sv[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) sv[e] = __uint_as_float(su[e]);
          if (c + 1 < FA_TILE / 16) tmem_ld16(acc + (c + 1) * 16, su);
          if (masked) {
            const float4* mt = reinterpret_cast<const float4*>(sMask + st * FA_TILE + c * 16);
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const float4 m = mt[j4];
              sv[j4 * 4] += m.x; sv[j4 * 4 + 1] += m.y; sv[j4 * 4 + 2] += m.z; sv[j4 * 4 + 3] += m.w;
            }
          }
          if (masked && p.clamp) {
#pragma unroll
            for (int e = 0; e < 16; ++e)   // keys past the end stay at -inf: they are not keys at all
              sv[e] = sv[e] == -INFINITY ? sv[e] : fminf(fmaxf(sv[e], -1e8f), 1e8f);
          }
          float cm = sv[0];
#pragma unroll
          for (int e = 1; e < 16; ++e) cm = fmaxf(cm, sv[e]);
          if (c == 0) {
            m_ref = fmaxf(m_run, cm);
            neg = -m_ref * L2E;
          } else if (__any_sync(0xffffffffu, cm - m_ref > kSlack)) {
            // raise the reference of the rows that need it and rescale what they have written so far
            const float m_up = cm - m_ref > kSlack ? cm : m_ref;
            const float f = ex2f((m_ref - m_up) * L2E);       // 1 for the rows that are fine
            tmem_st_wait();
            for (int cc = 0; cc < c; ++cc) {
              uint32_t w[8];
              tmem_ld8(acc + cc * 8, w);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float2 pv = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
                w[e] = pack_half2(pv.x * f, pv.y * f);
              }
              tmem_st8(acc + cc * 8, w);
            }
            sum *= f;
            m_ref = m_up;
            neg = -m_ref * L2E;
          }
          uint32_t w8[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float p0 = ex2f(fmaf(sv[2 * e], L2E, neg));
            const float p1 = ex2f(fmaf(sv[2 * e + 1], L2E, neg));
            sum += p0 + p1;
            w8[e] = pack_half2(p0, p1);
          }
          tmem_st8(acc + c * 8, w8);      // keys c*16 .. +15 -> columns c*8 .. +7 (below the S columns still unread)
        }
        tmem_st_wait();
        const float corr = ex2f((m_run - m_ref) * L2E);
        m_run = m_ref;
        l_run = l_run * corr + sum;
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[sidx]);
        if (q == 0 && lane == 0) FA_TRACE(sidx, n_tile, 1);
        // P V of this tile lands in columns 64..95 of the stream's region
        if (!mbar_wait(&o_full[sidx], n_tile & 1, abort_flag, p.status, 42)) { ok = false; break; }
        tc_fence_after();
        if (q == 0 && lane == 0) FA_TRACE(sidx, n_tile, 2);
        {
          uint32_t o[32];
          tmem_ld32(acc + 64, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) O[e] = fmaf(O[e], corr, __uint_as_float(o[e]));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[sidx]);
        if (q == 0 && lane == 0) FA_TRACE(sidx, n_tile, 3);
      }
      if (!ok) break;
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
  if (warp == 17) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

void configure_attention() {
  cudaFuncSetAttribute(flash_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM);
  cudaGetLastError();
}

lf_status make_map_f16_3d_ext(lf_context* ctx, CUtensorMap* map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2,
                              uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1);

lf_status attention_core(lf_context* ctx, ArenaCursor& cur, const op16* q, const op16* k, const op16* v, const op16* g,
                         const op16* bias, int ldb, const float* mask, int batch, int Q, int transpose,
                         int mask_mode, int clamp, op16* out) {
  if (cur.dry) return LF_OK;
  CUtensorMap mq, mk, mv, mb;
  const uint64_t row = 256, plane = (uint64_t)Q * 256;
  LF_TRY(make_map_f16_3d_ext(ctx, &mq, q, 128, Q, batch, row, plane, 64, FA_TILE));
  LF_TRY(make_map_f16_3d_ext(ctx, &mk, k, 128, Q, batch, row, plane, 64, FA_TILE));
  LF_TRY(make_map_f16_3d_ext(ctx, &mv, v, 128, Q, batch, row, plane, 64, FA_TILE));
  // bias [4][Q][ldb]: boxes of 64 keys x 128 queries; without a bias the map is a stand-in that is never used
  if (bias) LF_TRY(make_map_f16_3d_ext(ctx, &mb, bias, ldb, Q, 4, (uint64_t)ldb * 2, (uint64_t)Q * ldb * 2, 64, FA_TILE));
  else mb = mq;
  FlashParams p{};
  p.batch = batch; p.Q = Q; p.qtiles = (Q + FA_TILE - 1) / FA_TILE; p.qpairs = (p.qtiles + 1) / 2; p.ktiles = p.qtiles;
  p.transpose = transpose; p.mask_mode = mask_mode; p.clamp = clamp; p.mask = mask; p.has_bias = bias ? 1 : 0; p.ldb = ldb;
  p.gate = g; p.out = out; p.status = (Status*)ctx->tc_status;
  const int64_t items = (int64_t)batch * p.qpairs * 2;
  const int grid = (int)(items < ctx->sm_count ? items : ctx->sm_count);
  lf_prof_begin(ctx, LF_KERNEL_ATTENTION);
  flash_kernel<<<grid, FA_THREADS, FA_SMEM, ctx->stream>>>(mq, mk, mv, mb, p);
  lf_prof_end(ctx);
  ctx->launches++;
  return LF_OK;
}

}  // namespace tc

#ifdef LF_FLASH_TRACE
extern "C" __attribute__((visibility("default"))) int lf_debug_flash_trace(long long* host, int count) {
  return (int)cudaMemcpyFromSymbol(host, tc::lf_flash_trace, sizeof(long long) * count);
}
#endif
