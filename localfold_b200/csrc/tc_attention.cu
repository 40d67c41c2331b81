// Gated attention core on tcgen05 for 4 heads x 32 (128-channel) activations.
//
// Work item = (batch row b, pair of 128-query tiles, pair of heads): four independent streams
// (query tile g, head h) that share the K and V tiles of the head pair, which stream through a
// five-stage TMA ring of 48-key tiles.  Q, K, V (and the gate and the output) live in memory as
// 8-row x 8-channel pieces of 128 bytes; 5-d tensor maps bring a tile's pieces in as
// [rows / 8][8 pieces of the head pair][8 rows][16 B], which is the tensor core's unswizzled
// operand format (K-major for Q and K, MN-major for V).
//
// Per stream, tensor memory holds two S / P buffers (48 columns each) and the output accumulator O
// (32 columns): 128 columns per stream, 512 in all.
// Per key tile: S = Q K^T (+ the pair bias tile, added by the tensor core against an identity
// operand) lands in the S columns; the stream's four softmax warps (one thread per query row, so
// every row reduction is thread-local) read S in 16-column pieces, add the key-mask terms,
// exponentiate against a per-row reference and write P as packed fp16 over the S columns already
// consumed; O += P V then runs with P as the A operand straight from tensor memory.  The row
// reference is the maximum of the row's first 16 logits and is only raised when the exponentials
// of a later piece sum to more than 2^15 (so P stays inside fp16); raising it rescales, in place, the P
// columns of the current tile, the O columns and the running sum.  So in the common case a softmax
// warp hands P over and goes straight on to the next tile, whose S already waits in the other
// buffer: the only hand-off per tile is "P of tile u written" -> the issuer queues O += P V and,
// into the buffer P V frees, S of tile u+2 (the tensor pipe keeps their order).  The N x N x N
// logits and probabilities never exist outside tensor memory.
//
// What bounds the kernel is the softmax warps' per-tile chain, not a pipe: every shared-memory or
// tensor-memory round trip in it (barrier test, tcgen05.ld / st, wait) queues behind the exponentials
// the other warps have in flight.  So the chain is kept to the waits it cannot do without ("S is
// there" implies the K/V stage and its mask terms; "P V landed" is waited once per item), and the two
// query tiles take turns at the exponentials so that one pair of streams computes while the other
// stores and loads.  Computing part of the exponentials on the FMA pipe (a polynomial 2^x) was
// measured and is slower: the kernel is short of issue slots before it is short of the exponent unit.
//
// Warp roles: warp w < 16: softmax of stream w / 4 (TMEM lane quadrant = w % 4); 16: TMA producer
// of Q, K, V and the mask terms; 17 / 18: MMA issuers of streams 0-1 / 2-3, each handling its two
// streams together (17 owns the TMEM allocation); 19: TMA producer of the bias tiles (one ring
// per issuer).
#include <cuda.h>

#include "tc05.cuh"
#include "tc_kernels.cuh"

namespace tc {

using namespace tc05;

constexpr int FA_THREADS = 20 * 32;
constexpr int FA_TILE = 128;                        // query rows per stream
constexpr int FA_KT = 48;                           // keys per tile
constexpr int FA_STAGES = 5;                        // K/V ring
constexpr int FA_Q_BYTES = FA_TILE * 128;           // per query tile: 128 rows x (2 heads x 32 x 2 B)
constexpr int FA_KV_BYTES = FA_KT * 128;            // K or V of one tile, both heads
constexpr int FA_BIAS_BYTES = FA_TILE * 64 * 2;     // one stream's bias tile: 128 queries x 64 keys fetched (48 used), fp16
constexpr int FA_BIAS_SLOTS = 2;                    // per issuer; a slot holds the tiles of both its streams
constexpr int FA_IDENT_BYTES = 2048;                // 16 x 16 identity, 128-byte swizzled rows
constexpr int FA_SMEM = 2 * FA_Q_BYTES + FA_STAGES * 2 * FA_KV_BYTES + 2 * FA_BIAS_SLOTS * 2 * FA_BIAS_BYTES +
                        FA_IDENT_BYTES + FA_STAGES * FA_KT * 4 + 512 + 1024;
// Register budget: the CTA starts with 20 warps x 96 registers, and setmaxnreg trades inside the CTA's
// own allocation: 16 softmax warps x 104 + 4 service warps x 64 = 20 x 96.
constexpr uint32_t FA_REGS_SOFTMAX = 104, FA_REGS_SERVICE = 64;
constexpr int FA_O_COL = 2 * FA_KT;                 // O accumulator columns inside a stream's region, after the two S / P buffers

struct FlashParams {
  int batch, Q, qtiles, qpairs, ktiles;
  int transpose, mask_mode, clamp;
  const float* mask;       // b*Q + j, or j*batch + b when transpose
  int has_bias, ldb;       // the bias [4][Q][ldb] fp16 arrives through its tensor map
  int ldq;                 // rows per batch row of q, k, v, gate, out (Q rounded up to 16)
  const op16* gate;        // sigmoid(gate), in 8 x 8 pieces like q: element (b, q, c) at b*ldq*128 + (q/8)*1024 + (c/8)*64 + (q%8)*8 + c%8
  op16* out;               // same layout
  Status* status;
};

__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}


__global__ void __launch_bounds__(FA_THREADS, 1)
flash_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
             const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapB, const FlashParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                                    // [2 query tiles]
  uint8_t* sK = sQ + 2 * FA_Q_BYTES;                     // [stage]
  uint8_t* sV = sK + FA_STAGES * FA_KV_BYTES;            // [stage]
  uint8_t* sBias = sV + FA_STAGES * FA_KV_BYTES;         // [issuer][slot]
  uint8_t* sIdent = sBias + 2 * FA_BIAS_SLOTS * 2 * FA_BIAS_BYTES;
  float* sMask = reinterpret_cast<float*>(sIdent + FA_IDENT_BYTES);   // [stage][64] additive key terms
  uint64_t* bars = reinterpret_cast<uint64_t*>(sMask + FA_STAGES * FA_KT);
  uint64_t* q_full = bars;           // 1
  uint64_t* q_empty = bars + 1;      // count 2: one commit per issuer
  uint64_t* kv_full = bars + 2;      // [stage] count 2: TMA bytes + mask terms
  uint64_t* kv_empty = kv_full + FA_STAGES;     // [stage] count 2: one commit per issuer
  uint64_t* s_full = kv_empty + FA_STAGES;      // [issuer][buffer]: S of both its streams is there
  uint64_t* p_full = s_full + 4;     // [issuer][buffer] count 8: the eight softmax warps of its two streams
  uint64_t* o_full = p_full + 4;     // [issuer] one phase per item: the last P V of both streams has landed
  uint64_t* b_full = o_full + 2;     // [issuer][slot]
  uint64_t* b_empty = b_full + 2 * FA_BIAS_SLOTS;     // [issuer][slot]
  uint64_t* turn = b_empty + 2 * FA_BIAS_SLOTS;        // [query tile] count 8: the other tile's softmax warps are through their exponentials
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(turn + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* mask_flag = abort_flag + 1;      // [stage]: the stage has a non-zero term

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t items = (int64_t)p.batch * p.qpairs * 2;
  const int T = p.ktiles;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 2);
    for (int s = 0; s < FA_STAGES; ++s) { mbar_init(&kv_full[s], 2); mbar_init(&kv_empty[s], 2); }
    for (int i = 0; i < 4; ++i) { mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 8); }
    for (int i = 0; i < 2; ++i) mbar_init(&o_full[i], 1);
    for (int i = 0; i < 2 * FA_BIAS_SLOTS; ++i) { mbar_init(&b_full[i], 1); mbar_init(&b_empty[i], 1); }
    for (int i = 0; i < 2; ++i) mbar_init(&turn[i], 8);
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

  // The 16 softmax warps (warpgroups 0-3) hold a tile's logits and probabilities in registers; the
  // producer and issuer warps (warpgroup 4) need few and hand theirs over.  Each role's code follows
  // its own setmaxnreg, which is what the register allocator goes by.
  if (warp >= 16) {
  reg_dec<FA_REGS_SERVICE>();
  if (warp == 16) {
    // ---------------- TMA producer of Q, K, V + mask terms ----------------
    if (lane == 0) { prefetch_tensormap(&mapQ); prefetch_tensormap(&mapK); prefetch_tensormap(&mapV); }
    uint32_t n_item = 0, n_kv = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x, ++n_item) {
      const int hp = (int)(item & 1);
      const int qp = (int)((item >> 1) % p.qpairs);
      const int b = (int)((item >> 1) / p.qpairs);
      if (lane == 0) {
        if (!mbar_wait_parked(q_empty, (n_item & 1) ^ 1, abort_flag, p.status, 20)) ok = false;
        else {
          mbar_expect_tx(q_full, 2 * FA_Q_BYTES);
          // coordinates: channel and row inside a piece, piece along channels (8 per head pair), piece along rows, batch row
          tma_load_5d(sQ, &mapQ, q_full, 0, 0, hp * 8, (2 * qp) * (FA_TILE / 8), b);
          tma_load_5d(sQ + FA_Q_BYTES, &mapQ, q_full, 0, 0, hp * 8, (2 * qp + 1) * (FA_TILE / 8), b);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      for (int t = 0; t < T && ok; ++t, ++n_kv) {
        const int st = n_kv % FA_STAGES;
        if (lane == 0) {
          if (!mbar_wait(&kv_empty[st], ((n_kv / FA_STAGES) & 1) ^ 1, abort_flag, p.status, 21)) ok = false;   // not parked: the ring is only a few tiles deep
          else {
            mbar_expect_tx(&kv_full[st], 2 * FA_KV_BYTES);
            tma_load_5d(sK + st * FA_KV_BYTES, &mapK, &kv_full[st], 0, 0, hp * 8, t * (FA_KT / 8), b);
            tma_load_5d(sV + st * FA_KV_BYTES, &mapV, &kv_full[st], 0, 0, hp * 8, t * (FA_KT / 8), b);
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        // additive key terms for this tile: 2 keys per lane, lanes 0..23
        bool any = false;
        float term[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int j = t * FA_KT + lane * 2 + e;
          float v = -INFINITY;
          if (lane * 2 < FA_KT && j < p.Q) {
            const float m = p.mask[p.transpose ? (int64_t)j * p.batch + b : (int64_t)b * p.Q + j];
            v = p.mask_mode == 0 ? 1e9f * (m - 1.0f) : (m > 0.f ? 0.f : -1e9f);
          }
          term[e] = v;
          any = any || (lane * 2 < FA_KT && v != 0.f);
        }
        if (lane * 2 < FA_KT) *reinterpret_cast<float2*>(sMask + st * FA_KT + lane * 2) = make_float2(term[0], term[1]);
        const unsigned ballot = __ballot_sync(0xffffffffu, any);
        __syncwarp();   // orders every lane's term stores before the publishing arrive
        if (lane == 0) { mask_flag[st] = ballot != 0; mbar_arrive(&kv_full[st]); }
      }
    }
  } else if (warp == 19) {
    // ---------------- bias tiles: per issuer a ring of slots, each the tiles of its two streams for one key tile ----------------
    if (lane == 0 && p.has_bias) {
      prefetch_tensormap(&mapB);
      uint32_t slot = 0, par = 1;      // both rings advance together
      bool ok = true;
      for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
        const int hp = (int)(item & 1);
        const int qp = (int)((item >> 1) % p.qpairs);
        for (int t = 0; t < T && ok; ++t) {
          for (int ring = 0; ring < 2 && ok; ++ring) {
            const uint32_t bs = ring * FA_BIAS_SLOTS + slot;
            if (!mbar_wait_parked(&b_empty[bs], par, abort_flag, p.status, 22)) { ok = false; break; }
            const int q0 = (2 * qp + ring) * FA_TILE;
            // no copy starts outside the tensor: a query tile past the last row is not fetched, and
            // the issuer leaves its bias steps out
            if (q0 >= p.Q) { mbar_arrive(&b_full[bs]); continue; }
            mbar_expect_tx(&b_full[bs], 2 * FA_BIAS_BYTES);
            tma_load_3d(sBias + bs * 2 * FA_BIAS_BYTES, &mapB, &b_full[bs], t * FA_KT, q0, hp * 2);
            tma_load_3d(sBias + bs * 2 * FA_BIAS_BYTES + FA_BIAS_BYTES, &mapB, &b_full[bs], t * FA_KT, q0, hp * 2 + 1);
          }
          if (++slot == FA_BIAS_SLOTS) { slot = 0; par ^= 1; }
        }
      }
    }
  } else if (warp == 17 || warp == 18) {
    // ---------------- MMA issuers: warp 17 streams 0,1 (query tile 0), warp 18 streams 2,3 ----------------
    // Per key tile u, once the eight softmax warps of the issuer's two streams have written P:
    // O += P V for both streams, then at once S of tile u + 2 = Q K^T (+ bias) into the buffer the
    // P V frees; the tensor pipe runs them in issue order, so the new S never overtakes the P it
    // replaces.  S of tile u + 1 is already in the other buffer.  The whole warp runs the loop
    // (uniform control flow and uniform operand values); one elected lane issues.
    {
      const int w = warp - 17;         // = query tile g of both streams
      constexpr uint32_t idesc_qk = make_idesc_f16(FA_TILE, FA_KT, 0, 0);     // S[q][k], both K-major
      constexpr uint32_t idesc_pv = make_idesc_f16(FA_TILE, 32, 0, 1);        // O[q][d]: P K-major, V MN-major
      constexpr uint32_t idesc_b = make_idesc_f16(FA_TILE, 16, 0, 0);         // S[:, 16 keys] += bias[:, 16 keys] I
      const uint64_t ident_desc = make_smem_desc(smem_u32(sIdent), 16, 1024);
      const uint32_t q_addr = smem_u32(sQ + w * FA_Q_BYTES);
      const uint32_t d0 = tmem_base + (w * 2) * FA_TILE;      // stream h at d0 + h * FA_TILE
      const bool has_bias = p.has_bias != 0;
      uint32_t my_items = 0;
      for (int64_t item = blockIdx.x; item < items; item += gridDim.x) ++my_items;
      const uint32_t U = my_items * (uint32_t)T;      // key tiles this CTA walks through, all items
      bool ok = true;

      // Running position of the next Q K^T (tiles are issued in order, so nothing is divided): tile
      // within the item, item parity, K/V stage and its phase, bias slot and its phase, and whether
      // the item's query tile has any row (else its bias was not fetched).
      uint32_t qk_t = 0, qk_item = blockIdx.x, qk_itpar = 0, qk_st = 0, qk_stpar = 0, qk_bslot = 0, qk_bpar = 0;
      auto q_tile_valid = [&](uint32_t item) { return (int)(2 * ((item >> 1) % (uint32_t)p.qpairs) + w) * FA_TILE < p.Q; };
      bool qk_valid = q_tile_valid(blockIdx.x);

      // waits for what S of the next tile reads
      auto qk_ready = [&]() -> bool {
        if (qk_t == 0 && !mbar_wait(q_full, qk_itpar, abort_flag, p.status, 30)) return false;
        if (!mbar_wait(&kv_full[qk_st], qk_stpar, abort_flag, p.status, 31)) return false;
        if (has_bias && !mbar_wait(&b_full[w * FA_BIAS_SLOTS + qk_bslot], qk_bpar, abort_flag, p.status, 32)) return false;
        return true;
      };
      // S of the next tile u for both streams into buffer u & 1 (elected lane only)
      auto qk_issue = [&](uint32_t u) {
        const uint32_t k_addr = smem_u32(sK + qk_st * FA_KV_BYTES);
        const uint32_t bs = w * FA_BIAS_SLOTS + qk_bslot;
        // key groups past the padded row and query tiles past the last row were not fetched
        const int groups = qk_valid ? min(FA_KT / 16, (p.ldb - (int)qk_t * FA_KT) >> 4) : 0;   // ldb is a multiple of 16
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t d = d0 + h * FA_TILE + (u & 1) * FA_KT;
#pragma unroll
          for (int kk = 0; kk < 2; ++kk) {
            // unswizzled K-major tiles [rows / 8][8 pieces][8 rows][16 B]: a head is 4 pieces (512 B), a k-step 2 pieces
            const uint64_t adesc = make_smem_desc_plain(q_addr + h * 512 + kk * 256, 128, 1024);
            const uint64_t bdesc = make_smem_desc_plain(k_addr + h * 512 + kk * 256, 128, 1024);
            umma_f16(d, adesc, bdesc, idesc_qk, kk);
          }
          if (has_bias) {
            // the tile's bias is added by the tensor core: 16 keys per step against the identity
            const uint32_t b_addr = smem_u32(sBias + (bs * 2 + h) * FA_BIAS_BYTES);
#pragma unroll
            for (int kk = 0; kk < FA_KT / 16; ++kk) {
              if (kk >= groups) break;
              const uint64_t adesc = make_smem_desc(b_addr + kk * 32, 16, 1024);
              umma_f16(d + kk * 16, adesc, ident_desc, idesc_b, 1);
            }
          }
        }
        if (has_bias) umma_commit(&b_empty[bs]);
        umma_commit(&s_full[w * 2 + (u & 1)]);
        if (qk_t + 1 == (uint32_t)T) umma_commit(q_empty);    // this issuer is done with the item's Q
      };
      auto qk_advance = [&]() {
        if (++qk_bslot == FA_BIAS_SLOTS) { qk_bslot = 0; qk_bpar ^= 1; }
        if (++qk_st == FA_STAGES) { qk_st = 0; qk_stpar ^= 1; }
        if (qk_t + 1 == (uint32_t)T) {
          qk_t = 0; qk_itpar ^= 1; qk_item += gridDim.x;
          qk_valid = q_tile_valid(qk_item);
        } else {
          ++qk_t;
        }
      };

      for (uint32_t u0 = 0; u0 < 2 && u0 < U && ok; ++u0) {
        ok = qk_ready();
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) qk_issue(u0);
        __syncwarp();
        qk_advance();
      }
      uint32_t pv_t = 0;
      for (uint32_t u = 0; u < U && ok; ++u) {
        const int st = u % FA_STAGES;
        const bool more = u + 2 < U;
        if (!mbar_wait(&p_full[w * 2 + (u & 1)], (u >> 1) & 1, abort_flag, p.status, 33)) { ok = false; break; }
        if (more && !qk_ready()) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + st * FA_KV_BYTES);
        if (elect_one()) {
          // P is the A operand straight from tensor memory: 16 keys per step = 8 packed columns.
          // The first tile of an item overwrites O: every softmax warp has read the previous item's
          // O before it wrote this P.
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t d = d0 + h * FA_TILE;
            const uint32_t pbuf = d + (u & 1) * FA_KT;
#pragma unroll
            for (int kk = 0; kk < FA_KT / 16; ++kk) {
              // V as the MN-major operand: a piece is 8 keys x 8 channels; 16 keys per step = two row groups (2048 B)
              const uint64_t bdesc = make_smem_desc_plain(v_addr + h * 512 + kk * 2048, 1024, 128);
              umma_f16_ts(d + FA_O_COL, pbuf + kk * 8, bdesc, idesc_pv, (pv_t != 0 || kk != 0) ? 1u : 0u);
            }
          }
          if (pv_t + 1 == (uint32_t)T) umma_commit(&o_full[w]);     // one phase per item: its last P V has landed
          umma_commit(&kv_empty[st]);      // this issuer's streams are done with the stage
          if (more) qk_issue(u + 2);       // into the buffers these P V steps free
        }
        __syncwarp();
        if (more) qk_advance();
        if (++pv_t == (uint32_t)T) pv_t = 0;
      }
    }
  }
  } else {
    reg_inc<FA_REGS_SOFTMAX>();
    // ---------------- softmax: one thread per query row of one stream ----------------
    const int sidx = warp >> 2, q = warp & 3;
    const int g = sidx >> 1, h = sidx & 1;
    const int row = q * 32 + lane;
    const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + sidx * FA_TILE;
    const float L2E = 1.4426950408889634f;
    constexpr float kBig = 32768.0f;    // a piece whose 16 exponentials sum to at most this has every P < 2^15
    uint32_t n_tile = 0, n_item = 0;
    bool ok = true;
    for (int64_t item = blockIdx.x; item < items && ok; item += gridDim.x) {
      const int hp = (int)(item & 1);
      const int qp = (int)((item >> 1) % p.qpairs);
      const int b = (int)((item >> 1) / p.qpairs);
      const int head = hp * 2 + h;
      const int qi = (2 * qp + g) * FA_TILE + row;
      const bool qvalid = qi < p.Q;
      float m_ref = 0.f, neg = 0.f, l_run = 0.f;
      for (int t = 0; t < T && ok; ++t, ++n_tile) {
        const int st = n_tile % FA_STAGES;
        const uint32_t sbuf = acc + (n_tile & 1) * FA_KT;
        if (!mbar_wait(&s_full[g * 2 + (n_tile & 1)], (n_tile >> 1) & 1, abort_flag, p.status, 40)) { ok = false; break; }
        // The key terms of this stage were published through kv_full, which the issuer waited for before it
        // queued this S: S being there implies them, and this warp spares itself the wait.  (Every wait in
        // this loop costs far more than its instructions: its shared-memory round trip queues behind the
        // other warps' exponentials, so the loop keeps to the waits it cannot do without.)
        tc_fence_after();
        const bool masked = mask_flag[st] != 0;
        // The tile's 48 S columns go to registers; the three 16-key pieces are then independent chains
        // (mask terms, exponentials, sums) that the scheduler interleaves, and one vote per tile decides
        // whether the row reference has to be raised.  P is stored only after that, so the rare slow
        // path can read S again.
        uint32_t s0[16], s1[16], s2[16];
        auto load_s = [&]() {
          tmem_ld16(sbuf, s0);
          tmem_ld16(sbuf + 16, s1);
          tmem_ld16(sbuf + 32, s2);
          tmem_ld_wait();
          if (masked) {
            auto add_terms = [&](uint32_t (&su)[16], const int c) {
              const float4* mt = reinterpret_cast<const float4*>(sMask + st * FA_KT + c * 16);
#pragma unroll
              for (int j4 = 0; j4 < 4; ++j4) {
                const float4 m = mt[j4];
                su[j4 * 4] = __float_as_uint(__uint_as_float(su[j4 * 4]) + m.x);
                su[j4 * 4 + 1] = __float_as_uint(__uint_as_float(su[j4 * 4 + 1]) + m.y);
                su[j4 * 4 + 2] = __float_as_uint(__uint_as_float(su[j4 * 4 + 2]) + m.z);
                su[j4 * 4 + 3] = __float_as_uint(__uint_as_float(su[j4 * 4 + 3]) + m.w);
              }
              if (p.clamp) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {   // keys past the end stay at -inf: they are not keys at all
                  const float v = __uint_as_float(su[e]);
                  su[e] = __float_as_uint(v == -INFINITY ? v : fminf(fmaxf(v, -1e8f), 1e8f));
                }
              }
            };
            add_terms(s0, 0);
            add_terms(s1, 1);
            add_terms(s2, 2);
          }
        };
        auto piece_max = [&](const uint32_t (&su)[16]) {
          float mx[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) mx[e] = fmaxf(__uint_as_float(su[e]), __uint_as_float(su[e + 8]));
          return fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
        };
        // float32 exponentials: the packed fp16 form (ex2.approx.f16x2) measured slower per element, and
        // handing the exponent unit from warp to warp in turn (to keep the four warps of a scheduler out
        // of step) measured no gain - the wake-up costs what the stagger saves
        auto exponentials = [&](const uint32_t (&su)[16], uint32_t (&w)[8]) {
          float ps[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float p0 = ex2f(fmaf(__uint_as_float(su[2 * e]), L2E, neg));
            const float p1 = ex2f(fmaf(__uint_as_float(su[2 * e + 1]), L2E, neg));
            ps[e] = p0 + p1;
            w[e] = pack_half2(p0, p1);
          }
          return ((ps[0] + ps[1]) + (ps[2] + ps[3])) + ((ps[4] + ps[5]) + (ps[6] + ps[7]));
        };
        load_s();
        if (t == 0) {
          m_ref = fmaxf(piece_max(s0), fmaxf(piece_max(s1), piece_max(s2)));   // key 0 exists, so this is finite
          neg = -m_ref * L2E;
        }
        uint32_t w0[8], w1[8], w2[8];
        // The two query tiles take turns at the exponentials: tile 1's warps start a key tile's
        // exponentials when tile 0's are through theirs, and the other way round for the next key tile,
        // so that on every scheduler two warps have the exponent unit while the other two store, hand
        // over, wait and load.  (Without the turns the four warps of a scheduler fall into step.)
        if (!mbar_wait(&turn[g], (g ^ 1 ^ n_tile) & 1, abort_flag, p.status, 45)) { ok = false; break; }
        tie48(s0, s1, s2);
        float a0 = exponentials(s0, w0), a1 = exponentials(s1, w1), a2 = exponentials(s2, w2);
        tie24(w0, w1, w2);
        __syncwarp();
        if (lane == 0) mbar_arrive(&turn[g ^ 1]);
        // The sum of a piece's 16 exponentials bounds each of them: while it stays below kBig every P is
        // far inside fp16 and the row reference is left alone (no maximum is searched at all).
        const bool over = !(a0 <= kBig) || !(a1 <= kBig) || !(a2 <= kBig);
        if (__any_sync(0xffffffffu, over)) {
          // Rare: raise the reference of the rows that need it to their maximum so far; rescale their O
          // columns (once the P V steps so far have landed) and their running sum; then redo the tile.
          load_s();
          const float m_up = over ? fmaxf(m_ref, fmaxf(piece_max(s0), fmaxf(piece_max(s1), piece_max(s2)))) : m_ref;
          const float f = ex2f((m_ref - m_up) * L2E);       // 1 for the rows that are fine
          if (t > 0) {
            // P V of every earlier tile of the item has landed once both issuers have released the
            // previous tile's K/V stage
            if (!mbar_wait(&kv_empty[(n_tile - 1) % FA_STAGES], ((n_tile - 1) / FA_STAGES) & 1, abort_flag, p.status, 43)) ok = false;
            tc_fence_after();
            if (ok) {
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                uint32_t o[16];
                tmem_ld16(acc + FA_O_COL + half * 16, o);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
                tmem_st16(acc + FA_O_COL + half * 16, o);
              }
            }
          }
          l_run *= f;
          m_ref = m_up;
          neg = -m_ref * L2E;
          a0 = exponentials(s0, w0);
          a1 = exponentials(s1, w1);
          a2 = exponentials(s2, w2);
        }
        l_run += (a0 + a1) + a2;
        tmem_st8(sbuf, w0);          // keys c*16 .. +15 -> columns c*8 .. +7
        tmem_st8(sbuf + 8, w1);
        tmem_st8(sbuf + 16, w2);
        if (!ok) break;
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[g * 2 + (n_tile & 1)]);
      }
      if (!ok) break;
      // the item's last P V has landed: normalise, gate, store
      if (!mbar_wait(&o_full[g], n_item & 1, abort_flag, p.status, 42)) { ok = false; break; }
      ++n_item;
      tc_fence_after();
      {
        uint32_t o[32];
        tmem_ld32(acc + FA_O_COL, o);
        tmem_ld_wait();
        if (qvalid) {
          // the head's 32 channels are four 8-channel pieces of this row, 64 elements apart
          const int64_t r = (int64_t)b * p.ldq * 128 + (int64_t)(qi >> 3) * 1024 + head * 256 + (qi & 7) * 8;
          const float inv = 1.0f / l_run;
          const op16* gsrc = p.gate + r;
          op16* dst = p.out + r;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t pk[8];
            const uint4 ga = *reinterpret_cast<const uint4*>(gsrc + c * 128), gb = *reinterpret_cast<const uint4*>(gsrc + c * 128 + 64);
            const uint32_t gw[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float2 gf = __half22float2(*reinterpret_cast<const __half2*>(&gw[e]));
              pk[e] = pack_half2(__uint_as_float(o[c * 16 + e * 2]) * inv * gf.x, __uint_as_float(o[c * 16 + e * 2 + 1]) * inv * gf.y);
            }
            *reinterpret_cast<uint4*>(dst + c * 128) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *reinterpret_cast<uint4*>(dst + c * 128 + 64) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
          }
        }
      }
      tc_fence_before();   // the O read is ordered before this warp's next "P written" arrive
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
lf_status make_map_tiled_act(lf_context* ctx, CUtensorMap* map, const void* base, int ldq, int batch, int rows);

lf_status attention_core(lf_context* ctx, ArenaCursor& cur, const op16* q, const op16* k, const op16* v, const op16* g,
                         const op16* bias, int ldb, const float* mask, int batch, int Q, int transpose,
                         int mask_mode, int clamp, op16* out) {
  if (cur.dry) return LF_OK;
  CUtensorMap mq, mk, mv, mb;
  const int ldq = (Q + 15) / 16 * 16;
  LF_TRY(make_map_tiled_act(ctx, &mq, q, ldq, batch, FA_TILE));
  LF_TRY(make_map_tiled_act(ctx, &mk, k, ldq, batch, FA_KT));
  LF_TRY(make_map_tiled_act(ctx, &mv, v, ldq, batch, FA_KT));
  // bias [4][Q][ldb]: boxes of 64 keys x 128 queries; without a bias the map is a stand-in that is never used
  if (bias) LF_TRY(make_map_f16_3d_ext(ctx, &mb, bias, ldb, Q, 4, (uint64_t)ldb * 2, (uint64_t)Q * ldb * 2, 64, FA_TILE));
  else mb = mq;
  FlashParams p{};
  p.batch = batch; p.Q = Q; p.qtiles = (Q + FA_TILE - 1) / FA_TILE; p.qpairs = (p.qtiles + 1) / 2; p.ktiles = (Q + FA_KT - 1) / FA_KT;
  p.transpose = transpose; p.mask_mode = mask_mode; p.clamp = clamp; p.mask = mask; p.has_bias = bias ? 1 : 0; p.ldb = ldb; p.ldq = ldq;
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
