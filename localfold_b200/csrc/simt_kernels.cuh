// Float32 SIMT kernels: the precision-"f32" path of every operator and the
// generic-shape path behind the tensor-core kernels.  All accumulation is
// float32 FMA; statistics use warp-shuffle reductions.
#pragma once

#include "common.cuh"

namespace simt {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f<bf16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float sigmoidf_(float v) { return 1.0f / (1.0f + expf(-v)); }

// o[0..7] = v[0..7] (+ r[0..7] when r is given): 16-byte accesses for float32 activations
template <typename TAct>
__device__ __forceinline__ void add_store8(float (&v)[8], const TAct* r, TAct* o) {
  if (sizeof(TAct) == 4) {
    if (r) {
      const float4 r0 = *reinterpret_cast<const float4*>(r), r1 = *reinterpret_cast<const float4*>(r + 4);
      v[0] += r0.x; v[1] += r0.y; v[2] += r0.z; v[3] += r0.w;
      v[4] += r1.x; v[5] += r1.y; v[6] += r1.z; v[7] += r1.w;
    }
    *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    if (r) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] += to_f(r[e]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = from_f<TAct>(v[e]);
  }
}

// ---------------------------------------------------------------------------
// LayerNorm over the last axis, one warp per row.  `rows` logical rows; logical
// row r = b*Q + i reads memory row i*batch + b when `transpose` (batch, Q > 0).
// variance: 1 two-pass, 2 fast (E[x^2]-E[x]^2, unclamped).
// PAD16: the output rows are ch + 16 long, a one and fifteen zeros after the channels (the k column through which a
// GEMM that follows adds its bias)
template <typename TIn, typename TOut = float, bool PAD16 = false>
__global__ void layer_norm_kernel(const TIn* __restrict__ in, int64_t rows, int ch,
                                  const float* __restrict__ gamma, const float* __restrict__ beta,
                                  float eps, int variance, int transpose, int batch, int Q,
                                  TOut* __restrict__ out) {
  int lane = threadIdx.x & 31;
  int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  int64_t src = row;
  if (transpose) { int64_t b = row / Q, i = row % Q; src = i * batch + b; }
  const TIn* x = in + src * ch;
  float s = 0.f, ss = 0.f;
  for (int c = lane; c < ch; c += 32) { float v = to_f(x[c]); s += v; ss += v * v; }
  s = warp_sum(s);
  float mean = s / ch, var;
  if (variance == 2) {
    ss = warp_sum(ss);
    var = ss / ch - mean * mean;
  } else {
    float acc = 0.f;
    for (int c = lane; c < ch; c += 32) { float d = to_f(x[c]) - mean; acc += d * d; }
    var = warp_sum(acc) / ch;
  }
  float inv = rsqrtf(var + eps);
  // one Newton step: rsqrtf is 2 ulp, the parity bar is tighter than that squared error allows
  inv = inv * (1.5f - 0.5f * (var + eps) * inv * inv);
  TOut* y = out + row * (PAD16 ? ch + 16 : ch);
  for (int c = lane; c < ch; c += 32) y[c] = from_f<TOut>((to_f(x[c]) - mean) * inv * gamma[c] + beta[c]);
  if (PAD16 && lane < 16) y[ch + lane] = from_f<TOut>(lane == 0 ? 1.f : 0.f);
}

// ---------------------------------------------------------------------------
// Tiled SGEMM, batched over blockIdx.z:  C[m][n] = epi(sum_k A(m,k) B(k,n) + bias[n])
//   A(m,k) = TA ? A[k*lda + m] : A[m*lda + k]
//   B(k,n) = TB ? B[n*ldb + k] : B[k*ldb + n]
// 64x64x16 tile, 256 threads, 4x4 micro-tile, every load and store bounds-checked.
enum { EPI_NONE = 0, EPI_RELU = 1, EPI_SIGMOID_FROM_COL = 2 };

template <bool TA, bool TB, int EPI>
__global__ void __launch_bounds__(256)
sgemm_kernel(int M, int N, int K, const float* __restrict__ A, int64_t lda, int64_t strideA,
             const float* __restrict__ B, int64_t ldb, int64_t strideB, float* __restrict__ C,
             int64_t ldc, int64_t strideC, const float* __restrict__ bias, int epi_col0) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  A += (int64_t)blockIdx.z * strideA;
  B += (int64_t)blockIdx.z * strideB;
  C += (int64_t)blockIdx.z * strideC;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  const int t = threadIdx.x;
  const int tx = t & 15, ty = t >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      int idx = t + 256 * r;
      int m, k;
      if (TA) { m = idx & 63; k = idx >> 6; } else { k = idx & 15; m = idx >> 4; }
      int gm = m0 + m, gk = k0 + k;
      float v = 0.f;
      if (gm < M && gk < K) v = TA ? A[(int64_t)gk * lda + gm] : A[(int64_t)gm * lda + gk];
      As[k][m] = v;
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      int idx = t + 256 * r;
      int n, k;
      if (TB) { k = idx & 15; n = idx >> 4; } else { n = idx & 63; k = idx >> 6; }
      int gn = n0 + n, gk = k0 + k;
      float v = 0.f;
      if (gn < N && gk < K) v = TB ? B[(int64_t)gn * ldb + gk] : B[(int64_t)gk * ldb + gn];
      Bs[k][n] = v;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= N) continue;
      float v = acc[i][j] + (bias ? bias[gn] : 0.f);
      if (EPI == EPI_RELU) v = fmaxf(v, 0.f);
      if (EPI == EPI_SIGMOID_FROM_COL) { if (gn >= epi_col0) v = sigmoidf_(v); }
      C[(int64_t)gm * ldc + gn] = v;
    }
  }
}

// ---------------------------------------------------------------------------
// Triangle multiplication glue.
// p4: [pairs][4c] = (ap | ag | bp | bg).  a[h][p] = mask[p] * ap * sigmoid(ag), b likewise,
// channel-major with row stride ld >= n (plane = n*ld elements).  32x32 tile transpose
// through shared memory so both sides coalesce.
template <typename TOut>
__global__ void trimul_gate_kernel(const float* __restrict__ p4, const float* __restrict__ mask,
                                   int64_t pairs, int c, int n, int ld, TOut* __restrict__ a, TOut* __restrict__ b) {
  __shared__ float ta[32][33];
  __shared__ float tb[32][33];
  int64_t p0 = (int64_t)blockIdx.x * 32;
  int h0 = blockIdx.y * 32;
  int tx = threadIdx.x, ty = threadIdx.y;   // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    int64_t p = p0 + r;
    int h = h0 + tx;
    float va = 0.f, vb = 0.f;
    if (p < pairs && h < c) {
      const float* row = p4 + p * 4 * c;
      float m = mask[p];
      va = row[h] * sigmoidf_(row[c + h]) * m;
      vb = row[2 * c + h] * sigmoidf_(row[3 * c + h]) * m;
    }
    ta[r][tx] = va;
    tb[r][tx] = vb;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    int h = h0 + r;
    int64_t p = p0 + tx;
    if (h < c && p < pairs) {
      int64_t o = ((int64_t)h * n + p / n) * ld + p % n;
      a[o] = from_f<TOut>(ta[tx][r]);
      b[o] = from_f<TOut>(tb[tx][r]);
    }
  }
}

// LayerNorm over the hidden channel of a channel-major tensor x[h][i][ld] -> xn[p][h].
// One block handles 32 pairs; the tile [c][32] sits in shared memory (c <= 512).
template <typename TIn>
__global__ void center_norm_kernel(const TIn* __restrict__ x, int64_t pairs, int c, int n, int ld,
                                   const float* __restrict__ gamma, const float* __restrict__ beta,
                                   float eps, int variance, float prescale, float* __restrict__ xn) {
  extern __shared__ float tile[];   // [c][33]
  int64_t p0 = (int64_t)blockIdx.x * 32;
  int tx = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int h = w; h < c; h += nw) {
    int64_t p = p0 + tx;
    tile[h * 33 + tx] = p < pairs ? to_f(x[((int64_t)h * n + p / n) * ld + p % n]) * prescale : 0.f;
  }
  __syncthreads();
  // warp w normalises pairs w, w+nw, ...
  for (int r = w; r < 32; r += nw) {
    int64_t p = p0 + r;
    if (p >= pairs) continue;
    float s = 0.f, ss = 0.f;
    for (int h = tx; h < c; h += 32) { float v = tile[h * 33 + r]; s += v; ss += v * v; }
    s = warp_sum(s);
    float mean = s / c, var;
    if (variance == 2) { ss = warp_sum(ss); var = ss / c - mean * mean; }
    else {
      float acc = 0.f;
      for (int h = tx; h < c; h += 32) { float d = tile[h * 33 + r] - mean; acc += d * d; }
      var = warp_sum(acc) / c;
    }
    float inv = rsqrtf(var + eps);
    inv = inv * (1.5f - 0.5f * (var + eps) * inv * inv);
    for (int h = tx; h < c; h += 32) xn[p * c + h] = (tile[h * 33 + r] - mean) * inv * gamma[h] + beta[h];
  }
}

// out[dst(r)][c] = (resid ? resid[dst(r)][c] : 0) + proj[r][c] * (gate ? sigmoid(gate[r][c]) : 1)
// dst(r) follows the transposed-orientation rule of the attention operator.
template <typename TAct>
__global__ void finish_kernel(const float* __restrict__ proj, const float* __restrict__ gate,
                              const TAct* __restrict__ resid, int64_t rows, int ch, int transpose,
                              int batch, int Q, TAct* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = rows * ch;
  if (idx >= total) return;
  int64_t r = idx / ch;
  int c = (int)(idx % ch);
  int64_t dst = r;
  if (transpose) { int64_t b = r / Q, i = r % Q; dst = i * batch + b; }
  float v = proj[idx];
  if (gate) v *= sigmoidf_(gate[idx]);
  if (resid) v += to_f(resid[dst * ch + c]);
  out[dst * ch + c] = from_f<TAct>(v);
}

// q, k, v, gate as four fp16 [rows][HD] tensors -> one float32 [rows][4*HD] tensor
__global__ void unpack_qkvg_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                                   const __half* __restrict__ g, int64_t rows, int HD, float* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * HD) return;
  int64_t r = idx / HD;
  int c = (int)(idx % HD);
  float* o = out + r * 4 * HD + c;
  o[0] = __half2float(q[idx]);
  o[HD] = __half2float(k[idx]);
  o[2 * HD] = __half2float(v[idx]);
  o[3 * HD] = __half2float(g[idx]);
}

template <typename TIn>
__global__ void to_float_kernel(const TIn* __restrict__ in, int64_t n, float* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = to_f(in[i]);
}

// ---------------------------------------------------------------------------
// Pair bias: out[h][dst(p)] = LN(pair[p,:]) . W[:,h] for p = i*Q + j, dst = j*Q+i if swap.
// One warp per pair row; `normalized` != 0 skips the LayerNorm (input already normalised).
template <typename TIn>
__global__ void pair_bias_kernel(const TIn* __restrict__ pair, int Q, int ch, int heads,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 const float* __restrict__ w, float eps, int variance, int normalized,
                                 int swap, float* __restrict__ out) {
  int lane = threadIdx.x & 31;
  int64_t pairs = (int64_t)Q * Q;
  int64_t p = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= pairs) return;
  const TIn* x = pair + p * ch;
  float mean = 0.f, inv = 1.f;
  if (!normalized) {
    float s = 0.f, ss = 0.f;
    for (int c = lane; c < ch; c += 32) { float v = to_f(x[c]); s += v; ss += v * v; }
    s = warp_sum(s);
    mean = s / ch;
    float var;
    if (variance == 2) { ss = warp_sum(ss); var = ss / ch - mean * mean; }
    else {
      float acc = 0.f;
      for (int c = lane; c < ch; c += 32) { float d = to_f(x[c]) - mean; acc += d * d; }
      var = warp_sum(acc) / ch;
    }
    inv = rsqrtf(var + eps);
    inv = inv * (1.5f - 0.5f * (var + eps) * inv * inv);
  }
  int64_t dst = p;
  if (swap) { int64_t i = p / Q, j = p % Q; dst = j * Q + i; }
  for (int h = 0; h < heads; ++h) {
    float acc = 0.f;
    for (int c = lane; c < ch; c += 32) {
      float v = to_f(x[c]);
      if (!normalized) v = (v - mean) * inv * gamma[c] + beta[c];
      acc = fmaf(v, w[c * heads + h], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[(int64_t)h * pairs + dst] = acc;
  }
}

// Global column attention (extra-MSA stack).  Query of a column: the masked mean over the sequences of the
// normalised rows, projected onto heads x d and scaled.  One block per column; shared memory: c floats.
__global__ void global_query_kernel(const float* __restrict__ nrm, const float* __restrict__ mask, int S, int n, int c,
                                    int HD, float scale, const float* __restrict__ wq, float* __restrict__ q) {
  extern __shared__ float means[];
  __shared__ float red[32];
  const int col = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  float count = 0.f;
  for (int s = tid; s < S; s += blockDim.x) count += mask[(int64_t)s * n + col];
  count = warp_sum(count);
  if (lane == 0) red[wid] = count;
  __syncthreads();
  float total_count = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total_count += red[w];
  const float denominator = 1e-10f + total_count;
  for (int ch = tid; ch < c; ch += blockDim.x) {
    float total = 0.f;
    for (int s = 0; s < S; ++s) total = fmaf(nrm[((int64_t)s * n + col) * c + ch], mask[(int64_t)s * n + col], total);
    means[ch] = total / denominator;
  }
  __syncthreads();
  for (int slot = tid; slot < HD; slot += blockDim.x) {
    float r = 0.f;
    for (int ch = 0; ch < c; ++ch) r = fmaf(means[ch], wq[(int64_t)ch * HD + slot], r);
    q[(int64_t)col * HD + slot] = r * scale;
  }
}

// Softmax over the sequences of q(column, head) . k(sequence, column) with masked sequences at -1e9, applied to
// the values: one block of 64 threads per (column, head), each thread an online softmax over its sequences,
// combined through shared memory.  k at columns 0..d-1 and v at d..2d-1 of rows of `ld` floats; d <= 32.
__global__ void global_attend_kernel(const float* __restrict__ q, const float* __restrict__ kv, int ld,
                                     const float* __restrict__ mask, int S, int n, int heads, int d,
                                     float* __restrict__ attended) {
  __shared__ float part_max[64], part_den[64], part_acc[64 * 32];
  const int col = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  float qv[32], acc[32];
  for (int e = 0; e < d; ++e) { qv[e] = q[((int64_t)col * heads + h) * d + e]; acc[e] = 0.f; }
  float maximum = -1e30f, den = 0.f;
  for (int s = tid; s < S; s += 64) {
    const float* row = kv + ((int64_t)s * n + col) * ld;
    float logit = 0.f;
    for (int e = 0; e < d; ++e) logit = fmaf(qv[e], row[e], logit);
    if (mask[(int64_t)s * n + col] == 0.f) logit = -1e9f;
    const float next = fmaxf(maximum, logit);
    const float prev_scale = __expf(maximum - next), weight = __expf(logit - next);
    den = den * prev_scale + weight;
    for (int e = 0; e < d; ++e) acc[e] = acc[e] * prev_scale + weight * row[d + e];
    maximum = next;
  }
  part_max[tid] = maximum;
  part_den[tid] = den;
  for (int e = 0; e < d; ++e) part_acc[tid * 32 + e] = acc[e];
  __syncthreads();
  if (tid < d) {
    float top = -1e30f;
    for (int t = 0; t < 64; ++t) top = fmaxf(top, part_max[t]);
    float dsum = 0.f, num = 0.f;
    for (int t = 0; t < 64; ++t) {
      const float w = __expf(part_max[t] - top);
      dsum += part_den[t] * w;
      num += part_acc[t * 32 + tid] * w;
    }
    attended[((int64_t)col * heads + h) * d + tid] = num / dsum;
  }
}

// gated[r][slot] = sigmoid-gate[r][slot] (columns gate0.. of rows of `ld`) * attended[column of r][slot]
__global__ void global_gate_kernel(const float* __restrict__ kvg, int ld, int gate0, const float* __restrict__ attended,
                                   int64_t rows, int n, int HD, float* __restrict__ gated) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * HD) return;
  const int64_t r = idx / HD;
  const int slot = (int)(idx % HD);
  gated[idx] = kvg[r * ld + gate0 + slot] * attended[(r % n) * HD + slot];
}

// Attention activations between the projections and the tensor-core attention core: 128 channels (four
// heads of 32) of logical rows (b, q) as fp16 8-row x 8-channel pieces, element (b, q, c) at
// b*ldq*128 + (q/8)*1024 + (c/8)*64 + (q%8)*8 + c%8.  `src` rows hold q | k | v | gate, HD columns each;
// blockIdx.y = which of the four, written to dst + blockIdx.y * kind_stride from columns kind*HD + group*128 ..;
// value = (src + bias[col]) (bias may be null), times qscale for the query, through a sigmoid for the gate.
template <typename TSrc>
__global__ void rows_to_pieces_kernel(const TSrc* __restrict__ src, int HD, int group, const float* __restrict__ bias,
                                      float qscale, int batch, int Q, int ldq, __half* __restrict__ dst, int64_t kind_stride) {
  // one thread per (row, 8-channel piece); a warp takes 8 rows x 4 pieces, which it writes as 512 contiguous bytes
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int q8 = (Q + 7) >> 3;
  if (idx >= (int64_t)batch * q8 * 128) return;
  const int kind = blockIdx.y;
  const int col0 = kind * HD + group * 128;
  const float scale = kind == 0 ? qscale : 1.0f;
  const int piece = (int)((idx >> 3) & 15);
  const int64_t rg = idx >> 7;
  const int b = (int)(rg / q8), q = (int)(rg % q8) * 8 + (int)(idx & 7);
  if (q >= Q) return;
  const int64_t r = (int64_t)b * Q + q;
  const TSrc* x = src + r * 4 * HD + col0 + piece * 8;
  float in[8];
  if (sizeof(TSrc) == 2) {      // fp16 rows: one 16-byte load
    const uint4 raw = *reinterpret_cast<const uint4*>(x);
    const __half* hx = reinterpret_cast<const __half*>(&raw);
#pragma unroll
    for (int e = 0; e < 8; ++e) in[e] = __half2float(hx[e]);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) in[e] = to_f(x[e]);
  }
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    float t = in[e];
    if (bias) t += bias[col0 + piece * 8 + e];
    t *= scale;
    v[e] = kind == 3 ? sigmoidf_(t) : t;
  }
  __half2 h[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) h[e] = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
  __half* out = dst + kind * kind_stride + (int64_t)b * ldq * 128 + (int64_t)(q >> 3) * 1024 + piece * 64 + (q & 7) * 8;
  *reinterpret_cast<uint4*>(out) = *reinterpret_cast<const uint4*>(h);
}

// ... and back: the core's output pieces into columns col0 .. col0+127 of rows of `ld` elements
template <typename TDst>
__global__ void pieces_to_rows_kernel(const __half* __restrict__ src, int batch, int Q, int ldq, int64_t ld, int col0,
                                      TDst* __restrict__ dst) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;      // the thread order of rows_to_pieces_kernel
  const int q8 = (Q + 7) >> 3;
  if (idx >= (int64_t)batch * q8 * 128) return;
  const int piece = (int)((idx >> 3) & 15);
  const int64_t rg = idx >> 7;
  const int b = (int)(rg / q8), q = (int)(rg % q8) * 8 + (int)(idx & 7);
  if (q >= Q) return;
  const int64_t r = (int64_t)b * Q + q;
  const __half* in = src + (int64_t)b * ldq * 128 + (int64_t)(q >> 3) * 1024 + piece * 64 + (q & 7) * 8;
  uint4 raw = *reinterpret_cast<const uint4*>(in);
  const __half* h = reinterpret_cast<const __half*>(&raw);
  TDst* out = dst + r * ld + col0 + piece * 8;
  if (sizeof(TDst) == 2) {      // fp16 rows: the piece's 16 bytes as they are
    *reinterpret_cast<uint4*>(out) = raw;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) out[e] = from_f<TDst>(__half2float(h[e]));
  }
}

// Glue of the 16-bit GEMM path (activations x weights on the tensor cores through the contraction kernel).
// out[dst(r)][c] = (resid ? resid[dst(r)][c] : 0) + (proj[r][c] * scale + bias[c]) for an fp16 projection;
// eight channels per thread (ch a multiple of 8)
template <typename TAct>
__global__ void finish_half_kernel(const __half* __restrict__ proj, float scale, const float* __restrict__ bias,
                                   const TAct* __restrict__ resid, int64_t rows, int ch, int transpose,
                                   int batch, int Q, TAct* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int c8 = ch >> 3;
  if (idx >= rows * c8) return;
  int64_t r = idx / c8;
  int c = (int)(idx % c8) * 8;
  int64_t dst = r;
  if (transpose) { int64_t b = r / Q, i = r % Q; dst = i * batch + b; }
  const uint4 raw = *reinterpret_cast<const uint4*>(proj + r * ch + c);
  const __half* h = reinterpret_cast<const __half*>(&raw);
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = __half2float(h[e]) * scale + (bias ? bias[c + e] : 0.f);
  const TAct* rs = resid ? resid + dst * ch + c : nullptr;
  TAct* o = out + dst * ch + c;
  add_store8<TAct>(v, rs, o);
}

// Transition hidden layer on the fp16 projection h [rows][wide] into out [rows][hidden] (out may be h when wide == hidden):
//   relu:   out[r][j] = relu(h[r][j] + b[j]), wide = hidden
//   swiglu: out[r][j] = silu(h[r][j] + b[j]) * (h[r][hidden + j] + b[hidden + j]), wide = 2 hidden
__global__ void hidden_act_half_kernel(const __half* h, const float* __restrict__ bias, int64_t rows, int hidden, int wide,
                                       int swiglu, __half* out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * hidden) return;
  int64_t r = idx / hidden;
  int j = (int)(idx % hidden);
  const __half* row = h + r * wide;
  float g = __half2float(row[j]) + (bias ? bias[j] : 0.f);
  if (swiglu) {
    float v = __half2float(row[hidden + j]) + (bias ? bias[hidden + j] : 0.f);
    out[idx] = __float2half_rn(g * sigmoidf_(g) * v);
  } else {
    out[idx] = __float2half_rn(fmaxf(g, 0.f));
  }
}

// fp16 pair bias [heads][Q][ld] (rows padded to ld) -> float32 [heads][Q][Q]
__global__ void widen_bias_kernel(const __half* __restrict__ in, int heads, int Q, int ld, float* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)heads * Q * Q;
  if (idx >= total) return;
  int k = (int)(idx % Q);
  int64_t hq = idx / Q;
  out[idx] = __half2float(in[hq * ld + k]);
}

// One key mask for every sequence of an MSA: out[s][t] = max over s' of mask[s'][t] (AF3 pair-weighted
// averaging: a token any sequence covers is a key for all of them).
__global__ void msa_key_mask_kernel(const float* __restrict__ mask, int sequences, int tokens, float* __restrict__ out) {
  int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= tokens) return;
  float largest = 0.f;
  for (int s = 0; s < sequences; ++s) largest = fmaxf(largest, mask[(int64_t)s * tokens + t]);
  for (int s = 0; s < sequences; ++s) out[(int64_t)s * tokens + t] = largest;
}

// out[i][j][b] = half[i][j][b] + half[j][i][b]: a sum over the two token orders, not a mean.
__global__ void symmetrise_sum_kernel(const float* __restrict__ half, int tokens, int bins, float* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)tokens * tokens * bins;
  if (idx >= total) return;
  int b = (int)(idx % bins);
  int64_t p = idx / bins;
  int i = (int)(p / tokens), j = (int)(p % tokens);
  out[idx] = half[idx] + half[((int64_t)j * tokens + i) * bins + b];
}

// ---------------------------------------------------------------------------
// Gated attention core, float32, online softmax.  One warp per query, 8 queries
// per block, key/value tiles of 32 rows staged in shared memory.
//   qkvg: [rows][4*HD] = (q | k | v | sigmoid(gate)) in logical row order
//   bias: [H][Q][Q] or null; mask: indexed b*Q+j, or j*batch+b when transpose
//   mask_mode 0: logit += 1e9*(m-1); 1: logit += (m > 0 ? 0 : -1e9)
//   clamp: limit the logit to +-1e8 after all terms are added
//   out: [rows][HD] = softmax(.) v * gate
__global__ void __launch_bounds__(256)
attention_kernel(const float* __restrict__ qkvg, const float* __restrict__ bias,
                 const float* __restrict__ mask, int batch, int Q, int heads, int d,
                 int transpose, int mask_mode, int clamp, float scale, float* __restrict__ out) {
  extern __shared__ float sm[];
  const int HD = heads * d;
  const int ld = 4 * HD;
  float* Ks = sm;                    // [32][d+1]
  float* Vs = Ks + 32 * (d + 1);     // [32][d+1]
  float* Qs = Vs + 32 * (d + 1);     // [8][d]
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int b = blockIdx.y, h = blockIdx.z;
  const int qi = blockIdx.x * 8 + w;
  const bool active = qi < Q;
  const int64_t rowbase = (int64_t)b * Q;
  if (active) for (int e = lane; e < d; e += 32) Qs[w * d + e] = qkvg[(rowbase + qi) * ld + h * d + e];
  float run_max = -INFINITY, run_sum = 0.f, o0 = 0.f, o1 = 0.f;
  for (int j0 = 0; j0 < Q; j0 += 32) {
    __syncthreads();
    for (int idx = threadIdx.x; idx < 32 * d; idx += 256) {
      int j = idx / d, e = idx % d;
      float kv = 0.f, vv = 0.f;
      if (j0 + j < Q) {
        const float* row = qkvg + (rowbase + j0 + j) * ld + h * d + e;
        kv = row[HD];
        vv = row[2 * HD];
      }
      Ks[j * (d + 1) + e] = kv;
      Vs[j * (d + 1) + e] = vv;
    }
    __syncthreads();
    if (!active) continue;
    int j = j0 + lane;
    float logit = -INFINITY;
    if (j < Q) {
      float dot = 0.f;
      for (int e = 0; e < d; ++e) dot = fmaf(Qs[w * d + e], Ks[lane * (d + 1) + e], dot);
      float m = mask[transpose ? (int64_t)j * batch + b : rowbase + j];
      logit = dot * scale;
      logit += mask_mode == 0 ? 1e9f * (m - 1.0f) : (m > 0.f ? 0.f : -1e9f);
      if (bias) logit += bias[((int64_t)h * Q + qi) * Q + j];
      if (clamp) logit = fminf(fmaxf(logit, -1e8f), 1e8f);
    }
    float tile_max = warp_max(logit);
    float new_max = fmaxf(run_max, tile_max);
    float corr = __expf(run_max - new_max);   // exp(-inf) = 0 on the first tile
    float p = j < Q ? expf(logit - new_max) : 0.f;
    run_sum = run_sum * corr + warp_sum(p);
    run_max = new_max;
    o0 *= corr; o1 *= corr;
    int lim = min(32, Q - j0);
    for (int jj = 0; jj < lim; ++jj) {
      float pj = __shfl_sync(0xffffffffu, p, jj);
      if (lane < d) o0 = fmaf(pj, Vs[jj * (d + 1) + lane], o0);
      if (lane + 32 < d) o1 = fmaf(pj, Vs[jj * (d + 1) + lane + 32], o1);
    }
  }
  if (!active) return;
  const float* grow = qkvg + (rowbase + qi) * ld + 3 * HD + h * d;
  float* orow = out + (rowbase + qi) * HD + h * d;
  if (lane < d) orow[lane] = o0 / run_sum * grow[lane];
  if (lane + 32 < d) orow[lane + 32] = o1 / run_sum * grow[lane + 32];
}

// ---------------------------------------------------------------------------
// Transition glue: SwiGLU over a [rows][2*inter] tensor, gate half first.
__global__ void swiglu_kernel(const float* __restrict__ wide, int64_t rows, int inter, float* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * inter) return;
  int64_t r = idx / inter;
  int i = (int)(idx % inter);
  float g = wide[r * 2 * inter + i];
  float v = wide[r * 2 * inter + inter + i];
  out[idx] = g * sigmoidf_(g) * v;
}

// ---------------------------------------------------------------------------
// Outer product mean glue.
// rows [S*N][c]: multiply every row by its mask value.
// the same into fp16 copies (operands of the tensor-core outer product)
__global__ void mask_rows_half_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ mask,
                                      int64_t rows, int c, __half* __restrict__ a16, __half* __restrict__ b16) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * c) return;
  float m = mask[idx / c];
  a16[idx] = __float2half_rn(a[idx] * m);
  b16[idx] = __float2half_rn(b[idx] * m);
}

// the fp16 projection lr [rows][2c] (left | right) + biases, masked, into the outer product's operands
__global__ void opm_split_half_kernel(const __half* __restrict__ lr, const float* __restrict__ bl, const float* __restrict__ br,
                                      const float* __restrict__ mask, int64_t rows, int c, __half* __restrict__ a16,
                                      __half* __restrict__ b16) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * c) return;
  int64_t r = idx / c;
  int a = (int)(idx % c);
  float m = mask[r];
  a16[idx] = __float2half_rn((__half2float(lr[r * 2 * c + a]) + bl[a]) * m);
  b16[idx] = __float2half_rn((__half2float(lr[r * 2 * c + c + a]) + br[a]) * m);
}

// counts[i][j] = sum_s mask[s][i] mask[s][j]
__global__ void opm_counts_kernel(const float* __restrict__ mask, int S, int N, float* __restrict__ counts) {
  // four rows i per thread: a value of column j is loaded once for four products
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int n4 = (N + 3) >> 2;
  if (idx >= (int64_t)n4 * N) return;
  const int i0 = (int)(idx / N) * 4, j = (int)(idx % N);
  int ii[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) ii[e] = i0 + e < N ? i0 + e : N - 1;
  float cnt[4] = {0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < S; ++s) {
    const float* row = mask + (int64_t)s * N;
    const float mj = row[j];
#pragma unroll
    for (int e = 0; e < 4; ++e) cnt[e] = fmaf(row[ii[e]], mj, cnt[e]);
  }
#pragma unroll
  for (int e = 0; e < 4; ++e)
    if (i0 + e < N) counts[(int64_t)(i0 + e) * N + j] = cnt[e];
}

// out[i][j][z] = (proj[(i - i0) N + j][z] * scale + bout[z]) / (eps + counts[i][j]) (+ resid), or with the bias after
// the division by max(count, 1); fp16 projection
template <typename TAct>
__global__ void opm_finish_half_kernel(const __half* __restrict__ proj, float scale, const float* __restrict__ bout,
                                       const float* __restrict__ counts, int N, int cz, int i0, int cnt, float norm_eps,
                                       int bias_after_norm, const TAct* __restrict__ resid, TAct* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;      // eight channels per thread (cz a multiple of 8)
  const int z8 = cz >> 3;
  if (idx >= (int64_t)cnt * N * z8) return;
  const int z = (int)(idx % z8) * 8;
  const int64_t pr = idx / z8;                 // (i - i0) * N + j
  const int64_t pair = (int64_t)i0 * N + pr;
  const uint4 raw = *reinterpret_cast<const uint4*>(proj + pr * cz + z);
  const __half* h = reinterpret_cast<const __half*>(&raw);
  const float count = counts[pair];
  const float inv = bias_after_norm ? 1.0f / fmaxf(count, 1.0f) : 1.0f / (norm_eps + count);
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const float t = __half2float(h[e]) * scale;
    v[e] = bias_after_norm ? t * inv + bout[z + e] : (t + bout[z + e]) * inv;
  }
  const int64_t o = pair * cz + z;
  add_store8<TAct>(v, resid ? resid + o : nullptr, out + o);
}

__global__ void mask_rows_kernel(float* __restrict__ a, float* __restrict__ b, const float* __restrict__ mask,
                                 int64_t rows, int c) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows * c) return;
  float m = mask[idx / c];
  a[idx] *= m;
  b[idx] *= m;
}

// outer: [(i - i0)*c + a][j*c + b] for i in [i0, i0+ni); out[i][j][z] =
// (sum_ab outer * wout[(a*c+b)][z] + bout[z]) / (eps + count(i,j)), + resid.
// One block per (i, group of JT columns j); thread z loops over the c*c products.
// (TOuter: float32 sums, or the tensor-core contraction's fp16 sums scaled by 1 / outer_scale)
template <typename TAct, int JT, typename TOuter>
__global__ void opm_output_kernel(const TOuter* __restrict__ outer, float outer_scale, const float* __restrict__ wout,
                                  const float* __restrict__ bout, const float* __restrict__ mask,
                                  int S, int N, int c, int cz, int i0, float norm_eps,
                                  int bias_after_norm, const TAct* __restrict__ resid,
                                  TAct* __restrict__ out) {
  extern __shared__ float sm[];     // [JT][c*c] + counts[JT]
  const int cc = c * c;
  float* tile = sm;
  float* counts = sm + JT * cc;
  const int i = i0 + blockIdx.y;
  const int j0 = blockIdx.x * JT;
  const int64_t ldo = (int64_t)N * c;
  for (int idx = threadIdx.x; idx < JT * cc; idx += blockDim.x) {
    int jj = idx / cc, ab = idx % cc, a = ab / c, b2 = ab % c;
    int j = j0 + jj;
    tile[idx] = j < N ? to_f(outer[((int64_t)(i - i0) * c + a) * ldo + (int64_t)j * c + b2]) * outer_scale : 0.f;
  }
  if (threadIdx.x < JT) {
    int j = j0 + threadIdx.x;
    float cnt = 0.f;
    if (j < N) for (int s = 0; s < S; ++s) cnt += mask[(int64_t)s * N + i] * mask[(int64_t)s * N + j];
    counts[threadIdx.x] = cnt;
  }
  __syncthreads();
  for (int z = threadIdx.x; z < cz; z += blockDim.x) {
    float acc[JT];
#pragma unroll
    for (int jj = 0; jj < JT; ++jj) acc[jj] = 0.f;
    for (int ab = 0; ab < cc; ++ab) {
      float wv = wout[(int64_t)ab * cz + z];
#pragma unroll
      for (int jj = 0; jj < JT; ++jj) acc[jj] = fmaf(tile[jj * cc + ab], wv, acc[jj]);
    }
#pragma unroll
    for (int jj = 0; jj < JT; ++jj) {
      int j = j0 + jj;
      if (j >= N) continue;
      float v;
      if (bias_after_norm) v = acc[jj] / fmaxf(counts[jj], 1.0f) + bout[z];
      else v = (acc[jj] + bout[z]) / (norm_eps + counts[jj]);
      int64_t o = ((int64_t)i * N + j) * cz + z;
      if (resid) v += to_f(resid[o]);
      out[o] = from_f<TAct>(v);
    }
  }
}

// int5 decode: one thread per value.  value = code*scale + zero.
__global__ void int5_decode_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scales,
                                   const __half* __restrict__ zeros, int64_t elements, int block,
                                   float* __restrict__ out) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= elements) return;
  int64_t g = i / block;
  int within = (int)(i % block);
  int bit = within * 5;
  const uint8_t* base = codes + g * (block * 5 / 8);
  unsigned two = base[bit >> 3] | ((unsigned)base[(bit >> 3) + 1] << 8);
  unsigned code = (two >> (bit & 7)) & 31u;
  out[i] = fmaf((float)code, __half2float(scales[g]), __half2float(zeros[g]));
}

}  // namespace simt
