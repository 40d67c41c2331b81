/*
 * CPU oracle for the pair-stack hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file restates, in plain C, the arithmetic of the reference's own CPU
 * implementations (JavaScript, which cannot be executed where this library is
 * built).  Each function names the reference file and lines it follows.  The
 * reference keeps every tensor in a Float32Array and evaluates scalar
 * expressions in double precision, so here every accumulator is a `double`
 * and every stored tensor element is a `float` (one rounding per store), and
 * every inner-product loop runs in the same ascending index order.
 *
 * Only tests, the smoke check and the CPU-baseline leg of the benchmark may
 * load this library; the product path never does.
 *
 * Parity pin: the AF2 outgoing triangle multiplication below reproduces the
 * four golden fixtures the reference ships (OpenFold N=5 and three AlphaFold
 * captures, N=9/59/59).  The AF3 primitives reproduce the hand-worked values
 * of the reference's unit tests, and the int5 decoder agrees with the
 * reference's Python quantiser.  The remaining operators have no golden data
 * in the reference checkout ("parity unpinned" for them): they are defined as
 * agreement with this restatement.
 *
 * OpenMP parallelises over independent output rows only; no reduction is
 * split across threads, so results do not depend on the thread count.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

static inline double sigmoid_d(double v) { return 1.0 / (1.0 + exp(-v)); }

ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

ORC_API void orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------------- */
/* LayerNorm over the last axis.
 * fast == 0: two-pass variance, webgpu/kernels/triangle/cpu-reference.js:5-30.
 * fast == 1: E[x^2]-E[x]^2, unclamped, cpu/af3/trunk/pairformer.js:68-87.     */
ORC_API void orc_layer_norm(const float* in, int64_t rows, int ch, const float* scale,
                            const float* offset, double eps, int fast, float* out) {
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const float* x = in + r * ch;
    float* y = out + r * ch;
    double mean, inv;
    if (fast) {
      double s = 0, ss = 0;
      for (int c = 0; c < ch; ++c) { double v = x[c]; s += v; ss += v * v; }
      mean = s / ch;
      double var = ss / ch - mean * mean;
      inv = 1.0 / sqrt(var + eps);
    } else {
      double s = 0;
      for (int c = 0; c < ch; ++c) s += x[c];
      mean = s / ch;
      double var = 0;
      for (int c = 0; c < ch; ++c) { double d = x[c] - mean; var += d * d; }
      inv = 1.0 / sqrt(var / ch + eps);
    }
    for (int c = 0; c < ch; ++c)
      y[c] = (float)(((double)x[c] - mean) * inv * (double)scale[c] + (double)offset[c]);
  }
}

/* rows x cin -> rows x cout.  transposed == 0: weights are (in,out);
 * transposed == 1: (out,in).  The accumulator starts from the bias and sums
 * over the input channel in ascending order.
 * cpu/af3/trunk/pairformer.js:100-147, webgpu/kernels/triangle/cpu-reference.js:32-53. */
ORC_API void orc_linear(const float* in, int64_t rows, int cin, int cout, const float* w,
                        const float* bias, int transposed, float* out) {
#pragma omp parallel
  {
    double* acc = (double*)malloc(sizeof(double) * (size_t)cout);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
      const float* x = in + r * cin;
      if (!transposed) {
        for (int o = 0; o < cout; ++o) acc[o] = bias ? (double)bias[o] : 0.0;
        for (int c = 0; c < cin; ++c) {
          double v = x[c];
          const float* wr = w + (size_t)c * cout;
          for (int o = 0; o < cout; ++o) acc[o] += v * (double)wr[o];
        }
        for (int o = 0; o < cout; ++o) out[r * cout + o] = (float)acc[o];
      } else {
        for (int o = 0; o < cout; ++o) {
          double t = bias ? (double)bias[o] : 0.0;
          const float* wr = w + (size_t)o * cin;
          for (int c = 0; c < cin; ++c) t += (double)x[c] * (double)wr[c];
          out[r * cout + o] = (float)t;
        }
      }
    }
    free(acc);
  }
}

/* Softmax over one row held as float32, in place.  The exponentials are
 * written back as float32 before they are summed and divided, exactly as the
 * reference's Float32Array row buffer does.  cpu/af3/trunk/pairformer.js:150-166. */
static void softmax_row_f32(float* v, int width) {
  float largest = -INFINITY;
  for (int i = 0; i < width; ++i) if (v[i] > largest) largest = v[i];
  double total = 0;
  for (int i = 0; i < width; ++i) {
    double e = exp((double)v[i] - (double)largest);
    v[i] = (float)e;
    total += e;
  }
  for (int i = 0; i < width; ++i) v[i] = (float)((double)v[i] / total);
}

/* ------------------------------------------------------------------------- */
/* Triangle multiplicative update: the contraction over channel-major a, b.
 * outgoing: x[c,i,j] = sum_k a[c,i,k] b[c,j,k]
 * incoming: x[c,i,j] = sum_k a[c,k,j] b[c,k,i]
 * cpu/af3/trunk/pairformer.js:237-270, webgpu/kernels/triangle/cpu-reference.js:77-88,
 * incoming form for the AF2 dialect: webgpu/kernels/triangle/shaders.js:672-675.
 * The incoming operands are transposed first so the k loop is contiguous; the
 * summation order over k is unchanged.                                       */
static void contract_planes(const float* a, const float* b, int n, int ch, int incoming,
                            int divide_by_length, float* x) {
  const size_t pairs = (size_t)n * n;
#pragma omp parallel
  {
    float* at = NULL; float* bt = NULL;
    if (incoming) { at = (float*)malloc(pairs * 4); bt = (float*)malloc(pairs * 4); }
#pragma omp for schedule(dynamic, 1)
    for (int c = 0; c < ch; ++c) {
      const float* pa = a + c * pairs;
      const float* pb = b + c * pairs;
      float* px = x + c * pairs;
      const float *L, *R;
      if (incoming) {
        /* L[i][k] = b[k][i], R[j][k] = a[k][j] */
        for (int k = 0; k < n; ++k)
          for (int i = 0; i < n; ++i) { bt[(size_t)i * n + k] = pb[(size_t)k * n + i]; at[(size_t)i * n + k] = pa[(size_t)k * n + i]; }
        L = bt; R = at;
      } else { L = pa; R = pb; }
      for (int i = 0; i < n; ++i) {
        const float* li = L + (size_t)i * n;
        for (int j = 0; j < n; ++j) {
          const float* rj = R + (size_t)j * n;
          double t = 0;
          /* outgoing: a[i,k]*b[j,k]; incoming: a[k,j]*b[k,i] = R[j][k]*L[i][k] */
          for (int k = 0; k < n; ++k) t += (double)li[k] * (double)rj[k];
          px[(size_t)i * n + j] = (float)(divide_by_length ? t / n : t);
        }
      }
    }
    free(at); free(bt);
  }
}

/* AF2 / OpenFold operator form: two-pass LayerNorm, biases on all six linears,
 * weights stored [out][in].  Returns the update (no residual add).
 * webgpu/kernels/triangle/cpu-reference.js:55-99.  `w` holds the 16 tensors in
 * the pack order of webgpu/kernels/triangle/weights.js:4-10.                */
ORC_API void orc_trimul_af2(const float* z, const float* mask, int n, int cz, int c,
                            const float* const* w, double eps, int incoming, float* out) {
  const size_t pairs = (size_t)n * n;
  float* zn = (float*)malloc(pairs * cz * 4);
  float* ap = (float*)malloc(pairs * c * 4);
  float* ag = (float*)malloc(pairs * c * 4);
  float* bp = (float*)malloc(pairs * c * 4);
  float* bg = (float*)malloc(pairs * c * 4);
  orc_layer_norm(z, (int64_t)pairs, cz, w[0], w[1], eps, 0, zn);
  orc_linear(zn, (int64_t)pairs, cz, c, w[2], w[3], 1, ap);
  orc_linear(zn, (int64_t)pairs, cz, c, w[4], w[5], 1, ag);
  orc_linear(zn, (int64_t)pairs, cz, c, w[6], w[7], 1, bp);
  orc_linear(zn, (int64_t)pairs, cz, c, w[8], w[9], 1, bg);
  /* channel-major gated operands */
  float* a = (float*)malloc(pairs * c * 4);
  float* b = (float*)malloc(pairs * c * 4);
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < (int64_t)pairs; ++p) {
    double m = mask[p];
    for (int h = 0; h < c; ++h) {
      size_t idx = (size_t)p * c + h;
      a[(size_t)h * pairs + p] = (float)((double)ap[idx] * sigmoid_d(ag[idx]) * m);
      b[(size_t)h * pairs + p] = (float)((double)bp[idx] * sigmoid_d(bg[idx]) * m);
    }
  }
  free(ap); free(ag); free(bp); free(bg);
  float* x = (float*)malloc(pairs * c * 4);
  contract_planes(a, b, n, c, incoming, 0, x);
  free(a); free(b);
  /* channel-major -> channel-minor, then LayerNorm over the hidden channels */
  float* xm = (float*)malloc(pairs * c * 4);
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < (int64_t)pairs; ++p)
    for (int h = 0; h < c; ++h) xm[(size_t)p * c + h] = x[(size_t)h * pairs + p];
  free(x);
  float* xn = (float*)malloc(pairs * c * 4);
  orc_layer_norm(xm, (int64_t)pairs, c, w[10], w[11], eps, 0, xn);
  free(xm);
  float* gate = (float*)malloc(pairs * cz * 4);
  orc_linear(xn, (int64_t)pairs, c, cz, w[12], w[13], 1, out);
  orc_linear(zn, (int64_t)pairs, cz, cz, w[14], w[15], 1, gate);
  const size_t total = pairs * cz;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)total; ++i)
    out[i] = (float)((double)out[i] * sigmoid_d(gate[i]));
  free(gate); free(xn); free(zn);
}

/* AF3 form: fast-variance LayerNorm (eps 1e-5), no biases, `projection` and
 * `gate` are (c, 2c) with a at column 2h and b at 2h+1; `outputProjection`
 * and `gatingLinear` are (c, c) stored (in,out).
 * cpu/af3/trunk/pairformer.js:213-300.                                       */
ORC_API void orc_trimul_af3(const float* pair, const float* mask, int n, int ch, int incoming,
                            const float* norm_scale, const float* norm_offset,
                            const float* projection, const float* gate_w,
                            const float* center_scale, const float* center_offset,
                            const float* output_projection, const float* gating_linear,
                            int divide_by_length, float* out) {
  const size_t pairs = (size_t)n * n;
  const double eps = 1e-5;
  float* zn = (float*)malloc(pairs * ch * 4);
  float* proj = (float*)malloc(pairs * ch * 2 * 4);
  float* gate = (float*)malloc(pairs * ch * 2 * 4);
  orc_layer_norm(pair, (int64_t)pairs, ch, norm_scale, norm_offset, eps, 1, zn);
  orc_linear(zn, (int64_t)pairs, ch, ch * 2, projection, NULL, 0, proj);
  orc_linear(zn, (int64_t)pairs, ch, ch * 2, gate_w, NULL, 0, gate);
  float* a = (float*)malloc(pairs * ch * 4);
  float* b = (float*)malloc(pairs * ch * 4);
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < (int64_t)pairs; ++p) {
    size_t wide = (size_t)p * ch * 2;
    double m = mask[p];
    for (int c = 0; c < ch; ++c) {
      double gated = m * sigmoid_d(gate[wide + c * 2]);
      a[(size_t)c * pairs + p] = (float)((double)proj[wide + c * 2] * gated);
      b[(size_t)c * pairs + p] = (float)((double)proj[wide + c * 2 + 1] * m * sigmoid_d(gate[wide + c * 2 + 1]));
    }
  }
  free(proj); free(gate);
  float* x = (float*)malloc(pairs * ch * 4);
  contract_planes(a, b, n, ch, incoming, divide_by_length, x);
  free(a); free(b);
  float* centred = (float*)malloc(pairs * ch * 4);
#pragma omp parallel for schedule(static)
  for (int64_t p = 0; p < (int64_t)pairs; ++p) {
    double s = 0, ss = 0;
    for (int c = 0; c < ch; ++c) { double v = x[(size_t)c * pairs + p]; s += v; ss += v * v; }
    double mean = s / ch;
    double inv = 1.0 / sqrt(ss / ch - mean * mean + eps);
    for (int c = 0; c < ch; ++c)
      centred[(size_t)p * ch + c] = (float)(((double)x[(size_t)c * pairs + p] - mean) * inv * (double)center_scale[c] + (double)center_offset[c]);
  }
  free(x);
  float* og = (float*)malloc(pairs * ch * 4);
  orc_linear(centred, (int64_t)pairs, ch, ch, output_projection, NULL, 0, out);
  orc_linear(zn, (int64_t)pairs, ch, ch, gating_linear, NULL, 0, og);
  const size_t total = pairs * ch;
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < (int64_t)total; ++i) out[i] = (float)((double)out[i] * sigmoid_d(og[i]));
  free(og); free(centred); free(zn);
}

/* ------------------------------------------------------------------------- */
/* AF2 gated multi-head attention (the operator behind MSA row / column and
 * triangle start / end attention).
 *
 * Logical row r = b*Q + i reads memory row i*batch + b when `transpose`
 * (webgpu/kernels/attention.js:162-167); the key mask index follows the same
 * rule (:889-892) and the output is stored back to the memory row (:2466).
 * Arithmetic follows tools/gpu/check-evoformer-attention.js:27-112 (two-pass
 * LayerNorm, weights (in,out), gate bias, output bias, softmax over float32
 * logits), extended with the pair bias and logit clamp of
 * webgpu/kernels/attention.js:695-756,917-921:
 *   logit = q.k/sqrt(d) + 1e9*(mask-1) + bias[h,i,j], clamped to +-1e8.
 * bias_mode 0: none.  1: "separate" - bias[h,i,j] = LN2(pair_act)[i,j,:].Wb
 * with its own norm.  2: "normalized-input" - bias[h,i,j] = n[b=i, q=j,:].Wb
 * from the logical normalised activations (needs batch == Q).               */
ORC_API void orc_attention_af2(const float* act, const float* mask, int batch, int Q, int ch,
                               int heads, int transpose,
                               const float* norm_scale, const float* norm_offset,
                               const float* wq, const float* wk, const float* wv,
                               const float* wg, const float* bg, const float* wo, const float* bo,
                               int bias_mode, const float* pair_act, int pair_ch,
                               const float* pair_norm_scale, const float* pair_norm_offset,
                               const float* pair_w, double eps, float* out) {
  const int d = ch / heads;
  const double scale = 1.0 / sqrt((double)d);
  const int64_t rows = (int64_t)batch * Q;
  /* logical normalised activations */
  float* gathered_in = (float*)malloc((size_t)rows * ch * 4);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    int64_t b = r / Q, i = r % Q;
    int64_t src = transpose ? i * batch + b : r;
    memcpy(gathered_in + r * ch, act + src * ch, (size_t)ch * 4);
  }
  float* nrm = (float*)malloc((size_t)rows * ch * 4);
  orc_layer_norm(gathered_in, rows, ch, norm_scale, norm_offset, eps, 0, nrm);
  free(gathered_in);
  float* q = (float*)malloc((size_t)rows * ch * 4);
  float* k = (float*)malloc((size_t)rows * ch * 4);
  float* v = (float*)malloc((size_t)rows * ch * 4);
  float* g = (float*)malloc((size_t)rows * ch * 4);
  orc_linear(nrm, rows, ch, ch, wq, NULL, 0, q);
  orc_linear(nrm, rows, ch, ch, wk, NULL, 0, k);
  orc_linear(nrm, rows, ch, ch, wv, NULL, 0, v);
  orc_linear(nrm, rows, ch, ch, wg, bg, 0, g);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < rows * ch; ++i) g[i] = (float)sigmoid_d(g[i]);
  /* pair bias, head-major [h][i][j] */
  float* bias = NULL;
  if (bias_mode != 0) {
    const int64_t pp = (int64_t)Q * Q;
    float* flat = (float*)malloc((size_t)pp * heads * 4);
    if (bias_mode == 1) {
      float* pn = (float*)malloc((size_t)pp * pair_ch * 4);
      orc_layer_norm(pair_act, pp, pair_ch, pair_norm_scale, pair_norm_offset, eps, 0, pn);
      orc_linear(pn, pp, pair_ch, heads, pair_w, NULL, 0, flat);
      free(pn);
    } else {
      orc_linear(nrm, pp, ch, heads, pair_w, NULL, 0, flat);
    }
    bias = (float*)malloc((size_t)pp * heads * 4);
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < pp; ++p)
      for (int h = 0; h < heads; ++h) bias[(size_t)h * pp + p] = flat[p * heads + h];
    free(flat);
  }
  float* gathered = (float*)malloc((size_t)rows * ch * 4);
#pragma omp parallel
  {
    float* logits = (float*)malloc((size_t)Q * 4);
#pragma omp for schedule(dynamic, 1) collapse(2)
    for (int b = 0; b < batch; ++b) {
      for (int h = 0; h < heads; ++h) {
        for (int i = 0; i < Q; ++i) {
          const float* qi = q + ((int64_t)b * Q + i) * ch + h * d;
          for (int j = 0; j < Q; ++j) {
            const float* kj = k + ((int64_t)b * Q + j) * ch + h * d;
            double dot = 0;
            for (int e = 0; e < d; ++e) dot += (double)qi[e] * (double)kj[e];
            double m = mask[transpose ? (int64_t)j * batch + b : (int64_t)b * Q + j];
            /* the shader works in float32: the scaled dot product, then the
             * mask term, then the bias, each rounded as it is added */
            float value = (float)(dot * scale);
            value = (float)((double)value + 1e9 * (m - 1.0));
            if (bias) value = (float)((double)value + (double)bias[((size_t)h * Q + i) * Q + j]);
            if (value > 1e8f) value = 1e8f;
            if (value < -1e8f) value = -1e8f;
            logits[j] = value;
          }
          /* exponentials are stored as float32, their stored values are
           * summed, and the division happens once per output element
           * (tools/gpu/check-evoformer-attention.js:87-99) */
          float largest = -INFINITY;
          for (int j = 0; j < Q; ++j) if (logits[j] > largest) largest = logits[j];
          double total = 0;
          for (int j = 0; j < Q; ++j) {
            logits[j] = (float)exp((double)logits[j] - (double)largest);
            total += (double)logits[j];
          }
          float* oi = gathered + ((int64_t)b * Q + i) * ch + h * d;
          for (int e = 0; e < d; ++e) {
            double t = 0;
            for (int j = 0; j < Q; ++j) t += (double)logits[j] * (double)v[((int64_t)b * Q + j) * ch + h * d + e];
            oi[e] = (float)(t / total);
          }
        }
      }
    }
    free(logits);
  }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < rows * ch; ++i) gathered[i] = (float)((double)gathered[i] * (double)g[i]);
  float* proj = (float*)malloc((size_t)rows * ch * 4);
  orc_linear(gathered, rows, ch, ch, wo, bo, 0, proj);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    int64_t b = r / Q, i = r % Q;
    int64_t dst = transpose ? i * batch + b : r;
    memcpy(out + dst * ch, proj + r * ch, (size_t)ch * 4);
  }
  free(proj); free(gathered); free(bias); free(g); free(v); free(k); free(q); free(nrm);
}

/* AF3 triangle ("grid") self-attention.  cpu/af3/trunk/pairformer.js:322-431.
 * q, k, gate weights are (out,in) = [H*d][c]; v is (in,out); out-projection is
 * (in,out) [H*d][c].  gate_bias / out_bias may be NULL.                       */
ORC_API void orc_grid_attention_af3(const float* pair, const float* mask, int n, int ch,
                                    int transpose, int heads, int dim, int swap_transposed_bias,
                                    const float* norm_scale, const float* norm_offset,
                                    const float* pair_bias_w, const float* wq, const float* wk,
                                    const float* wv, const float* wgate, const float* gate_bias,
                                    const float* wo, const float* out_bias, float* out) {
  const int64_t pairs = (int64_t)n * n;
  const int width = heads * dim;
  const double scale = 1.0 / sqrt((double)dim);
  float* nrm = (float*)malloc((size_t)pairs * ch * 4);
  orc_layer_norm(pair, pairs, ch, norm_scale, norm_offset, 1e-5, 1, nrm);
  float* raw = (float*)malloc((size_t)pairs * heads * 4);
  orc_linear(nrm, pairs, ch, heads, pair_bias_w, NULL, 0, raw);
  const int swap = transpose && swap_transposed_bias;
  float* bias = (float*)malloc((size_t)pairs * heads * 4);
#pragma omp parallel for schedule(static)
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j)
      for (int h = 0; h < heads; ++h) {
        int64_t src = swap ? ((int64_t)j * n + i) : ((int64_t)i * n + j);
        bias[(size_t)h * pairs + (int64_t)i * n + j] = raw[src * heads + h];
      }
  free(raw);
  float* act = (float*)malloc((size_t)pairs * ch * 4);
#pragma omp parallel for schedule(static)
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      int64_t from = transpose ? ((int64_t)j * n + i) : ((int64_t)i * n + j);
      memcpy(act + ((int64_t)i * n + j) * ch, nrm + from * ch, (size_t)ch * 4);
    }
  free(nrm);
  float* q = (float*)malloc((size_t)pairs * width * 4);
  float* k = (float*)malloc((size_t)pairs * width * 4);
  float* v = (float*)malloc((size_t)pairs * width * 4);
  orc_linear(act, pairs, ch, width, wq, NULL, 1, q);
  orc_linear(act, pairs, ch, width, wk, NULL, 1, k);
  orc_linear(act, pairs, ch, width, wv, NULL, 0, v);
  float* gathered = (float*)malloc((size_t)pairs * width * 4);
#pragma omp parallel
  {
    float* logits = (float*)malloc((size_t)n * 4);
#pragma omp for schedule(dynamic, 1) collapse(2)
    for (int row = 0; row < n; ++row) {
      for (int h = 0; h < heads; ++h) {
        for (int i = 0; i < n; ++i) {
          const float* qi = q + ((int64_t)row * n + i) * width + h * dim;
          for (int j = 0; j < n; ++j) {
            const float* kj = k + ((int64_t)row * n + j) * width + h * dim;
            double dot = 0;
            for (int e = 0; e < dim; ++e) dot += (double)qi[e] * (double)kj[e];
            float masked = mask[transpose ? ((int64_t)j * n + row) : ((int64_t)row * n + j)];
            logits[j] = (float)(dot * scale + (double)bias[(size_t)h * pairs + (int64_t)i * n + j] + (masked > 0 ? 0.0 : -1e9));
          }
          softmax_row_f32(logits, n);
          float* oi = gathered + ((int64_t)row * n + i) * width + h * dim;
          for (int e = 0; e < dim; ++e) {
            double t = 0;
            for (int j = 0; j < n; ++j) t += (double)logits[j] * (double)v[((int64_t)row * n + j) * width + h * dim + e];
            oi[e] = (float)t;
          }
        }
      }
    }
    free(logits);
  }
  float* gate = (float*)malloc((size_t)pairs * width * 4);
  orc_linear(act, pairs, ch, width, wgate, NULL, 1, gate);
  if (gate_bias) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < pairs; ++r)
      for (int w = 0; w < width; ++w) gate[r * width + w] = (float)((double)gate[r * width + w] + (double)gate_bias[w]);
  }
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < pairs * width; ++i) gathered[i] = (float)((double)gathered[i] * sigmoid_d(gate[i]));
  free(gate);
  float* proj = (float*)malloc((size_t)pairs * ch * 4);
  orc_linear(gathered, pairs, width, ch, wo, NULL, 0, proj);
  if (out_bias) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < pairs; ++r)
      for (int c = 0; c < ch; ++c) proj[r * ch + c] = (float)((double)proj[r * ch + c] + (double)out_bias[c]);
  }
  if (!transpose) {
    memcpy(out, proj, (size_t)pairs * ch * 4);
  } else {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < n; ++i)
      for (int j = 0; j < n; ++j)
        memcpy(out + ((int64_t)i * n + j) * ch, proj + ((int64_t)j * n + i) * ch, (size_t)ch * 4);
  }
  free(proj); free(gathered); free(v); free(k); free(q); free(act); free(bias);
}

/* ------------------------------------------------------------------------- */
/* AF2 transition: relu(LN2(x).W1 + b1).W2 + b2, weights (in,out).
 * tools/gpu/check-evoformer-transition.js:30-66.  The hidden row is float32. */
ORC_API void orc_transition_af2(const float* act, int64_t rows, int ch, int hidden,
                                const float* norm_scale, const float* norm_offset,
                                const float* w1, const float* b1, const float* w2, const float* b2,
                                double eps, float* out) {
  float* nrm = (float*)malloc((size_t)rows * ch * 4);
  orc_layer_norm(act, rows, ch, norm_scale, norm_offset, eps, 0, nrm);
  float* hid = (float*)malloc((size_t)rows * hidden * 4);
  orc_linear(nrm, rows, ch, hidden, w1, b1, 0, hid);
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < rows * hidden; ++i) if (!(hid[i] > 0)) hid[i] = 0;
  orc_linear(hid, rows, hidden, ch, w2, b2, 0, out);
  free(hid); free(nrm);
}

/* AF3 transition: LN_fast -> (c, 2*f*c) -> swish(first half) * second half ->
 * (f*c, c).  cpu/af3/trunk/pairformer.js:180-201.                            */
ORC_API void orc_transition_af3(const float* act, int64_t rows, int ch, int factor,
                                const float* norm_scale, const float* norm_offset,
                                const float* t1, const float* t2, float* out) {
  const int inter = ch * factor;
  float* nrm = (float*)malloc((size_t)rows * ch * 4);
  orc_layer_norm(act, rows, ch, norm_scale, norm_offset, 1e-5, 1, nrm);
  float* wide = (float*)malloc((size_t)rows * inter * 2 * 4);
  orc_linear(nrm, rows, ch, inter * 2, t1, NULL, 0, wide);
  float* gated = (float*)malloc((size_t)rows * inter * 4);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r)
    for (int i = 0; i < inter; ++i) {
      double gv = wide[r * inter * 2 + i];
      double swish = gv * sigmoid_d(gv);
      gated[r * inter + i] = (float)(swish * (double)wide[r * inter * 2 + inter + i]);
    }
  orc_linear(gated, rows, inter, ch, t2, NULL, 0, out);
  free(gated); free(wide); free(nrm);
}

/* ------------------------------------------------------------------------- */
/* Outer product mean.
 * AF2 (bias_after_norm == 0, biases given): tools/gpu/check-evoformer-opm.js:29-94.
 * AF3 (af2_dialect == 0): cpu/af3/trunk/msa.js:72-155 (left/right biases optional;
 * fast-variance LayerNorm; multiplies by 1/(eps+count) where AF2 divides;
 * bias_after_norm selects the OpenDDE form).
 * The per-pair outer product accumulates in a float32 buffer, as both
 * references do.                                                             */
ORC_API void orc_outer_product_mean(const float* msa, const float* mask, int S, int n, int cm,
                                    int co, int cz, const float* norm_scale, const float* norm_offset,
                                    const float* wl, const float* bl, const float* wr, const float* br,
                                    const float* wout, const float* bout, double ln_eps,
                                    double norm_eps, int af2_dialect, int bias_after_norm,
                                    float* out) {
  const int64_t rows = (int64_t)S * n;
  float* nrm = (float*)malloc((size_t)rows * cm * 4);
  orc_layer_norm(msa, rows, cm, norm_scale, norm_offset, ln_eps, af2_dialect ? 0 : 1, nrm);
  float* left = (float*)malloc((size_t)rows * co * 4);
  float* right = (float*)malloc((size_t)rows * co * 4);
  orc_linear(nrm, rows, cm, co, wl, bl, 0, left);
  orc_linear(nrm, rows, cm, co, wr, br, 0, right);
  free(nrm);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    double keep = mask[r];
    for (int c = 0; c < co; ++c) {
      left[r * co + c] = (float)(keep * (double)left[r * co + c]);
      right[r * co + c] = (float)(keep * (double)right[r * co + c]);
    }
  }
#pragma omp parallel
  {
    float* outer = (float*)malloc((size_t)co * co * 4);
#pragma omp for schedule(dynamic, 1)
    for (int i = 0; i < n; ++i) {
      for (int j = 0; j < n; ++j) {
        memset(outer, 0, (size_t)co * co * 4);
        double count = 0;
        for (int s = 0; s < S; ++s) {
          count += (double)mask[(int64_t)s * n + i] * (double)mask[(int64_t)s * n + j];
          const float* l = left + ((int64_t)s * n + i) * co;
          const float* r = right + ((int64_t)s * n + j) * co;
          for (int a = 0; a < co; ++a) {
            double lv = l[a];
            for (int b = 0; b < co; ++b)
              outer[a * co + b] = (float)((double)outer[a * co + b] + lv * (double)r[b]);
          }
        }
        float* o = out + ((int64_t)i * n + j) * cz;
        double sc = bias_after_norm ? 1.0 / (count > 1.0 ? count : 1.0) : 1.0 / (norm_eps + count);
        for (int zc = 0; zc < cz; ++zc) {
          double value = bias_after_norm ? 0.0 : (double)bout[zc];
          for (int a = 0; a < co; ++a)
            for (int b = 0; b < co; ++b)
              value += (double)outer[a * co + b] * (double)wout[((size_t)a * co + b) * cz + zc];
          if (af2_dialect) o[zc] = (float)(value / (norm_eps + count));
          else o[zc] = (float)(bias_after_norm ? value * sc + (double)bout[zc] : value * sc);
        }
      }
    }
    free(outer);
  }
  free(left); free(right);
}

/* ------------------------------------------------------------------------- */
/* AF3 single-representation attention with pair bias.
 * cpu/af3/trunk/pairformer.js:446-485.  All weights (in,out); q has a bias.  */
ORC_API void orc_single_attention_af3(const float* single, const float* pair_logits,
                                      const float* seq_mask, int n, int ch, int heads, int dim,
                                      const float* norm_scale, const float* norm_offset,
                                      const float* wq, const float* bq, const float* wk,
                                      const float* wv, const float* wgate, const float* wo,
                                      float* out) {
  const int width = heads * dim;
  const double scale = 1.0 / sqrt((double)dim);
  float* nrm = (float*)malloc((size_t)n * ch * 4);
  orc_layer_norm(single, n, ch, norm_scale, norm_offset, 1e-5, 1, nrm);
  float* q = (float*)malloc((size_t)n * width * 4);
  float* k = (float*)malloc((size_t)n * width * 4);
  float* v = (float*)malloc((size_t)n * width * 4);
  orc_linear(nrm, n, ch, width, wq, bq, 0, q);
  orc_linear(nrm, n, ch, width, wk, NULL, 0, k);
  orc_linear(nrm, n, ch, width, wv, NULL, 0, v);
  float* gathered = (float*)malloc((size_t)n * width * 4);
#pragma omp parallel
  {
    float* logits = (float*)malloc((size_t)n * 4);
#pragma omp for schedule(dynamic, 1)
    for (int h = 0; h < heads; ++h) {
      for (int i = 0; i < n; ++i) {
        for (int j = 0; j < n; ++j) {
          double dot = 0;
          for (int e = 0; e < dim; ++e) dot += (double)q[(size_t)i * width + h * dim + e] * (double)k[(size_t)j * width + h * dim + e];
          logits[j] = (float)(dot * scale + (double)pair_logits[(size_t)h * n * n + (size_t)i * n + j] + 1e9 * ((double)seq_mask[j] - 1.0));
        }
        softmax_row_f32(logits, n);
        for (int e = 0; e < dim; ++e) {
          double t = 0;
          for (int j = 0; j < n; ++j) t += (double)logits[j] * (double)v[(size_t)j * width + h * dim + e];
          gathered[(size_t)i * width + h * dim + e] = (float)t;
        }
      }
    }
    free(logits);
  }
  float* gate = (float*)malloc((size_t)n * width * 4);
  orc_linear(nrm, n, ch, width, wgate, NULL, 0, gate);
  for (int64_t i = 0; i < (int64_t)n * width; ++i) gathered[i] = (float)((double)gathered[i] * sigmoid_d(gate[i]));
  orc_linear(gathered, n, width, ch, wo, NULL, 0, out);
  free(gate); free(gathered); free(v); free(k); free(q); free(nrm);
}

/* Head-major pair logits for the single attention:
 * logits[h,i,j] = LN_fast(pair)[i,j,:] . W[:,h].  cpu/af3/trunk/pairformer.js:516-532. */
ORC_API void orc_pair_logits_af3(const float* pair, int n, int ch, int heads,
                                 const float* norm_scale, const float* norm_offset,
                                 const float* w, float* out) {
  const int64_t pairs = (int64_t)n * n;
  float* nrm = (float*)malloc((size_t)pairs * ch * 4);
  orc_layer_norm(pair, pairs, ch, norm_scale, norm_offset, 1e-5, 1, nrm);
  float* flat = (float*)malloc((size_t)pairs * heads * 4);
  orc_linear(nrm, pairs, ch, heads, w, NULL, 0, flat);
  for (int64_t p = 0; p < pairs; ++p)
    for (int h = 0; h < heads; ++h) out[(size_t)h * pairs + p] = flat[p * heads + h];
  free(flat); free(nrm);
}

/* ------------------------------------------------------------------------- */
/* AF3 MSA pair-weighted averaging: values from the MSA, weights from the pair only (no query, no key).
 * cpu/af3/trunk/msa.js:164-224.  All weights (in,out); LayerNorms are the fast-variance form; one key mask
 * for every sequence, the maximum of the MSA mask over the depth (:179-187); the softmax row is float32
 * (softmaxRows, msa.js:34-52).  width = heads * dim need not equal the MSA channels.                     */
ORC_API void orc_msa_attention_af3(const float* msa, const float* msa_mask, const float* pair, int sequences,
                                   int tokens, int cm, int cz, int heads, int dim, const float* act_scale,
                                   const float* act_offset, const float* pair_scale, const float* pair_offset,
                                   const float* pair_logits, const float* wv, const float* wgate, const float* wo,
                                   float* out) {
  const int width = heads * dim;
  const int64_t rows = (int64_t)sequences * tokens, pairs = (int64_t)tokens * tokens;
  float* nrm = (float*)malloc((size_t)rows * cm * 4);
  orc_layer_norm(msa, rows, cm, act_scale, act_offset, 1e-5, 1, nrm);
  float* pnrm = (float*)malloc((size_t)pairs * cz * 4);
  orc_layer_norm(pair, pairs, cz, pair_scale, pair_offset, 1e-5, 1, pnrm);
  float* flat = (float*)malloc((size_t)pairs * heads * 4);
  orc_linear(pnrm, pairs, cz, heads, pair_logits, NULL, 0, flat);
  float* key_mask = (float*)malloc((size_t)tokens * 4);
  for (int t = 0; t < tokens; ++t) {
    float largest = 0;
    for (int s = 0; s < sequences; ++s) if (msa_mask[(size_t)s * tokens + t] > largest) largest = msa_mask[(size_t)s * tokens + t];
    key_mask[t] = largest;
  }
  float* weights = (float*)malloc((size_t)heads * pairs * 4);
#pragma omp parallel for schedule(static)
  for (int h = 0; h < heads; ++h)
    for (int i = 0; i < tokens; ++i) {
      float* row = weights + (size_t)h * pairs + (size_t)i * tokens;
      for (int j = 0; j < tokens; ++j)
        row[j] = (float)((double)flat[((size_t)i * tokens + j) * heads + h] + 1e9 * ((double)key_mask[j] - 1.0));
      softmax_row_f32(row, tokens);
    }
  float* values = (float*)malloc((size_t)rows * width * 4);
  orc_linear(nrm, rows, cm, width, wv, NULL, 0, values);
  float* averaged = (float*)malloc((size_t)rows * width * 4);
#pragma omp parallel for schedule(static)
  for (int64_t si = 0; si < rows; ++si) {
    const int s = (int)(si / tokens), i = (int)(si % tokens);
    for (int h = 0; h < heads; ++h) {
      const float* wrow = weights + (size_t)h * pairs + (size_t)i * tokens;
      for (int d = 0; d < dim; ++d) {
        double total = 0;
        for (int j = 0; j < tokens; ++j) total += (double)wrow[j] * (double)values[((size_t)s * tokens + j) * width + h * dim + d];
        averaged[(size_t)si * width + h * dim + d] = (float)total;
      }
    }
  }
  float* gate = (float*)malloc((size_t)rows * width * 4);
  orc_linear(nrm, rows, cm, width, wgate, NULL, 0, gate);
  for (int64_t i = 0; i < rows * width; ++i) averaged[i] = (float)((double)averaged[i] * sigmoid_d(gate[i]));
  orc_linear(averaged, rows, width, cm, wo, NULL, 0, out);
  free(gate); free(averaged); free(values); free(weights); free(key_mask); free(flat); free(pnrm); free(nrm);
}

/* Distogram logits: one half from a linear over the pair, symmetrised by a SUM with its transpose over the
 * two token axes (not a mean).  cpu/af3/trunk/trunk.js:47-60.  `bias` may be null (AlphaFold 3 has none).  */
ORC_API void orc_distogram_logits(const float* pair, int tokens, int cz, int bins, const float* w, const float* bias,
                                  float* out) {
  const int64_t pairs = (int64_t)tokens * tokens;
  float* half = (float*)malloc((size_t)pairs * bins * 4);
  orc_linear(pair, pairs, cz, bins, w, bias, 0, half);
#pragma omp parallel for schedule(static)
  for (int i = 0; i < tokens; ++i)
    for (int j = 0; j < tokens; ++j) {
      const float* f = half + ((size_t)i * tokens + j) * bins;
      const float* b = half + ((size_t)j * tokens + i) * bins;
      float* o = out + ((size_t)i * tokens + j) * bins;
      for (int k = 0; k < bins; ++k) o[k] = f[k] + b[k];
    }
  free(half);
}

/* ------------------------------------------------------------------------- */
/* AF2 global column attention of the extra-MSA stack, as the reference's shaders define it
 * (webgpu/af2/evoformer/block.js:100-482, encodeGlobalAttention :953-1032): per column, one query - the
 * masked mean over the sequences of the two-pass-normalised MSA, projected onto the heads and scaled by
 * head_dim^-1/2 - against one shared key/value head per sequence; masked sequences get the logit -1e9;
 * the attended vector of the column is gated per sequence by sigmoid(x.Wg + bg) and projected.  Weights
 * (in,out); float32 is stored where the shaders store it (normalised MSA, means, query, keys, values,
 * attended, gated).                                                                                       */
ORC_API void orc_global_column_attention_af2(const float* msa, const float* mask, int S, int n, int c, int heads,
                                             int dim, const float* norm_scale, const float* norm_offset,
                                             const float* wq, const float* wk, const float* wv,
                                             const float* wgate, const float* bgate, const float* wo,
                                             const float* bo, double eps, float* out) {
  const int gates = heads * dim;
  const int64_t rows = (int64_t)S * n;
  float* nrm = (float*)malloc((size_t)rows * c * 4);
  orc_layer_norm(msa, rows, c, norm_scale, norm_offset, eps, 0, nrm);
  float* keys = (float*)malloc((size_t)rows * dim * 4);
  float* values = (float*)malloc((size_t)rows * dim * 4);
  orc_linear(nrm, rows, c, dim, wk, NULL, 0, keys);
  orc_linear(nrm, rows, c, dim, wv, NULL, 0, values);
  float* attended = (float*)malloc((size_t)n * gates * 4);
  const double scale = 1.0 / sqrt((double)dim);
#pragma omp parallel
  {
    float* means = (float*)malloc((size_t)c * 4);
    float* query = (float*)malloc((size_t)gates * 4);
    float* logits = (float*)malloc((size_t)S * 4);
#pragma omp for schedule(static)
    for (int col = 0; col < n; ++col) {
      double count = 0;
      for (int s = 0; s < S; ++s) count += (double)mask[(size_t)s * n + col];
      const double denominator = 1e-10 + count;
      for (int ch = 0; ch < c; ++ch) {
        double total = 0;
        for (int s = 0; s < S; ++s) total += (double)nrm[((size_t)s * n + col) * c + ch] * (double)mask[(size_t)s * n + col];
        means[ch] = (float)(total / denominator);
      }
      for (int slot = 0; slot < gates; ++slot) {
        double r = 0;
        for (int ch = 0; ch < c; ++ch) r += (double)means[ch] * (double)wq[(size_t)ch * gates + slot];
        query[slot] = (float)(r * scale);
      }
      for (int h = 0; h < heads; ++h) {
        for (int s = 0; s < S; ++s) {
          double l = 0;
          for (int d = 0; d < dim; ++d) l += (double)query[h * dim + d] * (double)keys[((size_t)s * n + col) * dim + d];
          logits[s] = mask[(size_t)s * n + col] == 0.0f ? -1e9f : (float)l;
        }
        softmax_row_f32(logits, S);
        for (int d = 0; d < dim; ++d) {
          double t = 0;
          for (int s = 0; s < S; ++s) t += (double)logits[s] * (double)values[((size_t)s * n + col) * dim + d];
          attended[(size_t)col * gates + h * dim + d] = (float)t;
        }
      }
    }
    free(logits); free(query); free(means);
  }
  float* gate = (float*)malloc((size_t)rows * gates * 4);
  orc_linear(nrm, rows, c, gates, wgate, bgate, 0, gate);
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < rows; ++r) {
    const int col = (int)(r % n);
    for (int slot = 0; slot < gates; ++slot)
      gate[r * gates + slot] = (float)((double)attended[(size_t)col * gates + slot] * sigmoid_d(gate[r * gates + slot]));
  }
  orc_linear(gate, rows, gates, c, wo, bo, 0, out);
  free(gate); free(attended); free(values); free(keys); free(nrm);
}

/* ------------------------------------------------------------------------- */
/* int5 tensor decode: groups of `block` codes, 5 bits each, least significant
 * bit first in a little-endian bit stream (block*5/8 bytes per group), one
 * fp16 scale and one fp16 zero point per group; value = code*scale + zero in
 * double, stored float32.  shared/weights/dtype.js:330-378;
 * tools/quantize_af3.py:60-101.                                              */
static double half_to_double(uint16_t h) {
  int sign = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023;
  double v;
  if (e == 0) v = ldexp((double)m, -24);
  else if (e == 31) v = m ? NAN : INFINITY;
  else v = ldexp((double)(m + 1024), e - 25);
  return sign ? -v : v;
}

ORC_API void orc_int5_decode(const uint8_t* codes, const uint16_t* scales, const uint16_t* zeros,
                             int64_t elements, int block, float* out) {
  const int group_bytes = block * 5 / 8;
  const int64_t groups = (elements + block - 1) / block;
  for (int64_t g = 0; g < groups; ++g) {
    double scale = half_to_double(scales[g]);
    double zero = half_to_double(zeros[g]);
    const uint8_t* base = codes + g * group_bytes;
    int64_t start = g * block;
    int64_t end = start + block < elements ? start + block : elements;
    int bit = 0;
    for (int64_t i = start; i < end; ++i) {
      int at = bit >> 3;
      unsigned two = base[at] | ((unsigned)base[at + 1] << 8);
      unsigned code = (two >> (bit & 7)) & 31u;
      out[i] = (float)((double)code * scale + zero);
      bit += 5;
    }
  }
}
