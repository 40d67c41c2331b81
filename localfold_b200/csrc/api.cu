// C ABI of the pair-stack library: context, weights, operators.
// The float32 path composes the SIMT kernels of simt_kernels.cuh; the bf16 path
// routes the shapes they cover to the tcgen05 kernels declared in tc_kernels.cuh.
#include <cuda_fp16.h>

#include <cmath>
#include <cstring>
#include <map>
#include <mutex>

#include "simt_kernels.cuh"
#include "tc_kernels.cuh"

// ---------------------------------------------------------------------------
// context

static void profile_collect(lf_context* ctx) {
  cudaStreamSynchronize(ctx->stream);
  for (auto& t : ctx->timed) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess) {
      ctx->family_ms[t.family] += ms;
      ctx->family_launches[t.family] += 1;
    }
    cudaEventDestroy(t.start);
    cudaEventDestroy(t.stop);
  }
  ctx->timed.clear();
  cudaGetLastError();
}


lf_status lf_arena_ensure(lf_context* ctx, size_t bytes) {
  if (ctx->arena_limit && bytes > ctx->arena_limit)
    return lf_fail(ctx, LF_ERR_MEMORY, "scratch arena of %zu bytes exceeds the limit of %zu bytes set for this context", bytes, ctx->arena_limit);
  if (bytes <= ctx->arena_bytes) return LF_OK;
  // Work that still reads the old arena must finish before it is freed.
  LF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->arena) { cudaFree(ctx->arena); ctx->arena = nullptr; ctx->arena_bytes = 0; }
  size_t want = lf_align_up(bytes + bytes / 8, (size_t)1 << 21);
  cudaError_t e = cudaMalloc(&ctx->arena, want);
  if (e != cudaSuccess) {
    cudaGetLastError();
    want = lf_align_up(bytes, (size_t)1 << 21);
    e = cudaMalloc(&ctx->arena, want);
  }
  if (e != cudaSuccess) {
    cudaGetLastError();
    return lf_fail(ctx, LF_ERR_MEMORY, "scratch arena of %zu bytes refused: %s", want, cudaGetErrorString(e));
  }
  ctx->arena_bytes = want;
  return LF_OK;
}

extern "C" {

const char* lf_version(void) { return "localfold-pairstack-b200 0.1 (sm_100a)"; }

static lf_status context_create(int device_ordinal, void* stream, bool make_stream, lf_context** out);

lf_status lf_context_create(int device_ordinal, void* stream, lf_context** out) {
  return context_create(device_ordinal, stream, stream == nullptr, out);
}

lf_status lf_context_create_on_stream(int device_ordinal, void* stream, lf_context** out) {
  return context_create(device_ordinal, stream, false, out);
}

void* lf_context_stream(const lf_context* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

static lf_status context_create(int device_ordinal, void* stream, bool make_stream, lf_context** out) {
  if (!out) return LF_ERR_ARGUMENT;
  *out = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count == 0) { cudaGetLastError(); return LF_ERR_CUDA; }
  if (device_ordinal < 0 || device_ordinal >= count) return LF_ERR_ARGUMENT;
  if (cudaSetDevice(device_ordinal) != cudaSuccess) return LF_ERR_CUDA;
  lf_context* ctx = new lf_context();
  ctx->device = device_ordinal;
  if (!make_stream) { ctx->stream = (cudaStream_t)stream; ctx->owns_stream = false; }
  else {
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) { delete ctx; return LF_ERR_CUDA; }
    ctx->owns_stream = true;
  }
  cudaEventCreate(&ctx->ev0);
  cudaEventCreate(&ctx->ev1);
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device_ordinal) == cudaSuccess) ctx->sm_count = prop.multiProcessorCount;
  tc::configure_once();
  {   // the centre LayerNorm of the generic path stages c x 33 floats: up to cHidden = 512 is accepted
    static std::once_flag per_device[64];
    if (device_ordinal < 64)
      std::call_once(per_device[device_ordinal], [] {
        cudaFuncSetAttribute(simt::center_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 512 * 33 * 4);
        cudaFuncSetAttribute(simt::center_norm_kernel<op16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 512 * 33 * 4);
        cudaGetLastError();
      });
  }
  if (cudaMalloc(&ctx->tc_status, 16) == cudaSuccess) cudaMemset(ctx->tc_status, 0, 16);
  *out = ctx;
  return LF_OK;
}

void lf_context_destroy(lf_context* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  profile_collect(ctx);
  if (ctx->arena) cudaFree(ctx->arena);
  if (ctx->tc_status) cudaFree(ctx->tc_status);
  if (ctx->ev0) cudaEventDestroy(ctx->ev0);
  if (ctx->ev1) cudaEventDestroy(ctx->ev1);
  if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
}

const char* lf_last_error(const lf_context* ctx) { return ctx ? ctx->error.c_str() : "no context"; }

lf_status lf_context_synchronize(lf_context* ctx) {
  if (!ctx) return LF_ERR_ARGUMENT;
  LF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return tc::check_status(ctx);
}

uint64_t lf_context_launch_count(const lf_context* ctx) { return ctx ? ctx->launches : 0; }

lf_status lf_context_profile(lf_context* ctx, int enable) {
  if (!ctx) return LF_ERR_ARGUMENT;
  cudaSetDevice(ctx->device);
  profile_collect(ctx);
  ctx->profiling = enable != 0;
  return LF_OK;
}

lf_status lf_context_profile_read(lf_context* ctx, int family, double* total_ms, uint64_t* launches) {
  if (!ctx || family < 0 || family >= LF_KERNEL_FAMILY_COUNT) return LF_ERR_ARGUMENT;
  cudaSetDevice(ctx->device);
  profile_collect(ctx);
  if (total_ms) *total_ms = ctx->family_ms[family];
  if (launches) *launches = ctx->family_launches[family];
  ctx->family_ms[family] = 0;
  ctx->family_launches[family] = 0;
  return LF_OK;
}

lf_status lf_context_reserve(lf_context* ctx, uint64_t bytes) {
  if (!ctx) return LF_ERR_ARGUMENT;
  cudaSetDevice(ctx->device);
  return lf_arena_ensure(ctx, (size_t)bytes);
}

lf_status lf_context_limit_scratch(lf_context* ctx, uint64_t bytes) {
  if (!ctx) return LF_ERR_ARGUMENT;
  ctx->arena_limit = (size_t)bytes;
  return LF_OK;
}

void lf_context_release_scratch(lf_context* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->arena) cudaFree(ctx->arena);
  ctx->arena = nullptr;
  ctx->arena_bytes = 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// weights: canonical device layout, every linear (in,out) row-major float32

namespace {


typedef std::vector<float> hvec;

// [out][in] -> [in][out]
hvec transposed(const float* w, int out, int in) {
  hvec r((size_t)out * in);
  for (int o = 0; o < out; ++o)
    for (int i = 0; i < in; ++i) r[(size_t)i * out + o] = w[(size_t)o * in + i];
  return r;
}

// place a [in][n] block at column col0 of a [in][total] matrix
void put_columns(hvec& dst, int total, int col0, const float* src, int in, int n, int src_ld, int src_col0, int src_step) {
  for (int i = 0; i < in; ++i)
    for (int j = 0; j < n; ++j) dst[(size_t)i * total + col0 + j] = src[(size_t)i * src_ld + src_col0 + (size_t)j * src_step];
}

// Tensors of one operator are staged here while it is being built, then go to the device in one
// allocation with one synchronisation (finish_uploads).
struct PendingUploads {
  struct Item { int slot; hvec data; };
  std::vector<Item> items;
};
thread_local PendingUploads g_pending;

lf_status upload(lf_context* ctx, lf_weights* w, int slot, hvec host) {
  (void)ctx; (void)w;
  g_pending.items.push_back({slot, std::move(host)});
  return LF_OK;
}

lf_status finish_uploads(lf_context* ctx, lf_weights* w) {
  size_t total = 0;
  std::vector<size_t> offset;
  for (auto& it : g_pending.items) {
    offset.push_back(total);
    total += lf_align_up(it.data.size() * sizeof(float) + 4, 256);
  }
  char* base = nullptr;
  cudaError_t e = cudaMalloc(&base, total ? total : 256);
  if (e != cudaSuccess) {
    g_pending.items.clear();
    cudaGetLastError();
    return lf_fail(ctx, LF_ERR_MEMORY, "weight allocation of %zu bytes refused: %s", total, cudaGetErrorString(e));
  }
  w->owned.push_back(base);
  lf_status s = LF_OK;
  for (size_t i = 0; i < g_pending.items.size() && s == LF_OK; ++i) {
    auto& it = g_pending.items[i];
    float* dev = reinterpret_cast<float*>(base + offset[i]);
    if (!it.data.empty() &&
        cudaMemcpyAsync(dev, it.data.data(), it.data.size() * sizeof(float), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess) {
      cudaGetLastError();
      s = lf_fail(ctx, LF_ERR_CUDA, "weight upload failed");
    }
    w->f[it.slot] = dev;
  }
  if (cudaStreamSynchronize(ctx->stream) != cudaSuccess && s == LF_OK) s = lf_fail(ctx, LF_ERR_CUDA, "weight upload failed");
  return s;      // the staged host copies stay until the tensor-core repacks have read them (lf_weights_create)
}

struct Expect { const char* name; int64_t count; };

lf_status check_counts(lf_context* ctx, const Expect* e, int n_expected, const int64_t* counts, int n_given,
                       const float* const* tensors) {
  if (n_given != n_expected)
    return lf_fail(ctx, LF_ERR_ARGUMENT, "expected %d weight tensors; received %d", n_expected, n_given);
  for (int i = 0; i < n_expected; ++i) {
    if (counts[i] != e[i].count)
      return lf_fail(ctx, LF_ERR_SHAPE, "%s has %lld values; expected %lld", e[i].name, (long long)counts[i], (long long)e[i].count);
    if (e[i].count > 0 && tensors[i] == nullptr)
      return lf_fail(ctx, LF_ERR_ARGUMENT, "%s is null", e[i].name);
  }
  return LF_OK;
}

lf_status build_triangle_af2(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt) {
  const int cz = w->dims.channels, c = w->dims.hidden;
  const Expect e[16] = {
      {"layerNormInWeight", cz}, {"layerNormInBias", cz}, {"linearAPWeight", (int64_t)c * cz}, {"linearAPBias", c},
      {"linearAGWeight", (int64_t)c * cz}, {"linearAGBias", c}, {"linearBPWeight", (int64_t)c * cz}, {"linearBPBias", c},
      {"linearBGWeight", (int64_t)c * cz}, {"linearBGBias", c}, {"layerNormOutWeight", c}, {"layerNormOutBias", c},
      {"linearZWeight", (int64_t)cz * c}, {"linearZBias", cz}, {"linearGWeight", (int64_t)cz * cz}, {"linearGBias", cz}};
  LF_TRY(check_counts(ctx, e, 16, n, nt, t));
  w->f.assign(TRI_COUNT, nullptr);
  hvec w4((size_t)cz * 4 * c), b4((size_t)4 * c);
  const int order[4] = {2, 4, 6, 8};   // ap, ag, bp, bg
  for (int r = 0; r < 4; ++r) {
    hvec tr = transposed(t[order[r]], c, cz);
    put_columns(w4, 4 * c, r * c, tr.data(), cz, c, c, 0, 1);
    memcpy(&b4[(size_t)r * c], t[order[r] + 1], sizeof(float) * c);
  }
  LF_TRY(upload(ctx, w, TRI_LN_G, hvec(t[0], t[0] + cz)));
  LF_TRY(upload(ctx, w, TRI_LN_B, hvec(t[1], t[1] + cz)));
  LF_TRY(upload(ctx, w, TRI_W4, w4));
  LF_TRY(upload(ctx, w, TRI_B4, b4));
  LF_TRY(upload(ctx, w, TRI_LNO_G, hvec(t[10], t[10] + c)));
  LF_TRY(upload(ctx, w, TRI_LNO_B, hvec(t[11], t[11] + c)));
  LF_TRY(upload(ctx, w, TRI_WZ, transposed(t[12], cz, c)));
  LF_TRY(upload(ctx, w, TRI_BZ, hvec(t[13], t[13] + cz)));
  LF_TRY(upload(ctx, w, TRI_WG, transposed(t[14], cz, cz)));
  LF_TRY(upload(ctx, w, TRI_BG, hvec(t[15], t[15] + cz)));
  return LF_OK;
}

lf_status build_triangle_af3(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt) {
  const int cz = w->dims.channels, c = w->dims.hidden;
  if (c != cz) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "AF3 triangle weights need hidden == channels; got %d and %d", c, cz);
  const Expect e[8] = {{"leftNormInputScale", cz}, {"leftNormInputOffset", cz}, {"projection", (int64_t)cz * 2 * c},
                       {"gate", (int64_t)cz * 2 * c}, {"centerNormScale", c}, {"centerNormOffset", c},
                       {"outputProjection", (int64_t)c * cz}, {"gatingLinear", (int64_t)cz * cz}};
  LF_TRY(check_counts(ctx, e, 8, n, nt, t));
  w->f.assign(TRI_COUNT, nullptr);
  // projection / gate are (cz, 2c) with a at column 2h and b at 2h+1
  hvec w4((size_t)cz * 4 * c), b4((size_t)4 * c, 0.f);
  put_columns(w4, 4 * c, 0 * c, t[2], cz, c, 2 * c, 0, 2);
  put_columns(w4, 4 * c, 1 * c, t[3], cz, c, 2 * c, 0, 2);
  put_columns(w4, 4 * c, 2 * c, t[2], cz, c, 2 * c, 1, 2);
  put_columns(w4, 4 * c, 3 * c, t[3], cz, c, 2 * c, 1, 2);
  LF_TRY(upload(ctx, w, TRI_LN_G, hvec(t[0], t[0] + cz)));
  LF_TRY(upload(ctx, w, TRI_LN_B, hvec(t[1], t[1] + cz)));
  LF_TRY(upload(ctx, w, TRI_W4, w4));
  LF_TRY(upload(ctx, w, TRI_B4, b4));
  LF_TRY(upload(ctx, w, TRI_LNO_G, hvec(t[4], t[4] + c)));
  LF_TRY(upload(ctx, w, TRI_LNO_B, hvec(t[5], t[5] + c)));
  LF_TRY(upload(ctx, w, TRI_WZ, hvec(t[6], t[6] + (size_t)c * cz)));
  LF_TRY(upload(ctx, w, TRI_BZ, hvec((size_t)cz, 0.f)));
  LF_TRY(upload(ctx, w, TRI_WG, hvec(t[7], t[7] + (size_t)cz * cz)));
  LF_TRY(upload(ctx, w, TRI_BG, hvec((size_t)cz, 0.f)));
  return LF_OK;
}

// q | k | v | gate columns of the fused projection, plus output projection and pair bias
lf_status finish_attention(lf_context* ctx, lf_weights* w, const float* ln_g, const float* ln_b, const hvec& w4,
                           const hvec& b4, const float* wo, const float* bo, const float* pln_g,
                           const float* pln_b, const float* wb, int pair_ch) {
  const int c = w->dims.channels, H = w->dims.heads, HD = H * w->dims.head_dim;
  w->f.assign(ATT_COUNT, nullptr);
  LF_TRY(upload(ctx, w, ATT_LN_G, hvec(ln_g, ln_g + c)));
  LF_TRY(upload(ctx, w, ATT_LN_B, hvec(ln_b, ln_b + c)));
  LF_TRY(upload(ctx, w, ATT_W4, w4));
  LF_TRY(upload(ctx, w, ATT_B4, b4));
  LF_TRY(upload(ctx, w, ATT_WO, hvec(wo, wo + (size_t)HD * c)));
  LF_TRY(upload(ctx, w, ATT_BO, bo ? hvec(bo, bo + c) : hvec((size_t)c, 0.f)));
  if (pln_g) {
    LF_TRY(upload(ctx, w, ATT_PLN_G, hvec(pln_g, pln_g + pair_ch)));
    LF_TRY(upload(ctx, w, ATT_PLN_B, hvec(pln_b, pln_b + pair_ch)));
    w->has_pair_norm = true;
  }
  if (wb) {
    LF_TRY(upload(ctx, w, ATT_WB, hvec(wb, wb + (size_t)pair_ch * H)));
    w->has_pair_proj = true;
  }
  return LF_OK;
}

lf_status build_attention_af2(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt) {
  const int c = w->dims.channels, H = w->dims.heads;
  if (H <= 0 || c % H != 0) return lf_fail(ctx, LF_ERR_SHAPE, "attention channels %d are not a multiple of heads %d", c, H);
  w->dims.head_dim = c / H;
  const int64_t cc = (int64_t)c * c;
  Expect e[12] = {{"queryNormScale", c}, {"queryNormOffset", c}, {"queryWeight", cc}, {"keyWeight", cc},
                  {"valueWeight", cc}, {"gatingWeight", cc}, {"gatingBias", c}, {"outputWeight", cc},
                  {"outputBias", c}, {"", 0}, {"", 0}, {"", 0}};
  const float *pg = nullptr, *pb = nullptr, *wb = nullptr;
  int pair_ch = 0, expected = 9;
  if (nt == 10) {
    pair_ch = c;
    e[9] = {"pair projection", (int64_t)c * H};
    expected = 10;
  } else if (nt == 12) {
    pair_ch = w->dims.pair_channels;
    if (pair_ch <= 0) return lf_fail(ctx, LF_ERR_ARGUMENT, "separate pair bias needs pair_channels");
    e[9] = {"pair norm scale", pair_ch};
    e[10] = {"pair norm offset", pair_ch};
    e[11] = {"pair projection", (int64_t)pair_ch * H};
    expected = 12;
  }
  LF_TRY(check_counts(ctx, e, expected, n, nt, t));
  if (nt == 10) wb = t[9];
  if (nt == 12) { pg = t[9]; pb = t[10]; wb = t[11]; }
  hvec w4((size_t)c * 4 * c), b4((size_t)4 * c, 0.f);
  for (int r = 0; r < 4; ++r) put_columns(w4, 4 * c, r * c, t[2 + r], c, c, c, 0, 1);
  memcpy(&b4[(size_t)3 * c], t[6], sizeof(float) * c);
  w->has_gate_bias = true;
  w->has_out_bias = true;
  return finish_attention(ctx, w, t[0], t[1], w4, b4, t[7], t[8], pg, pb, wb, pair_ch);
}

lf_status build_grid_attention_af3(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt) {
  const int c = w->dims.channels, H = w->dims.heads, d = w->dims.head_dim, HD = H * d;
  if (H <= 0 || d <= 0) return lf_fail(ctx, LF_ERR_ARGUMENT, "grid attention needs heads and head_dim");
  const Expect e[10] = {{"actNormScale", c}, {"actNormOffset", c}, {"pairBiasProjection", (int64_t)c * H},
                        {"qProjection", (int64_t)HD * c}, {"kProjection", (int64_t)HD * c},
                        {"vProjection", (int64_t)c * HD}, {"gatingQuery", (int64_t)HD * c},
                        {"outputProjection", (int64_t)HD * c}, {"gatingQueryBias", n && nt == 10 ? n[8] : 0},
                        {"outputProjectionBias", n && nt == 10 ? n[9] : 0}};
  LF_TRY(check_counts(ctx, e, 10, n, nt, t));
  if (n[8] != 0 && n[8] != HD) return lf_fail(ctx, LF_ERR_SHAPE, "gatingQueryBias has %lld values; expected %d", (long long)n[8], HD);
  if (n[9] != 0 && n[9] != c) return lf_fail(ctx, LF_ERR_SHAPE, "outputProjectionBias has %lld values; expected %d", (long long)n[9], c);
  hvec w4((size_t)c * 4 * HD), b4((size_t)4 * HD, 0.f);
  hvec q = transposed(t[3], HD, c), k = transposed(t[4], HD, c), g = transposed(t[6], HD, c);
  put_columns(w4, 4 * HD, 0 * HD, q.data(), c, HD, HD, 0, 1);
  put_columns(w4, 4 * HD, 1 * HD, k.data(), c, HD, HD, 0, 1);
  put_columns(w4, 4 * HD, 2 * HD, t[5], c, HD, HD, 0, 1);
  put_columns(w4, 4 * HD, 3 * HD, g.data(), c, HD, HD, 0, 1);
  if (n[8]) { memcpy(&b4[(size_t)3 * HD], t[8], sizeof(float) * HD); w->has_gate_bias = true; }
  w->has_out_bias = n[9] != 0;
  return finish_attention(ctx, w, t[0], t[1], w4, b4, t[7], n[9] ? t[9] : nullptr, nullptr, nullptr, t[2], c);
}

lf_status build_single_attention_af3(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt) {
  const int c = w->dims.channels, H = w->dims.heads, d = w->dims.head_dim, HD = H * d, pc = w->dims.pair_channels;
  if (H <= 0 || d <= 0 || pc <= 0) return lf_fail(ctx, LF_ERR_ARGUMENT, "single attention needs heads, head_dim and pair_channels");
  const Expect e[11] = {{"layerNormScale", c}, {"layerNormOffset", c}, {"qProjection", (int64_t)c * HD}, {"qBias", HD},
                        {"kProjection", (int64_t)c * HD}, {"vProjection", (int64_t)c * HD}, {"gatingQuery", (int64_t)c * HD},
                        {"outputProjection", (int64_t)HD * c}, {"singlePairLogitsNormScale", pc},
                        {"singlePairLogitsNormOffset", pc}, {"singlePairLogitsProjection", (int64_t)pc * H}};
  LF_TRY(check_counts(ctx, e, 11, n, nt, t));
  hvec w4((size_t)c * 4 * HD), b4((size_t)4 * HD, 0.f);
  put_columns(w4, 4 * HD, 0 * HD, t[2], c, HD, HD, 0, 1);
  put_columns(w4, 4 * HD, 1 * HD, t[4], c, HD, HD, 0, 1);
  put_columns(w4, 4 * HD, 2 * HD, t[5], c, HD, HD, 0, 1);
  put_columns(w4, 4 * HD, 3 * HD, t[6], c, HD, HD, 0, 1);
  memcpy(b4.data(), t[3], sizeof(float) * HD);
  return finish_attention(ctx, w, t[0], t[1], w4, b4, t[7], nullptr, t[8], t[9], t[10], pc);
}

// AF3 MSA pair-weighted averaging as the gated attention engine sees it: no query and no key (zero
// columns, so every logit is the pair bias alone), values and gate from the normalised MSA, the pair
// bias from a pair tensor with a LayerNorm of its own.
lf_status build_msa_attention_af3(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt) {
  const int c = w->dims.channels, H = w->dims.heads, d = w->dims.head_dim, HD = H * d, pc = w->dims.pair_channels;
  if (H <= 0 || d <= 0 || pc <= 0) return lf_fail(ctx, LF_ERR_ARGUMENT, "MSA attention needs heads, head_dim and pair_channels");
  const Expect e[8] = {{"actNormScale", c}, {"actNormOffset", c}, {"pairNormScale", pc}, {"pairNormOffset", pc},
                       {"pairLogits", (int64_t)pc * H}, {"vProjection", (int64_t)c * HD}, {"gatingQuery", (int64_t)c * HD},
                       {"outputProjection", (int64_t)HD * c}};
  LF_TRY(check_counts(ctx, e, 8, n, nt, t));
  hvec w4((size_t)c * 4 * HD, 0.f), b4((size_t)4 * HD, 0.f);
  put_columns(w4, 4 * HD, 2 * HD, t[5], c, HD, HD, 0, 1);
  put_columns(w4, 4 * HD, 3 * HD, t[6], c, HD, HD, 0, 1);
  return finish_attention(ctx, w, t[0], t[1], w4, b4, t[7], nullptr, t[2], t[3], t[4], pc);
}

lf_status build_global_attention_af2(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt) {
  const int c = w->dims.channels, H = w->dims.heads;
  if (H <= 0 || nt != 9 || !n || n[6] <= 0 || n[6] % H != 0) return lf_fail(ctx, LF_ERR_SHAPE, "global attention: gatingBias must hold heads x head_dim values");
  const int HD = (int)n[6], d = HD / H;
  w->dims.head_dim = d;
  const Expect e[9] = {{"queryNormScale", c}, {"queryNormOffset", c}, {"queryWeight", (int64_t)c * HD}, {"keyWeight", (int64_t)c * d},
                       {"valueWeight", (int64_t)c * d}, {"gatingWeight", (int64_t)c * HD}, {"gatingBias", HD},
                       {"outputWeight", (int64_t)HD * c}, {"outputBias", c}};
  LF_TRY(check_counts(ctx, e, 9, n, nt, t));
  const int wide = 2 * d + HD;
  hvec w3((size_t)c * wide), b3((size_t)wide, 0.f);
  put_columns(w3, wide, 0, t[3], c, d, d, 0, 1);
  put_columns(w3, wide, d, t[4], c, d, d, 0, 1);
  put_columns(w3, wide, 2 * d, t[5], c, HD, HD, 0, 1);
  memcpy(&b3[(size_t)2 * d], t[6], sizeof(float) * HD);
  w->f.assign(GLB_COUNT, nullptr);
  LF_TRY(upload(ctx, w, GLB_LN_G, hvec(t[0], t[0] + c)));
  LF_TRY(upload(ctx, w, GLB_LN_B, hvec(t[1], t[1] + c)));
  LF_TRY(upload(ctx, w, GLB_WQ, hvec(t[2], t[2] + (size_t)c * HD)));
  LF_TRY(upload(ctx, w, GLB_W3, w3));
  LF_TRY(upload(ctx, w, GLB_B3, b3));
  LF_TRY(upload(ctx, w, GLB_WO, hvec(t[7], t[7] + (size_t)HD * c)));
  LF_TRY(upload(ctx, w, GLB_BO, hvec(t[8], t[8] + c)));
  return LF_OK;
}

lf_status build_transition(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt, bool af3) {
  const int c = w->dims.channels, hdn = w->dims.hidden;
  if (hdn <= 0) return lf_fail(ctx, LF_ERR_ARGUMENT, "transition needs hidden channels");
  w->f.assign(TRN_COUNT, nullptr);
  if (!af3) {
    const Expect e[6] = {{"layerNormScale", c}, {"layerNormOffset", c}, {"firstWeight", (int64_t)c * hdn},
                         {"firstBias", hdn}, {"secondWeight", (int64_t)hdn * c}, {"secondBias", c}};
    LF_TRY(check_counts(ctx, e, 6, n, nt, t));
    LF_TRY(upload(ctx, w, TRN_LN_G, hvec(t[0], t[0] + c)));
    LF_TRY(upload(ctx, w, TRN_LN_B, hvec(t[1], t[1] + c)));
    LF_TRY(upload(ctx, w, TRN_W1, hvec(t[2], t[2] + (size_t)c * hdn)));
    LF_TRY(upload(ctx, w, TRN_B1, hvec(t[3], t[3] + hdn)));
    LF_TRY(upload(ctx, w, TRN_W2, hvec(t[4], t[4] + (size_t)hdn * c)));
    LF_TRY(upload(ctx, w, TRN_B2, hvec(t[5], t[5] + c)));
  } else {
    const Expect e[4] = {{"inputLayerNormScale", c}, {"inputLayerNormOffset", c},
                         {"transition1", (int64_t)c * 2 * hdn}, {"transition2", (int64_t)hdn * c}};
    LF_TRY(check_counts(ctx, e, 4, n, nt, t));
    LF_TRY(upload(ctx, w, TRN_LN_G, hvec(t[0], t[0] + c)));
    LF_TRY(upload(ctx, w, TRN_LN_B, hvec(t[1], t[1] + c)));
    LF_TRY(upload(ctx, w, TRN_W1, hvec(t[2], t[2] + (size_t)c * 2 * hdn)));
    LF_TRY(upload(ctx, w, TRN_B1, hvec((size_t)2 * hdn, 0.f)));
    LF_TRY(upload(ctx, w, TRN_W2, hvec(t[3], t[3] + (size_t)hdn * c)));
    LF_TRY(upload(ctx, w, TRN_B2, hvec((size_t)c, 0.f)));
  }
  return LF_OK;
}

lf_status build_opm_af2(lf_context* ctx, lf_weights* w, const float* const* t, const int64_t* n, int nt) {
  const int cm = w->dims.channels, c = w->dims.hidden, cz = w->dims.out_channels;
  if (c <= 0 || cz <= 0) return lf_fail(ctx, LF_ERR_ARGUMENT, "outer product mean needs hidden and out_channels");
  const Expect e[8] = {{"layerNormScale", cm}, {"layerNormOffset", cm}, {"leftWeight", (int64_t)cm * c}, {"leftBias", c},
                       {"rightWeight", (int64_t)cm * c}, {"rightBias", c}, {"outputWeight", (int64_t)c * c * cz},
                       {"outputBias", cz}};
  LF_TRY(check_counts(ctx, e, 8, n, nt, t));
  w->f.assign(OPM_COUNT, nullptr);
  LF_TRY(upload(ctx, w, OPM_LN_G, hvec(t[0], t[0] + cm)));
  LF_TRY(upload(ctx, w, OPM_LN_B, hvec(t[1], t[1] + cm)));
  LF_TRY(upload(ctx, w, OPM_WL, hvec(t[2], t[2] + (size_t)cm * c)));
  LF_TRY(upload(ctx, w, OPM_BL, hvec(t[3], t[3] + c)));
  LF_TRY(upload(ctx, w, OPM_WR, hvec(t[4], t[4] + (size_t)cm * c)));
  LF_TRY(upload(ctx, w, OPM_BR, hvec(t[5], t[5] + c)));
  LF_TRY(upload(ctx, w, OPM_WOUT, hvec(t[6], t[6] + (size_t)c * c * cz)));
  LF_TRY(upload(ctx, w, OPM_BOUT, hvec(t[7], t[7] + cz)));
  return LF_OK;
}

}  // namespace

// Lays the operator's tensors out in the canonical arrays (staged on the host in g_pending).
static lf_status build_weights(lf_context* ctx, lf_weights* w, const float* const* tensors, const int64_t* counts, int n_tensors) {
  switch (w->kind) {
    case LF_WEIGHTS_TRIANGLE_AF2: return build_triangle_af2(ctx, w, tensors, counts, n_tensors);
    case LF_WEIGHTS_TRIANGLE_AF3: return build_triangle_af3(ctx, w, tensors, counts, n_tensors);
    case LF_WEIGHTS_ATTENTION_AF2: return build_attention_af2(ctx, w, tensors, counts, n_tensors);
    case LF_WEIGHTS_GRID_ATTENTION_AF3: return build_grid_attention_af3(ctx, w, tensors, counts, n_tensors);
    case LF_WEIGHTS_SINGLE_ATTENTION_AF3: return build_single_attention_af3(ctx, w, tensors, counts, n_tensors);
    case LF_WEIGHTS_MSA_ATTENTION_AF3: return build_msa_attention_af3(ctx, w, tensors, counts, n_tensors);
    case LF_WEIGHTS_GLOBAL_ATTENTION_AF2: return build_global_attention_af2(ctx, w, tensors, counts, n_tensors);
    case LF_WEIGHTS_TRANSITION_AF2: return build_transition(ctx, w, tensors, counts, n_tensors, false);
    case LF_WEIGHTS_TRANSITION_AF3: return build_transition(ctx, w, tensors, counts, n_tensors, true);
    case LF_WEIGHTS_OPM_AF2: return build_opm_af2(ctx, w, tensors, counts, n_tensors);
    default: return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown weight kind %d", w->kind);
  }
}

// ---------------------------------------------------------------------------
// Weights from encoded tensors (int5 payloads as they sit in a bundle): the codes go to the device as they
// are and one gather kernel decodes them straight into the canonical arrays, through a layout map that says,
// for every element of every canonical array, which input tensor and which of its elements it is (or that it
// is a constant zero).  The map is derived from the very functions that lay out float32 inputs, by running
// them on stand-in tensors that hold their own element numbers, so the two paths cannot disagree; it
// depends only on the operator's kind and shape and is cached per device.

namespace {

constexpr int kMaxSources = 16;
struct SourceTable {
  const uint8_t* base[kMaxSources];
  const __half* scales[kMaxSources];
  const __half* zeros[kMaxSources];
  int block[kMaxSources];           // 0 = float32 values
};

__global__ void gather_decode_kernel(const int32_t* __restrict__ map, int64_t count, const __grid_constant__ SourceTable src,
                                     float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const int32_t tensor = map[2 * i], index = map[2 * i + 1];
  float v = 0.f;
  if (tensor >= 0) {
    const int block = src.block[tensor];
    if (block == 0) {
      v = reinterpret_cast<const float*>(src.base[tensor])[index];
    } else {
      const int g = index / block, bit = (index - g * block) * 5;
      const uint8_t* codes = src.base[tensor] + (size_t)g * (block * 5 / 8);
      const unsigned two = codes[bit >> 3] | ((unsigned)codes[(bit >> 3) + 1] << 8);
      v = fmaf((float)((two >> (bit & 7)) & 31u), __half2float(src.scales[tensor][g]), __half2float(src.zeros[tensor][g]));
    }
  }
  out[i] = v;
}

struct LayoutMaps {
  std::vector<std::vector<int32_t>> slot;      // per canonical array: (tensor, element) pairs; tensor -1 = zero
  lf_weights flags;                            // what the layout functions set besides the arrays
  int32_t* device[64] = {nullptr};             // per device ordinal: all slots' maps, one after the other
};
std::mutex g_maps_mutex;
std::map<std::vector<int64_t>, LayoutMaps> g_maps;

// Runs the layout functions once per input tensor, that tensor holding 1, 2, 3, ... and the others zeros: a
// canonical element that comes out as v > 0 is element v - 1 of that tensor.
lf_status derive_maps(lf_context* ctx, int kind, const lf_weight_dims& dims, const int64_t* counts, int n, LayoutMaps& maps) {
  std::vector<std::vector<float>> fake(n);
  std::vector<const float*> ptr(n);
  for (int i = 0; i < n; ++i) {
    if (counts[i] >= (1 << 24)) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "tensor %d has %lld elements; encoded tensors are limited to 16777215", i, (long long)counts[i]);
    fake[i].assign((size_t)counts[i], 0.f);
    ptr[i] = counts[i] ? fake[i].data() : nullptr;
  }
  for (int i = 0; i < n; ++i) {
    if (!counts[i]) continue;
    for (int64_t e = 0; e < counts[i]; ++e) fake[i][(size_t)e] = (float)(e + 1);
    lf_weights tmp;
    tmp.kind = kind;
    tmp.dims = dims;
    g_pending.items.clear();
    lf_status s = build_weights(ctx, &tmp, ptr.data(), counts, n);
    if (s != LF_OK) { g_pending.items.clear(); return s; }
    if (maps.slot.empty()) {
      maps.slot.resize(tmp.f.size());
      for (auto& it : g_pending.items) maps.slot[it.slot].assign(it.data.size() * 2, -1);
      maps.flags = tmp;
      maps.flags.f.clear();
    }
    for (auto& it : g_pending.items) {
      auto& m = maps.slot[it.slot];
      for (size_t e = 0; e < it.data.size(); ++e)
        if (it.data[e] > 0.f) { m[2 * e] = i; m[2 * e + 1] = (int32_t)it.data[e] - 1; }
    }
    g_pending.items.clear();
    std::fill(fake[i].begin(), fake[i].end(), 0.f);
  }
  if (maps.slot.empty()) return lf_fail(ctx, LF_ERR_ARGUMENT, "no tensor has any element");
  return LF_OK;
}

}  // namespace

extern "C" {

lf_status lf_weights_create(lf_context* ctx, lf_weight_kind kind, const lf_weight_dims* dims,
                            const float* const* tensors, const int64_t* counts, int32_t n_tensors,
                            lf_weights** out) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!dims || !tensors || !counts || !out) return lf_fail(ctx, LF_ERR_ARGUMENT, "lf_weights_create: null argument");
  *out = nullptr;
  if (dims->channels <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "channels must be a positive integer; received %d", dims->channels);
  cudaSetDevice(ctx->device);
  g_pending.items.clear();
  lf_weights* w = new lf_weights();
  w->ctx = ctx;
  w->kind = (int)kind;
  w->dims = *dims;
  lf_status s = build_weights(ctx, w, tensors, counts, n_tensors);
  if (s == LF_OK) s = finish_uploads(ctx, w);
  if (s == LF_OK) s = tc::prepare_weights(ctx, w);
  g_pending.items.clear();
  if (s != LF_OK) { lf_weights_destroy(w); return s; }
  *out = w;
  return LF_OK;
}

lf_status lf_weights_create_encoded(lf_context* ctx, lf_weight_kind kind, const lf_weight_dims* dims,
                                    const lf_encoded_tensor* tensors, int32_t n_tensors, lf_weights** out) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!dims || !tensors || !out) return lf_fail(ctx, LF_ERR_ARGUMENT, "lf_weights_create_encoded: null argument");
  *out = nullptr;
  if (dims->channels <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "channels must be a positive integer; received %d", dims->channels);
  if (n_tensors <= 0 || n_tensors > kMaxSources) return lf_fail(ctx, LF_ERR_ARGUMENT, "expected 1 to %d tensors; received %d", kMaxSources, n_tensors);
  if (ctx->device < 0 || ctx->device >= 64) return lf_fail(ctx, LF_ERR_ARGUMENT, "device ordinal %d is out of range", ctx->device);
  std::vector<int64_t> counts(n_tensors);
  size_t input_bytes = 0;
  for (int i = 0; i < n_tensors; ++i) {
    const lf_encoded_tensor& t = tensors[i];
    counts[i] = t.count;
    if (t.count < 0 || (t.count > 0 && !t.data)) return lf_fail(ctx, LF_ERR_ARGUMENT, "tensor %d is null", i);
    if (t.dtype == LF_TENSOR_F32) input_bytes += lf_align_up((size_t)t.count * 4 + 4, 256);
    else if (t.dtype == LF_TENSOR_INT5) {
      if (t.block <= 0 || (t.block * 5) % 8) return lf_fail(ctx, LF_ERR_ARGUMENT, "tensor %d: group %d of 5 bits does not pack into whole bytes", i, t.block);
      const uint64_t groups = ((uint64_t)t.count + t.block - 1) / t.block, code_bytes = groups * (t.block * 5 / 8) + 1;
      if (t.scale_offset < code_bytes || t.scale_offset % 2 || t.zero_offset % 2 || t.scale_offset + groups * 2 > t.payload_bytes ||
          t.zero_offset + groups * 2 > t.payload_bytes)
        return lf_fail(ctx, LF_ERR_SHAPE, "tensor %d: int5 payload of %llu bytes does not hold %lld codes, scales and zeros", i,
                       (unsigned long long)t.payload_bytes, (long long)t.count);
      input_bytes += lf_align_up((size_t)t.payload_bytes + 4, 256);
    } else return lf_fail(ctx, LF_ERR_ARGUMENT, "tensor %d has unknown encoding %d", i, t.dtype);
  }
  cudaSetDevice(ctx->device);

  // the layout map of this kind and shape
  std::vector<int64_t> key = {(int64_t)kind, dims->channels, dims->hidden, dims->heads, dims->head_dim, dims->pair_channels, dims->out_channels};
  key.insert(key.end(), counts.begin(), counts.end());
  LayoutMaps* maps = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    auto found = g_maps.find(key);
    if (found == g_maps.end()) {
      LayoutMaps fresh;
      LF_TRY(derive_maps(ctx, (int)kind, *dims, counts.data(), n_tensors, fresh));
      found = g_maps.emplace(key, std::move(fresh)).first;
    }
    maps = &found->second;
    if (!maps->device[ctx->device]) {
      size_t total = 0;
      for (auto& m : maps->slot) total += m.size();
      int32_t* dev = nullptr;
      LF_CUDA(ctx, cudaMalloc(&dev, (total ? total : 1) * sizeof(int32_t)));
      size_t at = 0;
      for (auto& m : maps->slot) {
        if (!m.empty()) LF_CUDA(ctx, cudaMemcpyAsync(dev + at, m.data(), m.size() * sizeof(int32_t), cudaMemcpyHostToDevice, ctx->stream));
        at += m.size();
      }
      LF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
      maps->device[ctx->device] = dev;      // kept for the life of the process: one per operator shape
    }
  }

  // inputs to the device as they are (scratch arena), canonical arrays in one allocation
  LF_TRY(lf_arena_ensure(ctx, input_bytes));
  ArenaCursor cur{ctx, 0, false};
  SourceTable table{};
  for (int i = 0; i < n_tensors; ++i) {
    const lf_encoded_tensor& t = tensors[i];
    if (!t.count) continue;
    const size_t bytes = t.dtype == LF_TENSOR_F32 ? (size_t)t.count * 4 : (size_t)t.payload_bytes;
    uint8_t* dev = cur.take<uint8_t>(bytes + 4);
    LF_CUDA(ctx, cudaMemcpyAsync(dev, t.data, bytes, cudaMemcpyHostToDevice, ctx->stream));
    table.base[i] = dev;
    if (t.dtype == LF_TENSOR_INT5) {
      table.block[i] = t.block;
      table.scales[i] = reinterpret_cast<const __half*>(dev + t.scale_offset);
      table.zeros[i] = reinterpret_cast<const __half*>(dev + t.zero_offset);
    }
  }
  lf_weights* w = new lf_weights();
  w->ctx = ctx;
  w->kind = (int)kind;
  w->dims = maps->flags.dims;
  w->has_gate_bias = maps->flags.has_gate_bias; w->has_out_bias = maps->flags.has_out_bias;
  w->has_pair_norm = maps->flags.has_pair_norm; w->has_pair_proj = maps->flags.has_pair_proj;
  w->f.assign(maps->slot.size(), nullptr);
  size_t total = 0;
  std::vector<size_t> offset;
  for (auto& m : maps->slot) { offset.push_back(total); total += lf_align_up(m.size() / 2 * sizeof(float) + 4, 256); }
  char* base = nullptr;
  cudaError_t e = cudaMalloc(&base, total ? total : 256);
  if (e != cudaSuccess) { cudaGetLastError(); delete w; return lf_fail(ctx, LF_ERR_MEMORY, "weight allocation of %zu bytes refused: %s", total, cudaGetErrorString(e)); }
  w->owned.push_back(base);
  size_t at = 0;
  for (size_t sl = 0; sl < maps->slot.size(); ++sl) {
    const int64_t count = (int64_t)maps->slot[sl].size() / 2;
    float* dst = reinterpret_cast<float*>(base + offset[sl]);
    if (count) {
      gather_decode_kernel<<<lf_ceil_div(count, 256), 256, 0, ctx->stream>>>(maps->device[ctx->device] + at, count, table, dst);
      ctx->launches++;
    }
    w->f[sl] = dst;
    at += maps->slot[sl].size();
  }
  lf_status s = cudaGetLastError() == cudaSuccess ? LF_OK : lf_fail(ctx, LF_ERR_CUDA, "weight decode launch failed");
  g_pending.items.clear();                 // nothing is staged on the host: the repacks read the device arrays
  if (s == LF_OK) s = tc::prepare_weights(ctx, w);
  if (s == LF_OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) s = lf_fail(ctx, LF_ERR_CUDA, "weight decode failed");   // the caller's payloads may go
  if (s != LF_OK) { lf_weights_destroy(w); return s; }
  *out = w;
  return LF_OK;
}

void lf_weights_destroy(lf_weights* w) {
  if (!w) return;
  if (w->ctx) { cudaSetDevice(w->ctx->device); cudaStreamSynchronize(w->ctx->stream); }
  for (void* p : w->owned) cudaFree(p);
  delete w;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// operator plumbing

namespace {

#define LAUNCH(ctx, cur, kernel, grid, block, smem, ...)                     \
  do {                                                                       \
    if (!(cur).dry) {                                                        \
      lf_prof_begin((ctx), LF_KERNEL_SIMT);                                  \
      kernel<<<(grid), (block), (smem), (ctx)->stream>>>(__VA_ARGS__);       \
      lf_prof_end((ctx));                                                    \
      (ctx)->launches++;                                                     \
    }                                                                        \
  } while (0)

void sgemm(lf_context* ctx, ArenaCursor& cur, bool ta, bool tb, int epi, int M, int N, int K, const float* A,
           int64_t lda, int64_t sA, const float* B, int64_t ldb, int64_t sB, float* C, int64_t ldc, int64_t sC,
           const float* bias, int epi_col0, int batch) {
  dim3 grid(lf_ceil_div(M, 64), lf_ceil_div(N, 64), batch), block(256);
#define SG(TA_, TB_, E_) LAUNCH(ctx, cur, (simt::sgemm_kernel<TA_, TB_, E_>), grid, block, 0, M, N, K, A, lda, sA, B, ldb, sB, C, ldc, sC, bias, epi_col0)
  if (!ta && !tb) {
    if (epi == simt::EPI_NONE) SG(false, false, simt::EPI_NONE);
    else if (epi == simt::EPI_RELU) SG(false, false, simt::EPI_RELU);
    else SG(false, false, simt::EPI_SIGMOID_FROM_COL);
  } else if (!ta && tb) SG(false, true, simt::EPI_NONE);
  else if (ta && !tb) SG(true, false, simt::EPI_NONE);
  else SG(true, true, simt::EPI_NONE);
#undef SG
}

// Device views of a call's activation buffers: staged through the arena for
// host-space calls, used in place for device-space calls.
struct Staging {
  lf_context* ctx;
  ArenaCursor* cur;
  bool host;
  struct Out { void* host_ptr; void* dev_ptr; size_t bytes; };
  std::vector<Out> outs;
  const void* in(const void* p, size_t bytes) {
    if (!host || !p) return p;
    char* d = cur->take<char>(bytes);
    if (!cur->dry) cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, ctx->stream);
    return d;
  }
  void* out(void* p, size_t bytes) {
    if (!host) return p;
    char* d = cur->take<char>(bytes);
    if (!cur->dry) outs.push_back({p, d, bytes});
    return d;
  }
  void flush() {
    for (auto& o : outs) cudaMemcpyAsync(o.host_ptr, o.dev_ptr, o.bytes, cudaMemcpyDeviceToHost, ctx->stream);
    outs.clear();
  }
};

size_t dtype_size(int dt) { return dt == LF_DTYPE_BF16 ? 2 : 4; }

// ---- triangle multiplication, float32 SIMT path ----
struct TriArgs {
  int n, cz, c, incoming, variance, residual, divide;
  float eps;
  int act_dtype;
  const void* z; const float* mask; void* out;
  const lf_weights* w;
};

template <typename T>
void tri_f32(lf_context* ctx, ArenaCursor& cur, const TriArgs& a) {
  const int64_t P = (int64_t)a.n * a.n;
  const int cz = a.cz, c = a.c, n = a.n;
  const auto& f = a.w->f;
  float* zn = cur.take<float>(P * cz);
  float* p4 = cur.take<float>(P * 4 * c);
  float* ga = cur.take<float>(P * c);
  float* gb = cur.take<float>(P * c);
  float* x = cur.take<float>(P * c);
  LAUNCH(ctx, cur, (simt::layer_norm_kernel<T>), lf_ceil_div(P, 8), 256, 0, (const T*)a.z, P, cz, f[TRI_LN_G],
         f[TRI_LN_B], a.eps, a.variance, 0, 1, 1, zn);
  sgemm(ctx, cur, false, false, simt::EPI_NONE, (int)P, 4 * c, cz, zn, cz, 0, f[TRI_W4], 4 * c, 0, p4, 4 * c, 0, f[TRI_B4], 0, 1);
  LAUNCH(ctx, cur, (simt::trimul_gate_kernel<float>), dim3(lf_ceil_div(P, 32), lf_ceil_div(c, 32)), dim3(32, 8), 0, p4,
         a.mask, P, c, n, n, ga, gb);
  if (!a.incoming)   // x[i][j] = sum_k a[i][k] b[j][k]
    sgemm(ctx, cur, false, true, 0, n, n, n, ga, n, P, gb, n, P, x, n, P, nullptr, 0, c);
  else               // x[i][j] = sum_k b[k][i] a[k][j]
    sgemm(ctx, cur, true, false, 0, n, n, n, gb, n, P, ga, n, P, x, n, P, nullptr, 0, c);
  // xn reuses p4's storage (p4 is dead), then the two output GEMMs
  float* xn = p4;
  float* proj = p4 + P * c;
  float* gate = p4 + P * c + P * cz;   // needs 4c >= c + 2cz: checked by the caller
  LAUNCH(ctx, cur, (simt::center_norm_kernel<float>), lf_ceil_div(P, 32), 256, (size_t)c * 33 * sizeof(float), x, P, c, n, n,
         f[TRI_LNO_G], f[TRI_LNO_B], a.eps, a.variance, a.divide ? 1.0f / n : 1.0f, xn);
  sgemm(ctx, cur, false, false, 0, (int)P, cz, c, xn, c, 0, f[TRI_WZ], cz, 0, proj, cz, 0, f[TRI_BZ], 0, 1);
  sgemm(ctx, cur, false, false, 0, (int)P, cz, cz, zn, cz, 0, f[TRI_WG], cz, 0, gate, cz, 0, f[TRI_BG], 0, 1);
  LAUNCH(ctx, cur, (simt::finish_kernel<T>), lf_ceil_div(P * cz, 256), 256, 0, proj, gate,
         a.residual ? (const T*)a.z : (const T*)nullptr, P, cz, 0, 1, 1, (T*)a.out);
}

// 16-bit path: float32 LayerNorm statistics and gates, fp16 operands a, b, x with
// float32 accumulation on the tensor cores for the contraction.
template <typename T>
lf_status tri_bf16(lf_context* ctx, ArenaCursor& cur, const TriArgs& a) {
  const int64_t P = (int64_t)a.n * a.n;
  const int cz = a.cz, c = a.c, n = a.n;
  const int ld = (n + 15) / 16 * 16;        // rows start on 32-byte boundaries (TMA needs 16, the 256-bit stores 32)
  const int64_t plane = (int64_t)n * ld;
  const auto& f = a.w->f;
  float* zn = cur.take<float>(P * cz);
  float* p4 = cur.take<float>(P * 4 * c);
  op16* ga = cur.take<op16>(plane * c);
  op16* gb = cur.take<op16>(plane * c);
  op16* x = cur.take<op16>(plane * c);
  if (!tc::ln_gemm_supported(a.w))
    LAUNCH(ctx, cur, (simt::layer_norm_kernel<T>), lf_ceil_div(P, 8), 256, 0, (const T*)a.z, P, cz, f[TRI_LN_G],
           f[TRI_LN_B], a.eps, a.variance, 0, 1, 1, zn);
  if (tc::ln_gemm_supported(a.w)) {
    LF_TRY(tc::triangle_project(ctx, cur, a.z, a.act_dtype, a.mask, n, n, ld, a.variance, a.eps, a.w, ga, gb));
  } else {
    sgemm(ctx, cur, false, false, simt::EPI_NONE, (int)P, 4 * c, cz, zn, cz, 0, f[TRI_W4], 4 * c, 0, p4, 4 * c, 0, f[TRI_B4], 0, 1);
    LAUNCH(ctx, cur, (simt::trimul_gate_kernel<op16>), dim3(lf_ceil_div(P, 32), lf_ceil_div(c, 32)), dim3(32, 8), 0, p4,
           a.mask, P, c, n, ld, ga, gb);
  }
  // x is stored as fp16 scaled by a power of two near 1/sqrt(n) so that sums over n terms
  // stay far from the fp16 limits; the centre LayerNorm undoes the scale exactly.
  const float xscale = ldexpf(1.0f, -(int)(0.5f * log2f((float)n)));
  LF_TRY(tc::contract(ctx, cur, ga, gb, x, n, ld, c, a.incoming, xscale));
  if (tc::ln_gemm_supported(a.w)) {
    const float xs = xscale * (a.divide ? (float)n : 1.0f);
    LF_TRY(tc::triangle_output(ctx, cur, x, n, n, ld, a.eps * xs * xs, a.z, a.act_dtype, a.variance, a.eps, a.w,
                               a.residual ? a.z : nullptr, a.out));
    return LF_OK;
  }
  float* xn = p4;
  float* proj = p4 + P * c;
  float* gate = p4 + P * c + P * cz;
  LAUNCH(ctx, cur, (simt::center_norm_kernel<op16>), lf_ceil_div(P, 32), 256, (size_t)c * 33 * sizeof(float), x, P, c, n, ld,
         f[TRI_LNO_G], f[TRI_LNO_B], a.eps, a.variance, (a.divide ? 1.0f / n : 1.0f) / xscale, xn);
  sgemm(ctx, cur, false, false, 0, (int)P, cz, c, xn, c, 0, f[TRI_WZ], cz, 0, proj, cz, 0, f[TRI_BZ], 0, 1);
  sgemm(ctx, cur, false, false, 0, (int)P, cz, cz, zn, cz, 0, f[TRI_WG], cz, 0, gate, cz, 0, f[TRI_BG], 0, 1);
  LAUNCH(ctx, cur, (simt::finish_kernel<T>), lf_ceil_div(P * cz, 256), 256, 0, proj, gate,
         a.residual ? (const T*)a.z : (const T*)nullptr, P, cz, 0, 1, 1, (T*)a.out);
  return LF_OK;
}

lf_status tri_dispatch(lf_context* ctx, ArenaCursor& cur, const TriArgs& a, int precision) {
  if (precision == LF_PRECISION_BF16 && tc::contract_supported(a.n, a.c)) {
    return a.act_dtype == LF_DTYPE_BF16 ? tri_bf16<bf16>(ctx, cur, a) : tri_bf16<float>(ctx, cur, a);
  }
  if (a.act_dtype == LF_DTYPE_BF16) tri_f32<bf16>(ctx, cur, a); else tri_f32<float>(ctx, cur, a);
  return LF_OK;
}

// ---- attention engine, float32 SIMT path ----
struct AttArgs {
  int batch, Q, ch, heads, d, transpose, variance, residual;
  int bias_mode;       // 0 none, 1 from a separate pair tensor, 2 from the normalised input
  int bias_swap;       // store the bias transposed
  int pair_ch, pair_dtype, pair_variance;
  int mask_mode, clamp;
  int tc_pair_bias;    // 16-bit mode: a separate pair bias is projected on the tensor cores when its weights allow
  float eps, pair_eps;
  int act_dtype;
  const void* act; const float* mask; const void* pair; void* out;
  const lf_weights* w;
};

template <typename T>
void att_f32(lf_context* ctx, ArenaCursor& cur, const AttArgs& a) {
  const int64_t R = (int64_t)a.batch * a.Q;
  const int HD = a.heads * a.d, c = a.ch;
  const auto& f = a.w->f;
  float* nrm = cur.take<float>(R * c);
  float* qkvg = cur.take<float>(R * 4 * HD);
  float* bias = a.bias_mode ? cur.take<float>((int64_t)a.heads * a.Q * a.Q) : nullptr;
  float* o = cur.take<float>(R * HD);
  LAUNCH(ctx, cur, (simt::layer_norm_kernel<T>), lf_ceil_div(R, 8), 256, 0, (const T*)a.act, R, c, f[ATT_LN_G],
         f[ATT_LN_B], a.eps, a.variance, a.transpose, a.batch, a.Q, nrm);
  sgemm(ctx, cur, false, false, simt::EPI_SIGMOID_FROM_COL, (int)R, 4 * HD, c, nrm, c, 0, f[ATT_W4], 4 * HD, 0, qkvg,
        4 * HD, 0, f[ATT_B4], 3 * HD, 1);
  const int64_t QQ = (int64_t)a.Q * a.Q;
  if (a.bias_mode == 1 && a.tc_pair_bias && tc::pair_bias_supported(a.w) && !a.bias_swap) {
    // the pair-sized pass of this operator: LayerNorm of the pair and its projection onto the heads, fp16 out
    const int ldb = (a.Q + 15) / 16 * 16;
    op16* b16 = cur.take<op16>((int64_t)a.heads * a.Q * ldb);
    (void)tc::pair_bias_project(ctx, cur, a.pair, a.pair_dtype, a.Q, a.pair_variance, a.pair_eps, a.heads, a.w, b16, ldb);
    LAUNCH(ctx, cur, simt::widen_bias_kernel, lf_ceil_div(QQ * a.heads, 256), 256, 0, b16, a.heads, a.Q, ldb, bias);
  } else if (a.bias_mode == 1) {
    if (a.pair_dtype == LF_DTYPE_BF16)
      LAUNCH(ctx, cur, (simt::pair_bias_kernel<bf16>), lf_ceil_div(QQ, 8), 256, 0, (const bf16*)a.pair, a.Q, a.pair_ch,
             a.heads, f[ATT_PLN_G], f[ATT_PLN_B], f[ATT_WB], a.pair_eps, a.pair_variance, 0, a.bias_swap, bias);
    else
      LAUNCH(ctx, cur, (simt::pair_bias_kernel<float>), lf_ceil_div(QQ, 8), 256, 0, (const float*)a.pair, a.Q, a.pair_ch,
             a.heads, f[ATT_PLN_G], f[ATT_PLN_B], f[ATT_WB], a.pair_eps, a.pair_variance, 0, a.bias_swap, bias);
  } else if (a.bias_mode == 2) {
    LAUNCH(ctx, cur, (simt::pair_bias_kernel<float>), lf_ceil_div(QQ, 8), 256, 0, nrm, a.Q, c, a.heads, nullptr, nullptr,
           f[ATT_WB], a.eps, a.variance, 1, a.bias_swap, bias);
  }
  size_t smem = (size_t)(2 * 32 * (a.d + 1) + 8 * a.d) * sizeof(float);
  LAUNCH(ctx, cur, simt::attention_kernel, dim3(lf_ceil_div(a.Q, 8), a.batch, a.heads), 256, smem, qkvg, bias, a.mask,
         a.batch, a.Q, a.heads, a.d, a.transpose, a.mask_mode, a.clamp, 1.0f / sqrtf((float)a.d), o);
  float* proj = nrm;   // the normalised input is dead
  sgemm(ctx, cur, false, false, 0, (int)R, c, HD, o, HD, 0, f[ATT_WO], c, 0, proj, c, 0, f[ATT_BO], 0, 1);
  LAUNCH(ctx, cur, (simt::finish_kernel<T>), lf_ceil_div(R * c, 256), 256, 0, proj, (const float*)nullptr,
         a.residual ? (const T*)a.act : (const T*)nullptr, R, c, a.transpose, a.batch, a.Q, (T*)a.out);
}

// 16-bit path: tensor-core LayerNorm + q/k/v/gate/bias projection, then the attention core.
template <typename T>
lf_status att_bf16(lf_context* ctx, ArenaCursor& cur, const AttArgs& a) {
  const int HD = a.heads * a.d, c = a.ch;
  const auto& f = a.w->f;
  const int ldb = (a.Q + 15) / 16 * 16;        // rows and keys padded to whole groups of 16
  const int64_t RP = (int64_t)a.batch * ldb;   // q, k, v, gate and o are stored in 8 x 8 pieces: rows padded per batch row
  op16* q = cur.take<op16>(RP * HD);
  op16* k = cur.take<op16>(RP * HD);
  op16* v = cur.take<op16>(RP * HD);
  op16* g = cur.take<op16>(RP * HD);
  op16* bias = a.bias_mode ? cur.take<op16>((int64_t)a.heads * a.Q * ldb) : nullptr;
  op16* o16 = cur.take<op16>(RP * HD);
  if (ldb != a.Q && !cur.dry) {
    // the padding rows and columns are read (as keys past the end, masked out): they must hold finite values
    if (bias) cudaMemsetAsync(bias, 0, (size_t)a.heads * a.Q * ldb * sizeof(op16), ctx->stream);
    cudaMemsetAsync(k, 0, (size_t)RP * HD * sizeof(op16), ctx->stream);
    cudaMemsetAsync(v, 0, (size_t)RP * HD * sizeof(op16), ctx->stream);
  }
  LF_TRY(tc::attention_project(ctx, cur, a.act, a.act_dtype, a.batch, a.Q, a.transpose, a.variance, a.eps, a.heads, a.d,
                               a.bias_swap, a.w, q, k, v, g, bias, ldb));
  LF_TRY(tc::attention_core(ctx, cur, q, k, v, g, bias, ldb, a.mask, a.batch, a.Q, a.transpose, a.mask_mode, a.clamp, o16));
  LF_TRY(tc::attention_output(ctx, cur, o16, a.batch, a.Q, a.transpose, a.w, a.residual ? a.act : nullptr, a.out, a.act_dtype));
  (void)f; (void)c;
  return LF_OK;
}

// 16-bit GEMM on the tensor cores for activations of any width: out[m][n] = sum_k a[m][k] w[n][k], fp16 operands
// with k contiguous, float32 accumulation, fp16 result (the triangle contraction's kernel on one plane).
lf_status hgemm(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* w, op16* out, int64_t M, int N, int K,
                const float* bias = nullptr, int relu = 0) {
  if (M > 0x7fffffff) return lf_fail(ctx, LF_ERR_SHAPE, "too many rows for one projection");
  return tc::contract_gemm(ctx, cur, a, w, out, (int)M, N, K, bias, relu);
}

// the weights' fp16 [n_out][k] GEMM operands, made when the weights were prepared (null: none for this width)
const op16* gemm_operand(const lf_weights* w, int slot) {
  return slot < (int)w->g.size() ? (const op16*)w->g[slot] : nullptr;
}

bool hgemm_supported(const lf_weights* w) { return gemm_operand(w, 0) && gemm_operand(w, 1) && tc::contract_supported(1, 1); }

// 16-bit path for the shapes the fused projection kernel does not take (MSA row attention with pair bias: c_m = 256,
// 8 heads of 32; MSA column attention): LayerNorm to fp16, the q/k/v/gate projection as one tensor-core GEMM, the
// attention core on four heads at a time (logits, softmax and P V in tensor memory), the output projection as a
// second GEMM, bias and residual in float32.
template <typename T>
lf_status att_mixed(lf_context* ctx, ArenaCursor& cur, const AttArgs& a) {
  const int64_t R = (int64_t)a.batch * a.Q;
  const int HD = a.heads * a.d, c = a.ch, groups = a.heads / 4;
  const auto& f = a.w->f;
  const int ldb = (a.Q + 15) / 16 * 16;
  const int64_t RP = (int64_t)a.batch * ldb;
  op16* nrm = cur.take<op16>(R * c);
  op16* qkvg = cur.take<op16>(R * 4 * HD);
  op16* o = cur.take<op16>(R * HD);
  op16* bias16 = a.bias_mode ? cur.take<op16>((int64_t)a.heads * a.Q * ldb) : nullptr;
  op16* q16 = cur.take<op16>(4 * RP * 128);      // q | k | v | gate of one group of four heads
  op16* k16 = q16 + RP * 128;
  op16* v16 = k16 + RP * 128;
  op16* g16 = v16 + RP * 128;
  op16* o16 = cur.take<op16>(RP * 128);
  LAUNCH(ctx, cur, (simt::layer_norm_kernel<T, op16>), lf_ceil_div(R, 8), 256, 0, (const T*)a.act, R, c, f[ATT_LN_G],
         f[ATT_LN_B], a.eps, a.variance, a.transpose, a.batch, a.Q, nrm);
  LF_TRY(hgemm(ctx, cur, nrm, gemm_operand(a.w, 0), qkvg, R, 4 * HD, c));
  if (ldb != a.Q && !cur.dry) {
    // padding rows and columns are read as keys past the end (masked out): they must hold finite values
    if (bias16) cudaMemsetAsync(bias16, 0, (size_t)a.heads * a.Q * ldb * sizeof(op16), ctx->stream);
    cudaMemsetAsync(k16, 0, (size_t)RP * 128 * sizeof(op16), ctx->stream);
    cudaMemsetAsync(v16, 0, (size_t)RP * 128 * sizeof(op16), ctx->stream);
  }
  if (a.bias_mode == 1)
    LF_TRY(tc::pair_bias_project(ctx, cur, a.pair, a.pair_dtype, a.Q, a.pair_variance, a.pair_eps, a.heads, a.w, bias16, ldb));
  const int64_t pieces = (int64_t)a.batch * ((a.Q + 7) / 8) * 128;      // threads of the repack kernels
  const float qscale = 1.0f / sqrtf((float)a.d);
  for (int gi = 0; gi < groups; ++gi) {
    LAUNCH(ctx, cur, simt::rows_to_pieces_kernel<op16>, dim3((unsigned)lf_ceil_div(pieces, 256), 4), 256, 0, qkvg, HD, gi, f[ATT_B4], qscale,
           a.batch, a.Q, ldb, q16, RP * 128);
    LF_TRY(tc::attention_core(ctx, cur, q16, k16, v16, g16, bias16 ? bias16 + (int64_t)gi * 4 * a.Q * ldb : nullptr, ldb, a.mask, a.batch,
                              a.Q, a.transpose, a.mask_mode, a.clamp, o16));
    LAUNCH(ctx, cur, simt::pieces_to_rows_kernel<op16>, lf_ceil_div(pieces, 256), 256, 0, o16, a.batch, a.Q, ldb, (int64_t)HD, gi * 128, o);
  }
  op16* proj = nrm;   // the normalised input is dead
  LF_TRY(hgemm(ctx, cur, o, gemm_operand(a.w, 1), proj, R, c, HD));
  LAUNCH(ctx, cur, (simt::finish_half_kernel<T>), lf_ceil_div(R * c / 8, 256), 256, 0, proj, 1.0f, f[ATT_BO],
         a.residual ? (const T*)a.act : (const T*)nullptr, R, c, a.transpose, a.batch, a.Q, (T*)a.out);
  return LF_OK;
}

lf_status att_dispatch(lf_context* ctx, ArenaCursor& cur, const AttArgs& a, int precision) {
  if (precision == LF_PRECISION_BF16 && a.bias_mode != 1 && a.heads == 4 && a.d == 32 && tc::ln_gemm_supported(a.w)) {
    return a.act_dtype == LF_DTYPE_BF16 ? att_bf16<bf16>(ctx, cur, a) : att_bf16<float>(ctx, cur, a);
  }
  if (precision == LF_PRECISION_BF16 && a.d == 32 && a.heads % 4 == 0 && hgemm_supported(a.w) &&
      (a.bias_mode == 0 || (a.bias_mode == 1 && tc::pair_bias_supported(a.w) && !a.bias_swap))) {
    return a.act_dtype == LF_DTYPE_BF16 ? att_mixed<bf16>(ctx, cur, a) : att_mixed<float>(ctx, cur, a);
  }
  AttArgs b = a;
  b.tc_pair_bias = precision == LF_PRECISION_BF16 ? 1 : 0;
  if (b.act_dtype == LF_DTYPE_BF16) att_f32<bf16>(ctx, cur, b); else att_f32<float>(ctx, cur, b);
  return LF_OK;
}

// ---- transition, float32 SIMT path (row-chunked so the wide hidden stays bounded) ----
struct TrnArgs {
  int64_t rows; int ch, hidden, swiglu, variance, residual; float eps; int act_dtype;
  const void* act; void* out; const lf_weights* w;
};

template <typename T>
void trn_f32(lf_context* ctx, ArenaCursor& cur, const TrnArgs& a) {
  const auto& f = a.w->f;
  const int c = a.ch, hd = a.hidden, wide = a.swiglu ? 2 * hd : hd;
  const int64_t chunk = a.rows < (1 << 18) ? a.rows : (1 << 18);
  float* nrm = cur.take<float>(chunk * c);
  float* h1 = cur.take<float>(chunk * wide);
  float* h2 = a.swiglu ? cur.take<float>(chunk * hd) : h1;
  float* proj = cur.take<float>(chunk * c);
  for (int64_t r0 = 0; r0 < a.rows; r0 += chunk) {
    int64_t rows = a.rows - r0 < chunk ? a.rows - r0 : chunk;
    const T* in = (const T*)a.act + r0 * c;
    T* out = (T*)a.out + r0 * c;
    LAUNCH(ctx, cur, (simt::layer_norm_kernel<T>), lf_ceil_div(rows, 8), 256, 0, in, rows, c, f[TRN_LN_G], f[TRN_LN_B],
           a.eps, a.variance, 0, 1, 1, nrm);
    sgemm(ctx, cur, false, false, a.swiglu ? simt::EPI_NONE : simt::EPI_RELU, (int)rows, wide, c, nrm, c, 0, f[TRN_W1],
          wide, 0, h1, wide, 0, f[TRN_B1], 0, 1);
    if (a.swiglu) LAUNCH(ctx, cur, simt::swiglu_kernel, lf_ceil_div(rows * hd, 256), 256, 0, h1, rows, hd, h2);
    sgemm(ctx, cur, false, false, 0, (int)rows, c, hd, h2, hd, 0, f[TRN_W2], c, 0, proj, c, 0, f[TRN_B2], 0, 1);
    LAUNCH(ctx, cur, (simt::finish_kernel<T>), lf_ceil_div(rows * c, 256), 256, 0, proj, (const float*)nullptr,
           a.residual ? in : (const T*)nullptr, rows, c, 0, 1, 1, out);
  }
}

// 16-bit path for the widths the fused transition kernel does not take (the MSA transitions, other pair widths):
// LayerNorm to fp16, both projections as tensor-core GEMMs, the hidden activation in place on fp16.
template <typename T>
lf_status trn_half(lf_context* ctx, ArenaCursor& cur, const TrnArgs& a) {
  const auto& f = a.w->f;
  const int c = a.ch, hd = a.hidden, wide = a.swiglu ? 2 * hd : hd, c16 = c + 16;
  const int64_t chunk = a.rows < (1 << 18) ? a.rows : (1 << 18);
  // normalised rows with a column of ones after the channels: the first projection's operand carries its bias there
  op16* nrm = cur.take<op16>(chunk * c16);
  op16* h1 = cur.take<op16>(chunk * wide);
  op16* h2 = a.swiglu ? cur.take<op16>(chunk * hd) : h1;
  const op16* w1 = gemm_operand(a.w, 0);
  const op16* w2 = gemm_operand(a.w, 1);
  for (int64_t r0 = 0; r0 < a.rows; r0 += chunk) {
    int64_t rows = a.rows - r0 < chunk ? a.rows - r0 : chunk;
    const T* in = (const T*)a.act + r0 * c;
    T* out = (T*)a.out + r0 * c;
    LAUNCH(ctx, cur, (simt::layer_norm_kernel<T, op16, true>), lf_ceil_div(rows, 8), 256, 0, in, rows, c, f[TRN_LN_G], f[TRN_LN_B],
           a.eps, a.variance, 0, 1, 1, nrm);
    if (a.swiglu) {
      LF_TRY(hgemm(ctx, cur, nrm, w1, h1, rows, wide, c16));
      LAUNCH(ctx, cur, simt::hidden_act_half_kernel, lf_ceil_div(rows * hd, 256), 256, 0, h1, (const float*)nullptr, rows, hd, wide, 1, h2);
    } else {
      LF_TRY(hgemm(ctx, cur, nrm, w1, h1, rows, wide, c16, nullptr, 1));     // ReLU in the GEMM's epilogue
    }
    LF_TRY(hgemm(ctx, cur, h2, w2, nrm, rows, c, hd));
    LAUNCH(ctx, cur, (simt::finish_half_kernel<T>), lf_ceil_div(rows * c / 8, 256), 256, 0, nrm, 1.0f, f[TRN_B2],
           a.residual ? in : (const T*)nullptr, rows, c, 0, 1, 1, out);
  }
  return LF_OK;
}

lf_status trn_dispatch(lf_context* ctx, ArenaCursor& cur, const TrnArgs& a, int precision) {
  if (precision == LF_PRECISION_BF16 && tc::transition_supported(a.w))
    return tc::transition_run(ctx, cur, a.act, a.act_dtype, a.rows, a.variance, a.eps, a.w, a.residual ? a.act : nullptr, a.out);
  if (precision == LF_PRECISION_BF16 && hgemm_supported(a.w))
    return a.act_dtype == LF_DTYPE_BF16 ? trn_half<bf16>(ctx, cur, a) : trn_half<float>(ctx, cur, a);
  if (a.act_dtype == LF_DTYPE_BF16) trn_f32<bf16>(ctx, cur, a); else trn_f32<float>(ctx, cur, a);
  return LF_OK;
}

// Runs `body` twice: a dry pass that sizes the arena, then the real pass.
template <typename F>
lf_status run_with_arena(lf_context* ctx, lf_result* r, bool timed, F body) {
  cudaSetDevice(ctx->device);
  ArenaCursor dry{ctx, 0, true};
  dry.sized_by_dry_pass = true;
  LF_TRY(body(dry));
  LF_TRY(lf_arena_ensure(ctx, dry.peak));
  uint64_t before = ctx->launches;
  if (timed) cudaEventRecord(ctx->ev0, ctx->stream);
  ArenaCursor cur{ctx, 0, false};
  cur.sized_by_dry_pass = true;
  LF_TRY(body(cur));
  if (cur.peak > ctx->arena_peak) ctx->arena_peak = cur.peak;
  float ms = 0.f;
  if (timed) {
    cudaEventRecord(ctx->ev1, ctx->stream);
    LF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1);
    LF_TRY(tc::check_status(ctx));
  }
  LF_CUDA(ctx, cudaGetLastError());
  if (r) { r->elapsed_ms = ms; r->peak_bytes = ctx->arena_peak; r->launches = (uint32_t)(ctx->launches - before); }
  return LF_OK;
}

lf_status check_common(lf_context* ctx, int variance, int precision, int space, int act_dtype, float eps) {
  if (variance != LF_VARIANCE_TWO_PASS && variance != LF_VARIANCE_FAST)
    return lf_fail(ctx, LF_ERR_ARGUMENT, "variance has no default: pass LF_VARIANCE_TWO_PASS or LF_VARIANCE_FAST");
  if (precision != LF_PRECISION_F32 && precision != LF_PRECISION_BF16) return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown precision %d", precision);
  if (space != LF_SPACE_HOST && space != LF_SPACE_DEVICE) return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown space %d", space);
  if (act_dtype != LF_DTYPE_F32 && act_dtype != LF_DTYPE_BF16) return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown activation dtype %d", act_dtype);
  if (space == LF_SPACE_HOST && act_dtype != LF_DTYPE_F32) return lf_fail(ctx, LF_ERR_ARGUMENT, "host-space activations are float32");
  if (!(eps > 0.f) || !std::isfinite(eps)) return lf_fail(ctx, LF_ERR_ARGUMENT, "epsilon must be finite and positive; received %g", (double)eps);
  return LF_OK;
}

}  // namespace

extern "C" {

lf_status lf_triangle_multiplication_run(lf_context* ctx, const lf_triangle_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->z || !d->mask || !d->out || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "triangle multiplication: null argument");
  if (d->length <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "length must be a positive safe integer; received %d", d->length);
  if (d->c_z <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "cZ must be a positive safe integer; received %d", d->c_z);
  if (d->c_hidden <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "cHidden must be a positive safe integer; received %d", d->c_hidden);
  LF_TRY(check_common(ctx, d->variance, d->precision, d->space, d->act_dtype, d->epsilon));
  const lf_weights* w = d->weights;
  if (w->kind != LF_WEIGHTS_TRIANGLE_AF2 && w->kind != LF_WEIGHTS_TRIANGLE_AF3) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights are not triangle weights");
  if (w->dims.channels != d->c_z || w->dims.hidden != d->c_hidden)
    return lf_fail(ctx, LF_ERR_SHAPE, "weights were packed for cZ %d, cHidden %d; the call has %d, %d", w->dims.channels, w->dims.hidden, d->c_z, d->c_hidden);
  if (4 * d->c_hidden < d->c_hidden + 2 * d->c_z) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "cHidden %d is too small for cZ %d (needs 3*cHidden >= 2*cZ)", d->c_hidden, d->c_z);
  if (d->c_hidden > 512) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "cHidden %d exceeds 512", d->c_hidden);
  const bool host = d->space == LF_SPACE_HOST;
  const size_t P = (size_t)d->length * d->length, es = dtype_size(d->act_dtype);
  return run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    TriArgs a{d->length, d->c_z, d->c_hidden, d->incoming ? 1 : 0, d->variance, d->residual ? 1 : 0, d->divide_by_length ? 1 : 0,
              d->epsilon, d->act_dtype, nullptr, nullptr, nullptr, w};
    a.z = st.in(d->z, P * d->c_z * es);
    a.mask = (const float*)st.in(d->mask, P * sizeof(float));
    a.out = st.out(d->out, P * d->c_z * es);
    LF_TRY(tri_dispatch(ctx, cur, a, d->precision));
    st.flush();
    return LF_OK;
  });
}

lf_status lf_attention_run(lf_context* ctx, const lf_attention_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->activations || !d->mask || !d->out || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "attention: null argument");
  if (d->batch <= 0 || d->query_length <= 0 || d->channels <= 0 || d->heads <= 0)
    return lf_fail(ctx, LF_ERR_SHAPE, "attention dimensions must be positive safe integers");
  LF_TRY(check_common(ctx, d->variance, d->precision, d->space, d->act_dtype, d->epsilon));
  const lf_weights* w = d->weights;
  const bool af3 = w->kind == LF_WEIGHTS_GRID_ATTENTION_AF3;
  if (!af3 && w->kind != LF_WEIGHTS_ATTENTION_AF2) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights are not attention weights");
  if (w->dims.channels != d->channels || w->dims.heads != d->heads)
    return lf_fail(ctx, LF_ERR_SHAPE, "weights were packed for %d channels, %d heads; the call has %d, %d", w->dims.channels, w->dims.heads, d->channels, d->heads);
  const int hd = w->dims.head_dim;
  if (hd > 64) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "head dimension %d exceeds 64", hd);
  AttArgs a{};
  a.batch = d->batch; a.Q = d->query_length; a.ch = d->channels; a.heads = d->heads; a.d = hd;
  a.transpose = d->transpose ? 1 : 0; a.variance = d->variance; a.residual = d->residual ? 1 : 0;
  a.eps = d->epsilon; a.pair_eps = d->epsilon; a.pair_variance = d->variance; a.act_dtype = d->act_dtype; a.w = w;
  a.pair_dtype = d->act_dtype;
  if (af3) {
    if (d->swap_transposed_bias != 0 && d->swap_transposed_bias != 1)
      return lf_fail(ctx, LF_ERR_ARGUMENT, "dialect.swapTransposedBias has no default: pass 0 or 1");
    if (d->batch != d->query_length) return lf_fail(ctx, LF_ERR_SHAPE, "grid attention needs batch == query_length");
    a.bias_mode = 2;
    a.bias_swap = (a.transpose && !d->swap_transposed_bias) ? 1 : 0;
    a.mask_mode = 1; a.clamp = 0;
  } else {
    a.mask_mode = 0; a.clamp = 1;
    if (d->pair_bias == LF_PAIR_BIAS_NONE) a.bias_mode = 0;
    else if (d->pair_bias == LF_PAIR_BIAS_SEPARATE) {
      if (!w->has_pair_norm || !w->has_pair_proj) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights carry no separate pair-bias tensors");
      if (!d->pair_activations) return lf_fail(ctx, LF_ERR_ARGUMENT, "pair activations are null");
      if (d->pair_channels != w->dims.pair_channels) return lf_fail(ctx, LF_ERR_SHAPE, "pair activations have %d channels; expected %d", d->pair_channels, w->dims.pair_channels);
      a.bias_mode = 1; a.pair_ch = d->pair_channels;
    } else if (d->pair_bias == LF_PAIR_BIAS_NORMALIZED_INPUT) {
      if (!w->has_pair_proj || w->has_pair_norm) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights carry no normalized-input pair projection");
      if (d->batch != d->query_length) return lf_fail(ctx, LF_ERR_SHAPE, "normalized-input pair bias needs batch == query_length");
      a.bias_mode = 2;
    } else return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown pair bias source %d", d->pair_bias);
  }
  const bool host = d->space == LF_SPACE_HOST;
  const size_t R = (size_t)d->batch * d->query_length, es = dtype_size(d->act_dtype);
  return run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    AttArgs b = a;
    b.act = st.in(d->activations, R * d->channels * es);
    b.mask = (const float*)st.in(d->mask, R * sizeof(float));
    if (a.bias_mode == 1) b.pair = st.in(d->pair_activations, (size_t)d->query_length * d->query_length * d->pair_channels * es);
    b.out = st.out(d->out, R * d->channels * es);
    LF_TRY(att_dispatch(ctx, cur, b, d->precision));
    st.flush();
    return LF_OK;
  });
}

lf_status lf_transition_run(lf_context* ctx, const lf_transition_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->activations || !d->out || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "transition: null argument");
  if (d->rows <= 0 || d->channels <= 0 || d->hidden <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "transition dimensions must be positive safe integers");
  LF_TRY(check_common(ctx, d->variance, d->precision, d->space, d->act_dtype, d->epsilon));
  const lf_weights* w = d->weights;
  const bool af3 = w->kind == LF_WEIGHTS_TRANSITION_AF3;
  if (!af3 && w->kind != LF_WEIGHTS_TRANSITION_AF2) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights are not transition weights");
  if (w->dims.channels != d->channels || w->dims.hidden != d->hidden)
    return lf_fail(ctx, LF_ERR_SHAPE, "weights were packed for %d channels, %d hidden; the call has %d, %d", w->dims.channels, w->dims.hidden, d->channels, d->hidden);
  const bool host = d->space == LF_SPACE_HOST;
  const size_t bytes = (size_t)d->rows * d->channels * dtype_size(d->act_dtype);
  return run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    TrnArgs a{d->rows, d->channels, d->hidden, af3 ? 1 : 0, d->variance, d->residual ? 1 : 0, d->epsilon, d->act_dtype,
              nullptr, nullptr, w};
    a.act = st.in(d->activations, bytes);
    a.out = st.out(d->out, bytes);
    LF_TRY(trn_dispatch(ctx, cur, a, d->precision));
    st.flush();
    return LF_OK;
  });
}

lf_status lf_outer_product_mean_run(lf_context* ctx, const lf_opm_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->activations || !d->mask || !d->out || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "outer product mean: null argument");
  if (d->sequences <= 0 || d->length <= 0 || d->c_m <= 0 || d->c_outer <= 0 || d->c_z <= 0)
    return lf_fail(ctx, LF_ERR_SHAPE, "outer product mean dimensions must be positive safe integers");
  if (d->c_outer > 32) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "cOuter %d exceeds 32", d->c_outer);
  LF_TRY(check_common(ctx, d->variance, d->precision, d->space, d->act_dtype, d->layer_norm_epsilon));
  const lf_weights* w = d->weights;
  if (w->kind != LF_WEIGHTS_OPM_AF2) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights are not outer-product-mean weights");
  if (w->dims.channels != d->c_m || w->dims.hidden != d->c_outer || w->dims.out_channels != d->c_z)
    return lf_fail(ctx, LF_ERR_SHAPE, "weights were packed for cM %d, cOuter %d, cZ %d", w->dims.channels, w->dims.hidden, w->dims.out_channels);
  const bool host = d->space == LF_SPACE_HOST;
  const int S = d->sequences, N = d->length, cm = d->c_m, c = d->c_outer, cz = d->c_z;
  const int64_t rows = (int64_t)S * N;
  const size_t es = dtype_size(d->act_dtype);
  return run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    const float* msa = (const float*)st.in(d->activations, (size_t)rows * cm * 4);
    const float* mask = (const float*)st.in(d->mask, (size_t)rows * 4);
    const void* resid = nullptr;
    void* out;
    if (host) {
      out = st.out(d->out, (size_t)N * N * cz * es);
      if (d->residual) {   // host residual: the pair is read from the output buffer
        if (!cur.dry) cudaMemcpyAsync(out, d->out, (size_t)N * N * cz * es, cudaMemcpyHostToDevice, ctx->stream);
        resid = out;
      }
    } else { out = d->out; resid = d->residual ? d->out : nullptr; }
    const auto& f = w->f;
    const int ban = d->bias_after_norm ? 1 : 0;
    // 16-bit mode, widths in whole groups of 8: every GEMM of the operator runs on the tensor cores
    const bool tc_full = d->precision == LF_PRECISION_BF16 && c % 8 == 0 && hgemm_supported(w);
    float* nrm = tc_full ? nullptr : cur.take<float>(rows * cm);
    float* left = tc_full ? nullptr : cur.take<float>(rows * c);
    float* right = tc_full ? nullptr : cur.take<float>(rows * c);
    // 16-bit mode: the outer product sum over the sequences, [(i,a)] x [(j,b)] over s, is one tensor-core GEMM
    // (the triangle contraction's kernel in its MN-major form, one plane) with fp16 operands and fp16 sums scaled
    // by a power of two near 1 / S so that they stay far inside fp16 whatever the depth
    const bool tc_outer = d->precision == LF_PRECISION_BF16 && ((int64_t)N * c) % 8 == 0 && tc::contract_supported(N, 1);
    const float outer_scale = tc_outer ? ldexpf(1.0f, -(int)ceilf(log2f((float)S))) : 1.0f;
    // output rows per chunk: bound the [ni*c][N*c] outer-product buffer near 1 GiB
    int64_t per_row = (int64_t)c * N * c * (tc_outer ? 2 : 4);
    int ni = (int)((((int64_t)1 << 30) + per_row - 1) / per_row);
    if (ni > N) ni = N;
    float* outer = tc_outer ? nullptr : cur.take<float>((int64_t)ni * c * N * c);
    op16* outer16 = tc_outer ? cur.take<op16>((int64_t)ni * c * N * c) : nullptr;
    op16* left16 = tc_outer ? cur.take<op16>(rows * c) : nullptr;
    op16* right16 = tc_outer ? cur.take<op16>(rows * c) : nullptr;
    if (tc_full) {
      // LayerNorm to fp16, left | right projection as one GEMM; then per chunk of output rows the outer product
      // summed over the sequences (GEMM over s, stored grouped per pair), projected onto c_z (GEMM over (a, b))
      op16* nrm16 = cur.take<op16>(rows * cm);
      op16* lr16 = cur.take<op16>(rows * 2 * c);
      const op16* wlr = gemm_operand(w, 0);
      const op16* wout = gemm_operand(w, 1);
      op16* proj16 = cur.take<op16>((int64_t)ni * N * cz);
      float* counts = cur.take<float>((int64_t)N * N);
      LAUNCH(ctx, cur, (simt::layer_norm_kernel<float, op16>), lf_ceil_div(rows, 8), 256, 0, msa, rows, cm, f[OPM_LN_G], f[OPM_LN_B],
             d->layer_norm_epsilon, d->variance, 0, 1, 1, nrm16);
      LF_TRY(hgemm(ctx, cur, nrm16, wlr, lr16, rows, 2 * c, cm));
      LAUNCH(ctx, cur, simt::opm_split_half_kernel, lf_ceil_div(rows * c, 256), 256, 0, lr16, f[OPM_BL], f[OPM_BR], mask, rows, c, left16, right16);
      LAUNCH(ctx, cur, simt::opm_counts_kernel, lf_ceil_div((int64_t)((N + 3) / 4) * N, 256), 256, 0, mask, S, N, counts);
      for (int i0 = 0; i0 < N; i0 += ni) {
        int cnt = N - i0 < ni ? N - i0 : ni;
        LF_TRY(tc::contract_outer(ctx, cur, left16 + (int64_t)i0 * c, right16, outer16, cnt, N, c, S, outer_scale));
        LF_TRY(hgemm(ctx, cur, outer16, wout, proj16, (int64_t)cnt * N, cz, c * c));
        if (d->act_dtype == LF_DTYPE_BF16)
          LAUNCH(ctx, cur, (simt::opm_finish_half_kernel<bf16>), lf_ceil_div((int64_t)cnt * N * (cz / 8), 256), 256, 0, proj16, 1.0f / outer_scale,
                 f[OPM_BOUT], counts, N, cz, i0, cnt, d->normalization_epsilon, ban, (const bf16*)resid, (bf16*)out);
        else
          LAUNCH(ctx, cur, (simt::opm_finish_half_kernel<float>), lf_ceil_div((int64_t)cnt * N * (cz / 8), 256), 256, 0, proj16, 1.0f / outer_scale,
                 f[OPM_BOUT], counts, N, cz, i0, cnt, d->normalization_epsilon, ban, (const float*)resid, (float*)out);
      }
      st.flush();
      return LF_OK;
    }
    LAUNCH(ctx, cur, (simt::layer_norm_kernel<float>), lf_ceil_div(rows, 8), 256, 0, msa, rows, cm, f[OPM_LN_G], f[OPM_LN_B],
           d->layer_norm_epsilon, d->variance, 0, 1, 1, nrm);
    sgemm(ctx, cur, false, false, 0, (int)rows, c, cm, nrm, cm, 0, f[OPM_WL], c, 0, left, c, 0, f[OPM_BL], 0, 1);
    sgemm(ctx, cur, false, false, 0, (int)rows, c, cm, nrm, cm, 0, f[OPM_WR], c, 0, right, c, 0, f[OPM_BR], 0, 1);
    if (tc_outer) LAUNCH(ctx, cur, simt::mask_rows_half_kernel, lf_ceil_div(rows * c, 256), 256, 0, left, right, mask, rows, c, left16, right16);
    else LAUNCH(ctx, cur, simt::mask_rows_kernel, lf_ceil_div(rows * c, 256), 256, 0, left, right, mask, rows, c);
    constexpr int JT = 8;
    size_t smem = (size_t)(JT * c * c + JT) * sizeof(float);
    for (int i0 = 0; i0 < N; i0 += ni) {
      int cnt = N - i0 < ni ? N - i0 : ni;
      // outer[(i-i0)*c + a][j*c + b] = sum_s left[s][i][a] * right[s][j][b]
      dim3 grid(lf_ceil_div(N, JT), cnt);
      if (tc_outer) {
        // x[(i,a)][(j,b)] = scale * sum_s left[s][(i,a)] right[s][(j,b)]: rows of the operands are s, so both are
        // MN-major; the kernel's "b" is its M operand
        LF_TRY(tc::contract_rect(ctx, cur, right16, left16 + (int64_t)i0 * c, outer16, cnt * c, N * c, S, N * c, N * c,
                                 (int64_t)cnt * c * N * c, 0, 1, 1, outer_scale));
        if (d->act_dtype == LF_DTYPE_BF16)
          LAUNCH(ctx, cur, (simt::opm_output_kernel<bf16, JT, op16>), grid, 128, smem, outer16, 1.0f / outer_scale, f[OPM_WOUT], f[OPM_BOUT],
                 mask, S, N, c, cz, i0, d->normalization_epsilon, ban, (const bf16*)resid, (bf16*)out);
        else
          LAUNCH(ctx, cur, (simt::opm_output_kernel<float, JT, op16>), grid, 128, smem, outer16, 1.0f / outer_scale, f[OPM_WOUT], f[OPM_BOUT],
                 mask, S, N, c, cz, i0, d->normalization_epsilon, ban, (const float*)resid, (float*)out);
        continue;
      }
      sgemm(ctx, cur, true, false, 0, cnt * c, N * c, S, left + (int64_t)i0 * c, (int64_t)N * c, 0, right, (int64_t)N * c, 0,
            outer, (int64_t)N * c, 0, nullptr, 0, 1);
      if (d->act_dtype == LF_DTYPE_BF16)
        LAUNCH(ctx, cur, (simt::opm_output_kernel<bf16, JT, float>), grid, 128, smem, outer, 1.0f, f[OPM_WOUT], f[OPM_BOUT], mask, S, N, c, cz,
               i0, d->normalization_epsilon, ban, (const bf16*)resid, (bf16*)out);
      else
        LAUNCH(ctx, cur, (simt::opm_output_kernel<float, JT, float>), grid, 128, smem, outer, 1.0f, f[OPM_WOUT], f[OPM_BOUT], mask, S, N, c, cz,
               i0, d->normalization_epsilon, ban, (const float*)resid, (float*)out);
    }
    st.flush();
    return LF_OK;
  });
}

lf_status lf_single_attention_run(lf_context* ctx, const lf_single_attention_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->single || !d->pair || !d->seq_mask || !d->out || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "single attention: null argument");
  if (d->tokens <= 0 || d->channels <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "single attention dimensions must be positive safe integers");
  const lf_weights* w = d->weights;
  if (w->kind != LF_WEIGHTS_SINGLE_ATTENTION_AF3) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights are not single-attention weights");
  if (w->dims.channels != d->channels || w->dims.heads != d->heads || w->dims.head_dim != d->head_dim || w->dims.pair_channels != d->pair_channels)
    return lf_fail(ctx, LF_ERR_SHAPE, "weights were packed for %d channels, %d heads x %d, %d pair channels", w->dims.channels, w->dims.heads, w->dims.head_dim, w->dims.pair_channels);
  LF_TRY(check_common(ctx, LF_VARIANCE_FAST, d->precision, d->space, d->space == LF_SPACE_HOST ? LF_DTYPE_F32 : d->pair_dtype, 1e-5f));
  if (d->head_dim > 64) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "head dimension %d exceeds 64", d->head_dim);
  const bool host = d->space == LF_SPACE_HOST;
  const int n = d->tokens;
  return run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    AttArgs a{};
    a.batch = 1; a.Q = n; a.ch = d->channels; a.heads = d->heads; a.d = d->head_dim; a.transpose = 0;
    a.variance = LF_VARIANCE_FAST; a.residual = d->residual ? 1 : 0; a.bias_mode = 1; a.bias_swap = 0;
    a.pair_ch = d->pair_channels; a.pair_dtype = host ? LF_DTYPE_F32 : d->pair_dtype; a.pair_variance = LF_VARIANCE_FAST;
    a.mask_mode = 0; a.clamp = 0; a.eps = 1e-5f; a.pair_eps = 1e-5f; a.act_dtype = LF_DTYPE_F32; a.w = w;
    a.tc_pair_bias = d->precision == LF_PRECISION_BF16 ? 1 : 0;
    a.act = st.in(d->single, (size_t)n * d->channels * 4);
    a.mask = (const float*)st.in(d->seq_mask, (size_t)n * 4);
    a.pair = st.in(d->pair, (size_t)n * n * d->pair_channels * dtype_size(a.pair_dtype));
    a.out = st.out(d->out, (size_t)n * d->channels * 4);
    att_f32<float>(ctx, cur, a);
    st.flush();
    return LF_OK;
  });
}

lf_status lf_msa_attention_run(lf_context* ctx, const lf_msa_attention_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->msa || !d->msa_mask || !d->pair || !d->out || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "MSA attention: null argument");
  if (d->sequences <= 0 || d->tokens <= 0 || d->channels <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "MSA attention dimensions must be positive safe integers");
  const lf_weights* w = d->weights;
  if (w->kind != LF_WEIGHTS_MSA_ATTENTION_AF3) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights are not MSA attention weights");
  if (w->dims.channels != d->channels || w->dims.heads != d->heads || w->dims.head_dim != d->head_dim || w->dims.pair_channels != d->pair_channels)
    return lf_fail(ctx, LF_ERR_SHAPE, "weights were packed for %d channels, %d heads x %d, %d pair channels", w->dims.channels, w->dims.heads, w->dims.head_dim, w->dims.pair_channels);
  LF_TRY(check_common(ctx, LF_VARIANCE_FAST, d->precision, d->space, d->space == LF_SPACE_HOST ? LF_DTYPE_F32 : d->pair_dtype, 1e-5f));
  if (d->head_dim > 64) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "head dimension %d exceeds 64", d->head_dim);
  const bool host = d->space == LF_SPACE_HOST;
  const int S = d->sequences, n = d->tokens;
  const size_t R = (size_t)S * n;
  return run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    AttArgs a{};
    a.batch = S; a.Q = n; a.ch = d->channels; a.heads = d->heads; a.d = d->head_dim; a.transpose = 0;
    a.variance = LF_VARIANCE_FAST; a.residual = d->residual ? 1 : 0; a.bias_mode = 1; a.bias_swap = 0;
    a.pair_ch = d->pair_channels; a.pair_dtype = host ? LF_DTYPE_F32 : d->pair_dtype; a.pair_variance = LF_VARIANCE_FAST;
    a.mask_mode = 0; a.clamp = 0; a.eps = 1e-5f; a.pair_eps = 1e-5f; a.act_dtype = LF_DTYPE_F32; a.w = w;
    a.tc_pair_bias = d->precision == LF_PRECISION_BF16 ? 1 : 0;
    a.act = st.in(d->msa, R * d->channels * 4);
    const float* msa_mask = (const float*)st.in(d->msa_mask, R * 4);
    float* key_mask = cur.take<float>(R);
    LAUNCH(ctx, cur, simt::msa_key_mask_kernel, lf_ceil_div(n, 128), 128, 0, msa_mask, S, n, key_mask);
    a.mask = key_mask;
    a.pair = st.in(d->pair, (size_t)n * n * d->pair_channels * dtype_size(a.pair_dtype));
    a.out = st.out(d->out, R * d->channels * 4);
    att_f32<float>(ctx, cur, a);
    st.flush();
    return LF_OK;
  });
}

}  // extern "C"

namespace {
template <typename T>
void global_attention(lf_context* ctx, ArenaCursor& cur, const lf_global_attention_desc* d, const void* act, const float* mask,
                      void* out) {
  const lf_weights* w = d->weights;
  const auto& f = w->f;
  const int S = d->sequences, n = d->length, c = d->channels, H = d->heads, hd = w->dims.head_dim, HD = H * hd, wide = 2 * hd + HD;
  const int64_t R = (int64_t)S * n;
  float* nrm = cur.take<float>(R * c);
  float* kvg = cur.take<float>(R * wide);
  float* q = cur.take<float>((int64_t)n * HD);
  float* attended = cur.take<float>((int64_t)n * HD);
  float* gated = cur.take<float>(R * HD);
  LAUNCH(ctx, cur, (simt::layer_norm_kernel<T>), lf_ceil_div(R, 8), 256, 0, (const T*)act, R, c, f[GLB_LN_G], f[GLB_LN_B],
         d->epsilon, d->variance, 0, 1, 1, nrm);
  sgemm(ctx, cur, false, false, simt::EPI_SIGMOID_FROM_COL, (int)R, wide, c, nrm, c, 0, f[GLB_W3], wide, 0, kvg, wide, 0, f[GLB_B3],
        2 * hd, 1);
  LAUNCH(ctx, cur, simt::global_query_kernel, n, 128, (size_t)c * sizeof(float), nrm, mask, S, n, c, HD, 1.0f / sqrtf((float)hd),
         f[GLB_WQ], q);
  LAUNCH(ctx, cur, simt::global_attend_kernel, dim3(n, H), 64, 0, q, kvg, wide, mask, S, n, H, hd, attended);
  LAUNCH(ctx, cur, simt::global_gate_kernel, lf_ceil_div(R * HD, 256), 256, 0, kvg, wide, 2 * hd, attended, R, n, HD, gated);
  float* proj = nrm;   // the normalised input is dead
  sgemm(ctx, cur, false, false, 0, (int)R, c, HD, gated, HD, 0, f[GLB_WO], c, 0, proj, c, 0, f[GLB_BO], 0, 1);
  LAUNCH(ctx, cur, (simt::finish_kernel<T>), lf_ceil_div(R * c, 256), 256, 0, proj, (const float*)nullptr,
         d->residual ? (const T*)act : (const T*)nullptr, R, c, 0, 1, 1, (T*)out);
}
}  // namespace

extern "C" {

lf_status lf_global_column_attention_run(lf_context* ctx, const lf_global_attention_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->activations || !d->mask || !d->out || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "global attention: null argument");
  if (d->sequences <= 0 || d->length <= 0 || d->channels <= 0 || d->heads <= 0)
    return lf_fail(ctx, LF_ERR_SHAPE, "global attention dimensions must be positive safe integers");
  LF_TRY(check_common(ctx, d->variance, d->precision, d->space, d->act_dtype, d->epsilon));
  const lf_weights* w = d->weights;
  if (w->kind != LF_WEIGHTS_GLOBAL_ATTENTION_AF2) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights are not global attention weights");
  if (w->dims.channels != d->channels || w->dims.heads != d->heads)
    return lf_fail(ctx, LF_ERR_SHAPE, "weights were packed for %d channels, %d heads; the call has %d, %d", w->dims.channels, w->dims.heads, d->channels, d->heads);
  if (w->dims.head_dim > 32) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "global attention head dimension %d exceeds 32", w->dims.head_dim);
  const bool host = d->space == LF_SPACE_HOST;
  const size_t R = (size_t)d->sequences * d->length, es = dtype_size(d->act_dtype);
  return run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    const void* act = st.in(d->activations, R * d->channels * es);
    const float* mask = (const float*)st.in(d->mask, R * sizeof(float));
    void* out = st.out(d->out, R * d->channels * es);
    if (d->act_dtype == LF_DTYPE_BF16) global_attention<bf16>(ctx, cur, d, act, mask, out);
    else global_attention<float>(ctx, cur, d, act, mask, out);
    st.flush();
    return LF_OK;
  });
}

lf_status lf_distogram_logits_run(lf_context* ctx, const lf_distogram_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->pair || !d->half_logits || !d->out) return lf_fail(ctx, LF_ERR_ARGUMENT, "distogram: null argument");
  if (d->tokens <= 0 || d->channels <= 0 || d->bins <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "distogram dimensions must be positive safe integers");
  LF_TRY(check_common(ctx, LF_VARIANCE_FAST, LF_PRECISION_F32, d->space, d->space == LF_SPACE_HOST ? LF_DTYPE_F32 : d->pair_dtype, 1e-5f));
  const bool host = d->space == LF_SPACE_HOST;
  const int n = d->tokens, c = d->channels, bins = d->bins;
  const size_t P = (size_t)n * n;
  const int dt = host ? LF_DTYPE_F32 : d->pair_dtype;
  if (dt != LF_DTYPE_F32) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "distogram logits take a float32 pair");
  return run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    const void* pair = st.in(d->pair, P * c * dtype_size(dt));
    const float* w = (const float*)st.in(d->half_logits, (size_t)c * bins * 4);
    const float* bias = d->bias ? (const float*)st.in(d->bias, (size_t)bins * 4) : nullptr;
    float* out = (float*)st.out(d->out, P * bins * 4);
    const float* x = (const float*)pair;
    float* half = cur.take<float>(P * bins);
    sgemm(ctx, cur, false, false, 0, (int)P, bins, c, x, c, 0, w, bins, 0, half, bins, 0, bias, 0, 1);
    LAUNCH(ctx, cur, simt::symmetrise_sum_kernel, lf_ceil_div((int64_t)P * bins, 256), 256, 0, half, n, bins, out);
    st.flush();
    return LF_OK;
  });
}

lf_status lf_pair_stack_run(lf_context* ctx, const lf_pair_stack_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->pair || !d->mask || !d->blocks) return lf_fail(ctx, LF_ERR_ARGUMENT, "pair stack: null argument");
  if (d->length <= 0 || d->c_z <= 0 || d->c_hidden <= 0 || d->heads <= 0 || d->transition_hidden <= 0)
    return lf_fail(ctx, LF_ERR_SHAPE, "pair stack dimensions must be positive safe integers");
  if (d->first_block < 0 || d->n_blocks < 0 || d->first_block + d->n_blocks > d->block_count)
    return lf_fail(ctx, LF_ERR_ARGUMENT, "blocks [%d, %d) are outside the table of %d", d->first_block, d->first_block + d->n_blocks, d->block_count);
  LF_TRY(check_common(ctx, d->variance, d->precision, d->space, d->act_dtype, d->epsilon));
  if (d->order != LF_ORDER_EVOFORMER && d->order != LF_ORDER_TEMPLATE) return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown block order %d", d->order);
  if (d->c_z % d->heads != 0) return lf_fail(ctx, LF_ERR_SHAPE, "cZ %d is not a multiple of heads %d", d->c_z, d->heads);
  for (int b = d->first_block; b < d->first_block + d->n_blocks; ++b) {
    const lf_pair_block_weights& bw = d->blocks[b];
    if (!bw.triangle_outgoing || !bw.triangle_incoming || !bw.attention_starting || !bw.attention_ending || !bw.transition)
      return lf_fail(ctx, LF_ERR_ARGUMENT, "block %d has a null weight handle", b);
    const bool af3 = bw.attention_starting->kind == LF_WEIGHTS_GRID_ATTENTION_AF3;
    if (af3 && d->swap_transposed_bias != 0 && d->swap_transposed_bias != 1)
      return lf_fail(ctx, LF_ERR_ARGUMENT, "dialect.swapTransposedBias has no default: pass 0 or 1");
    if (!af3 && (bw.attention_starting->has_pair_norm || !bw.attention_starting->has_pair_proj))
      return lf_fail(ctx, LF_ERR_ARGUMENT, "block %d: triangle attention needs a normalized-input pair projection", b);
  }
  const bool host = d->space == LF_SPACE_HOST;
  const int n = d->length, cz = d->c_z;
  const size_t P = (size_t)n * n, es = dtype_size(d->act_dtype);
  const lf_status status = run_with_arena(ctx, r, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, host};
    void* pair = host ? st.out(d->pair, P * cz * es) : d->pair;
    if (host && !cur.dry) cudaMemcpyAsync(pair, d->pair, P * cz * es, cudaMemcpyHostToDevice, ctx->stream);
    const float* mask = (const float*)st.in(d->mask, P * 4);
    const size_t scratch_base = cur.offset;
    for (int b = d->first_block; b < d->first_block + d->n_blocks; ++b) {
      const lf_pair_block_weights& bw = d->blocks[b];
      auto triangles = [&]() -> lf_status {
        for (int dir = 0; dir < 2; ++dir) {
          cur.offset = scratch_base;
          TriArgs a{n, cz, d->c_hidden, dir, d->variance, 1, 0, d->epsilon, d->act_dtype, pair, mask, pair,
                    dir ? bw.triangle_incoming : bw.triangle_outgoing};
          LF_TRY(tri_dispatch(ctx, cur, a, d->precision));
        }
        return LF_OK;
      };
      auto attentions = [&]() -> lf_status {
        for (int t = 0; t < 2; ++t) {
          cur.offset = scratch_base;
          const lf_weights* w = t ? bw.attention_ending : bw.attention_starting;
          const bool af3 = w->kind == LF_WEIGHTS_GRID_ATTENTION_AF3;
          AttArgs a{};
          a.batch = n; a.Q = n; a.ch = cz; a.heads = d->heads; a.d = w->dims.head_dim; a.transpose = t;
          a.variance = d->variance; a.residual = 1; a.bias_mode = 2;
          a.bias_swap = (af3 && t && !d->swap_transposed_bias) ? 1 : 0;
          a.mask_mode = af3 ? 1 : 0; a.clamp = af3 ? 0 : 1; a.eps = d->epsilon; a.pair_eps = d->epsilon;
          a.pair_variance = d->variance; a.act_dtype = d->act_dtype; a.pair_dtype = d->act_dtype;
          a.act = pair; a.mask = mask; a.out = pair; a.w = w;
          LF_TRY(att_dispatch(ctx, cur, a, d->precision));
        }
        return LF_OK;
      };
      if (d->order == LF_ORDER_TEMPLATE) { LF_TRY(attentions()); LF_TRY(triangles()); }
      else { LF_TRY(triangles()); LF_TRY(attentions()); }
      cur.offset = scratch_base;
      TrnArgs a{(int64_t)P, cz, d->transition_hidden, bw.transition->kind == LF_WEIGHTS_TRANSITION_AF3 ? 1 : 0, d->variance, 1,
                d->epsilon, d->act_dtype, pair, pair, bw.transition};
      LF_TRY(trn_dispatch(ctx, cur, a, d->precision));
    }
    st.flush();
    return LF_OK;
  });
  // The device cannot hold the pair beside the operators' scratch: leave the pair in the caller's buffer and stream it through in chunks.
  if (status == LF_ERR_MEMORY && host) return lf_pair_stack_spilled(ctx, d, r);
  return status;
}

lf_status lf_pair_shard_step(lf_context* ctx, const lf_shard_step_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "shard step: null argument");
  if (d->rows <= 0 || d->length <= 0 || d->ranks <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "shard dimensions must be positive safe integers");
  if (d->act_dtype != LF_DTYPE_F32 && d->act_dtype != LF_DTYPE_BF16) return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown activation dtype %d", d->act_dtype);
  const lf_weights* w = d->weights;
  const int R = d->rows, n = d->length, ld = (n + 15) / 16 * 16;
  const bool tri = d->op >= LF_SHARD_TRIANGLE_PROJECT && d->op <= LF_SHARD_TRIANGLE_OUTPUT;
  const bool att = d->op >= LF_SHARD_ATTENTION_PROJECT && d->op <= LF_SHARD_ATTENTION_OUTPUT;
  if (tri && !((w->kind == LF_WEIGHTS_TRIANGLE_AF2 || w->kind == LF_WEIGHTS_TRIANGLE_AF3) && tc::ln_gemm_supported(w)))
    return lf_fail(ctx, LF_ERR_UNSUPPORTED, "shard step needs triangle weights with cZ = cHidden = 128");
  if (att && !(w->kind == LF_WEIGHTS_ATTENTION_AF2 && tc::ln_gemm_supported(w) && w->dims.heads == 4 && w->has_pair_proj && !w->has_pair_norm))
    return lf_fail(ctx, LF_ERR_UNSUPPORTED, "shard step needs AF2 attention weights: 128 channels, 4 heads, normalized-input pair bias");
  if (d->op == LF_SHARD_TRANSITION && !tc::transition_supported(w))
    return lf_fail(ctx, LF_ERR_UNSUPPORTED, "shard step needs transition weights 128 -> 512 -> 128");
  if ((tri || d->op == LF_SHARD_ATTENTION_PROJECT) && d->variance != LF_VARIANCE_TWO_PASS && d->variance != LF_VARIANCE_FAST)
    return lf_fail(ctx, LF_ERR_ARGUMENT, "variance has no default: pass LF_VARIANCE_TWO_PASS or LF_VARIANCE_FAST");
  cudaSetDevice(ctx->device);
  const uint64_t before = ctx->launches;
  ArenaCursor cur{ctx, 0, false};
  const float xscale = ldexpf(1.0f, -(int)(0.5f * log2f((float)n)));
  op16** b = (op16**)d->buf;
  lf_status s = LF_OK;
  switch (d->op) {
    case LF_SHARD_TRIANGLE_PROJECT:
      if (!d->pair || !d->mask || !b[0] || !b[1]) return lf_fail(ctx, LF_ERR_ARGUMENT, "triangle project: null buffer");
      s = tc::triangle_project(ctx, cur, d->pair, d->act_dtype, d->mask, R, n, ld, d->variance, d->epsilon, w, b[0], b[1]);
      break;
    case LF_SHARD_TRIANGLE_CONTRACT:
      if (!b[0] || !b[1] || !b[2]) return lf_fail(ctx, LF_ERR_ARGUMENT, "triangle contract: null buffer");
      if (d->chunk < 0 || d->chunk >= d->ranks) return lf_fail(ctx, LF_ERR_ARGUMENT, "chunk %d is outside %d ranks", d->chunk, d->ranks);
      if (d->ranks > 1 && R % 16 != 0) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "sharded rows must be a multiple of 16; received %d", R);
      s = tc::contract_rect(ctx, cur, b[0], b[1], b[2], R, d->ranks > 1 ? R : n, n, ld, ld, (int64_t)R * ld, d->chunk * R, 128, 0, xscale);
      break;
    case LF_SHARD_TRIANGLE_OUTPUT:
      if (!d->pair || !b[2]) return lf_fail(ctx, LF_ERR_ARGUMENT, "triangle output: null buffer");
      s = tc::triangle_output(ctx, cur, b[2], R, n, ld, d->epsilon * xscale * xscale, d->pair, d->act_dtype, d->variance, d->epsilon, w, d->pair, d->pair);
      break;
    case LF_SHARD_ATTENTION_PROJECT:
      if (!d->pair || !b[0] || !b[1] || !b[2] || !b[3] || !b[4]) return lf_fail(ctx, LF_ERR_ARGUMENT, "attention project: null buffer");
      s = tc::attention_project(ctx, cur, d->pair, d->act_dtype, R, n, 0, d->variance, d->epsilon, 4, 32, 0, w, b[0], b[1], b[2], b[3], b[4], ld);
      break;
    case LF_SHARD_ATTENTION_CORE:
      if (!d->mask || !b[0] || !b[1] || !b[2] || !b[3] || !b[4] || !b[5]) return lf_fail(ctx, LF_ERR_ARGUMENT, "attention core: null buffer");
      s = tc::attention_core(ctx, cur, b[0], b[1], b[2], b[3], b[4], ld, d->mask, R, n, 0, 0, 1, b[5]);
      break;
    case LF_SHARD_ATTENTION_OUTPUT:
      if (!d->pair || !b[5]) return lf_fail(ctx, LF_ERR_ARGUMENT, "attention output: null buffer");
      s = tc::attention_output(ctx, cur, b[5], R, n, 0, w, d->pair, d->pair, d->act_dtype);
      break;
    case LF_SHARD_TRANSITION:
      if (!d->pair) return lf_fail(ctx, LF_ERR_ARGUMENT, "transition: null buffer");
      s = tc::transition_run(ctx, cur, d->pair, d->act_dtype, (int64_t)R * n, d->variance, d->epsilon, w, d->pair, d->pair);
      break;
    default: return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown shard step %d", d->op);
  }
  if (s != LF_OK) return s;
  LF_CUDA(ctx, cudaGetLastError());
  if (r) { r->elapsed_ms = 0.f; r->peak_bytes = ctx->arena_peak; r->launches = (uint32_t)(ctx->launches - before); }
  return LF_OK;
}

lf_status lf_pair_shard_exchange_step(lf_context* ctx, const lf_shard_step_desc* d, const lf_shard_peers* peers, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->weights || !peers) return lf_fail(ctx, LF_ERR_ARGUMENT, "exchange step: null argument");
  if (d->rows <= 0 || d->length <= 0 || d->ranks <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "shard dimensions must be positive safe integers");
  if (d->ranks > tc::kMaxPeers || 128 % d->ranks != 0) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "exchange step: %d ranks do not divide 128 channels", d->ranks);
  if (peers->rank < 0 || peers->rank >= d->ranks) return lf_fail(ctx, LF_ERR_ARGUMENT, "exchange step: rank %d of %d", peers->rank, d->ranks);
  if ((int64_t)d->rows * d->ranks != d->length) return lf_fail(ctx, LF_ERR_SHAPE, "exchange step: rows %d x ranks %d must equal length %d", d->rows, d->ranks, d->length);
  if (d->length % 16 != 0 || (d->ranks > 1 && d->rows % 128 != 0))
    return lf_fail(ctx, LF_ERR_UNSUPPORTED, "exchange step: length must be a multiple of 16 and rows a multiple of 128; received %d, %d", d->length, d->rows);
  if (d->act_dtype != LF_DTYPE_F32 && d->act_dtype != LF_DTYPE_BF16) return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown activation dtype %d", d->act_dtype);
  const lf_weights* w = d->weights;
  const int R = d->rows, n = d->length, ld = n, G = d->ranks, rank = peers->rank, cpr = 128 / G;
  auto table = [&](void* const* src, tc::PeerPtrs& out, const char* name) -> lf_status {
    for (int g = 0; g < G; ++g) {
      if (!src[g]) return lf_fail(ctx, LF_ERR_ARGUMENT, "exchange step: %s buffer of rank %d is null", name, g);
      out.p[g] = src[g];
    }
    return LF_OK;
  };
  cudaSetDevice(ctx->device);
  const uint64_t before = ctx->launches;
  ArenaCursor cur{ctx, 0, false};
  const float xscale = ldexpf(1.0f, -(int)(0.5f * log2f((float)n)));
  lf_status s = LF_OK;
  switch (d->op) {
    case LF_SHARD_TRIANGLE_PROJECT: {
      if (!((w->kind == LF_WEIGHTS_TRIANGLE_AF2 || w->kind == LF_WEIGHTS_TRIANGLE_AF3) && tc::ln_gemm_supported(w)))
        return lf_fail(ctx, LF_ERR_UNSUPPORTED, "exchange step needs triangle weights with cZ = cHidden = 128");
      if (d->variance != LF_VARIANCE_TWO_PASS && d->variance != LF_VARIANCE_FAST)
        return lf_fail(ctx, LF_ERR_ARGUMENT, "variance has no default: pass LF_VARIANCE_TWO_PASS or LF_VARIANCE_FAST");
      if (!d->pair || !d->mask) return lf_fail(ctx, LF_ERR_ARGUMENT, "triangle project: null buffer");
      tc::PeerPtrs pa{}, pb{};
      LF_TRY(table(peers->a, pa, "a"));
      LF_TRY(table(peers->b, pb, "b"));
      s = tc::triangle_project_scatter(ctx, cur, d->pair, d->act_dtype, d->mask, R, n, ld, d->variance, d->epsilon, w, pa, pb, G, rank * R);
      break;
    }
    case LF_SHARD_TRIANGLE_CONTRACT: {
      tc::PeerPtrs px{};
      LF_TRY(table(peers->x, px, "x"));
      if (!peers->a[rank] || !peers->b[rank]) return lf_fail(ctx, LF_ERR_ARGUMENT, "triangle contract: null operand buffer");
      s = tc::contract_scatter(ctx, cur, (const op16*)peers->a[rank], (const op16*)peers->b[rank], n, ld, cpr, peers->incoming ? 1 : 0,
                               xscale, px, R, 128, rank * cpr);
      break;
    }
    case LF_SHARD_ATTENTION_PROJECT: {
      if (!(w->kind == LF_WEIGHTS_ATTENTION_AF2 && tc::ln_gemm_supported(w) && w->dims.heads == 4 && w->has_pair_proj && !w->has_pair_norm))
        return lf_fail(ctx, LF_ERR_UNSUPPORTED, "exchange step needs AF2 attention weights: 128 channels, 4 heads, normalized-input pair bias");
      if (d->variance != LF_VARIANCE_TWO_PASS && d->variance != LF_VARIANCE_FAST)
        return lf_fail(ctx, LF_ERR_ARGUMENT, "variance has no default: pass LF_VARIANCE_TWO_PASS or LF_VARIANCE_FAST");
      op16** b = (op16**)d->buf;
      if (!d->pair || !b[0] || !b[1] || !b[2] || !b[3]) return lf_fail(ctx, LF_ERR_ARGUMENT, "attention project: null buffer");
      tc::PeerPtrs pbias{};
      LF_TRY(table(peers->bias, pbias, "bias"));
      s = tc::attention_project_scatter(ctx, cur, d->pair, d->act_dtype, R, n, d->variance, d->epsilon, 4, w, b[0], b[1], b[2], b[3],
                                        pbias, G, n, rank * R, ld);
      break;
    }
    default: return lf_fail(ctx, LF_ERR_ARGUMENT, "exchange step: step %d has no exchange form", d->op);
  }
  if (s != LF_OK) return s;
  LF_CUDA(ctx, cudaGetLastError());
  if (r) { r->elapsed_ms = 0.f; r->peak_bytes = ctx->arena_peak; r->launches = (uint32_t)(ctx->launches - before); }
  return LF_OK;
}

lf_status lf_int5_decode(lf_context* ctx, const uint8_t* payload, uint64_t payload_bytes, uint64_t scale_offset,
                         uint64_t zero_offset, int64_t elements, int32_t block, lf_space out_space, float* out) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!payload || !out) return lf_fail(ctx, LF_ERR_ARGUMENT, "int5 decode: null argument");
  if (elements <= 0 || block <= 0 || (block * 5) % 8 != 0) return lf_fail(ctx, LF_ERR_ARGUMENT, "group %d of 5 bits does not pack into whole bytes", block);
  const int64_t groups = (elements + block - 1) / block;
  const uint64_t code_bytes = (uint64_t)groups * (block * 5 / 8) + 1;   // one slack byte
  if (scale_offset < code_bytes || scale_offset % 2 || zero_offset < scale_offset + (uint64_t)groups * 2 || zero_offset % 2 ||
      zero_offset + (uint64_t)groups * 2 > payload_bytes)
    return lf_fail(ctx, LF_ERR_SHAPE, "int5 payload of %llu bytes does not hold %lld codes, scales and zeros", (unsigned long long)payload_bytes, (long long)elements);
  const bool host = out_space == LF_SPACE_HOST;
  return run_with_arena(ctx, nullptr, host, [&](ArenaCursor& cur) -> lf_status {
    Staging st{ctx, &cur, true};
    const uint8_t* dev = (const uint8_t*)st.in(payload, payload_bytes);
    float* o = host ? (float*)st.out(out, (size_t)elements * 4) : out;
    LAUNCH(ctx, cur, simt::int5_decode_kernel, lf_ceil_div(elements, 256), 256, 0, dev, (const __half*)(dev + scale_offset),
           (const __half*)(dev + zero_offset), elements, block, o);
    st.flush();
    if (!host && !cur.dry) cudaStreamSynchronize(ctx->stream);   // `payload` may be freed by the caller
    return LF_OK;
  });
}

}  // extern "C"
