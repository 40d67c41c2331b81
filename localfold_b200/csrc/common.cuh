// Shared host-side plumbing of the pair-stack library: context, scratch arena,
// resident weights, error reporting.  No torch types anywhere in this library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../include/localfold_pairstack.h"

typedef __nv_bfloat16 bf16;
// Operand type of the tensor-core kernels: fp16 (11-bit significand) for the bounded
// intermediates (normalised activations, gated projections, probabilities); products
// accumulate in float32.  The pair stream itself is float32 or bf16.
typedef __half op16;

struct lf_context {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool owns_stream = false;
  std::string error;
  // Scratch arena: one device allocation, bump-allocated per operator call.
  char* arena = nullptr;
  size_t arena_bytes = 0;
  size_t arena_used = 0;
  size_t arena_peak = 0;
  size_t arena_limit = 0;      // 0 = none; otherwise requests above it are refused without asking the driver (lf_context_limit_scratch)
  uint64_t launches = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  int sm_count = 148;
  void* tc_status = nullptr;   // device word the tensor-core kernels set when a bounded wait expires
  // Optional per-kernel-family timing (CUDA events on the context's stream).
  bool profiling = false;
  struct Timed { int family; cudaEvent_t start, stop; };
  std::vector<Timed> timed;
  double family_ms[LF_KERNEL_FAMILY_COUNT] = {0};
  uint64_t family_launches[LF_KERNEL_FAMILY_COUNT] = {0};
};

static inline void lf_prof_begin(lf_context* ctx, int family) {
  if (!ctx->profiling) return;
  lf_context::Timed t{family, nullptr, nullptr};
  cudaEventCreate(&t.start);
  cudaEventCreate(&t.stop);
  cudaEventRecord(t.start, ctx->stream);
  ctx->timed.push_back(t);
}
static inline void lf_prof_end(lf_context* ctx) {
  if (!ctx->profiling || ctx->timed.empty()) return;
  cudaEventRecord(ctx->timed.back().stop, ctx->stream);
}

// Slots of lf_weights::f per operator kind.
enum { TRI_LN_G, TRI_LN_B, TRI_W4, TRI_B4, TRI_LNO_G, TRI_LNO_B, TRI_WZ, TRI_BZ, TRI_WG, TRI_BG, TRI_COUNT };
enum { ATT_LN_G, ATT_LN_B, ATT_W4, ATT_B4, ATT_WO, ATT_BO, ATT_PLN_G, ATT_PLN_B, ATT_WB, ATT_COUNT };
enum { TRN_LN_G, TRN_LN_B, TRN_W1, TRN_B1, TRN_W2, TRN_B2, TRN_COUNT };
enum { OPM_LN_G, OPM_LN_B, OPM_WL, OPM_BL, OPM_WR, OPM_BR, OPM_WOUT, OPM_BOUT, OPM_COUNT };
// global column attention: W3 = (key | value | gate) columns, B3 their biases (zero but for the gate)
enum { GLB_LN_G, GLB_LN_B, GLB_WQ, GLB_W3, GLB_B3, GLB_WO, GLB_BO, GLB_COUNT };

// Canonical device-resident weights.  Every linear is stored (in,out) row-major
// float32 in `f[...]`; tensor-core kernels keep extra fp16 repacks (swizzled operand images) in `h[...]`.
struct lf_weights {
  lf_context* ctx = nullptr;
  int kind = 0;
  lf_weight_dims dims{};
  std::vector<float*> f;     // named by the per-kind enums in weights.cuh
  std::vector<void*> h;      // fp16 repacks (tensor-core path)
  std::vector<void*> g;      // fp16 [n_out][k] operands of the plain tensor-core GEMM (widths the fused kernels do not take)
  std::vector<void*> owned;  // every device allocation, for destroy
  int bias_flags = 0;        // per 128-column group of the fused projection: bias is non-zero
  bool has_gate_bias = false, has_out_bias = false, has_pair_norm = false, has_pair_proj = false;
};

static inline lf_status lf_fail(lf_context* ctx, lf_status code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->error = buf;
  return code;
}

#define LF_CUDA(ctx, expr)                                                             \
  do {                                                                                 \
    cudaError_t e_ = (expr);                                                           \
    if (e_ != cudaSuccess)                                                             \
      return lf_fail((ctx), e_ == cudaErrorMemoryAllocation ? LF_ERR_MEMORY : LF_ERR_CUDA, \
                     "%s failed: %s", #expr, cudaGetErrorString(e_));                  \
  } while (0)

#define LF_TRY(expr)                  \
  do {                                \
    lf_status s_ = (expr);            \
    if (s_ != LF_OK) return s_;       \
  } while (0)

// Bump allocation out of the arena.  Sizing happens before any kernel of the
// call is enqueued (see Arena::plan in api.cu): the arena is never reallocated
// while work that uses it may still be in flight on the stream.
static inline size_t lf_align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct ArenaCursor {
  lf_context* ctx;
  size_t offset;
  bool dry;       // planning pass: only adds sizes up
  size_t peak = 0;   // high-water mark (callers may rewind `offset` between operators)
  bool sized_by_dry_pass = false;   // the arena was sized by a planning pass over the same calls: a launcher may take
                                    // scratch of its own (entry points that laid the arena out themselves leave it false)
  template <typename T>
  T* take(size_t count) {
    size_t bytes = lf_align_up(count * sizeof(T), 256);
    T* p = dry ? nullptr : reinterpret_cast<T*>(ctx->arena + offset);
    offset += bytes;
    if (offset > peak) peak = offset;
    return p;
  }
};

lf_status lf_arena_ensure(lf_context* ctx, size_t bytes);
// The pair stack with the pair left in host memory (pair_spill.cu).
lf_status lf_pair_stack_spilled(lf_context* ctx, const lf_pair_stack_desc* d, lf_result* r);

static inline int lf_ceil_div(int64_t a, int64_t b) { return (int)((a + b - 1) / b); }
