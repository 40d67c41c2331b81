// Triangle multiplication for callers that must not allocate device memory.
//
// Some hosts cannot let a library call cudaMalloc once they are running: an inference server that
// handed the whole device to its own memory pool at start-up (a later cudaMalloc fails or fragments
// what is left), or a service whose latency rules forbid driver allocations in steady state because
// cudaMalloc / cudaFree synchronise the device and stall every other stream.  The regular entry
// point sizes and grows a scratch arena with cudaMalloc on demand; this one never allocates: its
// scratch (the fp16 operands a, b and the product x of the triangle multiplication) is a fixed
// array that lives in the library's device image, so every GPU that loads the library holds it
// (12 MiB) until the process exits.
#include <cuda_runtime.h>

#include <cmath>
#include <mutex>

#include "tc_kernels.cuh"

#define LF_STATIC_MAX_LENGTH 128   // largest pair length the static scratch covers (c_z = c_hidden = 128)

namespace {

constexpr size_t kStaticPlane = (size_t)LF_STATIC_MAX_LENGTH * LF_STATIC_MAX_LENGTH;   // one channel of a, b or x
constexpr size_t kStaticBytes = 3 * 128 * kStaticPlane * sizeof(op16);                 // a, b, x: 12 MiB

// The array's name is a host-side stand-in in host code, not a device address: the address the
// kernels get comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
// Per device: device address of g_static_scratch (null = not resolved) and the error of the one attempt.
// std::call_once makes the first call per device safe from several host threads at once.
static void* g_static_ptr[kMaxDevices];
static cudaError_t g_static_err[kMaxDevices];
static std::once_flag g_static_once[kMaxDevices];

// Once per device, with that device current: resolve the array's device address.  With CUDA's lazy
// module loading this is also the moment the driver loads the module that holds the array.
lf_status static_scratch_setup(lf_context* ctx, void** out) {
  if (ctx->device < 0 || ctx->device >= kMaxDevices) return lf_fail(ctx, LF_ERR_ARGUMENT, "device ordinal %d is out of range", ctx->device);
  const int dev = ctx->device;
  std::call_once(g_static_once[dev], [dev]() {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess) cudaGetLastError();
    g_static_err[dev] = (e == cudaSuccess && ptr == nullptr) ? cudaErrorInvalidSymbol : e;
    g_static_ptr[dev] = e == cudaSuccess ? ptr : nullptr;
  });
  if (!g_static_ptr[dev])
    return lf_fail(ctx, LF_ERR_CUDA, "cudaGetSymbolAddress for the static scratch failed: %s", cudaGetErrorString(g_static_err[dev]));
  *out = g_static_ptr[dev];
  return LF_OK;
}

}  // namespace

extern "C" lf_status lf_triangle_multiplication_run_static(lf_context* ctx, const lf_triangle_desc* d, lf_result* r) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!d || !d->z || !d->mask || !d->out || !d->weights) return lf_fail(ctx, LF_ERR_ARGUMENT, "triangle multiplication: null argument");
  if (d->space != LF_SPACE_DEVICE)
    return lf_fail(ctx, LF_ERR_ARGUMENT, "the no-allocation entry point takes device buffers only (host buffers would need a staging allocation)");
  if (d->precision != LF_PRECISION_BF16)
    return lf_fail(ctx, LF_ERR_UNSUPPORTED, "the no-allocation entry point runs the 16-bit tensor-core path only");
  if (d->act_dtype != LF_DTYPE_F32 && d->act_dtype != LF_DTYPE_BF16) return lf_fail(ctx, LF_ERR_ARGUMENT, "unknown activation dtype %d", d->act_dtype);
  if (d->variance != LF_VARIANCE_TWO_PASS && d->variance != LF_VARIANCE_FAST)
    return lf_fail(ctx, LF_ERR_ARGUMENT, "variance has no default: pass LF_VARIANCE_TWO_PASS or LF_VARIANCE_FAST");
  if (!(d->epsilon > 0.f) || !std::isfinite(d->epsilon)) return lf_fail(ctx, LF_ERR_ARGUMENT, "epsilon must be finite and positive; received %g", (double)d->epsilon);
  if (d->length <= 0) return lf_fail(ctx, LF_ERR_SHAPE, "length must be a positive safe integer; received %d", d->length);
  if (d->length > LF_STATIC_MAX_LENGTH)
    return lf_fail(ctx, LF_ERR_UNSUPPORTED, "length %d exceeds the static scratch, which covers lengths up to %d; use lf_triangle_multiplication_run",
                   d->length, LF_STATIC_MAX_LENGTH);
  const lf_weights* w = d->weights;
  if (w->kind != LF_WEIGHTS_TRIANGLE_AF2 && w->kind != LF_WEIGHTS_TRIANGLE_AF3) return lf_fail(ctx, LF_ERR_ARGUMENT, "weights are not triangle weights");
  if (d->c_z != 128 || d->c_hidden != 128 || w->dims.channels != 128 || w->dims.hidden != 128 || !tc::ln_gemm_supported(w) ||
      !tc::contract_supported(d->length, 128))
    return lf_fail(ctx, LF_ERR_UNSUPPORTED, "the no-allocation entry point covers cZ = cHidden = 128 on a device with tensor-map support");

  cudaSetDevice(ctx->device);
  void* scratch = nullptr;
  LF_TRY(static_scratch_setup(ctx, &scratch));

  const int n = d->length;
  const int ld = (n + 15) / 16 * 16;
  const size_t plane = (size_t)n * ld;
  op16* a = reinterpret_cast<op16*>(scratch);
  op16* b = a + 128 * plane;
  op16* x = b + 128 * plane;
  // Nothing in the scratch has to start at zero: a, b and x are fully written before they are read
  // (columns between n and ld are never read), so the previous call's contents are simply overwritten.

  const bool was_profiling = ctx->profiling;   // the profiler creates events per launch; keep this path allocation-free
  ctx->profiling = false;
  const uint64_t before = ctx->launches;
  ArenaCursor cur{ctx, 0, false};
  const float xscale = ldexpf(1.0f, -(int)(0.5f * log2f((float)n)));
  const float xs = xscale * (d->divide_by_length ? (float)n : 1.0f);
  lf_status s = tc::triangle_project(ctx, cur, d->z, d->act_dtype, d->mask, n, n, ld, d->variance, d->epsilon, w, a, b);
  if (s == LF_OK) s = tc::contract(ctx, cur, a, b, x, n, ld, 128, d->incoming ? 1 : 0, xscale);
  if (s == LF_OK)
    s = tc::triangle_output(ctx, cur, x, n, n, ld, d->epsilon * xs * xs, d->z, d->act_dtype, d->variance, d->epsilon, w,
                            d->residual ? d->z : nullptr, d->out);
  ctx->profiling = was_profiling;
  if (s != LF_OK) return s;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return lf_fail(ctx, LF_ERR_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
  if (r) { r->elapsed_ms = 0.f; r->peak_bytes = kStaticBytes; r->launches = (uint32_t)(ctx->launches - before); }
  return LF_OK;
}
