// Transpose of a row-sharded pair tensor across the GPUs of one box, written straight into the
// peers' memory.
//
// Rank g of G owns rows [g R, (g+1) R) of z [N][N][C] as a local [R][N][C] tensor (R = N / G).  The
// transposed shard of rank d is zT[m][n] = z[n][d R + m]: vector (r, n) of this rank goes to rank
// n / R, row n % R, column g R + r.  One kernel per rank reads its shard once and stores every
// channel vector (C x 4 or C x 2 bytes, 16 bytes per lane) to its owner through a peer mapping
// (plain st.global over NVLink; no TMA, no multicast).  Destination rows are walked so that
// consecutive warps write consecutive vectors of one destination row.  The buffers are allocated
// by this library with cudaMalloc and shared between the ranks' processes as CUDA IPC handles; the
// caller orders "all stores have landed" with its own barrier (an NCCL collective on the stream).
#include <cuda_runtime.h>

#include "common.cuh"

namespace {

constexpr int kMaxRanks = 16;
struct PeerPtrs { unsigned char* p[kMaxRanks]; };

// vec16: 16-byte pieces per channel vector (32 for 128 float channels, 16 for 128 bf16 channels)
__global__ void __launch_bounds__(256) transpose_scatter_kernel(const uint4* __restrict__ src, PeerPtrs dst, int R, int N, int vec16,
                                                                int rank, long long vectors) {
  const int lanes_per_vec = vec16;                   // 16 or 32 lanes move one vector
  const int vec_per_warp = 32 / lanes_per_vec;       // 2 or 1
  const int lane = threadIdx.x & 31;
  const long long warp_global = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int sub = lane / lanes_per_vec, piece = lane % lanes_per_vec;
  // destination-major order: idx = n * R + r, so a destination row (fixed n) is written front to back
  for (long long base = warp_global * vec_per_warp * 4; base < vectors; base += warps * vec_per_warp * 4) {
    uint4 v[4];
    long long idx[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      idx[u] = base + u * vec_per_warp + sub;
      if (idx[u] < vectors) {
        const int n = (int)(idx[u] / R), r = (int)(idx[u] % R);
        v[u] = __ldcs(src + ((long long)r * N + n) * vec16 + piece);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (idx[u] < vectors) {
        const int n = (int)(idx[u] / R), r = (int)(idx[u] % R);
        uint4* out = reinterpret_cast<uint4*>(dst.p[n / R]) + ((long long)(n % R) * N + (long long)rank * R + r) * vec16 + piece;
        *out = v[u];
      }
    }
  }
}

// Channel planes of a row shard to their channel owners: src [C][R][ld] fp16; plane h goes to rank
// h / cpr, plane h % cpr of its [cpr][N][ld] buffer, rows rank R ..: one contiguous run of R x ld
// elements per plane, copied 16 bytes per lane.
__global__ void __launch_bounds__(256) planes_scatter_kernel(const uint4* __restrict__ src, PeerPtrs dst, int channels, int cpr,
                                                             long long run16, long long dst_plane16, long long dst_row16) {
  const long long total = (long long)channels * run16;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int h = (int)(i / run16);
    const long long within = i - (long long)h * run16;
    const int owner = h / cpr;
    reinterpret_cast<uint4*>(dst.p[owner])[(long long)(h - owner * cpr) * dst_plane16 + dst_row16 + within] = __ldcs(src + i);
  }
}

}  // namespace

extern "C" {

LF_API lf_status lf_peer_buffer_create(lf_context* ctx, size_t bytes, void** ptr, unsigned char handle[64]) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!ptr || !handle || bytes == 0) return lf_fail(ctx, LF_ERR_ARGUMENT, "peer buffer: null output or zero size");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  LF_CUDA(ctx, cudaSetDevice(ctx->device));
  void* p = nullptr;
  LF_CUDA(ctx, cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    cudaGetLastError();
    return lf_fail(ctx, LF_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
  }
  memcpy(handle, &h, 64);
  *ptr = p;
  return LF_OK;
}

LF_API lf_status lf_peer_buffer_open(lf_context* ctx, const unsigned char handle[64], void** ptr) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!ptr || !handle) return lf_fail(ctx, LF_ERR_ARGUMENT, "peer buffer: null argument");
  LF_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return lf_fail(ctx, LF_ERR_CUDA, "cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
  }
  *ptr = p;
  return LF_OK;
}

LF_API lf_status lf_peer_buffer_close(lf_context* ctx, void* ptr) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (ptr) LF_CUDA(ctx, cudaIpcCloseMemHandle(ptr));
  return LF_OK;
}

LF_API lf_status lf_peer_buffer_destroy(lf_context* ctx, void* ptr) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (ptr) LF_CUDA(ctx, cudaFree(ptr));
  return LF_OK;
}

LF_API lf_status lf_pair_transpose_scatter(lf_context* ctx, const void* src, int rows, int length, int vector_bytes, int ranks,
                                           int rank, void* const* dst) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!src || !dst) return lf_fail(ctx, LF_ERR_ARGUMENT, "transpose scatter: null buffer");
  if (ranks < 1 || ranks > kMaxRanks || rank < 0 || rank >= ranks) return lf_fail(ctx, LF_ERR_ARGUMENT, "transpose scatter: rank %d of %d", rank, ranks);
  if (rows <= 0 || (int64_t)rows * ranks != length) return lf_fail(ctx, LF_ERR_SHAPE, "transpose scatter: rows %d x ranks %d must equal length %d", rows, ranks, length);
  if (vector_bytes != 512 && vector_bytes != 256) return lf_fail(ctx, LF_ERR_UNSUPPORTED, "transpose scatter: channel vectors of 512 or 256 bytes; received %d", vector_bytes);
  PeerPtrs pp{};
  for (int g = 0; g < ranks; ++g) {
    if (!dst[g]) return lf_fail(ctx, LF_ERR_ARGUMENT, "transpose scatter: destination %d is null", g);
    pp.p[g] = (unsigned char*)dst[g];
  }
  LF_CUDA(ctx, cudaSetDevice(ctx->device));
  const long long vectors = (long long)rows * length;
  const int grid = ctx->sm_count * 8;
  lf_prof_begin(ctx, LF_KERNEL_ELEMENTWISE);
  transpose_scatter_kernel<<<grid, 256, 0, ctx->stream>>>((const uint4*)src, pp, rows, length, vector_bytes / 16, rank, vectors);
  lf_prof_end(ctx);
  ctx->launches++;
  LF_CUDA(ctx, cudaGetLastError());
  return LF_OK;
}

LF_API lf_status lf_pair_planes_scatter(lf_context* ctx, const void* src, int channels, int rows, int length, int ranks, int rank,
                                        void* const* dst) {
  if (!ctx) return LF_ERR_ARGUMENT;
  if (!src || !dst) return lf_fail(ctx, LF_ERR_ARGUMENT, "planes scatter: null buffer");
  if (ranks < 1 || ranks > kMaxRanks || rank < 0 || rank >= ranks || channels <= 0 || channels % ranks != 0)
    return lf_fail(ctx, LF_ERR_ARGUMENT, "planes scatter: rank %d of %d, %d channels", rank, ranks, channels);
  if (rows <= 0 || (int64_t)rows * ranks != length || length % 8 != 0)
    return lf_fail(ctx, LF_ERR_SHAPE, "planes scatter: rows %d x ranks %d must equal length %d, a multiple of 8", rows, ranks, length);
  PeerPtrs pp{};
  for (int g = 0; g < ranks; ++g) {
    if (!dst[g]) return lf_fail(ctx, LF_ERR_ARGUMENT, "planes scatter: destination %d is null", g);
    pp.p[g] = (unsigned char*)dst[g];
  }
  LF_CUDA(ctx, cudaSetDevice(ctx->device));
  const long long run16 = (long long)rows * length / 8;             // 16-byte pieces per plane of the shard
  const long long plane16 = (long long)length * length / 8, row16 = (long long)rank * rows * length / 8;
  lf_prof_begin(ctx, LF_KERNEL_ELEMENTWISE);
  planes_scatter_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>((const uint4*)src, pp, channels, channels / ranks, run16, plane16, row16);
  lf_prof_end(ctx);
  ctx->launches++;
  LF_CUDA(ctx, cudaGetLastError());
  return LF_OK;
}

}  // extern "C"
