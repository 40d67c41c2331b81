// The pair stack with the pair tensor left in host memory.
//
// The regular host-buffer path copies the whole pair to the device and keeps every operator's scratch
// beside it.  When the device cannot hold that (the scratch arena is refused), the block runs here
// instead: the pair stays in the caller's buffer, pinned for the duration, and streams through the
// device in chunks of pair rows (columns for the ending-node attention), one cudaMemcpyAsync /
// cudaMemcpy2DAsync per chunk and direction on two copy streams, double-buffered against the kernels.
// It replaces the reference's host-spill and row-chunked pair tracks (webgpu/runtime/host-spill.js:13-78,
// webgpu/af3/trunk/pair-track.js:967-1000).
//
// Per update (all on the 16-bit tensor-core kernels, c_z = c_hidden = 128, 4 heads):
//   triangle out / in   pass 1 over the chunks: project -> the chunk's rows of a, b inside whole channel planes
//                       (which stay on the device: the contraction needs every row); contraction; pass 2:
//                       output on the chunk's rows of x, the chunk goes back to the host
//   attention start     pass 1: project, for the pair bias of the chunk's query rows (the bias of ALL query
//   / end               rows is needed by every chunk); pass 2: project again, core, output, back to the host.
//                       The ending node walks column chunks, held on the device as [row][chunk column],
//                       which is the kernels' transposed orientation with batch = chunk columns.
//   transition          one pass
// What stays resident is a, b, x (3 x N^2 x 256 bytes) and the bias; what streams is the pair (N^2 x 512 bytes
// in and out per pass).  The path is PCIe-bound by design: it exists so that a length which does not fit
// still runs.
#include <cuda_runtime.h>

#include <cmath>

#include "tc_kernels.cuh"

namespace {

struct Pipeline {
  lf_context* ctx;
  cudaStream_t in = nullptr, out = nullptr;
  cudaEvent_t loaded[2] = {nullptr, nullptr}, computed[2] = {nullptr, nullptr}, stored[2] = {nullptr, nullptr};
  bool stored_valid[2] = {false, false};
  lf_status open() {
    LF_CUDA(ctx, cudaStreamCreateWithFlags(&in, cudaStreamNonBlocking));
    LF_CUDA(ctx, cudaStreamCreateWithFlags(&out, cudaStreamNonBlocking));
    for (int i = 0; i < 2; ++i) {
      LF_CUDA(ctx, cudaEventCreateWithFlags(&loaded[i], cudaEventDisableTiming));
      LF_CUDA(ctx, cudaEventCreateWithFlags(&computed[i], cudaEventDisableTiming));
      LF_CUDA(ctx, cudaEventCreateWithFlags(&stored[i], cudaEventDisableTiming));
    }
    return LF_OK;
  }
  void close() {
    if (in) cudaStreamSynchronize(in);
    if (out) cudaStreamSynchronize(out);
    for (int i = 0; i < 2; ++i) {
      if (loaded[i]) cudaEventDestroy(loaded[i]);
      if (computed[i]) cudaEventDestroy(computed[i]);
      if (stored[i]) cudaEventDestroy(stored[i]);
    }
    if (in) cudaStreamDestroy(in);
    if (out) cudaStreamDestroy(out);
    cudaGetLastError();
  }
};

struct Chunking {
  int n, rows;          // pair length, rows (or columns) per chunk
  int count() const { return (n + rows - 1) / rows; }
  int first(int c) const { return c * rows; }
  int size(int c) const { return first(c) + rows <= n ? rows : n - first(c); }
};

// One pass over the chunks.  `columns`: chunks are columns of the pair, held as [n][chunk].  load -> compute -> store
// (store optional), the buffer of chunk c + 2 reused once chunk c's store has finished.
template <typename Compute>
lf_status pass(lf_context* ctx, Pipeline& pl, const Chunking& ck, bool columns, bool store, float* host_pair, const float* host_mask,
               float* zbuf[2], float* mbuf[2], Compute compute) {
  const int n = ck.n;
  for (int c = 0; c < ck.count(); ++c) {
    const int b = c & 1, r0 = ck.first(c), rc = ck.size(c);
    // the buffer is free once the kernels of chunk c - 2 (and its store, if any) are done with it
    if (c >= 2) LF_CUDA(ctx, cudaStreamWaitEvent(pl.in, store && pl.stored_valid[b] ? pl.stored[b] : pl.computed[b], 0));
    if (!columns) {
      LF_CUDA(ctx, cudaMemcpyAsync(zbuf[b], host_pair + (size_t)r0 * n * 128, (size_t)rc * n * 512, cudaMemcpyHostToDevice, pl.in));
      LF_CUDA(ctx, cudaMemcpyAsync(mbuf[b], host_mask + (size_t)r0 * n, (size_t)rc * n * 4, cudaMemcpyHostToDevice, pl.in));
    } else {
      LF_CUDA(ctx, cudaMemcpy2DAsync(zbuf[b], (size_t)rc * 512, host_pair + (size_t)r0 * 128, (size_t)n * 512, (size_t)rc * 512, n,
                                     cudaMemcpyHostToDevice, pl.in));
      LF_CUDA(ctx, cudaMemcpy2DAsync(mbuf[b], (size_t)rc * 4, host_mask + r0, (size_t)n * 4, (size_t)rc * 4, n, cudaMemcpyHostToDevice, pl.in));
    }
    LF_CUDA(ctx, cudaEventRecord(pl.loaded[b], pl.in));
    LF_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, pl.loaded[b], 0));
    LF_TRY(compute(c, r0, rc, zbuf[b], mbuf[b]));
    LF_CUDA(ctx, cudaEventRecord(pl.computed[b], ctx->stream));
    if (store) {
      LF_CUDA(ctx, cudaStreamWaitEvent(pl.out, pl.computed[b], 0));
      if (!columns)
        LF_CUDA(ctx, cudaMemcpyAsync(host_pair + (size_t)r0 * n * 128, zbuf[b], (size_t)rc * n * 512, cudaMemcpyDeviceToHost, pl.out));
      else
        LF_CUDA(ctx, cudaMemcpy2DAsync(host_pair + (size_t)r0 * 128, (size_t)n * 512, zbuf[b], (size_t)rc * 512, (size_t)rc * 512, n,
                                       cudaMemcpyDeviceToHost, pl.out));
      LF_CUDA(ctx, cudaEventRecord(pl.stored[b], pl.out));
      pl.stored_valid[b] = true;
    }
  }
  // the next pass reads what this one wrote (host) and reuses the buffers
  LF_CUDA(ctx, cudaStreamSynchronize(pl.out));
  LF_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  pl.stored_valid[0] = pl.stored_valid[1] = false;
  return LF_OK;
}

size_t aligned(size_t bytes) { return lf_align_up(bytes, 256); }

}  // namespace

// Called by lf_pair_stack_run (host space, 16-bit mode) after the scratch arena for the regular path was refused.
lf_status lf_pair_stack_spilled(lf_context* ctx, const lf_pair_stack_desc* d, lf_result* r) {
  const int n = d->length;
  if (d->space != LF_SPACE_HOST || d->precision != LF_PRECISION_BF16 || d->c_z != 128 || d->c_hidden != 128 || d->heads != 4 ||
      d->order != LF_ORDER_EVOFORMER || n % 16 != 0)
    return lf_fail(ctx, LF_ERR_MEMORY, "the pair does not fit on the device and the host-resident path covers the 16-bit mode, cZ = cHidden = 128, "
                                       "4 heads and lengths that are multiples of 16");
  for (int b = d->first_block; b < d->first_block + d->n_blocks; ++b) {
    const lf_pair_block_weights& bw = d->blocks[b];
    const bool af3 = bw.attention_starting->kind == LF_WEIGHTS_GRID_ATTENTION_AF3;
    if (!tc::ln_gemm_supported(bw.triangle_outgoing) || !tc::ln_gemm_supported(bw.triangle_incoming) ||
        !tc::ln_gemm_supported(bw.attention_starting) || !tc::ln_gemm_supported(bw.attention_ending) || !tc::transition_supported(bw.transition) ||
        (af3 && !d->swap_transposed_bias))
      return lf_fail(ctx, LF_ERR_MEMORY, "the pair does not fit on the device and block %d has weights the host-resident path does not cover", b);
  }
  const int ld = n;
  const size_t plane = (size_t)n * ld;
  // resident: a, b, x, the pair bias; per chunk (twice): pair rows, mask rows; per chunk: q, k, v, gate, o
  const size_t resident = 3 * aligned(plane * 128 * 2) + aligned(plane * 4 * 2) + 4096;
  auto per_chunk = [&](int rows) { return 2 * (aligned((size_t)rows * n * 512) + aligned((size_t)rows * n * 4)) + 5 * aligned((size_t)rows * n * 256); };
  int rows = n;
  const size_t limit = ctx->arena_limit;
  if (limit) {
    while (rows > 16 && resident + per_chunk(rows) > limit) rows = (rows / 2 + 15) / 16 * 16;
    if (resident + per_chunk(rows) > limit)
      return lf_fail(ctx, LF_ERR_MEMORY, "the triangle operands alone (%zu bytes) exceed the scratch limit of %zu bytes", resident, limit);
  }
  lf_status s = LF_ERR_MEMORY;
  for (; rows >= 16; rows = rows > 16 ? (rows / 2 + 15) / 16 * 16 : 0) {      // halve the chunk until the driver grants the arena
    s = lf_arena_ensure(ctx, resident + per_chunk(rows));
    if (s == LF_OK || rows == 16) break;
  }
  if (s != LF_OK) return s;

  ArenaCursor cur{ctx, 0, false};
  op16* a = cur.take<op16>(plane * 128);
  op16* b = cur.take<op16>(plane * 128);
  op16* x = cur.take<op16>(plane * 128);
  op16* bias = cur.take<op16>(plane * 4);
  float* zbuf[2]; float* mbuf[2];
  for (int i = 0; i < 2; ++i) { zbuf[i] = cur.take<float>((size_t)rows * n * 128); mbuf[i] = cur.take<float>((size_t)rows * n); }
  op16* qkvgo[5];
  for (int i = 0; i < 5; ++i) qkvgo[i] = cur.take<op16>((size_t)rows * n * 128);
  if (cur.peak > ctx->arena_peak) ctx->arena_peak = cur.peak;

  float* host_pair = (float*)d->pair;
  const float* host_mask = d->mask;
  const size_t pair_bytes = plane * 512;
  const bool pinned_pair = cudaHostRegister(host_pair, pair_bytes, cudaHostRegisterDefault) == cudaSuccess;
  const bool pinned_mask = cudaHostRegister((void*)host_mask, plane * 4, cudaHostRegisterDefault) == cudaSuccess;
  cudaGetLastError();     // a buffer that is already pinned (or cannot be) is copied from as it is

  Pipeline pl{ctx};
  const uint64_t before = ctx->launches;
  cudaEventRecord(ctx->ev0, ctx->stream);
  s = pl.open();
  const Chunking ck{n, rows};
  const float xscale = ldexpf(1.0f, -(int)(0.5f * log2f((float)n)));
  tc::PeerPtrs pa{}, pb{}, pbias{};
  pa.p[0] = a; pb.p[0] = b; pbias.p[0] = bias;
  if (s == LF_OK) s = (cudaMemsetAsync(bias, 0, plane * 4 * 2, ctx->stream) == cudaSuccess) ? LF_OK : lf_fail(ctx, LF_ERR_CUDA, "memset failed");

  for (int blk = d->first_block; blk < d->first_block + d->n_blocks && s == LF_OK; ++blk) {
    const lf_pair_block_weights& bw = d->blocks[blk];
    for (int dir = 0; dir < 2 && s == LF_OK; ++dir) {
      const lf_weights* w = dir ? bw.triangle_incoming : bw.triangle_outgoing;
      s = pass(ctx, pl, ck, false, false, host_pair, host_mask, zbuf, mbuf, [&](int, int r0, int rc, float* z, float* m) {
        return tc::triangle_project_scatter(ctx, cur, z, LF_DTYPE_F32, m, rc, n, ld, d->variance, d->epsilon, w, pa, pb, 1, r0);
      });
      if (s == LF_OK) s = tc::contract(ctx, cur, a, b, x, n, ld, 128, dir, xscale);
      if (s == LF_OK)
        s = pass(ctx, pl, ck, false, true, host_pair, host_mask, zbuf, mbuf, [&](int, int r0, int rc, float* z, float*) {
          return tc::triangle_output(ctx, cur, x + (size_t)r0 * ld, rc, n, ld, d->epsilon * xscale * xscale, z, LF_DTYPE_F32, d->variance,
                                     d->epsilon, w, z, z, (int64_t)plane);
        });
    }
    for (int t = 0; t < 2 && s == LF_OK; ++t) {
      const lf_weights* w = t ? bw.attention_ending : bw.attention_starting;
      const bool af3 = w->kind == LF_WEIGHTS_GRID_ATTENTION_AF3;
      const int mask_mode = af3 ? 1 : 0, clamp = af3 ? 0 : 1;
      // the chunk's logical rows (b, q): memory (b, q) for the starting node; for the ending node the chunk holds
      // [q][b] with batch = the chunk's columns, which is the kernels' transposed orientation
      auto project = [&](int r0, int rc, float* z) {
        return tc::attention_project_scatter(ctx, cur, z, LF_DTYPE_F32, rc, n, d->variance, d->epsilon, 4, w, qkvgo[0], qkvgo[1], qkvgo[2],
                                             qkvgo[3], pbias, 1, n, r0, ld, t);
      };
      s = pass(ctx, pl, ck, t != 0, false, host_pair, host_mask, zbuf, mbuf, [&](int, int r0, int rc, float* z, float*) { return project(r0, rc, z); });
      if (s == LF_OK)
        s = pass(ctx, pl, ck, t != 0, true, host_pair, host_mask, zbuf, mbuf, [&](int, int r0, int rc, float* z, float* m) {
          LF_TRY(project(r0, rc, z));
          LF_TRY(tc::attention_core(ctx, cur, qkvgo[0], qkvgo[1], qkvgo[2], qkvgo[3], bias, ld, m, rc, n, t, mask_mode, clamp, qkvgo[4]));
          return tc::attention_output(ctx, cur, qkvgo[4], rc, n, t, w, z, z, LF_DTYPE_F32);
        });
    }
    if (s == LF_OK)
      s = pass(ctx, pl, ck, false, true, host_pair, host_mask, zbuf, mbuf, [&](int, int, int rc, float* z, float*) {
        return tc::transition_run(ctx, cur, z, LF_DTYPE_F32, (int64_t)rc * n, d->variance, d->epsilon, bw.transition, z, z);
      });
  }
  cudaEventRecord(ctx->ev1, ctx->stream);
  cudaStreamSynchronize(ctx->stream);
  pl.close();
  if (pinned_pair) cudaHostUnregister(host_pair);
  if (pinned_mask) cudaHostUnregister((void*)host_mask);
  cudaGetLastError();
  if (s != LF_OK) return s;
  LF_TRY(tc::check_status(ctx));
  float ms = 0.f;
  cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1);
  if (r) { r->elapsed_ms = ms; r->peak_bytes = ctx->arena_peak; r->launches = (uint32_t)(ctx->launches - before); }
  return LF_OK;
}
