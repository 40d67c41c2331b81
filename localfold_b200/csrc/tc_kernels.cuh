// Tensor-core (tcgen05 / TMEM / TMA) kernels for sm_100a: launchers used by api.cu.
// Each *_supported() says whether a kernel covers a shape; api.cu routes
// everything else to the float32 SIMT kernels.
#pragma once

#include "common.cuh"

namespace tc {

// Device buffers of the other ranks of a box as mapped into this process (entry `rank` = the local
// buffer).  Kernels only ever store to them with plain st.global.
constexpr int kMaxPeers = 16;
struct PeerPtrs { void* p[kMaxPeers]; };

void configure_once();
lf_status prepare_weights(lf_context* ctx, lf_weights* w);
// Reads the device status word; LF_ERR_TIMEOUT if a bounded wait expired in a kernel.
lf_status check_status(lf_context* ctx);

// Triangle contraction, batched over the c channels of channel-major fp16
// operands a, b [c][n][ld] (ld a multiple of 8, elements past n never read):
//   outgoing: x[h][i][j] = scale * sum_k a[h][i][k] * b[h][j][k]
//   incoming: x[h][i][j] = scale * sum_k a[h][k][j] * b[h][k][i]
bool contract_supported(int n, int c);
lf_status contract(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, op16* x, int n, int ld, int c,
                   int incoming, float scale);
// Rectangular form for row shards: x[h][i][col0 + j] = scale * sum_k a[h][i][k] b[h][j][k], i < m_rows, j < n_rows,
// k < k_len; a, b have row stride ld_ab and dense planes, x has row stride ldx and plane stride x_plane.
lf_status contract_rect(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, op16* x, int m_rows, int n_rows,
                        int k_len, int ld_ab, int ldx, int64_t x_plane, int col0, int c, int incoming, float scale);

// The same kernel as a plain fp16 GEMM: out[m][n] = act(sum_k a[m][k] w[n][k] + bias[n]) (k contiguous in both
// operands, k_len and n_out multiples of 8; bias may be null; act = ReLU when `relu`), fp16 result.
lf_status contract_gemm(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* w, op16* out, int m_rows, int n_out,
                        int k_len, const float* bias, int relu);
// ... and as the outer product mean's sum over the sequences, stored grouped per pair:
// out[((i * n + j) * c + a) * c + b] = scale * sum_s left[s][i*c + a] right[s][j*c + b] for i < cnt, j < n
// (left, right: k_len rows of n*c, left already offset to its first i), so that the c*c -> c_z projection that
// follows is a plain GEMM over rows (i, j).
lf_status contract_outer(lf_context* ctx, ArenaCursor& cur, const op16* left, const op16* right, op16* out, int cnt, int n, int c,
                         int k_len, float scale);

// Channel-sharded form for the GPUs of one box: a, b are this rank's `c` channels over all n rows
// ([c][n][ld]); row i of channel h of the product goes to rank i / rows_per_rank, into its buffer
// x_peers[...] laid out [all channels][rows_per_rank][ldx], at channel ch0 + h.
lf_status contract_scatter(lf_context* ctx, ArenaCursor& cur, const op16* a, const op16* b, int n, int ld, int c, int incoming,
                           float scale, const PeerPtrs& x_peers, int rows_per_rank, int total_channels, int ch0);

// LayerNorm + projection kernels for 128-channel activations (weights repacked by
// prepare_weights into lf_weights::h).
bool ln_gemm_supported(const lf_weights* w);
void configure_ln_gemm();
void pack_weight_image(lf_context* ctx, const float* w, int K, int n_out, int n_pad, int col0, int ld, op16* img, int row0,
                       float scale, const float* kscale = nullptr);
void fold_bias(lf_context* ctx, const float* w, int K, int n_out, int col0, int ld, const float* offset, const float* b_in, float scale,
               float* b_out);
// a, b [c][n][ld] fp16 = mask * (LN(z) Wp + bp) * sigmoid(LN(z) Wg + bg)
// `rows` pair rows of length n (rows = n for the whole pair, fewer for a row shard)
lf_status triangle_project(lf_context* ctx, ArenaCursor& cur, const void* z, int act_dtype, const float* mask, int rows,
                           int n, int ld, int variance, float eps, const lf_weights* w, op16* a, op16* b);
// The same for a row shard whose operands are wanted channel-sharded: channel h of the shard's rows goes
// to rank h / (128 / ranks), into its buffers a_peers / b_peers laid out [128 / ranks][n][ld], at rows
// row0 .. row0 + rows (row0 = this rank's first pair row).
lf_status triangle_project_scatter(lf_context* ctx, ArenaCursor& cur, const void* z, int act_dtype, const float* mask, int rows,
                                   int n, int ld, int variance, float eps, const lf_weights* w, const PeerPtrs& a_peers,
                                   const PeerPtrs& b_peers, int ranks, int row0);
// q (pre-scaled by head_dim^-1/2), k, v, sigmoid(gate) as fp16 logical rows [batch][ld][128] stored in 8-row x
// 8-channel pieces (element (b, q, c) at b*ld*128 + (q/8)*1024 + (c/8)*64 + (q%8)*8 + c%8, ld = Q rounded up to 16) and the
// pair bias fp16 [heads][batch rows][ldb] (null = none) from the normalised input
lf_status pair_bias_project(lf_context* ctx, ArenaCursor& cur, const void* pair, int pair_dtype, int Q, int variance, float eps,
                            int heads, const lf_weights* w, op16* bias, int ldb);
bool pair_bias_supported(const lf_weights* w);
lf_status attention_project(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int batch, int Q,
                            int transpose, int variance, float eps, int heads, int head_dim, int bias_swap,
                            const lf_weights* w, op16* q, op16* k, op16* v, op16* g, op16* bias, int ldb);
// The same for a row shard: its bias rows are written into every rank's copy of the whole bias
// [heads][bias_rows][ldb] at query rows row0 .. row0 + batch.  `transpose`: the shard is held as [Q][batch]
// (logical row (b, q) at memory row q*batch + b), as for a block of columns of the pair.
lf_status attention_project_scatter(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int batch, int Q,
                                    int variance, float eps, int heads, const lf_weights* w, op16* q, op16* k, op16* v,
                                    op16* g, const PeerPtrs& bias_peers, int ranks, int bias_rows, int row0, int ldb,
                                    int transpose = 0);
lf_status attention_output(lf_context* ctx, ArenaCursor& cur, const op16* o, int batch, int Q, int transpose,
                           const lf_weights* w, const void* resid, void* out, int act_dtype);
// `x_plane_elems`: distance between the channel planes of x (0 = rows * ld, a dense shard; n * ld when x points at
// `rows` rows inside whole planes)
lf_status triangle_output(lf_context* ctx, ArenaCursor& cur, const op16* x, int rows, int n, int ld, float x_eps,
                          const void* z, int act_dtype, int variance, float eps, const lf_weights* w, const void* resid,
                          void* out, int64_t x_plane_elems = 0);
// out[b*Q+i][128] = (softmax_j(q_i.k_j + bias[h][i][j] + mask term_j) v_j) * gate, 4 heads x 32
void configure_attention();
// `bias`: fp16 [4][Q][ldb] (head, query, key; ldb a multiple of 16) or null
lf_status attention_core(lf_context* ctx, ArenaCursor& cur, const op16* q, const op16* k, const op16* v, const op16* g,
                         const op16* bias, int ldb, const float* mask, int batch, int Q, int transpose,
                         int mask_mode, int clamp, op16* out);

// Fused AF2 pair transition (128 channels, 512 hidden): out = resid + relu(LN(x) W1 + b1) W2 + b2
void configure_transition();
bool transition_supported(const lf_weights* w);
lf_status transition_run(lf_context* ctx, ArenaCursor& cur, const void* act, int act_dtype, int64_t rows, int variance,
                         float eps, const lf_weights* w, const void* resid, void* out);

}  // namespace tc
