/*
 * localfold_pairstack.h - C ABI of the B200 (sm_100a) pair-stack library.
 *
 * Every entry point below replaces one operator of the reference's kernel
 * library (JavaScript classes over WebGPU); the reference interface each one
 * stands in for is cited as path:line within the reference project.  The ABI
 * carries plain pointers, sizes and enums only.  Nothing here throws: every
 * call returns an lf_status and lf_last_error() holds the message, which
 * names the tensor and the expected length for shape errors in the same
 * words as webgpu/kernels/triangle/types.js:7-11.
 *
 * Conventions
 *  - The caller owns every input and output buffer.  `space` says where the
 *    activation buffers of a call live: LF_SPACE_HOST (float32 host memory;
 *    the call copies in, runs, copies out and returns when the output is
 *    ready) or LF_SPACE_DEVICE (device memory of the context's GPU; the call
 *    only enqueues work on the context's stream - use lf_context_synchronize).
 *  - Activations in host space are float32.  In device space `act_dtype`
 *    gives their storage type.
 *  - Weights are handed over once per operator as float32 host arrays in the
 *    reference's own layouts and field order; the library keeps its own
 *    device-resident copy (repacked for its kernels) until lf_weights_destroy.
 *  - One context per host thread; calls on one context are serialised by the
 *    caller.  There is no CPU fallback anywhere behind this header.
 */
#ifndef LOCALFOLD_PAIRSTACK_H
#define LOCALFOLD_PAIRSTACK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define LF_API __attribute__((visibility("default")))
#else
#define LF_API
#endif

typedef enum lf_status {
  LF_OK = 0,
  LF_ERR_SHAPE = 1,       /* a tensor has the wrong number of elements */
  LF_ERR_ARGUMENT = 2,    /* null pointer, unknown enum, missing dialect bit */
  LF_ERR_CUDA = 3,        /* a CUDA runtime call failed */
  LF_ERR_MEMORY = 4,      /* device allocation refused */
  LF_ERR_UNSUPPORTED = 5, /* shape outside what the kernels cover */
  LF_ERR_TIMEOUT = 6      /* a bounded device-side wait ran out */
} lf_status;

typedef enum lf_space { LF_SPACE_HOST = 0, LF_SPACE_DEVICE = 1 } lf_space;
typedef enum lf_dtype { LF_DTYPE_F32 = 0, LF_DTYPE_BF16 = 1 } lf_dtype;

/* Arithmetic mode.  F32: float32 storage and float32 FMA accumulation
 * (the reference's `precision: "f32"`).  BF16 names the 16-bit tensor-core
 * mode: its tensor-core operands are fp16 (11-bit significand; every rounded
 * operand is bounded by construction), products accumulate in float32, and
 * LayerNorm statistics, softmax and gates are float32.  It stands where the
 * reference has `precision: "f16"`; the enumerator keeps its name because the
 * pair stream this mode is usually paired with is bf16 or float32 (lf_dtype). */
typedef enum lf_precision { LF_PRECISION_F32 = 0, LF_PRECISION_BF16 = 1 } lf_precision;

/* LayerNorm variance: the reference's `variance: "two-pass" | "fast"`
 * (webgpu/kernels/triangle/shaders.js:43-58). No default: 0 is rejected. */
typedef enum lf_variance { LF_VARIANCE_TWO_PASS = 1, LF_VARIANCE_FAST = 2 } lf_variance;

typedef struct lf_context lf_context;
typedef struct lf_weights lf_weights;

/* {elapsedMilliseconds, memory} of every reference operator result
 * (webgpu/kernels/triangle/webgpu.js:165). elapsed_ms is device time between
 * CUDA events for host-space calls and 0 for device-space calls. */
typedef struct lf_result {
  float elapsed_ms;
  uint64_t peak_bytes;   /* high-water mark of the context's scratch arena */
  uint32_t launches;     /* kernels of this library launched by the call */
} lf_result;

/* ---- context ------------------------------------------------------------ */

/* Replaces createNodeDevice() + per-device runtime (webgpu/node.js:51-81,
 * webgpu/runtime/execution.js:156).  `stream` may be NULL (the context makes
 * its own) or a cudaStream_t the caller owns. */
LF_API lf_status lf_context_create(int device_ordinal, void* stream, lf_context** out);
/* The same with the stream taken as given: NULL here means CUDA's default stream (which
 * lf_context_create cannot express, NULL being "make one").  For callers whose other work - their
 * own kernels, NCCL collectives - runs on that stream and must stay ordered with this library's. */
LF_API lf_status lf_context_create_on_stream(int device_ordinal, void* stream, lf_context** out);
/* The cudaStream_t every call of this context enqueues on.  Work the caller enqueues elsewhere is
 * not ordered with the library's: use this stream, or events, or lf_context_synchronize. */
LF_API void* lf_context_stream(const lf_context* ctx);
LF_API void lf_context_destroy(lf_context* ctx);
LF_API const char* lf_last_error(const lf_context* ctx);
LF_API lf_status lf_context_synchronize(lf_context* ctx);
/* Total kernels launched through this context since creation. */
LF_API uint64_t lf_context_launch_count(const lf_context* ctx);
/* Scratch arena: grows on demand; reserve up front to keep allocation out of
 * timed regions; release returns it to the driver. */
LF_API lf_status lf_context_reserve(lf_context* ctx, uint64_t bytes);
LF_API void lf_context_release_scratch(lf_context* ctx);
/* Upper bound on the scratch arena (0 = none): larger requests are refused with LF_ERR_MEMORY without
 * asking the driver.  For hosts that budget device memory, and for exercising the paths that run when
 * the device is short of memory (lf_pair_stack_run then leaves a host-space pair in the caller's buffer
 * and streams it through the device in chunks of rows: see there). */
LF_API lf_status lf_context_limit_scratch(lf_context* ctx, uint64_t bytes);
LF_API const char* lf_version(void);

/* Per-kernel timing, the counterpart of the reference's timestamp-query
 * profile (webgpu/runtime/execution.js:673-703): when enabled, every kernel
 * launch is bracketed by CUDA events on the context's stream.
 * lf_context_profile_read synchronises, then returns and clears the device
 * time and launch count accumulated for one kernel family. */
typedef enum lf_kernel_family {
  LF_KERNEL_SIMT = 0,              /* float32 SIMT kernels (all of them)        */
  LF_KERNEL_TRIANGLE_CONTRACT = 1, /* tcgen05 triangle contraction              */
  LF_KERNEL_LN_GEMM = 2,           /* tcgen05 LayerNorm + projection kernels    */
  LF_KERNEL_TRIANGLE_OUTPUT = 3,   /* tcgen05 centre-norm + output projection   */
  LF_KERNEL_ATTENTION = 4,         /* tcgen05 attention core                    */
  LF_KERNEL_TRANSITION = 5,        /* tcgen05 fused transition                  */
  LF_KERNEL_ELEMENTWISE = 6,       /* memory-bound vectorised kernels           */
  LF_KERNEL_FAMILY_COUNT = 7
} lf_kernel_family;
LF_API lf_status lf_context_profile(lf_context* ctx, int enable);
LF_API lf_status lf_context_profile_read(lf_context* ctx, int family, double* total_ms, uint64_t* launches);

/* ---- weights ------------------------------------------------------------ */

typedef enum lf_weight_kind {
  /* 16 tensors in the order of webgpu/kernels/triangle/weights.js:4-10
   * (layerNormInWeight ... linearGBias); linear weights are [out][in]. */
  LF_WEIGHTS_TRIANGLE_AF2 = 1,
  /* 8 tensors of shared/af3/weights/weights.js:407-416: leftNormInputScale,
   * leftNormInputOffset, projection (c,2c interleaved), gate (c,2c),
   * centerNormScale, centerNormOffset, outputProjection, gatingLinear. */
  LF_WEIGHTS_TRIANGLE_AF3 = 2,
  /* 9 tensors of webgpu/kernels/attention.js:64-80 (queryNormScale,
   * queryNormOffset, queryWeight, keyWeight, valueWeight, gatingWeight,
   * gatingBias, outputWeight, outputBias), then the pair bias tensors:
   * none; or projectionWeight ("normalized-input"); or layerNormScale,
   * layerNormOffset, projectionWeight ("separate"). All linears (in,out). */
  LF_WEIGHTS_ATTENTION_AF2 = 3,
  /* shared/af3/weights/weights.js:417-442: actNormScale, actNormOffset,
   * pairBiasProjection (c,H), qProjection (H*d,c), kProjection (H*d,c),
   * vProjection (c,H*d), gatingQuery (H*d,c), outputProjection (H*d,c),
   * then optional gatingQueryBias, outputProjectionBias (count 0 = absent). */
  LF_WEIGHTS_GRID_ATTENTION_AF3 = 4,
  /* webgpu/kernels/transition.js:477-480: layerNormScale, layerNormOffset,
   * firstWeight (c,h), firstBias, secondWeight (h,c), secondBias. */
  LF_WEIGHTS_TRANSITION_AF2 = 5,
  /* shared/af3/weights/weights.js:447-452: inputLayerNormScale,
   * inputLayerNormOffset, transition1 (c, 2*f*c gate half first),
   * transition2 (f*c, c). */
  LF_WEIGHTS_TRANSITION_AF3 = 6,
  /* webgpu/kernels/outer-product-mean.js:72-75: layerNormScale,
   * layerNormOffset, leftWeight (cm,c), leftBias, rightWeight, rightBias,
   * outputWeight (c*c, cz), outputBias. */
  LF_WEIGHTS_OPM_AF2 = 7,
  /* shared/af3/weights/weights.js:699-727 (singleAttention): layerNormScale,
   * layerNormOffset, qProjection (c,H*d), qBias, kProjection, vProjection,
   * gatingQuery, outputProjection (H*d,c), then the block's
   * singlePairLogitsNormScale, singlePairLogitsNormOffset,
   * singlePairLogitsProjection (cz,H). */
  LF_WEIGHTS_SINGLE_ATTENTION_AF3 = 8,
  /* msaAttention1 of shared/af3/weights/weights.js:670-680: actNormScale,
   * actNormOffset, pairNormScale, pairNormOffset, pairLogits (cz,H),
   * vProjection (cm,H*d), gatingQuery (cm,H*d), outputProjection (H*d,cm).
   * dims: channels = cm, heads, head_dim (not tied to cm / heads),
   * pair_channels = cz. */
  LF_WEIGHTS_MSA_ATTENTION_AF3 = 9,
  /* The extra-MSA stack's global column attention
   * (webgpu/af2/evoformer/block.js:963-966): queryNormScale, queryNormOffset,
   * queryWeight (c, H*d), keyWeight (c, d), valueWeight (c, d), gatingWeight
   * (c, H*d), gatingBias (H*d), outputWeight (H*d, c), outputBias.  dims:
   * channels, heads, head_dim = gatingBias / heads. */
  LF_WEIGHTS_GLOBAL_ATTENTION_AF2 = 10
} lf_weight_kind;

/* Shape of the operator the weights belong to; unused fields are 0. */
typedef struct lf_weight_dims {
  int32_t channels;        /* c_z for pair operators, c_m / c_s otherwise   */
  int32_t hidden;          /* triangle c_hidden, transition hidden, OPM c   */
  int32_t heads;           /* attention heads                                */
  int32_t head_dim;        /* attention head dimension                       */
  int32_t pair_channels;   /* channels of a separate pair-bias source / c_z  */
  int32_t out_channels;    /* OPM c_z                                        */
} lf_weight_dims;

/* Replaces packWeights / packAttentionWeights and the resident-weight upload
 * (webgpu/kernels/triangle/weights.js:85-171, webgpu/kernels/attention.js:82-97,
 * webgpu/runtime/resident.js).  `tensors[i]` holds `counts[i]` float32 values
 * on the host; counts are checked against `dims`. */
LF_API lf_status lf_weights_create(lf_context* ctx, lf_weight_kind kind, const lf_weight_dims* dims,
                                   const float* const* tensors, const int64_t* counts,
                                   int32_t n_tensors, lf_weights** out);
/* The same from tensors as a bundle stores them: int5 payloads (and float32 for what the exporters keep
 * in float32 - norms, offsets, biases) go to the device as they are, and one kernel decodes the codes
 * straight into the resident weight arrays in the layout the operator's kernels use - the transposes,
 * interleaves and column placements of lf_weights_create applied on the device.  No float32 copy of a
 * quantised weight is made on the host.  Stands where the reference decodes on the device with its
 * transpose / interleave maps (webgpu/weights/quantised-upload.js:100-120).  Tensor order and counts are
 * those of lf_weights_create.  An int5 tensor is given by the bytes of its (group-aligned) range: the
 * codes of whole groups of `block`, then - anywhere after them - one fp16 scale and one fp16 zero point
 * per group at the two offsets; value = code * scale + zero (shared/weights/dtype.js:330-378). */
typedef enum lf_tensor_encoding { LF_TENSOR_F32 = 0, LF_TENSOR_INT5 = 1 } lf_tensor_encoding;
typedef struct lf_encoded_tensor {
  int32_t dtype;               /* lf_tensor_encoding */
  int32_t block;               /* int5: codes per group (32) */
  const void* data;            /* host memory: `count` float32 values, or the int5 payload */
  int64_t count;               /* elements */
  uint64_t payload_bytes;      /* int5: bytes at `data` */
  uint64_t scale_offset;       /* int5: byte offsets of the scales and of the zero points inside the payload */
  uint64_t zero_offset;
} lf_encoded_tensor;
LF_API lf_status lf_weights_create_encoded(lf_context* ctx, lf_weight_kind kind, const lf_weight_dims* dims,
                                           const lf_encoded_tensor* tensors, int32_t n_tensors, lf_weights** out);
LF_API void lf_weights_destroy(lf_weights* w);

/* ---- int5 tensor decode ------------------------------------------------- */

/* Replaces readTensorRange for dtype "int5" (shared/weights/dtype.js:330-378)
 * and the on-device decode of webgpu/weights/quantised-upload.js:100-120:
 * `elements` values, groups of `block` codes of 5 bits, least significant bit
 * first, one fp16 scale and one fp16 zero per group; value = code*scale+zero.
 * `payload` is the tensor's bytes as stored in a shard (host memory);
 * scale_offset / zero_offset are byte offsets inside it.  Output: float32 on
 * the host (`out_space` HOST) or on the device. */
LF_API lf_status lf_int5_decode(lf_context* ctx, const uint8_t* payload, uint64_t payload_bytes,
                                uint64_t scale_offset, uint64_t zero_offset, int64_t elements,
                                int32_t block, lf_space out_space, float* out);

/* ---- operators ---------------------------------------------------------- */

/* TriangleMultiplication{Outgoing,Incoming}Gpu.run
 * (webgpu/kernels/triangle/webgpu.js:25-182) and af3TriangleMultiplication
 * (webgpu/af3/trunk/triangle.js:148-169).  out = update, or z + update when
 * `residual` (the in-place form of webgpu/af2/evoformer/block.js:1288-1534;
 * `out` may alias `z`). */
typedef struct lf_triangle_desc {
  int32_t length, c_z, c_hidden;
  int32_t incoming;            /* 0 outgoing (ikc,jkc->ijc), 1 incoming (kjc,kic->ijc) */
  int32_t variance;            /* lf_variance */
  int32_t precision;           /* lf_precision */
  int32_t residual;
  int32_t divide_by_length;    /* dialect bit triangleMulDivideByLength */
  float epsilon;
  int32_t space;               /* lf_space */
  int32_t act_dtype;           /* lf_dtype of z/out in device space */
  const void* z;               /* [length, length, c_z] */
  const float* mask;           /* [length, length] float32 (same space) */
  void* out;                   /* [length, length, c_z] */
  const lf_weights* weights;   /* TRIANGLE_AF2 or TRIANGLE_AF3 */
} lf_triangle_desc;
LF_API lf_status lf_triangle_multiplication_run(lf_context* ctx, const lf_triangle_desc* d, lf_result* r);

/* Triangle multiplication that allocates nothing.  It has no counterpart in the reference; it exists
 * for hosts that cannot let a library allocate device memory while they run - a server that gave
 * the whole GPU to its own pool at start-up, or one whose latency rules forbid cudaMalloc/cudaFree
 * in steady state because they synchronise the device.  Same descriptor and result as
 * lf_triangle_multiplication_run, with these limits: device-space buffers only, the 16-bit
 * tensor-core path only (precision LF_PRECISION_BF16), c_z = c_hidden = 128, and length <= 128
 * (longer inputs are refused with LF_ERR_UNSUPPORTED).  The operands a, b and the product x live in
 * a fixed 12 MiB array inside the library's device image instead of the scratch arena, so the call
 * makes no cudaMalloc, cudaFree or other allocating call; every GPU that loads the library holds
 * that array until the process exits.  The first call on each device looks the array's address up
 * once (cudaGetSymbolAddress; safe from several host threads at once); make that first call before
 * any stream capture, and during start-up: CUDA loads modules lazily, so this look-up and the first
 * launch of each kernel are also when the driver loads the library's device code, which may take
 * driver-side memory.  All calls share
 * the one array and it keeps the last call's contents (nothing in it needs clearing): two calls
 * that overlap on the GPU - different contexts or streams on one device - race on it, so run them
 * one after the other. */
LF_API lf_status lf_triangle_multiplication_run_static(lf_context* ctx, const lf_triangle_desc* d, lf_result* r);

/* AttentionGpu.run (webgpu/kernels/attention.js:2580-2739): gated multi-head
 * attention over `batch` rows of `query_length` positions with optional pair
 * bias and transposed orientation; and Af3GridSelfAttentionGpu.run
 * (webgpu/af3/trunk/grid-attention.js:1264) when the weights are
 * GRID_ATTENTION_AF3 (batch = query_length = n; `swap_transposed_bias` is the
 * dialect bit and must be 0 or 1 explicitly). */
typedef enum lf_pair_bias { LF_PAIR_BIAS_NONE = 0, LF_PAIR_BIAS_SEPARATE = 1, LF_PAIR_BIAS_NORMALIZED_INPUT = 2 } lf_pair_bias;
typedef struct lf_attention_desc {
  int32_t batch, query_length, channels, heads;
  int32_t transpose;
  int32_t pair_bias;           /* lf_pair_bias */
  int32_t pair_channels;       /* channels of pair_activations (SEPARATE) */
  int32_t swap_transposed_bias;/* AF3 dialect bit; -1 = not applicable (AF2 weights) */
  int32_t variance, precision, residual;
  float epsilon;
  int32_t space, act_dtype;
  const void* activations;     /* [batch*query_length, channels] in memory order */
  const float* mask;           /* [batch*query_length] in memory order */
  const void* pair_activations;/* [Q, Q, pair_channels] when SEPARATE */
  void* out;
  const lf_weights* weights;
} lf_attention_desc;
LF_API lf_status lf_attention_run(lf_context* ctx, const lf_attention_desc* d, lf_result* r);

/* TransitionGpu.run (webgpu/kernels/transition.js:1009-1105) for
 * TRANSITION_AF2 weights and Af3TransitionGpu.run
 * (webgpu/af3/trunk/transition.js:579) for TRANSITION_AF3. */
typedef struct lf_transition_desc {
  int64_t rows;
  int32_t channels, hidden;    /* hidden = hiddenChannels (AF2) or factor*channels (AF3) */
  int32_t variance, precision, residual;
  float epsilon;
  int32_t space, act_dtype;
  const void* activations;
  void* out;
  const lf_weights* weights;
} lf_transition_desc;
LF_API lf_status lf_transition_run(lf_context* ctx, const lf_transition_desc* d, lf_result* r);

/* OuterProductMeanGpu.run (webgpu/kernels/outer-product-mean.js:1748).
 * out[length,length,c_z] = update, or pair + update when `residual`. */
typedef struct lf_opm_desc {
  int32_t sequences, length, c_m, c_outer, c_z;
  int32_t variance, precision, residual;
  float layer_norm_epsilon;    /* 1e-5 in the reference */
  float normalization_epsilon; /* 1e-3 in the reference */
  int32_t space, act_dtype;    /* act_dtype applies to `out` (the pair) */
  const float* activations;    /* msa [sequences, length, c_m] float32 */
  const float* mask;           /* [sequences, length] */
  void* out;                   /* pair */
  const lf_weights* weights;
  int32_t bias_after_norm;     /* 0: (sum + bias) / (epsilon + count); 1: sum / max(count, 1) + bias, the
                                * dialect key opmBiasAfterNorm (cpu/af3/trunk/msa.js:81,141-150) */
} lf_opm_desc;
LF_API lf_status lf_outer_product_mean_run(lf_context* ctx, const lf_opm_desc* d, lf_result* r);

/* Af3SingleAttentionGpu.run (webgpu/af3/trunk/single-attention.js:504) fused
 * with the pair-logits pass that feeds it
 * (webgpu/af3/trunk/pairformer-block.js:157-230): single += attention(single,
 * LN(pair).W). */
typedef struct lf_single_attention_desc {
  int32_t tokens, channels, heads, head_dim, pair_channels;
  int32_t precision, residual;
  int32_t space, pair_dtype;
  const float* single;         /* [tokens, channels] float32 */
  const void* pair;            /* [tokens, tokens, pair_channels] */
  const float* seq_mask;       /* [tokens] */
  float* out;                  /* [tokens, channels] */
  const lf_weights* weights;
} lf_single_attention_desc;
LF_API lf_status lf_single_attention_run(lf_context* ctx, const lf_single_attention_desc* d, lf_result* r);

/* Af3MsaAttentionGpu.run (webgpu/af3/trunk/msa-attention.js:501-520; CPU form
 * cpu/af3/trunk/msa.js:164-224): MSA pair-weighted averaging.  The attention
 * weights come from the pair alone - softmax over keys of LN(pair).pairLogits
 * with one key mask for every sequence, the maximum of msa_mask over the
 * depth - and average the values v = LN(msa).vProjection of each sequence;
 * the result is gated by sigmoid(LN(msa).gatingQuery) and projected back to
 * the MSA channels.  Float32 arithmetic in either precision mode. */
typedef struct lf_msa_attention_desc {
  int32_t sequences, tokens, channels, heads, head_dim, pair_channels;
  int32_t precision, residual; /* residual: out = msa + update */
  int32_t space, pair_dtype;   /* lf_dtype of pair in device space */
  const float* msa;            /* [sequences, tokens, channels] float32 */
  const float* msa_mask;       /* [sequences, tokens] float32 */
  const void* pair;            /* [tokens, tokens, pair_channels] */
  float* out;                  /* [sequences, tokens, channels] float32 */
  const lf_weights* weights;   /* MSA_ATTENTION_AF3 */
} lf_msa_attention_desc;
LF_API lf_status lf_msa_attention_run(lf_context* ctx, const lf_msa_attention_desc* d, lf_result* r);

/* encodeGlobalAttention (webgpu/af2/evoformer/block.js:953-1032, shaders
 * :100-482): the global column attention of the extra-MSA stack.  Per column
 * one query - the masked mean over the sequences of the normalised MSA,
 * projected onto the heads - against one shared key/value head per sequence
 * (masked sequences at -1e9); the attended vector is gated per sequence and
 * projected.  Float32 arithmetic in either precision mode; head_dim <= 32. */
typedef struct lf_global_attention_desc {
  int32_t sequences, length, channels, heads;
  int32_t variance, precision, residual;
  float epsilon;
  int32_t space, act_dtype;
  const void* activations;     /* msa [sequences, length, channels] */
  const float* mask;           /* [sequences, length] float32 */
  void* out;
  const lf_weights* weights;   /* GLOBAL_ATTENTION_AF2 */
} lf_global_attention_desc;
LF_API lf_status lf_global_column_attention_run(lf_context* ctx, const lf_global_attention_desc* d, lf_result* r);

/* The logits of distogramHead (cpu/af3/trunk/trunk.js:47-60): half =
 * pair.half_logits (+ bias), logits[i,j] = half[i,j] + half[j,i] - a sum, not a
 * mean.  `half_logits` (channels, bins) and the optional `bias` (bins) live in
 * the same space as the pair; the logits are float32. */
typedef struct lf_distogram_desc {
  int32_t tokens, channels, bins;
  int32_t space, pair_dtype;
  const void* pair;            /* [tokens, tokens, channels] */
  const float* half_logits;    /* [channels, bins] */
  const float* bias;           /* [bins] or null */
  float* out;                  /* [tokens, tokens, bins] */
} lf_distogram_desc;
LF_API lf_status lf_distogram_logits_run(lf_context* ctx, const lf_distogram_desc* d, lf_result* r);

/* One block's worth of pair updates on a caller-owned pair, in the
 * reference's order with each update added into the running pair:
 * triangle out, triangle in, attention start, attention end, transition
 * (webgpu/af2/evoformer/block.js:1575-1612 for AF2 weights;
 * cpu/af3/trunk/pairformer.js:505-513 and webgpu/af3/trunk/pair-track.js:929
 * for AF3 weights).  Runs blocks [first_block, first_block + n_blocks) of the
 * `blocks` table on the same pair, which is what EvoformerStackGpu /
 * ExtraMsaPairStackGpu / Af3PairformerStackGpu do with a resident pair
 * (webgpu/af2/evoformer/stack.js:44-163, webgpu/af3/trunk/pairformer-block.js:290-343).
 *
 * Host-space calls whose pair does not fit on the device beside the operators' scratch (the arena is
 * refused) do not fail: in the 16-bit mode with cZ = cHidden = 128, 4 heads and a length that is a
 * multiple of 16 the pair stays in the caller's buffer (pinned for the call) and streams through the
 * device in chunks of rows - columns for the ending-node attention - with one cudaMemcpyAsync /
 * cudaMemcpy2DAsync per chunk and direction, double-buffered against the kernels; only the fp16
 * triangle operands and the pair bias stay resident.  This stands where the reference has its host
 * spill and row-chunked pair track (webgpu/runtime/host-spill.js:13-78,
 * webgpu/af3/trunk/pair-track.js:967-1000).  Results are those of the resident path. */
/* Order of the five updates inside a block.  EVOFORMER: triangle out, triangle in, attention start,
 * attention end, transition (main and extra-MSA stacks, AF3 pair track).  TEMPLATE: attention start,
 * attention end, triangle out, triangle in, transition - the template pair stack, which is the same
 * block at 64 channels (encodeTemplatePairBlock: webgpu/af2/evoformer/block.js:1746-1781). */
typedef enum lf_pair_block_order { LF_ORDER_EVOFORMER = 0, LF_ORDER_TEMPLATE = 1 } lf_pair_block_order;
typedef struct lf_pair_block_weights {
  const lf_weights* triangle_outgoing;
  const lf_weights* triangle_incoming;
  const lf_weights* attention_starting;
  const lf_weights* attention_ending;
  const lf_weights* transition;
} lf_pair_block_weights;
typedef struct lf_pair_stack_desc {
  int32_t length, c_z, c_hidden, heads, transition_hidden;
  int32_t variance, precision;
  int32_t swap_transposed_bias;/* AF3 dialect bit; -1 for AF2 weights */
  float epsilon;
  int32_t space, act_dtype;
  void* pair;                  /* updated in place */
  const float* mask;           /* [length, length] */
  const lf_pair_block_weights* blocks;
  int32_t block_count, first_block, n_blocks;
  int32_t order;               /* lf_pair_block_order */
} lf_pair_stack_desc;
LF_API lf_status lf_pair_stack_run(lf_context* ctx, const lf_pair_stack_desc* d, lf_result* r);

/* ---- row-sharded pair stack (several GPUs) ------------------------------- */

/* The reference is single-device; for large N this library shards the pair by rows over the GPUs
 * of one box (one process per GPU).  The host runs the block as a sequence of shard-local steps and
 * puts the collectives between them (all-gather of the triangle operand b and of the pair bias,
 * all-to-all transposes of the pair): see localfold_b200/sharded.py.  One entry point runs any
 * step on the local shard `pair` [rows][length][128] (device memory, 16-bit tensor-core path,
 * c_z = c_hidden = 128, 4 heads); `buf` holds the step's fp16 device buffers, which the caller
 * allocates and moves between ranks.  With ld = length rounded up to 16:
 *   TRIANGLE_PROJECT   buf0 = a, buf1 = b                      [128][rows][ld]
 *   TRIANGLE_CONTRACT  buf0 = a, buf1 = b of rank `chunk`, buf2 = x [128][rows][ld]: fills
 *                      x[:, :, chunk*rows : (chunk+1)*rows]    (outgoing form; rows % 16 == 0)
 *   TRIANGLE_OUTPUT    buf2 = x; pair += output(x, pair)
 *   ATTENTION_PROJECT  buf0..3 = q, k, v, gate: rows*length*128 fp16 each, in the library's own piece order
 *                      (scratch between the attention steps, not meant to be read); buf4 = this shard's pair bias
 *                      [4][rows][ld] (head, query row of the shard, key)
 *   ATTENTION_CORE     buf0..3; buf4 = the bias of all query rows [4][length][ld], the shards'
 *                      rows in rank order under each head; buf5 = o
 *   ATTENTION_OUTPUT   buf5 = o; pair += o Wo + bo
 *   TRANSITION         pair += transition(pair)
 * The incoming triangle update and the ending-node attention run as the outgoing / starting forms
 * on the transposed shard (incoming(z) = outgoing(z^T)^T), with the mask rows of the transposed mask. */
typedef enum lf_shard_op {
  LF_SHARD_TRIANGLE_PROJECT = 1, LF_SHARD_TRIANGLE_CONTRACT = 2, LF_SHARD_TRIANGLE_OUTPUT = 3,
  LF_SHARD_ATTENTION_PROJECT = 4, LF_SHARD_ATTENTION_CORE = 5, LF_SHARD_ATTENTION_OUTPUT = 6,
  LF_SHARD_TRANSITION = 7
} lf_shard_op;
typedef struct lf_shard_step_desc {
  int32_t op;                  /* lf_shard_op */
  int32_t rows, length;        /* pair rows on this rank, row length */
  int32_t ranks, chunk;        /* number of row shards; TRIANGLE_CONTRACT: whose b rows buf1 holds */
  int32_t variance;            /* lf_variance */
  float epsilon;
  int32_t act_dtype;           /* lf_dtype of `pair` */
  void* pair;
  const float* mask;           /* [rows][length] */
  void* buf[6];
  const lf_weights* weights;
} lf_shard_step_desc;
LF_API lf_status lf_pair_shard_step(lf_context* ctx, const lf_shard_step_desc* d, lf_result* r);

/* ------------------------------------------------------------------------------------------
 * The same steps with the exchange between the GPUs of one box fused into the kernels that produce
 * the data (plain stores into the peers' memory over NVLink; buffers shared as for the transpose
 * below).  The reference is single-device: no counterpart there.
 *
 * Triangle multiplication, channel-sharded: rank g contracts channels [g c, (g+1) c), c = 128 / ranks,
 * over the whole N x N plane, so every tile of the contraction is full-size and neither direction
 * needs a transposed pair.
 *   TRIANGLE_PROJECT   the epilogue of the LayerNorm + projection kernel stores channel h of this
 *                      shard's rows into a[h / c], b[h / c] (rank h / c's [c][length][ld] buffers) at
 *                      rows rank*rows ..: 7/8 of the operands leave over NVLink while the kernel runs
 *   TRIANGLE_CONTRACT  a[rank], b[rank] (complete after a barrier of the caller's) -> rows i of
 *                      the product of channel h go to x[i / rows] (rank i / rows's [128][rows][ld] buffer)
 *                      at channel rank*c + h; `incoming` picks the form
 *   ATTENTION_PROJECT  buf0..3 = q, k, v, gate as for lf_pair_shard_step; the shard's pair-bias rows are
 *                      stored into every bias[g] ([4][length][ld], all query rows) at rows rank*rows ..
 * After each step the caller runs a barrier on the same stream (e.g. a one-element NCCL all-reduce):
 * when it has passed on a rank, every peer's stores into that rank's buffers have landed.  The
 * remaining steps (TRIANGLE_OUTPUT on x[rank], ATTENTION_CORE on bias[rank], ...) are lf_pair_shard_step's.
 * length must be a multiple of 16 and rows a multiple of 128; 128 % ranks == 0.
 * ------------------------------------------------------------------------------------------ */
typedef struct lf_shard_peers {
  int32_t rank;          /* this rank */
  int32_t incoming;      /* TRIANGLE_CONTRACT: 0 outgoing, 1 incoming */
  void* a[16];           /* per rank, as mapped in this process (entry `rank` is the local buffer) */
  void* b[16];
  void* x[16];
  void* bias[16];
} lf_shard_peers;
LF_API lf_status lf_pair_shard_exchange_step(lf_context* ctx, const lf_shard_step_desc* d, const lf_shard_peers* peers,
                                             lf_result* r);
/* The operand exchange as a copy of its own, for comparison with the fused form: src [channels][rows][length] fp16
 * (what TRIANGLE_PROJECT of lf_pair_shard_step writes) -> plane h to rank h / (channels / ranks), plane
 * h % (channels / ranks) of dst[...] ([channels / ranks][length][length]), rows rank*rows ..; each plane of the shard is
 * one contiguous run, copied 16 bytes per lane over NVLink. */
LF_API lf_status lf_pair_planes_scatter(lf_context* ctx, const void* src, int32_t channels, int32_t rows, int32_t length,
                                        int32_t ranks, int32_t rank, void* const* dst);

/* ------------------------------------------------------------------------------------------
 * Transpose of the row-sharded pair across the GPUs of one box, written directly into the
 * peers' memory.  The reference is single-device: no counterpart there.
 *
 * lf_peer_buffer_create allocates a device buffer and returns its 64-byte CUDA IPC handle; the
 * ranks (one process per GPU) exchange handles by their own means and map each other's buffers
 * with lf_peer_buffer_open.  lf_pair_transpose_scatter then moves this rank's shard
 * src [rows][length][vector_bytes] so that dst[d] (rank d's buffer, as mapped in this process;
 * dst[rank] is the local one) receives zT[m][rank*rows + r] = z[r][d*rows + m]: after every rank
 * has run it and a barrier of the caller's (e.g. an NCCL collective on the same stream) has
 * passed, each buffer holds that rank's rows of the transposed pair.  vector_bytes = 512 (128
 * float32 channels) or 256 (128 bf16 channels).  The kernel uses plain peer stores over NVLink.
 * ------------------------------------------------------------------------------------------ */
LF_API lf_status lf_peer_buffer_create(lf_context* ctx, size_t bytes, void** ptr, unsigned char handle[64]);
LF_API lf_status lf_peer_buffer_open(lf_context* ctx, const unsigned char handle[64], void** ptr);
LF_API lf_status lf_peer_buffer_close(lf_context* ctx, void* ptr);
LF_API lf_status lf_peer_buffer_destroy(lf_context* ctx, void* ptr);
LF_API lf_status lf_pair_transpose_scatter(lf_context* ctx, const void* src, int32_t rows, int32_t length,
                                           int32_t vector_bytes, int32_t ranks, int32_t rank, void* const* dst);

#ifdef __cplusplus
}
#endif
#endif /* LOCALFOLD_PAIRSTACK_H */
