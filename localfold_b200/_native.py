"""ctypes binding of ``liblocalfold_pairstack.so`` (the C ABI in
``include/localfold_pairstack.h``).  There is no fallback: if the library is
missing or a call fails, an exception is raised."""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# the in-tree build; LOCALFOLD_PAIRSTACK_LIB points at another build of the same ABI (e.g. a variant being measured)
LIB_PATH = os.environ.get("LOCALFOLD_PAIRSTACK_LIB") or os.path.join(HERE, "lib", "liblocalfold_pairstack.so")

LF_OK, LF_ERR_SHAPE, LF_ERR_ARGUMENT, LF_ERR_CUDA, LF_ERR_MEMORY, LF_ERR_UNSUPPORTED, LF_ERR_TIMEOUT = range(7)
SPACE_HOST, SPACE_DEVICE = 0, 1
DTYPE_F32, DTYPE_BF16 = 0, 1
PRECISION_F32, PRECISION_BF16 = 0, 1
VARIANCE_TWO_PASS, VARIANCE_FAST = 1, 2
PAIR_BIAS_NONE, PAIR_BIAS_SEPARATE, PAIR_BIAS_NORMALIZED_INPUT = 0, 1, 2
ORDER_EVOFORMER, ORDER_TEMPLATE = 0, 1
(WEIGHTS_TRIANGLE_AF2, WEIGHTS_TRIANGLE_AF3, WEIGHTS_ATTENTION_AF2, WEIGHTS_GRID_ATTENTION_AF3,
 WEIGHTS_TRANSITION_AF2, WEIGHTS_TRANSITION_AF3, WEIGHTS_OPM_AF2, WEIGHTS_SINGLE_ATTENTION_AF3,
 WEIGHTS_MSA_ATTENTION_AF3, WEIGHTS_GLOBAL_ATTENTION_AF2) = range(1, 11)

KERNEL_FAMILIES = ("simt", "triangle_contract", "ln_gemm", "triangle_output", "attention", "transition",
                   "elementwise")

c_void_p, c_int32, c_int64, c_float = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_float


class RangeError(ValueError):
    """Shape validation failure (the reference throws RangeError)."""


class NativeError(RuntimeError):
    pass


class Result(ctypes.Structure):
    _fields_ = [("elapsed_ms", c_float), ("peak_bytes", ctypes.c_uint64), ("launches", ctypes.c_uint32)]


class WeightDims(ctypes.Structure):
    _fields_ = [("channels", c_int32), ("hidden", c_int32), ("heads", c_int32), ("head_dim", c_int32),
                ("pair_channels", c_int32), ("out_channels", c_int32)]


class TriangleDesc(ctypes.Structure):
    _fields_ = [("length", c_int32), ("c_z", c_int32), ("c_hidden", c_int32), ("incoming", c_int32),
                ("variance", c_int32), ("precision", c_int32), ("residual", c_int32),
                ("divide_by_length", c_int32), ("epsilon", c_float), ("space", c_int32),
                ("act_dtype", c_int32), ("z", c_void_p), ("mask", c_void_p), ("out", c_void_p),
                ("weights", c_void_p)]


class AttentionDesc(ctypes.Structure):
    _fields_ = [("batch", c_int32), ("query_length", c_int32), ("channels", c_int32), ("heads", c_int32),
                ("transpose", c_int32), ("pair_bias", c_int32), ("pair_channels", c_int32),
                ("swap_transposed_bias", c_int32), ("variance", c_int32), ("precision", c_int32),
                ("residual", c_int32), ("epsilon", c_float), ("space", c_int32), ("act_dtype", c_int32),
                ("activations", c_void_p), ("mask", c_void_p), ("pair_activations", c_void_p),
                ("out", c_void_p), ("weights", c_void_p)]


class TransitionDesc(ctypes.Structure):
    _fields_ = [("rows", c_int64), ("channels", c_int32), ("hidden", c_int32), ("variance", c_int32),
                ("precision", c_int32), ("residual", c_int32), ("epsilon", c_float), ("space", c_int32),
                ("act_dtype", c_int32), ("activations", c_void_p), ("out", c_void_p), ("weights", c_void_p)]


class OpmDesc(ctypes.Structure):
    _fields_ = [("sequences", c_int32), ("length", c_int32), ("c_m", c_int32), ("c_outer", c_int32),
                ("c_z", c_int32), ("variance", c_int32), ("precision", c_int32), ("residual", c_int32),
                ("layer_norm_epsilon", c_float), ("normalization_epsilon", c_float), ("space", c_int32),
                ("act_dtype", c_int32), ("activations", c_void_p), ("mask", c_void_p), ("out", c_void_p),
                ("weights", c_void_p), ("bias_after_norm", c_int32)]


class SingleAttentionDesc(ctypes.Structure):
    _fields_ = [("tokens", c_int32), ("channels", c_int32), ("heads", c_int32), ("head_dim", c_int32),
                ("pair_channels", c_int32), ("precision", c_int32), ("residual", c_int32),
                ("space", c_int32), ("pair_dtype", c_int32), ("single", c_void_p), ("pair", c_void_p),
                ("seq_mask", c_void_p), ("out", c_void_p), ("weights", c_void_p)]


class MsaAttentionDesc(ctypes.Structure):
    _fields_ = [("sequences", c_int32), ("tokens", c_int32), ("channels", c_int32), ("heads", c_int32),
                ("head_dim", c_int32), ("pair_channels", c_int32), ("precision", c_int32), ("residual", c_int32),
                ("space", c_int32), ("pair_dtype", c_int32), ("msa", c_void_p), ("msa_mask", c_void_p),
                ("pair", c_void_p), ("out", c_void_p), ("weights", c_void_p)]


class GlobalAttentionDesc(ctypes.Structure):
    _fields_ = [("sequences", c_int32), ("length", c_int32), ("channels", c_int32), ("heads", c_int32),
                ("variance", c_int32), ("precision", c_int32), ("residual", c_int32), ("epsilon", c_float),
                ("space", c_int32), ("act_dtype", c_int32), ("activations", c_void_p), ("mask", c_void_p),
                ("out", c_void_p), ("weights", c_void_p)]


class DistogramDesc(ctypes.Structure):
    _fields_ = [("tokens", c_int32), ("channels", c_int32), ("bins", c_int32), ("space", c_int32),
                ("pair_dtype", c_int32), ("pair", c_void_p), ("half_logits", c_void_p), ("bias", c_void_p),
                ("out", c_void_p)]


class PairBlockWeights(ctypes.Structure):
    _fields_ = [("triangle_outgoing", c_void_p), ("triangle_incoming", c_void_p),
                ("attention_starting", c_void_p), ("attention_ending", c_void_p), ("transition", c_void_p)]


class PairStackDesc(ctypes.Structure):
    _fields_ = [("length", c_int32), ("c_z", c_int32), ("c_hidden", c_int32), ("heads", c_int32),
                ("transition_hidden", c_int32), ("variance", c_int32), ("precision", c_int32),
                ("swap_transposed_bias", c_int32), ("epsilon", c_float), ("space", c_int32),
                ("act_dtype", c_int32), ("pair", c_void_p), ("mask", c_void_p),
                ("blocks", ctypes.POINTER(PairBlockWeights)), ("block_count", c_int32),
                ("first_block", c_int32), ("n_blocks", c_int32), ("order", c_int32)]


(SHARD_TRIANGLE_PROJECT, SHARD_TRIANGLE_CONTRACT, SHARD_TRIANGLE_OUTPUT, SHARD_ATTENTION_PROJECT,
 SHARD_ATTENTION_CORE, SHARD_ATTENTION_OUTPUT, SHARD_TRANSITION) = range(1, 8)


class ShardStepDesc(ctypes.Structure):
    _fields_ = [("op", c_int32), ("rows", c_int32), ("length", c_int32), ("ranks", c_int32), ("chunk", c_int32),
                ("variance", c_int32), ("epsilon", c_float), ("act_dtype", c_int32), ("pair", c_void_p),
                ("mask", c_void_p), ("buf", c_void_p * 6), ("weights", c_void_p)]


class EncodedTensorDesc(ctypes.Structure):
    _fields_ = [("dtype", c_int32), ("block", c_int32), ("data", c_void_p), ("count", c_int64),
                ("payload_bytes", ctypes.c_uint64), ("scale_offset", ctypes.c_uint64), ("zero_offset", ctypes.c_uint64)]


TENSOR_F32, TENSOR_INT5 = 0, 1


class ShardPeers(ctypes.Structure):
    _fields_ = [("rank", c_int32), ("incoming", c_int32), ("a", c_void_p * 16), ("b", c_void_p * 16),
                ("x", c_void_p * 16), ("bias", c_void_p * 16)]


EXPORTS = (
    "lf_version", "lf_context_create", "lf_context_create_on_stream", "lf_context_stream", "lf_context_destroy", "lf_last_error", "lf_context_synchronize",
    "lf_context_launch_count", "lf_context_profile", "lf_context_profile_read", "lf_context_reserve", "lf_context_release_scratch", "lf_context_limit_scratch", "lf_weights_create", "lf_weights_create_encoded",
    "lf_weights_destroy", "lf_int5_decode", "lf_triangle_multiplication_run",
    "lf_triangle_multiplication_run_static", "lf_attention_run",
    "lf_transition_run", "lf_outer_product_mean_run", "lf_single_attention_run", "lf_msa_attention_run",
    "lf_global_column_attention_run", "lf_distogram_logits_run", "lf_pair_stack_run",
    "lf_pair_shard_step", "lf_pair_shard_exchange_step", "lf_pair_planes_scatter", "lf_peer_buffer_create", "lf_peer_buffer_open", "lf_peer_buffer_close",
    "lf_peer_buffer_destroy", "lf_pair_transpose_scatter",
)

_lib = None


def load():
    """Load the shared library; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise NativeError(f"{LIB_PATH} is missing: run `python -m localfold_b200.build` (there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    lib.lf_version.restype = ctypes.c_char_p
    lib.lf_last_error.restype = ctypes.c_char_p
    lib.lf_last_error.argtypes = [c_void_p]
    lib.lf_context_create.argtypes = [ctypes.c_int, c_void_p, ctypes.POINTER(c_void_p)]
    lib.lf_context_create_on_stream.argtypes = [ctypes.c_int, c_void_p, ctypes.POINTER(c_void_p)]
    lib.lf_context_stream.argtypes = [c_void_p]
    lib.lf_context_stream.restype = c_void_p
    lib.lf_context_destroy.argtypes = [c_void_p]
    lib.lf_context_destroy.restype = None
    lib.lf_context_synchronize.argtypes = [c_void_p]
    lib.lf_context_launch_count.argtypes = [c_void_p]
    lib.lf_context_launch_count.restype = ctypes.c_uint64
    lib.lf_context_profile.argtypes = [c_void_p, ctypes.c_int]
    lib.lf_context_profile_read.argtypes = [c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_double),
                                            ctypes.POINTER(ctypes.c_uint64)]
    lib.lf_context_reserve.argtypes = [c_void_p, ctypes.c_uint64]
    lib.lf_context_limit_scratch.argtypes = [c_void_p, ctypes.c_uint64]
    lib.lf_context_release_scratch.argtypes = [c_void_p]
    lib.lf_context_release_scratch.restype = None
    lib.lf_weights_create.argtypes = [c_void_p, ctypes.c_int, ctypes.POINTER(WeightDims),
                                      ctypes.POINTER(c_void_p), ctypes.POINTER(c_int64), c_int32,
                                      ctypes.POINTER(c_void_p)]
    lib.lf_weights_create_encoded.argtypes = [c_void_p, ctypes.c_int, ctypes.POINTER(WeightDims),
                                              ctypes.POINTER(EncodedTensorDesc), c_int32, ctypes.POINTER(c_void_p)]
    lib.lf_weights_destroy.argtypes = [c_void_p]
    lib.lf_weights_destroy.restype = None
    lib.lf_int5_decode.argtypes = [c_void_p, c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
                                   c_int64, c_int32, ctypes.c_int, c_void_p]
    for name, desc in (("lf_triangle_multiplication_run", TriangleDesc),
                       ("lf_triangle_multiplication_run_static", TriangleDesc), ("lf_attention_run", AttentionDesc),
                       ("lf_transition_run", TransitionDesc), ("lf_outer_product_mean_run", OpmDesc),
                       ("lf_single_attention_run", SingleAttentionDesc), ("lf_msa_attention_run", MsaAttentionDesc),
                       ("lf_global_column_attention_run", GlobalAttentionDesc),
                       ("lf_distogram_logits_run", DistogramDesc), ("lf_pair_stack_run", PairStackDesc),
                       ("lf_pair_shard_step", ShardStepDesc)):
        getattr(lib, name).argtypes = [c_void_p, ctypes.POINTER(desc), ctypes.POINTER(Result)]
    lib.lf_pair_shard_exchange_step.argtypes = [c_void_p, ctypes.POINTER(ShardStepDesc), ctypes.POINTER(ShardPeers),
                                                ctypes.POINTER(Result)]
    lib.lf_pair_planes_scatter.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, ctypes.POINTER(c_void_p)]
    lib.lf_peer_buffer_create.argtypes = [c_void_p, ctypes.c_size_t, ctypes.POINTER(c_void_p), ctypes.c_char_p]
    lib.lf_peer_buffer_open.argtypes = [c_void_p, ctypes.c_char_p, ctypes.POINTER(c_void_p)]
    lib.lf_peer_buffer_close.argtypes = [c_void_p, c_void_p]
    lib.lf_peer_buffer_destroy.argtypes = [c_void_p, c_void_p]
    lib.lf_pair_transpose_scatter.argtypes = [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32,
                                              ctypes.POINTER(c_void_p)]
    _lib = lib
    return lib


def check(lib, ctx, status):
    if status == LF_OK:
        return
    message = lib.lf_last_error(ctx).decode() if ctx else "no context"
    if status == LF_ERR_SHAPE:
        raise RangeError(message)
    if status == LF_ERR_ARGUMENT:
        raise ValueError(message)
    if status == LF_ERR_MEMORY:
        raise MemoryError(message)
    if status == LF_ERR_UNSUPPORTED:
        raise NotImplementedError(message)
    raise NativeError(f"status {status}: {message}")
