"""Host-side mirror of the reference's operator API for the pair stack.

Same class names, ``run(input[, options])`` signatures, input field names, weight
field names and error behaviour as the reference's kernel library
(``webgpu/index.js:1-10,60-61``); each class forwards to one entry point of the
C ABI (``include/localfold_pairstack.h``).  Inputs are numpy float32 arrays
(host space) or CUDA tensors exposing ``data_ptr()`` / ``is_cuda`` (device
space, e.g. torch tensors; outputs are then written into caller tensors).

Where the reference takes ``precision: "f32" | "f16"``, this library takes
``"f32" | "bf16"``.  ``variance`` has no default where the reference has none.
"""
from __future__ import annotations

import ctypes
import weakref

import numpy as np

from . import _native as nat
from ._native import RangeError  # noqa: F401  (re-exported)

TRIANGLE_WEIGHT_ORDER = (
    "layerNormInWeight", "layerNormInBias", "linearAPWeight", "linearAPBias",
    "linearAGWeight", "linearAGBias", "linearBPWeight", "linearBPBias",
    "linearBGWeight", "linearBGBias", "layerNormOutWeight", "layerNormOutBias",
    "linearZWeight", "linearZBias", "linearGWeight", "linearGBias",
)  # webgpu/kernels/triangle/weights.js:4-10
TRIANGLE_AF3_ORDER = ("leftNormInputScale", "leftNormInputOffset", "projection", "gate",
                      "centerNormScale", "centerNormOffset", "outputProjection", "gatingLinear")
ATTENTION_WEIGHT_ORDER = ("queryNormScale", "queryNormOffset", "queryWeight", "keyWeight", "valueWeight",
                          "gatingWeight", "gatingBias", "outputWeight", "outputBias")  # attention.js:64-80
GRID_ATTENTION_AF3_ORDER = ("actNormScale", "actNormOffset", "pairBiasProjection", "qProjection",
                            "kProjection", "vProjection", "gatingQuery", "outputProjection")
TRANSITION_WEIGHT_ORDER = ("layerNormScale", "layerNormOffset", "firstWeight", "firstBias",
                           "secondWeight", "secondBias")  # transition.js:477-480
TRANSITION_AF3_ORDER = ("inputLayerNormScale", "inputLayerNormOffset", "transition1", "transition2")
OPM_WEIGHT_ORDER = ("layerNormScale", "layerNormOffset", "leftWeight", "leftBias", "rightWeight",
                    "rightBias", "outputWeight", "outputBias")  # outer-product-mean.js:72-75
SINGLE_ATTENTION_AF3_ORDER = ("layerNormScale", "layerNormOffset", "qProjection", "qBias", "kProjection",
                              "vProjection", "gatingQuery", "outputProjection")

_PRECISION = {"f32": nat.PRECISION_F32, "bf16": nat.PRECISION_BF16}
_VARIANCE = {"two-pass": nat.VARIANCE_TWO_PASS, "fast": nat.VARIANCE_FAST}


def _precision(options, default="f32"):
    value = (options or {}).get("precision", default)
    if value not in _PRECISION:
        raise ValueError(f'precision must be "f32" or "bf16"; received {value!r}')
    return _PRECISION[value]


def _variance(options, default=None):
    value = (options or {}).get("variance", default)
    if value not in _VARIANCE:
        raise ValueError('variance has no default here: pass "two-pass" or "fast"')
    return _VARIANCE[value]


class Device:
    """One GPU context (stands where the reference passes a ``GPUDevice``;
    ``createNodeDevice``: ``webgpu/node.js:51-81``)."""

    def __init__(self, ordinal: int = 0, stream: int | None = None):
        """``stream``: None - the context makes a stream of its own; an integer - that ``cudaStream_t``
        (0 is CUDA's default stream).  Every call enqueues on that stream and returns without waiting, so
        a device-tensor ``output`` is ready only after ``synchronize()`` or for work enqueued on the
        same stream (``stream`` gives its handle).  Inputs: a context with a stream of its own waits, on
        the device, for what torch has enqueued on its current stream when a device tensor is handed to a
        call (``wait_for_torch``); nothing orders torch's later work after the call's results."""
        self.lib = nat.load()
        handle = ctypes.c_void_p()
        if stream is None:
            status = self.lib.lf_context_create(int(ordinal), None, ctypes.byref(handle))
        else:
            status = self.lib.lf_context_create_on_stream(int(ordinal), ctypes.c_void_p(int(stream)), ctypes.byref(handle))
        if status != nat.LF_OK:
            raise nat.NativeError(f"lf_context_create({ordinal}) failed with status {status}: no usable CUDA device")
        self.handle = handle
        self.ordinal = ordinal
        self.stream = int(self.lib.lf_context_stream(handle) or 0)
        self._finalizer = weakref.finalize(self, self.lib.lf_context_destroy, handle)
        self._torch_stream = None
        if stream is None:
            _own_stream_devices.setdefault(int(ordinal), weakref.WeakSet()).add(self)

    def wait_for_torch(self):
        """Makes the context's own stream wait (on the device, no host wait) for the work torch has enqueued so
        far on its current stream of this GPU: device tensors handed to a call are usually produced there."""
        import torch
        current = torch.cuda.current_stream(self.ordinal)
        if int(current.cuda_stream) == self.stream:
            return
        if self._torch_stream is None:
            self._torch_stream = torch.cuda.ExternalStream(self.stream, device=self.ordinal)
        self._torch_stream.wait_event(current.record_event())

    def require_current_stream(self, what):
        """Raises unless torch's current stream on this device is the context's stream: collectives and
        tensor operations that ``what`` mixes with library calls are ordered only on one stream."""
        import torch
        current = int(torch.cuda.current_stream(self.ordinal).cuda_stream)
        if current != self.stream:
            raise RuntimeError(f"{what}: torch's current stream ({current:#x}) is not the library context's stream "
                               f"({self.stream:#x}); create the Device on torch's stream (Device(ordinal, stream="
                               f"torch.cuda.current_stream().cuda_stream)) or make that stream current")

    def check(self, status):
        nat.check(self.lib, self.handle, status)

    def synchronize(self):
        self.check(self.lib.lf_context_synchronize(self.handle))

    def launch_count(self) -> int:
        return int(self.lib.lf_context_launch_count(self.handle))

    def profile(self, enable: bool):
        """Bracket every kernel launch with CUDA events (off by default)."""
        self.check(self.lib.lf_context_profile(self.handle, 1 if enable else 0))

    def profile_read(self) -> dict:
        """{family: (total device ms, launches)} accumulated since the last read."""
        out = {}
        for index, name in enumerate(nat.KERNEL_FAMILIES):
            ms, count = ctypes.c_double(), ctypes.c_uint64()
            self.check(self.lib.lf_context_profile_read(self.handle, index, ctypes.byref(ms), ctypes.byref(count)))
            out[name] = (ms.value, int(count.value))
        return out

    def reserve(self, nbytes: int):
        self.check(self.lib.lf_context_reserve(self.handle, int(nbytes)))

    def limit_scratch(self, nbytes: int):
        """Upper bound on the scratch arena (0 = none); a host-space pair stack that needs more keeps the pair
        in host memory and streams it through the device in chunks."""
        self.check(self.lib.lf_context_limit_scratch(self.handle, int(nbytes)))

    def release_scratch(self):
        self.lib.lf_context_release_scratch(self.handle)

    def close(self):
        self._finalizer()


_default_device = None
_own_stream_devices = {}      # GPU ordinal -> contexts that run on a stream of their own


def create_device(ordinal: int = 0) -> Device:
    return Device(ordinal)


def _device(device):
    global _default_device
    if device is not None:
        return device
    if _default_device is None:
        _default_device = Device(0)
    return _default_device


class EncodedTensor:
    """A tensor as a bundle stores it: the bytes of an int5 range (the codes of whole groups, then fp16 scales and
    zero points at the two offsets) with its element count and shape.  Handed to the operators in place of a
    float32 array, it goes to the device as it is and is decoded there, straight into the operator's resident
    weight layout (``lf_weights_create_encoded``); ``decode()`` gives the float32 values on the host, for
    reference arithmetic."""

    def __init__(self, payload: bytes, scale_offset: int, zero_offset: int, count: int, shape, block: int = 32):
        self.payload = bytes(payload)
        self.scale_offset, self.zero_offset, self.count, self.block = int(scale_offset), int(zero_offset), int(count), int(block)
        self.shape = tuple(int(v) for v in shape)

    @property
    def size(self):
        return self.count

    def decode(self):
        from .bundle import decode_int5_host
        return decode_int5_host(self.payload, self.scale_offset, self.zero_offset, self.count, self.block).reshape(self.shape)

    def __array__(self, dtype=None, copy=None):
        out = self.decode()
        return out if dtype is None else out.astype(dtype)


class PreparedWeights:
    """Device-resident weights of one operator (``lf_weights``).  Tensors are float32 arrays or
    ``EncodedTensor``s; with any of the latter the codes are decoded on the device."""

    def __init__(self, device: Device, kind: int, dims: dict, tensors):
        self.device = device
        self.kind = kind
        self.dims = dict(dims)
        wd = nat.WeightDims(**{k: int(v) for k, v in dims.items()})
        handle = ctypes.c_void_p()
        if any(isinstance(t, EncodedTensor) for t in tensors):
            n = len(tensors)
            descs = (nat.EncodedTensorDesc * n)()
            keep = []
            for d, t in zip(descs, tensors):
                if isinstance(t, EncodedTensor):
                    raw = np.frombuffer(t.payload, np.uint8)
                    keep.append(raw)
                    d.dtype, d.block, d.data, d.count = nat.TENSOR_INT5, t.block, raw.ctypes.data, t.count
                    d.payload_bytes, d.scale_offset, d.zero_offset = raw.size, t.scale_offset, t.zero_offset
                else:
                    a = np.zeros(0, np.float32) if t is None else np.ascontiguousarray(np.asarray(t, dtype=np.float32)).reshape(-1)
                    keep.append(a)
                    d.dtype, d.block, d.data, d.count = nat.TENSOR_F32, 0, (a.ctypes.data if a.size else None), a.size
            device.check(device.lib.lf_weights_create_encoded(device.handle, kind, ctypes.byref(wd), descs, n, ctypes.byref(handle)))
        else:
            arrays = []
            for t in tensors:
                if t is None:
                    arrays.append(np.zeros(0, np.float32))
                else:
                    arrays.append(np.ascontiguousarray(np.asarray(t, dtype=np.float32)).reshape(-1))
            n = len(arrays)
            ptrs = (ctypes.c_void_p * n)(*[a.ctypes.data if a.size else None for a in arrays])
            counts = (ctypes.c_int64 * n)(*[a.size for a in arrays])
            device.check(device.lib.lf_weights_create(device.handle, kind, ctypes.byref(wd), ptrs, counts, n,
                                                       ctypes.byref(handle)))
        self.handle = handle
        self._finalizer = weakref.finalize(self, device.lib.lf_weights_destroy, handle)

    def close(self):
        self._finalizer()


class _Buffer:
    """Host numpy array or device tensor behind one pointer."""

    def __init__(self, value, dtype=np.float32):
        self.is_device = bool(getattr(value, "is_cuda", False))
        if self.is_device:
            if not value.is_contiguous():
                raise ValueError("device tensors must be contiguous")
            # a context with a stream of its own reads this tensor after torch's pending work on it
            for ctx in tuple(_own_stream_devices.get(value.device.index, ())):
                ctx.wait_for_torch()
            self.keep = value
            self.ptr = value.data_ptr()
            self.count = value.numel()
            name = str(value.dtype)
            self.dtype = nat.DTYPE_BF16 if "bfloat16" in name else nat.DTYPE_F32
            if "bfloat16" not in name and "float32" not in name:
                raise ValueError(f"device tensors must be float32 or bfloat16; received {name}")
        else:
            arr = np.ascontiguousarray(np.asarray(value, dtype=dtype))
            self.keep = arr
            self.ptr = arr.ctypes.data
            self.count = arr.size
            self.dtype = nat.DTYPE_F32


def _expect_length(name, buf, length):
    if buf.count != length:
        raise RangeError(f"{name} has {buf.count} values; expected {length}")


def _positive(name, value):
    if not isinstance(value, (int, np.integer)) or value <= 0:
        raise RangeError(f"{name} must be a positive safe integer; received {value}")


def _result(device, res, output):
    return {"output": output, "elapsedMilliseconds": float(res.elapsed_ms),
            "memory": {"peakBytes": int(res.peak_bytes)}, "launches": int(res.launches)}


def _out_like(buf: _Buffer, shape, out=None):
    """Output buffer: a fresh float32 array for host calls, ``out`` (or a new
    tensor like the input) for device calls."""
    if buf.is_device:
        target = out if out is not None else buf.keep.new_empty(buf.keep.shape)
        return _Buffer(target), target
    arr = np.empty(shape, np.float32)
    return _Buffer(arr), arr


# ---------------------------------------------------------------------------
# triangle multiplication


def validate_triangle_input(inp):
    """``validateTriangleInput`` (``webgpu/kernels/triangle/types.js:13-48``)."""
    shape = inp["shape"]
    length, cz, ch = shape["length"], shape["cZ"], shape["cHidden"]
    _positive("length", length)
    _positive("cZ", cz)
    _positive("cHidden", ch)
    pairs = length * length

    def count(v):
        return v.numel() if hasattr(v, "numel") else np.asarray(v).size

    def expect(name, value, n):
        if count(value) != n:
            raise RangeError(f"{name} has {count(value)} values; expected {n}")

    expect("z", inp["z"], pairs * cz)
    expect("mask", inp["mask"], pairs)
    w = inp["weights"]
    if not isinstance(w, PreparedWeights):
        sizes = {"layerNormInWeight": cz, "layerNormInBias": cz, "linearAPWeight": ch * cz, "linearAPBias": ch,
                 "linearAGWeight": ch * cz, "linearAGBias": ch, "linearBPWeight": ch * cz, "linearBPBias": ch,
                 "linearBGWeight": ch * cz, "linearBGBias": ch, "layerNormOutWeight": ch, "layerNormOutBias": ch,
                 "linearZWeight": cz * ch, "linearZBias": cz, "linearGWeight": cz * cz, "linearGBias": cz}
        for name in TRIANGLE_WEIGHT_ORDER:
            expect(name, w[name], sizes[name])
    eps = inp.get("epsilon")
    if eps is not None and (not (eps > 0) or not np.isfinite(eps)):
        raise RangeError(f"epsilon must be finite and positive; received {eps}")


def error_metrics(actual, expected):
    """``errorMetrics`` (``webgpu/kernels/triangle/types.js:50-69``)."""
    a = np.asarray(actual, np.float64).reshape(-1)
    e = np.asarray(expected, np.float64).reshape(-1)
    if a.size != e.size or a.size == 0:
        raise RangeError("error metrics require equally sized, non-empty arrays")
    delta = np.abs(a - e)
    return {"meanAbsoluteError": float(delta.mean()), "maxAbsoluteError": float(delta.max()),
            "rootMeanSquareError": float(np.sqrt((delta * delta).mean()))}


def prepare_triangle_weights(device, weights, c_z, c_hidden):
    if all(k in weights for k in TRIANGLE_WEIGHT_ORDER):
        return PreparedWeights(device, nat.WEIGHTS_TRIANGLE_AF2, {"channels": c_z, "hidden": c_hidden},
                               [weights[k] for k in TRIANGLE_WEIGHT_ORDER])
    return PreparedWeights(device, nat.WEIGHTS_TRIANGLE_AF3, {"channels": c_z, "hidden": c_hidden},
                           [weights[k] for k in TRIANGLE_AF3_ORDER])


class _TriangleMultiplicationGpu:
    incoming = False

    def __init__(self, device: Device | None = None):
        self.device = _device(device)

    def run(self, input, options=None, out=None):
        """``run(input, options)`` of ``webgpu/kernels/triangle/webgpu.js:38-170``.
        ``options``: precision "f32"|"bf16" (default "f32"), variance "two-pass"|"fast"
        (default "two-pass" as in the reference), residual (adds the update into z)."""
        validate_triangle_input(input)
        options = options or {}
        shape = input["shape"]
        n, cz, ch = int(shape["length"]), int(shape["cZ"]), int(shape["cHidden"])
        dev = self.device
        w = input["weights"]
        owned = None
        if not isinstance(w, PreparedWeights):
            owned = w = prepare_triangle_weights(dev, w, cz, ch)
        try:
            z = _Buffer(input["z"])
            mask = _Buffer(input["mask"])
            if z.is_device != mask.is_device:
                raise ValueError("z and mask must live in the same space")
            obuf, output = _out_like(z, (n, n, cz), out)
            desc = nat.TriangleDesc(n, cz, ch, 1 if self.incoming else 0, _variance(options, "two-pass"),
                                    _precision(options), 1 if options.get("residual") else 0,
                                    1 if options.get("divideByLength") else 0,
                                    float(input.get("epsilon") or 1e-5),
                                    nat.SPACE_DEVICE if z.is_device else nat.SPACE_HOST, z.dtype,
                                    z.ptr, mask.ptr, obuf.ptr, w.handle)
            res = nat.Result()
            dev.check(dev.lib.lf_triangle_multiplication_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


class TriangleMultiplicationOutgoingGpu(_TriangleMultiplicationGpu):
    incoming = False


class TriangleMultiplicationIncomingGpu(_TriangleMultiplicationGpu):
    incoming = True


def af3_triangle_multiplication(device, pair, mask, n, channels, direction, weights, options=None):
    """``af3TriangleMultiplication`` (``webgpu/af3/trunk/triangle.js:148-169``):
    AF3 weights, variance fixed "fast"."""
    if direction not in ("outgoing", "incoming"):
        raise ValueError(f'direction must be "outgoing" or "incoming"; received {direction!r}')
    op = (TriangleMultiplicationIncomingGpu if direction == "incoming" else TriangleMultiplicationOutgoingGpu)(device)
    dev = op.device
    owned = None
    if not isinstance(weights, PreparedWeights):
        owned = weights = PreparedWeights(dev, nat.WEIGHTS_TRIANGLE_AF3, {"channels": channels, "hidden": channels},
                                          [weights[k] for k in TRIANGLE_AF3_ORDER])
    try:
        opts = dict(options or {})
        opts["variance"] = "fast"
        return op.run({"shape": {"length": n, "cZ": channels, "cHidden": channels}, "z": pair, "mask": mask,
                       "weights": weights}, opts)
    finally:
        if owned is not None:
            dev.synchronize()
            owned.close()


# ---------------------------------------------------------------------------
# attention


def prepare_attention_weights(device, weights, channels, heads, pair_bias=None):
    tensors = [weights[k] for k in ATTENTION_WEIGHT_ORDER]
    dims = {"channels": channels, "heads": heads}
    if pair_bias is not None:
        if pair_bias.get("source") == "separate":
            tensors += [pair_bias["layerNormScale"], pair_bias["layerNormOffset"], pair_bias["projectionWeight"]]
            dims["pair_channels"] = int(pair_bias["channels"])
        else:
            tensors += [pair_bias["projectionWeight"]]
    return PreparedWeights(device, nat.WEIGHTS_ATTENTION_AF2, dims, tensors)


def prepare_grid_attention_weights(device, weights, channels):
    tensors = [weights[k] for k in GRID_ATTENTION_AF3_ORDER]
    tensors += [weights.get("gatingQueryBias"), weights.get("outputProjectionBias")]
    return PreparedWeights(device, nat.WEIGHTS_GRID_ATTENTION_AF3,
                           {"channels": channels, "heads": int(weights["heads"]), "head_dim": int(weights["dimension"])},
                           tensors)


class AttentionGpu:
    """``AttentionGpu`` (``webgpu/kernels/attention.js:2580-2739``)."""

    def __init__(self, device: Device | None = None, options=None):
        self.device = _device(device)
        self.options = dict(options or {})

    def run(self, input, options=None, out=None):
        opts = dict(self.options)
        opts.update(options or {})
        batch, q, c, heads = (input[k] for k in ("batch", "queryLength", "channels", "heads"))
        for v in (batch, q, c, heads):
            if not isinstance(v, (int, np.integer)) or v <= 0:
                raise RangeError("attention dimensions must be positive safe integers")
        if c % heads != 0 or c // heads > 64:
            raise RangeError("the fused attention path requires an integral head dimension no larger than 64")
        dev = self.device
        pair_bias = input.get("pairBias")
        w = input["weights"]
        owned = None
        act = _Buffer(input["activations"])
        mask = _Buffer(input["mask"])
        _expect_length("activations", act, batch * q * c)
        _expect_length("mask", mask, batch * q)
        if not isinstance(w, PreparedWeights):
            for name in ATTENTION_WEIGHT_ORDER:
                size = c if name in ("queryNormScale", "queryNormOffset", "gatingBias", "outputBias") else c * c
                if np.asarray(w[name]).size != size:
                    raise RangeError(f"{name} has {np.asarray(w[name]).size} values; expected {size}")
            owned = w = prepare_attention_weights(dev, w, c, heads, pair_bias)
        try:
            mode, pair_ptr, pair_ch = nat.PAIR_BIAS_NONE, None, 0
            pair = None
            if pair_bias is not None:
                if pair_bias.get("source") == "separate":
                    mode = nat.PAIR_BIAS_SEPARATE
                    pair_ch = int(pair_bias["channels"])
                    pair = _Buffer(pair_bias["activations"])
                    _expect_length("pair activations", pair, q * q * pair_ch)
                    pair_ptr = pair.ptr
                else:
                    mode = nat.PAIR_BIAS_NORMALIZED_INPUT
            obuf, output = _out_like(act, np.asarray(input["activations"]).shape if not act.is_device else None, out)
            desc = nat.AttentionDesc(batch, q, c, heads, 1 if input.get("transpose") else 0, mode, pair_ch, -1,
                                     _variance(opts, "two-pass"), _precision(opts), 1 if opts.get("residual") else 0,
                                     float(input.get("epsilon") or 1e-5),
                                     nat.SPACE_DEVICE if act.is_device else nat.SPACE_HOST, act.dtype,
                                     act.ptr, mask.ptr, pair_ptr, obuf.ptr, w.handle)
            res = nat.Result()
            dev.check(dev.lib.lf_attention_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


class Af3GridSelfAttentionGpu:
    """``Af3GridSelfAttentionGpu.run(pair, mask, {n, channels, transpose}, weights,
    dialect, options)`` (``webgpu/af3/trunk/grid-attention.js:1264``)."""

    def __init__(self, device: Device | None = None):
        self.device = _device(device)

    def run(self, pair, mask, shape, weights, dialect, options=None, out=None):
        if dialect is None or dialect.get("swapTransposedBias") not in (True, False):
            raise ValueError("dialect.swapTransposedBias has no default: openfold3 swaps the "
                             "transposed pair bias and alphafold3 does not")
        n, c, transpose = int(shape["n"]), int(shape["channels"]), bool(shape.get("transpose"))
        dev = self.device
        owned = None
        if not isinstance(weights, PreparedWeights):
            owned = weights = prepare_grid_attention_weights(dev, weights, c)
        try:
            p = _Buffer(pair)
            m = _Buffer(mask)
            _expect_length("pair", p, n * n * c)
            _expect_length("mask", m, n * n)
            obuf, output = _out_like(p, (n, n, c), out)
            opts = options or {}
            desc = nat.AttentionDesc(n, n, c, weights.dims["heads"], 1 if transpose else 0,
                                     nat.PAIR_BIAS_NORMALIZED_INPUT, 0, 1 if dialect["swapTransposedBias"] else 0,
                                     _variance(opts, "fast"), _precision(opts), 1 if opts.get("residual") else 0,
                                     float(opts.get("epsilon") or 1e-5),
                                     nat.SPACE_DEVICE if p.is_device else nat.SPACE_HOST, p.dtype,
                                     p.ptr, m.ptr, None, obuf.ptr, weights.handle)
            res = nat.Result()
            dev.check(dev.lib.lf_attention_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


# ---------------------------------------------------------------------------
# transition


class TransitionGpu:
    """``TransitionGpu`` (``webgpu/kernels/transition.js:1009-1105``)."""

    def __init__(self, device: Device | None = None, options=None):
        self.device = _device(device)
        self.options = dict(options or {})

    def run(self, input, options=None, out=None):
        opts = dict(self.options)
        opts.update(options or {})
        rows, c, hidden = int(input["rows"]), int(input["channels"]), int(input["hiddenChannels"])
        for name, v in (("rows", rows), ("channels", c), ("hiddenChannels", hidden)):
            _positive(name, v)
        dev = self.device
        w = input["weights"]
        owned = None
        act = _Buffer(input["activations"])
        _expect_length("activations", act, rows * c)
        if not isinstance(w, PreparedWeights):
            owned = w = PreparedWeights(dev, nat.WEIGHTS_TRANSITION_AF2, {"channels": c, "hidden": hidden},
                                        [w[k] for k in TRANSITION_WEIGHT_ORDER])
        try:
            obuf, output = _out_like(act, (rows, c), out)
            desc = nat.TransitionDesc(rows, c, hidden, _variance(opts, "two-pass"), _precision(opts),
                                      1 if opts.get("residual") else 0, float(input.get("epsilon") or 1e-5),
                                      nat.SPACE_DEVICE if act.is_device else nat.SPACE_HOST, act.dtype,
                                      act.ptr, obuf.ptr, w.handle)
            res = nat.Result()
            dev.check(dev.lib.lf_transition_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


class Af3TransitionGpu:
    """``Af3TransitionGpu.run(input, {rows, channels, factor}, weights, options)``
    (``webgpu/af3/trunk/transition.js:579``)."""

    def __init__(self, device: Device | None = None):
        self.device = _device(device)

    def run(self, input, shape, weights, options=None, out=None):
        rows, c, factor = int(shape["rows"]), int(shape["channels"]), int(shape.get("factor", 4))
        dev = self.device
        owned = None
        if not isinstance(weights, PreparedWeights):
            owned = weights = PreparedWeights(dev, nat.WEIGHTS_TRANSITION_AF3, {"channels": c, "hidden": c * factor},
                                              [weights[k] for k in TRANSITION_AF3_ORDER])
        try:
            act = _Buffer(input)
            _expect_length("input", act, rows * c)
            obuf, output = _out_like(act, (rows, c), out)
            opts = options or {}
            desc = nat.TransitionDesc(rows, c, c * factor, _variance(opts, "fast"), _precision(opts),
                                      1 if opts.get("residual") else 0, float(opts.get("epsilon") or 1e-5),
                                      nat.SPACE_DEVICE if act.is_device else nat.SPACE_HOST, act.dtype,
                                      act.ptr, obuf.ptr, weights.handle)
            res = nat.Result()
            dev.check(dev.lib.lf_transition_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


# ---------------------------------------------------------------------------
# outer product mean


class OuterProductMeanGpu:
    """``OuterProductMeanGpu`` (``webgpu/kernels/outer-product-mean.js:1748``).  ``input["biasAfterNorm"]`` selects the
    form of the dialect key ``opmBiasAfterNorm``: sum / max(count, 1) + bias (``cpu/af3/trunk/msa.js:141-150``)."""

    def __init__(self, device: Device | None = None):
        self.device = _device(device)

    def run(self, input, options=None, out=None):
        S, n, cm, co, cz = (int(input[k]) for k in ("sequences", "length", "cM", "cOuter", "cZ"))
        for name, v in (("sequences", S), ("length", n), ("cM", cm), ("cOuter", co), ("cZ", cz)):
            _positive(name, v)
        if co > 32:
            raise RangeError("the outer product mean requires cOuter no larger than 32")
        dev = self.device
        w = input["weights"]
        owned = None
        act = _Buffer(input["activations"])
        mask = _Buffer(input["mask"])
        _expect_length("activations", act, S * n * cm)
        _expect_length("mask", mask, S * n)
        if not isinstance(w, PreparedWeights):
            owned = w = PreparedWeights(dev, nat.WEIGHTS_OPM_AF2, {"channels": cm, "hidden": co, "out_channels": cz},
                                        [w[k] for k in OPM_WEIGHT_ORDER])
        try:
            opts = options or {}
            residual = out is not None and opts.get("residual")
            if act.is_device:
                if out is None:
                    raise ValueError("device-space outer product mean writes into `out` (the pair)")
                obuf, output = _Buffer(out), out
            else:
                arr = np.array(out, np.float32, copy=True) if residual else np.empty((n, n, cz), np.float32)
                obuf, output = _Buffer(arr), arr
            desc = nat.OpmDesc(S, n, cm, co, cz, _variance(opts, "two-pass"), _precision(opts), 1 if residual else 0,
                               float(input.get("layerNormEpsilon") or 1e-5),
                               float(input.get("normalizationEpsilon") or 1e-3),
                               nat.SPACE_DEVICE if act.is_device else nat.SPACE_HOST, obuf.dtype,
                               act.ptr, mask.ptr, obuf.ptr, w.handle, 1 if input.get("biasAfterNorm") else 0)
            res = nat.Result()
            dev.check(dev.lib.lf_outer_product_mean_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


# ---------------------------------------------------------------------------
# AF3 single attention (with the pair-logits pass that feeds it)


def prepare_single_attention_weights(device, block_weights, channels, pair_channels):
    """Resident weights of one block's single attention: its ``singleAttention`` object plus the block's
    ``singlePairLogitsNormScale/Offset/Projection`` (``shared/af3/weights/weights.js:699-727``)."""
    att = block_weights["singleAttention"]
    tensors = [att[k] for k in SINGLE_ATTENTION_AF3_ORDER]
    tensors += [block_weights["singlePairLogitsNormScale"], block_weights["singlePairLogitsNormOffset"],
                block_weights["singlePairLogitsProjection"]]
    return PreparedWeights(device, nat.WEIGHTS_SINGLE_ATTENTION_AF3,
                           {"channels": channels, "heads": int(att["heads"]), "head_dim": int(att["dimension"]),
                            "pair_channels": pair_channels}, tensors)


class Af3SingleAttentionGpu:
    """``Af3SingleAttentionGpu`` (``webgpu/af3/trunk/single-attention.js:504``) fused
    with the block's pair-logits projection
    (``webgpu/af3/trunk/pairformer-block.js:157-230``): ``run(single, pair, seqMask,
    {n, channels, pairChannels}, weights)`` where ``weights`` is the block's
    ``singleAttention`` object plus ``singlePairLogitsNormScale/Offset/Projection``."""

    def __init__(self, device: Device | None = None):
        self.device = _device(device)

    def run(self, single, pair, seq_mask, shape, weights, options=None):
        n, c, pc = int(shape["n"]), int(shape["channels"]), int(shape["pairChannels"])
        dev = self.device
        owned = None
        if not isinstance(weights, PreparedWeights):
            owned = weights = prepare_single_attention_weights(dev, weights, c, pc)
        try:
            s = _Buffer(single)
            p = _Buffer(pair)
            m = _Buffer(seq_mask)
            _expect_length("single", s, n * c)
            _expect_length("pair", p, n * n * pc)
            _expect_length("seqMask", m, n)
            obuf, output = _out_like(s, (n, c))
            opts = options or {}
            desc = nat.SingleAttentionDesc(n, c, weights.dims["heads"], weights.dims["head_dim"], pc, _precision(opts),
                                           1 if opts.get("residual") else 0,
                                           nat.SPACE_DEVICE if s.is_device else nat.SPACE_HOST, p.dtype,
                                           s.ptr, p.ptr, m.ptr, obuf.ptr, weights.handle)
            res = nat.Result()
            dev.check(dev.lib.lf_single_attention_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


GLOBAL_ATTENTION_ORDER = ("queryNormScale", "queryNormOffset", "queryWeight", "keyWeight", "valueWeight",
                          "gatingWeight", "gatingBias", "outputWeight", "outputBias")


class GlobalColumnAttentionGpu:
    """The extra-MSA stack's global column attention (``encodeGlobalAttention``,
    ``webgpu/af2/evoformer/block.js:953-1032``): ``run({activations, mask, sequences, length, channels, weights})``
    with ``weights`` the nine tensors of ``GLOBAL_ATTENTION_ORDER`` plus ``heads``; float32 arithmetic."""

    def __init__(self, device: Device | None = None):
        self.device = _device(device)

    def run(self, input, options=None, out=None):
        S, n, c = (int(input[k]) for k in ("sequences", "length", "channels"))
        for name, v in (("sequences", S), ("length", n), ("channels", c)):
            _positive(name, v)
        dev = self.device
        w = input["weights"]
        owned = None
        act = _Buffer(input["activations"])
        mask = _Buffer(input["mask"])
        _expect_length("activations", act, S * n * c)
        _expect_length("mask", mask, S * n)
        if not isinstance(w, PreparedWeights):
            heads = w.get("heads")
            if not isinstance(heads, (int, np.integer)) or heads <= 0:
                raise RangeError("global attention weights.heads must be a positive integer")
            owned = w = PreparedWeights(dev, nat.WEIGHTS_GLOBAL_ATTENTION_AF2, {"channels": c, "heads": int(heads)},
                                        [w[k] for k in GLOBAL_ATTENTION_ORDER])
        try:
            opts = options or {}
            obuf, output = _out_like(act, (S, n, c), out)
            desc = nat.GlobalAttentionDesc(S, n, c, w.dims["heads"], _variance(opts, "two-pass"), _precision(opts),
                                           1 if opts.get("residual") else 0, float(input.get("epsilon") or 1e-5),
                                           nat.SPACE_DEVICE if act.is_device else nat.SPACE_HOST, act.dtype,
                                           act.ptr, mask.ptr, obuf.ptr, w.handle)
            res = nat.Result()
            dev.check(dev.lib.lf_global_column_attention_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


MSA_ATTENTION_AF3_ORDER = ("actNormScale", "actNormOffset", "pairNormScale", "pairNormOffset", "pairLogits",
                           "vProjection", "gatingQuery", "outputProjection")


def prepare_msa_attention_weights(device, weights, channels, pair_channels):
    """Resident weights of ``msaAttention1`` (``shared/af3/weights/weights.js:670-680``); the head width is
    ``weights["dimension"]``, not ``channels / heads``."""
    return PreparedWeights(device, nat.WEIGHTS_MSA_ATTENTION_AF3,
                           {"channels": channels, "heads": int(weights["heads"]), "head_dim": int(weights["dimension"]),
                            "pair_channels": pair_channels}, [weights[k] for k in MSA_ATTENTION_AF3_ORDER])


class Af3MsaAttentionGpu:
    """``Af3MsaAttentionGpu`` (``webgpu/af3/trunk/msa-attention.js:501``; CPU form
    ``cpu/af3/trunk/msa.js:164-224``): ``run(msa, msaMask, pair, {sequences, tokens, msaChannels,
    pairChannels}, weights, options)`` - MSA pair-weighted averaging, float32 arithmetic."""

    def __init__(self, device: Device | None = None):
        self.device = _device(device)

    def run(self, msa, msa_mask, pair, shape, weights, options=None, out=None):
        S, n = int(shape["sequences"]), int(shape["tokens"])
        cm, cz = int(shape["msaChannels"]), int(shape["pairChannels"])
        dev = self.device
        owned = None
        if not isinstance(weights, PreparedWeights):
            if not isinstance(weights.get("heads"), (int, np.integer)) or not isinstance(weights.get("dimension"), (int, np.integer)):
                raise ValueError("weights.heads and weights.dimension must be integers")
            owned = weights = prepare_msa_attention_weights(dev, weights, cm, cz)
        try:
            a = _Buffer(msa)
            m = _Buffer(msa_mask)
            p = _Buffer(pair)
            _expect_length("msa", a, S * n * cm)
            _expect_length("msaMask", m, S * n)
            _expect_length("pair", p, n * n * cz)
            obuf, output = _out_like(a, (S, n, cm), out)
            opts = options or {}
            desc = nat.MsaAttentionDesc(S, n, cm, weights.dims["heads"], weights.dims["head_dim"], cz, _precision(opts),
                                        1 if opts.get("residual") else 0,
                                        nat.SPACE_DEVICE if a.is_device else nat.SPACE_HOST, p.dtype,
                                        a.ptr, m.ptr, p.ptr, obuf.ptr, weights.handle)
            res = nat.Result()
            dev.check(dev.lib.lf_msa_attention_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
            return _result(dev, res, output)
        finally:
            if owned is not None:
                dev.synchronize()
                owned.close()


def distogram_logits(device, pair, tokens, channels, half_logits, bias=None):
    """The logits of ``distogramHead`` (``cpu/af3/trunk/trunk.js:47-60``): ``pair . halfLogits`` plus its
    transpose over the token axes (a sum).  ``pair`` and the weights are host arrays or float32 device tensors."""
    dev = _device(device)
    p = _Buffer(pair)
    _expect_length("pair", p, tokens * tokens * channels)
    if p.is_device:
        import torch
        w = half_logits if getattr(half_logits, "is_cuda", False) else torch.as_tensor(np.asarray(half_logits, np.float32)).to(pair.device)
        b = None if bias is None else (bias if getattr(bias, "is_cuda", False) else torch.as_tensor(np.asarray(bias, np.float32)).to(pair.device))
    else:
        w, b = half_logits, bias
    wb = _Buffer(w)
    bins = wb.count // channels
    _expect_length("halfLogits", wb, channels * bins)
    bb = None if b is None else _Buffer(b)
    if p.is_device:
        output = pair.new_empty((tokens, tokens, bins), dtype=w.dtype)
        obuf = _Buffer(output)
    else:
        output = np.empty((tokens, tokens, bins), np.float32)
        obuf = _Buffer(output)
    desc = nat.DistogramDesc(tokens, channels, bins, nat.SPACE_DEVICE if p.is_device else nat.SPACE_HOST, p.dtype,
                             p.ptr, wb.ptr, None if bb is None else bb.ptr, obuf.ptr)
    res = nat.Result()
    dev.check(dev.lib.lf_distogram_logits_run(dev.handle, ctypes.byref(desc), ctypes.byref(res)))
    return _result(dev, res, output)


# ---------------------------------------------------------------------------
# int5


def int5_decode(device, payload: bytes, scale_offset: int, zero_offset: int, elements: int, block: int = 32):
    """Decode one int5 tensor payload (``shared/weights/dtype.js:330-378``) on the GPU."""
    dev = _device(device)
    raw = np.frombuffer(payload, np.uint8)
    out = np.empty(elements, np.float32)
    dev.check(dev.lib.lf_int5_decode(dev.handle, raw.ctypes.data, raw.size, scale_offset, zero_offset, elements,
                                     block, nat.SPACE_HOST, out.ctypes.data))
    return out
