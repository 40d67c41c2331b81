"""int5 weight bundles in the reference's on-disk format: manifest + shard files.

Format (``tools/quantize_af3.py:60-101,255-297``, ``shared/weights/dtype.js:330-378``): per tensor a
manifest record ``{file, shape, dtype, byteOffset[, block, scaleOffset, zeroOffset]}``.  An ``int5``
payload is ceil(n/32) groups of 20 bytes (32 five-bit codes, least significant bit first in a
little-endian bit stream), one slack byte, zero padding to 4 bytes, then one fp16 scale and one fp16
zero point per group; a value is ``code * scale + zero``.  Groups run over the flat row-major index of
the stored tensor.  Tensors whose names match ``/(scale|offset|bias)$|_bias$|_weight$|/output_b$`` stay
float32 (``quantize_af3.py:57``).  Every tensor starts 4-byte aligned inside its shard.

``write_bundle`` produces such a bundle from named float32 arrays (for synthetic weights);
``FileTensorStore`` reads one back, decoding int5 either on the GPU (``lf_int5_decode``) or, without a
device, with numpy (same arithmetic: float64 product, float32 store).
"""
from __future__ import annotations

import json
import os
import re

import numpy as np

GROUP = 32
BITS = 5
KEEP_FLOAT32 = re.compile(r"/(scale|offset|bias)$|_bias$|_weight$|/output_b$")


def quantise_int5(values, group=GROUP):
    """Asymmetric per-group codes with fp16 scale and zero point, rounded to fp16 before the codes are chosen."""
    values = np.asarray(values, np.float32).reshape(-1)
    levels = 2 ** BITS - 1
    padded = (-len(values)) % group
    grid = np.concatenate([values, np.zeros(padded, np.float32)]).reshape(-1, group)
    low = grid.min(1, keepdims=True).astype(np.float32)
    high = grid.max(1, keepdims=True).astype(np.float32)
    zeros = low.astype(np.float16)
    scales = ((high - low) / levels).astype(np.float16)
    safe = scales.astype(np.float32)
    safe[safe == 0] = 1.0
    codes = np.clip(np.rint((grid - zeros.astype(np.float32)) / safe), 0, levels).astype(np.uint8)
    return codes, scales.reshape(-1), zeros.reshape(-1)


def pack_int5(codes):
    """[groups, 32] codes -> [groups, 20] bytes, least significant bit first."""
    groups, group = codes.shape
    if (group * BITS) % 8:
        raise ValueError(f"group {group} of {BITS} bits does not pack into whole bytes")
    bits = np.unpackbits(codes[:, :, None], axis=2, count=BITS, bitorder="little")
    return np.packbits(bits.reshape(groups, group * BITS), axis=1, bitorder="little").astype(np.uint8)


def int5_payload(values):
    """Payload bytes of one tensor plus its (scaleOffset, zeroOffset) inside the payload."""
    codes, scales, zeros = quantise_int5(values)
    packed = pack_int5(codes).tobytes() + b"\x00"
    pad = (-len(packed)) % 4
    scale_offset = len(packed) + pad
    zero_offset = scale_offset + scales.nbytes
    payload = packed + b"\x00" * pad + scales.astype("<f2").tobytes() + zeros.astype("<f2").tobytes()
    return payload, scale_offset, zero_offset


def decode_int5_host(payload: bytes, scale_offset: int, zero_offset: int, elements: int, block: int = GROUP):
    raw = np.frombuffer(payload, np.uint8)
    groups = (elements + block - 1) // block
    group_bytes = block * BITS // 8
    bits = np.unpackbits(raw[:groups * group_bytes].reshape(groups, group_bytes), axis=1, bitorder="little")
    codes = np.packbits(bits.reshape(groups, block, BITS), axis=2, bitorder="little").reshape(groups, block)
    scales = np.frombuffer(payload, "<f2", groups, scale_offset).astype(np.float64)
    zeros = np.frombuffer(payload, "<f2", groups, zero_offset).astype(np.float64)
    out = codes.astype(np.float64) * scales[:, None] + zeros[:, None]
    return out.astype(np.float32).reshape(-1)[:elements]


def write_bundle(directory, tensors, shard_bytes=64 << 20, model="synthetic"):
    """Write ``manifest.json`` and ``weights-NN.int5.bin`` shards for a dict of named float32 arrays."""
    os.makedirs(directory, exist_ok=True)
    records, shards, cursor, current = {}, [], 0, []
    for name, array in tensors.items():
        array = np.ascontiguousarray(array, np.float32)
        record = {"shape": list(array.shape)}
        if KEEP_FLOAT32.search(name):
            payload = array.astype("<f4").tobytes()
            record["dtype"] = "float32"
        else:
            payload, scale_offset, zero_offset = int5_payload(array)
            record.update(dtype="int5", block=GROUP, scaleOffset=scale_offset, zeroOffset=zero_offset)
        pad = (-cursor) % 4
        if cursor + pad + len(payload) > shard_bytes and current:
            shards.append(b"".join(current))
            current, cursor, pad = [], 0, 0
        if pad:
            current.append(b"\x00" * pad)
            cursor += pad
        record["file"] = f"weights-{len(shards):02d}.int5.bin"
        record["byteOffset"] = cursor
        if record["dtype"] == "int5":
            record["scaleOffset"] += cursor
            record["zeroOffset"] += cursor
        current.append(payload)
        cursor += len(payload)
        records[name] = record
    shards.append(b"".join(current))
    for index, blob in enumerate(shards):
        with open(os.path.join(directory, f"weights-{index:02d}.int5.bin"), "wb") as f:
            f.write(blob)
    manifest = {"formatVersion": 1, "model": model, "tensors": records,
                "quantisation": {"scheme": "asymmetric-per-group", "bits": BITS, "group": GROUP,
                                 "scaleDtype": "float16", "zeroDtype": "float16"},
                "bundle": {"bytes": sum(len(b) for b in shards), "tensorCount": len(records)}}
    path = os.path.join(directory, "manifest.json")
    with open(path, "w") as f:
        json.dump(manifest, f)
    return path


class FileTensorStore:
    """Reads tensors of a bundle (``FileTensorStore``: ``shared/bundles/tensor-store.js:5``)."""

    def __init__(self, manifest_path, device=None):
        with open(manifest_path) as f:
            self.manifest = json.load(f)
        self.directory = os.path.dirname(manifest_path)
        self.device = device
        self._files = {}

    def names(self):
        return list(self.manifest["tensors"])

    def _bytes(self, name):
        if name not in self._files:
            with open(os.path.join(self.directory, name), "rb") as f:
                self._files[name] = f.read()
        return self._files[name]

    def read(self, name):
        record = self.manifest["tensors"].get(name)
        if record is None:
            raise KeyError(f"missing tensor {name}")
        blob = self._bytes(record["file"])
        count = int(np.prod(record["shape"])) if record["shape"] else 1
        start = record["byteOffset"]
        if record["dtype"] == "float32":
            return np.frombuffer(blob, "<f4", count, start).reshape(record["shape"]).copy()
        if record["dtype"] != "int5":
            raise ValueError(f"unsupported tensor dtype {record['dtype']}")
        groups = (count + record["block"] - 1) // record["block"]
        end = record["zeroOffset"] + groups * 2
        payload = blob[start:end]
        scale_offset, zero_offset = record["scaleOffset"] - start, record["zeroOffset"] - start
        if self.device is not None:
            from .operators import int5_decode
            flat = int5_decode(self.device, payload, scale_offset, zero_offset, count, record["block"])
        else:
            flat = decode_int5_host(payload, scale_offset, zero_offset, count, record["block"])
        return flat.reshape(record["shape"])


def quantise_weights_like_bundle(weights):
    """Round-trip every linear weight of a (nested) weight object through the int5 format, leaving the
    float32-kept names (norm scales/offsets, biases) alone: what a model loaded from an int5 bundle computes with."""
    out = {}
    for key, value in weights.items():
        if isinstance(value, dict):
            out[key] = quantise_weights_like_bundle(value)
        elif isinstance(value, np.ndarray) and value.ndim >= 2:
            payload, so, zo = int5_payload(value)
            out[key] = decode_int5_host(payload, so, zo, value.size).reshape(value.shape)
        else:
            out[key] = value
    return out
