"""Writes synthetic weight bundles in the reference's on-disk format.  TEST INFRASTRUCTURE ONLY.

The product reads bundles (``localfold_b200/bundle.py``); nothing in it writes them.  The tests need
bundles whose contents they know, so this module encodes named float32 arrays the way the reference's
exporter does (``tools/quantize_af3.py:60-101, 255-297``; int8: ``shared/weights/dtype.js:220-245``) and
is itself checked bit for bit against vectors produced by importing that exporter
(``tests/golden/int5-vectors.npz``).

int5: groups of 32 values over the flat index; per group zero = fp16(min), scale = fp16((max - min) / 31),
code = clip(rint((x - zero) / scale), 0, 31) with the rounded fp16 values (a zero scale divides as 1);
32 codes -> 20 bytes, least significant bit first; one slack byte; padding to 4 bytes; fp16 scales; fp16 zeros.
int8: groups of 64, symmetric, scale = fp16(max|x| / 127), code = clip(rint(x / scale), -127, 127); codes,
padding to 4 bytes, fp16 scales.
"""
from __future__ import annotations

import json
import os
import re

import numpy as np

from localfold_b200.bundle import decode_int5_host

FLOAT32_NAMES = re.compile(r"/(scale|offset|bias)$|_bias$|_weight$|/output_b$")


def _groups(values, size):
    flat = np.asarray(values, np.float32).ravel()
    count = -(-flat.size // size)
    grid = np.zeros((count, size), np.float32)
    grid.ravel()[:flat.size] = flat
    return grid


def int5_encode(values):
    """-> (codes [groups, 32] uint8, scales [groups] fp16, zeros [groups] fp16)"""
    grid = _groups(values, 32)
    lo, hi = grid.min(axis=1), grid.max(axis=1)
    zeros = lo.astype(np.float16)
    scales = ((hi - lo) / np.float32(31)).astype(np.float16)
    step = scales.astype(np.float32)
    step = np.where(step == 0, np.float32(1), step)
    codes = np.rint((grid - zeros.astype(np.float32)[:, None]) / step[:, None])
    return np.clip(codes, 0, 31).astype(np.uint8), scales, zeros


def int5_bytes(codes):
    """[groups, 32] five-bit codes -> [groups, 20] bytes; bit k of the stream is bit k % 5 of code k // 5."""
    bits = (codes[:, :, None] >> np.arange(5, dtype=np.uint8)) & 1
    return np.packbits(bits.reshape(codes.shape[0], -1), axis=1, bitorder="little")


def int5_payload(values):
    """(payload bytes, scale offset, zero offset) of one tensor."""
    codes, scales, zeros = int5_encode(values)
    body = int5_bytes(codes).tobytes() + b"\0"
    body += b"\0" * (-len(body) % 4)
    scale_offset = len(body)
    zero_offset = scale_offset + 2 * scales.size
    return body + scales.astype("<f2").tobytes() + zeros.astype("<f2").tobytes(), scale_offset, zero_offset


def packed_payload(values, bits, group):
    """Asymmetric ``bits``-bit codes at any whole-byte group (the delta bundles use int3 at 128): same scheme
    as int5 with 2^bits - 1 levels."""
    grid = _groups(values, group)
    levels = (1 << bits) - 1
    lo, hi = grid.min(axis=1), grid.max(axis=1)
    zeros = lo.astype(np.float16)
    scales = ((hi - lo) / np.float32(levels)).astype(np.float16)
    step = scales.astype(np.float32)
    step = np.where(step == 0, np.float32(1), step)
    codes = np.clip(np.rint((grid - zeros.astype(np.float32)[:, None]) / step[:, None]), 0, levels).astype(np.uint8)
    stream = (codes[:, :, None] >> np.arange(bits, dtype=np.uint8)) & 1
    body = np.packbits(stream.reshape(codes.shape[0], -1), axis=1, bitorder="little").tobytes() + b"\0"
    body += b"\0" * (-len(body) % 4)
    scale_offset = len(body)
    return body + scales.astype("<f2").tobytes() + zeros.astype("<f2").tobytes(), scale_offset, scale_offset + 2 * scales.size


def int8_payload(values):
    """(payload bytes, scale offset) of one int8 tensor, symmetric, groups of 64."""
    grid = _groups(values, 64)
    scales = (np.abs(grid).max(axis=1) / np.float32(127)).astype(np.float16)
    step = scales.astype(np.float32)
    step = np.where(step == 0, np.float32(1), step)
    codes = np.clip(np.rint(grid / step[:, None]), -127, 127).astype(np.int8)
    count = np.asarray(values).size
    body = codes.ravel()[:count].tobytes()
    body += b"\0" * (-len(body) % 4)
    return body + scales.astype("<f2").tobytes(), len(body)


def write_bundle(directory, tensors, shard_bytes=64 << 20, model="synthetic", dtypes=None, manifest_extra=None, prefix="weights"):
    """``manifest.json`` + ``weights-NN.int5.bin`` shards for a dict of named float32 arrays.  ``dtypes``
    optionally maps a name to "int5", "int8", "float16" or "float32"; by default names that the reference
    keeps in float32 stay float32 and every other tensor becomes int5."""
    os.makedirs(directory, exist_ok=True)
    dtypes = dtypes or {}
    shards, blob, records = [], bytearray(), {}
    for name, array in tensors.items():
        array = np.ascontiguousarray(array, np.float32)
        kind = dtypes.get(name) or ("float32" if FLOAT32_NAMES.search(name) else "int5")
        record = {"shape": list(array.shape), "dtype": kind}
        if kind == "float32":
            payload = array.astype("<f4").tobytes()
        elif kind == "float16":
            payload = array.astype("<f2").tobytes()
        elif kind == "int8":
            payload, scale_offset = int8_payload(array)
            record.update(block=64, scaleOffset=scale_offset)
        elif kind == "int3":
            payload, scale_offset, zero_offset = packed_payload(array, 3, 128)
            record.update(block=128, scaleOffset=scale_offset, zeroOffset=zero_offset)
        else:
            payload, scale_offset, zero_offset = int5_payload(array)
            record.update(block=32, scaleOffset=scale_offset, zeroOffset=zero_offset)
        start = len(blob) + (-len(blob) % 4)
        if blob and start + len(payload) > shard_bytes:
            shards.append(bytes(blob))
            blob, start = bytearray(), 0
        blob.extend(b"\0" * (start - len(blob)))
        record["file"] = f"{prefix}-{len(shards):02d}.int5.bin"
        record["byteOffset"] = start
        for key in ("scaleOffset", "zeroOffset"):
            if key in record:
                record[key] += start
        blob.extend(payload)
        records[name] = record
    shards.append(bytes(blob))
    for index, data in enumerate(shards):
        with open(os.path.join(directory, f"{prefix}-{index:02d}.int5.bin"), "wb") as f:
            f.write(data)
    manifest = {"formatVersion": 1, "model": model, "tensors": records,
                "quantisation": {"scheme": "asymmetric-per-group", "bits": 5, "group": 32,
                                 "scaleDtype": "float16", "zeroDtype": "float16"},
                "bundle": {"bytes": sum(map(len, shards)), "tensorCount": len(records)}}
    manifest.update(manifest_extra or {})
    path = os.path.join(directory, "manifest.json" if prefix == "weights" else f"{prefix}-manifest.json")
    with open(path, "w") as f:
        json.dump(manifest, f)
    return path


def quantise_weights_like_bundle(weights):
    """Every linear weight of a (nested) weight object after a round trip through the int5 format; norm
    scales / offsets and biases (one-dimensional) are left alone, as the exporter leaves them float32."""
    out = {}
    for key, value in weights.items():
        if isinstance(value, dict):
            out[key] = quantise_weights_like_bundle(value)
        elif isinstance(value, np.ndarray) and value.ndim >= 2:
            payload, scale_offset, zero_offset = int5_payload(value)
            out[key] = decode_int5_host(payload, scale_offset, zero_offset, value.size).reshape(value.shape)
        else:
            out[key] = value
    return out
