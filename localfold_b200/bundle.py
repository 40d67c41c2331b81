"""int5 weight bundles in the reference's on-disk format: manifest + shard files.

Format (``tools/quantize_af3.py:60-101,255-297``, ``shared/weights/dtype.js:330-378``): per tensor a
manifest record ``{file, shape, dtype, byteOffset[, block, scaleOffset, zeroOffset]}``.  An ``int5``
payload is ceil(n/32) groups of 20 bytes (32 five-bit codes, least significant bit first in a
little-endian bit stream), one slack byte, zero padding to 4 bytes, then one fp16 scale and one fp16
zero point per group; a value is ``code * scale + zero``.  Groups run over the flat row-major index of
the stored tensor.  Tensors whose names match ``/(scale|offset|bias)$|_bias$|_weight$|/output_b$`` stay
float32 (``quantize_af3.py:57``).  Every tensor starts 4-byte aligned inside its shard.

``FileTensorStore`` reads a bundle, decoding int5 either on the GPU (``lf_int5_decode``) or, without a
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
