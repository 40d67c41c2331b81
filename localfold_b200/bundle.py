"""Weight bundles in the reference's on-disk format: reading, and the mapping from bundle tensors to the
weight objects the operators take.

Format (``tools/quantize_af3.py:60-101,255-297``, ``shared/weights/dtype.js:212-406``): ``manifest.json``
holds per tensor a record ``{file, shape, dtype, byteOffset[, block, scaleOffset, zeroOffset]}``; the
payloads sit in shard files, each tensor 4-byte aligned.  Encodings:

* ``float32``, ``float16``: plain little-endian arrays;
* ``int8``: symmetric, groups of ``block`` (64) values over the flat index, one fp16 scale per group at
  ``scaleOffset``; value = code * scale (``dtype.js:220-245``);
* ``intN`` for N = 1..7 (``int5`` at group 32 is what the AF3 export writes): asymmetric, groups of ``block``
  codes packed least-significant-bit first into ``block * N / 8`` bytes, one slack byte, then fp16 scales at
  ``scaleOffset`` and fp16 zero points at ``zeroOffset``; value = code * scale + zero (``dtype.js:253-295,330-378``).

Every value is the float64 product (and sum) stored as float32, as the reference computes it.  Groups run
over the flat row-major index of the stored tensor, so a range of a tensor decodes to exactly what the whole
tensor holds there; stacked tensors ``[blocks, ...]`` are read one block at a time that way
(``readTensorRange``).  Offsets in a record are absolute within its shard file.

``FileTensorStore`` reads a bundle (int5 ranges that start on a group boundary are decoded on the GPU when a
device is given, everything else with numpy); ``DeltaTensorStore`` reads a model stored as a difference
against another (``shared/bundles/delta-tensor-store.js``).  ``AlphaFoldFixture`` and
``pairformer_block_weights`` turn a store into the weight objects of the AF2 Evoformer blocks
(``shared/bundles/alphafold-fixture.js:122-267``) and of the AF3 pairformer blocks
(``shared/af3/weights/weights.js:402-454,699-727``).
"""
from __future__ import annotations

import json
import os
import re

import numpy as np

GROUP = 32
BITS = 5

# where the AF3 exporters put the trunk's stacks (``shared/af3/weights/weights.js:14-26``)
EVO = "diffuser/evoformer"
PAIRFORMER = f"{EVO}/__layer_stack_no_per_layer_1/trunk_pairformer"
MSA_STACK = f"{EVO}/__layer_stack_no_per_layer/msa_stack"


def _packed_bits(dtype):
    m = re.fullmatch(r"int([1-9])", dtype)
    if m is None:
        return None
    bits = int(m.group(1))
    return bits if bits < 8 else None


def decode_packed_host(raw, bits, block, groups_first, groups_count, scales, zeros):
    """``groups_count`` whole groups of ``bits``-bit codes starting at group ``groups_first`` of the byte
    array ``raw`` (the tensor's code bytes from its first group on) -> float32 values."""
    group_bytes = block * bits // 8
    if block * bits % 8:
        raise ValueError(f"int{bits} at group {block} does not pack into whole bytes")
    body = np.frombuffer(raw, np.uint8, groups_count * group_bytes, groups_first * group_bytes)
    stream = np.unpackbits(body.reshape(groups_count, group_bytes), axis=1, bitorder="little")
    codes = stream.reshape(groups_count, block, bits)
    weights = (1 << np.arange(bits)).astype(np.int64)
    values = (codes.astype(np.int64) * weights).sum(axis=2).astype(np.float64)
    out = values * scales.astype(np.float64)[:, None] + zeros.astype(np.float64)[:, None]
    return out.astype(np.float32).reshape(-1)


def decode_int5_host(payload: bytes, scale_offset: int, zero_offset: int, elements: int, block: int = GROUP):
    """One whole int5 tensor payload (codes, slack byte, padding, scales, zeros) -> float32."""
    groups = (elements + block - 1) // block
    scales = np.frombuffer(payload, "<f2", groups, scale_offset)
    zeros = np.frombuffer(payload, "<f2", groups, zero_offset)
    return decode_packed_host(payload, BITS, block, 0, groups, scales, zeros)[:elements]


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

    def has(self, name):
        return name in self.manifest["tensors"]

    def record(self, name):
        record = self.manifest["tensors"].get(name)
        if record is None:
            raise KeyError(f"missing tensor {name}")
        return record

    def shape(self, name):
        return list(self.record(name)["shape"])

    def _bytes(self, name):
        if name not in self._files:
            with open(os.path.join(self.directory, name), "rb") as f:
                self._files[name] = f.read()
        return self._files[name]

    def tensor(self, name):
        record = self.record(name)
        count = int(np.prod(record["shape"])) if record["shape"] else 1
        return self.tensor_range(name, 0, count).reshape(record["shape"])

    read = tensor

    def tensor_as_float16(self, name):
        return self.tensor(name).astype(np.float16)

    def tensor_range(self, name, first, count):
        """Elements ``first .. first + count`` of the flat tensor, decoded without the rest
        (``readTensorRange``: ``shared/weights/dtype.js:212-406``)."""
        record = self.record(name)
        elements = int(np.prod(record["shape"])) if record["shape"] else 1
        if first < 0 or count < 0 or first + count > elements:
            raise ValueError(f"range {first}:{count} lies outside a tensor of {elements}")
        blob = self._bytes(record["file"])
        start = record.get("byteOffset", 0)
        dtype = record["dtype"]
        if dtype == "float32":
            return np.frombuffer(blob, "<f4", count, start + 4 * first).copy()
        if dtype == "float16":
            return np.frombuffer(blob, "<f2", count, start + 2 * first).astype(np.float32)
        block = record.get("block")
        if not isinstance(block, int) or block <= 0:
            raise ValueError(f"{dtype} tensor {name} has no block size")
        groups = (elements + block - 1) // block
        g0 = first // block
        g1 = min(groups, (first + count + block - 1) // block)
        scales = np.frombuffer(blob, "<f2", g1 - g0, record["scaleOffset"] + 2 * g0)
        lo = first - g0 * block
        if dtype == "int8":
            begin = g0 * block
            end = min(elements, g1 * block)
            codes = np.frombuffer(blob, np.int8, end - begin, start + begin).astype(np.float64)
            scale = np.repeat(scales.astype(np.float64), block)[:end - begin]
            return (codes * scale).astype(np.float32)[lo:lo + count]
        bits = _packed_bits(dtype)
        if bits is None:
            raise ValueError(f"unsupported tensor dtype {dtype}")
        if "zeroOffset" not in record:
            raise ValueError(f"{dtype} tensor {name} has no zero offset; it is asymmetric")
        zeros = np.frombuffer(blob, "<f2", g1 - g0, record["zeroOffset"] + 2 * g0)
        if bits == 5 and self.device is not None and lo == 0 and (count % block == 0 or first + count == elements):
            return self._int5_on_device(blob, record, start, g0, g1, count, block)
        raw = memoryview(blob)[start:]
        return decode_packed_host(raw, bits, block, g0, g1 - g0, scales, zeros)[lo:lo + count]

    def tensor_source(self, name, first, count, shape=None):
        """The stored bytes of a range, for decoding on the device: an ``EncodedTensor`` when the tensor is int5
        and the range starts on a group boundary (and ends on one, or at the tensor's end); otherwise the decoded
        float32 values (``tensorSource`` of the reference's stores: ``shared/bundles/alphafold-fixture.js:75-100``)."""
        from .operators import EncodedTensor
        record = self.record(name)
        elements = int(np.prod(record["shape"])) if record["shape"] else 1
        block = record.get("block")
        shape = (count,) if shape is None else shape
        if record["dtype"] != "int5" or first % block or not (count % block == 0 or first + count == elements):
            return self.tensor_range(name, first, count).reshape(shape)
        blob = self._bytes(record["file"])
        start = record.get("byteOffset", 0)
        g0, g1 = first // block, (first + count + block - 1) // block
        group_bytes = block * BITS // 8
        codes = blob[start + g0 * group_bytes:start + g1 * group_bytes] + b"\0"
        codes += b"\0" * (-len(codes) % 4)
        scales = blob[record["scaleOffset"] + 2 * g0:record["scaleOffset"] + 2 * g1]
        zeros = blob[record["zeroOffset"] + 2 * g0:record["zeroOffset"] + 2 * g1]
        return EncodedTensor(codes + scales + zeros, len(codes), len(codes) + len(scales), count, shape, block)

    def _int5_on_device(self, blob, record, start, g0, g1, count, block):
        """A group-aligned range through ``lf_int5_decode``: the codes of groups g0..g1 with their scales and
        zeros, laid out as a payload of their own."""
        from .operators import int5_decode
        group_bytes = block * BITS // 8
        codes = blob[start + g0 * group_bytes:start + g1 * group_bytes] + b"\0"
        codes += b"\0" * (-len(codes) % 4)
        scales = blob[record["scaleOffset"] + 2 * g0:record["scaleOffset"] + 2 * g1]
        zeros = blob[record["zeroOffset"] + 2 * g0:record["zeroOffset"] + 2 * g1]
        payload = codes + scales + zeros
        return int5_decode(self.device, payload, len(codes), len(codes) + len(scales), count, block)


class DeltaTensorStore:
    """A model stored as a difference against another, read as though it were whole
    (``shared/bundles/delta-tensor-store.js``).  The delta bundle's ``delta`` header lists the tensors to
    ADD to the base's value (``addTo``; the base rounded to fp16 first, because that is what the difference
    was taken against), to take whole from the delta (``whole``) and the base's tensors this model does not
    have (``absent``); everything else is the base's."""

    def __init__(self, base, delta):
        header = delta.manifest.get("delta")
        if header is None:
            raise ValueError("this bundle carries no `delta` header - it is not a delta")
        self.base, self.delta = base, delta
        self.add_to, self.whole, self.absent = (set(header.get(k, ())) for k in ("addTo", "whole", "absent"))
        tensors = {n: r for n, r in base.manifest["tensors"].items() if n not in self.absent}
        self.manifest = dict(base.manifest, tensors=tensors, delta=header)
        for section in ("templateEmbedding", "templateSingle"):
            parameters = (base.manifest.get(section) or {}).get("parameters")
            if parameters is None:
                continue
            names = [name for leaves in parameters.values() for name in leaves.values()]
            if any(n in self.absent for n in names):
                if not all(n in self.absent for n in names):
                    raise ValueError(f"{section} is only partly absent from this delta")
                self.manifest.pop(section, None)

    def names(self):
        return list(self.manifest["tensors"])

    def has(self, name):
        return name in self.manifest["tensors"]

    def shape(self, name):
        if name in self.absent:
            raise KeyError(f"missing tensor {name}")
        return self.base.shape(name)

    def _from(self, name):
        if name in self.absent:
            raise KeyError(f"missing tensor {name}")
        return self.delta if (name in self.whole or name in self.add_to) else self.base

    def tensor_range(self, name, first, count):
        if name not in self.add_to:
            return self._from(name).tensor_range(name, first, count)
        held = self.base.tensor_range(name, first, count).astype(np.float16).astype(np.float32)
        return held + self.delta.tensor_range(name, first, count)

    def tensor(self, name):
        shape = self.shape(name)
        count = int(np.prod(shape)) if shape else 1
        return self.tensor_range(name, 0, count).reshape(shape)

    def tensor_as_float16(self, name):
        return self.tensor(name).astype(np.float16)


# ---------------------------------------------------------------------------
# bundle tensors -> weight objects


def stacked(store, name, index, encoded=False):
    """Block ``index`` of a tensor stacked along its first axis, shaped as one block
    (``stacked``: ``shared/af3/weights/weights.js:154-184``).  ``encoded``: hand over the stored bytes
    (``EncodedTensor``) where the store can, for decoding on the device."""
    shape = store.shape(name)
    if index >= shape[0]:
        raise IndexError(f"{name} has {shape[0]} blocks; asked for {index}")
    stride = int(np.prod(shape[1:])) if len(shape) > 1 else 1
    if encoded and hasattr(store, "tensor_source"):
        return store.tensor_source(name, index * stride, stride, tuple(shape[1:]))
    return store.tensor_range(name, index * stride, stride).reshape(shape[1:])


class AlphaFoldFixture:
    """AF2 bundles: ``manifest.evoformerStack = {parameters: {module: {leaf: tensor name}}, blocks}`` with
    every tensor stacked ``[blocks, ...]`` (``shared/bundles/alphafold-fixture.js``).  Haiku stores every
    linear ``[in][out]``; the triangle operator takes ``[out][in]``, so its six projections are transposed here
    (``alphafold-fixture.js:181-191``); attention, transition and outer-product weights keep their layout."""

    def __init__(self, store):
        self.store = store
        self.manifest = store.manifest

    def _leaf(self, parameters, module, leaf, block, blocks):
        name = (parameters.get(module) or {}).get(leaf)
        if name is None:
            raise KeyError(f"missing {module}/{leaf}")
        shape = self.store.shape(name)
        if block is None:
            return self.store.tensor(name), shape
        if shape[0] != blocks:
            raise ValueError(f"{name} is stacked {shape[0]} deep; the manifest says {blocks} blocks")
        return stacked(self.store, name, block), shape[1:]

    def _gather(self, parameters, block, blocks, entries, transposed=()):
        out = {}
        for prop, module, leaf in entries:
            value, _ = self._leaf(parameters, module, leaf, block, blocks)
            if prop in transposed:
                rows, columns = transposed[prop]
                value = np.ascontiguousarray(value.reshape(rows, columns).T)
            out[prop] = np.ascontiguousarray(value, np.float32)
        return out

    def _attention(self, parameters, root, block, blocks):
        att = f"{root}/attention"
        weights = self._gather(parameters, block, blocks, [
            ("queryNormScale", f"{root}/query_norm", "scale"), ("queryNormOffset", f"{root}/query_norm", "offset"),
            ("queryWeight", att, "query_w"), ("keyWeight", att, "key_w"), ("valueWeight", att, "value_w"),
            ("gatingWeight", att, "gating_w"), ("gatingBias", att, "gating_b"), ("outputWeight", att, "output_w"),
            ("outputBias", att, "output_b")])
        _, gate_shape = self._leaf(parameters, att, "gating_b", block, blocks)
        return {"heads": int(gate_shape[0]), "attention": weights}

    def _triangle_attention(self, parameters, root, block, blocks):
        result = self._attention(parameters, root, block, blocks)
        result["pairBias"] = self._gather(parameters, block, blocks, [("projectionWeight", root, "feat_2d_weights")])
        return result

    def _transition(self, parameters, root, block, blocks):
        return self._gather(parameters, block, blocks, [
            ("layerNormScale", f"{root}/input_layer_norm", "scale"), ("layerNormOffset", f"{root}/input_layer_norm", "offset"),
            ("firstWeight", f"{root}/transition1", "weights"), ("firstBias", f"{root}/transition1", "bias"),
            ("secondWeight", f"{root}/transition2", "weights"), ("secondBias", f"{root}/transition2", "bias")])

    def _triangle(self, parameters, root, channels, block, blocks):
        _, bias_shape = self._leaf(parameters, f"{root}/left_projection", "bias", block, blocks)
        hidden = int(bias_shape[0])
        shapes = {"linearAPWeight": (channels, hidden), "linearAGWeight": (channels, hidden),
                  "linearBPWeight": (channels, hidden), "linearBGWeight": (channels, hidden),
                  "linearZWeight": (hidden, channels), "linearGWeight": (channels, channels)}
        return self._gather(parameters, block, blocks, [
            ("layerNormInWeight", f"{root}/layer_norm_input", "scale"), ("layerNormInBias", f"{root}/layer_norm_input", "offset"),
            ("linearAPWeight", f"{root}/left_projection", "weights"), ("linearAPBias", f"{root}/left_projection", "bias"),
            ("linearAGWeight", f"{root}/left_gate", "weights"), ("linearAGBias", f"{root}/left_gate", "bias"),
            ("linearBPWeight", f"{root}/right_projection", "weights"), ("linearBPBias", f"{root}/right_projection", "bias"),
            ("linearBGWeight", f"{root}/right_gate", "weights"), ("linearBGBias", f"{root}/right_gate", "bias"),
            ("layerNormOutWeight", f"{root}/center_layer_norm", "scale"), ("layerNormOutBias", f"{root}/center_layer_norm", "offset"),
            ("linearZWeight", f"{root}/output_projection", "weights"), ("linearZBias", f"{root}/output_projection", "bias"),
            ("linearGWeight", f"{root}/gating_linear", "weights"), ("linearGBias", f"{root}/gating_linear", "bias")], shapes)

    def _outer_product_mean(self, parameters, block, blocks):
        opm = "outer_product_mean"
        return self._gather(parameters, block, blocks, [
            ("layerNormScale", f"{opm}/layer_norm_input", "scale"), ("layerNormOffset", f"{opm}/layer_norm_input", "offset"),
            ("leftWeight", f"{opm}/left_projection", "weights"), ("leftBias", f"{opm}/left_projection", "bias"),
            ("rightWeight", f"{opm}/right_projection", "weights"), ("rightBias", f"{opm}/right_projection", "bias"),
            ("outputWeight", opm, "output_w"), ("outputBias", opm, "output_b")])

    def pair_block_weights(self, parameters, block, blocks, pair_channels=128):
        """The five pair updates of one block (also what the extra-MSA and template pair stacks hold)."""
        return {
            "triangleMultiplicationOutgoing": self._triangle(parameters, "triangle_multiplication_outgoing", pair_channels, block, blocks),
            "triangleMultiplicationIncoming": self._triangle(parameters, "triangle_multiplication_incoming", pair_channels, block, blocks),
            "triangleAttentionStarting": self._triangle_attention(parameters, "triangle_attention_starting_node", block, blocks),
            "triangleAttentionEnding": self._triangle_attention(parameters, "triangle_attention_ending_node", block, blocks),
            "pairTransition": self._transition(parameters, "pair_transition", block, blocks),
        }

    def main_stack_weights(self, pair_channels=128):
        """``mainStackWeights`` (``alphafold-fixture.js:229-267``): one weight object per Evoformer block."""
        section = self.manifest["evoformerStack"]
        parameters, blocks = section["parameters"], int(section["blocks"])
        result = []
        for block in range(blocks):
            row = self._attention(parameters, "msa_row_attention_with_pair_bias", block, blocks)
            row["pairBias"] = self._gather(parameters, block, blocks, [
                ("layerNormScale", "msa_row_attention_with_pair_bias/feat_2d_norm", "scale"),
                ("layerNormOffset", "msa_row_attention_with_pair_bias/feat_2d_norm", "offset"),
                ("projectionWeight", "msa_row_attention_with_pair_bias", "feat_2d_weights")])
            w = {"msaRowAttention": row,
                 "msaColumnAttention": self._attention(parameters, "msa_column_attention", block, blocks),
                 "msaTransition": self._transition(parameters, "msa_transition", block, blocks),
                 "outerProductMean": self._outer_product_mean(parameters, block, blocks)}
            w.update(self.pair_block_weights(parameters, block, blocks, pair_channels))
            result.append(w)
        return result


def pair_track(store, root, index, encoded=False):
    """The five pair-track modules of block ``index`` of an AF3-lineage stack (``pairTrack``:
    ``shared/af3/weights/weights.js:402-454``).  Heads and head dimension of the grid attention come from its
    own ``q_projection/weights`` ``[blocks, heads, dimension, channels]``; a block without
    ``pair_attention1`` (a PairMixer block) has no grid attention fields."""
    at = lambda leaf: stacked(store, f"{root}/{leaf}", index, encoded)
    has = lambda leaf: store.has(f"{root}/{leaf}")
    out = {}
    for direction in ("outgoing", "incoming"):
        t = f"triangle_multiplication_{direction}"
        out["triangleMultiplication" + direction.capitalize()] = {
            "leftNormInputScale": at(f"{t}/left_norm_input/scale"), "leftNormInputOffset": at(f"{t}/left_norm_input/offset"),
            "projection": at(f"{t}/projection/weights"), "gate": at(f"{t}/gate/weights"),
            "centerNormScale": at(f"{t}/center_norm/scale"), "centerNormOffset": at(f"{t}/center_norm/offset"),
            "outputProjection": at(f"{t}/output_projection/weights"), "gatingLinear": at(f"{t}/gating_linear/weights")}
    if has("pair_attention1/q_projection/weights"):
        _, heads, dimension = store.shape(f"{root}/pair_attention1/q_projection/weights")[:3]
        for which in (1, 2):
            a = f"pair_attention{which}"
            grid = {"heads": int(heads), "dimension": int(dimension),
                    "actNormScale": at(f"{a}/act_norm/scale"), "actNormOffset": at(f"{a}/act_norm/offset"),
                    "pairBiasProjection": at(f"{a}/pair_bias_projection/weights"),
                    "qProjection": at(f"{a}/q_projection/weights"), "kProjection": at(f"{a}/k_projection/weights"),
                    "vProjection": at(f"{a}/v_projection/weights"), "gatingQuery": at(f"{a}/gating_query/weights"),
                    "outputProjection": at(f"{a}/output_projection/weights"),
                    "gatingQueryBias": at(f"{a}/gating_query/bias") if has(f"{a}/gating_query/bias") else None,
                    "outputProjectionBias": at(f"{a}/output_projection/bias") if has(f"{a}/output_projection/bias") else None}
            out[f"pairAttention{which}"] = grid
    p = "pair_transition"
    out["pairTransition"] = {"inputLayerNormScale": at(f"{p}/input_layer_norm/scale"),
                             "inputLayerNormOffset": at(f"{p}/input_layer_norm/offset"),
                             "transition1": at(f"{p}/transition1/weights"), "transition2": at(f"{p}/transition2/weights")}
    return out


def pairformer_block_weights(store, index, root=PAIRFORMER, encoded=False):
    """``pairformerBlockWeights`` (``shared/af3/weights/weights.js:699-727``): block ``index`` of a pairformer
    stack.  The four widths come from the tensors: ``single_attention_q_projection/weights`` is
    ``[blocks, singleChannels, heads, dimension]`` and ``single_pair_logits_norm/scale`` ``[blocks, pairChannels]``."""
    at = lambda leaf: stacked(store, f"{root}/{leaf}", index, encoded)
    _, single_channels, heads, dimension = store.shape(f"{root}/single_attention_q_projection/weights")
    _, pair_channels = store.shape(f"{root}/single_pair_logits_norm/scale")
    out = {"pairChannels": int(pair_channels), "singleChannels": int(single_channels)}
    out.update(pair_track(store, root, index, encoded))
    out.update({
        "singlePairLogitsNormScale": at("single_pair_logits_norm/scale"),
        "singlePairLogitsNormOffset": at("single_pair_logits_norm/offset"),
        "singlePairLogitsProjection": at("single_pair_logits_projection/weights"),
        "singleAttention": {
            "heads": int(heads), "dimension": int(dimension),
            "layerNormScale": at("single_attention_layer_norm/scale"), "layerNormOffset": at("single_attention_layer_norm/offset"),
            "qProjection": at("single_attention_q_projection/weights"), "qBias": at("single_attention_q_projection/bias"),
            "kProjection": at("single_attention_k_projection/weights"), "vProjection": at("single_attention_v_projection/weights"),
            "gatingQuery": at("single_attention_gating_query/weights"),
            "outputProjection": at("single_attention_transition2/weights")},
        "singleTransition": {
            "inputLayerNormScale": at("single_transition/input_layer_norm/scale"),
            "inputLayerNormOffset": at("single_transition/input_layer_norm/offset"),
            "transition1": at("single_transition/transition1/weights"), "transition2": at("single_transition/transition2/weights")},
    })
    return out


def pairformer_stack_weights(store, root=PAIRFORMER, encoded=False):
    """Every block of a pairformer stack (block count from the stacked leading axis).  ``encoded``: int5 tensors
    stay encoded (``EncodedTensor``) and are decoded on the device when the operators prepare their weights
    (the reference's on-device decode: ``webgpu/weights/quantised-upload.js:100-120``)."""
    blocks = store.shape(f"{root}/single_pair_logits_norm/scale")[0]
    return [pairformer_block_weights(store, b, root, encoded) for b in range(blocks)]
