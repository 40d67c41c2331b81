"""Regenerates the golden vectors in this directory from a checkout of the reference.

    python tests/golden/make_golden.py /path/to/localfold

1. The four triangle-multiplication (outgoing) fixtures the reference ships under
   ``test/fixtures/`` (an OpenFold run at N=5 and three official-AlphaFold
   captures at N=9/59/59: ``test/cpu-reference.test.js:20-29``,
   ``test/alphafold-references.js:1-5``) are repacked, one ``.npz`` each, with
   float32 payloads unchanged.
2. int5 vectors: seeded values pushed through the reference's own quantiser
   (``tools/quantize_af3.py`` ``quantise`` + ``pack``, imported from the checkout)
   and decoded with the rule of ``shared/weights/dtype.js:330-378``
   (code*scale + zero in float64, stored float32).
"""
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURES = {
    "openfold-triangle-small": "test/fixtures/openfold-triangle-small",
    "alphafold-short-9": "test/fixtures/alphafold-single-sequence/short-9",
    "alphafold-single-59": "test/fixtures/alphafold-single-sequence/model1-reference-59",
    "alphafold-a3m-59": "test/fixtures/alphafold-a3m/model1-reference-59",
}


def pack_triangle(root, name, rel):
    d = os.path.join(root, rel)
    manifest = json.load(open(os.path.join(d, "manifest.json")))
    assert manifest["formatVersion"] == 1 and manifest["operator"] == "TriangleMultiplicationOutgoing"
    out = {}
    for tensor, record in manifest["tensors"].items():
        assert record["dtype"] == "float32"
        a = np.fromfile(os.path.join(d, record["file"]), dtype="<f4")
        out[tensor] = a.reshape(record["shape"])
    shape = manifest["shape"]
    out["shape"] = np.array([shape["length"], shape["cZ"], shape["cHidden"]], np.int64)
    out["epsilon"] = np.array(manifest.get("epsilon", 1e-5), np.float64)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(name, shape, manifest.get("source"))


def make_int5(root):
    spec = importlib.util.spec_from_file_location("quantize_af3", os.path.join(root, "tools/quantize_af3.py"))
    q = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(q)
    rng = np.random.default_rng(55)
    out = {}
    for i, n in enumerate((1, 7, 32, 33, 100, 1024, 4096 + 13)):
        values = (rng.standard_normal(n) * rng.uniform(0.01, 2.0)).astype(np.float32)
        if i == 2:
            values[:] = 0.25          # a constant group: scale 0
        codes, scales, zeros = q.quantise(values)
        packed = q.pack(codes)
        decoded = (codes.astype(np.float64) * scales.astype(np.float64)[:, None]
                   + zeros.astype(np.float64)[:, None]).astype(np.float32).reshape(-1)[:n]
        out[f"values_{i}"] = values
        out[f"packed_{i}"] = packed.reshape(-1)
        out[f"scales_{i}"] = scales
        out[f"zeros_{i}"] = zeros
        out[f"decoded_{i}"] = decoded
    np.savez_compressed(os.path.join(HERE, "int5-vectors.npz"), **out)
    print("int5 vectors", len(out) // 5)


if __name__ == "__main__":
    root = sys.argv[1]
    for name, rel in FIXTURES.items():
        pack_triangle(root, name, rel)
    make_int5(root)
