"""Pins the CPU oracle to every golden vector the reference ships for this path.

Bounds are the reference's own: ``test/cpu-reference.test.js:20-29`` (OpenFold
fixture: mean abs < 1e-7, max abs < 1e-6) and
``test/triangle-multiplication-outgoing.gpu.test.js:41-49`` (AlphaFold captures:
mean abs < 1e-5, max abs < 1e-4).
"""
import os

import numpy as np
import pytest

from oracle import oracle

TRIANGLE = [
    ("openfold-triangle-small", 1e-7, 1e-6),
    ("alphafold-short-9", 1e-5, 1e-4),
    ("alphafold-single-59", 1e-5, 1e-4),
    ("alphafold-a3m-59", 1e-5, 1e-4),
]


def load_triangle(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name + ".npz"))
    n, cz, c = (int(v) for v in d["shape"])
    weights = {k: d[k] for k in oracle.TRIANGLE_WEIGHT_ORDER}
    return d["z"], d["mask"], weights, c, float(d["epsilon"]), d["expected"]


@pytest.mark.parametrize("name,mean_bound,max_bound", TRIANGLE)
def test_trimul_outgoing_matches_golden(golden_dir, name, mean_bound, max_bound):
    z, mask, weights, c, eps, expected = load_triangle(golden_dir, name)
    got = oracle.trimul_af2(z, mask, weights, c, eps, incoming=False)
    delta = np.abs(got.astype(np.float64) - expected.astype(np.float64))
    assert delta.mean() < mean_bound
    assert delta.max() < max_bound
    assert oracle.relative_l2(got, expected) < 1e-6


def test_incoming_equals_outgoing_on_transposed_pair(golden_dir):
    """incoming(z)[i,j] = sum_k a[k,j] b[k,i]; with every per-pair quantity
    computed from the transposed pair this is the outgoing form, transposed back."""
    z, mask, w, c, eps, _ = load_triangle(golden_dir, "alphafold-short-9")
    rng = np.random.default_rng(3)
    mask = (rng.random(mask.shape) > 0.2).astype(np.float32)
    inc = oracle.trimul_af2(z, mask, w, c, eps, incoming=True)
    zt = np.ascontiguousarray(z.transpose(1, 0, 2))
    out_t = oracle.trimul_af2(zt, np.ascontiguousarray(mask.T), w, c, eps, incoming=False)
    np.testing.assert_array_equal(inc, out_t.transpose(1, 0, 2))


def test_int5_decode_matches_reference_quantiser(golden_dir):
    d = np.load(os.path.join(golden_dir, "int5-vectors.npz"))
    count = len([k for k in d.files if k.startswith("values_")])
    assert count >= 5
    for i in range(count):
        values = d[f"values_{i}"]
        got = oracle.int5_decode(d[f"packed_{i}"], d[f"scales_{i}"], d[f"zeros_{i}"], values.size)
        np.testing.assert_array_equal(got, d[f"decoded_{i}"])
        # a 5-bit code is at most half a step away from the value it encodes
        step = np.repeat(d[f"scales_{i}"].astype(np.float32), 32)[: values.size]
        assert np.all(np.abs(got - values) <= 0.5 * step + 2e-3 * np.abs(values) + 1e-6)
