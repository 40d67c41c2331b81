"""float32 parity of every operator, through the C ABI, against the CPU oracle.

Tolerance: relative L2 <= 1e-5 per operator and per block (the reference's own
f32 bound: ``tools/gpu/check-af3-triangle.js:92-122``, ``check-evoformer-*.js``)
and the golden-fixture bounds of ``test/triangle-multiplication-outgoing.gpu.test.js:41-49``.
"""
import os

import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    return lf.Device(0)


def load_triangle(golden_dir, name):
    d = np.load(os.path.join(golden_dir, name + ".npz"))
    n, cz, c = (int(v) for v in d["shape"])
    weights = {k: d[k] for k in oracle.TRIANGLE_WEIGHT_ORDER}
    return {"shape": {"length": n, "cZ": cz, "cHidden": c}, "z": d["z"], "mask": d["mask"], "weights": weights,
            "epsilon": float(d["epsilon"])}, d["expected"]


@pytest.mark.parametrize("name,mean_bound,max_bound", [
    ("openfold-triangle-small", 1e-6, 1e-5), ("alphafold-short-9", 1e-5, 1e-4),
    ("alphafold-single-59", 1e-5, 1e-4), ("alphafold-a3m-59", 1e-5, 1e-4)])
def test_triangle_outgoing_golden(dev, golden_dir, name, mean_bound, max_bound):
    import localfold_b200 as lf
    inp, expected = load_triangle(golden_dir, name)
    got = lf.TriangleMultiplicationOutgoingGpu(dev).run(inp, {"precision": "f32", "variance": "two-pass"})
    m = lf.error_metrics(got["output"], expected)
    assert m["meanAbsoluteError"] < mean_bound and m["maxAbsoluteError"] < max_bound
    assert got["launches"] > 0


@pytest.mark.parametrize("n,cz,c", [(37, 128, 128), (16, 24, 40), (5, 7, 6), (9, 64, 512)])      # 512: the widest cHidden accepted
@pytest.mark.parametrize("incoming", [False, True])
def test_triangle_af2_ragged(dev, n, cz, c, incoming):
    import localfold_b200 as lf
    d = syn.draw(100 + n)
    z = d.normal(n, n, cz)
    mask = (d.rng.random((n, n)) > 0.15).astype(np.float32)
    w = syn.af2_triangle_weights(d, cz, c)
    cls = lf.TriangleMultiplicationIncomingGpu if incoming else lf.TriangleMultiplicationOutgoingGpu
    got = cls(dev).run({"shape": {"length": n, "cZ": cz, "cHidden": c}, "z": z, "mask": mask, "weights": w},
                       {"precision": "f32", "variance": "two-pass"})["output"]
    want = oracle.trimul_af2(z, mask, w, c, 1e-5, incoming)
    assert oracle.relative_l2(got, want) <= TOL
    assert np.isfinite(got).all()


@pytest.mark.parametrize("direction", ["outgoing", "incoming"])
def test_triangle_af3(dev, direction):
    import localfold_b200 as lf
    n, c = 29, 64
    d = syn.draw(7)
    pair = d.normal(n, n, c)
    mask = syn.residue_pair_mask(n, 0.1)
    w = syn.af3_triangle_weights(d, c)
    got = lf.af3_triangle_multiplication(dev, pair, mask, n, c, direction, w, {"precision": "f32"})["output"]
    want = oracle.trimul_af3(pair, mask, w, direction == "incoming")
    assert oracle.relative_l2(got, want) <= TOL


@pytest.mark.parametrize("case", ["plain", "transpose", "normalized-input", "normalized-input-transpose", "separate"])
def test_attention_af2(dev, case):
    import localfold_b200 as lf
    d = syn.draw(11)
    heads, dim = 4, 8
    c = heads * dim
    if case.startswith("normalized"):
        batch = q = 13
    else:
        batch, q = 5, 13
    act = d.normal(batch * q, c)
    mask = (d.rng.random(batch * q) > 0.2).astype(np.float32)
    w = syn.af2_attention_weights(d, c, heads)["attention"]
    transpose = "transpose" in case
    pb = None
    if case.startswith("normalized"):
        pb = {"source": "normalized-input", "projectionWeight": d.linear(c, c, heads)}
    if case == "separate":
        pc = 24
        pb = {"source": "separate", "activations": d.normal(q, q, pc), "channels": pc,
              "layerNormScale": 1 + d.normal(pc, std=0.1), "layerNormOffset": d.normal(pc, std=0.1),
              "projectionWeight": d.linear(pc, pc, heads)}
    inp = {"activations": act, "mask": mask, "batch": batch, "queryLength": q, "channels": c, "heads": heads,
           "transpose": transpose, "weights": w}
    if pb:
        inp["pairBias"] = pb
    got = lf.AttentionGpu(dev).run(inp, {"precision": "f32", "variance": "two-pass"})["output"]
    want = oracle.attention_af2(act, mask, batch, q, c, heads, w, transpose, pb)
    assert oracle.relative_l2(got, want) <= TOL


def test_attention_fully_masked_row_is_uniform(dev):
    """Every key of batch row 2 is masked: float32 logits collapse to one value
    and the softmax is uniform, never 0/0."""
    import localfold_b200 as lf
    d = syn.draw(12)
    heads, dim, batch, q = 2, 16, 4, 40
    c = heads * dim
    act = d.normal(batch * q, c)
    mask = np.ones((batch, q), np.float32)
    mask[2, :] = 0
    w = syn.af2_attention_weights(d, c, heads)["attention"]
    inp = {"activations": act, "mask": mask, "batch": batch, "queryLength": q, "channels": c, "heads": heads,
           "weights": w}
    got = lf.AttentionGpu(dev).run(inp, {"precision": "f32", "variance": "two-pass"})["output"]
    want = oracle.attention_af2(act, mask, batch, q, c, heads, w, False, None)
    assert np.isfinite(got).all()
    assert oracle.relative_l2(got, want) <= TOL


@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("swap", [False, True])
def test_grid_attention_af3(dev, transpose, swap):
    import localfold_b200 as lf
    n, heads, dim = 21, 4, 8
    c = 32
    d = syn.draw(13)
    pair = d.normal(n, n, c)
    mask = (d.rng.random((n, n)) > 0.2).astype(np.float32)
    w = syn.af3_grid_attention_weights(d, c, heads, dim)
    got = lf.Af3GridSelfAttentionGpu(dev).run(pair, mask, {"n": n, "channels": c, "transpose": transpose}, w,
                                              {"swapTransposedBias": swap}, {"precision": "f32"})["output"]
    want = oracle.grid_attention_af3(pair, mask, w, transpose, swap)
    assert oracle.relative_l2(got, want) <= TOL


def test_transition_af2_ragged_primes(dev):
    import localfold_b200 as lf
    rows, c, hidden = 37, 67, 131    # the reference checker's shape
    d = syn.draw(14)
    act = d.normal(rows, c)
    w = {"layerNormScale": 1 + d.normal(c, std=0.1), "layerNormOffset": d.normal(c, std=0.1),
         "firstWeight": d.linear(c, c, hidden), "firstBias": d.normal(hidden, std=0.1),
         "secondWeight": d.linear(hidden, hidden, c), "secondBias": d.normal(c, std=0.1)}
    got = lf.TransitionGpu(dev).run({"activations": act, "rows": rows, "channels": c, "hiddenChannels": hidden,
                                     "weights": w}, {"precision": "f32", "variance": "two-pass"})["output"]
    want = oracle.transition_af2(act, w, hidden)
    assert oracle.relative_l2(got, want) <= TOL


def test_transition_af3(dev):
    import localfold_b200 as lf
    rows, c = 333, 48
    d = syn.draw(15)
    act = d.normal(rows, c)
    w = syn.af3_transition_weights(d, c, 4)
    got = lf.Af3TransitionGpu(dev).run(act, {"rows": rows, "channels": c, "factor": 4}, w, {"precision": "f32"})["output"]
    want = oracle.transition_af3(act, w, 4)
    assert oracle.relative_l2(got, want) <= TOL


def test_outer_product_mean_af2(dev):
    import localfold_b200 as lf
    S, n, cm, co, cz = 24, 9, 13, 7, 11   # the reference checker's shape
    d = syn.draw(16)
    msa = d.normal(S, n, cm)
    mask = (d.rng.random((S, n)) > 0.2).astype(np.float32)
    w = syn.af2_opm_weights(d, cm, co, cz)
    w["leftBias"] = d.normal(co, std=0.1)
    w["rightBias"] = d.normal(co, std=0.1)
    w["outputBias"] = d.normal(cz, std=0.1)
    got = lf.OuterProductMeanGpu(dev).run({"activations": msa, "mask": mask, "sequences": S, "length": n, "cM": cm,
                                           "cOuter": co, "cZ": cz, "weights": w},
                                          {"precision": "f32", "variance": "two-pass"})["output"]
    want = oracle.outer_product_mean_af2(msa, mask, w, co, cz)
    assert oracle.relative_l2(got, want) <= TOL


def test_single_attention_af3(dev):
    import localfold_b200 as lf
    n, cs, cz, heads = 19, 48, 32, 4
    d = syn.draw(17)
    single = d.normal(n, cs)
    pair = d.normal(n, n, cz)
    seq_mask = np.ones(n, np.float32)
    seq_mask[-3:] = 0
    w = {"singlePairLogitsNormScale": syn.ones(cz), "singlePairLogitsNormOffset": syn.zeros(cz),
         "singlePairLogitsProjection": d.linear(cz, cz, heads),
         "singleAttention": syn.af3_single_attention_weights(d, cs, heads, cs // heads)}
    got = lf.Af3SingleAttentionGpu(dev).run(single, pair, seq_mask, {"n": n, "channels": cs, "pairChannels": cz}, w,
                                            {"precision": "f32"})["output"]
    logits = oracle.pair_logits_af3(pair, w["singlePairLogitsNormScale"], w["singlePairLogitsNormOffset"],
                                    w["singlePairLogitsProjection"], heads)
    want = oracle.single_attention_af3(single, logits, seq_mask, w["singleAttention"])
    assert oracle.relative_l2(got, want) <= TOL


def test_int5_decode(dev, golden_dir):
    import localfold_b200 as lf
    d = np.load(os.path.join(golden_dir, "int5-vectors.npz"))
    count = len([k for k in d.files if k.startswith("values_")])
    for i in range(count):
        packed = d[f"packed_{i}"].tobytes() + b"\x00"
        pad = (-len(packed)) % 4
        scales, zeros = d[f"scales_{i}"], d[f"zeros_{i}"]
        payload = packed + b"\x00" * pad + scales.astype("<f2").tobytes() + zeros.astype("<f2").tobytes()
        scale_offset = len(packed) + pad
        got = lf.int5_decode(dev, payload, scale_offset, scale_offset + scales.nbytes, d[f"values_{i}"].size)
        np.testing.assert_array_equal(got, d[f"decoded_{i}"])


def test_af2_pair_block_config0(dev):
    """BASELINE config 0: N=64, c_z=128, float32, seed 0, mask ones."""
    import localfold_b200 as lf
    n = 64
    pair, mask, weights = syn.af2_pair_block(0, n)
    stages = []
    want = oracle.af2_pair_block(pair, mask, weights[0], 128, stages=stages)
    stack = lf.PairStackGpu(dev).prepare(weights, 128, 128)
    got = stack.run(pair, mask, {"precision": "f32", "variance": "two-pass"})
    assert oracle.relative_l2(got["pair"], want) <= TOL
    assert got["launches"] >= 5
    stack.close()


def test_af3_pairformer_block_small(dev):
    import localfold_b200 as lf
    n, cz, cs = 24, 32, 48
    pair, single, pair_mask, seq_mask, blocks = syn.af3_pairformer(2, n, cz, cs, blocks=2, pair_heads=4, single_heads=4)
    seq_mask[-2:] = 0
    pair_mask = np.outer(seq_mask, seq_mask).astype(np.float32)
    wp, ws = pair, single
    for w in blocks:
        wp, ws = oracle.af3_pairformer_block(wp, ws, pair_mask, seq_mask, w, True)
    got = lf.Af3PairformerStackGpu(dev).run({"pair": pair, "single": single, "pairMask": pair_mask,
                                             "seqMask": seq_mask, "tokens": n}, blocks,
                                            {"swapTransposedBias": True}, {"precision": "f32"})
    assert oracle.relative_l2(got["pair"], wp) <= 3 * TOL      # two blocks
    assert oracle.relative_l2(got["single"], ws) <= 3 * TOL


def test_shape_errors_name_the_tensor(dev):
    import localfold_b200 as lf
    pair, mask, weights = syn.af2_pair_block(0, 8)
    w = weights[0]["triangleMultiplicationOutgoing"]
    with pytest.raises(lf.RangeError, match="z has"):
        lf.TriangleMultiplicationOutgoingGpu(dev).run({"shape": {"length": 8, "cZ": 128, "cHidden": 128},
                                                       "z": pair[:-1], "mask": mask, "weights": w})
    bad = dict(w, linearGWeight=w["linearGWeight"][:-1])
    with pytest.raises(lf.RangeError, match="linearGWeight has"):
        lf.TriangleMultiplicationOutgoingGpu(dev).run({"shape": {"length": 8, "cZ": 128, "cHidden": 128},
                                                       "z": pair, "mask": mask, "weights": bad})
    with pytest.raises(ValueError, match="swapTransposedBias"):
        lf.Af3GridSelfAttentionGpu(dev).run(pair, mask, {"n": 8, "channels": 128}, {}, {})


@pytest.mark.parametrize("precision,tol", [("f32", 1e-5), ("bf16", 2e-3)])
def test_template_pair_stack_order_and_width(dev, precision, tol):
    """The template pair stack: the same block at 64 channels with the attentions first
    (``webgpu/af2/evoformer/block.js:1746-1781``; widths: ``shared/bundles/alphafold-fixture.js:418-451``)."""
    import localfold_b200 as lf
    n, cz = 40, 64
    pair, mask, weights = syn.af2_pair_block(90, n, cz, cz, 4, blocks=2, masked_tail=0.1)
    want = pair
    for w in weights:
        want = oracle.af2_template_pair_block(want, mask, w, cz)
    other = oracle.af2_pair_block(pair, mask, weights[0], cz)
    stack = lf.PairStackGpu(dev).prepare(weights, cz, cz)
    got = stack.run(pair, mask, {"precision": precision, "variance": "two-pass", "order": "template"})
    stack.close()
    assert oracle.relative_l2(got["pair"], want) <= tol
    assert oracle.relative_l2(want, oracle.af2_pair_block(other, mask, weights[1], cz)) > 1e-3      # the order matters
