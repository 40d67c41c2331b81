"""Cross-validates the C restatement against the independent torch-float64
formulation for the operators that have no golden data, checks the reference's
hand-worked unit cases (``test/af3-pairformer.test.js:24-103``), and the
uniform-softmax behaviour of fully masked rows."""
import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle, tier2_torch as t2

TOL = 2e-6   # float32 stores in the C restatement vs float64 throughout


def rel(a, b):
    return oracle.relative_l2(a, b)


def test_layer_norm_hand_values():
    x = np.array([1, 2, 3, 4, 10, 20, 30, 40], np.float32).reshape(2, 4)
    out = oracle.layer_norm(x, np.ones(4), np.zeros(4), fast=True)
    np.testing.assert_allclose(out[0], out[1], atol=1e-4)
    assert abs(out.sum(1)).max() < 1e-4
    out = oracle.layer_norm(np.array([[1, 2, 3, 4]], np.float32), np.zeros(4), np.array([5, 6, 7, 8]), fast=True)
    np.testing.assert_allclose(out[0], [5, 6, 7, 8], atol=1e-5)
    out = oracle.layer_norm(np.full((1, 4), 2, np.float32), np.ones(4), np.zeros(4), fast=True)
    np.testing.assert_allclose(out[0], 0, atol=1e-5)


def test_linear_layouts_hand_values():
    x = np.array([[1, 2]], np.float32)
    np.testing.assert_allclose(oracle.linear(x, np.array([[1, 2, 3], [10, 20, 30]], np.float32))[0], [21, 42, 63])
    np.testing.assert_allclose(oracle.linear(x, np.array([[1, 10], [2, 20], [3, 30]], np.float32), transposed=True)[0],
                               [21, 42, 63])
    np.testing.assert_allclose(oracle.linear(np.array([[1]], np.float32), np.array([[1, 1]], np.float32),
                                             np.array([5, -5], np.float32))[0], [6, -4])


def test_transition_af3_blocked_split_gate_first():
    inter = 4
    w = {"inputLayerNormScale": np.ones(1, np.float32), "inputLayerNormOffset": np.ones(1, np.float32),
         "transition1": np.zeros((1, inter * 2), np.float32), "transition2": np.zeros((inter, 1), np.float32)}
    w["transition1"][0, 0] = 1
    w["transition1"][0, inter] = 3
    w["transition2"][0, 0] = 1
    out = oracle.transition_af3(np.array([[7]], np.float32), w, 4)
    swish1 = 1 / (1 + np.exp(-1.0))
    assert abs(out[0, 0] - swish1 * 3) < 1e-6


@pytest.mark.parametrize("incoming", [False, True])
def test_trimul_af2_cross(incoming):
    d = syn.draw(1)
    n, cz, c = 17, 20, 12
    z = d.normal(n, n, cz)
    mask = (d.rng.random((n, n)) > 0.2).astype(np.float32)
    w = syn.af2_triangle_weights(d, cz, c)
    assert rel(oracle.trimul_af2(z, mask, w, c, 1e-5, incoming), t2.trimul_af2(z, mask, w, 1e-5, incoming)) < TOL


@pytest.mark.parametrize("incoming", [False, True])
def test_trimul_af3_cross(incoming):
    d = syn.draw(2)
    n, c = 15, 16
    z = d.normal(n, n, c)
    mask = (d.rng.random((n, n)) > 0.2).astype(np.float32)
    w = syn.af3_triangle_weights(d, c)
    assert rel(oracle.trimul_af3(z, mask, w, incoming), t2.trimul_af3(z, mask, w, incoming)) < TOL


@pytest.mark.parametrize("case", ["plain", "transpose", "normalized-input", "normalized-input-transpose", "separate"])
def test_attention_af2_cross(case):
    d = syn.draw(3)
    heads, dim = 3, 8
    c = heads * dim
    batch, q = (11, 11) if case.startswith("normalized") else (4, 11)
    act = d.normal(batch * q, c)
    mask = (d.rng.random(batch * q) > 0.25).astype(np.float32)
    w = syn.af2_attention_weights(d, c, heads)["attention"]
    pb = None
    if case.startswith("normalized"):
        pb = {"source": "normalized-input", "projectionWeight": d.linear(c, c, heads)}
    if case == "separate":
        pb = {"source": "separate", "activations": d.normal(q, q, 10), "channels": 10,
              "layerNormScale": 1 + d.normal(10, std=0.1), "layerNormOffset": d.normal(10, std=0.1),
              "projectionWeight": d.linear(10, 10, heads)}
    tr = "transpose" in case
    a = oracle.attention_af2(act, mask, batch, q, c, heads, w, tr, pb)
    b = t2.attention_af2(act, mask, batch, q, c, heads, w, tr, pb)
    assert rel(a, b) < TOL


def test_attention_fully_masked_row_uniform():
    d = syn.draw(4)
    heads, dim, batch, q = 2, 4, 3, 9
    c = heads * dim
    act = d.normal(batch * q, c)
    mask = np.ones((batch, q), np.float32)
    mask[1] = 0
    w = syn.af2_attention_weights(d, c, heads)["attention"]
    out = oracle.attention_af2(act, mask, batch, q, c, heads, w)
    assert np.isfinite(out).all()
    assert rel(out, t2.attention_af2(act, mask, batch, q, c, heads, w)) < TOL
    # row 1 attends uniformly: every query of that row gets the same value average
    n = t2.ln(t2.T(act).view(batch, q, c), w["queryNormScale"], w["queryNormOffset"])
    v = (n @ t2.T(w["valueWeight"]))[1].mean(0)
    g = 1 / (1 + np.exp(-((n[1] @ t2.T(w["gatingWeight"])).numpy() + w["gatingBias"])))
    want = (v.numpy()[None] * g) @ w["outputWeight"].astype(np.float64) + w["outputBias"]
    assert rel(out.reshape(batch, q, c)[1], want) < 1e-5


@pytest.mark.parametrize("transpose", [False, True])
@pytest.mark.parametrize("swap", [False, True])
def test_grid_attention_af3_cross(transpose, swap):
    d = syn.draw(5)
    n, heads, dim, c = 13, 2, 8, 16
    z = d.normal(n, n, c)
    mask = (d.rng.random((n, n)) > 0.2).astype(np.float32)
    w = syn.af3_grid_attention_weights(d, c, heads, dim)
    assert rel(oracle.grid_attention_af3(z, mask, w, transpose, swap), t2.grid_attention_af3(z, mask, w, transpose, swap)) < TOL


def test_af2_ending_attention_equals_af3_swapped_bias():
    """The AF2 ending-node attention takes its bias from the transposed
    normalised pair; AF3 with swapTransposedBias does the same thing."""
    d = syn.draw(6)
    n, heads, dim = 9, 2, 4
    c = heads * dim
    z = d.normal(n, n, c)
    mask = np.ones((n, n), np.float32)
    a2 = syn.af2_attention_weights(d, c, heads, c)
    att = a2["attention"]
    att["gatingBias"][:] = 0
    w3 = {"heads": heads, "dimension": dim, "actNormScale": att["queryNormScale"], "actNormOffset": att["queryNormOffset"],
          "pairBiasProjection": a2["pairBias"]["projectionWeight"], "qProjection": att["queryWeight"].T.copy(),
          "kProjection": att["keyWeight"].T.copy(), "vProjection": att["valueWeight"],
          "gatingQuery": att["gatingWeight"].T.copy(), "outputProjection": att["outputWeight"]}
    got2 = oracle.attention_af2(z, mask, n, n, c, heads, att, True, dict(a2["pairBias"], source="normalized-input"))
    got3 = oracle.grid_attention_af3(z, mask, w3, True, True)
    assert rel(got2.reshape(n, n, c), got3) < 2e-6


def test_transitions_cross():
    d = syn.draw(7)
    act = d.normal(37, 19)
    w = {"layerNormScale": 1 + d.normal(19, std=0.1), "layerNormOffset": d.normal(19, std=0.1),
         "firstWeight": d.linear(19, 19, 31), "firstBias": d.normal(31, std=0.1),
         "secondWeight": d.linear(31, 31, 19), "secondBias": d.normal(19, std=0.1)}
    assert rel(oracle.transition_af2(act, w, 31), t2.transition_af2(act, w)) < TOL
    w3 = syn.af3_transition_weights(d, 19, 4)
    assert rel(oracle.transition_af3(act, w3, 4), t2.transition_af3(act, w3)) < TOL


def test_opm_cross():
    d = syn.draw(8)
    S, n, cm, co, cz = 24, 9, 13, 7, 11
    msa = d.normal(S, n, cm)
    mask = (d.rng.random((S, n)) > 0.2).astype(np.float32)
    w = syn.af2_opm_weights(d, cm, co, cz)
    w["leftBias"] = d.normal(co, std=0.1)
    w["outputBias"] = d.normal(cz, std=0.1)
    assert rel(oracle.outer_product_mean_af2(msa, mask, w, co, cz), t2.outer_product_mean_af2(msa, mask, w)) < 5e-6


def test_single_attention_cross():
    d = syn.draw(9)
    n, cs, cz, heads = 11, 24, 16, 4
    single, pair = d.normal(n, cs), d.normal(n, n, cz)
    m = np.ones(n, np.float32)
    m[-2:] = 0
    w = {"singlePairLogitsNormScale": syn.ones(cz), "singlePairLogitsNormOffset": syn.zeros(cz),
         "singlePairLogitsProjection": d.linear(cz, cz, heads),
         "singleAttention": syn.af3_single_attention_weights(d, cs, heads, cs // heads)}
    logits = oracle.pair_logits_af3(pair, w["singlePairLogitsNormScale"], w["singlePairLogitsNormOffset"],
                                    w["singlePairLogitsProjection"], heads)
    assert rel(oracle.single_attention_af3(single, logits, m, w["singleAttention"]), t2.single_attention_af3(single, pair, m, w)) < TOL


def test_blocks_cross():
    pair, mask, weights = syn.af2_pair_block(0, 12, 16, 16, 2)
    assert rel(oracle.af2_pair_block(pair, mask, weights[0], 16), t2.af2_pair_block(pair, mask, weights[0])) < 5e-6
    pair, single, pm, sm, blocks = syn.af3_pairformer(2, 10, 16, 24, 1, 2, 4)
    got, _ = oracle.af3_pairformer_block(pair, single, pm, sm, blocks[0], True)
    assert rel(got, t2.af3_pair_block(pair, pm, blocks[0], True)) < 5e-6


def test_thread_count_does_not_change_results():
    pair, mask, weights = syn.af2_pair_block(0, 10, 16, 16, 2)
    oracle.set_threads(1)
    a = oracle.af2_pair_block(pair, mask, weights[0], 16)
    oracle.set_threads(oracle.max_threads())
    b = oracle.af2_pair_block(pair, mask, weights[0], 16)
    np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("flag", [False, True])
def test_sampled_positions_match_the_whole_tensor(flag):
    """The float64 sampled-position forms used at the benchmark's lengths equal the C restatement's
    whole-tensor results at those positions (triangle: flag = incoming; attention: flag = transpose)."""
    d = syn.draw(9)
    n = 37
    z = d.normal(n, n, 128)
    mask = syn.residue_pair_mask(n, 0.1)
    rows, cols = np.array([0, 5, 36, 20]), np.array([3, 4, 35, 1, 2])
    w = syn.af2_triangle_weights(d, 128, 128)
    full = oracle.trimul_af2(z, mask, w, 128, 1e-5, flag)
    assert rel(t2.trimul_af2_positions(z, mask, w, rows, cols, 1e-5, flag), full[np.ix_(rows, cols)]) < TOL
    t = syn.af2_attention_weights(d, 128, 4, 128)
    pb = dict(t["pairBias"], source="normalized-input")
    full = oracle.attention_af2(z, mask, n, n, 128, 4, t["attention"], flag, pb)
    ref = full[np.ix_(cols, rows)].transpose(1, 0, 2) if flag else full[np.ix_(rows, cols)]
    got = t2.attention_af2_positions(z, mask, n, 128, 4, t["attention"], rows, cols, flag, pb["projectionWeight"])
    assert rel(got, ref) < TOL
