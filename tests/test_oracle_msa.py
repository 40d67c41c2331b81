"""CPU checks of the oracle's AF3 MSA-block pieces (``cpu/af3/trunk/msa.js``, ``cpu/af3/trunk/trunk.js:47-60``).

No golden data exists for these operators in the reference checkout, so the C restatement is cross-checked
against an independent float64 numpy formulation and against the hand-computed cases the reference's own
tests use for the outer product mean (``test/af3-msa.test.js``: the sum over sequences comes before the
division, and the denominator is the per-pair coverage) and the MSA block (``test/opendde-branches.test.js``:
the two orders of the crossing lines give different blocks, and the order has no default)."""
import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle


def _ln(x, g, b):
    m = x.mean(-1, keepdims=True)
    v = (x * x).mean(-1, keepdims=True) - m * m
    return (x - m) / np.sqrt(v + 1e-5) * g + b


def _msa_attention_f64(msa, mask, pair, a):
    S, n, _ = msa.shape
    H, D = a["heads"], a["dimension"]
    x = _ln(msa.astype(np.float64), a["actNormScale"], a["actNormOffset"])
    z = _ln(pair.astype(np.float64), a["pairNormScale"], a["pairNormOffset"])
    logits = (z @ a["pairLogits"].astype(np.float64)).transpose(2, 0, 1) + 1e9 * (mask.max(0)[None, None, :] - 1)
    logits -= logits.max(-1, keepdims=True)
    w = np.exp(logits)
    w /= w.sum(-1, keepdims=True)
    v = (x @ a["vProjection"].astype(np.float64)).reshape(S, n, H, D)
    avg = np.einsum("hij,sjhd->sihd", w, v).reshape(S, n, H * D)
    gate = 1 / (1 + np.exp(-(x @ a["gatingQuery"].astype(np.float64))))
    return (avg * gate) @ a["outputProjection"].astype(np.float64)


@pytest.mark.parametrize("cm,heads,dim", [(16, 2, 8), (32, 4, 4)])      # the second: heads * dim != channels
def test_msa_attention_against_float64(cm, heads, dim):
    msa, pair, mask, _, w = syn.af3_msa_block(11, S=5, n=14, cm=cm, cz=16, co=4, msa_heads=heads, msa_dim=dim, pair_heads=2)
    got = oracle.msa_attention_af3(msa, mask, pair, w["msaAttention1"])
    want = _msa_attention_f64(msa, mask, pair, w["msaAttention1"])
    assert oracle.relative_l2(got, want) <= 1e-6


def test_msa_attention_key_mask_is_the_maximum_over_the_depth():
    msa, pair, _, _, w = syn.af3_msa_block(12, S=3, n=10, cm=16, cz=16, co=4, msa_heads=2, msa_dim=8, pair_heads=2)
    mask = np.ones((3, 10), np.float32)
    mask[:, 4] = 0          # no sequence covers token 4: nobody attends to it
    mask[1:, 7] = 0         # one sequence covers token 7: every sequence attends to it
    base = oracle.msa_attention_af3(msa, mask, pair, w["msaAttention1"])
    bumped = msa.copy()
    bumped[:, 4] *= -2.0     # (a constant shift would vanish in the LayerNorm)
    moved = oracle.msa_attention_af3(bumped, mask, pair, w["msaAttention1"])
    others = [t for t in range(10) if t != 4]
    assert np.allclose(moved[:, others], base[:, others], atol=1e-6)
    bumped = msa.copy()
    bumped[2, 7] *= -2.0    # sequence 2 does not cover token 7 itself, yet its own row reads it as a key
    moved = oracle.msa_attention_af3(bumped, mask, pair, w["msaAttention1"])
    assert np.abs(moved[2, others] - base[2, others]).max() > 1e-4
    assert np.allclose(moved[:2], base[:2], atol=1e-6)      # values are per sequence


def _pinned_opm(left, right):
    # one MSA channel, one outer channel: LayerNorm of a single channel is its offset, so left and right equal
    # the projection weights whatever the input holds
    return {"outerChannels": 1, "layerNormInputScale": np.zeros(1, np.float32), "layerNormInputOffset": np.ones(1, np.float32),
            "leftProjection": np.array([left], np.float32), "rightProjection": np.array([right], np.float32),
            "outputW": np.ones(1, np.float32), "outputB": np.zeros(1, np.float32)}


def test_outer_product_mean_sums_over_sequences_before_dividing():
    msa = np.zeros((2, 2, 1), np.float32)
    mask = np.ones((2, 2), np.float32)
    out = oracle.outer_product_mean_af3(msa, mask, _pinned_opm(2, 3), 1)
    assert np.allclose(out, 12 / (1e-3 + 2), atol=1e-4)


def test_outer_product_mean_divides_by_the_coverage_of_both_tokens():
    msa = np.zeros((2, 2, 1), np.float32)
    mask = np.array([[1, 1], [1, 0]], np.float32)        # sequence 1 covers token 0 only
    out = oracle.outer_product_mean_af3(msa, mask, _pinned_opm(2, 3), 1).reshape(2, 2)
    assert abs(out[0, 0] - 12 / (1e-3 + 2)) < 1e-4
    assert abs(out[1, 1] - 6 / (1e-3 + 1)) < 1e-4
    assert abs(out[0, 1] - 6 / (1e-3 + 1)) < 1e-4


def test_outer_product_mean_bias_after_the_division():
    """The dialect key ``opmBiasAfterNorm`` (``cpu/af3/trunk/msa.js:141-150``): sum / max(count, 1) + bias instead of
    (sum + bias) / (1e-3 + count); a pair no sequence covers divides by one and keeps the bare bias.  Hand values,
    then a float64 formulation on random inputs."""
    w = dict(_pinned_opm(2, 3), outputB=np.array([5.0], np.float32))
    msa = np.zeros((2, 2, 1), np.float32)
    mask = np.array([[1, 1], [1, 0]], np.float32)
    after = oracle.outer_product_mean_af3(msa, mask, w, 1, bias_after_norm=True).reshape(2, 2)
    before = oracle.outer_product_mean_af3(msa, mask, w, 1, bias_after_norm=False).reshape(2, 2)
    assert abs(after[0, 0] - (12 / 2 + 5)) < 1e-5 and abs(before[0, 0] - (12 + 5) / (1e-3 + 2)) < 1e-4
    assert abs(after[0, 1] - (6 / 1 + 5)) < 1e-5 and abs(after[1, 1] - (6 / 1 + 5)) < 1e-5
    none = oracle.outer_product_mean_af3(msa, np.zeros((2, 2), np.float32), w, 1, bias_after_norm=True)
    assert np.allclose(none, 5.0)
    rng = np.random.default_rng(12)
    S, n, cm, co, cz = 7, 9, 16, 4, 6
    msa = rng.standard_normal((S, n, cm)).astype(np.float32)
    mask = (rng.random((S, n)) > 0.3).astype(np.float32)
    w = {"outerChannels": co, "layerNormInputScale": (1 + 0.1 * rng.standard_normal(cm)).astype(np.float32),
         "layerNormInputOffset": (0.1 * rng.standard_normal(cm)).astype(np.float32),
         "leftProjection": (rng.standard_normal((cm, co)) / 4).astype(np.float32),
         "rightProjection": (rng.standard_normal((cm, co)) / 4).astype(np.float32),
         "outputW": (rng.standard_normal((co * co, cz)) / 4).astype(np.float32),
         "outputB": rng.standard_normal(cz).astype(np.float32)}
    x = msa.astype(np.float64)
    mean = x.mean(-1, keepdims=True)
    xn = (x - mean) / np.sqrt(((x - mean) ** 2).mean(-1, keepdims=True) + 1e-5) * w["layerNormInputScale"] + w["layerNormInputOffset"]
    left = xn @ w["leftProjection"].astype(np.float64) * mask[..., None]
    right = xn @ w["rightProjection"].astype(np.float64) * mask[..., None]
    outer = np.einsum("sia,sjb->ijab", left, right).reshape(n, n, co * co)
    count = np.einsum("si,sj->ij", mask.astype(np.float64), mask.astype(np.float64))
    want = outer @ w["outputW"].astype(np.float64) / np.maximum(count, 1.0)[..., None] + w["outputB"]
    got = oracle.outer_product_mean_af3(msa, mask, w, cz, bias_after_norm=True)
    assert oracle.relative_l2(got, want) < 1e-6


def test_msa_block_order_matters_and_has_no_default():
    msa, pair, mm, pm, w = syn.af3_msa_block(13, S=3, n=8, cm=16, cz=16, co=4, msa_heads=2, msa_dim=8, pair_heads=2)
    m_a, p_a = oracle.msa_block_af3(msa, pair, mm, pm, w, False, False)
    m_b, p_b = oracle.msa_block_af3(msa, pair, mm, pm, w, False, True)
    assert oracle.relative_l2(m_a, m_b) > 1e-6
    assert oracle.relative_l2(p_a, p_b) > 1e-6
    with pytest.raises(ValueError, match="no default"):
        oracle.msa_block_af3(msa, pair, mm, pm, w, False, None)


def test_distogram_logits_are_a_sum_with_the_transpose():
    rng = np.random.default_rng(3)
    pair = rng.standard_normal((7, 7, 12)).astype(np.float32)        # not symmetric in i and j
    w = rng.standard_normal((12, 6)).astype(np.float32)
    bias = rng.standard_normal(6).astype(np.float32)
    got = oracle.distogram_logits(pair, w, bias)
    half = pair.astype(np.float64) @ w + bias
    assert np.abs(got - (half + half.transpose(1, 0, 2))).max() < 1e-5
    assert np.abs(got - got.transpose(1, 0, 2)).max() == 0


def test_global_column_attention_against_float64():
    """The extra-MSA global column attention (defined by the reference's shaders only) against an independent
    float64 formulation of the same sums."""
    d = syn.draw(21)
    S, n, c, H, D = 9, 11, 32, 4, 8
    msa = d.normal(S, n, c)
    mask = (d.rng.random((S, n)) >= 0.3).astype(np.float32)
    mask[0] = 1
    w = syn.af2_global_attention_weights(d, c, H, D)
    got = oracle.global_column_attention_af2(msa, mask, w)
    x = msa.astype(np.float64)
    m = x.mean(-1, keepdims=True)
    v = ((x - m) ** 2).mean(-1, keepdims=True)
    nx = (x - m) / np.sqrt(v + 1e-5) * w["queryNormScale"] + w["queryNormOffset"]
    mk = mask.astype(np.float64)
    q_avg = (nx * mk[..., None]).sum(0) / (1e-10 + mk.sum(0))[:, None]
    q = (q_avg @ w["queryWeight"].astype(np.float64)).reshape(n, H, D) * D ** -0.5
    k = nx @ w["keyWeight"].astype(np.float64)
    val = nx @ w["valueWeight"].astype(np.float64)
    logits = np.where(mk.T[:, None, :] == 0, -1e9, np.einsum("nhd,snd->nhs", q, k))
    logits -= logits.max(-1, keepdims=True)
    p = np.exp(logits)
    p /= p.sum(-1, keepdims=True)
    att = np.einsum("nhs,snd->nhd", p, val).reshape(n, H * D)
    gate = 1 / (1 + np.exp(-(nx @ w["gatingWeight"].astype(np.float64) + w["gatingBias"])))
    want = (gate * att[None]) @ w["outputWeight"].astype(np.float64) + w["outputBias"]
    assert oracle.relative_l2(got, want) <= 1e-6
