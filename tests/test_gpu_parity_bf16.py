"""bf16 tensor-core path against the CPU oracle (float32 reference arithmetic).

Tolerances: per operator 8e-3 relative L2 (the reference's bound for its
half-precision arms: ``tools/gpu/check-evoformer-attention.js:162``,
``tools/gpu/check-triangle.js:59``); per block 2e-3 on the block's output pair,
the bound this library is specified to.
"""
import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle

pytestmark = pytest.mark.gpu
OP_TOL = 8e-3
BLOCK_TOL = 2e-3


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    return lf.Device(0)


@pytest.mark.parametrize("n", [64, 203, 300])
@pytest.mark.parametrize("incoming", [False, True])
def test_triangle_bf16(dev, n, incoming):
    import localfold_b200 as lf
    d = syn.draw(300 + n)
    z = d.normal(n, n, 128)
    mask = syn.residue_pair_mask(n, 0.05)
    w = syn.af2_triangle_weights(d, 128, 128)
    cls = lf.TriangleMultiplicationIncomingGpu if incoming else lf.TriangleMultiplicationOutgoingGpu
    got = cls(dev).run({"shape": {"length": n, "cZ": 128, "cHidden": 128}, "z": z, "mask": mask, "weights": w},
                       {"precision": "bf16", "variance": "two-pass"})["output"]
    want = oracle.trimul_af2(z, mask, w, 128, 1e-5, incoming)
    assert np.isfinite(got).all()
    assert oracle.relative_l2(got, want) <= OP_TOL


@pytest.mark.parametrize("incoming", [False, True])
def test_triangle_bf16_layer_norm_gains_and_offsets(dev, incoming):
    """The tensor-core path keeps the LayerNorm gains and offsets inside its weight images and biases: a case
    where they are far from (1, 0), for the input norm (projection and output gate) and the centre norm."""
    import localfold_b200 as lf
    from parity_report import record
    n = 128
    d = syn.draw(4242)
    z = d.normal(n, n, 128) + 0.5          # a mean that the offsets' path has to carry
    mask = syn.residue_pair_mask(n, 0.05)
    w = syn.af2_triangle_weights(d, 128, 128)
    w["layerNormInWeight"] = 1 + d.normal(128, std=0.3)
    w["layerNormInBias"] = d.normal(128, std=0.3)
    w["layerNormOutWeight"] = 1 + d.normal(128, std=0.3)
    w["layerNormOutBias"] = d.normal(128, std=0.3)
    for role in ("AP", "AG", "BP", "BG", "Z", "G"):
        w[f"linear{role}Bias"] = w[f"linear{role}Bias"] + d.normal(128, std=0.2)
    cls = lf.TriangleMultiplicationIncomingGpu if incoming else lf.TriangleMultiplicationOutgoingGpu
    got = cls(dev).run({"shape": {"length": n, "cZ": 128, "cHidden": 128}, "z": z, "mask": mask, "weights": w},
                       {"precision": "bf16", "variance": "two-pass"})["output"]
    want = oracle.trimul_af2(z, mask, w, 128, 1e-5, incoming)
    err = oracle.relative_l2(got, want)
    record("triangle_bf16", f"n={n} incoming={incoming} random LayerNorm gains and offsets", err, OP_TOL)
    assert np.isfinite(got).all()
    assert err <= OP_TOL


@pytest.mark.parametrize("transpose", [False, True])
def test_triangle_attention_bf16_layer_norm_gains_and_offsets(dev, transpose):
    """As above for the attention: the norm's offset reaches q, k, v, the gate and the pair-bias logits."""
    import localfold_b200 as lf
    from parity_report import record
    n = 96
    d = syn.draw(4343)
    z = d.normal(n, n, 128) + 0.5
    mask = syn.residue_pair_mask(n, 0.1)
    t = syn.af2_attention_weights(d, 128, 4, 128)
    t["attention"]["queryNormScale"] = 1 + d.normal(128, std=0.3)
    t["attention"]["queryNormOffset"] = d.normal(128, std=0.3)
    t["attention"]["gatingBias"] = t["attention"]["gatingBias"] + d.normal(128, std=0.2)
    t["attention"]["outputBias"] = d.normal(128, std=0.2)
    pb = dict(t["pairBias"], source="normalized-input")
    inp = {"activations": z, "mask": mask, "batch": n, "queryLength": n, "channels": 128, "heads": 4,
           "transpose": transpose, "weights": t["attention"], "pairBias": pb}
    got = lf.AttentionGpu(dev).run(inp, {"precision": "bf16", "variance": "two-pass"})["output"]
    want = oracle.attention_af2(z, mask, n, n, 128, 4, t["attention"], transpose, pb)
    err = oracle.relative_l2(got, want)
    record("attention_bf16", f"n={n} transpose={transpose} random LayerNorm gains and offsets", err, OP_TOL)
    assert np.isfinite(got).all()
    assert err <= OP_TOL


def test_triangle_bf16_af3_channels_64(dev):
    import localfold_b200 as lf
    n, c = 96, 64
    d = syn.draw(31)
    pair = d.normal(n, n, c)
    mask = syn.residue_pair_mask(n, 0.1)
    w = syn.af3_triangle_weights(d, c)
    for direction in ("outgoing", "incoming"):
        got = lf.af3_triangle_multiplication(dev, pair, mask, n, c, direction, w, {"precision": "bf16"})["output"]
        want = oracle.trimul_af3(pair, mask, w, direction == "incoming")
        assert oracle.relative_l2(got, want) <= OP_TOL


@pytest.mark.parametrize("n", [64, 300])
def test_af2_pair_block_bf16(dev, n):
    import localfold_b200 as lf
    from parity_report import record
    pair, mask, weights = syn.af2_pair_block(n - 64, n, masked_tail=0.05)
    want = oracle.af2_pair_block(pair, mask, weights[0], 128)
    stack = lf.PairStackGpu(dev).prepare(weights, 128, 128)
    got = stack.run(pair, mask, {"precision": "bf16", "variance": "two-pass"})
    stack.close()
    err = oracle.relative_l2(got["pair"], want)
    record("af2_pair_block", f"n={n}", err, BLOCK_TOL)
    assert err <= BLOCK_TOL


def test_af2_pair_block_bf16_at_the_metric_length(dev):
    """N = 384, the shorter of the two lengths the metric names: the whole block against the float64
    formulation (the scalar oracle takes tens of seconds there), at the per-block bound."""
    import localfold_b200 as lf
    from oracle import tier2_torch as t2
    from parity_report import record
    n = 384
    pair, mask, weights = syn.af2_pair_block(384, n, masked_tail=0.05)
    want = t2.af2_pair_block(pair, mask, weights[0])
    stack = lf.PairStackGpu(dev).prepare(weights, 128, 128)
    got = stack.run(pair, mask, {"precision": "bf16", "variance": "two-pass"})
    f32 = stack.run(pair, mask, {"precision": "f32", "variance": "two-pass"})
    stack.close()
    err = oracle.relative_l2(got["pair"], want)
    record("af2_pair_block", "n=384 vs float64", err, BLOCK_TOL)
    record("af2_pair_block", "n=384 f32 mode vs float64", oracle.relative_l2(f32["pair"], want), 1e-5)
    assert err <= BLOCK_TOL
    assert oracle.relative_l2(f32["pair"], want) <= 1e-5


@pytest.mark.parametrize("n", [64, 77, 260])
@pytest.mark.parametrize("transpose", [False, True])
def test_triangle_attention_af2_bf16(dev, n, transpose):
    import localfold_b200 as lf
    d = syn.draw(500 + n)
    z = d.normal(n, n, 128)
    mask = syn.residue_pair_mask(n, 0.1)
    t = syn.af2_attention_weights(d, 128, 4, 128)
    pb = dict(t["pairBias"], source="normalized-input")
    inp = {"activations": z, "mask": mask, "batch": n, "queryLength": n, "channels": 128, "heads": 4,
           "transpose": transpose, "weights": t["attention"], "pairBias": pb}
    got = lf.AttentionGpu(dev).run(inp, {"precision": "bf16", "variance": "two-pass"})["output"]
    want = oracle.attention_af2(z, mask, n, n, 128, 4, t["attention"], transpose, pb)
    assert np.isfinite(got).all()
    assert oracle.relative_l2(got, want) <= OP_TOL


@pytest.mark.parametrize("transpose,swap", [(False, False), (True, False), (True, True)])
def test_grid_attention_af3_bf16(dev, transpose, swap):
    import localfold_b200 as lf
    n = 72
    d = syn.draw(600)
    z = d.normal(n, n, 128)
    mask = (d.rng.random((n, n)) > 0.1).astype(np.float32)
    w = syn.af3_grid_attention_weights(d, 128, 4, 32)
    got = lf.Af3GridSelfAttentionGpu(dev).run(z, mask, {"n": n, "channels": 128, "transpose": transpose}, w,
                                              {"swapTransposedBias": swap}, {"precision": "bf16"})["output"]
    want = oracle.grid_attention_af3(z, mask, w, transpose, swap)
    assert oracle.relative_l2(got, want) <= OP_TOL


def test_triangle_attention_bf16_fully_masked_row(dev):
    """A residue masked out everywhere: its row of the pair mask is all zero, so every key of
    that batch row is masked and the softmax must come out uniform, not 0/0."""
    import localfold_b200 as lf
    n = 150
    d = syn.draw(700)
    z = d.normal(n, n, 128)
    res = np.ones(n, np.float32)
    res[[3, 77, 149]] = 0
    mask = np.outer(res, res).astype(np.float32)
    t = syn.af2_attention_weights(d, 128, 4, 128)
    pb = dict(t["pairBias"], source="normalized-input")
    inp = {"activations": z, "mask": mask, "batch": n, "queryLength": n, "channels": 128, "heads": 4,
           "weights": t["attention"], "pairBias": pb}
    got = lf.AttentionGpu(dev).run(inp, {"precision": "bf16", "variance": "two-pass"})["output"]
    want = oracle.attention_af2(z, mask, n, n, 128, 4, t["attention"], False, pb)
    assert np.isfinite(got).all()
    assert oracle.relative_l2(got, want) <= OP_TOL


@pytest.mark.parametrize("rows", [128, 1000, 40000])
def test_transition_af2_bf16(dev, rows):
    import localfold_b200 as lf
    d = syn.draw(800 + rows)
    act = d.normal(rows, 128)
    w = syn.af2_transition_weights(d, 128, 4)
    w["firstBias"] = d.normal(512, std=0.3)
    w["secondBias"] = d.normal(128, std=0.3)
    w["layerNormScale"] = 1 + d.normal(128, std=0.1)
    w["layerNormOffset"] = d.normal(128, std=0.1)
    got = lf.TransitionGpu(dev).run({"activations": act, "rows": rows, "channels": 128, "hiddenChannels": 512,
                                     "weights": w}, {"precision": "bf16", "variance": "two-pass"})
    want = oracle.transition_af2(act, w, 512)
    assert oracle.relative_l2(got["output"], want) <= OP_TOL
    assert got["launches"] == 1      # one fused kernel: the 4x-wide hidden is never written out


def test_triangle_attention_bf16_peaked_logits(dev):
    """Logits with a spread of tens of units: rows whose later keys outrun the reference taken from the
    tile's first keys must take the kernel's two-pass fallback and still match."""
    import localfold_b200 as lf
    n = 200
    d = syn.draw(701)
    z = d.normal(n, n, 128)
    mask = syn.residue_pair_mask(n, 0.05)
    t = syn.af2_attention_weights(d, 128, 4, 128)
    t["attention"]["queryWeight"] = t["attention"]["queryWeight"] * 4.0
    t["attention"]["keyWeight"] = t["attention"]["keyWeight"] * 4.0
    pb = dict(t["pairBias"], source="normalized-input")
    pb["projectionWeight"] = pb["projectionWeight"] * 5.0
    inp = {"activations": z, "mask": mask, "batch": n, "queryLength": n, "channels": 128, "heads": 4,
           "weights": t["attention"], "pairBias": pb}
    got = lf.AttentionGpu(dev).run(inp, {"precision": "bf16", "variance": "two-pass"})["output"]
    want = oracle.attention_af2(z, mask, n, n, 128, 4, t["attention"], False, pb)
    assert np.isfinite(got).all()
    assert oracle.relative_l2(got, want) <= OP_TOL


@pytest.mark.parametrize("rows", [128, 5000])
def test_transition_af3_bf16(dev, rows):
    import localfold_b200 as lf
    d = syn.draw(850 + rows)
    act = d.normal(rows, 128)
    w = syn.af3_transition_weights(d, 128, 4)
    w["inputLayerNormScale"] = 1 + d.normal(128, std=0.1)
    w["inputLayerNormOffset"] = d.normal(128, std=0.1)
    got = lf.Af3TransitionGpu(dev).run(act, {"rows": rows, "channels": 128, "factor": 4}, w, {"precision": "bf16"})
    want = oracle.transition_af3(act, w, 4)
    assert oracle.relative_l2(got["output"], want) <= OP_TOL
    assert got["launches"] == 1


def test_af3_pairformer_block_bf16_int5_weights(dev):
    """BASELINE config 2 shape at reduced N: AF3 pairformer blocks whose linear weights went through the
    int5 bundle format (quantised and decoded identically for the oracle and the GPU)."""
    import localfold_b200 as lf
    from bundle_writer import quantise_weights_like_bundle
    n = 96
    pair, single, pair_mask, seq_mask, blocks = syn.af3_pairformer(2, n, 128, 384, blocks=1)
    blocks = [quantise_weights_like_bundle(b) for b in blocks]
    wp, ws = oracle.af3_pairformer_block(pair, single, pair_mask, seq_mask, blocks[0], True)
    got = lf.Af3PairformerStackGpu(dev).run({"pair": pair, "single": single, "pairMask": pair_mask, "seqMask": seq_mask,
                                             "tokens": n}, blocks, {"swapTransposedBias": True}, {"precision": "bf16"})
    assert oracle.relative_l2(got["pair"], wp) <= BLOCK_TOL
    assert oracle.relative_l2(got["single"], ws) <= BLOCK_TOL


def test_af3_blocks_from_an_int5_bundle_on_disk(dev, tmp_path):
    """The whole loading path: an int5 bundle under the AF3 exporter's tensor names (stacked ``[blocks, ...]``
    tensors) is read with the device decoder, mapped to pairformer block weights and run; the oracle runs on
    the weights the host decoder gives, which must be the same numbers bit for bit."""
    import localfold_b200 as lf
    from localfold_b200 import bundle
    import bundle_writer as writer
    from test_bundle_mapping import af3_bundle_tensors
    n = 64
    pair, single, pair_mask, seq_mask, blocks = syn.af3_pairformer(3, n, 128, 384, blocks=2)
    path = writer.write_bundle(str(tmp_path), af3_bundle_tensors(blocks), shard_bytes=4 << 20)
    on_device = bundle.pairformer_stack_weights(bundle.FileTensorStore(path, device=dev))
    on_host = bundle.pairformer_stack_weights(bundle.FileTensorStore(path))
    for a, b in zip(on_device, on_host):
        for key in ("triangleMultiplicationOutgoing", "pairAttention2", "pairTransition", "singleAttention"):
            for field, value in a[key].items():
                if isinstance(value, np.ndarray):
                    np.testing.assert_array_equal(value, b[key][field], err_msg=f"{key}/{field}")
    wp, ws = pair, single
    for w in on_host:
        wp, ws = oracle.af3_pairformer_block(wp, ws, pair_mask, seq_mask, w, True)
    got = lf.Af3PairformerStackGpu(dev).run({"pair": pair, "single": single, "pairMask": pair_mask, "seqMask": seq_mask,
                                             "tokens": n}, on_device, {"swapTransposedBias": True}, {"precision": "bf16"})
    assert oracle.relative_l2(got["pair"], wp) <= 2 * BLOCK_TOL
    assert oracle.relative_l2(got["single"], ws) <= 2 * BLOCK_TOL
    # and with the int5 tensors left encoded: the codes go to the device and are decoded there, straight into the
    # operators' weight layout - the same weights, so the same result
    encoded = bundle.pairformer_stack_weights(bundle.FileTensorStore(path), encoded=True)
    assert isinstance(encoded[0]["pairTransition"]["transition1"], lf.EncodedTensor)
    assert isinstance(encoded[0]["pairTransition"]["inputLayerNormScale"], np.ndarray)       # kept float32 by the exporter
    again = lf.Af3PairformerStackGpu(dev).run({"pair": pair, "single": single, "pairMask": pair_mask, "seqMask": seq_mask,
                                               "tokens": n}, encoded, {"swapTransposedBias": True}, {"precision": "bf16"})
    np.testing.assert_array_equal(again["pair"], got["pair"])
    np.testing.assert_array_equal(again["single"], got["single"])
    f32 = lf.Af3PairformerStackGpu(dev).run({"pair": pair, "single": single, "pairMask": pair_mask, "seqMask": seq_mask,
                                             "tokens": n}, encoded, {"swapTransposedBias": True}, {"precision": "f32"})
    assert oracle.relative_l2(f32["pair"], wp) <= 2e-5


@pytest.mark.parametrize("n,precision,bound", [(384, "f32", 1e-5), (384, "bf16", 2e-3), (203, "bf16", 2e-3)])
def test_single_attention_af3_at_the_stack_shape(dev, n, precision, bound):
    """AF3 single attention at the 48-block stack's shape (c_s = 384, 16 heads of 24, c_z = 128).  In 16-bit mode
    its pair-sized pass - LayerNorm of the pair and the projection onto the 16 heads - runs on the tensor cores
    (fp16 logits); the attention over the N tokens stays float32."""
    import localfold_b200 as lf
    from parity_report import record
    cs, cz, heads = 384, 128, 16
    d = syn.draw(1700 + n)
    single = d.normal(n, cs)
    pair = d.normal(n, n, cz)
    seq_mask = np.ones(n, np.float32)
    seq_mask[-5:] = 0
    w = {"singlePairLogitsNormScale": 1 + d.normal(cz, std=0.1), "singlePairLogitsNormOffset": d.normal(cz, std=0.1),
         "singlePairLogitsProjection": d.linear(cz, cz, heads),
         "singleAttention": syn.af3_single_attention_weights(d, cs, heads, cs // heads)}
    r = lf.Af3SingleAttentionGpu(dev).run(single, pair, seq_mask, {"n": n, "channels": cs, "pairChannels": cz}, w,
                                          {"precision": precision})
    logits = oracle.pair_logits_af3(pair, w["singlePairLogitsNormScale"], w["singlePairLogitsNormOffset"],
                                    w["singlePairLogitsProjection"], heads)
    want = oracle.single_attention_af3(single, logits, seq_mask, w["singleAttention"])
    err = oracle.relative_l2(r["output"], want)
    record("single_attention_af3", f"n={n} 16x24 {precision}", err, bound)
    assert np.isfinite(r["output"]).all()
    assert err <= bound


def test_msa_row_attention_pair_bias_on_the_16_bit_path(dev):
    """MSA row attention with a separate pair bias (c_m = 256, 8 heads of 32): in 16-bit mode the pair bias - the
    pair-sized pass - comes from the tensor-core projection kernel; the rest of the operator is float32."""
    import localfold_b200 as lf
    from parity_report import record
    S, n, cm, cz, heads = 12, 96, 256, 128, 8
    d = syn.draw(1800)
    msa = d.normal(S, n, cm)
    pair = d.normal(n, n, cz)
    mask = np.ones((S, n), np.float32)
    mask[3] = 0
    t = syn.af2_attention_weights(d, cm, heads, cz, separate=True)
    t["pairBias"]["layerNormScale"] = 1 + d.normal(cz, std=0.2)
    t["pairBias"]["layerNormOffset"] = d.normal(cz, std=0.2)
    pb = dict(t["pairBias"], source="separate", activations=pair, channels=cz)
    inp = {"activations": msa, "mask": mask, "batch": S, "queryLength": n, "channels": cm, "heads": heads,
           "weights": t["attention"], "pairBias": pb}
    want = oracle.attention_af2(msa, mask, S, n, cm, heads, t["attention"], False, pb)
    for precision, bound in (("f32", 1e-5), ("bf16", 2e-3)):
        r = lf.AttentionGpu(dev).run(inp, {"precision": precision, "variance": "two-pass"})
        err = oracle.relative_l2(r["output"], want)
        record("msa_row_attention", f"S={S} n={n} 8x32 {precision}", err, bound)
        assert err <= bound


@pytest.mark.parametrize("S,n,cm,c", [(128, 256, 256, 32), (37, 50, 64, 32), (300, 24, 64, 8), (20, 33, 64, 24)])
def test_outer_product_mean_on_the_16_bit_path(dev, S, n, cm, c):
    """In 16-bit mode the three GEMMs of the operator run on the tensor cores: the left | right projection, the sum
    over the sequences of the outer products (fp16 sums scaled by a power of two near 1 / S) and the c*c -> c_z
    projection, a plain GEMM over the pairs because the sums are stored grouped per pair; the division by the
    coverage is float32.  First case: the Evoformer block's shape; last: a width that is not a power of two."""
    import localfold_b200 as lf
    from parity_report import record
    d = syn.draw(1900 + S)
    msa = d.normal(S, n, cm)
    mask = (d.rng.random((S, n)) >= 0.15).astype(np.float32)
    mask[0] = 1
    w = syn.af2_opm_weights(d, cm, c, 128)
    w["leftBias"] = d.normal(c, std=0.2)
    w["rightBias"] = d.normal(c, std=0.2)
    w["outputBias"] = d.normal(128, std=0.2)
    got = lf.OuterProductMeanGpu(dev).run({"activations": msa, "mask": mask, "sequences": S, "length": n, "cM": cm,
                                           "cOuter": c, "cZ": 128, "weights": w},
                                          {"precision": "bf16", "variance": "two-pass"})["output"]
    want = oracle.outer_product_mean_af2(msa, mask, w, c, 128)
    err = oracle.relative_l2(got, want)
    record("outer_product_mean", f"S={S} n={n} cM={cm} c={c} 16-bit", err, 2e-3)
    assert np.isfinite(got).all()
    assert err <= 2e-3
