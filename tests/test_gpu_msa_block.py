"""AF3 MSA-block operators on the GPU against the CPU oracle: MSA pair-weighted averaging
(``cpu/af3/trunk/msa.js:164-224``), the whole block in both orders of the dialect (``:235-287``) and the
distogram logits (``cpu/af3/trunk/trunk.js:47-60``).  Float32 mode: 1e-5 relative L2 per operator and per
block; 16-bit mode: the pair goes through the tensor-core pair block, bound 2e-3 on the pair, and the MSA,
whose operators stay float32, is bounded by what the pair's rounding feeds back into it."""
import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle

pytestmark = pytest.mark.gpu
F32_TOL = 1e-5


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    d = lf.Device(0)
    yield d
    d.close()


@pytest.mark.parametrize("S,n,cm,heads,dim", [(16, 64, 64, 8, 8), (5, 37, 128, 8, 8), (1, 20, 64, 8, 8)])
def test_msa_attention_f32(dev, S, n, cm, heads, dim):
    import localfold_b200 as lf
    from parity_report import record
    msa, pair, mask, _, w = syn.af3_msa_block(20 + S, S=S, n=n, cm=cm, cz=128, msa_heads=heads, msa_dim=dim)
    got = lf.Af3MsaAttentionGpu(dev).run(msa, mask, pair, {"sequences": S, "tokens": n, "msaChannels": cm, "pairChannels": 128},
                                         w["msaAttention1"], {"precision": "f32"})["output"]
    want = oracle.msa_attention_af3(msa, mask, pair, w["msaAttention1"])
    err = oracle.relative_l2(got, want)
    record("msa_attention_af3", f"S={S} n={n} cm={cm} heads={heads}x{dim}", err, F32_TOL)
    assert np.isfinite(got).all()
    assert err <= F32_TOL


def test_msa_attention_device_tensors_in_place(dev):
    import torch
    import localfold_b200 as lf
    S, n, cm = 6, 48, 64
    msa, pair, mask, _, w = syn.af3_msa_block(31, S=S, n=n, cm=cm, cz=128)
    want = msa + oracle.msa_attention_af3(msa, mask, pair, w["msaAttention1"])
    m = torch.from_numpy(msa).cuda()
    lf.Af3MsaAttentionGpu(dev).run(m, torch.from_numpy(mask).cuda(), torch.from_numpy(pair).cuda(),
                                   {"sequences": S, "tokens": n, "msaChannels": cm, "pairChannels": 128},
                                   w["msaAttention1"], {"precision": "f32", "residual": True}, out=m)
    dev.synchronize()
    assert oracle.relative_l2(m.cpu().numpy(), want) <= F32_TOL


def test_msa_attention_rejects_wrong_sizes(dev):
    import localfold_b200 as lf
    msa, pair, mask, _, w = syn.af3_msa_block(32, S=3, n=16, cm=64, cz=128)
    op = lf.Af3MsaAttentionGpu(dev)
    with pytest.raises(lf.RangeError):
        op.run(msa[:, :-1], mask, pair, {"sequences": 3, "tokens": 16, "msaChannels": 64, "pairChannels": 128}, w["msaAttention1"])
    bad = dict(w["msaAttention1"], heads=8.5)
    with pytest.raises(ValueError):
        op.run(msa, mask, pair, {"sequences": 3, "tokens": 16, "msaChannels": 64, "pairChannels": 128}, bad)


@pytest.mark.parametrize("update_first", [False, True])
def test_msa_block_f32(dev, update_first):
    import localfold_b200 as lf
    from parity_report import record
    S, n = 12, 48
    msa, pair, mm, pm, w = syn.af3_msa_block(40, S=S, n=n)
    dialect = {"swapTransposedBias": False, "msaUpdateBeforeOuterProduct": update_first}
    got = lf.Af3MsaBlockGpu(dev).run({"msa": msa, "pair": pair, "msaMask": mm, "pairMask": pm, "sequences": S, "tokens": n},
                                     w, dialect, {"precision": "f32"})
    want_msa, want_pair = oracle.msa_block_af3(msa, pair, mm, pm, w, False, update_first)
    e_msa, e_pair = oracle.relative_l2(got["msa"], want_msa), oracle.relative_l2(got["pair"], want_pair)
    record("msa_block_af3", f"S={S} n={n} f32 update_first={update_first} msa", e_msa, F32_TOL)
    record("msa_block_af3", f"S={S} n={n} f32 update_first={update_first} pair", e_pair, F32_TOL)
    assert e_msa <= F32_TOL and e_pair <= F32_TOL


def test_msa_block_16_bit_pair_path(dev):
    import localfold_b200 as lf
    from parity_report import record
    S, n = 12, 64
    msa, pair, mm, pm, w = syn.af3_msa_block(41, S=S, n=n)
    dialect = {"swapTransposedBias": True, "msaUpdateBeforeOuterProduct": False}
    got = lf.Af3MsaBlockGpu(dev).run({"msa": msa, "pair": pair, "msaMask": mm, "pairMask": pm, "sequences": S, "tokens": n},
                                     w, dialect, {"precision": "bf16"})
    want_msa, want_pair = oracle.msa_block_af3(msa, pair, mm, pm, w, True, False)
    e_msa, e_pair = oracle.relative_l2(got["msa"], want_msa), oracle.relative_l2(got["pair"], want_pair)
    record("msa_block_af3", f"S={S} n={n} 16-bit msa", e_msa, 2e-3)
    record("msa_block_af3", f"S={S} n={n} 16-bit pair", e_pair, 2e-3)
    assert e_pair <= 2e-3 and e_msa <= 2e-3


@pytest.mark.parametrize("precision,tol", [("f32", F32_TOL), ("bf16", 2e-3)])
def test_msa_block_bias_after_norm(dev, precision, tol):
    """The dialect key ``opmBiasAfterNorm``: sum / max(count, 1) + bias (``cpu/af3/trunk/msa.js:141-150``); the two
    forms differ by about (1 - 1/count) * bias on every pair, far above either bound."""
    import localfold_b200 as lf
    from parity_report import record
    S, n = 12, 48
    msa, pair, mm, pm, w = syn.af3_msa_block(43, S=S, n=n)
    assert np.abs(np.asarray(w["outerProductMean"]["outputB"])).max() > 0
    dialect = {"swapTransposedBias": False, "msaUpdateBeforeOuterProduct": False, "opmBiasAfterNorm": True}
    got = lf.Af3MsaBlockGpu(dev).run({"msa": msa, "pair": pair, "msaMask": mm, "pairMask": pm, "sequences": S, "tokens": n},
                                     w, dialect, {"precision": precision})
    want_msa, want_pair = oracle.msa_block_af3(msa, pair, mm, pm, w, False, False, bias_after_norm=True)
    _, other_pair = oracle.msa_block_af3(msa, pair, mm, pm, w, False, False, bias_after_norm=False)
    assert oracle.relative_l2(other_pair, want_pair) > 10 * tol      # the option is visible on this input
    e_msa, e_pair = oracle.relative_l2(got["msa"], want_msa), oracle.relative_l2(got["pair"], want_pair)
    record("msa_block_af3", f"S={S} n={n} {precision} bias after norm msa", e_msa, tol)
    record("msa_block_af3", f"S={S} n={n} {precision} bias after norm pair", e_pair, tol)
    assert e_msa <= tol and e_pair <= tol


def test_msa_block_needs_its_dialect(dev):
    import localfold_b200 as lf
    msa, pair, mm, pm, w = syn.af3_msa_block(42, S=2, n=16)
    state = {"msa": msa, "pair": pair, "msaMask": mm, "pairMask": pm, "sequences": 2, "tokens": 16}
    with pytest.raises(ValueError, match="msaUpdateBeforeOuterProduct has no default"):
        lf.Af3MsaBlockGpu(dev).run(state, w, {"swapTransposedBias": False})


@pytest.mark.parametrize("with_bias", [False, True])
def test_distogram_logits(dev, with_bias):
    import localfold_b200 as lf
    rng = np.random.default_rng(9)
    n, cz, bins = 45, 128, 64
    pair = rng.standard_normal((n, n, cz)).astype(np.float32)
    w = (rng.standard_normal((cz, bins)) / np.sqrt(cz)).astype(np.float32)
    bias = rng.standard_normal(bins).astype(np.float32) if with_bias else None
    got = lf.distogram_logits(dev, pair, n, cz, w, bias)["output"]
    want = oracle.distogram_logits(pair, w, bias)
    assert oracle.relative_l2(got, want) <= F32_TOL
    assert np.abs(got - got.transpose(1, 0, 2)).max() == 0


def test_msa_stack_hands_the_pair_to_the_pairformer(dev):
    """Two MSA blocks, then one pairformer block on the same resident pair (``keepPair``), against the oracle's
    composition of the same blocks."""
    import localfold_b200 as lf
    S, n = 6, 32
    d = syn.draw(50)
    msa, pair = d.normal(S, n, 64), d.normal(n, n, 128)
    mm = (d.rng.random((S, n)) >= 0.2).astype(np.float32)
    mm[0] = 1
    pm = np.ones((n, n), np.float32)
    blocks = [syn.af3_msa_block_weights(d) for _ in range(2)]
    pf = syn.af3_pairformer_block_weights(d, 128, 384)
    dialect = {"swapTransposedBias": False, "msaUpdateBeforeOuterProduct": False}
    seen = []
    r = lf.Af3MsaStackGpu(dev).run({"msa": msa, "pair": pair, "msaMask": mm, "pairMask": pm, "sequences": S, "tokens": n},
                                   blocks, dialect, {"precision": "f32", "keepPair": True, "onBlock": seen.append})
    assert seen == [0, 1] and r["pair"] is None
    out = lf.Af3PairformerStackGpu(dev).run({"pair": r["pairTensor"], "single": None, "pairMask": pm, "tokens": n}, [pf],
                                            {"swapTransposedBias": False}, {"precision": "f32"})
    want_msa, want_pair = msa, pair
    for w in blocks:
        want_msa, want_pair = oracle.msa_block_af3(want_msa, want_pair, mm, pm, w, False, False)
    want_pair, _ = oracle.af3_pairformer_block(want_pair, None, pm, None, pf, False)
    got_pair = out["pair"].cpu().numpy() if hasattr(out["pair"], "cpu") else out["pair"]
    assert oracle.relative_l2(r["msaTensor"].cpu().numpy(), want_msa) <= 2e-5
    assert oracle.relative_l2(got_pair, want_pair) <= 2e-5


@pytest.mark.parametrize("S,n,c,heads,dim", [(64, 48, 64, 8, 8), (5, 33, 64, 8, 8), (300, 17, 32, 4, 16), (1, 8, 64, 8, 8)])
def test_global_column_attention_f32(dev, S, n, c, heads, dim):
    import localfold_b200 as lf
    from parity_report import record
    d = syn.draw(60 + S)
    msa = d.normal(S, n, c)
    mask = (d.rng.random((S, n)) >= 0.2).astype(np.float32)
    mask[0] = 1
    w = syn.af2_global_attention_weights(d, c, heads, dim)
    got = lf.GlobalColumnAttentionGpu(dev).run({"activations": msa, "mask": mask, "sequences": S, "length": n, "channels": c,
                                                "weights": w}, {"precision": "f32", "variance": "two-pass"})["output"]
    want = oracle.global_column_attention_af2(msa, mask, w)
    err = oracle.relative_l2(got, want)
    record("global_column_attention", f"S={S} n={n} c={c} heads={heads}x{dim}", err, F32_TOL)
    assert np.isfinite(got).all()
    assert err <= F32_TOL


def test_global_column_attention_column_with_no_sequence(dev):
    """A column no sequence covers: every logit is -1e9, the softmax is uniform, the query is 0 / 1e-10 = 0."""
    import localfold_b200 as lf
    d = syn.draw(70)
    S, n, c = 6, 12, 64
    msa = d.normal(S, n, c)
    mask = np.ones((S, n), np.float32)
    mask[:, 5] = 0
    w = syn.af2_global_attention_weights(d, c, 8, 8)
    got = lf.GlobalColumnAttentionGpu(dev).run({"activations": msa, "mask": mask, "sequences": S, "length": n, "channels": c,
                                                "weights": w}, {"precision": "f32", "variance": "two-pass"})["output"]
    want = oracle.global_column_attention_af2(msa, mask, w)
    assert np.isfinite(got).all()
    assert oracle.relative_l2(got, want) <= F32_TOL


def test_extra_msa_block_f32(dev):
    import localfold_b200 as lf
    from parity_report import record
    S, n = 24, 40
    msa, pair, mm, pm, w = syn.af2_extra_msa_block(80, S=S, n=n)
    got = lf.ExtraMsaBlockGpu(dev).run({"msa": msa, "pair": pair, "msaMask": mm, "pairMask": pm, "sequences": S, "length": n,
                                        "cM": 64, "cZ": 128, "cOuter": 32, "triangleHidden": 128, "weights": w},
                                       {"precision": "f32", "variance": "two-pass"})
    want_msa, want_pair = oracle.af2_extra_msa_block(msa, pair, mm, pm, w, 32, 128)
    e_msa, e_pair = oracle.relative_l2(got["msa"], want_msa), oracle.relative_l2(got["pair"], want_pair)
    record("extra_msa_block", f"S={S} n={n} f32 msa", e_msa, F32_TOL)
    record("extra_msa_block", f"S={S} n={n} f32 pair", e_pair, F32_TOL)
    assert e_msa <= F32_TOL and e_pair <= F32_TOL


def test_extra_msa_stack_two_blocks(dev):
    import localfold_b200 as lf
    S, n = 10, 24
    d = syn.draw(90)
    msa, pair, mm, pm, w0 = syn.af2_extra_msa_block(90, S=S, n=n)
    _, _, _, _, w1 = syn.af2_extra_msa_block(91, S=S, n=n)
    seen = []
    got = lf.ExtraMsaStackGpu(dev).run({"msa": msa, "pair": pair, "msaMask": mm, "pairMask": pm, "sequences": S, "length": n,
                                        "cM": 64, "cZ": 128, "cOuter": 32, "triangleHidden": 128, "blockWeights": [w0, w1],
                                        "onBlockDone": seen.append}, {"precision": "f32", "variance": "two-pass"})
    want_msa, want_pair = msa, pair
    for w in (w0, w1):
        want_msa, want_pair = oracle.af2_extra_msa_block(want_msa, want_pair, mm, pm, w, 32, 128)
    assert seen == [0, 1]
    assert oracle.relative_l2(got["msa"], want_msa) <= 3 * F32_TOL
    assert oracle.relative_l2(got["pair"], want_pair) <= 3 * F32_TOL
