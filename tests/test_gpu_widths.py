"""The same graph at the other widths the reference ships (``docs/ARCHITECTURE.md:149-167``): OpenDDE's 384
pair channels with 12 heads, IntelliFold-2's 512, ESMFold2's 256 (triangle updates and transition, no grid
attention), a 64-channel track; and the rf3 dialect bits of the triangle update (divide by the length; gate
and output biases on the grid attention).  In float32 mode these widths run on the generic float32 kernels (bound 2e-5); in 16-bit mode the
triangle contraction still runs on the tensor cores with fp16 operands at any width, so the per-block 16-bit
bound applies there."""
import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 2e-5


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    d = lf.Device(0)
    yield d
    d.close()


@pytest.mark.parametrize("cz,heads,precision", [(384, 12, "f32"), (384, 12, "bf16"), (512, 16, "f32"), (256, 8, "f32"), (64, 2, "bf16")])
def test_af3_pairformer_block_at_other_widths(dev, cz, heads, precision):
    import localfold_b200 as lf
    from parity_report import record
    n = 20
    d = syn.draw(900 + cz)
    pair = d.normal(n, n, cz)
    single = d.normal(n, 96)
    mask = syn.residue_pair_mask(n, 0.1)
    seq_mask = np.ones(n, np.float32)
    w = syn.af3_pairformer_block_weights(d, cz, 96, heads, 4)
    got = lf.Af3PairformerStackGpu(dev).run({"pair": pair, "single": single, "pairMask": mask, "seqMask": seq_mask, "tokens": n},
                                            [w], {"swapTransposedBias": False}, {"precision": precision})
    want_pair, want_single = oracle.af3_pairformer_block(pair, single, mask, seq_mask, w, False)
    e_pair, e_single = oracle.relative_l2(got["pair"], want_pair), oracle.relative_l2(got["single"], want_single)
    bound = TOL if precision == "f32" else 2e-3
    record("af3_pairformer_block_widths", f"cz={cz} heads={heads} {precision} pair", e_pair, bound)
    record("af3_pairformer_block_widths", f"cz={cz} heads={heads} {precision} single", e_single, bound)
    assert e_pair <= bound and e_single <= bound


@pytest.mark.parametrize("cz", [256, 384])
def test_triangle_update_divided_by_length(dev, cz):
    """rf3's ``triangleMulDivideByLength`` (``cpu/af3/trunk/pairformer.js:253-267``)."""
    import localfold_b200 as lf
    n = 24
    d = syn.draw(950 + cz)
    pair = d.normal(n, n, cz)
    mask = syn.residue_pair_mask(n, 0.1)
    w = syn.af3_triangle_weights(d, cz)
    for direction in ("outgoing", "incoming"):
        got = lf.af3_triangle_multiplication(dev, pair, mask, n, cz, direction, w, {"precision": "f32", "divideByLength": True})["output"]
        want = oracle.trimul_af3(pair, mask, w, direction == "incoming", True)
        assert oracle.relative_l2(got, want) <= TOL


def test_grid_attention_with_gate_and_output_biases(dev):
    """rf3's biased gate and output projection of the grid attention (``cpu/af3/trunk/pairformer.js:397-408``)."""
    import localfold_b200 as lf
    n, cz, heads = 22, 256, 8
    d = syn.draw(960)
    pair = d.normal(n, n, cz)
    mask = syn.residue_pair_mask(n, 0.1)
    w = syn.af3_grid_attention_weights(d, cz, heads, cz // heads)
    w["gatingQueryBias"] = d.normal(cz, std=0.3)
    w["outputProjectionBias"] = d.normal(cz, std=0.3)
    for transpose in (False, True):
        got = lf.Af3GridSelfAttentionGpu(dev).run(pair, mask, {"n": n, "channels": cz, "transpose": transpose}, w,
                                                  {"swapTransposedBias": True}, {"precision": "f32"})["output"]
        want = oracle.grid_attention_af3(pair, mask, w, transpose, True)
        assert oracle.relative_l2(got, want) <= TOL
