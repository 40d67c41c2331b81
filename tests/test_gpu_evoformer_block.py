"""BASELINE config 1: one whole AF2 Evoformer block through ``EvoformerBlockGpu`` - MSA row attention with
pair bias (8 heads x 32, ``pairBias.source = "separate"``), MSA column attention, MSA transition,
OuterProductMean (c = 32), then the five pair updates - against the CPU oracle's block
(``webgpu/af2/evoformer/block.js:1546-1612``), c_m = 256, c_z = 128, a tenth of the MSA rows masked.

MSA rows that are masked out entirely take a uniform softmax in the row attention (every key is masked:
the float32 logits collapse to one value); their outputs never reach the pair (the outer product
multiplies by the mask) but they are part of the returned MSA, so MSA parity is reported on all rows and
on the unmasked rows separately.
"""
import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle
from parity_report import record

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    d = lf.Device(0)
    yield d
    d.close()


_WANT = {}


def block_input(S, n):
    msa, pair, msa_mask, pair_mask, w = syn.af2_evoformer_block(1, S=S, n=n)
    inp = {"msa": msa, "pair": pair, "msaMask": msa_mask, "pairMask": pair_mask, "sequences": S, "length": n,
           "cM": 256, "cZ": 128, "cOuter": 32, "triangleHidden": 128, "weights": w}
    return inp, msa_mask


@pytest.mark.parametrize("S,n", [(16, 40), (128, 96), (128, 256)])      # the last is configuration 1 in full
@pytest.mark.parametrize("precision,tol", [("f32", 1e-5), ("bf16", 2e-3)])
def test_evoformer_block(dev, S, n, precision, tol):
    import localfold_b200 as lf
    inp, msa_mask = block_input(S, n)
    if (S, n) not in _WANT:        # both precisions are checked against one oracle run
        _WANT[(S, n)] = oracle.af2_evoformer_block(inp["msa"], inp["pair"], inp["msaMask"], inp["pairMask"],
                                                   inp["weights"], 32, 128)
    want_msa, want_pair = _WANT[(S, n)]
    got = lf.EvoformerBlockGpu(dev).run(inp, {"precision": precision, "variance": "two-pass"})
    assert np.isfinite(got["msa"]).all() and np.isfinite(got["pair"]).all()
    live = msa_mask[:, 0] > 0
    assert 0 < live.sum() < S          # some rows are masked
    err_pair = oracle.relative_l2(got["pair"], want_pair)
    err_msa = oracle.relative_l2(got["msa"], want_msa)
    err_live = oracle.relative_l2(got["msa"][live], want_msa[live])
    for case, err in (("pair", err_pair), ("msa all rows", err_msa), ("msa unmasked rows", err_live)):
        record("evoformer_block", f"S={S} n={n} {precision} {case}", err, tol)
    assert err_pair <= tol
    assert err_msa <= tol
    assert err_live <= tol
    assert got["launches"] > 0
