"""bf16 storage of the pair stream (BASELINE config 4's "bf16 pair"): every operator of the 16-bit path
and one AF2 block with ``torch.bfloat16`` pair tensors, against the CPU oracle run on the same
bf16-rounded input.

What bf16 storage costs is known in advance: writing a float32 result to bf16 is a relative rounding of
up to 2^-9, 1.7e-3 relative L2 on its own.  So an operator's update (written once) stays inside the
per-operator bound of 8e-3, while a block writes the running pair five times and cannot meet the 2e-3
that the float32 stream meets: its bound here is 6e-3, and the measured value is recorded.  The float32
stream is the default for that reason; bf16 halves the pair's memory at this price.
"""
import numpy as np
import pytest
import torch

from localfold_b200 import synthetic as syn
from oracle import oracle
from parity_report import record

pytestmark = pytest.mark.gpu
OPTS = {"precision": "bf16", "variance": "two-pass"}
OP_TOL = 8e-3
BLOCK_TOL_BF16_STREAM = 6e-3


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    d = lf.Device(0, stream=torch.cuda.current_stream().cuda_stream)   # the inputs are made by torch on that stream
    yield d
    d.close()


def as_bf16(a):
    """(device bf16 tensor, the same values as float32 numpy for the oracle)"""
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda().to(torch.bfloat16)
    return t, t.float().cpu().numpy()


@pytest.mark.parametrize("n", [64, 203])
@pytest.mark.parametrize("incoming", [False, True])
def test_triangle_bf16_stream(dev, n, incoming):
    import localfold_b200 as lf
    d = syn.draw(1300 + n)
    z, z32 = as_bf16(d.normal(n, n, 128))
    mask = syn.residue_pair_mask(n, 0.05)
    w = syn.af2_triangle_weights(d, 128, 128)
    op = (lf.TriangleMultiplicationIncomingGpu if incoming else lf.TriangleMultiplicationOutgoingGpu)(dev)
    out = torch.empty_like(z)
    op.run({"shape": {"length": n, "cZ": 128, "cHidden": 128}, "z": z, "mask": torch.from_numpy(mask).cuda(), "weights": w},
           OPTS, out=out)
    dev.synchronize()
    assert out.dtype == torch.bfloat16
    err = oracle.relative_l2(out.float().cpu().numpy(), oracle.trimul_af2(z32, mask, w, 128, 1e-5, incoming))
    record("triangle_bf16_stream", f"n={n} incoming={incoming}", err, OP_TOL)
    assert err <= OP_TOL


def test_triangle_bf16_stream_in_place_residual(dev):
    """The block form: the update is added into z, which is also the output buffer."""
    import localfold_b200 as lf
    n = 96
    d = syn.draw(1400)
    z, z32 = as_bf16(d.normal(n, n, 128))
    mask = syn.residue_pair_mask(n, 0.05)
    w = syn.af2_triangle_weights(d, 128, 128)
    lf.TriangleMultiplicationOutgoingGpu(dev).run(
        {"shape": {"length": n, "cZ": 128, "cHidden": 128}, "z": z, "mask": torch.from_numpy(mask).cuda(), "weights": w},
        dict(OPTS, residual=True), out=z)
    dev.synchronize()
    want = z32 + oracle.trimul_af2(z32, mask, w, 128, 1e-5, False)
    err = oracle.relative_l2(z.float().cpu().numpy(), want)
    record("triangle_bf16_stream", "in-place residual n=96", err, 3e-3)
    assert err <= 3e-3      # one bf16 rounding of the sum (1.7e-3) plus the 16-bit operands


@pytest.mark.parametrize("n", [64, 203])
@pytest.mark.parametrize("transpose", [False, True])
def test_triangle_attention_bf16_stream(dev, n, transpose):
    import localfold_b200 as lf
    d = syn.draw(1500 + n)
    z, z32 = as_bf16(d.normal(n, n, 128))
    mask = syn.residue_pair_mask(n, 0.1)
    t = syn.af2_attention_weights(d, 128, 4, 128)
    pb = dict(t["pairBias"], source="normalized-input")
    out = torch.empty_like(z)
    lf.AttentionGpu(dev).run({"activations": z, "mask": torch.from_numpy(mask).cuda(), "batch": n, "queryLength": n,
                              "channels": 128, "heads": 4, "transpose": transpose, "weights": t["attention"],
                              "pairBias": pb}, OPTS, out=out)
    dev.synchronize()
    want = oracle.attention_af2(z32, mask, n, n, 128, 4, t["attention"], transpose, pb)
    err = oracle.relative_l2(out.float().cpu().numpy(), want)
    record("attention_bf16_stream", f"n={n} transpose={transpose}", err, OP_TOL)
    assert err <= OP_TOL


@pytest.mark.parametrize("rows", [128, 5000])
@pytest.mark.parametrize("af3", [False, True])
def test_transition_bf16_stream(dev, rows, af3):
    import localfold_b200 as lf
    d = syn.draw(1600 + rows)
    act, act32 = as_bf16(d.normal(rows, 128))
    out = torch.empty_like(act)
    if af3:
        w = syn.af3_transition_weights(d, 128, 4)
        lf.Af3TransitionGpu(dev).run(act, {"rows": rows, "channels": 128, "factor": 4}, w, {"precision": "bf16"}, out=out)
        want = oracle.transition_af3(act32, w, 4)
    else:
        w = syn.af2_transition_weights(d, 128, 4)
        lf.TransitionGpu(dev).run({"activations": act, "rows": rows, "channels": 128, "hiddenChannels": 512, "weights": w},
                                  OPTS, out=out)
        want = oracle.transition_af2(act32, w, 512)
    dev.synchronize()
    err = oracle.relative_l2(out.float().cpu().numpy(), want)
    record("transition_bf16_stream", f"rows={rows} af3={af3}", err, OP_TOL)
    assert err <= OP_TOL


@pytest.mark.parametrize("n", [64, 203])
def test_af2_pair_block_bf16_stream(dev, n):
    import localfold_b200 as lf
    pair, mask, weights = syn.af2_pair_block(40 + n, n, masked_tail=0.05)
    z, z32 = as_bf16(pair)
    want = oracle.af2_pair_block(z32, mask, weights[0], 128)
    stack = lf.PairStackGpu(dev).prepare(weights, 128, 128)
    stack.run(z, torch.from_numpy(mask).cuda(), OPTS)
    dev.synchronize()
    stack.close()
    err = oracle.relative_l2(z.float().cpu().numpy(), want)
    record("af2_pair_block_bf16_stream", f"n={n}", err, BLOCK_TOL_BF16_STREAM)
    assert err <= BLOCK_TOL_BF16_STREAM
