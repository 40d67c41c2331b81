"""The benchmarked sizes against an oracle: N = 512, 1024, 2048 (BASELINE config 3's sweep and config 4's
length), 16-bit tensor-core path.

A whole-tensor oracle would take minutes at these lengths, so the float64 formulation
(``oracle/tier2_torch.py``) computes a sample of output positions - rows and columns spread over the
tensor, some of them inside the masked tail - from exactly the inputs those positions depend on, and the
GPU result is compared there.  Unlike the relabelling properties this catches an error that commutes with
a permutation (a softmax scale, a rescale step at long rows, range loss of fp16 operands at N = 2048).

Tolerance: 8e-3 relative L2 per operator, the reference's bound for its half-precision arms
(``tools/gpu/check-triangle.js:59``, ``tools/gpu/check-evoformer-attention.js:162``).
"""
import numpy as np
import pytest
import torch

from localfold_b200 import synthetic as syn
from oracle import oracle, tier2_torch as t2
from parity_report import record

pytestmark = pytest.mark.gpu
OPTS = {"precision": "bf16", "variance": "two-pass"}
OP_TOL = 8e-3


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    d = lf.Device(0, stream=torch.cuda.current_stream().cuda_stream)   # the inputs are made by torch on that stream
    yield d
    d.close()


def make_pair(n, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    z = torch.randn((n, n, 128), generator=g, device="cuda", dtype=torch.float32)
    mask = torch.from_numpy(syn.residue_pair_mask(n, 0.05)).cuda()     # last 5 % of residues masked
    return z, mask


def sample_indices(n, seed, count):
    """Positions spread over the tensor: both ends, tile edges, the masked tail, and random ones."""
    rng = np.random.default_rng(seed)
    fixed = [0, 1, 127, 128, n // 2 - 1, n // 2, n - 1, n - 2, n - n // 40]
    extra = rng.choice(n, size=max(0, count - len(fixed)), replace=False)
    return np.unique(np.array(fixed + list(extra)) % n)


@pytest.mark.parametrize("n", [512, 1024, 2048])
@pytest.mark.parametrize("incoming", [False, True])
def test_triangle_positions_against_float64(dev, n, incoming):
    import localfold_b200 as lf
    z, mask = make_pair(n, 3000 + n)
    w = syn.af2_triangle_weights(syn.draw(3), 128, 128)
    op = (lf.TriangleMultiplicationIncomingGpu if incoming else lf.TriangleMultiplicationOutgoingGpu)(dev)
    out = torch.empty_like(z)
    op.run({"shape": {"length": n, "cZ": 128, "cHidden": 128}, "z": z, "mask": mask, "weights": w}, OPTS, out=out)
    dev.synchronize()
    assert bool(torch.isfinite(out).all())
    rows, cols = sample_indices(n, 1, 12), sample_indices(n, 2, 48)
    got = out[torch.from_numpy(rows).cuda()][:, torch.from_numpy(cols).cuda()].cpu().numpy()
    want = t2.trimul_af2_positions(z.cpu().numpy(), mask.cpu().numpy(), w, rows, cols, 1e-5, incoming)
    err = oracle.relative_l2(got, want)
    record("triangle_positions", f"n={n} incoming={incoming}", err, OP_TOL)
    assert err <= OP_TOL


@pytest.mark.parametrize("n", [1024, 2048])
@pytest.mark.parametrize("transpose", [False, True])
def test_attention_positions_against_float64(dev, n, transpose):
    import localfold_b200 as lf
    z, mask = make_pair(n, 4000 + n)
    t = syn.af2_attention_weights(syn.draw(4), 128, 4, 128)
    pb = dict(t["pairBias"], source="normalized-input")
    out = torch.empty_like(z)
    lf.AttentionGpu(dev).run({"activations": z, "mask": mask, "batch": n, "queryLength": n, "channels": 128, "heads": 4,
                              "transpose": transpose, "weights": t["attention"], "pairBias": pb}, OPTS, out=out)
    dev.synchronize()
    assert bool(torch.isfinite(out).all())
    brows, queries = sample_indices(n, 5, 10), sample_indices(n, 6, 40)
    want = t2.attention_af2_positions(z.cpu().numpy(), mask.cpu().numpy(), n, 128, 4, t["attention"], brows, queries,
                                      transpose, pb["projectionWeight"])
    bi, qi = torch.from_numpy(brows).cuda(), torch.from_numpy(queries).cuda()
    if transpose:      # logical (b, q) lives at memory (q, b)
        got = out[qi][:, bi].transpose(0, 1).cpu().numpy()
    else:
        got = out[bi][:, qi].cpu().numpy()
    err = oracle.relative_l2(got, want)
    record("attention_positions", f"n={n} transpose={transpose}", err, OP_TOL)
    assert err <= OP_TOL
