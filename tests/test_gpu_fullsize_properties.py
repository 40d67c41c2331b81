"""Full-size checks (N = 2048, the benchmark's length) through properties that do not need the oracle
to run at that size.

* Relabelling the residues (a permutation P applied to both pair indices and to the mask) must
  relabel the result: op(P z P^T) = P op(z) P^T.  The two runs walk the tiles in different orders,
  so agreement to the 16-bit path's rounding means no tile, ragged edge or ring slot is mishandled.
* The incoming triangle update equals the outgoing one on the transposed pair, transposed back
  (different tensor-core operand layouts for the same sums), and the ending-node attention equals the
  starting-node attention on the transposed pair.
* The pair transition is row-local, so a sample of rows of the full-size result is checked against
  the CPU oracle run on just those rows.

Everything stays on the device; the inputs are seeded.
"""
import numpy as np
import pytest
import torch

from localfold_b200 import synthetic as syn
from oracle import oracle

pytestmark = pytest.mark.gpu

N = 2048
OPTS = {"precision": "bf16", "variance": "two-pass"}


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    d = lf.Device(0, stream=torch.cuda.current_stream().cuda_stream)   # the inputs are made by torch on that stream
    yield d
    d.close()


@pytest.fixture(scope="module")
def pair():
    g = torch.Generator(device="cuda").manual_seed(2048)
    z = torch.randn((N, N, 128), generator=g, device="cuda", dtype=torch.float32)
    mask = (torch.rand((N, N), generator=g, device="cuda") > 0.05).to(torch.float32)
    perm = torch.randperm(N, generator=g, device="cuda")
    return z, mask, perm


def rel_l2(a, b):
    return float(torch.linalg.vector_norm((a - b).double()) / torch.linalg.vector_norm(b.double()))


def relabel(t, perm):
    return t.index_select(0, perm).index_select(1, perm).contiguous()


def run_triangle(dev, z, mask, w, incoming):
    import localfold_b200 as lf
    op = (lf.TriangleMultiplicationIncomingGpu if incoming else lf.TriangleMultiplicationOutgoingGpu)(dev)
    out = torch.empty_like(z)
    op.run({"shape": {"length": z.shape[0], "cZ": 128, "cHidden": 128}, "z": z, "mask": mask, "weights": w}, OPTS, out=out)
    dev.synchronize()
    return out


def run_attention(dev, z, mask, w, pb, transpose):
    import localfold_b200 as lf
    out = torch.empty_like(z)
    n = z.shape[0]
    lf.AttentionGpu(dev).run({"activations": z, "mask": mask, "batch": n, "queryLength": n, "channels": 128, "heads": 4,
                              "transpose": transpose, "weights": w, "pairBias": pb}, OPTS, out=out)
    dev.synchronize()
    return out


@pytest.mark.parametrize("incoming", [False, True])
def test_triangle_relabelling_fullsize(dev, pair, incoming):
    z, mask, perm = pair
    w = syn.af2_triangle_weights(syn.draw(77), 128, 128)
    base = run_triangle(dev, z, mask, w, incoming)
    assert bool(torch.isfinite(base).all())
    moved = run_triangle(dev, relabel(z, perm), relabel(mask, perm), w, incoming)
    assert rel_l2(moved, relabel(base, perm)) <= 2e-3


def test_triangle_incoming_is_outgoing_of_transpose_fullsize(dev, pair):
    z, mask, _ = pair
    w = syn.af2_triangle_weights(syn.draw(78), 128, 128)
    incoming = run_triangle(dev, z, mask, w, True)
    zt = z.transpose(0, 1).contiguous()
    outgoing_t = run_triangle(dev, zt, mask.t().contiguous(), w, False)
    assert rel_l2(incoming, outgoing_t.transpose(0, 1)) <= 2e-3


@pytest.mark.parametrize("transpose", [False, True])
def test_attention_relabelling_fullsize(dev, pair, transpose):
    z, mask, perm = pair
    t = syn.af2_attention_weights(syn.draw(79), 128, 4, 128)
    pb = dict(t["pairBias"], source="normalized-input")
    base = run_attention(dev, z, mask, t["attention"], pb, transpose)
    assert bool(torch.isfinite(base).all())
    moved = run_attention(dev, relabel(z, perm), relabel(mask, perm), t["attention"], pb, transpose)
    assert rel_l2(moved, relabel(base, perm)) <= 2e-3


def test_attention_ending_is_starting_of_transpose_fullsize(dev, pair):
    z, mask, _ = pair
    t = syn.af2_attention_weights(syn.draw(80), 128, 4, 128)
    pb = dict(t["pairBias"], source="normalized-input")
    ending = run_attention(dev, z, mask, t["attention"], pb, True)
    # the ending node attends along columns: the starting node on the transposed pair, transposed back,
    # with the bias taken from the transposed pair as well (which is what the AF2 ending node does)
    starting_t = run_attention(dev, z.transpose(0, 1).contiguous(), mask.t().contiguous(), t["attention"], pb, False)
    assert rel_l2(ending, starting_t.transpose(0, 1)) <= 2e-3


def test_transition_rows_against_oracle_fullsize(dev, pair):
    import localfold_b200 as lf
    z, _, _ = pair
    d = syn.draw(81)
    w = syn.af2_transition_weights(d, 128, 4)
    rows = z.reshape(N * N, 128)
    out = torch.empty_like(rows)
    lf.TransitionGpu(dev).run({"activations": rows, "rows": N * N, "channels": 128, "hiddenChannels": 512, "weights": w},
                              OPTS, out=out)
    dev.synchronize()
    g = torch.Generator(device="cuda").manual_seed(5)
    pick = torch.randint(0, N * N, (4096,), generator=g, device="cuda")
    got = out.index_select(0, pick).cpu().numpy()
    sample = rows.index_select(0, pick).cpu().numpy()
    want = oracle.transition_af2(sample, w, 512)
    assert np.isfinite(got).all()
    assert oracle.relative_l2(got, want) <= 8e-3


def test_pair_block_relabelling_fullsize(dev, pair):
    """The whole AF2 pair block (13 launches) commutes with a relabelling of the residues."""
    import localfold_b200 as lf
    z, mask, perm = pair
    _, _, weights = syn.af2_pair_block(4, 16, blocks=1)      # the weights do not depend on the length
    stack = lf.PairStackGpu(dev).prepare(weights, 128, 128)
    base = z.clone()
    stack.run(base, mask, OPTS, first_block=0, n_blocks=1)
    moved = relabel(z, perm)
    stack.run(moved, relabel(mask, perm), OPTS, first_block=0, n_blocks=1)
    dev.synchronize()
    stack.close()
    assert bool(torch.isfinite(base).all())
    assert rel_l2(moved, relabel(base, perm)) <= 2e-3


def test_context_with_its_own_stream_waits_for_torch_inputs(dev, pair):
    """A context that runs on a stream of its own is handed a tensor that torch is still producing (a 2 GB gather
    enqueued just before the call): the library orders its stream after torch's, so the result is the one computed
    from the finished tensor."""
    import localfold_b200 as lf
    z, _, perm = pair
    w = syn.af2_transition_weights(syn.draw(82), 128, 4)
    own = lf.Device(0)                       # a stream of its own
    try:
        moved = relabel(z, perm)             # torch's stream, not waited for here
        got = torch.empty((N * N, 128), device="cuda")
        lf.TransitionGpu(own).run({"activations": moved.reshape(N * N, 128), "rows": N * N, "channels": 128,
                                   "hiddenChannels": 512, "weights": w}, OPTS, out=got)
        own.synchronize()
        torch.cuda.synchronize()
        want = torch.empty_like(got)
        lf.TransitionGpu(dev).run({"activations": moved.reshape(N * N, 128), "rows": N * N, "channels": 128,
                                   "hiddenChannels": 512, "weights": w}, OPTS, out=want)
        dev.synchronize()
        assert torch.equal(got, want)
    finally:
        own.close()
