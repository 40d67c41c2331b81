"""The pair stack with the pair left in host memory: when the scratch arena for the resident path is
refused (here by a limit set on the context - no allocation is made to fail), ``lf_pair_stack_run`` keeps a
host-space pair in the caller's buffer and streams it through the device in chunks of rows (columns for the
ending-node attention).  The result must be the resident path's, and the oracle's within the per-block bound."""
import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle
from parity_report import record

pytestmark = pytest.mark.gpu
OPTS = {"precision": "bf16", "variance": "two-pass"}


@pytest.mark.parametrize("n,blocks", [(96, 1), (80, 2)])
def test_af2_block_with_the_pair_on_the_host(n, blocks):
    import localfold_b200 as lf
    dev = lf.Device(0)
    pair, mask, weights = syn.af2_pair_block(120 + n, n, blocks=blocks, masked_tail=0.1)
    want = pair
    for w in weights:
        want = oracle.af2_pair_block(want, mask, w, 128)
    stack = lf.PairStackGpu(dev).prepare(weights, 128, 128)
    resident = stack.run(pair, mask, OPTS)
    # room for the fp16 triangle operands and a few rows of everything else, not for the pair and its scratch
    resident_bytes = 3 * n * n * 256 + n * n * 8
    dev.release_scratch()
    dev.limit_scratch(resident_bytes + 16 * n * (2 * 516 + 5 * 256) + (1 << 16))
    spilled = stack.run(pair, mask, OPTS)
    dev.limit_scratch(0)
    stack.close()
    dev.close()
    assert spilled["launches"] > resident["launches"]          # several chunks per pass
    assert np.isfinite(spilled["pair"]).all()
    err = oracle.relative_l2(spilled["pair"], want)
    record("host_resident_pair", f"af2 n={n} blocks={blocks} vs oracle", err, 2e-3 * blocks)
    record("host_resident_pair", f"af2 n={n} blocks={blocks} vs resident path", oracle.relative_l2(spilled["pair"], resident["pair"]), 1e-6)
    assert err <= 2e-3 * blocks
    assert oracle.relative_l2(spilled["pair"], resident["pair"]) <= 1e-6


def test_af3_block_with_the_pair_on_the_host():
    import localfold_b200 as lf
    dev = lf.Device(0)
    n = 64
    pair, _, pair_mask, _, blocks = syn.af3_pairformer(130, n, 128, 384, blocks=1)
    pair_mask = (np.random.default_rng(1).random((n, n)) > 0.1).astype(np.float32)
    want, _ = oracle.af3_pairformer_block(pair, None, pair_mask, None, blocks[0], True)
    stack = lf.PairStackGpu(dev).prepare(blocks, 128, 128)
    opts = {"precision": "bf16"}
    dev.limit_scratch(3 * n * n * 256 + n * n * 8 + 16 * n * (2 * 516 + 5 * 256) + (1 << 16))
    got = stack.run(pair, pair_mask, opts, dialect={"swapTransposedBias": True})
    with pytest.raises(MemoryError):       # the non-swapped transposed bias is not covered: the refusal stands
        stack.run(pair, pair_mask, opts, dialect={"swapTransposedBias": False})
    dev.limit_scratch(0)
    stack.close()
    dev.close()
    assert oracle.relative_l2(got["pair"], want) <= 2e-3


def test_pipeline_of_host_pairs_matches_one_at_a_time():
    """``PairStackPipeline``: several host pairs in flight on one GPU, a context per lane; every pair's result is
    that of its own one-at-a-time call."""
    import torch
    import localfold_b200 as lf
    n, jobs = 96, 5
    pair, mask, blocks = syn.af2_pair_block(77, n, blocks=2)
    opts = {"precision": "bf16", "variance": "two-pass"}
    dev = lf.Device(0)
    stack = lf.PairStackGpu(dev).prepare(blocks, 128, 128)
    want = []
    for i in range(jobs):
        z = np.array(pair * (1.0 + 0.1 * i), np.float32)
        stack.run(z, mask, opts, inplace=True)
        want.append(z)
    stack.close()
    dev.close()
    pinned = [torch.from_numpy(np.array(pair * (1.0 + 0.1 * i), np.float32)).pin_memory() for i in range(jobs)]
    arrays = [p.numpy() for p in pinned]
    pipe = lf.PairStackPipeline(blocks, 128, 128, lanes=3)
    results = pipe.run_many(arrays, [mask] * jobs, opts)
    pipe.close()
    assert len(results) == jobs and all(r["launches"] > 0 for r in results)
    for got, ref in zip(arrays, want):
        assert np.array_equal(got, ref)
    with pytest.raises(ValueError):
        lf.PairStackPipeline(blocks, 128, 128, lanes=2).run_many([arrays[0], arrays[0]], [mask, mask], opts)
