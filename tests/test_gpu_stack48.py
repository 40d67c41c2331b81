"""48-block stacks (BASELINE configs 2 and 4 are 48-block stacks) against the CPU oracle at reduced N.

Three figures per stack, the way the reference judges multi-block runs
(``tools/gpu/check-af3-block.js:172-198, 258-268``): stacks of random-weight blocks amplify small
differences, so a free-running comparison alone says little.

* teacher-forced: every block is run on the oracle's input to that block; the per-block error must meet the
  per-block bound (2e-3) at every depth;
* free-running: the GPU stack runs all 48 blocks on its own output; the error against the oracle after 48;
* envelope: the oracle against itself with the input perturbed by 1e-7 relative - how much the stack
  amplifies a float32 rounding.  The free-running error must stay under max(1e-2, 20 x envelope).
"""
import numpy as np
import pytest

from localfold_b200 import synthetic as syn
from oracle import oracle
from parity_report import record

pytestmark = pytest.mark.gpu
BLOCKS = 48
BLOCK_TOL = 2e-3
STACK_TOL = 1e-2


@pytest.fixture(scope="module")
def dev():
    import localfold_b200 as lf
    d = lf.Device(0)
    yield d
    d.close()


def perturbed(x, seed):
    rng = np.random.default_rng(seed)
    return (x * (1.0 + 1e-7 * rng.standard_normal(x.shape))).astype(np.float32)


def test_af2_stack_48_blocks(dev):
    import localfold_b200 as lf
    n = 64
    pair, mask, weights = syn.af2_pair_block(4, n, blocks=BLOCKS)
    states = [pair]
    for b in range(BLOCKS):
        states.append(oracle.af2_pair_block(states[-1], mask, weights[b], 128))
    shadow = perturbed(pair, 1)
    for b in range(BLOCKS):
        shadow = oracle.af2_pair_block(shadow, mask, weights[b], 128)
    envelope = oracle.relative_l2(shadow, states[-1])
    stack = lf.PairStackGpu(dev).prepare(weights, 128, 128)
    opts = {"precision": "bf16", "variance": "two-pass"}
    worst = 0.0
    for b in range(BLOCKS):
        got = stack.run(states[b], mask, opts, first_block=b, n_blocks=1)["pair"]
        worst = max(worst, oracle.relative_l2(got, states[b + 1]))
    free = stack.run(pair, mask, opts)
    assert free["blocks"] == BLOCKS
    free_err = oracle.relative_l2(free["pair"], states[-1])
    f32 = stack.run(pair, mask, {"precision": "f32", "variance": "two-pass"})
    f32_err = oracle.relative_l2(f32["pair"], states[-1])
    stack.close()
    record("af2_stack48", "teacher-forced worst block, n=64", worst, BLOCK_TOL)
    record("af2_stack48", "free-running after 48, n=64", free_err, max(STACK_TOL, 20 * envelope), envelope=envelope)
    record("af2_stack48", "free-running after 48, f32 mode, n=64", f32_err, max(1e-4, 20 * envelope), envelope=envelope)
    assert np.isfinite(free["pair"]).all()
    assert worst <= BLOCK_TOL
    assert free_err <= max(STACK_TOL, 20 * envelope)
    assert f32_err <= max(1e-4, 20 * envelope)


def test_af3_stack_48_blocks_int5(dev):
    """Config 2 at reduced N: 48 AF3 pairformer blocks (pair and single tracks), int5-format weights."""
    import localfold_b200 as lf
    from bundle_writer import quantise_weights_like_bundle
    n = 48
    pair, single, pair_mask, seq_mask, blocks = syn.af3_pairformer(2, n, 128, 384, blocks=BLOCKS)
    blocks = [quantise_weights_like_bundle(b) for b in blocks]
    states = [(pair, single)]
    for b in range(BLOCKS):
        states.append(oracle.af3_pairformer_block(states[-1][0], states[-1][1], pair_mask, seq_mask, blocks[b], True))
    sp, ss = perturbed(pair, 2), perturbed(single, 3)
    for b in range(BLOCKS):
        sp, ss = oracle.af3_pairformer_block(sp, ss, pair_mask, seq_mask, blocks[b], True)
    env_pair, env_single = oracle.relative_l2(sp, states[-1][0]), oracle.relative_l2(ss, states[-1][1])
    runner = lf.Af3PairformerStackGpu(dev)
    dialect = {"swapTransposedBias": True}
    worst_p = worst_s = 0.0
    for b in range(BLOCKS):
        got = runner.run({"pair": states[b][0], "single": states[b][1], "pairMask": pair_mask, "seqMask": seq_mask,
                          "tokens": n}, blocks[b:b + 1], dialect, {"precision": "bf16"})
        worst_p = max(worst_p, oracle.relative_l2(got["pair"], states[b + 1][0]))
        worst_s = max(worst_s, oracle.relative_l2(got["single"], states[b + 1][1]))
    free = runner.run({"pair": pair, "single": single, "pairMask": pair_mask, "seqMask": seq_mask, "tokens": n},
                      blocks, dialect, {"precision": "bf16"})
    free_p = oracle.relative_l2(free["pair"], states[-1][0])
    free_s = oracle.relative_l2(free["single"], states[-1][1])
    record("af3_stack48", "teacher-forced worst block (pair), n=48", worst_p, BLOCK_TOL)
    record("af3_stack48", "teacher-forced worst block (single), n=48", worst_s, BLOCK_TOL)
    record("af3_stack48", "free-running pair after 48", free_p, max(STACK_TOL, 20 * env_pair), envelope=env_pair)
    record("af3_stack48", "free-running single after 48", free_s, max(STACK_TOL, 20 * env_single), envelope=env_single)
    assert np.isfinite(free["pair"]).all() and np.isfinite(free["single"]).all()
    assert worst_p <= BLOCK_TOL and worst_s <= BLOCK_TOL
    assert free_p <= max(STACK_TOL, 20 * env_pair)
    assert free_s <= max(STACK_TOL, 20 * env_single)
