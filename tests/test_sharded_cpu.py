"""The row-sharded pair stack on CPU: gloo ranks run ``ShardedPairStack`` with float64 CPU steps and must
reproduce the unsharded oracle block (checks the transposes, the gathers, incoming-as-outgoing on the
transposed shard and ending-as-starting attention with the transposed mask), in both forms of the triangle
multiplication: row-sharded with gathered b, and channel-sharded with the operands and the product
exchanged (what the GPU path does with stores into the peers' memory)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n, result_path, exchange):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from localfold_b200 import synthetic as syn
    from localfold_b200.sharded import ShardedPairStack, TorchComm, shard_rows
    from sharded_cpu_ops import CpuShardOps, block_weights

    pair, mask, weights = syn.af2_pair_block(11, n, 16, 16, 2, blocks=2, masked_tail=0.2)
    z = torch.from_numpy(np.ascontiguousarray(shard_rows(pair, rank, world))).double()
    m_rows = torch.from_numpy(np.ascontiguousarray(shard_rows(mask, rank, world))).double()
    m_t_rows = torch.from_numpy(np.ascontiguousarray(shard_rows(np.ascontiguousarray(mask.T), rank, world))).double()
    stack = ShardedPairStack(TorchComm(), CpuShardOps(n // world, n, world), exchange=True if exchange else None)
    z = stack.run(z, m_rows, m_t_rows, [block_weights(w) for w in weights])
    gathered = [torch.empty_like(z) for _ in range(world)]
    dist.all_gather(gathered, z)
    if rank == 0:
        np.save(result_path, torch.cat(gathered, 0).numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("exchange", [False, True])       # True: channel-sharded triangle multiplication
@pytest.mark.parametrize("world", [2, 4])
def test_sharded_stack_matches_unsharded_oracle(tmp_path, world, exchange):
    sys.path.insert(0, ROOT)
    from localfold_b200 import synthetic as syn
    from oracle import oracle
    n = 16
    port = 29600 + world + 10 * int(exchange) + os.getpid() % 200
    result = str(tmp_path / "pair.npy")
    mp.spawn(_worker, args=(world, port, n, result, exchange), nprocs=world, join=True)
    got = np.load(result)
    pair, mask, weights = syn.af2_pair_block(11, n, 16, 16, 2, blocks=2, masked_tail=0.2)
    want = pair
    for w in weights:
        want = oracle.af2_pair_block(want, mask, w, 16)
    assert oracle.relative_l2(got, want) < 5e-6


def test_transpose_shard_single_rank_is_a_transpose():
    from localfold_b200.sharded import transpose_shard

    class One:
        world, rank = 1, 0
        def all_to_all(self, t):
            return t
    z = torch.arange(4 * 4 * 3, dtype=torch.float64).reshape(4, 4, 3)
    assert torch.equal(transpose_shard(One(), z), z.transpose(0, 1))
