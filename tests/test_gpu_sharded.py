"""Row-sharded pair block on the GPU: two ranks (two processes on one device, exchanging through gloo
with host staging, so no NCCL and no second GPU is needed) run the library's shard steps and must
match the unsharded CPU oracle within the 16-bit per-block bound.  One case moves the transposes
to the peer-store kernel (buffers shared between the two processes as CUDA IPC handles), and one runs
the fused exchange: channel-sharded triangle multiplication and pair bias written by the producing
kernels straight into the other process's buffers.  The kernels never wait on one another: every
barrier is a host-side collective between the launches."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n, result_path, peer):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import localfold_b200 as lf
    from localfold_b200 import synthetic as syn
    from localfold_b200.sharded import (GpuShardOps, PeerExchange, PeerTranspose, ShardedPairStack, TorchComm,
                                        prepared_block_weights, shard_rows)

    torch.cuda.set_device(0)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = lf.Device(0, stream=stream.cuda_stream)
    pair, mask, weights = syn.af2_pair_block(21, n, blocks=2, masked_tail=0.1)
    blocks = [lf.PreparedPairBlock(dev, w, 128, 128) for w in weights]
    z = torch.from_numpy(np.ascontiguousarray(shard_rows(pair, rank, world))).cuda()
    m_rows = torch.from_numpy(np.ascontiguousarray(shard_rows(mask, rank, world))).cuda()
    m_t_rows = torch.from_numpy(np.ascontiguousarray(shard_rows(np.ascontiguousarray(mask.T), rank, world))).cuda()
    transposer = None
    if peer:   # transposes by peer stores between the two processes' buffers (CUDA IPC), barrier through gloo
        transposer = PeerTranspose(dev, None, n // world, n, torch.float32)
        transposer.shard().copy_(z)
        z = transposer.shard()
    exchange = PeerExchange(dev, None, n // world, n) if peer == "exchange" else None
    stack = ShardedPairStack(TorchComm(via_host=True), GpuShardOps(dev, n // world, n, world), transposer, exchange)
    z = stack.run(z, m_rows, m_t_rows, [prepared_block_weights(b) for b in blocks])
    dev.synchronize()
    host = z.cpu()
    if transposer is not None:
        transposer.close()
    if exchange is not None:
        exchange.close()
    gathered = [torch.empty_like(host) for _ in range(world)]
    dist.all_gather(gathered, host)
    if rank == 0:
        np.save(result_path, torch.cat(gathered, 0).numpy())
    dist.barrier()
    for b in blocks:
        b.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("n,peer", [(64, False), (160, False), (160, True), (256, "exchange")])
def test_sharded_gpu_block_matches_oracle(tmp_path, n, peer):
    sys.path.insert(0, ROOT)
    from localfold_b200 import synthetic as syn
    from oracle import oracle
    port = 29800 + os.getpid() % 150
    result = str(tmp_path / "pair.npy")
    mp.spawn(_worker, args=(2, port, n, result, peer), nprocs=2, join=True)
    got = np.load(result)
    pair, mask, weights = syn.af2_pair_block(21, n, blocks=2, masked_tail=0.1)
    want = pair
    for w in weights:
        want = oracle.af2_pair_block(want, mask, w, 128)
    assert np.isfinite(got).all()
    assert oracle.relative_l2(got, want) <= 3e-3       # two blocks at the 2e-3 per-block bound
