"""Row-sharded pair stack over the GPUs of one box (one process per GPU).

The reference is single-device.  Here the pair tensor is sharded by rows: rank g of G owns rows
[g*N/G, (g+1)*N/G) as a local `[N/G][N][128]` tensor.  Per AF2 pair block
(order and residual wiring of ``webgpu/af2/evoformer/block.js:1575-1612``):

    R layout   triangle outgoing   x[i,j] = sum_k a[i,k] b[j,k]: a rows are local, b is all-gathered;
                                   the contraction runs once per gathered chunk
    -> T       all-to-all transpose of the pair shard (rank g then owns rows of z^T)
    T layout   triangle incoming   = the outgoing form on z^T with the transposed mask rows
                                   (incoming(z) = outgoing(z^T)^T)
    -> R       transpose back
    R layout   attention starting  rows are local; the pair bias [H][N][N] is all-gathered by rows
    -> T       transpose
    T layout   attention ending    = the starting form on z^T (AF2 takes its bias from the transposed
                                   normalised pair); then the pair transition (row-local)
    -> R       transpose back

Collectives go through ``torch.distributed`` (NCCL between GPUs; gloo in the CPU tests).  The
arithmetic of every step is behind an ``ops`` object: ``GpuShardOps`` calls the library's
``lf_pair_shard_step``; tests plug in a float64 CPU implementation to check the orchestration.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _native as nat


class TorchComm:
    """all_gather / all_to_all over a torch.distributed group.  `via_host` stages CUDA tensors
    through host memory (for backends without CUDA support, e.g. gloo)."""

    def __init__(self, group=None, via_host=False):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.via_host = via_host

    def all_gather(self, t):
        import torch
        src = (t.cpu() if self.via_host else t).contiguous()
        if self.via_host or self.dist.get_backend(self.group) == "gloo":
            outs = [torch.empty_like(src) for _ in range(self.world)]
            self.dist.all_gather(outs, src, group=self.group)
            out = torch.stack(outs, 0)
        else:
            flat = torch.empty((self.world * src.shape[0],) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
            self.dist.all_gather_into_tensor(flat, src, group=self.group)
            out = flat.view((self.world,) + tuple(src.shape))
        return out.to(t.device) if self.via_host else out

    def all_gather_async(self, t):
        """Starts the gather; returns (gathered [world, ...], work).  `work.wait()` orders the current
        stream after the transfer; work is None when the gather already completed (host-staged backends)."""
        import torch
        if self.via_host or self.dist.get_backend(self.group) == "gloo":
            return self.all_gather(t), None
        src = t.contiguous()
        flat = torch.empty((self.world * src.shape[0],) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
        work = self.dist.all_gather_into_tensor(flat, src, group=self.group, async_op=True)
        return flat.view((self.world,) + tuple(src.shape)), work

    def all_to_all(self, t):
        """t: [world, ...]; block g goes to rank g; returns the blocks received, by source rank."""
        import torch
        src = (t.cpu() if self.via_host else t).contiguous()
        out = torch.empty_like(src)
        if self.via_host or self.dist.get_backend(self.group) == "gloo":
            ins = list(src.unbind(0))
            outs = [torch.empty_like(x) for x in ins]
            # gloo has no all_to_all: pairwise exchange
            reqs = []
            for peer in range(self.world):
                if peer == self.rank:
                    outs[peer].copy_(ins[peer])
                    continue
                reqs.append(self.dist.isend(ins[peer].contiguous(), peer, group=self.group))
                reqs.append(self.dist.irecv(outs[peer], peer, group=self.group))
            for r in reqs:
                r.wait()
            out = torch.stack(outs, 0)
        else:
            self.dist.all_to_all_single(out, src, group=self.group)
        return out.to(t.device) if self.via_host else out


def shard_rows(full, rank, world):
    """Rows [rank*N/world, (rank+1)*N/world) of a [N, ...] array."""
    n = full.shape[0]
    if n % world:
        raise ValueError(f"length {n} is not a multiple of {world} ranks")
    r = n // world
    return full[rank * r:(rank + 1) * r]


def transpose_shard(comm, z):
    """Local rows of z ([R][N][C], R = N/G) -> local rows of z^T, by one all-to-all."""
    R, N, C = z.shape
    G = comm.world
    if R * G != N:
        raise ValueError("shard rows times ranks must equal the row length")
    send = z.reshape(R, G, R, C).permute(1, 0, 2, 3).contiguous()        # [dest][my row][dest's col][C]
    recv = comm.all_to_all(send)                                           # [src][src's row][my col][C]
    return recv.permute(2, 0, 1, 3).reshape(R, N, C).contiguous()          # [my col][src*R + row][C]


class _DeviceArray:
    """A raw device allocation seen through ``__cuda_array_interface__`` (for ``torch.as_tensor``)."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 3, "strides": None}


class PeerTranspose:
    """Transposes of the row-sharded pair with one kernel per rank that stores into the peers' memory
    (``lf_pair_transpose_scatter``), instead of pack -> all-to-all -> unpack.

    Each rank holds two shard-sized buffers allocated by the library and shared with the other ranks'
    processes as CUDA IPC handles; the pair shard lives in one of them, and a transpose writes every
    rank's other buffer.  An all-reduce of one element on the same stream follows the kernel: when it
    has passed, every peer's stores into this rank's buffer have landed.  A buffer is written again
    only two transposes later, after its owner's own reading kernel and a barrier, so one barrier per
    transpose is enough.  GPUs of one box only.
    """

    def __init__(self, device, group, rows, length, dtype):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.group, self.dev = torch, dist, group, device
        device.require_current_stream("PeerTranspose")
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.R, self.N = int(rows), int(length)
        if self.R * self.world != self.N:
            raise ValueError("shard rows times ranks must equal the row length")
        self.dtype = dtype
        self.vector_bytes = 128 * (4 if dtype == torch.float32 else 2)
        nbytes = self.R * self.N * self.vector_bytes
        lib = device.lib
        self.local, self.opened, self.mapped = [], [], []
        handles, error = [], None
        try:
            for _ in range(2):
                ptr = ctypes.c_void_p()
                handle = ctypes.create_string_buffer(64)
                device.check(lib.lf_peer_buffer_create(device.handle, nbytes, ctypes.byref(ptr), handle))
                self.local.append(ptr.value)
                handles.append(handle.raw)
        except Exception as exc:      # keep going: every rank must reach the collectives below
            error = exc
            handles = [b"", b""]
        gathered = [None] * self.world
        dist.all_gather_object(gathered, handles, group=group)
        if error is None and all(len(h[0]) == 64 for h in gathered):
            try:
                for b in range(2):       # [buffer][rank] -> device pointer valid in this process
                    row = []
                    for g in range(self.world):
                        if g == self.rank:
                            row.append(self.local[b])
                            continue
                        ptr = ctypes.c_void_p()
                        device.check(lib.lf_peer_buffer_open(device.handle, gathered[g][b], ctypes.byref(ptr)))
                        row.append(ptr.value)
                        self.opened.append(ptr.value)
                    self.mapped.append(row)
            except Exception as exc:
                error = exc
        elif error is None:
            error = RuntimeError("another rank could not allocate its peer buffers")
        # all ranks agree on the outcome before anyone relies on the mapping
        verdicts = [None] * self.world
        dist.all_gather_object(verdicts, error is None, group=group)
        if not all(verdicts):
            self._release()
            raise error if error is not None else RuntimeError("another rank could not map the peer buffers")
        typestr = "<f4" if dtype == torch.float32 else "<u2"
        views = [torch.as_tensor(_DeviceArray(p, (self.R, self.N, 128), typestr), device=f"cuda:{device.ordinal}") for p in self.local]
        self.views = [v if dtype == torch.float32 else v.view(torch.bfloat16) for v in views]
        self.flag = torch.zeros(1, device=f"cuda:{device.ordinal}")
        self.current = 0
        dist.barrier(group=group)

    def shard(self):
        """The tensor the pair shard lives in right now ([rows][length][128])."""
        return self.views[self.current]

    def transpose(self, z):
        """z must be `shard()`.  Returns the other buffer, holding this rank's rows of the transposed pair."""
        if z.data_ptr() != self.local[self.current]:
            raise ValueError("the pair shard must live in the buffer shard() returned")
        self.dev.require_current_stream("PeerTranspose.transpose")     # the barrier below orders one stream only
        other = 1 - self.current
        dst = (ctypes.c_void_p * self.world)(*self.mapped[other])
        self.dev.check(self.dev.lib.lf_pair_transpose_scatter(self.dev.handle, self.local[self.current], self.R, self.N,
                                                              self.vector_bytes, self.world, self.rank, dst))
        self.dist.all_reduce(self.flag, group=self.group)     # stream-ordered barrier: all stores have landed
        self.current = other
        return self.views[other]

    def _release(self):
        lib = self.dev.lib
        for p in self.opened:
            lib.lf_peer_buffer_close(self.dev.handle, p)
        self.dist.barrier(group=self.group)      # nobody frees a buffer a peer still has mapped
        for p in self.local:
            lib.lf_peer_buffer_destroy(self.dev.handle, p)
        self.opened, self.local = [], []

    def close(self):
        self.dev.synchronize()
        self.dist.barrier(group=self.group)
        self._release()


class ShardedPairStack:
    """Runs AF2 pair blocks on a row shard.  `ops` does the arithmetic, `comm` the exchanges;
    `transposer` (a ``PeerTranspose``) replaces the all-to-all transposes when given - the shard
    must then live in ``transposer.shard()``."""

    def __init__(self, comm, ops, transposer=None):
        self.comm = comm
        self.ops = ops
        self.transposer = transposer

    def _transpose(self, z):
        return self.transposer.transpose(z) if self.transposer is not None else transpose_shard(self.comm, z)

    def _triangle(self, z, mask, w):
        ops, comm = self.ops, self.comm
        a, b = ops.triangle_project(z, mask, w)
        b_all, work = comm.all_gather_async(b)
        x = ops.new_product()
        ops.triangle_contract(a, b, x, comm.rank, w)      # the local chunk runs while the others travel
        if work is not None:
            work.wait()
        for g in range(comm.world):
            if g != comm.rank:
                ops.triangle_contract(a, b_all[g], x, g, w)
        ops.triangle_output(x, z, w)

    def _attention(self, z, mask, w):
        ops, comm = self.ops, self.comm
        q, k, v, g, bias = ops.attention_project(z, w)
        bias_all = comm.all_gather(bias)
        o = ops.attention_core(q, k, v, g, bias_all, mask, w)
        ops.attention_output(o, z, w)

    def block(self, z, mask_rows, mask_t_rows, w):
        """One block on the local shard `z` (updated and returned; it may be a new tensor)."""
        comm = self.comm
        self._triangle(z, mask_rows, w["triangle_outgoing"])
        z = self._transpose(z)
        self._triangle(z, mask_t_rows, w["triangle_incoming"])
        z = self._transpose(z)
        self._attention(z, mask_rows, w["attention_starting"])
        z = self._transpose(z)
        self._attention(z, mask_t_rows, w["attention_ending"])
        self.ops.transition(z, w["transition"])
        z = self._transpose(z)
        return z

    def run(self, z, mask_rows, mask_t_rows, blocks):
        for w in blocks:
            z = self.block(z, mask_rows, mask_t_rows, w)
        return z


class GpuShardOps:
    """Shard-local steps on the GPU through ``lf_pair_shard_step`` (16-bit tensor-core path)."""

    def __init__(self, device, rows, length, ranks, variance="two-pass", epsilon=1e-5):
        import torch
        self.torch = torch
        self.dev = device
        # the collectives and tensor operations between the steps run on torch's current stream
        device.require_current_stream("GpuShardOps")
        self.R, self.N, self.G = int(rows), int(length), int(ranks)
        self.ld = (self.N + 15) // 16 * 16
        self.variance = nat.VARIANCE_TWO_PASS if variance == "two-pass" else nat.VARIANCE_FAST
        self.eps = float(epsilon)
        f16 = dict(dtype=torch.float16, device=f"cuda:{device.ordinal}")
        R, N, ld = self.R, self.N, self.ld
        # buffers are reused by every block: the steps of a block run in stream order
        self.a = torch.empty((128, R, ld), **f16)
        self.b = torch.empty((128, R, ld), **f16)
        self.x = torch.empty((128, R, ld), **f16)
        self.qkvg = [torch.empty((R * N, 128), **f16) for _ in range(4)]
        self.o = torch.empty((R * N, 128), **f16)
        self.bias = torch.zeros((4, R, ld), **f16)

    def _step(self, op, w, pair=None, mask=None, bufs=(), chunk=0):
        self.dev.require_current_stream("GpuShardOps")
        d = nat.ShardStepDesc()
        d.op, d.rows, d.length, d.ranks, d.chunk = op, self.R, self.N, self.G, chunk
        d.variance, d.epsilon = self.variance, self.eps
        d.act_dtype = nat.DTYPE_BF16 if (pair is not None and pair.dtype == self.torch.bfloat16) else nat.DTYPE_F32
        d.pair = pair.data_ptr() if pair is not None else None
        d.mask = mask.data_ptr() if mask is not None else None
        for i, t in enumerate(bufs):
            d.buf[i] = t.data_ptr() if t is not None else None
        d.weights = w.handle
        self.dev.check(self.dev.lib.lf_pair_shard_step(self.dev.handle, ctypes.byref(d), None))

    def new_product(self):
        return self.x

    def triangle_project(self, z, mask, w):
        self._step(nat.SHARD_TRIANGLE_PROJECT, w, z, mask, (self.a, self.b))
        return self.a, self.b

    def triangle_contract(self, a, b_chunk, x, chunk, w):
        self._step(nat.SHARD_TRIANGLE_CONTRACT, w, None, None, (a, b_chunk, x), chunk)

    def triangle_output(self, x, z, w):
        self._step(nat.SHARD_TRIANGLE_OUTPUT, w, z, None, (None, None, x))

    def attention_project(self, z, w):
        q, k, v, g = self.qkvg
        self._step(nat.SHARD_ATTENTION_PROJECT, w, z, None, (q, k, v, g, self.bias))
        return q, k, v, g, self.bias

    def attention_core(self, q, k, v, g, bias_all, mask, w):
        # gathered [rank][head][rows][ld] -> [head][all rows][ld]
        bias_all = bias_all.permute(1, 0, 2, 3).reshape(4, self.N, self.ld).contiguous()
        self._step(nat.SHARD_ATTENTION_CORE, w, None, mask, (q, k, v, g, bias_all, self.o))
        return self.o

    def attention_output(self, o, z, w):
        self._step(nat.SHARD_ATTENTION_OUTPUT, w, z, None, (None, None, None, None, None, o))

    def transition(self, z, w):
        self._step(nat.SHARD_TRANSITION, w, z)


def prepared_block_weights(prepared):
    """``PreparedPairBlock`` -> the weight dict ``ShardedPairStack.block`` takes."""
    return {"triangle_outgoing": prepared.tri_out, "triangle_incoming": prepared.tri_in,
            "attention_starting": prepared.att_start, "attention_ending": prepared.att_end,
            "transition": prepared.transition}
