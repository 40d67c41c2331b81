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

With a ``PeerExchange`` the triangle multiplication runs channel-sharded instead and the exchange is
fused into the kernels (stores into the peers' memory over NVLink, one barrier per step):

    R layout   triangle outgoing   projection epilogue stores channel h of the local rows into rank
               and incoming        h / (128/G)'s operand planes; that rank contracts its 128/G channels over
                                   the whole N x N plane (full tiles, either direction, no transposed pair) and
                                   its epilogue stores row i of the product to rank i / R; output is row-local
    R layout   attention starting  the projection epilogue stores the shard's pair-bias rows into every rank
    -> T, attention ending, transition, -> R as above: two transposes per block instead of four

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


def share_buffers(device, group, sizes):
    """Allocates one device buffer per entry of ``sizes`` (bytes) and maps every other rank's buffers into
    this process as CUDA IPC handles.  Returns (local pointers, mapped[buffer][rank] pointers valid here,
    pointers opened from peers).  Every rank reaches every collective even when its own part fails, and all
    ranks agree on the outcome before anyone relies on the mapping."""
    import torch.distributed as dist
    lib = device.lib
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    local, opened, mapped, handles, error = [], [], [], [], None
    try:
        for nbytes in sizes:
            ptr = ctypes.c_void_p()
            handle = ctypes.create_string_buffer(64)
            device.check(lib.lf_peer_buffer_create(device.handle, int(nbytes), ctypes.byref(ptr), handle))
            local.append(ptr.value)
            handles.append(handle.raw)
    except Exception as exc:      # keep going: every rank must reach the collectives below
        error = exc
        handles = [b""] * len(sizes)
    gathered = [None] * world
    dist.all_gather_object(gathered, handles, group=group)
    if error is None and all(len(h) == 64 for hs in gathered for h in hs):
        try:
            for b in range(len(sizes)):
                row = []
                for g in range(world):
                    if g == rank:
                        row.append(local[b])
                        continue
                    ptr = ctypes.c_void_p()
                    device.check(lib.lf_peer_buffer_open(device.handle, gathered[g][b], ctypes.byref(ptr)))
                    row.append(ptr.value)
                    opened.append(ptr.value)
                mapped.append(row)
        except Exception as exc:
            error = exc
    elif error is None:
        error = RuntimeError("another rank could not allocate its peer buffers")
    verdicts = [None] * world
    dist.all_gather_object(verdicts, error is None, group=group)
    if not all(verdicts):
        release_buffers(device, group, local, opened)
        raise error if error is not None else RuntimeError("another rank could not map the peer buffers")
    return local, mapped, opened


def release_buffers(device, group, local, opened):
    import torch.distributed as dist
    lib = device.lib
    for p in opened:
        lib.lf_peer_buffer_close(device.handle, p)
    dist.barrier(group=group)      # nobody frees a buffer a peer still has mapped
    for p in local:
        lib.lf_peer_buffer_destroy(device.handle, p)


class PeerExchange:
    """Buffers of the fused exchange (``lf_pair_shard_exchange_step``): per rank the channel-sharded triangle
    operands a, b ``[128/G][N][N]`` fp16, the product x ``[128][R][N]`` and the pair bias of all query rows
    ``[4][N][N]``, each shared with the other ranks' processes as CUDA IPC handles.  ``barrier()`` is a
    one-element all-reduce on the current stream: once it has passed on a rank, every peer kernel enqueued
    before its own barrier has finished, so its stores into this rank's buffers have landed.  Each buffer
    is written by one step and read by the next, with a barrier in between and the reader's kernel ahead of
    the writer's next barrier in stream order, so single buffers are enough.  GPUs of one box only."""

    def __init__(self, device, group, rows, length):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.group, self.dev = torch, dist, group, device
        device.require_current_stream("PeerExchange")
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.R, self.N = int(rows), int(length)
        if self.R * self.world != self.N:
            raise ValueError("shard rows times ranks must equal the row length")
        if 128 % self.world or self.N % 16 or (self.world > 1 and self.R % 128):
            raise ValueError("the fused exchange needs ranks dividing 128, length a multiple of 16 and shard rows a multiple of 128")
        cpr = 128 // self.world
        plane = self.N * self.N * 2
        sizes = [cpr * plane, cpr * plane, 128 * self.R * self.N * 2, 4 * plane]
        self.local, self.mapped, self.opened = share_buffers(device, group, sizes)
        where = f"cuda:{device.ordinal}"
        half = lambda ptr, shape: torch.as_tensor(_DeviceArray(ptr, shape, "<u2"), device=where).view(torch.float16)
        self.x = half(self.local[2], (128, self.R, self.N))
        self.bias = half(self.local[3], (4, self.N, self.N))
        self.bias.zero_()
        self.flag = torch.zeros(1, device=where)
        self.peers = nat.ShardPeers()
        self.peers.rank = self.rank
        for g in range(self.world):
            self.peers.a[g], self.peers.b[g] = self.mapped[0][g], self.mapped[1][g]
            self.peers.x[g], self.peers.bias[g] = self.mapped[2][g], self.mapped[3][g]
        torch.cuda.synchronize()
        dist.barrier(group=group)

    def barrier(self):
        self.dev.require_current_stream("PeerExchange.barrier")
        self.dist.all_reduce(self.flag, group=self.group)

    def close(self):
        self.dev.synchronize()
        self.dist.barrier(group=self.group)
        release_buffers(self.dev, self.group, self.local, self.opened)
        self.local, self.opened = [], []


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
        self.local, self.mapped, self.opened = share_buffers(device, group, [nbytes, nbytes])
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
        release_buffers(self.dev, self.group, self.local, self.opened)
        self.opened, self.local = [], []

    def close(self):
        self.dev.synchronize()
        self.dist.barrier(group=self.group)
        self._release()


class ShardedPairStack:
    """Runs AF2 pair blocks on a row shard.  `ops` does the arithmetic, `comm` the exchanges;
    `transposer` (a ``PeerTranspose``) replaces the all-to-all transposes when given - the shard
    must then live in ``transposer.shard()``."""

    def __init__(self, comm, ops, transposer=None, exchange=None):
        """``exchange``: a ``PeerExchange`` (GPU) or True (operations that exchange through ``comm``, as the
        CPU test operations do) switches to the channel-sharded triangle multiplication."""
        self.comm = comm
        self.ops = ops
        self.transposer = transposer
        self.exchange = exchange

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

    def _triangle_channel(self, z, mask, w, incoming):
        """Channel-sharded: project (operands leave for their channel owners), contract 128/G channels over the
        whole plane (product rows leave for their row owners), output on the local rows."""
        ops = self.ops
        ops.exchange_triangle_project(z, mask, w, self.exchange, self.comm)
        x = ops.exchange_triangle_contract(w, self.exchange, self.comm, incoming)
        ops.triangle_output(x, z, w)

    def _attention_channel(self, z, mask, w):
        ops = self.ops
        q, k, v, g, bias_all = ops.exchange_attention_project(z, w, self.exchange, self.comm)
        o = ops.attention_core(q, k, v, g, bias_all, mask, w)
        ops.attention_output(o, z, w)

    def block(self, z, mask_rows, mask_t_rows, w):
        """One block on the local shard `z` (updated and returned; it may be a new tensor)."""
        if self.exchange is not None:
            self._triangle_channel(z, mask_rows, w["triangle_outgoing"], False)
            self._triangle_channel(z, mask_rows, w["triangle_incoming"], True)
            self._attention_channel(z, mask_rows, w["attention_starting"])
            z = self._transpose(z)
            self._attention_channel(z, mask_t_rows, w["attention_ending"])
            self.ops.transition(z, w["transition"])
            return self._transpose(z)
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

    def __init__(self, device, rows, length, ranks, variance="two-pass", epsilon=1e-5, project_exchange="fused"):
        """``project_exchange``: how the triangle operands reach their channel owners in the fused-exchange form -
        "fused" (stores from the projection kernel's epilogue) or "copy" (a copy kernel after it)."""
        import torch
        self.project_exchange = project_exchange
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
        if bias_all.dim() == 4:      # gathered [rank][head][rows][ld] -> [head][all rows][ld]
            bias_all = bias_all.permute(1, 0, 2, 3).reshape(4, self.N, self.ld).contiguous()
        self._step(nat.SHARD_ATTENTION_CORE, w, None, mask, (q, k, v, g, bias_all, self.o))
        return self.o

    def attention_output(self, o, z, w):
        self._step(nat.SHARD_ATTENTION_OUTPUT, w, z, None, (None, None, None, None, None, o))

    # -- the fused exchange (``PeerExchange``): kernels store into the peers' buffers, then a barrier

    def _exchange_step(self, op, w, ex, pair=None, mask=None, bufs=(), incoming=False):
        self.dev.require_current_stream("GpuShardOps")
        d = nat.ShardStepDesc()
        d.op, d.rows, d.length, d.ranks, d.chunk = op, self.R, self.N, self.G, 0
        d.variance, d.epsilon = self.variance, self.eps
        d.act_dtype = nat.DTYPE_BF16 if (pair is not None and pair.dtype == self.torch.bfloat16) else nat.DTYPE_F32
        d.pair = pair.data_ptr() if pair is not None else None
        d.mask = mask.data_ptr() if mask is not None else None
        for i, t in enumerate(bufs):
            d.buf[i] = t.data_ptr() if t is not None else None
        d.weights = w.handle
        ex.peers.incoming = 1 if incoming else 0
        self.dev.check(self.dev.lib.lf_pair_shard_exchange_step(self.dev.handle, ctypes.byref(d), ctypes.byref(ex.peers), None))

    def exchange_triangle_project(self, z, mask, w, ex, comm):
        if self.project_exchange == "fused":        # the projection's epilogue stores into the owners' planes
            self._exchange_step(nat.SHARD_TRIANGLE_PROJECT, w, ex, z, mask)
        else:                                       # projection into local planes, then one copy kernel per operand
            self._step(nat.SHARD_TRIANGLE_PROJECT, w, z, mask, (self.a, self.b))
            for local, table in ((self.a, ex.mapped[0]), (self.b, ex.mapped[1])):
                dst = (ctypes.c_void_p * self.G)(*table)
                self.dev.check(self.dev.lib.lf_pair_planes_scatter(self.dev.handle, local.data_ptr(), 128, self.R, self.N,
                                                                   self.G, ex.rank, dst))
        ex.barrier()          # every rank's operand rows have landed in the channel owners' planes

    def exchange_triangle_contract(self, w, ex, comm, incoming):
        self._exchange_step(nat.SHARD_TRIANGLE_CONTRACT, w, ex, incoming=incoming)
        ex.barrier()          # every channel owner's product rows have landed here
        return ex.x

    def exchange_attention_project(self, z, w, ex, comm):
        q, k, v, g = self.qkvg
        self._exchange_step(nat.SHARD_ATTENTION_PROJECT, w, ex, z, None, (q, k, v, g))
        ex.barrier()          # the bias rows of every shard have landed
        return q, k, v, g, ex.bias

    def transition(self, z, w):
        self._step(nat.SHARD_TRANSITION, w, z)


def prepared_block_weights(prepared):
    """``PreparedPairBlock`` -> the weight dict ``ShardedPairStack.block`` takes."""
    return {"triangle_outgoing": prepared.tri_out, "triangle_incoming": prepared.tri_in,
            "attention_starting": prepared.att_start, "attention_ending": prepared.att_end,
            "transition": prepared.transition}
