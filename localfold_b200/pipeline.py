"""Throughput mode for pairs that live in host memory.

One host-space call of the pair stack is three phases in a row - the pair goes up over PCIe, the blocks run, the
pair comes back - and at N = 2048 the two copies together take about twice as long as the block itself.
``PairStackPipeline`` keeps several such calls in flight on one GPU: every lane is a context of its own (its
stream, its scratch arena, its prepared weights), so one lane's copies run while another lane's kernels do, and
the upload of one pair overlaps the read-back of another (the GPU has a copy engine per direction).  The results
are those of the one-at-a-time calls: the lanes share nothing but the GPU.

The reference has no counterpart (its pair lives in a ``GPUBuffer`` for the whole fold, ``webgpu/af2/evoformer/
stack.js:44-110``); this is the serving form for independent pairs, e.g. a batch of chains or of recycling states.
"""
from __future__ import annotations

import threading
from concurrent.futures import ThreadPoolExecutor

from .operators import Device
from .stack import PairStackGpu


class PairStackPipeline:
    """``lanes`` contexts on GPU ``ordinal`` with the blocks' weights prepared in each.

    ``run_many(pairs, masks, options)`` updates every host pair in place (contiguous float32 ``[n, n, c_z]`` arrays,
    pinned for the copies to be asynchronous) and returns one result dictionary per pair, in order.  A pair is
    handled by one lane from upload to read-back; the lanes work through the list side by side."""

    def __init__(self, block_weights, c_z, c_hidden, lanes=3, ordinal=0):
        if lanes < 1:
            raise ValueError("the pipeline needs at least one lane")
        self.devices = [Device(ordinal) for _ in range(lanes)]
        self.stacks = [PairStackGpu(dev).prepare(block_weights, c_z, c_hidden) for dev in self.devices]
        self._pool = ThreadPoolExecutor(max_workers=lanes)
        self._free = list(range(lanes))
        self._lock = threading.Lock()

    @property
    def lanes(self):
        return len(self.devices)

    def _one(self, pair, mask, options, kwargs):
        with self._lock:
            lane = self._free.pop()
        try:
            # a host-space call returns when its pair is back in host memory; the library call releases the
            # interpreter lock, so the lanes' calls overlap
            return self.stacks[lane].run(pair, mask, options, inplace=True, **kwargs)
        finally:
            with self._lock:
                self._free.append(lane)

    def submit(self, pair, mask, options=None, **kwargs):
        """Queues one pair; the returned future's ``result()`` is the call's result dictionary.  The pair must not
        be touched (nor queued again) until then."""
        return self._pool.submit(self._one, pair, mask, options, kwargs)

    def run_many(self, pairs, masks, options=None, **kwargs):
        if len(pairs) != len(masks):
            raise ValueError(f"{len(pairs)} pairs but {len(masks)} masks")
        if len({id(p) for p in pairs}) != len(pairs):
            raise ValueError("a pair appears twice in one run: its two updates would race")
        futures = [self.submit(p, m, options, **kwargs) for p, m in zip(pairs, masks)]
        return [f.result() for f in futures]

    def close(self):
        self._pool.shutdown(wait=True)
        for dev, stack in zip(self.devices, self.stacks):
            dev.synchronize()
            stack.close()
            dev.close()
        self.devices, self.stacks = [], []
