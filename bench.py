"""Benchmark of the pair-stack hot path: one AF2 pair-stack block per step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--length L]

A step is one block of the 48-block AF2 Evoformer pair stack (triangle
multiplication outgoing + incoming, triangle attention starting + ending node,
pair transition) on a resident N x N x 128 pair tensor: BASELINE config 4's
shape (N = 2048, c_z = 128, c = 128, 4 x 32 heads, 4x transition, seed 4, mask
of ones), synthetic N(0,1) pair and N(0, 1/fan_in) weights.  Successive steps
are successive blocks of the stack on the same pair, as in the stack runner.

The JSON line reports ms per block (lower is better) with the pair resident in
HBM (`value`, timed with per-kernel profiling off), the same through the
host-buffer API with copies in the timed region (`e2e`), the live roofline of
every kernel family from a second, profiled pass over the same steps, the
N = 384 block time the metric also names (`extra.n384_ms_per_block`, L2 flushed
between blocks because that pair fits in L2), and - at N = 1 - the CPU oracle
timed on this host on a bounded sample (`cpu_baseline`).  `--pair-dtype bf16`
stores the pair stream in bf16, as BASELINE config 4 words it; the default is
float32, the storage that meets the per-block accuracy bound.

`--impl reference` times the reference's CPU implementation of the same block
(the C restatement under oracle/; the reference itself is JavaScript and no
JavaScript engine exists on these machines) on all host cores, on a bounded
sample, scaled to the full workload by algorithmic FLOPs.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

C_Z = 128
C_HIDDEN = 128
HEADS = 4


def block_flops(n: int) -> float:
    """AF2 pair block: 1536 N^3 + 985088 N^2 (contractions + attention + dense)."""
    return 1536.0 * n ** 3 + 985088.0 * n ** 2


def contraction_flops(n: int) -> float:
    return 256.0 * n ** 3


# Algorithmic work of one launch of each kernel family on a shard of `rows` pair rows of length n
# (c_z = c_hidden = 128, 4 heads x 32): tensor-core FLOPs for the two contraction-shaped kernels,
# bytes that must cross HBM for the fused LayerNorm/projection kernels (pair stream f32, operands f16).
#   triangle_contract  128 channels x (rows x rows_b x n) GEMM            256 rows rows_b n FLOP
#   attention          Q K^T and P V over 4 heads x 32                    512 rows n n FLOP
# with w the bytes of a pair element (4 for the float32 stream, 2 for bf16):
#   ln_gemm            triangle projection: z in, a and b out             128 w + 512 B / position
#                      attention projection: z in, q k v gate + bias out  128 w + 1032 B / position
#                      attention output: o and z in, z out                256 w + 256 B / position
#   triangle_output    x and z in, z out                                  256 w + 256 B / position
#   transition         z in, z out                                        256 w B / position
FAMILY_WORK = {
    "triangle_contract": ("tensor", lambda rows, n, world, w: 256.0 * rows * rows * n),
    "attention": ("tensor", lambda rows, n, world, w: 512.0 * rows * n * n),
    "ln_gemm": ("hbm", lambda rows, n, world, w: (2 * (128 * w + 512) + 2 * (128 * w + 1032) + 2 * (256 * w + 256)) / 6.0 * rows * n),
    "triangle_output": ("hbm", lambda rows, n, world, w: (256.0 * w + 256) * rows * n),
    "transition": ("hbm", lambda rows, n, world, w: 256.0 * w * rows * n),
}


def traffic_per_position():
    """DRAM bytes per pair position and launch of each kernel family, as written by the profiling step from
    an ncu capture of this build (dram__bytes_read.sum + dram__bytes_write.sum at a smaller N, divided by
    the positions of that launch; every kernel's traffic grows with the positions).  None when no capture
    is on file: `traffic` is then null rather than a stale figure."""
    path = os.path.join(ROOT, "profiles", "traffic_af2_pair_block.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f)


FAMILY_NAME = {
    "triangle_contract": "triangle contraction (tcgen05, 128 batched GEMMs)",
    "attention": "attention core (tcgen05 Q K^T and P V, softmax between them in tensor memory)",
    "ln_gemm": "LayerNorm + projection kernels (average of the six launches)",
    "triangle_output": "triangle output (LayerNorm of x folded into the GEMM, gate, residual)",
    "transition": "pair transition (LayerNorm + two GEMMs, weights streamed)",
}


def roofline_table(families, n, world, peaks, pair_bytes=4):
    """Per kernel family: algorithmic work per launch / its measured launch time against the
    measured peak.  Returns (the entry of the family with the largest share of the step, all entries)."""
    rows = n // world
    total = sum(v[0] for v in families.values()) or 1.0
    traffic = traffic_per_position()
    out = []
    for fam, (bound, work) in FAMILY_WORK.items():
        ms, launches = families.get(fam, (0.0, 0))
        if not launches:
            continue
        per_launch_ms = ms / launches
        w = work(rows, n, world, pair_bytes)
        if bound == "tensor":
            achieved, peak, unit = w / (per_launch_ms * 1e-3) / 1e12, peaks["tflops_sustained"], "TFLOP/s"
            src = peaks["source"] + " (sustained cuBLAS bf16: the kernel runs inside a long step)"
        else:
            achieved, peak, unit = w / (per_launch_ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
            src = peaks["source"] + " (copy bandwidth)"
        out.append({"kernel": FAMILY_NAME[fam], "family": fam, "bound": bound, "achieved": achieved, "peak": peak,
                    "unit": unit, "frac": achieved / peak,
                    "traffic": traffic["bytes_per_position"][fam] * rows * n if traffic and fam in traffic.get("bytes_per_position", {}) else None,
                    "traffic_source": traffic.get("source") if traffic else None, "peak_source": src,
                    "launch_ms": per_launch_ms, "launches": launches, "share_of_step": ms / total,
                    "work_per_launch": w})
        if fam == "transition":      # a GEMM pair at 256-512 flop per byte: reported against both rooflines
            flops = 262144.0 * rows * n
            out[-1]["tensor"] = {"achieved": flops / (per_launch_ms * 1e-3) / 1e12, "peak": peaks["tflops_sustained"],
                                 "unit": "TFLOP/s", "frac": flops / (per_launch_ms * 1e-3) / 1e12 / peaks["tflops_sustained"]}
    out.sort(key=lambda e: -e["share_of_step"])
    return (out[0] if out else None), out


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                   parts[3:7]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def host_threads() -> int:
    """Cores this process may run on: the CPU legs use exactly these, whatever OMP_NUM_THREADS says
    (torchrun exports OMP_NUM_THREADS=1)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_sample(sample_n: int, full_n: int):
    """Times the CPU oracle on one AF2 pair block at `sample_n` and scales to `full_n` by FLOPs."""
    from localfold_b200 import synthetic as syn
    from oracle import oracle
    cores = host_threads()
    oracle.set_threads(cores)
    pair, mask, weights = syn.af2_pair_block(4, sample_n)
    t0 = time.perf_counter()
    oracle.af2_pair_block(pair, mask, weights[0], C_HIDDEN)
    seconds = time.perf_counter() - t0
    scaled_ms = seconds * 1e3 * block_flops(full_n) / block_flops(sample_n)
    return {"value": scaled_ms, "unit": "ms/block", "cores": cores, "kind": "port",
            "sample": f"one AF2 pair block at N={sample_n} ({seconds:.2f} s on {cores} threads), scaled to "
                      f"N={full_n} by algorithmic FLOPs (1536 N^3 + 985088 N^2)",
            "sample_seconds": seconds}


def run_reference(args, rank):
    """The reference arm: the CPU restatement on all host cores.  Rank 0 alone works; under torchrun the
    other ranks leave at once (no process group is formed, nothing waits on anything)."""
    if rank != 0:
        return
    full_n = args.length
    times = []
    sample_n = args.cpu_sample
    res = None
    for i in range(args.warmup + args.steps):
        res = cpu_sample(sample_n, full_n)
        if i >= args.warmup:
            times.append(res["value"])
        if times and (time.perf_counter() - START) > 150:
            break
    ms = float(np.mean(times))
    line = {
        "impl": "reference", "metric": "pair_stack_block_ms", "value": ms, "unit": "ms/block", "n_gpus": args.gpus,
        "steps": len(times), "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f64 accumulate / f32 store", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": ms, "unit": "ms/block", "cores": res["cores"], "kind": "port", "sample": res["sample"]},
        "e2e": {"value": ms, "unit": "ms/block", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def workload_config(args, n_gpus):
    return {"workload": f"AF2 Evoformer pair-stack block, N={args.length}, c_z=128, tri-mult c=128, "
                        f"tri-attention 4x32, transition 4x, seed 4, mask ones (BASELINE config 4 shape)",
            "length": args.length, "precision": args.precision, "pair_dtype": args.pair_dtype,
            "parallelism": "single GPU" if n_gpus == 1 else
            (f"pair rows sharded over {n_gpus} GPUs; triangle multiplication channel-sharded, its operands, product and the pair "
             f"bias stored into the peers' memory by the producing kernels over NVLink; 2 transposes per block by one peer-store "
             f"kernel each" if args.trimul == "channel" and args.transpose == "peer" else
             f"pair rows sharded over {n_gpus} GPUs (NCCL all-gather of the triangle operand b and of the pair bias; "
             f"4 transposes per block by " + ("one peer-store kernel each over NVLink" if args.transpose == "peer"
                                             else "NCCL all-to-all") + ")"),
            "l2": "inputs larger than L2 (pair tensor %.0f MiB)" % (args.length ** 2 * C_Z * (2 if args.pair_dtype == "bf16" else 4) / 2 ** 20)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--length", type=int, default=2048)
    ap.add_argument("--precision", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--pair-dtype", default="f32", choices=["f32", "bf16"],
                    help="storage of the pair stream (bf16: BASELINE config 4 as worded; f32 meets the 2e-3 per-block bound)")
    ap.add_argument("--cpu-sample", type=int, default=384, help="N of the CPU oracle's bounded sample")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-pipeline", action="store_true", help="skip the pipelined end-to-end leg (three host pairs in flight)")
    ap.add_argument("--no-n384", action="store_true", help="skip the N = 384 leg")
    ap.add_argument("--trimul", default="channel", choices=["channel", "rows"],
                    help="N > 1: triangle multiplication channel-sharded with the exchange fused into the kernels (peer stores), "
                         "or row-sharded with an NCCL all-gather of the operand b")
    ap.add_argument("--project-exchange", default="fused", choices=["fused", "copy"],
                    help="--trimul channel: triangle operands to their channel owners by stores from the projection kernel's "
                         "epilogue, or by a copy kernel after it")
    ap.add_argument("--transpose", default="peer", choices=["peer", "nccl"],
                    help="N > 1: transposes of the sharded pair by peer stores (one kernel) or by NCCL all-to-all")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist
    import localfold_b200 as lf
    from localfold_b200 import synthetic as syn

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    # a non-default stream: the library and the timing events share it
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    dev = lf.Device(local_rank, stream=stream.cuda_stream)

    n = args.length
    opts = {"precision": args.precision, "variance": "two-pass"}
    pair_dtype = torch.bfloat16 if args.pair_dtype == "bf16" else torch.float32
    pair_bytes = 2 if args.pair_dtype == "bf16" else 4
    sharded_check = None
    if world == 1:
        pair_h, mask_h, weights = syn.af2_pair_block(4, n, blocks=2)
        stack = lf.PairStackGpu(dev).prepare(weights, C_Z, C_HIDDEN)
        pair_d = torch.from_numpy(pair_h).cuda().to(pair_dtype)
        mask_d = torch.from_numpy(mask_h).cuda()

        def step(i):
            stack.run(pair_d, mask_d, opts, first_block=i % 2, n_blocks=1)
    else:
        # strong scaling: the same block, pair rows sharded over the ranks
        from localfold_b200.sharded import (GpuShardOps, PeerExchange, PeerTranspose, ShardedPairStack, TorchComm,
                                            prepared_block_weights, shard_rows)
        if n % (16 * world):
            raise SystemExit(f"--length {n} must be a multiple of 16 x {world} ranks")
        pair_h, mask_h, weights = syn.af2_pair_block(4, n, blocks=2)
        prepared = [lf.PreparedPairBlock(dev, w, C_Z, C_HIDDEN) for w in weights]
        block_w = [prepared_block_weights(b) for b in prepared]

        def build(length, full_pair, full_mask):
            """The sharded runner for one length: (shard holder, row masks, runner, transposer)."""
            rows = length // world
            local = np.ascontiguousarray(shard_rows(full_pair, rank, world))
            transposer = None
            if args.transpose == "peer":   # the shard lives in buffers the ranks share; transposes are peer stores
                try:
                    transposer = PeerTranspose(dev, None, rows, length, pair_dtype)
                    mapped = 1
                except Exception as exc:   # e.g. no peer access between two of the GPUs: every rank falls back together
                    print(f"rank {rank}: peer mapping failed ({exc}); using NCCL all-to-all transposes", file=sys.stderr)
                    mapped = 0
                flag = torch.tensor([mapped], device="cuda")
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if int(flag.item()) == 0:
                    transposer = None
                    args.transpose = "nccl"
            if transposer is not None:
                transposer.shard().copy_(torch.from_numpy(local).cuda().to(pair_dtype))
                holder = {"z": transposer.shard()}
            else:
                holder = {"z": torch.from_numpy(local).cuda().to(pair_dtype)}
            m_rows = torch.from_numpy(np.ascontiguousarray(shard_rows(full_mask, rank, world))).cuda()
            m_t_rows = torch.from_numpy(np.ascontiguousarray(shard_rows(np.ascontiguousarray(full_mask.T), rank, world))).cuda()
            exchange = None
            if args.trimul == "channel" and transposer is None:
                args.trimul = "rows"
            if args.trimul == "channel":    # the fused exchange needs the same peer mappings
                try:
                    exchange = PeerExchange(dev, None, rows, length)
                except Exception as exc:    # raised on every rank together (the ranks agree inside)
                    print(f"rank {rank}: fused exchange unavailable ({exc}); row-sharded triangle multiplication", file=sys.stderr)
                    args.trimul = "rows"
            runner = ShardedPairStack(TorchComm(), GpuShardOps(dev, rows, length, world, project_exchange=args.project_exchange),
                                      transposer, exchange)
            return holder, m_rows, m_t_rows, runner, (transposer, exchange), local

        # Numerical check of the path that is about to be timed (NCCL gathers, peer-store transposes): one
        # block at a small length, every rank's shard against the same block run unsharded on this GPU.
        if args.trimul == "channel" and (128 % world or (n // world) % 128):
            args.trimul = "rows"
        check_n = 128 * world if args.trimul == "channel" else 16 * world * max(1, 256 // (16 * world))
        small_pair, small_mask, _ = syn.af2_pair_block(5, check_n, masked_tail=0.05)
        holder, m_rows, m_t_rows, runner, tr, _ = build(check_n, small_pair, small_mask)
        holder["z"] = runner.block(holder["z"], m_rows, m_t_rows, block_w[0])
        single = torch.from_numpy(small_pair).cuda().to(pair_dtype)
        ref_stack = lf.PairStackGpu(dev).prepare([prepared[0]], C_Z, C_HIDDEN)
        ref_stack.run(single, torch.from_numpy(small_mask).cuda(), opts, first_block=0, n_blocks=1)
        torch.cuda.synchronize()
        mine = single[rank * (check_n // world):(rank + 1) * (check_n // world)].float()
        num = torch.linalg.vector_norm((holder["z"].float() - mine).double()) ** 2
        den = torch.linalg.vector_norm(mine.double()) ** 2
        both = torch.stack([num, den])
        dist.all_reduce(both)
        sharded_check = {"length": check_n, "rel_l2_vs_unsharded": float(torch.sqrt(both[0] / both[1]).item()),
                         "what": "one sharded block (NCCL gathers, transposes as timed) against the same block on one GPU"}
        for part in tr:
            if part is not None:
                part.close()
        del holder, runner

        shard, m_rows, m_t_rows, sharded, transposer, pair_h = build(n, pair_h, mask_h)
        stack = None

        def step(i):
            shard["z"] = sharded.block(shard["z"], m_rows, m_t_rows, block_w[i % 2])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    # timed region: K blocks, per-kernel profiling off
    launches0 = dev.launch_count()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(stream)
    for i in range(args.steps):
        step(i)
    e1.record(stream)
    barrier()
    total_ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    launches = dev.launch_count() - launches0
    if world > 1:
        t = torch.tensor([total_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_block = total_ms / args.steps
    finite = bool(torch.isfinite((pair_d if world == 1 else shard["z"]).float()).all().item())

    # second pass over the same steps with every launch bracketed by events: the per-family split
    dev.profile(True)
    dev.profile_read()
    for i in range(args.steps):
        step(i)
    barrier()
    families = dev.profile_read()
    dev.profile(False)

    # the metric's other length: N = 384 on one GPU.  That pair (75 MB in float32) fits in L2, so a
    # buffer larger than L2 is written between blocks and each block is timed by its own events.
    extra = {}
    if world == 1 and n != 384 and not args.no_n384:
        p384, m384, _ = syn.af2_pair_block(4, 384)
        z384 = torch.from_numpy(p384).cuda().to(pair_dtype)
        k384 = torch.from_numpy(m384).cuda()
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        times = []
        for i in range(3 + 10):
            flush.fill_(i & 0xff)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            stack.run(z384, k384, opts, first_block=i % 2, n_blocks=1)
            b.record(stream)
            torch.cuda.synchronize()
            if i >= 3:
                times.append(a.elapsed_time(b))
        extra["n384_ms_per_block"] = float(np.mean(times))
        extra["n384_note"] = "AF2 pair block at N=384 on one GPU, mean of 10 blocks, 256 MiB written between blocks to flush L2"
        extra["n384_tflops_block"] = block_flops(384) / (extra["n384_ms_per_block"] * 1e-3) / 1e12
        # the same length in the AF3 dialect (the five pair updates of a pairformer block: fast-variance LayerNorm,
        # SwiGLU transition, no biases), the shape of the 48-block pairformer stack
        d3 = syn.draw(2)
        af3_blocks = [syn.af3_pairformer_block_weights(d3, C_Z, 384, 4, 16) for _ in range(2)]
        stack3 = lf.PairStackGpu(dev).prepare(af3_blocks, C_Z, C_Z)
        opts3 = dict(opts, variance="fast")
        times = []
        for i in range(3 + 10):
            flush.fill_(i & 0xff)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            stack3.run(z384, k384, opts3, first_block=i % 2, n_blocks=1, dialect={"swapTransposedBias": False})
            b.record(stream)
            torch.cuda.synchronize()
            if i >= 3:
                times.append(a.elapsed_time(b))
        stack3.close()
        extra["n384_af3_ms_per_block"] = float(np.mean(times))
        extra["n384_af3_note"] = "pair part of an AF3 pairformer block at N=384 (the 48-block stack's shape), timed like n384_ms_per_block"
        del z384
        # config 1 of the baseline: one whole AF2 Evoformer block (MSA row / column attention, MSA transition, outer
        # product mean, the five pair updates) at S = 128 sequences, N = 256, c_m = 256, MSA and pair resident
        msa_h, pair_c1, mm_h, pm_h, w_c1 = syn.af2_evoformer_block(1, S=128, n=256)
        block_c1 = lf.PreparedMsaBlock(dev, w_c1, 256, C_Z, 32, C_Z)
        msa_d, pair_c1d = torch.from_numpy(msa_h).cuda(), torch.from_numpy(pair_c1).cuda()
        mm_d, pm_d = torch.from_numpy(mm_h).cuda(), torch.from_numpy(pm_h).cuda()
        for name, o in (("evoformer_block_ms", opts), ("evoformer_block_f32_ms", dict(opts, precision="f32"))):
            times = []
            for i in range(3 + 6):
                flush.fill_(i & 0xff)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                block_c1.run(msa_d, pair_c1d, mm_d, pm_d, 128, 256, o)
                b.record(stream)
                torch.cuda.synchronize()
                if i >= 3:
                    times.append(a.elapsed_time(b))
            extra[name] = float(np.mean(times))
        block_c1.close()
        # the shape of the reference's own published per-block figure (a whole Evoformer block at N = 825 residues,
        # 512 MSA rows, measured through WebGPU on another GPU): same operators, same widths, ragged length
        msa_h, pair_c1, mm_h, pm_h, w_c1 = syn.af2_evoformer_block(2, S=512, n=825)
        block_p = lf.PreparedMsaBlock(dev, w_c1, 256, C_Z, 32, C_Z)
        msa_d, pair_c1d = torch.from_numpy(msa_h).cuda(), torch.from_numpy(pair_c1).cuda()
        mm_d, pm_d = torch.from_numpy(mm_h).cuda(), torch.from_numpy(pm_h).cuda()
        times = []
        for i in range(2 + 4):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            block_p.run(msa_d, pair_c1d, mm_d, pm_d, 512, 825, opts)
            b.record(stream)
            torch.cuda.synchronize()
            if i >= 2:
                times.append(a.elapsed_time(b))
        extra["evoformer_block_n825_s512_ms"] = float(np.mean(times))
        extra["evoformer_block_n825_s512_finite"] = bool(torch.isfinite(pair_c1d).all().item() and torch.isfinite(msa_d).all().item())
        extra["evoformer_block_n825_s512_note"] = ("one AF2 Evoformer block at N=825, 512 MSA rows (432 MB MSA + 348 MB pair, larger than L2), mean of 4; "
                                                   "the reference documents 195.6 ms per block for this shape through WebGPU on an A100")
        block_p.close()
        extra["evoformer_block_note"] = ("one AF2 Evoformer block at S=128, N=256, c_m=256 (the baseline's CPU-runnable configuration), "
                                         "MSA and pair resident, mean of 6 blocks, L2 flushed between; _f32_ is the float32 SIMT mode")
        del flush, msa_d, pair_c1d

    # end to end through the public API with host buffers: pinned host pair in, pair out, every step
    e2e = None
    if not args.no_e2e:
        rows_local = n // world
        reps = max(2, min(args.steps, 3))
        if world == 1 and pair_dtype == torch.float32:
            pinned = torch.empty((rows_local, n, C_Z), dtype=torch.float32, pin_memory=True)
            pinned.copy_(torch.from_numpy(pair_h).reshape(rows_local, n, C_Z))
            mask_p = torch.empty((n, n), dtype=torch.float32, pin_memory=True)
            mask_p.copy_(torch.from_numpy(mask_h))
            host_pair, host_mask = pinned.numpy(), mask_p.numpy()

            def e2e_step(i):   # the public host-buffer call: pair in, block, pair out
                stack.run(host_pair, host_mask, opts, first_block=i % 2, n_blocks=1, inplace=True)
            h2d = int(pinned.numel() * 4 + mask_p.numel() * 4)
            d2h = int(pinned.numel() * 4)
        else:
            pinned = torch.empty((rows_local, n, C_Z), dtype=pair_dtype, pin_memory=True)
            pinned.copy_(torch.from_numpy(pair_h).reshape(rows_local, n, C_Z).to(pair_dtype))
            target = pair_d if world == 1 else None

            def e2e_step(i):   # each rank: its pinned shard in, the block on the device, its shard out
                dst = target if world == 1 else shard["z"]
                dst.copy_(pinned, non_blocking=True)
                step(i)
                pinned.copy_(target if world == 1 else shard["z"], non_blocking=True)
                torch.cuda.synchronize()
            h2d = int(pinned.numel() * pair_bytes) * world
            d2h = h2d
        e2e_step(0)   # warm the staging arena
        barrier()
        t0 = time.perf_counter()
        for i in range(reps):
            e2e_step(i)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3 / reps
        if world > 1:
            t = torch.tensor([wall], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            wall = float(t.item())
        e2e = {"value": wall, "unit": "ms/block", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        if world == 1 and pair_dtype == torch.float32 and not args.no_pipeline:
            # the same host-buffer call with three pairs in flight (PairStackPipeline: a context per lane), so that one
            # pair's copies overlap another's kernels: every block still has its pair uploaded from and read back
            # into pinned host memory inside the timed region
            lanes, jobs = 3, 12
            buffers = [pinned] + [torch.empty_like(pinned).pin_memory() for _ in range(lanes - 1)]
            for extra_buffer in buffers[1:]:
                extra_buffer.copy_(pinned)
            arrays = [bf.numpy() for bf in buffers]
            pipe = lf.PairStackPipeline(weights, C_Z, C_Z, lanes=lanes, ordinal=local_rank)
            for f in [pipe.submit(a, host_mask, opts, first_block=0, n_blocks=1) for a in arrays]:
                f.result()      # warm every lane's arena
            t0 = time.perf_counter()
            futures = []
            for i in range(jobs):
                if i >= lanes:
                    futures[i - lanes].result()      # the buffer's previous block is back in host memory
                futures.append(pipe.submit(arrays[i % lanes], host_mask, opts, first_block=i % 2, n_blocks=1))
            for f in futures:
                f.result()
            e2e["pipelined_value"] = (time.perf_counter() - t0) * 1e3 / jobs
            e2e["pipelined_note"] = ("%d blocks on %d pinned host pairs through %d lanes of one GPU, wall clock / blocks; value above is one "
                                     "pair at a time" % (jobs, lanes, lanes))
            pipe.close()
            del buffers, arrays

    # the ranks part here: the CPU leg below runs on rank 0 of a single-GPU run only, so nobody waits on it
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        peaks = measured_peaks()
        roofline, roofline_kernels = roofline_table(families, n, world, peaks, pair_bytes)
        cpu = None
        if not args.no_cpu and world == 1:
            cpu = cpu_sample(args.cpu_sample, n)
        line = {
            "metric": "pair_stack_block_ms", "value": ms_per_block, "unit": "ms/block", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_block, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None,
            "dtype": ("f16 operands / f32 accumulate (pair stream %s)" % args.pair_dtype) if args.precision == "bf16" else "f32",
            "data": "synthetic", "config": workload_config(args, world),
            "tflops_block": block_flops(n) / (ms_per_block * 1e-3) / 1e12,
            "roofline": roofline, "roofline_kernels": roofline_kernels, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches),
            "kernel_ms_per_step": {k: v[0] / args.steps for k, v in families.items() if v[1]},
            "clocks": clocks, "finite": finite, "extra": extra, "sharded_check": sharded_check,
        }
        print(json.dumps(line))
    if stack is not None:
        stack.close()


START = time.perf_counter()

if __name__ == "__main__":
    main()
