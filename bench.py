r"""Benchmark of the fused neural-field operators on B200.

    python bench.py --gpus N --steps K --warmup W [--workload NAME] [--impl reference]

Default workload ``train_step`` is benchmark configuration 3: per GPU 2^21 uniform 3-D points ->
hash encoding (16 levels x 2 features, T = 2^19, 16..2048, float16 table) -> fused MLP
32 -> 64 -> 64 -> 16 (ReLU, float16) -> MSE -> backward -> gradient all-reduce (NCCL) -> Adam.
A "step" is one such pass over one batch; ``value`` is points per second over all ranks with the
batch already in HBM; ``e2e`` runs the same step from pinned HOST buffers (coordinates and
targets copied in, the loss copied out, every step, inside the timed region).

Other workloads (``hash`` = configuration 0, ``mlp`` = 1, ``reversible`` = 2, ``contention`` = 4)
time forward + backward of one operator; with N > 1 every rank runs its own batch (no collective).
On one GPU these are timed as CUDA-graph replays of one captured step (``--graph off`` for eager
launches): their device work is shorter than the Python around it.  The per-kernel breakdown and
the roofline always come from an eager pass with CUDA events around every C-ABI call.

One JSON line is printed by rank 0.  ``--impl reference`` times the CPU port of the same step
(``oracle/``: the restatement of the reference's torch CPU path) on the host cores instead, on the
same 2^21-point batch.

The run fails (non-zero exit, no JSON line) when any rank's loss is not finite after a timed leg,
when the optimiser skipped non-finite gradients, or when a tensor-core kernel gave up on a wait.
"""
import argparse
import glob
import json
import math
import os
import re
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "fwd+bwd points/sec (hash-enc + fused MLP)"
TRAIN_POINTS = 2**21  # per GPU per step (benchmark configuration 3)

L2_BYTES = 126 * 1024 * 1024

# ncu figures are not typed in here: a summary under profiles/ that wants one of its captured figures
# quoted beside the timed number carries a line
#   bench-record: workload=<name> entry=<C-ABI entry> dram_bytes_per_launch=<int> l2_requests_per_launch=<int>
#                 l2_sectors_per_launch=<int> tensor_pipe_pct=<float>          (any subset of the four figures)
# and the JSON line names the file it took them from.  No such line -> null.
RECORD = re.compile(r"bench-record:\s*(.*)")


def ncu_records(workload):
    found = {}
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        try:
            text = open(path).read()
        except OSError:
            continue
        for m in RECORD.finditer(text):
            fields = dict(kv.split("=", 1) for kv in m.group(1).split() if "=" in kv)
            if fields.get("workload") == workload and "entry" in fields:
                rec = {"source": os.path.relpath(path, ROOT)}
                for key in ("dram_bytes_per_launch", "l2_requests_per_launch", "l2_sectors_per_launch", "tensor_pipe_pct"):
                    if key in fields:
                        rec[key] = float(fields[key])
                found[fields["entry"]] = rec
    return found


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"], tflops_sustained=p.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


# ---- clocks ------------------------------------------------------------------------------------


class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def __enter__(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL,
            )  # fmt: skip
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if not self.path or not os.path.exists(self.path):
            return out
        clocks, reasons, sm_max = [], set(), None
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    clocks.append(float(parts[0]))
                    sm_max = float(parts[1])
                except ValueError:
                    continue
                for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                    if flag == "Active":
                        reasons.add(name)
        os.unlink(self.path)
        if clocks:
            busy = sorted(clocks)[len(clocks) // 2 :]  # upper half: samples taken under load
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=sm_max, reasons=sorted(reasons), samples=len(clocks))
        return out


# ---- workloads ---------------------------------------------------------------------------------

HASH_CFG = dict(
    hash=dict(points=65536, feats=2, cap=2**19, n_max=2048, dtype=torch.float32, clustered=False),
    contention=dict(points=2**22, feats=4, cap=2**22, n_max=4096, dtype=torch.float32, clustered=True),
)


def hash_bytes_per_point(levels, feats, elem_bytes):
    # coordinates + 2^3 corner rows per level + the [N, L*F] output (forward) or gradient (backward)
    return 12 + levels * 8 * feats * elem_bytes + levels * feats * elem_bytes


def clustered_points(n, gen, device):
    centres = torch.rand(8, 3, device=device, generator=gen) * 0.6 + 0.2
    which = torch.randint(0, 8, (n,), device=device, generator=gen)
    pts = centres[which] + 0.02 * torch.randn(n, 3, device=device, generator=gen)
    return pts.clamp_(0, 1 - 2**-24)


class TrainStep:
    r"""benchmark configuration 3."""

    name = "cfg3: 2^21 pts/GPU, hash L16 F2 T2^19 16..2048 fp16 -> MLP 32-64-64-16 fp16 -> MSE -> allreduce -> Adam"
    dtype = "f16"

    def __init__(self, device, rank, points, args):
        from triton_helpers_b200.layers.fully_fused_mlp import FullyFusedMLP
        from triton_helpers_b200.layers.hash_encoding import HashEncoding
        from triton_helpers_b200.training import NeuralFieldTrainer

        self.device, self.points = device, points
        torch.manual_seed(0)  # identical parameters on every rank
        enc = HashEncoding(2**19, 16, 3, 2, 16, 2048)
        with torch.no_grad():
            enc.embeddings.uniform_(-1e-4, 1e-4)
        mlp = FullyFusedMLP(32, 64, 16, depth=2, bias=False)
        self.trainer = NeuralFieldTrainer(enc.to(device).half(), mlp.to(device).half(), lr=1e-2, betas=(0.9, 0.99), eps=1e-15,
                                          backward_passes=args.backward_passes, fused={"auto": None, "both": True, "backward": "backward", "none": False}[args.fused])
        gen = torch.Generator(device=device).manual_seed(1234 + rank)  # a different batch per rank
        self.coords = torch.rand(points, 3, device=device, generator=gen)
        self.targets = torch.rand(points, 16, device=device, generator=gen).half()
        self.table_elems = enc.embeddings.numel()
        self.units = points
        self.host = None
        self.last_loss = None

    def step(self):
        self.last_loss = self.trainer.step(self.coords, self.targets)
        return self.last_loss

    def skipped(self):
        return self.trainer.skipped_elements()

    def collective_buffer(self):
        return self.trainer._state.flat_grad

    # end to end: batch arrives from pinned host memory, loss goes back
    def prepare_e2e(self):
        # One pinned host buffer and one device buffer per slot hold [coordinates | targets], so a batch
        # crosses the host link as a single copy (two slots: the next batch copies in while this one computes).
        n_coord = self.coords.numel() * 4
        n_target = self.targets.numel() * 2
        self.h2d_bytes = n_coord + n_target
        self.host, self.dev_raw, self.dev = [], [], []
        for _ in range(2):
            host = torch.empty(self.h2d_bytes, dtype=torch.uint8).pin_memory()
            host[:n_coord].view(torch.float32).copy_(self.coords.cpu().reshape(-1))
            host[n_coord:].view(torch.float16).copy_(self.targets.cpu().reshape(-1))
            raw = torch.empty(self.h2d_bytes, dtype=torch.uint8, device=self.device)
            self.host.append(host)
            self.dev_raw.append(raw)
            self.dev.append((raw[:n_coord].view(torch.float32).view_as(self.coords),
                             raw[n_coord:].view(torch.float16).view_as(self.targets)))
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.ready = [torch.cuda.Event() for _ in range(2)]
        self.consumed = [torch.cuda.Event() for _ in range(2)]
        self.loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
        self.d2h_bytes = 4
        self.slot = 0
        self._prefetch(0)

    def _prefetch(self, slot):
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.consumed[slot])
            self.dev_raw[slot].copy_(self.host[slot], non_blocking=True)
            self.ready[slot].record(self.copy_stream)

    def step_e2e(self):
        slot = self.slot
        self._prefetch(slot ^ 1)  # next batch copies in while this one computes
        torch.cuda.current_stream().wait_event(self.ready[slot])
        loss = self.trainer.step(*self.dev[slot])
        self.consumed[slot].record()
        self.loss_host.copy_(loss, non_blocking=True)
        self.slot ^= 1

    def h2d_alone(self, world):
        r"""The batch's host-to-device copy by itself, every rank at once (what the host link gives N ranks):
        GB/s per rank (the slowest rank's) and summed over ranks."""
        copy = lambda: self.dev_raw[0].copy_(self.host[0], non_blocking=True)  # noqa: E731
        for _ in range(3):
            copy()
        reps = 20
        ms = timed_region(copy, reps, world) / reps
        per_rank = self.h2d_bytes / (ms * 1e-3) / 1e9
        return {"ms": ms, "gbs_per_rank": per_rank, "gbs_all_ranks": per_rank * world, "reps": reps}

    def work(self):
        S, n = 2, self.points
        mlp_flops = 2 * (32 * 64 + 64 * 64 + 64 * 16)
        enc = hash_bytes_per_point(16, 2, S) * n
        return {
            "th_hash_fwd": ("hbm", enc),
            "th_hash_bwd": ("hbm", enc),
            "th_field_fwd": ("hbm", enc),   # encoding + MLP forward + loss in one kernel: the encoding's bytes bound it
            "th_field_bwd": ("hbm", enc),   # MLP backward + encoding backward in one kernel
            "th_mlp_fwd": ("tensor", mlp_flops * n),
            "th_mlp_fwd_mse": ("tensor", mlp_flops * n),  # forward with the loss fused into its last layer
            "th_mlp_bwd": ("tensor", 2 * mlp_flops * n),
            "th_mse_grad": ("hbm", 3 * S * 16 * n),
            "th_scale_cast": ("hbm", 6 * 7168),
            "th_adam_step": ("hbm", (3 * S + 16) * self.table_elems),
        }


class HashOnly:
    dtype = "f32"

    def __init__(self, device, rank, key):
        from triton_helpers_b200.layers.hash_encoding import hash_encoding
        self.key = key
        self.allreduce = dist.is_initialized() and dist.get_world_size() > 1 and key == "contention"
        self.kernel_only_ms = None
        from triton_helpers_b200.layers.hash_encoding.helpers import level_geometry

        c = HASH_CFG[key]
        self.c, self.fn, self.device = c, hash_encoding, device
        self.name = (f"cfg{0 if key == 'hash' else 4}: {c['points']} pts, hash L16 F{c['feats']} T{c['cap']} 16..{c['n_max']} "
                     f"fp32 fwd+bwd" + (", 8 Gaussian clusters" if c["clustered"] else ""))  # fmt: skip
        gen = torch.Generator(device=device).manual_seed(rank)
        geo = level_geometry(16, c["cap"], 3, 16, c["n_max"])
        self.x = clustered_points(c["points"], gen, device) if c["clustered"] else torch.rand(c["points"], 3, device=device, generator=gen)
        self.table = ((torch.rand(geo.total_rows, c["feats"], device=device, generator=gen) * 2 - 1) * 1e-4).requires_grad_(True)
        self.go = torch.randn(c["points"], 16 * c["feats"], device=device, generator=gen)
        self.units = c["points"]

    def step(self):
        c = self.c
        out = self.fn(self.x, self.table, None, None, c["cap"], 16, c["n_max"], 16)
        (g,) = torch.autograd.grad(out, self.table, self.go)
        if self.allreduce:
            dist.all_reduce(g)  # cfg 4 data parallel: the 681 MB float32 table gradient, summed over ranks every step
        return g

    def collective_buffer(self):
        return torch.empty_like(self.table) if self.allreduce else torch.empty(0, device=self.device)

    def extra(self):
        # kernel-only number next to the one with the all-reduce
        if not self.allreduce:
            return {}
        self.allreduce = False
        for _ in range(3):
            self.step()
        ms = timed_region(self.step, 10, dist.get_world_size()) / 10
        self.allreduce = True
        return {"kernel_only": {"ms_per_step": ms, "value": self.units * dist.get_world_size() / (ms * 1e-3), "unit": "points/s"}}

    def work(self):
        b = hash_bytes_per_point(16, self.c["feats"], 4) * self.units
        return {"th_hash_fwd": ("hbm", b), "th_hash_bwd": ("hbm", b)}



class MlpOnly:
    name = "cfg1: 2^20 rows, fused MLP 32 -> 4x64 (ReLU) -> 16, fp16, no bias, fwd+bwd"
    dtype = "f16"

    def __init__(self, device, rank):
        from triton_helpers_b200.layers.fully_fused_mlp import fully_fused_mlp

        self.fn = fully_fused_mlp
        gen = torch.Generator(device=device).manual_seed(rank)
        rows = 2**20
        lin = lambda o, i: ((torch.rand(o, i, device=device, generator=gen) * 2 - 1) / i**0.5).half().requires_grad_(True)  # noqa: E731
        self.w = [lin(64, 32), lin(16, 64), lin(192, 64)]
        self.x = torch.randn(1, rows, 32, device=device, generator=gen).half().requires_grad_(True)
        self.go = (torch.randn(1, rows, 16, device=device, generator=gen) * 1e-2).half()
        self.units = rows

    def step(self):
        y = self.fn(self.x, self.w[0], None, self.w[1], None, self.w[2], None)
        return torch.autograd.grad(y, [self.x, *self.w], self.go)

    def work(self):
        f = 2 * (32 * 64 + 3 * 64 * 64 + 64 * 16) * self.units
        return {"th_mlp_fwd": ("tensor", f), "th_mlp_bwd": ("tensor", 2 * f)}



class ReversibleOnly:
    name = "cfg2: 2^20 rows x 128 bf16, 8 coupling blocks of 64 -> 64 -> 64 (ReLU), fwd+bwd with reconstruction"
    dtype = "bf16"

    def __init__(self, device, rank):
        from triton_helpers_b200.layers.reversible_mlp import reversible_mlp

        self.fn = reversible_mlp
        gen = torch.Generator(device=device).manual_seed(rank)
        rows = 2**20
        lin = lambda: ((torch.rand(512, 64, device=device, generator=gen) * 2 - 1) / 8).bfloat16().requires_grad_(True)  # noqa: E731
        self.w = [lin() for _ in range(4)]
        self.x = torch.randn(rows, 128, device=device, generator=gen).bfloat16().requires_grad_(True)
        self.go = torch.randn(rows, 128, device=device, generator=gen).bfloat16()
        self.units = rows

    def step(self):
        y = self.fn(self.x, *self.w)
        return torch.autograd.grad(y, [self.x, *self.w], self.go)

    def work(self):
        f = 8 * 4 * 2 * 64 * 64 * self.units
        return {"th_rev_fwd": ("tensor", f), "th_rev_bwd": ("tensor", 2 * f)}



def build_workload(name, device, rank, args):
    if name == "train_step":
        return TrainStep(device, rank, TRAIN_POINTS, args)
    if name in HASH_CFG:
        return HashOnly(device, rank, name)
    if name == "mlp":
        return MlpOnly(device, rank)
    if name == "reversible":
        return ReversibleOnly(device, rank)
    raise SystemExit(f"unknown workload {name}")


# ---- CPU arm -----------------------------------------------------------------------------------


def cpu_training_step_rate(steps, warmup, points):
    r"""points/s of the CPU port of the training step on all host threads."""
    from oracle.training_step import CpuNeuralField, make_batch

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    model = CpuNeuralField()
    coords, targets = make_batch(points)
    for _ in range(warmup):
        model.step(coords, targets)
    t0 = time.perf_counter()
    for _ in range(steps):
        model.step(coords, targets)
    dt = time.perf_counter() - t0
    return points * steps / dt, threads, dt / steps * 1e3


def cpu_operator_rate(workload):
    r"""(units/s, threads, sample text) of the CPU oracle of one operator's forward + backward, bounded sample."""
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    if workload in HASH_CFG:
        from oracle import hash_encoding as oracle

        c = HASH_CFG[workload]
        n = 2**16
        kw = dict(table_cap=c["cap"], levels=16, n_min=16, n_max=c["n_max"])
        rows = sum(oracle.level_rows(16, c["cap"], 3, 16, c["n_max"]))
        table = (torch.rand(rows, c["feats"], generator=g) * 2 - 1) * 1e-4
        x, go = torch.rand(n, 3, generator=g), torch.randn(n, 16 * c["feats"], generator=g)
        fn = lambda: (oracle.encode(x, table, **kw), oracle.encode_backward(x, go, table, **kw))  # noqa: E731
        sample = f"{n} uniform points, float32 table of {rows} rows (the reference's CPU path restated in oracle/)"
    elif workload == "mlp":
        from oracle import fused_mlp as oracle

        n = 2**18
        lin = lambda o, i: (torch.rand(o, i, generator=g) * 2 - 1) / i**0.5  # noqa: E731
        w = (lin(64, 32), lin(16, 64), lin(192, 64))
        x, go = torch.randn(1, n, 32, generator=g), torch.randn(1, n, 16, generator=g) * 1e-2
        fn = lambda: oracle.forward_backward(x, w[0], None, w[1], None, w[2], None, go)  # noqa: E731
        sample = f"{n} rows, float32 F.linear chain with autograd (oracle/)"
    else:
        from oracle import reversible_mlp as oracle

        n = 2**16
        w = tuple((torch.rand(512, 64, generator=g) * 2 - 1) / 8 for _ in range(4))
        x, go = torch.randn(n, 128, generator=g), torch.randn(n, 128, generator=g)
        fn = lambda: oracle.forward_backward(x, w, (None,) * 4, go)  # noqa: E731
        sample = f"{n} rows, float32 autograd with stored activations (oracle/)"
    fn()
    t0, reps = time.perf_counter(), 0
    while reps < 3 or (time.perf_counter() - t0 < 5 and reps < 50):
        fn()
        reps += 1
    return n * reps / (time.perf_counter() - t0), threads, sample


def workload_config(name):
    r"""The `config` object of the JSON line: identical for the GPU arm and the CPU arm of a workload."""
    return {
        "workload": name,
        "units_per_gpu_per_step": TRAIN_POINTS,
        "l2": "per-step inputs and intermediates (25 MB coordinates, 67 MB targets, 134 MB features per step) exceed "
              "the 126 MB L2; no explicit flush",
    }  # fmt: skip


def run_reference(args, rank):
    r"""The CPU arm: the float32 port of the same step, all host threads.  A step of the GPU arm's 2^21 points takes
    a few seconds; when K + W such steps would run beyond a few minutes, every step takes a smaller power-of-two
    sample of the batch instead (the rate is per point, and the line says which sample was timed)."""
    if rank != 0:
        return
    probe = 2**17
    probe_rate, _, _ = cpu_training_step_rate(1, 1, probe)
    budget_s = 150.0
    points = TRAIN_POINTS
    while points > 2**16 and (args.steps + args.warmup) * points / probe_rate > budget_s:
        points //= 2
    rate, threads, ms = cpu_training_step_rate(args.steps, args.warmup, points)
    sample = (f"{args.steps} steps of {points} points" +
              (" (the GPU arm's batch per GPU)" if points == TRAIN_POINTS else
               f" (a sample of the GPU arm's {TRAIN_POINTS}-point batch, sized so that the run ends within a few minutes)"))
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": "points/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(TrainStep.name),
        "arm": "CPU port of the same step (oracle/: the reference's torch CPU path restated), float32, host cores only; "
               "rank 0 alone runs it",
        "cpu_baseline": {"value": rate, "unit": "points/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": rate, "unit": "points/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


# ---- GPU arm -----------------------------------------------------------------------------------


def timed_region(fn, steps, world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    ms = torch.tensor([start.elapsed_time(stop)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.barrier()
    return float(ms)


def step_quantiles(fn, reps, world):
    r"""Per-step device times of `reps` more steps (CUDA events around each): the reference harness's
    statistic - median with the 20th and 80th percentile (triton_helpers/benchmark.py:153) - max over ranks
    per percentile."""
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    events = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
    events[0].record()
    for i in range(reps):
        fn()
        events[i + 1].record()
    torch.cuda.synchronize()
    times = sorted(events[i].elapsed_time(events[i + 1]) for i in range(reps))
    pick = lambda q: times[min(reps - 1, int(q * reps))]  # noqa: E731
    q = torch.tensor([pick(0.2), pick(0.5), pick(0.8)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(q, op=dist.ReduceOp.MAX)
    return {"reps": reps, "p20_ms": float(q[0]), "median_ms": float(q[1]), "p80_ms": float(q[2])}


def collective_alone(buffer, reps, world):
    r"""The step's one collective by itself: all-reduce of the flat gradient buffer, CUDA events, max over ranks."""
    scratch = torch.zeros_like(buffer)
    for _ in range(5):
        dist.all_reduce(scratch)
    ms = timed_region(lambda: dist.all_reduce(scratch), reps, world) / reps
    nbytes = scratch.numel() * scratch.element_size()
    return {"bytes": nbytes, "ms": ms, "reps": reps, "algbw_gbs": nbytes / (ms * 1e-3) / 1e9,
            "busbw_gbs": nbytes * 2 * (world - 1) / world / (ms * 1e-3) / 1e9}  # fmt: skip


def health(world, device, losses, skipped):
    r"""Stops the run when a loss is not finite on any rank, Adam skipped elements, or a tensor-core kernel
    reported a wait that ran out."""
    from triton_helpers_b200 import _lib

    lib = _lib.lib()
    flags = torch.tensor([int(any(not math.isfinite(v) for v in losses)), int(bool(skipped)),
                          int(lib.th_mlp_tc_status() != 0 or lib.th_rev_tc_status() != 0 or lib.th_hash_status() != 0)],
                         dtype=torch.int32, device=device)  # fmt: skip
    if world > 1:
        dist.all_reduce(flags, op=dist.ReduceOp.MAX)  # NCCL has no bitwise reductions: one 0/1 flag per reason
    bad = [bool(v) for v in flags.tolist()]
    if any(bad):
        reasons = [text for hit, text in zip(bad, ("a loss is not finite", "Adam skipped non-finite gradients",
                                                   "a tensor-core or encoding kernel gave up on a wait")) if hit]  # fmt: skip
        raise SystemExit(f"bench.py: invalid run on at least one rank: {'; '.join(reasons)} (losses here: {losses})")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_step", choices=["train_step", "hash", "mlp", "reversible", "contention"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--fused", default="auto", choices=["auto", "both", "backward", "none"],
                    help="train_step: which passes run in the kernels that fuse encoding and MLP (auto: the trainer's default)")
    ap.add_argument("--backward-passes", type=int, default=None,
                    help="train_step: run the encoding backward in this many level ranges with the gradient sums overlapped")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="time CUDA-graph replays of the step (auto: single-operator workloads on one GPU)")
    ap.add_argument("--quantile-reps", type=int, default=100, help="extra steps timed one by one for median / p20 / p80")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    from triton_helpers_b200 import _lib
    from triton_helpers_b200.parallel import init_from_env

    rank, world, local_rank = init_from_env("nccl")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the CUDA extension is the only compute path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    _lib.lib()  # fail loudly here if the extension is missing

    wl = build_workload(args.workload, device, rank, args)
    is_train = args.workload == "train_step"
    # the sampler starts before the warm-up (nvidia-smi takes ~100 ms to deliver its first line);
    # the busier half of its samples is what gets summarised
    use_graph = args.graph == "on" or (args.graph == "auto" and world == 1 and not is_train)
    timing = ("eager launches, CUDA events around the K timed steps; per-kernel times from a second pass of K steps "
              "with CUDA events around every C-ABI call (the extra events cost 2-3 % of the step)")
    losses = []
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.warmup):
            wl.step()
        torch.cuda.synchronize()
        launches_before = _lib.lib().th_launch_count()
        total_ms = timed_region(wl.step, args.steps, world)
        launches = _lib.lib().th_launch_count() - launches_before
        if is_train:
            losses.append(float(wl.last_loss))  # the loss of the last device-timed step
        with _lib.KernelTimer() as timer:
            timed_region(wl.step, args.steps, world)
        kernels = timer.summary()
        graph = None
        if use_graph:
            # The single-operator steps are tens of microseconds of GPU work behind hundreds of
            # microseconds of Python: replaying a captured step measures the kernels, the eager pass
            # above keeps the per-kernel CUDA-event breakdown.
            try:
                side = torch.cuda.Stream(device=device)
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    wl.step()
                torch.cuda.current_stream().wait_stream(side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    wl.step()
                for _ in range(args.warmup):
                    graph.replay()
                total_ms = timed_region(graph.replay, args.steps, world)
                timing = "CUDA-graph replays of one captured step, CUDA events around the timed replays; per-kernel times from an eager pass"
            except Exception as exc:  # noqa: BLE001  (report and keep the eager number)
                graph = None
                timing += f" (graph capture failed: {type(exc).__name__}: {exc})"[:300]
        quantiles = step_quantiles(graph.replay if graph is not None else wl.step, max(args.quantile_reps, 1), world)
        if is_train:
            losses.append(float(wl.last_loss))
    clock_summary = clocks.summary()
    ms_per_step = total_ms / args.steps
    value = wl.units * world / (ms_per_step * 1e-3)

    # per entry point: launches, time, share; roofline of the one that takes the most time
    peaks = measured_peaks()
    work = wl.work()
    in_kernels = sum(t for _, t in kernels.values()) or 1.0
    breakdown = {k: {"calls": c, "ms_per_step": t / args.steps, "share": t / in_kernels} for k, (c, t) in kernels.items()}
    top = max(kernels, key=lambda k: kernels[k][1])
    bound, amount = work[top]
    calls, top_ms = kernels[top]
    per_launch_s = top_ms / calls * 1e-3
    per_launch_amount = amount * (args.steps / calls)
    if bound == "hbm":
        achieved, peak, unit = per_launch_amount / per_launch_s / 1e9, peaks["hbm_gbs"], "GB/s"
    else:
        achieved, peak, unit = per_launch_amount / per_launch_s / 1e12, peaks["tflops"], "TFLOP/s"
    records = ncu_records(args.workload)
    record = records.get(top, {})
    # ncu figures of every entry point that has a summary: DRAM and L2 GB/s over this run's launch time, tensor-pipe
    # utilisation as captured
    for entry, info in breakdown.items():
        rec = records.get(entry)
        if not rec:
            continue
        launch_s = kernels[entry][1] / kernels[entry][0] * 1e-3
        ncu = {"source": rec["source"]}
        if "dram_bytes_per_launch" in rec:
            ncu["dram_gbs"] = rec["dram_bytes_per_launch"] / launch_s / 1e9
        if "l2_sectors_per_launch" in rec:
            ncu["l2_gbs"] = rec["l2_sectors_per_launch"] * 32 / launch_s / 1e9
        if "tensor_pipe_pct" in rec:
            ncu["tensor_pipe_pct"] = rec["tensor_pipe_pct"]
        info["ncu"] = ncu
    roofline = {"kernel": top, "bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                "traffic": record.get("dram_bytes_per_launch"), "traffic_source": record.get("source"),
                "peak_source": peaks["source"], "algorithmic_per_launch": per_launch_amount,
                "ms_per_launch": per_launch_s * 1e3}  # fmt: skip
    # The encoding kernels of cfg 0 / 3 run out of L2 (the table never leaves it): what bounds them is the
    # SM-to-L2 request path, one request per clock per SM.  Requests per launch come from the ncu summary
    # the record names; the ceiling uses this run's own SM clock.
    request_roofline = None
    if record.get("l2_requests_per_launch") and clock_summary.get("sm_mhz"):
        ceiling = torch.cuda.get_device_properties(device).multi_processor_count * clock_summary["sm_mhz"] * 1e6
        rate = record["l2_requests_per_launch"] / per_launch_s
        request_roofline = {"kernel": top, "bound": "sm_to_l2_requests", "achieved": rate / 1e9, "peak": ceiling / 1e9,
                            "unit": "G requests/s", "frac": rate / ceiling, "requests_per_launch": record["l2_requests_per_launch"],
                            "source": record["source"],
                            "peak_source": "SM count x median SM clock of this run (one L2 request per clock per SM)"}  # fmt: skip

    e2e = None
    if hasattr(wl, "prepare_e2e"):
        wl.prepare_e2e()
        for _ in range(args.warmup):
            wl.step_e2e()
        e2e_ms = timed_region(wl.step_e2e, args.steps, world) / args.steps
        losses.append(float(wl.loss_host[0]))
        e2e = {"value": wl.units * world / (e2e_ms * 1e-3), "unit": "points/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes,
               "last_loss": float(wl.loss_host[0]), "h2d_alone": wl.h2d_alone(world)}  # fmt: skip

    health(world, device, losses, wl.skipped() if is_train else 0)

    collective = None
    if world > 1 and hasattr(wl, "collective_buffer"):
        collective = collective_alone(wl.collective_buffer(), 100, world)

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and is_train:
        rate, threads, _ = cpu_training_step_rate(steps=2, warmup=1, points=TRAIN_POINTS)
        cpu_baseline = {"value": rate, "unit": "points/s", "cores": threads, "kind": "port",
                        "sample": f"2 steps (after 1 warm-up) of {TRAIN_POINTS} points, float32 CPU port of the same step (oracle/)"}  # fmt: skip
    elif rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, threads, sample = cpu_operator_rate(args.workload)
        cpu_baseline = {"value": rate, "unit": "points/s", "cores": threads, "kind": "port", "sample": sample}

    extra = wl.extra() if hasattr(wl, "extra") else {}  # may time more steps: every rank takes part
    if rank == 0:
        config = workload_config(wl.name)
        config["units_per_gpu_per_step"] = wl.units
        if args.workload == "hash":
            config["l2"] = "table (48.8 MB) is meant to stay L2 resident; no flush"
        line = {
            "metric": METRIC, "value": value, "unit": "points/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": config, "timing": timing,
            "step_quantiles": quantiles, "clocks": clock_summary, "e2e": e2e, "gpu_launches": launches,
            "roofline": roofline, "roofline_l2_requests": request_roofline, "kernels": breakdown,
            "collective_alone": collective, "cpu_baseline": cpu_baseline,
            "last_loss": losses[0] if losses else None,
        }  # fmt: skip
        line.update(extra)
        print(json.dumps(line, allow_nan=False), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
