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
(``oracle/``: the restatement of the reference's torch CPU path) on the host cores instead.
"""
import argparse
import json
import os
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

# dram__bytes_read.sum + dram__bytes_write.sum per launch, from the ncu captures summarised under
# profiles/ (hash_bwd_kernel_cfg3.md, hash_fwd_kernel_cfg3.md, mlp_bwd_pipe_kernel_cfg3.md,
# mlp_fwd_pipe_kernel_cfg3.md), all taken on the full cfg 3 workload; th_hash_bwd is the sum of its two
# kernels.  Other workloads have no capture yet: traffic is reported as null there.
NCU_TRAFFIC_BYTES = {
    "train_step": {"th_hash_bwd": 355.9e6, "th_hash_fwd": 131.4e6, "th_mlp_bwd": 298.8e6, "th_mlp_fwd": 174.6e6, "th_mlp_fwd_mse": 239.9e6},
}
L2_BYTES = 126 * 1024 * 1024


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

    def __init__(self, device, rank, points, backward_passes=None):
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
                                          backward_passes=backward_passes)
        gen = torch.Generator(device=device).manual_seed(1234 + rank)  # a different batch per rank
        self.coords = torch.rand(points, 3, device=device, generator=gen)
        self.targets = torch.rand(points, 16, device=device, generator=gen).half()
        self.table_elems = enc.embeddings.numel()
        self.units = points
        self.gathers_per_step = points * 16 * 8  # one table row per corner per level
        self.host = None

    def step(self):
        return self.trainer.step(self.coords, self.targets)

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

    def work(self):
        S, n = 2, self.points
        mlp_flops = 2 * (32 * 64 + 64 * 64 + 64 * 16)
        return {
            "th_hash_fwd": ("hbm", hash_bytes_per_point(16, 2, S) * n),
            "th_hash_bwd": ("hbm", hash_bytes_per_point(16, 2, S) * n),
            "th_mlp_fwd": ("tensor", mlp_flops * n),
            "th_mlp_fwd_mse": ("tensor", mlp_flops * n),  # forward with the loss fused into its last layer
            "th_mlp_bwd": ("tensor", 2 * mlp_flops * n),
            "th_mse_grad": ("hbm", 3 * S * 16 * n),
            "th_adam_step": ("hbm", (3 * S + 16) * self.table_elems),
        }



class HashOnly:
    dtype = "f32"

    def __init__(self, device, rank, key):
        from triton_helpers_b200.layers.hash_encoding import hash_encoding
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
        self.gathers_per_step = c["points"] * 16 * 8

    def step(self):
        c = self.c
        out = self.fn(self.x, self.table, None, None, c["cap"], 16, c["n_max"], 16)
        (g,) = torch.autograd.grad(out, self.table, self.go)
        return g

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



def build_workload(name, device, rank, backward_passes=None):
    if name == "train_step":
        return TrainStep(device, rank, 2**21, backward_passes)
    if name in HASH_CFG:
        return HashOnly(device, rank, name)
    if name == "mlp":
        return MlpOnly(device, rank)
    if name == "reversible":
        return ReversibleOnly(device, rank)
    raise SystemExit(f"unknown workload {name}")


# ---- CPU arm -----------------------------------------------------------------------------------


def cpu_training_step_rate(steps, warmup, points):
    r"""points/s of the CPU port of the training step on all host threads (bounded sample)."""
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


def run_reference(args, rank):
    if rank != 0:
        return
    points = 2**16
    rate, threads, ms = cpu_training_step_rate(args.steps, args.warmup, points)
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": "points/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": TrainStep.name, "arm": "CPU port of the same step (oracle/), float32, host cores only"},
        "cpu_baseline": {"value": rate, "unit": "points/s", "cores": threads, "kind": "port",
                         "sample": f"{points} points per step (the GPU arm uses 2^21 per GPU)"},
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


def l2_probe(device):
    r"""What the L2 delivers for the encoding's two access patterns, measured with ``th_probe_l2`` on a
    24 MB buffer (the size of the cfg 3 float16 table): coalesced streaming reads in GB/s, random
    32-byte-sector gathers and random float16-pair reductions in 1e9 per second.  CUDA events on the
    launching stream."""
    import ctypes

    from triton_helpers_b200 import _lib

    buf = torch.empty(24 * 2**20, dtype=torch.uint8, device=device).random_(0, 255)
    sink = torch.zeros(1, dtype=torch.int32, device=device)
    lib, stream = _lib.lib(), _lib.stream_ptr(device)
    out = {}
    for mode, iters, key, scale in ((0, 40, "stream_gbs", 1e9), (1, 64, "gather_g_per_s", 1e9), (2, 64, "update_g_per_s", 1e9)):
        work = ctypes.c_int64(0)
        call = lambda: _lib.check(lib.th_probe_l2(buf.data_ptr(), buf.numel(), mode, iters, sink.data_ptr(), ctypes.byref(work), stream), "th_probe_l2")  # noqa: E731
        for _ in range(3):
            call()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(5):
            call()
        stop.record()
        torch.cuda.synchronize()
        out[key] = work.value * 5 / (start.elapsed_time(stop) * 1e-3) / scale
    out["buffer_mb"] = 24
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="train_step", choices=["train_step", "hash", "mlp", "reversible", "contention"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--backward-passes", type=int, default=None,
                    help="train_step: run the encoding backward in this many level ranges with the gradient sums overlapped")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="time CUDA-graph replays of the step (auto: single-operator workloads on one GPU)")
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

    wl = build_workload(args.workload, device, rank, args.backward_passes)
    # the sampler starts before the warm-up (nvidia-smi takes ~100 ms to deliver its first line);
    # the busier half of its samples is what gets summarised
    use_graph = args.graph == "on" or (args.graph == "auto" and world == 1 and args.workload != "train_step")
    timing = ("eager launches, CUDA events around the K timed steps; per-kernel times from a second pass of K steps "
              "with CUDA events around every C-ABI call (the extra events cost 2-3 % of the step)")
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.warmup):
            wl.step()
        torch.cuda.synchronize()
        launches_before = _lib.lib().th_launch_count()
        total_ms = timed_region(wl.step, args.steps, world)
        launches = _lib.lib().th_launch_count() - launches_before
        with _lib.KernelTimer() as timer:
            timed_region(wl.step, args.steps, world)
        kernels = timer.summary()
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
                timing += f" (graph capture failed: {type(exc).__name__}: {exc})"[:300]
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
    if bound == "hbm":
        achieved, peak, unit = amount * (args.steps / calls) / per_launch_s / 1e9, peaks["hbm_gbs"], "GB/s"
    else:
        achieved, peak, unit = amount * (args.steps / calls) / per_launch_s / 1e12, peaks["tflops"], "TFLOP/s"
    roofline = {"kernel": top, "bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                "traffic": NCU_TRAFFIC_BYTES.get(args.workload, {}).get(top), "peak_source": peaks["source"], "algorithmic_per_launch": amount * (args.steps / calls),
                "ms_per_launch": per_launch_s * 1e3}  # fmt: skip

    e2e = None
    if hasattr(wl, "prepare_e2e"):
        wl.prepare_e2e()
        for _ in range(args.warmup):
            wl.step_e2e()
        e2e_ms = timed_region(wl.step_e2e, args.steps, world) / args.steps
        e2e = {"value": wl.units * world / (e2e_ms * 1e-3), "unit": "points/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes,
               "last_loss": float(wl.loss_host[0])}  # fmt: skip

    # the encoding kernels run out of L2 (cfg 0 / 3): put the cache's own figures beside the HBM roofline
    l2 = None
    if rank == 0 and args.workload in ("train_step", "hash", "contention"):
        l2 = l2_probe(device)
        fwd = kernels.get("th_hash_fwd")
        if fwd and hasattr(wl, "gathers_per_step"):
            l2["hash_fwd_gather_g_per_s"] = wl.gathers_per_step * args.steps / (fwd[1] * 1e-3) / 1e9
            l2["hash_fwd_frac_of_gather_probe"] = l2["hash_fwd_gather_g_per_s"] / l2["gather_g_per_s"]
        bwd = kernels.get("th_hash_bwd")
        if bwd and hasattr(wl, "gathers_per_step"):
            l2["hash_bwd_update_g_per_s"] = wl.gathers_per_step * args.steps / (bwd[1] * 1e-3) / 1e9
            l2["hash_bwd_frac_of_update_probe"] = l2["hash_bwd_update_g_per_s"] / l2["update_g_per_s"]

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and args.workload == "train_step":
        points = 2**17
        rate, threads, _ = cpu_training_step_rate(steps=8, warmup=1, points=points)
        cpu_baseline = {"value": rate, "unit": "points/s", "cores": threads, "kind": "port",
                        "sample": f"8 steps of {points} points, float32 CPU port of the same step (oracle/)"}  # fmt: skip
    elif rank == 0 and world == 1 and not args.no_cpu_baseline:
        rate, threads, sample = cpu_operator_rate(args.workload)
        cpu_baseline = {"value": rate, "unit": "points/s", "cores": threads, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "points/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": {"workload": wl.name, "units_per_gpu_per_step": wl.units,
                       "l2": "per-step inputs and intermediates exceed the 126 MB L2; no explicit flush"
                       if args.workload != "hash" else "table (48.8 MB) is meant to stay L2 resident; no flush",
                       "timing": timing},
            "clocks": clock_summary, "e2e": e2e, "gpu_launches": launches,
            "roofline": roofline, "l2_probe": l2, "kernels": breakdown, "cpu_baseline": cpu_baseline,
        }  # fmt: skip
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
