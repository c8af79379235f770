r"""Command-line harness for timing the fused operators against baselines.

Stands in for ``triton_helpers/benchmark.py``: the same two verbs (``benchmark``, ``profile``), the
same flags (``-p`` providers, ``-m`` modes, ``-d`` dtypes, ``-w`` warm-up, ``-r`` repetitions, ``-l``
line argument, ``-x`` x dimension, ``-o`` output directory, one flag per dimension with a
``--<dim>-mode`` of ``values`` / ``linspace`` / ``logspace``), the same statistic (median with the
20th and 80th percentile, reference :153) and the same result files: one CSV per chart named
``<task>-<mode>-<dim=value-...>-<dtype>.csv`` whose first column is the x dimension and whose other
columns are the title-cased line names (reference :410-412 and the files under
``triton_helpers/layers/*/benchmarks``).  A PNG of each chart is written next to its CSV when
matplotlib is importable.

What differs: timing uses CUDA events around every repetition on the current stream (an L2-sized
buffer is overwritten between repetitions) instead of ``triton.testing.do_bench``, and the kernels an
executor wraps are this package's CUDA kernels.

    python -m triton_helpers_b200.layers.hash_encoding benchmark -m fwd bwd -d fp16 -o out/
    python -m triton_helpers_b200.layers.fully_fused_mlp benchmark -m fwd-bwd -d fp16 bf16 -L 65536 1048576
"""
import argparse
import csv
import itertools
from dataclasses import dataclass, field
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch
from torch import Tensor


class Dtype(str, Enum):
    FP16 = "fp16"
    BF16 = "bf16"
    FP32 = "fp32"

    def __str__(self) -> str:
        return self.value

    @property
    def torch(self) -> torch.dtype:
        return {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[self.value]


class Mode(str, Enum):
    FORWARD = "fwd"
    BACKWARD = "bwd"
    FORWARD_BACKWARD = "fwd-bwd"

    def __str__(self) -> str:
        return self.value

    @property
    def long_name(self) -> str:
        return {"fwd": "Forward", "bwd": "Backward", "fwd-bwd": "Forward-Backward"}[self.value]


def dimension_values(values: Sequence[int], mode: str) -> List[int]:
    r"""``values``: as given; ``linspace``: ``(start, stop, step)`` inclusive; ``logspace``: ``(start, stop, steps)``
    exponents of two."""
    if mode == "values":
        return [int(v) for v in values]
    start, stop, step = (int(v) for v in values)
    if mode == "linspace":
        return list(range(start, stop + 1, step))
    if mode == "logspace":
        return torch.logspace(start, stop, step, base=2).int().tolist()
    raise ValueError(f"Unsupported mode {mode}")


@dataclass
class KernelExecutor:
    r"""One line of a chart: builds inputs for a point of the dimension grid and runs the operator.

    Subclasses implement ``prepare_inputs(**dims, dtype=..., device=..., requires_grad=...) -> kwargs`` and
    ``forward(**kwargs) -> Tensor``; ``backward`` and ``prepare_backward`` may be overridden.
    """

    provider: str
    warmup: int = 20
    rep: int = 100
    quantiles: Tuple[float, float, float] = (0.5, 0.2, 0.8)

    def __str__(self) -> str:
        return self.provider.title()

    def prepare_inputs(self, *, requires_grad: bool = False, **kwargs) -> Dict[str, Any]:
        raise NotImplementedError

    def forward(self, **kwargs) -> Tensor:
        raise NotImplementedError

    def prepare_backward(self, forward_output: Any) -> Tensor:
        if not isinstance(forward_output, Tensor):
            raise TypeError(f"override prepare_backward to pick a tensor out of {type(forward_output)}")
        return forward_output

    def backward(self, output: Tensor, do: Tensor) -> None:
        output.backward(do, retain_graph=True)

    def closure(self, mode: Mode, dtype: Dtype, **dims) -> Callable[[], Any]:
        if mode == Mode.FORWARD:
            inputs = self.prepare_inputs(**dims, dtype=dtype.torch, requires_grad=False)
            return lambda: self.forward(**inputs)
        inputs = self.prepare_inputs(**dims, dtype=dtype.torch, requires_grad=True)
        if mode == Mode.BACKWARD:
            output = self.prepare_backward(self.forward(**inputs))
            do = torch.randn_like(output)
            return lambda: self.backward(output, do)

        def both():
            output = self.prepare_backward(self.forward(**inputs))
            self.backward(output, torch.randn_like(output))
            return output

        return both

    def benchmark(self, mode: Mode, dtype: Dtype, **dims) -> Tuple[float, float, float]:
        r"""(median, 20th percentile, 80th percentile) in milliseconds over ``rep`` repetitions."""
        fn = self.closure(mode, dtype, **dims)
        device = dims.get("device", "cuda")
        flush = torch.empty(160 * 2**20, dtype=torch.uint8, device=device)  # larger than the 126 MB L2
        for _ in range(self.warmup):
            fn()
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(self.rep)]
        for start, stop in events:
            flush.zero_()
            start.record()
            fn()
            stop.record()
        torch.cuda.synchronize()
        times = torch.tensor([a.elapsed_time(b) for a, b in events], dtype=torch.float64)
        q = torch.quantile(times, torch.tensor(self.quantiles, dtype=torch.float64))
        return float(q[0]), float(q[1]), float(q[2])

    def profile(self, mode: Mode, dtype: Dtype, **dims) -> None:
        r"""Warm up, then run once inside a profiler range (cudaProfilerStart / NVTX), for ``ncu --profile-from-start off``."""
        fn = self.closure(mode, dtype, **dims)
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStart()
        torch.cuda.nvtx.range_push(f"{self.provider}-{mode}-{dtype}")
        fn()
        torch.cuda.nvtx.range_pop()
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()


@dataclass
class Chart:
    r"""One result table: rows over the x dimension, one column per line."""

    name: str
    x_name: str
    x_values: List[int]
    line_names: List[str]
    y_label: str
    rows: List[List[float]] = field(default_factory=list)  # medians, [x][line]
    spread: List[List[Tuple[float, float]]] = field(default_factory=list)

    def save(self, directory: Path) -> Path:
        path = directory / f"{self.name}.csv"
        with open(path, "w", newline="") as f:
            writer = csv.writer(f)
            writer.writerow([self.x_name, *self.line_names])
            for x, row in zip(self.x_values, self.rows):
                writer.writerow([f"{float(x):.1f}", *(f"{v:.4f}" for v in row)])
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except ImportError:
            return path
        fig, ax = plt.subplots()
        for i, line in enumerate(self.line_names):
            ax.plot(self.x_values, [r[i] for r in self.rows], label=line)
            ax.fill_between(self.x_values, [s[i][0] for s in self.spread], [s[i][1] for s in self.spread], alpha=0.15)
        ax.set_xlabel(self.x_name)
        ax.set_ylabel(self.y_label)
        ax.legend()
        fig.savefig(directory / f"{self.name}.png")
        plt.close(fig)
        return path

    def __str__(self) -> str:
        width = max(len(n) for n in [self.x_name, *self.line_names]) + 2
        lines = [self.name, "".join(n.rjust(width) for n in [self.x_name, *self.line_names])]
        for x, row in zip(self.x_values, self.rows):
            lines.append(str(x).rjust(width) + "".join(f"{v:.4f}".rjust(width) for v in row))
        return "\n".join(lines)


@dataclass
class CLI:
    task: str
    kernels: Sequence[KernelExecutor]
    dims: Dict[str, List[int]]
    modes: Sequence[Mode] = (Mode.FORWARD,)
    dtypes: Sequence[Dtype] = (Dtype.FP16,)
    line_arg: str = "kernel"
    x_dim: Optional[str] = None
    output: Optional[Path] = None
    device: str = "cuda"

    def charts(self) -> List[Tuple[Chart, List[Dict[str, Any]]]]:
        r"""Every chart with, per line, the fixed arguments of that line.  The x dimension runs along the rows, the
        line argument along the columns, every other factor (kernel, mode, dtype, other dimensions) makes a chart
        of its own - named ``<task>[-<kernel>]-<mode>-<dim=value...>-<dtype>`` as the reference does."""
        x_dim = self.x_dim or next(iter(self.dims))
        factors: Dict[str, List[Any]] = {"kernel": list(self.kernels), "mode": list(self.modes), "dtype": list(self.dtypes)}
        for name, values in self.dims.items():
            if name != x_dim:
                factors[name] = list(values)
        if self.line_arg not in factors:
            raise ValueError(f"line argument {self.line_arg} is not one of {list(factors)}")
        line_values = factors.pop(self.line_arg)
        out = []
        for combo in itertools.product(*factors.values()):
            fixed = dict(zip(factors.keys(), combo))
            dim_name = "-".join(f"{k}={v}" for k, v in fixed.items() if k not in ("kernel", "mode", "dtype"))
            parts = [self.task, str(fixed["kernel"]) if "kernel" in fixed else None, str(fixed["mode"]) if "mode" in fixed else None,
                     dim_name or None, str(fixed["dtype"]) if "dtype" in fixed else None]  # fmt: skip
            chart = Chart("-".join(p for p in parts if p), x_dim, list(self.dims[x_dim]), [str(v) for v in line_values], "Latency (ms)")
            out.append((chart, [{**fixed, self.line_arg: v} for v in line_values]))
        return out

    def run(self, endpoint: str) -> List[Chart]:
        done = []
        for chart, lines in self.charts():
            for x in chart.x_values:
                medians, spread = [], []
                for args in lines:
                    args = dict(args)
                    kernel, mode, dtype = args.pop("kernel"), args.pop("mode"), args.pop("dtype")
                    point = {**args, chart.x_name: x, "device": self.device}
                    if endpoint == "profile":
                        kernel.profile(mode, dtype, **point)
                        continue
                    ms, lo, hi = kernel.benchmark(mode, dtype, **point)
                    medians.append(ms)
                    spread.append((lo, hi))
                if endpoint == "benchmark":
                    chart.rows.append(medians)
                    chart.spread.append(spread)
            if endpoint == "benchmark":
                print(chart, flush=True)
                if self.output is not None:
                    chart.save(self.output)
                done.append(chart)
        return done

    @classmethod
    def entrypoint(
        cls,
        task: str,
        kernels: Sequence[KernelExecutor],
        dims: Dict[str, Tuple[Any, str]],
        argv: Optional[Sequence[str]] = None,
    ) -> List[Chart]:
        r"""Parse the command line and run.  ``dims`` maps a dimension name to ``(default value(s), default mode)``."""
        parser = argparse.ArgumentParser(description=f"Benchmark or profile: {task}", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
        sub = parser.add_subparsers(dest="endpoint", required=True)
        for verb in ("benchmark", "profile"):
            p = sub.add_parser(verb)
            p.add_argument("-p", "--providers", nargs="+", default=[k.provider for k in kernels], choices=[k.provider for k in kernels])
            p.add_argument("-m", "--modes", nargs="+", type=Mode, default=[Mode.FORWARD], choices=list(Mode))
            p.add_argument("-d", "--dtypes", nargs="+", type=Dtype, default=[Dtype.FP16], choices=list(Dtype))
            p.add_argument("-w", "--warmup", type=int, default=20)
            p.add_argument("--device", default="cuda")
            for name, (values, mode) in dims.items():
                flag = f"-{name}" if len(name) == 1 else f"--{name}"
                p.add_argument(flag, dest=name, type=int, nargs="+", default=[values] if isinstance(values, int) else list(values))
                p.add_argument(f"--{name}-mode", dest=f"{name}_mode", choices=["values", "linspace", "logspace"], default=mode)
            if verb == "benchmark":
                p.add_argument("-l", "--line-arg", default="kernel", choices=["kernel", "dtype", "mode", *dims.keys()])
                p.add_argument("-x", "--x-dim", default=next(iter(dims)), choices=list(dims.keys()))
                p.add_argument("-r", "--rep", type=int, default=100)
                p.add_argument("-o", "--output", type=Path, default=None)
        args = parser.parse_args(argv)
        if args.endpoint == "benchmark" and args.output is not None and not args.output.is_dir():
            raise NotADirectoryError(f"Output path {args.output} is not a directory")
        chosen = [k for k in kernels if k.provider in args.providers]
        for k in chosen:
            k.warmup = args.warmup
            k.rep = getattr(args, "rep", 100)
        grid = {name: dimension_values(getattr(args, name), getattr(args, f"{name}_mode")) for name in dims}
        cli = cls(task, chosen, grid, args.modes, args.dtypes, getattr(args, "line_arg", "kernel"), getattr(args, "x_dim", None),
                  getattr(args, "output", None), args.device)  # fmt: skip
        return cli.run(args.endpoint)
