r"""The benchmark harness: dimension grids, chart naming and CSV layout (the reference's file names and
columns, ``triton_helpers/benchmark.py:410-412`` and ``layers/*/benchmarks/*.csv``), on CPU with a stub executor;
one end-to-end run of the two layer entry points on the GPU."""
import csv
from dataclasses import dataclass

import pytest
import torch

from triton_helpers_b200.benchmark import CLI, Chart, Dtype, KernelExecutor, Mode, dimension_values


def test_dimension_values():
    assert dimension_values([512, 2048], "values") == [512, 2048]
    assert dimension_values([1, 10, 3], "linspace") == [1, 4, 7, 10]
    assert dimension_values([6, 10, 5], "logspace") == [64, 128, 256, 512, 1024]
    with pytest.raises(ValueError):
        dimension_values([1], "cubic")


@dataclass
class Stub(KernelExecutor):
    cost: float = 1.0

    def benchmark(self, mode, dtype, **dims):
        ms = self.cost * dims["L"] / 1000.0 * (2 if mode == Mode.BACKWARD else 1)
        return ms, 0.9 * ms, 1.1 * ms


def test_chart_names_and_csv_follow_the_reference(tmp_path):
    cli = CLI("InstantNGP Hash Encoding", [Stub("tiny-cuda-nn", cost=2.0), Stub("cuda-hash")],
              {"L": [512, 2048], "D": [3], "F": [2], "T": [16384], "N": [16], "X": [16], "Y": [512]},
              modes=[Mode.FORWARD, Mode.BACKWARD], dtypes=[Dtype.FP16], output=tmp_path)  # fmt: skip
    charts = cli.run("benchmark")
    assert [c.name for c in charts] == [
        "InstantNGP Hash Encoding-fwd-D=3-F=2-T=16384-N=16-X=16-Y=512-fp16",
        "InstantNGP Hash Encoding-bwd-D=3-F=2-T=16384-N=16-X=16-Y=512-fp16",
    ]
    rows = list(csv.reader(open(tmp_path / (charts[1].name + ".csv"))))
    assert rows[0] == ["L", "Tiny-Cuda-Nn", "Cuda-Hash"]
    assert rows[1][0] == "512.0" and float(rows[1][1]) == pytest.approx(2.048) and float(rows[2][2]) == pytest.approx(4.096)


def test_line_argument_can_be_the_dtype():
    cli = CLI("MLP", [Stub("fully-fused")], {"L": [512], "D": [64], "H": [8]}, modes=[Mode.FORWARD_BACKWARD],
              dtypes=[Dtype.FP16, Dtype.BF16], line_arg="dtype")  # fmt: skip
    (chart,) = cli.run("benchmark")
    assert chart.name == "MLP-Fully-Fused-fwd-bwd-D=64-H=8" and chart.line_names == ["fp16", "bf16"]


def test_entrypoint_parses_the_reference_flags(tmp_path):
    charts = CLI.entrypoint("MLP", [Stub("baseline"), Stub("fully-fused")], {"L": ((512, 2048), "values"), "D": (64, "values"), "H": (8, "values")},
                            ["benchmark", "-p", "fully-fused", "-m", "fwd", "bwd", "-d", "bf16", "-w", "1", "-r", "2", "-L", "6", "8", "3",
                             "--L-mode", "logspace", "-o", str(tmp_path)])  # fmt: skip
    assert [c.name for c in charts] == ["MLP-fwd-D=64-H=8-bf16", "MLP-bwd-D=64-H=8-bf16"]
    assert charts[0].x_values == [64, 128, 256] and charts[0].line_names == ["Fully-Fused"]
    assert (tmp_path / "MLP-fwd-D=64-H=8-bf16.csv").exists()
    with pytest.raises(NotADirectoryError):
        CLI.entrypoint("MLP", [Stub("baseline")], {"L": (512, "values")}, ["benchmark", "-o", str(tmp_path / "missing")])


@pytest.mark.gpu
def test_layer_entry_points_run_on_the_gpu(tmp_path):
    from triton_helpers_b200.layers.fully_fused_mlp.__main__ import Baseline, Fused
    from triton_helpers_b200.layers.hash_encoding.__main__ import CudaHash

    charts = CLI.entrypoint("MLP", [Baseline("baseline"), Fused("fully-fused")], {"L": ((512, 2048), "values"), "D": (64, "values"), "H": (2, "values")},
                            ["benchmark", "-m", "fwd", "fwd-bwd", "-w", "2", "-r", "5", "-o", str(tmp_path)])  # fmt: skip
    assert len(charts) == 2 and all(v > 0 for c in charts for row in c.rows for v in row)
    charts = CLI.entrypoint("InstantNGP Hash Encoding", [CudaHash("cuda-hash")],
                            {"L": ((512,), "values"), "D": (3, "values"), "F": (2, "values"), "T": (2**14, "values"), "N": (16, "values"),
                             "X": (16, "values"), "Y": (512, "values")}, ["benchmark", "-m", "bwd", "-d", "fp32", "-w", "2", "-r", "5"])  # fmt: skip
    assert charts[0].name == "InstantNGP Hash Encoding-bwd-D=3-F=2-T=16384-N=16-X=16-Y=512-fp32" and charts[0].rows[0][0] > 0
    CLI.entrypoint("MLP", [Fused("fully-fused")], {"L": (512, "values"), "D": (64, "values"), "H": (1, "values")}, ["profile", "-w", "1"])
