r"""Builds ``libth_b200.so`` in-tree with nvcc for sm_100a (no other architecture).

``python -m triton_helpers_b200.build`` compiles every ``csrc/*.cu`` to an object file (in
parallel, one nvcc process per file) and links them into
``triton_helpers_b200/csrc/libth_b200.so``.  Objects are rebuilt only when their source or a
header is newer.  nvcc cross-compiles, so no GPU is needed to build.
"""
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import List

CSRC = Path(__file__).resolve().parent / "csrc"
INCLUDE = Path(__file__).resolve().parent.parent / "include"
LIB_PATH = CSRC / "libth_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", str(INCLUDE),
]  # fmt: skip


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    return str(candidate) if candidate.exists() else "nvcc"


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def _compile(src: Path, obj: Path, verbose: bool) -> None:
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build(force: bool = False, verbose: bool = False) -> Path:
    sources: List[Path] = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    header_time = _newest_header()
    objects, stale = [], []
    for src in sources:
        obj = src.with_suffix(".o")
        objects.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time):
            stale.append((src, obj))
    with ThreadPoolExecutor(max_workers=max(1, min(len(stale), os.cpu_count() or 1))) as pool:
        list(pool.map(lambda job: _compile(job[0], job[1], verbose), stale))
    if stale or not LIB_PATH.exists():
        cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objects), "-gencode", "arch=compute_100a,code=sm_100a"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True)
    print(f"built {path}")
