r"""``python -m triton_helpers_b200.layers.hash_encoding benchmark|profile ...``: times the CUDA hash encoding
(and tiny-cuda-nn's when it is installed) over the point count ``L``, like
``triton_helpers/layers/hash_encoding/__main__.py``: 32 x L points, the same dimension names and defaults."""
import math
from dataclasses import dataclass
from typing import Any, Dict

import torch
from torch import Tensor

from ...benchmark import CLI, KernelExecutor
from .kernel import hash_encoding
from .module import HashEncoding

try:
    from tinycudann.modules import Encoding  # type: ignore
except ImportError:
    Encoding = None


@dataclass
class CudaHash(KernelExecutor):

    @torch.no_grad()
    def prepare_inputs(self, L, D, F, T, N, X, Y, dtype=torch.float32, device="cuda", requires_grad=False, **_) -> Dict[str, Any]:
        torch.random.manual_seed(0)
        x = torch.rand(32, L, D, device=device)
        layer = HashEncoding(T, N, D, F, X, Y).to(device)
        e = layer.embeddings.to(dtype).detach()
        e.requires_grad = requires_grad
        return {"x": x, "e": e, "pi": layer.pi, "geometry": (T, X, Y, N)}

    def forward(self, x: Tensor, e: Tensor, pi: Tensor, geometry) -> Tensor:
        T, X, Y, N = geometry
        return hash_encoding(x, e, None, pi, T, X, Y, N)


@dataclass
class TinyCudaNN(KernelExecutor):

    def prepare_inputs(self, L, D, F, T, N, X, Y, dtype=torch.float32, device="cuda", **_) -> Dict[str, Any]:
        assert Encoding is not None, "tiny-cuda-nn is not installed"
        scale = math.exp((math.log(Y) - math.log(X)) / (N - 1)) + 1e-5
        config = {"otype": "HashGrid", "n_levels": N, "n_features_per_level": F, "log2_hashmap_size": int(math.log2(T) + 1e-5),
                  "base_resolution": X, "per_level_scale": scale, "interpolation": "Linear"}  # fmt: skip
        torch.random.manual_seed(0)
        return {"x": torch.rand(32, L, D, device=device), "module": Encoding(D, config, dtype=dtype).to(device)}

    def forward(self, x: Tensor, module) -> Tensor:
        return module(x.view(-1, x.size(-1)))


if __name__ == "__main__":
    executors = [CudaHash("cuda-hash")] + ([TinyCudaNN("tiny-cuda-nn")] if Encoding is not None else [])
    CLI.entrypoint(
        "InstantNGP Hash Encoding",
        executors,
        dims={
            "L": ((512, 2048, 8192, 16384, 32768, 65536, 65536 * 2), "values"),
            "D": (3, "values"),
            "F": (2, "values"),
            "T": (2**14, "values"),
            "N": (16, "values"),
            "X": (16, "values"),
            "Y": (512, "values"),
        },
    )
