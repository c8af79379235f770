r"""``python -m triton_helpers_b200.layers.fully_fused_mlp benchmark|profile ...``: the fused MLP against a chain of
``F.linear`` calls over the row count ``L`` (32 x L rows, width ``D``, ``H`` hidden layers), like
``triton_helpers/layers/fully_fused_mlp/__main__.py``."""
from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch
import torch.nn.functional as F
from torch import Tensor

from ...benchmark import CLI, KernelExecutor
from .kernel import fully_fused_mlp
from .module import FullyFusedMLP


@dataclass
class Baseline(KernelExecutor):

    def prepare_inputs(self, L, D, H, dtype=torch.float16, device="cuda", requires_grad=False, **_) -> Dict[str, Any]:
        torch.random.manual_seed(0)
        layer = FullyFusedMLP(D, D, D, depth=H + 1).to(device=device, dtype=dtype)
        for p in layer.parameters():
            p.requires_grad = requires_grad
        x = torch.randn(32, L, D, device=device, dtype=dtype, requires_grad=requires_grad)
        return {"x": x, "w_in": layer.w_in, "b_in": layer.b_in, "w_out": layer.w_out, "b_out": layer.b_out,
                "w_hid": layer.w_hid, "b_hid": layer.b_hid}  # fmt: skip

    def forward(self, x: Tensor, w_in, b_in, w_out, b_out, w_hid: Optional[Tensor], b_hid: Optional[Tensor]) -> Tensor:
        h = F.relu(F.linear(x, w_in, b_in))
        if w_hid is not None:
            width = w_in.shape[0]
            for i in range(w_hid.shape[0] // width):
                h = F.relu(F.linear(h, w_hid[i * width : (i + 1) * width], b_hid[i]))
        return F.linear(h, w_out, b_out)


@dataclass
class Fused(Baseline):
    fp16_acc: bool = False

    def forward(self, x, w_in, b_in, w_out, b_out, w_hid, b_hid) -> Tensor:
        return fully_fused_mlp(x, w_in, b_in, w_out, b_out, w_hid, b_hid, fp16_acc=self.fp16_acc)


if __name__ == "__main__":
    CLI.entrypoint(
        "MLP",
        [Baseline("baseline"), Fused("fully-fused")],
        dims={
            "L": ((512, 2048, 8192, 16384, 32768, 65536), "values"),
            "D": (64, "values"),
            "H": (8, "values"),
        },
    )
