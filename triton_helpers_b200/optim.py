r"""Adam for 16-bit parameters with fp32 moments, one CUDA kernel per parameter tensor.

``torch.optim.Adam`` keeps its moments in the parameter dtype; with float16 hash tables the
second moment underflows (``g*g < 6e-8`` for ``|g| < 2.4e-4``) and the update divides by
``eps``.  ``FusedAdam`` follows the same update rule (no weight decay, no amsgrad) but stores
``exp_avg`` / ``exp_avg_sq`` in float32, scales the stored gradient by ``grad_scale`` on the fly
(inverse loss scale and world size) and can clear the gradient buffer in the same pass, which
replaces the separate zero-fill the hash-encoding backward needs before every step.
"""
from typing import Iterable

import torch
from torch import Tensor

from . import _lib


class FusedAdam(torch.optim.Optimizer):

    def __init__(self, params: Iterable[Tensor], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8):
        if lr < 0 or eps < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1):
            raise ValueError("invalid Adam hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps))

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, zero_grad: bool = False) -> None:
        r"""Update every parameter that has a gradient.

        ``grad_scale`` multiplies the stored gradients before use; ``zero_grad`` clears the
        gradient buffers (kept allocated) as part of the update kernel.
        """
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.dtype != p.dtype or not p.is_contiguous() or not p.grad.is_contiguous():
                    raise RuntimeError("FusedAdam needs contiguous parameters and same-dtype contiguous gradients")
                state = self.state[p]
                if not state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                    state["exp_avg_sq"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                state["step"] += 1
                device = _lib.require_cuda(p, p.grad)
                with torch.cuda.device(device):
                    _lib.check(
                        _lib.lib().th_adam_step(
                            p.data_ptr(), p.grad.data_ptr(), state["exp_avg"].data_ptr(), state["exp_avg_sq"].data_ptr(),
                            p.numel(), group["lr"], beta1, beta2, group["eps"], state["step"], grad_scale,
                            int(zero_grad), _lib.dtype_code(p), _lib.stream_ptr(device),
                        ),
                        "th_adam_step",
                    )  # fmt: skip
