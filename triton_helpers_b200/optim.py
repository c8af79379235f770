r"""Adam for 16-bit parameters with fp32 moments, one CUDA kernel per parameter tensor.

``torch.optim.Adam`` keeps its moments in the parameter dtype; with float16 hash tables the
second moment underflows (``g*g < 6e-8`` for ``|g| < 2.4e-4``) and the update divides by
``eps``.  ``FusedAdam`` follows the same update rule (no weight decay, no amsgrad) but stores
``exp_avg`` / ``exp_avg_sq`` in float32, scales the stored gradient by ``grad_scale`` on the fly
(inverse loss scale and world size) and can clear the gradient buffer in the same pass, which
replaces the separate zero-fill the hash-encoding backward needs before every step.

Elements whose gradient is not finite (an overflowed 16-bit sum, a NaN from upstream) are left
untouched - parameter and moments - and counted; ``FusedAdam.skipped_elements()`` reads the count.
"""
from typing import Dict, Iterable, Optional, Tuple

import torch
from torch import Tensor

from . import _lib


@torch.no_grad()
def adam_update(
    param: Tensor,
    grad: Tensor,
    exp_avg: Tensor,
    exp_avg_sq: Tensor,
    step: int,
    lr: float,
    betas: Tuple[float, float],
    eps: float,
    grad_scale: float = 1.0,
    zero_grad: bool = False,
    skipped: Optional[Tensor] = None,
) -> None:
    r"""One ``th_adam_step`` launch: ``param`` (float32 / float16 / bfloat16, contiguous) is updated in
    place from ``grad`` (same dtype and element count) times ``grad_scale``; ``exp_avg`` / ``exp_avg_sq``
    are float32.  ``skipped`` is an int32 device counter of elements passed over because their gradient
    was not finite."""
    if grad.dtype != param.dtype or not param.is_contiguous() or not grad.is_contiguous():
        raise RuntimeError("adam_update needs contiguous parameters and same-dtype contiguous gradients")
    device = _lib.require_cuda(param, grad, exp_avg, exp_avg_sq, skipped)
    with torch.cuda.device(device):
        _lib.check(
            _lib.lib().th_adam_step(
                param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), param.numel(), lr,
                betas[0], betas[1], eps, step, grad_scale, int(zero_grad), _lib.dtype_code(param), _lib.ptr(skipped),
                _lib.stream_ptr(device),
            ),
            "th_adam_step",
        )  # fmt: skip


class FusedAdam(torch.optim.Optimizer):

    def __init__(self, params: Iterable[Tensor], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8):
        if lr < 0 or eps < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1):
            raise ValueError("invalid Adam hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps))
        self._skipped: Dict[torch.device, Tensor] = {}

    def _skip_counter(self, device: torch.device) -> Tensor:
        counter = self._skipped.get(device)
        if counter is None:
            counter = self._skipped[device] = torch.zeros(1, dtype=torch.int32, device=device)
        return counter

    def skipped_elements(self) -> int:
        r"""Elements passed over so far because their gradient was not finite (reads the device: synchronises)."""
        return sum(int(c.item()) for c in self._skipped.values())

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, zero_grad: bool = False) -> None:
        r"""Update every parameter that has a gradient.

        ``grad_scale`` multiplies the stored gradients before use; ``zero_grad`` clears the
        gradient buffers (kept allocated) as part of the update kernel.
        """
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if not state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                    state["exp_avg_sq"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                state["step"] += 1
                adam_update(
                    p, p.grad, state["exp_avg"], state["exp_avg_sq"], state["step"], group["lr"], group["betas"],
                    group["eps"], grad_scale, zero_grad, self._skip_counter(p.device),
                )  # fmt: skip
