"""Optimizer step on the lattice values as one kernel.

The reference's training loops run ``torch.optim.AdamW`` over the table (reference:
examples/performance.py:161 -- ``amsgrad=False, betas=(0.9, 0.99), eps=1e-15, weight_decay=0.0``
-- and examples/train_toy_example.py:30); its published training throughput includes that step.
``LatticeAdamW`` has the same constructor arguments and update rule, but applies the step to each
fp32 CUDA parameter with a single launch of ``permuto_adam_step`` (C ABI) instead of the chain of
elementwise kernels a generic optimizer issues, can skip slots no point has touched yet, and can
clear the gradient in the same pass.  There is no CPU implementation.
"""
from __future__ import annotations

import torch

from . import _native as _C


def adam_step(values: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, step: int,
              lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, skip_untouched: bool = False,
              zero_grad: bool = False) -> None:
    """In-place AdamW step on raw tensors (all fp32, contiguous, same shape, same CUDA device)."""
    for name, t in (("values", values), ("grad", grad), ("exp_avg", exp_avg), ("exp_avg_sq", exp_avg_sq)):
        if not t.is_cuda:
            raise RuntimeError(f"{name} should be in GPU memory. There is no CPU path")
        if t.dtype != torch.float32 or not t.is_contiguous() or t.shape != values.shape or t.device != values.device:
            raise RuntimeError(f"{name} must be a contiguous float32 tensor of the shape and device of the values")
    flags = (_C.PERMUTO_ADAM_SKIP_UNTOUCHED if skip_untouched else 0) | (_C.PERMUTO_ADAM_ZERO_GRAD if zero_grad else 0)
    with _C._guard(values.device):
        _C.check(_C.lib.permuto_adam_step(values.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(),
                                          values.numel(), float(lr), float(betas[0]), float(betas[1]), float(eps),
                                          float(weight_decay), int(step), flags, _C._stream(values.device)))
    # the kernel wrote through the raw pointer: tell autograd (and the module's fp16 copy) so
    torch.autograd.graph.increment_version(values)


class LatticeAdamW(torch.optim.Optimizer):
    """``torch.optim.AdamW`` for fp32 CUDA parameters, one fused kernel per parameter.

    ``skip_untouched=True`` leaves entries alone whose gradient and moments are all zero (exact
    when ``weight_decay == 0``, ignored otherwise).  ``zero_grad_in_step=True`` clears each
    ``.grad`` inside the step kernel; ``zero_grad()`` then has nothing left to do when called
    with ``set_to_none=False``.  ``amsgrad`` and ``maximize`` are not supported.
    """

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2, amsgrad=False,
                 skip_untouched=False, zero_grad_in_step=False):
        if amsgrad:
            raise ValueError("LatticeAdamW does not implement amsgrad")
        if lr < 0 or eps < 0 or weight_decay < 0 or not (0 <= betas[0] < 1) or not (0 <= betas[1] < 1):
            raise ValueError("invalid AdamW hyper-parameters")
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, skip_untouched=skip_untouched,
                        zero_grad_in_step=zero_grad_in_step)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None:
                    continue
                state = self.state[p]
                if not state:
                    state["step"] = 0
                    state["exp_avg"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                    state["exp_avg_sq"] = torch.zeros_like(p, memory_format=torch.contiguous_format)
                state["step"] += 1
                grad = p.grad if p.grad.is_contiguous() else p.grad.contiguous()
                # the parameter itself, not p.data: the step must bump ITS version counter
                adam_step(p, grad, state["exp_avg"], state["exp_avg_sq"], state["step"], group["lr"],
                          group["betas"], group["eps"], group["weight_decay"], group["skip_untouched"],
                          group["zero_grad_in_step"] and grad is p.grad)
        return loss
