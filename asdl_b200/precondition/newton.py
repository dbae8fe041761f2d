"""Damped (optionally saddle-free) Newton step with the full Hessian.
Parity: asdl/precondition/newton.py:21-49.  The damped system is solved without modifying the
stored Hessian."""
from dataclasses import dataclass
from typing import Any, Tuple, Union

import torch
from torch import Tensor

from .. import ops
from ..grad_maker import GradientMaker
from ..hessian import HessianMaker, HessianConfig
from ..matrices import SHAPE_FULL

__all__ = ['NewtonGradientConfig', 'NewtonGradientMaker']


@dataclass
class NewtonGradientConfig:
    damping: float = 1.e-8
    absolute: bool = False


class NewtonGradientMaker(GradientMaker):
    """``grad <- (H + damping*I)^-1 grad``; with ``absolute=True`` H is replaced by |H| (absolute
    eigenvalues), which turns saddle directions into descent directions."""

    def __init__(self, model, config):
        super().__init__(model)
        self.config = config
        self.hessian_maker = HessianMaker(model, HessianConfig(hessian_shapes=[SHAPE_FULL]))

    def forward_and_backward(self, scale=1., accumulate=False) -> Union[Tuple[Any, Tensor], Any]:
        rst = self.delegate_forward_and_backward(self.hessian_maker, scale=scale,
                                                 accumulate=accumulate, calc_loss_grad=True)
        self.precondition()
        return rst

    @torch.no_grad()
    def precondition(self):
        hessian = self.model.hessian.data
        grads = [p.grad for p in self.model.parameters() if p.requires_grad and p.grad is not None]
        if self.config.absolute:
            evals, evecs = ops.eigh(hessian)
            hessian = (evecs * evals.abs()) @ evecs.T
        eye = torch.eye(hessian.shape[0], device=hessian.device, dtype=hessian.dtype)
        g = torch.cat([t.reshape(-1) for t in grads])
        sol = torch.linalg.solve(hessian + self.config.damping * eye, g)
        offset = 0
        for t in grads:
            t.copy_(sol[offset:offset + t.numel()].view_as(t))
            offset += t.numel()
