"""CurveBall (Henriques et al., "Small steps and giant leaps", ICCV 2019): a momentum buffer z is
driven by the gradient of the local quadratic model, z <- rho*z - beta*(H z + damping*z + g), and
the update direction left in ``param.grad`` is -z, so that a plain SGD step with learning rate 1
applies w <- w + z.

Parity: asdl/precondition/curve_ball.py:17-45.  In the reference the method is named
``_precondition`` and is therefore never reached (``precondition`` raises); here the template's
``precondition`` is implemented, the Hessian-vector product uses forward-over-reverse
differentiation and also yields the gradient, so no separate forward/backward is run.
"""
from dataclasses import dataclass

import torch
import torch.nn as nn

from .prec_grad_maker import PreconditionedGradientMaker, PreconditioningConfig

__all__ = ['CurveBallGradientMaker', 'CurveBallGradientConfig']


@dataclass
class CurveBallGradientConfig(PreconditioningConfig):
    damping: float = 1.e-7
    momentum: float = 0.9
    momentum_decay: float = 1.


class CurveBallGradientMaker(PreconditionedGradientMaker):
    """Args:
        momentum: step size beta of the momentum-buffer update.
        momentum_decay: forgetting factor rho of the buffer."""

    def __init__(self, model: nn.Module, config: PreconditioningConfig,
                 momentum: float = 0.9, momentum_decay: float = 1):
        super().__init__(model, config)
        self._params = [p for p in model.parameters() if p.requires_grad]
        self._momentum = tuple(torch.zeros_like(p) for p in self._params)
        self.momentum = momentum
        self.momentum_decay = momentum_decay

    def do_forward_and_backward(self, step=None) -> bool:
        return False  # the gradient comes out of the Hessian-vector product

    def precondition(self):
        damping = self.config.damping
        for p in self._params:
            p.grad = None
        hvps = self.loss_hvp(tangents=self._momentum, accumulate_grad=True)
        grads = [p.grad for p in self._params]
        if not (len(hvps) == len(grads) == len(self._momentum)):
            raise ValueError(f'len(hvps), len(grads), and len(momentum) have to be the same. '
                             f'Got {len(hvps)}, {len(grads)}, and {len(self._momentum)}')
        with torch.no_grad():
            for p, z, hvp, grad in zip(self._params, self._momentum, hvps, grads):
                quad_grad = hvp + damping * z + grad
                if self.momentum_decay != 1:
                    z.mul_(self.momentum_decay)
                z.sub_(quad_grad, alpha=self.momentum)
                p.grad = -z.clone()

    def _curvature_state(self):
        return {f'momentum{i}': z for i, z in enumerate(self._momentum)}

    def _load_curvature_state(self, tensors):
        for i, z in enumerate(self._momentum):
            if f'momentum{i}' in tensors:
                z.copy_(tensors[f'momentum{i}'])
