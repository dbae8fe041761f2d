"""Exact empirical natural gradient through the n x n Gram matrix of per-example gradients
(Sherman-Morrison-Woodbury; Ren & Goldfarb, arXiv:1906.02353).

Parity: asdl/precondition/smw.py:36-69.  The Gram matrix sum_l (a a^T) o (g g^T) is accumulated
into ``model.kernel`` by the ``gram_hada`` hooks during a first backward pass; solving
(K + damping*I) b = K 1 gives per-example weights, and a second backward pass with the weights
``(1 - b)/damping`` leaves (F + damping*I)^-1 grad in ``param.grad``.
"""
from dataclasses import dataclass
from typing import Any, Tuple

import torch
from torch import Tensor
import torch.nn as nn

from ..core import extend
from ..operations import OP_GRAM_HADAMARD
from ..grad_maker import GradientMaker

__all__ = ['SmwEmpNaturalGradientConfig', 'SmwEmpNaturalGradientMaker']


def zero_kernel(model: nn.Module, n_data1: int, n_data2: int):
    p = next(iter(model.parameters()))
    model.kernel = torch.zeros(n_data1, n_data2, device=p.device, dtype=p.dtype)


def cholesky_solve(A, b, eps=1e-8):
    """(A + eps*I)^-1 b without touching A."""
    eye = torch.eye(A.shape[-1], device=A.device, dtype=A.dtype)
    chol = torch.linalg.cholesky(A + eps * eye)
    return torch.cholesky_solve(b.unsqueeze(-1), chol).squeeze(-1)


@dataclass
class SmwEmpNaturalGradientConfig:
    data_size: int
    damping: float = 1.e-5


class SmwEmpNaturalGradientMaker(GradientMaker):
    """Exact empirical-Fisher natural gradient of a mini-batch through the n x n Gram matrix of per-example
    gradients (Sherman-Morrison-Woodbury): the kernel ``sum_l (a a^T) * (g g^T)`` is accumulated in hooks, one
    Cholesky solve re-weights the per-example losses and a second backward pass forms the gradient.
    Reference: asdl/precondition/smw.py:36-69.
    """
    _loss_reduction = 'none'

    def __init__(self, model, config):
        super().__init__(model)
        self.config = config

    def forward_and_backward(self) -> Tuple[Any, Tensor]:
        if isinstance(self._loss_fn, nn.Module):
            data_average = self._loss_fn.reduction == 'mean'
        else:
            data_average = self._loss_fn_kwargs.get('reduction', 'mean') == 'mean'
        model, n, damping = self.model, self.config.data_size, self.config.damping
        with extend(model, OP_GRAM_HADAMARD):
            zero_kernel(model, n, n)
            self.forward()
            batch_loss = self._loss
            params = [p for p in model.parameters() if p.requires_grad]
            torch.autograd.grad(batch_loss.sum(), params, retain_graph=True)
        UtU = model.kernel  # n x n Gram matrix of per-example gradients
        Utg = UtU.sum(dim=1)
        if data_average:
            UtU = UtU / n
        b = cholesky_solve(UtU, Utg, damping)
        ones = torch.ones_like(b)
        if data_average:
            b = b / n ** 2
            ones = ones / n
        batch_loss.backward(gradient=(ones - b) / damping)
        self._loss = batch_loss.mean() if data_average else batch_loss.sum()
        return self._model_output, self._loss
