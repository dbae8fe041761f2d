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
    """Fresh ``model.kernel`` (n_data1 x n_data2) for the Gram hooks to add into."""
    like = next(iter(model.parameters()))
    model.kernel = like.new_zeros(n_data1, n_data2)


def cholesky_solve(A, b, eps=1e-8):
    """(A + eps*I)^-1 b without touching A (a breakdown of the factorisation raises the damping, see
    :func:`asdl_b200.ops.damped_cholesky`)."""
    from .. import ops
    return torch.cholesky_solve(b.unsqueeze(-1), ops.damped_cholesky(A, eps)).squeeze(-1)


def woodbury_example_weights(gram: Tensor, damping: float, data_average: bool) -> Tensor:
    """Per-example loss weights w such that back-propagating ``sum_i w_i loss_i`` leaves
    ``(F + damping*I)^-1 grad`` in ``param.grad``, with F the empirical Fisher of the batch.

    With U the n x p matrix of per-example gradients, ``gram = U U^T`` and g = U^T 1 (divided by n when the
    loss is a mean), Woodbury gives ``(U^T U / n + damping I)^-1 g = U^T (1 - b) / damping`` where
    ``(gram / n + damping I) b = gram 1`` (and the 1/n factors of the mean distributed as below)."""
    n = gram.shape[0]
    rhs = gram.sum(dim=1)
    scale = n if data_average else 1
    b = cholesky_solve(gram / scale, rhs, damping)
    ones = torch.ones_like(b)
    if data_average:
        return (ones / n - b / n ** 2) / damping
    return (ones - b) / damping


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

    def _loss_is_a_mean(self) -> bool:
        if isinstance(self._loss_fn, nn.Module):
            return self._loss_fn.reduction == 'mean'
        return self._loss_fn_kwargs.get('reduction', 'mean') == 'mean'

    def forward_and_backward(self) -> Tuple[Any, Tensor]:
        n = self.config.data_size
        with extend(self.model, OP_GRAM_HADAMARD):
            zero_kernel(self.model, n, n)
            self.forward()                       # per-example losses (reduction forced to 'none')
            losses = self._loss
            trainable = [p for p in self.model.parameters() if p.requires_grad]
            torch.autograd.grad(losses.sum(), trainable, retain_graph=True)   # fills model.kernel through the hooks
        mean = self._loss_is_a_mean()
        losses.backward(gradient=woodbury_example_weights(self.model.kernel, self.config.damping, mean))
        self._loss = losses.mean() if mean else losses.sum()
        return self._model_output, self._loss
