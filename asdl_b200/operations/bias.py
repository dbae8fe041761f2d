"""A learnable scalar shift (Fixup-style ``Bias`` module) and its statistics: the per-example
gradient is the sum of the output-gradient, the "Kronecker factors" are 1x1.
Parity: asdl/operations/bias.py:8-52."""
import torch
from torch import nn

from .operation import (Operation, BASIC_OPS, OP_COV_KRON, OP_COV_SWIFT_KRON, OP_COV_DIAG,
                        OP_COV_DIAG_INV, OP_GRAM_DIRECT, OP_BATCH_GRADS)

__all__ = ['Bias', 'BiasExt']

_OPS = set(BASIC_OPS + [OP_COV_KRON, OP_COV_SWIFT_KRON, OP_COV_DIAG, OP_COV_DIAG_INV,
                        OP_GRAM_DIRECT, OP_BATCH_GRADS])


class Bias(nn.Module):
    """Learnable scalar added to its input (Fixup-style networks).  Reference: asdl/operations/bias.py:8-24."""
    supported_operations = _OPS

    def __init__(self):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(1))

    def reset_parameters(self):
        nn.init.constant_(self.weight, 0)

    def forward(self, input):
        return input + self.weight


def _per_example_sum(t):
    return t.reshape(t.shape[0], -1).sum(dim=1)


class BiasExt(Operation):
    """module.weight: 1;  in_data: n x f;  out_grads: n x f."""
    supported_operations = _OPS
    _supported_operations = _OPS

    @staticmethod
    def batch_grads_weight(module, in_data, out_grads):
        return _per_example_sum(out_grads).unsqueeze(-1)

    @staticmethod
    def cov_diag_weight(module, in_data, out_grads):
        return _per_example_sum(out_grads).square().sum()

    @staticmethod
    def cov_kron_A(module, in_data):
        return torch.ones((1, 1), device=in_data.device)

    @staticmethod
    def cov_kron_B(module, out_grads):
        return _per_example_sum(out_grads).square().sum().reshape(1, 1)

    cov_swift_kron_A = cov_kron_A
    cov_swift_kron_B = cov_kron_B
