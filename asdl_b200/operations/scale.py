"""A learnable scalar gain (Fixup-style ``Scale`` module) and its statistics: the per-example
gradient is sum(out_grad * input); the input seen in the forward hook is kept on the module
(``module.n_in_data``) for the backward statistic.  Parity: asdl/operations/scale.py:7-48."""
import torch
from torch import nn

from .operation import Operation

__all__ = ['Scale', 'ScaleExt']


class Scale(nn.Module):
    """Learnable scalar that multiplies its input (Fixup-style networks).  Reference: asdl/operations/scale.py:7-20."""
    def __init__(self):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(1))

    def reset_parameters(self):
        nn.init.constant_(self.weight, 1)

    def forward(self, input):
        return self.weight * input


def _per_example_dot(x, g):
    n = g.shape[0]
    return (x.reshape(n, -1) * g.reshape(n, -1)).sum(dim=1)


class ScaleExt(Operation):
    """module.weight: 1;  in_data: n x f;  out_grads: n x f."""

    @staticmethod
    def batch_grads_weight(module, in_data, out_grads):
        return _per_example_dot(in_data, out_grads).unsqueeze(-1)

    @staticmethod
    def cov_diag_weight(module, in_data, out_grads):
        return _per_example_dot(in_data, out_grads).square().sum()

    @staticmethod
    def cov_kron_A(module, in_data):
        module.n_in_data = in_data.reshape(in_data.shape[0], -1)
        return torch.ones(1, 1, device=in_data.device)

    @staticmethod
    def cov_kron_B(module, out_grads):
        return _per_example_dot(module.n_in_data, out_grads).square().sum().reshape(1, 1)
