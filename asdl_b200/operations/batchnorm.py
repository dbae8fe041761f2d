"""Statistics of ``nn.BatchNorm1d`` / ``nn.BatchNorm2d``.

The "input" of the affine part is the normalised activation x_hat, recovered from the layer
output as (out - bias) / weight (so every weight has to be non-zero).  Per-example gradients are
sum_hw(x_hat * g) for the scale and sum_hw(g) for the shift; the unit-wise curvature is one 2x2
block per feature.  Kronecker and Hadamard-Gram statistics do not exist for these layers.
Parity: asdl/operations/batchnorm.py:7-107.
"""
import torch
from torch import nn

from .operation import (Operation, BASIC_OPS, OP_COV_KRON, OP_GRAM_HADAMARD, OP_COV_UNIT_WISE,
                        OP_COV_UNIT_WISE_INV, OP_COV_DIAG, OP_COV_DIAG_INV, OP_GRAM_DIRECT,
                        OP_BATCH_GRADS)

__all__ = ['BatchNorm1d', 'BatchNorm2d']


def two_by_two_blocks(gw, gb):
    """n x f per-example (scale, shift) gradients -> f x 2 x 2 second-moment blocks."""
    ww = gw.square().sum(dim=0).flatten()
    bb = gb.square().sum(dim=0).flatten()
    wb = (gw * gb).sum(dim=0).flatten()
    return torch.stack([torch.stack([ww, wb], dim=1), torch.stack([wb, bb], dim=1)], dim=1)


class _BatchNormNd(Operation):
    supported_operations = set(BASIC_OPS + [OP_COV_UNIT_WISE, OP_COV_UNIT_WISE_INV, OP_COV_DIAG,
                                            OP_COV_DIAG_INV, OP_GRAM_DIRECT, OP_BATCH_GRADS])
    _spatial_dims = ()

    @staticmethod
    def preprocess_in_data(module, in_data, out_data):
        if getattr(module, 'fused_output', False):
            raise ValueError(f'{module} fuses an activation or a residual add: its output does not determine '
                             f'the normalised input.  Build the model without fusion for this gradient '
                             f'maker, or use FusedKfacGradientMaker.')
        shape = (1, module.num_features) + (1,) * (out_data.ndim - 2)
        return (out_data - module.bias.view(shape)).div(module.weight.view(shape))

    def _reduce(self, tensor):
        return tensor.sum(dim=self._spatial_dims) if self._spatial_dims else tensor

    def batch_grads_weight(self, module, in_data, out_grads):
        return self._reduce(in_data * out_grads)  # n x f

    def batch_grads_bias(self, module, out_grads):
        return self._reduce(out_grads)  # n x f

    def grad_weight(self, module, in_data, out_grads):
        return self.batch_grads_weight(module, in_data, out_grads).sum(dim=0)

    def grad_bias(self, module, out_grads):
        return self.batch_grads_bias(module, out_grads).sum(dim=0)

    def cov_diag_weight(self, module, in_data, out_grads):
        return self.batch_grads_weight(module, in_data, out_grads).square().sum(dim=0)

    def cov_diag_bias(self, module, out_grads):
        return self.batch_grads_bias(module, out_grads).square().sum(dim=0)

    def cov_unit_wise(self, module, in_data, out_grads):
        return two_by_two_blocks(self.batch_grads_weight(module, in_data, out_grads),
                                 self.batch_grads_bias(module, out_grads))

    @staticmethod
    def _unsupported(what):
        raise ValueError(f'{what} operation is not supported in BatchNormNd.')

    @classmethod
    def cov_kron_A(cls, module, in_data):
        cls._unsupported(OP_COV_KRON)

    @classmethod
    def cov_kron_B(cls, module, out_grads):
        cls._unsupported(OP_COV_KRON)

    @classmethod
    def gram_A(cls, module, in_data1, in_data2=None):
        cls._unsupported(OP_GRAM_HADAMARD)

    @classmethod
    def gram_B(cls, module, out_grads1, out_grads2=None):
        cls._unsupported(OP_GRAM_HADAMARD)

    @staticmethod
    def in_data_mean(module, in_data):
        return in_data.transpose(0, 1).flatten(start_dim=1).mean(dim=1)

    @staticmethod
    def out_data_mean(module, out_data):
        return out_data.transpose(0, 1).flatten(start_dim=1).mean(dim=1)

    @staticmethod
    def out_grads_mean(module, out_grads):
        return out_grads.transpose(0, 1).flatten(start_dim=1).mean(dim=1)

    @staticmethod
    def out_spatial_size(module, out_data):
        size = 1
        for d in out_data.shape[2:]:
            size *= d
        return size


class BatchNorm1d(_BatchNormNd):
    """weight, bias: f;  in_data, out_grads: n x f."""
    _spatial_dims = ()


class BatchNorm2d(_BatchNormNd):
    """weight, bias: c;  in_data, out_grads: n x c x h x w."""
    _spatial_dims = (2, 3)
