"""Statistics of ``nn.LayerNorm``: as for batch norm the affine part sees the normalised input
(out - bias) / weight; leading dimensions beyond the normalised shape are folded into the batch.
Parity: asdl/operations/layernorm.py:7-102."""
import torch

from .batchnorm import two_by_two_blocks
from .operation import (Operation, BASIC_OPS, OP_COV_KRON, OP_GRAM_HADAMARD, OP_COV_UNIT_WISE,
                        OP_COV_UNIT_WISE_INV, OP_COV_DIAG, OP_COV_DIAG_INV, OP_GRAM_DIRECT,
                        OP_BATCH_GRADS)

__all__ = ['LayerNorm']


def _fold(module, t):
    k = module.weight.ndim
    return t.reshape(-1, *t.shape[-k:]) if t.ndim > k + 1 else t


class LayerNorm(Operation):
    """weight, bias: normalized_shape;  in_data, out_grads: n x normalized_shape."""
    supported_operations = set(BASIC_OPS + [OP_COV_UNIT_WISE, OP_COV_UNIT_WISE_INV, OP_COV_DIAG,
                                            OP_COV_DIAG_INV, OP_GRAM_DIRECT, OP_BATCH_GRADS])

    @staticmethod
    def preprocess_in_data(module, in_data, out_data):
        return _fold(module, (out_data - module.bias).div(module.weight))

    @staticmethod
    def preprocess_out_grads(module, out_grads):
        return _fold(module, out_grads)

    @staticmethod
    def batch_grads_weight(module, in_data, out_grads):
        return in_data * out_grads

    @staticmethod
    def batch_grads_bias(module, out_grads):
        return out_grads

    @staticmethod
    def grad_weight(module, in_data, out_grads):
        return (in_data * out_grads).sum(dim=0)

    @staticmethod
    def grad_bias(module, out_grads):
        return out_grads.sum(dim=0)

    @staticmethod
    def cov_diag_weight(module, in_data, out_grads):
        return (in_data * out_grads).square().sum(dim=0)

    @staticmethod
    def cov_diag_bias(module, out_grads):
        return out_grads.square().sum(dim=0)

    @staticmethod
    def cov_unit_wise(module, in_data, out_grads):
        return two_by_two_blocks(in_data * out_grads, out_grads)  # n_features x 2 x 2

    @staticmethod
    def _unsupported(what):
        raise ValueError(f'{what} operation is not supported in LayerNorm.')

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
        return in_data.mean(dim=0)

    @staticmethod
    def out_data_mean(module, out_data):
        return _fold(module, out_data).mean(dim=0)

    @staticmethod
    def out_grads_mean(module, out_grads):
        return out_grads.mean(dim=0)

    @staticmethod
    def out_spatial_size(module, out_data):
        return 1
