"""Statistics of ``nn.Conv2d``.

Shapes after preprocessing: ``a`` n x (c_in*kh*kw) x L patches (column order (c, kh, kw), matching
``weight.view(c_out, -1)``), ``g`` n x c_out x L with L = h_out*w_out.  A = M M^T / L with M the
(c_in*kh*kw) x (n*L) patch matrix, B = G G^T (no spatial normalisation).
Parity: asdl/operations/conv.py:9-225.  On CUDA the A factor is produced from the raw layer input
by :func:`asdl_b200.ops.conv_patch_gram` (bf16 im2col kernel feeding the tcgen05 SYRK) when the
patches themselves are not needed.
"""
import torch
from torch import nn

from .. import ops
from ..utils import im2col_2d
from .operation import Operation, ALL_OPS, OP_RFIM_RELU, OP_RFIM_SOFTMAX

__all__ = ['Conv2d']


def _rows(t):
    """n x d x L -> (n*L) x d sample matrix."""
    return t.permute(0, 2, 1).reshape(-1, t.shape[1])


class Conv2d(Operation):
    """Statistics of ``nn.Conv2d``.  in_data becomes the patch matrix n x (c_in kh kw) x (h_out w_out),
    out_grads n x c_out x (h_out w_out); the input-side Kronecker factor is divided by the number of output
    positions.  Everything but the rFIM operations.  Reference: asdl/operations/conv.py:9-225.
    """
    supported_operations = set(ALL_OPS) - {OP_RFIM_RELU, OP_RFIM_SOFTMAX}

    def __init__(self, module, op_names, model_for_kernel=None):
        if getattr(module, 'groups', 1) != 1:
            raise ValueError(f'{module}: convolutions with groups > 1 are not supported (every group has its own '
                             f'patch matrix); list the layer in ignore_modules.')
        super().__init__(module, op_names, model_for_kernel)

    @staticmethod
    def preprocess_in_data(module, in_data, out_data):
        return im2col_2d(in_data, module)

    @staticmethod
    def preprocess_out_grads(module, out_grads):
        return out_grads.flatten(start_dim=2)

    @staticmethod
    def extend_in_data(in_data):
        n, _, L = in_data.shape
        return torch.cat([in_data, in_data.new_ones(n, 1, L)], dim=1)

    # gradients --------------------------------------------------------------------------------
    @staticmethod
    def batch_grads_weight(module, in_data, out_grads):
        return torch.bmm(out_grads, in_data.transpose(1, 2)).view(-1, *module.weight.shape)

    @staticmethod
    def batch_grads_bias(module, out_grads):
        return out_grads.sum(dim=2)

    @staticmethod
    def grad_weight(module, in_data, out_grads):
        return torch.einsum('nol,nil->oi', out_grads, in_data).view_as(module.weight)

    @staticmethod
    def grad_bias(module, out_grads):
        return out_grads.sum(dim=(0, 2))

    # diagonal ---------------------------------------------------------------------------------
    @staticmethod
    def cov_diag_weight(module, in_data, out_grads):
        c_out, d = module.weight.shape[0], in_data.shape[1]
        L = in_data.shape[-1]
        if L == 1:
            # each per-example gradient is an outer product, so its square factorises
            return (_rows(out_grads).square().T @ _rows(in_data).square()).view_as(module.weight)
        # chunk over examples so the n x c_out x d per-example gradients are never all resident
        acc = in_data.new_zeros(c_out, d, dtype=torch.float32)
        step = max(1, (1 << 26) // max(1, c_out * d))
        for lo in range(0, in_data.shape[0], step):
            bg = torch.bmm(out_grads[lo:lo + step], in_data[lo:lo + step].transpose(1, 2))
            acc += bg.float().square().sum(dim=0)
        return acc.view_as(module.weight).to(in_data.dtype)

    @staticmethod
    def cov_diag_bias(module, out_grads):
        return out_grads.sum(dim=2).square().sum(dim=0)

    # Kronecker factors ------------------------------------------------------------------------
    @staticmethod
    def cov_kron_A(module, in_data):
        L = in_data.shape[-1]
        return ops.gram(_rows(in_data), scale=1.0 / L)

    @staticmethod
    def cov_kron_B(module, out_grads):
        return ops.gram(_rows(out_grads))

    @classmethod
    def cov_swift_kron_A(cls, module, in_data):
        n, d, _ = in_data.shape
        return in_data.sum(dim=-1) if n < d else cls.cov_kron_A(module, in_data)

    @classmethod
    def cov_swift_kron_B(cls, module, out_grads):
        n, c_out, _ = out_grads.shape
        return out_grads.sum(dim=-1) if n < c_out else cls.cov_kron_B(module, out_grads)

    @classmethod
    def _basis(cls, t, gram_fn):
        n, d, L = t.shape
        if n * L < d:
            return torch.linalg.svd(_rows(t).float(), full_matrices=True)[2].T
        return ops.eigh(gram_fn(t))[1]

    @classmethod
    def cov_kfe_A(cls, module, in_data):
        return cls._basis(in_data, lambda t: cls.cov_kron_A(module, t))

    @classmethod
    def cov_kfe_B(cls, module, out_grads):
        return cls._basis(out_grads, lambda t: cls.cov_kron_B(module, t))

    @classmethod
    def cov_kfe_scale(cls, module, in_data, out_grads, Ua, Ub, bias=True):
        n = in_data.shape[0]
        a_rot = (_rows(in_data) @ Ua).square()
        g_rot = (_rows(out_grads) @ Ub).square()
        scale_w = g_rot.T @ a_rot / n
        return (scale_w, g_rot.mean(dim=0)) if bias else (scale_w,)

    # unit-wise / Gram -------------------------------------------------------------------------
    @staticmethod
    def cov_unit_wise(module, in_data, out_grads):
        bg = torch.bmm(out_grads, in_data.transpose(1, 2))  # n x c_out x d
        return torch.einsum('noi,noj->oij', bg, bg)  # c_out x d x d

    def _gram_hadamard_scale(self, a, g):
        return 1.0 / g.shape[-1] if (a.ndim == 3 and g.ndim == 3) else None

    @staticmethod
    def gram_A(module, in_data1, in_data2=None):
        m1 = in_data1.flatten(start_dim=1)
        m2 = m1 if in_data2 is None else in_data2.flatten(start_dim=1)
        return m1 @ m2.T

    @staticmethod
    def gram_B(module, out_grads1, out_grads2=None):
        L = out_grads1.shape[-1]
        m1 = out_grads1.flatten(start_dim=1)
        m2 = m1 if out_grads2 is None else out_grads2.flatten(start_dim=1)
        return (m1 @ m2.T).div(L)

    # means ------------------------------------------------------------------------------------
    @staticmethod
    def in_data_mean(module, in_data):
        return in_data.mean(dim=(0, 2))

    @staticmethod
    def out_data_mean(module, out_data):
        return out_data.mean(dim=(0, 2, 3))

    def out_data_spatial_mean(self, module, out_data):
        return out_data.flatten(start_dim=2).mean(dim=2)  # n x c_out

    @staticmethod
    def out_spatial_size(module, out_data):
        return out_data.shape[-2] * out_data.shape[-1]

    @staticmethod
    def out_grads_mean(module, out_grads):
        return out_grads.mean(dim=(0, 2))

    def out_grads_spatial_mean(self, module, out_grads):
        return out_grads.mean(dim=2)  # n x c_out

    @staticmethod
    def bfgs_kron_s_As(module, in_data):
        H = module.bfgs.kron.A_inv
        pooled = in_data.mean(dim=2)  # n x d
        s = H @ pooled.mean(dim=0)
        return s, pooled.T @ (pooled @ s)

    def random_sketch_and_gram(self, module, in_data, out_grads):
        """Optionally compress the spatial dimension to ``truncated_rank`` with a truncated SVD of
        the output-gradients before the column sketch."""
        rank = self._truncated_rank
        if rank is not None and rank < in_data.shape[2]:
            u, s, vt = torch.linalg.svd(out_grads, full_matrices=False)
            in_data = torch.bmm(in_data, vt.transpose(1, 2)[:, :, :rank])  # n x d x r
            out_grads = u[:, :, :rank] * s[:, None, :rank]  # n x c_out x r
        return super().random_sketch_and_gram(module, in_data, out_grads)
