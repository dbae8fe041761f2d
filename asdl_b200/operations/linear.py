"""Statistics of ``nn.Linear``.

Shapes: ``a`` (layer input) n x f_in, ``g`` (output-gradient of the summed loss) n x f_out; any
extra leading dimensions (sequence, ...) are folded into n.  There is no homogeneous coordinate:
A = a^T a, B = g^T g and the bias shares B.  Parity: asdl/operations/linear.py:9-190.
The factor products run through :func:`asdl_b200.ops.gram` (tcgen05 SYRK on CUDA tensors).
"""
import torch
from torch import nn
import torch.nn.functional as F

from .. import ops
from .operation import Operation, ALL_OPS

__all__ = ['Linear']


def _fold_leading(t):
    return t.reshape(-1, t.shape[-1]) if t.ndim > 2 else t


def _eigenbasis(x, gram_fn):
    """Right singular / eigen basis of the sample matrix x (rows = samples)."""
    n, d = x.shape
    if n < d:
        return torch.linalg.svd(x.float(), full_matrices=True)[2].T
    return ops.eigh(gram_fn(x))[1]


class Linear(Operation):
    """Statistics of ``nn.Linear``.  module.weight: f_out x f_in, module.bias: f_out; in_data: n x f_in and
    out_grads: n x f_out after leading dimensions (sequence positions) are folded into n.  Supports every
    operation.  Reference: asdl/operations/linear.py:9-190.
    """
    supported_operations = set(ALL_OPS)

    @staticmethod
    def preprocess_in_data(module, in_data, out_data):
        return _fold_leading(in_data)

    @staticmethod
    def preprocess_out_grads(module, out_grads):
        return _fold_leading(out_grads)

    @staticmethod
    def extend_in_data(in_data):
        return torch.cat([in_data, in_data.new_ones(in_data.shape[0], 1)], dim=1)

    # gradients --------------------------------------------------------------------------------
    @staticmethod
    def batch_grads_weight(module, in_data, out_grads):
        return torch.einsum('no,ni->noi', out_grads, in_data)  # n x f_out x f_in

    @staticmethod
    def batch_grads_bias(module, out_grads):
        return out_grads

    @staticmethod
    def grad_weight(module, in_data, out_grads):
        return out_grads.T @ in_data

    @staticmethod
    def grad_bias(module, out_grads):
        return out_grads.sum(dim=0)

    # diagonal ---------------------------------------------------------------------------------
    @staticmethod
    def cov_diag_weight(module, in_data, out_grads):
        return out_grads.square().T @ in_data.square()  # f_out x f_in

    @staticmethod
    def cov_diag_bias(module, out_grads):
        return out_grads.square().sum(dim=0)

    # Kronecker factors ------------------------------------------------------------------------
    @staticmethod
    def cov_kron_A(module, in_data):
        return ops.gram(in_data)  # f_in x f_in

    @staticmethod
    def cov_kron_B(module, out_grads):
        return ops.gram(out_grads)  # f_out x f_out

    @classmethod
    def cov_swift_kron_A(cls, module, in_data):
        n, f_in = in_data.shape
        return in_data if n < f_in else cls.cov_kron_A(module, in_data)

    @classmethod
    def cov_swift_kron_B(cls, module, out_grads):
        n, f_out = out_grads.shape
        return out_grads if n < f_out else cls.cov_kron_B(module, out_grads)

    @classmethod
    def cov_kfe_A(cls, module, in_data):
        return _eigenbasis(in_data, lambda x: cls.cov_kron_A(module, x))

    @classmethod
    def cov_kfe_B(cls, module, out_grads):
        return _eigenbasis(out_grads, lambda x: cls.cov_kron_B(module, x))

    @classmethod
    def cov_kfe_scale(cls, module, in_data, out_grads, Ua, Ub, bias=True):
        n = in_data.shape[0]
        a_rot = (in_data @ Ua).square()
        g_rot = (out_grads @ Ub).square()
        scale_w = g_rot.T @ a_rot / n
        return (scale_w, g_rot.mean(dim=0)) if bias else (scale_w,)

    # unit-wise / Gram -------------------------------------------------------------------------
    @staticmethod
    def cov_unit_wise(module, in_data, out_grads):
        f_in = in_data.shape[1]
        outer = torch.einsum('ni,nj->nij', in_data, in_data).flatten(start_dim=1)
        return (out_grads.square().T @ outer).view(-1, f_in, f_in)  # f_out x f_in x f_in

    def _cvp_without_batch_grads(self, a, g, vector, has_w, has_b):
        """With per-example gradients g_n a_n^T (and g_n for the bias) the coefficient of example n is
        c_n = g_n^T V_w a_n + g_n . v_b, and the product is (g o c)^T a (and its column sums): two
        GEMMs over the batch instead of an n x d_out x d_in tensor (asdl/operations/operation.py:247-263
        forms the per-example gradients)."""
        if a.ndim != 2 or g.ndim != 2:
            return None
        module = self._module
        d_out, d_in = module.weight.shape
        nw = d_out * d_in if has_w else 0
        coef = torch.zeros(g.shape[0], device=g.device, dtype=torch.float32)
        if has_w:
            coef += (ops.matmul_nn(g, vector[:nw].view(d_out, d_in)) * a).sum(dim=1)
        if has_b:
            coef += g.float() @ vector[nw:].float()
        weighted = g.float() * coef.unsqueeze(1)
        out_w = ops.matmul_tn(weighted, a).to(module.weight.dtype) if has_w else None
        out_b = weighted.sum(dim=0).to(module.bias.dtype) if has_b else None
        return out_w, out_b

    def _gram_hadamard_scale(self, a, g):
        return 1.0 if (a.ndim == 2 and g.ndim == 2) else None

    @staticmethod
    def gram_A(module, in_data1, in_data2=None):
        return in_data1 @ (in_data1 if in_data2 is None else in_data2).T

    @staticmethod
    def gram_B(module, out_grads1, out_grads2=None):
        return out_grads1 @ (out_grads1 if out_grads2 is None else out_grads2).T

    # relative FIM -----------------------------------------------------------------------------
    @staticmethod
    def rfim_relu(module, in_data, out_data):
        nu = torch.sigmoid(out_data).square()
        return torch.einsum('bo,bi,bj->oij', nu, in_data, in_data)  # f_out x f_in x f_in

    @staticmethod
    def rfim_softmax(module, in_data, out_data):
        probs = F.softmax(out_data, dim=1)
        hess = torch.diag_embed(probs) - torch.einsum('bi,bj->bij', probs, probs)
        return torch.einsum('bij,bk,bl->ikjl', hess, in_data, in_data)

    # means ------------------------------------------------------------------------------------
    @staticmethod
    def in_data_mean(module, in_data):
        return in_data.mean(dim=0)

    @staticmethod
    def out_data_mean(module, out_data):
        return _fold_leading(out_data).mean(dim=0)

    @staticmethod
    def out_spatial_size(module, out_data):
        return 1

    @staticmethod
    def out_grads_mean(module, out_grads):
        return out_grads.mean(dim=0)

    @staticmethod
    def bfgs_kron_s_As(module, in_data):
        H = module.bfgs.kron.A_inv
        s = H @ in_data.mean(dim=0)
        return s, in_data.T @ (in_data @ s)
