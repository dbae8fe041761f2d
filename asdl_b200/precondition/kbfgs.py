"""K-BFGS: Kronecker-factored quasi-Newton preconditioning (Goldfarb, Ren, Bahamou,
arXiv:2006.08877; mini-batch Hessian-action variant arXiv:2102.06737).

Parity: asdl/precondition/kbfgs.py:18-217.  Per layer the inverse of the input factor A is
maintained by BFGS updates on the moving average of A (or on a mini-batch Hessian action), and
the inverse of the output factor B by BFGS updates from pairs (change of the mean layer output,
change of the mean output-gradient) that are obtained by running the *previous* batch through the
model once more after the parameters moved.  Powell damping and Levenberg-Marquardt damping keep
the pairs admissible; convolutions split the damping by sqrt(spatial size).

Difference: the rank-two inverse update is applied to the stored matrix itself (the reference
symmetrises into a temporary and updates the temporary, so its stored inverses never change).
"""
import math

import torch
import torch.nn as nn
from torch import Tensor

from .. import ops
from ..core import extend
from ..operations import (OP_MEAN_INPUTS, OP_SPATIAL_MEAN_OUTPUTS, OP_SPATIAL_MEAN_OUTGRADS,
                          OP_OUT_SPATIAL_SIZE, OP_COV_KRON, OP_BFGS_KRON_S_AS, OperationContext)
from ..utils import cholesky_inv
from ..symmatrix import SymMatrix, Kron
from .prec_grad_maker import PreconditionedGradientMaker, PreconditioningConfig

__all__ = ['KronBfgsGradientMaker', 'powell_lm_damping_', 'bfgs_inv_update_']


class KronBfgsGradientMaker(PreconditionedGradientMaker):
    r"""GradientMaker for K-BFGS.

    Args:
        model: module to precondition (Linear / Conv2d layers).
        config: :class:`PreconditioningConfig` (``data_size``, ``damping``, ``ema_decay`` used).
        minibatch_hessian_action: update :math:`A^{-1}` from the action of the current
            mini-batch factor on :math:`s` instead of from the moving average of A.
        mu1: Powell damping threshold :math:`\mu_1\in(0,1)`.
    """
    _supported_classes = (nn.Linear, nn.Conv2d)

    def __init__(self, model: nn.Module, config: PreconditioningConfig,
                 minibatch_hessian_action: bool = False, mu1: float = 0.2):
        super().__init__(model, config)
        self._last_call = ((), {})
        self._A_inv_exists = False
        self._B_inv_exists = False
        self.minibatch_hessian_action = minibatch_hessian_action
        self.bfgs_attr = 'bfgs'
        self.mu1 = mu1
        self.mean_outputs_attr = 'mean_outputs'
        self.mean_outgrads_attr = 'mean_outgrads'

    def do_forward_and_backward(self, step=None):
        return not self.do_update_preconditioner(step)

    def _startup(self):
        step = self.state['step']
        if step > 0 and self.do_update_preconditioner(step - 1):
            if not self._last_call[0] and not self._last_call[1]:
                return  # resumed from a checkpoint: the batch of the open (s, y) pair is gone, drop the pair
            self._post_preconditioner_update()

    def update_preconditioner(self):
        """Forward/backward on the current batch with hooks: update A^-1, remember the mean
        outputs and output-gradients (the B pair is completed at the next step)."""
        if self.minibatch_hessian_action and self._A_inv_exists:
            op_names = (OP_BFGS_KRON_S_AS, OP_SPATIAL_MEAN_OUTPUTS, OP_OUT_SPATIAL_SIZE)
        else:
            op_names = (OP_COV_KRON, OP_MEAN_INPUTS, OP_SPATIAL_MEAN_OUTPUTS, OP_OUT_SPATIAL_SIZE)
        op_names += (OP_SPATIAL_MEAN_OUTGRADS,)
        with extend(self.module_dict, *op_names) as cxt:
            self.forward()
            self._update_A_inv(cxt)
            self._store_mean(cxt, is_forward=True)
            self._loss.backward()
            self._store_mean(cxt, is_forward=False)
        self._last_call = (self._model_args, dict(self._model_kwargs))

    def _post_preconditioner_update(self):
        """Re-run the previous batch with the updated parameters and update B^-1 from the
        differences of the means."""
        current = (self._model_args, self._model_kwargs)
        saved_grads = [(p, p.grad) for p in self.model.parameters()]
        for p, _ in saved_grads:
            p.grad = None
        self._model_args, self._model_kwargs = self._last_call[0], dict(self._last_call[1])
        op_names = (OP_SPATIAL_MEAN_OUTPUTS, OP_SPATIAL_MEAN_OUTGRADS, OP_OUT_SPATIAL_SIZE)
        with extend(self.module_dict, *op_names) as cxt:
            self.forward()
            self._loss.backward()
            self._update_B_inv(cxt)
        self._model_args, self._model_kwargs = current
        for p, g in saved_grads:
            p.grad = g
        self._B_inv_exists = True

    def precondition(self):
        if not self._B_inv_exists:
            return
        for module in self.module_dict.values():
            matrix: SymMatrix = getattr(module, self.bfgs_attr)
            vec_weight = module.weight.grad
            if vec_weight is None:
                raise ValueError('gradient has not been calculated.')
            vec_bias = None
            if module.bias is not None and module.bias.requires_grad:
                vec_bias = module.bias.grad
                if vec_bias is None:
                    raise ValueError('gradient has not been calculated.')
            matrix.kron.mvp(vec_weight=vec_weight, vec_bias=vec_bias, use_inv=True, inplace=True)

    def _update_A_inv(self, cxt: OperationContext):
        config = self.config
        for module in self.module_dict.values():
            damping = self._get_damping(cxt, module, is_A=True)
            bfgs = getattr(module, self.bfgs_attr, None)
            if self.minibatch_hessian_action and self._A_inv_exists:
                s, As = cxt.bfgs_kron_s_As(module)
                n = self.config.data_size
                y = As / n + damping * s
            else:
                new = cxt.cov_symmatrix(module, pop=True).mul_(1 / config.data_size)
                if bfgs is None:
                    setattr(module, self.bfgs_attr, new)
                    bfgs = new
                else:
                    ema = config.ema_decay if 0 < config.ema_decay <= 1 else 1.0  # unset: keep the newest
                    bfgs.mul_(1 - ema)
                    bfgs += new.mul_(ema)  # in-place add keeps the stored inverses
                A = bfgs.kron.A
                if bfgs.kron.A_inv is None:
                    bfgs.kron.A_inv = cholesky_inv(A, damping)
                s = torch.mv(bfgs.kron.A_inv, cxt.mean_in_data(module))
                y = torch.mv(A, s) + damping * s
            if bfgs is None:
                raise ValueError(f'Matrix for {module} is not calculated yet.')
            bfgs_inv_update_(bfgs.kron.A_inv, s, y)
        self._A_inv_exists = True

    def _store_mean(self, cxt: OperationContext, is_forward=True):
        for module in self.module_dict.values():
            if is_forward:
                setattr(module, self.mean_outputs_attr, cxt.spatial_mean_out_data(module))
            else:
                setattr(module, self.mean_outgrads_attr, cxt.spatial_mean_out_grads(module))

    def _update_B_inv(self, cxt: OperationContext):
        for module in self.module_dict.values():
            damping = self._get_damping(cxt, module, is_A=False)
            bfgs = getattr(module, self.bfgs_attr)
            s = cxt.spatial_mean_out_data(module) - getattr(module, self.mean_outputs_attr)
            y = cxt.spatial_mean_out_grads(module) - getattr(module, self.mean_outgrads_attr)
            if s.ndim > 1:  # n x c_out per-example means (Conv2d) -> batch mean
                s, y = s.mean(dim=0), y.mean(dim=0)
            if bfgs.kron.B_inv is None:
                bfgs.kron.B_inv = torch.eye(s.shape[-1], device=s.device, dtype=s.dtype)
            s, y = s.clone(), y.clone()
            powell_lm_damping_(bfgs.kron.B_inv, s, y, mu1=self.mu1, mu2=damping)
            bfgs_inv_update_(bfgs.kron.B_inv, s, y)

    def _get_damping(self, cxt: OperationContext, module: nn.Module, is_A=True):
        root = math.sqrt(self.config.damping)
        if isinstance(module, nn.Conv2d):
            spatial = math.sqrt(cxt.out_spatial_size(module))
            return root * spatial if is_A else root / spatial
        return root

    def _curvature_state(self):
        out = {}
        for name, module in self.module_dict.items():
            bfgs = getattr(module, self.bfgs_attr, None)
            if bfgs is not None:
                out.update(bfgs.tensors(prefix=f'{name}.'))
        return out

    def _load_curvature_state(self, tensors):
        grouped = {}
        for key, value in tensors.items():
            name, rest = key.split('.', 1)
            grouped.setdefault(name, {})[rest] = value
        for name, module in self.module_dict.items():
            if name in grouped:
                setattr(module, self.bfgs_attr, SymMatrix.from_tensors(
                    {k: v.to(self.device) for k, v in grouped[name].items()}))
                kron = getattr(module, self.bfgs_attr).kron
                self._A_inv_exists = self._A_inv_exists or kron.A_inv is not None
                self._B_inv_exists = self._B_inv_exists or kron.B_inv is not None


def _bfgs_kernels_ok(H, s, y):
    """The CUDA kernels of the BFGS update take fp32 tensors in their natural layout."""
    return (ops.cuda_kernels_enabled(H, s, y) and H.dtype == s.dtype == y.dtype == torch.float32
            and H.ndim == 2 and H.stride(1) == 1 and s.is_contiguous() and y.is_contiguous())


def powell_lm_damping_(H: Tensor, s: Tensor, y: Tensor, mu1: float, mu2: float):
    """Make the pair (s, y) safe for a BFGS update of H = B^-1: Powell's damping pulls s towards
    H y when s^T y < mu1 * y^T H y, then y <- y + mu2 * s (Levenberg-Marquardt on H^-1).
    s and y are modified in place."""
    if mu1 <= 0 or 1 <= mu1:
        raise ValueError(f'mu1 has to be in (0, 1). Got {mu1}.')
    if mu2 <= 0:
        raise ValueError(f'mu2 has to be > 0. Got {mu2}.')
    if _bfgs_kernels_ok(H, s, y):
        ops.extension().bfgs_powell_damping(H, s, y, float(mu1), float(mu2))
        return
    Hy = torch.mv(H, y)
    ytHy = torch.dot(y, Hy)
    sty = torch.dot(s, y)
    gap = ytHy - sty
    theta = torch.where((sty < mu1 * ytHy) & (gap > 0), (1 - mu1) * ytHy / gap.clamp_min(1e-30),
                        torch.ones_like(sty))
    s.mul_(theta).add_(Hy * (1 - theta))
    y.add_(s, alpha=mu2)


def bfgs_inv_update_(H: Tensor, s: Tensor, y: Tensor):
    """In-place BFGS update of the inverse Hessian approximation H (Sherman-Morrison form):
    H <- H + (s^T y + y^T H y) s s^T / (s^T y)^2 - (H y s^T + s y^T H) / (s^T y)."""
    if H.ndim != 2 or H.shape[0] != H.shape[1]:
        raise ValueError(f'H has to be a {Tensor} containing a symmetric matrix.')
    n = H.shape[0]
    for name, v in (('s', s), ('y', y)):
        if v.ndim != 1 or v.shape[0] != n:
            raise ValueError(f'{name} has to be a {Tensor} containing a vector of same dimension as H.')
    if _bfgs_kernels_ok(H, s, y):
        ops.extension().bfgs_inv_update(H, s, y)
        return H
    H.copy_((H + H.T) / 2)
    sty = torch.dot(s, y)
    Hy = torch.mv(H, y)
    ytHy = torch.dot(y, Hy)
    cross = torch.outer(Hy, s)
    # a pair without usable curvature (s^T y not safely positive, e.g. a layer whose mean output
    # gradient is removed by a following BatchNorm) leaves H as it is; decided on the device
    ok = torch.isfinite(sty) & (sty > 1e-12 * (1 + s.norm() * y.norm()))
    safe = torch.where(ok, sty, torch.ones_like(sty))
    update = torch.outer(s, s) * ((safe + ytHy) / safe ** 2) - (cross + cross.T) / safe
    H.add_(torch.where(ok & torch.isfinite(update).all(), update, torch.zeros_like(update)))
    return H
