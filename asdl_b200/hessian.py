"""Hessians of the registered loss: full, layer-wise and diagonal matrices, Hessian-vector
products, and the matrix-free tools built on them (power iteration, conjugate gradients,
quadratic forms).

Parity: asdl/hessian.py:18-289.  Results are stored on the modules as ``module.hessian``
(``SymMatrix``) / ``model.hvp`` (``ParamVector``) and accumulate across calls.
The dense Hessian is built from double backward passes over *batches* of basis vectors
(``is_grads_batched``) instead of one backward per row.
"""
from dataclasses import dataclass
from typing import Any, List, Tuple, Union

import torch
from torch import Tensor
import torch.nn as nn

from .grad_maker import GradientMaker
from .matrices import SHAPE_FULL, SHAPE_LAYER_WISE, SHAPE_DIAG
from .symmatrix import SymMatrix, Diag
from .vector import ParamVector
from .mvp import power_method, conjugate_gradient_method, quadratic_form

__all__ = ['HessianConfig', 'HessianMaker']

_supported_shapes = [SHAPE_FULL, SHAPE_LAYER_WISE, SHAPE_DIAG]


@dataclass
class HessianConfig:
    hessian_attr: str = 'hessian'
    tmp_hessian_attr: str = 'tmp_hessian'
    hvp_attr: str = 'hvp'
    tmp_hvp_attr: str = 'tmp_hvp'
    hessian_shapes: List[str] = None


class HessianMaker(GradientMaker):
    """Hessian of the loss in the shapes full / layer_wise / diag (row-by-row double backward), stored as
    ``module.hessian`` (``SymMatrix``), Hessian-vector products as ``module.hvp``, and the matrix-free tools
    ``hessian_eig`` / ``hessian_free`` / ``hessian_quadratic_form``.  Reference: asdl/hessian.py:27-289.
    """
    def __init__(self, model: nn.Module, config):
        super().__init__(model)
        self.config = config

    def zero_hessian(self, hvp=False):
        attr = self.config.hvp_attr if hvp else self.config.hessian_attr
        for module in self.model.modules():
            if hasattr(module, attr):
                delattr(module, attr)

    def forward_and_backward(self, scale=1., accumulate=False, calc_loss_grad=False, hvp=False,
                             vec: ParamVector = None) -> Union[Tuple[Any, Tensor], Any]:
        """Computes the Hessian in the configured shapes (or ``H @ vec`` with ``hvp=True``),
        multiplies by ``scale`` and stores / accumulates it on the modules."""
        if not accumulate:
            self.zero_hessian(hvp)
        self.forward()
        if hvp:
            params = [p for p in self.model.parameters() if p.requires_grad]
            v, g = _hvp(self._loss, params, vec)
            setattr(self.model, self.config.tmp_hvp_attr, v)
            if calc_loss_grad:
                for param, grad in zip(params, g.values()):
                    param.grad = grad.detach()
        else:
            self._hessian(calc_loss_grad)
        self.accumulate(scale)
        return self._model_output, self._loss

    def _hessian(self, calc_loss_grad=False):
        model, loss = self.model, self._loss
        shapes = self.config.hessian_shapes
        shapes = {shapes} if isinstance(shapes, str) else set(shapes)
        for shape in shapes:
            if shape not in _supported_shapes:
                raise ValueError(f'Invalid hessian_shape: {shape}. {_supported_shapes} are supported.')
        attr = self.config.tmp_hessian_attr
        params = [p for p in model.parameters() if p.requires_grad]
        full = None
        if SHAPE_FULL in shapes:
            full = _hessian(loss, params, save_grad=calc_loss_grad)
            setattr(model, attr, SymMatrix(data=full))
        if SHAPE_LAYER_WISE not in shapes and SHAPE_DIAG not in shapes:
            return
        # offsets of every parameter inside the full matrix
        offsets, offset = {}, 0
        for p in params:
            offsets[id(p)] = offset
            offset += p.numel()
        for module in model.modules():
            w, b = getattr(module, 'weight', None), getattr(module, 'bias', None)
            own = [p for p in (w, b) if isinstance(p, Tensor) and p.requires_grad]
            if not own:
                continue
            if full is None:
                block = _hessian(loss, own, save_grad=calc_loss_grad)
            else:
                idx = torch.cat([torch.arange(offsets[id(p)], offsets[id(p)] + p.numel(),
                                              device=full.device) for p in own])
                block = full[idx][:, idx]
            if SHAPE_LAYER_WISE in shapes:
                existing = getattr(module, attr, None)
                if existing is not None and module is model:
                    pass  # the root module already carries the full matrix
                else:
                    setattr(module, attr, SymMatrix(data=block))
            if SHAPE_DIAG in shapes:
                d = torch.diag(block)
                pieces, start = {}, 0
                for name, p in (('weight', w), ('bias', b)):
                    if isinstance(p, Tensor) and p.requires_grad:
                        pieces[name] = d[start:start + p.numel()].view_as(p).clone()
                        start += p.numel()
                diag = Diag(weight=pieces.get('weight'), bias=pieces.get('bias'))
                existing = getattr(module, attr, None)
                if existing is not None:
                    existing.diag = diag
                else:
                    setattr(module, attr, SymMatrix(diag=diag))

    def _pop(self, module, attr):
        value = getattr(module, attr, None)
        if value is not None:
            delattr(module, attr)
        return value

    def accumulate(self, scale=1.):
        """Move the freshly computed (temporary) results into the accumulated attributes."""
        cfg = self.config
        for module in self.model.modules():
            self._accumulate(module, self._pop(module, cfg.tmp_hessian_attr), cfg.hessian_attr, scale)
            self._accumulate(module, self._pop(module, cfg.tmp_hvp_attr), cfg.hvp_attr, scale)

    @staticmethod
    def _accumulate(module, new, dst_attr, scale):
        if new is None:
            return
        if scale != 1:
            new.mul_(scale)
        existing = getattr(module, dst_attr, None)
        if existing is None:
            setattr(module, dst_attr, new)
        else:
            existing += new  # in place, so that stored inverses survive

    # ------------------------------------------------------------------ matrix-free tools
    def _get_hvp_fn(self):
        def hvp_fn(vec: ParamVector) -> ParamVector:
            self.forward_and_backward(hvp=True, vec=vec)
            return getattr(self.model, self.config.hvp_attr)
        return hvp_fn

    def _grad_vector(self):
        grads = {p: p.grad for p in self.model.parameters() if p.requires_grad}
        return ParamVector(grads.keys(), grads.values())

    def hessian_eig(self, top_n=1, max_iters=100, tol=1e-7, is_distributed=False, print_progress=False):
        return power_method(self._get_hvp_fn(), self.model, top_n=top_n, max_iters=max_iters,
                            tol=tol, is_distributed=is_distributed, print_progress=print_progress)

    def hessian_free(self, b=None, init_x=None, damping=1e-3, max_iters=None, tol=1e-8,
                     print_progress=False):
        if b is None:
            b = self._grad_vector()
        return conjugate_gradient_method(self._get_hvp_fn(), b, init_x=init_x, damping=damping,
                                         max_iters=max_iters, tol=tol, print_progress=print_progress)

    def hessian_quadratic_form(self, vec: ParamVector = None):
        if vec is None:
            vec = self._grad_vector()
        return quadratic_form(self._get_hvp_fn(), vec)


def _hvp(output, inputs, vec: ParamVector):
    grads = torch.autograd.grad(output, inputs=inputs, create_graph=True)
    v = torch.autograd.grad(grads, inputs=inputs, grad_outputs=tuple(vec.values()))
    return ParamVector(inputs, v), ParamVector(inputs, grads)


def _gradient(outputs, inputs, grad_outputs=None, retain_graph=None, create_graph=False):
    """Flattened gradient of ``outputs`` w.r.t. a list of tensors (zeros where unused)."""
    inputs = [inputs] if torch.is_tensor(inputs) else list(inputs)
    grads = torch.autograd.grad(outputs, inputs, grad_outputs, allow_unused=True,
                                retain_graph=retain_graph, create_graph=create_graph)
    return torch.cat([(g if g is not None else torch.zeros_like(x)).reshape(-1)
                      for g, x in zip(grads, inputs)])


def _hessian(output, inputs, out=None, allow_unused=False, create_graph=False, save_grad=False,
             chunk=256):
    """Dense Hessian of a scalar ``output`` w.r.t. ``inputs`` (a tensor or list of tensors)."""
    if output.ndim != 0:
        raise ValueError(f'Number of output dimensions has to be 0. Got {output.ndim}')
    inputs = [inputs] if torch.is_tensor(inputs) else list(inputs)
    n = sum(p.numel() for p in inputs)
    grads = torch.autograd.grad(output, inputs, create_graph=True, allow_unused=True)
    if save_grad:
        for p, g in zip(inputs, grads):
            if g is not None and p.requires_grad:
                p.grad = g.detach().clone()
    flat = torch.cat([(g if g is not None else torch.zeros_like(p)).reshape(-1)
                      for g, p in zip(grads, inputs)])
    hess = output.new_zeros(n, n) if out is None else out
    if not flat.requires_grad:
        return hess
    eye = torch.eye(n, device=flat.device, dtype=flat.dtype)
    for lo in range(0, n, chunk):
        basis = eye[lo:lo + chunk]
        try:
            rows = torch.autograd.grad(flat, inputs, grad_outputs=basis, retain_graph=True,
                                       create_graph=create_graph, allow_unused=True,
                                       is_grads_batched=True)
            rows = torch.cat([(r if r is not None else p.new_zeros(basis.shape[0], *p.shape))
                              .reshape(basis.shape[0], -1) for r, p in zip(rows, inputs)], dim=1)
        except RuntimeError:  # an op without a batching rule: fall back to one backward per row
            rows = torch.stack([_gradient(flat[lo + k], inputs, retain_graph=True,
                                          create_graph=create_graph) for k in range(basis.shape[0])])
        hess[lo:lo + basis.shape[0]] += rows
    return hess
