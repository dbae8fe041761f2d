"""SENG: sketched empirical natural gradient (Yang, Xu, Wen, Chen, Wang, J. Sci. Comput. 2022).

Parity: asdl/precondition/seng.py:32-142.  Per layer the empirical Fisher F = lambda*I + U^T U / N
(U: per-example gradients) is inverted by Woodbury through the n x n Gram matrix of *sketched*
activations and output-gradients (column subsampling to ``sketching_size``; for convolutions the
spatial dimension is first compressed by a rank-``truncated_rank`` SVD).  The low-rank correction
applied to the gradient is re-expanded with a rank-one (per spatial rank) surrogate of
U^T (lambda*I + U U^T)^-1 U g.
"""
from dataclasses import dataclass
from typing import Dict

import torch
import torch.nn as nn
from torch import Tensor

from .prec_grad_maker import PreconditionedGradientMaker, PreconditioningConfig
from ..core import extend
from ..utils import cholesky_inv
from ..operations import OP_SKETCHED_GRAM

__all__ = ['SengGradientMaker']

_invalid_data_size = -1


@dataclass
class SketchedEmpFisherInfo:
    in_data: Tensor
    out_grads: Tensor
    sub_in_data: Tensor
    sub_out_grads: Tensor
    in_indices: Tensor
    out_indices: Tensor
    gram_inv: Tensor


def _as_3d(t: Tensor):
    return t.unsqueeze(-1) if t.ndim == 2 else t


def maybe_unsqueeze_to_3d(tensor: Tensor):
    """n x d -> n x d x 1; three-dimensional tensors pass through."""
    return _as_3d(tensor)


def maybe_flatten_to_2d(tensor: Tensor):
    """n x d x 1 -> n x d; two-dimensional tensors pass through."""
    return tensor.flatten(start_dim=1) if tensor.ndim == 3 and tensor.shape[-1] == 1 else tensor


class SengGradientMaker(PreconditionedGradientMaker):
    r"""GradientMaker for SENG.

    Args:
        model: module to precondition (Linear / Conv2d layers).
        config: :class:`PreconditioningConfig` (``data_size`` is mandatory).
        sketching_size: number of input / output features kept by the sketch.
        truncated_rank: (Conv2d) rank of the truncated SVD over the spatial dimension.
    """
    _loss_reduction = 'sum'
    _supported_classes = (nn.Linear, nn.Conv2d)

    def __init__(self, model: nn.Module, config: PreconditioningConfig,
                 sketching_size: int = 256, truncated_rank: int = 16):
        super().__init__(model, config)
        if config.data_size == _invalid_data_size:
            raise ValueError('data_size is not set.')
        self._curvature_info: Dict[nn.Module, SketchedEmpFisherInfo] = {}
        self.sketching_size = sketching_size
        self.truncated_rank = truncated_rank

    def do_forward_and_backward(self, step=None):
        return not self.do_update_curvature(step)

    def update_curvature(self):
        config = self.config
        with extend(self.model, OP_SKETCHED_GRAM, ignore_modules=config.ignore_modules) as cxt:
            cxt.set_sketching_size(self.sketching_size)
            cxt.set_truncated_rank(self.truncated_rank)
            self.forward()
            self.backward()
            for module in self.module_dict.values():
                data, sketches, indices, gram = cxt.sketched_inputs_outgrads_gram(module)
                gram_inv = cholesky_inv(gram / config.data_size, config.damping)
                self._curvature_info[module] = SketchedEmpFisherInfo(*data, *sketches, *indices, gram_inv)

    @torch.no_grad()
    def precondition(self):
        """F^-1 g = g/lambda - U^T (lambda*I + U U^T)^-1 U g / lambda with sketched U."""
        N, damping = self.config.data_size, self.config.damping
        for module, info in self._curvature_info.items():
            bias = module.bias is not None and module.bias.requires_grad
            g = module.weight.grad.flatten(start_dim=1)  # d_out x d_in
            if bias:
                g = torch.cat([g, module.bias.grad.unsqueeze(-1)], dim=1)
            g = g / (N * damping)
            # sketched U g: one scalar per example
            sub_g = g[:, :-1] if bias else g
            ratio = 1.
            if info.out_indices is not None:
                sub_g = sub_g.index_select(0, info.out_indices)
                ratio *= g.shape[0] / sub_g.shape[0]
            if info.in_indices is not None:
                sub_g = sub_g.index_select(1, info.in_indices)
                ratio *= g.shape[1] / sub_g.shape[1]
            sub_a, sub_e = _as_3d(info.sub_in_data), _as_3d(info.sub_out_grads)
            v = torch.einsum('ij,nir,njr->n', sub_g * ratio, sub_e, sub_a)
            v = torch.mv(info.gram_inv, v)
            # re-expansion with the full activations / errors
            a, e = _as_3d(info.in_data), _as_3d(info.out_grads)
            if bias:
                a = torch.cat([a, a.new_ones(a.shape[0], 1, a.shape[2])], dim=1)
            root = v.abs().sqrt()
            # all-zero v (the sampled coordinates saw dead units only) leaves the gradient as it is
            mat_in = torch.einsum('n,nir->ir', v / root.sum().clamp_min(torch.finfo(v.dtype).tiny), a)
            mat_out = torch.einsum('n,nor->or', root, e)
            g = g - (mat_out @ mat_in.T) / N ** 2
            if bias:
                module.weight.grad.copy_(g[:, :-1].reshape(module.weight.shape))
                module.bias.grad.copy_(g[:, -1])
            else:
                module.weight.grad.copy_(g.reshape(module.weight.shape))

    def _teardown(self):
        with torch.no_grad():
            self._loss /= self.config.data_size

    # ------------------------------------------------------------------ checkpointing
    _INFO_FIELDS = ('in_data', 'out_grads', 'sub_in_data', 'sub_out_grads', 'in_indices', 'out_indices', 'gram_inv')

    def _curvature_state(self):
        out = {}
        names = {module: name for name, module in self.module_dict.items()}
        for module, info in self._curvature_info.items():
            for field in self._INFO_FIELDS:
                value = getattr(info, field)
                if value is not None:
                    out[f'{names[module]}.seng.{field}'] = value
        return out

    def _load_curvature_state(self, tensors):
        grouped: Dict[str, Dict[str, Tensor]] = {}
        for key, value in tensors.items():
            name, _, field = key.rsplit('.', 2)
            grouped.setdefault(name, {})[field] = value
        for name, module in self.module_dict.items():
            if name in grouped:
                fields = {f: grouped[name].get(f) for f in self._INFO_FIELDS}
                fields = {f: (v.to(self.device) if v is not None else None) for f, v in fields.items()}
                self._curvature_info[module] = SketchedEmpFisherInfo(**fields)
