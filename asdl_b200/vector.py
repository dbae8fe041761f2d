"""Parameter-shaped vectors and the few collectives / orthogonalisation helpers built on them.

Parity: asdl/vector.py:11-135 (``ParamVector``, ``reduce_vectors``, ``normalization``,
``orthnormal``).  A ``ParamVector`` maps each parameter (identity-keyed) to a tensor of the same
shape; arithmetic is elementwise over the shared key order.  Reductions that need one scalar
(``dot``, ``norm``) are evaluated with ``torch._foreach`` style fused reductions rather than by
materialising the flattened concatenation.
"""
from collections import OrderedDict
from typing import Iterable, List, Union

import torch
import torch.distributed as dist
import torch.nn as nn

__all__ = ['ParamVector', 'reduce_vectors', 'normalization', 'orthnormal']


class ParamVector:
    """Ordered map parameter -> tensor of the same shape with vector-space arithmetic (``+``, ``add_``, ``mul_``,
    ``dot``, ``norm``), slicing by module or parameter, and a flat view for collectives and dense algebra.
    Reference: asdl/vector.py:11-102.
    """
    def __init__(self, params: Iterable[torch.Tensor],
                 values: Union[torch.Tensor, Iterable[torch.Tensor]]):
        params = list(params)
        if len(params) == 0:
            raise ValueError('params cannot be empty.')
        self.vectors: 'OrderedDict[torch.Tensor, torch.Tensor]' = OrderedDict()
        if isinstance(values, torch.Tensor):
            if values.ndim != 1:
                raise ValueError(f'values.ndim has to be 1. Got {values.ndim}.')
            total = sum(p.numel() for p in params)
            if total != values.numel():
                raise ValueError(f'pointer has to be {values.numel()}. Got {total}.')
            chunks = torch.split(values, [p.numel() for p in params])
            for p, chunk in zip(params, chunks):
                self.vectors[p] = chunk.view_as(p)
        elif isinstance(values, Iterable):
            for p, v in zip(params, values):
                if p.shape != v.shape:
                    raise ValueError(f'param.shape ({p.shape}) does not match value.shape ({v.shape}).')
                self.vectors[p] = v
        else:
            raise TypeError(f'Invalid vectors type: {type(values)}')

    # -- dict-like access -------------------------------------------------------------------
    def params(self):
        return self.vectors.keys()

    def values(self):
        return self.vectors.values()

    def _pairs(self, other):
        return zip(self.values(), other.values())

    # -- arithmetic -------------------------------------------------------------------------
    def __add__(self, other):
        return ParamVector(self.params(), [a + b for a, b in self._pairs(other)])

    def __iadd__(self, other):
        for a, b in self._pairs(other):
            a += b
        return self

    def add(self, other, alpha=1):
        return ParamVector(self.params(), [a.add(b, alpha=alpha) for a, b in self._pairs(other)])

    def add_(self, other, alpha=1):
        for a, b in self._pairs(other):
            a.add_(b, alpha=alpha)
        return self

    def mul(self, value):
        return ParamVector(self.params(), [v.mul(value) for v in self.values()])

    def mul_(self, value):
        for v in self.values():
            v.mul_(value)
        return self

    def extend(self, other):
        if set(self.params()) & set(other.params()):
            raise ValueError('self.params and other.params cannot have a common element.')
        self.vectors.update(other.vectors)

    def dot(self, other):
        parts = [torch.sum(a * b) for a, b in self._pairs(other)]
        return torch.stack(parts).sum()

    def norm(self):
        return torch.sqrt(self.dot(self))

    # -- slicing ----------------------------------------------------------------------------
    def get_vectors_by_module(self, module: nn.Module):
        return self.get_vectors_by_params(list(module.parameters()))

    def get_vectors_by_params(self, params: List[torch.Tensor]):
        picked = OrderedDict((p, self.vectors[p]) for p in params if p in self.vectors)
        if not picked:
            return None
        return ParamVector(picked.keys(), picked.values())

    def get_vector_by_param(self, param: torch.Tensor, default=None) -> torch.Tensor:
        if param is None:
            return default
        return self.vectors.get(param, default)

    def get_flatten_vector(self):
        return torch.cat([v.reshape(-1) for v in self.values()])

    def numel(self):
        return sum(v.numel() for v in self.values())

    def copy(self):
        return ParamVector(self.params(), [v.detach().clone() for v in self.values()])


def reduce_vectors(vectors: ParamVector, is_master=True, all_reduce=False) -> ParamVector:
    """Sum a ParamVector over all ranks (``all_reduce``) or onto rank 0."""
    packed = vectors.get_flatten_vector()
    if all_reduce:
        dist.all_reduce(packed)
    else:
        dist.reduce(packed, dst=0)
    out = ParamVector(vectors.params(), packed) if (all_reduce or is_master) else None
    dist.barrier()
    return out


def normalization(v: ParamVector) -> ParamVector:
    """In-place scaling to (almost) unit norm, matching ``v / (|v| + 1e-6)``."""
    length = float(v.norm())
    v.mul_(1.0 / (length + 1e-6))
    return v


def orthnormal(w: ParamVector, v_list: List[ParamVector]) -> ParamVector:
    """One Gram-Schmidt sweep of ``w`` against ``v_list`` followed by normalisation."""
    for v in v_list:
        w = w.add(v, alpha=-w.dot(v))
    return normalization(w)
