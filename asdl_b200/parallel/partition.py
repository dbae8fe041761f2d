"""Assignment of per-layer inverse / preconditioning work to ranks.

The reference splits the layer list into contiguous chunks by ``numel(weight)**0.3``
(asdl/precondition/natural_gradient.py:162-321; ``sum(dim**0.4)`` for Shampoo,
asdl/precondition/shampoo.py:58-198).  Here the cost model is the actual arithmetic of the owner's
work - cubic in the factor sizes for the inverse plus the two-sided product for the
preconditioning - and the assignment is longest-processing-time-first onto the least loaded rank,
which needs no contiguity and leaves no rank idle while another holds two large layers.
The result is a pure function of the layer list, so every rank computes the same table.
"""
import heapq
from typing import List, Optional, Sequence

import torch.nn as nn

__all__ = ['assign_owners', 'curvature_cost', 'shampoo_cost', 'balance_report']


def _kron_dims(module: nn.Module):
    if isinstance(module, nn.Linear):
        return module.in_features, module.out_features
    if isinstance(module, nn.Conv2d):
        kh, kw = module.kernel_size
        return module.in_channels // module.groups * kh * kw, module.out_channels
    if isinstance(module, nn.Embedding):
        return module.num_embeddings, module.embedding_dim
    weight = getattr(module, 'weight', None)
    if weight is not None and weight.ndim >= 2:
        return weight[0].numel(), weight.shape[0]
    return 1, 1


def curvature_cost(module: nn.Module, shape: str) -> float:
    """Estimated FLOPs of one inverse update plus one preconditioning of ``module``."""
    n_params = sum(p.numel() for p in module.parameters() if p.requires_grad)
    if shape in ('kron', 'swift_kron', 'kfe'):
        d_in, d_out = _kron_dims(module)
        inverse = float(d_in) ** 3 + float(d_out) ** 3
        apply = 2.0 * d_in * d_out * (d_in + d_out)
        return inverse + apply
    if shape == 'layer_wise':
        return float(n_params) ** 3 + 2.0 * float(n_params) ** 2
    if shape == 'unit_wise':
        if isinstance(module, (nn.BatchNorm1d, nn.BatchNorm2d, nn.LayerNorm)):
            return 16.0 * n_params
        d_in, d_out = _kron_dims(module)
        return d_out * float(d_in + 1) ** 3
    return 4.0 * n_params  # diagonal


def shampoo_cost(shape: Sequence[int], block_size: int, newton_iters: int = 20) -> float:
    """Estimated FLOPs of the inverse-root updates of one parameter tensor of ``shape``."""
    total = 0.0
    for dim in shape:
        n_blocks = (dim + block_size - 1) // block_size
        size = min(dim, block_size)
        total += n_blocks * newton_iters * 8.0 * float(size) ** 3
    return total


def assign_owners(costs: Sequence[float], world_size: int,
                  fixed: Optional[Sequence[Optional[int]]] = None) -> List[int]:
    """Owner rank for each item.  ``fixed[i]`` pins item i to a rank; the rest are placed
    largest-first on the currently least loaded rank (ties broken by rank index)."""
    n = len(costs)
    owners = [0] * n
    load = [0.0] * world_size
    if fixed is not None:
        for i, rank in enumerate(fixed):
            if rank is not None:
                owners[i] = rank
                load[rank] += costs[i]
    heap = [(load[r], r) for r in range(world_size)]
    heapq.heapify(heap)
    free = [i for i in range(n) if fixed is None or fixed[i] is None]
    for i in sorted(free, key=lambda k: (-costs[k], k)):
        cur, rank = heapq.heappop(heap)
        owners[i] = rank
        heapq.heappush(heap, (cur + costs[i], rank))
    return owners


def balance_report(costs: Sequence[float], owners: Sequence[int], world_size: int):
    """(max load / mean load, per-rank loads) - 1.0 is a perfect balance."""
    load = [0.0] * world_size
    for c, o in zip(costs, owners):
        load[o] += c
    mean = sum(load) / world_size if world_size else 0.0
    return (max(load) / mean if mean > 0 else 1.0), load
