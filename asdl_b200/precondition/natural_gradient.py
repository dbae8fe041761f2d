"""Natural-gradient preconditioning with Fisher matrices of any shape - full, layer-wise,
Kronecker-factored (K-FAC, optionally "swift"/SKFAC), Kronecker-factored eigenbasis (EKFAC),
unit-wise and diagonal - with an optional exponential moving average of the curvature and
data-parallel execution where the inverse + precondition work of each layer belongs to one
"owner" rank.

Parity: asdl/precondition/natural_gradient.py:28-936 (``NaturalGradientMaker`` and the eight
wrapper classes).  Single-process numerics are the reference's: on a curvature step the Fisher
maker runs the forward/backward (MC/exact Fisher backward passes, then the true-loss backward),
without EMA the damped inverses are produced inside the hooks, with EMA the stored factors are
scaled by ``1-ema_decay`` and the new statistics (scaled by ``ema_decay``) are added, and
``update_preconditioner`` inverts on its own interval.  The gradient is preconditioned in place.

Data-parallel rule (one rule for every mode, replacing the reference's mode-dependent behaviour):
  1. every rank computes statistics and gradients on its shard;
  2. the statistics and gradients of a layer are averaged onto the layer's owner;
  3. the owner keeps the running curvature, inverts it and preconditions the averaged gradient;
  4. owners broadcast the preconditioned gradients; gradients of parameters that carry no
     curvature are all-reduced.
Every rank therefore ends a step with identical ``param.grad`` for *all* parameters.  Owners are
chosen by balancing an n^3-type cost estimate (``asdl_b200.parallel.partition``), not by
contiguous chunks.  Without EMA the inverse is still taken by the owner from the averaged
statistics (the reference inverts each rank's local statistics).  Any ``torch.distributed``
backend works (gloo on CPU included); on CUDA the communication can be taken over by the fused
kernels of :mod:`asdl_b200.parallel`.
"""
from typing import Any, Dict, List, Union

import torch
from torch import nn
import torch.distributed as dist

from ..core import module_wise_assignments, modules_to_assign
from ..matrices import *  # noqa: F401,F403
from ..matrices import (FISHER_MC, FISHER_EMP, SHAPE_FULL, SHAPE_LAYER_WISE, SHAPE_KRON,
                        SHAPE_SWIFT_KRON, SHAPE_KFE, SHAPE_UNIT_WISE, SHAPE_DIAG)
from ..symmatrix import SymMatrix
from ..vector import ParamVector
from ..fisher import LOSS_CROSS_ENTROPY, get_fisher_maker, FisherConfig
from ..utils import nvtx_range
from .prec_grad_maker import PreconditionedGradientMaker, PreconditioningConfig

_invalid_ema_decay = -1
_module_level_shapes = [SHAPE_LAYER_WISE, SHAPE_KRON, SHAPE_SWIFT_KRON, SHAPE_KFE, SHAPE_UNIT_WISE,
                        SHAPE_DIAG]

__all__ = [
    'NaturalGradientMaker', 'FullNaturalGradientMaker', 'LayerWiseNaturalGradientMaker',
    'KfacGradientMaker', 'EkfacGradientMaker', 'UnitWiseNaturalGradientMaker',
    'DiagNaturalGradientMaker', 'EmpNaturalGradientMaker'
]


def _bias_requires_grad(module):
    bias = getattr(module, 'bias', None)
    return bias is not None and bias.requires_grad


def _pack(tensors):
    return torch.cat([t.reshape(-1) for t in tensors])


def _unpack(flat, tensors):
    offset = 0
    for t in tensors:
        n = t.numel()
        t.copy_(flat[offset:offset + n].view_as(t))
        offset += n


class NaturalGradientMaker(PreconditionedGradientMaker):
    """Natural gradient: ``grad <- F^-1 grad`` with F the Fisher information in the chosen shape.

    Args:
        model: module to precondition.
        config: :class:`PreconditioningConfig`.
        fisher_type: ``"fisher_exact"``, ``"fisher_mc"`` (default) or ``"fisher_emp"``.
        fisher_shape: one shape or an assignment list, e.g.
            ``["kron", (nn.BatchNorm2d, "unit_wise")]``.
        loss_type: ``"cross_entropy"`` or ``"mse"`` (ignored for the empirical Fisher).
        scale: multiplier of the Fisher.  grad_scale: multiplier applied to the gradient before
            preconditioning.
        sync_group / sync_group_ranks: process group (and its global ranks) for the collectives.
        module_partitions: optional explicit owner assignment, ``module_partitions[r]`` being the
            modules owned by rank ``r``; modules not listed are assigned automatically.
        n_mc_samples, var, seed: Monte-Carlo Fisher options.
    """
    _supported_classes = (nn.Linear, nn.Conv2d, nn.BatchNorm1d, nn.BatchNorm2d, nn.LayerNorm,
                          nn.Embedding)

    def __init__(self, model, config: PreconditioningConfig,
                 fisher_type: str = FISHER_MC, fisher_shape: Union[str, List[Any]] = SHAPE_FULL,
                 loss_type: str = LOSS_CROSS_ENTROPY, scale: float = 1, grad_scale: float = 1,
                 sync_group: dist.ProcessGroup = None, sync_group_ranks: List[int] = None,
                 module_partitions: List[List[nn.Module]] = None,
                 n_mc_samples: int = 1, var: float = 1., seed: int = None):
        from torch.nn.parallel import DistributedDataParallel as DDP
        if isinstance(model, DDP):
            raise TypeError(f'{DDP} is not supported: this maker synchronises gradients itself.')
        super().__init__(model, config)
        if isinstance(fisher_shape, str):
            fisher_shape = [fisher_shape]
        if not self.do_accumulate and config.curvature_upd_ratio is not None:
            raise ValueError('curvature_upd_ratio cannot be specified when no curvature accumulation is performed.')

        self.named_modules_for_curvature = []
        self.modules_for_curvature = []
        self.shape_for = {}
        for name, module, shapes in module_wise_assignments(self.module_dict, *fisher_shape, named=True):
            if len(shapes) != 1:
                raise ValueError(f'Each module has to be assigned one Fisher shape. '
                                 f'{name} is assigned {len(shapes)} shapes.')
            self.modules_for_curvature.append(module)
            self.named_modules_for_curvature.append((name, module))
            self.shape_for[module] = shapes[0]
            self.shape_for[name] = shapes[0]
        self._named_modules_for = {}

        self.fisher_maker = get_fisher_maker(model, FisherConfig(
            fisher_type=fisher_type, fisher_shapes=fisher_shape, loss_type=loss_type,
            n_mc_samples=n_mc_samples, ignore_modules=config.ignore_modules, var=var, seed=seed))
        self.fisher_type = fisher_type
        self.fisher_shape = fisher_shape
        self.scale = scale
        self.grad_scale = grad_scale

        if sync_group is not None:
            if sync_group_ranks is None:
                raise ValueError('sync_group_ranks is not set.')
            if sync_group.size() != len(sync_group_ranks):
                raise ValueError(f'sync_group.size() ({sync_group.size()}) does not match '
                                 f'len(sync_group_ranks) ({len(sync_group_ranks)}).')
        self.sync_group = sync_group
        self.sync_group_ranks = sync_group_ranks
        if dist.is_available() and dist.is_initialized():
            self.world_rank = dist.get_rank(sync_group)
            self.world_size = dist.get_world_size(sync_group)
        else:
            self.world_rank, self.world_size = 0, 1
        self.module_partitions = module_partitions
        self.partitioned_modules = []
        if module_partitions is not None:
            if len(module_partitions) != self.world_size:
                raise ValueError(f'Number of partitions has to be world_size. Got {len(module_partitions)}')
            self.partitioned_modules = [m for part in module_partitions for m in part]
        self.partitions = self.get_distr_prec_partition()
        self._owner = {}
        for i, shape in enumerate(_module_level_shapes):
            for j, module in enumerate(self.modules_for(shape)):
                self._owner[module] = self.partitions[i][j]

        self.curvature_sync_handles = []
        self.grad_sync_handles = []
        self.grads = []
        self.packed_grads = []

    # ------------------------------------------------------------------ module bookkeeping
    def named_modules_for(self, shape):
        if shape not in self._named_modules_for:
            self._named_modules_for[shape] = list(modules_to_assign(
                self.model, shape, *self.fisher_shape, ignore_modules=self.config.ignore_modules,
                named=True))
        return self._named_modules_for[shape]

    def modules_for(self, shape):
        return [m for _, m in self.named_modules_for(shape)]

    def parameters_for(self, shape):
        for module in self.modules_for(shape):
            for p in module.parameters():
                if p.requires_grad:
                    yield p

    def get_distr_prec_partition(self):
        """Owner rank of every module, as ``partitions[shape_index][module_index]`` with shapes in
        the order layer_wise, kron, swift_kron, kfe, unit_wise, diag."""
        from ..parallel.partition import assign_owners, curvature_cost
        entries = []
        for i, shape in enumerate(_module_level_shapes):
            for j, module in enumerate(self.modules_for(shape)):
                entries.append((i, j, module, curvature_cost(module, shape)))
        fixed = {}
        if self.module_partitions is not None:
            for rank, part in enumerate(self.module_partitions):
                for module in part:
                    fixed[module] = rank
        owners = assign_owners([e[3] for e in entries], self.world_size,
                               fixed=[fixed.get(e[2]) for e in entries])
        partitions = [[0] * len(self.modules_for(s)) for s in _module_level_shapes]
        for (i, j, _, _), owner in zip(entries, owners):
            partitions[i][j] = owner
        return partitions

    def is_module_for_inv_and_precondition(self, module: nn.Module):
        """Whether this rank inverts / preconditions ``module``."""
        if module not in self.shape_for:
            return False
        return self._owner.get(module, 0) == self.world_rank

    # ------------------------------------------------------------------ fisher storage
    @property
    def _fisher_attr(self):
        return self.fisher_maker.config.fisher_attr

    def _get_module_fisher(self, module, postfix=None):
        attr = self._fisher_attr if postfix is None else f'{self._fisher_attr}_{postfix}'
        return getattr(module, attr, None)

    def _set_module_fisher(self, module, fisher, postfix=None):
        attr = self._fisher_attr if postfix is None else f'{self._fisher_attr}_{postfix}'
        setattr(module, attr, fisher)

    def _get_full_fisher(self):
        return self._get_module_fisher(self.model)

    def _get_module_symmatrix(self, module, shape, postfix=None):
        fisher = self._get_module_fisher(module, postfix)
        if fisher is None:
            return None
        if shape in (SHAPE_FULL, SHAPE_LAYER_WISE):
            return fisher
        if shape in (SHAPE_KRON, SHAPE_SWIFT_KRON):
            return fisher.kron
        if shape == SHAPE_KFE:
            return fisher.kfe
        if shape == SHAPE_UNIT_WISE:
            return fisher.unit
        if shape == SHAPE_DIAG:
            return fisher.diag
        raise ValueError(f'Invalid shape: {shape}.')

    @staticmethod
    def _keys_list_from_shape(shape, kron=None, diag=None):
        if shape in (SHAPE_FULL, SHAPE_LAYER_WISE):
            return [['data']]
        if shape in (SHAPE_KRON, SHAPE_SWIFT_KRON):
            kron = ['A', 'B'] if kron is None else kron
            if any(k not in ('A', 'B') for k in kron):
                raise ValueError(f'kron has to be a list of "A" or "B". Got {kron}')
            return [['kron', k] for k in kron]
        if shape == SHAPE_UNIT_WISE:
            return [['unit', 'data']]
        if shape == SHAPE_DIAG:
            diag = ['weight', 'bias'] if diag is None else diag
            if any(k not in ('weight', 'bias') for k in diag):
                raise ValueError(f'diag has to be a list of "weight" or "bias". Got {diag}')
            return [['diag', k] for k in diag]
        if shape == SHAPE_KFE:
            return []
        raise ValueError(f'Invalid shape: {shape}.')

    def _curvature_tensors(self, module, shape):
        out = []
        for keys in self._keys_list_from_shape(shape):
            t = self.fisher_maker.get_fisher_tensor(module, *keys)
            if t is not None:
                out.append(t)
        if shape == SHAPE_KFE:
            kfe = self._get_module_symmatrix(module, shape)
            if kfe is not None and kfe.has_scale:
                out.extend(kfe.scale)
        return out

    def get_fisher_from_model(self):
        """All curvature tensors currently stored on the modules (module-level shapes)."""
        tensors = []
        for shape in _module_level_shapes:
            for module in self.modules_for(shape):
                tensors.extend(self._curvature_tensors(module, shape))
        return tensors

    def _scale_fisher(self, scale):
        for shape in _module_level_shapes:
            for module in self.modules_for(shape):
                matrix = self._get_module_symmatrix(module, shape)
                if matrix is not None:
                    matrix.mul_(scale)
        fisher = self._get_full_fisher()
        if fisher is not None and fisher.has_data:
            fisher.data.mul_(scale)

    # ------------------------------------------------------------------ schedule hooks
    @property
    def do_accumulate(self):
        return self.config.ema_decay != _invalid_ema_decay

    @property
    def _owner_inverts(self):
        """Inverses are taken in ``update_preconditioner`` (not inside the hooks) when the
        curvature is accumulated or has to be averaged over ranks first."""
        return self.do_accumulate or self.world_size > 1

    def do_forward_and_backward(self, step=None):
        return not self.do_update_curvature(step)

    def do_update_preconditioner(self, step=None) -> bool:
        has_curvature_rule = (self.curvature_upd_schedule is not None
                              or self.config.curvature_upd_interval is not None)
        if not self.do_accumulate and self.world_size > 1 and has_curvature_rule:
            return self.do_update_curvature(step)  # nothing is kept, so invert whenever measured
        return super().do_update_preconditioner(step)

    # ------------------------------------------------------------------ the three phases
    def update_curvature(self):
        config = self.config
        scale = self.scale
        distributed = self.world_size > 1
        if self.do_accumulate:
            scale = scale * config.ema_decay
        stored = None
        if distributed:
            # measure the new statistics on their own, average them onto the owners, and let the
            # owners fold them into their running curvature
            stored = self._detach_fisher()
        elif self.do_accumulate:
            self._scale_fisher(1 - config.ema_decay)
        self.delegate_forward_and_backward(self.fisher_maker,
                                           data_size=config.data_size,
                                           scale=scale,
                                           accumulate=self.do_accumulate and not distributed,
                                           calc_loss_grad=True,
                                           calc_inv=not self._owner_inverts,
                                           damping=config.damping)
        if distributed:
            self.reduce_scatter_curvature()
            self._merge_fisher(stored)

    def _fisher_holders(self):
        holders = list(self.modules_for_curvature)
        if any(True for _ in self.parameters_for(SHAPE_FULL)) and self.model not in holders:
            holders.append(self.model)
        return holders

    def _detach_fisher(self):
        """Remove the running curvature from the modules (returned as {module: SymMatrix})."""
        stored = {}
        for module in self._fisher_holders():
            fisher = self._get_module_fisher(module)
            if fisher is not None:
                stored[module] = fisher
                delattr(module, self._fisher_attr)
        return stored

    def _merge_fisher(self, stored):
        """Owners: running <- (1 - ema_decay) * running + averaged new statistics (or just the new
        statistics without EMA).  Other ranks keep no curvature for the layer."""
        decay = 1 - self.config.ema_decay if self.do_accumulate else 0.0
        for module in self._fisher_holders():
            new = self._get_module_fisher(module)
            owns = module is self.model or self.is_module_for_inv_and_precondition(module)
            if not owns:
                if new is not None:
                    delattr(module, self._fisher_attr)
                continue
            old = stored.get(module)
            if old is None or decay == 0.0 or new is None:
                continue
            old.mul_(decay)
            old += new  # in place: the stored inverses stay attached
            self._set_module_fisher(module, old)

    def update_preconditioner(self, damping=None, module_name=None, kron=None, zero_curvature=False,
                              partition_aware=False):
        """Invert the stored curvature of the layers this rank owns (``module_name`` / ``kron``
        restrict the update to one module / one Kronecker factor)."""
        if not self._owner_inverts:
            return
        kron = ['A', 'B'] if kron is None else kron
        damping = self.config.damping if damping is None else damping
        for shape in _module_level_shapes:
            for name, module in self.named_modules_for(shape):
                if module_name is not None and name != module_name:
                    continue
                if not self.is_module_for_inv_and_precondition(module):
                    continue
                matrix = self._get_module_symmatrix(module, shape)
                if matrix is None:
                    continue
                is_kron = shape in (SHAPE_KRON, SHAPE_SWIFT_KRON)
                tag = f'inv_{shape}' + (''.join(f'_{k}' for k in kron) if is_kron else '') + f'_{name}'
                with nvtx_range(tag):
                    if is_kron:
                        matrix.update_inv(damping, calc_A_inv='A' in kron, calc_B_inv='B' in kron)
                    else:
                        matrix.update_inv(damping)
                    if zero_curvature:
                        with torch.no_grad():
                            if is_kron:
                                for k in kron:
                                    getattr(matrix, k).mul_(0)
                            else:
                                matrix.mul_(0)
        fisher = self._get_full_fisher()
        if fisher is not None and fisher.has_data and module_name is None:
            fisher.update_inv(damping)
            if zero_curvature:
                with torch.no_grad():
                    fisher.data.mul_(0)

    def precondition(self, vectors: ParamVector = None, grad_scale=None, use_inv=True):
        """``grad <- F^-1 grad`` in place (or on ``vectors``).  In data-parallel runs gradients
        are averaged first and the owners' results are distributed afterwards."""
        grad_scale = self.grad_scale if grad_scale is None else grad_scale
        distributed = self.world_size > 1 and vectors is None
        if distributed:
            self.sync_grad_pre_precondition()
        for shape in _module_level_shapes:
            for module in self.modules_for(shape):
                if self.is_module_for_inv_and_precondition(module):
                    self._precondition_module(module, shape, vectors, grad_scale=grad_scale,
                                              use_inv=use_inv)
        params = list(self.parameters_for(SHAPE_FULL))
        if params:
            fisher = self._get_full_fisher()
            if fisher is None:
                raise ValueError(f'Fisher of shape {SHAPE_FULL} has not been calculated.')
            if vectors is None:
                vectors_full = ParamVector(params, [p.grad for p in params])
            else:
                vectors_full = vectors
            if grad_scale != 1:
                vectors_full.mul_(grad_scale)
            fisher.mvp(vectors=vectors_full, use_inv=use_inv, inplace=True)
        if distributed:
            self.sync_grad_post_precondition()

    def precondition_module(self, module, vec_weight=None, vec_bias=None, use_inv=True):
        """Precondition explicit weight/bias-shaped tensors with ``module``'s curvature (used by
        the kernel utilities for per-example gradients)."""
        weight = getattr(module, 'weight', None)
        if vec_weight is not None and weight is not None and vec_weight.ndim == weight.ndim + 1:
            for i in range(vec_weight.shape[0]):   # a batch of per-example gradients: one at a time, in place
                self._precondition_module(module, vec_weight=vec_weight[i],
                                          vec_bias=None if vec_bias is None else vec_bias[i], grad_scale=1,
                                          use_inv=use_inv)
            return
        self._precondition_module(module, vec_weight=vec_weight, vec_bias=vec_bias, grad_scale=1,
                                  use_inv=use_inv)

    def precondition_vector(self, vectors, use_inv=True):
        """``F^-1`` applied in place to a list of tensors aligned with ``model.parameters()`` (used by the
        kernel utilities between two Jacobians).  Runs on plain PyTorch operations, so the result stays
        differentiable with respect to what the tensors were computed from."""
        from .. import ops
        vectors = list(vectors)
        params = list(self.model.parameters())
        if len(vectors) != len(params):
            raise ValueError(f'{len(params)} tensors are expected, one per parameter. Got {len(vectors)}.')
        backend = ops.get_backend()
        ops.set_backend('torch')
        try:
            self.precondition(vectors=ParamVector(params, vectors), grad_scale=1, use_inv=use_inv)
        finally:
            ops.set_backend(backend)
        return vectors

    def _precondition_module(self, module, shape=None, vectors: ParamVector = None,
                             vec_weight: torch.Tensor = None, vec_bias: torch.Tensor = None,
                             grad_scale=None, use_inv=True):
        grad_scale = self.grad_scale if grad_scale is None else grad_scale
        if shape is None:
            shape = self.shape_for.get(module)
        if shape is None:
            raise ValueError(f'No shape is assigned to module: {module}.')
        if vectors is not None:
            vec_weight = vectors.get_vector_by_param(getattr(module, 'weight', None), None)
            vec_bias = vectors.get_vector_by_param(getattr(module, 'bias', None), None)
        matrix = self._get_module_symmatrix(module, shape)
        if matrix is None:
            raise ValueError(f'Matrix of shape {shape} for module {module} has not been calculated.')
        weight = getattr(module, 'weight', None)
        if vec_weight is None and weight is not None and weight.requires_grad:
            vec_weight = weight.grad
        if vec_weight is None and shape not in (SHAPE_DIAG, SHAPE_LAYER_WISE):
            raise ValueError(f'weight gradient for module {module} has not been calculated.')
        if _bias_requires_grad(module) and vec_bias is None:
            vec_bias = module.bias.grad
            if vec_bias is None:
                raise ValueError(f'bias gradient for module {module} has not been calculated.')
        if grad_scale != 1:
            for v in (vec_weight, vec_bias):
                if v is not None:
                    v.data.mul_(grad_scale)
        if shape == SHAPE_KFE:
            matrix.mvp(vec_weight=vec_weight, vec_bias=vec_bias, inplace=True, eps=self.config.damping)
        elif not use_inv or matrix.has_inv:
            matrix.mvp(vec_weight=vec_weight, vec_bias=vec_bias, use_inv=use_inv, inplace=True)

    # ------------------------------------------------------------------ collectives
    def _owner_groups(self):
        """{owner rank: [(module, shape), ...]} in a deterministic order shared by all ranks."""
        groups: Dict[int, list] = {r: [] for r in range(self.world_size)}
        for shape in _module_level_shapes:
            for module in self.modules_for(shape):
                groups[self._owner.get(module, 0)].append((module, shape))
        return groups

    def _global_rank(self, rank_in_group):
        if self.sync_group_ranks is not None:
            return self.sync_group_ranks[rank_in_group]
        return rank_in_group

    def _reduce_avg(self, tensors, dst=None):
        """Average ``tensors`` over ranks onto ``dst`` (or onto everyone) with one message."""
        if not tensors:
            return
        flat = _pack(tensors)
        if dst is None:
            dist.all_reduce(flat, group=self.sync_group)
        else:
            dist.reduce(flat, self._global_rank(dst), group=self.sync_group)
        if dst is None or dst == self.world_rank:
            _unpack(flat.div_(self.world_size), tensors)

    @staticmethod
    def _module_grads(module):
        return [p.grad for p in module.parameters() if p.requires_grad and p.grad is not None]

    def reduce_scatter_curvature(self, kron=None, diag=None, with_grad=True):
        """Average the freshly measured statistics (and, by default, the gradients) of every layer
        onto its owner: one packed message per owner rank."""
        assert kron is None and diag is None
        with nvtx_range('reduce_scatter_curvature'):
            for owner, members in self._owner_groups().items():
                tensors = []
                for module, shape in members:
                    tensors.extend(self._curvature_tensors(module, shape))
                    if with_grad:
                        tensors.extend(self._module_grads(module))
                self._reduce_avg(tensors, dst=owner)
            fisher = self._get_full_fisher()
            if fisher is not None and fisher.has_data:
                self._reduce_avg([fisher.data])
        if with_grad:
            self._owned_grads_synced = True

    def sync_curvature(self, module_name=None, kron=None, diag=None, with_grad=False, enabled=True,
                       async_op=False):
        """Average curvature tensors onto their owners (optionally one module / one factor)."""
        if not enabled or self.world_size == 1:
            return
        for owner, members in self._owner_groups().items():
            tensors = []
            for module, shape in members:
                if module_name is not None and self._name_of(module) != module_name:
                    continue
                for keys in self._keys_list_from_shape(shape, kron=kron, diag=diag):
                    t = self.fisher_maker.get_fisher_tensor(module, *keys)
                    if t is not None:
                        tensors.append(t)
                if with_grad:
                    tensors.extend(self._module_grads(module))
            self._reduce_avg(tensors, dst=owner)

    def _name_of(self, module):
        for name, m in self.named_modules_for_curvature:
            if m is module:
                return name
        return None

    def sync_grad_pre_precondition(self, enabled=True, async_op=False):
        """Make the averaged gradient available where it is needed: owners get the average of
        their layers (skipped when the curvature reduction already carried it)."""
        if not enabled or self.world_size == 1:
            return
        if getattr(self, '_owned_grads_synced', False):
            self._owned_grads_synced = False
            return
        with nvtx_range('reduce_scatter_grad'):
            for owner, members in self._owner_groups().items():
                tensors = []
                for module, _ in members:
                    tensors.extend(self._module_grads(module))
                self._reduce_avg(tensors, dst=owner)

    def sync_grad_post_precondition(self, enabled=True, async_op=False):
        if not enabled or self.world_size == 1:
            return
        self.all_gather_or_reduce_grad()

    def all_gather_or_reduce_grad(self):
        """Owners broadcast their preconditioned gradients; every other trainable parameter of the
        model gets the plain average."""
        with nvtx_range('all_gather_grad'):
            covered = set()
            for owner, members in self._owner_groups().items():
                tensors = []
                for module, _ in members:
                    grads = self._module_grads(module)
                    tensors.extend(grads)
                    covered.update(id(g) for g in grads)
                if not tensors:
                    continue
                flat = _pack(tensors)
                dist.broadcast(flat, self._global_rank(owner), group=self.sync_group)
                if owner != self.world_rank:
                    _unpack(flat, tensors)
            full_params = {id(p) for p in self.parameters_for(SHAPE_FULL)}
            rest = [p.grad for p in self.model.parameters()
                    if p.requires_grad and p.grad is not None and id(p.grad) not in covered
                    and id(p) not in full_params]
            self._reduce_avg(rest)

    def all_reduce_all_grad(self, async_op=False):
        """Average every gradient of the model over ranks."""
        with nvtx_range('all_reduce_all_grad'):
            self._reduce_avg([p.grad for p in self.model.parameters() if p.grad is not None])

    # -- members of the reference's explicit-partition interface (asdl/precondition/natural_gradient.py:288-320,
    #    587-700, 802-811), kept so that code written against them keeps running --------------------------
    def computational_cost(self, shape, module):
        """Cost that the owner assignment attributes to ``module`` with curvature ``shape`` (inverse and
        preconditioning, cubic in the factor sizes); 0 for modules this rank does not own."""
        from ..parallel.partition import curvature_cost
        return curvature_cost(module, shape) if self.is_module_for_inv_and_precondition(module) else 0

    @staticmethod
    def next_split(subset_partitions):
        """Index at which a list of costs is cut into two parts of nearly equal sums (the first part is
        the shortest prefix reaching half of the total, and never the whole list)."""
        if len(subset_partitions) < 2:
            raise ValueError('at least two costs are needed for a split.')
        half, running = sum(subset_partitions) / 2, 0.0
        for index, cost in enumerate(subset_partitions):
            running += cost
            if running >= half:
                return min(index + 1, len(subset_partitions) - 1)
        return len(subset_partitions) - 1

    def _distinct_keys(self, kron=None, diag=None):
        """Key paths of every module-level shape, each once (kron and swift_kron share theirs)."""
        out = []
        for shape in _module_level_shapes:
            for keys in self._keys_list_from_shape(shape, kron=kron, diag=diag):
                if keys not in out:
                    out.append(keys)
        return out

    def _modules_outside_partitions(self, module_name=None):
        return [m for name, m in self.named_modules_for_curvature
                if m not in self.partitioned_modules and (module_name is None or name == module_name)]

    def reduce_scatter_curvature_module_partitions(self, kron=None, diag=None, with_grad=False):
        """Sum the curvature of ``module_partitions[r]`` onto rank r (explicit partitions only)."""
        if self.module_partitions is None:
            raise ValueError('module_partitions is not set.')
        handles = []
        for keys in self._distinct_keys(kron, diag):
            handles += self.fisher_maker.reduce_scatter_fisher(self.module_partitions, *keys, with_grad=with_grad,
                                                               group=self.sync_group, async_op=True)
        self.curvature_sync_handles += [h for h in handles if h is not None]
        return handles

    def reduce_curvature(self, module_name, kron=None, diag=None, with_grad=False):
        """Sum the curvature of the named module onto the rank whose explicit partition holds it."""
        if self.module_partitions is None:
            raise ValueError('module_partitions is not set.')
        module = dict(self.named_modules_for_curvature).get(module_name)
        if module is None or module not in self.partitioned_modules:
            return []
        dst = next(i for i, part in enumerate(self.module_partitions) if module in part)
        if self.sync_group is not None and self.sync_group_ranks is not None:
            dst = self.sync_group_ranks[dst]
        handles = []
        for keys in self._keys_list_from_shape(self.shape_for[module], kron=kron, diag=diag):
            handles += self.fisher_maker.reduce_fisher([module], *keys, all_reduce=False, dst=dst, with_grad=with_grad,
                                                       group=self.sync_group, async_op=True)
        self.curvature_sync_handles += [h for h in handles if h is not None]
        return handles

    def all_reduce_undivided_curvature(self, module_name=None, kron=None, diag=None, with_grad=False):
        """Sum over ranks the curvature of the modules that no explicit partition holds."""
        modules = self._modules_outside_partitions(module_name)
        handles = []
        for keys in self._distinct_keys(kron, diag):
            handles += self.fisher_maker.reduce_fisher(modules, *keys, all_reduce=True, with_grad=with_grad,
                                                       group=self.sync_group, async_op=True)
        self.curvature_sync_handles += [h for h in handles if h is not None]
        return handles

    def _all_reduce_sum(self, grads):
        grads = [g for g in grads if g is not None]
        if not grads or not dist.is_initialized():
            return
        packed = torch.cat([g.reshape(-1) for g in grads])
        dist.all_reduce(packed, group=self.sync_group)
        offset = 0
        for g in grads:
            g.copy_(packed[offset:offset + g.numel()].view_as(g))
            offset += g.numel()

    def all_reduce_undivided_grad(self, async_op=False):
        """Sum over ranks the gradients of the curvature modules that no explicit partition holds."""
        if not dist.is_initialized():
            raise EnvironmentError('torch.distributed is not initialized.')
        self._all_reduce_sum([p.grad for m in self._modules_outside_partitions() for p in m.parameters()])

    def all_reduce_no_curvature_grad(self, async_op=False):
        """Sum over ranks the gradients of the leaf modules without curvature."""
        with_curvature = set(self.modules_for_curvature)
        self._all_reduce_sum([p.grad for m in self.model.modules()
                              if len(list(m.children())) == 0 and m not in with_curvature for p in m.parameters()])

    def reduce_scatter_grad(self, async_op=False):
        self._owned_grads_synced = False
        self.sync_grad_pre_precondition()

    def all_gather_grad(self, async_op=False):
        self.all_gather_or_reduce_grad()

    def wait_all_curvature_sync(self):
        while self.curvature_sync_handles:
            self.curvature_sync_handles.pop(0).wait()

    def wait_all_grad_sync(self):
        while self.grad_sync_handles:
            self.grad_sync_handles.pop(0).wait()

    # ------------------------------------------------------------------ checkpointing
    def _curvature_state(self):
        out = {}
        for name, module in self.named_modules_for_curvature:
            fisher = self._get_module_fisher(module)
            if fisher is not None:
                out.update(fisher.tensors(prefix=f'{name}.'))
        fisher = self._get_full_fisher()
        if fisher is not None and SHAPE_FULL in [s for s in self.fisher_shape if isinstance(s, str)]:
            out.update(fisher.tensors(prefix='__model__.'))
        return out

    def _load_curvature_state(self, tensors):
        grouped: Dict[str, Dict[str, torch.Tensor]] = {}
        for key, value in tensors.items():
            name, rest = key.split('.', 1)
            grouped.setdefault(name, {})[rest] = value
        by_name = dict(self.named_modules_for_curvature)
        for name, items in grouped.items():
            module = self.model if name == '__model__' else by_name.get(name)
            if module is None:
                continue
            device = next(module.parameters()).device
            items = {k: v.to(device) for k, v in items.items()}
            if name != '__model__':
                _check_state_shapes(name, module, items)
            self._set_module_fisher(module, SymMatrix.from_tensors(items))


def _check_state_shapes(name, module, items):
    """A checkpoint written for another architecture fails at load time, with the offending key,
    instead of at the first preconditioning product."""
    weight = getattr(module, 'weight', None)
    if weight is None:
        return

    def fail(key, why):
        raise ValueError(f'curvature checkpoint entry {name}.{key} of shape {tuple(items[key].shape)} does not fit '
                         f'{module.__class__.__name__} with weight {tuple(weight.shape)}: {why}')

    sides = {}
    for key, value in items.items():
        if key in ('kron.A', 'kron.A_inv', 'kron.B', 'kron.B_inv'):
            if value.ndim == 2 and value.shape[0] != value.shape[1]:
                fail(key, 'a Kronecker factor is square')
            side = key[5]
            if sides.setdefault(side, value.shape[0]) != value.shape[0]:
                fail(key, 'factor and inverse differ in size')
        elif key in ('diag.weight', 'diag.weight_inv') and value.shape != weight.shape:
            fail(key, 'the diagonal has the shape of the weight')
    if 'B' in sides and sides['B'] != weight.shape[0] and not isinstance(module, nn.Embedding):
        fail('kron.B' if 'kron.B' in items else 'kron.B_inv', 'the output-side factor has one row per output feature')
    if 'A' in sides and 'B' in sides and not isinstance(module, nn.Embedding) \
            and sides['A'] * sides['B'] != weight.numel():
        fail('kron.A' if 'kron.A' in items else 'kron.A_inv', 'the factor sizes do not multiply to the weight size')


class FullNaturalGradientMaker(NaturalGradientMaker):
    """Natural gradient with one dense Fisher matrix over all parameters."""
    def __init__(self, model, config: PreconditioningConfig, *args, **kwargs):
        super().__init__(model, config, *args, **kwargs, fisher_shape=SHAPE_FULL)


class LayerWiseNaturalGradientMaker(NaturalGradientMaker):
    """Natural gradient with one dense Fisher block per layer."""
    def __init__(self, model, config: PreconditioningConfig, *args, **kwargs):
        super().__init__(model, config, *args, **kwargs, fisher_shape=SHAPE_LAYER_WISE)


class KfacGradientMaker(NaturalGradientMaker):
    """K-FAC: Kronecker-factored Fisher for Linear / Conv2d / Embedding layers and unit-wise 2x2
    blocks for normalisation layers.  ``swift=True`` selects SKFAC (factors with fewer samples
    than dimensions are inverted by Woodbury)."""

    def __init__(self, model, config: PreconditioningConfig,
                 fisher_type: str = FISHER_MC, loss_type: str = LOSS_CROSS_ENTROPY,
                 scale: float = 1, grad_scale: float = 1,
                 n_mc_samples: int = 1, var: float = 1., seed: int = None, swift=False, **kwargs):
        fisher_shape = [SHAPE_SWIFT_KRON if swift else SHAPE_KRON,
                        (nn.BatchNorm1d, SHAPE_UNIT_WISE),
                        (nn.BatchNorm2d, SHAPE_UNIT_WISE),
                        (nn.LayerNorm, SHAPE_UNIT_WISE)]
        super().__init__(model, config, fisher_type=fisher_type, fisher_shape=fisher_shape,
                         loss_type=loss_type, scale=scale, grad_scale=grad_scale,
                         n_mc_samples=n_mc_samples, var=var, seed=seed, **kwargs)


class EkfacGradientMaker(NaturalGradientMaker):
    """EKFAC: the gradient is rescaled in the Kronecker-factored eigenbasis by second moments
    measured in that basis.  Empirical Fisher only."""

    def __init__(self, model, config: PreconditioningConfig, *args, **kwargs):
        if not args:
            kwargs.setdefault('fisher_type', FISHER_EMP)
        # normalisation layers have no Kronecker eigenbasis: unit-wise blocks as in K-FAC
        fisher_shape = [SHAPE_KFE, (nn.BatchNorm1d, SHAPE_UNIT_WISE), (nn.BatchNorm2d, SHAPE_UNIT_WISE),
                        (nn.LayerNorm, SHAPE_UNIT_WISE)]
        super().__init__(model, config, *args, **kwargs, fisher_shape=fisher_shape)
        if self.fisher_type != FISHER_EMP:
            raise ValueError(f'{EkfacGradientMaker} supports only {FISHER_EMP}.')


class UnitWiseNaturalGradientMaker(NaturalGradientMaker):
    """Natural gradient with one small Fisher block per output unit (2 x 2 per feature for normalisation layers)."""
    def __init__(self, model, config: PreconditioningConfig, *args, **kwargs):
        super().__init__(model, config, *args, **kwargs, fisher_shape=SHAPE_UNIT_WISE)


class DiagNaturalGradientMaker(NaturalGradientMaker):
    """Natural gradient with the diagonal of the Fisher matrix."""
    def __init__(self, model, config: PreconditioningConfig, *args, **kwargs):
        super().__init__(model, config, *args, **kwargs, fisher_shape=SHAPE_DIAG)


class EmpNaturalGradientMaker(NaturalGradientMaker):
    """Natural gradient with the empirical Fisher (gradients of the observed labels) in the given shape."""
    def __init__(self, model, config: PreconditioningConfig, *args, **kwargs):
        super().__init__(model, config, *args, **kwargs, fisher_type=FISHER_EMP)
