"""Fisher information matrices (exact / Monte-Carlo / empirical, for cross-entropy or MSE) in any
of the supported shapes, their inverses, Fisher-vector products and spectral tools.

Parity: asdl/fisher.py (``FisherConfig`` :29-45, ``FisherMaker`` :48-416, variants :419-497,
``get_fisher_maker`` :500-521).  Semantics kept: losses are forced to ``reduction='sum'`` and
gradients / loss are divided by ``data_size`` afterwards; ``scale / data_size`` multiplies *each*
Kronecker factor; results are stored on the modules as ``module.fisher`` (``SymMatrix``) and
``module.fvp`` (``ParamVector``).

Exact cross-entropy Fisher is evaluated with one backward pass per class with ``sqrt(p_c)``
weighting; the Monte-Carlo estimate samples labels from the model.  Backward passes that only
serve the curvature run with every ``param.grad`` frozen (see ``skip_param_grad``).
"""
from dataclasses import dataclass
from typing import Any, List, Tuple, Union

import numpy as np
import torch
from torch import Tensor
import torch.nn as nn
import torch.nn.functional as F
import torch.distributed as dist

from .core import no_centered_cov
from .operations import OperationContext
from .utils import skip_param_grad
from .grad_maker import GradientMaker, LOSS_CROSS_ENTROPY, LOSS_MSE
from .matrices import *  # noqa: F401,F403
from .matrices import FISHER_EXACT, FISHER_MC, FISHER_EMP, SHAPE_FULL
from .vector import ParamVector, reduce_vectors
from .mvp import power_method, stochastic_lanczos_quadrature, conjugate_gradient_method, quadratic_form
from .symmatrix import SymMatrix

__all__ = ['FisherConfig', 'get_fisher_maker']

_supported_types = [FISHER_EXACT, FISHER_MC, FISHER_EMP]
_invalid_data_size = -1


@dataclass
class FisherConfig:
    fisher_type: str
    fisher_shapes: List[Any]
    loss_type: str = None
    n_mc_samples: int = 1
    var: float = 1.
    seed: int = None
    fisher_attr: str = 'fisher'
    fvp_attr: str = 'fvp'
    ignore_modules: List[Any] = None
    data_size: int = _invalid_data_size
    scale: float = 1.
    is_distributed: bool = False
    all_reduce: bool = False
    is_master: bool = True
    ignore_index: int = -1


class FisherMaker(GradientMaker):
    _loss_reduction = 'sum'

    def __init__(self, model, config):
        super().__init__(model)
        self.config: FisherConfig = config

    def zero_fisher(self, fvp=False):
        attr = self.config.fvp_attr if fvp else self.config.fisher_attr
        for module in self.model.modules():
            if hasattr(module, attr):
                delattr(module, attr)

    @property
    def is_fisher_emp(self):
        return False

    @property
    def do_local_accumulate(self) -> bool:
        """True when the Fisher needs several backward passes, so that an inverse can only be
        taken after all of them have been accumulated."""
        raise NotImplementedError

    def forward_and_backward(self, data_size=_invalid_data_size, scale=None, accumulate=False,
                             calc_loss_grad=False, calc_inv=False, fvp=False, damping=None,
                             vec: ParamVector = None) -> Union[Tuple[Any, Tensor], Any]:
        """Computes the Fisher (or its inverse, or Fisher-vector products) of the registered
        model/loss and stores it on the modules.

        data_size: mandatory (here or in the config); everything is scaled by ``1/data_size``.
        scale: extra factor (the EMA weight is passed here by the K-FAC maker).
        accumulate: add to the existing ``module.fisher`` instead of replacing it.
        calc_loss_grad: also leave the gradient of the true loss in ``param.grad`` (divided by
            ``data_size``) and return the loss.
        calc_inv: store damped inverses instead of the matrices.
        fvp / vec: compute ``F @ vec`` into ``module.fvp`` instead of matrices.
        """
        if accumulate and calc_inv:
            raise ValueError('accumulate and calc_inv cannot be True at the same time.')
        if fvp and calc_inv:
            raise ValueError('fvp and calc_inv cannot be True at the same time.')
        model, config = self.model, self.config
        shapes = config.fisher_shapes
        if isinstance(shapes, str):
            shapes = [shapes]
        if data_size == _invalid_data_size:
            data_size = config.data_size
        if data_size == _invalid_data_size:
            raise ValueError('data_size is not specified.')
        scale = (config.scale if scale is None else scale) / data_size
        if not accumulate:
            self.zero_fisher(fvp=fvp)
        if config.seed is not None:
            torch.random.manual_seed(config.seed)

        grad_with_fisher = calc_loss_grad and self.is_fisher_emp
        grad_after_fisher = calc_loss_grad and not self.is_fisher_emp
        inv_in_hooks = calc_inv and not self.do_local_accumulate
        inv_after = calc_inv and not inv_in_hooks

        with no_centered_cov(model, shapes, ignore_modules=config.ignore_modules, cvp=fvp,
                             vectors=vec, calc_inv=inv_in_hooks) as cxt:
            if accumulate:
                self._register_fisher(cxt)
            if damping is not None:
                cxt.set_damping(damping)
            cxt.set_cov_scale(scale)

            self.call_model()
            loss = None
            if self.is_fisher_emp or calc_loss_grad:
                loss = self.call_loss()

            def closure(nll_expr, retain_graph=False):
                cxt.clear_batch_grads()
                with skip_param_grad(model, disable=grad_with_fisher):
                    nll_expr().backward(retain_graph=retain_graph or grad_after_fisher)
                if fvp:
                    cxt.calc_full_cvp(model, scale=scale)
                else:
                    cxt.calc_full_cov(model, scale=scale, calc_inv=inv_in_hooks, damping=damping)

            if self.is_fisher_emp:
                closure(lambda: loss)
            else:
                self._fisher_loop(closure)
            self._extract_fisher(cxt)

        if inv_after:
            self.replace_fisher_with_inv(damping)
        if grad_after_fisher:
            loss.backward()
        if calc_loss_grad:
            for p in model.parameters():
                if p.grad is not None:
                    p.grad.div_(data_size)
            with torch.no_grad():
                loss.div_(data_size)
        self._loss = loss
        return self._model_output, loss

    def _register_fisher(self, cxt: OperationContext):
        attr = self.config.fisher_attr
        for module in self.model.modules():
            fisher = getattr(module, attr, None)
            if fisher is None:
                continue
            if cxt.is_operation_registered(module) and module is not self.model:
                cxt.register_symmatrix(module, fisher)
        fisher = getattr(self.model, attr, None)
        if fisher is not None and fisher.has_data:
            cxt.register_full_symmatrix(self.model, fisher)

    def _extract_fisher(self, cxt: OperationContext):
        """Move results from the context to ``module.<fisher_attr>`` / ``module.<fvp_attr>``
        (only where nothing is stored yet: accumulated results were added in place)."""
        model = self.model
        fisher_attr, fvp_attr = self.config.fisher_attr, self.config.fvp_attr

        def extract(module, getter, attr):
            if getattr(module, attr, None) is None:
                value = getter(module, pop=True)
                if value is not None:
                    setattr(module, attr, value)

        def adopt_promoted_factors(module):
            # a wide swift factor that received a second contribution was replaced by the square matrix it
            # stands for (it cannot be updated in place): hand the new tensor to the stored Kron
            stored = getattr(module, fisher_attr, None)
            if stored is None or not stored.has_kron or not cxt.is_operation_registered(module):
                return
            results = cxt.cov_kron(module) or {}
            for key in ('A', 'B'):
                value = results.get(key)
                if value is not None and value is not getattr(stored.kron, key):
                    setattr(stored.kron, key, value)

        for module in model.modules():
            adopt_promoted_factors(module)
            extract(module, cxt.cov_symmatrix, fisher_attr)
            extract(module, cxt.cvp_paramvector, fvp_attr)
        extract(model, cxt.full_cov_symmatrix, fisher_attr)
        extract(model, cxt.full_cvp_paramvector, fvp_attr)

    def replace_fisher_with_inv(self, damping):
        attr = self.config.fisher_attr
        kwargs = {} if damping is None else {'damping': damping}
        seen = set()
        for module in list(self.model.modules()) + [self.model]:
            fisher: SymMatrix = getattr(module, attr, None)
            if fisher is not None and id(fisher) not in seen:
                seen.add(id(fisher))
                fisher.update_inv(replace=True, **kwargs)

    def _fisher_loop(self, closure):
        raise NotImplementedError

    def get_fisher_tensor(self, module: nn.Module, *keys) -> Union[torch.Tensor, None]:
        """``get_fisher_tensor(m, 'kron', 'A')`` -> ``m.fisher.kron.A`` (None if absent)."""
        data = getattr(module, self.config.fisher_attr, None)
        for key in keys:
            if data is None:
                return None
            data = getattr(data, key, None)
        if data is not None and not isinstance(data, torch.Tensor):
            raise TypeError(f'data have to be {torch.Tensor}, got {type(data)}.')
        return data

    # ------------------------------------------------------------------ collectives
    def _tensors_for(self, modules, keys, with_grad):
        out = []
        for module in modules:
            tensor = self.get_fisher_tensor(module, *keys)
            if tensor is None:
                continue
            out.append(tensor)
            if with_grad:
                out.extend(p.grad for p in module.parameters() if p.requires_grad and p.grad is not None)
        return out

    def reduce_scatter_fisher(self, module_partitions: List[List[torch.nn.Module]], *keys,
                              with_grad=False, group: dist.ProcessGroup = None, async_op=False):
        """Partition i (a list of modules, same length and tensor shapes for every rank) is summed
        onto rank i.  Works with any backend: backends without a list reduce-scatter fall back to
        one ``reduce`` per slot."""
        if not dist.is_initialized():
            raise EnvironmentError('torch.distributed is not initialized.')
        world_size = dist.get_world_size(group)
        if len(module_partitions) != world_size:
            raise ValueError(f'Number of partitions has to be world_size. Got {len(module_partitions)}')
        sizes = [len(p) for p in module_partitions]
        if len(set(sizes)) != 1:
            raise ValueError(f'Number of members in each partition has to be the same. Got {sizes}')
        per_rank = [self._tensors_for(mods, keys, with_grad) for mods in module_partitions]
        counts = [len(t) for t in per_rank]
        if len(set(counts)) != 1:
            raise ValueError(f'Number of tensors in every partition has to be {counts[0]}. Got {counts}')
        rank = dist.get_rank(group)
        use_rs = dist.get_backend(group) == dist.Backend.NCCL
        handles = []
        for slot in range(counts[0]):
            inputs = [tensors[slot] for tensors in per_rank]
            if use_rs:
                handles.append(dist.reduce_scatter(inputs[rank], inputs, group=group, async_op=async_op))
            else:
                for dst, tensor in enumerate(inputs):
                    dst_global = dist.get_global_rank(group, dst) if group is not None else dst
                    handles.append(dist.reduce(tensor, dst_global, group=group, async_op=async_op))
        return handles

    def reduce_fisher(self, modules, *keys, all_reduce=True, with_grad=False, dst=0,
                      group: dist.ProcessGroup = None, async_op=False):
        if not dist.is_initialized():
            raise ValueError('torch.distributed is not initialized.')
        handles = []
        for tensor in self._tensors_for(modules, keys, with_grad):
            if all_reduce:
                handles.append(dist.all_reduce(tensor, group=group, async_op=async_op))
            else:
                handles.append(dist.reduce(tensor, dst=dst, group=group, async_op=async_op))
        return handles

    def reduce_fvp(self, fisher_shape, is_master=True, all_reduce=False):
        v = reduce_vectors(self.load_fvp(fisher_shape), is_master, all_reduce)
        attr = self.config.fvp_attr
        if fisher_shape == SHAPE_FULL:
            setattr(self.model, attr, v)
        else:
            for module in self.model.modules():
                if hasattr(module, attr):
                    setattr(module, attr, v.get_vectors_by_module(module) if v is not None else None)

    def load_fvp(self, fisher_shape: str) -> ParamVector:
        attr = self.config.fvp_attr
        if fisher_shape == SHAPE_FULL:
            v = getattr(self.model, attr, None)
            return None if v is None else v.copy()
        out = None
        for module in self.model.modules():
            if module is self.model and len(list(module.children())) > 0:
                continue
            v = getattr(module, attr, None)
            if v is None:
                continue
            if out is None:
                out = v.copy()
            else:
                out.extend(v.copy())
        return out

    # ------------------------------------------------------------------ spectral tools
    def _get_fvp_fn(self):
        def fvp_fn(vec: ParamVector) -> ParamVector:
            self.forward_and_backward(fvp=True, vec=vec)
            return self.load_fvp(self.config.fisher_shapes[0])
        return fvp_fn

    def _mc_seed(self):
        # one seed for the whole solve turns the MC Fisher into a fixed matrix across iterations
        return int(torch.rand(1).item() * 100) + 1 if self.config.fisher_type == FISHER_MC else None

    def fisher_eig(self, top_n=1, max_iters=100, tol=1e-7, is_distributed=False, print_progress=False):
        return power_method(self._get_fvp_fn(), self.model, top_n=top_n, max_iters=max_iters,
                            tol=tol, is_distributed=is_distributed, print_progress=print_progress,
                            random_seed=self._mc_seed())

    def fisher_esd(self, n_v=1, num_iter=100, num_bins=10000, sigma_squared=1e-5, overhead=None,
                   is_distributed=False):
        """Eigenvalue spectral density by SLQ with Gaussian smoothing on a regular grid
        (PyHessian-style).  Returns (density, grid)."""
        eigvals, weights = stochastic_lanczos_quadrature(self._get_fvp_fn(), self.model, n_v=n_v,
                                                         num_iter=num_iter,
                                                         is_distributed=is_distributed,
                                                         random_seed=self._mc_seed())
        eigvals, weights = np.array(eigvals), np.array(weights)
        lam_max = np.mean(np.max(eigvals, axis=1))
        lam_min = np.mean(np.min(eigvals, axis=1))
        sigma_squared = sigma_squared * max(1, lam_max - lam_min)
        if overhead is None:
            overhead = np.sqrt(sigma_squared)
        grid = np.linspace(np.maximum(0., lam_min - overhead), lam_max + overhead, num=num_bins)
        diffs = grid[None, :, None] - eigvals[:, None, :]  # n_v x bins x iters
        gauss = np.exp(-diffs ** 2 / (2.0 * sigma_squared)) / np.sqrt(2 * np.pi * sigma_squared)
        density = np.mean(np.sum(gauss * weights[:, None, :], axis=2), axis=0)
        density = density / (np.sum(density) * (grid[1] - grid[0]))
        return density, grid

    def _grad_vector(self):
        grads = {p: p.grad for p in self.model.parameters() if p.requires_grad}
        return ParamVector(grads.keys(), grads.values())

    def fisher_free(self, b=None, init_x=None, damping=1e-3, max_iters=None, tol=1e-8,
                    preconditioner=None, print_progress=False, random_seed=None) -> ParamVector:
        """(F + damping*I)^-1 b by conjugate gradients (b defaults to the current gradient)."""
        if b is None:
            b = self._grad_vector()
        if random_seed is None:
            random_seed = self._mc_seed()
        return conjugate_gradient_method(self._get_fvp_fn(), b, init_x=init_x, damping=damping,
                                         max_iters=max_iters, tol=tol, preconditioner=preconditioner,
                                         print_progress=print_progress, random_seed=random_seed)

    def fisher_quadratic_form(self, vec: ParamVector = None):
        if vec is None:
            vec = self._grad_vector()
        return quadratic_form(self._get_fvp_fn(), vec)


def _flat_classes(t):
    return t.reshape(-1, t.shape[-1])


class FisherExactCrossEntropy(FisherMaker):
    @property
    def do_local_accumulate(self) -> bool:
        return True if self._logits is None else self._logits.shape[-1] > 1

    def _fisher_loop(self, closure):
        logits = self._logits
        log_probs = _flat_classes(F.log_softmax(logits, dim=-1))
        n, n_classes = log_probs.shape
        with torch.no_grad():
            sqrt_probs = _flat_classes(F.softmax(logits, dim=-1)).sqrt()
        for c in range(n_classes):
            targets = torch.full((n,), c, device=logits.device, dtype=torch.long)

            def nll_expr():
                nll = F.nll_loss(log_probs, targets, reduction='none',
                                 ignore_index=self.config.ignore_index)
                return (nll * sqrt_probs[:, c]).sum()

            closure(nll_expr, retain_graph=c < n_classes - 1)


class FisherMCCrossEntropy(FisherMaker):
    @property
    def do_local_accumulate(self) -> bool:
        return self.config.n_mc_samples > 1

    def _fisher_loop(self, closure):
        logits = self._logits
        n_mc = self.config.n_mc_samples
        log_probs = _flat_classes(F.log_softmax(logits.float(), dim=-1))
        with torch.no_grad():
            probs = log_probs.exp()
        for i in range(n_mc):
            with torch.no_grad():
                targets = torch.multinomial(probs, 1).squeeze(1)
            closure(lambda: F.nll_loss(log_probs, targets, reduction='sum',
                                       ignore_index=self.config.ignore_index) / n_mc,
                    retain_graph=i < n_mc - 1)


class FisherExactMSE(FisherMaker):
    @property
    def do_local_accumulate(self) -> bool:
        return True if self._logits is None else self._logits.shape[-1] > 1

    def _fisher_loop(self, closure):
        logits = self._logits
        n_dims = logits.size(-1)
        for d in range(n_dims):
            closure(lambda: logits[..., d].sum(), retain_graph=d < n_dims - 1)


class FisherMCMSE(FisherMaker):
    @property
    def do_local_accumulate(self) -> bool:
        return self.config.n_mc_samples > 1

    def _fisher_loop(self, closure):
        logits = self._logits
        n_mc = self.config.n_mc_samples
        std = float(np.sqrt(self.config.var))
        for i in range(n_mc):
            with torch.no_grad():
                targets = logits + std * torch.randn_like(logits)
            closure(lambda: 0.5 * F.mse_loss(logits, targets, reduction='sum') / n_mc,
                    retain_graph=i < n_mc - 1)


class FisherEmp(FisherMaker):
    @property
    def do_local_accumulate(self) -> bool:
        return False

    @property
    def is_fisher_emp(self):
        return True


def get_fisher_maker(model: nn.Module, config: FisherConfig):
    """The FisherMaker subclass for ``config.fisher_type`` (exact / Monte-Carlo / empirical) and
    ``config.loss_type`` (cross-entropy / MSE).  Reference: asdl/fisher.py:500-521.
    """
    fisher_type, loss_type = config.fisher_type, config.loss_type
    if fisher_type not in _supported_types:
        raise ValueError(f'Invalid fisher_type: {fisher_type}. {_supported_types} are supported.')
    if fisher_type == FISHER_EMP:
        return FisherEmp(model, config)
    if loss_type not in [LOSS_CROSS_ENTROPY, LOSS_MSE]:
        raise ValueError(f'Invalid loss_type: {loss_type}. {[LOSS_CROSS_ENTROPY, LOSS_MSE]} are supported.')
    table = {(FISHER_EXACT, LOSS_CROSS_ENTROPY): FisherExactCrossEntropy,
             (FISHER_EXACT, LOSS_MSE): FisherExactMSE,
             (FISHER_MC, LOSS_CROSS_ENTROPY): FisherMCCrossEntropy,
             (FISHER_MC, LOSS_MSE): FisherMCMSE}
    return table[(fisher_type, loss_type)](model, config)
