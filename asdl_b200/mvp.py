"""Matrix-free solvers that only need a matrix-vector product on :class:`ParamVector`:
power iteration with deflation, stochastic Lanczos quadrature, conjugate gradients and quadratic
forms.  Parity: asdl/mvp.py:18-231 (the algorithms follow PyHessian's formulation).

The scalars that steer the iterations (Rayleigh quotients, residual norms) are needed on the host
every step anyway, so they are read with a single ``.item()`` per iteration.
"""
import math
from typing import Callable, List

import numpy as np
import torch
import torch.nn as nn
import torch.distributed as dist

from . import ops
from .vector import ParamVector, normalization, orthnormal

__all__ = ['power_method', 'stochastic_lanczos_quadrature', 'conjugate_gradient_method',
           'quadratic_form']

MvpFn = Callable[[ParamVector], ParamVector]


def _mvp(mvp_fn: MvpFn, vec: ParamVector, random_seed=None, damping=None) -> ParamVector:
    """mvp_fn(vec) (+ damping*vec).  Re-seeding makes stochastic matrices (MC Fisher) behave as
    one fixed matrix across iterations."""
    if random_seed:
        torch.manual_seed(int(random_seed))
    out = mvp_fn(vec)
    if damping:
        out.add_(vec, alpha=damping)
    return out


def _trainable(model):
    return [p for p in model.parameters() if p.requires_grad]


def _synchronised(vec: ParamVector, params, is_distributed):
    """Rank 0's vector on every rank."""
    if not is_distributed:
        return vec
    flat = vec.get_flatten_vector()
    dist.broadcast(flat, src=0)
    return ParamVector(params, flat)


def power_method(mvp_fn: MvpFn, model: nn.Module, top_n=1, max_iters=100, tol=1e-7,
                 is_distributed=False, print_progress=False, random_seed=None):
    """Top ``top_n`` eigenpairs by power iteration; found eigenvectors are projected out before
    every product.  Returns (eigenvalues, eigenvectors) sorted by decreasing eigenvalue."""
    if top_n < 1:
        raise ValueError(f'top_n has to be >=1. Got {top_n}.')
    if max_iters < 1:
        raise ValueError(f'max_iters has to be >=1. Got {max_iters}.')
    params = _trainable(model)
    eigvals: List[float] = []
    eigvecs: List[ParamVector] = []
    for i in range(top_n):
        if print_progress:
            print(f'start power iteration for lambda({i+1}).')
        vec = _synchronised(ParamVector(params, [torch.randn_like(p) for p in params]), params,
                            is_distributed)
        eigval = last = None
        for j in range(max_iters):
            vec = orthnormal(vec, eigvecs)
            Mv = _mvp(mvp_fn, vec, random_seed=random_seed)
            eigval = Mv.dot(vec).item()
            if j > 0:
                diff = abs(eigval - last) / (abs(last) + 1e-6)
                if print_progress:
                    print(f'{j}/{max_iters} diff={diff}')
                if diff < tol:
                    break
            last = eigval
            vec = Mv
        eigvals.append(eigval)
        eigvecs.append(vec)
    order = np.argsort(eigvals)[::-1]
    return [eigvals[k] for k in order], [eigvecs[k] for k in order]


def stochastic_lanczos_quadrature(mvp_fn: MvpFn, model: nn.Module, n_v=1, num_iter=100,
                                  is_distributed=False, random_seed=None):
    """``n_v`` Lanczos runs of ``num_iter`` steps from Rademacher start vectors with full
    re-orthogonalisation.  Returns the Ritz values and the squared first components of the Ritz
    vectors (quadrature weights) of each run."""
    if n_v < 1:
        raise ValueError(f'n_v has to be >=1. Got {n_v}.')
    if num_iter < 1:
        raise ValueError(f'num_iter has to be >=1. Got {num_iter}.')
    params = _trainable(model)
    device = params[0].device
    all_eigvals: List[List[float]] = []
    all_weights: List[List[float]] = []
    for _ in range(n_v):
        start = [torch.randint_like(p, high=2).mul_(2).sub_(1) for p in params]
        vec = _synchronised(normalization(ParamVector(params, start)), params, is_distributed)
        basis = [vec]
        alphas, betas = [], []
        w = None
        for i in range(num_iter):
            if i > 0:
                beta = float(w.norm())
                betas.append(beta)
                if beta != 0.:
                    vec = orthnormal(w, basis)
                else:  # invariant subspace found: restart with a fresh direction
                    fresh = ParamVector(params, [torch.randn_like(p) for p in params])
                    vec = _synchronised(orthnormal(fresh, basis), params, is_distributed)
                basis.append(vec)
            w = _mvp(mvp_fn, vec, random_seed=random_seed)
            alpha = w.dot(vec)
            alphas.append(alpha.item())
            w = w.add(vec, alpha=-alpha)
            if i > 0:
                w = w.add(basis[-2], alpha=-betas[-1])
        T = torch.diag(torch.tensor(alphas, device=device))
        if betas:
            off = torch.tensor(betas, device=device)
            T = T + torch.diag(off, 1) + torch.diag(off, -1)
        eigval, eigvec = ops.eigh(T)
        all_eigvals.append(eigval.tolist())
        all_weights.append((eigvec[0, :] ** 2).tolist())
    return all_eigvals, all_weights


def conjugate_gradient_method(mvp_fn: MvpFn, b: ParamVector, init_x: ParamVector = None,
                              damping=1e-3, max_iters=None, tol=1e-8, preconditioner=None,
                              print_progress=False, random_seed=None) -> ParamVector:
    """Solve (A + damping*I) x = b.  ``preconditioner`` needs a ``precondition(ParamVector)``
    method that returns M^-1 r."""
    if not isinstance(b, ParamVector):
        raise TypeError(f'b has to be an instance of {ParamVector}. {type(b)} is given.')
    if max_iters is None:
        max_iters = b.numel()

    def A(v):
        return _mvp(mvp_fn, v, random_seed, damping)

    if init_x is None:
        x = ParamVector(b.params(), [torch.zeros_like(p) for p in b.params()])
        r = b.copy()
    else:
        x = init_x
        r = b.add(A(x), alpha=-1)
    if preconditioner is None:
        p = r.copy()
        rz = r.dot(r)
    else:
        p = preconditioner.precondition(r)
        rz = r.dot(p)
    b_norm = float(b.norm())
    for i in range(max_iters):
        Ap = A(p)
        alpha = rz / p.dot(Ap)
        x.add_(p, alpha)
        r.add_(Ap, -alpha)
        rr = r.dot(r)
        err = math.sqrt(float(rr)) / b_norm
        if print_progress:
            print(f'{i+1}/{max_iters} err={err}')
        if err < tol:
            break
        if preconditioner is None:
            z, new_rz = r, rr
        else:
            z = preconditioner.precondition(r)
            new_rz = r.dot(z)
        p = z.add(p, new_rz / rz)  # Fletcher-Reeves
        rz = new_rz
    return x


def quadratic_form(mvp_fn: MvpFn, v: ParamVector, random_seed=None, damping=0):
    """v^T (A + damping*I) v."""
    return v.dot(_mvp(mvp_fn, v, random_seed, damping))
