"""PSGD: the preconditioner P = Q^T Q is fitted online so that it whitens pairs
(dx, dg = H dx) of a random parameter perturbation and the resulting gradient perturbation
(Li, "Preconditioned Stochastic Gradient Descent", arXiv:1512.04202).

Parity: asdl/precondition/psgd.py:25-629 - ``PsgdGradientMaker`` (one P x P triangular factor for
the whole model), ``KronPsgdGradientMaker`` (per layer P = (Qr^T Qr) (x) (Ql^T Ql), bias folded in
as an extra column), and the factor-format functions ``update_precond_kron`` /
``precond_grad_kron`` for dense, normalisation (diagonal + last column) and scaling (diagonal)
factors.

The update rule is the same for every format: with A = Ql dG Qr^T and B = Ql^-T dX Qr^-1,
    Ql <- Ql - mu/max|G_l| * G_l Ql,   G_l = proj(A A^T - B B^T)
    Qr <- Qr - mu/max|G_r| * G_r Qr,   G_r = proj(A^T A - B^T B)
where ``proj`` keeps the entries the factor format owns (upper triangle / diagonal / diagonal and
last column).  Here each format is a small class that knows how to multiply, solve and project,
so the nine (left, right) combinations share one code path.  The Hessian-vector product comes
from a double backward (or ``torch.func`` when ``use_functorch=True``); step-size normalisation
stays on the device (no host round trip for ``max|G|``).
"""
from typing import Iterable, List, Tuple

import numpy as np
import torch
import torch.nn as nn
from torch import Tensor
from torch.linalg import solve_triangular

from .. import ops

from .prec_grad_maker import PreconditionedGradientMaker, PreconditioningConfig

__all__ = ['PsgdGradientMaker', 'KronPsgdGradientMaker', 'update_precond_kron', 'precond_grad_kron',
           'update_precond_splu', 'precond_grad_splu']

_TINY = 1.2e-38


def parameters_to_vector(parameters: Iterable[Tensor]) -> Tensor:
    return torch.cat([p.reshape(-1) for p in parameters])


def _write_back(flat: Tensor, tensors: List[Tensor]):
    offset = 0
    for t in tensors:
        t.copy_(flat[offset:offset + t.numel()].view_as(t))
        offset += t.numel()


class PsgdGradientMaker(PreconditionedGradientMaker):
    r"""PSGD with one dense triangular factor over all preconditioned parameters.

    The factor is :math:`P\times P` (P = number of trainable parameters of the supported layers),
    so this maker is only meant for very small networks; use :class:`KronPsgdGradientMaker`
    otherwise.

    Args:
        model: module to precondition (Linear / Conv2d layers).
        config: :class:`PreconditioningConfig`.
        precond_lr: normalised step size of the factor update.
        init_scale: the factor starts as ``init_scale * I``.
        use_functorch: compute the Hessian-vector product with ``torch.func`` (forward-over-reverse)
            instead of a double backward.
    """
    _supported_classes = (nn.Linear, nn.Conv2d)

    def __init__(self, model: nn.Module, config: PreconditioningConfig,
                 precond_lr: float = 0.01, init_scale: float = 1., use_functorch=False):
        super().__init__(model, config)
        self.precond_lr = precond_lr
        self.init_scale = init_scale
        self._init_cholesky_factors()
        self.use_functorch = use_functorch

    def _init_cholesky_factors(self):
        n = sum(p.numel() for p in self.module_dict.parameters())
        self.cholesky_factor = self.init_scale * torch.eye(n, device=self.device)

    def do_forward_and_backward(self, step=None):
        return not self.do_update_preconditioner(step)

    def _probe_and_hvp(self, retain_graph=False):
        params = list(self.module_dict.parameters())
        if self.use_functorch:
            vs = self._get_random_tangents()
            hvs = self.loss_hvp(tangents=vs)
            wanted = {id(p) for p in params}
            keep = [i for i, p in enumerate(q for q in self.model.parameters() if q.requires_grad)
                    if id(p) in wanted]
            return [vs[i] for i in keep], [hvs[i] for i in keep]
        self.forward()
        everything = [p for p in self.model.parameters() if p.requires_grad]
        all_grads = torch.autograd.grad(self._loss, everything, create_graph=True, allow_unused=True)
        by_id = {id(p): g for p, g in zip(everything, all_grads)}
        grads = [by_id[id(p)] for p in params]
        vs = [torch.randn_like(p) for p in params]
        hvs = torch.autograd.grad(grads, params, vs, retain_graph=retain_graph)
        for p, g in zip(everything, all_grads):  # every trainable parameter gets its gradient
            if g is not None:
                p.grad = g.detach()
        return vs, list(hvs)

    def update_preconditioner(self, retain_graph=False):
        vs, hvs = self._probe_and_hvp(retain_graph)
        self._update_preconditioner(list(vs), list(hvs))

    @torch.no_grad()
    def _update_preconditioner(self, dxs: List[Tensor], dgs: List[Tensor], eps=_TINY):
        dx = parameters_to_vector(dxs)
        dg = parameters_to_vector(dgs)
        Q = self.cholesky_factor
        a = Q.mv(dg)
        b = solve_triangular(Q.T, dx.unsqueeze(-1), upper=False).squeeze(-1)
        grad = torch.triu(torch.outer(a, a) - torch.outer(b, b))
        lr = self.precond_lr / (grad.abs().max() + eps)
        Q.sub_(lr * grad.mm(Q))

    @torch.no_grad()
    def precondition(self):
        grads = [p.grad for p in self.module_dict.parameters()]
        Q = self.cholesky_factor
        _write_back(Q.T.mv(Q.mv(parameters_to_vector(grads))), grads)

    def criterion(self, n_samples=1):
        """Fitting criterion E[dx^T P^-1 dx + dg^T P dg] (lower is better)."""
        total = 0.
        for _ in range(n_samples):
            vs = self._get_random_tangents()
            hvs = self.loss_hvp(tangents=vs, accumulate_grad=False)
            total += self._criterion(vs, hvs)
        return total / n_samples

    @torch.no_grad()
    def _criterion(self, dxs: Tuple[Tensor], dgs: Tuple[Tensor]):
        dx = parameters_to_vector(dxs)
        dg = parameters_to_vector(dgs)
        Q = self.cholesky_factor
        y = solve_triangular(Q.T, dx.unsqueeze(-1), upper=False)
        return float((y * y).sum() + Q.mv(dg).square().sum())

    def _curvature_state(self):
        return {'cholesky_factor': self.cholesky_factor}

    def _load_curvature_state(self, tensors):
        if 'cholesky_factor' in tensors:
            self.cholesky_factor = tensors['cholesky_factor'].to(self.device)


class KronPsgdGradientMaker(PsgdGradientMaker):
    r"""PSGD with a layer-wise Kronecker-factored preconditioner
    :math:`P = (Q_r^\top Q_r)\otimes(Q_l^\top Q_l)`; a bias is appended to the weight as one more
    input column."""

    def _init_cholesky_factors(self):
        self.cholesky_factors = {}
        for module in self.module_dict.children():
            in_dim = int(np.prod(module.weight.shape[1:])) + (1 if module.bias is not None else 0)
            out_dim = module.weight.shape[0]
            self.cholesky_factors[module] = (self.init_scale * torch.eye(out_dim, device=self.device),
                                             self.init_scale * torch.eye(in_dim, device=self.device))

    @staticmethod
    def _as_matrix(module, pieces: List[Tensor]):
        w = pieces.pop(0)
        mat = w.flatten(start_dim=1)
        if module.bias is not None:
            mat = torch.cat([mat, pieces.pop(0).unsqueeze(-1)], dim=1)
        return mat

    @torch.no_grad()
    def _update_preconditioner(self, dxs: List[Tensor], dgs: List[Tensor]):
        for module in self.module_dict.children():
            dX = self._as_matrix(module, dxs)
            dG = self._as_matrix(module, dgs)
            Ql, Qr = self.cholesky_factors[module]
            self.cholesky_factors[module] = update_precond_kron(Ql, Qr, dX, dG, step=self.precond_lr)
        if dxs or dgs:
            raise ValueError('perturbations are still remaining.')

    @torch.no_grad()
    def precondition(self):
        grads = [p.grad for p in self.module_dict.parameters()]
        for module in self.module_dict.children():
            G = self._as_matrix(module, grads)
            G = precond_grad_kron(*self.cholesky_factors[module], G)
            if module.bias is not None:
                module.weight.grad.copy_(G[:, :-1].reshape(module.weight.shape))
                module.bias.grad.copy_(G[:, -1])
            else:
                module.weight.grad.copy_(G.reshape(module.weight.shape))
        if grads:
            raise ValueError('grads are still remaining')

    def _criterion(self, dxs, dgs):
        dxs, dgs = list(dxs), list(dgs)
        total = 0.
        for module in self.module_dict.children():
            dX, dG = self._as_matrix(module, dxs), self._as_matrix(module, dgs)
            Ql, Qr = self.cholesky_factors[module]
            fl, fr = _factor(Ql), _factor(Qr)
            A = fr.right_mul_t(fl.left_mul(dG))
            B = fr.right_solve(fl.left_solve_t(dX))
            total += float(A.square().sum() + B.square().sum())
        return total

    def _curvature_state(self):
        out = {}
        for name, module in self.module_dict.items():
            Ql, Qr = self.cholesky_factors[module]
            out[f'{name}.Ql'] = Ql
            out[f'{name}.Qr'] = Qr
        return out

    def _load_curvature_state(self, tensors):
        for name, module in self.module_dict.items():
            if f'{name}.Ql' in tensors:
                self.cholesky_factors[module] = (tensors[f'{name}.Ql'].to(self.device),
                                                 tensors[f'{name}.Qr'].to(self.device))


# ----------------------------------------------------------------------------------------------
# factor formats
# ----------------------------------------------------------------------------------------------
class _Dense:
    """Upper-triangular n x n factor."""

    def __init__(self, Q):
        self.Q = Q

    def max_diag(self):
        return torch.diagonal(self.Q).max()

    def scaled(self, s):
        return _Dense(self.Q * s)

    def _tc(self, *others):
        """Dense products of factors from 256 x 256 on run on the tensor-core GEMM (fp32 operands as three
        bf16 part products, fp32 accumulation); smaller ones are launch-bound either way."""
        return (self.Q.shape[0] >= 256 and self.Q.dtype == torch.float32
                and ops.cuda_kernels_enabled(self.Q, *others) and all(o.dtype == torch.float32 and o.ndim == 2 for o in others))

    def left_mul(self, X):            # Q X
        return ops.matmul(self.Q, X) if self._tc(X) else self.Q @ X

    def right_mul_t(self, X):         # X Q^T
        return ops.matmul(X, self.Q, trans_b=True) if self._tc(X) else X @ self.Q.T

    def left_solve_t(self, X):        # Q^-T X
        return solve_triangular(self.Q.T, X, upper=False)

    def right_solve(self, X):         # X Q^-1
        return solve_triangular(self.Q, X, upper=True, left=False)

    def updated(self, A, B, step, on_rows):
        if self._tc(A, B):
            # A A^T - B B^T (rows) or A^T A - B^T B (columns): two symmetric products into one matrix
            M = ops.matmul(A, A, trans_a=not on_rows, trans_b=on_rows, sym=True)
            ops.matmul(B, B, trans_a=not on_rows, trans_b=on_rows, alpha=-1.0, out=M, beta=1.0, sym=True)
            G = torch.triu(M)
            return self.Q - (step / (G.abs().max() + _TINY)) * ops.matmul(G, self.Q)
        M = (A @ A.T - B @ B.T) if on_rows else (A.T @ A - B.T @ B)
        G = torch.triu(M)
        return self.Q - (step / (G.abs().max() + _TINY)) * (G @ self.Q)

    def gram_apply_left(self, X):     # Q^T Q X
        if self._tc(X):
            return ops.matmul(self.Q, ops.matmul(self.Q, X), trans_a=True)
        return self.Q.T @ (self.Q @ X)

    def gram_apply_right(self, X):    # X Q^T Q
        if self._tc(X):
            return ops.matmul(ops.matmul(X, self.Q, trans_b=True), self.Q)
        return (X @ self.Q.T) @ self.Q


class _Scale:
    """Diagonal factor stored as 1 x n."""

    def __init__(self, q):
        self.q = q

    def max_diag(self):
        return self.q.max()

    def scaled(self, s):
        return _Scale(self.q * s)

    def left_mul(self, X):
        return self.q.T * X

    def right_mul_t(self, X):
        return X * self.q

    def left_solve_t(self, X):
        return X / self.q.T

    def right_solve(self, X):
        return X / self.q

    def updated(self, A, B, step, on_rows):
        dim = 1 if on_rows else 0
        g = (A * A).sum(dim=dim) - (B * B).sum(dim=dim)
        return self.q - (step / (g.abs().max() + _TINY)) * g.view_as(self.q) * self.q

    def gram_apply_left(self, X):
        return (self.q * self.q).T * X

    def gram_apply_right(self, X):
        return X * (self.q * self.q)


class _Norm:
    """"Normalisation" factor: upper triangular with a free diagonal d (row 0 of the 2 x n
    storage) and a free last column c (row 1, its last entry unused)."""

    def __init__(self, q):
        self.q = q
        self.d = q[0]
        self.c = q[1].clone()
        self.c[-1] = 0

    def _dense(self):
        Q = torch.diag(self.d)
        Q[:-1, -1] += self.c[:-1]
        return Q

    def max_diag(self):
        return self.d.max()

    def scaled(self, s):
        return _Norm(self.q * s)

    def left_mul(self, X):            # Q X = d * X + c x_last
        return self.d.unsqueeze(1) * X + self.c.unsqueeze(1) * X[-1:]

    def right_mul_t(self, X):         # X Q^T = (Q X^T)^T
        return self.left_mul(X.T).T

    def left_solve_t(self, X):        # Q^-T X  (Q^T is lower triangular: diag d, last row c)
        out = X / self.d.unsqueeze(1)
        out[-1] = (X[-1] - (self.c[:-1].unsqueeze(1) * out[:-1]).sum(dim=0)) / self.d[-1]
        return out

    def right_solve(self, X):         # X Q^-1 = (Q^-T X^T)^T
        return self.left_solve_t(X.T).T

    def updated(self, A, B, step, on_rows):
        if not on_rows:
            A, B = A.T, B.T
        g_diag = (A * A).sum(dim=1) - (B * B).sum(dim=1)
        g_col = A[:-1] @ A[-1] - B[:-1] @ B[-1]
        g_col = torch.cat([g_col, g_col.new_zeros(1)])
        s = step / (torch.maximum(g_diag.abs().max(), g_col.abs().max()) + _TINY)
        new_d = self.d - s * g_diag * self.d
        new_c = self.c - s * (g_diag * self.c + self.d[-1] * g_col)
        return torch.stack([new_d, new_c])

    def gram_apply_left(self, X):     # Q^T (Q X)
        Y = self.left_mul(X)
        out = self.d.unsqueeze(1) * Y
        out[-1] = out[-1] + (self.c.unsqueeze(1) * Y).sum(dim=0)
        return out

    def gram_apply_right(self, X):
        return self.gram_apply_left(X.T).T


def _factor(Q):
    rows, cols = Q.shape
    if rows == cols:
        return _Dense(Q)
    if rows == 2:
        return _Norm(Q)
    if rows == 1:
        return _Scale(Q)
    raise Exception('Unknown Kronecker product preconditioner')


@torch.no_grad()
def update_precond_kron(Ql, Qr, dX, dG, step=0.01, _tiny=_TINY):
    """One fitting step of P = kron(Qr^T Qr, Ql^T Ql).  Each factor is dense upper triangular
    (n x n), a normalisation factor (2 x n) or a scaling factor (1 x n).  Returns the new
    (Ql, Qr); dense factors are also updated in place.

    dX: perturbation of the (matrix) parameter, dG: perturbation of its gradient."""
    fl, fr = _factor(Ql), _factor(Qr)
    rho = torch.sqrt(fl.max_diag() / fr.max_diag())  # keep both factors in a similar range
    fl, fr = fl.scaled(1 / rho), fr.scaled(rho)
    A = fr.right_mul_t(fl.left_mul(dG))        # Ql dG Qr^T
    B = fr.right_solve(fl.left_solve_t(dX))    # Ql^-T dX Qr^-1
    new_l = fl.updated(A, B, step, on_rows=True)
    new_r = fr.updated(A, B, step, on_rows=False)
    if Ql.shape == new_l.shape:
        Ql.copy_(new_l)
        new_l = Ql
    if Qr.shape == new_r.shape:
        Qr.copy_(new_r)
        new_r = Qr
    return new_l, new_r


@torch.no_grad()
def precond_grad_kron(Ql, Qr, Grad):
    """``Ql^T Ql . Grad . Qr^T Qr`` for any combination of factor formats."""
    return _factor(Qr).gram_apply_right(_factor(Ql).gram_apply_left(Grad))


# ----------------------------------------------------------------------------------------------
# sparse-LU preconditioner  P = Q^T Q,  Q = L U  with "arrow" factors
#     L = [[L1, 0], [L2, diag(l3)]]   (L1: r x r lower triangular)
#     U = [[U1, U2], [0, diag(u3)]]   (U1: r x r upper triangular)
# stored as L12 = [L1; L2] (n x r), l3 ((n-r) x 1), U12 = [U1, U2] (r x n), u3 ((n-r) x 1).
# Parity: asdl/precondition/psgd.py:498-629 (a format no gradient maker uses; kept as functions).
# ----------------------------------------------------------------------------------------------
class _ArrowLU:
    """Products and solves with the arrow factors on (head, tail) = (first r, remaining) parts."""

    def __init__(self, L12, l3, U12, u3):
        r = U12.shape[0]
        self.r = r
        self.L1, self.L2, self.l3 = L12[:r], L12[r:], l3.reshape(-1)
        self.U1, self.U2, self.u3 = U12[:, :r], U12[:, r:], u3.reshape(-1)

    def split(self, v):
        return v[:self.r], v[self.r:]

    def U(self, h, t):
        return self.U1 @ h + self.U2 @ t, self.u3 * t

    def L(self, h, t):
        return self.L1 @ h, self.L2 @ h + self.l3 * t

    def Lt(self, h, t):
        return self.L1.T @ h + self.L2.T @ t, self.l3 * t

    def Ut(self, h, t):
        return self.U1.T @ h, self.U2.T @ h + self.u3 * t

    @staticmethod
    def _tri(mat, rhs, upper, transpose=False):
        a = mat.T if transpose else mat
        return torch.linalg.solve_triangular(a, rhs.unsqueeze(1), upper=(upper != transpose)).squeeze(1)

    def Ut_solve(self, h, t):      # U^-T
        x = self._tri(self.U1, h, upper=True, transpose=True)
        return x, (t - self.U2.T @ x) / self.u3

    def Lt_solve(self, h, t):      # L^-T
        y = t / self.l3
        return self._tri(self.L1, h - self.L2.T @ y, upper=False, transpose=True), y

    def L_solve(self, h, t):       # L^-1
        x = self._tri(self.L1, h, upper=False)
        return x, (t - self.L2 @ x) / self.l3

    def U_solve(self, h, t):       # U^-1
        y = t / self.u3
        return self._tri(self.U1, h - self.U2 @ y, upper=True), y


def _flatten_list(tensors):
    return torch.cat([t.reshape(-1) for t in tensors])


@torch.no_grad()
def update_precond_splu(L12, l3, U12, u3, dxs, dgs, step=0.01, _tiny=_TINY):
    """One fitting step of the sparse-LU preconditioner from a parameter perturbation ``dxs`` and
    the resulting gradient perturbation ``dgs`` (lists of tensors).  Returns the new
    ``(L12, l3, U12, u3)``; the inputs are rescaled in place so that L and U keep a similar range."""
    rho = torch.sqrt(torch.maximum(torch.diagonal(L12).max(), l3.max())
                     / torch.maximum(torch.diagonal(U12).max(), u3.max()))
    L12 /= rho
    l3 /= rho
    U12 *= rho
    u3 *= rho
    f = _ArrowLU(L12, l3, U12, u3)
    dx_h, dx_t = f.split(_flatten_list(dxs))
    dg_h, dg_t = f.split(_flatten_list(dgs))
    qg_h, qg_t = f.L(*f.U(dg_h, dg_t))                      # Q dg
    iq_h, iq_t = f.Lt_solve(*f.Ut_solve(dx_h, dx_t))        # Q^-T dx
    pg_h, pg_t = f.Ut(*f.Lt(qg_h, qg_t))                    # P dg
    ip_h, ip_t = f.U_solve(*f.L_solve(iq_h, iq_t))          # P^-1 dx

    def normalised(step_, *grads):
        return step_ / (torch.stack([g.abs().max() for g in grads]).max() + _tiny)

    # L <- L - mu * [[tril(g1), 0], [g2, diag(g3)]] L
    g1 = torch.tril(torch.outer(qg_h, qg_h) - torch.outer(iq_h, iq_h))
    g2 = torch.outer(qg_t, qg_h) - torch.outer(iq_t, iq_h)
    g3 = qg_t * qg_t - iq_t * iq_t
    mu = normalised(step, g1, g2, g3)
    new_L1 = f.L1 - mu * (g1 @ f.L1)
    new_L2 = f.L2 - mu * (g2 @ f.L1) - mu * g3.unsqueeze(1) * f.L2
    new_l3 = f.l3 - mu * g3 * f.l3
    # U <- U - mu * U [[triu(h1), h2], [0, diag(h3)]]
    h1 = torch.triu(torch.outer(pg_h, dg_h) - torch.outer(dx_h, ip_h))
    h2 = torch.outer(pg_h, dg_t) - torch.outer(dx_h, ip_t)
    h3 = pg_t * dg_t - dx_t * ip_t
    mu = normalised(step, h1, h2, h3)
    new_U1 = f.U1 - mu * (f.U1 @ h1)
    new_U2 = f.U2 - mu * (f.U1 @ h2) - mu * h3.unsqueeze(0) * f.U2
    new_u3 = f.u3 - mu * h3 * f.u3
    return (torch.cat([new_L1, new_L2], dim=0), new_l3.reshape(-1, 1),
            torch.cat([new_U1, new_U2], dim=1), new_u3.reshape(-1, 1))


@torch.no_grad()
def precond_grad_splu(L12, l3, U12, u3, grads):
    """``P g`` with the sparse-LU preconditioner for a list of gradient tensors; returns a list of
    tensors with the shapes of ``grads``."""
    f = _ArrowLU(L12, l3, U12, u3)
    h, t = f.split(_flatten_list(grads))
    out = torch.cat(f.Ut(*f.Lt(*f.L(*f.U(h, t)))))
    result, offset = [], 0
    for g in grads:
        result.append(out[offset:offset + g.numel()].view_as(g))
        offset += g.numel()
    return result
