"""Curvature containers: dense symmetric blocks, Kronecker factors, Kronecker-factored
eigenbases, unit-wise blocks and diagonals.

Parity: asdl/symmatrix.py (``matrix_to_tril`` :25-38, ``tril_to_matrix`` :41-58,
``SymMatrix`` :94-358, ``Kron`` :361-548, ``KFE`` :551-614, ``UnitWise`` :617-719,
``Diag`` :722-869).  The on-disk layout written by ``save`` (float32 ``.npy`` files holding the
row-major lower triangle: ``tril.npy``, ``kron/A_tril.npy``, ``kron/B_tril.npy``,
``diag/weight.npy``, ``diag/bias.npy``, ``unit_wise.npy``) is the same.

What is different:
  * inverses never mutate the stored matrix (damping is applied inside the factorisation);
  * the dense inverse, the Kronecker two-sided product and the damped inverse go through
    :mod:`asdl_b200.ops`, which runs the library's sm_100a kernels for CUDA tensors;
  * every container exposes ``tensors()`` / ``load_tensors()`` so that gradient makers can put
    the curvature into their ``state_dict``.
"""
import math
import os
from typing import Dict, Iterable, Optional, Tuple

import numpy as np
import torch
from torch import Tensor

from . import ops
from .utils import smw_inv
from .vector import ParamVector

__all__ = [
    'matrix_to_tril', 'tril_to_matrix', 'get_n_cols_by_tril',
    'SymMatrix', 'Kron', 'KFE', 'Diag', 'UnitWise'
]

_default_damping = 1e-5


# ----------------------------------------------------------------------------------------------
# triangle packing
# ----------------------------------------------------------------------------------------------
def matrix_to_tril(mat: torch.Tensor):
    """Row-major lower triangle of a matrix as a 1-D tensor: [[1,.,.],[2,3,.],[4,5,6]] -> 1..6."""
    if mat.ndim != 2:
        raise ValueError(f'mat.ndim has to be 2. Got {mat.ndim}.')
    rows, cols = torch.tril_indices(mat.shape[0], mat.shape[1], device=mat.device)
    return mat[rows, cols]


def get_n_cols_by_tril(tril: torch.Tensor):
    """Side length n of the matrix whose packed triangle has n(n+1)/2 entries."""
    if tril.ndim != 1:
        raise ValueError(f'tril.ndim has to be 1. Got {tril.ndim}.')
    return int(math.sqrt(2 * tril.numel() + 0.25) - 0.5)


def tril_to_matrix(tril: torch.Tensor):
    """Inverse of :func:`matrix_to_tril` for a symmetric matrix."""
    if tril.ndim != 1:
        raise ValueError(f'tril.ndim has to be 1. Got {tril.ndim}.')
    n = get_n_cols_by_tril(tril)
    if n * (n + 1) // 2 != tril.numel():
        raise ValueError(f'{tril.numel()} entries are not the packed triangle of any square matrix.')
    rows, cols = torch.tril_indices(n, n, device=tril.device)
    out = torch.zeros(n, n, device=tril.device, dtype=tril.dtype)
    out[rows, cols] = tril
    out[cols, rows] = tril
    return out


def _eigvalsh(mat: torch.Tensor):
    return torch.linalg.eigvalsh(mat, UPLO='U')


def symeig(A: torch.Tensor, upper=True):
    """Eigenvalues of a symmetric matrix from its upper (default) or lower triangle, ascending."""
    return torch.linalg.eigvalsh(A, UPLO='U' if upper else 'L')


def is_all_none(xs: Iterable):
    """Whether every item is None."""
    return all(x is None for x in xs)


def _npy_save(path, tensor):
    os.makedirs(os.path.dirname(path), exist_ok=True)
    np.save(path, tensor.detach().cpu().numpy().astype('float32'))


def _npy_load(path, device='cpu'):
    return torch.from_numpy(np.load(path)).to(device)


def _all_none(items: Iterable):
    return all(item is None for item in items)


def _is_zero(t: Tensor):
    return not bool(torch.any(t != 0))


def _merge(a: Optional[Tensor], b: Optional[Tensor], inplace: bool):
    if b is None:
        return a
    if a is None:
        return b
    if inplace:
        a.add_(b)
        return a
    return a + b


def swift_gram(x: Tensor) -> Tensor:
    """The square matrix a "swift" factor stands for: a wide n x d factor x (n < d) represents
    ``x^T x / n`` (the Woodbury inverse in :func:`asdl_b200.utils.smw_inv` is the inverse of exactly that
    plus damping); a square factor is itself."""
    return x if x.shape[0] == x.shape[1] else x.T @ x / x.shape[0]


def _merge_factor(a: Optional[Tensor], b: Optional[Tensor], inplace: bool):
    """Sum of two Kronecker factors; wide swift factors of different batches cannot be added as they
    are, so a sum involving one is formed from the square matrices they stand for."""
    if a is None or b is None or (a.shape[0] == a.shape[1] and b.shape[0] == b.shape[1]):
        return _merge(a, b, inplace)
    a, b = swift_gram(a), swift_gram(b)
    return a.add_(b) if inplace and a.shape == b.shape and a.shape[0] == a.shape[1] and a.is_leaf else a + b


# ----------------------------------------------------------------------------------------------
# containers
# ----------------------------------------------------------------------------------------------
class Kron:
    """Kronecker-factored block ``A (x) B`` of one layer: A over inputs, B over outputs.  A factor
    may also be a raw "swift" n x d sample matrix (n < d), inverted by Woodbury."""

    def __init__(self, A, B, A_inv=None, B_inv=None):
        self.A, self.B, self.A_inv, self.B_inv = A, B, A_inv, B_inv

    # presence ---------------------------------------------------------------------------------
    @property
    def data(self):
        return [self.A, self.B]

    @property
    def has_A(self):
        return self.A is not None

    @property
    def has_B(self):
        return self.B is not None

    @property
    def has_data(self):
        return self.has_A or self.has_B

    @property
    def has_inv(self):
        return self.A_inv is not None and self.B_inv is not None

    def _dim(self, name):
        for t in (getattr(self, name), getattr(self, name + '_inv')):
            if t is not None:
                return t.shape[-1]
        raise ValueError(f'{name} nor {name}_inv has not been set.')

    @property
    def A_dim(self):
        return self._dim('A')

    @property
    def B_dim(self):
        return self._dim('B')

    @property
    def A_is_square(self):
        return self.A.shape[0] == self.A.shape[1]

    @property
    def B_is_square(self):
        return self.B.shape[0] == self.B.shape[1]

    # algebra ----------------------------------------------------------------------------------
    def __add__(self, other):  # inverses are dropped
        if not other.has_data:
            return self
        return Kron(_merge_factor(self.A, other.A, False), _merge_factor(self.B, other.B, False))

    def __iadd__(self, other):
        if other.has_data:
            self.A = _merge_factor(self.A, other.A, True)
            self.B = _merge_factor(self.B, other.B, True)
        return self

    def mul_(self, value):
        for t in (self.A, self.B):
            if t is not None:
                # a wide swift factor x stands for x^T x / n: scaling that by v scales x by sqrt(v)
                t.mul_(value if t.shape[0] == t.shape[1] else math.sqrt(value))
        return self

    def eigenvalues(self):
        eig = torch.outer(_eigvalsh(self.A), _eigvalsh(self.B)).flatten()
        return torch.sort(eig, descending=True)[0]

    def top_eigenvalue(self):
        return (_eigvalsh(self.A).max() * _eigvalsh(self.B).max()).item()

    def trace(self):
        return torch.diag(self.A).sum().item() * torch.diag(self.B).sum().item()

    # persistence ------------------------------------------------------------------------------
    def save(self, root, relative_dir):
        paths = {}
        for name in ('A', 'B'):
            mat = getattr(self, name)
            if mat is None:
                continue
            rel = os.path.join(relative_dir, 'kron', f'{name}_tril.npy')
            _npy_save(os.path.join(root, rel), matrix_to_tril(mat))
            paths[f'{name}_tril'] = rel
        return paths

    def load(self, A_path, B_path, device):
        self.A = tril_to_matrix(_npy_load(A_path, device))
        self.B = tril_to_matrix(_npy_load(B_path, device))

    def to_matrices(self, unflatten, pointer):
        pointer = unflatten(self.A, pointer)
        return unflatten(self.B, pointer)

    def tensors(self) -> Dict[str, Tensor]:
        return {k: getattr(self, k) for k in ('A', 'B', 'A_inv', 'B_inv')
                if getattr(self, k) is not None}

    def load_tensors(self, tensors: Dict[str, Tensor]):
        for k in ('A', 'B', 'A_inv', 'B_inv'):
            if k in tensors:
                setattr(self, k, tensors[k])

    # inverse / products -----------------------------------------------------------------------
    def damping_split(self, damping, eps=1e-7):
        """pi-corrected split of the damping between the two factors:
        pi = sqrt((tr A / dim A) / (tr B / dim B)); A gets sqrt(damping)*pi, B sqrt(damping)/pi."""
        if not (self.has_A and self.has_B):
            return damping, damping

        def mean_eig(mat):  # a wide swift factor x stands for x^T x / n
            total = mat.trace() if mat.shape[0] == mat.shape[1] else (mat ** 2).sum() / mat.shape[0]
            return total / mat.shape[-1]

        pi = float(torch.sqrt(mean_eig(self.A) / mean_eig(self.B)))
        if pi == 0 or math.isinf(pi) or math.isnan(pi):
            return damping, damping
        root = damping ** 0.5
        return max(root * pi, eps), max(root / pi, eps)

    def update_inv(self, damping=_default_damping, calc_A_inv=True, calc_B_inv=True, eps=1e-7,
                   replace=False):
        if not self.has_data:
            raise ValueError('data do not exist.')
        damping_A, damping_B = self.damping_split(damping, eps)
        for name, wanted, damp in (('A', calc_A_inv, damping_A), ('B', calc_B_inv, damping_B)):
            if not wanted:
                continue
            mat = getattr(self, name)
            if mat is None:
                raise ValueError(f'{name} does not exist.')
            if _is_zero(mat):
                continue
            if mat.shape[0] == mat.shape[1]:
                inv = ops.spd_inverse(mat, damp)
            else:
                inv = smw_inv(mat, damp)
            setattr(self, name + '_inv', inv)
            if replace:
                setattr(self, name, None)

    def mvp(self, vec_weight, vec_bias=None, use_inv=False, inplace=False):
        """``B . W2d . A`` on the weight (viewed d_out x -1) and ``B . b`` on the bias."""
        left = self.B_inv if use_inv else self.B
        right = self.A_inv if use_inv else self.A
        w2d = vec_weight.reshape(self.B_dim, -1)
        mvp_w = ops.kron_apply(left, w2d, right).view_as(vec_weight)
        if inplace:
            vec_weight.copy_(mvp_w)
        if vec_bias is None:
            return mvp_w
        mvp_b = torch.mv(left.to(vec_bias.dtype), vec_bias)
        if inplace:
            vec_bias.copy_(mvp_b)
        return mvp_w, mvp_b


class KFE:
    """Kronecker-factored eigenbasis: rotate by (Ub, Ua), divide by the second-moment ``scale``
    in that basis, rotate back.  There is no explicit inverse."""

    def __init__(self, Ua: Tensor, Ub: Tensor, scale: Tuple[Tensor]):
        self.Ua, self.Ub, self.scale = Ua, Ub, scale

    @property
    def has_Ua(self):
        return self.Ua is not None

    @property
    def has_Ub(self):
        return self.Ub is not None

    @property
    def has_scale(self):
        return self.scale is not None

    @property
    def has_inv(self):
        return False

    def update_inv(self, *args, **kwargs):
        pass

    def __add__(self, other):
        raise NotImplementedError

    def __iadd__(self, other):  # only the scales accumulate; bases are kept
        if other.has_scale:
            if self.has_scale:
                for mine, theirs in zip(self.scale, other.scale):
                    mine.add_(theirs)
            else:
                self.scale = other.scale
        return self

    def mul_(self, value):
        if self.has_scale:
            for s in self.scale:
                s.mul_(value)
        return self

    def tensors(self):
        out = {}
        if self.has_Ua:
            out['Ua'] = self.Ua
        if self.has_Ub:
            out['Ub'] = self.Ub
        if self.has_scale:
            for i, s in enumerate(self.scale):
                out[f'scale{i}'] = s
        return out

    def load_tensors(self, tensors):
        self.Ua = tensors.get('Ua', self.Ua)
        self.Ub = tensors.get('Ub', self.Ub)
        scales = [tensors[k] for k in sorted(k for k in tensors if k.startswith('scale'))]
        if scales:
            self.scale = tuple(scales)

    def mvp(self, vec_weight, vec_bias=None, use_inv=False, inplace=False, eps=1.e-7):
        """Applies ``(Ub (x) Ua) diag(1/(scale+eps)) (Ub (x) Ua)^T`` to the gradient.

        The eigenbases hold eigenvectors in their columns, so going *into* the basis multiplies
        by ``Ub^T`` on the left and ``Ua`` on the right, and coming back uses the transposes.
        (``use_inv`` is accepted for interface symmetry: the KFE product already is the
        preconditioning step.)"""
        Ua, Ub = self.Ua, self.Ub
        w2d = vec_weight.reshape(Ub.shape[0], -1)
        rotated = Ub.T.mm(w2d).mm(Ua) / (self.scale[0] + eps)
        mvp_w = Ub.mm(rotated).mm(Ua.T).view_as(vec_weight)
        if inplace:
            vec_weight.copy_(mvp_w)
        if vec_bias is None:
            return mvp_w
        mvp_b = Ub.mv(Ub.T.mv(vec_bias) / (self.scale[1] + eps))
        if inplace:
            vec_bias.copy_(mvp_b)
        return mvp_w, mvp_b


class UnitWise:
    """One small block per output unit: ``f x 2 x 2`` for normalisation layers (scale, shift),
    ``f_out x (f_in+1) x (f_in+1)`` for Linear/Conv2d with bias."""

    def __init__(self, data=None, inv=None):
        self.data = data.contiguous() if isinstance(data, Tensor) else data
        self.inv = inv

    @property
    def has_data(self):
        return self.data is not None

    @property
    def has_inv(self):
        return self.inv is not None

    def __add__(self, other):
        if not other.has_data:
            return self
        return UnitWise(data=_merge(self.data, other.data, False))

    def __iadd__(self, other):
        if other.has_data:
            self.data = _merge(self.data, other.data, True)
        return self

    def mul_(self, value):
        if self.has_data:
            self.data.mul_(value)
        return self

    def eigenvalues(self):
        if not self.has_data:
            raise ValueError('data do not exist.')
        return torch.sort(_eigvalsh(self.data).flatten(), descending=True)[0]

    def top_eigenvalue(self):
        return _eigvalsh(self.data).max().item()

    def trace(self):
        return torch.diagonal(self.data, dim1=-2, dim2=-1).sum().item()

    def save(self, root, relative_dir):
        rel = os.path.join(relative_dir, 'unit_wise.npy')
        _npy_save(os.path.join(root, rel), self.data)
        return rel

    def load(self, path=None, device='cpu'):
        if path:
            self.data = _npy_load(path, device)

    def to_matrices(self, unflatten, pointer):
        return unflatten(self.data, pointer) if self.has_data else pointer

    def tensors(self):
        return {k: getattr(self, k) for k in ('data', 'inv') if getattr(self, k) is not None}

    def load_tensors(self, tensors):
        for k in ('data', 'inv'):
            if k in tensors:
                setattr(self, k, tensors[k])

    def update_inv(self, damping=_default_damping, replace=False):
        if not self.has_data:
            raise ValueError('data do not exist.')
        if _is_zero(self.data):
            return
        self.inv = ops.unitwise_inverse(self.data, damping)
        if replace:
            self.data = None

    def mvp(self, vec_weight, vec_bias, use_inv=False, inplace=False):
        mat = self.inv if use_inv else self.data
        if vec_weight.shape == vec_bias.shape:  # normalisation layers: f x 2 x 2 blocks
            stacked = torch.stack([vec_weight.flatten(), vec_bias.flatten()], dim=1)
            prod = torch.einsum('fij,fj->fi', mat, stacked)
            mvp_w = prod[:, 0].view_as(vec_weight)
            mvp_b = prod[:, 1].view_as(vec_bias)
        else:  # f_out x (f_in+1) x (f_in+1): weight row with the bias appended
            w2d = vec_weight.reshape(vec_weight.shape[0], -1)
            stacked = torch.cat([w2d, vec_bias.unsqueeze(1)], dim=1)
            prod = torch.einsum('fij,fj->fi', mat, stacked)
            mvp_w = prod[:, :-1].reshape(vec_weight.shape)
            mvp_b = prod[:, -1]
        if inplace:
            vec_weight.copy_(mvp_w)
            vec_bias.copy_(mvp_b)
        return mvp_w, mvp_b


class Diag:
    """Diagonal curvature of the weight and bias."""

    def __init__(self, weight=None, bias=None, weight_inv=None, bias_inv=None):
        self.weight, self.bias = weight, bias
        self.weight_inv, self.bias_inv = weight_inv, bias_inv

    @property
    def data(self):
        return [t for t in (self.weight, self.bias) if t is not None]

    @property
    def has_weight(self):
        return self.weight is not None

    @property
    def has_bias(self):
        return self.bias is not None

    @property
    def has_inv(self):
        ok = self.weight_inv is not None
        if self.has_bias:
            ok = ok and self.bias_inv is not None
        return ok

    def __add__(self, other):
        return Diag(weight=_merge(self.weight, other.weight, False),
                    bias=_merge(self.bias, other.bias, False))

    def __iadd__(self, other):
        self.weight = _merge(self.weight, other.weight, True)
        self.bias = _merge(self.bias, other.bias, True)
        return self

    def mul_(self, value):
        for t in self.data:
            t.mul_(value)
        return self

    def eigenvalues(self):
        return torch.sort(torch.cat([t.flatten() for t in self.data]), descending=True)[0]

    def top_eigenvalue(self):
        return max([-1] + [t.max().item() for t in self.data])

    def trace(self):
        return sum(t.sum().item() for t in self.data)

    def save(self, root, relative_dir):
        paths = {}
        for name in ('weight', 'bias'):
            t = getattr(self, name)
            if t is None:
                continue
            rel = os.path.join(relative_dir, 'diag', f'{name}.npy')
            _npy_save(os.path.join(root, rel), t)
            paths[name] = rel
        return paths

    def load(self, w_path=None, b_path=None, device='cpu'):
        if w_path:
            self.weight = _npy_load(w_path, device)
        if b_path:
            self.bias = _npy_load(b_path, device)

    def to_matrices(self, unflatten, pointer):
        for t in self.data:
            pointer = unflatten(t, pointer)
        return pointer

    def tensors(self):
        return {k: getattr(self, k) for k in ('weight', 'bias', 'weight_inv', 'bias_inv')
                if getattr(self, k) is not None}

    def load_tensors(self, tensors):
        for k in ('weight', 'bias', 'weight_inv', 'bias_inv'):
            if k in tensors:
                setattr(self, k, tensors[k])

    def update_inv(self, damping=_default_damping, replace=False):
        for name in ('weight', 'bias'):
            t = getattr(self, name)
            if t is None or _is_zero(t):
                continue
            setattr(self, name + '_inv', 1 / (t + damping))
            if replace:
                setattr(self, name, None)

    def mvp(self, vec_weight=None, vec_bias=None, use_inv=False, inplace=False):
        if vec_weight is None and vec_bias is None:
            raise ValueError('Either vec_weight or vec_bias has to be set.')
        out = []
        for vec, name in ((vec_weight, 'weight'), (vec_bias, 'bias')):
            if vec is None:
                continue
            mat = getattr(self, name + '_inv' if use_inv else name)
            out.append(vec.mul_(mat) if inplace else vec.mul(mat))
        return out


class SymMatrix:
    """Curvature of one module (or of the whole model): an optional dense block plus optional
    Kronecker / eigenbasis / unit-wise / diagonal representations."""

    _parts = ('data', 'kron', 'kfe', 'diag', 'unit')

    def __init__(self, data=None, inv=None, kron=None, kfe=None, diag=None, unit=None,
                 kron_A=None, kron_B=None, kron_A_inv=None, kron_B_inv=None,
                 kfe_A=None, kfe_B=None, kfe_scale=None,
                 unit_data=None, unit_inv=None,
                 diag_weight=None, diag_bias=None, diag_weight_inv=None, diag_bias_inv=None):
        self.data: Tensor = data
        self.inv: Tensor = inv
        self.kron: Kron = kron
        self.kfe: KFE = kfe
        self.unit: UnitWise = unit
        self.diag: Diag = diag
        if not _all_none([kron_A, kron_B, kron_A_inv, kron_B_inv]):
            self.kron = Kron(kron_A, kron_B, kron_A_inv, kron_B_inv)
        if not _all_none([kfe_A, kfe_B, kfe_scale]):
            self.kfe = KFE(kfe_A, kfe_B, kfe_scale)
        if not _all_none([unit_data, unit_inv]):
            self.unit = UnitWise(unit_data, unit_inv)
        if not _all_none([diag_weight, diag_bias, diag_weight_inv, diag_bias_inv]):
            self.diag = Diag(diag_weight, diag_bias, diag_weight_inv, diag_bias_inv)

    def __repr__(self):
        items = []
        if self.has_data:
            items.append(f'data {tuple(self.data.shape)}')
        if self.has_kron:
            items += [f'kron.{k} {tuple(v.shape)}' for k, v in self.kron.tensors().items()]
        if self.has_kfe:
            items += [f'kfe.{k} {tuple(v.shape)}' for k, v in self.kfe.tensors().items()]
        if self.has_unit:
            items += [f'unit.{k} {tuple(v.shape)}' for k, v in self.unit.tensors().items()]
        if self.has_diag:
            items += [f'diag.{k} {tuple(v.shape)}' for k, v in self.diag.tensors().items()]
        return 'SymMatrix(' + ', '.join(items) + ')'

    @property
    def has_data(self):
        return self.data is not None

    @property
    def has_inv(self):
        return self.inv is not None

    @property
    def has_kron(self):
        return self.kron is not None

    @property
    def has_kfe(self):
        return self.kfe is not None

    @property
    def has_diag(self):
        return self.diag is not None

    @property
    def has_unit(self):
        return self.unit is not None

    # algebra ----------------------------------------------------------------------------------
    def __add__(self, other):  # inverses are not carried over
        merged = {}
        for part in self._parts:
            mine, theirs = getattr(self, part), getattr(other, part)
            if theirs is None:
                merged[part] = mine
            elif mine is None:
                merged[part] = theirs
            else:
                merged[part] = mine + theirs
        return SymMatrix(**merged)

    def __iadd__(self, other):
        for part in self._parts:
            mine, theirs = getattr(self, part), getattr(other, part)
            if theirs is None:
                continue
            if mine is None:
                setattr(self, part, theirs)
            else:
                mine += theirs
        return self

    def mul_(self, value):
        for part in self._parts:
            obj = getattr(self, part)
            if obj is not None:
                obj.mul_(value)
        return self

    def _need_data(self):
        if not self.has_data:
            raise ValueError('data do not exist.')

    def eigenvalues(self):
        self._need_data()
        return torch.sort(_eigvalsh(self.data), descending=True)[0]

    def top_eigenvalue(self):
        self._need_data()
        return _eigvalsh(self.data).max().item()

    def trace(self):
        self._need_data()
        return torch.diag(self.data).sum().item()

    # persistence ------------------------------------------------------------------------------
    def save(self, root, relative_dir):
        paths = {}
        if self.has_data:
            rel = os.path.join(relative_dir, 'tril.npy')
            _npy_save(os.path.join(root, rel), matrix_to_tril(self.data))
            paths['tril'] = rel
        if self.has_kron:
            paths['kron'] = self.kron.save(root, relative_dir)
        if self.has_diag:
            paths['diag'] = self.diag.save(root, relative_dir)
        if self.has_unit:
            paths['unit_wise'] = self.unit.save(root, relative_dir)
        return paths

    def load(self, path=None, kron_path=None, diag_path=None, unit_path=None, device='cpu'):
        if path:
            self.data = tril_to_matrix(_npy_load(path, device))
        if kron_path is not None:
            if not self.has_kron:
                self.kron = Kron(A=None, B=None)
            self.kron.load(A_path=kron_path['A_tril'], B_path=kron_path['B_tril'], device=device)
        if diag_path is not None:
            if not self.has_diag:
                self.diag = Diag()
            self.diag.load(w_path=diag_path.get('weight'), b_path=diag_path.get('bias'), device=device)
        if unit_path is not None:
            if not self.has_unit:
                self.unit = UnitWise()
            self.unit.load(path=unit_path, device=device)

    def tensors(self, prefix='') -> Dict[str, Tensor]:
        """Flat ``{name: tensor}`` view of everything stored (for state dicts)."""
        out = {}
        if self.has_data:
            out[prefix + 'data'] = self.data
        if self.has_inv:
            out[prefix + 'inv'] = self.inv
        for part in ('kron', 'kfe', 'unit', 'diag'):
            obj = getattr(self, part)
            if obj is not None:
                for k, v in obj.tensors().items():
                    out[f'{prefix}{part}.{k}'] = v
        return out

    @classmethod
    def from_tensors(cls, tensors: Dict[str, Tensor]):
        mat = cls()
        grouped: Dict[str, Dict[str, Tensor]] = {}
        for key, value in tensors.items():
            if key in ('data', 'inv'):
                setattr(mat, key, value)
            else:
                part, name = key.split('.', 1)
                grouped.setdefault(part, {})[name] = value
        makers = {'kron': lambda: Kron(None, None), 'kfe': lambda: KFE(None, None, None),
                  'unit': UnitWise, 'diag': Diag}
        for part, items in grouped.items():
            obj = makers[part]()
            obj.load_tensors(items)
            setattr(mat, part, obj)
        return mat

    def to_vector(self):
        parts = []
        if self.has_data:
            parts.append(self.data)
        if self.has_kron:
            parts.extend(self.kron.data)
        if self.has_diag:
            parts.extend(self.diag.data)
        if self.has_unit:
            parts.append(self.unit.data)
        return [p.flatten() for p in parts]

    def to_matrices(self, vec, pointer):
        def unflatten(mat, start):
            stop = start + mat.numel()
            mat.copy_(vec[start:stop].view_as(mat))
            return stop

        if self.has_data:
            pointer = unflatten(self.data, pointer)
        for part in ('kron', 'diag', 'unit'):
            obj = getattr(self, part)
            if obj is not None:
                pointer = obj.to_matrices(unflatten, pointer)
        return pointer

    # inverse / products -----------------------------------------------------------------------
    def update_inv(self, damping=_default_damping, replace=False):
        if self.has_data and not _is_zero(self.data):
            self.inv = ops.spd_inverse(self.data, damping)
            if replace:
                self.data = None
        for part in ('kron', 'diag', 'unit'):
            obj = getattr(self, part)
            if obj is not None:
                obj.update_inv(damping, replace=replace)

    def mvp(self, vectors: ParamVector = None, vec_weight: Tensor = None, vec_bias: Tensor = None,
            use_inv=False, inplace=False):
        """Dense block times a vector.  ``vectors``: whole-model ParamVector (full shape);
        ``vec_weight``/``vec_bias``: one layer's weight-then-bias ordering (layer-wise shape)."""
        mat = self.inv if use_inv else self.data
        if vectors is not None:
            out = ParamVector(vectors.params(), torch.mv(mat, vectors.get_flatten_vector()))
            if inplace:
                for dst, src in zip(vectors.values(), out.values()):
                    dst.copy_(src)
            return out
        if vec_weight is None and vec_bias is None:
            raise ValueError('Either vec_weight or vec_bias has to be set.')
        pieces = [v for v in (vec_weight, vec_bias) if v is not None]
        prod = torch.mv(mat, torch.cat([p.flatten() for p in pieces]))
        outs, start = [], 0
        for p in pieces:
            seg = prod[start:start + p.numel()].view_as(p)
            start += p.numel()
            if inplace:
                p.copy_(seg)
            outs.append(seg)
        return tuple(outs) if len(outs) == 2 else outs
