"""Names of curvature types / shapes and :class:`MatrixManager`, which accumulates, stores,
reduces and analyses the curvature matrices (``module.<matrix_type>``) of a model.

Parity: asdl/matrices.py (constants :10-21, ``MatrixManager`` :52-394).  The reference's
``accumulate_matrices`` calls a method that does not exist on its containers; here accumulation
with an optional scale is implemented with ``mul_``.  The directory layout written by
``save_matrices`` is ``<root>/<relative_dir>/<matrix_type>/<module_name>/...`` with the per-module
files of ``SymMatrix.save``.
"""
import copy
import os
from typing import List

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn

HESSIAN = 'hessian'  # Hessian
FISHER_EXACT = 'fisher_exact'  # exact Fisher
FISHER_MC = 'fisher_mc'  # Fisher estimation by Monte-Carlo sampling
FISHER_EMP = 'fisher_emp'  # empirical Fisher

SHAPE_FULL = 'full'  # full
SHAPE_LAYER_WISE = 'layer_wise'  # layer-wise block-diagonal
SHAPE_KRON = 'kron'  # Kronecker-factored
SHAPE_SWIFT_KRON = 'swift_kron'  # swift Kronecker-factored
SHAPE_KFE = 'kfe'  # Kronecker-factored eigenbasis
SHAPE_UNIT_WISE = 'unit_wise'  # unit-wise block-diagonal
SHAPE_DIAG = 'diag'  # diagonal

__all__ = ['MatrixManager', 'FISHER_EXACT', 'FISHER_MC', 'FISHER_EMP', 'HESSIAN',
           'SHAPE_FULL', 'SHAPE_LAYER_WISE', 'SHAPE_KRON', 'SHAPE_SWIFT_KRON', 'SHAPE_KFE',
           'SHAPE_UNIT_WISE', 'SHAPE_DIAG']

_supported_types = [HESSIAN, FISHER_EXACT, FISHER_MC, FISHER_EMP]
_supported_shapes = [SHAPE_FULL, SHAPE_LAYER_WISE, SHAPE_KRON, SHAPE_SWIFT_KRON, SHAPE_KFE,
                     SHAPE_UNIT_WISE, SHAPE_DIAG]
_normalizations = (nn.BatchNorm1d, nn.BatchNorm2d)


def _check_types(matrix_types):
    if isinstance(matrix_types, str):
        matrix_types = [matrix_types]
    for mt in matrix_types:
        if mt not in _supported_types:
            raise ValueError(f'Invalid matrix_type: {mt}. matrix_type must be in {_supported_types}.')
    return list(matrix_types)


def _requires_matrix(module: nn.Module):
    """Leaf module with at least one trainable parameter."""
    if len(list(module.children())) > 0:
        return False
    return any(p.requires_grad for p in module.parameters())


def _part_for_shape(matrix, shape):
    """The sub-container of a SymMatrix that represents ``shape``."""
    if shape in (SHAPE_FULL, SHAPE_LAYER_WISE):
        return matrix if matrix.has_data else None
    if shape in (SHAPE_KRON, SHAPE_SWIFT_KRON):
        return matrix.kron
    if shape == SHAPE_KFE:
        return matrix.kfe
    if shape == SHAPE_UNIT_WISE:
        return matrix.unit
    if shape == SHAPE_DIAG:
        return matrix.diag
    raise ValueError(f'Invalid matrix_shape: {shape}. matrix_shape must be in {_supported_shapes}.')


class MatrixManager:
    """Bookkeeping for curvature stored as attributes on modules.

    A Fisher/Hessian maker writes the *latest* matrix to ``module.<matrix_type>``;
    ``accumulate_matrices(stats_name)`` folds it into the running statistic
    ``module.<stats_name>_<matrix_type>`` (a plain sum, or an exponential moving average when a
    smoothing weight is set).  With ``stats_name=None`` the latest matrix itself is the statistic
    and accumulation only applies the scale.
    """

    def __init__(self, model, matrix_types, scale=1., smoothing_weight=None):
        self._model = model
        self._device = next(model.parameters()).device
        self._matrix_types = set(_check_types(matrix_types))
        self._scale = scale
        self._smoothing_weight = smoothing_weight
        self._stats_names = set()

    # naming -----------------------------------------------------------------------------------
    @staticmethod
    def _get_save_field(matrix_type, stats_name=None):
        return matrix_type if stats_name is None else f'{stats_name}_{matrix_type}'

    def _check_stats_name(self, stats_name):
        if stats_name is not None and stats_name not in self._stats_names:
            raise ValueError(f'stats {stats_name} does not exist.')

    def _stats(self, module, matrix_type, stats_name=None):
        return getattr(module, self._get_save_field(matrix_type, stats_name), None)

    def get_matrix(self, module, matrix_type, stats_name=None):
        return self._stats(module, matrix_type, stats_name)

    # accumulation -----------------------------------------------------------------------------
    def accumulate_matrices(self, stats_name=None, scale=None, smoothing_weight=None):
        """stats <- stats + scale*new, or stats <- (1-w)*stats + w*scale*new with smoothing
        weight w.  The latest matrix ``module.<matrix_type>`` is scaled in place."""
        self._stats_names.add(stats_name)
        scale = self._scale if scale is None else scale
        w = self._smoothing_weight if smoothing_weight is None else smoothing_weight
        for module in self._model.modules():
            for mt in self._matrix_types:
                new = getattr(module, mt, None)
                if new is None:
                    continue
                if scale != 1:
                    new.mul_(scale)
                if stats_name is None:
                    continue
                attr = self._get_save_field(mt, stats_name)
                stats = getattr(module, attr, None)
                if stats is None:
                    setattr(module, attr, copy.deepcopy(new))
                elif w:
                    stats.mul_(1 - w)
                    stats += copy.deepcopy(new).mul_(w)
                else:
                    stats += new

    def clear_matrices(self, stats_name):
        self._check_stats_name(stats_name)
        for mt in self._matrix_types:
            attr = self._get_save_field(mt, stats_name)
            for module in self._model.modules():
                if hasattr(module, attr):
                    delattr(module, attr)
        self._stats_names.discard(stats_name)

    # persistence ------------------------------------------------------------------------------
    def save_matrices(self, root, relative_dir='', stats_name=None):
        """Writes every statistic as npy-tril files under
        ``<root>/<relative_dir>/<matrix_type>/<module_name>/`` and returns the nested dict of
        relative paths ``{matrix_type: {module_name: {...}}}`` (entries of the root module sit
        directly under the matrix type)."""
        self._check_stats_name(stats_name)
        paths = {}
        for mt in self._matrix_types:
            per_type = paths[mt] = {}
            for name, module in self._model.named_modules():
                stats = self._stats(module, mt, stats_name)
                if stats is None:
                    continue
                saved = stats.save(root, os.path.join(relative_dir, mt, name))
                if module is self._model:
                    per_type.update(saved)
                else:
                    per_type[name] = saved
        return paths

    def load_matrices(self, root, relative_paths, matrix_shapes):
        """Rebuilds ``module.<matrix_type>`` for the requested shapes from a ``save_matrices``
        path dict.  Raises ValueError when a requested piece is missing."""
        from .symmatrix import SymMatrix
        for shape in matrix_shapes:
            if shape not in _supported_shapes:
                raise ValueError(f'Invalid matrix_shape: {shape}. {_supported_shapes} are supported.')

        def absolute(value):
            if isinstance(value, dict):
                return {k: absolute(v) for k, v in value.items()}
            return os.path.join(root, value)

        paths = absolute(relative_paths)
        for mt in self._matrix_types:
            per_type = paths.get(mt)
            if per_type is None:
                raise ValueError(f'matrix type {mt} does not exist.')

            def load_piece(matrix, shape, load_key, path_key, module_name=None):
                try:
                    entry = per_type[module_name] if module_name else per_type
                    matrix.load(**{load_key: entry[path_key]}, device=self._device)
                except (KeyError, FileNotFoundError):
                    where = f' for module {module_name}' if module_name else ''
                    raise ValueError(f'{mt}.{shape}{where} does not exist.')

            for name, module in self._model.named_modules():
                if module is self._model or not _requires_matrix(module):
                    continue
                matrix = SymMatrix()
                if SHAPE_LAYER_WISE in matrix_shapes:
                    load_piece(matrix, SHAPE_LAYER_WISE, 'path', 'tril', name)
                if SHAPE_KRON in matrix_shapes:
                    if isinstance(module, _normalizations):
                        load_piece(matrix, SHAPE_UNIT_WISE, 'unit_path', 'unit_wise', name)
                    else:
                        load_piece(matrix, SHAPE_KRON, 'kron_path', 'kron', name)
                if SHAPE_UNIT_WISE in matrix_shapes:
                    load_piece(matrix, SHAPE_UNIT_WISE, 'unit_path', 'unit_wise', name)
                if SHAPE_DIAG in matrix_shapes:
                    load_piece(matrix, SHAPE_DIAG, 'diag_path', 'diag', name)
                setattr(module, mt, matrix)
            if SHAPE_FULL in matrix_shapes:
                matrix = SymMatrix()
                load_piece(matrix, SHAPE_FULL, 'path', 'tril')
                setattr(self._model, mt, matrix)

    def matrices_exist(self, root, relative_paths, matrix_shapes):
        try:
            self.load_matrices(root, relative_paths, matrix_shapes)
            return True
        except ValueError:
            return False

    # collectives ------------------------------------------------------------------------------
    def matrices_to_vector(self, stats_name):
        self._check_stats_name(stats_name)
        parts = []
        for mt in self._matrix_types:
            for module in self._model.modules():
                stats = self._stats(module, mt, stats_name)
                if stats is not None:
                    parts.extend(stats.to_vector())
        return torch.cat(parts) if parts else torch.zeros(0, device=self._device)

    def vector_to_matrices(self, vec, stats_name):
        self._check_stats_name(stats_name)
        pointer = 0
        for mt in self._matrix_types:
            for module in self._model.modules():
                stats = self._stats(module, mt, stats_name)
                if stats is not None:
                    pointer = stats.to_matrices(vec, pointer)
        if pointer != vec.numel():
            raise ValueError(f'pointer has to be {vec.numel()}. Got {pointer}.')

    def reduce_matrices(self, stats_name=None, is_master=True, all_reduce=False):
        """Average the statistics over ranks with one flat message, unpacked in place."""
        packed = self.matrices_to_vector(stats_name)
        if all_reduce:
            dist.all_reduce(packed)
        else:
            dist.reduce(packed, dst=0)
        if all_reduce or is_master:
            self.vector_to_matrices(packed.div_(dist.get_world_size()), stats_name)
        dist.barrier()

    # spectra ----------------------------------------------------------------------------------
    def _collect_metrics(self, matrix_type, matrix_shape, stats_name, metrics_fn):
        self._check_stats_name(stats_name)
        if matrix_shape == SHAPE_FULL:
            stats = self._stats(self._model, matrix_type, stats_name)
            part = None if stats is None else _part_for_shape(stats, matrix_shape)
            return [] if part is None else [metrics_fn(part)]
        out = []
        for module in self._model.modules():
            if module is self._model and len(list(module.children())) > 0:
                continue
            stats = self._stats(module, matrix_type, stats_name)
            if stats is None:
                continue
            shape = matrix_shape
            if isinstance(module, _normalizations) and matrix_shape in (SHAPE_KRON, SHAPE_SWIFT_KRON):
                shape = SHAPE_UNIT_WISE
            part = _part_for_shape(stats, shape)
            if part is not None:
                out.append(metrics_fn(part))
        return out

    def get_eigenvalues(self, matrix_type, matrix_shape, stats_name=None):
        eigs = self._collect_metrics(matrix_type, matrix_shape, stats_name, lambda p: p.eigenvalues())
        if not eigs:
            return torch.zeros(0, device=self._device)
        return torch.sort(torch.cat(eigs), descending=True)[0]

    def get_top_eigenvalue(self, matrix_type, matrix_shape, stats_name=None):
        tops = self._collect_metrics(matrix_type, matrix_shape, stats_name, lambda p: p.top_eigenvalue())
        return max(tops) if tops else None

    def get_trace(self, matrix_type, matrix_shape, stats_name=None):
        return sum(self._collect_metrics(matrix_type, matrix_shape, stats_name, lambda p: p.trace()))

    def get_effective_dim(self, matrix_type, matrix_shape, reg, stats_name=None):
        """sum_i lambda_i / (lambda_i + reg)."""
        eigs = self.get_eigenvalues(matrix_type, matrix_shape, stats_name)
        return float(torch.sum(eigs / (eigs + reg)))
