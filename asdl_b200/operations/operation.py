"""Per-module curvature "operations" and the context that owns them.

An :class:`Operation` is attached to one ``nn.Module`` for the lifetime of an ``extend`` context.
It is told which statistics (``OP_*`` names) to produce, receives the layer input / output in the
forward hook and the output-gradient in the backward hook, and stores results in a nested dict.
Layer subclasses (``Linear``, ``Conv2d``, ...) only implement the primitives (how to turn ``a``/``g``
into Kronecker factors, per-example gradients, diagonals, Gram matrices ...); the bookkeeping is
shared here.

Parity: asdl/operations/operation.py (op-name registry :12-84, ``Operation`` :87-548,
``OperationContext`` :551-964).  Results live under the same keys as in the reference, e.g.
``['cov_kron']['A']``; swift-Kron results are stored under ``'cov_kron'`` as well.
Implementation differences: dispatch is table driven (``_FWD_HANDLERS`` / ``_BWD_HANDLERS``)
instead of a chain of ``if``; the pi-damping split is evaluated without mutating the factors; the
Kronecker factor GEMMs are issued through :mod:`asdl_b200.ops` (tcgen05 SYRK on CUDA tensors).
"""
from typing import Dict, List, Tuple

import math

import torch
import torch.nn as nn

from .. import ops
from ..utils import original_requires_grad, cholesky_inv, smw_inv, nvtx_range
from ..symmatrix import SymMatrix
from ..vector import ParamVector

# compute first and second-order derivative
OP_FULL_COV = 'full_cov'  # full covariance
OP_FULL_CVP = 'full_cvp'  # full covariance-vector product
OP_COV = 'cov'  # layer-wise covariance
OP_COV_INV = 'cov_inv'  # layer-wise covariance inverse
OP_CVP = 'cvp'  # layer-wise covariance-vector product
OP_COV_KRON = 'cov_kron'  # Kronecker-factored covariance
OP_COV_KRON_INV = 'cov_kron_inv'  # Kronecker-factored covariance inverse
OP_COV_SWIFT_KRON = 'cov_swift_kron'  # swift Kronecker-factored covariance
OP_COV_SWIFT_KRON_INV = 'cov_swift_kron_inv'  # swift Kronecker-factored covariance inverse
OP_COV_KFE = 'cov_kfe'  # Kronecker-factored covariance eigenbasis
OP_COV_UNIT_WISE = 'cov_unit_wise'  # unit-wise covariance
OP_COV_UNIT_WISE_INV = 'cov_unit_wise_inv'  # unit-wise covariance inverse
OP_COV_DIAG = 'cov_diag'  # diagonal covariance
OP_COV_DIAG_INV = 'cov_diag_inv'  # diagonal covariance inverse
OP_RFIM_RELU = 'rfim_relu'  # relative FIM for ReLU
OP_RFIM_SOFTMAX = 'rfim_softmax'  # relative FIM for softmax
OP_GRAM_DIRECT = 'gram_direct'  # direct Gram matrix
OP_GRAM_HADAMARD = 'gram_hada'  # Hadamard-factored Gram matrix
OP_BATCH_GRADS = 'batch_grads'  # per-example gradients
OP_SAVE_INPUTS = 'save_inputs'
OP_SAVE_OUTPUTS = 'save_outputs'
OP_SAVE_OUTGRADS = 'save_outgrads'
OP_MEAN_INPUTS = 'mean_inputs'
OP_MEAN_OUTPUTS = 'mean_outputs'
OP_SPATIAL_MEAN_OUTPUTS = 'spatial_mean_outputs'
OP_OUT_SPATIAL_SIZE = 'out_spatial_size'
OP_MEAN_OUTGRADS = 'mean_outgrads'
OP_SPATIAL_MEAN_OUTGRADS = 'spatial_mean_outgrads'
OP_SKETCHED_GRAM = 'sketched_gram'
OP_BFGS_KRON_S_AS = 'bfgs_kron_s_As'

ALL_OPS = [OP_FULL_COV, OP_FULL_CVP, OP_COV, OP_COV_INV, OP_CVP,
           OP_COV_KRON, OP_COV_KRON_INV, OP_COV_SWIFT_KRON, OP_COV_SWIFT_KRON_INV,
           OP_COV_KFE, OP_COV_UNIT_WISE, OP_COV_UNIT_WISE_INV, OP_COV_DIAG, OP_COV_DIAG_INV,
           OP_RFIM_RELU, OP_RFIM_SOFTMAX, OP_GRAM_DIRECT, OP_GRAM_HADAMARD, OP_BATCH_GRADS,
           OP_SAVE_INPUTS, OP_SAVE_OUTPUTS, OP_SAVE_OUTGRADS,
           OP_MEAN_INPUTS, OP_MEAN_OUTPUTS, OP_SPATIAL_MEAN_OUTPUTS, OP_OUT_SPATIAL_SIZE,
           OP_MEAN_OUTGRADS, OP_SPATIAL_MEAN_OUTGRADS, OP_SKETCHED_GRAM, OP_BFGS_KRON_S_AS]

# statistics that are complete after the forward pass
FWD_OPS = [OP_SAVE_INPUTS, OP_SAVE_OUTPUTS, OP_COV_KRON, OP_COV_SWIFT_KRON,
           OP_RFIM_RELU, OP_RFIM_SOFTMAX, OP_MEAN_INPUTS, OP_MEAN_OUTPUTS,
           OP_SPATIAL_MEAN_OUTPUTS, OP_OUT_SPATIAL_SIZE, OP_BFGS_KRON_S_AS]
# statistics evaluated in the backward pass that also need the layer input
BWD_OPS_WITH_INPUTS = [OP_COV, OP_COV_INV, OP_CVP, OP_COV_KRON_INV, OP_COV_SWIFT_KRON_INV,
                       OP_COV_KFE, OP_COV_UNIT_WISE, OP_COV_UNIT_WISE_INV,
                       OP_COV_DIAG, OP_COV_DIAG_INV, OP_GRAM_HADAMARD, OP_GRAM_DIRECT,
                       OP_BATCH_GRADS, OP_SKETCHED_GRAM]
# everything that needs the backward pass
BWD_OPS = [OP_SAVE_OUTGRADS, OP_COV_KRON, OP_COV_SWIFT_KRON, OP_RFIM_RELU, OP_RFIM_SOFTMAX,
           OP_MEAN_OUTGRADS, OP_SPATIAL_MEAN_OUTGRADS] + BWD_OPS_WITH_INPUTS
# what every layer type supports: saved tensors and means, and everything that follows from per-example
# gradients alone (layer-wise blocks and their inverses, matrix-free products, the model-wide matrix, Gram rows)
BASIC_OPS = [OP_SAVE_INPUTS, OP_SAVE_OUTPUTS, OP_SAVE_OUTGRADS,
             OP_MEAN_INPUTS, OP_MEAN_OUTPUTS, OP_SPATIAL_MEAN_OUTPUTS, OP_OUT_SPATIAL_SIZE,
             OP_MEAN_OUTGRADS, OP_SPATIAL_MEAN_OUTGRADS,
             OP_FULL_COV, OP_FULL_CVP, OP_COV, OP_COV_INV, OP_CVP, OP_GRAM_DIRECT]

# local copies of the shape names (the canonical definitions live in asdl_b200.matrices)
SHAPE_FULL = 'full'
SHAPE_LAYER_WISE = 'layer_wise'
SHAPE_KRON = 'kron'
SHAPE_SWIFT_KRON = 'swift_kron'
SHAPE_KFE = 'kfe'
SHAPE_UNIT_WISE = 'unit_wise'
SHAPE_DIAG = 'diag'
HESSIAN = 'hessian'
FISHER_EXACT = 'fisher_exact'
FISHER_MC = 'fisher_mc'
FISHER_EMP = 'fisher_emp'

__all__ = ['Operation', 'OperationContext', 'ALL_OPS', 'FWD_OPS', 'BWD_OPS', 'BWD_OPS_WITH_INPUTS',
           'BASIC_OPS'] + [name for name in list(globals()) if name.startswith('OP_')]


def _is_norm_layer(module):
    return isinstance(module, (nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d, nn.LayerNorm))


class Operation:
    """Statistics extractor bound to one module.  Subclasses provide the primitives."""
    supported_operations = set(ALL_OPS)

    def __init__(self, module, op_names, model_for_kernel=None):
        weight = getattr(module, 'weight', None)
        if weight is not None:
            bias = getattr(module, 'bias', None)
            if not (weight.requires_grad or (bias is not None and bias.requires_grad)):
                raise ValueError(f'One of weight or bias has to require grad (module: {module}).')
        if isinstance(op_names, str):
            op_names = [op_names]
        if not isinstance(op_names, list):
            raise TypeError(f'op_names has to be a list. Got {type(op_names)}.')
        names = set(op_names)
        unknown = names - set(ALL_OPS)
        if unknown:
            raise ValueError(f'Invalid operation name: {sorted(unknown)}. {ALL_OPS} are supported.')
        if names & set(BWD_OPS_WITH_INPUTS):
            names |= {OP_SAVE_INPUTS, OP_SAVE_OUTPUTS}
        self._module = module
        self._model_for_kernel = model_for_kernel
        self._op_names = names
        self._op_results = {}
        self._bwd_calls = 0           # backward hook calls so far (pairs each one with its forward call)
        self._kron_inv_sums = None    # (A, B) behind the hook-time inverses, for layers applied more than once
        self._damping = 1.e-7
        self._cov_scale = 1.
        self._sketching_size = 256
        self._truncated_rank = None

    # ------------------------------------------------------------------ result store
    def _walk(self, keys, create):
        node = self._op_results
        for key in keys:
            nxt = node.get(key)
            if nxt is None:
                if not create:
                    return None
                nxt = node[key] = {}
            node = nxt
        return node

    def accumulate_result(self, value, *keys, extend=False):
        """First call stores, later calls add in place (or extend a list).
        ``accumulate_result(A, OP_COV_KRON, 'A')`` -> ``results['cov_kron']['A']``."""
        node = self._walk(keys[:-1], create=True)
        leaf = keys[-1]
        if node.get(leaf) is None:
            node[leaf] = value
        elif extend:
            node[leaf].extend(value)
        else:
            node[leaf] += value

    def get_result(self, *keys, pop=False, default=None):
        node = self._walk(keys[:-1], create=False)
        if node is None:
            return None
        return node.pop(keys[-1], default) if pop else node.get(keys[-1], default)

    def clear_result(self, *keys):
        node = self._walk(keys[:-1], create=False)
        if node is not None:
            node.pop(keys[-1], None)

    def clear_results(self):
        self._op_results = {}
        self._bwd_calls = 0
        self._kron_inv_sums = None

    # ------------------------------------------------------------------ knobs
    def add_op_name(self, op_name):
        self._op_names.add(op_name)

    def remove_op_name(self, op_name):
        self._op_names.discard(op_name)

    def set_damping(self, value):
        self._damping = value

    def set_cov_scale(self, value):
        self._cov_scale = value

    def set_sketching_size(self, value):
        self._sketching_size = value

    def set_truncated_rank(self, value):
        self._truncated_rank = value

    # ------------------------------------------------------------------ forward
    def forward_post_process(self, in_data: torch.Tensor, out_data: torch.Tensor):
        names = self._op_names
        if OP_SAVE_INPUTS in names:
            self.accumulate_result([in_data], OP_SAVE_INPUTS, extend=True)
        if OP_SAVE_OUTPUTS in names:
            self.accumulate_result([out_data], OP_SAVE_OUTPUTS, extend=True)
        todo = [n for n in names if n in _FWD_HANDLERS]
        if not todo:
            return
        a = self.preprocess_in_data(self._module, in_data, out_data)
        a32 = out32 = None
        for name in todo:
            with nvtx_range(_RANGE_NAMES_FWD.get(name, name)):
                if name in _HALF_PRECISION_OK:
                    _FWD_HANDLERS[name](self, a, out_data)
                else:   # everything but the Gram products computes in fp32 (activations may be bf16 under autocast)
                    a32 = _as_fp32(a) if a32 is None else a32
                    out32 = _as_fp32(out_data) if out32 is None else out32
                    _FWD_HANDLERS[name](self, a32, out32)

    def _fwd_kron(self, a, out_data):
        self.accumulate_result(self.cov_kron_A(self._module, a).mul_(self._cov_scale), OP_COV_KRON, 'A')

    def _fwd_swift_kron(self, a, out_data):
        self._accumulate_swift(self.cov_swift_kron_A(self._module, a), 'A')

    def _accumulate_swift(self, mat, key):
        """A swift factor is either the square statistic or, with fewer samples than features, the raw
        n x d matrix x itself, which stands for ``x^T x / n`` (what ``smw_inv`` inverts).  A raw factor is
        stored as ``x * sqrt(cov_scale * n)`` so that it stands for ``cov_scale * x^T x``, out of place
        (x is the layer input or the output gradient that autograd still uses).  Anything that has to be
        added to an existing entry (moving averages, several backward passes) is added as the square
        matrix it stands for: raw matrices of different passes have no meaningful sum."""
        scale = self._cov_scale
        node = self._walk((OP_COV_KRON,), create=True)
        old = node.get(key)
        raw = mat.shape[0] != mat.shape[1]
        if old is None:
            node[key] = mat * (math.sqrt(scale * mat.shape[0]) if raw else scale)
            return
        new = (mat.T @ mat if raw else mat) * scale
        if old.shape[0] == old.shape[1]:
            old += new          # in place: a registered accumulator keeps its identity
        else:
            node[key] = old.T @ old / old.shape[0] + new

    def _fwd_simple(name, fn_name, needs_out):  # noqa: N805  (builder, not a method)
        def handler(self, a, out_data):
            fn = getattr(self, fn_name)
            self.accumulate_result(fn(self._module, out_data if needs_out else a), name)
        return handler

    def _fwd_rfim(name, fn_name):  # noqa: N805
        def handler(self, a, out_data):
            self.accumulate_result(getattr(self, fn_name)(self._module, a, out_data), name)
        return handler

    # ------------------------------------------------------------------ backward
    def backward_pre_process(self, out_grads, vector: torch.Tensor = None):
        module, names = self._module, self._op_names
        if not any(n in BWD_OPS for n in names):
            return
        g = self.preprocess_out_grads(module, out_grads)
        if OP_SAVE_OUTGRADS in names:
            self.accumulate_result([g], OP_SAVE_OUTGRADS, extend=True)
        a = None
        if any(n in BWD_OPS_WITH_INPUTS for n in names):
            # a layer applied k times in the forward pass saved k inputs; its output gradients arrive in
            # reverse order (and again in that order in every further backward pass of the same graph)
            saved_in, saved_out = self.get_result(OP_SAVE_INPUTS), self.get_result(OP_SAVE_OUTPUTS)
            use = -1 - self._bwd_calls % len(saved_in)
            self._bwd_calls += 1
            a = self.preprocess_in_data(module, saved_in[use], saved_out[use])
        a32 = g32 = None
        for name in list(names):
            handler = _BWD_HANDLERS.get(name)
            if handler is not None:
                with nvtx_range(_RANGE_NAMES_BWD.get(name, name)):
                    if name in _HALF_PRECISION_OK:
                        handler(self, name, a, g, vector)
                    else:
                        a32 = _as_fp32(a) if a32 is None and a is not None else a32
                        g32 = _as_fp32(g) if g32 is None else g32
                        handler(self, name, a32, g32, vector)

    def _bwd_cov(self, name, a, g, vector):
        _, _, bg = self.collect_batch_grads(a, g)
        cov = ops.gram(bg, scale=self._cov_scale)     # bg^T bg: the tensor-core SYRK on CUDA
        if name == OP_COV:
            self.accumulate_result(cov, OP_COV, 'data')
        else:
            self.accumulate_result(cholesky_inv(cov, self._damping), OP_COV, 'inv')

    def _bwd_cvp(self, name, a, g, vector):
        if vector is None:
            raise ValueError('vector is not set.')
        if vector.ndim != 1:
            raise ValueError(f'vector.ndim has to be 1. Got {vector.ndim}.')
        module = self._module
        has_w = original_requires_grad(module, 'weight')
        has_b = original_requires_grad(module, 'bias')
        direct = self._cvp_without_batch_grads(a, g, vector, has_w, has_b)
        if direct is not None:
            for key, value in zip(('weight', 'bias'), direct):
                if value is not None:
                    self.accumulate_result(value.mul_(self._cov_scale), OP_CVP, key)
            return
        _, _, bg = self.collect_batch_grads(a, g)
        cvp = torch.mv(bg.T, torch.mv(bg, vector)).mul_(self._cov_scale)
        if has_w and has_b:
            nw = module.weight.numel()
            self.accumulate_result(cvp[:nw].view_as(module.weight), OP_CVP, 'weight')
            self.accumulate_result(cvp[nw:].view_as(module.bias), OP_CVP, 'bias')
        elif has_w:
            self.accumulate_result(cvp.view_as(module.weight), OP_CVP, 'weight')
        else:
            self.accumulate_result(cvp.view_as(module.bias), OP_CVP, 'bias')

    def _bwd_kron(self, name, a, g, vector):
        if name == OP_COV_KRON:
            self.accumulate_result(self.cov_kron_B(self._module, g).mul_(self._cov_scale), OP_COV_KRON, 'B')
        else:
            self._accumulate_swift(self.cov_swift_kron_B(self._module, g), 'B')

    def _bwd_kron_inv(self, name, a, g, vector):
        module, scale = self._module, self._cov_scale
        A = self.cov_kron_A(module, a).mul_(scale)
        B = self.cov_kron_B(module, g).mul_(scale)
        if self._kron_inv_sums is not None:   # the layer was applied before in this pass: invert the sums
            A += self._kron_inv_sums[0]
            B += self._kron_inv_sums[1]
        self._kron_inv_sums = (A, B)
        damping_A, damping_B = self.cov_kron_damping(A, B)
        node = self._walk((OP_COV_KRON,), create=True)
        node['A_inv'] = cholesky_inv(A, damping_A)
        node['B_inv'] = cholesky_inv(B, damping_B)

    def _bwd_swift_kron_inv(self, name, a, g, vector):
        module, scale = self._module, self._cov_scale

        def scaled(mat):  # same convention as _accumulate_swift: a raw n x d factor stands for x^T x / n
            return mat * (scale if mat.shape[0] == mat.shape[1] else math.sqrt(scale * mat.shape[0]))

        A = scaled(self.cov_swift_kron_A(module, a))
        B = scaled(self.cov_swift_kron_B(module, g))
        damping_A, damping_B = self.cov_kron_damping(A, B)

        def invert(mat, damp):
            return cholesky_inv(mat, damp) if mat.shape[0] == mat.shape[1] else smw_inv(mat, damp)

        self.accumulate_result(invert(A, damping_A), OP_COV_KRON, 'A_inv')
        self.accumulate_result(invert(B, damping_B), OP_COV_KRON, 'B_inv')

    def _bwd_kfe(self, name, a, g, vector):
        module = self._module
        Ua = self.cov_kfe_A(module, a)
        Ub = self.cov_kfe_B(module, g)
        bias = original_requires_grad(module, 'bias')
        self.accumulate_result(Ua, OP_COV_KFE, 'A')
        self.accumulate_result(Ub, OP_COV_KFE, 'B')
        self.accumulate_result(self.cov_kfe_scale(module, a, g, Ua, Ub, bias=bias), OP_COV_KFE, 'scale')

    def _bwd_unit_wise(self, name, a, g, vector):
        module = self._module
        if _is_norm_layer(module):
            if not (original_requires_grad(module, 'weight') and original_requires_grad(module, 'bias')):
                raise ValueError(f'Both weight and bias have to require grad for {OP_COV_UNIT_WISE} '
                                 f'(module: {module}).')
        elif original_requires_grad(module, 'bias'):
            a = self.extend_in_data(a)
        cov = self.cov_unit_wise(module, a, g).mul_(self._cov_scale)
        if name == OP_COV_UNIT_WISE:
            self.accumulate_result(cov, OP_COV_UNIT_WISE, 'data')
        else:
            self.accumulate_result(ops.unitwise_inverse(cov, self._damping), OP_COV_UNIT_WISE, 'inv')

    def _bwd_diag(self, name, a, g, vector):
        module, scale, damping = self._module, self._cov_scale, self._damping
        inv = name == OP_COV_DIAG_INV
        if original_requires_grad(module, 'weight'):
            cov = self.cov_diag_weight(module, a, g).mul_(scale)
            self.accumulate_result(1 / (cov + damping) if inv else cov,
                                   OP_COV_DIAG, 'weight_inv' if inv else 'weight')
        if original_requires_grad(module, 'bias'):
            cov = self.cov_diag_bias(module, g).mul_(scale)
            self.accumulate_result(1 / (cov + damping) if inv else cov,
                                   OP_COV_DIAG, 'bias_inv' if inv else 'bias')

    def _kernel_owner(self, name):
        owner = self._model_for_kernel
        if owner is None:
            raise ValueError(f'model_for_kernel needs to be set for {name}.')
        return owner

    def _bwd_gram_hadamard(self, name, a, g, vector):
        """kernel += gram_B(g) o (gram_A(a) [+1 with a bias]).  When the batch holds two
        concatenated sets (n1 rows then the rest) the rectangular n1 x n2 block is produced."""
        owner, module = self._kernel_owner(name), self._module
        n1 = owner.kernel.shape[0]
        fused_scale = self._gram_hadamard_scale(a, g)
        if fused_scale is not None and ops.cuda_kernels_enabled(owner.kernel, a, g) and owner.kernel.dtype == torch.float32:
            # both Gram tiles in TMEM, multiplied in the epilogue of one launch
            a2d, g2d = a.flatten(start_dim=1), g.flatten(start_dim=1)
            one = 1.0 if original_requires_grad(module, 'bias') else 0.0
            if g.shape[0] == n1:
                ops.gram_hadamard(owner.kernel, a2d, g2d, one=one, scale=fused_scale)
            else:
                ops.gram_hadamard(owner.kernel, a2d[:n1], g2d[:n1], a2d[n1:], g2d[n1:], one=one, scale=fused_scale)
            return
        if g.shape[0] == n1:
            A = self.gram_A(module, a)
            B = self.gram_B(module, g)
        else:
            A = self.gram_A(module, a[:n1], a[n1:])
            B = self.gram_B(module, g[:n1], g[n1:])
        if original_requires_grad(module, 'bias'):
            A = A + 1.
        owner.kernel += B.mul(A)

    def _cvp_without_batch_grads(self, a, g, vector, has_w, has_b):
        """sum_n g_n (g_n . v) split into (weight, bias) without forming the per-example gradients, or
        None when the layer has no such form (the per-example gradients are then collected)."""
        return None

    def _gram_hadamard_scale(self, a, g):
        """Factor of gram_B when gram_A / gram_B are plain products of the flattened operands (Linear:
        1, Conv2d: 1 / spatial size), else None (the layer's own gram_A / gram_B are called)."""
        return None

    def _bwd_gram_direct(self, name, a, g, vector):
        owner, module = self._kernel_owner(name), self._module
        n1 = owner.kernel.shape[0]
        bg_w, bg_b, bg = self.collect_batch_grads(a, g)
        precond = getattr(module, 'gram_precond', None)
        if precond is not None:
            # copies: the per-example bias gradient of a Linear layer is the output gradient itself, which
            # autograd still propagates
            bg_w = None if bg_w is None else bg_w.clone()
            bg_b = None if bg_b is None else bg_b.clone()
            precond.precondition_module(module, vec_weight=bg_w, vec_bias=bg_b)
            bg2 = torch.cat([t.flatten(start_dim=1) for t in (bg_w, bg_b) if t is not None], dim=1)
        else:
            bg2 = bg
        if a.shape[0] == n1:
            owner.kernel += torch.matmul(bg, bg2.T)
        else:
            owner.kernel += torch.matmul(bg[:n1], bg2[n1:].T)

    def _bwd_batch_grads(self, name, a, g, vector):
        module = self._module
        if original_requires_grad(module, 'weight'):
            self.accumulate_result(self.batch_grads_weight(module, a, g), OP_BATCH_GRADS, 'weight')
        if original_requires_grad(module, 'bias'):
            self.accumulate_result(self.batch_grads_bias(module, g), OP_BATCH_GRADS, 'bias')

    def _bwd_mean_outgrads(self, name, a, g, vector):
        fn = self.out_grads_mean if name == OP_MEAN_OUTGRADS else self.out_grads_spatial_mean
        self.accumulate_result(fn(self._module, g), name)

    def _bwd_sketched_gram(self, name, a, g, vector):
        self.accumulate_result(self.random_sketch_and_gram(self._module, a, g), OP_SKETCHED_GRAM)

    # ------------------------------------------------------------------ shared helpers
    @torch.no_grad()
    def collect_batch_grads(self, in_data, out_grads):
        """Per-example gradients of weight and bias and their flattened concatenation (n x p)."""
        module = self._module
        bg_w = bg_b = None
        if original_requires_grad(module, 'weight'):
            bg_w = self.batch_grads_weight(module, in_data, out_grads)
        if original_requires_grad(module, 'bias'):
            bg_b = self.batch_grads_bias(module, out_grads)
        if bg_w is None and bg_b is None:
            raise ValueError(f'At least one of weight or bias has to require grad (module: {module}).')
        flat = torch.cat([t.flatten(start_dim=1) for t in (bg_w, bg_b) if t is not None], dim=1)
        return bg_w, bg_b, flat

    def cov_kron_damping(self, A, B, eps=1.e-7):
        """pi-split of the damping between the two Kronecker factors."""
        from ..symmatrix import Kron
        return Kron(A, B).damping_split(self._damping, eps)

    def random_sketch_and_gram(self, module, in_data, out_grads):
        """Column-subsampled (rescaled) a and g and the Hadamard product of their n x n Grams.
        in_data: n x d_in (x r); out_grads: n x d_out (x r)."""
        size = self._sketching_size

        def sketch(t):
            dim = t.shape[1]
            if size >= dim:
                return t, None
            idx = torch.randperm(dim, device=t.device)[:size]
            return torch.index_select(t, 1, idx).mul(dim / size), idx

        sub_a, idx_a = sketch(in_data)
        sub_g, idx_g = sketch(out_grads)
        gram = self.gram_A(module, sub_a).mul(self.gram_B(module, sub_g))
        return (in_data, out_grads), (sub_a, sub_g), (idx_a, idx_g), gram

    # ------------------------------------------------------------------ primitives
    @staticmethod
    def preprocess_in_data(module, in_data, out_data):
        return in_data

    @staticmethod
    def preprocess_out_grads(module, out_grads):
        return out_grads

    @staticmethod
    def extend_in_data(in_data):
        return in_data

    def out_data_spatial_mean(self, module, out_data):
        return self.out_data_mean(module, out_data)

    def out_grads_spatial_mean(self, module, out_grads):
        return self.out_grads_mean(module, out_grads)


def _unimplemented(name):
    def primitive(*args, **kwargs):
        raise NotImplementedError(name)
    primitive.__name__ = name
    return staticmethod(primitive)


for _name in ('batch_grads_weight', 'batch_grads_bias', 'grad_weight', 'grad_bias',
              'cov_diag_weight', 'cov_diag_bias', 'cov_kron_A', 'cov_kron_B',
              'cov_swift_kron_A', 'cov_swift_kron_B', 'cov_kfe_A', 'cov_kfe_B', 'cov_kfe_scale',
              'cov_unit_wise', 'gram_A', 'gram_B', 'rfim_relu', 'rfim_softmax', 'in_data_mean',
              'out_data_mean', 'out_spatial_size', 'out_grads_mean', 'bfgs_kron_s_As'):
    setattr(Operation, _name, _unimplemented(_name))

_FWD_HANDLERS = {
    OP_COV_KRON: Operation._fwd_kron,
    OP_COV_SWIFT_KRON: Operation._fwd_swift_kron,
    OP_RFIM_RELU: Operation._fwd_rfim(OP_RFIM_RELU, 'rfim_relu'),
    OP_RFIM_SOFTMAX: Operation._fwd_rfim(OP_RFIM_SOFTMAX, 'rfim_softmax'),
    OP_MEAN_INPUTS: Operation._fwd_simple(OP_MEAN_INPUTS, 'in_data_mean', False),
    OP_MEAN_OUTPUTS: Operation._fwd_simple(OP_MEAN_OUTPUTS, 'out_data_mean', True),
    OP_SPATIAL_MEAN_OUTPUTS: Operation._fwd_simple(OP_SPATIAL_MEAN_OUTPUTS, 'out_data_spatial_mean', True),
    OP_OUT_SPATIAL_SIZE: Operation._fwd_simple(OP_OUT_SPATIAL_SIZE, 'out_spatial_size', True),
    OP_BFGS_KRON_S_AS: Operation._fwd_simple(OP_BFGS_KRON_S_AS, 'bfgs_kron_s_As', False),
}
_BWD_HANDLERS = {
    OP_COV: Operation._bwd_cov, OP_COV_INV: Operation._bwd_cov,
    OP_CVP: Operation._bwd_cvp,
    OP_COV_KRON: Operation._bwd_kron, OP_COV_SWIFT_KRON: Operation._bwd_kron,
    OP_COV_KRON_INV: Operation._bwd_kron_inv,
    OP_COV_SWIFT_KRON_INV: Operation._bwd_swift_kron_inv,
    OP_COV_KFE: Operation._bwd_kfe,
    OP_COV_UNIT_WISE: Operation._bwd_unit_wise, OP_COV_UNIT_WISE_INV: Operation._bwd_unit_wise,
    OP_COV_DIAG: Operation._bwd_diag, OP_COV_DIAG_INV: Operation._bwd_diag,
    OP_GRAM_HADAMARD: Operation._bwd_gram_hadamard,
    OP_GRAM_DIRECT: Operation._bwd_gram_direct,
    OP_BATCH_GRADS: Operation._bwd_batch_grads,
    OP_MEAN_OUTGRADS: Operation._bwd_mean_outgrads,
    OP_SPATIAL_MEAN_OUTGRADS: Operation._bwd_mean_outgrads,
    OP_SKETCHED_GRAM: Operation._bwd_sketched_gram,
}
#: operations whose primitives take bf16 / fp16 activations as they are (Gram products with fp32 accumulation:
#: tensor-core kernels on CUDA, an fp32 product elsewhere); every other operation gets fp32 copies
_HALF_PRECISION_OK = {OP_COV_KRON, OP_COV_KRON_INV}


def _as_fp32(t):
    if isinstance(t, torch.Tensor) and t.dtype in (torch.bfloat16, torch.float16):
        return t.float()
    return t


#: range names of the hook-time work (NVTX and phase profiles); the Kronecker ops have a forward and a backward half
_RANGE_NAMES_FWD = {OP_COV_KRON: 'cov_kron_A', OP_COV_SWIFT_KRON: 'cov_swift_kron_A'}
_RANGE_NAMES_BWD = {OP_COV_KRON: 'cov_kron_B', OP_COV_SWIFT_KRON: 'cov_swift_kron_B',
                    OP_COV_KRON_INV: 'cov_kron_inv', OP_COV_SWIFT_KRON_INV: 'cov_swift_kron_inv'}


class OperationContext:
    """Module -> Operation map with result accessors and post-hoc calculators that work from the
    saved inputs / output-gradients instead of from hooks."""

    def __init__(self, vectors: ParamVector = None):
        self._operations: Dict[nn.Module, Operation] = {}
        self._vectors: ParamVector = vectors
        self._input_scale = 1.
        self._output_scale = 1.

    # registration -----------------------------------------------------------------------------
    def is_operation_registered(self, module: nn.Module):
        return module in self._operations

    def register_operation(self, module: nn.Module, operation: Operation):
        self._operations[module] = operation

    def get_operation(self, module: nn.Module) -> Operation:
        try:
            return self._operations[module]
        except KeyError:
            raise KeyError(f'No operation is registered to {module}.')

    def clear_operation(self, module: nn.Module):
        if self._operations.pop(module, None) is None:
            raise KeyError(f'No operation is registered to {module}.')

    def clear_operations(self):
        self._operations.clear()

    def get_vectors_by_module(self, module: nn.Module, flatten=False):
        if self._vectors is None:
            return None
        vectors = self._vectors.get_vectors_by_module(module)
        if vectors is None:
            return None
        return vectors.get_flatten_vector() if flatten else vectors

    # hook entry points --------------------------------------------------------------------------
    def call_operations_in_forward(self, module, in_data, out_data):
        self.get_operation(module).forward_post_process(in_data, out_data)

    def call_operations_in_backward(self, module, out_grads):
        vector = self.get_vectors_by_module(module, flatten=True)
        self.get_operation(module).backward_pre_process(out_grads, vector)

    # result access ------------------------------------------------------------------------------
    def get_result(self, module, *keys, pop=False, default=None):
        op = self._operations.get(module)
        if op is None:
            return default
        return op.get_result(*keys, pop=pop, default=default)

    def accumulate_result(self, module, value, *keys):
        return self.get_operation(module).accumulate_result(value, *keys)

    def clear_result(self, module, *keys):
        return self.get_operation(module).clear_result(*keys)

    def _for_all(self, method, *args):
        for op in self._operations.values():
            getattr(op, method)(*args)

    def turn_on_op(self, op_name):
        self._for_all('add_op_name', op_name)

    def turn_off_op(self, op_name):
        self._for_all('remove_op_name', op_name)

    def turn_on_save_inputs_outgrads(self):
        self.turn_on_op(OP_SAVE_INPUTS)
        self.turn_on_op(OP_SAVE_OUTGRADS)

    def turn_off_save_inputs_outgrads(self):
        self.turn_off_op(OP_SAVE_INPUTS)
        self.turn_off_op(OP_SAVE_OUTGRADS)

    def set_damping(self, value):
        self._for_all('set_damping', value)

    def set_cov_scale(self, value):
        self._for_all('set_cov_scale', value)

    def set_sketching_size(self, value):
        self._for_all('set_sketching_size', value)

    def set_truncated_rank(self, value):
        self._for_all('set_truncated_rank', value)

    def set_input_scale(self, scale):
        self._input_scale = scale

    def set_output_scale(self, scale):
        self._output_scale = scale

    # named accessors ----------------------------------------------------------------------------
    def in_data(self, module, pop=False):
        return self.get_result(module, OP_SAVE_INPUTS, pop=pop)

    def out_data(self, module, pop=False):
        return self.get_result(module, OP_SAVE_OUTPUTS, pop=pop)

    def out_grads(self, module, pop=False):
        return self.get_result(module, OP_SAVE_OUTGRADS, pop=pop)

    def cov(self, module):
        return self.get_result(module, OP_COV)

    def cvp(self, module):
        return self.get_result(module, OP_CVP)

    def cov_kron(self, module):
        return self.get_result(module, OP_COV_KRON)

    def cov_unit_wise(self, module):
        return self.get_result(module, OP_COV_UNIT_WISE)

    def cov_diag(self, module):
        return self.get_result(module, OP_COV_DIAG)

    def full_cov(self, module):
        return self.get_result(module, OP_FULL_COV)

    def full_cvp(self, module):
        return self.get_result(module, OP_FULL_CVP)

    def rfim_relu(self, module):
        return self.get_result(module, OP_RFIM_RELU)

    def rfim_softmax(self, module):
        return self.get_result(module, OP_RFIM_SOFTMAX)

    def mean_in_data(self, module):
        return self.get_result(module, OP_MEAN_INPUTS)

    def mean_out_data(self, module):
        return self.get_result(module, OP_MEAN_OUTPUTS)

    def spatial_mean_out_data(self, module):
        return self.get_result(module, OP_SPATIAL_MEAN_OUTPUTS)

    def out_spatial_size(self, module):
        return self.get_result(module, OP_OUT_SPATIAL_SIZE)

    def mean_out_grads(self, module):
        return self.get_result(module, OP_MEAN_OUTGRADS)

    def spatial_mean_out_grads(self, module):
        return self.get_result(module, OP_SPATIAL_MEAN_OUTGRADS)

    def bfgs_kron_s_As(self, module):
        return self.get_result(module, OP_BFGS_KRON_S_AS)

    def sketched_inputs_outgrads_gram(self, module):
        return self.get_result(module, OP_SKETCHED_GRAM)

    # per-example gradients ------------------------------------------------------------------------
    def batch_grads(self, module, flatten=False):
        grads = self.get_result(module, OP_BATCH_GRADS)
        if grads is not None and flatten:
            return torch.cat([g.flatten(start_dim=1) for g in grads.values()], dim=1)
        return grads

    def clear_batch_grads(self):
        for op in self._operations.values():
            if op.get_result(OP_BATCH_GRADS) is not None:
                op.clear_result(OP_BATCH_GRADS)

    def full_batch_grads(self, module):
        parts = [self.batch_grads(m, flatten=True) for m in module.modules()]
        parts = [p for p in parts if p is not None]
        return torch.cat(parts, dim=1) if parts else None  # n x p

    def calc_full_cov(self, module, scale=1., calc_inv=False, damping=1.e-7):
        """Dense p x p covariance sum_n g_n g_n^T over all hooked modules (or its damped inverse)."""
        bg = self.full_batch_grads(module)
        if bg is None:
            return
        cov = torch.matmul(bg.T, bg).mul_(scale)
        if calc_inv:
            self.accumulate_result(module, cholesky_inv(cov, damping), OP_FULL_COV, 'inv')
        else:
            self.accumulate_result(module, cov, OP_FULL_COV, 'data')

    def calc_full_cvp(self, module, scale=1.):
        """sum_n g_n (g_n^T v) without forming the covariance."""
        vector = self.get_vectors_by_module(module, flatten=True)
        bg = self.full_batch_grads(module)
        if bg is None:
            return
        if bg.shape[1] != vector.shape[0]:
            raise ValueError(f'bg.shape[1] ({bg.shape[1]}) does not match vector.shape[0] ({vector.shape[0]}).')
        cvp = torch.mv(bg.T, torch.mv(bg, vector)).mul_(scale)
        self.accumulate_result(module, cvp, OP_FULL_CVP)

    # post-hoc calculators from saved tensors ------------------------------------------------------
    def load_op_in_out(self, module) -> Tuple[Operation, List[torch.Tensor], List[torch.Tensor]]:
        return self.get_operation(module), self.in_data(module), self.out_grads(module)

    def calc_grads(self, scale=None):
        for module in list(self._operations.keys()):
            if original_requires_grad(module, 'weight') or original_requires_grad(module, 'bias'):
                self.calc_grad(module, scale)

    def calc_grad(self, module, scale=None):
        """Recompute weight/bias gradients from the saved input and output-gradient, optionally
        re-weighting each example by ``scale``."""
        op, in_data, out_grads = self.load_op_in_out(module)
        a = op.preprocess_in_data(module, in_data[-1], (self.out_data(module) or [None])[-1]) \
            if isinstance(in_data, list) else in_data
        g = out_grads[-1] if isinstance(out_grads, list) else out_grads
        if scale is not None:
            if scale.shape[0] != g.shape[0]:
                raise ValueError(f'scale and out_grads have to have the same first dimension. '
                                 f'Got {scale.shape[0]} and {g.shape[0]}')
            g = g * scale.view(-1, *([1] * (g.ndim - 1)))
        for attr, fn, args in (('weight', op.grad_weight, (module, a, g)),
                               ('bias', op.grad_bias, (module, g))):
            if not original_requires_grad(module, attr):
                continue
            grad = fn(*args)
            param = getattr(module, attr)
            if param.grad is None:
                param.grad = grad
            else:
                param.grad.data.copy_(grad)

    def calc_kernel(self):
        """sum over modules of gram_A o gram_B (+ gram_B for the bias) from saved tensors."""
        kernel = None
        for module in self._operations.keys():
            if not original_requires_grad(module, 'weight'):
                continue
            op, in_data, out_grads = self.load_op_in_out(module)
            a = op.preprocess_in_data(module, in_data[-1], (self.out_data(module) or [None])[-1])
            g = out_grads[-1]
            A = op.gram_A(module, a, a)
            B = op.gram_B(module, g, g)
            if kernel is None:
                kernel = torch.zeros_like(A)
            kernel += A.mul(B)
            if original_requires_grad(module, 'bias'):
                kernel += B
        return kernel

    def calc_cov(self, module, shape=SHAPE_LAYER_WISE, kron=None, clear_in_out=False,
                 num_batches=None, swift=False, tag=''):
        """Curvature of ``shape`` for ``module`` from the lists of saved inputs / out-grads."""
        op, in_list, g_list = self.load_op_in_out(module)
        out_list = self.out_data(module)

        def take(lst, i):
            return lst.pop(0) if clear_in_out else lst[i]

        def limit(*lists):
            n = min(len(l) for l in lists)
            return n if num_batches is None else min(n, num_batches)

        def prep_in(i):
            raw = take(in_list, i)
            out = take(out_list, i) if out_list else None
            t = op.preprocess_in_data(module, raw, out)
            return t * self._input_scale if self._input_scale != 1 else t

        def prep_g(i):
            t = take(g_list, i)
            return t * self._output_scale if self._output_scale != 1 else t

        if shape == SHAPE_KRON:
            kron = ['A', 'B'] if kron is None else kron
            if 'A' in kron and in_list is not None:
                with nvtx_range('cov_kron_A' + tag):
                    for i in range(limit(in_list)):
                        a = prep_in(i)
                        A = op.cov_swift_kron_A(module, a) if swift else op.cov_kron_A(module, a)
                        self.accumulate_result(module, A, OP_COV_KRON, 'A')
            if 'B' in kron and g_list is not None:
                with nvtx_range('cov_kron_B' + tag):
                    for i in range(limit(g_list)):
                        g = prep_g(i)
                        B = op.cov_swift_kron_B(module, g) if swift else op.cov_kron_B(module, g)
                        self.accumulate_result(module, B, OP_COV_KRON, 'B')
            return
        if in_list is None or g_list is None:
            return
        with nvtx_range(f'cov_{shape}' + tag):
            for i in range(limit(in_list, g_list)):
                a, g = prep_in(i), prep_g(i)
                if shape == SHAPE_LAYER_WISE:
                    _, _, bg = op.collect_batch_grads(a, g)
                    self.accumulate_result(module, torch.matmul(bg.T, bg), OP_COV, 'data')
                elif shape == SHAPE_UNIT_WISE:
                    if not _is_norm_layer(module) and original_requires_grad(module, 'bias'):
                        a = op.extend_in_data(a)
                    self.accumulate_result(module, op.cov_unit_wise(module, a, g), OP_COV_UNIT_WISE, 'data')
                elif shape == SHAPE_DIAG:
                    self.accumulate_result(module, op.cov_diag_weight(module, a, g), OP_COV_DIAG, 'weight')
                    if original_requires_grad(module, 'bias'):
                        self.accumulate_result(module, op.cov_diag_bias(module, g), OP_COV_DIAG, 'bias')

    def calc_cov_kron(self, module, clear_in_out=False):
        self.calc_cov(module, shape=SHAPE_KRON, clear_in_out=clear_in_out)

    def calc_cov_unit_wise(self, module, clear_in_out=False):
        self.calc_cov(module, shape=SHAPE_UNIT_WISE, clear_in_out=clear_in_out)

    def calc_cov_diag(self, module, clear_in_out=False):
        self.calc_cov(module, shape=SHAPE_DIAG, clear_in_out=clear_in_out)

    # results -> containers --------------------------------------------------------------------------
    def cov_symmatrix(self, module, pop=False):
        """Collect whatever curvature was computed for ``module`` into a SymMatrix (or None)."""
        kwargs = {}

        def gather(op_name, mapping):
            res = self.get_result(module, op_name, pop=pop)
            if res is None:
                return
            for src, dst in mapping.items():
                kwargs[dst] = res.pop(src, None) if pop else res.get(src)

        gather(OP_COV, {'data': 'data', 'inv': 'inv'})
        gather(OP_COV_KRON, {'A': 'kron_A', 'B': 'kron_B', 'A_inv': 'kron_A_inv', 'B_inv': 'kron_B_inv'})
        gather(OP_COV_KFE, {'A': 'kfe_A', 'B': 'kfe_B', 'scale': 'kfe_scale'})
        gather(OP_COV_UNIT_WISE, {'data': 'unit_data', 'inv': 'unit_inv'})
        diag_map = {}
        if original_requires_grad(module, 'weight'):
            diag_map.update(weight='diag_weight', weight_inv='diag_weight_inv')
        if original_requires_grad(module, 'bias'):
            diag_map.update(bias='diag_bias', bias_inv='diag_bias_inv')
        gather(OP_COV_DIAG, diag_map)
        if all(v is None for v in kwargs.values()):
            return None
        return SymMatrix(**kwargs)

    def full_cov_symmatrix(self, module, pop=False):
        cov = self.get_result(module, OP_FULL_COV, pop=pop)
        if cov is None:
            return None
        return SymMatrix(data=cov.get('data'), inv=cov.get('inv'))

    def register_symmatrix(self, module, matrix: SymMatrix):
        """Pre-load existing curvature into the accumulators so new statistics add in place
        (this is how accumulation over micro-batches and the EMA are realised)."""
        op = self.get_operation(module)
        if matrix.has_data:
            op.accumulate_result(matrix.data, OP_COV, 'data')
        if matrix.has_kron:
            if matrix.kron.has_A:
                op.accumulate_result(matrix.kron.A, OP_COV_KRON, 'A')
            if matrix.kron.has_B:
                op.accumulate_result(matrix.kron.B, OP_COV_KRON, 'B')
        if matrix.has_kfe:
            for key, value in (('A', matrix.kfe.Ua), ('B', matrix.kfe.Ub), ('scale', matrix.kfe.scale)):
                if value is not None:
                    op.accumulate_result(value, OP_COV_KFE, key)
        if matrix.has_unit and matrix.unit.has_data:
            op.accumulate_result(matrix.unit.data, OP_COV_UNIT_WISE, 'data')
        if matrix.has_diag:
            if matrix.diag.has_weight:
                op.accumulate_result(matrix.diag.weight, OP_COV_DIAG, 'weight')
            if matrix.diag.has_bias:
                op.accumulate_result(matrix.diag.bias, OP_COV_DIAG, 'bias')

    def register_full_symmatrix(self, module, matrix: SymMatrix):
        if not matrix.has_data:
            raise ValueError('data do not exist')
        self.get_operation(module).accumulate_result(matrix.data, OP_FULL_COV, 'data')

    def cvp_paramvector(self, module, pop=False):
        cvp = self.get_result(module, OP_CVP, pop=pop)
        if cvp is None:
            return None
        params, vectors = [], []
        for attr in ('weight', 'bias'):
            if original_requires_grad(module, attr):
                params.append(getattr(module, attr))
                vectors.append(cvp[attr])
        return ParamVector(params, vectors)

    def full_cvp_paramvector(self, module, pop=False):
        cvp = self.get_result(module, OP_FULL_CVP, pop=pop)
        if cvp is None:
            return None
        params = []
        for m in module.modules():
            if m in self._operations and m is not module:
                for attr in ('weight', 'bias'):
                    if original_requires_grad(m, attr):
                        params.append(getattr(m, attr))
        if sum(p.numel() for p in params) != cvp.numel():
            params = [p for p in module.parameters() if original_requires_grad(param=p)]
        return ParamVector(params, cvp)
