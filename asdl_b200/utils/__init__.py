"""General helpers: requires_grad bookkeeping, patch extraction, damped SPD solves, pseudo-batch
loaders and NVTX ranges.

Parity notes (reference: asdl/utils.py):
  * ``original_requires_grad`` / ``skip_param_grad``       <- asdl/utils.py:21-48
  * ``im2col_2d`` / ``im2col_2d_slow``                     <- asdl/utils.py:51-88
  * ``cholesky_inv`` / ``cholesky_solve`` / ``smw_inv``    <- asdl/utils.py:91-115
  * ``PseudoBatchLoaderGenerator``                         <- asdl/utils.py:118-186
  * ``nvtx_range`` / ``has_reduction``                     <- asdl/utils.py:189-202
Differences on purpose: the damped solves never touch the caller's matrix (the reference adds the
damping to the diagonal in place and subtracts it afterwards), ``im2col_2d`` is a single strided
view (and therefore also handles dilation), and on CUDA tensors the SPD inverse is routed to the
library's own fp32 Cholesky kernels through :mod:`asdl_b200.ops`.
"""
import inspect
from contextlib import contextmanager, nullcontext

import torch
from torch import nn
import torch.nn.functional as F
from torch.utils.data import BatchSampler, DataLoader, Subset

from . import profiling
from .profiling import PhaseProfile, time_funcs

__all__ = [
    'original_requires_grad', 'record_original_requires_grad',
    'restore_original_requires_grad', 'skip_param_grad', 'im2col_2d',
    'im2col_2d_slow', 'cholesky_inv', 'cholesky_solve', 'smw_inv',
    'PseudoBatchLoaderGenerator', 'nvtx_range', 'has_reduction', 'PhaseProfile', 'time_funcs'
]

_FLAG = '_original_requires_grad'


def record_original_requires_grad(param):
    """Remember whether ``param`` is trainable before any temporary freezing."""
    setattr(param, _FLAG, param.requires_grad)


def restore_original_requires_grad(param):
    """Puts back the ``requires_grad`` value that :func:`record_original_requires_grad` stored on ``param``."""
    param.requires_grad = getattr(param, _FLAG, param.requires_grad)


def original_requires_grad(module=None, param_name=None, param=None):
    """True if the parameter exists and was trainable when it was last recorded."""
    if param is None:
        if module is None or param_name is None:
            raise ValueError('Both module and param_name have to be set.')
        param = getattr(module, param_name, None)
    if param is None:
        return False
    return bool(getattr(param, _FLAG, param.requires_grad))


@contextmanager
def skip_param_grad(model, disable=False):
    """Backward passes inside this context produce activation gradients (so module hooks fire) but
    leave every ``param.grad`` untouched."""
    if disable:
        yield
        return
    params = list(model.parameters())
    for p in params:
        record_original_requires_grad(p)
        p.requires_grad = False
    try:
        yield
    finally:
        for p in params:
            restore_original_requires_grad(p)


def _conv_geometry(conv2d):
    pad = conv2d.padding
    if isinstance(pad, str):
        if pad not in ('valid', 'same'):
            raise ValueError(f'padding="{pad}" is not supported.')
        pad = (0, 0)   # 'same' is applied to the input by _explicit_padding (it may be asymmetric)
    return tuple(conv2d.kernel_size), tuple(conv2d.stride), tuple(pad), tuple(conv2d.dilation)


def _explicit_padding(x: torch.Tensor, conv2d):
    """(input, (pad_h, pad_w)) for patch extraction: reflect / replicate / circular padding is applied to
    the input here (patch extraction itself pads with zeros), zero padding is left to the caller."""
    (kh, kw), _, (ph, pw), (dh, dw) = _conv_geometry(conv2d)
    mode = getattr(conv2d, 'padding_mode', 'zeros')
    if conv2d.padding == 'same':   # stride 1: total padding d * (k - 1), the extra element on the right / bottom
        th, tw = dh * (kh - 1), dw * (kw - 1)
        pads = (tw // 2, tw - tw // 2, th // 2, th - th // 2)
        if not any(pads):
            return x, (0, 0)
        return F.pad(x, pads, mode='constant' if mode == 'zeros' else mode), (0, 0)
    if mode == 'zeros' or (ph == 0 and pw == 0):
        return x, (ph, pw)
    return F.pad(x, (pw, pw, ph, ph), mode=mode), (0, 0)


def im2col_2d(x: torch.Tensor, conv2d: nn.Module):
    """Patch matrix of a conv input: ``n x c x h x w -> n x (c*kh*kw) x (h_out*w_out)`` with the
    column order (c, kh, kw) of ``conv2d.weight.view(c_out, -1)``."""
    if x.ndim != 4:
        raise ValueError(f'x.ndim has to be 4. Got {x.ndim}.')
    if not isinstance(conv2d, (nn.Conv2d, nn.ConvTranspose2d)):
        raise TypeError(f'conv2d has to be {nn.Conv2d} or {nn.ConvTranspose2d}. Got {type(conv2d)}.')
    (kh, kw), (sh, sw), _, (dh, dw) = _conv_geometry(conv2d)
    x, (ph, pw) = _explicit_padding(x, conv2d)
    if ph or pw:
        x = F.pad(x, (pw, pw, ph, ph))
    n, c, h, w = x.shape
    ho = (h - dh * (kh - 1) - 1) // sh + 1
    wo = (w - dw * (kw - 1) - 1) // sw + 1
    x = x.contiguous()
    sn, sc, s_h, s_w = x.stride()
    patches = x.as_strided((n, c, kh, kw, ho, wo),
                           (sn, sc, s_h * dh, s_w * dw, s_h * sh, s_w * sw))
    return patches.reshape(n, c * kh * kw, ho * wo)


def im2col_2d_slow(x: torch.Tensor, conv2d: nn.Module):
    """Same result through ``F.unfold`` (kept as an independent oracle)."""
    if x.ndim != 4:
        raise ValueError(f'x.ndim has to be 4. Got {x.ndim}.')
    if not isinstance(conv2d, (nn.Conv2d, nn.ConvTranspose2d)):
        raise TypeError(f'conv2d has to be {nn.Conv2d} or {nn.ConvTranspose2d}. Got {type(conv2d)}.')
    k, s, _, d = _conv_geometry(conv2d)
    x, p = _explicit_padding(x, conv2d)
    return F.unfold(x, k, dilation=d, padding=p, stride=s)


def cholesky_inv(X, damping=1e-7):
    """(X + damping*I)^-1 for a symmetric positive (semi-)definite X.  X is not modified."""
    from .. import ops
    return ops.spd_inverse(X, damping)


def cholesky_solve(X, b, damping=1e-7):
    """Solve (X + damping*I) y = b.  X is not modified."""
    from .. import ops
    chol = ops.damped_cholesky(X, damping)
    if b.ndim == 1:
        return torch.cholesky_solve(b.unsqueeze(-1), chol).squeeze(-1)
    return torch.cholesky_solve(b, chol)


def smw_inv(x, damping=1e-7):
    """Woodbury inverse of ``x^T x / n + damping*I`` (up to the ``1/n`` folded into the damping)
    for a wide factor ``x`` (n x d, n < d): ``(I - x^T (x x^T + damping*n*I)^-1 x) / damping``."""
    n, d = x.shape
    gram = x @ x.T
    gram = gram + (damping * n) * torch.eye(n, device=x.device, dtype=x.dtype)
    sol = torch.linalg.solve(gram, x)
    eye = torch.eye(d, device=x.device, dtype=x.dtype)
    return (eye - x.T @ sol) / damping


class PseudoBatchLoaderGenerator:
    """Iterates a dataset in large logical "pseudo-batches"; each item is a DataLoader that walks
    one pseudo-batch in micro-batches of ``batch_size``.

    >>> loader = DataLoader(TensorDataset(torch.arange(10)), shuffle=True)
    >>> for pb_loader in PseudoBatchLoaderGenerator(loader, 5):
    ...     for (x,) in pb_loader: ...
    """

    def __init__(self, base_data_loader, pseudo_batch_size, batch_size=None, drop_last=None):
        if batch_size is None:
            batch_size = base_data_loader.batch_size
        if pseudo_batch_size % batch_size != 0:
            raise ValueError(f'pseudo_batch_size ({pseudo_batch_size}) '
                             f'needs to be divisible by batch_size ({batch_size})')
        if drop_last is None:
            drop_last = base_data_loader.drop_last
        dataset = base_data_loader.dataset
        sampler = type(base_data_loader.sampler)(range(len(dataset)))
        self.batch_size = batch_size
        self.base_dataset = dataset
        self.base_data_loader = base_data_loader
        self.pseudo_batch_sampler = BatchSampler(sampler, batch_size=pseudo_batch_size,
                                                 drop_last=drop_last)

    def __iter__(self):
        base = self.base_data_loader
        for indices in self.pseudo_batch_sampler:
            kwargs = dict(batch_size=self.batch_size, shuffle=False, num_workers=base.num_workers,
                          collate_fn=base.collate_fn, pin_memory=base.pin_memory, drop_last=False,
                          timeout=base.timeout, worker_init_fn=base.worker_init_fn,
                          generator=base.generator)
            if base.num_workers > 0:
                kwargs.update(multiprocessing_context=base.multiprocessing_context,
                              prefetch_factor=base.prefetch_factor,
                              persistent_workers=base.persistent_workers)
            yield DataLoader(Subset(self.base_dataset, indices), **kwargs)

    def __len__(self) -> int:
        return len(self.pseudo_batch_sampler)


@contextmanager
def nvtx_range(msg, *args, **kwargs):
    """NVTX range when CUDA is present; while a :class:`~asdl_b200.utils.profiling.PhaseProfile`
    is active the range is also timed (CUDA events, or the wall clock on CPU) under the same name."""
    profile = profiling.active_profile()
    timed = profile.range(msg) if profile is not None else nullcontext()
    if torch.cuda.is_available():
        with torch.cuda.nvtx.range(msg, *args, **kwargs), timed:
            yield
    else:
        with timed:
            yield


def has_reduction(func):
    """Whether a loss callable (module or function) exposes a ``reduction`` option."""
    if isinstance(func, nn.Module):
        return hasattr(func, 'reduction')
    try:
        return 'reduction' in inspect.signature(func).parameters
    except (TypeError, ValueError):
        return False
