"""Analytic FLOP / memory (element count) models per layer for the forward and backward passes and
for the statistics / inverse / preconditioning phases of Adam, K-FAC, Shampoo, L-BFGS and SMW-NG.

Parity: asdl/counter.py:15-334 (same public classes, ``set_counter`` context, ``linear`` /
``conv2d`` / ``attn`` entry points and the same conventions: a multiply-add counts as 2 FLOPs for
matrix products, convolution products are counted as in the reference, ``numel`` is the number of
elements the phase has to keep).

Structure: every layer is reduced to a :class:`LayerDims` record (rows = samples x positions,
d_in, d_out, the raw weight shape); a counter only has to say what its phase costs for such a
record.  ``roofline_ms`` turns a (FLOP, bytes) pair into the time bound implied by a measured
peak pair, for quick "is this phase compute- or bandwidth-bound" estimates.
"""
import math
from contextlib import contextmanager
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from torch import Tensor
import torch.nn as nn

__all__ = ['Counter', 'set_counter', 'Forward', 'BackwardWeight', 'BackwardInput',
           'AdamStats', 'AdamPrecond', 'KFACStats', 'KFACInv', 'KFACPrecond',
           'ShampooStats', 'ShampooInv', 'ShampooPrecond', 'LBFGSPrecond',
           'SMWNGStats', 'SMWNGPrecond', 'LayerDims', 'roofline_ms']


@dataclass
class LayerDims:
    batch_size: int
    d_out: int
    d_in: int            # fan-in of one output unit (c_in*kh*kw for convolutions)
    weight_shape: Tuple[int, ...]
    in_positions: int = 1    # h_in*w_in
    out_positions: int = 1   # h_out*w_out
    c_in: int = 0
    is_conv: bool = False

    @property
    def n_params(self):
        return self.d_out * self.d_in


def roofline_ms(flop: float, n_bytes: float, peak_tflops: float = 1413.5, peak_gbs: float = 6539.9):
    """max(compute time, memory time) in milliseconds for the given peaks (defaults: sustained
    bf16 matmul TFLOP/s and copy GB/s measured on a B200)."""
    return max(flop / (peak_tflops * 1e12), n_bytes / (peak_gbs * 1e9)) * 1e3


class Counter:
    """Base of the analytic cost models: ``count_flop_numel(module, ...)`` returns the floating-point
    operations and the number of stored values one phase of a method costs on ``module`` (Linear, Conv2d or
    MultiheadAttention); subclasses define ``cost`` (and ``attn``).  Reference: asdl/counter.py:15-120.
    """

    supported_types = (nn.Linear, nn.Conv2d, nn.MultiheadAttention)

    def count_flop_numel(self, module: nn.Module, inputs: Optional[Tensor] = None,
                         outputs: Optional[Tensor] = None, batch_size: int = 32,
                         seq_len: int = 128) -> Tuple[int, int]:
        if type(module) == nn.Linear:
            return self.linear(batch_size, *module.weight.shape)
        if type(module) == nn.Conv2d:
            h_in, w_in = inputs.shape[2:]
            h_out, w_out = outputs.shape[2:]
            return self.conv2d(batch_size, *module.weight.shape, h_in * w_in, h_out * w_out)
        if type(module) == nn.MultiheadAttention:
            return self.attn(seq_len, batch_size, module.embed_dim, module.num_heads)
        raise TypeError(f'Invalid module type: {type(module)}')

    # the phase model -----------------------------------------------------------------------------
    def cost(self, dims: LayerDims) -> Tuple[int, int]:
        raise NotImplementedError

    # reference-compatible entry points -------------------------------------------------------------
    def linear(self, batch_size, f_out, f_in) -> Tuple[int, int]:
        return self.cost(LayerDims(batch_size, f_out, f_in, (f_out, f_in)))

    def conv2d(self, batch_size, c_out, c_in, kh, kw, f_in, f_out) -> Tuple[int, int]:
        return self.cost(LayerDims(batch_size, c_out, c_in * kh * kw, (c_out, c_in, kh, kw),
                                   in_positions=f_in, out_positions=f_out, c_in=c_in, is_conv=True))

    def attn(self, seq_len, batch_size, emb_dim, num_heads) -> Tuple[int, int]:
        flop, numel = self.linear(seq_len * batch_size, emb_dim, emb_dim)
        return flop * 4, numel * 4  # q, k, v and output projections


@contextmanager
def set_counter(model: nn.Module, counters: List[Counter], batch_size=32, seq_len=128, keys=None):
    """Accumulates the counters over all supported layers of ``model``.  Linear and attention
    layers are counted immediately; convolutions are counted in a forward hook (their spatial
    sizes are only known then), so run one forward pass inside the context::

        with set_counter(model, [Forward(), KFACStats()]) as counts:
            model(x)
        counts['KFACStats']['flop']
    """
    handles = []
    keys = [type(c).__name__ for c in counters] if keys is None else keys
    counts: Dict[str, Any] = {key: {'flop': 0, 'numel': 0} for key in keys}
    counts['params'] = 0

    def add(module, inputs=None, outputs=None):
        for key, counter in zip(keys, counters):
            flop, numel = counter.count_flop_numel(module, inputs, outputs, batch_size, seq_len)
            counts[key]['flop'] += flop
            counts[key]['numel'] += numel

    try:
        for module in model.modules():
            if type(module) not in Counter.supported_types:
                continue
            if type(module) == nn.Conv2d:
                handles.append(module.register_forward_hook(lambda m, i, o: add(m, i[0], o)))
            else:
                add(module)
            counts['params'] += sum(p.numel() for p in module.parameters())
        yield counts
    finally:
        for handle in handles:
            handle.remove()


def _conv_or_linear_macs(d: LayerDims):
    """Product count used for the three passes (the reference counts convolutions without the
    factor two it uses for Linear)."""
    if d.is_conv:
        return d.batch_size * d.d_in * d.d_out * d.out_positions
    return d.batch_size * d.d_in * d.d_out * 2


class Forward(Counter):
    """Forward pass: one multiply-add per weight and output position; stores the outputs."""

    def cost(self, d):
        return _conv_or_linear_macs(d), d.batch_size * d.d_out * d.out_positions

    def attn(self, seq_len, batch_size, emb_dim, num_heads):
        hd = int(emb_dim / num_heads)
        tokens, heads = seq_len * batch_size, batch_size * num_heads
        scores = heads * seq_len * seq_len
        flop = tokens * emb_dim * 3 * emb_dim * 2          # q, k, v projections
        flop += heads * seq_len * hd * seq_len * 2           # q k^T
        flop += scores * 2 + scores * 3                      # softmax, dropout
        flop += scores * hd * 2                              # attention x v
        flop += tokens * emb_dim * emb_dim * 2               # output projection
        numel = 3 * tokens * emb_dim + 3 * scores + heads * seq_len * hd + tokens * emb_dim
        return flop, numel


class BackwardWeight(Counter):
    """Weight gradient: the same multiply-adds as the forward pass; stores one value per parameter."""

    def cost(self, d):
        return _conv_or_linear_macs(d), d.n_params

    def attn(self, seq_len, batch_size, emb_dim, num_heads):
        tokens = seq_len * batch_size
        flop = tokens * emb_dim * emb_dim * 2 + tokens * emb_dim * 3 * emb_dim * 2
        return flop, 4 * emb_dim * emb_dim


class BackwardInput(Counter):
    """Input gradient: the same multiply-adds as the forward pass; stores one value per input element."""

    def cost(self, d):
        return _conv_or_linear_macs(d), d.batch_size * (d.c_in * d.in_positions if d.is_conv else d.d_in)

    def attn(self, seq_len, batch_size, emb_dim, num_heads):
        hd = emb_dim / num_heads
        tokens, heads = seq_len * batch_size, batch_size * num_heads
        scores = heads * seq_len * seq_len
        flop = tokens * emb_dim * emb_dim * 2                # output projection
        flop += 2 * scores * hd * 2                          # d(attention x v)
        flop += scores * 2 + scores * 4                      # dropout, softmax
        flop += 2 * scores * hd * 2                          # dq, dk
        flop += tokens * emb_dim * 3 * emb_dim * 2           # q, k, v projections
        numel = 4 * heads * seq_len * hd + 3 * scores + tokens * emb_dim
        return flop, numel


class AdamStats(Counter):
    """square, two scalings and one add per element."""

    def cost(self, d):
        return d.n_params * 4, d.n_params

    def attn(self, seq_len, batch_size, emb_dim, num_heads):
        n = 4 * emb_dim * emb_dim
        return n * 4, n


class AdamPrecond(Counter):
    """sqrt and divide per element."""

    def cost(self, d):
        return d.n_params * 2, 0


def _im2col_flop(d: LayerDims):
    return d.batch_size * d.c_in * d.d_out * d.out_positions if d.is_conv else 0


class KFACStats(Counter):
    """K-FAC statistics: patch extraction for convolutions plus the two Gram products ``a^T a`` (d_in^2 per
    sample) and ``g^T g`` (d_out^2 per sample); stores both factors."""

    def cost(self, d):
        a, b = d.d_in ** 2, d.d_out ** 2
        return _im2col_flop(d) + d.batch_size * (a + b) * 2, a + b


class KFACInv(Counter):
    """K-FAC inverses: n^3 per factor (Cholesky factorisation, triangular inverse and product)."""

    def cost(self, d):
        return d.d_in ** 3 + d.d_out ** 3, d.d_in ** 2 + d.d_out ** 2


class KFACPrecond(Counter):
    """K-FAC preconditioning ``B^-1 G A^-1``: two matrix products per layer."""

    def cost(self, d):
        return d.d_in * d.d_in * d.d_out * 2 + d.d_in * d.d_out * d.d_out * 2, 0


def _prod(shape):
    out = 1
    for s in shape:
        out *= s
    return out


class ShampooStats(Counter):
    """Shampoo statistics: for every tensor mode of size s the contraction of the gradient with itself over
    the other modes (2 * numel * s operations, s^2 stored values)."""

    @staticmethod
    def flop(*shape):
        return sum(_prod(shape) * s * 2 for s in shape)

    @staticmethod
    def numel(*shape):
        return sum(s ** 2 for s in shape)

    def cost(self, d):
        return self.flop(*d.weight_shape), self.numel(*d.weight_shape)


class ShampooInv(Counter):
    """Eigendecomposition-based root: (9 + 1/3) n^3 per factor."""

    @staticmethod
    def flop(*shape):
        return math.ceil(sum((9 + 1 / 3) * s ** 3 for s in shape))

    @staticmethod
    def numel(*shape):
        return sum(s ** 2 * 2 + s for s in shape)

    def cost(self, d):
        return self.flop(*d.weight_shape), self.numel(*d.weight_shape)


class ShampooPrecond(Counter):
    """Shampoo preconditioning: one mode product with an s x s root per tensor mode."""

    @staticmethod
    def flop(*shape):
        return sum(_prod(shape) * s * 2 for s in shape)

    def cost(self, d):
        return self.flop(*d.weight_shape), 0


class LBFGSPrecond(Counter):
    """Two-loop recursion: five axpy/dot passes per history entry."""

    def __init__(self, hist_size=20):
        self.hist_size = hist_size

    def flop(self, nparams):
        return nparams * 2 * 5 * self.hist_size

    def numel(self, nparams):
        return nparams * 2 * self.hist_size

    def cost(self, d):
        return self.flop(d.n_params), self.numel(d.n_params)


class SMWNGStats(Counter):
    """Sherman-Morrison-Woodbury natural gradient statistics: the n x n Gram matrices of inputs and
    output gradients (n = batch size) and their element-wise product."""

    def cost(self, d):
        n2 = d.batch_size ** 2
        if d.is_conv:
            return _im2col_flop(d) + n2 * d.d_in + n2 * d.d_out, n2
        return n2 * d.d_in * 2 + n2 * d.d_out * 2, n2


class SMWNGPrecond(Counter):
    """SMW natural gradient solve: Cholesky solve of the n x n kernel and the two reductions around it."""

    @staticmethod
    def flop(n):
        return n ** 2 + 1 / 3 * n ** 3 + n ** 2  # Gram row sums + Cholesky solve

    @staticmethod
    def numel(n):
        return n

    def cost(self, d):
        return self.flop(d.batch_size), self.numel(d.batch_size)
