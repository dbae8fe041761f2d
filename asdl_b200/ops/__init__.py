"""Numerical primitives with two implementations each:

  * a plain PyTorch one (any device / dtype) that doubles as the oracle in the tests, and
  * the library's sm_100a CUDA kernels (tcgen05 GEMM/SYRK fed by TMA, bf16 staging kernels,
    fp32 Cholesky inverse, fused elementwise epilogues), used automatically for CUDA tensors.

The CUDA path never falls back silently: if a CUDA tensor is passed and the extension cannot be
loaded an ImportError is raised.  ``set_backend('torch')`` selects the PyTorch implementation
explicitly (used to build reference results on the GPU).

What each primitive stands in for in the reference (file:line inside its project):
  * ``gram`` / ``matmul_tn``: asdl/operations/linear.py:77,89 (A = a^T a, B = g^T g),
    asdl/precondition/shampoo.py:335-339 (mode statistics);
  * ``conv_patch_gram``: asdl/utils.py:51-88 (im2col) + asdl/operations/conv.py:80-88;
  * ``kron_apply``: asdl/symmatrix.py:536-548 (B W A) and asdl/precondition/shampoo.py:351-367;
  * ``spd_inverse`` / ``spd_inverse_grouped``: asdl/utils.py:91-96 (cholesky_inv);
  * ``unitwise_inverse``: asdl/symmatrix.py:687-698;
  * ``eigh`` / ``eigvalsh``: the ``torch.linalg.eigh`` calls of asdl/operations/linear.py:103-118,
    asdl/precondition/newton.py:43, asdl/mvp.py:140 (matrices up to 128 x 128: the library's batched
    Jacobi kernel);
  * ``layernorm_unitwise_stats``: asdl/operations/layernorm.py:70-78;
  * ``diag_linear_stats``: asdl/operations/linear.py:57-66;
  * ``batchnorm_unitwise_stats``: asdl/operations/batchnorm.py:11-55;
  * ``batch_norm_train`` / ``layer_norm``: the models' own normalisation layers (no reference
    counterpart; PyTorch's kernels were the hot spot of the benchmark models).

Precision policy of the tensor-core products (``set_precision``):
  * ``'auto'``   : bf16/fp16 inputs -> one bf16 pass (fp32 accumulation);
                   fp32 inputs      -> three bf16 passes on hi/lo splits ("bf16x3", ~2^-16 relative);
  * ``'bf16'``   : always one pass;  ``'bf16x3'``: always three passes.
"""
from typing import Optional

import os

import torch

from . import _build

__all__ = ['gram', 'matmul_tn', 'split3', 'matmul_fp32_tc', 'eigh', 'eigvalsh', 'layernorm_unitwise_stats',
           'diag_linear_stats', 'kron_apply', 'conv_patch_gram', 'spd_inverse', 'spd_inverse_grouped', 'damped_cholesky',
           'unitwise_inverse', 'batchnorm_unitwise_stats', 'batchnorm_unitwise_stats_from_input',
           'batch_norm_train', 'layer_norm',
           'set_backend', 'get_backend', 'set_precision', 'get_precision', 'extension',
           'cuda_kernels_enabled', 'check_status']

_backend = 'auto'      # 'auto' | 'torch'
_precision = 'auto'    # 'auto' | 'bf16' | 'bf16x3'
_ext = None

#: which of the library's grouped SPD inverses runs on CUDA: ``'tensor_core'`` (128-wide panels, every
#: O(n^3) product on the tcgen05 GEMM from three-way bf16 splits) or ``'cuda_core'`` (64-wide
#: panels, fp32 FMA tile products)
CHOLESKY_BACKEND = 'tensor_core'



def set_backend(name: str):
    global _backend
    if name not in ('auto', 'torch'):
        raise ValueError("backend has to be 'auto' or 'torch'")
    _backend = name


def get_backend():
    return _backend


def set_precision(name: str):
    global _precision
    if name not in ('auto', 'bf16', 'bf16x3'):
        raise ValueError("precision has to be 'auto', 'bf16' or 'bf16x3'")
    _precision = name


def get_precision():
    return _precision


def extension():
    """The compiled extension module (built in-tree on first use)."""
    global _ext
    if _ext is None:
        _ext = _build.load()
        tiles = os.environ.get('ASDL_B200_GEMM_TILES')   # tile policy of the GEMM, see set_gemm_tiles
        if tiles is not None:
            _ext.set_gemm_wide(int(tiles))
    return _ext


def set_gemm_tiles(mode: int = -1):
    """Tile policy of the tcgen05 GEMM's single-problem launches: 0 = 128 x 128 tiles, 1 / 2 = 128 x 256
    tiles for large / all outputs, 3 = 256 x 256 tiles on CTA pairs (``cta_group::2``) for large
    products and 128 x 128 otherwise (the default, also -1), 4 = CTA pairs for every product.  The
    environment variable ``ASDL_B200_GEMM_TILES`` sets the initial policy."""
    extension().set_gemm_wide(int(mode))


def cuda_kernels_enabled(*tensors):
    """True when the custom kernels should handle these tensors."""
    if _backend == 'torch':
        return False
    return all(t.is_cuda for t in tensors) and all(
        t.dtype in (torch.float32, torch.bfloat16, torch.float16) for t in tensors)


def check_status(device=None):
    """Raises if a kernel reported a problem (timed-out wait, non-SPD matrix) since the last
    check.  Synchronises the current stream."""
    if not torch.cuda.is_available():
        return
    dev = torch.cuda.current_device() if device is None else torch.device(device).index
    code = extension().read_status(dev or 0)
    if code != 0:
        names = {1: 'timed out waiting for a TMA stage', 2: 'timed out waiting for a free stage',
                 3: 'timed out waiting for the accumulator', 4: 'timed out waiting for a peer GPU',
                 5: 'matrix is not positive definite', 6: 'bad argument'}
        raise RuntimeError(f'asdl_b200 CUDA kernel error {code}: {names.get(code, "unknown")}')


# --------------------------------------------------------------------------------------------
# staging helpers
# --------------------------------------------------------------------------------------------
def _round_up(v, m):
    return (v + m - 1) // m * m


def _use_x3(dtype):
    if _precision == 'bf16':
        return False
    if _precision == 'bf16x3':
        return True
    return dtype == torch.float32


def _stage_bf16(x: torch.Tensor, want_lo: bool):
    """[rows, n] -> bf16 operand(s) with a 16-byte aligned row pitch.  Returns (hi, lo|None),
    both views [rows, n] into padded storage."""
    rows, n = x.shape
    if (not want_lo and x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        return x, None
    ld = _round_up(max(n, 8), 8)
    hi = torch.empty(rows, ld, device=x.device, dtype=torch.bfloat16)
    lo = torch.empty_like(hi) if want_lo else None
    src = x if x.stride(1) == 1 else x.contiguous()
    extension().cast_pad_bf16(src, hi, lo, 1.0)
    return hi[:, :n], (lo[:, :n] if want_lo else None)


def _segments(a_hi, a_lo, b_hi, b_lo):
    if a_lo is None or b_lo is None:
        return [a_hi], [b_hi]
    return [a_hi, a_hi, a_lo], [b_hi, b_lo, b_hi]


# --------------------------------------------------------------------------------------------
# products
# --------------------------------------------------------------------------------------------
def _f32(t: torch.Tensor) -> torch.Tensor:
    """Half-precision tensors as fp32 (the PyTorch paths accumulate and return fp32, like the kernels do)."""
    return t.float() if t.dtype in (torch.bfloat16, torch.float16) else t


def split3(x: torch.Tensor):
    """fp32 [rows, n] -> three bf16 parts (hi, mid, lo) with hi + mid + lo == x to 24 bits, as views
    [rows, n] into storage whose row pitch is a multiple of 64 elements (CUDA only)."""
    rows, n = x.shape
    ld = _round_up(max(n, 8), 64)
    parts = [torch.empty(rows, ld, device=x.device, dtype=torch.bfloat16) for _ in range(3)]
    src = x if (x.stride(1) == 1 and x.dtype == torch.float32) else x.float().contiguous()
    extension().cast_split3(src, *parts)
    return [p[:, :n] for p in parts]


def matmul_fp32_tc(a_parts, b_parts, a_kmajor: bool, b_kmajor: bool, out=None, alpha: float = 1.0, beta: float = 0.0,
                   sym: bool = False, out_parts=None):
    """fp32-grade product on the bf16 tensor cores from three-way splits of both operands
    (``a_parts`` / ``b_parts``: the (hi, mid, lo) triples of :func:`split3`): the kernel loads the
    six part tiles of a K block once, issues the six significant part products
    small-magnitude-first into a fresh TMEM accumulator and adds every K block to a running fp32
    sum in registers.  ``out_parts``: optional (hi, mid, lo) bf16 buffers that receive the split of
    the result from the epilogue."""
    oh, om, ol = out_parts if out_parts is not None else (None, None, None)
    extension().umma_gemm(list(a_parts), list(b_parts), a_kmajor, b_kmajor, out, float(alpha), float(beta), sym,
                          oh, ol, 1, om, True)
    return out


def gram(x: torch.Tensor, scale: float = 1.0, out: Optional[torch.Tensor] = None,
         beta: float = 0.0) -> torch.Tensor:
    """``scale * x^T x (+ beta * out)`` for a sample matrix x [rows, n] -> [n, n].

    This is the Kronecker-factor product of K-FAC (A = a^T a, B = g^T g) and Shampoo's R = G^T G.
    CUDA: tcgen05 SYRK (lower-triangular tiles mirrored in the epilogue, split-K over rows,
    the EMA ``beta`` folded into the epilogue); the result is fp32 and exactly symmetric."""
    if x.ndim != 2:
        raise ValueError(f'x has to be 2-D. Got {x.ndim}-D.')
    if not cuda_kernels_enabled(x) or x.shape[0] == 0:
        x = _f32(x)
        prod = (x.T @ x) * scale if scale != 1.0 else x.T @ x
        if out is None:
            return prod
        if beta != 0.0:
            out.mul_(beta).add_(prod.to(out.dtype))
        else:
            out.copy_(prod)
        return out
    hi, lo = _stage_bf16(x, _use_x3(x.dtype))
    n = x.shape[1]
    if out is None:
        out = torch.empty(n, n, device=x.device, dtype=torch.float32)
        beta = 0.0
    a_segs, b_segs = _segments(hi, lo, hi, lo)
    extension().umma_gemm(a_segs, b_segs, False, False, out, float(scale), float(beta), True,
                          None, None, 0)
    return out


def matmul_tn(a: torch.Tensor, b: torch.Tensor, scale: float = 1.0,
              out: Optional[torch.Tensor] = None, beta: float = 0.0) -> torch.Tensor:
    """``scale * a^T b (+ beta*out)`` with a: [k, m], b: [k, n] (both "sample-major")."""
    if not cuda_kernels_enabled(a, b) or a.shape[0] == 0:
        prod = (_f32(a).T @ _f32(b)) * scale
        if out is None:
            return prod
        return out.mul_(beta).add_(prod.to(out.dtype)) if beta != 0.0 else out.copy_(prod)
    x3 = _use_x3(a.dtype) or _use_x3(b.dtype)
    a_hi, a_lo = _stage_bf16(a, x3)
    b_hi, b_lo = _stage_bf16(b, x3)
    if out is None:
        out = torch.empty(a.shape[1], b.shape[1], device=a.device, dtype=torch.float32)
        beta = 0.0
    a_segs, b_segs = _segments(a_hi, a_lo, b_hi, b_lo)
    extension().umma_gemm(a_segs, b_segs, False, False, out, float(scale), float(beta), False,
                          None, None, 0)
    return out


def matmul(a: torch.Tensor, b: torch.Tensor, trans_a: bool = False, trans_b: bool = False, alpha: float = 1.0,
           out: Optional[torch.Tensor] = None, beta: float = 0.0, sym: bool = False) -> torch.Tensor:
    """``alpha * op(a) op(b) (+ beta * out)`` for row-major matrices, op = transpose where asked.  No operand
    is copied for its layout: the tcgen05 GEMM takes either operand K-major or MN-major.  ``sym``: the
    result is known to be symmetric (a a^T, a^T a); only its lower tiles are multiplied and mirrored."""
    if not cuda_kernels_enabled(a, b) or a.numel() == 0 or b.numel() == 0:
        prod = (_f32(a).T if trans_a else _f32(a)) @ (_f32(b).T if trans_b else _f32(b))
        if alpha != 1.0:
            prod = prod * alpha
        if out is None:
            return prod
        return out.mul_(beta).add_(prod.to(out.dtype)) if beta != 0.0 else out.copy_(prod)
    x3 = _use_x3(a.dtype) or _use_x3(b.dtype)
    a_hi, a_lo = _stage_bf16(a, x3)
    b_hi, b_lo = (a_hi, a_lo) if b is a else _stage_bf16(b, x3)
    m = a.shape[1] if trans_a else a.shape[0]
    n = b.shape[0] if trans_b else b.shape[1]
    if out is None:
        out = torch.empty(m, n, device=a.device, dtype=torch.float32)
        beta = 0.0
    a_segs, b_segs = _segments(a_hi, a_lo, b_hi, b_lo)
    # A operand: stored [m, k] (not transposed) is K-major; B operand: stored [n, k] (transposed) is K-major
    extension().umma_gemm(a_segs, b_segs, not trans_a, trans_b, out, float(alpha), float(beta), bool(sym), None, None, 0)
    return out


def matmul_nn(a: torch.Tensor, b: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """``scale * a b`` with a: [m, k], b: [k, n] in their natural row-major layouts (a is the K-major
    operand of the tcgen05 GEMM, b the MN-major one: no transpose copy)."""
    if not cuda_kernels_enabled(a, b) or a.numel() == 0 or b.numel() == 0:
        prod = _f32(a) @ _f32(b)
        return prod * scale if scale != 1.0 else prod
    x3 = _use_x3(a.dtype) or _use_x3(b.dtype)
    a_hi, a_lo = _stage_bf16(a, x3)
    b_hi, b_lo = _stage_bf16(b, x3)
    out = torch.empty(a.shape[0], b.shape[1], device=a.device, dtype=torch.float32)
    a_segs, b_segs = _segments(a_hi, a_lo, b_hi, b_lo)
    extension().umma_gemm(a_segs, b_segs, True, False, out, float(scale), 0.0, False, None, None, 0)
    return out


def gram_hadamard(kernel: torch.Tensor, a1: torch.Tensor, g1: torch.Tensor, a2: Optional[torch.Tensor] = None,
                  g2: Optional[torch.Tensor] = None, one: float = 0.0, scale: float = 1.0) -> torch.Tensor:
    """``kernel += scale * (a1 a2^T + one) o (g1 g2^T)``: one layer's term of the Hadamard-factored
    Gram / NTK matrix (asdl/operations/operation.py:335-351).  a*: layer inputs [n, d_in], g*: output
    gradients [n, d_out] of the two example sets (the second defaults to the first); ``one`` = 1 for a
    layer with a bias.

    CUDA: one launch; every CTA forms both 128 x 128 Gram tiles in its two TMEM accumulators and
    multiplies them in the epilogue, so neither Gram matrix is written to memory.  fp32 inputs are
    split into (hi, lo) bf16 parts and every Gram is the sum of three part products."""
    a2 = a1 if a2 is None else a2
    g2 = g1 if g2 is None else g2
    if (not cuda_kernels_enabled(kernel, a1, g1) or kernel.dtype != torch.float32 or kernel.ndim != 2
            or kernel.stride(1) != 1 or a1.shape[1] == 0 or g1.shape[1] == 0):
        A = _f32(a1) @ _f32(a2).T
        B = _f32(g1) @ _f32(g2).T
        if scale != 1.0:
            B = B * scale
        kernel += B.mul(A + one if one != 0.0 else A).to(kernel.dtype)
        return kernel
    x3 = _use_x3(a1.dtype) or _use_x3(g1.dtype)

    def parts(t):
        return [p for p in _stage_bf16(t, x3) if p is not None]

    pa1, pg1 = parts(a1), parts(g1)
    pa2 = pa1 if a2 is a1 else parts(a2)
    pg2 = pg1 if g2 is g1 else parts(g2)
    if len(pa1) != len(pa2):      # one side was already an aligned bf16 matrix: use single parts on both
        pa1, pa2 = pa1[:1], pa2[:1]
    if len(pg1) != len(pg2):
        pg1, pg2 = pg1[:1], pg2[:1]
    extension().gram_hadamard(pa1, pa2, pg1, pg2, kernel, float(scale), float(one))
    return kernel


def kron_apply(left: torch.Tensor, mid: torch.Tensor, right: torch.Tensor) -> torch.Tensor:
    """``left @ mid @ right`` with symmetric ``left`` [m, m] and ``right`` [n, n]: the K-FAC
    preconditioning step B^-1 . grad . A^-1 (also used un-inverted for curvature products).

    CUDA: two chained tcgen05 GEMMs.  The symmetry of the outer matrices lets both be read in
    their stored row-major layout as MN-major operands; the intermediate is written by the first
    GEMM's epilogue directly as bf16 hi/lo pairs in the K-major layout the second one consumes."""
    if not cuda_kernels_enabled(left, mid, right) or mid.numel() == 0:
        dt = mid.dtype
        return left.to(dt) @ mid @ right.to(dt)
    ext = extension()
    m, n = mid.shape
    x3 = _use_x3(torch.float32) if (left.dtype == torch.float32 or mid.dtype == torch.float32) \
        else _use_x3(mid.dtype)
    l_hi, l_lo = _stage_bf16(left, x3)
    g_hi, g_lo = _stage_bf16(mid, x3)
    r_hi, r_lo = _stage_bf16(right, x3)
    ld = _round_up(max(n, 8), 8)
    t_hi = torch.empty(m, ld, device=mid.device, dtype=torch.bfloat16)
    t_lo = torch.empty_like(t_hi) if x3 else None
    # T = left^T-as-stored . mid : A operand = left ([k=m, m] row-major, symmetric), B = mid [k=m, n]
    out = torch.empty(m, n, device=mid.device, dtype=torch.float32)
    if x3:   # (hi, lo) parts, loaded once per K block by the x3wide flavour
        ext.umma_gemm([l_hi, l_lo], [g_hi, g_lo], False, False, None, 1.0, 0.0, False, t_hi, t_lo, 0, None, False, True)
        ext.umma_gemm([t_hi[:, :n], t_lo[:, :n]], [r_hi, r_lo], True, False, out, 1.0, 0.0, False, None, None, 0,
                      None, False, True)
        return out.to(mid.dtype) if mid.dtype != torch.float32 else out
    ext.umma_gemm([l_hi], [g_hi], False, False, None, 1.0, 0.0, False, t_hi, t_lo, 0)
    # Y = T . right : A operand = T ([m, k=n] K-major), B = right ([k=n, n] row-major, symmetric)
    ext.umma_gemm([t_hi[:, :n]], [r_hi], True, False, out, 1.0, 0.0, False, None, None, 0)
    return out.to(mid.dtype) if mid.dtype != torch.float32 else out


#: stride-1 convolutions on channels_last bf16 inputs with a multiple of 64 channels: gather the patch tiles
#: inside the SYRK (4-D TMA boxes) instead of writing the patch matrix to memory first
IMPLICIT_IM2COL = os.environ.get('ASDL_B200_IMPLICIT_IM2COL', '1') != '0'
#: ... when the patch matrix would take at least this many MiB.  Measured on single layers (32 images): at 56 x 56 x 64
#: channels (110 MiB of patches) the implicit SYRK takes the time of im2col + SYRK (0.128 vs 0.124 ms); on the small
#: maps of deep layers (14 x 14 x 256: 28 MiB) the 4-D boxes of 2 x 2 pixels x 16 images load at half the rate of the
#: 2-D boxes of an explicit matrix (0.144 vs 0.077 ms), so those keep the explicit path.
IMPLICIT_IM2COL_MIN_MB = float(os.environ.get('ASDL_B200_IMPLICIT_IM2COL_MIN_MB', '64'))


def implicit_im2col_eligible(x: torch.Tensor, kernel, stride, dilation, padding, out_hw, khwc_order: bool) -> bool:
    """True when the input-side factor of this convolution is formed without a patch matrix (4-D TMA gather
    inside the SYRK): stride 1, no dilation, channels_last bf16 input with a multiple of 64 channels, at most 12
    filter taps, (kh, kw, c) column order, and a patch matrix large enough for the saved memory traffic to pay."""
    (kh, kw), (sh, sw), (dh, dw), (ph, pw), (ho, wo) = kernel, stride, dilation, padding, out_hw
    n, c = x.shape[0], x.shape[1]
    return bool(IMPLICIT_IM2COL and khwc_order and x.is_cuda and x.dtype == torch.bfloat16 and not _use_x3(x.dtype)
                and sh == sw == dh == dw == 1 and c % 64 == 0 and kh * kw <= 12 and ph < kh and pw < kw
                and ho > ph and wo > pw and x.is_contiguous(memory_format=torch.channels_last)
                and n * ho * wo * c * kh * kw * 2 >= IMPLICIT_IM2COL_MIN_MB * 2 ** 20)


def conv_patch_gram(x: torch.Tensor, conv: torch.nn.Conv2d, scale: float = 1.0,
                    out: Optional[torch.Tensor] = None, beta: float = 0.0,
                    channels_last_order: bool = False) -> torch.Tensor:
    """K-FAC A factor of a convolution straight from its input:
    ``scale * M M^T`` with M the (c_in*kh*kw) x (n*h_out*w_out) patch matrix.

    ``channels_last_order=False`` orders rows/columns as (c, kh, kw) (matching
    ``weight.view(c_out, -1)``); ``True`` uses (kh, kw, c), the order of a channels_last weight.
    CUDA: stride-1 convolutions on channels_last bf16 inputs with a multiple of 64 channels whose patch matrix
    would take ``IMPLICIT_IM2COL_MIN_MB`` or more never form it - the SYRK's producer gathers 8 x 8 pixel blocks of one filter tap with 4-D TMA boxes, padding
    and image edges being TMA's zero fill (``IMPLICIT_IM2COL``); 1x1 stride-1 convolutions read the activations
    in place; everything else goes through a bf16 im2col kernel (vectorised for channels_last inputs).  fp32 inputs are
    staged as bf16 hi/lo patch pairs and multiplied in three passes (precision policy 'auto')."""
    from ..utils import im2col_2d, _conv_geometry, _explicit_padding
    (kh, kw), (sh, sw), _, (dh, dw) = _conv_geometry(conv)
    if not cuda_kernels_enabled(x):
        patches = im2col_2d(_f32(x), conv)  # n x (c kh kw) x L
        if channels_last_order:
            n, _, L = patches.shape
            patches = patches.view(n, x.shape[1], kh * kw, L).permute(0, 2, 1, 3).reshape(n, -1, L)
        rows = patches.permute(0, 2, 1).reshape(-1, patches.shape[1])
        return gram(rows, scale=scale, out=out, beta=beta)
    x, (ph, pw) = _explicit_padding(x, conv)   # reflect / replicate / circular padding becomes part of the input
    n, c, h, w = x.shape
    ho = (h + 2 * ph - dh * (kh - 1) - 1) // sh + 1
    wo = (w + 2 * pw - dw * (kw - 1) - 1) // sw + 1
    ncol = c * kh * kw
    pointwise = (kh == 1 and kw == 1 and sh == 1 and sw == 1 and ph == 0 and pw == 0)
    if (pointwise and x.dtype == torch.bfloat16 and x.is_contiguous(memory_format=torch.channels_last)
            and c % 8 == 0 and not _use_x3(x.dtype)):
        rows = x.permute(0, 2, 3, 1).reshape(n * h * w, c)  # a view: NHWC memory is already [rows, c]
        return gram(rows, scale=scale, out=out, beta=beta)
    if (implicit_im2col_eligible(x, (kh, kw), (sh, sw), (dh, dw), (ph, pw), (ho, wo), channels_last_order)
            and (out is None or (out.dtype == torch.float32 and out.stride(1) == 1))):
        # no patch matrix: the SYRK's producer gathers its operand tiles from x with 4-D TMA boxes
        if out is None:
            out = torch.empty(ncol, ncol, device=x.device, dtype=torch.float32)
            beta = 0.0
        extension().umma_syrk_conv(x, out, kh, kw, ph, pw, float(scale), float(beta), 0)
        return out
    ld = _round_up(max(ncol, 8), 8)
    x3 = _use_x3(x.dtype)
    patches = torch.empty(n * ho * wo, ld, device=x.device, dtype=torch.bfloat16)
    patches_lo = torch.empty_like(patches) if x3 else None
    extension().im2col_bf16(x, patches, patches_lo, [kh, kw], [sh, sw], [ph, pw], [dh, dw],
                            not channels_last_order)
    if not x3:
        return gram(patches[:, :ncol], scale=scale, out=out, beta=beta)
    hi, lo = patches[:, :ncol], patches_lo[:, :ncol]
    if out is None:
        out = torch.empty(ncol, ncol, device=x.device, dtype=torch.float32)
        beta = 0.0
    extension().umma_gemm([hi, hi, lo], [hi, lo, hi], False, False, out, float(scale), float(beta),
                          True, None, None, 0)
    return out


# --------------------------------------------------------------------------------------------
# inverses
# --------------------------------------------------------------------------------------------
#: a factorisation that breaks down is retried with the damping multiplied by this, this many times
DAMPING_ESCALATION, DAMPING_ESCALATION_TRIES = 10.0, 6


def damped_cholesky(mat: torch.Tensor, damping) -> torch.Tensor:
    """Lower Cholesky factor of ``mat + damping*I`` (PyTorch path).  A matrix that is not positive
    definite at that damping (rounding in an ill-conditioned factor, a negative curvature estimate) is
    retried with 10x the damping, up to six times, with a warning that names the damping finally used;
    non-finite entries raise at once, since no damping repairs them."""
    eye = torch.eye(mat.shape[-1], device=mat.device, dtype=mat.dtype)
    damping = damping.to(mat.dtype) if isinstance(damping, torch.Tensor) else damping
    chol, info = torch.linalg.cholesky_ex(mat + damping * eye)
    if not bool(info.any()):
        return chol
    if not bool(torch.isfinite(mat).all()):
        raise torch.linalg.LinAlgError(f'a {tuple(mat.shape)} curvature matrix has non-finite entries and cannot be '
                                       f'factorised (non-finite activations or gradients in the statistics pass)')
    used = float(damping) if float(damping) > 0 else 1e-8 * float(mat.diagonal(dim1=-2, dim2=-1).abs().max() + 1e-30)
    for _ in range(DAMPING_ESCALATION_TRIES):
        used *= DAMPING_ESCALATION
        chol, info = torch.linalg.cholesky_ex(mat + used * eye)
        if not bool(info.any()):
            import warnings
            warnings.warn(f'a {tuple(mat.shape)} curvature matrix is not positive definite with damping '
                          f'{float(damping):.3g}; factorised with damping {used:.3g} instead.')
            return chol
    raise torch.linalg.LinAlgError(f'a {tuple(mat.shape)} curvature matrix is not positive definite even with damping '
                                   f'{used:.3g} (asked for {float(damping):.3g})')


def spd_inverse(mat: torch.Tensor, damping=0.0) -> torch.Tensor:
    """``(mat + damping*I)^-1`` for symmetric positive (semi-)definite ``mat``; the input is left
    untouched.  ``damping`` may be a Python number or a 0-d / 1-element tensor (kept on the
    device).  CUDA fp32: the library's grouped blocked Cholesky-inverse kernels (``CHOLESKY_BACKEND``)."""
    if cuda_kernels_enabled(mat) and mat.dtype == torch.float32 and mat.ndim == 2:
        out = torch.empty(mat.shape, device=mat.device, dtype=torch.float32)
        spd_inverse_grouped([mat], [out], damping)
        return out
    return torch.cholesky_inverse(damped_cholesky(mat, damping))


def spd_inverse_grouped(mats, outs, damping):
    """``outs[i] <- (mats[i] + damping[i]*I)^-1`` for a list of square fp32 matrices of arbitrary
    sizes.  ``damping``: one number for all, a list of numbers, or a device tensor with one entry
    per matrix (no host synchronisation).  On CUDA all matrices advance together through one
    sequence of grouped kernel launches."""
    count = len(mats)
    if count == 0:
        return outs
    dev = mats[0].device
    if isinstance(damping, torch.Tensor):
        damp = damping.to(device=dev, dtype=torch.float32).reshape(-1)
        if damp.numel() == 1 and count > 1:
            damp = damp.expand(count)
        damp = damp.contiguous()
    elif isinstance(damping, (list, tuple)):
        damp = torch.tensor([float(d) for d in damping], device=dev, dtype=torch.float32)
    else:
        damp = torch.full((count,), float(damping), device=dev, dtype=torch.float32)
    if cuda_kernels_enabled(*mats) and all(m.dtype == torch.float32 for m in mats):
        mats = [m if m.stride(-1) == 1 else m.contiguous() for m in mats]
        if CHOLESKY_BACKEND == 'tensor_core':
            extension().chol_inverse_tc(list(mats), list(outs), damp)
        else:
            extension().chol_inverse(list(mats), list(outs), damp)
        return outs
    for m, o, d in zip(mats, outs, damp):
        o.copy_(torch.cholesky_inverse(damped_cholesky(m, d)))
    return outs


def batchnorm_unitwise_stats(y: torch.Tensor, g: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                             out: Optional[torch.Tensor] = None, alpha: float = 1.0,
                             beta: float = 0.0) -> torch.Tensor:
    """Unit-wise curvature blocks of a BatchNorm layer from its output ``y`` and output gradient
    ``g`` ([n, c, *spatial]):  ``out <- beta * out + alpha * sum_n [[gw^2, gw gb], [gw gb, gb^2]]``
    with per-sample ``gw = sum_spatial ((y - bias) / weight) * g`` and ``gb = sum_spatial g``
    (out: [c, 2, 2] fp32).  CUDA, 4-d channels_last bf16/fp32: one pass over y and g with the
    library's kernel; anything else: PyTorch."""
    c = y.shape[1]
    if out is None:
        out = torch.zeros(c, 2, 2, device=y.device, dtype=torch.float32)
        beta = 0.0
    vec = 8 if y.dtype == torch.bfloat16 else 4
    if (cuda_kernels_enabled(y, g) and y.ndim == 4 and y.dtype in (torch.bfloat16, torch.float32)
            and g.dtype == y.dtype and c % vec == 0 and weight.dtype == torch.float32
            and y.is_contiguous(memory_format=torch.channels_last) and out.is_contiguous()):
        if not g.is_contiguous(memory_format=torch.channels_last):
            g = g.contiguous(memory_format=torch.channels_last)
        extension().bn_unitwise_stats(y, g, weight.detach().contiguous(), bias.detach().contiguous(), out,
                                      float(alpha), float(beta))
        return out
    shape = (1, -1) + (1,) * (y.ndim - 2)
    xh = (y.float() - bias.view(shape)) / weight.view(shape)
    dims = tuple(range(2, y.ndim))
    gw = (xh * g).sum(dim=dims) if dims else xh * g
    gb = g.float().sum(dim=dims) if dims else g.float()
    ww, wb, bb = gw.square().sum(dim=0), (gw * gb).sum(dim=0), gb.square().sum(dim=0)
    new = torch.stack([torch.stack([ww, wb], dim=1), torch.stack([wb, bb], dim=1)], dim=1)
    return out.mul_(beta).add_(new, alpha=alpha)


#: ReLU mask of the fused BatchNorm backward: recomputed from x (True) or read from the saved output (False)
BN_RELU_MASK_FROM_X = os.environ.get('ASDL_B200_BN_MASK_FROM_X', '1') != '0'


class _BatchNormTrain(torch.autograd.Function):
    """Training-mode batch normalisation (+ residual add, + ReLU) on the library's NHWC bf16 kernels."""

    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, num_batches_tracked, momentum, eps,
                residual, relu):
        y, mean, invstd = extension().bn_forward_train(x, weight.detach(), bias.detach(), running_mean,
                                                       running_var, num_batches_tracked, float(momentum),
                                                       float(eps), residual, bool(relu))
        ctx.relu, ctx.has_residual = bool(relu), residual is not None
        # ReLU without a residual: y > 0 exactly when x * scale + shift > 0, so the backward kernels recompute the
        # mask from x (which they read anyway) and the bias, instead of reading y once more in each pass
        ctx.mask_from_x = ctx.relu and not ctx.has_residual and BN_RELU_MASK_FROM_X
        ctx.save_for_backward(x, weight, mean, invstd, *([bias] if ctx.mask_from_x else ([y] if relu else [])))
        ctx.mark_non_differentiable(mean, invstd)
        return y, mean, invstd

    @staticmethod
    def backward(ctx, dy, _dmean, _dinvstd):
        x, weight, mean, invstd, *rest = ctx.saved_tensors
        if not dy.is_contiguous(memory_format=torch.channels_last):
            dy = dy.contiguous(memory_format=torch.channels_last)
        y = rest[0] if (ctx.relu and not ctx.mask_from_x) else None
        bias = rest[0].detach() if ctx.mask_from_x else None
        out = extension().bn_backward_train(x, dy, weight.detach(), mean, invstd, y, ctx.has_residual, bias)
        dx, dweight, dbias = out[:3]
        dres = None
        if ctx.has_residual:
            dres = out[3] if ctx.relu else dy
        return dx, dweight, dbias, None, None, None, None, None, dres, None


def batch_norm_train_supported(x: torch.Tensor, weight, bias, residual=None) -> bool:
    """True when :func:`batch_norm_train` runs on the library's kernels for this input."""
    ok = (weight is not None and bias is not None and cuda_kernels_enabled(x) and x.ndim == 4
          and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.numel() > 0
          and weight.dtype == torch.float32 and bias.dtype == torch.float32
          and x.is_contiguous(memory_format=torch.channels_last))
    if ok and residual is not None:
        ok = (residual.shape == x.shape and residual.dtype == torch.bfloat16
              and residual.is_contiguous(memory_format=torch.channels_last))
    return ok


def batch_norm_train(x, weight, bias, running_mean=None, running_var=None, momentum=0.1, eps=1e-5,
                     residual=None, relu=False, num_batches_tracked=None, return_stats=False):
    """``act(batch_norm(x) + residual)`` with batch statistics (running statistics and the batch
    counter updated in place), differentiable in x, weight, bias and residual.  CUDA, channels_last
    bf16 activations with fp32 parameters: three kernels forward (sums, finalize, transform) and
    three backward, each pass reading / writing every activation once with 16-byte accesses;
    anything else: ``F.batch_norm`` followed by the add and the ReLU.  With ``return_stats`` the
    result is ``(y, mean, invstd)`` (``None`` statistics on the PyTorch path)."""
    if batch_norm_train_supported(x, weight, bias, residual):
        y, mean, invstd = _BatchNormTrain.apply(x, weight, bias, running_mean, running_var,
                                                num_batches_tracked, momentum, eps, residual, relu)
        return (y, mean, invstd) if return_stats else y
    if num_batches_tracked is not None:
        num_batches_tracked.add_(1)
    y = torch.nn.functional.batch_norm(x, running_mean, running_var, weight, bias, True, momentum, eps)
    if residual is not None:
        y = y + residual
    if relu:
        y = torch.relu(y)
    return (y, None, None) if return_stats else y


def batchnorm_unitwise_stats_from_input(x, dy, y, mean, invstd, out, alpha=1.0, beta=0.0):
    """Unit-wise curvature blocks of a BatchNorm layer with a fused activation: the normalised
    input is ``(x - mean) * invstd`` and the output gradient ``dy`` is masked by the ReLU that
    produced ``y`` (``y=None``: no activation).  Same result layout as
    :func:`batchnorm_unitwise_stats`."""
    if (cuda_kernels_enabled(x, dy) and x.ndim == 4 and x.dtype == torch.bfloat16 and dy.dtype == torch.bfloat16
            and x.shape[1] % 8 == 0 and x.is_contiguous(memory_format=torch.channels_last)
            and (y is None or y.is_contiguous(memory_format=torch.channels_last)) and out.is_contiguous()):
        if not dy.is_contiguous(memory_format=torch.channels_last):
            dy = dy.contiguous(memory_format=torch.channels_last)
        extension().bn_unitwise_stats_xhat(x, dy, y, mean, invstd, out, float(alpha), float(beta))
        return out
    shape = (1, -1) + (1,) * (x.ndim - 2)
    xh = (x.float() - mean.view(shape)) * invstd.view(shape)
    g = dy.float() if y is None else dy.float() * (y > 0)
    dims = tuple(range(2, x.ndim))
    gw, gb = (xh * g).sum(dim=dims), g.sum(dim=dims)
    ww, wb, bb = gw.square().sum(dim=0), (gw * gb).sum(dim=0), gb.square().sum(dim=0)
    new = torch.stack([torch.stack([ww, wb], dim=1), torch.stack([wb, bb], dim=1)], dim=1)
    return out.mul_(beta).add_(new, alpha=alpha)


class _LayerNormFn(torch.autograd.Function):
    """LayerNorm over the last dimension on the library's bf16 kernels."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        y, mean, rstd = extension().ln_forward(x, weight.detach(), bias.detach(), float(eps))
        ctx.save_for_backward(x, weight, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, mean, rstd = ctx.saved_tensors
        dx, dweight, dbias = extension().ln_backward(x, dy.contiguous(), weight.detach(), mean, rstd)
        return dx, dweight, dbias, None


_LN_SIZES = {256 * v for v in (1, 2, 3, 4, 6, 8, 12, 16)}


def layer_norm_supported(x: torch.Tensor, weight, bias) -> bool:
    return (weight is not None and bias is not None and weight.ndim == 1 and cuda_kernels_enabled(x)
            and x.dtype == torch.bfloat16 and x.is_contiguous() and x.numel() > 0
            and x.shape[-1] == weight.numel() and weight.numel() in _LN_SIZES
            and weight.dtype == torch.float32 and bias.dtype == torch.float32)


def layer_norm(x, weight, bias, eps=1e-5):
    """LayerNorm over the last dimension, differentiable.  CUDA, contiguous bf16 input with fp32
    parameters and a feature size of 256 * {1, 2, 3, 4, 6, 8, 12, 16}: one kernel forward, two
    backward (the input gradient and the weight / bias gradients come out of one pass over dy and
    x); anything else: ``F.layer_norm``."""
    if layer_norm_supported(x, weight, bias):
        return _LayerNormFn.apply(x, weight, bias, eps)
    return torch.nn.functional.layer_norm(x, (weight.numel(),) if weight is not None else x.shape[-1:],
                                          weight, bias, eps)


#: largest matrix the Jacobi eigensolver kernel takes (it keeps the matrix and the vectors in shared memory)
JACOBI_MAX_N = 160


def _jacobi_ok(mat: torch.Tensor) -> bool:
    return (cuda_kernels_enabled(mat) and mat.dtype == torch.float32 and mat.ndim in (2, 3)
            and mat.shape[-1] == mat.shape[-2] and 1 <= mat.shape[-1] <= JACOBI_MAX_N)


def eigh(mat: torch.Tensor):
    """``(eigenvalues ascending, eigenvectors as columns)`` of a symmetric matrix or a batch of them.
    CUDA fp32 up to 160 x 160: the library's batched parallel-Jacobi kernel (one CTA per matrix, the
    input is symmetrised on load); anything else: ``torch.linalg.eigh``."""
    if _jacobi_ok(mat):
        batched = mat.ndim == 3
        w, v = extension().jacobi_eigh((mat if batched else mat.unsqueeze(0)).contiguous(), True)
        return (w, v) if batched else (w[0], v[0])
    return torch.linalg.eigh(mat)


def eigvalsh(mat: torch.Tensor) -> torch.Tensor:
    """Eigenvalues (ascending) of a symmetric matrix or a batch of them; see :func:`eigh`."""
    if _jacobi_ok(mat):
        batched = mat.ndim == 3
        w, _ = extension().jacobi_eigh((mat if batched else mat.unsqueeze(0)).contiguous(), False)
        return w if batched else w[0]
    return torch.linalg.eigvalsh(mat)


def layernorm_unitwise_stats(y: torch.Tensor, g: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
                             out: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0) -> torch.Tensor:
    """Unit-wise curvature blocks of a LayerNorm over the last dimension from its output ``y`` and output
    gradient ``g`` ([..., d]): ``out <- beta * out + alpha * sum_rows [[gw^2, gw gb], [gw gb, gb^2]]`` with
    ``gw = (y - bias) / weight * g`` and ``gb = g`` per feature (out: [d, 2, 2] fp32).  CUDA bf16 / fp32:
    one pass over y and g with the library's kernel; anything else: PyTorch."""
    d = weight.numel()
    if out is None:
        out = torch.zeros(d, 2, 2, device=y.device, dtype=torch.float32)
        beta = 0.0
    if (cuda_kernels_enabled(y, g) and weight.ndim == 1 and y.shape[-1] == d and y.dtype == g.dtype
            and y.dtype in (torch.bfloat16, torch.float32) and weight.dtype == torch.float32 and out.is_contiguous()):
        extension().ln_unitwise_stats(y.reshape(-1, d).contiguous(), g.reshape(-1, d).contiguous(),
                                      weight.detach().contiguous(), bias.detach().contiguous(), out,
                                      float(alpha), float(beta))
        return out
    k = weight.ndim
    xh = (y.float() - bias) / weight
    gw = (xh * g).reshape(-1, *y.shape[-k:]).flatten(start_dim=1)
    gb = g.float().reshape(-1, *y.shape[-k:]).flatten(start_dim=1)
    ww, wb, bb = gw.square().sum(dim=0), (gw * gb).sum(dim=0), gb.square().sum(dim=0)
    new = torch.stack([torch.stack([ww, wb], dim=1), torch.stack([wb, bb], dim=1)], dim=1)
    return out.mul_(beta).add_(new, alpha=alpha)


def diag_linear_stats(a: torch.Tensor, g: torch.Tensor, out: Optional[torch.Tensor] = None,
                      out_bias: Optional[torch.Tensor] = None, alpha: float = 1.0, beta: float = 0.0):
    """Diagonal Fisher of a linear layer: ``out[o, i] <- beta*out + alpha * sum_rows g[r, o]^2 a[r, i]^2`` and
    ``out_bias[o] <- ... sum_rows g[r, o]^2`` for inputs ``a`` [rows, in] and output gradients ``g``
    [rows, out].  CUDA bf16 / fp32: one kernel that squares in registers; anything else: PyTorch."""
    d_in, d_out = a.shape[1], g.shape[1]
    if out is None:
        out = torch.zeros(d_out, d_in, device=a.device, dtype=torch.float32)
        beta = 0.0
    if (cuda_kernels_enabled(a, g) and a.dtype == g.dtype and a.dtype in (torch.bfloat16, torch.float32)
            and out.is_contiguous() and out.dtype == torch.float32
            and (out_bias is None or (out_bias.is_contiguous() and out_bias.dtype == torch.float32))):
        extension().diag_linear_stats(a.contiguous(), g.contiguous(), out, out_bias, float(alpha), float(beta))
        return out, out_bias
    g2, a2 = g.float().square(), a.float().square()
    out.mul_(beta).add_(g2.T @ a2, alpha=alpha)
    if out_bias is not None:
        out_bias.mul_(beta).add_(g2.sum(dim=0), alpha=alpha)
    return out, out_bias


def unitwise_inverse(blocks: torch.Tensor, damping: float = 0.0) -> torch.Tensor:
    """Batched ``(block + damping*I)^-1`` for f x k x k blocks.  2x2 blocks (normalisation
    layers) use the closed form, evaluated in one fused elementwise pass."""
    k = blocks.shape[-1]
    if k == 2 and blocks.shape[-2] == 2:
        a = blocks[..., 0, 0] + damping
        b = blocks[..., 0, 1]
        c = blocks[..., 1, 0]
        d = blocks[..., 1, 1] + damping
        det = a * d - b * c
        inv = torch.stack([torch.stack([d, -b], dim=-1), torch.stack([-c, a], dim=-1)], dim=-2)
        return inv / det[..., None, None]
    eye = torch.eye(k, device=blocks.device, dtype=blocks.dtype)
    return torch.linalg.inv(blocks + damping * eye)
