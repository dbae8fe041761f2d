"""Device-timed micro-benchmarks of the library's sm_100a kernels, one JSON line per case.

    python benchmarks/kernels.py                    # all cases
    python benchmarks/kernels.py --only syrk --rows 8192 --n 4096 --iters 3 --warmup 1   # one small case (profiling)

Every case reports the CUDA-event time (L2 flushed between iterations by writing a 256 MiB buffer),
the algorithmic FLOP/s or bytes/s, the fraction of the measured peak of the GPU
(MEASURED_PEAKS.json beside the repository root if present, else 6.65 TB/s and 1.59 PFLOP/s) and,
where a library routine computes the same thing, its time (cuBLAS through torch.matmul,
cuSOLVER through torch.linalg).
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from asdl_b200 import ops  # noqa: E402


def peaks():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p['hbm_gbs'] * 1e9, p['bf16_tflops'] * 1e12, 'measured'
    return 6.65e12, 1.59e15, 'fallback'


class Timer:
    def __init__(self, iters, warmup):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda')

    def __call__(self, fn):
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(self.iters):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        times.sort()
        return times[len(times) // 2]


def emit(**kw):
    print(json.dumps(kw), flush=True)


def bench_syrk(timer, rows, n, hbm, flops_peak, src):
    """C = X^T X, X bf16 [rows, n]; useful FLOPs counted as the full 2*rows*n^2 product (what the
    library GEMM computes), so a SYRK that only forms the lower triangle can exceed 1.0."""
    ext = ops.extension()
    x = torch.randn(rows, n, device='cuda').to(torch.bfloat16)
    out = torch.empty(n, n, device='cuda')
    ms = timer(lambda: ext.umma_gemm([x], [x], False, False, out, 1.0, 0.0, True, None, None, 0))
    ms_lib = timer(lambda: torch.matmul(x.T, x))
    fl = 2.0 * rows * n * n
    by = 2.0 * rows * n + 4.0 * n * n
    emit(case='syrk_bf16', rows=rows, n=n, ms=round(ms, 4), tflops=round(fl / ms / 1e9, 1),
         frac_of_peak_flops=round(fl / (ms * 1e-3) / flops_peak, 3),
         frac_of_peak_hbm=round(by / (ms * 1e-3) / hbm, 3), peak_source=src,
         cublas_bf16_ms=round(ms_lib, 4), speedup_vs_cublas=round(ms_lib / ms, 2))


def bench_syrk_x3(timer, rows, n, hbm, flops_peak, src):
    """fp32-grade X^T X from bf16 hi/lo splits (three tensor-core passes) against cuBLAS fp32."""
    x = torch.randn(rows, n, device='cuda')
    out = torch.empty(n, n, device='cuda')
    ms = timer(lambda: ops.gram(x, out=out))
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    ms_lib = timer(lambda: torch.matmul(x.T, x))
    torch.backends.cuda.matmul.allow_tf32 = True
    ms_tf32 = timer(lambda: torch.matmul(x.T, x))
    torch.backends.cuda.matmul.allow_tf32 = prev
    emit(case='syrk_fp32_as_bf16x3', rows=rows, n=n, ms=round(ms, 4), cublas_fp32_ms=round(ms_lib, 4),
         cublas_tf32_ms=round(ms_tf32, 4), includes='hi/lo split cast of the input')


def bench_precond(timer, m, n, hbm, flops_peak, src):
    left = torch.randn(m, m, device='cuda')
    left = left @ left.T / m
    right = torch.randn(n, n, device='cuda')
    right = right @ right.T / n
    g = torch.randn(m, n, device='cuda')
    ms = timer(lambda: ops.kron_apply(left, g, right))
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    ms_lib = timer(lambda: left @ g @ right)
    torch.backends.cuda.matmul.allow_tf32 = prev
    emit(case='kron_apply_fp32', m=m, n=n, ms=round(ms, 4), cublas_fp32_ms=round(ms_lib, 4),
         includes='hi/lo split casts of all three operands (the K-FAC maker caches those of the inverses)')


def bench_inverse(timer, sizes, hbm, flops_peak, src):
    mats = []
    for s in sizes:
        a = torch.randn(s, 2 * s, device='cuda')
        mats.append(a @ a.T / (2 * s))
    outs = [torch.empty_like(m) for m in mats]
    ms = timer(lambda: ops.spd_inverse_grouped(mats, outs, 1e-3))

    def lib():
        for m in mats:
            eye = torch.eye(m.shape[0], device='cuda')
            torch.cholesky_inverse(torch.linalg.cholesky(m + 1e-3 * eye))
    ms_lib = timer(lib)
    fl = sum(float(s) ** 3 for s in sizes)  # potrf n^3/3 + trtri n^3/3 + lauum n^3/3
    n = sizes[0]
    eye = torch.eye(n, device='cuda', dtype=torch.float64)
    resid = ((mats[0].double() + 1e-3 * eye) @ outs[0].double() - eye).abs().max().item()
    emit(case='chol_inverse_grouped_fp32', backend=ops.CHOLESKY_BACKEND, sizes=sizes if len(sizes) < 8 else
         f'{len(sizes)} factors {min(sizes)}..{max(sizes)}', ms=round(ms, 3), tflops_fp32=round(fl / ms / 1e9, 2),
         cusolver_loop_ms=round(ms_lib, 3), speedup_vs_cusolver=round(ms_lib / ms, 2), residual_first=float(f'{resid:.2e}'))


def bench_roots(timer, b, n, p, ridge):
    """Shampoo inverse p-th roots of a batch: the grouped tensor-core chain against the batched fp32
    matrix products of PyTorch (cuBLAS), same iteration, same stopping rule."""
    from asdl_b200.precondition import shampoo
    a = torch.randn(b, n, n // 2, device='cuda')
    mats = a @ a.transpose(1, 2) / n
    out = {}
    for mode in ('auto', 'never'):
        shampoo.TENSOR_CORE_ROOTS = mode
        out[mode] = timer(lambda: shampoo.inverse_pth_root_batched(mats, p, ridge_epsilon=ridge))
        roots = shampoo.inverse_pth_root_batched(mats, p, ridge_epsilon=ridge)
        ev, evec = torch.linalg.eigh(mats[0].double())
        ev = ev.clamp_min(0) + ridge * ev.max()
        exact = (evec * ev.pow(-1.0 / p)) @ evec.T
        out[mode + '_err'] = ((roots[0].double() - exact).norm() / exact.norm()).item()
    shampoo.TENSOR_CORE_ROOTS = 'auto'
    emit(case='inverse_pth_root_batched', batch=b, n=n, p=p, ridge=ridge, ms=round(out['auto'], 3),
         rel_err_vs_fp64=float(f"{out['auto_err']:.2e}"), torch_bmm_ms=round(out['never'], 3),
         torch_bmm_rel_err=float(f"{out['never_err']:.2e}"), speedup_vs_torch=round(out['never'] / out['auto'], 2))


def bench_layouts(timer, m, n, k, flops_peak, src):
    """One bf16 GEMM in the four operand layouts (MN-major = [K, M] row-major, K-major = [M, K])."""
    ext = ops.extension()
    a = torch.randn(k, m, device='cuda').to(torch.bfloat16)
    b = torch.randn(k, n, device='cuda').to(torch.bfloat16)
    ak, bk = a.T.contiguous(), b.T.contiguous()
    out = torch.empty(m, n, device='cuda')
    res = {}
    for name, (x, y, xk, yk) in {'mn_mn': (a, b, False, False), 'k_k': (ak, bk, True, True),
                                 'k_mn': (ak, b, True, False), 'mn_k': (a, bk, False, True)}.items():
        res[name] = round(timer(lambda: ext.umma_gemm([x], [y], xk, yk, out, 1.0, 0.0, False, None, None, 1)), 4)
    ms_lib = timer(lambda: torch.matmul(ak, b))
    fl = 2.0 * m * n * k
    emit(case='gemm_bf16_layouts', m=m, n=n, k=k, ms=res, cublas_ms=round(ms_lib, 4),
         frac_of_peak_flops={kk: round(fl / (v * 1e-3) / flops_peak, 3) for kk, v in res.items()}, peak_source=src)


def bench_eigh(timer, batch, n):
    """Batched Jacobi eigensolver (n <= 128) against torch.linalg.eigh (cuSOLVER)."""
    a = torch.randn(batch, n, 2 * n, device='cuda')
    mats = a @ a.transpose(1, 2) / (2 * n)
    ms = timer(lambda: ops.eigh(mats))
    ms_lib = timer(lambda: torch.linalg.eigh(mats))
    w, v = ops.eigh(mats)
    ref = torch.linalg.eigvalsh(mats.double())
    err = ((w.double() - ref).abs().max() / ref.abs().max()).item()
    emit(case='jacobi_eigh_fp32', batch=batch, n=n, ms=round(ms, 4), cusolver_ms=round(ms_lib, 4),
         speedup_vs_cusolver=round(ms_lib / ms, 2), max_rel_eigenvalue_error=float(f'{err:.2e}'))


def bench_lnstats(timer, rows, d, hbm, src):
    """Unit-wise LayerNorm statistics: one pass over y and g against the chain of PyTorch elementwise ops."""
    y = torch.randn(rows, d, device='cuda').to(torch.bfloat16)
    g = torch.randn(rows, d, device='cuda').to(torch.bfloat16)
    w, b = torch.rand(d, device='cuda') + 0.5, torch.randn(d, device='cuda')
    out = torch.zeros(d, 2, 2, device='cuda')
    ms = timer(lambda: ops.layernorm_unitwise_stats(y, g, w, b, out=out, alpha=0.05, beta=0.95))
    ops.set_backend('torch')
    ms_lib = timer(lambda: ops.layernorm_unitwise_stats(y, g, w, b, out=out, alpha=0.05, beta=0.95))
    ops.set_backend('auto')
    by = 2.0 * 2 * rows * d
    emit(case='layernorm_unitwise_stats_bf16', rows=rows, d=d, ms=round(ms, 4), gbs=round(by / ms / 1e6, 1),
         frac_of_peak_hbm=round(by / (ms * 1e-3) / hbm, 3), peak_source=src, torch_ms=round(ms_lib, 4),
         speedup_vs_torch=round(ms_lib / ms, 2))


def bench_conv_syrk(timer, n, c, hw, k, flops_peak, src):
    """Input-side factor of a stride-1 k x k convolution (padding k // 2) on a channels_last bf16 input: patches
    gathered inside the SYRK by 4-D TMA boxes against the bf16 im2col kernel followed by the SYRK."""
    conv = torch.nn.Conv2d(c, 8, k, padding=k // 2).cuda()
    x = torch.randn(n, c, hw, hw, device='cuda').to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    ncol = c * k * k
    out = torch.empty(ncol, ncol, device='cuda')
    saved, saved_mb = ops.IMPLICIT_IM2COL, ops.IMPLICIT_IM2COL_MIN_MB
    ops.IMPLICIT_IM2COL, ops.IMPLICIT_IM2COL_MIN_MB = True, 0.0
    ms = timer(lambda: ops.conv_patch_gram(x, conv, out=out, channels_last_order=True))
    ops.IMPLICIT_IM2COL = False
    ms_explicit = timer(lambda: ops.conv_patch_gram(x, conv, out=out, channels_last_order=True))
    ops.IMPLICIT_IM2COL, ops.IMPLICIT_IM2COL_MIN_MB = saved, saved_mb
    fl = 2.0 * n * hw * hw * ncol * ncol
    emit(case='conv_patch_syrk_bf16', n=n, c=c, hw=hw, k=k, ncol=ncol, implicit_ms=round(ms, 4),
         explicit_im2col_ms=round(ms_explicit, 4), speedup=round(ms_explicit / ms, 2),
         tflops_full_product=round(fl / ms / 1e9, 1), frac_of_peak_flops=round(fl / (ms * 1e-3) / flops_peak, 3),
         patch_matrix_mb=round(n * hw * hw * ncol * 2 / 2 ** 20, 1), peak_source=src)


def bench_gram_hadamard(timer, n, d_in, d_out, flops_peak, src):
    """kernel += (a a^T + 1) o (g g^T): both Gram tiles in TMEM, multiplied in the epilogue, against the
    PyTorch ops of the same update (two matmuls, an add, a multiply, an accumulate)."""
    a = torch.randn(n, d_in, device='cuda').to(torch.bfloat16)
    g = torch.randn(n, d_out, device='cuda').to(torch.bfloat16)
    kernel = torch.zeros(n, n, device='cuda')
    ms = timer(lambda: ops.gram_hadamard(kernel, a, g, one=1.0))
    ops.set_backend('torch')
    ms_lib = timer(lambda: ops.gram_hadamard(kernel, a, g, one=1.0))
    ops.set_backend('auto')
    fl = 2.0 * n * n * (d_in + d_out)
    emit(case='gram_hadamard_bf16', n=n, d_in=d_in, d_out=d_out, ms=round(ms, 4), tflops=round(fl / ms / 1e9, 1),
         frac_of_peak_flops=round(fl / (ms * 1e-3) / flops_peak, 3), peak_source=src, torch_ms=round(ms_lib, 4),
         speedup_vs_torch=round(ms_lib / ms, 2))


def bench_bfgs(timer, n):
    """Powell damping + rank-2 update of the inverse (5 launches) against the PyTorch ops of the same update."""
    from asdl_b200.precondition.kbfgs import powell_lm_damping_, bfgs_inv_update_
    base = torch.randn(n, n, device='cuda')
    H = base @ base.T / n + torch.eye(n, device='cuda')
    s0 = torch.randn(n, device='cuda')
    y0 = torch.randn(n, device='cuda') + 2 * s0

    def run():
        s, y = s0.clone(), y0.clone()
        powell_lm_damping_(H, s, y, 0.2, 1e-3)
        bfgs_inv_update_(H, s, y)

    ms = timer(run)
    ops.set_backend('torch')
    ms_lib = timer(run)
    ops.set_backend('auto')
    emit(case='bfgs_damping_and_update_fp32', n=n, ms=round(ms, 4), torch_ms=round(ms_lib, 4),
         speedup_vs_torch=round(ms_lib / ms, 2), passes_over_H='mat-vec read, symmetrise read + write, update read + write')


def bench_embedding(timer, tokens, vocab, dim):
    """Diagonal statistics of an embedding table (reductions per token row) against index_add_ of the squares."""
    from asdl_b200.operations.embedding import Embedding as EmbOp
    emb = torch.nn.Embedding(vocab, dim).cuda()
    idx = torch.randint(0, vocab, (tokens,), device='cuda')
    g = torch.randn(tokens, dim, device='cuda').to(torch.bfloat16)
    ms = timer(lambda: EmbOp.cov_diag_weight(emb, idx, g))
    ops.set_backend('torch')
    ms_lib = timer(lambda: EmbOp.cov_diag_weight(emb, idx, g.float()))
    ops.set_backend('auto')
    emit(case='embedding_diag_stats_bf16', tokens=tokens, vocab=vocab, dim=dim, ms=round(ms, 4), torch_ms=round(ms_lib, 4),
         speedup_vs_torch=round(ms_lib / ms, 2), includes='zero-fill of the vocab x dim output')


def bench_symm(timer, world, mb, hbm, src):
    """The segment kernels of the NVLink transport on ranks emulated on ONE GPU (every "peer" buffer is
    local memory, so this measures the kernels against HBM, not the link): owner pull-reduce and push."""
    from asdl_b200.parallel.symmetric import SymmetricArena
    numel = int(mb * (1 << 20) / 4)
    arenas = SymmetricArena.local_group(numel + 1024, world)
    offs = [a.alloc(numel)[0] for a in arenas]
    for a in arenas:
        a.buffer.normal_()
    segs = arenas[0].segments([(offs[0], numel)])
    ms_r = timer(lambda: arenas[0].reduce_segments(segs, 1.0 / world))
    ms_b = timer(lambda: arenas[0].bcast_segments(segs))
    emit(case='symm_reduce_segments_emulated', world=world, mbytes=mb, ms=round(ms_r, 4),
         frac_of_peak_hbm=round(4.0 * numel * (world + 1) / (ms_r * 1e-3) / hbm, 3), peak_source=src)
    emit(case='symm_bcast_segments_emulated', world=world, mbytes=mb, ms=round(ms_b, 4),
         frac_of_peak_hbm=round(4.0 * numel * world / (ms_b * 1e-3) / hbm, 3), peak_source=src)
    # owner-side pull of a factor's statistics: every emulated rank holds its share (lower triangle) at the same offset
    n = 4096
    group = SymmetricArena.local_group(2 * n * n + 1024, world)
    offs = [(g.alloc(n, n), g.alloc(n, n)) for g in group]
    for g in group:
        g.buffer.normal_()
    table = torch.tensor([[offs[0][0][0], offs[0][1][0], n]], dtype=torch.int64, device='cuda')
    ms_p = timer(lambda: group[0].pull_slots(table, n, 0.95))
    by = 4.0 * n * n * (0.5 * world + 0.5 + 1.0)   # lower triangles of all ranks and of the factor read, full factor written
    emit(case='symm_pull_slots_emulated', world=world, n=n, ms=round(ms_p, 4),
         frac_of_peak_hbm=round(by / (ms_p * 1e-3) / hbm, 3), peak_source=src)


def bench_im2col(timer, n, c, hw, k, stride, pad, hbm, flops_peak, src):
    ext = ops.extension()
    x = torch.randn(n, c, hw, hw, device='cuda').to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    ho = (hw + 2 * pad - k) // stride + 1
    ncol = c * k * k
    ld = (ncol + 7) // 8 * 8
    out = torch.empty(n * ho * ho, ld, device='cuda', dtype=torch.bfloat16)
    ms = timer(lambda: ext.im2col_bf16(x, out, None, [k, k], [stride, stride], [pad, pad], [1, 1], False))
    by = 2.0 * x.numel() + 2.0 * out.numel()
    emit(case='im2col_bf16_nhwc', shape=[n, c, hw, hw], kernel=k, stride=stride, ms=round(ms, 4),
         gbs=round(by / ms / 1e6, 1), frac_of_peak_hbm=round(by / (ms * 1e-3) / hbm, 3), peak_source=src)


def bench_batchnorm(timer, n, c, hw, hbm, flops_peak, src):
    """Training BatchNorm forward + backward on NHWC bf16 (fused ReLU) against F.batch_norm + relu."""
    import torch.nn.functional as F
    cl = dict(memory_format=torch.channels_last)
    x = torch.randn(n, c, hw, hw, device='cuda').to(torch.bfloat16).contiguous(**cl).requires_grad_(True)
    dy = torch.randn(n, c, hw, hw, device='cuda').to(torch.bfloat16).contiguous(**cl)
    w = torch.ones(c, device='cuda', requires_grad=True)
    b = torch.zeros(c, device='cuda', requires_grad=True)

    def ours():
        y = ops.batch_norm_train(x, w, b, None, None, 0.1, 1e-5, relu=True)
        torch.autograd.grad(y, (x, w, b), dy)

    def lib():
        y = torch.relu(F.batch_norm(x, None, None, w, b, True, 0.1, 1e-5))
        torch.autograd.grad(y, (x, w, b), dy)
    ms, ms_lib = timer(ours), timer(lib)
    numel = n * c * hw * hw
    by = 2.0 * numel * (3 + 7)           # fwd 3 passes; bwd sums (x, dy, y) + dx (dy, x, y, write)
    emit(case='batchnorm_relu_train_fwd_bwd_nhwc_bf16', shape=[n, c, hw, hw], ms=round(ms, 4),
         gbs=round(by / ms / 1e6, 1), frac_of_peak_hbm=round(by / (ms * 1e-3) / hbm, 3), peak_source=src,
         torch_ms=round(ms_lib, 4), speedup_vs_torch=round(ms_lib / ms, 2))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--only', default=None, choices=['syrk', 'syrk_x3', 'layouts', 'precond', 'inverse', 'roots', 'eigh', 'lnstats', 'conv_syrk', 'gram_hadamard', 'bfgs', 'embedding', 'symm', 'im2col', 'batchnorm'])
    ap.add_argument('--wide', type=int, default=-1, help='tile policy of the GEMM: -1 = default (3), 0 = 128 wide, 1 = 256 wide for large outputs, 2 = 256 wide wherever legal, 3 = CTA pairs (256 x 256, cta_group::2) for large products, 4 = CTA pairs everywhere')
    ap.add_argument('--chol', default=None, choices=['tensor_core', 'cuda_core'], help='grouped inverse backend')
    ap.add_argument('--rows', type=int, default=None)
    ap.add_argument('--n', type=int, default=None)
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    args = ap.parse_args()
    hbm, fl, src = peaks()
    ops.extension().set_gemm_wide(args.wide)
    if args.chol:
        ops.CHOLESKY_BACKEND = args.chol
    timer = Timer(args.iters, args.warmup)
    want = lambda name: args.only in (None, name)  # noqa: E731
    if want('syrk'):
        cases = [(args.rows, args.n)] if args.rows and args.n else \
            [(100352, 64), (100352, 256), (25088, 512), (25088, 1152), (6272, 2304), (6272, 1024), (1568, 4608),
             (1568, 2048), (8192, 1024), (8192, 4096), (4096, 8192), (32768, 4096)]
        for rows, n in cases:
            bench_syrk(timer, rows, n, hbm, fl, src)
    if want('syrk_x3'):
        for rows, n in ([(args.rows, args.n)] if args.rows and args.n else [(8192, 1024), (8192, 4096)]):
            bench_syrk_x3(timer, rows, n, hbm, fl, src)
    if want('precond'):
        for m, n in [(512, 4608), (2048, 512), (1024, 4096), (4096, 1024)]:
            bench_precond(timer, m, n, hbm, fl, src)
    if want('inverse'):
        resnet = ([147, 64] + [64, 64] + [64, 256] * 4 + [256, 64] * 2 + [576, 64] * 3 + [256, 128] + [1152, 128] * 4
                  + [128, 512] * 4 + [256, 512] + [512, 128] * 3 + [512, 256] + [2304, 256] * 6 + [256, 1024] * 6
                  + [512, 1024] + [1024, 256] * 5 + [1024, 512] + [4608, 512] * 3 + [512, 2048] * 3 + [1024, 2048]
                  + [2048, 512] * 2 + [2048, 1000])
        cases = [[args.n]] if args.n else [[2048], [4608], [1024] * 8,
                                           [64] * 16 + [256] * 16 + [512] * 8 + [1024] * 8 + [2304] * 6, resnet]
        for sizes in cases:
            bench_inverse(timer, sizes, hbm, fl, src)
    if want('roots'):
        for b, n, p, ridge in [(8, 1024, 4, 1e-6), (30, 1024, 4, 1e-6), (30, 768, 4, 1e-6)]:
            bench_roots(timer, b, n, p, ridge)
    if want('layouts'):
        for m, n, k in [(4096, 4096, 8192), (2048, 2048, 2048)]:
            bench_layouts(timer, m, n, k, fl, src)
    if want('eigh'):
        for batch, n in [(64, 64), (16, 128), (256, 32)]:
            bench_eigh(timer, batch, n)
    if want('lnstats'):
        for rows, d in [(8192, 1024), (12608, 768)]:
            bench_lnstats(timer, rows, d, hbm, src)
    if want('conv_syrk'):
        for n, c, hw in [(32, 64, 56), (32, 128, 28), (32, 256, 14), (32, 512, 7)]:
            bench_conv_syrk(timer, n, c, hw, 3, fl, src)
    if want('gram_hadamard'):
        for n, d_in, d_out in [(2048, 4608, 512), (1024, 1024, 1024), (4096, 768, 3072)]:
            bench_gram_hadamard(timer, n, d_in, d_out, fl, src)
    if want('bfgs'):
        for n in (1024, 4608):
            bench_bfgs(timer, n)
    if want('embedding'):
        bench_embedding(timer, 8192, 50304, 1024)
    if want('symm'):
        bench_symm(timer, 4, 64, hbm, src)
    if want('im2col'):
        bench_im2col(timer, 32, 64, 56, 3, 1, 1, hbm, fl, src)
        bench_im2col(timer, 32, 256, 14, 3, 1, 1, hbm, fl, src)
    if want('batchnorm'):
        for n, c, hw in [(32, 64, 112), (32, 256, 56), (32, 512, 28), (32, 1024, 14), (32, 2048, 7)]:
            bench_batchnorm(timer, n, c, hw, hbm, fl, src)
    ops.check_status()


if __name__ == '__main__':
    main()
