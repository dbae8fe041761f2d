"""sm_100a kernels against plain PyTorch fp32 references of the same operation."""
import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as asdl
from asdl_b200 import ops

pytestmark = pytest.mark.gpu
DEV = 'cuda'


def rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-30)).item()


@pytest.fixture(scope='module')
def ext():
    e = ops.extension()
    yield e
    ops.check_status()


@pytest.mark.parametrize('rows,n', [(64, 128), (100, 8), (1000, 200), (777, 152), (4096, 512),
                                    (8192, 64), (1568, 1024), (33, 17), (5000, 320)])
@pytest.mark.parametrize('nsplit', [1, 0])
def test_syrk_bf16(ext, rows, n, nsplit):
    x = torch.randn(rows, n, device=DEV).to(torch.bfloat16)
    ld = (n + 7) // 8 * 8
    buf = torch.zeros(rows, ld, device=DEV, dtype=torch.bfloat16)
    buf[:, :n] = x
    c = torch.full((n, n), float('nan'), device=DEV)
    ext.umma_gemm([buf[:, :n]], [buf[:, :n]], False, False, c, 1.0, 0.0, True, None, None, nsplit)
    ref = (x.double().T @ x.double()).float()
    assert rel_err(c, ref) < 1e-4  # the tensor core accumulates long sums with truncation
    assert torch.equal(c, c.T)


def test_syrk_ema_epilogue(ext):
    rows, n = 2048, 384
    x = torch.randn(rows, n, device=DEV).to(torch.bfloat16)
    c0 = torch.randn(n, n, device=DEV)
    c0 = c0 + c0.T
    for nsplit in (1, 4):
        c = c0.clone()
        ext.umma_gemm([x], [x], False, False, c, 0.05 / rows, 0.95, True, None, None, nsplit)
        ref = 0.95 * c0 + 0.05 / rows * (x.double().T @ x.double()).float()
        assert rel_err(c, ref) < 1e-5


@pytest.mark.parametrize('m,n,k', [(128, 128, 64), (256, 384, 512), (200, 304, 1000), (512, 4608, 512),
                                   (64, 2048, 2048), (1000, 2048, 1000)])
def test_gemm_all_layouts(ext, m, n, k):
    a = torch.randn(k, m, device=DEV).to(torch.bfloat16)
    b = torch.randn(k, n, device=DEV).to(torch.bfloat16)
    ref = (a.double().T @ b.double()).float()
    ak, bk = a.T.contiguous(), b.T.contiguous()
    for a_op, b_op, a_k, b_k in ((a, b, False, False), (ak, b, True, False), (ak, bk, True, True),
                                 (a, bk, False, True)):
        c = torch.empty(m, n, device=DEV)
        ext.umma_gemm([a_op], [b_op], a_k, b_k, c, 1.0, 0.0, False, None, None, 0)
        assert rel_err(c, ref) < 1e-5


def test_bf16x3_and_bf16_outputs(ext):
    m, n, k = 256, 320, 1024
    af, bf = torch.randn(k, m, device=DEV), torch.randn(k, n, device=DEV)
    ah, al = torch.empty(k, m, device=DEV, dtype=torch.bfloat16), torch.empty(k, m, device=DEV, dtype=torch.bfloat16)
    bh, bl = torch.empty(k, n, device=DEV, dtype=torch.bfloat16), torch.empty(k, n, device=DEV, dtype=torch.bfloat16)
    ext.cast_pad_bf16(af, ah, al, 1.0)
    ext.cast_pad_bf16(bf, bh, bl, 1.0)
    assert rel_err(ah.float() + al.float(), af) < 1e-4
    c = torch.empty(m, n, device=DEV)
    ext.umma_gemm([ah, ah, al], [bh, bl, bh], False, False, c, 1.0, 0.0, False, None, None, 1)
    ref = (af.double().T @ bf.double()).float()
    assert rel_err(c, ref) < 5e-5
    oh, ol = torch.empty(m, n, device=DEV, dtype=torch.bfloat16), torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ext.umma_gemm([ah], [bh], False, False, None, 1.0, 0.0, False, oh, ol, 1)
    assert rel_err(oh.float() + ol.float(), ah.float().T @ bh.float()) < 1e-4


@pytest.mark.parametrize('cfg', [(2, 16, 10, 10, 3, 1, 1), (2, 8, 9, 9, 3, 2, 1), (2, 3, 12, 12, 7, 2, 3),
                                 (2, 16, 8, 8, 1, 2, 0), (3, 24, 7, 7, 3, 1, 1)])
def test_im2col(ext, cfg):
    n, c, h, w, k, s, p = cfg
    x = torch.randn(n, c, h, w, device=DEV)
    ref = F.unfold(x, k, padding=p, stride=s)
    ho = (h + 2 * p - k) // s + 1
    rows, ncol = n * ho * ho, c * k * k
    ld = (ncol + 7) // 8 * 8
    out = torch.empty(rows, ld, device=DEV, dtype=torch.bfloat16)
    ext.im2col_bf16(x, out, None, [k, k], [s, s], [p, p], [1, 1], True)
    want = ref.transpose(1, 2).reshape(rows, ncol).to(torch.bfloat16)
    assert torch.equal(out[:, :ncol], want) and out[:, ncol:].abs().sum() == 0
    xb = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    out2 = torch.empty(rows, ld, device=DEV, dtype=torch.bfloat16)
    ext.im2col_bf16(xb, out2, None, [k, k], [s, s], [p, p], [1, 1], False)
    want2 = ref.view(n, c, k * k, -1).permute(0, 3, 2, 1).reshape(rows, ncol).to(torch.bfloat16)
    assert torch.equal(out2[:, :ncol], want2)


def test_ops_gram_and_kron_apply():
    x = torch.randn(3000, 200, device=DEV)
    ops.set_backend('torch')
    ref = ops.gram(x, scale=0.5)
    ops.set_backend('auto')
    got = ops.gram(x, scale=0.5)
    assert rel_err(got, ref) < 5e-5  # fp32 input -> bf16x3
    xb = x.to(torch.bfloat16)
    assert rel_err(ops.gram(xb), xb.float().T @ xb.float()) < 1e-5
    left = torch.randn(96, 96, device=DEV)
    left = left @ left.T / 96
    right = torch.randn(200, 200, device=DEV)
    right = right @ right.T / 200
    mid = torch.randn(96, 200, device=DEV)
    assert rel_err(ops.kron_apply(left, mid, right), left @ mid @ right) < 1e-4
    conv = nn.Conv2d(16, 8, 3, padding=1, stride=2).to(DEV)
    xc = torch.randn(4, 16, 10, 10, device=DEV)
    ops.set_backend('torch')
    ref = ops.conv_patch_gram(xc, conv, scale=0.1)
    ops.set_backend('auto')
    assert rel_err(ops.conv_patch_gram(xc, conv, scale=0.1), ref) < 1e-4  # fp32 input -> hi/lo patches
    xcl = xc.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    got = ops.conv_patch_gram(xcl, conv, scale=0.1, channels_last_order=True)
    perm = torch.arange(16 * 9, device=DEV).view(16, 9).T.reshape(-1)
    assert rel_err(got, ref[perm][:, perm]) < 1e-2
    ops.check_status()


def _small_cnn():
    torch.manual_seed(0)
    return nn.Sequential(nn.Conv2d(3, 16, 3, padding=1, bias=False), nn.BatchNorm2d(16), nn.ReLU(),
                         nn.Conv2d(16, 32, 1, bias=False), nn.BatchNorm2d(32), nn.ReLU(),
                         nn.Conv2d(32, 16, 3, stride=2, padding=1), nn.ReLU(),
                         nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(16, 5))


def _fused_kfac_gpu_matches_cpu(graph, **extra):
    torch.backends.cudnn.allow_tf32 = False
    x, t = torch.randn(8, 3, 16, 16), torch.randint(0, 5, (8,))
    cfg = asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=0.3,
                                     curvature_upd_interval=4, preconditioner_upd_interval=4)
    base = _small_cnn()

    def run(model, x, t, **kw):
        gm = asdl.FusedKfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP, **kw)
        opt = torch.optim.SGD(model.parameters(), lr=0.01)
        out = []
        for _ in range(8):
            opt.zero_grad()
            d = gm.setup_model_call(model, x)
            gm.setup_loss_call(F.cross_entropy, d, t)
            _, loss = gm.forward_and_backward()
            out.append((loss.item(), [p.grad.detach().cpu().clone() for p in model.parameters()]))
            opt.step()
        return out

    ref = run(copy.deepcopy(base), x, t)
    model = copy.deepcopy(base).to(DEV).to(memory_format=torch.channels_last)
    got = run(model, x.to(DEV).contiguous(memory_format=torch.channels_last), t.to(DEV), cuda_graph=graph, **extra)
    for (l1, g1), (l2, g2) in zip(ref, got):
        assert abs(l1 - l2) < 2e-3 * max(1, abs(l1))
        for a, b in zip(g1, g2):
            assert rel_err(b, a) < 5e-3, (rel_err(b, a), a.shape)
    ops.check_status()


def test_fused_kfac_gpu_matches_cpu():
    _fused_kfac_gpu_matches_cpu(False)


def test_fused_kfac_per_layer_launches_match_cpu():
    _fused_kfac_gpu_matches_cpu(False, grouped=False)


def test_smoke_entry():
    import __graft_entry__ as entry
    entry.smoke()


@pytest.mark.parametrize('sizes', [[64], [100], [65, 130, 17], [512, 256, 64, 1000], [2304, 576]])
def test_chol_inverse_grouped(sizes):
    torch.manual_seed(0)
    mats, damp = [], []
    for i, n in enumerate(sizes):
        a = torch.randn(n, 2 * n, device=DEV)
        mats.append(a @ a.T / (2 * n))
        damp.append(1e-2 * (i + 1))
    keep = [m.clone() for m in mats]
    outs = [torch.empty_like(m) for m in mats]
    ops.spd_inverse_grouped(mats, outs, torch.tensor(damp, device=DEV))
    ops.check_status()
    for m, k, o, d in zip(mats, keep, outs, damp):
        assert torch.equal(m, k)  # inputs untouched
        n = m.shape[0]
        eye = torch.eye(n, device=DEV, dtype=torch.float64)
        ref = torch.linalg.inv(m.double() + d * eye)
        assert rel_err(o, ref.float()) < 1e-4
        assert torch.equal(o, o.T)
        resid = ((m.double() + d * eye) @ o.double() - eye).abs().max().item()
        assert resid < 1e-3
    single = ops.spd_inverse(mats[0], damp[0])
    assert rel_err(single, outs[0]) < 1e-6


@pytest.mark.parametrize('shape,dtype', [((6, 64, 9, 7), torch.bfloat16), ((3, 24, 5, 5), torch.bfloat16),
                                         ((4, 40, 12, 12), torch.float32), ((32, 256, 14, 14), torch.bfloat16),
                                         ((2, 8, 1, 1), torch.float32)])
def test_batchnorm_unitwise_stats_kernel(ext, shape, dtype):
    torch.manual_seed(0)
    c = shape[1]
    y = torch.randn(shape, device=DEV).to(dtype).contiguous(memory_format=torch.channels_last)
    g = torch.randn(shape, device=DEV).to(dtype).contiguous(memory_format=torch.channels_last)
    w = torch.rand(c, device=DEV) + 0.5
    b = torch.randn(c, device=DEV)
    prev = torch.randn(c, 2, 2, device=DEV)
    ops.set_backend('torch')
    ref = ops.batchnorm_unitwise_stats(y, g, w, b, out=prev.clone(), alpha=0.3, beta=0.7)
    ops.set_backend('auto')
    before = ext.launch_count()
    got = ops.batchnorm_unitwise_stats(y, g, w, b, out=prev.clone(), alpha=0.3, beta=0.7)
    assert ext.launch_count() == before + 2
    assert rel_err(got, ref) < 2e-5
    fresh = ops.batchnorm_unitwise_stats(y, g, w, b)
    assert rel_err(fresh, (ref - 0.7 * prev) / 0.3) < 1e-4
    assert torch.equal(fresh[:, 0, 1], fresh[:, 1, 0])


@pytest.mark.parametrize('shape', [(8, 64, 14, 14), (4, 24, 7, 5), (32, 256, 28, 28), (2, 8, 1, 3), (3, 72, 33, 9)])
def test_batch_norm_train_kernels(ext, shape):
    """Forward (output, running statistics) and backward (input, weight, bias gradients) against
    F.batch_norm evaluated in fp32 on the same bf16-rounded input."""
    torch.manual_seed(0)
    c = shape[1]
    x = (torch.randn(shape, device=DEV) * 2 + 0.7).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    w = (torch.rand(c, device=DEV) + 0.5).requires_grad_(True)
    b = torch.randn(c, device=DEV).requires_grad_(True)
    dy = torch.randn(shape, device=DEV).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    rm, rv = torch.zeros(c, device=DEV), torch.ones(c, device=DEV)
    xr = x.detach().float().requires_grad_(True)
    wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    rm_ref, rv_ref = rm.clone(), rv.clone()
    y_ref = F.batch_norm(xr, rm_ref, rv_ref, wr, br, True, 0.1, 1e-5)
    y_ref.backward(dy.float())
    xk = x.detach().requires_grad_(True)
    assert ops.batch_norm_train_supported(xk, w, b)
    before = ext.launch_count()
    y = ops.batch_norm_train(xk, w, b, rm, rv, 0.1, 1e-5)
    y.backward(dy)
    assert ext.launch_count() == before + 6
    assert y.dtype == torch.bfloat16 and y.is_contiguous(memory_format=torch.channels_last)
    assert rel_err(y, y_ref) < 4e-3                      # bf16 rounding of the output
    assert rel_err(rm, rm_ref) < 1e-5 and rel_err(rv, rv_ref) < 1e-5
    assert rel_err(w.grad, wr.grad) < 1e-4 and rel_err(b.grad, br.grad) < 1e-4
    assert rel_err(xk.grad, xr.grad) < 6e-3
    ops.check_status()


def test_shampoo_grouped_launches_match_per_block_path():
    """Grouped statistics / root application on CUDA against the per-block PyTorch path on CPU."""
    torch.manual_seed(0)
    base = nn.Sequential(nn.Linear(40, 96), nn.Tanh(), nn.Linear(96, 72, bias=False), nn.Tanh(), nn.Linear(72, 8))
    x, t = torch.randn(16, 40), torch.randint(0, 8, (16,))

    def run(model, x, t, **kw):
        cfg = asdl.PreconditioningConfig(damping=1e-4, preconditioner_upd_interval=2)
        gm = asdl.ShampooGradientMaker(model, cfg, block_size=32, **kw)
        opt = torch.optim.SGD(model.parameters(), lr=1e-3)
        out, launches = [], []
        ext = ops.extension()
        for _ in range(5):
            before = ext.launch_count()
            opt.zero_grad(set_to_none=False)
            d = gm.setup_model_call(model, x)
            gm.setup_loss_call(F.cross_entropy, d, t)
            gm.forward_and_backward()
            launches.append(ext.launch_count() - before)
            out.append([p.grad.detach().cpu().clone() for p in model.parameters()])
            opt.step()
        return gm, out, launches

    _, ref, _ = run(copy.deepcopy(base), x, t)
    gm, got, launches = run(copy.deepcopy(base).to(DEV), x.to(DEV), t.to(DEV))
    assert gm._group is not None and len(gm._group.blocks) == 2 * 3 + 3 * 3 + 3
    # a step without a root update: 1 staging + 1 statistics + 2 application launches for all 18
    # blocks together; the steps that refresh the roots add the power iteration and the root chain
    assert max(sorted(launches)[:2]) <= 4, launches
    for step, (g_ref, g_got) in enumerate(zip(ref, got)):
        for a, b in zip(g_ref, g_got):
            assert rel_err(b, a) < 5e-3, (step, rel_err(b, a), a.shape)
    ops.check_status()


def test_three_way_split_reproduces_fp32(ext):
    torch.manual_seed(0)
    x = torch.randn(300, 200, device=DEV) * torch.logspace(-6, 3, 200, device=DEV)
    parts = [torch.empty(300, 200, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    ext.cast_split3(x, *parts)
    total = parts[0].double() + parts[1].double() + parts[2].double()
    assert ((total - x.double()).abs() <= x.double().abs() * 2.0 ** -23).all()


@pytest.mark.parametrize('n,p', [(192, 4), (128, 2), (200, 8)])
def test_inverse_root_chain_on_tensor_cores(n, p):
    """Batched coupled Newton with grouped tcgen05 products against the exact root from an
    eigendecomposition in fp64."""
    from asdl_b200.precondition.shampoo import inverse_pth_root_batched
    torch.manual_seed(0)
    a = torch.randn(3, n, 2 * n, device=DEV)
    mats = a @ a.transpose(1, 2) / (2 * n)
    mats[1] *= 50.0                                  # different scales in one batch
    ext = ops.extension()
    before = ext.launch_count()
    roots = inverse_pth_root_batched(mats, p, ridge_epsilon=1e-4)
    assert ext.launch_count() > before               # ran on the library's kernels
    for m, r in zip(mats.double(), roots.double()):
        evals, evecs = torch.linalg.eigh(m)
        evals = evals + 1e-4 * evals.max()
        exact = (evecs * evals.pow(-1.0 / p)) @ evecs.T
        assert rel_err(r, exact) < 2e-3, rel_err(r, exact)
    ops.check_status()


@pytest.mark.parametrize('relu,residual', [(True, False), (False, True), (True, True)])
def test_batch_norm_train_fused_activation_and_residual(ext, relu, residual):
    torch.manual_seed(0)
    shape, c = (8, 64, 14, 14), 64
    cl = dict(memory_format=torch.channels_last)
    x = (torch.randn(shape, device=DEV) * 2 + 0.7).to(torch.bfloat16).contiguous(**cl)
    r = torch.randn(shape, device=DEV).to(torch.bfloat16).contiguous(**cl) if residual else None
    w = (torch.rand(c, device=DEV) + 0.5).requires_grad_(True)
    b = torch.randn(c, device=DEV).requires_grad_(True)
    dy = torch.randn(shape, device=DEV).to(torch.bfloat16).contiguous(**cl)
    xr = x.detach().float().requires_grad_(True)
    rr = r.detach().float().requires_grad_(True) if residual else None
    wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    y_ref = F.batch_norm(xr, None, None, wr, br, True, 0.1, 1e-5)
    if residual:
        y_ref = y_ref + rr
    if relu:
        y_ref = torch.relu(y_ref)
    y_ref.backward(dy.float())
    xk = x.detach().requires_grad_(True)
    rk = r.detach().requires_grad_(True) if residual else None
    tracked = torch.zeros((), dtype=torch.long, device=DEV)
    y, mean, invstd = ops.batch_norm_train(xk, w, b, None, None, 0.1, 1e-5, residual=rk, relu=relu,
                                           num_batches_tracked=tracked, return_stats=True)
    y.backward(dy)
    assert tracked.item() == 1
    assert rel_err(y, y_ref) < 5e-3
    assert rel_err(w.grad, wr.grad) < 2e-3 and rel_err(b.grad, br.grad) < 2e-3
    assert rel_err(xk.grad, xr.grad) < 8e-3
    if residual:
        assert rel_err(rk.grad, rr.grad) < 5e-3
    # unit-wise curvature from (x, mean, invstd, y) against the PyTorch formulation
    stats = torch.zeros(c, 2, 2, device=DEV)
    ops.batchnorm_unitwise_stats_from_input(xk.detach(), dy, y.detach() if relu else None, mean, invstd, stats)
    ops.set_backend('torch')
    ref = ops.batchnorm_unitwise_stats_from_input(xk.detach(), dy, y.detach() if relu else None, mean, invstd,
                                                  torch.zeros(c, 2, 2, device=DEV))
    ops.set_backend('auto')
    assert rel_err(stats, ref) < 1e-4
    ops.check_status()


def test_fused_resnet_under_autocast_matches_unfused_model():
    """Fused normalisation / activation / residual kernels plus the grouped weight cast against
    the same network made of separate PyTorch layers (bf16 autocast, channels_last)."""
    from asdl_b200.models import resnet_tiny
    torch.manual_seed(0)
    plain = resnet_tiny(width=16, fused=False).to(DEV).to(memory_format=torch.channels_last)
    fused = resnet_tiny(width=16, fused=True).to(DEV).to(memory_format=torch.channels_last)
    fused.load_state_dict(copy.deepcopy(plain.state_dict()))
    x = torch.randn(8, 3, 64, 64, device=DEV).contiguous(memory_format=torch.channels_last)
    t = torch.randint(0, 10, (8,), device=DEV)
    grads = []
    for model in (plain, fused):
        with torch.autocast('cuda', dtype=torch.bfloat16):
            loss = F.cross_entropy(model(x), t)
        loss.backward()
        grads.append((loss.item(), [p.grad.float().clone() for p in model.parameters()]))
        assert all(p.grad.dtype == torch.float32 and p.grad.shape == p.shape for p in model.parameters())
    assert abs(grads[0][0] - grads[1][0]) < 5e-2, (grads[0][0], grads[1][0])
    # both networks round to bf16 at different places (the fused kernels round once after the
    # residual add and the ReLU), so compare directions and overall size rather than digits
    flat_a = torch.cat([g.flatten() for g in grads[0][1]])
    flat_b = torch.cat([g.flatten() for g in grads[1][1]])
    cosine = F.cosine_similarity(flat_a, flat_b, dim=0).item()
    assert cosine > 0.95, cosine
    assert 0.8 < (flat_b.norm() / flat_a.norm()).item() < 1.25
    assert torch.allclose(plain.bn1.running_mean, fused.bn1.running_mean, atol=2e-3), \
        (plain.bn1.running_mean - fused.bn1.running_mean).abs().max().item()
    assert plain.bn1.num_batches_tracked.item() == fused.bn1.num_batches_tracked.item() == 1


@pytest.mark.parametrize('rows,cols', [(96, 40), (1000, 768), (33, 65), (4096, 1024)])
def test_transposing_cast_kernel(ext, rows, cols):
    """Column-major bf16 gradient -> row-major fp32 tensor (what autograd hands over for linear layers)."""
    torch.manual_seed(0)
    base = torch.randn(cols, rows, device=DEV).to(torch.bfloat16)   # storage of the transposed matrix
    src = base.t()                                                  # [rows, cols], strides (1, rows)
    dst = torch.full((rows, cols), float('nan'), device=DEV)
    ext.transpose_cast(src, dst)
    assert torch.equal(dst, src.float())
    # through the grouped weight cast: a linear layer under autocast gets an fp32 gradient in its own layout
    from asdl_b200.models.layers import grouped_bf16_weights
    lin_a, lin_b = nn.Linear(cols, 24).to(DEV), nn.Linear(cols, 24).to(DEV)
    lin_b.load_state_dict(lin_a.state_dict())
    x = torch.randn(rows, cols, device=DEV)
    with torch.autocast('cuda', dtype=torch.bfloat16):
        with grouped_bf16_weights(lin_a):
            ya = lin_a(x)
        yb = lin_b(x)
    ya.float().square().sum().backward()
    yb.float().square().sum().backward()
    assert lin_a.weight.grad.dtype == torch.float32 and lin_a.weight.grad.is_contiguous()
    assert rel_err(lin_a.weight.grad, lin_b.weight.grad) < 1e-2
    ops.check_status()


@pytest.mark.parametrize('rows,d', [(64, 256), (197 * 3, 768), (1000, 1024), (9, 4096), (33, 1536), (1001, 2048),
                                    (517, 3072), (600, 4096)])
def test_layer_norm_kernels(ext, rows, d):
    """Forward and backward (input, weight, bias gradients) against F.layer_norm in fp32."""
    torch.manual_seed(0)
    x = (torch.randn(rows, d, device=DEV) * 1.5 + 0.3).to(torch.bfloat16)
    w = (torch.rand(d, device=DEV) + 0.5).requires_grad_(True)
    b = torch.randn(d, device=DEV).requires_grad_(True)
    dy = torch.randn(rows, d, device=DEV).to(torch.bfloat16)
    xr = x.float().requires_grad_(True)
    wr, br = w.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    F.layer_norm(xr, (d,), wr, br, 1e-5).backward(dy.float())
    xk = x.detach().requires_grad_(True)
    assert ops.layer_norm_supported(xk, w, b)
    before = ext.launch_count()
    y = ops.layer_norm(xk, w, b, 1e-5)
    y.backward(dy)
    assert ext.launch_count() == before + 3
    assert rel_err(y, F.layer_norm(x.float(), (d,), w, b, 1e-5)) < 4e-3
    assert rel_err(xk.grad, xr.grad) < 6e-3
    assert rel_err(w.grad, wr.grad) < 1e-4 and rel_err(b.grad, br.grad) < 1e-4
    # a 3-d input and the module wrapper under autocast
    from asdl_b200.models.layers import FusedLayerNorm
    ln = FusedLayerNorm(d).to(DEV)
    x3 = torch.randn(2, 5, d, device=DEV, requires_grad=True)
    with torch.autocast('cuda', dtype=torch.bfloat16):
        out = ln(x3)
    assert out.dtype == torch.bfloat16 and out.shape == x3.shape
    out.float().sum().backward()
    assert x3.grad is not None and ln.weight.grad.shape == (d,)
    ops.check_status()


def test_symmetric_segment_kernels_on_emulated_ranks(ext):
    """Pull-reduce, push-broadcast and decay kernels with three ranks emulated on one GPU."""
    from asdl_b200.parallel.symmetric import SymmetricArena
    arenas = SymmetricArena.local_group(5000, 3)
    slots = [[a.alloc(37, 20), a.alloc(1000), a.alloc(8)] for a in arenas]
    torch.manual_seed(0)
    for per_rank in slots:
        for _, view in per_rank:
            view.copy_(torch.randn_like(view))
    before = [[v.clone() for _, v in per_rank] for per_rank in slots]
    owner = arenas[1]
    segs = owner.segments([(slots[1][0][0], 37 * 20), (slots[1][2][0], 8)])
    owner.reduce_segments(segs, 1.0 / 3)
    for k in (0, 2):
        ref = sum(before[r][k] for r in range(3)) / 3
        assert torch.allclose(slots[1][k][1], ref, atol=1e-6)
        assert torch.equal(slots[0][k][1], before[0][k])  # peers are only read
    assert torch.equal(slots[1][1][1], before[1][1])      # segments not listed stay
    owner.bcast_segments(segs)
    for r in (0, 2):
        for k in (0, 2):
            assert torch.equal(slots[r][k][1], slots[1][k][1])
        assert torch.equal(slots[r][1][1], before[r][1])
    owner.scale_segments(owner.segments([(slots[1][1][0], 1000)]), 0.25)
    assert torch.allclose(slots[1][1][1], before[1][1] * 0.25)
    with pytest.raises(RuntimeError):
        owner.barrier()
    ops.check_status()


def test_gemm_epilogue_reduces_into_and_replicates_to_other_buffers(ext):
    """The epilogue paths of the data-parallel transport, aimed at plain buffers of this GPU: tiles
    added into a destination that already holds data (statistics pushed to an owner) and results
    stored to several destinations (preconditioned gradients replicated to every rank)."""
    torch.manual_seed(0)
    x = torch.randn(3000, 200, device=DEV).to(torch.bfloat16)
    ref = x.float().T @ x.float()
    target = torch.randn(200, 200, device=DEV)
    held = target.clone()
    for _ in range(2):  # two ranks' contributions
        ext.umma_gemm_to_ptr([x], [x], False, False, target.data_ptr(), 200, 0.5, True, True, [], 0)
    assert rel_err(target, held + ref) < 1e-4
    # lower-triangle-only reductions (what travels between GPUs) completed by a local mirror pass
    from asdl_b200.parallel.symmetric import SymmetricArena
    arena = SymmetricArena.local_group(200 * 200 + 64, 1)[0]
    off, fac = arena.alloc(200, 200)
    for _ in range(2):
        ext.umma_gemm_to_ptr([x], [x], False, False, arena.ptr(0, off), 200, 0.5, True, 2, [], 0)
    assert rel_err(torch.tril(fac), torch.tril(ref)) < 1e-4 and torch.triu(fac, 1).abs().max() == 0
    arena.mirror_lower(torch.tensor([[off, 200]], dtype=torch.int64, device=DEV), 200)
    assert rel_err(fac, ref) < 1e-4 and torch.equal(fac, fac.T)
    # slot transport: every rank stores its lower-triangular tiles into its own slot on the owner
    # (plain stores), the owner folds the slots into its running factor and mirrors
    owner, other = SymmetricArena.local_group(3 * 200 * 200 + 256, 2)
    (f_off, factor), (s_off, _) = owner.alloc(200, 200), owner.alloc(2, 200, 200)
    other.alloc(200, 200), other.alloc(2, 200, 200)
    factor.copy_(held + held.T)
    x2 = torch.randn(1000, 200, device=DEV).to(torch.bfloat16)
    for rank, data in enumerate((x, x2)):   # both emulated ranks send to rank 0
        ext.umma_gemm_to_ptr([data], [data], False, False, owner.ptr(0, s_off + rank * 200 * 200), 200, 0.5,
                             True, 3, [], 0)
    owner.reduce_slots(torch.tensor([[f_off, s_off, 200]], dtype=torch.int64, device=DEV), 200 * 200, 200, 0.25)
    want = 0.25 * (held + held.T) + 0.5 * (ref + x2.float().T @ x2.float())
    assert rel_err(factor, want) < 1e-4 and torch.equal(factor, factor.T)
    # pull transport: every rank stores its share into ITS OWN buffer (same offset everywhere) and the owner
    # reads all ranks' copies while it sums (five emulated ranks: the kernel loads from four ranks at a time, so
    # both the full group and the remainder are exercised)
    group = SymmetricArena.local_group(2 * 200 * 200 + 256, 5)
    offs = [(g.alloc(200, 200), g.alloc(200, 200)) for g in group]
    (pf_off, pfactor), (share_off, _) = offs[0]
    pfactor.copy_(held + held.T)
    datas = [torch.randn(300 + 8 * r, 200, device=DEV).to(torch.bfloat16) for r in range(5)]
    for r, (g, data) in enumerate(zip(group, datas)):
        ext.umma_gemm_to_ptr([data], [data], False, False, g.ptr(r, share_off), 200, 0.5, True, 3, [], 0)
    group[0].pull_slots(torch.tensor([[pf_off, share_off, 200]], dtype=torch.int64, device=DEV), 200, 0.25)
    want = 0.25 * (held + held.T) + 0.5 * sum(d.float().T @ d.float() for d in datas)
    assert rel_err(pfactor, want) < 1e-4 and torch.equal(pfactor, pfactor.T)
    a = torch.randn(96, 160, device=DEV).to(torch.bfloat16)   # [K, M]
    b = torch.randn(96, 72, device=DEV).to(torch.bfloat16)    # [K, N]
    outs = [torch.zeros(160, 72, device=DEV) for _ in range(4)]
    ext.umma_gemm_to_ptr([a], [b], False, False, outs[0].data_ptr(), 72, 2.0, False, False,
                         [o.data_ptr() for o in outs[1:]], 0)
    want = 2.0 * a.float().T @ b.float()
    for o in outs:
        assert rel_err(o, want) < 1e-5
    ops.check_status()


def test_barrier_completes_alone_and_gives_up_on_a_missing_peer(ext):
    """A one-rank barrier passes.  A two-rank barrier whose peer never arrives runs into its wait
    limit, reports it through the status word and leaves the context usable."""
    from asdl_b200.parallel.symmetric import SymmetricArena
    solo = SymmetricArena.local_group(64, 1)[0]
    for _ in range(3):
        solo.barrier()
    ops.check_status()
    assert solo.buffer[:256].view(torch.int32)[63].item() == 3   # entered three times
    pair = SymmetricArena.local_group(64, 2)
    ext.symm_barrier(pair[0].peers_dev, 0, 2, 0, 50)             # nothing ever sets rank 1's flag
    with pytest.raises(RuntimeError, match='peer'):
        ops.check_status()
    ops.check_status()                                           # the status was cleared by the read
    y = torch.randn(256, 64, device=DEV)
    assert rel_err(ops.gram(y), y.T @ y) < 5e-5                   # the GPU still works


def test_fused_kfac_cuda_graph_matches_cpu():
    _fused_kfac_gpu_matches_cpu(True)


@pytest.mark.parametrize('m,n,k,sym', [(256, 256, 2048, False), (200, 328, 1000, False), (384, 384, 4096, True),
                                       (130, 130, 192, True)])
def test_fp32_grade_product_from_three_way_splits(ext, m, n, k, sym):
    """Six part products, one accumulation chunk per K block: the result has to be as good as an fp32
    product (a single long bf16x3 accumulation in TMEM is off by ~1e-5 from truncation alone)."""
    torch.manual_seed(0)
    a = torch.randn(k, m, device=DEV) * torch.logspace(-2, 2, m, device=DEV)
    b = a if sym else torch.randn(k, n, device=DEV)
    ap, bp = ops.split3(a), ops.split3(b)
    out = torch.full((m, n), float('nan'), device=DEV)
    parts = [torch.zeros(m, (n + 63) // 64 * 64, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    ops.matmul_fp32_tc(ap, bp, False, False, out=out, sym=sym, out_parts=parts)
    ref = a.double().T @ b.double()
    fp32 = (a.T @ b).double()
    err, err32 = (out.double() - ref).abs().max().item(), (fp32 - ref).abs().max().item()
    assert err <= 4 * err32 + 1e-30, (err, err32)
    assert rel_err(out, ref.float()) < 3e-7
    total = sum(p[:, :n].double() for p in parts)
    assert (total - out.double()).abs().max().item() <= out.abs().max().item() * 2.0 ** -22
    if sym:
        assert torch.equal(out, out.T)
    # K-major operands give the same product
    out2 = torch.empty(m, n, device=DEV)
    ak, bk = ops.split3(a.T.contiguous()), ops.split3(b.T.contiguous())
    ops.matmul_fp32_tc(ak, bk, True, True, out=out2)
    assert rel_err(out2, ref.float()) < 3e-7


@pytest.mark.parametrize('mode', [2])
def test_wide_tiles_match_narrow_tiles(ext, mode):
    torch.manual_seed(0)
    try:
        for rows, n in [(2048, 1024), (704, 392), (4096, 136)]:
            x = torch.randn(rows, n, device=DEV).to(torch.bfloat16)
            y = torch.randn(rows, 520, device=DEV).to(torch.bfloat16)
            for nsplit in (1, 3):
                ext.set_gemm_wide(0)
                c0 = torch.empty(n, n, device=DEV)
                ext.umma_gemm([x], [x], False, False, c0, 1.0, 0.0, True, None, None, nsplit)
                g0 = torch.empty(n, 520, device=DEV)
                ext.umma_gemm([x], [y], False, False, g0, 1.0, 0.0, False, None, None, nsplit)
                ext.set_gemm_wide(mode)
                c1 = torch.full((n, n), float('nan'), device=DEV)
                ext.umma_gemm([x], [x], False, False, c1, 1.0, 0.0, True, None, None, nsplit)
                g1 = torch.full((n, 520), float('nan'), device=DEV)
                ext.umma_gemm([x], [y], False, False, g1, 1.0, 0.0, False, None, None, nsplit)
                g2 = torch.full((n, 520), float('nan'), device=DEV)
                ext.umma_gemm([x], [y.T.contiguous()], False, True, g2, 1.0, 0.0, False, None, None, nsplit)
                assert rel_err(c1, c0) < 1e-6 and torch.equal(c1, c1.T)
                assert rel_err(g1, g0) < 1e-6 and rel_err(g2, g0) < 1e-6
    finally:
        ext.set_gemm_wide(-1)
    ops.check_status()


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
@pytest.mark.parametrize('n1,n2,d_in,d_out', [(200, 200, 300, 10), (130, 77, 72, 260), (5, 300, 9, 1)])
def test_gram_hadamard_kernel(n1, n2, d_in, d_out, dtype):
    """kernel += scale * (a1 a2^T + one) o (g1 g2^T) against fp64 from the same (rounded) inputs."""
    torch.manual_seed(0)
    a1, g1 = torch.randn(n1, d_in, device=DEV).to(dtype), torch.randn(n1, d_out, device=DEV).to(dtype)
    same = n1 == n2
    a2 = a1 if same else torch.randn(n2, d_in, device=DEV).to(dtype)
    g2 = g1 if same else torch.randn(n2, d_out, device=DEV).to(dtype)
    start = torch.randn(n1, n2, device=DEV)
    kernel = start.clone()
    before = ops.extension().launch_count()
    ops.gram_hadamard(kernel, a1, g1, None if same else a2, None if same else g2, one=1.0, scale=0.25)
    assert ops.extension().launch_count() - before <= 1 + 4          # the product itself + operand staging
    ref = start.double() + 0.25 * (a1.double() @ a2.double().T + 1.0) * (g1.double() @ g2.double().T)
    # fp32 inputs: three bf16 part products per Gram (the lo . lo term, 2^-16 relative, is left out)
    assert rel_err(kernel, ref.float()) < (2e-5 if dtype == torch.float32 else 2e-6), rel_err(kernel, ref.float())
    ops.check_status()


def test_hadamard_ntk_on_cuda_matches_cpu():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(), nn.Flatten(), nn.Linear(8 * 36, 32), nn.ReLU(),
                          nn.Linear(32, 4, bias=False))
    x1, x2 = torch.randn(9, 3, 6, 6), torch.randn(5, 3, 6, 6)
    want = asdl.empirical_class_wise_hadamard_ntk(model, x1, x2)
    before = ops.extension().launch_count()
    got = asdl.empirical_class_wise_hadamard_ntk(copy.deepcopy(model).to(DEV), x1.to(DEV), x2.to(DEV))
    assert ops.extension().launch_count() > before
    assert rel_err(got.cpu(), want) < 1e-5
    want1 = asdl.empirical_class_wise_hadamard_ntk(model, x1)
    got1 = asdl.empirical_class_wise_hadamard_ntk(copy.deepcopy(model).to(DEV), x1.to(DEV))
    assert rel_err(got1.cpu(), want1) < 1e-5
    ops.check_status()


@pytest.mark.parametrize('n', [1, 33, 200, 1000])
def test_bfgs_kernels_match_the_pytorch_path(n):
    """Powell damping and the rank-2 update of the inverse on CUDA against the same functions on CPU
    (PyTorch ops), for a pair with and a pair without usable curvature."""
    from asdl_b200.precondition.kbfgs import powell_lm_damping_, bfgs_inv_update_
    torch.manual_seed(n)
    base = torch.randn(n, n)
    H0 = base @ base.T / n + torch.eye(n) + 1e-3 * torch.randn(n, n)       # not exactly symmetric
    for flip in (1.0, -1.0):
        s0, y0 = torch.randn(n), torch.randn(n)
        y0 = flip * (y0 + 2 * s0)                                          # flip = -1: s^T y < 0
        Hc, sc, yc = H0.clone(), s0.clone(), y0.clone()
        Hg, sg, yg = H0.to(DEV), s0.to(DEV), y0.to(DEV)
        before = ops.extension().launch_count()
        powell_lm_damping_(Hc, sc, yc, 0.2, 0.1)
        powell_lm_damping_(Hg, sg, yg, 0.2, 0.1)
        assert rel_err(sg.cpu(), sc) < 1e-5 and rel_err(yg.cpu(), yc) < 1e-5
        bfgs_inv_update_(Hc, sc, yc)
        bfgs_inv_update_(Hg, sg, yg)
        assert ops.extension().launch_count() - before == 5
        assert rel_err(Hg.cpu(), Hc) < 1e-5, rel_err(Hg.cpu(), Hc)
        assert torch.equal(Hg, Hg.T)
        # a pair without curvature leaves the (symmetrised) matrix alone
        Hc2, Hg2 = H0.clone(), H0.to(DEV)
        bfgs_inv_update_(Hc2, s0.clone(), -s0.clone())
        bfgs_inv_update_(Hg2, s0.to(DEV), -s0.to(DEV))
        assert rel_err(Hg2.cpu(), Hc2) < 1e-6
    ops.check_status()


def test_embedding_statistics_kernels():
    torch.manual_seed(0)
    emb = nn.Embedding(37, 20, padding_idx=3)
    idx = torch.randint(0, 37, (6, 11))
    idx[0, :4] = 3
    g = torch.randn(6, 11, 20)
    from asdl_b200.operations.embedding import Embedding as EmbOp
    want_diag = EmbOp.cov_diag_weight(emb, idx, g)
    want_A = EmbOp.cov_kron_A(emb, idx)
    emb_g = copy.deepcopy(emb).to(DEV)
    before = ops.extension().launch_count()
    got_diag = EmbOp.cov_diag_weight(emb_g, idx.to(DEV), g.to(DEV))
    got_diag16 = EmbOp.cov_diag_weight(emb_g, idx.to(DEV), g.to(DEV).to(torch.bfloat16))
    got_A = EmbOp.cov_kron_A(emb_g, idx.to(DEV))
    assert ops.extension().launch_count() - before >= 4
    assert rel_err(got_diag.cpu(), want_diag) < 1e-6
    assert rel_err(got_diag16.cpu(), want_diag) < 1e-2
    assert got_diag[3].abs().max().item() == 0.0
    assert torch.equal(got_A.cpu(), want_A)        # small integer counts: exact
    ops.check_status()


def test_cvp_and_cov_on_cuda_match_cpu():
    """Layer-wise covariance (SYRK of the per-example gradients) and covariance-vector products (two
    GEMMs over the batch for Linear layers) against the CPU path."""
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(12, 20), nn.Tanh(), nn.Linear(20, 7, bias=False), nn.Tanh(), nn.Linear(7, 3))
    x, t = torch.randn(16, 12), torch.randint(0, 3, (16,))
    vec = [torch.randn_like(p) for p in model.parameters()]

    def run(model, x, t, vec):
        cfg = asdl.FisherConfig(fisher_type=asdl.FISHER_EMP, fisher_shapes=[asdl.SHAPE_LAYER_WISE], data_size=16)
        fm = asdl.get_fisher_maker(model, cfg)
        d = fm.setup_model_call(model, x)
        fm.setup_loss_call(F.cross_entropy, d, t)
        fm.forward_and_backward()
        covs = [m.fisher.data.detach().cpu().clone() for m in model if hasattr(m, 'fisher')]
        fm = asdl.get_fisher_maker(model, cfg)
        d = fm.setup_model_call(model, x)
        fm.setup_loss_call(F.cross_entropy, d, t)
        fm.forward_and_backward(fvp=True, vec=asdl.ParamVector(list(model.parameters()), vec))
        fvps = [v.detach().cpu().clone() for m in model if hasattr(m, 'fvp') for v in m.fvp.values()]
        return covs, fvps

    covs_c, fvps_c = run(model, x, t, vec)
    before = ops.extension().launch_count()
    covs_g, fvps_g = run(copy.deepcopy(model).to(DEV), x.to(DEV), t.to(DEV), [v.to(DEV) for v in vec])
    assert ops.extension().launch_count() > before
    assert len(covs_c) == 3 and len(fvps_c) == 5
    for a, b in zip(covs_c, covs_g):
        assert rel_err(b, a) < 2e-5
    for a, b in zip(fvps_c, fvps_g):
        assert rel_err(b, a) < 2e-5
    ops.check_status()


def test_general_matmul_and_psgd_dense_products():
    """ops.matmul in its four operand layouts (no transpose copies) and the dense Kronecker PSGD step and
    application built on it, against fp64 / the CPU path."""
    from asdl_b200.precondition.psgd import update_precond_kron, precond_grad_kron
    torch.manual_seed(0)
    a, b = torch.randn(300, 520, device=DEV), torch.randn(520, 264, device=DEV)
    ref = a.double() @ b.double()
    for ta in (False, True):
        for tb in (False, True):
            x = a.T.contiguous() if ta else a
            y = b.T.contiguous() if tb else b
            assert rel_err(ops.matmul(x, y, trans_a=ta, trans_b=tb), ref.float()) < 2e-5
    acc = torch.ones(300, 300, device=DEV)
    ops.matmul(a, a, trans_b=True, alpha=-0.5, out=acc, beta=2.0, sym=True)
    assert rel_err(acc, (2.0 - 0.5 * (a.double() @ a.double().T)).float()) < 2e-5
    # one PSGD fitting step and one application with 320 x 320 and 260 x 260 upper-triangular factors
    m, n = 320, 260
    Ql = torch.triu(torch.randn(m, m) * 0.05) + torch.eye(m)
    Qr = torch.triu(torch.randn(n, n) * 0.05) + torch.eye(n)
    dX, dG, grad = torch.randn(m, n) * 0.1, torch.randn(m, n), torch.randn(m, n)
    Ql_g, Qr_g = Ql.to(DEV), Qr.to(DEV)
    before = ops.extension().launch_count()
    new_l, new_r = update_precond_kron(Ql.clone(), Qr.clone(), dX, dG, step=0.05)
    got_l, got_r = update_precond_kron(Ql_g, Qr_g, dX.to(DEV), dG.to(DEV), step=0.05)
    assert ops.extension().launch_count() > before
    assert rel_err(got_l.cpu(), new_l) < 1e-4 and rel_err(got_r.cpu(), new_r) < 1e-4
    assert rel_err(got_l.cpu() - Ql, new_l - Ql) < 2e-3          # the update itself, not only the factor
    want = precond_grad_kron(new_l, new_r, grad)
    got = precond_grad_kron(got_l, got_r, grad.to(DEV))
    assert rel_err(got.cpu(), want) < 1e-4
    ops.check_status()


@pytest.mark.parametrize('n,c,h,w,kh,kw,ph,pw', [(4, 64, 20, 20, 3, 3, 1, 1), (3, 128, 14, 14, 3, 3, 1, 1),
                                                 (2, 64, 7, 7, 3, 3, 1, 1), (2, 64, 10, 13, 3, 2, 1, 0),
                                                 (2, 192, 9, 9, 3, 3, 0, 0), (1, 64, 33, 17, 2, 3, 1, 2)])
def test_implicit_im2col_syrk_matches_the_explicit_patch_matrix(ext, n, c, h, w, kh, kw, ph, pw):
    """A factor of a stride-1 convolution gathered inside the SYRK by 4-D TMA boxes (padding, ragged image
    edges, pixel blocks past the image) against the same product from the explicit bf16 patch matrix and
    against fp64; alone, with a moving average, and inside a deferred batch."""
    torch.manual_seed(0)
    conv = nn.Conv2d(c, 8, (kh, kw), padding=(ph, pw)).to(DEV)
    x = torch.randn(n, c, h, w, device=DEV).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    saved, saved_mb = ops.IMPLICIT_IM2COL, ops.IMPLICIT_IM2COL_MIN_MB
    try:
        ops.IMPLICIT_IM2COL_MIN_MB = 0.0          # the size threshold is a speed policy: every eligible layer here
        ops.IMPLICIT_IM2COL = False
        want = ops.conv_patch_gram(x, conv, scale=0.5, channels_last_order=True)
        ops.IMPLICIT_IM2COL = True
        before = ext.launch_count()
        got = ops.conv_patch_gram(x, conv, scale=0.5, channels_last_order=True)
        assert ext.launch_count() - before <= 2            # the SYRK (+ its split-K reduction), no im2col kernel
        assert rel_err(got, want) < 1e-5 and torch.equal(got, got.T)
        patches = F.unfold(x.float(), (kh, kw), padding=(ph, pw))                      # n x (c kh kw) x L, (c, kh, kw) order
        patches = patches.view(n, c, kh * kw, -1).permute(0, 2, 1, 3).reshape(n, c * kh * kw, -1)
        rows = patches.permute(0, 2, 1).reshape(-1, c * kh * kw).double()
        assert rel_err(got, (0.5 * rows.T @ rows).float()) < 1e-5
        # moving average into an existing factor, and the same product recorded in a deferred batch
        acc = want.clone()
        ops.conv_patch_gram(x, conv, scale=0.5, out=acc, beta=0.25, channels_last_order=True)
        assert rel_err(acc, 1.25 * want) < 1e-5
        out_b = torch.full_like(want, float('nan'))
        other = torch.randn(300, 72, device=DEV).to(torch.bfloat16)
        ext.gemm_batch_begin()
        try:
            ops.conv_patch_gram(x, conv, scale=0.5, out=out_b, channels_last_order=True)
            g_other = ops.gram(other)
        finally:
            ext.gemm_batch_end()
        assert rel_err(out_b, want) < 1e-5     # another split of the pixel range: another summation order
        # the data-parallel statistics path: lower-triangular tiles stored to / added at a raw address
        ncol = c * kh * kw
        slot = torch.zeros(ncol, ncol, device=DEV)
        ext.umma_syrk_conv(x, None, kh, kw, ph, pw, 0.5, 0.0, 0, slot.data_ptr(), ncol, 3)
        assert rel_err(torch.tril(slot), torch.tril(want)) < 1e-5 and torch.triu(slot, 1).abs().max() == 0
        ext.umma_syrk_conv(x, None, kh, kw, ph, pw, 0.5, 0.0, 0, slot.data_ptr(), ncol, 2)
        assert rel_err(torch.tril(slot), 2 * torch.tril(want)) < 1e-5 and torch.triu(slot, 1).abs().max() == 0
        assert rel_err(g_other, other.float().T @ other.float()) < 1e-5
    finally:
        ops.IMPLICIT_IM2COL, ops.IMPLICIT_IM2COL_MIN_MB = saved, saved_mb
    ops.check_status()


def test_cta_pair_tiles_match_narrow_tiles(ext):
    """cta_group::2 flavour (256 x 256 tiles over two SMs) against the 128 x 128 flavour: even and odd
    counts of 128-row tiles, ragged edges, split-K, K-major operands, several segments, beta and the
    bf16 images of the result."""
    torch.manual_seed(0)
    try:
        for rows, n, ny in [(2048, 1024, 1032), (704, 1160, 1288), (1000, 1288, 2048), (304, 200, 72), (64, 136, 520)]:
            x = torch.randn(rows, n, device=DEV).to(torch.bfloat16)
            y = torch.randn(rows, ny, device=DEV).to(torch.bfloat16)
            x2 = torch.randn(rows, n, device=DEV).to(torch.bfloat16)
            for nsplit in (1, 3):
                res = []
                for mode in (0, 4):
                    ext.set_gemm_wide(mode)
                    c = torch.full((n, n), float('nan'), device=DEV)
                    ext.umma_gemm([x], [x], False, False, c, 1.0, 0.0, True, None, None, nsplit)
                    g = torch.full((n, ny), float('nan'), device=DEV)
                    ext.umma_gemm([x], [y], False, False, g, 1.0, 0.0, False, None, None, nsplit)
                    gk = torch.full((n, ny), float('nan'), device=DEV)
                    ext.umma_gemm([x.T.contiguous()], [y.T.contiguous()], True, True, gk, 1.0, 0.0, False, None, None, nsplit)
                    s2 = torch.ones(n, n, device=DEV)
                    hi = torch.zeros(n, (n + 63) // 64 * 64, device=DEV, dtype=torch.bfloat16)
                    lo = torch.zeros_like(hi)
                    ext.umma_gemm([x, x2], [x, x2], False, False, s2, 0.5, 0.25, True, hi, lo, nsplit)
                    res.append((c, g, gk, s2, hi, lo))
                (c0, g0, gk0, s0, hi0, lo0), (c1, g1, gk1, s1, hi1, lo1) = res
                assert rel_err(c1, c0) < 1e-6 and torch.equal(c1, c1.T)
                assert rel_err(g1, g0) < 1e-6 and rel_err(gk1, g0) < 1e-6
                assert rel_err(s1, s0) < 1e-6 and torch.equal(s1, s1.T)
                assert rel_err(hi1[:, :n].float() + lo1[:, :n].float(), s1) < 1e-4
                assert rel_err(hi1.float(), hi0.float()) < 1e-2   # a last-bit difference of the sum may flip a bf16 rounding
            ref = x.float().T @ y.float()
            assert rel_err(g1, ref) < 1e-5
    finally:
        ext.set_gemm_wide(-1)
    ops.check_status()


@pytest.mark.parametrize('backend', ['tensor_core', 'cuda_core'])
@pytest.mark.parametrize('sizes', [[1], [128], [129, 300, 40], [1500, 640, 257], [2304, 576, 64, 64]])
def test_chol_inverse_backends(backend, sizes):
    """Both grouped inverses against fp64, on well and badly conditioned matrices."""
    torch.manual_seed(1)
    saved = ops.CHOLESKY_BACKEND
    ops.CHOLESKY_BACKEND = backend
    try:
        mats, damp = [], []
        for i, n in enumerate(sizes):
            a = torch.randn(n, max(n // 2, 1), device=DEV)      # rank-deficient: the damping carries the inverse
            mats.append(a @ a.T / max(n // 2, 1))
            damp.append(1e-3 * (i + 1))
        outs = [torch.empty_like(m) for m in mats]
        for _ in range(2):                                       # the second call runs from the cached tables
            ops.spd_inverse_grouped(mats, outs, torch.tensor(damp, device=DEV))
        ops.check_status()
        for m, o, d in zip(mats, outs, damp):
            n = m.shape[0]
            eye = torch.eye(n, device=DEV, dtype=torch.float64)
            ref = torch.linalg.inv(m.double() + d * eye)
            assert rel_err(o, ref.float()) < 2e-4, (n, rel_err(o, ref.float()))
            assert torch.equal(o, o.T)
            resid = ((m.double() + d * eye) @ o.double() - eye).abs().max().item()
            assert resid < 1e-3, (n, resid)
    finally:
        ops.CHOLESKY_BACKEND = saved


def test_inverse_root_chain_at_small_ridge():
    """The ViT Shampoo configuration: blocks of 1024, fourth roots, ridge 1e-6, condition number 1e6.
    At that conditioning any fp32 iteration is a few percent off the exact root (a perturbation of
    2^-24 of the largest eigenvalue is 6 % of the smallest); the tensor-core chain has to converge
    and be as accurate as the same iteration on fp32 matrix products of the library."""
    from asdl_b200.precondition import shampoo
    torch.manual_seed(0)
    n, p = 1024, 4
    q, _ = torch.linalg.qr(torch.randn(n, n, device=DEV, dtype=torch.float64))
    evals = torch.logspace(-8, 0, n, device=DEV, dtype=torch.float64)
    mats = torch.stack([(q * evals) @ q.T, (q * evals.flip(0) * 30) @ q.T]).float()
    ext = ops.extension()

    def errors(roots):
        out = []
        for m, r in zip(mats.double(), roots.double()):
            ev, evec = torch.linalg.eigh(m)
            ev = ev.clamp_min(0) + 1e-6 * ev.max()
            exact = (evec * ev.pow(-1.0 / p)) @ evec.T
            out.append(rel_err(r, exact))
        return out

    before = ext.launch_count()
    assert shampoo.TENSOR_CORE_ROOTS == 'auto'
    got = errors(shampoo.inverse_pth_root_batched(mats, p, ridge_epsilon=1e-6))
    assert ext.launch_count() - before > 10                # the grouped tensor-core chain ran
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    shampoo.TENSOR_CORE_ROOTS = 'never'
    try:
        want = errors(shampoo.inverse_pth_root_batched(mats, p, ridge_epsilon=1e-6))
    finally:
        shampoo.TENSOR_CORE_ROOTS = 'auto'
        torch.backends.cuda.matmul.allow_tf32 = prev
    print('inverse root errors: tensor-core chain', got, 'fp32 matmul', want)
    for g, w in zip(got, want):
        assert g < 0.1 and g < 1.5 * w + 2e-3, (got, want)
    ops.check_status()


def test_graph_is_captured_again_when_a_captured_hyper_parameter_changes():
    """Damping is read at capture time; changing it later has to take effect: the graphs are dropped
    (with a warning) and captured again.  The replayed run with the change has to follow the eager run
    with the same change, and to differ from a replayed run without it."""
    torch.backends.cudnn.allow_tf32 = False
    x = torch.randn(8, 3, 16, 16, device=DEV).contiguous(memory_format=torch.channels_last)
    t = torch.randint(0, 5, (8,), device=DEV)

    def run(graph, change):
        torch.manual_seed(0)
        model = _small_cnn().to(DEV).to(memory_format=torch.channels_last)
        cfg = asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=0.3, curvature_upd_interval=4,
                                         preconditioner_upd_interval=4)
        gm = asdl.FusedKfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP, cuda_graph=graph)
        out = []
        for step in range(10):      # no optimizer step: all runs see the same weights, only the maker differs
            if step == 6 and change:
                cfg.damping = 1.0
            for p in model.parameters():
                p.grad = None
            d = gm.setup_model_call(model, x)
            gm.setup_loss_call(F.cross_entropy, d, t)
            gm.forward_and_backward()
            out.append(torch.cat([p.grad.detach().flatten() for p in model.parameters()]).clone())
        return out, gm

    import warnings
    eager, _ = run(False, True)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter('always')
        replayed, gm = run(True, True)
    assert any('captured again' in str(w.message) for w in caught)
    assert gm.replayed_launches > 0 and gm._graphs                     # replaying again after the change
    unchanged, _ = run(True, False)
    for step in range(10):
        assert rel_err(replayed[step], eager[step]) < 5e-3, (step, rel_err(replayed[step], eager[step]))
    # the inverses are refreshed at step 8 with the new damping: from then on the change has to show
    assert rel_err(replayed[9], unchanged[9]) > 0.05
    assert rel_err(replayed[5], unchanged[5]) < 1e-6
    ops.check_status()


@pytest.mark.parametrize('fisher,loss', [('fisher_mc', 'mse'), ('fisher_exact', 'cross_entropy'),
                                         ('fisher_exact', 'mse'), ('fisher_mc2', 'cross_entropy')])
def test_fused_kfac_fisher_variants_and_reused_layer_match_cpu(fisher, loss):
    """Several backward passes per curvature step (exact Fisher: one per output; Monte-Carlo with two
    samples) and a layer applied twice: every further contribution adds to the statistics of the step
    through the GEMM's accumulate epilogue.  Compared with the same maker on the CPU (PyTorch path),
    with a fixed sampling seed where labels are sampled."""
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(0)
            self.conv = nn.Conv2d(3, 8, 3, padding=1)
            self.shared = nn.Linear(8, 8)
            self.head = nn.Linear(8, 4)

        def forward(self, x):
            x = F.relu(self.conv(x)).mean(dim=(2, 3))
            x = F.relu(self.shared(x))
            x = F.relu(self.shared(x))
            return self.head(x)

    n_mc = 2 if fisher == 'fisher_mc2' else 1
    ftype = asdl.FISHER_EXACT if fisher == 'fisher_exact' else asdl.FISHER_MC
    ltype = asdl.LOSS_MSE if loss == 'mse' else asdl.LOSS_CROSS_ENTROPY
    x = torch.randn(6, 3, 8, 8)
    t = torch.randn(6, 4) if loss == 'mse' else torch.randint(0, 4, (6,))
    loss_fn = F.mse_loss if loss == 'mse' else F.cross_entropy

    def factors(dev):
        model = Net().to(dev)
        cfg = asdl.PreconditioningConfig(data_size=6, damping=1e-2, ema_decay=0.5, curvature_upd_interval=1,
                                         preconditioner_upd_interval=1)
        gm = asdl.FusedKfacGradientMaker(model, cfg, fisher_type=ftype, loss_type=ltype, n_mc_samples=n_mc, seed=3)
        for _ in range(2):
            d = gm.setup_model_call(model, x.to(dev))
            gm.setup_loss_call(loss_fn, d, t.to(dev))
            gm.forward_and_backward()
        return [(st.A.cpu(), st.B.cpu()) for st in gm._kron], [p.grad.cpu() for p in model.parameters()]

    exact = fisher == 'fisher_exact'           # sampled labels come from different generators on CPU and GPU
    f_cpu, g_cpu = factors(torch.device('cpu'))
    f_gpu, g_gpu = factors(torch.device(DEV))
    for (a1, b1), (a2, b2) in zip(f_cpu, f_gpu):
        assert rel_err(a2, a1) < 1e-4                    # input-side statistics never depend on the sampling
        if exact:
            assert rel_err(b2, b1) < 1e-3
        else:
            assert torch.isfinite(b2).all() and b2.abs().sum() > 0
    if exact:
        for a, b in zip(g_cpu, g_gpu):
            assert rel_err(b, a) < 5e-3
    ops.check_status()


@pytest.mark.parametrize('n,batch', [(1, 2), (2, 3), (7, 2), (64, 4), (100, 2), (127, 1), (128, 2), (160, 2)])
def test_jacobi_eigh_kernel(ext, n, batch):
    """Batched Jacobi eigensolver against float64 torch.linalg.eigh: eigenvalues, residual and
    orthogonality, on matrices with eigenvalues spread over eight decades."""
    torch.manual_seed(n)
    q, _ = torch.linalg.qr(torch.randn(batch, n, n, device=DEV, dtype=torch.float64))
    lam = torch.logspace(-6, 2, n, device=DEV, dtype=torch.float64).expand(batch, n) * (1 + torch.rand(batch, n, device=DEV))
    mats = ((q * lam.unsqueeze(1)) @ q.transpose(1, 2)).float()
    before = ext.launch_count()
    w, v = ops.eigh(mats)
    assert ext.launch_count() > before
    ref = torch.linalg.eigvalsh(mats.double())
    scale = ref.abs().amax(dim=1, keepdim=True)
    assert ((w.double() - ref).abs() <= 5e-5 * scale).all()
    assert (w[:, 1:] >= w[:, :-1]).all()
    eye = torch.eye(n, device=DEV, dtype=torch.float64)
    vd = v.double()
    assert (vd.transpose(1, 2) @ vd - eye).abs().max().item() < 5e-5
    resid = (mats.double() @ vd - vd * w.double().unsqueeze(1)).abs().amax(dim=(1, 2)) / scale.squeeze(1)
    assert resid.max().item() < 5e-5
    assert ((ops.eigvalsh(mats[0]).double() - ref[0]).abs() <= 5e-5 * scale[0]).all()
    ops.check_status()


@pytest.mark.parametrize('rows,d,dtype', [(37, 24, torch.float32), (512, 768, torch.bfloat16), (4099, 1000, torch.bfloat16)])
def test_layernorm_unitwise_and_diag_stats_kernels(ext, rows, d, dtype):
    torch.manual_seed(0)
    y = torch.randn(rows, d, device=DEV).to(dtype)
    g = torch.randn(rows, d, device=DEV).to(dtype)
    weight, bias = torch.rand(d, device=DEV) + 0.5, torch.randn(d, device=DEV)
    old = torch.rand(d, 2, 2, device=DEV)
    got = ops.layernorm_unitwise_stats(y, g, weight, bias, out=old.clone(), alpha=0.3, beta=0.7)
    ops.set_backend('torch')
    want = ops.layernorm_unitwise_stats(y, g, weight, bias, out=old.clone(), alpha=0.3, beta=0.7)
    ops.set_backend('auto')
    assert rel_err(got, want) < 2e-5
    a = torch.randn(rows, 40, device=DEV).to(dtype)
    o0, b0 = torch.rand(d, 40, device=DEV), torch.rand(d, device=DEV)
    got_w, got_b = ops.diag_linear_stats(a, g, out=o0.clone(), out_bias=b0.clone(), alpha=0.5, beta=0.25)
    want_w = 0.25 * o0 + 0.5 * (g.double().square().T @ a.double().square()).float()
    want_b = 0.25 * b0 + 0.5 * g.double().square().sum(dim=0).float()
    assert rel_err(got_w, want_w) < 2e-5 and rel_err(got_b, want_b) < 2e-5
    ops.check_status()


def test_multi_tensor_unitwise_and_bias_kernels(ext):
    torch.manual_seed(0)
    sizes = [8, 24, 257, 1000]
    stats = [torch.rand(f, 2, 2, device=DEV) for f in sizes]
    stats = [s @ s.transpose(1, 2) for s in stats]
    invs = [torch.empty_like(s) for s in stats]
    ext.unitwise_inverse_mt([[s.data_ptr(), i.data_ptr(), s.shape[0]] for s, i in zip(stats, invs)], 0.1)
    for s, i in zip(stats, invs):
        assert rel_err(i, torch.linalg.inv(s.double() + 0.1 * torch.eye(2, device=DEV, dtype=torch.float64)).float()) < 1e-5
    gw = [torch.randn(f, device=DEV) for f in sizes]
    gb = [torch.randn(f, device=DEV) for f in sizes]
    want = [(i.double() @ torch.stack([w, b], dim=1).double().unsqueeze(2) * 0.5).squeeze(2) for i, w, b in zip(invs, gw, gb)]
    ext.unitwise_apply_mt([[i.data_ptr(), w.data_ptr(), b.data_ptr(), i.shape[0]] for i, w, b in zip(invs, gw, gb)], 0.5)
    for (w, b), ref in zip(zip(gw, gb), want):
        assert rel_err(w, ref[:, 0].float()) < 1e-5 and rel_err(b, ref[:, 1].float()) < 1e-5
    mats = [torch.randn(n, n, device=DEV) for n in (5, 64, 1000)]
    vecs = [torch.randn(m.shape[0], device=DEV) for m in mats]
    want = [(m.double() @ v.double() * 2.0).float() for m, v in zip(mats, vecs)]
    scratch = [torch.empty_like(v) for v in vecs]
    ext.bias_precondition_mt([[m.data_ptr(), v.data_ptr(), s.data_ptr(), m.shape[0]] for m, v, s in zip(mats, vecs, scratch)], 2.0)
    for v, ref in zip(vecs, want):
        assert rel_err(v, ref) < 1e-5
    ops.check_status()


@pytest.mark.parametrize('b,n', [(3, 257), (8, 1024), (1, 5)])
def test_batched_matrix_vector_kernel(ext, b, n):
    torch.manual_seed(0)
    a, x = torch.randn(b, n, n, device=DEV), torch.randn(b, n, device=DEV)
    got = ext.batched_mv(a, x)
    want = torch.bmm(a.double(), x.double().unsqueeze(2)).squeeze(2).float()
    assert rel_err(got, want) < 1e-5
