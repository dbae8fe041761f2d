"""The PyTorch paths of ``asdl_b200.ops`` (the oracles that the CUDA kernels are tested against)
checked against independent formulas: per-example loops, ``torch.linalg`` and autograd."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from asdl_b200 import ops


def test_gram_matmul_and_kron_apply():
    torch.manual_seed(0)
    a, b = torch.randn(10, 4), torch.randn(10, 3)
    torch.testing.assert_close(ops.gram(a, scale=0.5), 0.5 * sum(torch.outer(r, r) for r in a))
    out = torch.ones(4, 4)
    ops.gram(a, scale=2.0, out=out, beta=0.25)                       # moving average in place
    torch.testing.assert_close(out, 0.25 * torch.ones(4, 4) + 2.0 * a.T @ a)
    torch.testing.assert_close(ops.matmul_tn(a, b, scale=3.0), 3.0 * a.T @ b)
    out = torch.full((4, 3), 2.0)
    ops.matmul_tn(a, b, out=out, beta=0.5)
    torch.testing.assert_close(out, 1.0 + a.T @ b)
    left, right = ops.gram(torch.randn(7, 4)), ops.gram(torch.randn(9, 3))
    mid = torch.randn(4, 3)
    torch.testing.assert_close(ops.kron_apply(left, mid, right), left @ mid @ right)
    # ... which is the Kronecker product applied to the row-major flattened matrix
    torch.testing.assert_close(ops.kron_apply(left, mid, right).flatten(), torch.kron(left, right) @ mid.flatten(),
                               rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize('conv_kw', [dict(kernel_size=3), dict(kernel_size=3, stride=2, padding=1),
                                     dict(kernel_size=(2, 3), padding=(1, 0), dilation=(1, 2)), dict(kernel_size=1)])
def test_conv_patch_gram_in_both_column_orders(conv_kw):
    torch.manual_seed(0)
    conv = nn.Conv2d(3, 4, **conv_kw)
    x = torch.randn(2, 3, 7, 7)
    kh, kw = conv.kernel_size
    cols = F.unfold(x, conv.kernel_size, conv.dilation, conv.padding, conv.stride)        # n x (c kh kw) x L
    rows = cols.permute(0, 2, 1).reshape(-1, cols.shape[1])
    torch.testing.assert_close(ops.conv_patch_gram(x, conv, scale=0.1), 0.1 * rows.T @ rows, rtol=1e-4, atol=1e-5)
    reordered = rows.view(-1, 3, kh * kw).permute(0, 2, 1).reshape(rows.shape[0], -1)    # (kh, kw, c) columns
    torch.testing.assert_close(ops.conv_patch_gram(x, conv, channels_last_order=True), reordered.T @ reordered,
                               rtol=1e-4, atol=1e-5)


def test_spd_inverses():
    torch.manual_seed(0)
    mats = [ops.gram(torch.randn(n + 3, n)) for n in (3, 8, 5)]
    single = ops.spd_inverse(mats[1], 0.1)
    torch.testing.assert_close(single, torch.linalg.inv(mats[1] + 0.1 * torch.eye(8)), rtol=1e-4, atol=1e-5)
    before = [m.clone() for m in mats]
    for damping in (0.2, [0.1, 0.2, 0.3], torch.tensor([0.1, 0.2, 0.3])):
        outs = ops.spd_inverse_grouped(mats, [torch.empty_like(m) for m in mats], damping)
        values = [damping] * 3 if isinstance(damping, float) else [float(d) for d in damping]
        for m, o, d in zip(mats, outs, values):
            torch.testing.assert_close(o, torch.linalg.inv(m + d * torch.eye(m.shape[0])), rtol=1e-4, atol=1e-5)
    assert all(torch.equal(m, k) for m, k in zip(mats, before))
    blocks = torch.stack([ops.gram(torch.randn(4, 2)) for _ in range(6)])
    torch.testing.assert_close(ops.unitwise_inverse(blocks, 0.05), torch.linalg.inv(blocks + 0.05 * torch.eye(2)),
                               rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize('relu', [False, True])
def test_unit_wise_batchnorm_statistics(relu):
    """[[sum gw^2, sum gw gb], [sum gw gb, sum gb^2]] per channel, with the per-sample gradients of scale and
    shift gw = sum_hw xhat * g and gb = sum_hw g (normalised input held fixed, g masked by a fused ReLU)."""
    torch.manual_seed(0)
    bn = nn.BatchNorm2d(5)
    bn.weight.data.uniform_(0.5, 1.5)
    bn.bias.data.normal_()
    x = torch.randn(6, 5, 4, 4)
    y = bn(x).detach()
    dy = torch.randn(6, 5, 4, 4)
    mean = x.mean(dim=(0, 2, 3))
    invstd = torch.rsqrt(x.var(dim=(0, 2, 3), unbiased=False) + bn.eps)
    want = torch.zeros(5, 2, 2)
    for n in range(6):
        for c in range(5):
            g = dy[n, c] * ((y[n, c] > 0).float() if relu else 1.0)
            xh = (x[n, c] - mean[c]) * invstd[c]
            v = torch.stack([(xh * g).sum(), g.sum()])
            want[c] += torch.outer(v, v)
    if relu:
        got = ops.batchnorm_unitwise_stats_from_input(x, dy, torch.relu(y), mean, invstd, torch.zeros(5, 2, 2))
    else:   # from the output (xhat recovered as (y - bias) / weight) and from the input: the same blocks
        got = ops.batchnorm_unitwise_stats(y, dy, bn.weight.detach(), bn.bias.detach())
        also = ops.batchnorm_unitwise_stats_from_input(x, dy, None, mean, invstd, torch.zeros(5, 2, 2))
        torch.testing.assert_close(also, want, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-4)
    running = torch.ones(5, 2, 2)
    ops.batchnorm_unitwise_stats(y, dy * (y > 0 if relu else 1), bn.weight.detach(), bn.bias.detach(), out=running,
                                 alpha=0.5, beta=0.25)
    if not relu:
        torch.testing.assert_close(running, 0.25 + 0.5 * want, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize('residual,relu', [(False, False), (True, False), (False, True), (True, True)])
def test_batch_norm_train_matches_autograd_of_the_unfused_ops(residual, relu):
    torch.manual_seed(0)
    x = torch.randn(4, 6, 5, 5, requires_grad=True)
    w, b = torch.randn(6, requires_grad=True), torch.randn(6, requires_grad=True)
    res = torch.randn(4, 6, 5, 5, requires_grad=True) if residual else None
    rm, rv, count = torch.zeros(6), torch.ones(6), torch.zeros((), dtype=torch.long)
    y = ops.batch_norm_train(x, w, b, rm, rv, 0.1, 1e-5, residual=res, relu=relu, num_batches_tracked=count)
    ref_rm, ref_rv = torch.zeros(6), torch.ones(6)
    x2, w2, b2 = (t.detach().clone().requires_grad_(True) for t in (x, w, b))
    res2 = res.detach().clone().requires_grad_(True) if residual else None
    y2 = F.batch_norm(x2, ref_rm, ref_rv, w2, b2, True, 0.1, 1e-5)
    y2 = y2 + res2 if residual else y2
    y2 = torch.relu(y2) if relu else y2
    torch.testing.assert_close(y, y2)
    torch.testing.assert_close(rm, ref_rm)
    torch.testing.assert_close(rv, ref_rv)
    assert int(count) == 1
    weight = torch.randn_like(y)
    (y * weight).sum().backward()
    (y2 * weight).sum().backward()
    for got, want in ((x.grad, x2.grad), (w.grad, w2.grad), (b.grad, b2.grad)):
        torch.testing.assert_close(got, want)
    if residual:
        torch.testing.assert_close(res.grad, res2.grad)


def test_layer_norm_and_backends():
    torch.manual_seed(0)
    x = torch.randn(3, 7, 16, requires_grad=True)
    w, b = torch.randn(16, requires_grad=True), torch.randn(16, requires_grad=True)
    y = ops.layer_norm(x, w, b, 1e-5)
    mean, var = x.mean(-1, keepdim=True), x.var(-1, unbiased=False, keepdim=True)
    torch.testing.assert_close(y, (x - mean) / torch.sqrt(var + 1e-5) * w + b)
    assert ops.get_backend() in ('auto', 'torch')
    ops.set_backend('torch')
    try:
        assert not ops.cuda_kernels_enabled(x)
    finally:
        ops.set_backend('auto')
    with pytest.raises(ValueError):
        ops.set_backend('no_such_backend')
    ops.check_status()     # nothing to report without a GPU


def test_general_matmul_gram_hadamard_and_small_statistics():
    """PyTorch paths of the products and statistics added with the second kernel set: the general matmul
    in its four layouts, the Hadamard-factored Gram update, the BFGS pair damping / inverse update, and
    the embedding statistics, each against an independent formula."""
    torch.manual_seed(0)
    a, b = torch.randn(6, 9), torch.randn(9, 4)
    for ta in (False, True):
        for tb in (False, True):
            x, y = (a.T.contiguous() if ta else a), (b.T.contiguous() if tb else b)
            torch.testing.assert_close(ops.matmul(x, y, trans_a=ta, trans_b=tb, alpha=2.0), 2.0 * a @ b)
    out = torch.ones(6, 6)
    ops.matmul(a, a, trans_b=True, alpha=-1.0, out=out, beta=3.0, sym=True)
    torch.testing.assert_close(out, 3.0 - a @ a.T)
    torch.testing.assert_close(ops.matmul_nn(a, b, scale=0.5), 0.5 * a @ b)
    # kernel += scale * (a1 a2^T + one) o (g1 g2^T), entry by entry
    a1, a2, g1, g2 = torch.randn(5, 7), torch.randn(3, 7), torch.randn(5, 2), torch.randn(3, 2)
    kernel = torch.full((5, 3), 0.5)
    ops.gram_hadamard(kernel, a1, g1, a2, g2, one=1.0, scale=0.25)
    want = torch.tensor([[0.5 + 0.25 * (a1[i] @ a2[j] + 1.0) * (g1[i] @ g2[j]) for j in range(3)] for i in range(5)])
    torch.testing.assert_close(kernel, want)
    # BFGS: the updated inverse satisfies the secant equation H y = s for the damped pair and stays symmetric
    from asdl_b200.precondition.kbfgs import powell_lm_damping_, bfgs_inv_update_
    base = torch.randn(8, 8, dtype=torch.float64)
    H = base @ base.T / 8 + torch.eye(8, dtype=torch.float64)
    s, y = torch.randn(8, dtype=torch.float64), torch.randn(8, dtype=torch.float64)
    powell_lm_damping_(H, s, y, 0.2, 0.1)
    assert (s @ y) > 0
    bfgs_inv_update_(H, s, y)
    torch.testing.assert_close(H @ y, s)
    torch.testing.assert_close(H, H.T)
    # embedding: diagonal statistics and per-example counts against loops over tokens
    from asdl_b200.operations.embedding import Embedding as EmbOp
    emb = nn.Embedding(11, 4, padding_idx=2)
    idx, g = torch.randint(0, 11, (3, 5)), torch.randn(3, 5, 4)
    diag = torch.zeros(11, 4)
    counts = torch.zeros(3, 11)
    for n in range(3):
        for t in range(5):
            counts[n, idx[n, t]] += 1
            if idx[n, t] != 2:
                diag[idx[n, t]] += g[n, t] ** 2
    torch.testing.assert_close(EmbOp.cov_diag_weight(emb, idx, g), diag)
    torch.testing.assert_close(EmbOp.cov_kron_A(emb, idx), counts.T @ counts)


def test_gpu_only_policies_fall_back_on_cpu():
    """The tile policy, the implicit-im2col policy and the fused BatchNorm are CUDA paths: CPU tensors never
    qualify, and the convolution factor of a CPU input equals the product of its explicit patch matrix."""
    torch.manual_seed(0)
    conv = nn.Conv2d(64, 4, 3, padding=1)
    x = torch.randn(2, 64, 6, 6).to(memory_format=torch.channels_last)
    assert not ops.implicit_im2col_eligible(x.bfloat16(), (3, 3), (1, 1), (1, 1), (1, 1), (6, 6), True)
    assert not ops.batch_norm_train_supported(x.bfloat16(), torch.ones(64), torch.zeros(64))
    got = ops.conv_patch_gram(x, conv, scale=0.5, channels_last_order=True)
    patches = F.unfold(x, 3, padding=1).view(2, 64, 9, -1).permute(0, 2, 1, 3).reshape(2, 64 * 9, -1)
    rows = patches.permute(0, 2, 1).reshape(-1, 64 * 9)
    torch.testing.assert_close(got, 0.5 * rows.T @ rows, rtol=1e-4, atol=1e-4)
