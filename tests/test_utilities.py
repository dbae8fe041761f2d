"""Containers, helpers, kernels (NTK), counters and the matrix manager against plain-PyTorch oracles."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import DataLoader, TensorDataset

import asdl_b200 as asdl
from asdl_b200 import counter as C


def _mlp():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 5), nn.Tanh(), nn.Linear(5, 3))


def test_tril_roundtrip_and_symmatrix_files(tmp_path):
    torch.manual_seed(0)
    a = torch.randn(7, 7)
    a = a + a.T
    tril = asdl.matrix_to_tril(a)
    assert tril.numel() == 28 and asdl.get_n_cols_by_tril(tril) == 7
    torch.testing.assert_close(asdl.tril_to_matrix(tril), a)
    kron = asdl.Kron(torch.eye(3) * 2, a[:4, :4].clone())
    sym = asdl.SymMatrix(data=a.clone(), kron=kron)
    paths = sym.save(str(tmp_path), 'layer0')
    files = [os.path.join(dp, f) for dp, _, fs in os.walk(tmp_path) for f in fs]
    assert files and all(f.endswith('.npy') for f in files)
    assert paths == {'tril': 'layer0/tril.npy',
                     'kron': {'A_tril': 'layer0/kron/A_tril.npy', 'B_tril': 'layer0/kron/B_tril.npy'}}
    stored = np.load(os.path.join(tmp_path, paths['tril']))
    assert stored.ndim == 1 and stored.dtype == np.float32 and stored.size == 28   # row-major lower triangle
    loaded = asdl.SymMatrix()
    loaded.load(path=os.path.join(tmp_path, paths['tril']),
                kron_path={k: os.path.join(tmp_path, v) for k, v in paths['kron'].items()})
    torch.testing.assert_close(loaded.data, a)
    torch.testing.assert_close(loaded.kron.A, kron.A)
    torch.testing.assert_close(loaded.kron.B, kron.B)


def test_param_vector_algebra():
    model = _mlp()
    params = list(model.parameters())
    v = asdl.ParamVector(params, [torch.ones_like(p) for p in params])
    w = asdl.ParamVector(params, [torch.full_like(p, 2.0) for p in params])
    n = sum(p.numel() for p in params)
    assert v.numel() == n and abs(v.dot(w).item() - 2 * n) < 1e-4
    assert abs((v + w).norm().item() - 3 * n ** 0.5) < 1e-4
    u = v.copy().mul_(3.0).add_(w, alpha=-1)
    torch.testing.assert_close(u.get_flatten_vector(), torch.ones(n))
    sub = v.get_vectors_by_module(model[0])
    assert sub.numel() == 6 * 5 + 5
    torch.manual_seed(1)
    r = asdl.ParamVector(params, [torch.randn_like(p) for p in params])
    unit_v = asdl.normalization(v.copy())
    q = asdl.orthnormal(r, [unit_v])
    assert abs(q.norm().item() - 1) < 1e-4 and abs(q.dot(unit_v).item()) < 1e-5


def test_im2col_variants_and_woodbury_inverse():
    torch.manual_seed(0)
    conv = nn.Conv2d(3, 4, 3, stride=2, padding=1)
    x = torch.randn(2, 3, 9, 8)
    cols = asdl.im2col_2d(x, conv)
    torch.testing.assert_close(cols, asdl.im2col_2d_slow(x, conv))
    torch.testing.assert_close(cols, F.unfold(x, 3, padding=1, stride=2))
    out = torch.einsum('ok,nkp->nop', conv.weight.flatten(1), cols) + conv.bias.view(1, -1, 1)
    torch.testing.assert_close(out.view(2, 4, 5, 4), conv(x), rtol=1e-4, atol=1e-5)
    a = torch.randn(4, 9).double()                             # n < d: "swift" factor
    damping = 0.1
    dense = torch.linalg.inv(a.T @ a / 4 + damping * torch.eye(9).double())
    torch.testing.assert_close(asdl.smw_inv(a, damping), dense, rtol=1e-6, atol=1e-8)
    spd = a @ a.T + torch.eye(4).double()
    torch.testing.assert_close(asdl.cholesky_inv(spd.clone(), 0.5), torch.linalg.inv(spd + 0.5 * torch.eye(4).double()))


def test_pseudo_batch_loader_covers_the_dataset_once():
    data = TensorDataset(torch.arange(24).float())
    loader = DataLoader(data, batch_size=4, shuffle=True, drop_last=True)
    gen = asdl.PseudoBatchLoaderGenerator(loader, 12)
    seen = []
    assert len(gen) == 2
    for pb in gen:
        micro = [b[0] for b in pb]
        assert len(micro) == 3 and all(m.numel() == 4 for m in micro)
        seen += [int(v) for m in micro for v in m]
    assert sorted(seen) == list(range(24))


def test_empirical_ntk_matches_jacobian_products():
    model = _mlp()
    x1, x2 = torch.randn(4, 6), torch.randn(3, 6)

    def jac(x):
        rows = []
        for i in range(x.shape[0]):
            out = model(x[i:i + 1])[0]
            rows.append(torch.stack([torch.cat([g.flatten() for g in torch.autograd.grad(o, model.parameters(),
                                                                                        retain_graph=True)])
                                     for o in out]))
        return torch.stack(rows)                               # n x c x p
    j1, j2 = jac(x1), jac(x2)
    oracle = torch.einsum('ncp,mdp->nmcd', j1, j2)
    got = asdl.empirical_direct_ntk(model, x1, x2)
    torch.testing.assert_close(got, oracle, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(asdl.empirical_implicit_ntk(model, x1, x2), oracle, rtol=1e-4, atol=1e-5)
    class_wise = asdl.empirical_class_wise_direct_ntk(model, x1, x2)
    torch.testing.assert_close(class_wise, torch.einsum('ncp,mcp->nmc', j1, j2), rtol=1e-4, atol=1e-5)


def test_kernel_natural_gradient_equals_parameter_space_solution():
    """Function-space natural gradient with the full NTK equals J^T (K + damping)^-1 applied to the
    second-order output gradient (the identity behind asdl/kernel.py's natural_gradient_cross_entropy)."""
    model = _mlp()
    x, t = torch.randn(5, 6), torch.randint(0, 3, (5,))
    kernel = asdl.empirical_direct_ntk(model, x)
    model.zero_grad()
    asdl.natural_gradient_cross_entropy(model, x, t, kernel, damping=1e-3)
    grads = [p.grad.clone() for p in model.parameters()]
    assert all(torch.isfinite(g).all() for g in grads) and any(g.abs().sum() > 0 for g in grads)
    top = asdl.kernel_eigenvalues(model, x, top_n=1)
    dense = kernel.permute(0, 2, 1, 3).reshape(15, 15)         # (n c) x (m d)
    assert abs(float(top[0]) - torch.linalg.eigvalsh(dense)[-1].item()) < 1e-2 * abs(float(top[0]))


def test_counters_follow_their_formulas():
    model = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.ReLU(), nn.Flatten(), nn.Linear(8 * 6 * 6, 10))
    counters = [C.Forward(), C.KFACStats(), C.KFACInv(), C.ShampooStats()]
    with C.set_counter(model, counters, batch_size=4) as counts:
        model(torch.randn(1, 3, 6, 6))
    conv_macs = 4 * 36 * 8 * 27
    lin_macs = 4 * 10 * 288
    assert conv_macs + lin_macs <= counts['Forward']['flop'] <= 2 * (conv_macs + lin_macs) + 10 ** 4
    assert counts['KFACInv']['flop'] > 0 and counts['ShampooStats']['flop'] > 0
    assert counts['params'] == sum(p.numel() for p in model.parameters())
    assert C.roofline_ms(1e12, 1e9) == pytest.approx(max(1e12 / 1413.5e12, 1e9 / 6539.9e9) * 1e3)


def test_matrix_manager_accumulates_and_measures():
    model = _mlp()
    x, t = torch.randn(8, 6), torch.randint(0, 3, (8,))
    mm = asdl.MatrixManager(model, asdl.FISHER_EMP)
    for k in range(2):
        maker = asdl.get_fisher_maker(model, asdl.FisherConfig(fisher_type=asdl.FISHER_EMP,
                                                               fisher_shapes=[asdl.SHAPE_LAYER_WISE],
                                                               loss_type=asdl.LOSS_CROSS_ENTROPY, data_size=8,
                                                               fisher_attr=asdl.FISHER_EMP))
        d = maker.setup_model_call(model, x)
        maker.setup_loss_call(F.cross_entropy, d, t)
        maker.forward_and_backward()
        mm.accumulate_matrices('run')
    single = getattr(model[0], asdl.FISHER_EMP).data.clone()
    acc = mm.get_matrix(model[0], asdl.FISHER_EMP, 'run').data
    torch.testing.assert_close(acc, 2 * single, rtol=1e-5, atol=1e-7)
    trace = mm.get_trace(asdl.FISHER_EMP, asdl.SHAPE_LAYER_WISE, 'run')
    assert trace is not None


def test_gradient_utilities_against_autograd():
    model = _mlp()
    x, t = torch.randn(6, 6), torch.randint(0, 3, (6,))
    params = list(model.parameters())

    def per_example():
        rows = []
        for i in range(6):
            loss = F.cross_entropy(model(x[i:i + 1]), t[i:i + 1], reduction='sum')
            rows.append(torch.cat([g.flatten() for g in torch.autograd.grad(loss, params)]))
        return torch.stack(rows)
    oracle = per_example()

    def closure():
        loss = F.cross_entropy(model(x), t, reduction='sum')
        loss.backward()
        return loss
    model.zero_grad()
    grads = asdl.batch_gradient(model, closure)
    # per-example gradients are listed module by module (weight, then bias): the parameter order here
    torch.testing.assert_close(grads, oracle, rtol=1e-4, atol=1e-6)
    model.zero_grad()
    asdl.save_batch_gradient(model, closure)
    torch.testing.assert_close(model[0].weight.batch_grad.sum(0), model[0].weight.grad, rtol=1e-4, atol=1e-6)
    jac = asdl.jacobian(model, x)
    assert jac.shape == (6, 3, sum(p.numel() for p in params))
    out0 = model(x)[2, 1]
    g = torch.cat([v.flatten() for v in torch.autograd.grad(out0, params)])
    torch.testing.assert_close(jac[2, 1], g, rtol=1e-4, atol=1e-6)
    model.zero_grad()
    loader = DataLoader(TensorDataset(x, t), batch_size=2)
    mean_loss = asdl.data_loader_gradient(model, lambda y, tt: F.cross_entropy(y, tt, reduction='sum'), loader)
    ref_loss = F.cross_entropy(model(x), t)
    assert abs(mean_loss - ref_loss.item()) < 1e-5
    ref = torch.autograd.grad(ref_loss, params)
    for p, r in zip(params, ref):
        torch.testing.assert_close(p.grad, r, rtol=1e-4, atol=1e-6)


def test_phase_profile_times_library_and_user_ranges():
    from asdl_b200.utils import PhaseProfile, nvtx_range, time_funcs
    from asdl_b200.utils.profiling import active_profile
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 5), nn.ReLU(), nn.Linear(5, 3))
    x, t = torch.randn(8, 6), torch.randint(0, 3, (8,))
    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=0.5,
                                                                  preconditioner_upd_interval=2,
                                                                  curvature_upd_interval=1))

    def step():
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        gm.forward_and_backward()

    assert active_profile() is None
    with PhaseProfile(cuda=False) as prof:
        assert active_profile() is prof
        for _ in range(4):
            with nvtx_range('user_step'):
                step()
    assert active_profile() is None
    table = prof.table()
    assert table['user_step']['ncalls'] == 4 and table['update_curvature']['ncalls'] == 4
    assert table['update_preconditioner']['ncalls'] == 2          # every second step
    assert table['cov_kron_A']['ncalls'] == 8 and table['cov_kron_B']['ncalls'] == 8   # two layers, four steps
    assert table['user_step']['total_ms'] >= table['update_curvature']['total_ms'] > 0
    assert any(name.startswith('inv_kron') for name in table)
    assert 'user_step' in prof.report().splitlines()[1]            # sorted by total time: the enclosing range first
    with PhaseProfile(cuda=False, skip_first=3) as prof:
        for _ in range(4):
            with nvtx_range('user_step'):
                step()
    assert prof.table()['user_step']['ncalls'] == 1 and prof.reduce_max()['user_step']['ncalls'] == 1
    table = time_funcs([step, lambda: None], name='kfac_', func_names=['step', 'noop'], num_iters=3, num_warmups=1)
    assert table['kfac_step']['ncalls'] == 3 and table['kfac_Iter']['mean_ms'] >= table['kfac_step']['mean_ms']
    assert table['kfac_noop']['mean_ms'] < table['kfac_step']['mean_ms']


def test_preconditioned_ntk_is_jacobian_inverse_fisher_jacobian():
    """``get_preconditioned_kernel_fn``: J1 F^-1 J2^T with the K-FAC inverse of a gradient maker, for the
    direct, the implicit and the class-wise direct kernel."""
    from asdl_b200 import kernel as K
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 5), nn.Tanh(), nn.Linear(5, 3))
    x, t = torch.randn(4, 6), torch.randint(0, 3, (4,))
    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=4, damping=1e-2), fisher_type=asdl.FISHER_EMP)
    dummy = gm.setup_model_call(model, x)
    gm.setup_loss_call(F.cross_entropy, dummy, t)
    gm.forward_and_backward()
    model.zero_grad()
    params = list(model.parameters())
    y = model(x)
    jac, right = [], []
    for i in range(4):
        for c in range(3):
            grads = torch.autograd.grad(y[i, c], params, retain_graph=True)
            jac.append(torch.cat([g.flatten() for g in grads]))
            vec = asdl.ParamVector(params, [g.clone() for g in grads])
            gm.precondition(vectors=vec, grad_scale=1)
            right.append(vec.get_flatten_vector())
    jac, right = torch.stack(jac).view(4, 3, -1), torch.stack(right).view(4, 3, -1)
    want = torch.einsum('ncp,mdp->nmcd', jac, right)
    plain = torch.einsum('ncp,mdp->nmcd', jac, jac)
    for fn in (K.empirical_direct_ntk, K.empirical_implicit_ntk):
        torch.testing.assert_close(K.batch(fn, model, x, batch_size=2), plain, rtol=1e-4, atol=1e-5)
        got = K.batch(K.get_preconditioned_kernel_fn(fn, gm), model, x, batch_size=4)
        torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-4)
    class_wise = K.batch(K.get_preconditioned_kernel_fn(K.empirical_class_wise_direct_ntk, gm), model, x, batch_size=4)
    torch.testing.assert_close(class_wise, torch.einsum('ncp,mcp->nmc', jac, right), rtol=1e-3, atol=1e-4)
