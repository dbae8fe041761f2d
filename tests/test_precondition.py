"""Preconditioned gradient makers: dense oracles for K-FAC and its relatives, behavioural checks
for Shampoo / PSGD / K-BFGS / SENG / SMW-NG / Newton / CurveBall, schedules and state dicts."""
import copy
import math

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as asdl
from asdl_b200.precondition.shampoo import (BlockPartitioner, ComputePower, Preconditioner,
                                            inverse_pth_root_batched, _merge_small_dims)
from conftest import make_net, make_data


def mlp_784():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(784, 512), nn.ReLU(), nn.Linear(512, 512), nn.ReLU(),
                         nn.Linear(512, 10))


def step(gm, model, x, t, loss_fn=F.cross_entropy, **kw):
    dummy = gm.setup_model_call(model, x)
    gm.setup_loss_call(loss_fn, dummy, t, **kw)
    return gm.forward_and_backward()


def capture_a_g(model, x, t):
    """Layer inputs a and output-gradients g of the SUM-reduced loss for every Linear."""
    with asdl.save_inputs_outgrads(model) as cxt:
        F.cross_entropy(model(x), t, reduction='sum').backward()
        out = {m: (cxt.in_data(m)[0], cxt.out_grads(m)[0]) for m in model if isinstance(m, nn.Linear)}
    model.zero_grad()
    return out


def test_kfac_matches_dense_oracle():
    """Preconditioned gradients equal (B + d_B I)^-1 grad (A + d_A I)^-1 with the pi-split damping
    on the flagship CPU configuration (MLP 784-512-512-10, batch 128, damping 0.01)."""
    model = mlp_784()
    x = torch.randn(128, 784)
    t = torch.randint(0, 10, (128,))
    damping, n = 0.01, 128
    acts = capture_a_g(model, x, t)
    F.cross_entropy(model(x), t).backward()
    raw = {m: (m.weight.grad.clone(), m.bias.grad.clone()) for m in acts}
    model.zero_grad()

    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=n, damping=damping),
                                fisher_type=asdl.FISHER_EMP)
    _, loss = step(gm, model, x, t)
    assert torch.isfinite(loss)
    for m, (a, g) in acts.items():
        A, B = a.T @ a / n, g.T @ g / n
        pi = math.sqrt((A.trace() / A.shape[0]) / (B.trace() / B.shape[0]))
        dA, dB = max(damping ** 0.5 * pi, 1e-7), max(damping ** 0.5 / pi, 1e-7)
        Ainv = torch.linalg.inv(A.double() + dA * torch.eye(A.shape[0], dtype=torch.double))
        Binv = torch.linalg.inv(B.double() + dB * torch.eye(B.shape[0], dtype=torch.double))
        gw, gb = raw[m]
        want_w = (Binv @ gw.double() @ Ainv).float()
        want_b = (Binv @ gb.double()).float()
        torch.testing.assert_close(m.weight.grad, want_w, rtol=2e-3, atol=1e-5)
        torch.testing.assert_close(m.bias.grad, want_b, rtol=2e-3, atol=1e-5)


def test_kfac_training_reduces_loss_and_ema_mode():
    model = mlp_784()
    x, t = torch.randn(128, 784), torch.randint(0, 10, (128,))
    cfg = asdl.PreconditioningConfig(data_size=128, damping=0.01, ema_decay=0.5,
                                     curvature_upd_interval=2, preconditioner_upd_interval=4)
    gm = asdl.KfacGradientMaker(model, cfg)
    opt = torch.optim.SGD(model.parameters(), lr=0.02)
    losses = []
    for _ in range(12):
        opt.zero_grad()
        _, loss = step(gm, model, x, t)
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0] * 0.5
    assert model[0].fisher.kron.A is not None and model[0].fisher.kron.A_inv is not None
    # EMA semantics: after a curvature step A = (1-e) A_old + e * a^T a / n
    sd = gm.state_dict()
    assert sd['step'] == 12 and any(k.endswith('kron.A') for k in sd['curvature'])


def test_kfac_cnn_with_batchnorm_unit_wise():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Conv2d(3, 8, 3, padding=1), nn.BatchNorm2d(8), nn.ReLU(),
                          nn.Conv2d(8, 8, 3, stride=2), nn.ReLU(), nn.Flatten(), nn.Linear(8 * 3 * 3, 5))
    x, t = torch.randn(16, 3, 8, 8), torch.randint(0, 5, (16,))
    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=16, damping=1e-2))
    _, loss = step(gm, model, x, t)
    assert model[1].fisher.unit.inv.shape == (8, 2, 2)
    assert model[0].fisher.kron.A_inv.shape == (27, 27)
    assert all(torch.isfinite(p.grad).all() for p in model.parameters())


@pytest.mark.parametrize('maker_cls,kwargs', [
    (asdl.FullNaturalGradientMaker, {}),
    (asdl.LayerWiseNaturalGradientMaker, {}),
    (asdl.UnitWiseNaturalGradientMaker, {}),
    (asdl.DiagNaturalGradientMaker, {}),
    (asdl.EkfacGradientMaker, {}),
    (asdl.KfacGradientMaker, {'swift': True}),
])
def test_natural_gradient_family_against_dense(maker_cls, kwargs):
    """With the exact empirical Fisher of the same shape, preconditioning is a dense solve."""
    kind, n, damping = 'mlp', 6, 1e-2
    model = make_net(kind)
    x, t = make_data(kind, n, 'cross_entropy')
    F.cross_entropy(model(x), t).backward()
    raw = torch.cat([p.grad.flatten() for p in model.parameters()])
    model.zero_grad()
    cfg = asdl.PreconditioningConfig(data_size=n, damping=damping)
    gm = maker_cls(model, cfg, fisher_type=asdl.FISHER_EMP, **kwargs)
    step(gm, model, x, t)
    got = torch.cat([p.grad.flatten() for p in model.parameters()])
    assert torch.isfinite(got).all()
    if maker_cls is asdl.FullNaturalGradientMaker:
        per = asdl.batch_gradient(model, lambda: F.cross_entropy(model(x), t, reduction='sum').backward())
        Fm = per.T @ per / n
        want = torch.linalg.solve(Fm + damping * torch.eye(Fm.shape[0]), raw)
        torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-5)
    elif maker_cls is asdl.DiagNaturalGradientMaker:
        per = asdl.batch_gradient(model, lambda: F.cross_entropy(model(x), t, reduction='sum').backward())
        d = (per ** 2).sum(0) / n
        torch.testing.assert_close(got, raw / (d + damping), rtol=1e-3, atol=1e-6)
    else:
        # preconditioning with an SPD matrix keeps a positive inner product with the gradient
        assert torch.dot(got, raw) > 0


def test_schedules():
    cfg = asdl.PreconditioningConfig(preconditioner_upd_interval=5, preconditioner_warmup_steps=3,
                                     curvature_upd_interval=2)
    gm = asdl.KfacGradientMaker(make_net('mlp'), cfg)
    prec = [gm.do_update_preconditioner(s) for s in range(12)]
    assert prec == [True, True, True, True, False, False, False, False, True, False, False, False]
    curv = [gm.do_update_curvature(s) for s in range(6)]
    assert curv == [True, False, True, False, True, False]
    sched = asdl.get_update_schedule(20, update_ratio=0.5, warmup_ratio=0.1)
    assert len(sched) == 20 and sum(sched) == 10 and sched[:2] == [True, True]
    assert sum(asdl.get_update_schedule(20, 0.5, 0.1, asdl.INTERVAL_STEP)) == 10
    lin = asdl.get_update_schedule(100, 0.1, 0.0, asdl.INTERVAL_LINEAR)
    assert len(lin) == 100 and sum(lin) == 10
    with pytest.raises(ValueError):
        asdl.get_update_schedule(10, update_ratio=0.1, warmup_ratio=0.5)
    gm2 = asdl.KfacGradientMaker(make_net('mlp'), asdl.PreconditioningConfig(
        num_total_steps=10, preconditioner_upd_ratio=0.5, ema_decay=0.1, curvature_upd_ratio=1.0))
    assert sum(gm2.do_update_preconditioner(s) for s in range(10)) == 5


def test_state_dict_roundtrip_and_reference_format():
    model = make_net('mlp')
    x, t = make_data('mlp', 8, 'cross_entropy')
    cfg = asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=0.5)
    gm = asdl.KfacGradientMaker(model, cfg)
    for _ in range(3):
        step(gm, model, x, t)
    sd = copy.deepcopy(gm.state_dict())
    model2 = make_net('mlp')
    model2.load_state_dict(model.state_dict())
    gm2 = asdl.KfacGradientMaker(model2, cfg)
    gm2.load_state_dict(sd)
    assert gm2.state['step'] == 3
    for m1, m2 in zip(model, model2):
        if isinstance(m1, nn.Linear):
            torch.testing.assert_close(m1.fisher.kron.A, m2.fisher.kron.A)
            torch.testing.assert_close(m1.fisher.kron.B_inv, m2.fisher.kron.B_inv)
    gm2.load_state_dict({'step': 7})  # the reference's state dict has only the step
    assert gm2.state['step'] == 7


def test_block_partitioner_and_merge_dims():
    bp = BlockPartitioner((5, 7), 3)
    t = torch.arange(35.).view(5, 7)
    parts = bp.partition(t)
    assert len(parts) == 2 * 3 and [tuple(p.shape) for p in parts][:3] == [(3, 3), (3, 3), (3, 1)]
    torch.testing.assert_close(bp.merge_partitions(parts), t)
    assert [s[0] for s in bp.kronecker_factor_shapes()][:4] == [3, 3, 3, 3]
    assert _merge_small_dims([1, 2, 512, 1, 2048, 1, 3, 4], 1024) == [1024, 2048, 12]


@pytest.mark.parametrize('p', [2, 4, 8])
def test_inverse_pth_root(p):
    torch.manual_seed(0)
    mats = []
    for n in (6, 6, 6):
        a = torch.randn(n, n, dtype=torch.float64)
        mats.append(a @ a.T + 0.1 * torch.eye(n, dtype=torch.float64))
    stack = torch.stack(mats)
    roots = inverse_pth_root_batched(stack, p, ridge_epsilon=1e-8, error_tolerance=1e-10)
    for m, r in zip(mats, roots):
        w, v = torch.linalg.eigh(m + 1e-8 * torch.linalg.eigvalsh(m).max() * torch.eye(6, dtype=torch.float64))
        want = (v * w.pow(-1.0 / p)) @ v.T
        torch.testing.assert_close(r, want, rtol=1e-5, atol=1e-7)
    single = ComputePower(mats[0], p, ridge_epsilon=1e-8, error_tolerance=1e-10)
    torch.testing.assert_close(single, roots[0], rtol=1e-6, atol=1e-8)


def test_shampoo_blocked_equals_reference_math():
    torch.manual_seed(0)
    lin = nn.Linear(6, 5, bias=False)
    lin.weight.grad = torch.randn(5, 6)
    cfg = asdl.PreconditioningConfig(damping=1e-6)
    prec = Preconditioner(lin.weight, cfg, block_size=3)
    g = lin.weight.grad.clone()
    prec.update_statistics()
    prec.update_preconditioners()
    prec.precondition()
    out = torch.empty_like(g)
    for rs in (slice(0, 3), slice(3, 5)):
        for cs in (slice(0, 3), slice(3, 6)):
            blk = g[rs, cs]
            L = blk @ blk.T + 1e-12 * torch.eye(blk.shape[0])
            R = blk.T @ blk + 1e-12 * torch.eye(blk.shape[1])
            out[rs, cs] = ComputePower(L, 4) @ blk @ ComputePower(R, 4)
    torch.testing.assert_close(lin.weight.grad, out, rtol=1e-4, atol=1e-5)


MAKERS = {
    'shampoo': lambda m: asdl.ShampooGradientMaker(m, asdl.PreconditioningConfig(damping=1e-6), block_size=4),
    'kron_psgd': lambda m: asdl.KronPsgdGradientMaker(m, asdl.PreconditioningConfig()),
    'psgd': lambda m: asdl.PsgdGradientMaker(m, asdl.PreconditioningConfig()),
    'psgd_func': lambda m: asdl.KronPsgdGradientMaker(m, asdl.PreconditioningConfig(), use_functorch=True),
    'kbfgs': lambda m: asdl.KronBfgsGradientMaker(m, asdl.PreconditioningConfig(
        data_size=8, damping=1e-2, ema_decay=0.1)),
    'kbfgs_mb': lambda m: asdl.KronBfgsGradientMaker(m, asdl.PreconditioningConfig(
        data_size=8, damping=1e-2, ema_decay=0.1), minibatch_hessian_action=True),
    'seng': lambda m: asdl.SengGradientMaker(m, asdl.PreconditioningConfig(data_size=8, damping=1e-1),
                                             sketching_size=3, truncated_rank=2),
    'curve_ball': lambda m: asdl.CurveBallGradientMaker(m, asdl.PreconditioningConfig(damping=1e-2),
                                                        momentum=0.1),
}


@pytest.mark.parametrize('name', sorted(MAKERS))
@pytest.mark.parametrize('kind', ['mlp', 'cnn'])
def test_makers_train(name, kind):
    model = make_net(kind)
    x, t = make_data(kind, 8, 'cross_entropy')
    gm = MAKERS[name](model)
    lr = {'seng': 0.01, 'curve_ball': 1.0, 'shampoo': 0.02}.get(name, 0.05)
    opt = torch.optim.SGD(model.parameters(), lr=lr)
    first = F.cross_entropy(model(x), t).item()
    for _ in range(25):
        opt.zero_grad()
        _, loss = step(gm, model, x, t)
        assert torch.isfinite(loss)
        opt.step()
    last = F.cross_entropy(model(x), t).item()
    assert last < first, (name, first, last)


CHECKPOINTED = dict(MAKERS)
CHECKPOINTED.update({
    'kfac_ema': lambda m: asdl.KfacGradientMaker(m, asdl.PreconditioningConfig(
        data_size=8, damping=1e-2, ema_decay=0.3), fisher_type=asdl.FISHER_EMP),
    'kfac_fused': lambda m: asdl.FusedKfacGradientMaker(m, asdl.PreconditioningConfig(
        data_size=8, damping=1e-2, ema_decay=0.3), fisher_type=asdl.FISHER_EMP),
    'ekfac': lambda m: asdl.EkfacGradientMaker(m, asdl.PreconditioningConfig(data_size=8, damping=1e-2)),
    'diag': lambda m: asdl.DiagNaturalGradientMaker(m, asdl.PreconditioningConfig(
        data_size=8, damping=1e-2, ema_decay=0.3), fisher_type=asdl.FISHER_EMP),
})


@pytest.mark.parametrize('name', sorted(CHECKPOINTED))
@pytest.mark.parametrize('kind', ['mlp', 'cnn'])
def test_resume_from_state_dict_continues_the_run(name, kind):
    """A fresh model and maker that load the weights and ``state_dict()`` of a run produce the gradients
    the interrupted run would have produced at its next step.  K-BFGS is the exception: its open
    (s, y) pair needs the previous batch, which no checkpoint holds, so the pair is dropped."""
    torch.manual_seed(1)
    model = make_net(kind)
    x, t = make_data(kind, 8, 'cross_entropy')
    gm = CHECKPOINTED[name](model)
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    for _ in range(3):
        opt.zero_grad()
        step(gm, model, x, t)
        opt.step()
    state, weights = copy.deepcopy(gm.state_dict()), copy.deepcopy(model.state_dict())
    rng = torch.get_rng_state()
    opt.zero_grad()
    step(gm, model, x, t)
    want = [p.grad.clone() for p in model.parameters()]

    model2 = make_net(kind)
    model2.load_state_dict(weights)
    gm2 = CHECKPOINTED[name](model2)
    gm2.load_state_dict(state)
    assert gm2.state['step'] == 3
    torch.set_rng_state(rng)
    step(gm2, model2, x, t)
    for p, w in zip(model2.parameters(), want):
        assert torch.isfinite(p.grad).all()
        if not name.startswith('kbfgs'):
            torch.testing.assert_close(p.grad, w)


def test_smw_natural_gradient_matches_dense():
    model = make_net('mlp')
    n, damping = 6, 1e-2
    x, t = make_data('mlp', n, 'cross_entropy')
    per = asdl.batch_gradient(model, lambda: F.cross_entropy(model(x), t, reduction='sum').backward())
    model.zero_grad()
    Fm = per.T @ per / n
    g = per.mean(0)
    want = torch.linalg.solve(Fm + damping * torch.eye(Fm.shape[0]), g)
    gm = asdl.SmwEmpNaturalGradientMaker(model, asdl.SmwEmpNaturalGradientConfig(data_size=n, damping=damping))
    step(gm, model, x, t)
    got = torch.cat([p.grad.flatten() for p in model.parameters()])
    torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize('absolute', [False, True])
def test_newton(absolute):
    model = make_net('mlp')
    x, t = make_data('mlp', 8, 'cross_entropy')
    gm = asdl.NewtonGradientMaker(model, asdl.NewtonGradientConfig(damping=1e-1, absolute=absolute))
    step(gm, model, x, t)
    H = model.hessian.data
    params = list(model.parameters())
    g = torch.cat([v.flatten() for v in torch.autograd.grad(F.cross_entropy(model(x), t), params)])
    if absolute:
        w, v = torch.linalg.eigh(H)
        H = (v * w.abs()) @ v.T
    want = torch.linalg.solve(H + 1e-1 * torch.eye(H.shape[0]), g)
    got = torch.cat([p.grad.flatten() for p in params])
    torch.testing.assert_close(got, want, rtol=1e-3, atol=1e-5)


def test_hessian_shapes_and_tools():
    model = make_net('mlp')
    x, t = make_data('mlp', 8, 'cross_entropy')
    hm = asdl.HessianMaker(model, asdl.HessianConfig(hessian_shapes=[asdl.SHAPE_FULL, asdl.SHAPE_LAYER_WISE,
                                                                     asdl.SHAPE_DIAG]))
    d = hm.setup_model_call(model, x)
    hm.setup_loss_call(F.cross_entropy, d, t)
    hm.forward_and_backward()
    H = model.hessian.data
    torch.testing.assert_close(H, H.T, rtol=1e-5, atol=1e-6)
    ref = torch.autograd.functional.hessian(
        lambda *ps: F.cross_entropy(torch.func.functional_call(model, dict(zip([k for k, _ in model.named_parameters()], ps)), (x,)), t),
        tuple(model.parameters()))
    n0 = model[0].weight.numel()
    torch.testing.assert_close(H[:n0, :n0], ref[0][0].reshape(n0, n0), rtol=1e-4, atol=1e-6)
    blk = model[0].hessian.data
    nb = n0 + model[0].bias.numel()
    torch.testing.assert_close(blk, H[:nb, :nb])
    torch.testing.assert_close(model[0].hessian.diag.weight.flatten(), torch.diag(H)[:n0])
    params = list(model.parameters())
    v = asdl.ParamVector(params, [torch.randn_like(p) for p in params])
    hm.forward_and_backward(hvp=True, vec=v)
    torch.testing.assert_close(model.hvp.get_flatten_vector(), H @ v.get_flatten_vector(), rtol=1e-4, atol=1e-6)
    eig, _ = hm.hessian_eig(top_n=1, max_iters=300, tol=1e-9)
    top = torch.linalg.eigvalsh(H).abs().max().item()
    assert abs(abs(eig[0]) - top) / top < 1e-2


def test_psgd_sparse_lu_fits_a_quadratic():
    """P = Q^T Q with arrow-shaped LU factors: P g equals the dense product, and fitting on
    (dx, H dx) pairs of a fixed SPD Hessian drives P H towards the identity on the criterion
    E[dg^T P dg + dx^T P^-1 dx]."""
    from asdl_b200.precondition.psgd import update_precond_splu, precond_grad_splu
    torch.manual_seed(0)
    n, r = 12, 4
    L12 = torch.cat([torch.eye(r), torch.zeros(n - r, r)]).double()
    U12 = torch.cat([torch.eye(r), torch.zeros(r, n - r)], dim=1).double()
    l3, u3 = torch.ones(n - r, 1).double(), torch.ones(n - r, 1).double()
    a = torch.randn(n, n).double()
    H = a @ a.T / n + 0.5 * torch.eye(n).double()

    def dense_P(L12, l3, U12, u3):
        L = torch.zeros(n, n).double()
        L[:, :r] = L12
        L[r:, r:] = torch.diag(l3.reshape(-1))
        U = torch.zeros(n, n).double()
        U[:r] = U12
        U[r:, r:] = torch.diag(u3.reshape(-1))
        Q = L @ U
        return Q.T @ Q

    def criterion(P):
        return (torch.trace(P @ H @ H) + torch.trace(torch.linalg.inv(P))).item()

    start = criterion(dense_P(L12, l3, U12, u3))
    for _ in range(400):
        dx = torch.randn(n).double()
        L12, l3, U12, u3 = update_precond_splu(L12, l3, U12, u3, [dx[:5].reshape(5, 1), dx[5:]],
                                               [(H @ dx)[:5].reshape(5, 1), (H @ dx)[5:]], step=0.05)
    P = dense_P(L12, l3, U12, u3)
    assert criterion(P) < 0.8 * start
    g = [torch.randn(3, 2).double(), torch.randn(6).double()]
    out = precond_grad_splu(L12, l3, U12, u3, g)
    flat = P @ torch.cat([t.reshape(-1) for t in g])
    torch.testing.assert_close(torch.cat([t.reshape(-1) for t in out]), flat)
    assert out[0].shape == (3, 2) and out[1].shape == (6,)


def test_seng_state_roundtrip():
    """The sketched curvature of SENG travels through state_dict: a fresh maker that loads it
    preconditions a given gradient exactly like the original."""
    import copy
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 5), nn.ReLU(), nn.Linear(5, 3))
    x, t = torch.randn(8, 6), torch.randint(0, 3, (8,))
    cfg = asdl.PreconditioningConfig(data_size=8, damping=1e-2, curvature_upd_interval=100)
    gm = asdl.SengGradientMaker(model, cfg, sketching_size=4)
    d = gm.setup_model_call(model, x)
    gm.setup_loss_call(F.cross_entropy, d, t)
    gm.forward_and_backward()
    state = copy.deepcopy(gm.state_dict())
    assert any(k.endswith('seng.gram_inv') for k in state['curvature'])
    fresh = asdl.SengGradientMaker(model, cfg, sketching_size=4)
    fresh.load_state_dict(state)
    grads = [torch.randn_like(p) for p in model.parameters()]
    results = []
    for maker in (gm, fresh):
        for p, g in zip(model.parameters(), grads):
            p.grad = g.clone()
        maker.precondition()
        results.append([p.grad.clone() for p in model.parameters()])
    for a, b in zip(*results):
        torch.testing.assert_close(a, b)


@pytest.mark.parametrize('ema,fisher_type,steps,kwargs', [
    (-1, asdl.FISHER_EMP, 1, {}), (1.0, asdl.FISHER_EMP, 1, {}), (0.3, asdl.FISHER_EMP, 3, {}),
    (-1, asdl.FISHER_MC, 1, {'n_mc_samples': 2}), (0.3, asdl.FISHER_MC, 3, {'n_mc_samples': 2}),
    (-1, asdl.FISHER_EXACT, 1, {})])
def test_swift_kfac_equals_kfac(ema, fisher_type, steps, kwargs):
    """With fewer samples than features the swift factors are the raw n x d matrices and the inverse
    is taken by Woodbury: exact, so the preconditioned gradients equal those of ordinary K-FAC in
    every mode (inverse in the hooks, moving average, several backward passes per step)."""
    def run(swift):
        torch.manual_seed(0)
        model = nn.Sequential(nn.Linear(12, 9), nn.Tanh(), nn.Linear(9, 3))
        x, t = torch.randn(4, 12), torch.randint(0, 3, (4,))
        cfg = asdl.PreconditioningConfig(data_size=4, damping=1e-2, ema_decay=ema)
        gm = asdl.KfacGradientMaker(model, cfg, fisher_type=fisher_type, swift=swift, **kwargs)
        opt = torch.optim.SGD(model.parameters(), lr=0.05)
        for s in range(steps):
            opt.zero_grad()
            torch.manual_seed(100 + s)           # the same sampled labels in both runs
            step(gm, model, x, t)
            grads = torch.cat([p.grad.flatten() for p in model.parameters()])
            opt.step()
        if swift and ema == -1:
            assert model[0].fisher.kron.A_inv.shape == (12, 12)
        return grads

    torch.testing.assert_close(run(True), run(False), rtol=1e-4, atol=1e-6)


def test_members_of_the_explicit_partition_interface():
    model = make_net('mlp')
    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=8, damping=1e-2))
    linears = [m for m in model.modules() if isinstance(m, nn.Linear)]
    assert gm.computational_cost(asdl.SHAPE_KRON, linears[0]) > 0
    assert gm.next_split([1, 1, 1, 1]) == 2 and gm.next_split([10, 1, 1]) == 1 and gm.next_split([1, 1, 10]) == 2
    with pytest.raises(ValueError):
        gm.next_split([1])
    with pytest.raises(ValueError, match='module_partitions'):
        gm.reduce_scatter_curvature_module_partitions()
    with pytest.raises(ValueError, match='module_partitions'):
        gm.reduce_curvature('0')
    gm.all_reduce_no_curvature_grad()       # no process group: nothing to do
    shampoo = asdl.ShampooGradientMaker(model, asdl.PreconditioningConfig(damping=1e-6))
    assert shampoo.computational_cost([[4, 4], [2, 2]]) == 72 and shampoo.next_split([3, 1, 1, 1]) == 1


AUTOCAST_MAKERS = {
    'kfac': lambda m: asdl.KfacGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-2, ema_decay=0.3),
                                             fisher_type=asdl.FISHER_EMP),
    'kfac_mc_inv_in_hooks': lambda m: asdl.KfacGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-2), seed=1),
    'kfac_fused': lambda m: asdl.FusedKfacGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-2, ema_decay=0.3),
                                                        fisher_type=asdl.FISHER_EMP),
    'ekfac': lambda m: asdl.EkfacGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-2)),
    'unit_wise': lambda m: asdl.UnitWiseNaturalGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-2),
                                                             fisher_type=asdl.FISHER_EMP),
    'diag': lambda m: asdl.DiagNaturalGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-2),
                                                    fisher_type=asdl.FISHER_EMP),
    'layer_wise': lambda m: asdl.LayerWiseNaturalGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-2),
                                                               fisher_type=asdl.FISHER_EMP),
    'shampoo': lambda m: asdl.ShampooGradientMaker(m, asdl.PreconditioningConfig(damping=1e-4)),
    'kron_psgd': lambda m: asdl.KronPsgdGradientMaker(m, asdl.PreconditioningConfig()),
    'kbfgs': lambda m: asdl.KronBfgsGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-2, ema_decay=0.1)),
    'seng': lambda m: asdl.SengGradientMaker(m, asdl.PreconditioningConfig(data_size=16, damping=1e-1)),
    'smw': lambda m: asdl.SmwEmpNaturalGradientMaker(m, asdl.SmwEmpNaturalGradientConfig(data_size=16, damping=1e-2)),
}


@pytest.mark.parametrize('name', sorted(AUTOCAST_MAKERS))
def test_makers_under_bf16_autocast(name):
    """The model may run under bf16 autocast: hooks see bf16 activations and run inside the autocast
    region, statistics and factors stay fp32, and the result stays close to the fp32 run."""
    def run(bf16):
        torch.manual_seed(0)
        norm_layers = name not in ('kbfgs', 'seng', 'kron_psgd')     # those makers handle Linear / Conv2d only
        layers = ([nn.Conv2d(2, 4, 3, padding=1)] + ([nn.BatchNorm2d(4)] if norm_layers else [])
                  + [nn.Tanh(), nn.Flatten(), nn.Linear(4 * 36, 8)] + ([nn.LayerNorm(8)] if norm_layers else [])
                  + [nn.Linear(8, 3)])
        model = nn.Sequential(*layers)
        x, t = torch.randn(16, 2, 6, 6), torch.randint(0, 3, (16,))
        gm = AUTOCAST_MAKERS[name](model)

        def model_fn(inp):
            with torch.autocast('cpu', dtype=torch.bfloat16, enabled=bf16):
                return model(inp)

        for _ in range(2):
            model.zero_grad()
            dummy = gm.setup_model_call(model_fn, x)
            gm.setup_loss_call(F.cross_entropy, dummy, t)
            gm.forward_and_backward()
        assert all(p.grad.dtype == torch.float32 for p in model.parameters())
        return torch.cat([p.grad.flatten() for p in model.parameters()])

    full, mixed = run(False), run(True)
    assert torch.isfinite(mixed).all()
    assert F.cosine_similarity(full, mixed, dim=0) > 0.98


@pytest.mark.parametrize('maker', [asdl.KfacGradientMaker, asdl.FusedKfacGradientMaker])
@pytest.mark.parametrize('stop', [1, 2, 4, 5])
def test_resume_at_any_point_of_the_update_schedule(maker, stop):
    """Curvature every 2nd and inverses every 3rd step: a run resumed after ``stop`` steps continues with
    the gradients of the uninterrupted run."""
    def make(model):
        cfg = asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=0.3, curvature_upd_interval=2,
                                         preconditioner_upd_interval=3)
        return maker(model, cfg, fisher_type=asdl.FISHER_EMP)

    def one_step(gm, model, opt):
        opt.zero_grad()
        step(gm, model, x, t)
        grads = torch.cat([p.grad.flatten() for p in model.parameters()]).clone()
        opt.step()
        return grads

    torch.manual_seed(1)
    model = make_net('cnn')
    x, t = make_data('cnn', 8, 'cross_entropy')
    gm, opt = make(model), torch.optim.SGD(model.parameters(), lr=0.01)
    for _ in range(stop):
        one_step(gm, model, opt)
    state, weights = copy.deepcopy(gm.state_dict()), copy.deepcopy(model.state_dict())
    want = [one_step(gm, model, opt) for _ in range(3)]
    resumed = make_net('cnn')
    resumed.load_state_dict(weights)
    gm2, opt2 = make(resumed), torch.optim.SGD(resumed.parameters(), lr=0.01)
    gm2.load_state_dict(state)
    for w in want:
        torch.testing.assert_close(one_step(gm2, resumed, opt2), w, rtol=1e-5, atol=1e-7)
