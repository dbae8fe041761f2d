"""Failures are raised on the host with a usable message and leave the model as it was: exceptions
inside hooked passes, checkpoints that do not fit, damaged curvature files, misuse of the API."""
import copy
import os

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as asdl
from conftest import make_net, make_data


def _step(gm, model, x, t):
    dummy = gm.setup_model_call(model, x)
    gm.setup_loss_call(F.cross_entropy, dummy, t)
    return gm.forward_and_backward()


def _n_hooks(model):
    return sum(len(m._forward_hooks) + len(m._forward_pre_hooks) + len(m._backward_hooks) + len(m._backward_pre_hooks)
               for m in model.modules())


class _Boom(nn.Module):
    def forward(self, x):
        raise RuntimeError('boom')


@pytest.mark.parametrize('maker', [asdl.KfacGradientMaker, asdl.FusedKfacGradientMaker, asdl.DiagNaturalGradientMaker])
def test_exception_in_forward_removes_the_hooks(maker):
    model = nn.Sequential(nn.Linear(5, 4), _Boom())
    x, t = make_data('mlp', 8, 'cross_entropy')
    gm = maker(model, asdl.PreconditioningConfig(data_size=8, damping=1e-2))
    before = _n_hooks(model)
    with pytest.raises(RuntimeError, match='boom'):
        _step(gm, model, x, t)
    assert _n_hooks(model) == before
    model[1] = nn.Identity()   # the maker is usable again once the model is
    gm = maker(model, asdl.PreconditioningConfig(data_size=8, damping=1e-2))
    _, loss = _step(gm, model, x, t)
    assert torch.isfinite(loss)


def test_exception_in_loss_removes_the_hooks():
    model = make_net('mlp')
    x, t = make_data('mlp', 8, 'cross_entropy')
    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=8, damping=1e-2))

    def bad_loss(y, t, reduction="mean"):
        raise ValueError('bad loss')

    dummy = gm.setup_model_call(model, x)
    gm.setup_loss_call(bad_loss, dummy, t)
    with pytest.raises(ValueError, match='bad loss'):
        gm.forward_and_backward()
    assert _n_hooks(model) == 0


def test_checkpoint_of_another_architecture_is_refused_at_load():
    model = make_net('mlp')
    x, t = make_data('mlp', 8, 'cross_entropy')
    cfg = asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=0.3)
    gm = asdl.KfacGradientMaker(model, cfg)
    _step(gm, model, x, t)
    state = copy.deepcopy(gm.state_dict())
    key = next(k for k in state['curvature'] if k.endswith('kron.A'))
    state['curvature'][key] = torch.zeros(3, 3)
    fresh = asdl.KfacGradientMaker(make_net('mlp'), cfg)
    with pytest.raises(ValueError, match='curvature checkpoint entry'):
        fresh.load_state_dict(state)


def test_damaged_curvature_file_is_reported(tmp_path):
    model = make_net('mlp')
    x, t = make_data('mlp', 8, 'cross_entropy')
    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=0.3))
    _step(gm, model, x, t)
    fisher = model[0].fisher
    paths = fisher.save(str(tmp_path), 'layer0')
    a_file = os.path.join(str(tmp_path), paths['kron']['A_tril'])
    good = np.load(a_file)
    np.save(a_file, good[:-1])  # a lower triangle with one element missing is not a triangle of any n
    kron_paths = {k: os.path.join(str(tmp_path), v) for k, v in paths['kron'].items()}
    with pytest.raises(ValueError, match='packed triangle'):
        fisher.load(kron_path=kron_paths)
    with open(a_file, 'wb') as f:
        f.write(b'not an npy file')
    with pytest.raises(Exception):
        fisher.load(kron_path=kron_paths)
    np.save(a_file, good)
    fisher.load(kron_path=kron_paths)  # and the intact file loads again
    assert fisher.kron.A.shape == (5, 5)


def test_api_misuse_messages():
    model = make_net('mlp')
    x, t = make_data('mlp', 8, 'cross_entropy')
    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=8, damping=1e-2))
    with pytest.raises((ValueError, RuntimeError)):
        gm.forward_and_backward()  # nothing set up
    gm.setup_model_call(model, x)
    with pytest.raises((ValueError, RuntimeError)):
        gm.forward_and_backward()  # no loss set up
    with pytest.raises((ValueError, TypeError)):
        asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=8), fisher_type='no_such_type')
    with pytest.raises(ValueError):
        asdl.get_update_schedule(1.5, 0.0, 10)


def test_non_finite_factor_is_reported_not_inverted():
    """A factor with a NaN cannot be inverted; the maker says which step failed instead of
    writing NaNs into the gradients."""
    model = make_net('mlp')
    x, t = make_data('mlp', 8, 'cross_entropy')
    gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=0.3),
                                fisher_type=asdl.FISHER_EMP)
    x_bad = x.clone()
    x_bad[0, 0] = float('nan')
    with pytest.raises(Exception):
        _step(gm, model, x_bad, t)


def test_indefinite_factor_is_factorised_with_more_damping_and_a_warning():
    """Cholesky breakdown does not end the run: the damping is raised tenfold until the factor is
    positive definite, and the warning names the damping that was used."""
    torch.manual_seed(0)
    q = torch.linalg.qr(torch.randn(6, 6))[0]
    mat = (q * torch.tensor([2.0, 1.0, 0.5, 0.1, 0.0, -3e-4])) @ q.T          # one slightly negative eigenvalue
    mat = (mat + mat.T) / 2
    with pytest.warns(UserWarning, match='not positive definite with damping 1e-05'):
        inv = asdl.cholesky_inv(mat, 1e-5)
    assert torch.isfinite(inv).all()
    used = 1e-3                                                               # 1e-5 -> 1e-4 (still < 3e-4) -> 1e-3
    torch.testing.assert_close(inv, torch.linalg.inv(mat + used * torch.eye(6)), rtol=1e-3, atol=1e-3)
    with pytest.warns(UserWarning):
        y = asdl.cholesky_solve(mat, torch.ones(6), 1e-5)
    torch.testing.assert_close((mat + used * torch.eye(6)) @ y, torch.ones(6), rtol=1e-3, atol=1e-3)
    bad = mat.clone()
    bad[0, 0] = float('nan')
    with pytest.raises(torch.linalg.LinAlgError, match='non-finite'):
        asdl.cholesky_inv(bad, 1e-5)
    with pytest.raises(torch.linalg.LinAlgError, match='even with damping'):
        asdl.cholesky_inv(-1e6 * torch.eye(4), 1e-5)
    spd = q @ q.T + torch.eye(6)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter('error')
        asdl.cholesky_inv(spd, 1e-5)                                          # the normal case stays silent


def test_grouped_convolution_is_refused_with_advice():
    model = nn.Sequential(nn.Conv2d(4, 6, 3, groups=2), nn.Flatten(), nn.Linear(6 * 4 * 4, 3))
    x, t = torch.randn(4, 4, 6, 6), torch.randint(0, 3, (4,))
    cfg = asdl.PreconditioningConfig(data_size=4, damping=1e-2)
    with pytest.raises(ValueError, match='groups > 1'):
        asdl.FusedKfacGradientMaker(model, cfg)
    with pytest.raises(ValueError, match='groups > 1'):
        _step(asdl.KfacGradientMaker(model, cfg), model, x, t)
    ok = asdl.PreconditioningConfig(data_size=4, damping=1e-2, ignore_modules=[model[0]])
    for maker in (asdl.KfacGradientMaker, asdl.FusedKfacGradientMaker):   # the advice works
        _, loss = _step(maker(model, ok), model, x, t)
        assert torch.isfinite(loss) and model[0].weight.grad is not None


def test_fused_maker_refuses_float64_models():
    model = nn.Sequential(nn.Linear(5, 3)).double()
    with pytest.raises(ValueError, match='float64'):
        asdl.FusedKfacGradientMaker(model, asdl.PreconditioningConfig(data_size=4, damping=1e-2))
