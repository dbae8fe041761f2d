"""The persistent-buffer K-FAC path reproduces the generic maker step for step."""
import copy

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as asdl


def small_cnn():
    torch.manual_seed(0)
    return nn.Sequential(nn.Conv2d(3, 8, 3, padding=1, bias=False), nn.BatchNorm2d(8), nn.ReLU(),
                         nn.Conv2d(8, 16, 1, bias=False), nn.BatchNorm2d(16), nn.ReLU(),
                         nn.Conv2d(16, 8, 3, stride=2, padding=1), nn.ReLU(),
                         nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(8, 5))


def run(maker_cls, model, steps, cfg, x, t, **kw):
    gm = maker_cls(model, cfg, fisher_type=asdl.FISHER_EMP, **kw)
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    out = []
    for _ in range(steps):
        opt.zero_grad()
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        _, loss = gm.forward_and_backward()
        out.append((loss.item(), [p.grad.clone() for p in model.parameters()]))
        opt.step()
    return gm, out


@pytest.mark.parametrize('ema', [-1, 0.3])
@pytest.mark.parametrize('channels_last', [False, True])
def test_fused_equals_generic(ema, channels_last):
    x, t = torch.randn(6, 3, 8, 8), torch.randint(0, 5, (6,))
    cfg = asdl.PreconditioningConfig(data_size=6, damping=1e-2, ema_decay=ema,
                                     curvature_upd_interval=2 if ema > 0 else None,
                                     preconditioner_upd_interval=2)
    base = small_cnn()
    m1, m2 = copy.deepcopy(base), copy.deepcopy(base)
    if channels_last:
        m2 = m2.to(memory_format=torch.channels_last)
    _, ref = run(asdl.KfacGradientMaker, m1, 5, cfg, x, t)
    x2 = x.contiguous(memory_format=torch.channels_last) if channels_last else x
    gm, got = run(asdl.FusedKfacGradientMaker, m2, 5, cfg, x2, t)
    for (l1, g1), (l2, g2) in zip(ref, got):
        assert abs(l1 - l2) < 1e-4 * max(1, abs(l1))
        for a, b in zip(g1, g2):
            torch.testing.assert_close(b, a, rtol=2e-3, atol=2e-5)
    sd = gm.state_dict()
    assert any(k.endswith('kron.A_inv') for k in sd['curvature'])
    m3 = copy.deepcopy(base)
    gm3 = asdl.FusedKfacGradientMaker(m3, cfg, fisher_type=asdl.FISHER_EMP)
    gm3.load_state_dict(copy.deepcopy(sd))
    torch.testing.assert_close(m3[0].fisher.kron.A, m2[0].fisher.kron.A)


def test_fused_mc_fisher_trains():
    model = small_cnn()
    x, t = torch.randn(16, 3, 8, 8), torch.randint(0, 5, (16,))
    cfg = asdl.PreconditioningConfig(data_size=16, damping=1e-2, ema_decay=0.5,
                                     curvature_upd_interval=2, preconditioner_upd_interval=4)
    gm = asdl.FusedKfacGradientMaker(model, cfg, seed=1)
    opt = torch.optim.SGD(model.parameters(), lr=0.02)
    losses = []
    for _ in range(20):
        opt.zero_grad()
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        _, loss = gm.forward_and_backward()
        opt.step()
        losses.append(loss.item())
    assert losses[-1] < losses[0]


@pytest.mark.parametrize('loss', ['cross_entropy', 'mse'])
@pytest.mark.parametrize('options', [
    {'fisher_type': 'fisher_mc'}, {'fisher_type': 'fisher_exact'}, {'fisher_type': 'fisher_mc', 'n_mc_samples': 3},
    {'fisher_type': 'fisher_mc', 'var': 0.5}, {'fisher_type': 'fisher_exact', 'ema': 0.3},
    {'fisher_type': 'fisher_mc', 'scale': 2.0}, {'fisher_type': 'fisher_emp', 'grad_scale': 0.5},
    {'fisher_type': 'fisher_mc', 'seed': 3}], ids=lambda o: '-'.join(f'{k}={v}' for k, v in o.items()))
def test_fused_follows_the_generic_maker_for_every_fisher_type_and_option(options, loss):
    """Sampled labels / Gaussian targets, several samples per step (statistics of the passes add up),
    one pass per class or output for the exact Fisher, scales and seeds."""
    import torch.nn as nn
    import torch.nn.functional as F

    def run(maker_cls):
        kw = dict(options)
        torch.manual_seed(0)
        model = nn.Sequential(nn.Conv2d(2, 3, 3, padding=1), nn.BatchNorm2d(3), nn.Tanh(), nn.Flatten(), nn.Linear(108, 3))
        x = torch.randn(8, 2, 6, 6)
        t = torch.randn(8, 3) if loss == 'mse' else torch.randint(0, 3, (8,))
        cfg = asdl.PreconditioningConfig(data_size=8, damping=1e-2, ema_decay=kw.pop('ema', -1))
        gm = maker_cls(model, cfg, loss_type=loss, **kw)
        opt = torch.optim.SGD(model.parameters(), lr=0.01)
        grads = []
        for s in range(3):
            opt.zero_grad()
            torch.manual_seed(9 + s)
            dummy = gm.setup_model_call(model, x)
            gm.setup_loss_call(F.mse_loss if loss == 'mse' else F.cross_entropy, dummy, t)
            gm.forward_and_backward()
            grads.append(torch.cat([p.grad.flatten() for p in model.parameters()]).clone())
            opt.step()
        return grads

    for want, got in zip(run(asdl.KfacGradientMaker), run(asdl.FusedKfacGradientMaker)):
        assert ((want - got).norm() / want.norm()).item() < 1e-4


def test_capture_key_covers_what_a_graph_bakes_in():
    """The key that decides whether captured steps may be replayed changes with every value that a
    capture reads once: damping, the moving-average weight, the data size, the training mode and
    non-tensor arguments of the registered calls."""
    import torch.nn as nn
    import asdl_b200 as asdl
    model = nn.Sequential(nn.Linear(4, 3))
    cfg = asdl.PreconditioningConfig(data_size=4, damping=1e-2, ema_decay=0.1)
    gm = asdl.FusedKfacGradientMaker(model, cfg)
    x = torch.randn(4, 4)
    gm.setup_model_call(model, x)
    gm.setup_loss_call(lambda y, scale=1.0: y.sum() * scale, gm._model_output if False else x, scale=2.0)
    key0 = gm._capture_key(gm._tensor_slots())
    assert key0 == gm._capture_key(gm._tensor_slots())
    cfg.damping = 1e-1
    key1 = gm._capture_key(gm._tensor_slots())
    assert key1 != key0 and key1[0] == key0[0]          # same layouts, different captured values
    cfg.damping = 1e-2
    cfg.ema_decay = 0.2
    assert gm._capture_key(gm._tensor_slots()) != key0
    cfg.ema_decay = 0.1
    model.eval()
    assert gm._capture_key(gm._tensor_slots()) != key0
    model.train()
    gm.setup_loss_call(lambda y, scale=1.0: y.sum() * scale, x, scale=3.0)
    assert gm._capture_key(gm._tensor_slots()) != key0
