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
