"""Every operation name against a plain-autograd value: what the hook-time handlers store for
Linear and Conv2d layers, under which key, and that the post-hoc calculators (from saved inputs
and output gradients) agree with the hook-time ones."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as asdl
from asdl_b200.operations import (OP_COV_KRON, OP_COV_SWIFT_KRON, OP_COV_KFE, OP_COV, OP_CVP, OP_COV_UNIT_WISE,
                                  OP_COV_DIAG, OP_GRAM_HADAMARD, OP_GRAM_DIRECT, OP_BATCH_GRADS, OP_MEAN_INPUTS,
                                  OP_MEAN_OUTPUTS, OP_SPATIAL_MEAN_OUTPUTS, OP_OUT_SPATIAL_SIZE, OP_MEAN_OUTGRADS,
                                  OP_SPATIAL_MEAN_OUTGRADS, OP_SAVE_INPUTS, OP_SAVE_OUTGRADS, OP_RFIM_RELU,
                                  OP_RFIM_SOFTMAX)


def _linear_net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(5, 4), nn.Tanh(), nn.Linear(4, 3))


def _conv_net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Conv2d(2, 3, 3, padding=1), nn.Tanh(), nn.Conv2d(3, 4, 2, stride=2), nn.Flatten(),
                         nn.Linear(4 * 3 * 3, 3))


def _data(kind, n=6):
    g = torch.Generator().manual_seed(1)
    x = torch.randn(n, 5, generator=g) if kind == 'linear' else torch.randn(n, 2, 6, 6, generator=g)
    return x, torch.randint(0, 3, (n,), generator=g)


def _per_example_grads(model, layer, x, t):
    """n x (weight.numel + bias.numel), weight first, by one backward pass per example."""
    rows = []
    for i in range(x.shape[0]):
        model.zero_grad()
        F.cross_entropy(model(x[i:i + 1]), t[i:i + 1], reduction='sum').backward()
        rows.append(torch.cat([layer.weight.grad.flatten(), layer.bias.grad.flatten()]))
    model.zero_grad()
    return torch.stack(rows)


def _run(model, x, t, *ops, read, **kw):
    """``read(cxt)`` evaluated inside the hooked pass (results are released when the context closes)."""
    with asdl.extend(model, *ops, **kw) as cxt:
        F.cross_entropy(model(x), t, reduction='sum').backward()
        out = read(cxt)
    model.zero_grad()
    return out


@pytest.mark.parametrize('kind', ['linear', 'conv'])
def test_per_example_gradient_family(kind):
    """batch_grads, cov, cov_diag, cov_unit_wise, cvp and gram_direct are all functions of the
    per-example gradients of the layer."""
    model = _linear_net() if kind == 'linear' else _conv_net()
    layer = model[0]
    x, t = _data(kind)
    bg = _per_example_grads(model, layer, x, t)
    nw = layer.weight.numel()
    vec = asdl.ParamVector(list(model.parameters()), [torch.randn_like(p) for p in model.parameters()])
    got, cov, diag, unit, cvp = _run(
        model, x, t, OP_BATCH_GRADS, OP_COV, OP_COV_DIAG, OP_COV_UNIT_WISE, OP_CVP, vectors=vec,
        read=lambda c: (dict(c.batch_grads(layer)), c.cov(layer)['data'], dict(c.cov_diag(layer)),
                        c.cov_unit_wise(layer)['data'], dict(c.cvp(layer))))
    torch.testing.assert_close(torch.cat([got['weight'].flatten(1), got['bias'].flatten(1)], dim=1), bg)
    torch.testing.assert_close(cov, bg.T @ bg, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(torch.cat([diag['weight'].flatten(), diag['bias'].flatten()]), bg.square().sum(0),
                               rtol=1e-4, atol=1e-6)
    f_out = layer.weight.shape[0]
    rows = torch.cat([bg[:, :nw].reshape(-1, f_out, nw // f_out), bg[:, nw:].unsqueeze(-1)], dim=2)
    torch.testing.assert_close(unit, torch.einsum('nfi,nfj->fij', rows, rows), rtol=1e-4, atol=1e-6)
    flat_v = torch.cat([vec.get_vector_by_param(p).flatten() for p in layer.parameters()])
    torch.testing.assert_close(torch.cat([cvp['weight'].flatten(), cvp['bias'].flatten()]), bg.T @ (bg @ flat_v),
                               rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize('kind', ['linear', 'conv'])
def test_gram_ops_equal_the_gram_of_per_example_gradients(kind):
    model = _linear_net() if kind == 'linear' else _conv_net()
    x, t = _data(kind)
    layers = [m for m in model if isinstance(m, (nn.Linear, nn.Conv2d))]
    bg = torch.cat([_per_example_grads(model, layer, x, t) for layer in layers], dim=1)
    want = bg @ bg.T
    n = x.shape[0]
    for op in (OP_GRAM_DIRECT,) + ((OP_GRAM_HADAMARD,) if kind == 'linear' else ()):
        with asdl.extend(model, op):
            model.kernel = torch.zeros(n, n)
            F.cross_entropy(model(x), t, reduction='sum').backward()
        torch.testing.assert_close(model.kernel, want, rtol=1e-4, atol=1e-5)
        model.zero_grad()


@pytest.mark.parametrize('kind', ['linear', 'conv'])
def test_kron_swift_and_kfe(kind):
    model = _linear_net() if kind == 'linear' else _conv_net()
    layer = model[0]
    x, t = _data(kind, n=3)                                        # fewer samples than input features: swift keeps a raw
    with asdl.save_inputs_outgrads(model) as saved:
        F.cross_entropy(model(x), t, reduction='sum').backward()
        a_raw, g_raw = saved.in_data(layer)[0], saved.out_grads(layer)[0]
    model.zero_grad()
    if kind == 'linear':
        a, g, positions = a_raw, g_raw, 1
    else:
        a = asdl.im2col_2d(a_raw, layer).transpose(1, 2).reshape(-1, 2 * 3 * 3)   # (n * positions) x (c kh kw)
        positions = g_raw.shape[-1] * g_raw.shape[-2] if g_raw.ndim == 4 else g_raw.shape[-1]
        g = g_raw.reshape(3, 3, -1).transpose(1, 2).reshape(-1, 3)
    kron = _run(model, x, t, OP_COV_KRON, read=lambda c: dict(c.cov_kron(layer)))
    torch.testing.assert_close(kron['A'], a.T @ a / positions, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(kron['B'], g.T @ g, rtol=1e-4, atol=1e-6)
    swift = _run(model, x, t, OP_COV_SWIFT_KRON, read=lambda c: dict(c.cov_kron(layer)))
    if kind == 'linear':                                           # 3 samples < 5 features: the raw 3 x 5 matrix
        assert swift['A'].shape == (3, 5)
        from asdl_b200.symmatrix import swift_gram                 # the raw factor x stands for x^T x / n
        torch.testing.assert_close(swift_gram(swift['A']), a.T @ a, rtol=1e-4, atol=1e-6)
        assert swift['B'].shape == (3, 4) or swift['B'].shape == (4, 4)
    kfe = _run(model, x, t, OP_COV_KFE, read=lambda c: dict(c.get_result(layer, OP_COV_KFE)))
    Ua, Ub = kfe['A'], kfe['B']
    torch.testing.assert_close(Ua.T @ Ua, torch.eye(Ua.shape[1]), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(Ub.T @ Ub, torch.eye(Ub.shape[1]), rtol=1e-4, atol=1e-5)
    assert bool((kfe['scale'][0] >= 0).all())


def test_means_and_sizes():
    model = _conv_net()
    conv, x, t = model[0], *_data('conv')
    r = _run(model, x, t, OP_MEAN_INPUTS, OP_MEAN_OUTPUTS, OP_SPATIAL_MEAN_OUTPUTS, OP_OUT_SPATIAL_SIZE,
             OP_MEAN_OUTGRADS, OP_SPATIAL_MEAN_OUTGRADS, OP_SAVE_INPUTS, OP_SAVE_OUTGRADS,
             read=lambda c: dict(size=c.out_spatial_size(conv), sm_out=c.spatial_mean_out_data(conv),
                                 m_out=c.mean_out_data(conv), g=c.out_grads(conv)[0], a=c.in_data(conv)[0],
                                 sm_g=c.spatial_mean_out_grads(conv), m_in=c.mean_in_data(conv)))
    y = conv(x)
    assert r['size'] == 36
    torch.testing.assert_close(r['sm_out'], y.mean(dim=(2, 3)))
    torch.testing.assert_close(r['m_out'].flatten(), y.mean(dim=(0, 2, 3)), rtol=1e-4, atol=1e-6)
    assert r['g'].shape[0] == 6 and r['a'].shape == x.shape
    torch.testing.assert_close(r['sm_g'], r['g'].reshape(6, 3, -1).mean(dim=2), rtol=1e-4, atol=1e-7)
    patches = asdl.im2col_2d(x, conv)                               # n x (c kh kw) x positions
    torch.testing.assert_close(r['m_in'].flatten(), patches.mean(dim=(0, 2)), rtol=1e-4, atol=1e-6)


def test_relative_fisher_ops_are_linear_only():
    model = _linear_net()
    x, t = _data('linear')
    relu, softmax = _run(model, x, t, OP_RFIM_RELU, OP_RFIM_SOFTMAX,
                         read=lambda c: (c.rfim_relu(model[0]), c.rfim_softmax(model[2])))
    assert relu is not None and softmax is not None
    assert OP_RFIM_RELU not in asdl.Conv2d.supported_operations and OP_RFIM_RELU in asdl.Linear.supported_operations


@pytest.mark.parametrize('kind', ['linear', 'conv'])
@pytest.mark.parametrize('shape', [asdl.SHAPE_LAYER_WISE, asdl.SHAPE_KRON, asdl.SHAPE_UNIT_WISE, asdl.SHAPE_DIAG])
def test_post_hoc_calculators_agree_with_hooks(kind, shape):
    """calc_cov from saved inputs / output gradients == the statistics computed inside the hooks."""
    model = _linear_net() if kind == 'linear' else _conv_net()
    layer = model[0]
    x, t = _data(kind)
    op = {asdl.SHAPE_LAYER_WISE: OP_COV, asdl.SHAPE_KRON: OP_COV_KRON, asdl.SHAPE_UNIT_WISE: OP_COV_UNIT_WISE,
          asdl.SHAPE_DIAG: OP_COV_DIAG}[shape]
    hooked = _run(model, x, t, op, read=lambda c: c.cov_symmatrix(layer))
    with asdl.save_inputs_outgrads(model) as cxt:
        F.cross_entropy(model(x), t, reduction='sum').backward()
        cxt.calc_cov(layer, shape)
        post = cxt.cov_symmatrix(layer)
    for key, value in hooked.tensors().items():
        torch.testing.assert_close(post.tensors()[key], value, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize('mode', ['zeros', 'reflect', 'replicate', 'circular'])
def test_convolution_statistics_honour_the_padding_mode(mode):
    """Patches are taken from the input padded the way the layer pads it (the reference pads with
    zeros whatever the mode: asdl/utils.py:51-70)."""
    torch.manual_seed(0)
    conv = nn.Conv2d(2, 3, 3, padding=1, padding_mode=mode)
    model = nn.Sequential(conv, nn.Flatten(), nn.Linear(3 * 36, 3))
    x, t = torch.randn(4, 2, 6, 6), torch.randint(0, 3, (4,))
    want = _per_example_grads(model, conv, x, t)
    got = _run(model, x, t, OP_BATCH_GRADS, read=lambda c: dict(c.batch_grads(conv)))
    torch.testing.assert_close(torch.cat([got['weight'].flatten(1), got['bias'].flatten(1)], dim=1), want)
    torch.testing.assert_close(asdl.im2col_2d(x, conv), asdl.im2col_2d_slow(x, conv))


@pytest.mark.parametrize('kernel', [3, (2, 4)])
def test_convolution_with_same_padding(kernel):
    torch.manual_seed(0)
    conv = nn.Conv2d(2, 3, kernel, padding='same')
    model = nn.Sequential(conv, nn.Flatten(), nn.Linear(3 * 36, 3))
    x, t = torch.randn(4, 2, 6, 6), torch.randint(0, 3, (4,))
    want = _per_example_grads(model, conv, x, t)
    got = _run(model, x, t, OP_BATCH_GRADS, read=lambda c: dict(c.batch_grads(conv)))
    torch.testing.assert_close(torch.cat([got['weight'].flatten(1), got['bias'].flatten(1)], dim=1), want)
    for maker in (asdl.KfacGradientMaker, asdl.FusedKfacGradientMaker):
        gm = maker(model, asdl.PreconditioningConfig(data_size=4, damping=1e-2), fisher_type=asdl.FISHER_EMP)
        dummy = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, dummy, t)
        gm.forward_and_backward()
        assert torch.isfinite(conv.weight.grad).all()
