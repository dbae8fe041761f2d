"""Differential check against the reference package where it is installed beside the repository
(``baseline/_ref``; skipped otherwise): the same model, data and seeds go through both libraries'
gradient makers for three optimizer steps and the preconditioned gradients are compared."""
import os
import sys
import warnings

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as ours

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), 'baseline', '_ref')


@pytest.fixture(scope='module')
def reference():
    if not os.path.isdir(os.path.join(REF_DIR, 'asdl')):
        pytest.skip('reference package not installed under baseline/_ref')
    sys.path.insert(0, REF_DIR)
    try:
        import asdl
    except Exception as exc:  # an environment without the reference's imports
        pytest.skip(f'reference package not importable: {exc}')
    finally:
        sys.path.remove(REF_DIR)
    return asdl


def _net(kind):
    torch.manual_seed(0)
    if kind == 'mlp':
        return nn.Sequential(nn.Linear(6, 5), nn.Tanh(), nn.Linear(5, 3)), torch.randn(8, 6), torch.randint(0, 3, (8,))
    if kind == 'batchnorm':
        model = nn.Sequential(nn.Conv2d(2, 4, 3, padding=1), nn.BatchNorm2d(4), nn.ReLU(), nn.Flatten(),
                              nn.Linear(4 * 36, 6), nn.BatchNorm1d(6), nn.ReLU(), nn.Linear(6, 3))
        return model, torch.randn(8, 2, 6, 6), torch.randint(0, 3, (8,))
    if kind == 'layernorm_sequence':     # n x sequence x features, some positions ignored by the loss
        model = nn.Sequential(nn.Linear(6, 5), nn.LayerNorm(5), nn.Tanh(), nn.Linear(5, 3))
        t = torch.randint(0, 3, (4, 7))
        t[0, :3] = -1
        return model, torch.randn(4, 7, 6), t
    if kind == 'embedding':
        return (nn.Sequential(nn.Embedding(11, 4), nn.Flatten(), nn.Linear(12, 3)), torch.randint(0, 11, (8, 3)),
                torch.randint(0, 3, (8,)))
    model = nn.Sequential(nn.Conv2d(2, 3, 3, padding=1), nn.Tanh(), nn.Conv2d(3, 4, 2, stride=2), nn.Flatten(),
                          nn.Linear(36, 3))
    return model, torch.randn(8, 2, 6, 6), torch.randint(0, 3, (8,))


def _run(lib, make, kind, steps=3):
    model, x, t = _net(kind)
    gm = make(lib, model)
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    out = []
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        for s in range(steps):
            opt.zero_grad()
            torch.manual_seed(50 + s)      # sampled labels and random probes agree between the libraries
            dummy = gm.setup_model_call(model, x)
            if t.ndim == 2:
                gm.setup_loss_call(F.cross_entropy, dummy.view(-1, 3), t.view(-1), ignore_index=-1)
            else:
                gm.setup_loss_call(F.cross_entropy, dummy, t)
            gm.forward_and_backward()
            out.append(torch.cat([p.grad.flatten() for p in model.parameters()]).clone())
            opt.step()
    return out


def _cfg(lib, **kw):
    return lib.PreconditioningConfig(**kw)


#: name -> (constructor, relative tolerance, steps compared)
CASES = {
    'kfac_emp': (lambda L, m: L.KfacGradientMaker(m, _cfg(L, data_size=8, damping=1e-2), fisher_type='fisher_emp'), 1e-4, 3),
    'kfac_mc': (lambda L, m: L.KfacGradientMaker(m, _cfg(L, data_size=8, damping=1e-2)), 1e-4, 3),
    'kfac_ema': (lambda L, m: L.KfacGradientMaker(m, _cfg(L, data_size=8, damping=1e-2, ema_decay=0.3),
                                                  fisher_type='fisher_emp'), 1e-4, 3),
    'diag': (lambda L, m: L.DiagNaturalGradientMaker(m, _cfg(L, data_size=8, damping=1e-2), fisher_type='fisher_emp'), 1e-5, 3),
    'full': (lambda L, m: L.FullNaturalGradientMaker(m, _cfg(L, data_size=8, damping=1e-2), fisher_type='fisher_emp'), 1e-4, 3),
    # inverse roots come from different iterations (batched here), probes pass through different triangular solves
    'shampoo': (lambda L, m: L.ShampooGradientMaker(m, _cfg(L, damping=1e-6)), 1e-2, 3),
    'kron_psgd': (lambda L, m: L.KronPsgdGradientMaker(m, _cfg(L)), 5e-3, 3),
    'psgd': (lambda L, m: L.PsgdGradientMaker(m, _cfg(L)), 1e-5, 3),
    # the first K-BFGS step is plain; afterwards this library updates the stored inverse, the reference a temporary
    'kbfgs': (lambda L, m: L.KronBfgsGradientMaker(m, _cfg(L, data_size=8, damping=1e-2, ema_decay=0.1)), 1e-6, 1),
    'seng': (lambda L, m: L.SengGradientMaker(m, _cfg(L, data_size=8, damping=1e-1), sketching_size=256,
                                              truncated_rank=16), 1e-5, 3),
    'smw': (lambda L, m: L.SmwEmpNaturalGradientMaker(m, L.SmwEmpNaturalGradientConfig(data_size=8, damping=1e-2)), 1e-5, 3),
    'newton': (lambda L, m: L.NewtonGradientMaker(m, L.NewtonGradientConfig(damping=1e-1)), 1e-4, 3),
}


@pytest.mark.parametrize('kind', ['mlp', 'cnn'])
@pytest.mark.parametrize('name', sorted(CASES))
def test_same_gradients_as_the_reference(reference, name, kind):
    make, rtol, steps = CASES[name]
    want = _run(reference, make, kind)
    got = _run(ours, make, kind)
    for w, g in list(zip(want, got))[:steps]:
        assert ((w - g).norm() / w.norm()).item() < rtol


@pytest.mark.parametrize('kind', ['batchnorm', 'layernorm_sequence', 'embedding'])
@pytest.mark.parametrize('name', ['kfac_emp', 'kfac_mc', 'kfac_ema', 'diag', 'seng'])
def test_same_gradients_on_norm_layers_sequences_and_embeddings(reference, name, kind):
    if kind == 'embedding' and name in ('kfac_emp', 'kfac_mc'):
        pytest.skip('the reference raises on embeddings without a moving average')
    make, rtol, steps = CASES[name]
    for w, g in zip(_run(reference, make, kind), _run(ours, make, kind)):
        assert ((w - g).norm() / w.norm()).item() < rtol


def test_unit_wise_on_a_linear_network(reference):
    """(The reference's unit-wise maker fails on convolutions: it concatenates a 4-D and a 2-D tensor.)"""
    def make(L, m):
        return L.UnitWiseNaturalGradientMaker(m, _cfg(L, data_size=8, damping=1e-2), fisher_type='fisher_emp')
    for w, g in zip(_run(reference, make, 'mlp'), _run(ours, make, 'mlp')):
        assert ((w - g).norm() / w.norm()).item() < 1e-5
    assert all(torch.isfinite(g).all() for g in _run(ours, make, 'cnn'))


def _mlp():
    return _net('mlp')


def _fisher_maker(L, **kw):
    model, x, t = _mlp()
    fm = L.get_fisher_maker(model, L.FisherConfig(fisher_type='fisher_emp', fisher_shapes=['full'],
                                                  loss_type='cross_entropy', data_size=8, **kw))
    dummy = fm.setup_model_call(model, x)
    fm.setup_loss_call(F.cross_entropy, dummy, t)
    return model, fm


def _ones(L, model):
    return L.ParamVector(list(model.parameters()), [torch.ones_like(p) for p in model.parameters()])


def _fisher_eig(L):
    _, fm = _fisher_maker(L)
    fm.forward_and_backward()
    return torch.tensor([float(v) for v in fm.fisher_eig(top_n=2, max_iters=300, tol=1e-9)[0]])


def _fisher_free(L):
    model, fm = _fisher_maker(L)
    return fm.fisher_free(_ones(L, model), damping=1e-2, max_iters=200, tol=1e-10).get_flatten_vector()


def _fisher_quadratic_form(L):
    model, fm = _fisher_maker(L)
    return torch.tensor(float(fm.fisher_quadratic_form(_ones(L, model))))


def _hessian(shape):
    def run(L):
        model, x, t = _mlp()
        hm = L.HessianMaker(model, L.HessianConfig(hessian_shapes=[shape]))
        dummy = hm.setup_model_call(model, x)
        hm.setup_loss_call(F.cross_entropy, dummy, t)
        hm.forward_and_backward()
        if shape == 'full':
            return model.hessian.data
        return model[0].hessian.data if shape == 'layer_wise' else model[0].hessian.diag.weight
    return run


def _hessian_eig(L):
    model, x, t = _mlp()
    hm = L.HessianMaker(model, L.HessianConfig(hessian_shapes=['full']))
    dummy = hm.setup_model_call(model, x)
    hm.setup_loss_call(F.cross_entropy, dummy, t)
    return torch.tensor([float(v) for v in hm.hessian_eig(top_n=1, max_iters=500, tol=1e-10)[0]])


def _ntk(name):
    def run(L):
        model, x, _ = _mlp()
        return getattr(L, name)(model, x)
    return run


def _gradient_after(call):
    def run(L):
        model, x, t = _mlp()
        call(L, model, x, t)
        return torch.cat([p.grad.flatten() for p in model.parameters()])
    return run


ANALYSES = {
    'fisher_eig': _fisher_eig, 'fisher_free': _fisher_free, 'fisher_quadratic_form': _fisher_quadratic_form,
    'hessian_full': _hessian('full'), 'hessian_layer_wise': _hessian('layer_wise'), 'hessian_diag': _hessian('diag'),
    'hessian_eig': _hessian_eig,
    'ntk_implicit': _ntk('empirical_implicit_ntk'), 'ntk_class_wise_direct': _ntk('empirical_class_wise_direct_ntk'),
    'ntk_class_wise_hadamard': _ntk('empirical_class_wise_hadamard_ntk'),
    'kernel_free': _gradient_after(lambda L, m, x, t: L.kernel_free_cross_entropy(m, x, t, damping=1e-2, tol=1e-9)),
    'kernel_eigenvalues': lambda L: torch.tensor([float(v) for v in L.kernel_eigenvalues(
        _mlp()[0], _mlp()[1], top_n=2, max_iters=500, tol=1e-10)]),
    'empirical_natural_gradient': _gradient_after(lambda L, m, x, t: L.empirical_natural_gradient(m, x, t, damping=1e-2)),
}


@pytest.mark.parametrize('name', sorted(ANALYSES))
def test_same_analysis_results_as_the_reference(reference, name):
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        torch.manual_seed(3)
        want = torch.as_tensor(ANALYSES[name](reference)).double().flatten()
        torch.manual_seed(3)
        got = torch.as_tensor(ANALYSES[name](ours)).double().flatten()
    assert ((want - got).norm() / want.norm()).item() < 1e-5


def _fisher_tensors(model):
    out = {}
    for name, module in model.named_modules():
        fisher = getattr(module, 'fisher', None)
        if fisher is None:
            continue
        parts = {'': fisher, 'kron.': getattr(fisher, 'kron', None), 'unit.': getattr(fisher, 'unit', None),
                 'diag.': getattr(fisher, 'diag', None)}
        for prefix, part in parts.items():
            if part is None:
                continue
            for attr in ('data', 'inv', 'A', 'B', 'A_inv', 'B_inv', 'weight', 'bias', 'weight_inv', 'bias_inv'):
                value = getattr(part, attr, None)
                if isinstance(value, torch.Tensor):
                    out[f'{name}.{prefix}{attr}'] = value
    return out


def _fisher_net(kind):
    torch.manual_seed(0)
    if kind == 'mlp':
        return nn.Sequential(nn.Linear(6, 5), nn.Tanh(), nn.Linear(5, 3)), torch.randn(8, 6)
    if kind == 'cnn_bn':
        return (nn.Sequential(nn.Conv2d(2, 3, 3, padding=1), nn.BatchNorm2d(3), nn.Tanh(), nn.Flatten(), nn.Linear(108, 3)),
                torch.randn(8, 2, 6, 6))
    # token-level model: every layer sees (examples x tokens) rows
    return nn.Sequential(nn.Embedding(11, 4), nn.LayerNorm(4), nn.Linear(4, 3)), torch.randint(0, 11, (8, 3))


@pytest.mark.parametrize('kind', ['mlp', 'cnn_bn', 'embedding_ln'])
@pytest.mark.parametrize('fisher_type', ['fisher_exact', 'fisher_mc', 'fisher_emp'])
@pytest.mark.parametrize('loss', ['cross_entropy', 'mse'])
def test_same_fisher_tensors_as_the_reference(reference, kind, fisher_type, loss):
    """Every shape, with and without the fused inverse: the same tensors under the same names."""
    shapes = ['full', 'layer_wise', 'kron', 'unit_wise', 'diag']
    if kind == 'embedding_ln' and fisher_type == 'fisher_exact':
        pytest.skip('on n x tokens x classes outputs the reference raises (cross-entropy) or loops over the wrong '
                    'dimension (MSE); tests/test_fisher.py checks this library against J^T J there')
    if kind == 'embedding_ln':
        shapes = ['full', 'layer_wise', 'diag']   # no unit-wise blocks for embeddings, no Kronecker factors for LayerNorm
    for shape in shapes:
        for calc_inv in (False, True):
            results = []
            for lib in (reference, ours):
                model, x = _fisher_net(kind)
                rows = 24 if kind == 'embedding_ln' else 8
                t = torch.randint(0, 3, (rows,)) if loss == 'cross_entropy' else torch.randn(rows, 3)
                fm = lib.get_fisher_maker(model, lib.FisherConfig(fisher_type=fisher_type, fisher_shapes=[shape],
                                                                  loss_type=loss, data_size=8, seed=1, n_mc_samples=2))
                dummy = fm.setup_model_call(model, x)
                fm.setup_loss_call(F.cross_entropy if loss == 'cross_entropy' else F.mse_loss,
                                   dummy.view(-1, 3) if kind == 'embedding_ln' else dummy, t)
                with warnings.catch_warnings():
                    warnings.simplefilter('ignore')
                    fm.forward_and_backward(calc_inv=calc_inv, damping=1e-2)
                results.append(_fisher_tensors(model))
            want, got = results
            assert set(want) == set(got), (shape, calc_inv, sorted(set(want) ^ set(got)))
            for key in want:
                assert ((want[key] - got[key]).norm() / (want[key].norm() + 1e-30)).item() < 1e-4, (shape, calc_inv, key)


def _conv_net():
    torch.manual_seed(0)
    return (nn.Sequential(nn.Conv2d(2, 3, 3, padding=1), nn.Tanh(), nn.Flatten(), nn.Linear(108, 3)), torch.randn(8, 2, 6, 6),
            torch.randint(0, 3, (8,)))


def _leaves(value):
    if isinstance(value, torch.Tensor):
        return [value.double().flatten()]
    if isinstance(value, dict):
        value = list(value.values())
    if isinstance(value, (list, tuple)):
        return [leaf for v in value for leaf in _leaves(v)]
    return [torch.as_tensor(value).double().flatten()]


def _counters(L):
    model, x, _ = _conv_net()
    flat = torch.randn(8, 108)
    out = []
    for cls in ('Forward', 'BackwardWeight', 'BackwardInput', 'AdamStats', 'AdamPrecond', 'KFACStats', 'KFACInv',
                'KFACPrecond', 'ShampooStats', 'ShampooInv', 'ShampooPrecond', 'SMWNGStats'):
        counter = getattr(L, cls)()
        for module, inputs in ((model[0], x), (model[3], flat)):
            out += list(counter.count_flop_numel(module, inputs, module(inputs), batch_size=8))
    return [float(v) for v in out]


def _loader_gradient(L):
    model, x, t = _conv_net()
    loader = torch.utils.data.DataLoader(torch.utils.data.TensorDataset(x, t), batch_size=4)
    loss = L.data_loader_gradient(model, lambda y, tt: F.cross_entropy(y, tt, reduction='sum'), loader)
    return [loss] + [p.grad for p in model.parameters()]


def _functional(name):
    def run(L):
        model, x, t = _conv_net()
        gm = L.GradientMaker(model)
        dummy = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, dummy, t)
        return getattr(gm, name)()
    return run


def _esd(L):
    model, x, t = _conv_net()
    fm = L.get_fisher_maker(model, L.FisherConfig(fisher_type='fisher_emp', fisher_shapes=['full'],
                                                  loss_type='cross_entropy', data_size=8))
    dummy = fm.setup_model_call(model, x)
    fm.setup_loss_call(F.cross_entropy, dummy, t)
    return list(fm.fisher_esd(n_v=2, num_iter=10)[:2])


def _schedules(L):
    out = []
    for ratio, warmup in ((0.1, 0.0), (0.5, 0.0), (0.5, 0.2), (1.0, 0.2)):
        for kind in ('constant', 'step', 'linear'):
            out += [float(v) for v in L.get_update_schedule(num_total_steps=50, update_ratio=ratio, warmup_ratio=warmup,
                                                            interval_type=kind)]
    return out


UTILITIES = {
    'schedules': _schedules, 'counters': _counters, 'data_loader_gradient': _loader_gradient, 'fisher_esd': _esd,
    'batch_gradient': lambda L: _batch_gradient(L),
    'loss_grad': _functional('loss_grad'), 'per_example_loss_grads': _functional('per_example_loss_grads'),
    'loss_hessian': _functional('loss_hessian'), 'logit_jacobian': _functional('logit_jacobian'),
}


def _batch_gradient(L):
    model, x, t = _conv_net()
    return L.batch_gradient(model, lambda: F.cross_entropy(model(x), t, reduction='sum').backward())


@pytest.mark.parametrize('name', sorted(UTILITIES))
def test_same_utility_results_as_the_reference(reference, name):
    with warnings.catch_warnings():
        warnings.simplefilter('ignore')
        torch.manual_seed(3)
        want = torch.cat(_leaves(UTILITIES[name](reference)))
        torch.manual_seed(3)
        got = torch.cat(_leaves(UTILITIES[name](ours)))
    assert want.shape == got.shape
    assert ((want - got).norm() / (want.norm() + 1e-30)).item() < 1e-4


def test_curvature_files_interchange_with_the_reference(reference, tmp_path):
    """Lower-triangle ``.npy`` files written by either library load in the other."""
    for writer, reader in ((reference, ours), (ours, reference)):
        model, x, t = _conv_net()
        fm = writer.get_fisher_maker(model, writer.FisherConfig(fisher_type='fisher_emp', fisher_shapes=['kron', 'diag'],
                                                                loss_type='cross_entropy', data_size=8))
        dummy = fm.setup_model_call(model, x)
        fm.setup_loss_call(F.cross_entropy, dummy, t)
        fm.forward_and_backward()
        root = str(tmp_path / writer.__name__)
        paths = model[0].fisher.save(root, 'conv')
        assert paths['kron']['A_tril'].replace(os.sep, '/') == 'conv/kron/A_tril.npy'
        assert paths['diag']['weight'].replace(os.sep, '/') == 'conv/diag/weight.npy'
        loaded = reader.SymMatrix()
        loaded.load(kron_path={k: os.path.join(root, v) for k, v in paths['kron'].items()},
                    diag_path={k: os.path.join(root, v) for k, v in paths['diag'].items()})
        torch.testing.assert_close(loaded.kron.A, model[0].fisher.kron.A)
        torch.testing.assert_close(loaded.kron.B, model[0].fisher.kron.B)
        torch.testing.assert_close(loaded.diag.weight, model[0].fisher.diag.weight)


class _LossInside(nn.Module):
    """Returns logits, or ``(logits, loss)`` / ``{'loss', 'logits'}`` when given targets."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.body = nn.Sequential(nn.Linear(6, 5), nn.BatchNorm1d(5), nn.ReLU(), nn.Linear(5, 3))

    def forward(self, x, t=None, as_dict=False):
        y = self.body(x)
        if t is None:
            return y
        loss = F.cross_entropy(y, t)
        return {'loss': loss, 'logits': y} if as_dict else (y, loss)


SCHEDULED = {
    'intervals_and_warmup': lambda L, m: L.KfacGradientMaker(m, _cfg(
        L, data_size=8, damping=1e-2, ema_decay=0.2, curvature_upd_interval=2, preconditioner_upd_interval=3,
        preconditioner_warmup_steps=2), fisher_type='fisher_emp'),
    'ratios': lambda L, m: L.KfacGradientMaker(m, _cfg(
        L, data_size=8, damping=1e-2, ema_decay=0.2, num_total_steps=6, preconditioner_upd_ratio=0.5,
        curvature_upd_ratio=0.5), fisher_type='fisher_emp'),
    'ignore_class': lambda L, m: L.KfacGradientMaker(m, _cfg(L, data_size=8, damping=1e-2, ignore_modules=[nn.BatchNorm1d]),
                                                     fisher_type='fisher_emp'),
    'ignore_name': lambda L, m: L.KfacGradientMaker(m, _cfg(L, data_size=8, damping=1e-2, ignore_modules=['body.0']),
                                                    fisher_type='fisher_emp'),
    'sampled_labels': lambda L, m: L.KfacGradientMaker(m, _cfg(L, data_size=8, damping=1e-2)),
}


@pytest.mark.parametrize('convention', ['tensor', 'tuple', 'dict'])
@pytest.mark.parametrize('name', sorted(SCHEDULED))
def test_same_gradients_for_every_output_convention_and_schedule(reference, name, convention):
    runs = []
    for lib in (reference, ours):
        model = _LossInside()
        torch.manual_seed(1)
        x, t = torch.randn(8, 6), torch.randint(0, 3, (8,))
        gm = SCHEDULED[name](lib, model)
        opt = torch.optim.SGD(model.parameters(), lr=0.05)
        grads = []
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            for s in range(6):
                opt.zero_grad()
                torch.manual_seed(20 + s)
                if convention == 'tuple':
                    dummy = gm.setup_model_call(model, x, t)
                    gm.setup_logits_repr(dummy[0])
                    gm.setup_loss_repr(dummy[1])
                elif convention == 'dict':
                    dummy = gm.setup_model_call(model, x, t, as_dict=True)
                    gm.setup_logits_repr(dummy['logits'])
                    gm.setup_loss_repr(dummy['loss'])
                else:
                    dummy = gm.setup_model_call(model, x)
                    gm.setup_loss_call(F.cross_entropy, dummy, t)
                gm.forward_and_backward()
                grads.append(torch.cat([p.grad.flatten() for p in model.parameters()]).clone())
                opt.step()
        runs.append(grads)
    for want, got in zip(*runs):
        assert ((want - got).norm() / want.norm()).item() < 1e-4


def _plain_norm_layers(module):
    """The library's normalisation subclasses replaced by their parents (the reference matches layer
    types exactly and refuses subclasses); same parameters and buffers."""
    for name, child in list(module.named_children()):
        kind = type(child).__name__
        if kind == 'FusedLayerNorm':
            new = nn.LayerNorm(child.normalized_shape, eps=child.eps)
        elif kind == 'FusedBatchNorm2d':
            assert child.act is None
            new = nn.BatchNorm2d(child.num_features, eps=child.eps, momentum=child.momentum)
        else:
            _plain_norm_layers(child)
            continue
        new.load_state_dict(child.state_dict())
        setattr(module, name, new)
    return module


def _family(kind, plain):
    from asdl_b200 import models
    torch.manual_seed(0)
    images, labels = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    if kind == 'gpt2':
        model = models.gpt2_tiny()
        tokens = torch.randint(0, 97, (4, 16))
        images, labels = tokens, tokens
    else:
        model = {'resnet_bottleneck': models.resnet_tiny, 'resnet18': lambda: models.resnet18(width=8),
                 'wideresnet': models.wideresnet_tiny, 'vit': models.vit_tiny, 'mixer': models.mixer_tiny}[kind]()
    return (_plain_norm_layers(model) if plain else model), images, labels


@pytest.mark.parametrize('kind', ['resnet_bottleneck', 'resnet18', 'wideresnet', 'vit', 'mixer', 'gpt2'])
@pytest.mark.parametrize('fisher_type,ema', [('fisher_emp', 0.3), ('fisher_mc', -1)])
def test_model_families_generic_and_fused_kfac(reference, kind, fisher_type, ema):
    """Two K-FAC steps on the tiny version of every model family: the reference's maker, this library's
    generic maker and its fused maker give the same gradients."""
    def run(lib, maker_name, plain):
        model, x, t = _family(kind, plain)
        ignore = [nn.Embedding] if kind == 'gpt2' else None
        gm = getattr(lib, maker_name)(model, _cfg(lib, data_size=4, damping=1e-2, ema_decay=ema, ignore_modules=ignore),
                                      fisher_type=fisher_type)
        opt = torch.optim.SGD(model.parameters(), lr=0.01)
        grads = []
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            for s in range(2):
                opt.zero_grad()
                torch.manual_seed(9 + s)
                dummy = gm.setup_model_call(model, x)
                if kind == 'gpt2':
                    gm.setup_loss_call(F.cross_entropy, dummy.view(-1, model(x).shape[-1]), t.view(-1))
                else:
                    gm.setup_loss_call(F.cross_entropy, dummy, t)
                gm.forward_and_backward()
                grads.append(torch.cat([p.grad.flatten() for p in model.parameters() if p.grad is not None]).clone())
                opt.step()
        return grads

    want = run(reference, 'KfacGradientMaker', True)
    for maker_name in ('KfacGradientMaker', 'FusedKfacGradientMaker'):
        for w, g in zip(want, run(ours, maker_name, False)):
            assert ((w - g).norm() / w.norm()).item() < 2e-4, maker_name


def test_mixed_shape_rules_on_a_language_model(reference):
    """Shape assignment by class and by name substring: Kronecker factors for the Linear layers, the
    diagonal for the embeddings and the output head, unit-wise blocks for LayerNorm."""
    runs = []
    for lib, plain in ((reference, True), (ours, False)):
        model, tokens, _ = _family('gpt2', plain)
        rules = ['kron', (nn.Embedding, 'diag'), (nn.LayerNorm, 'unit_wise'), ('lm_head', 'diag')]
        gm = lib.NaturalGradientMaker(model, _cfg(lib, data_size=4, damping=1e-2, ema_decay=0.3), fisher_type='fisher_emp',
                                      fisher_shape=rules)
        grads = []
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            for _ in range(2):
                model.zero_grad()
                dummy = gm.setup_model_call(model, tokens)
                gm.setup_loss_call(F.cross_entropy, dummy.view(-1, model(tokens).shape[-1]), tokens.view(-1))
                gm.forward_and_backward()
                grads.append(torch.cat([p.grad.flatten() for p in model.parameters() if p.grad is not None]).clone())
                with torch.no_grad():
                    for p in model.parameters():
                        if p.grad is not None:
                            p -= 0.01 * p.grad
        runs.append(grads)
    for want, got in zip(*runs):
        assert ((want - got).norm() / want.norm()).item() < 1e-4


@pytest.mark.parametrize('options', [
    {'fisher_type': 'fisher_emp'}, {'fisher_type': 'fisher_mc'}, {'fisher_type': 'fisher_exact'},
    {'fisher_type': 'fisher_mc', 'n_mc_samples': 3}, {'fisher_type': 'fisher_mc', 'var': 0.5},
    {'fisher_type': 'fisher_exact', 'ema': 0.3}, {'fisher_type': 'fisher_mc', 'scale': 2.0},
    {'fisher_type': 'fisher_emp', 'grad_scale': 0.5}], ids=lambda o: '-'.join(f'{k}={v}' for k, v in o.items()))
def test_same_gradients_with_a_regression_loss_and_every_constructor_option(reference, options):
    runs = []
    for lib in (reference, ours):
        kw = dict(options)
        model, x, _ = _conv_net()
        torch.manual_seed(4)
        t = torch.randn(8, 3)
        gm = lib.KfacGradientMaker(model, _cfg(lib, data_size=8, damping=1e-2, ema_decay=kw.pop('ema', -1)),
                                   loss_type='mse', **kw)
        opt = torch.optim.SGD(model.parameters(), lr=0.01)
        grads = []
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            for s in range(3):
                opt.zero_grad()
                torch.manual_seed(9 + s)
                dummy = gm.setup_model_call(model, x)
                gm.setup_loss_call(F.mse_loss, dummy, t)
                gm.forward_and_backward()
                grads.append(torch.cat([p.grad.flatten() for p in model.parameters()]).clone())
                opt.step()
        runs.append(grads)
    for want, got in zip(*runs):
        assert ((want - got).norm() / want.norm()).item() < 1e-4


@pytest.mark.parametrize('name,loss', [('loss_hvp', 'cross_entropy'), ('logit_jvp', 'cross_entropy'),
                                       ('fvp', 'cross_entropy'), ('fvp', 'mse')])
def test_same_functional_products_as_the_reference(reference, name, loss):
    results = []
    for lib in (reference, ours):
        model, x, t = _mlp()
        if loss == 'mse':
            torch.manual_seed(2)
            t = torch.randn(8, 3)
        gm = lib.GradientMaker(model)
        dummy = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy if loss == 'cross_entropy' else F.mse_loss, dummy, t)
        tangents = tuple(torch.ones_like(p) for p in model.parameters())
        kwargs = {'tangents': tangents, **({'loss_type': loss} if name == 'fvp' else {})}
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            results.append(torch.cat(_leaves(getattr(gm, name)(**kwargs))))
    want, got = results
    assert want.shape == got.shape and ((want - got).norm() / want.norm()).item() < 1e-5


def test_public_surface_covers_the_reference(reference):
    """Every public name of the reference's flat namespace exists here; every public member of its
    classes and every parameter of its functions and constructors is accepted."""
    import inspect
    problems = []
    for name in dir(reference):
        if name.startswith('_'):
            continue
        if not hasattr(ours, name):
            problems.append(f'missing name {name}')
            continue
        theirs, mine = getattr(reference, name), getattr(ours, name)
        if inspect.isclass(theirs) and inspect.isclass(mine):
            problems += [f'{name}.{m}' for m in dir(theirs) if not m.startswith('_') and not hasattr(mine, m)]
            pairs = [(theirs.__init__, mine.__init__)]
        elif inspect.isfunction(theirs) and inspect.isfunction(mine):
            pairs = [(theirs, mine)]
        else:
            continue
        for f_theirs, f_mine in pairs:
            try:
                wanted, have = inspect.signature(f_theirs).parameters, inspect.signature(f_mine).parameters
            except (TypeError, ValueError):
                continue
            if any(p.kind == p.VAR_KEYWORD for p in have.values()):
                continue
            problems += [f'{name}({p})' for p in wanted if p not in have]
    assert not problems, problems


def test_every_submodule_name_of_the_reference_exists(reference):
    """``from asdl.<module> import <name>`` keeps working with ``asdl_b200.<module>``."""
    import importlib
    import inspect
    import pkgutil
    missing = []
    for info in pkgutil.walk_packages(reference.__path__, 'asdl.'):
        theirs = importlib.import_module(info.name)
        mine = importlib.import_module(info.name.replace('asdl.', 'asdl_b200.', 1))
        for name, obj in vars(theirs).items():
            if name.startswith('_') or inspect.ismodule(obj):
                continue
            defined_here = getattr(obj, '__module__', info.name) == info.name or isinstance(obj, (str, int, float, list, tuple))
            if defined_here and not hasattr(mine, name):
                missing.append(f'{mine.__name__}.{name}')
            elif inspect.isclass(obj) and obj.__module__ == info.name:      # and every public member of its classes
                missing += [f'{mine.__name__}.{name}.{member}' for member in dir(obj)
                            if not member.startswith('_') and not hasattr(getattr(mine, name), member)]
    assert not missing, missing


def test_psgd_factor_formats_and_sparse_lu_match_the_reference(reference):
    import importlib
    theirs = importlib.import_module('asdl.precondition.psgd')
    mine = importlib.import_module('asdl_b200.precondition.psgd')
    torch.manual_seed(0)
    m, n = 5, 7
    dX, dG, G = torch.randn(m, n), torch.randn(m, n), torch.randn(m, n)

    def dense(k):
        return torch.triu(torch.randn(k, k)) * 0.3 + torch.eye(k)

    def scale(k):
        return 1 + 0.1 * torch.rand(1, k)

    def norm(k):      # row 0: diagonal, row 1: last column without its last entry
        q = torch.cat([1 + 0.1 * torch.rand(1, k), 0.1 * torch.randn(1, k)], dim=0)
        q[1, -1] = 0
        return q

    formats = {'scale,dense': (scale(m), dense(n)), 'dense,scale': (dense(m), scale(n)), 'norm,dense': (norm(m), dense(n)),
               'norm,scale': (norm(m), scale(n)), 'dense,norm': (dense(m), norm(n)), 'scale,norm': (scale(m), norm(n))}
    for name, (Ql, Qr) in formats.items():
        results = []
        for lib in (theirs, mine):
            a, b = lib.update_precond_kron(Ql.clone(), Qr.clone(), dX, dG)
            results.append((a, b, lib.precond_grad_kron(a, b, G)))
        for want, got in zip(*results):
            assert ((want - got).norm() / want.norm()).item() < 1e-5, name
    # (dense, dense) and (scale, scale): the reference's dispatcher does not reach them; this library's do something sensible
    a, b = mine.update_precond_kron(dense(m), dense(n), dX, dG)
    assert torch.isfinite(mine.precond_grad_kron(a, b, G)).all()
    a, b = mine.update_precond_kron(scale(m), scale(n), dX, dG)
    assert torch.isfinite(mine.precond_grad_kron(a, b, G)).all()

    r, size = 2, 9
    L12 = torch.cat([torch.eye(r), torch.zeros(size - r, r)], 0) + 0.1 * torch.tril(torch.randn(size, r))
    U12 = torch.cat([torch.eye(r), torch.zeros(r, size - r)], 1) + 0.1 * torch.triu(torch.randn(r, size))
    l3, u3 = 1 + 0.1 * torch.rand(size - r, 1), 1 + 0.1 * torch.rand(size - r, 1)
    dxs, dgs, grads = ([torch.randn(3, 2), torch.randn(3)] for _ in range(3))
    results = []
    for lib in (theirs, mine):
        state = lib.update_precond_splu(L12.clone(), l3.clone(), U12.clone(), u3.clone(), dxs, dgs)
        results.append(list(state) + list(lib.precond_grad_splu(*state, grads)))
    for want, got in zip(*results):
        assert ((want - got).norm() / want.norm()).item() < 1e-5


def _random_network(rng):
    """A random small classifier: 0-3 convolutions (random kernel / stride / padding / bias, optional BatchNorm2d),
    0-2 hidden Linear layers (optional LayerNorm / BatchNorm1d), random activations."""
    layers = []
    if rng.random() < 0.6:
        channels, side = 2, 8
        for _ in range(rng.randint(1, 3)):
            out_channels, k, stride = rng.choice([3, 4, 6]), rng.choice([1, 2, 3]), rng.choice([1, 1, 2])
            pad = rng.choice([0, 1]) if k > 1 else 0
            new_side = (side + 2 * pad - k) // stride + 1
            if new_side < 2:
                continue
            layers.append(nn.Conv2d(channels, out_channels, k, stride=stride, padding=pad, bias=rng.random() < 0.7))
            channels, side = out_channels, new_side
            if rng.random() < 0.5:
                layers.append(nn.BatchNorm2d(channels))
            layers.append(rng.choice([nn.Tanh, nn.ReLU, nn.Sigmoid])())
        layers.append(nn.Flatten())
        width, x = channels * side * side, torch.randn(8, 2, 8, 8)
    else:
        width, x = 7, torch.randn(8, 7)
    for _ in range(rng.randint(0, 2)):
        new_width = rng.choice([4, 5, 9])
        layers.append(nn.Linear(width, new_width, bias=rng.random() < 0.7))
        width = new_width
        draw = rng.random()
        if draw < 0.3:
            layers.append(nn.LayerNorm(width))
        elif draw < 0.5:
            layers.append(nn.BatchNorm1d(width))
        layers.append(rng.choice([nn.Tanh, nn.ReLU])())
    layers.append(nn.Linear(width, 3))
    return nn.Sequential(*layers), x


@pytest.mark.parametrize('seed', range(12))
def test_random_networks_kfac_generic_and_fused(reference, seed):
    import random
    rng = random.Random(seed)
    ema, fisher_type = rng.choice([-1, 0.3, 1.0]), rng.choice(['fisher_emp', 'fisher_mc', 'fisher_exact'])
    damping = rng.choice([1e-1, 1e-2, 1e-3])
    runs = []
    for lib, maker in ((reference, 'KfacGradientMaker'), (ours, 'KfacGradientMaker'), (ours, 'FusedKfacGradientMaker')):
        torch.manual_seed(seed)
        model, x = _random_network(random.Random(seed))
        t = torch.randint(0, 3, (8,))
        gm = getattr(lib, maker)(model, _cfg(lib, data_size=8, damping=damping, ema_decay=ema), fisher_type=fisher_type)
        opt = torch.optim.SGD(model.parameters(), lr=0.01)
        grads = []
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            for s in range(2):
                opt.zero_grad()
                torch.manual_seed(100 + s)
                dummy = gm.setup_model_call(model, x)
                gm.setup_loss_call(F.cross_entropy, dummy, t)
                gm.forward_and_backward()
                grads.append(torch.cat([p.grad.flatten() for p in model.parameters()]).clone())
                opt.step()
        runs.append(grads)
    for other in runs[1:]:
        for want, got in zip(runs[0], other):
            assert ((want - got).norm() / want.norm()).item() < 1e-3


@pytest.mark.parametrize('seed', range(12))
def test_random_networks_fisher_flags(reference, seed):
    import random
    rng = random.Random(seed + 500)
    shape = rng.choice(['full', 'layer_wise', 'kron', 'unit_wise', 'diag'])
    fisher_type = rng.choice(['fisher_exact', 'fisher_mc', 'fisher_emp'])
    loss = rng.choice(['cross_entropy', 'mse'])
    flags = dict(accumulate=rng.random() < 0.4, calc_loss_grad=rng.random() < 0.5, scale=rng.choice([1.0, 0.5, 3.0]))
    if not flags['accumulate'] and rng.random() < 0.4:
        flags.update(calc_inv=True, damping=rng.choice([1e-1, 1e-2]))
    results = []
    for lib in (reference, ours):
        torch.manual_seed(seed)
        model, x = _random_network(random.Random(seed))
        t = torch.randint(0, 3, (8,)) if loss == 'cross_entropy' else torch.randn(8, 3)
        fm = lib.get_fisher_maker(model, lib.FisherConfig(fisher_type=fisher_type, fisher_shapes=[shape], loss_type=loss,
                                                          data_size=8, seed=2))
        with warnings.catch_warnings():
            warnings.simplefilter('ignore')
            for _ in range(2 if flags['accumulate'] else 1):
                dummy = fm.setup_model_call(model, x)
                fm.setup_loss_call(F.cross_entropy if loss == 'cross_entropy' else F.mse_loss, dummy, t)
                out = fm.forward_and_backward(**flags)
        tensors = _fisher_tensors(model)
        if flags['calc_loss_grad']:
            tensors.update({'grad.' + n: p.grad for n, p in model.named_parameters() if p.grad is not None})
            tensors['loss'] = torch.as_tensor(float(out[1]))
        results.append(tensors)
    want, got = results
    assert set(want) == set(got)
    for key in want:
        assert ((want[key] - got[key]).norm() / (want[key].norm() + 1e-30)).item() < 1e-3, key
