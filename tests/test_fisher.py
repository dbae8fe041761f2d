"""Curvature oracle tests (strategy of the reference's test/grad_maker/test_fisher.py): the full
Fisher of one sample is the ground truth; every other shape has to be the matching slice of it."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as asdl
from asdl_b200 import (FISHER_EXACT, FISHER_MC, FISHER_EMP, SHAPE_FULL, SHAPE_LAYER_WISE, SHAPE_KRON,
                       SHAPE_UNIT_WISE, SHAPE_DIAG, LOSS_CROSS_ENTROPY, LOSS_MSE)
from conftest import make_net, make_data

KINDS = ['mlp', 'cnn']
TYPES = [FISHER_EXACT, FISHER_MC, FISHER_EMP]
LOSSES = [LOSS_CROSS_ENTROPY, LOSS_MSE]
BS = 4


def loss_fn_for(loss_type):
    return F.cross_entropy if loss_type == LOSS_CROSS_ENTROPY else F.mse_loss


def make_maker(model, fisher_type, shape, loss_type, **kw):
    config = asdl.FisherConfig(fisher_type=fisher_type, fisher_shapes=[shape], loss_type=loss_type,
                               seed=1, **kw)
    return asdl.get_fisher_maker(model, config)


def run(maker, model, x, t, loss_type, **kw):
    dummy = maker.setup_model_call(model, x)
    maker.setup_loss_call(loss_fn_for(loss_type), dummy, t)
    return maker.forward_and_backward(**kw)


def full_fisher(model, fisher_type, loss_type, x, t, data_size=1):
    maker = make_maker(model, fisher_type, SHAPE_FULL, loss_type)
    run(maker, model, x, t, loss_type, data_size=data_size)
    return model.fisher.data.clone()


def layer_slices(model):
    out, start = {}, 0
    for m in model.modules():
        if isinstance(m, (nn.Linear, nn.Conv2d)):
            n = m.weight.numel() + m.bias.numel()
            out[m] = (start, start + n)
            start += n
    return out


@pytest.mark.parametrize('kind', KINDS)
@pytest.mark.parametrize('fisher_type', TYPES)
@pytest.mark.parametrize('loss_type', LOSSES)
def test_batch_of_copies_scales(kind, fisher_type, loss_type):
    if fisher_type == FISHER_MC:
        pytest.skip('sampling differs between the two runs')
    model = make_net(kind)
    x1, t1 = make_data(kind, 1, loss_type)
    f1 = full_fisher(model, fisher_type, loss_type, x1, t1)
    reps = (BS,) + (1,) * (x1.ndim - 1)
    xb, tb = x1.repeat(*reps), t1.repeat(*((BS,) + (1,) * (t1.ndim - 1)))
    fb = full_fisher(model, fisher_type, loss_type, xb, tb)
    factor = BS if fisher_type != FISHER_EMP or loss_type == LOSS_CROSS_ENTROPY else BS
    if fisher_type == FISHER_EMP and loss_type == LOSS_MSE:
        pytest.skip('sum-reduced MSE of copies is not a per-sample sum of the same quantity')
    torch.testing.assert_close(fb, f1 * factor, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize('kind', KINDS)
@pytest.mark.parametrize('fisher_type', TYPES)
@pytest.mark.parametrize('loss_type', LOSSES)
def test_shapes_are_slices_of_full(kind, fisher_type, loss_type):
    model = make_net(kind)
    x, t = make_data(kind, 1, loss_type)
    full = full_fisher(model, fisher_type, loss_type, x, t)
    assert full.shape[0] == sum(p.numel() for p in model.parameters())
    torch.testing.assert_close(full, full.T)
    slices = layer_slices(model)

    # layer-wise = diagonal blocks
    maker = make_maker(model, fisher_type, SHAPE_LAYER_WISE, loss_type)
    run(maker, model, x, t, loss_type, data_size=1)
    for m, (a, b) in slices.items():
        torch.testing.assert_close(m.fisher.data, full[a:b, a:b], rtol=1e-4, atol=1e-6)

    # Kronecker factors: for ONE sample kron(B, A) is the weight block (Linear), B the bias block
    maker = make_maker(model, fisher_type, SHAPE_KRON, loss_type)
    run(maker, model, x, t, loss_type, data_size=1)
    for m, (a, b) in slices.items():
        A, B = m.fisher.kron.A, m.fisher.kron.B
        torch.testing.assert_close(A, A.T)
        torch.testing.assert_close(B, B.T)
        assert A.shape[0] == m.weight[0].numel() and B.shape[0] == m.weight.shape[0]
        if isinstance(m, nn.Linear) and not (fisher_type != FISHER_EMP and False):
            nw = m.weight.numel()
            if fisher_type == FISHER_EMP or full[a:b, a:b].abs().sum() > 0:
                if fisher_type == FISHER_EMP or fisher_type == FISHER_MC:
                    torch.testing.assert_close(torch.kron(B, A), full[a:a + nw, a:a + nw],
                                               rtol=1e-4, atol=1e-6)
                torch.testing.assert_close(B, full[a + nw:b, a + nw:b], rtol=1e-4, atol=1e-6)

    # unit-wise blocks
    maker = make_maker(model, fisher_type, SHAPE_UNIT_WISE, loss_type)
    run(maker, model, x, t, loss_type, data_size=1)
    for m, (a, b) in slices.items():
        blk = full[a:b, a:b]
        f_out = m.weight.shape[0]
        f_in = m.weight[0].numel()
        nw = m.weight.numel()
        for o in range(f_out):
            idx = list(range(o * f_in, (o + 1) * f_in)) + [nw + o]
            idx = torch.tensor(idx)
            torch.testing.assert_close(m.fisher.unit.data[o], blk[idx][:, idx], rtol=1e-4, atol=1e-6)

    # diagonal
    maker = make_maker(model, fisher_type, SHAPE_DIAG, loss_type)
    run(maker, model, x, t, loss_type, data_size=1)
    for m, (a, b) in slices.items():
        d = torch.cat([m.fisher.diag.weight.flatten(), m.fisher.diag.bias.flatten()])
        torch.testing.assert_close(d, torch.diag(full[a:b, a:b]), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize('kind', KINDS)
@pytest.mark.parametrize('loss_type', LOSSES)
def test_exact_fisher_is_ggn(kind, loss_type):
    model = make_net(kind)
    x, t = make_data(kind, 3, loss_type)
    full = full_fisher(model, FISHER_EXACT, loss_type, x, t, data_size=3)
    params = list(model.parameters())
    logits = model(x)
    n, c = logits.shape
    rows = []
    for i in range(n):
        for k in range(c):
            g = torch.autograd.grad(logits[i, k], params, retain_graph=True)
            rows.append(torch.cat([v.flatten() for v in g]))
    J = torch.stack(rows).view(n, c, -1)
    if loss_type == LOSS_CROSS_ENTROPY:
        p = F.softmax(logits, dim=1).detach()
        H = torch.diag_embed(p) - torch.einsum('ni,nj->nij', p, p)
    else:
        H = torch.eye(c).expand(n, c, c)
    ggn = torch.einsum('nip,nij,njq->pq', J, H, J) / n
    torch.testing.assert_close(full, ggn, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize('shape', [SHAPE_FULL, SHAPE_LAYER_WISE, SHAPE_KRON, SHAPE_UNIT_WISE, SHAPE_DIAG])
@pytest.mark.parametrize('fisher_type', [FISHER_EXACT, FISHER_EMP])
def test_accumulate_scale_data_size(shape, fisher_type):
    kind, loss_type = 'mlp', LOSS_CROSS_ENTROPY
    model = make_net(kind)
    x, t = make_data(kind, BS, loss_type)

    def tensors():
        out = {}
        for name, m in model.named_modules():
            f = getattr(m, 'fisher', None)
            if f is not None:
                out.update({f'{name}.{k}': v.clone() for k, v in f.tensors().items()})
        return out

    maker = make_maker(model, fisher_type, shape, loss_type)
    run(maker, model, x, t, loss_type, data_size=BS)
    base = tensors()
    assert base
    for _ in range(2):
        run(maker, model, x, t, loss_type, data_size=BS, accumulate=True)
    for k, v in tensors().items():
        torch.testing.assert_close(v, base[k] * 3, rtol=1e-4, atol=1e-6)
    run(maker, model, x, t, loss_type, data_size=BS, scale=10.)
    for k, v in tensors().items():
        torch.testing.assert_close(v, base[k] * 10, rtol=1e-4, atol=1e-6)
    run(maker, model, x, t, loss_type, data_size=BS * 2)
    for k, v in tensors().items():
        torch.testing.assert_close(v, base[k] / 2, rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize('kind', KINDS)
@pytest.mark.parametrize('shape', [SHAPE_FULL, SHAPE_LAYER_WISE, SHAPE_KRON, SHAPE_UNIT_WISE, SHAPE_DIAG])
@pytest.mark.parametrize('fisher_type', TYPES)
def test_inverse(kind, shape, fisher_type):
    loss_type, damping = LOSS_CROSS_ENTROPY, 1.0
    model = make_net(kind)
    x, t = make_data(kind, BS, loss_type)
    maker = make_maker(model, fisher_type, shape, loss_type)
    run(maker, model, x, t, loss_type, data_size=BS)
    data = {m: m.fisher for m in model.modules() if getattr(m, 'fisher', None) is not None}
    for m in data:
        del m.fisher
    maker = make_maker(model, fisher_type, shape, loss_type)
    run(maker, model, x, t, loss_type, data_size=BS, calc_inv=True, damping=damping)

    def check(mat, inv, damp):
        eye = torch.eye(mat.shape[-1])
        torch.testing.assert_close((mat + damp * eye) @ inv, eye.expand_as(inv), rtol=1e-3, atol=1e-4)

    for m, f in data.items():
        g = m.fisher
        if shape in (SHAPE_FULL, SHAPE_LAYER_WISE):
            assert g.data is None
            check(f.data, g.inv, damping)
        elif shape == SHAPE_KRON:
            assert g.kron.A is None and g.kron.B is None
            A, B = f.kron.A, f.kron.B
            pi = torch.sqrt((A.trace() / A.shape[0]) / (B.trace() / B.shape[0]))
            check(A, g.kron.A_inv, max(damping ** 0.5 * pi.item(), 1e-7))
            check(B, g.kron.B_inv, max(damping ** 0.5 / pi.item(), 1e-7))
        elif shape == SHAPE_UNIT_WISE:
            assert g.unit.data is None
            check(f.unit.data, g.unit.inv, damping)
        else:
            torch.testing.assert_close(g.diag.weight_inv, 1 / (f.diag.weight + damping))
            torch.testing.assert_close(g.diag.bias_inv, 1 / (f.diag.bias + damping))


def test_inverse_data_size_law():
    """Kron inverse with (data_size=N, damping=d) equals N x the inverse with damping d*N^2
    taken at data_size=1 ... i.e. inv_N(d) = N * inv_1(d*N) per factor."""
    kind, loss_type, damping, N = 'mlp', LOSS_CROSS_ENTROPY, 1e-2, 4
    model = make_net(kind)
    x, t = make_data(kind, BS, loss_type)
    for shape in (SHAPE_LAYER_WISE, SHAPE_KRON, SHAPE_DIAG):
        maker = make_maker(model, FISHER_EMP, shape, loss_type)
        run(maker, model, x, t, loss_type, data_size=1, calc_inv=True,
            damping=damping * (N * N if shape == SHAPE_KRON else N))
        ref = {m: {k: v.clone() for k, v in m.fisher.tensors().items()}
               for m in model.modules() if getattr(m, 'fisher', None) is not None}
        run(maker, model, x, t, loss_type, data_size=N, calc_inv=True, damping=damping)
        for m, items in ref.items():
            for k, v in m.fisher.tensors().items():
                torch.testing.assert_close(v, items[k] * N, rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize('kind', KINDS)
@pytest.mark.parametrize('shape', [SHAPE_FULL, SHAPE_LAYER_WISE])
@pytest.mark.parametrize('fisher_type', TYPES)
def test_fvp_and_eig(kind, shape, fisher_type):
    loss_type = LOSS_CROSS_ENTROPY
    model = make_net(kind)
    x, t = make_data(kind, BS, loss_type)
    maker = make_maker(model, fisher_type, shape, loss_type, data_size=BS)
    run(maker, model, x, t, loss_type)
    params = list(model.parameters())
    vec = asdl.ParamVector(params, [torch.randn_like(p) for p in params])
    if shape == SHAPE_FULL:
        want = model.fisher.data @ vec.get_flatten_vector()
        top = torch.linalg.eigvalsh(model.fisher.data).max().item()
    else:
        pieces, tops = [], []
        for m in model.modules():
            f = getattr(m, 'fisher', None)
            if f is None or m is model:
                continue
            v = vec.get_vectors_by_module(m).get_flatten_vector()
            pieces.append(f.data @ v)
            tops.append(torch.linalg.eigvalsh(f.data).max().item())
        want, top = torch.cat(pieces), max(tops)
    run(maker, model, x, t, loss_type, fvp=True, vec=vec)
    got = maker.load_fvp(shape).get_flatten_vector()
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-6)
    if fisher_type != FISHER_MC:
        eigvals, _ = maker.fisher_eig(top_n=1, max_iters=500, tol=1e-10)
        assert abs(eigvals[0] - top) / top < 1e-3


def test_fisher_free_and_quadratic_form():
    kind, loss_type = 'mlp', LOSS_CROSS_ENTROPY
    model = make_net(kind)
    x, t = make_data(kind, BS, loss_type)
    maker = make_maker(model, FISHER_EMP, SHAPE_FULL, loss_type, data_size=BS)
    run(maker, model, x, t, loss_type, calc_loss_grad=True)
    F_ = model.fisher.data.clone()
    g = torch.cat([p.grad.flatten() for p in model.parameters()])
    sol = maker.fisher_free(damping=1e-2, tol=1e-10)
    want = torch.linalg.solve(F_ + 1e-2 * torch.eye(F_.shape[0]), g)
    torch.testing.assert_close(sol.get_flatten_vector(), want, rtol=1e-3, atol=1e-5)
    params = list(model.parameters())
    v = asdl.ParamVector(params, [torch.randn_like(p) for p in params])
    q = maker.fisher_quadratic_form(v)
    flat = v.get_flatten_vector()
    torch.testing.assert_close(q, flat @ (F_ @ flat), rtol=1e-4, atol=1e-6)


def test_norm_embedding_layers():
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 8), nn.BatchNorm1d(8), nn.ReLU(), nn.Linear(8, 8),
                          nn.LayerNorm(8), nn.Linear(8, 3))
    x, t = torch.randn(5, 6), torch.randint(3, (5,))
    config = asdl.FisherConfig(fisher_type=FISHER_EMP, fisher_shapes=[SHAPE_LAYER_WISE])
    maker = asdl.get_fisher_maker(model, config)
    # per-example gradients via the hook path vs torch.func
    with asdl.extend(model, asdl.OP_BATCH_GRADS) as cxt:
        F.cross_entropy(model(x), t, reduction='sum').backward()
        got = {m: cxt.batch_grads(m) for m in model if isinstance(m, (nn.LayerNorm, nn.Linear))}
    gm = asdl.GradientMaker(model)
    # LayerNorm and Linear after BN see the batch statistics as constants only approximately;
    # check the last Linear and LayerNorm, which are exact
    ln, last = model[4], model[5]
    h = model[:4](x)
    hn = ((ln(h) - ln.bias) / ln.weight).detach()
    hh = ln(h).detach().requires_grad_(True)
    loss = F.cross_entropy(last(hh), t, reduction='sum')
    gout, = torch.autograd.grad(loss, hh)
    torch.testing.assert_close(got[ln]['weight'], hn * gout, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(got[ln]['bias'], gout, rtol=1e-4, atol=1e-6)
    # unit-wise 2x2 blocks
    with asdl.extend(model, asdl.OP_COV_UNIT_WISE, ignore_modules=[nn.Linear]) as cxt:
        F.cross_entropy(model(x), t, reduction='sum').backward()
        blocks = cxt.cov_unit_wise(ln)['data']
    gw, gb = hn * gout, gout
    torch.testing.assert_close(blocks[:, 0, 0], (gw ** 2).sum(0), rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(blocks[:, 0, 1], (gw * gb).sum(0), rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(blocks[:, 1, 1], (gb ** 2).sum(0), rtol=1e-4, atol=1e-6)

    emb = nn.Sequential(nn.Embedding(11, 4), nn.Flatten(), nn.Linear(12, 3))
    idx = torch.randint(11, (5, 3))
    with asdl.extend(emb, asdl.OP_BATCH_GRADS, asdl.OP_COV_DIAG, asdl.OP_COV_KRON) as cxt:
        F.cross_entropy(emb(idx), t, reduction='sum').backward()
        bg = cxt.batch_grads(emb[0])['weight']
        kron = cxt.cov_kron(emb[0])
    emb.zero_grad()
    F.cross_entropy(emb(idx), t, reduction='sum').backward()
    torch.testing.assert_close(bg.sum(0), emb[0].weight.grad, rtol=1e-4, atol=1e-6)
    assert kron['A'].shape == (11, 11) and kron['B'].shape == (4, 4)


@pytest.mark.parametrize('loss_type', LOSSES)
def test_exact_fisher_of_a_token_level_model_is_the_ggn(loss_type):
    """Outputs n x tokens x classes: every token is an example; the exact Fisher is J^T H J / data_size
    over all (example, token) rows."""
    torch.manual_seed(0)
    model = nn.Sequential(nn.Embedding(11, 4), nn.LayerNorm(4), nn.Linear(4, 3))
    tokens = torch.randint(0, 11, (8, 3))
    ce = loss_type == asdl.LOSS_CROSS_ENTROPY
    t = torch.randint(0, 3, (24,)) if ce else torch.randn(24, 3)
    fm = asdl.get_fisher_maker(model, asdl.FisherConfig(fisher_type=FISHER_EXACT, fisher_shapes=[SHAPE_FULL],
                                                        loss_type=loss_type, data_size=8))
    dummy = fm.setup_model_call(model, tokens)
    fm.setup_loss_call(F.cross_entropy if ce else F.mse_loss, dummy.view(-1, 3), t)
    fm.forward_and_backward()
    y = model(tokens).view(-1, 3)
    params = list(model.parameters())
    rows = []
    for i in range(24):
        for c in range(3):
            grads = torch.autograd.grad(y[i, c], params, retain_graph=True)
            rows.append(torch.cat([g.flatten() for g in grads]))
    J = torch.stack(rows).view(24, 3, -1)
    if ce:
        p = y.softmax(dim=1).detach()
        H = torch.diag_embed(p) - p.unsqueeze(2) * p.unsqueeze(1)
    else:
        H = torch.eye(3).expand(24, 3, 3)
    want = torch.einsum('ncp,ncd,ndq->pq', J, H, J) / 8
    torch.testing.assert_close(model.fisher.data, want, rtol=1e-4, atol=1e-6)
