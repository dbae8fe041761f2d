"""GradientMaker interface: every way of describing the model / loss call reproduces the plain
hand-written loop (strategy of the reference's test/grad_maker/test_grad_maker.py)."""
from dataclasses import dataclass

import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as asdl
from conftest import make_mlp, make_net, make_data


class WithLoss(nn.Module):
    def __init__(self, kind):
        super().__init__()
        self.body = make_net(kind)

    def forward(self, inputs, targets=None, flip=False):
        logits = self.body(inputs)
        if targets is None:
            return logits
        loss = F.cross_entropy(logits, targets)
        return (loss, logits) if flip else (logits, loss)


@dataclass
class Output:
    loss: torch.Tensor
    logits: torch.Tensor


class SeqModel(nn.Module):
    def __init__(self):
        super().__init__()
        self.body = make_mlp()

    def forward(self, inputs, targets=None, return_dict=True):
        logits = self.body(inputs)
        loss = None
        if targets is not None:
            loss = F.cross_entropy(logits.view(-1, logits.size(-1)), targets.view(-1), ignore_index=-1)
        return Output(loss=loss, logits=logits) if return_dict else (loss, logits)


def flat_grads(model):
    return torch.cat([p.grad.flatten() for p in model.parameters()])


def reference_step(model, fn):
    model.zero_grad()
    out = fn()
    return out


@pytest.mark.parametrize('kind', ['mlp', 'cnn'])
def test_tensor_output_with_loss_call(kind):
    model = WithLoss(kind)
    x, t = make_data(kind, 4, 'cross_entropy')
    model.zero_grad()
    logits = model(x)
    loss = F.cross_entropy(logits, t)
    loss.backward()
    want = flat_grads(model).clone()

    model.zero_grad()
    gm = asdl.GradientMaker(model)
    dummy = gm.setup_model_call(model, x)
    gm.setup_loss_call(F.cross_entropy, dummy, t)
    y, l = gm.forward_and_backward()
    torch.testing.assert_close(y, logits)
    torch.testing.assert_close(l, loss)
    torch.testing.assert_close(flat_grads(model), want)


@pytest.mark.parametrize('flip', [False, True])
def test_tuple_output_with_loss_repr(flip):
    model = WithLoss('mlp')
    x, t = make_data('mlp', 4, 'cross_entropy')
    model.zero_grad()
    out = model(x, targets=t, flip=flip)
    loss = out[0] if flip else out[1]
    loss.backward()
    want = flat_grads(model).clone()

    model.zero_grad()
    gm = asdl.GradientMaker(model)
    dummy = gm.setup_model_call(model, x, targets=t, flip=flip)
    gm.setup_loss_repr(dummy[0] if flip else dummy[1])
    y, l = gm.forward_and_backward()
    torch.testing.assert_close(l, loss)
    torch.testing.assert_close(y[1] if flip else y[0], out[1] if flip else out[0])
    torch.testing.assert_close(flat_grads(model), want)


def test_dataclass_output_and_placeholder_calls():
    model = SeqModel()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 8, 5, generator=g)
    t = torch.randint(-1, 3, (2, 8), generator=g)
    model.zero_grad()
    out = model(x, targets=t)
    out.loss.backward()
    want = flat_grads(model).clone()

    # (a) the model's own loss
    model.zero_grad()
    gm = asdl.GradientMaker(model)
    dummy = gm.setup_model_call(model, x, targets=t)
    gm.setup_loss_repr(dummy.loss)
    y, l = gm.forward_and_backward()
    torch.testing.assert_close(l, out.loss)
    torch.testing.assert_close(flat_grads(model), want)

    # (b) pseudo-calls on the placeholder, evaluated at forward time
    model.zero_grad()
    gm = asdl.GradientMaker(model)
    dummy = gm.setup_model_call(model, x)
    logits = dummy.logits.view(-1, dummy.logits.size(-1))
    gm.setup_loss_call(F.cross_entropy, logits, t.view(-1), ignore_index=-1)
    y, l = gm.forward_and_backward()
    torch.testing.assert_close(l, out.loss)
    torch.testing.assert_close(flat_grads(model), want)


def test_dict_output():
    body = make_mlp()

    def model_fn(x, t):
        logits = body(x)
        return {'logits': logits, 'loss': F.cross_entropy(logits, t)}

    x, t = make_data('mlp', 4, 'cross_entropy')
    gm = asdl.GradientMaker(body)
    dummy = gm.setup_model_call(model_fn, x, t)
    gm.setup_loss_repr(dummy['loss'])
    out, loss = gm.forward_and_backward()
    assert loss is out['loss']
    assert all(p.grad is not None for p in body.parameters())


def test_missing_setup_raises():
    gm = asdl.GradientMaker(make_mlp())
    with pytest.raises(ValueError):
        gm.forward_and_backward()
    gm.setup_model_call(gm.model, torch.randn(2, 5))
    with pytest.raises(ValueError):
        gm.forward_and_backward()
    with pytest.raises(TypeError):
        gm.setup_loss_repr('not a dummy')


def test_dummy_object_eval():
    lin = nn.Linear(5, 3)
    assert asdl.DummyObject().weight[0].numel().eval(lin) == 5
    d = asdl.DummyObject()
    expr = d[0].add(d[1])
    assert expr.eval((torch.ones(2), torch.ones(2))).tolist() == [2., 2.]


def test_functional_utilities():
    model = make_mlp()
    x, t = make_data('mlp', 6, 'cross_entropy')
    gm = asdl.GradientMaker(model)
    dummy = gm.setup_model_call(model, x)
    gm.setup_loss_call(F.cross_entropy, dummy, t)
    # gradient
    grads = gm.loss_grad()
    model.zero_grad()
    F.cross_entropy(model(x), t).backward()
    for g, p in zip(grads, model.parameters()):
        torch.testing.assert_close(g, p.grad)
    # per-example gradients sum to the batch gradient (mean reduction -> each is for batch of 1)
    per = gm.per_example_loss_grads()
    for g, p in zip(per, model.parameters()):
        assert g.shape == (6, *p.shape)
        torch.testing.assert_close(g.mean(0), p.grad, rtol=1e-4, atol=1e-6)
    # hessian-vector product against the explicit Hessian
    tang = tuple(torch.randn_like(p) for p in model.parameters())
    hvp = gm.loss_hvp(tangents=tang, accumulate_grad=False)
    H = gm.loss_hessian()
    params = list(model.parameters())
    for i in range(len(params)):
        want = sum((H[i][j].reshape(params[i].numel(), -1) @ tang[j].flatten()) for j in range(len(params)))
        torch.testing.assert_close(hvp[i].flatten(), want, rtol=1e-4, atol=1e-5)
    # fvp equals J^T H J v built from the Jacobian
    fvp = gm.fvp(asdl.LOSS_CROSS_ENTROPY, tangents=tang)
    J = gm.logit_jacobian()
    Jv = sum(torch.einsum('nc...,...->nc', j, v) for j, v in zip(J, tang))
    probs = F.softmax(model(x), dim=1).detach()
    HJv = probs * Jv - probs * (probs * Jv).sum(1, keepdim=True)
    for f, j in zip(fvp, J):
        want = torch.einsum('nc...,nc->...', j, HJv) / 6
        torch.testing.assert_close(f, want, rtol=1e-4, atol=1e-6)
