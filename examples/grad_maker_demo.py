"""The gradient-maker interface on models with different output conventions.

    python examples/grad_maker_demo.py

Four ways a model hands back its result, each trained for a few steps with the same K-FAC maker code:
logits; a (logits, loss) tuple; an object with ``.logits`` / ``.loss`` attributes (the convention of
Hugging Face models); and logits that the loss wants reshaped.  Role of the reference's
examples/grad_maker_demo1.py and grad_maker_demo2.py.
"""
import os
import sys
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402


@dataclass
class Output:
    loss: torch.Tensor
    logits: torch.Tensor


class Net(nn.Module):
    def __init__(self, mode):
        super().__init__()
        self.mode = mode
        self.body = nn.Sequential(nn.Linear(12, 16), nn.ReLU(), nn.Linear(16, 4))

    def forward(self, x, labels=None):
        logits = self.body(x)
        if self.mode == 'logits':
            return logits
        # curvature makers work with the *summed* loss and divide by data_size themselves
        loss = F.cross_entropy(logits.view(-1, 4), labels.view(-1), reduction='sum') if labels is not None else None
        return (logits, loss) if self.mode == 'tuple' else Output(loss=loss, logits=logits)


def train(mode):
    torch.manual_seed(0)
    model = Net(mode if mode != 'reshape' else 'logits')
    x = torch.randn(32, 12) if mode != 'reshape' else torch.randn(8, 4, 12)      # (batch, seq, features)
    t = torch.randint(0, 4, x.shape[:-1])
    config = asdl.PreconditioningConfig(data_size=t.numel(), damping=1e-2)
    grad_maker = asdl.KfacGradientMaker(model, config, fisher_type=asdl.FISHER_EMP)
    optimizer = torch.optim.SGD(model.parameters(), lr=0.1)
    losses = []
    for _ in range(10):
        optimizer.zero_grad()
        if mode == 'logits':
            dummy_y = grad_maker.setup_model_call(model, x)
            grad_maker.setup_loss_call(F.cross_entropy, dummy_y, t)
        elif mode == 'tuple':          # the model computes the loss: pick it out of the tuple
            dummy_y = grad_maker.setup_model_call(model, x, labels=t)
            grad_maker.setup_loss_repr(dummy_y[1])
        elif mode == 'object':         # ... or out of an attribute
            dummy_y = grad_maker.setup_model_call(model, x, labels=t)
            grad_maker.setup_loss_repr(dummy_y.loss)
        else:                          # operations on the placeholder are replayed on the real output
            dummy_y = grad_maker.setup_model_call(model, x)
            grad_maker.setup_loss_call(F.cross_entropy, dummy_y.view(-1, dummy_y.size(-1)), t.view(-1))
        _, loss = grad_maker.forward_and_backward()
        optimizer.step()
        losses.append(float(loss.detach()))
    print(f'{mode:8s} loss {losses[0]:.4f} -> {losses[-1]:.4f}')


if __name__ == '__main__':
    for mode in ('logits', 'tuple', 'object', 'reshape'):
        train(mode)
