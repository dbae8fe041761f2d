"""Gradient helpers: dataset-level gradients (optionally reduced over ranks), per-example
gradients and logit Jacobians through the hook engine.
Parity: asdl/gradient.py:10-106 (``jacobian`` reads the per-example gradients from the context;
the reference reads an attribute that is never written)."""
import torch
import torch.distributed as dist

from .core import extend
from .operations import OP_BATCH_GRADS

__all__ = ['data_loader_gradient', 'batch_gradient', 'save_batch_gradient', 'jacobian']


def data_loader_gradient(model, loss_fn, data_loader, is_distributed=False, all_reduce=False,
                         is_master=True, data_average=True):
    """Accumulates ``loss_fn(model(x), t)`` gradients over a loader (``loss_fn`` is expected to
    use ``reduction='sum'``), optionally averages over the dataset, and optionally averages the
    result over ranks with a single packed message.  Returns the (averaged) loss."""
    device = next(model.parameters()).device
    total = torch.zeros((), device=device)
    for inputs, targets in data_loader:
        inputs, targets = inputs.to(device), targets.to(device)
        loss = loss_fn(model(inputs), targets)
        loss.backward()
        total += loss.detach()
    total_loss = total.item()
    if data_average:
        n = len(data_loader.dataset)
        for p in model.parameters():
            if p.grad is not None:
                p.grad.div_(n)
        total_loss /= n
    if is_distributed:
        grads = [p.grad for p in model.parameters() if p.requires_grad]
        packed = torch.cat([g.reshape(-1) for g in grads] + [torch.tensor([total_loss], device=device)])
        if all_reduce:
            dist.all_reduce(packed)
        else:
            dist.reduce(packed, dst=0)
        if is_master or all_reduce:
            packed.div_(dist.get_world_size())
            total_loss = packed[-1].item()
            offset = 0
            for g in grads:
                g.copy_(packed[offset:offset + g.numel()].view_as(g))
                offset += g.numel()
        dist.barrier()
    return total_loss


def batch_gradient(model, closure, return_outputs=False):
    """Per-example gradients (n x p) of whatever ``closure`` back-propagates."""
    with extend(model, OP_BATCH_GRADS) as cxt:
        outputs = closure()
        parts = [cxt.batch_grads(m, flatten=True) for m in model.modules()]
        grads = torch.cat([g for g in parts if g is not None], dim=-1)
    return (grads, outputs) if return_outputs else grads


def save_batch_gradient(model, closure, return_outputs=False):
    """Like :func:`batch_gradient` but stores (accumulates) ``param.batch_grad``."""
    with extend(model, OP_BATCH_GRADS) as cxt:
        outputs = closure()
        for module in model.modules():
            grads = cxt.batch_grads(module)
            if grads is None:
                continue
            for key, value in grads.items():
                param = getattr(module, key)
                if hasattr(param, 'batch_grad'):
                    param.batch_grad += value
                else:
                    param.batch_grad = value
    if return_outputs:
        return outputs


def jacobian(model, x):
    """Jacobian of the (n x c) model output w.r.t. the parameters: n x c x p."""
    with extend(model, OP_BATCH_GRADS) as cxt:
        f = model(x)
        if f.ndim != 2:
            raise ValueError(f'Number of output dimensions has to be 2. Got {f.ndim}')
        n, c = f.shape
        rows = []
        for i in range(c):
            cxt.clear_batch_grads()
            params = [p for p in model.parameters() if p.requires_grad]
            torch.autograd.grad(f[:, i].sum(), params, retain_graph=i < c - 1, allow_unused=True)
            parts = [cxt.batch_grads(m, flatten=True) for m in model.modules()]
            rows.append(torch.cat([g for g in parts if g is not None], dim=1))
    return torch.stack(rows).transpose(0, 1)
