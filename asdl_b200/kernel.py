"""Neural-tangent-kernel utilities and function-space natural gradients.

Parity: asdl/kernel.py:42-795.
  * ``batch`` assembles a kernel matrix block by block over mini-batches, serially or with the
    blocks spread over ranks (gathered on the master, on all ranks, or redistributed class-wise);
  * ``empirical_direct_ntk`` (explicit Jacobians), ``empirical_implicit_ntk`` (double backward),
    class-wise NTKs from Gram hooks (direct or Hadamard-factored), optionally preconditioned;
  * natural gradients in function space for cross-entropy: dense (n*c x n*c), class-wise
    "efficient" form, its data->class->data parallel version, and the matrix-free CG solver
    ``kernel_free_cross_entropy``; kernel spectra by power iteration;
  * Woodbury empirical natural gradients from hooks or from a saved-tensor context.

The reference's ``empirical_direct_ntk`` reads results through an accessor that no longer exists
in its own code base; here the per-example gradients come from the hook context.  Rank-to-rank
redistribution uses ``all_to_all`` where the backend has it and falls back to gathers otherwise.
"""
from functools import partial
from typing import List

import numpy as np
import torch
from torch import Tensor
from torch.nn import functional as F
from torch.utils.data import DataLoader, Subset, TensorDataset
import torch.distributed as dist

from .core import extend, save_inputs_outgrads
from .operations import *  # noqa: F401,F403
from .operations import OP_BATCH_GRADS, OP_GRAM_HADAMARD, OP_GRAM_DIRECT, OperationContext
from .utils import skip_param_grad

__all__ = [
    'batch', 'empirical_direct_ntk', 'empirical_implicit_ntk', 'empirical_class_wise_direct_ntk',
    'empirical_class_wise_hadamard_ntk', 'get_preconditioned_kernel_fn',
    'logits_hessian_cross_entropy', 'natural_gradient_cross_entropy',
    'efficient_natural_gradient_cross_entropy', 'parallel_efficient_natural_gradient_cross_entropy',
    'kernel_vector_product', 'kernel_free_cross_entropy', 'kernel_eigenvalues',
    'empirical_natural_gradient', 'empirical_natural_gradient2', 'empirical_natural_gradient_by_context'
]

_MASTER, _ALL, _SPLIT = 'master', 'all', 'split'


# ----------------------------------------------------------------------------------------------
# block-wise kernel assembly
# ----------------------------------------------------------------------------------------------
def batch(kernel_fn, model, x1, x2=None, batch_size=1, store_on_device=True, is_distributed=False,
          gather_type=_MASTER):
    """Kernel matrix between ``x1`` and ``x2`` (or ``x1`` with itself) built from
    ``kernel_fn(model, batch1, batch2)`` blocks.  Result: n1 x n2 x c or n1 x n2 x c x c."""
    def loader_of(x):
        if isinstance(x, DataLoader):
            return x
        if isinstance(x, Tensor):
            if x.shape[0] % batch_size != 0:
                raise ValueError(f'data size ({x.shape[0]}) has to be divisible by batch size ({batch_size}).')
            return DataLoader(TensorDataset(x), batch_size)
        raise ValueError(f'x1 and x2 have to be {DataLoader} or {Tensor}. {type(x)} was given.')

    loader1 = loader_of(x1)
    loader2 = None if x2 is None else loader_of(x2)
    if is_distributed:
        return _parallel(kernel_fn, model, loader1, loader2, store_on_device, gather_type)
    return _serial(kernel_fn, model, loader1, loader2, store_on_device)


def _inputs_of(item):
    inputs = item[0] if isinstance(item, (tuple, list)) else item
    if not isinstance(inputs, torch.Tensor):
        raise TypeError(f'inputs have to be {torch.Tensor}. Got {type(inputs)}.')
    return inputs


def _mirror(block):
    """Block (j, i) of a symmetric kernel from block (i, j)."""
    out = block.transpose(0, 1)
    return out.transpose(2, 3) if out.ndim == 4 else out


def _assemble(blocks, n_rows, n_cols, symmetric):
    if symmetric:
        for i in range(n_rows):
            for j in range(i):
                blocks[i][j] = _mirror(blocks[j][i])
    return torch.cat([torch.cat(blocks[i], dim=1) for i in range(n_rows)], dim=0)


def _serial(kernel_fn, model, loader1, loader2=None, store_on_device=True):
    device = next(iter(model.parameters())).device
    keep = device if store_on_device else 'cpu'
    symmetric = loader2 is None
    batches1 = [_inputs_of(b).to(device) for b in loader1]
    batches2 = batches1 if symmetric else [_inputs_of(b).to(device) for b in loader2]
    blocks = [[None] * len(batches2) for _ in batches1]
    for i, b1 in enumerate(batches1):
        for j, b2 in enumerate(batches2):
            if symmetric and j < i:
                continue
            block = kernel_fn(model, b1) if (symmetric and i == j) else kernel_fn(model, b1, b2)
            blocks[i][j] = block.to(keep)
    return _assemble(blocks, len(batches1), len(batches2), symmetric).to(device)


def _subset_loader(loader: DataLoader, batch_indices: List[int]):
    bs, n = loader.batch_size, len(loader.dataset)
    samples = [s for b in batch_indices for s in range(b * bs, min((b + 1) * bs, n))]
    return DataLoader(Subset(loader.dataset, samples), bs, pin_memory=loader.pin_memory,
                      num_workers=loader.num_workers)


def _gather_to(tensor, dst, rank, world_size):
    """``dist.gather`` with the receive list only on ``dst``."""
    if rank == dst:
        out = [torch.zeros_like(tensor) for _ in range(world_size)]
        dist.gather(tensor, out, dst=dst)
        return out
    dist.gather(tensor, dst=dst)
    return None


def _parallel(kernel_fn, model, loader1, loader2=None, store_on_device=True, gather_type=_MASTER):
    """Blocks (upper triangle only when symmetric) are dealt out to the ranks in contiguous runs;
    ``gather_type`` decides who ends up with what: the master, everybody, or - ``'split'`` - each
    rank the full n x n kernels of its own slice of classes."""
    device = next(iter(model.parameters())).device
    keep = device if store_on_device else 'cpu'
    if gather_type not in (_MASTER, _ALL, _SPLIT):
        raise ValueError(f'Invalid gather_type: {gather_type}. {[_MASTER, _ALL, _SPLIT]} are supported.')
    n1 = len(loader1)
    symmetric = loader2 is None
    if symmetric:
        loader2, n2 = loader1, n1
        pairs = [(i, j) for i in range(n1) for j in range(i, n1)]
    else:
        n2 = len(loader2)
        pairs = [(i, j) for i in range(n1) for j in range(n2)]
    rank, world_size = dist.get_rank(), dist.get_world_size()
    if len(pairs) < world_size:
        raise ValueError(f'At least 1 block have to be assigned to each process. '
                         f'There are only {len(pairs)} blocks for {world_size} processes.')
    shares = [list(map(tuple, s)) for s in np.array_split(np.array(pairs), world_size)]
    mine = shares[rank]
    sub1 = _subset_loader(loader1, [i for i, _ in mine])
    sub2 = _subset_loader(loader2, [j for _, j in mine])
    local = []
    for (i, j), b1, b2 in zip(mine, sub1, sub2):
        b1 = _inputs_of(b1).to(device)
        b2 = None if (symmetric and i == j) else _inputs_of(b2).to(device)
        local.append(kernel_fn(model, b1, b2).to(keep))
    local = torch.stack(local).to(device)
    pad = len(shares[0]) - len(mine)  # equal message sizes
    if pad > 0:
        local = torch.cat([local, local.new_zeros(pad, *local.shape[1:])])

    def build(per_rank_blocks):
        blocks = [[None] * n2 for _ in range(n1)]
        for rank_blocks, share in zip(per_rank_blocks, shares):
            for block, (i, j) in zip(rank_blocks, share):
                blocks[i][j] = block
        return _assemble(blocks, n1, n2, symmetric)

    if gather_type == _MASTER:
        gathered = _gather_to(local, 0, rank, world_size)
        return build(gathered) if gathered is not None else None
    if gather_type == _ALL:
        gathered = [torch.zeros_like(local) for _ in range(world_size)]
        dist.all_gather(gathered, local)
        return build(gathered)
    if local.ndim != 4:  # blocks x bs x bs x c
        raise ValueError(f'local_blocks.ndim has to be 4. Got {local.ndim}')
    n_classes = local.shape[-1]
    class_split = np.array_split(range(n_classes), world_size)
    received = None
    for dst, classes in enumerate(class_split):
        got = _gather_to(local[..., list(classes)].contiguous(), dst, rank, world_size)
        if got is not None:
            received = got
    if len(class_split[rank]) == 0:
        return None
    return torch.stack([build([blocks[..., k] for blocks in received])
                        for k in range(len(class_split[rank]))])  # local_c x n x n


# ----------------------------------------------------------------------------------------------
# empirical NTKs
# ----------------------------------------------------------------------------------------------
def empirical_direct_ntk(model, x1, x2=None, precond=None):
    """J1 J2^T from explicit per-example logit Jacobians: n1 x n2 x c x c.  With ``precond`` (a gradient maker
    with curvature) the kernel is J1 F^-1 J2^T: the second Jacobian's rows are preconditioned layer by layer."""
    n1 = x1.shape[0]
    inputs = x1 if x2 is None else torch.cat([x1, x2], dim=0)
    with extend(model, OP_BATCH_GRADS) as cxt:
        outputs = model(inputs)
        n_classes = outputs.shape[1]
        params = [p for p in model.parameters() if p.requires_grad]
        rows, right_rows = [], []
        for k in range(n_classes):
            cxt.clear_batch_grads()
            torch.autograd.grad(outputs[:, k].sum(), params, retain_graph=k < n_classes - 1,
                                allow_unused=True)
            parts = [cxt.batch_grads(m, flatten=True) for m in model.modules()]
            rows.append(torch.cat([p for p in parts if p is not None], dim=1))
            if precond is not None:
                for m in model.modules():
                    grads = cxt.batch_grads(m)
                    if grads is not None:   # in place on the stored per-example gradients
                        precond.precondition_module(m, vec_weight=grads.get('weight'), vec_bias=grads.get('bias'))
                parts = [cxt.batch_grads(m, flatten=True) for m in model.modules()]
                right_rows.append(torch.cat([p for p in parts if p is not None], dim=1))
    jac = torch.stack(rows, dim=1)  # n x c x p
    j1 = jac[:n1]
    right = jac if precond is None else torch.stack(right_rows, dim=1)
    j2 = right[:n1] if x2 is None else right[n1:]
    return torch.einsum('ncp,mdp->nmcd', j1, j2)


def empirical_implicit_ntk(model, x1, x2=None, precond=None):
    """The same kernel without materialising Jacobians (vjp then jvp-by-double-backward), with an
    optional preconditioner applied between the two Jacobians."""
    params = list(model.parameters())
    y1 = model(x1)
    n1, n_classes = y1.shape
    v1 = torch.ones_like(y1).requires_grad_()
    vjp1 = torch.autograd.grad(y1, params, v1, create_graph=True)
    mid = [v.clone() for v in vjp1]
    if precond is not None:
        precond.precondition_vector(mid)
    if x2 is None:
        n2 = n1
        ntk_dot_v = torch.autograd.grad(vjp1, v1, mid, create_graph=True)[0]
    else:
        n2 = x2.shape[0]
        y2 = model(x2)
        v2 = torch.ones_like(y2).requires_grad_()
        vjp2 = torch.autograd.grad(y2, params, v2, create_graph=True)
        ntk_dot_v = torch.autograd.grad(vjp2, v2, mid, create_graph=True)[0]
    ntk = y1.new_zeros(n1, n2, n_classes, n_classes)
    for j in range(n2):
        for k in range(n_classes):
            last = j == n2 - 1 and k == n_classes - 1
            ntk[:, j, :, k] = torch.autograd.grad(ntk_dot_v[j][k], v1, retain_graph=not last)[0]
    return ntk


def get_preconditioned_kernel_fn(kernel_fn, precond):
    """``kernel_fn`` with its ``precond`` argument bound to a gradient maker whose ``precondition`` is applied to one side's Jacobian."""
    return partial(kernel_fn, precond=precond)


def empirical_class_wise_direct_ntk(model, x1, x2=None, precond=None):
    """Empirical NTK per output class, c x n1 x n2, from per-example gradients of each logit."""
    return _empirical_class_wise_ntk(model, x1, x2, hadamard=False, precond=precond)


def empirical_class_wise_hadamard_ntk(model, x1, x2=None, precond=None):
    """Empirical NTK per output class, c x n1 x n2, from layer-wise Hadamard products of input and output-gradient Gram matrices."""
    return _empirical_class_wise_ntk(model, x1, x2, hadamard=True, precond=precond)


def _empirical_class_wise_ntk(model, x1, x2=None, hadamard=False, precond=None):
    """Per-class kernels K_c = J_c J_c^T accumulated by the Gram hooks: n1 x n2 x c."""
    n1 = x1.shape[0]
    if x2 is None:
        inputs, n2 = x1, n1
    else:
        inputs, n2 = torch.cat([x1, x2], dim=0), x2.shape[0]
    modules = list(model.modules())
    for module in modules:
        module.gram_precond = precond
    try:
        with extend(model, OP_GRAM_HADAMARD if hadamard else OP_GRAM_DIRECT):
            _zero_kernel(model, n1, n2)
            outputs = model(inputs)
            n_classes = outputs.shape[-1]
            params = [p for p in model.parameters() if p.requires_grad]
            kernels = []
            for k in range(n_classes):
                torch.autograd.grad(outputs[:, k].sum(), params, retain_graph=k < n_classes - 1,
                                    allow_unused=True)
                kernels.append(model.kernel.detach().clone())
                _zero_kernel(model, n1, n2)
            _clear_kernel(model)
    finally:
        for module in modules:
            if hasattr(module, 'gram_precond'):
                delattr(module, 'gram_precond')
    return torch.stack(kernels, dim=-1)


# ----------------------------------------------------------------------------------------------
# function-space natural gradient for cross-entropy
# ----------------------------------------------------------------------------------------------
def logits_hessian_cross_entropy(logits):
    """diag(p) - p p^T per example: n x c x c."""
    probs = F.softmax(logits, dim=1)
    return torch.diag_embed(probs) - torch.einsum('ni,nj->nij', probs, probs)


def _add_value_to_diagonal(X, value):
    if X.ndim not in (2, 3):
        raise ValueError(f'X.ndim has to be 2 or 3. Got {X.ndim}.')
    return X + value * torch.eye(X.shape[-1], device=X.device, dtype=X.dtype)


def _cholesky_solve(A, b, eps=1e-8):
    """(A + eps*I)^-1 b, batched over leading dimensions of A."""
    chol = torch.linalg.cholesky(_add_value_to_diagonal(A, eps))
    vec = b.ndim < A.ndim
    out = torch.cholesky_solve(b.unsqueeze(-1) if vec else b, chol)
    return out.squeeze(-1) if vec else out


def logits_second_order_grad_cross_entropy(logits, targets, damping=1e-5):
    hessian = _add_value_to_diagonal(logits_hessian_cross_entropy(logits), damping)
    loss = F.cross_entropy(logits, targets, reduction='sum')
    grads = torch.autograd.grad(loss, logits, retain_graph=True)[0]
    return _cholesky_solve(hessian, grads, eps=0.)


def natural_gradient_cross_entropy(model, inputs, targets, kernel, damping=1e-5):
    """Exact natural gradient through the (n*c x n*c) system (H K / n + damping*I) v = g; the
    parameter-space gradient is obtained by back-propagating v.  ``kernel``: n x n x c (class-wise)
    or n x n x c x c."""
    outputs = model(inputs)
    n, c = outputs.shape
    hessian = logits_hessian_cross_entropy(outputs)
    if kernel.ndim == 3:
        mat = torch.einsum('ijd,icd->icjd', kernel, hessian)
    else:
        mat = torch.einsum('ice,ijed->icjd', hessian, kernel)
    mat = _add_value_to_diagonal(mat.reshape(n * c, n * c) / n, damping)
    model.zero_grad()
    loss = F.cross_entropy(outputs, targets)
    grads = torch.autograd.grad(loss, outputs, retain_graph=True)[0].flatten()
    v = torch.linalg.solve(mat, grads).reshape(n, c)
    torch.autograd.backward(outputs, grad_tensors=v)
    return loss


def efficient_natural_gradient_cross_entropy(model, inputs, targets, class_kernels, damping=1e-5):
    """Class-wise approximation: solve with the logits Hessian per example, then with the n x n
    kernel per class."""
    if class_kernels.ndim != 3:  # c x n x n
        raise ValueError(f'class_kernels.ndim has to be 3. Got {class_kernels.ndim}')
    model.zero_grad()
    outputs = model(inputs)
    v = logits_second_order_grad_cross_entropy(outputs, targets, damping)  # n x c
    v = _cholesky_solve(class_kernels, v.T).T
    torch.autograd.backward(outputs, grad_tensors=v)


def _exchange(chunks, rank, world_size):
    """All-to-all of equally shaped tensors (``chunks[d]`` goes to rank d)."""
    try:
        out = [torch.zeros_like(c) for c in chunks]
        dist.all_to_all(out, [c.contiguous() for c in chunks])
        return out
    except (RuntimeError, NotImplementedError):
        received = None
        for dst in range(world_size):
            got = _gather_to(chunks[dst].contiguous(), dst, rank, world_size)
            if got is not None:
                received = got
        return received


def parallel_efficient_natural_gradient_cross_entropy(model, inputs, targets, local_class_kernels,
                                                      damping=1e-5):
    """Data-parallel logits solve -> all-to-all to class-parallel -> per-class kernel solve ->
    all-to-all back -> backward -> all-reduce of the parameter gradient."""
    rank, world_size = dist.get_rank(), dist.get_world_size()
    local_n = inputs.shape[0]
    outputs = model(inputs)
    n_classes = outputs.shape[-1]
    v = logits_second_order_grad_cross_entropy(outputs, targets, damping)  # local_n x c
    class_split = [list(s) for s in np.array_split(range(n_classes), world_size)]
    width = len(class_split[0])

    def padded(t, cols):  # local_n x len(cols) -> local_n x width
        out = t.new_zeros(t.shape[0], width)
        out[:, :len(cols)] = t[:, cols]
        return out

    received = _exchange([padded(v, cols) for cols in class_split], rank, world_size)
    mine = class_split[rank]
    if mine:
        if local_class_kernels is None:
            raise ValueError('local_class_kernels is not set.')
        if local_class_kernels.ndim != 3:
            raise ValueError(f'local_class_kernels.ndim has to be 3. Got {local_class_kernels.ndim}.')
        local_c, n, _ = local_class_kernels.shape
        if n != local_n * world_size:
            raise ValueError(f'n ({n}) does not match local_n * world_size ({local_n * world_size}).')
        stacked = torch.cat(received)[:, :local_c].T  # local_c x n
        solved = _cholesky_solve(local_class_kernels, stacked)  # local_c x n
        full = solved.new_zeros(width, n)
        full[:local_c] = solved
    else:
        full = inputs.new_zeros(width, local_n * world_size)
    back = _exchange([full[:, d * local_n:(d + 1) * local_n] for d in range(world_size)], rank, world_size)
    v = torch.cat([chunk[:len(cols)] for chunk, cols in zip(back, class_split) if cols]).T  # local_n x c
    model.zero_grad()
    torch.autograd.backward(outputs, grad_tensors=v.contiguous())
    params = [p for p in model.parameters() if p.requires_grad]
    for p, g in zip(params, _all_reduce_tensor_list([p.grad for p in params])):
        p.grad.copy_(g)


def empirical_natural_gradient(model, inputs, targets, loss_fn=F.cross_entropy, damping=1e-5,
                               data_average=True):
    """(F_emp + damping*I)^-1 grad by Woodbury with the Hadamard-Gram hooks; leaves the result in
    ``param.grad`` and returns the loss."""
    n = inputs.shape[0]
    with extend(model, OP_GRAM_HADAMARD):
        _zero_kernel(model, n, n)
        outputs = model(inputs)
        batch_loss = loss_fn(outputs, targets, reduction='none')
        params = [p for p in model.parameters() if p.requires_grad]
        torch.autograd.grad(batch_loss.sum(), params, retain_graph=True)
    from .precondition.smw import woodbury_example_weights
    batch_loss.backward(gradient=woodbury_example_weights(model.kernel, damping, data_average))
    return batch_loss.mean() if data_average else batch_loss.sum()


def empirical_natural_gradient2(model, inputs, targets, loss_fn=F.cross_entropy, damping=1e-5,
                                data_average=True):
    """Same quantity from saved inputs / output-gradients (no second backward pass)."""
    n = inputs.shape[0]
    with save_inputs_outgrads(model) as cxt:
        outputs = model(inputs)
        loss = loss_fn(outputs, targets, reduction='sum')
        with skip_param_grad(model):
            loss.backward()
        empirical_natural_gradient_by_context(cxt, damping, n if data_average else None)
    return loss.detach() / n if data_average else loss.detach()


def empirical_natural_gradient_by_context(cxt: OperationContext, damping=1e-5, data_average_n=None):
    """Re-weights every example by (1 - b)/damping with (K + damping*I) b = K 1 and rebuilds the
    parameter gradients from the saved tensors of ``cxt`` (sum-reduced output-gradients)."""
    from .precondition.smw import woodbury_example_weights
    gram = cxt.calc_kernel()
    if data_average_n and data_average_n != gram.shape[0]:
        raise ValueError(f'data_average_n ({data_average_n}) has to be the batch size ({gram.shape[0]}).')
    cxt.calc_grads(woodbury_example_weights(gram, damping, bool(data_average_n)))


def kernel_vector_product(model, inputs, vec):
    """J J^T vec."""
    outputs = model(inputs)
    vec = vec.detach().requires_grad_(True)
    params = list(model.parameters())
    vjp = torch.autograd.grad(outputs, params, grad_outputs=vec, create_graph=True)
    return torch.autograd.grad(vjp, vec, grad_outputs=[v.detach() for v in vjp])[0]


def _dist_sum(t, is_distributed):
    if is_distributed:
        dist.all_reduce(t)
    return t


def kernel_free_cross_entropy(model, inputs, targets, damping=1e-5, tol=1e-3, max_iters=None,
                              is_distributed=False, print_progress=False):
    """Function-space natural gradient by conjugate gradients on (H J J^T / n + damping*I) x = g
    without forming the kernel; the result is back-propagated into ``param.grad``."""
    outputs = model(inputs)
    n_data, n_classes = outputs.shape
    if is_distributed:
        n_data *= dist.get_world_size()
    if max_iters is None:
        max_iters = n_data * n_classes
    params = list(model.parameters())
    hessian = logits_hessian_cross_entropy(outputs)
    loss = F.cross_entropy(outputs, targets, reduction='sum').div(n_data)
    grads = torch.autograd.grad(loss, outputs, retain_graph=True)[0]
    g_norm = torch.sqrt(_dist_sum(grads.square().sum(), is_distributed))
    x = torch.zeros_like(outputs)
    p = grads.clone().requires_grad_(True)
    r = grads.clone()
    rr = _dist_sum(r.square().sum(), is_distributed)
    for i in range(max_iters):
        vjp = torch.autograd.grad(outputs, params, grad_outputs=p, retain_graph=True, create_graph=True)
        g = [t.detach().clone() for t in vjp]
        if is_distributed:
            g = _all_reduce_tensor_list(g)
        kvp = torch.autograd.grad(vjp, p, grad_outputs=g)[0]
        u = torch.einsum('nij,nj->ni', hessian, kvp).div(n_data).add_(p.detach(), alpha=damping)
        alpha = (rr / _dist_sum((p.detach() * u).sum(), is_distributed)).item()
        x.add_(p.detach(), alpha=alpha)
        r.sub_(u, alpha=alpha)
        new_rr = _dist_sum(r.square().sum(), is_distributed)
        err = new_rr.sqrt() / g_norm
        if print_progress:
            print(f'{i+1}/{max_iters} err={err}')
        if err < tol:
            break
        p = r.add(p.detach(), alpha=(new_rr / rr).item()).requires_grad_(True)
        rr = new_rr
    model.zero_grad()
    torch.autograd.backward(outputs, grad_tensors=x)
    if is_distributed:
        trainable = [q for q in model.parameters() if q.requires_grad]
        for q, g in zip(trainable, _all_reduce_tensor_list([q.grad for q in trainable])):
            q.grad.copy_(g)


def kernel_eigenvalues(model, inputs, top_n=1, max_iters=100, tol=1e-3, eps=1e-6, eigenvectors=False,
                       cross_entropy=False, is_distributed=False, gather_type=_ALL, print_progress=False):
    """Top eigenvalues of J J^T (or H J J^T with ``cross_entropy``) by deflated power iteration
    in function space."""
    if top_n < 1:
        raise ValueError(f'top_n has to be >= 1. Got {top_n}.')
    if max_iters < 1:
        raise ValueError(f'max_inters has to be >=1. Got {max_iters}.')
    params = list(model.parameters())
    outputs = model(inputs)
    hessian = logits_hessian_cross_entropy(outputs) if cross_entropy else None
    eigvals, eigvecs = [], []
    for i in range(top_n):
        if print_progress:
            print(f'start power iteration for lambda({i+1}).')
        vec = torch.randn_like(outputs)
        eigval = last = None
        for j in range(max_iters):
            vec = vec.detach()
            for v in eigvecs:
                vec = vec - v * _dist_sum((vec * v).sum(), is_distributed)
            vec = vec / torch.sqrt(_dist_sum(vec.square().sum(), is_distributed))
            vec.requires_grad_(True)
            vjp = torch.autograd.grad(outputs, params, grad_outputs=vec, create_graph=True)
            g = [t.detach().clone() for t in vjp]
            if is_distributed:
                g = _all_reduce_tensor_list(g)
            kvp = torch.autograd.grad(vjp, vec, grad_outputs=g, retain_graph=True)[0]
            if cross_entropy:
                kvp = torch.einsum('nij,nj->ni', hessian, kvp)
            eigval = _dist_sum((kvp * vec.detach()).sum(), is_distributed)
            if j > 0:
                diff = abs(eigval - last) / (abs(last) + eps)
                if print_progress:
                    print(f'{j}/{max_iters} diff={diff}')
                if diff < tol:
                    break
            last = eigval
            vec = kvp
        eigvals.append(eigval)
        eigvecs.append(vec.detach())
    order = sorted(range(top_n), key=lambda k: float(eigvals[k]), reverse=True)
    eigvals = [eigvals[k] for k in order]
    eigvecs = [eigvecs[k] for k in order]
    if not eigenvectors:
        return eigvals
    if is_distributed:
        world_size, rank = dist.get_world_size(), dist.get_rank()
        for i, v in enumerate(eigvecs):
            if gather_type == _MASTER:
                got = _gather_to(v, 0, rank, world_size)
            elif gather_type == _ALL:
                got = [torch.zeros_like(v) for _ in range(world_size)]
                dist.all_gather(got, v)
            else:
                raise ValueError(f'Invalid gather type {gather_type}.')
            if got is not None:
                eigvecs[i] = torch.cat([t.flatten() for t in got])
    return eigvals, eigvecs


def _all_reduce_tensor_list(tensor_list):
    packed = torch.cat([t.detach().reshape(-1) for t in tensor_list])
    dist.all_reduce(packed)
    out, offset = [], 0
    for t in tensor_list:
        out.append(packed[offset:offset + t.numel()].clone().reshape(t.shape))
        offset += t.numel()
    return out


def _zero_kernel(model, n_data1, n_data2):
    p = next(iter(model.parameters()))
    model.kernel = torch.zeros(n_data1, n_data2, device=p.device, dtype=p.dtype)


def _clear_kernel(model):
    if hasattr(model, 'kernel'):
        delattr(model, 'kernel')
