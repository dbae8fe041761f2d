"""Optimal-Brain-Surgeon style pruning with a Kronecker-factored inverse Fisher.

    python examples/one_shot_pruning.py --sparsity 0.8

A small classifier is trained on a synthetic task, then pruned in a few rounds.  Every round
  1. estimates the empirical Fisher in K-FAC form and inverts it (``FisherMaker`` with
     ``fisher_shapes=[SHAPE_KRON]``, ``calc_inv=True``),
  2. scores every weight by the loss increase of removing it, ``w^2 / (2 [F^-1]_ww)`` with the
     diagonal of the Kronecker inverse ``diag(B^-1) x diag(A^-1)``,
  3. removes the lowest-scoring weights up to the scheduled sparsity, and
  4. moves the surviving weights along ``-F^-1 v`` (``v`` = removed weights over their inverse
     diagonal), which compensates the removal to second order.
Magnitude pruning at the same sparsity is printed for comparison.
Role of the reference's examples/one_shot_pruning.py.
"""
import argparse
import copy
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402


def accuracy(model, x, t):
    with torch.no_grad():
        return (model(x).argmax(dim=1) == t).float().mean().item()


def prune_with_fisher(model, x, t, sparsity, rounds, damping):
    layers = [m for m in model.modules() if isinstance(m, nn.Linear)]
    masks = {m: torch.ones_like(m.weight, dtype=torch.bool) for m in layers}
    total = sum(m.weight.numel() for m in layers)
    config = asdl.FisherConfig(fisher_type=asdl.FISHER_EMP, fisher_shapes=[asdl.SHAPE_KRON],
                               loss_type=asdl.LOSS_CROSS_ENTROPY, data_size=x.shape[0])
    for r in range(1, rounds + 1):
        target = sparsity * (1 - (1 - r / rounds) ** 3)              # polynomial schedule
        for m in layers:
            if hasattr(m, 'fisher'):
                delattr(m, 'fisher')
        maker = asdl.get_fisher_maker(model, config)
        dummy_y = maker.setup_model_call(model, x)
        maker.setup_loss_call(F.cross_entropy, dummy_y, t)
        maker.forward_and_backward(calc_inv=True, damping=damping)
        scores, inv_diags = [], {}
        for m in layers:
            kron = m.fisher.kron
            inv_diag = torch.outer(torch.diagonal(kron.B_inv), torch.diagonal(kron.A_inv))
            inv_diags[m] = inv_diag
            score = m.weight.detach() ** 2 / (2 * inv_diag)
            scores.append(torch.where(masks[m], score, torch.full_like(score, float('inf'))).flatten())
        already = total - sum(int(mask.sum()) for mask in masks.values())
        n_new = int(target * total) - already
        if n_new <= 0:
            continue
        threshold = torch.cat(scores).kthvalue(n_new).values
        with torch.no_grad():
            for m, score in zip(layers, scores):
                drop = (score.view_as(m.weight) <= threshold) & masks[m]
                v = torch.where(drop, m.weight / inv_diags[m], torch.zeros_like(m.weight))
                bias_zero = torch.zeros_like(m.bias) if m.bias is not None else None
                m.fisher.kron.mvp(vec_weight=v, vec_bias=bias_zero, use_inv=True, inplace=True)  # v <- F^-1 v
                m.weight.sub_(v)
                masks[m] &= ~drop
                m.weight.mul_(masks[m])
    return 1 - sum(int(mask.sum()) for mask in masks.values()) / total


def prune_by_magnitude(model, sparsity):
    layers = [m for m in model.modules() if isinstance(m, nn.Linear)]
    flat = torch.cat([m.weight.detach().abs().flatten() for m in layers])
    threshold = flat.kthvalue(int(sparsity * flat.numel())).values
    with torch.no_grad():
        for m in layers:
            m.weight.mul_(m.weight.abs() > threshold)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--sparsity', type=float, default=0.8)
    ap.add_argument('--rounds', type=int, default=8)
    ap.add_argument('--damping', type=float, default=1e-3)
    args = ap.parse_args()
    torch.manual_seed(0)
    device = 'cuda' if torch.cuda.is_available() else 'cpu'
    n, d, classes = 2048, 32, 10
    teacher = torch.randn(classes, d)
    x = torch.randn(n, d)
    t = (x @ teacher.T).argmax(dim=1)
    x, t = x.to(device), t.to(device)
    model = nn.Sequential(nn.Linear(d, 64), nn.ReLU(), nn.Linear(64, 64), nn.ReLU(), nn.Linear(64, classes)).to(device)
    opt = torch.optim.Adam(model.parameters(), lr=3e-3)
    for _ in range(300):
        opt.zero_grad()
        F.cross_entropy(model(x), t).backward()
        opt.step()
    print(f'dense accuracy: {accuracy(model, x, t):.4f}')
    magnitude = copy.deepcopy(model)
    prune_by_magnitude(magnitude, args.sparsity)
    print(f'magnitude pruning to {args.sparsity:.0%}: accuracy {accuracy(magnitude, x, t):.4f}')
    reached = prune_with_fisher(model, x[:512], t[:512], args.sparsity, args.rounds, args.damping)
    print(f'K-FAC OBS pruning to {reached:.0%}: accuracy {accuracy(model, x, t):.4f}')


if __name__ == '__main__':
    main()
