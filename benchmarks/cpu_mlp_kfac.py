"""CPU K-FAC on an MLP: time per step and agreement with the dense oracle.

    python benchmarks/cpu_mlp_kfac.py [--impl reference]

MLP 784-512-512-10 (ReLU, bias, fp32), batch 128 of N(0,1) inputs with uniform labels, cross-entropy,
``KfacGradientMaker(damping=0.01, data_size=128)`` with curvature and inverses refreshed every step, SGD
lr 0.01, 20 steps.  Prints one JSON line: mean ms/step (after 3 warm-up steps), first / last loss, and the
relative error of the preconditioned weight gradients of the first step against
``(B + d_B I)^-1 grad_W (A + d_A I)^-1`` and ``(B + d_B I)^-1 grad_b`` formed densely in float64 from the
same factors (pi-split damping).
``--impl reference`` runs the reference package from baseline/_ref through the same loop;
``--optim shampoo | kron_psgd | kbfgs | seng`` times another method on the same network (no oracle).
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference', 'fused'])
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--optim', default='kfac', choices=['kfac', 'shampoo', 'kron_psgd', 'kbfgs', 'seng'],
                    help='kfac (default, with the dense-oracle check) or another method on the same network (time only)')
    args = ap.parse_args()
    if args.impl == 'reference':
        sys.path.insert(0, os.path.join(ROOT, 'baseline', '_ref'))
        import asdl
    else:
        sys.path.insert(0, ROOT)
        import asdl_b200 as asdl
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(784, 512), nn.ReLU(), nn.Linear(512, 512), nn.ReLU(), nn.Linear(512, 10))
    x, t = torch.randn(128, 784), torch.randint(0, 10, (128,))
    config = asdl.PreconditioningConfig(data_size=128, damping=0.01)
    if args.optim == 'kfac':
        maker_cls = asdl.FusedKfacGradientMaker if args.impl == 'fused' else asdl.KfacGradientMaker
        gm = maker_cls(model, config, fisher_type='fisher_emp')
    elif args.optim == 'shampoo':
        gm = asdl.ShampooGradientMaker(model, asdl.PreconditioningConfig(damping=1e-6))
    elif args.optim == 'kron_psgd':
        gm = asdl.KronPsgdGradientMaker(model, asdl.PreconditioningConfig())
    elif args.optim == 'kbfgs':
        gm = asdl.KronBfgsGradientMaker(model, asdl.PreconditioningConfig(data_size=128, damping=0.01, ema_decay=0.1))
    else:
        gm = asdl.SengGradientMaker(model, asdl.PreconditioningConfig(data_size=128, damping=0.1))
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    losses, times, oracle_err = [], [], None
    for step in range(args.steps + 3):
        opt.zero_grad(set_to_none=True)
        t0 = time.perf_counter()
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        _, loss = gm.forward_and_backward()
        times.append(time.perf_counter() - t0)
        if step == 0 and args.optim == 'kfac':   # dense oracle from plain autograd quantities
            errs = []
            linears = [m for m in model if isinstance(m, nn.Linear)]
            have = [torch.cat([m.weight.grad, m.bias.grad.unsqueeze(1)], dim=1).double() for m in linears]
            acts, h = [], x
            for layer in model:
                if isinstance(layer, nn.Linear):
                    acts.append(h)
                h = layer(h)
            outs = []
            h = x
            for layer in model:
                h = layer(h)
                if isinstance(layer, nn.Linear):
                    h.retain_grad()
                    outs.append(h)
            F.cross_entropy(h, t, reduction='sum').backward()
            for got, a, o in zip(have, acts, outs):
                a, g = a.detach(), o.grad
                A, B = a.T @ a / 128, g.T @ g / 128
                pi = torch.sqrt((A.trace() / A.shape[0]) / (B.trace() / B.shape[0]))
                root = 0.01 ** 0.5
                Ai = torch.linalg.inv(A.double() + root * pi * torch.eye(A.shape[0], dtype=torch.double))
                Bi = torch.linalg.inv(B.double() + root / pi * torch.eye(B.shape[0], dtype=torch.double))
                want = torch.cat([Bi @ (g.T @ a / 128).double() @ Ai, Bi @ g.sum(0, keepdim=True).T.double() / 128], dim=1)
                errs.append(((got - want).norm() / want.norm()).item())
            oracle_err = max(errs)
            for m, g in zip(linears, have):   # put the preconditioned gradients back for the optimizer
                m.weight.grad, m.bias.grad = g[:, :-1].float().contiguous(), g[:, -1].float().contiguous()
        opt.step()
        losses.append(float(loss.detach()))
    print(json.dumps({'case': 'cpu_mlp_' + args.optim, 'impl': args.impl, 'threads': torch.get_num_threads(),
                      'ms_per_step': round(1e3 * sum(times[3:]) / len(times[3:]), 2), 'first_loss': round(losses[0], 4),
                      'last_loss': round(losses[-1], 4), 'max_rel_err_vs_dense_oracle': oracle_err}))


if __name__ == '__main__':
    main()
