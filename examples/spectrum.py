"""Top eigenvalues and eigenvalue spectral density of the Fisher / Hessian of a small classifier.

    python examples/spectrum.py --matrix fisher_emp --top-n 5
    python examples/spectrum.py --matrix hessian --esd

Matrix-free: power iteration (deflated) and stochastic Lanczos quadrature on Fisher- / Hessian-vector
products.  Covers the use cases of the reference's examples/eigenvalues.py and examples/esd.py.
"""
import argparse
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--matrix', default='fisher_emp', choices=['fisher_emp', 'fisher_mc', 'fisher_exact', 'hessian'])
    ap.add_argument('--top-n', type=int, default=3)
    ap.add_argument('--esd', action='store_true', help='also estimate the spectral density')
    ap.add_argument('--batch-size', type=int, default=64)
    args = ap.parse_args()
    torch.manual_seed(0)
    device = 'cuda' if torch.cuda.is_available() else 'cpu'
    model = nn.Sequential(nn.Flatten(), nn.Linear(3 * 16 * 16, 64), nn.ReLU(), nn.Linear(64, 10)).to(device)
    x = torch.randn(args.batch_size, 3, 16, 16, device=device)
    t = torch.randint(0, 10, (args.batch_size,), device=device)
    if args.matrix == 'hessian':
        maker = asdl.HessianMaker(model, asdl.HessianConfig(hessian_shapes=[]))
        eig, esd = maker.hessian_eig, getattr(maker, 'hessian_esd', None)
    else:
        maker = asdl.get_fisher_maker(model, asdl.FisherConfig(fisher_type=args.matrix, fisher_shapes=[asdl.SHAPE_FULL],
                                                               loss_type=asdl.LOSS_CROSS_ENTROPY,
                                                               data_size=args.batch_size))
        eig, esd = maker.fisher_eig, maker.fisher_esd
    dummy_y = maker.setup_model_call(model, x)
    maker.setup_loss_call(F.cross_entropy, dummy_y, t)
    eigvals, _ = eig(top_n=args.top_n, max_iters=200, tol=1e-5)
    print(f'top {args.top_n} eigenvalues of the {args.matrix}: ' + ', '.join(f'{v:.5g}' for v in eigvals))
    if args.esd and esd is not None:
        density, grid = esd(n_v=2, num_iter=40, num_bins=200)
        peak = int(density.argmax())
        print(f'spectral density on [{grid[0]:.4g}, {grid[-1]:.4g}]: peak at {grid[peak]:.4g}, '
              f'mass above half of the largest eigenvalue: '
              f'{float(density[grid > 0.5 * max(eigvals)].sum() / density.sum()):.4f}')


if __name__ == '__main__':
    main()
