"""K-FAC with large logical batches ("pseudo-batches") iterated in micro-batches.

    python examples/pseudo_batch_train.py --pseudo-batch-size 256 --batch-size 64

The curvature and the gradient of one optimizer step are accumulated over the micro-batches of a
pseudo-batch: every micro-batch calls ``forward_and_backward(accumulate=True)`` on a
``FisherMaker`` with ``scale = micro_batch / pseudo_batch`` (so the sums become averages over the
pseudo-batch); the factors are then inverted and the K-FAC preconditioner is applied once.
Role of the reference's examples/pseudo_batch_train.py.
"""
import argparse
import os
import sys

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--pseudo-batch-size', type=int, default=256)
    ap.add_argument('--batch-size', type=int, default=64)
    ap.add_argument('--epochs', type=int, default=2)
    ap.add_argument('--lr', type=float, default=0.05)
    ap.add_argument('--damping', type=float, default=1e-2)
    args = ap.parse_args()
    torch.manual_seed(0)
    device = 'cuda' if torch.cuda.is_available() else 'cpu'
    n = 4 * args.pseudo_batch_size
    x = torch.randn(n, 1, 16, 16)
    teacher = torch.randn(10, 256) / 8
    t = (x.flatten(1) @ teacher.T).argmax(dim=1)
    loader = DataLoader(TensorDataset(x, t), batch_size=args.batch_size, shuffle=True, drop_last=True)
    model = nn.Sequential(nn.Conv2d(1, 8, 3, padding=1), nn.ReLU(), nn.Flatten(), nn.Linear(8 * 256, 10)).to(device)
    optimizer = torch.optim.SGD(model.parameters(), lr=args.lr, momentum=0.9)
    fisher_cfg = asdl.FisherConfig(fisher_type=asdl.FISHER_EMP, fisher_shapes=[asdl.SHAPE_KRON],
                                   loss_type=asdl.LOSS_CROSS_ENTROPY)
    maker = asdl.get_fisher_maker(model, fisher_cfg)
    for epoch in range(1, args.epochs + 1):
        total, count = 0.0, 0
        for pb_loader in asdl.PseudoBatchLoaderGenerator(loader, args.pseudo_batch_size):
            optimizer.zero_grad(set_to_none=True)
            for module in model.modules():      # a fresh curvature estimate per pseudo-batch
                if hasattr(module, 'fisher'):
                    delattr(module, 'fisher')
            micro = list(pb_loader)
            for i, (xb, tb) in enumerate(micro):
                xb, tb = xb.to(device), tb.to(device)
                dummy_y = maker.setup_model_call(model, xb)
                maker.setup_loss_call(F.cross_entropy, dummy_y, tb)
                _, loss = maker.forward_and_backward(data_size=args.pseudo_batch_size, accumulate=True,
                                                     calc_loss_grad=True)
                total += float(loss.detach()) * args.pseudo_batch_size   # the maker returns sum / data_size
                count += xb.shape[0]
            for module in model.modules():      # natural gradient = inverse Fisher times gradient
                fisher = getattr(module, 'fisher', None)
                if fisher is not None and fisher.kron is not None:
                    fisher.update_inv(args.damping)
                    fisher.kron.mvp(vec_weight=module.weight.grad, vec_bias=module.bias.grad, use_inv=True, inplace=True)
            optimizer.step()
        print(f'epoch {epoch}: mean loss {total / count:.4f}')


if __name__ == '__main__':
    main()
