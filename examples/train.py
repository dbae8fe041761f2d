"""Train a small classifier with any gradient maker of the library.

    python examples/train.py --optim kfac --model cnn --dataset synthetic --epochs 2
    python examples/train.py --config examples/configs/cnn_shampoo.json
    python examples/train.py --optim kron_psgd --dataset mnist --data-root /data      # needs the files on disk

The training loop is the same for every method: the gradient maker replaces
``loss = F.cross_entropy(model(x), t); loss.backward()`` and leaves the (preconditioned) gradient in
``param.grad`` for a first-order optimizer to apply.  Prints per-epoch loss / accuracy and, at the
end, the average step time and the peak device memory.

Covers the use cases of the reference's examples/train.py, examples/train_cpu.py and
examples/arxiv_results/train.py (one script; JSON files override the command line; no logging
service).
"""
import argparse
import json
import os
import sys
import time

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402
from asdl_b200.models import resnet_tiny, vit_tiny  # noqa: E402

OPTIMS = ['sgd', 'adam', 'kfac', 'kfac_fused', 'ekfac', 'unit_wise', 'diag', 'shampoo', 'smw_ngd', 'full_psgd',
          'kron_psgd', 'kbfgs', 'seng', 'newton', 'curve_ball']


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--config', default=None, help='JSON file whose keys override the command line')
    ap.add_argument('--optim', default='kfac', choices=OPTIMS)
    ap.add_argument('--model', default='mlp', choices=['mlp', 'cnn', 'resnet_tiny', 'vit_tiny'])
    ap.add_argument('--dataset', default='synthetic', choices=['synthetic', 'mnist', 'cifar10'])
    ap.add_argument('--data-root', default='./data')
    ap.add_argument('--batch-size', type=int, default=128)
    ap.add_argument('--epochs', type=int, default=2)
    ap.add_argument('--steps-per-epoch', type=int, default=50, help='synthetic data only')
    ap.add_argument('--lr', type=float, default=0.05)
    ap.add_argument('--momentum', type=float, default=0.9)
    ap.add_argument('--weight-decay', type=float, default=0.0)
    ap.add_argument('--damping', type=float, default=1e-3)
    ap.add_argument('--ema-decay', type=float, default=-1)
    ap.add_argument('--curvature-upd-interval', type=int, default=1)
    ap.add_argument('--preconditioner-upd-interval', type=int, default=1)
    ap.add_argument('--block-size', type=int, default=128, help='Shampoo block size')
    ap.add_argument('--clip-grad-norm', type=float, default=1.0)
    ap.add_argument('--bf16', action='store_true', help='bf16 autocast')
    ap.add_argument('--cuda-graph', action='store_true', help='kfac_fused: replay steps from CUDA graphs')
    ap.add_argument('--seed', type=int, default=1)
    ap.add_argument('--no-cuda', action='store_true')
    args = ap.parse_args()
    if args.config:
        with open(args.config) as f:
            for key, value in json.load(f).items():
                if not hasattr(args, key):
                    raise KeyError(f'unknown option {key} in {args.config}')
                setattr(args, key, value)
    return args


def make_model(name, in_shape, classes):
    c, h, w = in_shape
    if name == 'mlp':
        return nn.Sequential(nn.Flatten(), nn.Linear(c * h * w, 256), nn.ReLU(), nn.Linear(256, 256), nn.ReLU(),
                             nn.Linear(256, classes))
    if name == 'cnn':
        return nn.Sequential(nn.Conv2d(c, 32, 3, padding=1), nn.BatchNorm2d(32), nn.ReLU(), nn.MaxPool2d(2),
                             nn.Conv2d(32, 64, 3, padding=1), nn.BatchNorm2d(64), nn.ReLU(),
                             nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(64, classes))
    if name == 'resnet_tiny':
        from asdl_b200.models import ResNet
        return ResNet((1, 1, 1, 1), num_classes=classes, width=8, in_channels=c)
    return vit_tiny(classes, image_size=h)


def make_loaders(args, device):
    """(train batches, test batches, input shape, classes); each an iterable of (x, t) on CPU."""
    if args.dataset == 'synthetic':
        shape, classes = (3, 32, 32), 10
        g = torch.Generator().manual_seed(args.seed)
        teacher = torch.randn(classes, shape[0] * shape[1] * shape[2], generator=g) / 30

        def batches(count):
            out = []
            for _ in range(count):
                x = torch.randn(args.batch_size, *shape, generator=g)
                out.append((x, (x.flatten(1) @ teacher.T).argmax(dim=1)))  # learnable labels
            return out
        return batches(args.steps_per_epoch), batches(max(1, args.steps_per_epoch // 5)), shape, classes
    from torchvision import datasets, transforms
    if args.dataset == 'mnist':
        tf = transforms.Compose([transforms.ToTensor(), transforms.Normalize((0.1307,), (0.3081,))])
        cls, shape = datasets.MNIST, (1, 28, 28)
    else:
        tf = transforms.Compose([transforms.ToTensor(),
                                 transforms.Normalize((0.4914, 0.4822, 0.4465), (0.2470, 0.2435, 0.2616))])
        cls, shape = datasets.CIFAR10, (3, 32, 32)
    train = cls(args.data_root, train=True, download=False, transform=tf)
    test = cls(args.data_root, train=False, download=False, transform=tf)
    kw = dict(batch_size=args.batch_size, num_workers=2, pin_memory=device.type == 'cuda')
    return (torch.utils.data.DataLoader(train, shuffle=True, drop_last=True, **kw),
            torch.utils.data.DataLoader(test, **kw), shape, 10)


def make_grad_maker(args, model):
    name = args.optim
    if name in ('sgd', 'adam'):
        return asdl.GradientMaker(model)
    cfg = asdl.PreconditioningConfig(data_size=args.batch_size, damping=args.damping, ema_decay=args.ema_decay,
                                     curvature_upd_interval=args.curvature_upd_interval,
                                     preconditioner_upd_interval=args.preconditioner_upd_interval)
    if name == 'kfac':
        return asdl.KfacGradientMaker(model, cfg)
    if name == 'kfac_fused':
        return asdl.FusedKfacGradientMaker(model, cfg, cuda_graph=args.cuda_graph)
    if name == 'ekfac':
        return asdl.EkfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP)
    if name == 'unit_wise':
        return asdl.UnitWiseNaturalGradientMaker(model, cfg)
    if name == 'diag':
        return asdl.DiagNaturalGradientMaker(model, cfg)
    if name == 'shampoo':
        return asdl.ShampooGradientMaker(model, cfg, block_size=args.block_size)
    if name == 'smw_ngd':
        return asdl.SmwEmpNaturalGradientMaker(model, cfg)
    if name == 'full_psgd':
        return asdl.PsgdGradientMaker(model, cfg)
    if name == 'kron_psgd':
        return asdl.KronPsgdGradientMaker(model, cfg)
    if name == 'kbfgs':
        return asdl.KronBfgsGradientMaker(model, cfg)
    if name == 'seng':
        return asdl.SengGradientMaker(model, cfg)
    if name == 'newton':
        return asdl.NewtonGradientMaker(model, cfg)
    return asdl.CurveBallGradientMaker(model, cfg)


def main():
    args = parse_args()
    torch.manual_seed(args.seed)
    device = torch.device('cuda' if torch.cuda.is_available() and not args.no_cuda else 'cpu')
    train_batches, test_batches, shape, classes = make_loaders(args, device)
    model = make_model(args.model, shape, classes).to(device)
    if device.type == 'cuda' and args.model != 'mlp':
        model = model.to(memory_format=torch.channels_last)
    if args.optim == 'adam':
        optimizer = torch.optim.Adam(model.parameters(), lr=args.lr, weight_decay=args.weight_decay)
    else:
        optimizer = torch.optim.SGD(model.parameters(), lr=args.lr, momentum=args.momentum,
                                    weight_decay=args.weight_decay)
    grad_maker = make_grad_maker(args, model)

    def model_fn(x):
        with torch.autocast(device.type, dtype=torch.bfloat16, enabled=args.bf16):
            return model(x)

    def to_device(x, t):
        x = x.to(device, non_blocking=True)
        if x.ndim == 4 and device.type == 'cuda' and args.model != 'mlp':
            x = x.contiguous(memory_format=torch.channels_last)
        return x, t.to(device, non_blocking=True)

    steps, train_time = 0, 0.0
    for epoch in range(1, args.epochs + 1):
        model.train()
        if device.type == 'cuda':
            torch.cuda.synchronize()
        start = time.time()
        running = 0.0
        for x, t in train_batches:
            x, t = to_device(x, t)
            optimizer.zero_grad(set_to_none=False)
            dummy_y = grad_maker.setup_model_call(model_fn, x)
            grad_maker.setup_loss_call(F.cross_entropy, dummy_y, t)
            _, loss = grad_maker.forward_and_backward()
            if args.clip_grad_norm > 0:
                torch.nn.utils.clip_grad_norm_(model.parameters(), args.clip_grad_norm)
            optimizer.step()
            running += float(loss)
            steps += 1
        if device.type == 'cuda':
            torch.cuda.synchronize()
        train_time += time.time() - start
        model.eval()
        correct = total = 0
        with torch.no_grad():
            for x, t in test_batches:
                x, t = to_device(x, t)
                correct += (model_fn(x).argmax(dim=1) == t).sum().item()
                total += t.numel()
        print(f'epoch {epoch}: train loss {running / len(train_batches):.4f}  test acc {100 * correct / total:.2f}%')
    print(f'total_train_time: {train_time:.2f}s')
    print(f'avg_step_time: {1000 * train_time / max(steps, 1):.2f}ms')
    if device.type == 'cuda':
        print(f'cuda_max_memory: {torch.cuda.max_memory_allocated() / 2 ** 20:.1f}MiB')
        asdl.ops.check_status()


if __name__ == '__main__':
    main()
