"""ResNet-50 with K-FAC, single GPU or data parallel (one process per GPU).

    python examples/train_resnet50_with_kfac.py --steps 50
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        examples/train_resnet50_with_kfac.py --data-dir /data/imagenet --epochs 40

The recipe of the reference's examples/train_resnet50_with_kfac.py: batch 32 per GPU, SGD with momentum 0.9,
lr 0.1 with linear warm-up and polynomial decay, weight decay 5e-5, damping 1e-3, curvature every 10 steps,
inverses every 100 steps, moving-average weight 0.05, KL clipping 1e-3.  Without ``--data-dir`` it trains on
synthetic images (there is no dataset on this machine), which exercises the whole step:
``FusedKfacGradientMaker`` with CUDA-graph replay, bf16 autocast, channels_last, and the NVLink
symmetric-memory transport when several ranks run.
"""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402
from asdl_b200.models import resnet50, resnet_tiny  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--data-dir', default=None, help='ImageFolder root with train/ (synthetic data if omitted)')
    ap.add_argument('--batch-size', type=int, default=32, help='per GPU')
    ap.add_argument('--epochs', type=int, default=1)
    ap.add_argument('--steps', type=int, default=None, help='stop after this many steps')
    ap.add_argument('--lr', type=float, default=0.1)
    ap.add_argument('--warmup-steps', type=int, default=500)
    ap.add_argument('--momentum', type=float, default=0.9)
    ap.add_argument('--weight-decay', type=float, default=5e-5)
    ap.add_argument('--damping', type=float, default=1e-3)
    ap.add_argument('--cov-update-freq', type=int, default=10)
    ap.add_argument('--inv-update-freq', type=int, default=100)
    ap.add_argument('--ema-decay', type=float, default=0.05)
    ap.add_argument('--kl-clip', type=float, default=1e-3)
    ap.add_argument('--no-graph', action='store_true')
    ap.add_argument('--cpu-smoke', action='store_true',
                    help='run the same loop on the CPU with the tiny bottleneck ResNet and 32 x 32 images (checks the script)')
    return ap.parse_args()


def synthetic_batches(batch_size, count, seed, side=224, classes=1000, pin=True):
    g = torch.Generator().manual_seed(seed)
    data = []
    for _ in range(8):
        x = torch.randn(batch_size, 3, side, side, generator=g).contiguous(memory_format=torch.channels_last)
        t = torch.randint(0, classes, (batch_size,), generator=g)
        data.append((x.pin_memory(), t.pin_memory()) if pin else (x, t))
    for i in range(count):
        yield data[i % len(data)]


def main():
    args = parse_args()
    rank, local, world = (int(os.environ.get(k, d)) for k, d in (('RANK', 0), ('LOCAL_RANK', 0), ('WORLD_SIZE', 1)))
    cuda = not args.cpu_smoke
    if cuda and not torch.cuda.is_available():
        raise SystemExit('this example needs a CUDA device (or --cpu-smoke)')
    if cuda:
        torch.cuda.set_device(local)
    device = torch.device('cuda', local) if cuda else torch.device('cpu')
    if world > 1:
        dist.init_process_group('nccl', device_id=device) if cuda else dist.init_process_group('gloo')
    torch.manual_seed(0)
    model = (resnet50() if cuda else resnet_tiny()).to(device).to(memory_format=torch.channels_last)
    config = asdl.PreconditioningConfig(data_size=args.batch_size, damping=args.damping, ema_decay=args.ema_decay,
                                        curvature_upd_interval=args.cov_update_freq,
                                        preconditioner_upd_interval=args.inv_update_freq)
    grad_maker = asdl.FusedKfacGradientMaker(model, config, cuda_graph=cuda and not args.no_graph)
    decay, no_decay = [], []
    for p in model.parameters():
        (decay if p.ndim > 1 else no_decay).append(p)
    optimizer = torch.optim.SGD([{'params': decay, 'weight_decay': args.weight_decay},
                                 {'params': no_decay, 'weight_decay': 0.0}], lr=args.lr, momentum=args.momentum)
    if args.data_dir:
        from torchvision import datasets, transforms
        tf = transforms.Compose([transforms.RandomResizedCrop(224), transforms.RandomHorizontalFlip(), transforms.ToTensor(),
                                 transforms.Normalize((0.485, 0.456, 0.406), (0.229, 0.224, 0.225))])
        dataset = datasets.ImageFolder(os.path.join(args.data_dir, 'train'), tf)
        sampler = torch.utils.data.distributed.DistributedSampler(dataset) if world > 1 else None
        loader = torch.utils.data.DataLoader(dataset, batch_size=args.batch_size, shuffle=sampler is None, sampler=sampler,
                                             num_workers=8, pin_memory=True, drop_last=True)
        steps_per_epoch = len(loader)
    else:
        steps_per_epoch = args.steps or 200
        loader = None
    total_steps = args.steps or args.epochs * steps_per_epoch

    def model_fn(x):
        with torch.autocast(device.type, dtype=torch.bfloat16, enabled=cuda):
            return model(x)

    step, t0 = 0, time.time()
    for epoch in range(args.epochs):
        batches = loader if loader is not None else synthetic_batches(
            args.batch_size, steps_per_epoch, seed=rank, side=224 if cuda else 32, classes=1000 if cuda else 10, pin=cuda)
        if loader is not None and world > 1:
            loader.sampler.set_epoch(epoch)
        for x, t in batches:
            if step >= total_steps:
                break
            lr = args.lr * min(1.0, (step + 1) / args.warmup_steps) * (1 - step / total_steps) ** 2
            for group in optimizer.param_groups:
                group['lr'] = lr
            x = x.to(device, non_blocking=True).contiguous(memory_format=torch.channels_last)
            t = t.to(device, non_blocking=True)
            optimizer.zero_grad(set_to_none=True)
            dummy_y = grad_maker.setup_model_call(model_fn, x)
            grad_maker.setup_loss_call(F.cross_entropy, dummy_y, t)
            _, loss = grad_maker.forward_and_backward()
            if args.kl_clip > 0:   # scale the step so that lr^2 * g_prec . g_prec stays below the KL bound
                grads = [p.grad for p in model.parameters() if p.grad is not None]
                sq = torch.stack([(g.float() ** 2).sum() for g in grads]).sum()
                nu = torch.clamp(torch.sqrt(args.kl_clip / (lr * lr * sq + 1e-30)), max=1.0)
                torch._foreach_mul_(grads, nu)
            optimizer.step()
            step += 1
            if rank == 0 and (step % 50 == 0 or step == total_steps):
                if cuda:
                    torch.cuda.synchronize()
                rate = step * args.batch_size * world / (time.time() - t0)
                print(f'step {step}/{total_steps} lr {lr:.4f} loss {float(loss.detach()):.4f} {rate:.0f} images/s', flush=True)
    if cuda:
        asdl.ops.check_status()
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
