"""Train a small classifier with any gradient maker of the library.

    python examples/train.py --optim kfac --model cnn --dataset synthetic --epochs 2
    python examples/train.py --config examples/configs/cnn_shampoo.json
    python examples/train.py --recipe resnet18/kfac --data-root /data        # a paper run of the reference
    python examples/train.py --optim kron_psgd --dataset mnist --data-root /data      # needs the files on disk

The training loop is the same for every method: the gradient maker replaces
``loss = F.cross_entropy(model(x), t); loss.backward()`` and leaves the (preconditioned) gradient in
``param.grad`` for a first-order optimizer to apply.  Prints per-epoch loss / accuracy and, at the
end, the average step time and the peak device memory.

Covers the use cases of the reference's examples/train.py, examples/train_cpu.py and
examples/arxiv_results/train.py: one script; JSON files override the command line and may use the
reference's key names (``curvature_update_interval``, ``clipping_norm``, ``optim: kfac_mc`` ...);
train / validation split (``--train-size``), label smoothing, Nesterov momentum, AdamW, cosine
learning-rate decay, crop + flip / Cutout / AutoAugment, a stop on a non-finite loss, an
out-of-memory report instead of a traceback, and a JSON-lines log (``--log-json``) in place of a
logging service.  Crop, flip and Cutout run on the whole batch on the device (examples/augment.py).
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
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import asdl_b200 as asdl  # noqa: E402
from asdl_b200 import models  # noqa: E402
from augment import batch_cutout, batch_random_crop_flip  # noqa: E402

OPTIMS = ['sgd', 'adam', 'adamw', 'kfac', 'kfac_fused', 'ekfac', 'unit_wise', 'diag', 'shampoo', 'smw_ngd', 'full_psgd',
          'kron_psgd', 'kbfgs', 'seng', 'newton', 'curve_ball']
MODELS = ['mlp', 'cnn', 'resnet_tiny', 'vit_tiny', 'resnet18', 'resnet34', 'wideresnet28', 'wideresnet_tiny',
          'vit_tiny_patch16_224', 'mixer_b16_224', 'mixer_tiny']
#: key names of the reference's JSON files -> options of this script
ALIASES = {'curvature_update_interval': 'curvature_upd_interval', 'clipping_norm': 'clip_grad_norm',
           'auto_augment': 'auto_augment', 'data_augmentation': 'data_augmentation'}
OPTIM_ALIASES = {'kfac_mc': 'kfac', 'psgd': 'kron_psgd', 'smw_ng': 'smw_ngd'}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--config', default=None, help='JSON file whose keys override the command line')
    ap.add_argument('--recipe', default=None, metavar='FAMILY/METHOD',
                    help='entry of examples/configs/recipes.json (the paper runs of the reference), e.g. resnet18/kfac; '
                         'explicit command-line options still win')
    ap.add_argument('--optim', default='kfac', choices=OPTIMS)
    ap.add_argument('--model', default='mlp', choices=MODELS)
    ap.add_argument('--width', type=int, default=256, help='mlp: hidden units')
    ap.add_argument('--depth', type=int, default=3, help='mlp: number of linear layers')
    ap.add_argument('--dataset', default='synthetic', choices=['synthetic', 'mnist', 'cifar10'])
    ap.add_argument('--train-size', type=int, default=None,
                    help='real datasets: this many training samples, the rest of the training set validates')
    ap.add_argument('--data-augmentation', action='store_true', help='random crop + flip on the device')
    ap.add_argument('--cutout', action='store_true', help='Cutout on the device')
    ap.add_argument('--n-holes', type=int, default=1)
    ap.add_argument('--length', type=int, default=16)
    ap.add_argument('--auto-augment', action='store_true', help='real CIFAR-10 only: torchvision AutoAugment policy')
    ap.add_argument('--label-smoothing', type=float, default=0.0)
    ap.add_argument('--nesterov', action='store_true')
    ap.add_argument('--cosine', action='store_true', help='cosine learning-rate decay over the epochs')
    ap.add_argument('--ignore-norm-layers', action='store_true',
                    help='leave BatchNorm / LayerNorm parameters to the first-order optimizer')
    ap.add_argument('--log-interval', type=int, default=0, help='print the running loss every N steps')
    ap.add_argument('--log-json', default=None, help='append one JSON line per epoch and a summary line here')
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
    if args.recipe:
        family, method = args.recipe.split('/')
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'configs', 'recipes.json')) as f:
            table = json.load(f)[family]
        given = {a.lstrip('-').split('=')[0].replace('-', '_') for a in sys.argv[1:] if a.startswith('--')}
        for key, value in {**table['common'], **table[method]}.items():
            if key not in given:
                setattr(args, key, value)
    if args.config:
        with open(args.config) as f:
            for key, value in json.load(f).items():
                key = ALIASES.get(key, key)
                if not hasattr(args, key):
                    raise KeyError(f'unknown option {key} in {args.config}')
                setattr(args, key, value)
    args.dataset = args.dataset.lower()
    args.optim = OPTIM_ALIASES.get(args.optim, args.optim)
    if args.optim not in OPTIMS:
        raise KeyError(f'unknown optim {args.optim}')
    if args.curvature_upd_interval > 1 and args.preconditioner_upd_interval == 1:
        args.preconditioner_upd_interval = args.curvature_upd_interval  # the reference ties the two
    return args


def make_model(name, in_shape, classes, width=256, depth=3):
    c, h, w = in_shape
    if name == 'mlp':
        return models.MLP(width, depth, c * h * w, classes)
    if name == 'cnn':
        return nn.Sequential(nn.Conv2d(c, 32, 3, padding=1), nn.BatchNorm2d(32), nn.ReLU(), nn.MaxPool2d(2),
                             nn.Conv2d(32, 64, 3, padding=1), nn.BatchNorm2d(64), nn.ReLU(),
                             nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.Linear(64, classes))
    if name == 'resnet_tiny':
        return models.ResNet((1, 1, 1, 1), num_classes=classes, width=8, in_channels=c)
    if name in ('resnet18', 'resnet34'):
        return getattr(models, name)(classes, in_channels=c)
    if name == 'wideresnet28':
        return models.WideResNet(28, 10, classes, dropout=0.3, in_channels=c)
    if name == 'wideresnet_tiny':
        return models.WideResNet(10, 1, classes, in_channels=c)
    if name == 'vit_tiny_patch16_224':
        return models.VisionTransformer(h, 16 if h % 16 == 0 and h >= 64 else 4, 12, 3, 192, 768, classes, in_channels=c)
    if name == 'mixer_b16_224':
        return models.mixer_b_16(classes) if h == 224 else models.mixer_tiny(classes, image_size=h)
    if name == 'mixer_tiny':
        return models.mixer_tiny(classes, image_size=h)
    return models.vit_tiny(classes, image_size=h)


def make_loaders(args, device):
    """(train, validation or None, test, input shape, classes); each an iterable of (x, t) on CPU."""
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
        return batches(args.steps_per_epoch), None, batches(max(1, args.steps_per_epoch // 5)), shape, classes
    from torchvision import datasets, transforms
    big = args.model.endswith('_224')  # transformers of the reference's recipes train on 224 x 224 crops
    if args.dataset == 'mnist':
        norm = transforms.Normalize((0.1307,), (0.3081,))
        cls, shape = datasets.MNIST, (1, 28, 28)
    else:
        norm = transforms.Normalize((0.4914, 0.4822, 0.4465), (0.2470, 0.2435, 0.2616))
        cls, shape = datasets.CIFAR10, (3, 224, 224) if big else (3, 32, 32)
    pre = [transforms.Resize(224)] if big and args.dataset == 'cifar10' else []
    train_tf = list(pre)
    if args.auto_augment and args.dataset == 'cifar10':
        train_tf.append(transforms.AutoAugment(transforms.AutoAugmentPolicy.CIFAR10))
    train_tf = transforms.Compose(train_tf + [transforms.ToTensor(), norm])
    test_tf = transforms.Compose(pre + [transforms.ToTensor(), norm])
    train = cls(args.data_root, train=True, download=False, transform=train_tf)
    held_out = cls(args.data_root, train=True, download=False, transform=test_tf)
    test = cls(args.data_root, train=False, download=False, transform=test_tf)
    kw = dict(batch_size=args.batch_size, num_workers=2, pin_memory=device.type == 'cuda')
    val_loader = None
    if args.train_size is not None and args.train_size < len(train):
        order = torch.randperm(len(train), generator=torch.Generator().manual_seed(args.seed)).tolist()
        val_loader = torch.utils.data.DataLoader(torch.utils.data.Subset(held_out, order[args.train_size:]), **kw)
        train = torch.utils.data.Subset(train, order[:args.train_size])
    return (torch.utils.data.DataLoader(train, shuffle=True, drop_last=True, **kw), val_loader,
            torch.utils.data.DataLoader(test, **kw), shape, 10)


def make_grad_maker(args, model):
    name = args.optim
    if name in ('sgd', 'adam', 'adamw'):
        return asdl.GradientMaker(model)
    ignore = [nn.BatchNorm1d, nn.BatchNorm2d, nn.BatchNorm3d, nn.LayerNorm] if args.ignore_norm_layers else None
    cfg = asdl.PreconditioningConfig(data_size=args.batch_size, damping=args.damping, ema_decay=args.ema_decay,
                                     curvature_upd_interval=args.curvature_upd_interval,
                                     preconditioner_upd_interval=args.preconditioner_upd_interval,
                                     ignore_modules=ignore)
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


def evaluate(model_fn, batches, to_device):
    """(mean loss, accuracy in percent) over ``batches``."""
    loss = correct = total = 0
    with torch.no_grad():
        for x, t in batches:
            x, t = to_device(x, t)
            y = model_fn(x)
            loss += F.cross_entropy(y.float(), t, reduction='sum').item()
            correct += (y.argmax(dim=1) == t).sum().item()
            total += t.numel()
    return loss / max(total, 1), 100 * correct / max(total, 1)


def main():
    args = parse_args()
    torch.manual_seed(args.seed)
    device = torch.device('cuda' if torch.cuda.is_available() and not args.no_cuda else 'cpu')
    train_batches, val_batches, test_batches, shape, classes = make_loaders(args, device)
    model = make_model(args.model, shape, classes, args.width, args.depth).to(device)
    nhwc = device.type == 'cuda' and args.model != 'mlp'
    if nhwc:
        model = model.to(memory_format=torch.channels_last)
    if args.optim in ('adam', 'adamw'):
        cls = torch.optim.Adam if args.optim == 'adam' else torch.optim.AdamW
        optimizer = cls(model.parameters(), lr=args.lr, weight_decay=args.weight_decay)
    else:
        optimizer = torch.optim.SGD(model.parameters(), lr=args.lr, momentum=args.momentum,
                                    weight_decay=args.weight_decay, nesterov=args.nesterov)
    scheduler = torch.optim.lr_scheduler.CosineAnnealingLR(optimizer, T_max=args.epochs) if args.cosine else None
    grad_maker = make_grad_maker(args, model)
    aug_rng = torch.Generator(device=device).manual_seed(args.seed)

    def model_fn(x):
        with torch.autocast(device.type, dtype=torch.bfloat16, enabled=args.bf16):
            return model(x)

    def to_device(x, t, train=False):
        x = x.to(device, non_blocking=True)
        if train and x.ndim == 4:  # whole-batch augmentation on the device
            if args.data_augmentation:
                x = batch_random_crop_flip(x, padding=max(1, x.shape[-1] // 8), generator=aug_rng)
            if args.cutout:
                x = batch_cutout(x, args.n_holes, args.length * x.shape[-1] // 32, generator=aug_rng)
        if x.ndim == 4 and nhwc:
            x = x.contiguous(memory_format=torch.channels_last)
        return x, t.to(device, non_blocking=True)

    def log(record):
        if args.log_json:
            with open(args.log_json, 'a') as f:
                f.write(json.dumps(record) + '\n')

    steps, train_time, best_val, stopped = 0, 0.0, 0.0, None
    try:
        for epoch in range(1, args.epochs + 1):
            model.train()
            if device.type == 'cuda':
                torch.cuda.synchronize()
            start = time.time()
            running = 0.0
            for i, (x, t) in enumerate(train_batches, 1):
                x, t = to_device(x, t, train=True)
                optimizer.zero_grad(set_to_none=False)
                dummy_y = grad_maker.setup_model_call(model_fn, x)
                grad_maker.setup_loss_call(F.cross_entropy, dummy_y, t, label_smoothing=args.label_smoothing)
                _, loss = grad_maker.forward_and_backward()
                if args.clip_grad_norm > 0:
                    torch.nn.utils.clip_grad_norm_(model.parameters(), args.clip_grad_norm)
                optimizer.step()
                value = float(loss.detach())
                if value != value or value in (float('inf'), float('-inf')):
                    stopped = f'non-finite loss at epoch {epoch}, step {i}'
                    break
                running += value
                steps += 1
                if args.log_interval and i % args.log_interval == 0:
                    print(f'  epoch {epoch} step {i}: loss {running / i:.4f}')
            if device.type == 'cuda':
                torch.cuda.synchronize()
            train_time += time.time() - start
            if stopped:
                print(stopped)
                break
            if scheduler is not None:
                scheduler.step()
            model.eval()
            record = {'epoch': epoch, 'train_loss': running / len(train_batches), 'lr': optimizer.param_groups[0]['lr']}
            line = f'epoch {epoch}: train loss {record["train_loss"]:.4f}'
            if val_batches is not None:
                record['val_loss'], record['val_acc'] = evaluate(model_fn, val_batches, to_device)
                best_val = max(best_val, record['val_acc'])
                line += f'  val acc {record["val_acc"]:.2f}%'
            record['test_loss'], record['test_acc'] = evaluate(model_fn, test_batches, to_device)
            print(line + f'  test acc {record["test_acc"]:.2f}%')
            log(record)
    except torch.OutOfMemoryError as err:  # report like the reference does, with the memory figure marked
        print(err)
        stopped = 'out of memory'
    summary = {'total_train_time_s': train_time, 'avg_step_time_ms': 1000 * train_time / max(steps, 1), 'stopped': stopped}
    print(f'total_train_time: {train_time:.2f}s')
    print(f'avg_step_time: {summary["avg_step_time_ms"]:.2f}ms')
    if val_batches is not None:
        summary['max_val_accuracy'] = best_val
        print(f'max_val_accuracy: {best_val:.2f}%')
    if device.type == 'cuda':
        peak = -1 if stopped == 'out of memory' else torch.cuda.max_memory_allocated() / 2 ** 20
        summary['cuda_max_memory_mib'] = peak
        print(f'cuda_max_memory: {peak:.1f}MiB')
        if stopped != 'out of memory':
            asdl.ops.check_status()
    log(summary)
    if stopped and stopped != 'out of memory':
        sys.exit(1)


if __name__ == '__main__':
    main()
