"""Device time per phase of a training step, for any method and model of examples/train.py.

    python benchmarks/time_step.py --optim kfac --model resnet18 --batch-size 128 --bf16
    python benchmarks/time_step.py --config benchmarks/time_step_example.yaml
    python benchmarks/time_step.py --optim shampoo --model vit_tiny --no-cuda --iters 5      # CPU: wall clock

Runs ``--warmup`` untimed steps, then ``--iters`` steps under a ``PhaseProfile``: every named range of
the library (forward_and_backward, update_curvature, cov_kron_A/B, inv_*, update_preconditioner,
precondition, collectives) plus the optimizer step is timed with CUDA events on the device (one
synchronisation at the end), and the table of calls / mean / standard deviation per range is printed,
as JSON with ``--json``.  Synthetic data of the model's input shape.  A YAML (or JSON) file may give
any of the options.  Role of the reference's examples/prof/time_step.py + parse_nvtx_events.py, without
an external profiler.
"""
import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, 'examples'))
import train as recipes  # noqa: E402  (examples/train.py: model and gradient-maker factories)
from asdl_b200.utils import PhaseProfile, nvtx_range  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--config', default=None, help='YAML or JSON file with any of the options below')
    ap.add_argument('--optim', default='kfac', choices=recipes.OPTIMS)
    ap.add_argument('--model', default='resnet18', choices=recipes.MODELS)
    ap.add_argument('--width', type=int, default=256)
    ap.add_argument('--depth', type=int, default=3)
    ap.add_argument('--image-size', type=int, default=32)
    ap.add_argument('--batch-size', type=int, default=128)
    ap.add_argument('--damping', type=float, default=1e-3)
    ap.add_argument('--ema-decay', type=float, default=-1)
    ap.add_argument('--curvature-upd-interval', type=int, default=1)
    ap.add_argument('--preconditioner-upd-interval', type=int, default=1)
    ap.add_argument('--block-size', type=int, default=128)
    ap.add_argument('--ignore-norm-layers', action='store_true')
    ap.add_argument('--cuda-graph', action='store_true')
    ap.add_argument('--bf16', action='store_true')
    ap.add_argument('--iters', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--no-cuda', action='store_true')
    ap.add_argument('--json', action='store_true', help='print the table as one JSON line')
    args = ap.parse_args()
    if args.config:
        with open(args.config) as f:
            if args.config.endswith(('.yaml', '.yml')):
                import yaml
                loaded = yaml.safe_load(f)
            else:
                loaded = json.load(f)
        for key, value in loaded.items():
            key = key.replace('-', '_')
            if not hasattr(args, key):
                raise KeyError(f'unknown option {key} in {args.config}')
            setattr(args, key, value)
    device = torch.device('cuda' if torch.cuda.is_available() and not args.no_cuda else 'cpu')
    torch.manual_seed(0)
    channels = 1 if args.model == 'mlp' else 3
    model = recipes.make_model(args.model, (channels, args.image_size, args.image_size), 10, args.width, args.depth).to(device)
    x = torch.randn(args.batch_size, channels, args.image_size, args.image_size, device=device)
    if device.type == 'cuda' and args.model != 'mlp':
        model = model.to(memory_format=torch.channels_last)
        x = x.contiguous(memory_format=torch.channels_last)
    t = torch.randint(0, 10, (args.batch_size,), device=device)
    optimizer = torch.optim.SGD(model.parameters(), lr=1e-3, momentum=0.9)
    grad_maker = recipes.make_grad_maker(args, model)

    def model_fn(inp):
        with torch.autocast(device.type, dtype=torch.bfloat16, enabled=args.bf16):
            return model(inp)

    def step():
        with nvtx_range('step'):
            optimizer.zero_grad(set_to_none=False)
            dummy_y = grad_maker.setup_model_call(model_fn, x)
            grad_maker.setup_loss_call(F.cross_entropy, dummy_y, t)
            grad_maker.forward_and_backward()
            with nvtx_range('optimizer_step'):
                optimizer.step()

    for _ in range(args.warmup):
        step()
    with PhaseProfile() as prof:
        for _ in range(args.iters):
            step()
    if args.json:
        print(json.dumps({'optim': args.optim, 'model': args.model, 'batch_size': args.batch_size,
                          'device': device.type, 'ranges': prof.reduce_max()}))
    else:
        print(prof.report())
    if device.type == 'cuda':
        import asdl_b200
        asdl_b200.ops.check_status()


if __name__ == '__main__':
    main()
