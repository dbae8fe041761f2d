"""Device time per phase of the ResNet-50 K-FAC step (plain step, curvature step, inverse update,
gradient reduction / preconditioning / broadcast), measured with CUDA events inside the gradient
maker.

    python benchmarks/kfac_phases.py [--no-graph] [--precond-precision bf16] [--no-overlap]
    python benchmarks/kfac_phases.py --impl reference    # the unmodified reference: plain / curvature / inverse steps
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29561 benchmarks/kfac_phases.py

Rank 0 prints one JSON line {phase: [calls, mean milliseconds]}.  Batch 32 per GPU, bf16 autocast,
channels_last, curvature every 10 steps, inverses every 30 steps (so that a short run sees them).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402
from asdl_b200.models import resnet50  # noqa: E402


def reference_phases(args):
    """Step kinds of the reference package (stock fp32 / TF32 path on torchvision's ResNet-50), timed
    the way ``bench.py`` times them for its ``phases`` entry: CUDA events around single steps whose
    kind is chosen through the maker's step counter."""
    import bench
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    ns = argparse.Namespace(impl='reference', precision='bf16', no_graph=True, precond_precision='bf16x3')
    step, _, to_device, dtype, gm = bench.build_reference(ns, dev, world)
    xs, ts = bench.make_batches(4, dev, seed=1234 + local)
    batches = [to_device(x, t) for x, t in zip(xs, ts)]
    flush = torch.empty(bench.L2_FLUSH_BYTES, dtype=torch.uint8, device=dev)
    for i in range(max(args.warmup, 3)):
        step(*batches[i % 4])
    phases = bench.measure_phases(step, gm, batches, flush)
    if local == 0:
        print(json.dumps({'case': 'resnet50_kfac_phases', 'impl': 'reference', 'dtype': dtype, 'n_gpus': world,
                          'phases_ms': phases}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--no-graph', action='store_true')
    ap.add_argument('--precond-precision', default='bf16x3', choices=['bf16', 'bf16x3'])
    ap.add_argument('--steps', type=int, default=60)
    ap.add_argument('--warmup', type=int, default=12)
    ap.add_argument('--no-overlap', action='store_true',
                    help='reduce the gradients after the backward pass instead of bucket by bucket during it')
    ap.add_argument('--bucket-mb', type=float, default=16.0, help='size of a gradient bucket of the overlapped reduction')
    ap.add_argument('--comm-blocks', type=int, default=None, help='CTAs of a bucket kernel')
    ap.add_argument('--impl', choices=['ours', 'reference'], default='ours')
    args = ap.parse_args()
    if args.impl == 'reference':
        return reference_phases(args)
    world = int(os.environ.get('WORLD_SIZE', '1'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    torch.manual_seed(0)
    model = resnet50().to(dev).to(memory_format=torch.channels_last)
    cfg = asdl.PreconditioningConfig(data_size=32, damping=1e-3, ema_decay=0.05, curvature_upd_interval=10,
                                     preconditioner_upd_interval=30)
    gm = asdl.FusedKfacGradientMaker(model, cfg, cuda_graph=not args.no_graph,
                                     precond_precision=args.precond_precision,
                                     overlap_grad_reduce=not args.no_overlap, bucket_mb=args.bucket_mb)
    if args.comm_blocks:
        gm.comm_blocks = args.comm_blocks
    opt = torch.optim.SGD(model.parameters(), lr=1e-4, momentum=0.9)
    x = torch.randn(32, 3, 224, 224, device=dev).contiguous(memory_format=torch.channels_last)
    t = torch.randint(0, 1000, (32,), device=dev)

    def model_fn(inp):
        with torch.autocast('cuda', dtype=torch.bfloat16):
            return model(inp)

    def step():
        opt.zero_grad(set_to_none=False)
        d = gm.setup_model_call(model_fn, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        gm.forward_and_backward()
        opt.step()

    for _ in range(args.warmup):
        step()
    gm.enable_phase_timing()
    for _ in range(args.steps):
        step()
    phases = gm.phase_times()
    if local == 0:
        print(json.dumps({'case': 'resnet50_kfac_phases', 'n_gpus': world, 'cuda_graph': not args.no_graph,
                          'precond_precision': args.precond_precision, 'overlap': not args.no_overlap,
                          'bucket_mb': args.bucket_mb, 'comm_blocks': gm.comm_blocks,
                          'phases_ms': {k: [n, round(ms, 3)] for k, (n, ms) in phases.items()}}), flush=True)
    asdl.ops.check_status()
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
