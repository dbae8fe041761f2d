"""Data-parallel fused K-FAC on 2+ GPUs of one node: the NVLink symmetric-memory transport (eager and
replayed from a CUDA graph) and the torch.distributed transport give every rank the same gradients
as a single-process run on the concatenated batch.  Skipped on boxes with one GPU; the kernels of
the transport are also exercised on one GPU by test_gpu_kernels.py (emulated ranks)."""
import copy
import os
import socket
import sys
import tempfile
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402
from asdl_b200 import ops  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2,
                                 reason='needs two GPUs')]

STEPS = 7


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


class _Reuse(nn.Module):
    """Ten curvature layers (more owners than ranks at every world size tested), one of them
    applied twice in a forward pass, a LayerNorm, and a bias-free head."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.stem = nn.Conv2d(3, 16, 3, padding=1, bias=False)
        self.convs = nn.ModuleList([nn.Conv2d(16, 16, 3, padding=1) for _ in range(3)])
        self.down = nn.Conv2d(16, 32, 3, stride=2, padding=1, bias=False)
        self.point = nn.Conv2d(32, 24, 1)
        self.norm = nn.LayerNorm(24)
        self.shared = nn.Linear(24, 24)
        self.mid = nn.Linear(24, 24)
        self.head = nn.Linear(24, 5, bias=False)

    def forward(self, x):
        x = F.relu(self.stem(x))
        for c in self.convs:
            x = F.relu(c(x)) + x
        x = F.relu(self.point(F.relu(self.down(x))))
        x = self.norm(x.mean(dim=(2, 3)))
        x = F.relu(self.shared(x))
        x = F.relu(self.mid(x))
        x = F.relu(self.shared(x))          # second application of the same layer
        return self.head(x)


def _net():
    return _Reuse()


def _data(n):
    g = torch.Generator().manual_seed(3)
    return torch.randn(n, 3, 12, 12, generator=g), torch.randint(0, 5, (n,), generator=g)


def _train(model, x, t, data_size, multimem=True, **kw):
    os.environ['ASDL_B200_MULTIMEM'] = '1' if multimem else '0'   # read when the symmetric buffer is set up
    cfg = asdl.PreconditioningConfig(data_size=data_size, damping=1e-2, ema_decay=0.4,
                                     curvature_upd_interval=3, preconditioner_upd_interval=3)
    push = kw.pop('push', False)
    gm = asdl.FusedKfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP, **kw)
    if push:   # statistics and preconditioned gradients sent from the GEMM epilogues instead of pulled / broadcast
        gm.pull_statistics, gm.replicate_in_epilogue = False, True
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    out = []
    for _ in range(STEPS):
        opt.zero_grad(set_to_none=False)
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        _, loss = gm.forward_and_backward()
        out.append(torch.cat([p.grad.flatten() for p in model.parameters()]).cpu().clone())
        opt.step()
    ops.check_status()
    return out


def _train_resnet(dev, world, rank):
    """BatchNorm model under autocast, two Monte-Carlo samples, graph replay: batch statistics and
    sampled labels are per rank, so the check is that all ranks end up with the same gradients."""
    from asdl_b200.models import resnet_tiny
    torch.manual_seed(0)
    # width 64 and no size threshold: the 3 x 3 convolutions take the implicit-im2col statistics path
    ops.IMPLICIT_IM2COL_MIN_MB = 0.0
    model = resnet_tiny(num_classes=10, width=64, fused=True).to(dev).to(memory_format=torch.channels_last)
    cfg = asdl.PreconditioningConfig(data_size=8, damping=1e-3, ema_decay=0.05,
                                     curvature_upd_interval=2, preconditioner_upd_interval=4)
    gm = asdl.FusedKfacGradientMaker(model, cfg, n_mc_samples=2, cuda_graph=True)
    g = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(8, 3, 32, 32, generator=g).to(dev).contiguous(memory_format=torch.channels_last)
    t = torch.randint(0, 10, (8,), generator=g).to(dev)

    def model_fn(inp):
        with torch.autocast('cuda', dtype=torch.bfloat16):
            return model(inp)

    opt = torch.optim.SGD(model.parameters(), lr=1e-3)
    out = []
    for _ in range(9):
        opt.zero_grad(set_to_none=True)
        d = gm.setup_model_call(model_fn, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        gm.forward_and_backward()
        out.append(torch.cat([p.grad.flatten().float() for p in model.parameters()]).cpu().clone())
        opt.step()
    ops.check_status()
    return out


def _train_shampoo(model, x, t, **kw):
    cfg = asdl.PreconditioningConfig(damping=1e-4, preconditioner_upd_interval=2)
    gm = asdl.ShampooGradientMaker(model, cfg, block_size=16, **kw)
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    out = []
    for _ in range(5):
        opt.zero_grad(set_to_none=True)
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        gm.forward_and_backward()
        out.append(torch.cat([p.grad.flatten() for p in model.parameters()]).cpu().clone())
        opt.step()
    ops.check_status()
    return out


TRANSPORTS = (('torch', dict(comm='torch')),
              ('symmetric', dict(comm='symmetric', overlap_grad_reduce=False)),
              ('symmetric_overlap', dict(comm='symmetric', bucket_mb=0.01)),      # several buckets on a tiny model
              ('symmetric_overlap_peer_loads', dict(comm='symmetric', bucket_mb=0.01, multimem=False)),
              ('symmetric_graph', dict(comm='symmetric', cuda_graph=True, overlap_grad_reduce=False)),
              ('symmetric_graph_overlap', dict(comm='symmetric', cuda_graph=True, bucket_mb=0.01)),
              ('symmetric_push', dict(comm='symmetric', overlap_grad_reduce=False, push=True)),
              ('symmetric_graph_push', dict(comm='symmetric', cuda_graph=True, overlap_grad_reduce=False, push=True)))


def _worker(rank, world, port, out_dir):
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world,
                            timeout=timedelta(seconds=120), device_id=dev)
    try:
        x, t = _data(8 * world)
        n = x.shape[0] // world
        xs = x[rank * n:(rank + 1) * n].to(dev).contiguous(memory_format=torch.channels_last)
        ts = t[rank * n:(rank + 1) * n].to(dev)
        results = {}
        for name, kw in TRANSPORTS:
            model = _net().to(dev).to(memory_format=torch.channels_last)
            results[name] = _train(model, xs, ts, n, **kw)
            torch.cuda.synchronize()
            dist.barrier()
        for name, kw in (('shampoo_torch', dict(comm='torch')), ('shampoo_symmetric', dict(comm='symmetric'))):
            model = _net().to(dev)
            results[name] = _train_shampoo(model, xs.contiguous(), ts, **kw)
            torch.cuda.synchronize()
            dist.barrier()
        results['resnet'] = _train_resnet(dev, world, rank)
        torch.cuda.synchronize()
        dist.barrier()
        torch.save(results, os.path.join(out_dir, f'rank{rank}.pt'))
    finally:
        dist.destroy_process_group()


def rel_err(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)).item()


@pytest.mark.parametrize('world', [2, 4, 8])
def test_data_parallel_transports_match_single_process(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    with tempfile.TemporaryDirectory() as out_dir:
        mp.spawn(_worker, args=(world, _free_port(), out_dir), nprocs=world, join=True)
        per_rank = [torch.load(os.path.join(out_dir, f'rank{r}.pt')) for r in range(world)]
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    x, t = _data(8 * world)
    dev = torch.device('cuda', 0)
    model = _net().to(dev).to(memory_format=torch.channels_last)
    single = _train(model, x.to(dev).contiguous(memory_format=torch.channels_last), t.to(dev), x.shape[0])
    worst = {}
    for name, _ in TRANSPORTS:
        for step in range(STEPS):
            a = per_rank[0][name][step]
            for r in range(1, world):
                assert rel_err(per_rank[r][name][step], a) < 1e-6, (name, step, r, 'ranks disagree')
            worst[name] = max(worst.get(name, 0.0), rel_err(a, single[step]))
            assert rel_err(a, single[step]) < 5e-3, (name, step, rel_err(a, single[step]))
    single_shampoo = _train_shampoo(_net().to(dev), x.to(dev), t.to(dev))
    for name in ('shampoo_torch', 'shampoo_symmetric'):
        for step, ref in enumerate(single_shampoo):
            a = per_rank[0][name][step]
            for r in range(1, world):
                assert rel_err(per_rank[r][name][step], a) < 1e-6, (name, step, r, 'ranks disagree')
            worst[name] = max(worst.get(name, 0.0), rel_err(a, ref))
            assert rel_err(a, ref) < 5e-3, (name, step, rel_err(a, ref))
    for step, a in enumerate(per_rank[0]['resnet']):
        assert torch.isfinite(a).all(), ('resnet', step)
        for r in range(1, world):
            assert rel_err(per_rank[r]['resnet'][step], a) < 1e-6, ('resnet', step, r, 'ranks disagree')
    print(f'world {world}: largest relative difference to the single-process run per transport: {worst}')
