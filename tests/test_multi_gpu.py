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


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Conv2d(3, 16, 3, padding=1, bias=False), nn.ReLU(),
                         nn.Conv2d(16, 32, 3, stride=2, padding=1, bias=False), nn.ReLU(),
                         nn.Conv2d(32, 24, 1), nn.ReLU(),
                         nn.AdaptiveAvgPool2d(1), nn.Flatten(), nn.LayerNorm(24), nn.Linear(24, 5))


def _data(n):
    g = torch.Generator().manual_seed(3)
    return torch.randn(n, 3, 12, 12, generator=g), torch.randint(0, 5, (n,), generator=g)


def _train(model, x, t, data_size, **kw):
    cfg = asdl.PreconditioningConfig(data_size=data_size, damping=1e-2, ema_decay=0.4,
                                     curvature_upd_interval=3, preconditioner_upd_interval=3)
    gm = asdl.FusedKfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP, **kw)
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


def _worker(rank, world, port, out_dir):
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    torch.backends.cudnn.allow_tf32 = False
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world,
                            timeout=timedelta(seconds=120), device_id=dev)
    try:
        x, t = _data(8 * world)
        n = x.shape[0] // world
        xs = x[rank * n:(rank + 1) * n].to(dev).contiguous(memory_format=torch.channels_last)
        ts = t[rank * n:(rank + 1) * n].to(dev)
        results = {}
        for name, kw in (('torch', dict(comm='torch')), ('symmetric', dict(comm='symmetric')),
                         ('symmetric_graph', dict(comm='symmetric', cuda_graph=True))):
            model = _net().to(dev).to(memory_format=torch.channels_last)
            results[name] = _train(model, xs, ts, n, **kw)
            torch.cuda.synchronize()
            dist.barrier()
        torch.save(results, os.path.join(out_dir, f'rank{rank}.pt'))
    finally:
        dist.destroy_process_group()


def rel_err(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)).item()


def test_data_parallel_transports_match_single_process():
    world = 2
    with tempfile.TemporaryDirectory() as out_dir:
        mp.spawn(_worker, args=(world, _free_port(), out_dir), nprocs=world, join=True)
        per_rank = [torch.load(os.path.join(out_dir, f'rank{r}.pt')) for r in range(world)]
    torch.backends.cudnn.allow_tf32 = False
    x, t = _data(8 * world)
    dev = torch.device('cuda', 0)
    model = _net().to(dev).to(memory_format=torch.channels_last)
    single = _train(model, x.to(dev).contiguous(memory_format=torch.channels_last), t.to(dev), x.shape[0])
    for name in ('torch', 'symmetric', 'symmetric_graph'):
        for step in range(STEPS):
            a, b = per_rank[0][name][step], per_rank[1][name][step]
            assert rel_err(a, b) < 1e-6, (name, step, 'ranks disagree')
            assert rel_err(a, single[step]) < 2e-2, (name, step, rel_err(a, single[step]))
