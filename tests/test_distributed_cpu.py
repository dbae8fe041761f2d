"""Multi-process semantics on CPU ranks (gloo): data-parallel K-FAC / Shampoo equal the
single-process run on the concatenated batch, owner assignment is balanced and deterministic,
state dicts move between world sizes, and a rank that disappears ends the others' next collective
with an error instead of a hang."""
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
from asdl_b200.parallel import assign_owners, balance_report  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Conv2d(3, 6, 3, padding=1), nn.ReLU(), nn.Conv2d(6, 4, 3, stride=2), nn.ReLU(),
                         nn.Flatten(), nn.LayerNorm(4 * 3 * 3), nn.Linear(4 * 3 * 3, 5))


def _data(n=8):
    g = torch.Generator().manual_seed(3)
    return torch.randn(n, 3, 8, 8, generator=g), torch.randint(0, 5, (n,), generator=g)


def _make(kind, model, data_size):
    if kind == 'kfac':
        cfg = asdl.PreconditioningConfig(data_size=data_size, damping=1e-2, ema_decay=0.5,
                                         curvature_upd_interval=2, preconditioner_upd_interval=2)
        return asdl.KfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP)
    if kind == 'kfac_noema':
        cfg = asdl.PreconditioningConfig(data_size=data_size, damping=1e-2)
        return asdl.KfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP)
    if kind in ('fused', 'fused_exact'):   # the exact Fisher takes one backward pass per class: statistics add up
        cfg = asdl.PreconditioningConfig(data_size=data_size, damping=1e-2, ema_decay=0.5,
                                         curvature_upd_interval=2, preconditioner_upd_interval=2)
        fisher_type = asdl.FISHER_EMP if kind == 'fused' else asdl.FISHER_EXACT
        return asdl.FusedKfacGradientMaker(model, cfg, fisher_type=fisher_type, comm='torch')
    cfg = asdl.PreconditioningConfig(damping=1e-3, preconditioner_upd_interval=2)
    return asdl.ShampooGradientMaker(model, cfg, block_size=8)


def _train(kind, model, x, t, data_size, steps=4):
    gm = _make(kind, model, data_size)
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    grads = None
    for _ in range(steps):
        opt.zero_grad()
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        gm.forward_and_backward()
        grads = torch.cat([p.grad.flatten() for p in model.parameters()]).clone()
        opt.step()
    return gm, grads


def _worker(rank, world, port, kind, out_dir):
    dist.init_process_group('gloo', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world,
                            timeout=timedelta(seconds=60))
    try:
        x, t = _data(4 * world)
        n = x.shape[0] // world
        xs, ts = x[rank * n:(rank + 1) * n], t[rank * n:(rank + 1) * n]
        model = _net()
        gm, grads = _train(kind, model, xs, ts, data_size=n)
        torch.save({'grads': grads, 'state': gm.state_dict() if kind != 'shampoo' else None,
                    'weights': model.state_dict()}, os.path.join(out_dir, f'rank{rank}.pt'))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('kind,world', [('kfac', 2), ('kfac_noema', 2), ('fused', 2), ('shampoo', 2),
                                        ('kfac', 3), ('fused', 3), ('shampoo', 3), ('fused_exact', 2)])
def test_data_parallel_matches_single_process(kind, world):
    with tempfile.TemporaryDirectory() as out_dir:
        mp.spawn(_worker, args=(world, _free_port(), kind, out_dir), nprocs=world, join=True)
        results = [torch.load(os.path.join(out_dir, f'rank{r}.pt'), weights_only=False) for r in range(world)]
    for other in results[1:]:
        torch.testing.assert_close(results[0]['grads'], other['grads'])  # ranks agree on every gradient
    x, t = _data(4 * world)
    _, single = _train(kind, _net(), x, t, data_size=x.shape[0])
    if kind == 'shampoo':
        # the statistic of the averaged gradient is what the owner sees: identical to single process
        torch.testing.assert_close(results[0]['grads'], single, rtol=1e-3, atol=1e-5)
    else:
        torch.testing.assert_close(results[0]['grads'], single, rtol=2e-3, atol=1e-5)
    if kind == 'kfac':
        # owner-sharded state from 2 ranks loads into a single-process maker
        merged = {'step': results[0]['state']['step'], 'curvature': {}}
        for r in results:
            merged['curvature'].update(r['state']['curvature'])
        model = _net()
        model.load_state_dict(results[0]['weights'])
        gm = _make('kfac', model, 4 * world)
        gm.load_state_dict(merged)
        assert gm.state['step'] == 4
        assert model[0].fisher.kron.A is not None


def _vanishing_worker(rank, world, port, out_dir):
    dist.init_process_group('gloo', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world,
                            timeout=timedelta(seconds=5))
    t = torch.ones(4)
    dist.all_reduce(t)  # everybody is here for the first step
    if rank == 1:
        # leaves between steps, with nothing in flight
        os._exit(0)
    try:
        dist.all_reduce(t)
        outcome = 'completed'
    except Exception as exc:  # the missing peer surfaces as an error on the host
        outcome = f'error:{type(exc).__name__}'
    with open(os.path.join(out_dir, 'rank0.txt'), 'w') as fh:
        fh.write(outcome)
    os._exit(0)


def test_vanished_rank_ends_the_collective_with_an_error():
    with tempfile.TemporaryDirectory() as out_dir:
        ctx = mp.get_context('spawn')
        port = _free_port()
        procs = [ctx.Process(target=_vanishing_worker, args=(r, 2, port, out_dir)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=90)
            assert not p.is_alive()
        outcome = open(os.path.join(out_dir, 'rank0.txt')).read()
    assert outcome.startswith('error:'), outcome


def _vanishing_maker_worker(rank, world, port, out_dir):
    """A data-parallel maker runs one step on two ranks; rank 1 then leaves between steps.  Rank 0's next
    step has to raise within the process-group timeout, leave no hooks on the model and not advance
    the maker's step counter."""
    dist.init_process_group('gloo', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world,
                            timeout=timedelta(seconds=5))
    x, t = _data(4 * world)
    n = x.shape[0] // world
    model = _net()
    gm = _make('fused', model, n)
    xs, ts = x[rank * n:(rank + 1) * n], t[rank * n:(rank + 1) * n]

    def one_step():
        for p in model.parameters():
            p.grad = None
        d = gm.setup_model_call(model, xs)
        gm.setup_loss_call(F.cross_entropy, d, ts)
        gm.forward_and_backward()

    one_step()
    if rank == 1:
        os._exit(0)                      # leaves between steps, with nothing in flight
    before = gm.state['step']
    try:
        one_step()
        outcome = 'completed'
    except Exception as exc:
        hooks = sum(len(m._forward_hooks) + len(m._forward_pre_hooks) + len(m._backward_hooks) for m in model.modules())
        outcome = f'error:{type(exc).__name__}:hooks={hooks}:step_advanced={gm.state["step"] != before}'
    with open(os.path.join(out_dir, 'rank0.txt'), 'w') as fh:
        fh.write(outcome)
    os._exit(0)


def test_vanished_rank_makes_the_next_maker_step_raise_and_leaves_the_model_clean():
    with tempfile.TemporaryDirectory() as out_dir:
        ctx = mp.get_context('spawn')
        port = _free_port()
        procs = [ctx.Process(target=_vanishing_maker_worker, args=(r, 2, port, out_dir)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert not p.is_alive()
        outcome = open(os.path.join(out_dir, 'rank0.txt')).read()
    assert outcome.startswith('error:'), outcome
    assert 'hooks=0' in outcome and 'step_advanced=False' in outcome, outcome


def test_owner_assignment_is_balanced_and_deterministic():
    costs = [4608 ** 3] * 3 + [2304 ** 3] * 6 + [1024 ** 3] * 12 + [64 ** 3] * 30
    owners = assign_owners(costs, 8)
    assert owners == assign_owners(costs, 8)
    ratio, load = balance_report(costs, owners, 8)
    # three items dominate: no assignment can do better than one of them alone on a rank
    assert max(load) == 4608 ** 3 and min(load) > 0
    even = assign_owners([1024 ** 3] * 64, 8)
    assert balance_report([1024 ** 3] * 64, even, 8)[0] == pytest.approx(1.0)
    pinned = assign_owners(costs, 8, fixed=[7] + [None] * (len(costs) - 1))
    assert pinned[0] == 7
    assert assign_owners([1.0, 2.0], 4) == [1, 0]  # more ranks than layers: nobody holds two
