"""The lower-level distributed entry points on two CPU ranks (gloo), each against its
single-process value: summed Fisher blocks and Fisher-vector products, packed ParamVector and
MatrixManager reductions, loader gradients averaged over ranks, a power iteration whose start
vectors are broadcast, partitioned (reduce-scatter) Fisher blocks and the rank-parallel kernel
assembly."""
import os
import socket
import sys
import tempfile
from datetime import timedelta

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.data import DataLoader, TensorDataset

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import asdl_b200 as asdl  # noqa: E402
from asdl_b200 import kernel as K  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _net():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(6, 5), nn.Tanh(), nn.Linear(5, 3))


def _data(n=8):
    g = torch.Generator().manual_seed(5)
    return torch.randn(n, 6, generator=g), torch.randint(0, 3, (n,), generator=g)


def _fisher(model, x, t, shape, **kw):
    cfg = asdl.FisherConfig(fisher_type=asdl.FISHER_EMP, fisher_shapes=[shape], loss_type=asdl.LOSS_CROSS_ENTROPY)
    fm = asdl.get_fisher_maker(model, cfg)
    dummy = fm.setup_model_call(model, x)
    fm.setup_loss_call(F.cross_entropy, dummy, t)
    fm.forward_and_backward(**kw)
    return fm


def _manager_fisher(model, x, t, data_size):
    cfg = asdl.FisherConfig(fisher_type=asdl.FISHER_EMP, fisher_shapes=[asdl.SHAPE_LAYER_WISE], data_size=data_size,
                            loss_type=asdl.LOSS_CROSS_ENTROPY, fisher_attr=asdl.FISHER_EMP)
    fm = asdl.get_fisher_maker(model, cfg)
    dummy = fm.setup_model_call(model, x)
    fm.setup_loss_call(F.cross_entropy, dummy, t)
    fm.forward_and_backward()


def _probe(model):
    g = torch.Generator().manual_seed(9)
    return asdl.ParamVector(list(model.parameters()), [torch.randn(p.shape, generator=g) for p in model.parameters()])


def _results(model, x, t, world, rank=0, distributed=False):
    """Everything the test compares, computed on (x, t); with ``distributed`` the rank-local
    values are combined through the library's collectives."""
    out = {}
    linears = [m for m in model if isinstance(m, nn.Linear)]
    # Fisher blocks: unnormalised sums add up over ranks
    fm = _fisher(model, x, t, asdl.SHAPE_KRON, data_size=1)
    if distributed:
        fm.reduce_fisher(linears, 'kron', 'A', all_reduce=True)
        fm.reduce_fisher(linears, 'kron', 'B', all_reduce=True)
    out['kron_A'] = linears[0].fisher.kron.A.clone()
    out['kron_B'] = linears[1].fisher.kron.B.clone()
    out['kron_A_of'] = [m.fisher.kron.A.clone() for m in linears]
    # partitioned reduction: module i is complete on rank i only
    fm = _fisher(model, x, t, asdl.SHAPE_LAYER_WISE, data_size=1)
    if distributed:
        fm.reduce_scatter_fisher([[m] for m in linears], 'data')
        out['layer_block'] = linears[rank].fisher.data.clone()
    else:
        out['layer_blocks'] = [m.fisher.data.clone() for m in linears]
    # Fisher-vector product
    fm = _fisher(model, x, t, asdl.SHAPE_FULL, fvp=True, vec=_probe(model), data_size=1)
    if distributed:
        fm.reduce_fvp(asdl.SHAPE_FULL, all_reduce=True)
    out['fvp'] = model.fvp.get_flatten_vector().clone()
    # packed vector sum
    v = _probe(model).mul_(float(rank + 1) if distributed else float(sum(range(1, world + 1))))
    out['vector'] = (asdl.reduce_vectors(v, all_reduce=True) if distributed else v).get_flatten_vector().clone()
    # gradient over a loader, averaged over ranks (equal shard sizes: the mean of means is the mean)
    model.zero_grad()
    loader = DataLoader(TensorDataset(x, t), batch_size=2)
    out['loader_loss'] = asdl.data_loader_gradient(model, lambda y, tt: F.cross_entropy(y, tt, reduction='sum'), loader,
                                                   is_distributed=distributed, all_reduce=True)
    out['loader_grad'] = torch.cat([p.grad.flatten() for p in model.parameters()]).clone()
    model.zero_grad()
    return out


def _worker(rank, world, port, out_dir):
    dist.init_process_group('gloo', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world,
                            timeout=timedelta(seconds=60))
    try:
        x, t = _data()
        n = x.shape[0] // world
        model = _net()
        out = _results(model, x[rank * n:(rank + 1) * n], t[rank * n:(rank + 1) * n], world, rank, distributed=True)
        # rank-parallel kernel assembly over the FULL inputs (every rank computes its share of the blocks)
        out['ntk'] = K.batch(K.empirical_direct_ntk, model, x, batch_size=2, is_distributed=True, gather_type='all')
        # power iteration on the summed Fisher with broadcast start vectors: same top eigenvalue on both ranks
        local = _fisher(model, x[rank * n:(rank + 1) * n], t[rank * n:(rank + 1) * n], asdl.SHAPE_FULL, data_size=1)

        def summed_fvp(vec):
            local.forward_and_backward(fvp=True, vec=vec, data_size=1)
            local.reduce_fvp(asdl.SHAPE_FULL, all_reduce=True)
            return local.load_fvp(asdl.SHAPE_FULL)

        eigvals, _ = asdl.power_method(summed_fvp, model, top_n=1, max_iters=300, tol=1e-9, is_distributed=True)
        out['top_eig'] = float(eigvals[0])
        xs, ts = x[rank * n:(rank + 1) * n], t[rank * n:(rank + 1) * n]
        # MatrixManager: per-rank means, one packed message, average over ranks
        mm = asdl.MatrixManager(model, asdl.FISHER_EMP)
        _manager_fisher(model, xs, ts, n)
        mm.accumulate_matrices('run')
        mm.reduce_matrices('run', all_reduce=True)
        out['manager'] = mm.get_matrix(model[0], asdl.FISHER_EMP, 'run').data.clone()
        # function-space solvers
        torch.manual_seed(7)
        K.kernel_free_cross_entropy(model, xs, ts, damping=1e-2, tol=1e-8, is_distributed=True)
        out['kernel_free'] = torch.cat([p.grad.flatten() for p in model.parameters()]).clone()
        torch.manual_seed(11 + rank)
        out['kernel_eig'] = float(K.kernel_eigenvalues(model, xs, top_n=1, max_iters=500, tol=1e-10, is_distributed=True)[0])
        class_kernels = K.batch(K.empirical_class_wise_direct_ntk, model, x, batch_size=2).permute(2, 0, 1).contiguous()
        split = [[0, 1], [2]][rank]                      # 3 classes over 2 ranks
        damped = class_kernels[split] / x.shape[0] + 1e-2 * torch.eye(x.shape[0])
        K.parallel_efficient_natural_gradient_cross_entropy(model, xs, ts, damped, damping=1e-2)
        out['parallel_ngd'] = torch.cat([p.grad.flatten() for p in model.parameters()]).clone()
        # explicit partitions (the reference's older interface): module r is summed onto rank r
        linears = [m for m in model if isinstance(m, nn.Linear)]
        gm = asdl.KfacGradientMaker(model, asdl.PreconditioningConfig(data_size=n, damping=1e-2, ema_decay=0.5),
                                    fisher_type=asdl.FISHER_EMP, module_partitions=[[m] for m in linears])
        dummy = gm.setup_model_call(model, xs)
        gm.setup_loss_call(F.cross_entropy, dummy, ts)
        gm.delegate_forward_and_backward(gm.fisher_maker, data_size=1, scale=1., accumulate=False)
        gm.reduce_scatter_curvature_module_partitions()
        gm.wait_all_curvature_sync()
        out['partition_A'] = linears[rank].fisher.kron.A.clone()
        assert gm.reduce_curvature('no_such_module') == [] and gm.computational_cost(asdl.SHAPE_KRON, linears[rank]) > 0
        torch.save(out, os.path.join(out_dir, f'rank{rank}.pt'))
    finally:
        dist.destroy_process_group()


def test_distributed_entry_points_match_single_process():
    world = 2
    with tempfile.TemporaryDirectory() as out_dir:
        mp.spawn(_worker, args=(world, _free_port(), out_dir), nprocs=world, join=True)
        ranks = [torch.load(os.path.join(out_dir, f'rank{r}.pt'), weights_only=False) for r in range(world)]
    x, t = _data()
    model = _net()
    single = _results(model, x, t, world)
    for r in ranks:
        for key in ('kron_A', 'kron_B', 'fvp', 'vector', 'loader_grad'):
            torch.testing.assert_close(r[key], single[key], rtol=1e-4, atol=1e-6)
        assert abs(r['loader_loss'] - single['loader_loss']) < 1e-5
    for rank, r in enumerate(ranks):
        torch.testing.assert_close(r['layer_block'], single['layer_blocks'][rank], rtol=1e-4, atol=1e-6)
        torch.testing.assert_close(r['partition_A'], single['kron_A_of'][rank], rtol=1e-4, atol=1e-6)
    ntk = K.batch(K.empirical_direct_ntk, model, x, batch_size=2)
    for r in ranks:
        torch.testing.assert_close(r['ntk'], ntk, rtol=1e-4, atol=1e-6)
    full = _fisher(model, x, t, asdl.SHAPE_FULL, data_size=1)
    top = torch.linalg.eigvalsh(model.fisher.data)[-1].item()
    assert abs(ranks[0]['top_eig'] - ranks[1]['top_eig']) < 1e-6 * top
    assert abs(ranks[0]['top_eig'] - top) < 1e-3 * top
    del full
    fresh = _net()
    _manager_fisher(fresh, x, t, x.shape[0])
    K.kernel_free_cross_entropy(model, x, t, damping=1e-2, tol=1e-8)
    kernel_free = torch.cat([p.grad.flatten() for p in model.parameters()]).clone()
    jac_kernel = K.batch(K.empirical_direct_ntk, model, x, batch_size=2)           # n x n x c x c
    n, c = x.shape[0], 3
    top_kernel = torch.linalg.eigvalsh(jac_kernel.permute(0, 2, 1, 3).reshape(n * c, n * c))[-1].item()
    class_kernels = K.batch(K.empirical_class_wise_direct_ntk, model, x, batch_size=2).permute(2, 0, 1).contiguous()
    K.efficient_natural_gradient_cross_entropy(model, x, t, class_kernels / n + 1e-2 * torch.eye(n), damping=1e-2)
    ngd = torch.cat([p.grad.flatten() for p in model.parameters()]).clone()
    for r in ranks:
        torch.testing.assert_close(r['manager'], getattr(fresh[0], asdl.FISHER_EMP).data, rtol=1e-4, atol=1e-6)
        torch.testing.assert_close(r['kernel_free'], kernel_free, rtol=1e-3, atol=1e-5)
        assert abs(r['kernel_eig'] - top_kernel) < 1e-3 * top_kernel
        torch.testing.assert_close(r['parallel_ngd'], ngd, rtol=1e-3, atol=1e-5)
