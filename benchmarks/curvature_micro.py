"""The data-parallel curvature path in isolation, fused kernels against library calls.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29533 benchmarks/curvature_micro.py --sizes 256 512 1024 2048 4096 8192

Work of one iteration on W ranks: W Kronecker factors of size n, factor r owned by rank r.  Every
rank holds activations a [B, n] (bf16, N(0,1)) and contributes a^T a / (B W) to every factor; the
owner adds damping, inverts in fp32 and applies the inverse to an n x n gradient; every rank ends
up with all W preconditioned gradients.

  fused    --transport pull (default): tcgen05 SYRKs whose epilogues store lower-triangular tiles into this
           rank's own symmetric buffer, bounded flag barrier, owner-side kernel that reads every rank's
           share with coalesced loads over NVLink while it sums and mirrors (reduce + transfer in one
           kernel), grouped Cholesky inverse on the tensor cores, tcgen05 GEMM, coalesced broadcast of the
           result into every rank's buffer (multimem.st through the switch where mapped), barrier.
           --transport push: the SYRK epilogue stores its tiles into this rank's slot on the owner and the
           GEMM epilogue stores the result into every rank's buffer (compute + send in one kernel); a
           lane of the epilogue holds a row of the accumulator, so these are 16-byte stores over NVLink.
  library  torch.matmul (cuBLAS, fp32 output) + dist.all_reduce (NCCL) + torch.linalg.cholesky /
           cholesky_inverse (cuSOLVER) + torch.matmul + dist.all_gather.

One JSON line per size from rank 0: device time (CUDA events, max over ranks, median of the
iterations) of both arms and the roofline of the fused arm: the slower of its tensor-core FLOPs at
the measured GEMM peak and the bytes each GPU must send over NVLink at 770 GB/s (the inverse is
fp32 CUDA-core work and is reported separately).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from asdl_b200 import ops  # noqa: E402
from asdl_b200.parallel.symmetric import SymmetricArena  # noqa: E402

NVLINK_BPS = 770e9


def gemm_peak():
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)['bf16_tflops'] * 1e12, 'measured'
    return 1.59e15, 'fallback'


def timed(fn, iters, warmup, world, flush):
    for _ in range(warmup):
        fn()
    out = []
    for _ in range(iters):
        flush.zero_()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    t = torch.tensor(out, device='cuda', dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.median().item()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--sizes', type=int, nargs='+', default=[256, 512, 1024, 2048, 4096, 8192])
    ap.add_argument('--batch', type=int, default=4096)
    ap.add_argument('--iters', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--damping', type=float, default=1e-3)
    ap.add_argument('--transport', default='pull', choices=['pull', 'push'],
                    help="pull: SYRK epilogues store locally, the owner reads every rank's share with coalesced peer loads "
                         "while it sums, and the result is pushed by the coalesced broadcast kernel; "
                         "push: the SYRK and GEMM epilogues store straight into the other GPUs' buffers")
    args = ap.parse_args()
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    ext = ops.extension()
    peak, src = gemm_peak()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    B = args.batch
    for n in args.sizes:
        torch.manual_seed(100 + rank)
        a = torch.randn(B, n, device=dev).to(torch.bfloat16)
        grad = torch.randn(n, n, device=dev)
        nn_ = n * n
        arena = SymmetricArena(3 * world * nn_ + 1024) if world > 1 else SymmetricArena.local_group(3 * nn_ + 1024, 1)[0]
        f_off = [arena.alloc(n, n) for _ in range(world)]   # factor r (only the copy on rank r is used)
        slots_off, _ = arena.alloc(world, n, n)             # slot q: the statistics that rank q stored here
        y_off = [arena.alloc(n, n) for _ in range(world)]   # preconditioned gradient r (replicated)
        slot_table = torch.tensor([[f_off[rank][0], slots_off, n]], dtype=torch.int64, device=dev)
        inv = torch.empty(n, n, device=dev)
        ld = (n + 7) // 8 * 8
        mk = lambda: torch.empty(n, ld, device=dev, dtype=torch.bfloat16)  # noqa: E731
        g_hi, g_lo, i_hi, i_lo = mk(), mk(), mk(), mk()
        damp = torch.full((1,), args.damping, device=dev)
        peers_y = [arena.ptr(r, y_off[rank][0]) for r in range(world) if r != rank]

        pull_table = torch.tensor([[f_off[rank][0], slots_off + rank * nn_, n]], dtype=torch.int64, device=dev)
        y_segs = arena.segments([(y_off[rank][0], nn_)])
        pull = args.transport == 'pull'

        def fused():
            for k in range(world):
                r = (rank + 1 + k) % world
                if pull:   # region r of this rank's own buffer holds its share of factor r
                    target = arena.ptr(rank, slots_off + r * nn_)
                else:      # staggered: at any time every owner receives from one peer
                    target = arena.ptr(r, slots_off + rank * nn_)
                ext.umma_gemm_to_ptr([a], [a], False, False, target, n,
                                     1.0 / (B * world), True, 3, [], 0)   # lower-triangular tiles, plain stores
            arena.barrier()
            if pull:
                arena.pull_slots(pull_table, n, 0.0)
            else:
                arena.reduce_slots(slot_table, nn_, n, 0.0)
            ops.spd_inverse_grouped([f_off[rank][1]], [inv], damp)
            ext.cast_pad_bf16(inv, i_hi, i_lo, 1.0)
            ext.cast_pad_bf16(grad, g_hi, g_lo, 1.0)
            gh, gl, ih, il = g_hi[:, :n], g_lo[:, :n], i_hi[:, :n], i_lo[:, :n]
            # Y = G A^-1: G is [n(M), n(K)] K-major; A^-1 symmetric, read as [K, N] MN-major
            ext.umma_gemm_to_ptr([gh, gh, gl], [ih, il, ih], True, False, arena.ptr(rank, y_off[rank][0]), n,
                                 1.0, False, False, [] if pull else peers_y, 0)
            if pull and world > 1:
                arena.bcast_segments(y_segs)
            arena.barrier()

        stack = torch.empty(world, n, n, device=dev)
        ys = [torch.empty(n, n, device=dev) for _ in range(world)]
        eye = torch.eye(n, device=dev)
        af = a.float()

        def library():
            for r in range(world):
                try:
                    torch.mm(a.T, a, out_dtype=torch.float32, out=stack[r])
                except (TypeError, RuntimeError):
                    torch.mm(af.T, af, out=stack[r])
            stack.div_(B * world)
            if world > 1:
                dist.all_reduce(stack)
            m = stack[rank] + args.damping * eye
            minv = torch.cholesky_inverse(torch.linalg.cholesky(m))
            y = grad @ minv
            if world > 1:
                dist.all_gather(ys, y)
            else:
                ys[0].copy_(y)

        ms_fused = timed(fused, args.iters, args.warmup, world, flush)
        ops.check_status()
        ms_lib = timed(library, args.iters, args.warmup, world, flush)
        ms_inv = timed(lambda: ops.spd_inverse_grouped([f_off[rank][1]], [inv], damp), args.iters, args.warmup, world, flush)
        err = ((y_off[rank][1] - ys[rank]).norm() / ys[rank].norm()).item()
        if world > 1:  # a replicated copy written by a peer's epilogue
            other = (rank + 1) % world
            err = max(err, ((y_off[other][1] - ys[other]).norm() / ys[other].norm()).item())
        # tensor-core FLOPs per GPU: W SYRKs (lower triangle ~ half of 2 B n^2) + 3 passes of 2 n^3
        flops = world * B * n * n + 3 * 2.0 * n ** 3
        wire = (world - 1) * (nn_ / 2 + nn_) * 4.0   # exported triangles of W-1 factors + replicated result
        roof_ms = max(flops / peak, wire / NVLINK_BPS) * 1e3
        if rank == 0:
            print(json.dumps({
                'case': 'curvature_micro', 'n': n, 'batch': B, 'n_gpus': world, 'transport': args.transport,
                'fused_ms': round(ms_fused, 4),
                'library_ms': round(ms_lib, 4), 'speedup': round(ms_lib / ms_fused, 2),
                'inverse_ms_in_fused': round(ms_inv, 4),
                'roofline_ms_excl_inverse': round(roof_ms, 4),
                'frac_of_roofline_excl_inverse': round(roof_ms / max(ms_fused - ms_inv, 1e-6), 3),
                'peak_source': src, 'rel_diff_fused_vs_library': err}), flush=True)
        del arena
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
