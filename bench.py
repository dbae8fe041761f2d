"""Headline benchmark: ResNet-50 K-FAC training throughput (images/s) on N B200 GPUs of one node.

    python bench.py --gpus 1 --steps 40 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 40 --warmup 5
    python bench.py --impl reference ...      # the unmodified reference package, same workload
    python bench.py --precision tf32 ...      # this library at the reference's precision (fp32 + TF32)
    python bench.py --impl reference-autocast # the reference under bf16 autocast (shimmed, see below)

Workload (both arms): torchvision-topology ResNet-50 with random initialisation, synthetic
N(0,1) images [32, 3, 224, 224] per GPU and uniform labels over 1000 classes, K-FAC with damping
1e-3, curvature update every 10 steps, inverse update every 100 steps, factor EMA 0.95
(``ema_decay=0.05``), Monte-Carlo Fisher, SGD step included.  Weak scaling: the per-GPU batch is
fixed.  This arm runs bf16 autocast / channels_last with fp32 factors and inverses; the reference
arm runs its stock fp32 path (its hooks cannot consume bf16 activations).

Two numbers are reported.  ``value`` is timed on the device with CUDA events around exactly K
steps whose inputs already sit in device memory; ``e2e`` repeats K steps through the same public
API but copies every step's batch from pinned host memory and reads the loss back to the host.
One JSON line is printed by rank 0.

Attribution aids (none of them changes the two timed regions):
  * ``--precision tf32`` runs this library without autocast (fp32 activations, TF32 convolutions and
    matrix products, statistics from bf16 hi/lo splits): the same precision as the stock reference.
  * ``--impl reference-autocast`` is a SECOND reference line, never a replacement of the stock
    one: the reference package under bf16 autocast.  Its hooks cannot consume bf16 activations
    (its factor products would run in bf16 and its Cholesky rejects bf16), so the two hook entry
    points of its ``Operation`` class are wrapped here, at run time, to up-cast what they receive
    to fp32.  Nothing under ``baseline/_ref`` is modified.
  * ``phases``: after the timed regions single steps of each kind (plain / with curvature / with
    curvature and inverses) are timed with CUDA events, the maker's step counter being set to a
    step of that kind through its public ``state``; ``amortised_ms_per_step_100`` is
    (89 plain + 10 curvature + 1 inverse step) / 100, the figure a 100-step window would show.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PER_GPU_BATCH = 32
NUM_CLASSES = 1000
IMAGE = (3, 224, 224)
L2_FLUSH_BYTES = 256 << 20


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=40)
    ap.add_argument('--warmup', type=int, default=5)
    ap.add_argument('--impl', choices=['ours', 'reference', 'reference-autocast'], default='ours')
    ap.add_argument('--precision', choices=['bf16', 'tf32'], default='bf16',
                    help="compute precision of this library's arm: bf16 autocast (default) or fp32 with TF32")
    ap.add_argument('--no-phases', action='store_true', help='skip the per-step-kind timing after the timed regions')
    ap.add_argument('--grad-overlap', choices=['auto', 'on', 'off'], default='auto',
                    help='bucketed gradient reduction during the backward pass (multi-GPU runs of this library)')
    ap.add_argument('--no-graph', action='store_true', help='disable CUDA-graph replay of plain steps')
    ap.add_argument('--nvtx', action='store_true',
                    help="wrap every device-timed step in an NVTX range ('plain_step' / 'curvature_step')")
    ap.add_argument('--precond-precision', default='bf16x3', choices=['bf16', 'bf16x3'])
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks / throttle reasons of the job's GPUs while the timed region runs: an NVML thread
    (a reading every 10 ms, no start-up delay, so even a 150 ms region gets a dozen samples per GPU), or an
    ``nvidia-smi -lms`` child process where the NVML bindings are missing.  Reads only; sets nothing."""
    QUERY = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,'
             'clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,'
             'clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')
    REASON_BITS = {'sw_power_cap': 0x4, 'hw_slowdown': 0x8, 'sw_thermal_slowdown': 0x20, 'hw_thermal_slowdown': 0x40}

    def __init__(self):
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []
        self.max_clocks = []
        self.reason_mask = 0
        self._stop = False

    def _nvml_handles(self, gpu_indices):
        import pynvml
        pynvml.nvmlInit()
        handles = []
        for i in gpu_indices:
            try:
                uuid = str(torch.cuda.get_device_properties(i).uuid)
                handles.append(pynvml.nvmlDeviceGetHandleByUUID(('GPU-' + uuid) if not uuid.startswith('GPU-') else uuid))
            except Exception:
                handles.append(pynvml.nvmlDeviceGetHandleByIndex(i))
        return pynvml, handles

    def _run(self, pynvml, handles):
        reasons = getattr(pynvml, 'nvmlDeviceGetCurrentClocksEventReasons', None) or \
            getattr(pynvml, 'nvmlDeviceGetCurrentClocksThrottleReasons')
        while not self._stop:
            for h in handles:
                try:
                    self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    self.reason_mask |= int(reasons(h))
                except Exception:
                    pass
            time.sleep(0.01)

    def start(self, gpu_indices=(0,)):
        try:
            pynvml, handles = self._nvml_handles(list(gpu_indices))
            self.max_clocks = [float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)) for h in handles]
            self.thread = threading.Thread(target=self._run, args=(pynvml, handles), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix='.csv')
            os.close(fd)
            self.proc = subprocess.Popen(
                ['nvidia-smi', f'--query-gpu={self.QUERY}', '--format=csv,noheader,nounits', '-lms', '200'],
                stdout=open(self.path, 'w'), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, gpu_indices):
        out = {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': []}
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            if self.samples:
                out['sm_mhz'] = statistics.median(self.samples)
                out['sm_max_mhz'] = max(self.max_clocks) if self.max_clocks else None
                out['samples'] = len(self.samples)
                out['source'] = 'nvml, every 10 ms during the timed region'
            out['reasons'] = sorted(n for n, bit in self.REASON_BITS.items() if self.reason_mask & bit)
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, max_clocks, reasons = [], [], set()
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(',')]
                if len(parts) < 9 or not parts[0].isdigit() or int(parts[0]) not in gpu_indices:
                    continue
                clocks.append(float(parts[1]))
                max_clocks.append(float(parts[2]))
                for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown',
                                      'sw_power_cap'), parts[5:9]):
                    if val.lower().startswith('active'):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if clocks:
            out['sm_mhz'] = statistics.median(clocks)
            out['sm_max_mhz'] = max(max_clocks)
            out['samples'] = len(clocks)
            out['source'] = 'nvidia-smi -lms 200'
        out['reasons'] = sorted(reasons)
        return out


def init_distributed(n):
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    assert world == n, f'--gpus {n} but WORLD_SIZE={world}'
    return rank, local, world


def make_batches(count, device, seed, channels_last=False):
    g = torch.Generator().manual_seed(seed)
    fmt = torch.channels_last if channels_last else torch.contiguous_format
    xs = [torch.randn(PER_GPU_BATCH, *IMAGE, generator=g).contiguous(memory_format=fmt).pin_memory()
          for _ in range(count)]
    ts = [torch.randint(0, NUM_CLASSES, (PER_GPU_BATCH,), generator=g).pin_memory() for _ in range(count)]
    return xs, ts


# ----------------------------------------------------------------------------------------------
# the two arms: each returns step(x_dev, t_dev) -> loss tensor, plus a launch counter
# ----------------------------------------------------------------------------------------------
def build_ours(args, device, world):
    import asdl_b200 as asdl
    from asdl_b200.models import resnet50
    torch.manual_seed(0)
    model = resnet50(NUM_CLASSES).to(device).to(memory_format=torch.channels_last)
    config = asdl.PreconditioningConfig(data_size=PER_GPU_BATCH, damping=1e-3, ema_decay=0.05,
                                        curvature_upd_interval=10, preconditioner_upd_interval=100)
    gm = asdl.FusedKfacGradientMaker(model, config, precond_precision=args.precond_precision,
                                     cuda_graph=not args.no_graph,
                                     overlap_grad_reduce={'auto': 'auto', 'on': True, 'off': False}[args.grad_overlap])
    opt = torch.optim.SGD(model.parameters(), lr=1e-4, momentum=0.9)

    bf16 = args.precision == 'bf16'
    if not bf16:
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True

    def model_fn(x):
        with torch.autocast('cuda', dtype=torch.bfloat16, enabled=bf16):
            return model(x)

    def step(x, t):
        opt.zero_grad(set_to_none=True)
        dummy = gm.setup_model_call(model_fn, x)
        gm.setup_loss_call(F.cross_entropy, dummy, t)
        _, loss = gm.forward_and_backward()
        opt.step()
        return loss

    def launches():  # host-issued launches plus those replayed from the captured step graph
        return asdl.ops.extension().launch_count() + gm.replayed_launches

    def to_device(x, t):
        return (x.to(device, non_blocking=True).contiguous(memory_format=torch.channels_last),
                t.to(device, non_blocking=True))

    return step, launches, to_device, ('bf16' if bf16 else 'fp32 (tf32 matmul/conv)'), gm


def build_reference(args, device, world):
    ref_dir = os.path.join(ROOT, 'baseline', '_ref')
    if not os.path.isdir(os.path.join(ref_dir, 'asdl')):
        raise ImportError('reference package is not installed under baseline/_ref')
    sys.path.insert(0, ref_dir)
    import asdl  # the unmodified reference
    import torchvision
    torch.manual_seed(0)
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True
    model = torchvision.models.resnet50(num_classes=NUM_CLASSES)
    for m in model.modules():  # its norm-layer statistics read the layer output after the forward pass
        if isinstance(m, nn.ReLU):
            m.inplace = False
    model = model.to(device)
    config = asdl.PreconditioningConfig(data_size=PER_GPU_BATCH, damping=1e-3, ema_decay=0.05,
                                        curvature_upd_interval=10, preconditioner_upd_interval=100)
    gm = asdl.KfacGradientMaker(model, config)
    opt = torch.optim.SGD(model.parameters(), lr=1e-4, momentum=0.9)
    autocast = args.impl == 'reference-autocast'
    if autocast:
        # second reference line: bf16 autocast, with the tensors that reach the reference's hooks
        # up-cast to fp32 (wrappers installed here; the package itself stays as it is)
        from asdl.operations.operation import Operation

        def upcast(v):
            if isinstance(v, torch.Tensor) and v.dtype in (torch.bfloat16, torch.float16):
                return v.float()
            if isinstance(v, (tuple, list)):
                return type(v)(upcast(e) for e in v)
            return v

        fwd, bwd = Operation.forward_post_process, Operation.backward_pre_process

        def forward_post_process(self, in_data, out_data):
            with torch.autocast('cuda', enabled=False):
                return fwd(self, upcast(in_data), upcast(out_data))

        def backward_pre_process(self, out_grads, vector=None):
            with torch.autocast('cuda', enabled=False):
                return bwd(self, upcast(out_grads), vector)

        Operation.forward_post_process = forward_post_process
        Operation.backward_pre_process = backward_pre_process

    def model_fn(x):
        with torch.autocast('cuda', dtype=torch.bfloat16, enabled=autocast):
            return model(x)

    def step(x, t):
        opt.zero_grad(set_to_none=True)
        dummy = gm.setup_model_call(model_fn, x)
        gm.setup_loss_call(F.cross_entropy, dummy, t)
        _, loss = gm.forward_and_backward()
        opt.step()
        return loss

    def to_device(x, t):
        return x.to(device, non_blocking=True), t.to(device, non_blocking=True)

    dtype = 'bf16 autocast, hook tensors up-cast to fp32 (second reference line)' if autocast \
        else 'fp32 (tf32 matmul/conv)'
    return step, (lambda: 0), to_device, dtype, gm


def measure_phases(step, gm, dev_batches, flush):
    """Device time of one step of each kind, measured after the timed regions.  The step kind is
    chosen by setting the maker's step counter (curvature every 10 steps, inverses every 100)."""
    def timed(step_index):
        gm.state['step'] = step_index
        flush.zero_()
        x, t = dev_batches[step_index % len(dev_batches)]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step(x, t)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    saved = gm.state['step']
    plain = statistics.median(timed(1001 + i) for i in range(7))
    curvature = statistics.median(timed(1010 + 10 * i) for i in range(3))
    update = statistics.median(timed(1100 + 100 * i) for i in range(2))
    gm.state['step'] = saved
    return {'plain_ms': round(plain, 3), 'curvature_ms': round(curvature, 3), 'update_ms': round(update, 3),
            'amortised_ms_per_step_100': round((89 * plain + 10 * curvature + update) / 100, 3),
            'how': 'CUDA events around single steps after the timed regions; medians of 7 / 3 / 2 steps'}


def barrier(world):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def main():
    args = parse_args()
    args.warmup = max(args.warmup, 3)  # the step graphs are captured at the second step
    if args.impl != 'ours' and not os.path.isdir(os.path.join(ROOT, 'baseline', '_ref', 'asdl')):
        if int(os.environ.get('RANK', '0')) == 0:
            print(json.dumps({'impl': args.impl,
                              'unavailable': 'reference package not installed under baseline/_ref'}))
        return
    rank, local, world = init_distributed(args.gpus)
    device = torch.device('cuda', local)
    torch.backends.cudnn.benchmark = True  # both arms: fixed shapes, let cuDNN pick its kernels once
    build = build_ours if args.impl == 'ours' else build_reference
    step, launches, to_device, dtype, gm = build(args, device, world)

    n_host = 8
    xs, ts = make_batches(n_host, device, seed=1234 + rank, channels_last=args.impl == 'ours')
    dev_batches = [to_device(x, t) for x, t in zip(xs, ts)]
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)
    torch.cuda.synchronize()

    it = 0
    for _ in range(args.warmup):
        x, t = dev_batches[it % n_host]
        step(x, t)
        it += 1

    # ---- device-timed region: exactly K steps, inputs resident on the device ------------------
    sampler = ClockSampler()
    barrier(world)
    if rank == 0:
        sampler.start(list(range(world)))
    l0 = launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    e0.record()
    for _ in range(args.steps):
        flush.zero_()
        x, t = dev_batches[it % n_host]
        if args.nvtx:  # a profiler can select one kind of step by range name
            torch.cuda.nvtx.range_push('curvature_step' if it % 10 == 0 else 'plain_step')
        loss = step(x, t)
        if args.nvtx:
            torch.cuda.nvtx.range_pop()
        it += 1
    e1.record()
    barrier(world)
    ms = e0.elapsed_time(e1)
    n_launch = launches() - l0
    clocks = sampler.stop(list(range(world))) if rank == 0 else None

    # ---- end-to-end region: H2D of every batch from pinned memory, loss read back -------------
    barrier(world)
    t0 = time.perf_counter()
    h2d = d2h = 0
    last = 0.0
    # Input pipeline as a training loop would run it: two device buffers per input; the copy of the
    # next step's batch from pinned host memory is issued on a copy stream while the current step
    # computes, and the loss of a step is copied to pinned host memory behind it and read by the host
    # one step later (the host never idles the GPU to read a number).  Every batch is copied and every
    # loss is read inside the timed region; nothing is allocated in the loop.
    copy_stream = torch.cuda.Stream()
    main_stream = torch.cuda.current_stream()
    x_bufs = [torch.empty_like(dev_batches[0][0]) for _ in range(2)]
    t_bufs = [torch.empty_like(dev_batches[0][1]) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    loss_host = None
    loss_done = [torch.cuda.Event() for _ in range(2)]

    def fetch(index):
        slot = index % 2
        xh, th = xs[index % n_host], ts[index % n_host]
        copy_stream.wait_stream(main_stream)  # the step that last read this slot has been queued before
        with torch.cuda.stream(copy_stream):
            x_bufs[slot].copy_(xh, non_blocking=True)
            t_bufs[slot].copy_(th, non_blocking=True)
            ready[slot].record(copy_stream)
        return xh.numel() * xh.element_size() + th.numel() * th.element_size()

    first = it
    h2d += fetch(it)
    for k in range(args.steps):
        flush.zero_()
        slot = it % 2
        main_stream.wait_event(ready[slot])
        if k + 1 < args.steps:
            h2d += fetch(it + 1)
        loss = step(x_bufs[slot], t_bufs[slot])
        if loss_host is None:
            loss_host = torch.empty(2, dtype=loss.dtype).pin_memory()
        loss_host[k % 2].copy_(loss.detach(), non_blocking=True)
        loss_done[k % 2].record(main_stream)
        d2h += loss.element_size()
        if k >= 1:
            loss_done[(k - 1) % 2].synchronize()
            last = float(loss_host[(k - 1) % 2])
        it += 1
    loss_done[(args.steps - 1) % 2].synchronize()
    last = float(loss_host[(args.steps - 1) % 2])
    del first
    barrier(world)
    e2e_s = time.perf_counter() - t0

    phases = None
    if not args.no_phases:
        phases = measure_phases(step, gm, dev_batches, flush)
        barrier(world)
    if args.impl == 'ours':  # a kernel that gave up on a wait (peer barrier, pipeline stage) reports it here
        import asdl_b200
        asdl_b200.ops.check_status()
    times = torch.tensor([ms, e2e_s * 1e3], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = times.tolist()
    if rank == 0:
        global_batch = PER_GPU_BATCH * world
        value = args.steps * global_batch / (ms / 1e3)
        e2e_value = args.steps * global_batch / (e2e_ms / 1e3)
        out = {
            'metric': 'ResNet-50 K-FAC images/sec', 'value': round(value, 2), 'unit': 'images/s',
            'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': round(ms / args.steps, 3), 'higher_is_better': True, 'scaling': 'weak',
            'vs_baseline': None, 'dtype': dtype, 'data': 'synthetic N(0,1) images, uniform labels, random-init weights',
            'impl': args.impl,
            'config': {'model': 'resnet50', 'global_batch': global_batch, 'per_gpu_batch': PER_GPU_BATCH,
                       'image': list(IMAGE), 'parallelism': f'dp{world}', 'damping': 1e-3,
                       'curvature_upd_interval': 10, 'preconditioner_upd_interval': 100,
                       'ema_decay': 0.05, 'fisher': 'mc', 'optimizer': 'sgd(momentum=0.9) step included',
                       'l2': 'flushed every step by a 256 MiB memset; per-step activations exceed L2',
                       'cuda_graph': (not args.no_graph) if args.impl == 'ours' else False,
                       'e2e_loop': 'every batch copied from pinned memory into one of two static device buffers on a '
                                   'copy stream; every loss copied to pinned memory and read one step later',
                       **({'transport': ('nvlink symmetric memory: statistics pulled by the owners, gradients pull-reduced, '
                                         'preconditioned gradients broadcast; no NCCL call inside a step')}
                          if args.impl == 'ours' and world > 1 else {})},
            'e2e': {'value': round(e2e_value, 2), 'unit': 'images/s',
                    'ms_per_step': round(e2e_ms / args.steps, 3),
                    'h2d_bytes_per_step': h2d // args.steps, 'd2h_bytes_per_step': d2h // args.steps,
                    'last_loss': last},
            'gpu_launches': int(n_launch),
            'clocks': clocks,
            'phases': phases,
        }
        print(json.dumps(out), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
