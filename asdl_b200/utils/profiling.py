"""In-process phase timing: every named range of the library (the NVTX ranges ``cov_kron_A``,
``inv_*``, ``reduce_scatter_curvature``, ``kfac_precondition`` ...) and of user code is timed on the
device with CUDA events while a :class:`PhaseProfile` is active, and summarised as calls / mean /
standard deviation per name.

The reference gets the same table offline: it wraps phases in NVTX ranges
(examples/prof/profiling.py:7-23), records a trace with an external profiler and joins range and
kernel tables of the exported database (examples/prof/parse_nvtx_events.py:28-111).  Here the
ranges carry their own events, so the table needs no external tool and no trace file; the NVTX
ranges stay, for those who do record a trace (benchmarks/nsys_nvtx_report.py reads its export).

    with PhaseProfile() as prof:
        for _ in range(20):
            step()
    print(prof.report())

Events are recorded on the current stream and resolved when the table is asked for (one
synchronisation at the end, none per range).  Ranges entered while the stream is being captured
into a CUDA graph are skipped: a replayed graph has no host-visible ranges.  On CPU tensors the
ranges are timed with the wall clock.
"""
import math
import time
from contextlib import contextmanager
from typing import Callable, Dict, List, Optional, Sequence

import torch

__all__ = ['PhaseProfile', 'time_funcs', 'active_profile']

_active: Optional['PhaseProfile'] = None


def active_profile() -> Optional['PhaseProfile']:
    """The profile that currently collects ranges, or None."""
    return _active


class PhaseProfile:
    """Collects named ranges while it is the active profile (``with PhaseProfile() as prof``).

    Args:
        cuda: time with CUDA events on the current stream (default: whether CUDA is available).
        skip_first: leave the first ``skip_first`` occurrences of every name out of the statistics
            (allocator warm-up, lazy initialisation).
    """

    def __init__(self, cuda: Optional[bool] = None, skip_first: int = 0):
        self.cuda = torch.cuda.is_available() if cuda is None else bool(cuda)
        self.skip_first = int(skip_first)
        self._pending: List[tuple] = []          # (name, start event, end event) on CUDA
        self._times: Dict[str, List[float]] = {}  # name -> milliseconds per call, in call order
        self._previous = None

    # -- activation ----------------------------------------------------------------------------
    def __enter__(self):
        global _active
        self._previous, _active = _active, self
        return self

    def __exit__(self, *exc):
        global _active
        _active = self._previous
        return False

    # -- recording -----------------------------------------------------------------------------
    @contextmanager
    def range(self, name: str):
        if self.cuda:
            if torch.cuda.is_current_stream_capturing():
                yield
                return
            start = torch.cuda.Event(enable_timing=True)
            end = torch.cuda.Event(enable_timing=True)
            start.record()
            try:
                yield
            finally:
                end.record()
                self._pending.append((name, start, end))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._times.setdefault(name, []).append(1e3 * (time.perf_counter() - t0))

    def _resolve(self):
        if self._pending:
            torch.cuda.synchronize()
            for name, start, end in self._pending:
                self._times.setdefault(name, []).append(start.elapsed_time(end))
            self._pending.clear()

    # -- results -------------------------------------------------------------------------------
    def table(self) -> Dict[str, Dict[str, float]]:
        """``{name: {'ncalls', 'mean_ms', 'stdev_ms', 'total_ms', 'min_ms', 'max_ms'}}`` in order of first use."""
        self._resolve()
        out = {}
        for name, values in self._times.items():
            values = values[self.skip_first:]
            if not values:
                continue
            mean = sum(values) / len(values)
            var = sum((v - mean) ** 2 for v in values) / (len(values) - 1) if len(values) > 1 else 0.0
            out[name] = {'ncalls': len(values), 'mean_ms': mean, 'stdev_ms': math.sqrt(var), 'total_ms': sum(values),
                         'min_ms': min(values), 'max_ms': max(values)}
        return out

    def report(self, sort_by_total: bool = True) -> str:
        rows = list(self.table().items())
        if sort_by_total:
            rows.sort(key=lambda kv: -kv[1]['total_ms'])
        width = max([len(name) for name, _ in rows] + [5])
        lines = [f'{"range":<{width}}  {"calls":>6}  {"mean ms":>10}  {"stdev ms":>10}  {"total ms":>10}']
        for name, r in rows:
            lines.append(f'{name:<{width}}  {r["ncalls"]:>6d}  {r["mean_ms"]:>10.4f}  {r["stdev_ms"]:>10.4f}  '
                         f'{r["total_ms"]:>10.3f}')
        return '\n'.join(lines)

    def reduce_max(self, group=None) -> Dict[str, Dict[str, float]]:
        """The table with every figure replaced by its maximum over the ranks of ``group`` (the slowest
        rank defines a phase's time in a data-parallel step).  Ranks must have timed the same names."""
        import torch.distributed as dist
        table = self.table()
        if not (dist.is_available() and dist.is_initialized()):
            return table
        names = sorted(table)
        keys = ('mean_ms', 'stdev_ms', 'total_ms', 'min_ms', 'max_ms')
        device = torch.device('cuda', torch.cuda.current_device()) if dist.get_backend(group) == 'nccl' else 'cpu'
        flat = torch.tensor([[table[n][k] for k in keys] for n in names], dtype=torch.float64, device=device)
        dist.all_reduce(flat, op=dist.ReduceOp.MAX, group=group)
        for i, n in enumerate(names):
            for j, k in enumerate(keys):
                table[n][k] = float(flat[i, j])
        return table


def time_funcs(funcs: Sequence[Callable[[], object]], name: str = '', func_names: Optional[Sequence[str]] = None,
               num_iters: int = 100, num_warmups: int = 5, emit_nvtx: bool = False) -> Dict[str, Dict[str, float]]:
    """Calls ``funcs`` one after the other ``num_iters`` times (after ``num_warmups`` untimed rounds) and
    returns the :meth:`PhaseProfile.table` of ``<name><function name>`` and of the whole round
    ``<name>Iter``.  Every call sits in an NVTX range of the same name and the timed part sits between
    ``cudaProfilerStart`` / ``Stop``, so an external profiler started with capture range "cudaProfilerApi"
    sees the same phases (``emit_nvtx`` adds autograd's per-operator ranges for it)."""
    from . import nvtx_range
    if func_names is None:
        func_names = [f.__name__ for f in funcs]
    cuda = torch.cuda.is_available()
    with nvtx_range(name + 'Warmup'):
        for _ in range(num_warmups):
            for f in funcs:
                f()
    if cuda:
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
    try:
        with PhaseProfile() as prof:
            for _ in range(num_iters):
                with nvtx_range(name + 'Iter'):
                    for f, fname in zip(funcs, func_names):
                        with nvtx_range(name + fname):
                            if emit_nvtx and cuda:
                                with torch.autograd.profiler.emit_nvtx():
                                    f()
                            else:
                                f()
            table = prof.table()
    finally:
        if cuda:
            torch.cuda.profiler.stop()
    return table
