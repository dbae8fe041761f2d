"""K-FAC with persistent curvature buffers and fused statistics kernels - the production path for
CUDA (it also runs, through the PyTorch implementations of :mod:`asdl_b200.ops`, on CPU, which is
how it is tested against :class:`KfacGradientMaker`).

Compared with the generic maker (same numerics, see asdl/precondition/natural_gradient.py:397-506
for the reference life cycle) nothing is allocated or re-packed per step:

  * every Kronecker factor lives in a persistent fp32 buffer; the statistics hooks launch one SYRK
    per factor whose epilogue performs the whole moving-average update
    ``A <- (1-e) A + e*s * a^T a`` (conv layers: bf16 im2col kernel -> SYRK, 1x1 convolutions on
    channels_last activations read the activation tensor in place);
  * convolution factors use the (kh, kw, c) column order of channels_last weights, so weight
    gradients are preconditioned through a view, without layout copies;
  * the pi-damping split and "is this factor still zero" tests stay on the device: no host
    synchronisation anywhere in a step;
  * inverses are cached as bf16 hi/lo pairs, the two-sided product B^-1 G A^-1 runs as chained
    tcgen05 GEMMs writing straight into ``param.grad``;
  * the 2x2 unit-wise blocks of all normalisation layers are applied with multi-tensor kernels.
"""
from typing import Dict, List

import os

import torch
import torch.nn as nn
import torch.distributed as dist
import torch.nn.functional as F

from .. import ops
from ..matrices import FISHER_EMP, FISHER_MC, SHAPE_KRON, SHAPE_UNIT_WISE
from ..symmatrix import SymMatrix, Kron, UnitWise
from ..utils import skip_param_grad, nvtx_range
from ..grad_maker import LOSS_CROSS_ENTROPY
from .natural_gradient import KfacGradientMaker
from .prec_grad_maker import PreconditioningConfig

__all__ = ['FusedKfacGradientMaker']

_NORMS = (nn.BatchNorm1d, nn.BatchNorm2d, nn.LayerNorm)


def _khwc_order(module):
    """True when the conv weight is stored channels_last, i.e. its rows are ordered (kh, kw, c)."""
    w = module.weight
    return (isinstance(module, nn.Conv2d) and w.shape[2] * w.shape[3] > 1
            and w.is_contiguous(memory_format=torch.channels_last) and not w.is_contiguous())


class _KronState:
    def __init__(self, name, module, device):
        self.name, self.module = name, module
        w = module.weight
        self.d_out = w.shape[0]
        self.d_in = w[0].numel()
        self.khwc = _khwc_order(module)
        self.has_bias = getattr(module, 'bias', None) is not None and module.bias.requires_grad
        f32 = dict(device=device, dtype=torch.float32)
        self.A = torch.zeros(self.d_in, self.d_in, **f32)
        self.B = torch.zeros(self.d_out, self.d_out, **f32)
        self.A_inv = torch.zeros(self.d_in, self.d_in, **f32)
        self.B_inv = torch.zeros(self.d_out, self.d_out, **f32)
        self.has_inv = False
        self.kron = Kron(self.A, self.B)
        module.fisher = SymMatrix(kron=self.kron)

    def grad_matrix(self):
        """(d_out x d_in view of the weight gradient, tensor to copy back into or None)."""
        g = self.module.weight.grad
        if g.ndim == 2:
            return g, None
        if self.khwc:
            if g.is_contiguous(memory_format=torch.channels_last):
                return g.permute(0, 2, 3, 1).reshape(self.d_out, self.d_in), None
            staged = g.contiguous(memory_format=torch.channels_last)
            return staged.permute(0, 2, 3, 1).reshape(self.d_out, self.d_in), staged
        if g.is_contiguous():
            return g.view(self.d_out, self.d_in), None
        staged = g.contiguous()
        return staged.view(self.d_out, self.d_in), staged


class _NormState:
    def __init__(self, name, module, device):
        self.name, self.module = name, module
        f = module.weight.numel()
        self.stats = torch.zeros(f, 2, 2, device=device, dtype=torch.float32)
        self.inv = torch.zeros(f, 2, 2, device=device, dtype=torch.float32)
        self.has_inv = False
        self.unit = UnitWise(self.stats)
        module.fisher = SymMatrix(unit=self.unit)


class FusedKfacGradientMaker(KfacGradientMaker):
    """Drop-in replacement of :class:`KfacGradientMaker` for Linear / Conv2d (Kronecker factors)
    and BatchNorm / LayerNorm (unit-wise 2x2 blocks) with persistent state.

    Extra args:
        precond_precision: ``'bf16x3'`` (default, ~2^-16 relative) or ``'bf16'`` for the products
            that apply the inverses.
        clone_norm_outputs: copy normalisation-layer outputs in the statistics hook (needed only
            if the model modifies them in place afterwards, e.g. ``ReLU(inplace=True)``).
        cuda_graph: replay whole steps from CUDA graphs: the plain step (forward, loss, backward,
            preconditioning), the step that also measures the curvature, and the step that measures
            it and inverts (the last two unless a sampling seed is configured).  They are captured
            at the first plain step after the first inverses exist; hyper-parameters (damping,
            moving-average weights) are read at capture time.  The registered tensor arguments are
            copied into static buffers before every replay, ``param.grad`` is (re)bound to static
            gradient tensors that each replay overwrites (so gradients are not accumulated across
            calls in this mode), and the returned output / loss are static tensors as well.
            CUDA runs, single process or data parallel with ``comm='symmetric'`` (all ranks must
            then see the same sequence of input shapes); anything else uses the eager path.
        grouped: apply the inverses of all layers with grouped launches (one staging kernel and
            two GEMM launches for the whole model) instead of a few launches per layer.
        comm: data-parallel transport.  ``'symmetric'`` keeps factors and gradients in NVLink
            symmetric memory and uses the library's own kernels: the statistics SYRKs store their
            lower-triangular tiles into this rank's buffer and the owner of a factor reads every
            rank's share over NVLink while it sums them into the running factor
            (``pull_statistics``), owners pull-reduce the gradients of their layers - bucket by
            bucket while the backward pass is still running with ``overlap_grad_reduce`` - and push
            their preconditioned gradients into every rank's gradient buffer with a coalesced
            broadcast kernel (``replicate_in_epilogue`` selects the GEMM epilogue instead).  ``'torch'`` uses
            ``torch.distributed`` collectives (any backend).  ``'auto'`` picks ``'symmetric'``
            for multi-rank CUDA runs.
        batch_statistics: record the statistics products of a curvature pass (one per Kronecker
            factor, asdl/operations/linear.py:77,89 and conv.py:80-103) and run them as ONE
            persistent tcgen05 launch after the backward pass instead of one launch per factor; the
            layer inputs and output gradients are kept alive until then.  Switch it off for models
            that modify a layer's input in place after the layer has run.
        overlap_grad_reduce: ``True`` / ``False`` / ``'auto'`` (on from ``OVERLAP_MIN_MB`` MiB of gradients
            per rank).  With ``comm='symmetric'``, reduce the gradients in buckets on a
            communication stream as the backward pass produces them (asdl/precondition/
            natural_gradient.py:753-757,814-829 reduce them after the backward pass): a tensor hook
            per parameter copies its gradient into the symmetric buffer, and when a bucket is
            complete one kernel on the communication stream exchanges flags with the peers and lets
            every owner pull the sum of its layers' gradients (``multimem.ld_reduce`` through the
            NVSwitch where the buffer has a multicast mapping).  The main stream joins the
            communication stream before preconditioning.  ``bucket_mb``: bucket size in MiB.
    Embedding layers are not handled here; list them in ``config.ignore_modules``.
    """

    #: gradient volume (MiB of fp32 gradients per rank) from which ``overlap_grad_reduce='auto'`` switches the
    #: bucketed reduction during the backward pass on
    OVERLAP_MIN_MB = 256.0

    #: Replicate the preconditioned gradients from the GEMM epilogue with ``multimem.st`` (one store through
    #: the NVSwitch instead of one store per peer).  Off: in the epilogue every lane of a warp holds a
    #: different row, so a store instruction is 32 separate 16-byte multicast writes, and on 2 GPUs the
    #: step was measured 0.48 ms SLOWER with it than with plain peer stores (7.11 vs 6.63 ms); the coalesced
    #: segment kernels (gradient pull, broadcast of the rest) do use the multicast mapping.
    multicast_epilogue = False

    #: Where the owners' preconditioned gradients of the Kronecker layers reach the other ranks: True - the
    #: final GEMM's epilogue stores every tile into every rank's buffer (no extra pass, but world - 1 peer
    #: stores of 16 bytes per lane); False - the epilogue stores locally and the coalesced broadcast kernel
    #: that pushes the remaining gradients (``multimem.st`` where the buffer has a multicast mapping) pushes
    #: these too.  Measured (ResNet-50, 20-step window): 7.15 against 7.68 ms per step at 4 GPUs, 7.27 against
    #: 7.39 at 2.  The environment variable ASDL_B200_REPLICATE_IN_EPILOGUE (0 / 1) overrides it.
    replicate_in_epilogue = False

    #: How a rank's share of a factor's statistics reaches the factor's owner: True - every rank's SYRK epilogue
    #: stores its lower-triangular tiles into its OWN buffer and the owner pulls them from all ranks with
    #: coalesced loads while it sums; False - the epilogue stores them into a slot in the owner's buffer
    #: (16 bytes per lane and store over NVLink).  ASDL_B200_PULL_STATISTICS (0 / 1) overrides it.
    pull_statistics = True

    #: plain steps that run eagerly before the CUDA graphs are captured (the capture itself warms
    #: every step kind up twice, so none are needed)
    eager_plain_steps_before_capture = 0

    def __init__(self, model, config: PreconditioningConfig, fisher_type: str = FISHER_MC,
                 loss_type: str = LOSS_CROSS_ENTROPY, scale: float = 1, grad_scale: float = 1,
                 n_mc_samples: int = 1, var: float = 1., seed: int = None,
                 precond_precision: str = 'bf16x3', clone_norm_outputs: bool = False,
                 cuda_graph: bool = False, comm: str = 'auto', grouped: bool = True,
                 overlap_grad_reduce='auto', bucket_mb: float = 16.0, batch_statistics: bool = True,
                 **kwargs):
        super().__init__(model, config, fisher_type=fisher_type, loss_type=loss_type, scale=scale,
                         grad_scale=grad_scale, n_mc_samples=n_mc_samples, var=var, seed=seed, **kwargs)
        self.precond_precision = precond_precision
        self.clone_norm_outputs = clone_norm_outputs
        device = self.device
        if any(p.dtype == torch.float64 for p in model.parameters()):
            raise ValueError('FusedKfacGradientMaker keeps its factors and inverses in fp32 buffers; '
                             'use KfacGradientMaker for a float64 model.')
        self._kron: List[_KronState] = []
        self._norm: List[_NormState] = []
        for name, module in self.named_modules_for_curvature:
            shape = self.shape_for[module]
            if shape == SHAPE_KRON and isinstance(module, (nn.Linear, nn.Conv2d)):
                if getattr(module, 'groups', 1) != 1:
                    raise ValueError(f'{name}: convolutions with groups > 1 are not supported (every group has its '
                                     f'own patch matrix); list the layer in config.ignore_modules.')
                self._kron.append(_KronState(name, module, device))
            elif shape == SHAPE_UNIT_WISE and isinstance(module, _NORMS):
                self._norm.append(_NormState(name, module, device))
            else:
                raise ValueError(f'{type(module).__name__} with shape {shape} is not supported by the '
                                 f'fused K-FAC path; add it to config.ignore_modules.')
        self._by_module: Dict[nn.Module, object] = {s.module: s for s in self._kron + self._norm}
        self._bf16_cache = {}
        self.grouped = grouped
        self._group = None
        if comm not in ('auto', 'symmetric', 'torch'):
            raise ValueError("comm has to be 'auto', 'symmetric' or 'torch'")
        if comm == 'auto':
            comm = 'symmetric' if (self.world_size > 1 and device.type == 'cuda') else 'torch'
        self.comm = comm if self.world_size > 1 else 'torch'
        self._arena = None
        if overlap_grad_reduce == 'auto':
            # The pull of one step's gradients takes about 2 us per MB per peer once the backward pass
            # is over; bucketing hides it but adds a copy and a kernel per bucket and lets the pull
            # kernels share the SMs with the backward pass.  Below this volume the plain reduction
            # after the backward pass was measured to be the faster one.
            grad_mb = sum(p.numel() for p in model.parameters() if p.requires_grad) * 4 / 2 ** 20
            overlap_grad_reduce = grad_mb >= self.OVERLAP_MIN_MB
        self.overlap_grad_reduce = bool(overlap_grad_reduce)
        self.batch_statistics = bool(batch_statistics)
        self.bucket_mb = float(bucket_mb)
        # CTAs of a bucket's pull kernel: one per SM (256 threads each, it shares the GPU with the backward pass)
        self.comm_blocks = (torch.cuda.get_device_properties(device).multi_processor_count
                            if device.type == 'cuda' else 1)
        self._buckets, self._comm_stream, self._reduced_in_backward = [], None, False
        if self.comm == 'symmetric':
            self._setup_symmetric()
        elif self.world_size > 1:
            # torch.distributed transport: new statistics are measured into staging buffers,
            # averaged onto the owners, and folded into the running factors there
            for st in self._kron:
                st.A_new, st.B_new = torch.zeros_like(st.A), torch.zeros_like(st.B)
            for st in self._norm:
                st.stage = torch.zeros_like(st.stats)
        # multi-rank replay needs a transport made of this library's own kernels only: their
        # barriers keep their epochs on the device, so a replay needs no per-step host arguments
        self._graph_enabled = (bool(cuda_graph) and device.type == 'cuda'
                               and (self.world_size == 1 or self.comm == 'symmetric'))
        self._graphs = {}              # 'plain' / 'curvature' / 'update' -> captured step
        self._graph_key = None
        self._plain_steps_seen = 0
        self.replayed_launches = 0     # ... summed over all replays so far
        self._timing = None            # phase -> list of (start, end) CUDA events
        if self._graph_enabled:
            ops.extension().reserve_scratch(device.index or 0, 64 << 20)

    # ------------------------------------------------------------------ device-side phase timing
    def enable_phase_timing(self, enabled=True):
        """Record CUDA events around the phases of every step (plain step, curvature update,
        inverse update, preconditioning).  Read the result with :meth:`phase_times`."""
        self._timing = {} if (enabled and self.device.type == 'cuda') else None

    def _phase(self, name):
        maker = self

        class _Ctx:
            def __enter__(self_inner):
                self_inner.start = None
                if maker._timing is not None and not torch.cuda.is_current_stream_capturing():
                    self_inner.start = torch.cuda.Event(enable_timing=True)
                    self_inner.start.record()

            def __exit__(self_inner, *exc):
                if maker._timing is not None and self_inner.start is not None:
                    end = torch.cuda.Event(enable_timing=True)
                    end.record()
                    maker._timing.setdefault(name, []).append((self_inner.start, end))
                return False

        return _Ctx()

    def phase_times(self, reset=True):
        """{phase: (calls, mean milliseconds)} measured on the device since the last reset."""
        if self._timing is None:
            return {}
        torch.cuda.synchronize()
        out = {k: (len(v), sum(a.elapsed_time(b) for a, b in v) / len(v)) for k, v in self._timing.items()}
        if reset:
            self._timing = {}
        return out

    # ------------------------------------------------------------------ symmetric-memory transport
    def _setup_symmetric(self):
        from ..parallel.symmetric import SymmetricArena, _round_up
        pad = lambda n: _round_up(n, 64)  # noqa: E731
        params = [p for p in self.model.parameters() if p.requires_grad]
        total = sum(pad(st.A.numel()) + pad(st.B.numel()) for st in self._kron)
        total += sum(pad(st.stats.numel()) for st in self._norm)
        total += sum(pad(p.numel()) for p in params)
        # per-rank slots that the peers' SYRK epilogues store their (lower-triangular) statistics
        # into: every owner needs world x (size of its factors); the symmetric region is sized for
        # the largest owner and every rank can compute every owner's layout
        owned_total = [0] * self.world_size
        for st in self._kron:
            o = self._owner.get(st.module, 0)
            st.slot_rel = (owned_total[o], owned_total[o] + pad(st.A.numel()))
            owned_total[o] += pad(st.A.numel()) + pad(st.B.numel())
        self._slot_stride = max(owned_total + [64])
        total += self.world_size * self._slot_stride + 64
        arena = self._arena = SymmetricArena(total, group=self.sync_group, device=self.device)
        rank = self.world_rank
        self._slots_off, _ = arena.alloc(self.world_size * self._slot_stride)
        stage_segs, grad_segs, mirror_rows, slot_rows, pull_rows = [], [], [], [], []
        for st in self._kron:
            st.A_off, st.A = arena.alloc(st.d_in, st.d_in)
            st.B_off, st.B = arena.alloc(st.d_out, st.d_out)
            st.kron.A, st.kron.B = st.A, st.B
            st.owner = self._owner.get(st.module, 0)
            if st.owner == rank:
                mirror_rows += [[st.A_off, st.d_in], [st.B_off, st.d_out]]
                slot_rows += [[st.A_off, self._slots_off + st.slot_rel[0], st.d_in],
                              [st.B_off, self._slots_off + st.slot_rel[1], st.d_out]]
                # pull variant: region `rank` of every rank's slot area holds that rank's share of this owner's factors
                pull_rows += [[st.A_off, self._slots_off + rank * self._slot_stride + st.slot_rel[0], st.d_in],
                              [st.B_off, self._slots_off + rank * self._slot_stride + st.slot_rel[1], st.d_out]]
        for st in self._norm:
            st.stage_off, st.stage = arena.alloc(*st.stats.shape)
            st.owner = self._owner.get(st.module, 0)
            if st.owner == rank:
                stage_segs.append((st.stage_off, st.stage.numel()))
        owner_of_param = {}
        for st in self._kron + self._norm:
            for p in st.module.parameters():
                owner_of_param[p] = st.owner
        self._grad_slot = {}
        kron_weights = {st.module.weight for st in self._kron}
        rest_segs = []  # owned gradients that no GEMM epilogue replicates
        for i, p in enumerate(params):
            off, flat = arena.alloc(p.numel())
            view = flat.as_strided(p.shape, p.stride())
            self._grad_slot[p] = (off, view)
            if owner_of_param.get(p, i % self.world_size) == rank:
                grad_segs.append((off, p.numel()))
                if p not in kron_weights:
                    rest_segs.append((off, p.numel()))
        self._rest_segs = arena.segments(rest_segs)
        self._sym_params = params
        # gradient buckets in the order the backward pass produces them (last parameters first); a
        # bucket's table lists the segments this rank owns in it
        target = max(int(self.bucket_mb * (1 << 20) / 4), 1)
        self._buckets, cur, cur_numel = [], [], 0
        for i in reversed(range(len(params))):
            cur.append(i)
            cur_numel += params[i].numel()
            if cur_numel >= target or i == 0:
                owned = [(self._grad_slot[params[j]][0], params[j].numel()) for j in cur
                         if owner_of_param.get(params[j], j % self.world_size) == rank]
                self._buckets.append(dict(params=cur, segs=arena.segments(owned)))
                cur, cur_numel = [], 0
        if self.overlap_grad_reduce and self.device.type == 'cuda':
            self._comm_stream = torch.cuda.Stream(device=self.device)
        self._mirror_n_max = max([r[1] for r in mirror_rows], default=0)
        self._slot_table = torch.tensor(slot_rows, dtype=torch.int64, device=self.device).reshape(-1, 3)
        self._pull_table = torch.tensor(pull_rows, dtype=torch.int64, device=self.device).reshape(-1, 3)
        self._stage_segs = arena.segments(stage_segs)
        self._grad_segs = arena.segments(grad_segs)

    def _bind_grads_to_arena(self):
        """Gradients live in the symmetric arena; anything autograd allocated elsewhere is moved."""
        with torch.no_grad():
            moved_dst, moved_src = [], []
            for p in self._sym_params:
                _, view = self._grad_slot[p]
                g = p.grad
                if g is None:
                    view.zero_()
                elif g.data_ptr() != view.data_ptr():
                    moved_dst.append(view)
                    moved_src.append(g)
                p.grad = view
            if moved_dst:
                torch._foreach_copy_(moved_dst, moved_src)

    # ------------------------------------------------------------------ gradient buckets overlapped with backward
    def _overlap_active(self):
        return self._arena is not None and self._comm_stream is not None and self.overlap_grad_reduce

    def _overlap_begin(self, views=None, scale=1.0):
        """Arms the bucketed reduction for the next backward pass that produces parameter gradients.
        ``views``: the leaf tensors the model runs on instead of its parameters (graph capture), in the
        order of ``self._sym_params``.  ``scale``: factor applied to the reduced gradients."""
        params = self._sym_params
        st = dict(pending=[len(b['params']) for b in self._buckets], fired=set(), next=0, handles=[],
                  scale=float(scale), copies=[[] for _ in self._buckets])

        def on_view_grad(i, b, grad):
            st['copies'][b].append((self._grad_slot[params[i]][1], grad))
            self._bucket_progress(st, i, b)

        def on_param_grad(i, b, param):
            view = self._grad_slot[param][1]
            g = param.grad
            if g is None:
                with torch.no_grad():
                    view.zero_()
            elif g.data_ptr() != view.data_ptr():
                st['copies'][b].append((view, g))
            param.grad = view
            self._bucket_progress(st, i, b)

        for b, bucket in enumerate(self._buckets):
            for i in bucket['params']:
                if views is not None:
                    h = views[i].register_hook(lambda grad, i=i, b=b: on_view_grad(i, b, grad))
                else:
                    h = params[i].register_post_accumulate_grad_hook(lambda prm, i=i, b=b: on_param_grad(i, b, prm))
                st['handles'].append(h)
        return st

    def _bucket_progress(self, st, i, b):
        if i in st['fired']:
            return   # a parameter used twice in the graph reports once per use: the last copy wins
        st['fired'].add(i)
        st['pending'][b] -= 1
        # buckets go out in their fixed order on every rank, so kernel k of one rank meets kernel k of the others
        while st['next'] < len(self._buckets) and st['pending'][st['next']] == 0:
            self._launch_bucket(st, st['next'])
            st['next'] += 1

    def _launch_bucket(self, st, b):
        current = torch.cuda.current_stream(self.device)
        pairs = st['copies'][b]
        if pairs:   # the bucket's gradients go into the symmetric buffer with one multi-tensor copy
            with torch.no_grad():
                torch._foreach_copy_([v for v, _ in pairs], [g for _, g in pairs])
            st['copies'][b] = []
        ready = torch.cuda.Event()
        ready.record(current)
        self._comm_stream.wait_event(ready)
        with torch.cuda.stream(self._comm_stream):
            self._arena.bucket_reduce(self._buckets[b]['segs'], st['scale'] / self.world_size, blocks=self.comm_blocks)

    def _overlap_end(self, st, ok=True):
        """Removes the hooks; parameters that received no gradient count as zero, the remaining buckets
        go out, and every ``param.grad`` is the parameter's slot in the symmetric buffer."""
        for h in st['handles']:
            h.remove()
        if not ok:
            return
        params = self._sym_params
        with torch.no_grad():
            for b in range(st['next'], len(self._buckets)):
                for i in self._buckets[b]['params']:
                    if i not in st['fired']:
                        self._grad_slot[params[i]][1].zero_()
                        st['fired'].add(i)
                self._launch_bucket(st, b)
            st['next'] = len(self._buckets)
        for prm in params:
            prm.grad = self._grad_slot[prm][1]
        self._reduced_in_backward = True

    def backward(self):
        if not self._overlap_active():
            return super().backward()
        st = self._overlap_begin()
        ok = False
        try:
            super().backward()
            ok = True
        finally:
            self._overlap_end(st, ok)

    # ------------------------------------------------------------------ CUDA-graph replay
    def _capture_key(self, slots):
        """Everything a captured step depends on besides the contents of its tensor arguments: their
        layouts first, then the values read at capture time."""
        cfg = self.config
        layouts = tuple((tuple(v.shape), v.dtype, v.stride()) for _, _, v in slots)
        others = []
        for container in (self._model_args, self._model_kwargs, self._loss_fn_args, self._loss_fn_kwargs):
            items = container.items() if isinstance(container, dict) else enumerate(container)
            for k, v in items:
                if not isinstance(v, torch.Tensor) and isinstance(v, (int, float, bool, str, type(None))):
                    others.append((k, v))
        return (layouts, float(cfg.damping), float(cfg.ema_decay), cfg.data_size, float(self.grad_scale),
                float(self.scale), bool(self.model.training), tuple(others))

    def _tensor_slots(self):
        """(container, key) of every tensor among the registered model / loss arguments."""
        slots = []
        for container in (self._model_args, self._model_kwargs, self._loss_fn_args, self._loss_fn_kwargs):
            items = container.items() if isinstance(container, dict) else enumerate(container)
            for key, value in items:
                if isinstance(value, torch.Tensor):
                    slots.append((container, key, value))
        return slots

    def forward_and_backward(self):
        step = self.state['step']
        curv, prec = self.do_update_curvature(step), self.do_update_preconditioner(step)
        plain = not curv and not prec
        kind = 'plain' if plain else ('curvature' if curv and not prec else ('update' if curv and prec else None))
        ready = all(st.has_inv for st in self._kron + self._norm
                    if self.is_module_for_inv_and_precondition(st.module))
        if not (self._graph_enabled and kind is not None and ready):
            return self._eager_step(step, plain)
        slots = self._tensor_slots()
        key = self._capture_key(slots)
        if self._graphs and key != self._graph_key and key[:1] == self._graph_key[:1]:
            # same tensor shapes, but something that a capture bakes in has changed (damping, moving
            # average, data size, gradient scale, training mode, a non-tensor argument): the graphs
            # are dropped and captured again at the next plain step.  Every rank sees the same
            # configuration, so every rank takes this decision at the same step.
            import warnings
            warnings.warn('FusedKfacGradientMaker: a hyper-parameter or argument captured in the CUDA graphs '
                          'changed; the steps are captured again.')
            self._graphs = {}
            self._graph_key = None
            self._plain_steps_seen = 0
        if not self._graphs:
            if kind != 'plain':
                return self._eager_step(step, plain)
            self._plain_steps_seen += 1
            if self._plain_steps_seen <= self.eager_plain_steps_before_capture:
                return self._eager_step(step, plain)
            self._capture(slots, key)  # runs its own warm-up rounds before recording
        if key != self._graph_key or kind not in self._graphs:
            return self._eager_step(step, plain)
        captured = self._graphs[kind]
        with torch.no_grad():
            for static, (_, _, value) in zip(self._static_inputs, slots):
                if static.data_ptr() != value.data_ptr():
                    static.copy_(value, non_blocking=True)
        with self._phase({'plain': 'plain_step_graph', 'curvature': 'curvature_step_graph',
                          'update': 'update_step_graph'}[kind]):
            captured['graph'].replay()
        self.replayed_launches += captured['launches']
        for p, g in zip(self._graph_params, captured['grads']):
            p.grad = g
        self._model_output, self._loss = captured['output'], captured['loss']
        self.state['step'] += 1
        return self._model_output, self._loss

    def _eager_step(self, step, plain):
        with self._phase('plain_step_eager' if plain else 'update_step'):
            return KfacGradientMaker.forward_and_backward(self)

    def _capture(self, slots, key):
        """Capture the step without updates and, where possible, the step that also measures the
        curvature and the step that measures it and inverts.  Both run on fresh leaf views of the parameters: autograd's gradient
        accumulators remember the stream they were created on - for the real parameters that may
        be the legacy default stream, which a capture must not touch, and they stay alive as long
        as anybody holds an output of an earlier step.  Views created inside the capture get their
        accumulators on the capture stream; gradients come from ``torch.autograd.grad`` and are
        bound to ``param.grad`` by hand.  Two warm-up rounds run on the capture stream first;
        everything they change (running statistics of the model, curvature) is restored after."""
        self._static_inputs = [v.clone() for _, _, v in slots]

        def rebound(container, index_of):
            if isinstance(container, dict):
                return {k: (self._static_inputs[index_of[(id(container), k)]]
                            if (id(container), k) in index_of else v) for k, v in container.items()}
            return tuple(self._static_inputs[index_of[(id(container), i)]]
                         if (id(container), i) in index_of else v for i, v in enumerate(container))

        index_of = {(id(c), k): i for i, (c, k, _) in enumerate(slots)}
        saved = (self._model_args, self._model_kwargs, self._loss_fn_args, self._loss_fn_kwargs)
        self._model_args, self._model_kwargs, self._loss_fn_args, self._loss_fn_kwargs = (
            rebound(c, index_of) for c in saved)
        self._graph_params = [p for p in self.model.parameters() if p.requires_grad]
        from torch.nn.utils.stateless import _reparametrize_module
        names = [n for n, p in self.model.named_parameters() if p.requires_grad]

        def fresh_views():
            return [p.detach().requires_grad_(True) for p in self._graph_params]

        def detach_results():
            self._loss = self._loss.detach()
            if isinstance(self._model_output, torch.Tensor):
                self._model_output = self._model_output.detach()

        def plain_step():
            views = fresh_views()
            with _reparametrize_module(self.model, dict(zip(names, views))):
                self.forward()
            if self._overlap_active():
                st = self._overlap_begin(views)
                torch.autograd.grad(self._loss, views, allow_unused=True)
                self._overlap_end(st)
            else:
                grads = torch.autograd.grad(self._loss, views, allow_unused=True)
                for p, g in zip(self._graph_params, grads):
                    p.grad = g if g is not None else torch.zeros_like(p)
            detach_results()
            self.precondition()

        # the sampling passes of the Monte-Carlo Fisher only need gradients of activations: ask for
        # the gradient of a floating-point model input, which every layer's output leads to
        float_inputs = [t for t in self._static_inputs
                        if t.is_floating_point() and any(t is a for a in self._model_args)]

        def curvature_step():
            for t in float_inputs:
                t.requires_grad_(True)
            try:
                self.update_curvature(views=fresh_views(), names=names, through=float_inputs or None)
            finally:
                for t in float_inputs:
                    t.requires_grad_(False)
            detach_results()
            self.precondition()

        def update_step():  # curvature, inverses of the owned layers, preconditioning
            for t in float_inputs:
                t.requires_grad_(True)
            try:
                self.update_curvature(views=fresh_views(), names=names, through=float_inputs or None)
            finally:
                for t in float_inputs:
                    t.requires_grad_(False)
            detach_results()
            self.update_preconditioner()
            self.precondition()

        stream = torch.cuda.Stream()
        kinds = [('plain', plain_step)]
        if self.fisher_maker.config.seed is None:
            kinds += [('curvature', curvature_step), ('update', update_step)]
        restore = [b for b in self.model.buffers()]
        restore += [t for st in self._kron for t in (st.A, st.B, st.A_inv, st.B_inv)]
        restore += [t for st in self._norm for t in (st.stats, st.inv)]
        restore += [t for pair in self._bf16_cache.values() for t in pair if isinstance(t, torch.Tensor)]
        pool = None
        try:
            for kind, fn in kinds:
                saved_state = [b.detach().clone() for b in restore]
                stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(stream):
                    for _ in range(2):
                        for p in self._graph_params:
                            p.grad = None
                        fn()
                torch.cuda.current_stream().wait_stream(stream)
                torch.cuda.synchronize()
                if self.world_size > 1:
                    dist.barrier(self.sync_group)  # peers have stopped adding to this rank's factors
                with torch.no_grad():
                    torch._foreach_copy_(restore, saved_state)
                del saved_state
                for p in self._graph_params:
                    p.grad = None
                self._model_output = self._loss = None
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                launches_before = ops.extension().launch_count()
                with torch.cuda.graph(graph, stream=stream, pool=pool):
                    fn()
                pool = graph.pool()
                self._graphs[kind] = dict(graph=graph, grads=[p.grad for p in self._graph_params],
                                          output=self._model_output, loss=self._loss,
                                          launches=ops.extension().launch_count() - launches_before)
        finally:
            self._model_args, self._model_kwargs, self._loss_fn_args, self._loss_fn_kwargs = saved
        self._graph_key = key
        if self.world_size > 1:
            # capturing takes host time that differs between ranks; nobody replays (and waits at a
            # device-side barrier) before everybody is done
            torch.cuda.synchronize()
            dist.barrier(self.sync_group)

    # ------------------------------------------------------------------ curvature
    def _stat_weights(self):
        """(alpha, beta): new statistics enter with alpha, stored curvature is kept with beta."""
        cfg = self.config
        if cfg.data_size == -1:
            raise ValueError('data_size is not specified.')
        if self.do_accumulate:
            return self.scale * cfg.ema_decay / cfg.data_size, 1.0 - cfg.ema_decay
        return self.scale / cfg.data_size, 0.0

    def _install_hooks(self):
        alpha, beta = self._stat_weights()
        staged = self._arena is None and self.world_size > 1
        if staged:
            beta = 0.0
        handles = []
        # 'seen': layers whose output-gradient statistics were already written in this curvature pass; further
        # backward passes of the same pass (several Monte-Carlo samples) add to them instead of starting over
        state = {'on': True, 'seen': set(), 'seen_inputs': set()}

        def kron_hook(st: _KronState):
            module = st.module

            def fwd(_m, inputs, output):
                if not state['on']:
                    return
                x = inputs[0].detach()
                reused = st in state['seen_inputs']   # a layer applied more than once in one forward pass
                state['seen_inputs'].add(st)
                beta_a = 1.0 if reused else beta
                # the forward pass may run inside an autocast region: the statistics are not to be autocast
                with torch.no_grad(), torch.autocast(x.device.type, enabled=False):
                    if self._arena is not None:
                        self._push_factor(st, x, output, alpha, is_A=True, accumulate=reused)
                    elif isinstance(module, nn.Conv2d):
                        out_size = output.shape[-2] * output.shape[-1]
                        ops.conv_patch_gram(x, module, scale=alpha / out_size,
                                            out=st.A_new if staged else st.A, beta=beta_a,
                                            channels_last_order=st.khwc)
                    else:
                        ops.gram(x.reshape(-1, x.shape[-1]), scale=alpha,
                                 out=st.A_new if staged else st.A, beta=beta_a)
                if output.requires_grad:
                    def bwd(grad):
                        if not state['on']:
                            return
                        g = grad.detach()
                        again = st in state['seen']
                        state['seen'].add(st)
                        with torch.no_grad():
                            if self._arena is not None:
                                self._push_factor(st, g, None, alpha, is_A=False, accumulate=again)
                                return
                            if g.ndim == 4:
                                rows = g.permute(0, 2, 3, 1).reshape(-1, g.shape[1])
                            else:
                                rows = g.reshape(-1, g.shape[-1])
                            ops.gram(rows, scale=alpha, out=st.B_new if staged else st.B, beta=1.0 if again else beta)
                    output.register_hook(bwd)
            return fwd

        def norm_hook(st: _NormState):
            module = st.module

            def fwd(_m, inputs, output):
                if not state['on']:
                    return
                y = output.detach()
                if output.requires_grad:
                    fused = getattr(module, 'fused_output', False)
                    if fused:  # (x, mean, invstd, y) of this forward pass
                        saved = module.curvature_inputs
                        module.curvature_inputs = None
                    else:
                        saved = y.clone() if self.clone_norm_outputs else y

                    def bwd(grad):
                        if not state['on']:
                            return
                        again = st in state['seen']
                        state['seen'].add(st)
                        with torch.no_grad():
                            self._norm_statistics(st, saved, grad.detach(), alpha, beta, fused, accumulate=again)
                    output.register_hook(bwd)
            return fwd

        for st in self._kron:
            handles.append(st.module.register_forward_hook(kron_hook(st)))
        for st in self._norm:
            handles.append(st.module.register_forward_hook(norm_hook(st)))
            if hasattr(st.module, 'keep_curvature_inputs'):
                st.module.keep_curvature_inputs = True
        return handles, state

    def _push_factor(self, st: _KronState, t, output, alpha, is_A, accumulate=False):
        """Statistics product of this rank sent to the owner of the factor through NVLink: the SYRK
        epilogue stores its lower-triangular tiles (scaled by 1/world) straight into this rank's
        slot in the owner's symmetric buffer; after the barrier the owner sums its slots into the
        running factor (moving average folded in) and mirrors the result.  Deterministic, and the
        wire carries plain 16-byte stores."""
        ext = ops.extension()
        arena = self._arena
        module = st.module
        scale = alpha / self.world_size
        if is_A and isinstance(module, nn.Conv2d):
            from ..utils import _conv_geometry, _explicit_padding
            (kh, kw), (sh, sw), _, (dh, dw) = _conv_geometry(module)
            t, (ph, pw) = _explicit_padding(t, module)
            n, c, h, w = t.shape
            scale = scale / (output.shape[-2] * output.shape[-1])
            pointwise = kh == kw == sh == sw == 1 and ph == pw == 0
            if (pointwise and t.dtype == torch.bfloat16 and c % 8 == 0
                    and t.is_contiguous(memory_format=torch.channels_last)):
                segs_a = [t.permute(0, 2, 3, 1).reshape(-1, c)]
            elif ops.implicit_im2col_eligible(t, (kh, kw), (sh, sw), (dh, dw), (ph, pw), output.shape[-2:], st.khwc):
                # no patch matrix: the SYRK's producer gathers its tiles from the input with 4-D TMA boxes
                if self._pull_statistics():
                    off = self._slots_off + st.owner * self._slot_stride + st.slot_rel[0]
                    target = arena.ptr(self.world_rank, off)
                else:
                    off = self._slots_off + self.world_rank * self._slot_stride + st.slot_rel[0]
                    target = arena.ptr(st.owner, off)
                ext.umma_syrk_conv(t, None, kh, kw, ph, pw, float(scale), 0.0, 0, target, st.d_in,
                                   2 if accumulate else 3)
                return
            else:
                rows = n * output.shape[-2] * output.shape[-1]
                ncol = c * kh * kw
                ld = (max(ncol, 8) + 7) // 8 * 8
                x3 = t.dtype == torch.float32
                hi = torch.empty(rows, ld, device=t.device, dtype=torch.bfloat16)
                lo = torch.empty_like(hi) if x3 else None
                ext.im2col_bf16(t, hi, lo, [kh, kw], [sh, sw], [ph, pw], [dh, dw], not st.khwc)
                segs_a = [hi[:, :ncol], hi[:, :ncol], lo[:, :ncol]] if x3 else [hi[:, :ncol]]
        else:
            rows2d = t.permute(0, 2, 3, 1).reshape(-1, t.shape[1]) if t.ndim == 4 \
                else t.reshape(-1, t.shape[-1])
            hi, lo = ops._stage_bf16(rows2d, ops._use_x3(rows2d.dtype))
            segs_a = [hi, hi, lo] if lo is not None else [hi]
        segs_b = [segs_a[0], segs_a[2], segs_a[0]] if len(segs_a) == 3 else segs_a
        n_dim = st.d_in if is_A else st.d_out
        if self._pull_statistics():
            # this rank's own buffer, region of the factor's owner: the owner pulls it after the barrier
            off = self._slots_off + st.owner * self._slot_stride + st.slot_rel[0 if is_A else 1]
            target = arena.ptr(self.world_rank, off)
        else:
            # this rank's slot in the owner's buffer: peer stores from the epilogue
            off = self._slots_off + self.world_rank * self._slot_stride + st.slot_rel[0 if is_A else 1]
            target = arena.ptr(st.owner, off)
        # lower-triangular tiles only; a further backward pass of the same curvature pass adds to the region
        # (it has one writer, this rank)
        ext.umma_gemm_to_ptr(segs_a, segs_b, False, False, target, n_dim,
                             float(scale), True, 2 if accumulate else 3, [], 0)

    @staticmethod
    def _norm_statistics(st: _NormState, y, g, alpha, beta, fused=False, accumulate=False):
        module = st.module
        staged = getattr(st, 'stage', None) is not None  # reduced over ranks after the backward pass
        target = st.stage if staged else st.stats
        if staged:
            alpha, beta = 1.0, 0.0
        if accumulate:  # a further backward pass of the same curvature pass
            beta = 1.0
        if fused:
            x, mean, invstd, out = y
            ops.batchnorm_unitwise_stats_from_input(x, g, out, mean, invstd, target, alpha=alpha, beta=beta)
            return
        if not isinstance(module, nn.LayerNorm):
            ops.batchnorm_unitwise_stats(y, g, module.weight, module.bias, out=target, alpha=alpha, beta=beta)
            return
        # LayerNorm: one pass over y and g on CUDA (1-D weights), PyTorch otherwise
        ops.layernorm_unitwise_stats(y, g, module.weight, module.bias, out=target, alpha=alpha, beta=beta)

    def _sampling_losses(self, logits):
        """The scalar losses whose backward passes (activation gradients only) measure the output-side
        statistics of the Monte-Carlo and the exact Fisher, as in asdl/fisher.py:419-490: labels sampled
        from the model (cross-entropy) or Gaussian targets around the output (squared error), each
        divided by the number of samples; or one pass per class weighted by sqrt(p) / one per output."""
        cfg = self.fisher_maker.config
        cross_entropy = cfg.loss_type == LOSS_CROSS_ENTROPY
        if self.fisher_type == FISHER_MC:
            n_mc = cfg.n_mc_samples
            if cross_entropy:
                log_probs = F.log_softmax(logits.float(), dim=-1).reshape(-1, logits.shape[-1])
                for _ in range(n_mc):
                    with torch.no_grad():
                        targets = torch.multinomial(log_probs.exp(), 1).squeeze(1)
                    yield F.nll_loss(log_probs, targets, reduction='sum') / n_mc
            else:
                std = float(cfg.var) ** 0.5
                for _ in range(n_mc):
                    with torch.no_grad():
                        targets = logits + std * torch.randn_like(logits)
                    yield 0.5 * F.mse_loss(logits, targets, reduction='sum') / n_mc
        elif cross_entropy:
            log_probs = F.log_softmax(logits, dim=-1).reshape(-1, logits.shape[-1])
            with torch.no_grad():
                sqrt_probs = log_probs.exp().sqrt()
            for c in range(log_probs.shape[1]):
                yield -(log_probs[:, c] * sqrt_probs[:, c]).sum()
        else:
            for d in range(logits.shape[-1]):
                yield logits[..., d].sum()

    def update_curvature(self, views=None, names=None, through=None):
        """One pass that measures the statistics and leaves the (averaged) loss gradient in
        ``param.grad``.

        ``views`` / ``names`` (used while capturing a CUDA graph): fresh leaf views of the parameters
        that the model runs on; gradients then come from ``torch.autograd.grad`` instead of
        ``backward()``.  ``through``: tensors whose gradient is requested in the sampling passes of
        the Monte-Carlo Fisher so that the output hooks of every layer fire (``None``: the
        parameters' ``requires_grad`` is switched off and ``backward()`` is used)."""
        cfg = self.config
        model = self.model
        handles, state = self._install_hooks()
        if cfg is not None and self.fisher_maker.config.seed is not None:
            torch.random.manual_seed(self.fisher_maker.config.seed)

        overlapped = self._overlap_active()

        def backward(loss_, retain=False):
            # the pass that leaves the loss gradient in param.grad; with the bucketed reduction the
            # division by the data size is folded into the reduction's scale
            st = self._overlap_begin(views, scale=1.0 / cfg.data_size) if overlapped else None
            ok = False
            try:
                if views is None:
                    loss_.backward(retain_graph=retain)
                else:
                    grads = torch.autograd.grad(loss_, views, allow_unused=True, retain_graph=retain)
                    if not overlapped:
                        for p, g in zip(self._graph_params, grads):
                            p.grad = g if g is not None else torch.zeros_like(p)
                ok = True
            finally:
                if st is not None:
                    self._overlap_end(st, ok)

        batched = (self.batch_statistics and self.device.type == 'cuda' and ops.get_backend() != 'torch')
        if batched:
            ops.extension().gemm_batch_begin()
        try:
            with nvtx_range('kfac_curvature'), self._phase('curvature'):
                if views is None:
                    self.call_model()
                else:
                    from torch.nn.utils.stateless import _reparametrize_module
                    with _reparametrize_module(model, dict(zip(names, views))):
                        self.call_model()
                saved = self._loss_reduction
                self._loss_reduction = 'sum'
                try:
                    loss = self.call_loss()
                finally:
                    self._loss_reduction = saved
                if self.fisher_type == FISHER_EMP:
                    backward(loss)
                else:
                    for nll in self._sampling_losses(self._logits):
                        if views is None:
                            with skip_param_grad(model):
                                nll.backward(retain_graph=True)
                        else:
                            torch.autograd.grad(nll, through if through else views,
                                                retain_graph=True, allow_unused=True)
                    state['on'] = False
                    backward(loss)
                if batched:   # every statistics product of the pass in one launch
                    batched = False
                    ops.extension().gemm_batch_end()
        finally:
            if batched:
                ops.extension().gemm_batch_abort()
            state['on'] = False
            for h in handles:
                h.remove()
            for st in self._norm:
                if hasattr(st.module, 'keep_curvature_inputs'):
                    st.module.keep_curvature_inputs = False
                    st.module.curvature_inputs = None
        with torch.no_grad():
            grads = [p.grad for p in model.parameters() if p.grad is not None]
            if grads and not overlapped:
                torch._foreach_div_(grads, cfg.data_size)
            loss = loss.detach().div_(cfg.data_size) if views is not None else loss.div_(cfg.data_size)
        self._loss = loss
        if self._arena is not None:
            alpha, beta = self._stat_weights()
            self._arena.barrier()  # every rank's tiles have landed in the owners' slots
            if self._mirror_n_max > 0:  # running factor <- beta * factor + sum of the slots, mirrored
                if self._pull_statistics():
                    self._arena.pull_slots(self._pull_table, self._mirror_n_max, beta)
                else:
                    self._arena.reduce_slots(self._slot_table, self._slot_stride, self._mirror_n_max, beta)
            self._arena.reduce_segments(self._stage_segs, 1.0 / self.world_size)
            with torch.no_grad():
                mine = [st for st in self._norm if st.owner == self.world_rank]
                if mine:
                    torch._foreach_mul_([st.stats for st in mine], beta)
                    torch._foreach_add_([st.stats for st in mine], [st.stage for st in mine], alpha=alpha)
        elif self.world_size > 1:
            self._reduce_staged_statistics()

    def do_update_preconditioner(self, step=None) -> bool:
        if not self.do_accumulate and (self.curvature_upd_schedule is not None
                                       or self.config.curvature_upd_interval is not None):
            return self.do_update_curvature(step)  # nothing is kept: invert whenever measured
        return KfacGradientMaker.do_update_preconditioner(self, step)

    def _reduce_staged_statistics(self):
        """torch.distributed transport: average the new statistics (and the gradients) of every
        layer onto its owner with one packed message per owner, then update the running curvature
        on the owner."""
        alpha, beta = self._stat_weights()
        groups = {r: [] for r in range(self.world_size)}
        for st in self._kron:
            groups[self._owner.get(st.module, 0)] += [st.A_new, st.B_new] + self._module_grads(st.module)
        for st in self._norm:
            groups[self._owner.get(st.module, 0)] += [st.stage] + self._module_grads(st.module)
        for owner, tensors in groups.items():
            self._reduce_avg(tensors, dst=owner)
        self._owned_grads_synced = True
        with torch.no_grad():
            for st in self._kron:
                if self.is_module_for_inv_and_precondition(st.module):
                    st.A.mul_(beta).add_(st.A_new)
                    st.B.mul_(beta).add_(st.B_new)
            for st in self._norm:
                if self.is_module_for_inv_and_precondition(st.module):
                    st.stats.mul_(beta).add_(st.stage, alpha=alpha)

    # ------------------------------------------------------------------ inverses
    @torch.no_grad()
    def update_preconditioner(self, damping=None, **kwargs):
        damping = self.config.damping if damping is None else damping
        root = damping ** 0.5
        with nvtx_range('kfac_inverse'), self._phase('inverse'):
            owned = [st for st in self._kron if self.is_module_for_inv_and_precondition(st.module)]
            if owned:
                # pi-damping split from the traces, evaluated on the device for all layers at once
                tr_a = torch.stack([torch.diagonal(st.A).sum() / st.d_in for st in owned])
                tr_b = torch.stack([torch.diagonal(st.B).sum() / st.d_out for st in owned])
                pi = torch.sqrt(tr_a / tr_b)
                ok = torch.isfinite(pi) & (pi > 0)
                pi = torch.where(ok, pi, torch.ones_like(pi))
                flat = torch.full_like(pi, damping)
                d_a = torch.where(ok, (root * pi).clamp_min(1e-7), flat)
                d_b = torch.where(ok, (root / pi).clamp_min(1e-7), flat)
                mats = [st.A for st in owned] + [st.B for st in owned]
                outs = [st.A_inv for st in owned] + [st.B_inv for st in owned]
                ops.spd_inverse_grouped(mats, outs, torch.cat([d_a, d_b]))
                for st in owned:
                    st.kron.A_inv, st.kron.B_inv = st.A_inv, st.B_inv
                    st.has_inv = True
                    self._refresh_cache(st)
            norms = [st for st in self._norm if self.is_module_for_inv_and_precondition(st.module)]
            if norms and self._use_norm_kernels():
                # all 2x2 blocks of all normalisation layers: one launch, closed form
                ops.extension().unitwise_inverse_mt([[st.stats.data_ptr(), st.inv.data_ptr(), st.stats.shape[0]] for st in norms],
                                                    float(damping))
            else:
                for st in norms:
                    st.inv.copy_(ops.unitwise_inverse(st.stats, damping))
            for st in norms:
                st.unit.inv = st.inv
                st.has_inv = True

    def _refresh_cache(self, st: _KronState):
        """bf16 hi/lo images of the inverses used by the tensor-core preconditioning products."""
        if not st.A.is_cuda or ops.get_backend() == 'torch':
            return
        x3 = self.precond_precision == 'bf16x3'
        for key, mat in (('A', st.A_inv), ('B', st.B_inv)):
            n = mat.shape[0]
            ld = (max(n, 8) + 7) // 8 * 8
            slot = self._bf16_cache.get((st, key))
            if slot is None:
                hi = torch.empty(n, ld, device=mat.device, dtype=torch.bfloat16)
                lo = torch.empty_like(hi) if x3 else None
                slot = self._bf16_cache[(st, key)] = (hi, lo)
            ops.extension().cast_pad_bf16(mat, slot[0], slot[1], 1.0)

    # ------------------------------------------------------------------ preconditioning
    @torch.no_grad()
    def precondition(self, vectors=None, grad_scale=None, use_inv=True):
        if vectors is not None or not use_inv:
            return super().precondition(vectors=vectors, grad_scale=grad_scale, use_inv=use_inv)
        grad_scale = self.grad_scale if grad_scale is None else grad_scale
        if self._arena is not None:
            return self._precondition_symmetric(grad_scale)
        distributed = self.world_size > 1
        if distributed:
            self.sync_grad_pre_precondition()
        with nvtx_range('kfac_precondition'), self._phase('precondition'):
            todo = [st for st in self._kron
                    if st.has_inv and self.is_module_for_inv_and_precondition(st.module)
                    and st.module.weight.grad is not None]
            if todo and self._use_grouped(todo):
                self._precondition_kron_grouped(todo, grad_scale)
            else:
                for st in todo:
                    self._precondition_kron(st, grad_scale)
            self._precondition_norms(grad_scale)
        if distributed:
            self.sync_grad_post_precondition()

    def _precondition_symmetric(self, grad_scale):
        """barrier -> owners pull-reduce the gradients of their layers -> precondition -> owners push
        their gradients into every rank's buffer (only the small rest when the final GEMM's epilogue has
        already stored the Kronecker layers' results everywhere) -> barrier."""
        arena = self._arena
        with self._phase('grad_reduce'):
            if self._reduced_in_backward:
                # the buckets were reduced on the communication stream while the backward pass ran
                self._reduced_in_backward = False
                torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)
            else:
                self._bind_grads_to_arena()
                arena.barrier()
                arena.reduce_segments(self._grad_segs, 1.0 / self.world_size)
        with nvtx_range('kfac_precondition'), self._phase('precondition'):
            owned = [st for st in self._kron if st.owner == self.world_rank]
            todo = [st for st in owned if st.has_inv]
            replicated = len(todo) == len(owned) and self._replicate_in_epilogue()
            if todo and self._use_grouped(todo):
                self._precondition_kron_grouped(todo, grad_scale)
            else:
                for st in todo:
                    replicated &= self._precondition_kron(st, grad_scale, replicate=self._replicate_in_epilogue())
            self._precondition_norms(grad_scale)
        # with replicate_in_epilogue the GEMM epilogues have already stored the Kronecker layers' results on every rank
        with self._phase('grad_bcast'):
            arena.bcast_segments(self._rest_segs if replicated else self._grad_segs)
            arena.barrier()

    def _pull_statistics(self):
        env = os.environ.get('ASDL_B200_PULL_STATISTICS')
        return bool(int(env)) if env is not None else bool(self.pull_statistics)

    def _replicate_in_epilogue(self):
        env = os.environ.get('ASDL_B200_REPLICATE_IN_EPILOGUE')
        return bool(int(env)) if env is not None else bool(self.replicate_in_epilogue)

    # grouped path: all layers' products in a handful of launches ------------------------------------
    def _use_grouped(self, todo):
        return (self.grouped and todo[0].A.is_cuda and ops.get_backend() != 'torch')

    def _build_group(self, todo):
        """Persistent staging buffers, the cast table and the two GEMM plans for ``todo``."""
        ext = ops.extension()
        dev = todo[0].A.device
        x3 = self.precond_precision == 'bf16x3'
        arena = self._arena
        if arena is None:
            total = sum((st.d_out * st.d_in + 63) // 64 * 64 for st in todo)
            flat = torch.zeros(total, device=dev, dtype=torch.float32)
        rows, views, off = [], [], 0
        plan1, plan2 = ext.gemm_plan_new(), ext.gemm_plan_new()
        keep = []
        for st in todo:
            m, n = st.d_out, st.d_in
            w = st.module.weight
            mcast = False
            if arena is None:
                region = flat[off:off + m * n]
                off += (m * n + 63) // 64 * 64
                dst_ptr, extra = region.data_ptr(), []
            else:
                a_off, view = self._grad_slot[w]
                region = arena.buffer[a_off:a_off + m * n]
                if not self._replicate_in_epilogue():
                    dst_ptr, extra = arena.ptr(arena.rank, a_off), []
                elif arena.multicast_ptr and self.multicast_epilogue:
                    # one multimem.st per 16 bytes reaches every rank, this one included
                    dst_ptr, extra, mcast = 0, [arena.mc_ptr(a_off)], True
                else:
                    dst_ptr = arena.ptr(arena.rank, a_off)
                    extra = [arena.ptr(r, a_off) for r in range(arena.world) if r != arena.rank]
            # the region holds the gradient as a contiguous [d_out, d_in] matrix in the factor's order
            if w.ndim == 4 and st.khwc:
                view = region.view(m, w.shape[2], w.shape[3], w.shape[1]).permute(0, 3, 1, 2)
            else:
                view = region.view(w.shape)
            views.append(view)
            ld = (max(n, 8) + 7) // 8 * 8
            mk = lambda: torch.empty(m, ld, device=dev, dtype=torch.bfloat16)  # noqa: E731
            g_hi, g_lo, t_hi, t_lo = mk(), (mk() if x3 else None), mk(), (mk() if x3 else None)
            keep.append((g_hi, g_lo, t_hi, t_lo, region))
            rows.append([region.data_ptr(), g_hi.data_ptr(), g_lo.data_ptr() if x3 else 0, m, n, n, ld])
            b_hi, b_lo = self._bf16_cache[(st, 'B')]
            a_hi, a_lo = self._bf16_cache[(st, 'A')]
            bm, am = b_hi[:, :m], a_hi[:, :n]
            gh, th = g_hi[:, :n], t_hi[:, :n]
            if x3:
                # (hi, lo) parts of both operands: the x3wide flavour loads the four part tiles of a K block
                # once and forms lo*hi + hi*lo + hi*hi from them on 128 x 256 tiles
                s1a, s1b = [bm, b_lo[:, :m]], [gh, g_lo[:, :n]]
                s2a, s2b = [th, t_lo[:, :n]], [am, a_lo[:, :n]]
            else:
                s1a, s1b, s2a, s2b = [bm], [gh], [th], [am]
            ext.gemm_plan_add(plan1, s1a, s1b, False, False, None, 1.0, 0.0, False, t_hi, t_lo,
                              0, 0, False, [], 1, None, False, x3)
            ext.gemm_plan_add(plan2, s2a, s2b, True, False, None, 1.0, 0.0, False, None, None,
                              dst_ptr, n, False, extra, 1, None, False, x3, mcast)
        ext.gemm_plan_finalize(plan1)
        ext.gemm_plan_finalize(plan2)
        table = torch.tensor(rows, dtype=torch.int64, device=dev)
        max_elems = max(r[3] * r[6] for r in rows)
        return dict(key=tuple(id(st) for st in todo), views=views, table=table, plans=(plan1, plan2), max_elems=max_elems,
                    keep=keep, flat=None if arena is not None else flat)

    def _precondition_kron_grouped(self, todo, grad_scale):
        ext = ops.extension()
        group = self._group
        if group is None or group['key'] != tuple(id(st) for st in todo):
            group = self._group = self._build_group(todo)
        grads = [st.module.weight.grad for st in todo]
        moved = [(v, g) for v, g in zip(group['views'], grads) if g.data_ptr() != v.data_ptr()]
        if moved:
            torch._foreach_copy_([v for v, _ in moved], [g for _, g in moved])
        if grad_scale != 1:
            torch._foreach_mul_(group['views'], grad_scale)
        ext.cast_pad_bf16_grouped(group['table'], len(todo), group['max_elems'])
        ext.gemm_plan_run(group['plans'][0])
        ext.gemm_plan_run(group['plans'][1])
        if moved:
            torch._foreach_copy_([g for _, g in moved], [v for v, _ in moved])
        self._precondition_biases(todo, grad_scale)

    def _precondition_kron(self, st: _KronState, grad_scale, replicate=False):
        g2d, staged = st.grad_matrix()
        if grad_scale != 1:
            g2d.mul_(grad_scale)
        replicated = False
        if g2d.is_cuda and ops.get_backend() != 'torch':
            replicated = self._kron_apply_cached(st, g2d, replicate and staged is None)
        else:
            g2d.copy_(st.B_inv @ g2d @ st.A_inv)
        if staged is not None:
            st.module.weight.grad.copy_(staged)
        if st.has_bias and st.module.bias.grad is not None:
            b = st.module.bias.grad
            if grad_scale != 1:
                b.mul_(grad_scale)
            b.copy_(torch.mv(st.B_inv, b))
        return replicated

    def _kron_apply_cached(self, st: _KronState, g2d, replicate=False):
        """g2d <- B^-1 g2d A^-1 with the cached bf16 images of the inverses.  With ``replicate``
        the epilogue of the second GEMM also stores the result into the peers' gradient buffers
        (preconditioning fused with the all-gather of its result)."""
        ext = ops.extension()
        x3 = self.precond_precision == 'bf16x3'
        m, n = g2d.shape
        ld = (max(n, 8) + 7) // 8 * 8
        bufs = self._bf16_cache.get((st, 'work'))
        if bufs is None:
            mk = lambda: torch.empty(m, ld, device=g2d.device, dtype=torch.bfloat16)  # noqa: E731
            bufs = self._bf16_cache[(st, 'work')] = (mk(), mk() if x3 else None, mk(), mk() if x3 else None)
        g_hi, g_lo, t_hi, t_lo = bufs
        ext.cast_pad_bf16(g2d, g_hi, g_lo, 1.0)
        b_hi, b_lo = self._bf16_cache[(st, 'B')]
        a_hi, a_lo = self._bf16_cache[(st, 'A')]
        bm = b_hi[:, :m]
        am = a_hi[:, :n]
        if x3:
            seg_a, seg_b = [bm, bm, b_lo[:, :m]], [g_hi[:, :n], g_lo[:, :n], g_hi[:, :n]]
        else:
            seg_a, seg_b = [bm], [g_hi[:, :n]]
        ext.umma_gemm(seg_a, seg_b, False, False, None, 1.0, 0.0, False, t_hi, t_lo, 0)
        if x3:
            seg_a = [t_hi[:, :n], t_hi[:, :n], t_lo[:, :n]]
            seg_b = [am, a_lo[:, :n], am]
        else:
            seg_a, seg_b = [t_hi[:, :n]], [am]
        if replicate and g2d.stride(1) == 1 and g2d.stride(0) == n:
            off, _ = self._grad_slot[st.module.weight]
            arena = self._arena
            peers = [arena.ptr(r, off) for r in range(arena.world) if r != arena.rank]
            ext.umma_gemm_to_ptr(seg_a, seg_b, True, False, arena.ptr(arena.rank, off), n, 1.0,
                                 False, False, peers, 0)
            return True
        elif g2d.stride(1) == 1:
            ext.umma_gemm(seg_a, seg_b, True, False, g2d, 1.0, 0.0, False, None, None, 0)
        else:
            out = torch.empty(m, n, device=g2d.device, dtype=torch.float32)
            ext.umma_gemm(seg_a, seg_b, True, False, out, 1.0, 0.0, False, None, None, 0)
            g2d.copy_(out)
        return False

    def _use_norm_kernels(self):
        return self.device.type == 'cuda' and ops.get_backend() != 'torch'

    def _precondition_biases(self, todo, grad_scale):
        """bias.grad <- B^-1 bias.grad for every layer of ``todo`` that has a bias: one launch on CUDA."""
        with_bias = [st for st in todo if st.has_bias and st.module.bias.grad is not None]
        if not with_bias:
            return
        if self._use_norm_kernels() and all(st.module.bias.grad.is_contiguous() and st.B_inv.is_contiguous()
                                            and st.module.bias.grad.dtype == torch.float32 for st in with_bias):
            scratch = self.__dict__.setdefault('_bias_scratch', {})
            rows = []
            for st in with_bias:
                if st not in scratch:
                    scratch[st] = torch.empty(st.d_out, device=self.device, dtype=torch.float32)
                rows.append([st.B_inv.data_ptr(), st.module.bias.grad.data_ptr(), scratch[st].data_ptr(), st.d_out])
            ops.extension().bias_precondition_mt(rows, float(grad_scale))   # the addresses travel as kernel parameters
            return
        for st in with_bias:
            b = st.module.bias.grad
            if grad_scale != 1:
                b.mul_(grad_scale)
            b.copy_(torch.mv(st.B_inv, b))

    def _precondition_norms(self, grad_scale):
        if self._use_norm_kernels():
            norms, grads = [], []
            for st in self._norm:
                if not st.has_inv or not self.is_module_for_inv_and_precondition(st.module):
                    continue
                w, b = st.module.weight.grad, st.module.bias.grad
                if w is None or b is None:
                    continue
                if not (w.is_contiguous() and b.is_contiguous() and w.dtype == torch.float32 and b.dtype == torch.float32):
                    norms = None
                    break
                norms.append(st)
                grads.append((w, b))
            if norms is not None:
                if norms:   # every normalisation layer's 2x2 blocks applied in one launch
                    ops.extension().unitwise_apply_mt([[st.inv.data_ptr(), w.data_ptr(), b.data_ptr(), st.inv.shape[0]]
                                                       for st, (w, b) in zip(norms, grads)], float(grad_scale))
                return
        gw, gb, i00, i01, i10, i11 = [], [], [], [], [], []
        for st in self._norm:
            if not st.has_inv or not self.is_module_for_inv_and_precondition(st.module):
                continue
            w, b = st.module.weight.grad, st.module.bias.grad
            if w is None or b is None:
                continue
            gw.append(w.view(-1))
            gb.append(b.view(-1))
            i00.append(st.inv[:, 0, 0])
            i01.append(st.inv[:, 0, 1])
            i10.append(st.inv[:, 1, 0])
            i11.append(st.inv[:, 1, 1])
        if not gw:
            return
        if grad_scale != 1:
            torch._foreach_mul_(gw, grad_scale)
            torch._foreach_mul_(gb, grad_scale)
        new_w = torch._foreach_mul(gw, i00)
        torch._foreach_addcmul_(new_w, gb, i01)
        new_b = torch._foreach_mul(gw, i10)
        torch._foreach_addcmul_(new_b, gb, i11)
        torch._foreach_copy_(gw, new_w)
        torch._foreach_copy_(gb, new_b)

    # ------------------------------------------------------------------ checkpointing
    def _load_curvature_state(self, tensors):
        grouped: Dict[str, Dict[str, torch.Tensor]] = {}
        for key, value in tensors.items():
            name, rest = key.split('.', 1)
            grouped.setdefault(name, {})[rest] = value
        for st in self._kron:
            items = grouped.get(st.name, {})
            for key, buf in (('kron.A', st.A), ('kron.B', st.B), ('kron.A_inv', st.A_inv),
                             ('kron.B_inv', st.B_inv)):
                if key in items:
                    buf.copy_(items[key])
            if 'kron.A_inv' in items and 'kron.B_inv' in items:
                st.kron.A_inv, st.kron.B_inv = st.A_inv, st.B_inv
                st.has_inv = True
                self._refresh_cache(st)
        for st in self._norm:
            items = grouped.get(st.name, {})
            if 'unit.data' in items:
                st.stats.copy_(items['unit.data'])
            if 'unit.inv' in items:
                st.inv.copy_(items['unit.inv'])
                st.unit.inv = st.inv
                st.has_inv = True
