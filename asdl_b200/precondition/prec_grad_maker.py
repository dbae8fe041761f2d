"""Base class of the preconditioned gradient makers: configuration, update schedules and the
template ``forward_and_backward`` that every second-order method fills in.

Parity: asdl/precondition/prec_grad_maker.py (``PreconditioningConfig`` :22-75,
``PreconditionedGradientMaker`` :78-201, ``get_update_schedule`` :204-254).

Differences: ``curvature_interval_type`` is a real dataclass field and both interval types are
forwarded to the schedule builder; ``state_dict()`` carries the curvature state of the maker
(subclasses contribute through ``_curvature_state`` / ``_load_curvature_state``) in addition to
the step counter, and a dict holding only ``{'step': n}`` still loads.
"""
import math
import warnings
from dataclasses import dataclass
from typing import Any, Dict, List

import torch
import torch.nn as nn

from ..grad_maker import GradientMaker
from ..utils import nvtx_range

__all__ = ['PreconditionedGradientMaker', 'PreconditioningConfig', 'get_update_schedule',
           'INTERVAL_CONSTANT', 'INTERVAL_STEP', 'INTERVAL_LINEAR', 'INTERVAL_TYPES']

INTERVAL_CONSTANT = 'constant'
INTERVAL_STEP = 'step'
INTERVAL_LINEAR = 'linear'
INTERVAL_TYPES = [INTERVAL_CONSTANT, INTERVAL_STEP, INTERVAL_LINEAR]

_default_interval = 1
_invalid_value = -1


@dataclass
class PreconditioningConfig:
    """Configuration shared by all preconditioners.

    Args:
        num_total_steps: total number of training steps; when given, ratio-based boolean
            schedules replace the interval rules.
        preconditioner_upd_interval: steps between preconditioner (inverse / root) updates.
        preconditioner_warmup_steps: update every step until this step.
        preconditioner_upd_ratio / preconditioner_warmup_ratio: fractions of ``num_total_steps``
            spent on updates / warm-up (ratio mode).
        preconditioner_interval_type: ``"constant"``, ``"step"`` or ``"linear"`` (ratio mode).
        curvature_upd_interval, curvature_warmup_steps, curvature_upd_ratio,
        curvature_warmup_ratio, curvature_interval_type: the same for curvature (statistics)
            updates; when neither interval nor ratio is set the preconditioner rule is used.
        data_size: number of examples the curvature is averaged over.
        damping: value added to the diagonal before inversion.
        ema_decay: ``curv <- curv*(1-ema_decay) + new*ema_decay``; ``-1`` disables the EMA.
        ignore_modules: modules, module classes or name fragments excluded from preconditioning.
    """
    num_total_steps: int = None
    preconditioner_upd_interval: int = _default_interval
    preconditioner_warmup_steps: int = 0
    preconditioner_upd_ratio: float = 1.
    preconditioner_warmup_ratio: float = 0.
    preconditioner_interval_type: str = INTERVAL_CONSTANT
    curvature_upd_interval: int = None
    curvature_warmup_steps: int = 0
    curvature_upd_ratio: float = None
    curvature_warmup_ratio: float = 0.
    curvature_interval_type: str = INTERVAL_CONSTANT
    data_size: int = _invalid_value
    damping: float = 1.e-7
    ema_decay: float = _invalid_value
    ignore_modules: List[Any] = None


class PreconditionedGradientMaker(GradientMaker):
    """Template of every preconditioned gradient maker: ``forward_and_backward()`` runs the pass, then
    ``update_curvature`` / ``update_preconditioner`` when their schedules say so, then ``precondition`` (which
    rewrites ``param.grad`` in place), and counts the step.  ``state_dict()`` holds the step and the curvature
    state of the subclass.  Reference: asdl/precondition/prec_grad_maker.py:78-201.
    """
    _supported_classes = None

    def __init__(self, model: nn.Module, config: PreconditioningConfig):
        super().__init__(model)
        self.config = config
        self.curvature_upd_schedule = None
        self.preconditioner_upd_schedule = None
        if config.num_total_steps is not None:
            if config.preconditioner_upd_interval != _default_interval:
                warnings.warn('Since num_total_steps is specified, preconditioner_upd_interval '
                              'is ignored and preconditioner_upd_ratio is used.')
            self.preconditioner_upd_schedule = get_update_schedule(
                num_total_steps=config.num_total_steps, update_ratio=config.preconditioner_upd_ratio,
                warmup_ratio=config.preconditioner_warmup_ratio,
                interval_type=config.preconditioner_interval_type)
            if config.curvature_upd_ratio is not None:
                if config.curvature_upd_interval is not None:
                    warnings.warn('Since num_total_steps is specified, curvature_upd_interval '
                                  'is ignored and curvature_upd_ratio is used.')
                self.curvature_upd_schedule = get_update_schedule(
                    num_total_steps=config.num_total_steps, update_ratio=config.curvature_upd_ratio,
                    warmup_ratio=config.curvature_warmup_ratio,
                    interval_type=config.curvature_interval_type)
        self.state = dict(step=0)
        # a model that is itself a single layer has the empty name, which ModuleDict refuses
        self.module_dict = nn.ModuleDict({(name.replace('.', '/') or 'model'): m for name, m in model.named_modules()
                                          if self._is_supported(name, m)})
        params = list(self.module_dict.parameters())
        self.device = params[0].device if params else torch.device('cpu')

    def _is_supported(self, module_name: str, module: nn.Module) -> bool:
        """Leaf modules with trainable parameters that are not ignored (and of a supported class,
        when the subclass restricts them)."""
        if len(list(module.children())) > 0:
            return False
        if all(not p.requires_grad for p in module.parameters()):
            return False
        for item in self.config.ignore_modules or []:
            if isinstance(item, type):
                if isinstance(module, item):
                    return False
            elif isinstance(item, str):
                if item in module_name:
                    return False
            elif item is module:
                return False
        if self._supported_classes is not None and not isinstance(module, self._supported_classes):
            warnings.warn(f'This model contains {module}, but ASDL library does not support {module}.')
            return False
        return True

    # ------------------------------------------------------------------ checkpointing
    def _curvature_state(self) -> Dict[str, torch.Tensor]:
        """Flat ``{key: tensor}`` curvature state of the maker (overridden by subclasses)."""
        return {}

    def _load_curvature_state(self, tensors: Dict[str, torch.Tensor]):
        pass

    def state_dict(self) -> dict:
        out = dict(self.state)
        curvature = self._curvature_state()
        if curvature:
            out['curvature'] = curvature
        return out

    def load_state_dict(self, state_dict: dict):
        self.state['step'] = state_dict['step']
        for key, value in state_dict.items():
            if key not in ('step', 'curvature'):
                self.state[key] = value
        if state_dict.get('curvature'):
            self._load_curvature_state(state_dict['curvature'])

    # ------------------------------------------------------------------ the template
    def forward_and_backward(self):
        step = self.state['step']
        self._startup()
        if self.do_forward_and_backward(step):
            with nvtx_range('forward_and_backward'):
                self.forward()
                self.backward()
        if self.do_update_curvature(step):
            with nvtx_range('update_curvature'):
                self.update_curvature()
        if self.do_update_preconditioner(step):
            with nvtx_range('update_preconditioner'):
                self.update_preconditioner()
        with nvtx_range('precondition'):
            self.precondition()
        self._teardown()
        self.state['step'] += 1
        return self._model_output, self._loss

    def _startup(self):
        pass

    def update_curvature(self):
        pass

    def update_preconditioner(self):
        pass

    def precondition(self):
        raise NotImplementedError

    def _teardown(self):
        pass

    # ------------------------------------------------------------------ schedules
    def do_forward_and_backward(self, step=None) -> bool:
        raise NotImplementedError

    def do_update_curvature(self, step=None) -> bool:
        if self.curvature_upd_schedule is not None:
            return self._do_update_by_schedule(self.curvature_upd_schedule, step)
        config = self.config
        if config.curvature_upd_interval is not None:
            return self._do_update_by_interval(config.curvature_upd_interval,
                                               config.curvature_warmup_steps, step)
        return self.do_update_preconditioner(step)

    def do_update_preconditioner(self, step=None) -> bool:
        if self.preconditioner_upd_schedule is not None:
            return self._do_update_by_schedule(self.preconditioner_upd_schedule, step)
        return self._do_update_by_interval(self.config.preconditioner_upd_interval,
                                           self.config.preconditioner_warmup_steps, step)

    def _do_update_by_schedule(self, upd_schedule, step=None) -> bool:
        step = self.state['step'] if step is None else step
        if step >= len(upd_schedule):
            warnings.warn(f'Given step+1 ({step+1}) is larger than the total number of steps '
                          f'({self.config.num_total_steps})')
            return False
        return upd_schedule[step]

    def _do_update_by_interval(self, interval, warmup_steps=0, step=None) -> bool:
        step = self.state['step'] if step is None else step
        return step < warmup_steps or (step - warmup_steps) % interval == 0


def get_update_schedule(num_total_steps: int, update_ratio: float = 1., warmup_ratio: float = 0.,
                        interval_type: str = INTERVAL_CONSTANT, reverse=False):
    """Boolean list of length ``num_total_steps``: update every step during warm-up, then spread
    the remaining ``num_total_steps*update_ratio - warmup`` updates with a constant interval,
    all at once (``step``) or with linearly growing gaps (``linear``)."""
    if num_total_steps <= 0:
        raise ValueError(f'num_total_steps has to be > 0. Got {num_total_steps}.')
    if not 0 <= update_ratio <= 1:
        raise ValueError(f'update_ratio has to be in [0, 1]. Got {update_ratio}.')
    if not 0 <= warmup_ratio <= 1:
        raise ValueError(f'warmup_ratio has to be in [0, 1]. Got {warmup_ratio}.')
    n_updates = int(num_total_steps * update_ratio)
    n_warmup = int(num_total_steps * warmup_ratio)
    if n_warmup > n_updates:
        raise ValueError(f'num_warmup_steps cannot be larger than num_total_updates ({n_updates}). '
                         f'Got {n_warmup}.')
    if interval_type not in INTERVAL_TYPES:
        raise ValueError(f'Invalid interval_type: {interval_type}. {INTERVAL_TYPES} are supported.')
    schedule = [True] * n_warmup
    steps_left = num_total_steps - n_warmup
    updates_left = n_updates - n_warmup
    if updates_left > 0:
        if interval_type == INTERVAL_CONSTANT:
            interval = steps_left // updates_left
            done = n_warmup
            for i in range(steps_left):
                hit = i % interval == 0 and done < n_updates
                schedule.append(hit)
                done += hit
        elif interval_type == INTERVAL_STEP:
            schedule.extend([True] * updates_left)
        else:
            gaps = updates_left - 1
            schedule.append(True)
            if gaps > 0:
                growth = math.floor(2 * (steps_left - gaps) / gaps / (gaps - 1)) if gaps > 1 else 0
                for i in range(gaps):
                    schedule.extend([False] * (1 + growth * i - 1))
                    schedule.append(True)
    if len(schedule) > num_total_steps:
        raise ValueError(f'len(update_schedule) cannot be larger than num_total_steps '
                         f'({num_total_steps}). Got {len(schedule)}.')
    schedule.extend([False] * (num_total_steps - len(schedule)))
    return schedule[::-1] if reverse else schedule
