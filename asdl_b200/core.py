"""Hook engine: attach :class:`Operation` objects to the supported leaf modules of a model for the
duration of a ``with`` block.

Parity: asdl/core.py (``extend`` :20-80, ``no_centered_cov`` :83-97, ``save_inputs_outgrads``
and friends :100-121, ``module_wise_assignments`` :130-244, ``modules_to_assign`` :247-260).

How the capture works here: a forward hook on each module hands the detached input/output to the
operation and - if any backward statistic was requested - registers a *tensor* hook on the
module's output, which receives the output-gradient during backward.  Tensor hooks (rather than
the deprecated module backward hooks of the reference) are exact for modules that sit on several
autograd paths, work with in-place activations that follow the module, and fire once per backward
pass through that output, so several backward passes over one graph (MC / exact Fisher) each
contribute.  All hook work can be placed on a side CUDA stream with ``stream=``; the side stream
waits for the producing stream before reading and the consumer must wait on it afterwards.
"""
import warnings
from contextlib import contextmanager, nullcontext

import torch
import torch.nn as nn
from torch.cuda import Stream

from .utils import record_original_requires_grad
from .operations import *  # noqa: F401,F403
from .operations import Operation, OperationContext, get_op_class, Bias, Scale
from .operations import FWD_OPS, BWD_OPS, BWD_OPS_WITH_INPUTS
from .matrices import *  # noqa: F401,F403
from .vector import ParamVector

_supported_module_classes = (nn.Linear, nn.Conv2d, nn.BatchNorm1d, nn.BatchNorm2d, nn.LayerNorm,
                             nn.Embedding, Bias, Scale)

__all__ = ['extend', 'no_centered_cov', 'save_inputs_outgrads', 'save_inputs', 'save_outgrads',
           'module_wise_assignments', 'modules_to_assign']


@contextmanager
def extend(model, *op_names, ignore_modules=None, map_rule=None, vectors: ParamVector = None,
           stream: Stream = None) -> OperationContext:
    """``with extend(model, OP_COV_KRON) as cxt: loss = f(model(x)); loss.backward()`` collects the
    requested statistics in ``cxt``.  ``op_names`` follow the assignment mini-language of
    :func:`module_wise_assignments`."""
    handles = []
    cxt = OperationContext(vectors=vectors)
    use_stream = stream is not None and torch.cuda.is_available()
    state = {'alive': True}

    def on_side_stream(fn):
        if not use_stream:
            return fn()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            return fn()

    def make_hooks(needs_fwd, needs_bwd):
        def forward_hook(module, inputs, output):
            x = inputs[0].detach()
            y = output.detach()
            if needs_fwd:
                # the forward pass may run inside the user's autocast region: statistics are not to be autocast
                with torch.autocast(x.device.type, enabled=False):
                    on_side_stream(lambda: cxt.call_operations_in_forward(module, x, y))
            if needs_bwd and output.requires_grad:
                def grad_hook(grad):
                    if state['alive'] and cxt.is_operation_registered(module):
                        g = grad.detach()
                        with torch.autocast(g.device.type, enabled=False):
                            on_side_stream(lambda: cxt.call_operations_in_backward(module, g))
                output.register_hook(grad_hook)
        return forward_hook

    try:
        for module, names in module_wise_assignments(model, *op_names, ignore_modules=ignore_modules,
                                                     map_rule=map_rule):
            if not names:
                continue
            op_class = get_op_class(module)
            if op_class is None:
                continue
            usable = []
            for name in names:
                if name in op_class.supported_operations:
                    usable.append(name)
                else:
                    warnings.warn(f'{name} operation is not supported for {module}. Skip.')
            cxt.register_operation(module, op_class(module, usable, model_for_kernel=model))
            needs_fwd = any(n in FWD_OPS for n in usable) or any(n in BWD_OPS_WITH_INPUTS for n in usable)
            needs_bwd = any(n in BWD_OPS for n in usable)
            if needs_fwd or needs_bwd:
                handles.append(module.register_forward_hook(make_hooks(needs_fwd, needs_bwd)))
        if not cxt.is_operation_registered(model):
            cxt.register_operation(model, Operation(model, []))  # holder for whole-model results
        yield cxt
    finally:
        state['alive'] = False
        for handle in handles:
            handle.remove()
        cxt.clear_operations()


_SHAPE_TO_OP = {
    SHAPE_FULL: (OP_BATCH_GRADS, OP_BATCH_GRADS),
    SHAPE_LAYER_WISE: (OP_COV, OP_COV_INV),
    SHAPE_KRON: (OP_COV_KRON, OP_COV_KRON_INV),
    SHAPE_SWIFT_KRON: (OP_COV_SWIFT_KRON, OP_COV_SWIFT_KRON_INV),
    SHAPE_KFE: (OP_COV_KFE, OP_COV_KFE),
    SHAPE_UNIT_WISE: (OP_COV_UNIT_WISE, OP_COV_UNIT_WISE_INV),
    SHAPE_DIAG: (OP_COV_DIAG, OP_COV_DIAG_INV),
}


def no_centered_cov(model: nn.Module, shapes, ignore_modules=None, cvp=False,
                    vectors: ParamVector = None, stream: Stream = None,
                    calc_inv=False) -> OperationContext:
    """``extend`` with curvature *shapes* (``'kron'``, ``'diag'``, ...) instead of op names.
    ``cvp`` switches layer-wise blocks to matrix-free products; ``calc_inv`` selects the fused
    "statistic + damped inverse" variant of every shape that has one."""
    if cvp and calc_inv:
        raise ValueError('cvp and calc_inv cannot be True at the same time.')

    def to_op(shape):
        if cvp and shape == SHAPE_LAYER_WISE:
            return OP_CVP
        return _SHAPE_TO_OP[shape][1 if calc_inv else 0]

    return extend(model, *shapes, ignore_modules=ignore_modules, map_rule=to_op, vectors=vectors,
                  stream=stream)


def _save_context(model, ops_to_save, targets, ignore_modules):
    if targets is not None:
        rules = [(t, *ops_to_save) for t in targets]
    else:
        rules = list(ops_to_save)
    return extend(model, *rules, ignore_modules=ignore_modules)


def save_inputs_outgrads(model: nn.Module, targets=None, ignore_modules=None) -> OperationContext:
    """Context in which hooks keep every supported layer's inputs and output gradients (``cxt.in_data(module)``, ``cxt.out_grads(module)``)."""
    return _save_context(model, (OP_SAVE_INPUTS, OP_SAVE_OUTGRADS), targets, ignore_modules)


def save_inputs(model: nn.Module, targets=None, ignore_modules=None) -> OperationContext:
    """Context in which hooks keep every supported layer's inputs."""
    return _save_context(model, (OP_SAVE_INPUTS,), targets, ignore_modules)


def save_outgrads(model: nn.Module, targets=None, ignore_modules=None) -> OperationContext:
    """Context in which hooks keep every supported layer's output gradients."""
    return _save_context(model, (OP_SAVE_OUTGRADS,), targets, ignore_modules)


def named_supported_modules(model):
    for name, module in model.named_modules():
        if isinstance(module, _supported_module_classes):
            yield name, module


def _ignored(name, module, ignore_modules):
    for item in ignore_modules:
        if isinstance(item, type):
            if isinstance(module, item):
                return True
        elif isinstance(item, str):
            if item in name:
                return True
        elif item is module:
            return True
    return False


def module_wise_assignments(model, *assign_rules, ignore_modules=None, map_rule=None, named=False):
    """Yield ``(module, values)`` (or ``(name, module, values)``) for every supported module with
    trainable parameters.

    A rule is either a plain string (a value for every module that no keyed rule matched) or a
    tuple ``(key, value, ...)`` whose key is a module instance, a substring of the module name, or
    a module class - in that order of priority.  Example::

        module_wise_assignments(model, 'kron', ('conv', 'diag'), (nn.BatchNorm2d, 'unit_wise'),
                                (model.bn1, 'full'))

    Values are passed through ``map_rule`` when given.  ``ignore_modules`` accepts the same three
    kinds of keys.
    """
    for rule in assign_rules:
        if not isinstance(rule, (str, tuple)):
            raise TypeError(f'every assign rule has to be {str} or {tuple}.')
    ignore_modules = [] if ignore_modules is None else list(ignore_modules)
    convert = map_rule if map_rule is not None else (lambda v: v)

    default_values = []
    keyed = {}
    for rule in assign_rules:
        if isinstance(rule, str):
            default_values.append(convert(rule))
            continue
        if len(rule) < 2:
            raise ValueError(f'Tuple length has to be >= 2. Given: {rule}.')
        key, values = rule[0], rule[1:]
        if any(not isinstance(v, str) for v in values):
            raise TypeError(f'All values have to be {str}. Given: {values}.')
        if key in keyed:
            raise ValueError(f'({key}, _) is already assigned.')
        keyed[key] = [convert(v) for v in values]

    name_keys = [k for k in keyed if isinstance(k, str)]
    for name, module in named_supported_modules(model):
        if _ignored(name, module, ignore_modules):
            continue
        trainable = False
        for attr in ('weight', 'bias'):
            param = getattr(module, attr, None)
            if param is not None:
                trainable = trainable or param.requires_grad
                record_original_requires_grad(param)
        if not trainable:
            continue
        if module in keyed:
            values = keyed[module]
        else:
            hit = next((k for k in name_keys if k in name), None)
            if hit is not None:
                values = keyed[hit]
            elif any(cls in keyed for cls in type(module).__mro__):  # nearest base class wins
                values = keyed[next(cls for cls in type(module).__mro__ if cls in keyed)]
            elif default_values:
                values = list(default_values)
            else:
                continue
        yield (name, module, values) if named else (module, values)


def named_modules_to_assign(model, value, *assign_rules, ignore_modules=None):
    """``(name, module)`` pairs whose assigned values contain ``value``."""
    return modules_to_assign(model, value, *assign_rules, ignore_modules=ignore_modules, named=True)


def modules_to_assign(model, value, *assign_rules, ignore_modules=None, named=False):
    """Modules whose assigned values contain ``value``."""
    for item in module_wise_assignments(model, *assign_rules, ignore_modules=ignore_modules, named=True):
        name, module, values = item
        if value in values:
            yield (name, module) if named else module
