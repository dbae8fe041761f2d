"""The ``GradientMaker`` interface: the user registers *how* to call the model and the loss, the
maker decides *when* they are evaluated inside ``forward_and_backward()``.

    dummy_y = gm.setup_model_call(model, x)
    gm.setup_loss_call(F.cross_entropy, dummy_y, t)
    y, loss = gm.forward_and_backward()

``setup_model_call`` returns a :class:`DummyObject`, a placeholder for the future model output
that records item access, attribute access and calls; it can be passed (possibly manipulated) to
``setup_loss_call`` / ``setup_loss_repr`` / ``setup_logits_repr`` and is replayed on the real
output at evaluation time.

Parity: asdl/grad_maker.py (``DummyObject`` :45-119, ``GradientMaker`` :137-368, functional
utilities :370-581).  The functional utilities are built on ``torch.func.functional_call`` (the
reference uses the deprecated ``functorch.make_functional_with_buffers``); ``ft`` is exported as
an alias of ``torch.func`` for code that used the reference's ``ft`` handle.
"""
from collections import OrderedDict
from typing import Any, Callable, Dict, Tuple, Union

import torch
from torch import Tensor
import torch.nn as nn
import torch.nn.functional as F
import torch.func as ft

from .utils import has_reduction

__all__ = ['GradientMaker', 'DummyObject', 'ft', 'LOSS_CROSS_ENTROPY', 'LOSS_MSE']

LOSS_CROSS_ENTROPY = 'cross_entropy'
LOSS_MSE = 'mse'

_OP_FIRST, _OP_ITEM, _OP_ATTR, _OP_CALL = 'first', 'item', 'attr', 'call'


class GetFirstItem:
    """Marker: take element 0 of a tuple/list output, pass anything else through."""
    kind = _OP_FIRST

    def __repr__(self):
        return 'GetFirstItem()'


class GetItem(tuple):
    """``value[item]`` as an element of a DummyObject's operator list (``DummyObject([GetItem(0)])``)."""

    def __new__(cls, item):
        return tuple.__new__(cls, (_OP_ITEM, item))


class GetAttr(tuple):
    """``value.item`` as an element of a DummyObject's operator list."""

    def __new__(cls, item):
        return tuple.__new__(cls, (_OP_ATTR, item))


class Call(tuple):
    """``value(*args, **kwargs)`` as an element of a DummyObject's operator list."""

    def __new__(cls, args=(), kwargs=None):
        return tuple.__new__(cls, (_OP_CALL, tuple(args), dict(kwargs or {})))


class DummyObject:
    """Recorder of a chain of ``[]`` / ``.attr`` / ``()`` operations on a value that does not exist
    yet.  ``eval(base)`` replays the chain on ``base``; DummyObjects appearing inside call
    arguments are evaluated against the same base first.

        >>> DummyObject().weight[0].numel().eval(torch.nn.Linear(5, 3))
        5
    """
    __slots__ = ('_operators',)

    def __init__(self, operators=None):
        object.__setattr__(self, '_operators', list(operators) if operators else [])

    def _extended(self, op):
        return DummyObject(self._operators + [op])

    def __getitem__(self, item):
        return self._extended((_OP_ITEM, item))

    def __getattr__(self, item):
        if item.startswith('__') and item.endswith('__'):
            raise AttributeError(item)  # keep copy / pickle / inspection protocols sane
        return self._extended((_OP_ATTR, item))

    def __call__(self, *args, **kwargs):
        return self._extended((_OP_CALL, args, kwargs))

    def eval(self, base_value):
        def resolve(v):
            return v.eval(base_value) if isinstance(v, DummyObject) else v

        value = base_value
        for op in self._operators:
            if isinstance(op, GetFirstItem):
                value = value[0] if isinstance(value, (tuple, list)) else value
            elif op[0] == _OP_ITEM:
                value = value[op[1]]
            elif op[0] == _OP_ATTR:
                value = getattr(value, op[1])
            else:
                value = value(*[resolve(a) for a in op[1]], **{k: resolve(v) for k, v in op[2].items()})
        return value


class VmapInfo:
    """Batch dimension (int or None) of every positional / keyword argument for ``vmap``."""

    def __init__(self, *args, **kwargs):
        for v in list(args) + list(kwargs.values()):
            if v is not None and not isinstance(v, int):
                raise TypeError('Every argument has to be int or None.')
        self.args_batch_dims: Tuple[int] = args
        self.kwargs_batch_dims: Dict[str, int] = kwargs


class GradientMaker:
    """Base class of every ``XXXGradientMaker``; on its own it is the plain first-order drop-in.

    Args:
        model (Module): module whose parameters receive the gradient.
    """
    _loss_reduction = None  # subclasses force 'sum' / 'none' on the registered loss

    def __init__(self, model: nn.Module):
        self.model = model
        self._model_fn = None
        self._model_args = ()
        self._model_kwargs = dict()
        self._model_output = None
        self._model_vmap_info: VmapInfo = None
        self._logits: Tensor = None
        self._loss_fn = None
        self._loss_fn_args = ()
        self._loss_fn_kwargs = dict()
        self._loss_vmap_info: VmapInfo = None
        self._loss: Tensor = None
        self._dummy_loss: DummyObject = None
        self._dummy_logits = DummyObject([GetFirstItem()])

    # ------------------------------------------------------------------ registration
    def setup_model_call(self, model_fn: Callable, *args, **kwargs) -> DummyObject:
        """Registers ``model_fn(*args, **kwargs)`` as the forward computation and returns the
        placeholder of its output."""
        self._model_fn = model_fn
        self._model_args = args
        self._model_kwargs = kwargs
        return DummyObject()

    def setup_model_vmap_info(self, *args, **kwargs):
        self._model_vmap_info = VmapInfo(*args, **kwargs)

    def setup_loss_call(self, loss_fn: Callable, *args, **kwargs):
        """Registers ``loss_fn(*args, **kwargs)``; arguments may be (derived from) the placeholder
        returned by :meth:`setup_model_call`."""
        self._loss_fn = loss_fn
        self._loss_fn_args = args
        self._loss_fn_kwargs = kwargs

    def setup_loss_vmap_info(self, *args, **kwargs):
        self._loss_vmap_info = VmapInfo(*args, **kwargs)

    def setup_loss_repr(self, dummy_loss: DummyObject):
        """Alternative to :meth:`setup_loss_call` for models that return their own loss:
        ``gm.setup_loss_repr(dummy_y[1])`` / ``dummy_y.loss`` / ``dummy_y["loss"]``."""
        if not isinstance(dummy_loss, DummyObject):
            raise TypeError(f'dummy_loss has to be an {DummyObject}, not {type(dummy_loss)}.')
        self._dummy_loss = dummy_loss

    def setup_logits_repr(self, dummy_logits: DummyObject):
        """Tells Fisher-based makers where the logits are inside the model output."""
        if not isinstance(dummy_logits, DummyObject):
            raise TypeError(f'dummy_logits has to be an {DummyObject}, not {type(dummy_logits)}.')
        self._dummy_logits = dummy_logits

    @property
    def model_output(self):
        return self._model_output

    @property
    def loss(self):
        return self._loss

    # ------------------------------------------------------------------ evaluation
    def call_model(self) -> Any:
        if self._model_fn is None:
            raise ValueError('model_fn is not set. Call setup_model_call() before calling forward_and_backward().')
        self._model_output = self._model_fn(*self._model_args, **self._model_kwargs)
        self._logits = self._dummy_logits.eval(self._model_output)
        return self._model_output

    def call_loss(self) -> Tensor:
        if self._loss_fn is not None:
            self._loss = self._call_loss_fn()
        elif self._dummy_loss is not None:
            self._loss = self._dummy_loss.eval(self._model_output)
        else:
            raise ValueError('Neither loss_fn nor loss_repr is not set. '
                             'Call setup_loss_call() or setup_loss_repr() before calling forward_and_backward().')
        return self._loss

    def forward(self):
        self.call_model()
        self.call_loss()

    def backward(self):
        self._loss.backward()

    def forward_and_backward(self) -> Tuple[Any, Tensor]:
        """One forward and one backward pass; returns ``(model_output, loss)``."""
        self.forward()
        self.backward()
        return self._model_output, self._loss

    def delegate_forward_and_backward(self, other, *args, **kwargs):
        """Lets ``other`` (another GradientMaker) run the registered computation and mirrors its
        ``model_output`` / ``loss`` on ``self``."""
        if self._model_fn is None:
            raise ValueError('model_fn is not set. Call setup_model_call() before calling forward_and_backward().')
        if self._loss_fn is None and self._dummy_loss is None:
            raise ValueError('Neither loss_fn nor loss_repr is set. '
                             'Call setup_loss_call() or setup_loss_repr() before calling forward_and_backward().')
        other.setup_model_call(self._model_fn, *self._model_args, **self._model_kwargs)
        if self._loss_fn is None:
            other.setup_loss_repr(self._dummy_loss)
        else:
            other.setup_loss_call(self._loss_fn, *self._loss_fn_args, **self._loss_fn_kwargs)
        other.setup_logits_repr(self._dummy_logits)
        other.forward_and_backward(*args, **kwargs)
        self._model_output = other.model_output
        self._loss = other.loss
        return self._model_output, self._loss

    def _resolved_loss_args(self, output=None):
        output = self._model_output if output is None else output

        def resolve(v):
            return v.eval(output) if isinstance(v, DummyObject) else v

        return ([resolve(a) for a in self._loss_fn_args],
                {k: resolve(v) for k, v in self._loss_fn_kwargs.items()})

    def _call_loss_fn(self) -> Tensor:
        reduction = self._loss_reduction
        args, kwargs = self._resolved_loss_args()
        if reduction is None:
            return self._loss_fn(*args, **kwargs)
        if not has_reduction(self._loss_fn):
            raise AttributeError('loss_fn has to have "reduction" option')
        if isinstance(self._loss_fn, nn.Module):
            saved = self._loss_fn.reduction
            self._loss_fn.reduction = reduction
            try:
                return self._loss_fn(*args, **kwargs)
            finally:
                self._loss_fn.reduction = saved
        kwargs['reduction'] = reduction
        return self._loss_fn(*args, **kwargs)

    # ------------------------------------------------------------------ functional utilities
    def _functional_parts(self):
        if self._model_fn is None:
            raise ValueError('model_fn is not set. Call setup_model_call().')
        if not isinstance(self._model_fn, nn.Module):
            raise TypeError('model_fn has to be an object of torch.nn.Module.')
        module = self._model_fn
        params = OrderedDict((k, v.detach()) for k, v in module.named_parameters() if v.requires_grad)
        frozen = OrderedDict((k, v.detach()) for k, v in module.named_parameters() if not v.requires_grad)
        buffers = OrderedDict((k, v) for k, v in module.named_buffers())
        names = list(params.keys())

        def call(param_tuple, *args, **kwargs):
            state = dict(zip(names, param_tuple))
            state.update(frozen)
            state.update(buffers)
            return ft.functional_call(module, state, args, kwargs)

        return call, tuple(params.values())

    def _get_stateless_model_fn_params_only(self):
        call, params = self._functional_parts()
        return (lambda p: call(p, *self._model_args, **self._model_kwargs)), params

    def _get_stateless_logit_fn_params_only(self):
        model_fn, params = self._get_stateless_model_fn_params_only()
        return (lambda p: self._dummy_logits.eval(model_fn(p))), params

    def _get_stateless_model_loss_fn_params_only(self, return_output=False):
        if self._loss_reduction == 'none':
            raise ValueError('Stateless loss function is not available when _loss_reduction == "none".')
        model_fn, params = self._get_stateless_model_fn_params_only()

        def fn(p):
            self._model_output = model_fn(p)
            self.call_loss()
            return (self._loss, self._model_output) if return_output else self._loss

        return fn, params

    def _get_random_tangents(self):
        if not isinstance(self._model_fn, nn.Module):
            raise TypeError(f'_model_fn has to be {nn.Module}. Got {type(self._model_fn)}.')
        return tuple(torch.randn_like(p) for p in self._model_fn.parameters() if p.requires_grad)

    @torch.no_grad()
    def loss_grad(self, return_output=False) -> Tuple[Tensor, ...]:
        fn, params = self._get_stateless_model_loss_fn_params_only(return_output=return_output)
        return ft.grad(fn, has_aux=return_output)(params)

    @torch.no_grad()
    def per_example_loss_grads(self) -> Tuple[Tensor, ...]:
        """vmap(grad) over the batch dimension of every tensor argument (override the batch
        dimensions with ``setup_model_vmap_info`` / ``setup_loss_vmap_info``)."""
        call, params = self._functional_parts()
        m_args, m_kwargs = self._model_args, OrderedDict(self._model_kwargs)
        l_args, l_kwargs = self._loss_fn_args, OrderedDict(self._loss_fn_kwargs)

        def batch_dims(info: VmapInfo, args, kwargs):
            if info is None:
                return tuple(0 if isinstance(v, Tensor) else None for v in [*args, *kwargs.values()])
            if len(args) != len(info.args_batch_dims):
                raise ValueError(f'len(ref_args) ({len(args)}) does not match '
                                 f'args_batch_dims ({len(info.args_batch_dims)}).')
            if set(kwargs.keys()) != set(info.kwargs_batch_dims.keys()):
                raise ValueError('keyword arguments do not match kwargs_batch_dims.')
            return tuple(info.args_batch_dims) + tuple(info.kwargs_batch_dims[k] for k in kwargs)

        flat = [*m_args, *m_kwargs.values()]
        dims = batch_dims(self._model_vmap_info, m_args, m_kwargs)
        n_model = len(flat)
        if self._loss_fn is not None:
            flat += [*l_args, *l_kwargs.values()]
            dims += batch_dims(self._loss_vmap_info, l_args, l_kwargs)
        # DummyObjects are not tensors: they travel through a closure, not through vmap
        is_dummy = [isinstance(v, DummyObject) for v in flat]
        dims = tuple(None if d else dim for d, dim in zip(is_dummy, dims))
        tensors = [None if d else v for d, v in zip(is_dummy, flat)]

        def regroup(values, ref_args, ref_kwargs):
            args = tuple(values[:len(ref_args)])
            kwargs = {k: values[len(ref_args) + i] for i, k in enumerate(ref_kwargs.keys())}
            return args, kwargs

        def loss_of_one(p, *one):
            one = [flat[i] if is_dummy[i] else (v if dims[i] is None else v.unsqueeze(dims[i]))
                   for i, v in enumerate(one)]
            args, kwargs = regroup(one[:n_model], m_args, m_kwargs)
            output = call(p, *args, **kwargs)
            if self._loss_fn is None:
                return self._dummy_loss.eval(output)
            rest = [v.eval(output) if isinstance(v, DummyObject) else v for v in one[n_model:]]
            args, kwargs = regroup(rest, l_args, l_kwargs)
            return self._loss_fn(*args, **kwargs)

        return ft.vmap(ft.grad(loss_of_one), in_dims=(None,) + dims)(params, *tensors)

    @torch.no_grad()
    def loss_hessian(self) -> Tuple[Tuple[Tensor, ...], ...]:
        fn, params = self._get_stateless_model_loss_fn_params_only()
        return ft.hessian(fn)(params)

    @torch.no_grad()
    def loss_hvp(self, tangents=None, accumulate_grad=True) -> Tuple[Tensor, ...]:
        """Hessian-vector product by forward-over-reverse; optionally also accumulates the
        gradient into ``param.grad``."""
        fn, params = self._get_stateless_model_loss_fn_params_only()
        if tangents is None:
            tangents = self._get_random_tangents()
        grads, hvps = ft.jvp(ft.grad(fn), (params,), (tuple(tangents),))
        if accumulate_grad:
            targets = [p for p in self.model.parameters() if p.requires_grad]
            for p, g in zip(targets, grads):
                if p.grad is None:
                    p.grad = g.clone()
                else:
                    p.grad.add_(g)
        return hvps

    @torch.no_grad()
    def logit_jacobian(self) -> Tuple[Tensor, ...]:
        fn, params = self._get_stateless_logit_fn_params_only()
        return ft.jacrev(fn)(params)

    @torch.no_grad()
    def logit_jvp(self, tangents=None, return_model_output=False):
        fn, params = self._get_stateless_logit_fn_params_only()
        if tangents is None:
            tangents = self._get_random_tangents()
        logits, jvp = ft.jvp(fn, (params,), (tuple(tangents),))
        return (jvp, logits) if return_model_output else jvp

    def fvp(self, loss_type, data_size=None, tangents=None, return_model_output=False):
        """Fisher(GGN)-vector product J^T H_L J v for cross-entropy or MSE."""
        if loss_type not in [LOSS_MSE, LOSS_CROSS_ENTROPY]:
            raise ValueError(f'Invalid loss type: {loss_type}. {[LOSS_CROSS_ENTROPY, LOSS_MSE]} are supported.')
        if tangents is None:
            tangents = self._get_random_tangents()
        module = self._model_fn
        params = [p for p in module.parameters() if p.requires_grad]
        fn, flat_params = self._get_stateless_logit_fn_params_only()
        with torch.no_grad():
            y_detached, jvp = ft.jvp(fn, (flat_params,), (tuple(tangents),))
        if y_detached.ndim != 2:
            raise ValueError(f'Number of output dimensions has to be 2. Got {y_detached.ndim}.')
        if data_size is None:
            data_size = y_detached.shape[0]
        if loss_type == LOSS_CROSS_ENTROPY:
            probs = F.softmax(y_detached, dim=1)
            grad_outputs = probs * jvp - probs * (probs * jvp).sum(dim=1, keepdim=True)
        else:
            grad_outputs = jvp
        y = self._dummy_logits.eval(module(*self._model_args, **self._model_kwargs))
        out = torch.autograd.grad(y, params, grad_outputs=grad_outputs / data_size)
        return (out, y) if return_model_output else out

    @torch.no_grad()
    def nvp(self, cotangents=None, return_model_output=False):
        """NTK-vector product J J^T u."""
        fn, params = self._get_stateless_logit_fn_params_only()
        y, vjp_fn = ft.vjp(fn, params)
        if cotangents is None:
            cotangents = torch.randn_like(y)
        elif isinstance(cotangents, (tuple, list)):
            cotangents = cotangents[0]
        (vjp,) = vjp_fn(cotangents)
        nvp = ft.jvp(fn, (params,), (vjp,))[1]
        return (nvp, y) if return_model_output else nvp
