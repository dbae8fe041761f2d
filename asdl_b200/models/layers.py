"""Layers of the model zoo that run on the library's own kernels."""
import torch
import torch.nn as nn

from .. import ops

__all__ = ['FusedBatchNorm2d', 'FusedLayerNorm', 'grouped_bf16_weights']


class FusedBatchNorm2d(nn.BatchNorm2d):
    """``nn.BatchNorm2d`` with an optional fused residual add and ReLU,
    ``y = act(batch_norm(x) + residual)``, whose training-mode forward / backward run on the
    library's NHWC bf16 kernels (:func:`asdl_b200.ops.batch_norm_train`) when the input is a
    channels_last bf16 CUDA tensor, and as ``nn.BatchNorm2d`` + add + ReLU otherwise.  Same
    parameters, buffers and state dict as the parent.

    Args (beyond ``nn.BatchNorm2d``):
        act: ``None`` or ``'relu'``.

    With ``act=None`` and no residual the output is the plain normalised tensor and curvature
    hooks treat the layer like any BatchNorm2d.  With a fused activation or residual the module
    output no longer determines the normalised input; the layer then keeps ``(x, mean, invstd, y)``
    of its last training forward pass in ``curvature_inputs`` while ``keep_curvature_inputs`` is
    set (the fused K-FAC maker sets it during its curvature passes).
    """

    def __init__(self, num_features, eps=1e-5, momentum=0.1, affine=True, track_running_stats=True,
                 act=None, **kwargs):
        super().__init__(num_features, eps, momentum, affine, track_running_stats, **kwargs)
        if act not in (None, 'relu'):
            raise ValueError("act has to be None or 'relu'")
        self.act = act
        self.keep_curvature_inputs = False
        self.curvature_inputs = None

    @property
    def fused_output(self):
        """True when the module output is not the plain normalised tensor."""
        return self.act is not None or self._used_residual

    _used_residual = False

    def forward(self, x, residual=None):
        relu = self.act == 'relu'
        self._used_residual = residual is not None
        if (self.training and self.track_running_stats and self.momentum is not None
                and ops.batch_norm_train_supported(x, self.weight, self.bias, residual)):
            y, mean, invstd = ops.batch_norm_train(x, self.weight, self.bias, self.running_mean, self.running_var,
                                                   self.momentum, self.eps, residual=residual, relu=relu,
                                                   num_batches_tracked=self.num_batches_tracked,
                                                   return_stats=True)
            if self.keep_curvature_inputs:
                self.curvature_inputs = (x.detach(), mean, invstd, y.detach() if relu else None)
            return y
        y = super().forward(x)
        if self.keep_curvature_inputs:
            with torch.no_grad():
                if self.training or self.running_mean is None:
                    xf = x.detach().float()
                    mean = xf.mean(dim=(0, 2, 3))
                    invstd = torch.rsqrt(xf.var(dim=(0, 2, 3), unbiased=False) + self.eps)
                else:
                    mean, invstd = self.running_mean, torch.rsqrt(self.running_var + self.eps)
        if residual is not None:
            y = y + residual
        if relu:
            y = torch.relu(y)
        if self.keep_curvature_inputs:
            self.curvature_inputs = (x.detach(), mean, invstd, y.detach() if relu else None)
        return y

    def extra_repr(self):
        return super().extra_repr() + (f', act={self.act}' if self.act else '')


class FusedLayerNorm(nn.LayerNorm):
    """``nn.LayerNorm`` over the last dimension whose forward / backward run on the library's bf16
    kernels (:func:`asdl_b200.ops.layer_norm`) for contiguous bf16 CUDA inputs of a supported
    feature size, and exactly like the parent otherwise.  Under autocast the parent computes in
    fp32 and returns fp32; this layer keeps the activation in bf16 (statistics in fp32)."""

    def forward(self, x):
        if (len(self.normalized_shape) == 1 and self.elementwise_affine and self.bias is not None
                and x.is_cuda and torch.is_autocast_enabled('cuda')
                and torch.get_autocast_dtype('cuda') == torch.bfloat16):
            xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
            xb = xb if xb.is_contiguous() else xb.contiguous()
            if ops.layer_norm_supported(xb, self.weight, self.bias):
                return ops.layer_norm(xb, self.weight, self.bias, self.eps)
        return super().forward(x)


class _GroupedCast(torch.autograd.Function):
    """fp32 parameters -> bf16 copies that live in one flat buffer (a few multi-tensor launches
    instead of one cast kernel per parameter); the backward pass converts the bf16 gradients back to
    fp32 the same way.  Every copy keeps the memory format of its parameter."""

    @staticmethod
    def forward(ctx, *weights):
        total = sum((w.numel() + 7) // 8 * 8 for w in weights)
        flat = torch.empty(total, device=weights[0].device, dtype=torch.bfloat16)
        outs, off = [], 0
        for w in weights:
            chunk = flat[off:off + w.numel()]
            off += (w.numel() + 7) // 8 * 8
            outs.append(chunk.as_strided(w.shape, w.stride()) if w.is_contiguous() or _dense(w)
                        else chunk.view(w.shape))
        torch._foreach_copy_(outs, [w.detach() for w in weights])
        ctx.meta = [(w.shape, w.stride()) for w in weights]
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        present = [(i, g) for i, g in enumerate(grads) if g is not None]
        outs = [None] * len(grads)
        if present:
            dst = [torch.empty_strided(ctx.meta[i][0], ctx.meta[i][1], device=g.device, dtype=torch.float32)
                   if _dense_meta(*ctx.meta[i]) else torch.empty(ctx.meta[i][0], device=g.device, dtype=torch.float32)
                   for i, g in present]
            same, same_dst = [], []
            kernels = present[0][1].is_cuda and ops.cuda_kernels_enabled(present[0][1])
            for (i, g), d in zip(present, dst):
                # autograd hands the weight gradient of a linear layer over as a transposed tensor: a
                # tiled transposing cast instead of a strided element-wise copy
                if (kernels and g.ndim == 2 and g.dtype == torch.bfloat16 and d.is_contiguous()
                        and g.stride(0) == 1 and g.stride(1) >= g.shape[0] and g.shape[0] > 1):
                    ops.extension().transpose_cast(g, d)
                else:
                    same.append(g)
                    same_dst.append(d)
            if same:
                torch._foreach_copy_(same_dst, same)
            for (i, _), d in zip(present, dst):
                outs[i] = d
        return tuple(outs)


def _dense_meta(shape, stride):
    """True when (shape, stride) covers exactly numel elements without gaps (any dimension order)."""
    expected = 1
    for size, st in sorted(((s, t) for s, t in zip(shape, stride) if s > 1), key=lambda p: p[1]):
        if st != expected:
            return False
        expected *= size
    return True


def _dense(t):
    return _dense_meta(t.shape, t.stride())


class grouped_bf16_weights:
    """Context manager: inside it, the ``weight`` of every Conv2d / Linear of ``model`` is a bf16 copy
    made by one grouped cast (differentiable), so autocast finds nothing left to convert."""

    def __init__(self, model):
        self.model = model

    def __enter__(self):
        from torch.nn.utils.stateless import _reparametrize_module
        names, weights = [], []
        for name, module in self.model.named_modules():
            if isinstance(module, (nn.Conv2d, nn.Linear)) and module.weight.dtype == torch.float32:
                names.append(f'{name}.weight' if name else 'weight')
                weights.append(module.weight)
        self._ctx = None
        if weights:
            casts = _GroupedCast.apply(*weights)
            self._ctx = _reparametrize_module(self.model, dict(zip(names, casts)))
            self._ctx.__enter__()
        return self

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)
        return False
