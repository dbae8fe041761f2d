"""Layers of the model zoo that run on the library's own kernels."""
import torch
import torch.nn as nn

from .. import ops

__all__ = ['FusedBatchNorm2d']


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
