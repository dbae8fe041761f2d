"""Layers of the model zoo that run on the library's own kernels."""
import torch
import torch.nn as nn

from .. import ops

__all__ = ['FusedBatchNorm2d']


class FusedBatchNorm2d(nn.BatchNorm2d):
    """``nn.BatchNorm2d`` whose training-mode forward / backward run on the library's NHWC bf16
    kernels (:func:`asdl_b200.ops.batch_norm_train`) when the input is a channels_last bf16 CUDA
    tensor, and exactly like the parent otherwise.  Same parameters, buffers, state dict and
    output semantics as the parent, so curvature hooks treat it as a BatchNorm2d."""

    def forward(self, x):
        if (self.training and self.track_running_stats and self.momentum is not None
                and ops.batch_norm_train_supported(x, self.weight, self.bias)):
            self.num_batches_tracked.add_(1)
            return ops.batch_norm_train(x, self.weight, self.bias, self.running_mean, self.running_var,
                                        self.momentum, self.eps)
        return super().forward(x)
