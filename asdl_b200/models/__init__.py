"""Model definitions used by the benchmarks, examples and tests (random initialisation only)."""
from .resnet import ResNet, Bottleneck, resnet50, resnet_tiny

__all__ = ['ResNet', 'Bottleneck', 'resnet50', 'resnet_tiny']
