"""Model definitions used by the benchmarks, examples and tests (random initialisation only)."""
from .layers import FusedBatchNorm2d
from .resnet import ResNet, Bottleneck, resnet50, resnet_tiny
from .vit import VisionTransformer, vit_b_16, vit_tiny
from .gpt2 import GPT2, gpt2_medium, gpt2_tiny, next_token_loss

__all__ = ['FusedBatchNorm2d', 'ResNet', 'Bottleneck', 'resnet50', 'resnet_tiny', 'VisionTransformer', 'vit_b_16', 'vit_tiny',
           'GPT2', 'gpt2_medium', 'gpt2_tiny', 'next_token_loss']
