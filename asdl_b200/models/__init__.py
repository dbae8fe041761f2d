"""Model definitions used by the benchmarks, examples and tests (random initialisation only)."""
from .layers import FusedBatchNorm2d
from .resnet import ResNet, Bottleneck, resnet50, resnet_tiny
from .vit import VisionTransformer, vit_b_16, vit_tiny_patch16_224, vit_tiny
from .cifar import MLP, SmallCNN, BasicBlock, CifarResNet, resnet18, resnet34
from .gpt2 import GPT2, gpt2_medium, gpt2_tiny, next_token_loss
from .wideresnet import WideResNet, wideresnet28, wideresnet_tiny
from .mixer import MlpMixer, mixer_b_16, mixer_tiny

__all__ = ['FusedBatchNorm2d', 'ResNet', 'Bottleneck', 'resnet50', 'resnet_tiny', 'VisionTransformer', 'vit_b_16', 'vit_tiny',
           'GPT2', 'gpt2_medium', 'gpt2_tiny', 'next_token_loss', 'WideResNet', 'wideresnet28', 'wideresnet_tiny',
           'MlpMixer', 'mixer_b_16', 'mixer_tiny', 'vit_tiny_patch16_224', 'MLP', 'SmallCNN', 'BasicBlock', 'CifarResNet',
           'resnet18', 'resnet34']
