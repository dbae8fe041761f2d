"""ResNet-50 with the torchvision topology (stem 7x7/2 + max-pool, bottleneck stages
[3, 4, 6, 3] with the stride on the 3x3 convolution, global average pool, linear head), written
for curvature capture: activations that the statistics hooks read are never overwritten in place,
and the module runs in channels_last / bf16 autocast without layout changes between layers.
The reference trains the torchvision model (examples/train_resnet50_with_kfac.py:144-154) and CIFAR
ResNets of its own (examples/arxiv_results/models/resnet.py)."""
import torch
import torch.nn as nn

from .layers import FusedBatchNorm2d, grouped_bf16_weights

__all__ = ['ResNet', 'Bottleneck', 'resnet50', 'resnet_tiny']


class Bottleneck(nn.Module):
    expansion = 4

    def __init__(self, inplanes, planes, stride=1, downsample=None, fused=False):
        super().__init__()
        act = 'relu' if fused else None
        self.fused = fused
        self.conv1 = nn.Conv2d(inplanes, planes, 1, bias=False)
        self.bn1 = FusedBatchNorm2d(planes, act=act)
        self.conv2 = nn.Conv2d(planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn2 = FusedBatchNorm2d(planes, act=act)
        self.conv3 = nn.Conv2d(planes, planes * self.expansion, 1, bias=False)
        self.bn3 = FusedBatchNorm2d(planes * self.expansion, act=act)
        self.relu = nn.ReLU(inplace=False)
        self.downsample = downsample

    def forward(self, x):
        identity = x if self.downsample is None else self.downsample(x)
        if self.fused:  # the ReLUs and the residual add run inside the normalisation kernels
            out = self.bn2(self.conv2(self.bn1(self.conv1(x))))
            return self.bn3(self.conv3(out), identity)
        out = self.relu(self.bn1(self.conv1(x)))
        out = self.relu(self.bn2(self.conv2(out)))
        out = self.bn3(self.conv3(out))
        return self.relu(out + identity)


class ResNet(nn.Module):
    """``fused=True`` folds every ReLU and residual add into the preceding normalisation layer
    (:class:`FusedBatchNorm2d`); curvature of such layers is supported by
    ``FusedKfacGradientMaker``, while the generic makers need ``fused=False``."""

    def __init__(self, layers=(3, 4, 6, 3), num_classes=1000, width=64, in_channels=3, fused=False):
        super().__init__()
        self.inplanes = width
        self.fused = fused
        self.conv1 = nn.Conv2d(in_channels, width, 7, stride=2, padding=3, bias=False)
        self.bn1 = FusedBatchNorm2d(width, act='relu' if fused else None)
        self.relu = nn.ReLU(inplace=False)
        self.maxpool = nn.MaxPool2d(3, stride=2, padding=1)
        self.layer1 = self._make_layer(width, layers[0])
        self.layer2 = self._make_layer(width * 2, layers[1], stride=2)
        self.layer3 = self._make_layer(width * 4, layers[2], stride=2)
        self.layer4 = self._make_layer(width * 8, layers[3], stride=2)
        self.avgpool = nn.AdaptiveAvgPool2d((1, 1))
        self.fc = nn.Linear(width * 8 * Bottleneck.expansion, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')
            elif isinstance(m, nn.BatchNorm2d):
                nn.init.constant_(m.weight, 1)
                nn.init.constant_(m.bias, 0)

    def _make_layer(self, planes, blocks, stride=1):
        downsample = None
        if stride != 1 or self.inplanes != planes * Bottleneck.expansion:
            downsample = nn.Sequential(
                nn.Conv2d(self.inplanes, planes * Bottleneck.expansion, 1, stride=stride, bias=False),
                FusedBatchNorm2d(planes * Bottleneck.expansion))
        layers = [Bottleneck(self.inplanes, planes, stride, downsample, fused=self.fused)]
        self.inplanes = planes * Bottleneck.expansion
        layers += [Bottleneck(self.inplanes, planes, fused=self.fused) for _ in range(1, blocks)]
        return nn.Sequential(*layers)

    def forward(self, x):
        if self.fused and x.is_cuda and torch.is_autocast_enabled('cuda') and torch.get_autocast_dtype('cuda') == torch.bfloat16:
            with grouped_bf16_weights(self):  # one grouped cast instead of one cast kernel per layer
                return self._forward(x)
        return self._forward(x)

    def _forward(self, x):
        x = self.bn1(self.conv1(x))
        x = self.maxpool(x if self.fused else self.relu(x))
        x = self.layer4(self.layer3(self.layer2(self.layer1(x))))
        return self.fc(torch.flatten(self.avgpool(x), 1))


def resnet50(num_classes=1000, fused=True):
    return ResNet((3, 4, 6, 3), num_classes=num_classes, fused=fused)


def resnet_tiny(num_classes=10, width=8, fused=False):
    """Two-stage miniature with the same block structure, for tests and smoke runs."""
    return ResNet((1, 1, 1, 1), num_classes=num_classes, width=width, fused=fused)
