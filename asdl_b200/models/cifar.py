"""Small-image classifiers of the reference's training recipes: the fully connected network
(examples/arxiv_results/models/mlp.py, configs/mlp/*.json: width 2048, depth 3 on MNIST), the
two-convolution network (models/cnn.py) and the 32 x 32 ResNet-18 / 34 (models/resnet.py,
configs/resnet18/*.json: 3 x 3 stem without max-pooling, four stages of basic blocks).

Residual blocks can use :class:`~asdl_b200.models.layers.FusedBatchNorm2d` (``fused=True``: BatchNorm +
ReLU / residual add in one NHWC bf16 kernel on CUDA).  Activations that curvature hooks read are
never modified in place."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import FusedBatchNorm2d

__all__ = ['MLP', 'SmallCNN', 'BasicBlock', 'CifarResNet', 'resnet18', 'resnet34']


class MLP(nn.Module):
    """``depth`` linear layers (``depth - 1`` hidden ones of ``width`` units) with ReLU between them."""

    def __init__(self, width=2048, depth=3, in_features=28 * 28, num_classes=10, bias=True):
        super().__init__()
        if depth < 2:
            raise ValueError('depth counts the linear layers and has to be at least 2')
        dims = [in_features] + [width] * (depth - 1) + [num_classes]
        layers = []
        for i, (d_in, d_out) in enumerate(zip(dims[:-1], dims[1:])):
            layers.append(nn.Linear(d_in, d_out, bias=bias))
            if i < depth - 1:
                layers.append(nn.ReLU())
        self.layers = nn.Sequential(*layers)

    def forward(self, x):
        return self.layers(torch.flatten(x, 1))


class SmallCNN(nn.Module):
    """conv5-pool-conv5-pool-fc-fc for 28 x 28 or 32 x 32 inputs."""

    def __init__(self, in_channels=1, num_classes=10, image_size=28):
        super().__init__()
        self.conv1 = nn.Conv2d(in_channels, 32, 5, padding=2)
        self.conv2 = nn.Conv2d(32, 64, 5, padding=2)
        side = image_size // 4
        self.fc1 = nn.Linear(64 * side * side, 512)
        self.fc2 = nn.Linear(512, num_classes)

    def forward(self, x):
        x = F.max_pool2d(F.relu(self.conv1(x)), 2)
        x = F.max_pool2d(F.relu(self.conv2(x)), 2)
        return self.fc2(F.relu(self.fc1(torch.flatten(x, 1))))


def _bn(planes, fused, act=None):
    return FusedBatchNorm2d(planes, act=act) if fused else nn.BatchNorm2d(planes)


class BasicBlock(nn.Module):
    expansion = 1

    def __init__(self, in_planes, planes, stride=1, fused=False):
        super().__init__()
        self.fused = fused
        self.conv1 = nn.Conv2d(in_planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn1 = _bn(planes, fused, 'relu')
        self.conv2 = nn.Conv2d(planes, planes, 3, padding=1, bias=False)
        self.bn2 = _bn(planes, fused, 'relu')
        self.downsample = None
        if stride != 1 or in_planes != planes:
            self.downsample = nn.Sequential(nn.Conv2d(in_planes, planes, 1, stride=stride, bias=False), _bn(planes, fused))

    def forward(self, x):
        skip = x if self.downsample is None else self.downsample(x)
        if self.fused:
            return self.bn2(self.conv2(self.bn1(self.conv1(x))), residual=skip)
        out = F.relu(self.bn1(self.conv1(x)))
        return F.relu(self.bn2(self.conv2(out)) + skip)


class CifarResNet(nn.Module):
    def __init__(self, num_blocks=(2, 2, 2, 2), num_classes=10, in_channels=3, width=64, fused=False):
        super().__init__()
        self.fused = fused
        self.conv1 = nn.Conv2d(in_channels, width, 3, padding=1, bias=False)
        self.bn1 = _bn(width, fused, 'relu')
        stages, in_planes = [], width
        for stage, count in enumerate(num_blocks):
            planes = width * 2 ** stage
            for i in range(count):
                stages.append(BasicBlock(in_planes, planes, 2 if stage > 0 and i == 0 else 1, fused))
                in_planes = planes
        self.blocks = nn.Sequential(*stages)
        self.fc = nn.Linear(in_planes, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')

    def forward(self, x):
        x = self.bn1(self.conv1(x))
        if not self.fused:
            x = F.relu(x)
        x = self.blocks(x)
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def resnet18(num_classes=10, fused=False, **kwargs):
    return CifarResNet((2, 2, 2, 2), num_classes, fused=fused, **kwargs)


def resnet34(num_classes=10, fused=False, **kwargs):
    return CifarResNet((3, 4, 6, 3), num_classes, fused=fused, **kwargs)
