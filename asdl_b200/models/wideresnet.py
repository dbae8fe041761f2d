"""Wide residual network for 32 x 32 images (WRN-d-k: three stages of pre-activation basic blocks,
widths 16k / 32k / 64k, depth d = 6n + 4), the CIFAR model family of the reference's training
recipes (examples/arxiv_results/models/wideresnet.py, configs/wideresnet28/*.json).  Activations read by
curvature hooks are never modified in place."""
import torch
import torch.nn as nn
import torch.nn.functional as F

__all__ = ['WideResNet', 'wideresnet28', 'wideresnet_tiny']


class _PreActBlock(nn.Module):
    def __init__(self, in_planes, planes, stride, dropout):
        super().__init__()
        self.bn1 = nn.BatchNorm2d(in_planes)
        self.conv1 = nn.Conv2d(in_planes, planes, 3, stride=stride, padding=1, bias=False)
        self.bn2 = nn.BatchNorm2d(planes)
        self.conv2 = nn.Conv2d(planes, planes, 3, padding=1, bias=False)
        self.dropout = dropout
        self.shortcut = None
        if stride != 1 or in_planes != planes:
            self.shortcut = nn.Conv2d(in_planes, planes, 1, stride=stride, bias=False)

    def forward(self, x):
        out = F.relu(self.bn1(x))
        skip = x if self.shortcut is None else self.shortcut(out)
        out = self.conv1(out)
        out = F.relu(self.bn2(out))
        if self.dropout > 0:
            out = F.dropout(out, self.dropout, self.training)
        return self.conv2(out) + skip


class WideResNet(nn.Module):
    def __init__(self, depth=28, widen_factor=10, num_classes=10, dropout=0.0, in_channels=3):
        super().__init__()
        if (depth - 4) % 6 != 0:
            raise ValueError('depth has to be 6n + 4')
        n = (depth - 4) // 6
        widths = [16, 16 * widen_factor, 32 * widen_factor, 64 * widen_factor]
        self.conv1 = nn.Conv2d(in_channels, widths[0], 3, padding=1, bias=False)
        blocks, in_planes = [], widths[0]
        for stage, planes in enumerate(widths[1:]):
            for i in range(n):
                blocks.append(_PreActBlock(in_planes, planes, 2 if stage > 0 and i == 0 else 1, dropout))
                in_planes = planes
        self.blocks = nn.Sequential(*blocks)
        self.bn = nn.BatchNorm2d(in_planes)
        self.fc = nn.Linear(in_planes, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Conv2d):
                nn.init.kaiming_normal_(m.weight, mode='fan_out', nonlinearity='relu')

    def forward(self, x):
        x = F.relu(self.bn(self.blocks(self.conv1(x))))
        return self.fc(torch.flatten(F.adaptive_avg_pool2d(x, 1), 1))


def wideresnet28(num_classes=10, widen_factor=10):
    return WideResNet(28, widen_factor, num_classes)


def wideresnet_tiny(num_classes=10):
    """WRN-10-1 for tests."""
    return WideResNet(10, 1, num_classes)
