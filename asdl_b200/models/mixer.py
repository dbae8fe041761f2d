"""MLP-Mixer (patch embedding convolution, blocks of a token-mixing MLP across patches and a
channel-mixing MLP across features, global average pooling, linear head).  Every weight matrix is an
``nn.Linear`` (the token-mixing MLP acts on the transposed activation), so K-FAC hooks and
per-parameter methods see all of them.  Reference counterpart: the timm Mixer-B of
examples/arxiv_results/configs/mixer/*.json."""
import torch.nn as nn
import torch.nn.functional as F

__all__ = ['MlpMixer', 'mixer_b_16', 'mixer_tiny']


class _MixerBlock(nn.Module):
    def __init__(self, tokens, dim, token_hidden, channel_hidden):
        super().__init__()
        self.ln_1 = nn.LayerNorm(dim)
        self.token_fc1 = nn.Linear(tokens, token_hidden)
        self.token_fc2 = nn.Linear(token_hidden, tokens)
        self.ln_2 = nn.LayerNorm(dim)
        self.channel_fc1 = nn.Linear(dim, channel_hidden)
        self.channel_fc2 = nn.Linear(channel_hidden, dim)

    def forward(self, x):
        y = self.ln_1(x).transpose(1, 2)
        x = x + self.token_fc2(F.gelu(self.token_fc1(y))).transpose(1, 2)
        return x + self.channel_fc2(F.gelu(self.channel_fc1(self.ln_2(x))))


class MlpMixer(nn.Module):
    def __init__(self, image_size=224, patch_size=16, dim=768, depth=12, token_hidden=384, channel_hidden=3072,
                 num_classes=1000, in_channels=3):
        super().__init__()
        tokens = (image_size // patch_size) ** 2
        self.stem = nn.Conv2d(in_channels, dim, patch_size, stride=patch_size)
        self.blocks = nn.Sequential(*[_MixerBlock(tokens, dim, token_hidden, channel_hidden) for _ in range(depth)])
        self.ln = nn.LayerNorm(dim)
        self.head = nn.Linear(dim, num_classes)

    def forward(self, x):
        x = self.stem(x).flatten(2).transpose(1, 2)
        return self.head(self.ln(self.blocks(x)).mean(dim=1))


def mixer_b_16(num_classes=1000):
    return MlpMixer(224, 16, 768, 12, 384, 3072, num_classes)


def mixer_tiny(num_classes=10, image_size=32):
    return MlpMixer(image_size, 8, 32, 2, 24, 64, num_classes)
