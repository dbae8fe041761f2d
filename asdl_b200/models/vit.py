"""Vision Transformer (ViT-B/16 topology: patch-embedding convolution, class token, learned position
embedding, pre-norm encoder blocks, linear head) written so that every weight matrix is visible to
the curvature hooks: the attention projections are plain ``nn.Linear`` modules (a fused
``nn.MultiheadAttention`` keeps q/k/v in one bare parameter that module hooks never see).  The
reference takes its ViT / Mixer models from timm (examples/arxiv_results/train.py:349,
configs/vit/*.json)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import FusedLayerNorm, grouped_bf16_weights

__all__ = ['VisionTransformer', 'vit_b_16', 'vit_tiny_patch16_224', 'vit_tiny']


class SelfAttention(nn.Module):
    def __init__(self, dim, heads, causal=False):
        super().__init__()
        assert dim % heads == 0
        self.heads, self.causal = heads, causal
        self.qkv = nn.Linear(dim, 3 * dim)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x):
        b, s, d = x.shape
        qkv = self.qkv(x).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
        out = F.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2], is_causal=self.causal)
        return self.proj(out.transpose(1, 2).reshape(b, s, d))


class EncoderBlock(nn.Module):
    def __init__(self, dim, heads, mlp_dim, causal=False):
        super().__init__()
        self.ln_1 = FusedLayerNorm(dim, eps=1e-6)
        self.attn = SelfAttention(dim, heads, causal)
        self.ln_2 = FusedLayerNorm(dim, eps=1e-6)
        self.fc1 = nn.Linear(dim, mlp_dim)
        self.fc2 = nn.Linear(mlp_dim, dim)

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.fc2(F.gelu(self.fc1(self.ln_2(x))))


class VisionTransformer(nn.Module):
    def __init__(self, image_size=224, patch_size=16, num_layers=12, num_heads=12, hidden_dim=768,
                 mlp_dim=3072, num_classes=1000, in_channels=3):
        super().__init__()
        assert image_size % patch_size == 0
        self.conv_proj = nn.Conv2d(in_channels, hidden_dim, patch_size, stride=patch_size)
        seq = (image_size // patch_size) ** 2 + 1
        self.class_token = nn.Parameter(torch.zeros(1, 1, hidden_dim))
        self.pos_embedding = nn.Parameter(torch.empty(1, seq, hidden_dim).normal_(std=0.02))
        self.layers = nn.ModuleList(EncoderBlock(hidden_dim, num_heads, mlp_dim) for _ in range(num_layers))
        self.ln = FusedLayerNorm(hidden_dim, eps=1e-6)
        self.head = nn.Linear(hidden_dim, num_classes)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.trunc_normal_(m.weight, std=0.02)
                nn.init.zeros_(m.bias)

    def forward(self, x):
        if x.is_cuda and torch.is_autocast_enabled('cuda') and torch.get_autocast_dtype('cuda') == torch.bfloat16:
            with grouped_bf16_weights(self):  # one grouped cast instead of one cast kernel per layer
                return self._forward(x)
        return self._forward(x)

    def _forward(self, x):
        x = self.conv_proj(x).flatten(2).transpose(1, 2)
        x = torch.cat([self.class_token.expand(x.shape[0], -1, -1).to(x.dtype), x], dim=1)
        x = x + self.pos_embedding.to(x.dtype)
        for layer in self.layers:
            x = layer(x)
        return self.head(self.ln(x)[:, 0])


def vit_b_16(num_classes=1000):
    return VisionTransformer(224, 16, 12, 12, 768, 3072, num_classes)


def vit_tiny_patch16_224(num_classes=10):
    """ViT-Ti/16 (12 blocks of width 192 with 3 heads): the transformer of the reference's CIFAR-10
    recipes (examples/arxiv_results/configs/vit/*.json), there with pretrained weights, here random."""
    return VisionTransformer(224, 16, 12, 3, 192, 768, num_classes)


def vit_tiny(num_classes=10, image_size=32):
    """Two-block ViT for tests."""
    return VisionTransformer(image_size, 8, 2, 2, 32, 64, num_classes)
