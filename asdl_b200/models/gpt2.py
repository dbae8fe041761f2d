"""GPT-2 (decoder-only transformer, learned token and position embeddings, pre-norm blocks, tied
output head) with ``nn.Linear`` projections, so that K-FAC's Linear hooks see every weight matrix
of the blocks.  ``ignore_for_kfac`` lists the modules that K-FAC must skip on this model: the
embeddings and the output head (a vocabulary-sized factor is 50257 x 50257) and the LayerNorms.
The reference only has layer-shape tables of such models for its cost model
(examples/prof/models/transformer.py:27-42); its Embedding operation is asdl/operations/embedding.py."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from .layers import FusedLayerNorm, grouped_bf16_weights
from .vit import SelfAttention

__all__ = ['GPT2', 'gpt2_medium', 'gpt2_tiny']


class Block(nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.ln_1 = FusedLayerNorm(dim)
        self.attn = SelfAttention(dim, heads, causal=True)
        self.ln_2 = FusedLayerNorm(dim)
        self.fc = nn.Linear(dim, 4 * dim)
        self.proj = nn.Linear(4 * dim, dim)

    def forward(self, x):
        x = x + self.attn(self.ln_1(x))
        return x + self.proj(F.gelu(self.fc(self.ln_2(x)), approximate='tanh'))


class GPT2(nn.Module):
    def __init__(self, vocab_size=50257, n_positions=1024, n_layer=24, n_head=16, n_embd=1024,
                 pad_vocab_to_multiple_of=64):
        super().__init__()
        # The embedding / output matrix is stored with its row count rounded up: an odd vocabulary
        # size (50257) makes the rows of the logits unaligned and pushes the output GEMMs onto slow
        # unaligned kernels.  The extra logits are forced to -inf, so losses and sampled labels are
        # those of the unpadded vocabulary.
        self.vocab_size = vocab_size
        m = max(1, pad_vocab_to_multiple_of)
        padded = (vocab_size + m - 1) // m * m
        mask = torch.zeros(padded)
        mask[vocab_size:] = float('-inf')
        self.register_buffer('vocab_mask', mask, persistent=False)
        self.wte = nn.Embedding(padded, n_embd)
        self.wpe = nn.Embedding(n_positions, n_embd)
        self.blocks = nn.ModuleList(Block(n_embd, n_head) for _ in range(n_layer))
        self.ln_f = FusedLayerNorm(n_embd)
        self.lm_head = nn.Linear(n_embd, padded, bias=False)
        self.lm_head.weight = self.wte.weight  # tied
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, std=0.02)
                if getattr(m, 'bias', None) is not None:
                    nn.init.zeros_(m.bias)
        for blk in self.blocks:  # residual projections are scaled down with depth
            nn.init.normal_(blk.proj.weight, std=0.02 / (2 * n_layer) ** 0.5)
            nn.init.normal_(blk.attn.proj.weight, std=0.02 / (2 * n_layer) ** 0.5)

    def forward(self, tokens):
        if tokens.is_cuda and torch.is_autocast_enabled('cuda') and torch.get_autocast_dtype('cuda') == torch.bfloat16:
            with grouped_bf16_weights(self):  # one grouped cast instead of one cast kernel per layer
                return self._forward(tokens)
        return self._forward(tokens)

    def _forward(self, tokens):
        pos = torch.arange(tokens.shape[1], device=tokens.device)
        x = self.wte(tokens) + self.wpe(pos)
        for blk in self.blocks:
            x = blk(x)
        logits = self.lm_head(self.ln_f(x))
        if logits.shape[-1] != self.vocab_size:
            logits = logits + self.vocab_mask.to(logits.dtype)
        return logits

    def ignore_for_kfac(self):
        """Modules that K-FAC leaves to the plain gradient on this model."""
        return [self.wte, self.wpe, self.lm_head, nn.LayerNorm]


def next_token_loss(logits, tokens, reduction='mean'):
    """Cross-entropy of predicting token t+1 from position t (per predicted token)."""
    return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), tokens[:, 1:].reshape(-1),
                           reduction=reduction)


def gpt2_medium():
    return GPT2(50257, 1024, 24, 16, 1024)


def gpt2_tiny(vocab_size=97, n_positions=16):
    """Two-block GPT-2 for tests."""
    return GPT2(vocab_size, n_positions, 2, 2, 32)
