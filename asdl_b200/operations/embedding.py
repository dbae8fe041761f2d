"""Statistics of ``nn.Embedding``.

``a`` is the integer index tensor n x *, ``g`` is n x * x d.  The A factor of the one-hot input is
counts^T counts (V x V, only sensible for small vocabularies); per-example gradients and the
diagonal are built with scatter-adds (one fused ``index_add_`` instead of a Python loop over
tokens).  Parity: asdl/operations/embedding.py:7-78.
"""
import torch
from torch import nn

from .. import ops
from .operation import (Operation, BASIC_OPS, OP_COV_KRON, OP_COV_KRON_INV, OP_BATCH_GRADS, OP_COV_DIAG,
                        OP_COV_DIAG_INV, SHAPE_DIAG)

__all__ = ['Embedding']


class Embedding(Operation):
    """Statistics of ``nn.Embedding``.  in_data: token ids (any shape, flattened), out_grads: tokens x dim.
    The input-side Kronecker factor is ``counts^T counts`` of the per-example token-count vectors
    (vocabulary x vocabulary, so only for small vocabularies; larger ones use the diagonal shape or are
    ignored); counts, per-example gradients and the diagonal are scatter-adds over tokens.  Reference:
    asdl/operations/embedding.py:7-78 (``bincount`` per example and Python loops over tokens).
    """
    # the reference leaves out the fused "statistic + inverse" op, so K-FAC without a moving average
    # (which inverts inside the hooks) finds no curvature for an embedding and raises
    supported_operations = set(BASIC_OPS + [OP_COV_KRON, OP_COV_KRON_INV, OP_BATCH_GRADS, SHAPE_DIAG, OP_COV_DIAG,
                                            OP_COV_DIAG_INV])

    @classmethod
    def batch_grads_weight(cls, module, in_data, out_grads):
        """tokens x num_embeddings x embedding_dim (dense; intended for small vocabularies).  Every token
        is a row of its own, the convention of every layer for inputs with extra leading dimensions
        (a Linear layer after the embedding flattens n x sequence x features to (n sequence) x features),
        so the rows of all layers of a token-level model line up."""
        idx = in_data.reshape(-1).long()
        g = out_grads.reshape(idx.shape[0], -1)
        rows = idx.shape[0]
        out = g.new_zeros(rows * module.num_embeddings, module.embedding_dim)
        out.index_add_(0, idx + torch.arange(rows, device=idx.device) * module.num_embeddings, g)
        out = out.view(rows, module.num_embeddings, module.embedding_dim)
        if module.padding_idx is not None:
            out[:, module.padding_idx].zero_()
        return out

    @staticmethod
    def cov_kron_A(module, in_data):
        n = in_data.shape[0]
        idx = in_data.reshape(n, -1).long()
        counts = torch.zeros(n, module.num_embeddings, device=idx.device, dtype=torch.float32)
        if idx.is_cuda and ops.cuda_kernels_enabled(counts):
            ops.extension().embedding_counts(idx.contiguous(), counts)    # reductions, one thread per token
            return ops.gram(counts.to(module.weight.device))              # V x V on the tensor cores
        counts.scatter_add_(1, idx, torch.ones_like(idx, dtype=torch.float32))
        counts = counts.to(module.weight.device)
        return counts.T @ counts  # V x V

    @staticmethod
    def cov_kron_B(module, out_grads):
        return ops.gram(out_grads.reshape(-1, out_grads.shape[-1]))

    @staticmethod
    def cov_diag_weight(module, in_data, out_grads):
        """Sum over tokens of the squared output-gradient, scattered to the looked-up rows
        (every token counts as its own example, as in the reference)."""
        idx = in_data.reshape(-1).long()
        if (idx.is_cuda and ops.cuda_kernels_enabled(out_grads) and module.weight.dtype == torch.float32
                and out_grads.dtype in (torch.float32, torch.bfloat16)):
            cov = torch.zeros_like(module.weight, memory_format=torch.contiguous_format)
            g = out_grads.reshape(idx.shape[0], -1)
            g = g if g.stride(1) == 1 else g.contiguous()
            ops.extension().embedding_diag_stats(idx.contiguous(), g, cov,
                                                 -1 if module.padding_idx is None else int(module.padding_idx), 1.0)
            return cov
        g2 = out_grads.reshape(idx.shape[0], -1).square()
        cov = torch.zeros_like(module.weight)
        cov.index_add_(0, idx, g2.to(cov.dtype))
        if module.padding_idx is not None:
            cov[module.padding_idx].zero_()
        return cov

    @staticmethod
    def in_data_mean(module, in_data):
        return in_data.float().mean(dim=0)

    @staticmethod
    def out_data_mean(module, out_data):
        return out_data.reshape(-1, out_data.shape[-1]).mean(dim=0)

    @staticmethod
    def out_grads_mean(module, out_grads):
        return out_grads.reshape(-1, out_grads.shape[-1]).mean(dim=0)

    @staticmethod
    def out_spatial_size(module, out_data):
        return 1
