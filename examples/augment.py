"""Image augmentations that run on whole batches on the training device.

The reference augments sample by sample in data-loader workers (random crop + flip, the CIFAR-10
AutoAugment policy, Cutout: examples/arxiv_results/train.py:247-264, utils/cutout.py,
utils/autoaugment.py).  Here the batch is augmented after it reached the GPU: one indexing
kernel for crop + flip and one masking kernel for Cutout, no per-sample Python work; the AutoAugment
policy, where wanted, is torchvision's and stays in the loader.
"""
import torch

__all__ = ['batch_random_crop_flip', 'batch_cutout', 'Cutout']


def batch_random_crop_flip(x: torch.Tensor, padding: int = 4, flip: bool = True, generator=None) -> torch.Tensor:
    """Every image of ``x`` (n, c, h, w) is shifted by its own offset in ``[-padding, padding]`` per axis
    (zeros move in, as a crop of the zero-padded image does) and mirrored with probability 1/2."""
    n, _, h, w = x.shape
    dev = x.device
    dy = torch.randint(-padding, padding + 1, (n, 1, 1), device=dev, generator=generator)
    dx = torch.randint(-padding, padding + 1, (n, 1, 1), device=dev, generator=generator)
    rows = torch.arange(h, device=dev).view(1, h, 1) + dy
    cols = torch.arange(w, device=dev).view(1, 1, w)
    if flip:
        mirrored = torch.rand(n, 1, 1, device=dev, generator=generator) < 0.5
        cols = torch.where(mirrored, w - 1 - cols, cols)
    cols = cols + dx
    inside = ((rows >= 0) & (rows < h) & (cols >= 0) & (cols < w)).unsqueeze(1)
    rows, cols = rows.clamp(0, h - 1).expand(n, h, w), cols.clamp(0, w - 1).expand(n, h, w)
    batch = torch.arange(n, device=dev).view(n, 1, 1).expand(n, h, w)
    out = x.permute(0, 2, 3, 1)[batch, rows, cols].permute(0, 3, 1, 2)
    return out * inside


def batch_cutout(x: torch.Tensor, n_holes: int = 1, length: int = 16, generator=None) -> torch.Tensor:
    """Zeroes ``n_holes`` squares of side ``length`` per image; centres are uniform over the image, so
    squares are clipped at the border."""
    n, _, h, w = x.shape
    dev = x.device
    rows = torch.arange(h, device=dev).view(1, h, 1)
    cols = torch.arange(w, device=dev).view(1, 1, w)
    keep = torch.ones(n, h, w, dtype=torch.bool, device=dev)
    for _ in range(n_holes):
        cy = torch.randint(0, h, (n, 1, 1), device=dev, generator=generator)
        cx = torch.randint(0, w, (n, 1, 1), device=dev, generator=generator)
        hole = ((rows >= cy - length // 2) & (rows < cy + length // 2)
                & (cols >= cx - length // 2) & (cols < cx + length // 2))
        keep &= ~hole
    return x * keep.unsqueeze(1)


class Cutout:
    """Per-sample form of :func:`batch_cutout` for a transform pipeline (input: c x h x w tensor)."""

    def __init__(self, n_holes=1, length=16):
        self.n_holes, self.length = n_holes, length

    def __call__(self, img: torch.Tensor) -> torch.Tensor:
        return batch_cutout(img.unsqueeze(0), self.n_holes, self.length)[0]
