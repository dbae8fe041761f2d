"""Analytic FLOP and memory model of one training step per method, from the library's counters.

    python benchmarks/flops_memory.py --model resnet50 --batch-size 32
    python benchmarks/flops_memory.py --model vit_b_16 --batch-size 64 --seq-len 197
    python benchmarks/flops_memory.py --model gpt2_medium --batch-size 8 --seq-len 1024

Prints one row per phase (forward, backward, and statistics / inverse / preconditioning of K-FAC,
Shampoo, SMW-NG, Adam, L-BFGS): GFLOP, million stored numbers, and the roofline time on a B200.
Runs on CPU (convolution sizes are learnt from one forward pass of batch 1 on the meta-sized
input).  Role of the reference's examples/prof/flops_memory.py.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from asdl_b200 import counter as C  # noqa: E402
from asdl_b200.models import resnet50, vit_b_16, gpt2_medium, resnet_tiny  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='resnet50', choices=['resnet50', 'resnet_tiny', 'vit_b_16', 'gpt2_medium'])
    ap.add_argument('--batch-size', type=int, default=32)
    ap.add_argument('--seq-len', type=int, default=128)
    ap.add_argument('--json', default=None, help='also write {phase: {flop, numel, roofline_ms}} to this file')
    args = ap.parse_args()
    if args.model == 'resnet50':
        model, x = resnet50(), torch.randn(1, 3, 224, 224)
    elif args.model == 'resnet_tiny':
        model, x = resnet_tiny(), torch.randn(1, 3, 32, 32)
    elif args.model == 'vit_b_16':
        model, x = vit_b_16(), torch.randn(1, 3, 224, 224)
    else:
        model, x = gpt2_medium(), torch.randint(0, 50257, (1, min(args.seq_len, 1024)))
    rows = args.batch_size * (args.seq_len if args.model in ('vit_b_16', 'gpt2_medium') else 1)
    counters = [C.Forward(), C.BackwardWeight(), C.BackwardInput(), C.AdamStats(), C.AdamPrecond(),
                C.KFACStats(), C.KFACInv(), C.KFACPrecond(), C.ShampooStats(), C.ShampooInv(),
                C.ShampooPrecond(), C.LBFGSPrecond(), C.SMWNGStats(), C.SMWNGPrecond()]
    model.eval()
    with C.set_counter(model, counters, batch_size=rows, seq_len=args.seq_len) as counts, torch.no_grad():
        model(x)
    print(f'{args.model}: {counts["params"] / 1e6:.1f} M parameters in Linear / Conv2d / attention layers, '
          f'{rows} rows per step')
    print(f'{"phase":<16}{"GFLOP":>12}{"M numbers":>12}{"roofline ms":>14}')
    for c in counters:
        name = type(c).__name__
        flop, numel = counts[name]['flop'], counts[name]['numel']
        print(f'{name:<16}{flop / 1e9:>12.2f}{numel / 1e6:>12.2f}{C.roofline_ms(flop, 4 * numel):>14.4f}')
    if args.json:
        import json
        with open(args.json, 'w') as f:
            json.dump({'model': args.model, 'rows': rows,
                       'phases': {type(c).__name__: {'flop': counts[type(c).__name__]['flop'],
                                                     'numel': counts[type(c).__name__]['numel'],
                                                     'roofline_ms': C.roofline_ms(counts[type(c).__name__]['flop'],
                                                                                  4 * counts[type(c).__name__]['numel'])}
                                  for c in counters}}, f, indent=1)


if __name__ == '__main__':
    main()
