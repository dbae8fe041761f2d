"""Training-step benchmarks of the transformer configurations (synthetic data, random init).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29544 benchmarks/train_step.py --model vit_b_16 --steps 20 --warmup 3
    ... --model gpt2_medium            (K-FAC on the block Linears, embeddings/LayerNorm/head ignored)
    ... --impl reference               (the reference package from baseline/_ref; on stock model definitions:
                                        torchvision's vit_b_16, a plain nn.Linear GPT-2 with the 50257-row
                                        vocabulary; --ref-model ours runs it on this library's definitions)

vit_b_16     ViT-B/16, per-GPU batch 64 of N(0,1) images, Shampoo with block size 1024, inverse 4th
             roots in fp32 every 20 steps, epsilon 1e-6, bf16 autocast.
gpt2_medium  GPT-2 medium, per-GPU batch 8 x 1024 uniform token ids, next-token loss, K-FAC
             (damping 1e-3, curvature every 10 steps, inverses every 100 steps, EMA 0.05), bf16
             autocast, fp32 factors, inverses sharded layer-wise over the ranks.

Rank 0 prints one JSON line: device-timed (CUDA events, max over ranks) milliseconds per step over
exactly ``--steps`` steps after ``--warmup`` untimed ones, optimizer step included, L2 flushed
before every step.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class _PlainGPT2(torch.nn.Module):
    """GPT-2 as a stock PyTorch model for the reference arm: nn.Embedding, nn.LayerNorm, nn.Linear and
    scaled_dot_product_attention, the 50257-row vocabulary unpadded, output matrix tied to the embedding."""

    class Block(torch.nn.Module):
        def __init__(self, d, heads):
            super().__init__()
            nn = torch.nn
            self.heads = heads
            self.ln_1, self.ln_2 = nn.LayerNorm(d), nn.LayerNorm(d)
            self.attn_qkv, self.attn_proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
            self.mlp_fc, self.mlp_proj = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)

        def forward(self, x):
            b, s, d = x.shape
            q, k, v = self.attn_qkv(self.ln_1(x)).view(b, s, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(b, s, d)
            x = x + self.attn_proj(a)
            return x + self.mlp_proj(F.gelu(self.mlp_fc(self.ln_2(x)), approximate='tanh'))

    def __init__(self, vocab=50257, seq=1024, layers=24, d=1024, heads=16):
        super().__init__()
        nn = torch.nn
        self.wte, self.wpe = nn.Embedding(vocab, d), nn.Embedding(seq, d)
        self.blocks = nn.ModuleList([self.Block(d, heads) for _ in range(layers)])
        self.ln_f = nn.LayerNorm(d)
        self.lm_head = nn.Linear(d, vocab, bias=False)
        self.lm_head.weight = self.wte.weight

    def forward(self, idx):
        x = self.wte(idx) + self.wpe(torch.arange(idx.shape[1], device=idx.device))
        for blk in self.blocks:
            x = blk(x)
        return self.lm_head(self.ln_f(x))

    def ignore_for_kfac(self):
        return [torch.nn.Embedding, torch.nn.LayerNorm, self.lm_head]


def _plain_next_token_loss(logits, tokens, reduction='mean'):
    return F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), tokens[:, 1:].reshape(-1),
                           reduction=reduction)


def build(args, dev, world):
    from asdl_b200.models import vit_b_16, gpt2_medium, vit_tiny, gpt2_tiny, next_token_loss
    if args.impl == 'reference':
        sys.path.insert(0, os.path.join(ROOT, 'baseline', '_ref'))
        import asdl
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
    else:
        import asdl_b200 as asdl
    torch.manual_seed(0)
    g = torch.Generator().manual_seed(1 + int(os.environ.get('RANK', '0')))
    if args.model.startswith('vit'):
        tiny = args.model == 'vit_tiny'
        stock = args.impl == 'reference' and args.ref_model == 'stock' and not tiny
        if stock:
            import torchvision
            model = torchvision.models.vit_b_16(num_classes=1000).to(dev)
        else:
            model = (vit_tiny(10, 32) if tiny else vit_b_16()).to(dev)
        bs = args.batch or 64
        x = torch.randn(bs, 3, *((32, 32) if tiny else (224, 224)), generator=g).to(dev)
        t = torch.randint(0, 10 if tiny else 1000, (bs,), generator=g).to(dev)
        cfg = asdl.PreconditioningConfig(damping=1e-6, preconditioner_upd_interval=20)
        if args.impl == 'reference':
            gm = asdl.ShampooGradientMaker(model, cfg)  # the reference ignores its block_size argument
        else:
            gm = asdl.ShampooGradientMaker(model, cfg, block_size=1024)
        loss_fn, autocast = F.cross_entropy, args.impl != 'reference' or args.ref_autocast
        desc = dict(model=args.model, per_gpu_batch=bs, optimizer='shampoo', block_size=1024,
                    preconditioner_upd_interval=20, epsilon=1e-6)
    else:
        tiny = args.model == 'gpt2_tiny'
        stock = args.impl == 'reference' and args.ref_model == 'stock' and not tiny
        model = (_PlainGPT2() if stock else (gpt2_tiny() if tiny else gpt2_medium())).to(dev)
        bs, seq, vocab = args.batch or 8, (16 if tiny else 1024), (97 if tiny else 50257)
        x = torch.randint(0, vocab, (bs, seq), generator=g).to(dev)
        t = x
        cfg = asdl.PreconditioningConfig(data_size=bs, damping=1e-3, ema_decay=0.05,
                                         curvature_upd_interval=10, preconditioner_upd_interval=100,
                                         ignore_modules=model.ignore_for_kfac())
        if args.impl == 'reference':
            gm = asdl.KfacGradientMaker(model, cfg)
        else:
            gm = asdl.FusedKfacGradientMaker(model, cfg, cuda_graph=not args.no_graph)
        loss_fn, autocast = (_plain_next_token_loss if stock else next_token_loss), args.impl != 'reference' or args.ref_autocast
        desc = dict(model=args.model, per_gpu_batch=bs, seq_len=seq, optimizer='kfac', damping=1e-3,
                    curvature_upd_interval=10, preconditioner_upd_interval=100, ema_decay=0.05)
    opt = torch.optim.SGD(model.parameters(), lr=1e-4, momentum=0.9)

    def model_fn(inp):
        with torch.autocast('cuda', dtype=torch.bfloat16, enabled=autocast):
            return model(inp)

    def step():
        opt.zero_grad(set_to_none=False)
        d = gm.setup_model_call(model_fn, x)
        gm.setup_loss_call(loss_fn, d, t)
        _, loss = gm.forward_and_backward()
        opt.step()
        return loss

    desc['dtype'] = 'bf16 autocast' if autocast else 'fp32 (tf32)'
    if args.impl == 'reference':
        desc['model_definition'] = 'stock (torchvision / plain nn.Linear GPT-2)' if stock else "this library's"
    return step, desc


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--model', default='vit_b_16', choices=['vit_b_16', 'gpt2_medium', 'vit_tiny', 'gpt2_tiny'])
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--batch', type=int, default=None)
    ap.add_argument('--no-graph', action='store_true')
    ap.add_argument('--ref-model', default='stock', choices=['stock', 'ours'],
                    help="model definition of the reference arm: stock PyTorch models or this library's")
    ap.add_argument('--ref-autocast', action='store_true',
                    help='run the reference arm under bf16 autocast too (its factor products then run in bf16)')
    args = ap.parse_args()
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    world = int(os.environ.get('WORLD_SIZE', '1'))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)
    if world > 1:
        dist.init_process_group('nccl', device_id=dev)
    step, desc = build(args, dev, world)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        flush.zero_()
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({'case': 'train_step', 'impl': args.impl, 'n_gpus': world, 'steps': args.steps,
                          'warmup': args.warmup, 'ms_per_step': round(ms.item() / args.steps, 3),
                          'last_loss': float(loss), 'peak_mem_gb': round(torch.cuda.max_memory_allocated() / 2**30, 2),
                          'config': desc}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
