"""The benchmark model families step through their makers (tiny versions, CPU)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

import asdl_b200 as asdl
from asdl_b200.models import vit_tiny, gpt2_tiny, next_token_loss, resnet_tiny


def _steps(gm, model, x, loss_fn, t, n=3, lr=0.01):
    opt = torch.optim.SGD(model.parameters(), lr=lr)
    losses = []
    for _ in range(n):
        opt.zero_grad()
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(loss_fn, d, t)
        _, loss = gm.forward_and_backward()
        assert all(torch.isfinite(p.grad).all() for p in model.parameters() if p.grad is not None)
        opt.step()
        losses.append(loss.item())
    return losses


def test_vit_shampoo_blocks_every_matrix():
    torch.manual_seed(0)
    model = vit_tiny()
    x, t = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    cfg = asdl.PreconditioningConfig(damping=1e-6, preconditioner_upd_interval=2)
    gm = asdl.ShampooGradientMaker(model, cfg, block_size=16)
    losses = _steps(gm, model, x, F.cross_entropy, t, n=4, lr=1e-3)
    assert losses[-1] < losses[0]
    shapes = {tuple(p.shape) for p in model.parameters() if p.ndim > 1}
    assert (96, 32) in shapes and (32, 3, 8, 8) in shapes and (1, 17, 32) in shapes
    assert len(gm.preconditioners) == len([p for p in model.parameters() if p.ndim > 1])


def test_vit_kfac_sees_attention_projections():
    torch.manual_seed(0)
    model = vit_tiny()
    x, t = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    cfg = asdl.PreconditioningConfig(data_size=4, damping=1e-2)
    gm = asdl.FusedKfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP)
    _steps(gm, model, x, F.cross_entropy, t)
    assert model.layers[0].attn.qkv.fisher.kron.A.shape == (32, 32)
    assert model.layers[0].attn.qkv.fisher.kron.B.shape == (96, 96)


def test_gpt2_kfac_on_block_linears_only():
    torch.manual_seed(0)
    model = gpt2_tiny()
    tokens = torch.randint(0, 97, (2, 16))
    cfg = asdl.PreconditioningConfig(data_size=2, damping=1e-3, ignore_modules=model.ignore_for_kfac())
    gm = asdl.FusedKfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP)
    losses = _steps(gm, model, tokens, next_token_loss, tokens, n=3)
    assert losses[-1] < losses[0] + 1e-3
    assert len(gm._kron) == 2 * 4 and not gm._norm
    assert not hasattr(model.lm_head, 'fisher') and not hasattr(model.wte, 'fisher')
    assert model.blocks[1].proj.fisher.kron.A.shape == (128, 128)


def test_resnet_tiny_kfac_reference_maker():
    torch.manual_seed(0)
    model = resnet_tiny()
    x, t = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    cfg = asdl.PreconditioningConfig(data_size=4, damping=1e-2)
    gm = asdl.KfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP)
    _steps(gm, model, x, F.cross_entropy, t, n=2)


def test_fused_resnet_blocks_match_unfused_ones():
    """ReLUs and residual adds folded into the normalisation layers: same loss, same gradients and
    the same K-FAC preconditioned gradients as the model with separate layers."""
    import copy
    torch.manual_seed(0)
    plain = resnet_tiny(fused=False)
    fused = resnet_tiny(fused=True)
    fused.load_state_dict(copy.deepcopy(plain.state_dict()))
    x, t = torch.randn(6, 3, 32, 32), torch.randint(0, 10, (6,))
    results = []
    for model in (plain, fused):
        cfg = asdl.PreconditioningConfig(data_size=6, damping=1e-2)
        gm = asdl.FusedKfacGradientMaker(model, cfg, fisher_type=asdl.FISHER_EMP)
        d = gm.setup_model_call(model, x)
        gm.setup_loss_call(F.cross_entropy, d, t)
        _, loss = gm.forward_and_backward()
        results.append((loss.item(), [p.grad.clone() for p in model.parameters()],
                        model.layer1[0].bn3.fisher.unit.data.clone(), model.bn1.running_mean.clone()))
    assert abs(results[0][0] - results[1][0]) < 1e-6
    for a, b in zip(results[0][1], results[1][1]):
        torch.testing.assert_close(a, b, rtol=2e-4, atol=1e-6)
    torch.testing.assert_close(results[0][2], results[1][2], rtol=1e-4, atol=1e-8)
    torch.testing.assert_close(results[0][3], results[1][3])
    generic = asdl.KfacGradientMaker(fused, asdl.PreconditioningConfig(data_size=6, damping=1e-2),
                                     fisher_type=asdl.FISHER_EMP)
    d = generic.setup_model_call(fused, x)
    generic.setup_loss_call(F.cross_entropy, d, t)
    import pytest
    with pytest.raises(ValueError, match='fuses an activation'):
        generic.forward_and_backward()


def test_grouped_bf16_weight_cast_is_transparent():
    """One grouped cast of all Conv2d / Linear weights gives the same outputs and fp32 gradients
    (in the parameters' own memory format) as autocast's per-layer casts."""
    import copy
    from asdl_b200.models.layers import grouped_bf16_weights
    torch.manual_seed(0)
    a = resnet_tiny(fused=True).to(memory_format=torch.channels_last)
    b = copy.deepcopy(a)
    x = torch.randn(2, 3, 32, 32)
    with torch.autocast('cpu', dtype=torch.bfloat16):
        with grouped_bf16_weights(a):
            assert a.conv1.weight.dtype == torch.bfloat16 and a.conv1.weight.stride() == b.conv1.weight.stride()
            ya = a._forward(x)
        yb = b._forward(x)
    assert a.conv1.weight.dtype == torch.float32          # restored
    torch.testing.assert_close(ya, yb)
    ya.float().sum().backward()
    yb.float().sum().backward()
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert pa.grad.dtype == torch.float32 and pa.grad.stride() == pb.grad.stride()
        torch.testing.assert_close(pa.grad, pb.grad, rtol=2e-2, atol=1e-3 * pb.grad.abs().max().item())


def test_wideresnet_and_mixer_step_through_their_makers():
    from asdl_b200.models import wideresnet_tiny, mixer_tiny
    torch.manual_seed(0)
    x, t = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    wrn = wideresnet_tiny()
    cfg = asdl.PreconditioningConfig(data_size=4, damping=1e-2)
    _steps(asdl.FusedKfacGradientMaker(wrn, cfg, fisher_type=asdl.FISHER_EMP), wrn, x, F.cross_entropy, t, n=2)
    assert wrn.blocks[1].shortcut.fisher.kron.B.shape == (32, 32)
    mixer = mixer_tiny()
    _steps(asdl.KfacGradientMaker(mixer, cfg, fisher_type=asdl.FISHER_EMP), mixer, x, F.cross_entropy, t, n=2)
    assert mixer.blocks[0].token_fc1.fisher.kron.A_inv.shape == (16, 16)    # 16 patches of 8 x 8
    shampoo = asdl.ShampooGradientMaker(mixer, asdl.PreconditioningConfig(damping=1e-6), block_size=16)
    _steps(shampoo, mixer, x, F.cross_entropy, t, n=2, lr=1e-3)


def test_fused_layer_norm_is_layer_norm_on_cpu():
    from asdl_b200.models.layers import FusedLayerNorm
    torch.manual_seed(0)
    a, b = FusedLayerNorm(48), nn.LayerNorm(48)
    b.load_state_dict(a.state_dict())
    x = torch.randn(3, 7, 48)
    torch.testing.assert_close(a(x), b(x))
    assert isinstance(a, nn.LayerNorm)


def test_cifar_family_steps_through_its_makers():
    from asdl_b200.models import MLP, SmallCNN, resnet18, resnet34, vit_tiny_patch16_224
    torch.manual_seed(0)
    x, t = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    cfg = asdl.PreconditioningConfig(data_size=4, damping=1e-2)
    plain, fused = resnet18(width=8), resnet18(width=8, fused=True)
    fused.load_state_dict(plain.state_dict())
    torch.testing.assert_close(plain(x), fused(x))
    _steps(asdl.KfacGradientMaker(plain, cfg, fisher_type=asdl.FISHER_EMP), plain, x, F.cross_entropy, t, n=2)
    _steps(asdl.FusedKfacGradientMaker(fused, cfg, fisher_type=asdl.FISHER_EMP), fused, x, F.cross_entropy, t, n=2)
    assert plain.blocks[2].downsample[0].fisher.kron.A_inv.shape == (8, 8)         # 1 x 1 convolution, 8 -> 16 channels
    assert len(resnet34(width=8).blocks) == 16
    mlp = MLP(width=16, depth=4, in_features=3 * 32 * 32)
    assert sum(isinstance(m, nn.Linear) for m in mlp.modules()) == 4
    _steps(asdl.KronPsgdGradientMaker(mlp, asdl.PreconditioningConfig()), mlp, x, F.cross_entropy, t, n=2)
    cnn = SmallCNN(in_channels=3, image_size=32)
    _steps(asdl.SengGradientMaker(cnn, asdl.PreconditioningConfig(data_size=4, damping=1e-1), sketching_size=3,
                                  truncated_rank=2), cnn, x, F.cross_entropy, t, n=2)
    vit = vit_tiny_patch16_224()
    assert len(vit.layers) == 12 and vit.head.in_features == 192 and vit.layers[0].attn.heads == 3
