"""Fused AdamW arena vs torch.optim.AdamW on fp32 copies."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fused_adamw_matches_torch():
    from aicomp_b200 import FusedAdamW
    torch.manual_seed(0)
    shapes = [(256, 128), (1000,), (64, 64, 3), (8,)]
    params = [torch.nn.Parameter((torch.randn(s, device="cuda") * 0.1).bfloat16()) for s in shapes]
    ref = [torch.nn.Parameter(p.detach().float().clone()) for p in params]
    opt = FusedAdamW(params, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, grad_scale=0.5)
    ropt = torch.optim.AdamW(ref, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for step in range(5):
        opt.zero_grad()
        ropt.zero_grad()
        for p, r in zip(params, ref):
            g = torch.randn(p.shape, device="cuda")
            if step % 2 == 0:
                p.main_grad.add_(g)            # fused wgrad path writes the arena directly
                p.grad_accumulated = True
            else:
                p.grad = g.bfloat16()          # autograd path leaves .grad
                g = p.grad.float()
            r.grad = g * 0.5
        opt.step()
        ropt.step()
        assert float(opt.grad.abs().max()) == 0.0  # the update cleared the gradient arena
    for p, r, mo in zip(params, ref, opt.offsets):
        master = opt.master[mo:mo + p.numel()].view(p.shape)
        assert torch.allclose(master, r.detach(), rtol=2e-3, atol=2e-3)
        assert torch.allclose(p.detach().float(), master, rtol=1e-2, atol=1e-2)


def test_grad_clipping_uses_global_norm():
    from aicomp_b200 import FusedAdamW
    torch.manual_seed(0)
    p = torch.nn.Parameter(torch.zeros(4096, device="cuda", dtype=torch.bfloat16))
    opt = FusedAdamW([p], lr=1.0, betas=(0.0, 0.0), eps=1e-12, weight_decay=0.0, max_grad_norm=1.0)
    p.main_grad.fill_(10.0)
    p.grad_accumulated = True
    n = opt.grad_norm()
    assert abs(n.item() - 640.0) < 1e-2
    opt.step()  # with beta=0 the update is -lr * sign(g): clipping must not change the sign, only scale g
    assert torch.allclose(opt.master, torch.full_like(opt.master, -1.0), atol=1e-3)
