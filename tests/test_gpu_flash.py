"""tcgen05 flash attention forward vs an fp32 PyTorch reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,S", [(1, 128), (2, 256), (1, 1000), (1, 2048), (3, 77), (1, 4096)])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (4, 4)])
def test_flash_fwd_matches_reference(B, S, hq, hkv):
    from aicomp_b200 import ops
    from aicomp_b200.ops import flash
    from aicomp_b200.ops.attention import attention_reference
    torch.manual_seed(0)
    D = 128
    qkv = torch.randn(B * S, (hq + 2 * hkv) * D, device="cuda", dtype=torch.bfloat16)
    out, lse = flash.flash_fwd(qkv, B, S, hq, hkv, D, need_lse=True)
    torch.cuda.synchronize()
    ops.check_errors()
    q = qkv[:, : hq * D].view(B, S, hq, D).transpose(1, 2)
    k = qkv[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D).transpose(1, 2)
    v = qkv[:, (hq + hkv) * D:].view(B, S, hkv, D).transpose(1, 2)
    ref = attention_reference(q.float(), k.float(), v.float(), causal=True).transpose(1, 2).reshape(B * S, hq * D)
    err = (out.float() - ref).abs().max().item()
    assert err < 3e-2, err
    # log-sum-exp
    g = hq // hkv
    s = torch.einsum("bhgqd,bhkd->bhgqk", q.float().view(B, hkv, g, S, D), k.float()) / D ** 0.5
    mask = torch.ones(S, S, dtype=torch.bool, device="cuda").tril()
    ref_lse = torch.logsumexp(s.masked_fill(~mask, float("-inf")), -1).reshape(B, hq, S)
    assert (lse - ref_lse).abs().max().item() < 2e-2


def test_flash_used_for_inference_attention():
    from aicomp_b200.ops import attention, flash
    qkv = torch.randn(256, (4 + 2 * 2) * 128, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        assert flash.supported(qkv, 128)
        o = attention.causal_attention_packed(qkv, 1, 256, 4, 2, 128)
    assert o.shape == (256, 512)


@pytest.mark.parametrize("B,S", [(1, 128), (2, 256), (1, 1000), (1, 2048), (3, 77)])
@pytest.mark.parametrize("hq,hkv", [(8, 2), (4, 4)])
def test_flash_bwd_matches_reference(B, S, hq, hkv):
    """dQ, dK, dV of the tcgen05 backward kernel (packed layout) vs autograd through an fp32 reference."""
    from aicomp_b200 import ops
    from aicomp_b200.ops import flash
    from aicomp_b200.ops.attention import attention_reference
    torch.manual_seed(1)
    D = 128
    qkv = torch.randn(B * S, (hq + 2 * hkv) * D, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn(B * S, hq * D, device="cuda", dtype=torch.bfloat16)
    x = qkv.clone().requires_grad_(True)
    out = flash.flash_attention_packed(x, B, S, hq, hkv, D)
    out.backward(dout)
    torch.cuda.synchronize()
    ops.check_errors()
    ref_in = qkv.float().requires_grad_(True)
    q = ref_in[:, : hq * D].view(B, S, hq, D).transpose(1, 2)
    k = ref_in[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D).transpose(1, 2)
    v = ref_in[:, (hq + hkv) * D:].view(B, S, hkv, D).transpose(1, 2)
    ref = attention_reference(q, k, v, causal=True).transpose(1, 2).reshape(B * S, hq * D)
    ref.backward(dout.float())
    got, want = x.grad.float(), ref_in.grad
    for name, lo, hi in (("dq", 0, hq * D), ("dk", hq * D, (hq + hkv) * D), ("dv", (hq + hkv) * D, (hq + 2 * hkv) * D)):
        g, w = got[:, lo:hi], want[:, lo:hi]
        rel = ((g - w).norm() / w.norm()).item()
        assert rel < 2e-2, (name, rel)
        assert (g - w).abs().max().item() < 0.05 * w.abs().max().item() + 1e-2, name


def test_training_attention_runs_the_kernels():
    from aicomp_b200 import ops
    from aicomp_b200.ops import attention
    qkv = torch.randn(256, (4 + 2 * 2) * 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    before = ops.launch_count()
    o = attention.causal_attention_packed(qkv, 1, 256, 4, 2, 128)
    o.sum().backward()
    assert ops.launch_count() - before >= 4  # forward + (delta, backward, rounding)
    assert qkv.grad is not None and torch.isfinite(qkv.grad).all()
