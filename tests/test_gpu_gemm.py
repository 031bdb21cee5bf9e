"""tcgen05 GEMM vs an fp32 PyTorch reference, all operand layouts and epilogues."""
import pytest
import torch

from aicomp_b200 import ops

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    af = (a.t() if a_mn else a).float()
    bf = (b.t() if b_mn else b).float()
    return af @ bf.t()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 1024, 512), (200, 264, 136), (2048, 4096, 1024)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_layouts(a_mn, b_mn, M, N, K, bn):
    torch.manual_seed(0)
    dev = "cuda"
    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a row pitch that is a multiple of 8")
    a = torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16)
    c = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, bn=bn)
    torch.cuda.synchronize()
    ops.check_errors()
    ref = _ref(a, b, a_mn, b_mn)
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max err {err} (scale {scale})"


def test_gemm_fp32_accumulate_and_bias():
    torch.manual_seed(1)
    M, N, K = 512, 768, 320
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    acc0 = acc.clone()
    ops.gemm(a, b, out=acc, accumulate=True)
    ops.gemm(a, b, out=acc, accumulate=True)
    torch.cuda.synchronize()
    ref = acc0 + 2 * (a.float() @ b.float().t())
    assert torch.allclose(acc, ref, rtol=1e-3, atol=1e-2)
    c = ops.gemm(a, b, bias=bias, alpha=0.5)
    ref2 = 0.5 * (a.float() @ b.float().t()) + bias.float()
    assert (c.float() - ref2).abs().max().item() <= 1e-2 * ref2.abs().max().item()
    ops.check_errors()


def test_linear_autograd_matches_torch():
    torch.manual_seed(2)
    x = torch.randn(4, 96, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()
    bias = torch.randn(512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w, bias)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, bias))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    for got, ref in ((y, yr), (x.grad, xr.grad), (w.grad, wr.grad), (bias.grad, br.grad)):
        assert (got.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item() + 1e-3
    ops.check_errors()


def test_wgrad_accumulates_into_main_grad():
    torch.manual_seed(3)
    x = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    w = torch.nn.Parameter(torch.randn(384, 128, device="cuda", dtype=torch.bfloat16) * 0.05)
    w.main_grad = torch.zeros(384, 128, device="cuda", dtype=torch.float32)
    for _ in range(2):
        y = ops.linear(x, w)
        y.backward(torch.ones_like(y))
    assert w.grad is None
    ref = 2 * (torch.ones(256, 384, device="cuda").t() @ x.float())
    assert torch.allclose(w.main_grad, ref, rtol=1e-3, atol=1e-2)
    ops.check_errors()


@pytest.mark.parametrize("M,N,K", [(8, 4096, 4096), (64, 6144, 4096), (100, 4096, 14336), (256, 1024, 512)])
def test_small_m_linear_split_k(M, N, K):
    torch.manual_seed(4)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02
    b = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        y = ops.linear(x, w, b)
    ref = x.float() @ w.float().t() + b.float()
    assert (y.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-2
    acc = torch.zeros(M, N, device="cuda")
    ops.gemm(x, w, out=acc, accumulate=True, ksplit=7, bn=128)
    assert torch.allclose(acc, x.float() @ w.float().t(), rtol=1e-3, atol=2e-2)
    ops.check_errors()


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("M,N,K", [(512, 256, 64), (512, 512, 448), (2048, 6144, 4096), (4096, 4096, 2048), (1000, 520, 264),
                                   (640, 1032, 128)])
def test_pair_gemm_layouts(a_mn, b_mn, M, N, K):
    """CTA-pair kernel (cta_group::2, 256 x 256 tiles, each CTA stages half of B) vs fp32 PyTorch."""
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
    c = ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair=True)
    torch.cuda.synchronize()
    ops.check_errors()
    ref = _ref(a, b, a_mn, b_mn)
    err = (c.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 1e-2 * scale + 1e-2, f"max err {err} (scale {scale})"


def test_pair_gemm_fp32_accumulate_bias_and_repeat():
    torch.manual_seed(1)
    M, N, K = 1024, 768, 320
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
    acc = torch.randn(M, N, device="cuda", dtype=torch.float32)
    acc0 = acc.clone()
    for _ in range(3):
        ops.gemm(a, b, out=acc, accumulate=True, pair=True)
    torch.cuda.synchronize()
    ref = acc0 + 3 * (a.float() @ b.float().t())
    assert torch.allclose(acc, ref, rtol=1e-3, atol=2e-2)
    c = ops.gemm(a, b, bias=bias, alpha=0.5, pair=True)
    ref2 = 0.5 * (a.float() @ b.float().t()) + bias.float()
    assert (c.float() - ref2).abs().max().item() <= 1e-2 * ref2.abs().max().item()
    # many tiles per pair: exercises the ring wrap-around and both accumulator buffers
    a2 = torch.randn(8192, 512, device="cuda", dtype=torch.bfloat16)
    b2 = torch.randn(8192, 512, device="cuda", dtype=torch.bfloat16)
    c2 = ops.gemm(a2, b2, pair=True)
    ref3 = a2.float() @ b2.float().t()
    assert (c2.float() - ref3).abs().max().item() <= 1e-2 * ref3.abs().max().item()
    ops.check_errors()
