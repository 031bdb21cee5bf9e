"""Memory-bound sm_100a kernels vs fp32 PyTorch references."""
import pytest
import torch
import torch.nn.functional as F

from aicomp_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _close(got, ref, rtol=2e-2, atol=2e-2):
    err = (got.float() - ref.float()).abs().max().item()
    lim = rtol * ref.float().abs().max().item() + atol
    assert err <= lim, f"err {err} > {lim}"


@pytest.mark.parametrize("rows,H", [(7, 64), (300, 4096), (33, 8192), (1000, 768)])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm(rows, H, with_res):
    torch.manual_seed(0)
    x = torch.randn(rows, H, device=DEV, dtype=BF, requires_grad=True)
    r = torch.randn(rows, H, device=DEV, dtype=BF, requires_grad=True) if with_res else None
    w = (1 + 0.1 * torch.randn(H, device=DEV, dtype=BF)).requires_grad_()
    y, ro = ops.rmsnorm(x, w, 1e-5, residual=r)
    g = torch.randn_like(y)
    g2 = torch.randn_like(y) if with_res else None
    (y * g).sum().backward() if not with_res else ((y * g).sum() + (ro * g2).sum()).backward()
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    rf = r.detach().float().requires_grad_() if with_res else None
    s = xf + rf if with_res else xf
    yr = s * torch.rsqrt(s.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    ((yr * g.float()).sum() + ((s * g2.float()).sum() if with_res else 0)).backward()
    _close(y, yr)
    _close(x.grad, xf.grad)
    _close(w.grad, wf.grad, rtol=3e-2, atol=0.3)
    if with_res:
        _close(ro, s)
        _close(r.grad, rf.grad)


@pytest.mark.parametrize("rows,H", [(130, 768), (64, 1024)])
def test_layernorm(rows, H):
    torch.manual_seed(0)
    x = torch.randn(rows, H, device=DEV, dtype=BF, requires_grad=True)
    w = (1 + 0.1 * torch.randn(H, device=DEV, dtype=BF)).requires_grad_()
    b = (0.1 * torch.randn(H, device=DEV, dtype=BF)).requires_grad_()
    y, _ = ops.layernorm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf, bf = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = F.layer_norm(xf, (H,), wf, bf, 1e-5)
    yr.backward(g.float())
    _close(y, yr)
    _close(x.grad, xf.grad)
    _close(w.grad, wf.grad, rtol=3e-2, atol=0.3)
    _close(b.grad, bf.grad, rtol=3e-2, atol=0.3)


def test_rope_matches_hf_rotate_half():
    torch.manual_seed(0)
    tokens, hq, hkv, D = 50, 8, 2, 128
    qkv = torch.randn(tokens, (hq + 2 * hkv) * D, device=DEV, dtype=BF)
    pos = torch.randint(0, 4096, (tokens,), device=DEV)
    cos, sin = ops.rope_tables(4096, D, 500000.0, DEV)
    ref = qkv.clone().float()
    c = torch.cat([cos[pos], cos[pos]], -1)[:, None, :]
    s = torch.cat([sin[pos], sin[pos]], -1)[:, None, :]
    qk = ref[:, : (hq + hkv) * D].reshape(tokens, hq + hkv, D)
    rot = torch.cat([-qk[..., D // 2:], qk[..., : D // 2]], -1)
    ref[:, : (hq + hkv) * D] = (qk * c + rot * s).reshape(tokens, -1)
    x = qkv.clone().requires_grad_()
    out = ops.apply_rope_qkv(x * 1.0, pos, cos, sin, hq + hkv, D)
    _close(out, ref)
    g = torch.randn_like(out)
    out.backward(g)
    # rotation is orthogonal: backward of forward output gives the input back
    back = ops.rope_inplace(out.detach().clone(), pos, cos, sin, hq + hkv, D, sign=-1.0)
    _close(back, qkv)
    assert x.grad is not None and x.grad.shape == qkv.shape


def test_swiglu_and_gelu():
    torch.manual_seed(0)
    gu = torch.randn(70, 2 * 256, device=DEV, dtype=BF, requires_grad=True)
    y = ops.swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    guf = gu.detach().float().requires_grad_()
    yr = F.silu(guf[:, :256]) * guf[:, 256:]
    yr.backward(g.float())
    _close(y, yr)
    _close(gu.grad, guf.grad)
    x = torch.randn(33, 3072, device=DEV, dtype=BF, requires_grad=True)
    y = ops.gelu_tanh(x)
    y.backward(g := torch.randn_like(y))
    xf = x.detach().float().requires_grad_()
    yr = F.gelu(xf, approximate="tanh")
    yr.backward(g.float())
    _close(y, yr)
    _close(x.grad, xf.grad)


@pytest.mark.parametrize("rows,V", [(64, 1000), (37, 50264), (16, 128256)])
def test_cross_entropy(rows, V):
    torch.manual_seed(0)
    logits = (torch.randn(rows, V, device=DEV, dtype=BF) * 3).requires_grad_()
    labels = torch.randint(0, V, (rows,), device=DEV)
    labels[::5] = -100
    lf = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(lf, labels, ignore_index=-100)
    ref.backward()
    loss = ops.cross_entropy(logits * 1.0, labels)
    loss.backward()
    assert abs(loss.item() - ref.item()) <= 2e-3 * abs(ref.item()) + 1e-3
    _close(logits.grad, lf.grad, rtol=2e-2, atol=1e-5)


def test_embedding():
    torch.manual_seed(0)
    table = torch.randn(1000, 256, device=DEV, dtype=BF, requires_grad=True)
    ids = torch.randint(0, 1000, (4, 37), device=DEV)
    y = ops.embedding(ids, table)
    assert torch.equal(y, F.embedding(ids, table))
    g = torch.randn_like(y)
    y.backward(g)
    tf = table.detach().float().requires_grad_()
    F.embedding(ids, tf).backward(g.float())
    _close(table.grad, tf.grad)


@pytest.mark.parametrize("sk", [17, 128, 2048, 4100])
def test_softmax_masked_and_causal(sk):
    torch.manual_seed(0)
    b, h, sq = 2, 3, min(sk, 64)
    x = torch.randn(b, h, sq, sk, device=DEV, dtype=BF, requires_grad=True)
    mask = torch.rand(b, 1, sq, sk, device=DEV) < 0.2
    for kwargs in ({"mask": mask}, {"causal": True}, {}):
        y = ops.scaled_softmax(x, 0.3, **kwargs)
        xf = x.detach().float().requires_grad_()
        s = xf * 0.3
        if "mask" in kwargs:
            s = s.masked_fill(mask, -10000.0)
        if kwargs.get("causal"):
            keep = torch.ones(sq, sk, dtype=torch.bool, device=DEV).tril(sk - sq)
            s = s.masked_fill(~keep, float("-inf"))
        yr = torch.softmax(s, -1)
        g = torch.randn_like(y)
        x.grad = None
        y.backward(g)
        yr.backward(g.float())
        _close(y, yr, atol=4e-3)
        _close(x.grad, xf.grad, atol=4e-3)
