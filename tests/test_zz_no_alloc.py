"""The allocation-free RMSNorm backward entry point against the regular one.

Some users of the kernel library cannot allocate device memory when they call it: a server that gave all of its
HBM to a page pool at start-up, a plug-in running inside a runtime that owns the allocator, a loop that cannot
afford cudaMalloc's device-wide synchronisation.  ``b200_rmsnorm_bwd_noalloc`` serves them by keeping its scratch
in a fixed array inside the library.  This test calls it through its exported C symbol (ctypes, no wrapper of the
package in between) and checks dx and dw against ``b200_norm_bwd`` with caller-provided scratch, twice in a row so
that the shared scratch array is shown not to carry anything over, and checks that an over-limit size is refused.
The file sorts last so that a run stopping at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from aicomp_b200.ops import _lib as L
    lib = L.require()
    P, I = ctypes.c_void_p, ctypes.c_int
    fn = lib.b200_rmsnorm_bwd_noalloc
    fn.argtypes = [P, P, P, P, P, P, P, P, I, I, I, P]
    fn.restype = I
    return lib, fn


def _inputs(rows, H, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
    dy = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
    w = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16()
    dres = torch.randn(rows, H, device="cuda", generator=g).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5).contiguous()
    return x, dy, w, dres, rstd


def test_noalloc_rmsnorm_bwd_matches_regular_entry_twice():
    lib, fn = _lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, H) in enumerate([(777, 4096), (300, 1024)]):  # second call is smaller: stale partials would show
        x, dy, w, dres, rstd = _inputs(rows, H, seed=call)
        dx_ref = torch.empty_like(x)
        dw_ref = torch.zeros(H, device="cuda", dtype=torch.float32)
        scratch = torch.empty(2 * lib.b200_norm_bwd_ctas() * H, device="cuda", dtype=torch.float32)
        rc = lib.b200_norm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), None, dres.data_ptr(), dx_ref.data_ptr(),
                               scratch.data_ptr(), dw_ref.data_ptr(), None, None, None, 0, rows, H, 0, stream)
        assert rc == 0
        dx = torch.empty_like(x)
        dw = torch.full((H,), 123.0, device="cuda", dtype=torch.float32)
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), dw.data_ptr(), None,
                0, rows, H, stream)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        torch.cuda.synchronize()
        assert torch.equal(dx, dx_ref)
        err = (dw - dw_ref).abs().max().item()
        assert err <= 2e-2 * dw_ref.abs().max().item() + 2e-2, err  # partial sums are grouped differently (148 vs 296 CTAs)
        # and against plain PyTorch fp32 math, the oracle of the other norm tests
        xf, wf = x.float(), w.float()
        xh = xf * rstd[:, None]
        gvec = dy.float() * wf
        dx_t = rstd[:, None] * (gvec - xh * (gvec * xh).mean(-1, keepdim=True)) + dres.float()
        assert (dx.float() - dx_t).abs().max().item() <= 2e-2 * dx_t.abs().max().item() + 2e-2
        assert (dw - (dy.float() * xh).sum(0)).abs().max().item() <= 3e-2 * dw_ref.abs().max().item() + 0.3


def test_noalloc_rejects_sizes_beyond_its_scratch():
    lib, fn = _lib()
    x = torch.zeros(2, 16384, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), rstd.data_ptr(), None, x.data_ptr(), None, None, 0, 2, 16384,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -20
