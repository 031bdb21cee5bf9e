"""Device-timed micro-benchmarks of the sm_100a kernels against their library counterparts.

``python -m aicomp_b200.ops.microbench gemm`` times the tcgen05 GEMM and
``torch.matmul`` (cuBLAS) on the linear-layer shapes of Llama-3-8B with CUDA
events, L2 flushed between iterations, and prints one JSON line per shape.
"""
from __future__ import annotations

import json
import sys

import torch

from aicomp_b200 import ops


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2]


def bench_gemm(shapes=None):
    dev = "cuda"
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    shapes = shapes or [
        # (M, N, K, a_mn, b_mn, out_f32_accumulate, label)
        (2048, 6144, 4096, False, False, False, "qkv fwd"),
        (2048, 4096, 4096, False, False, False, "o_proj fwd"),
        (2048, 28672, 4096, False, False, False, "gate_up fwd"),
        (2048, 4096, 14336, False, False, False, "down fwd"),
        (2048, 4096, 28672, False, True, False, "gate_up dgrad"),
        (28672, 4096, 2048, True, True, True, "gate_up wgrad"),
        (4096, 14336, 2048, True, True, True, "down wgrad"),
        (6144, 4096, 2048, True, True, True, "qkv wgrad"),
        (8192, 8192, 8192, False, False, False, "square 8k"),
        (2048, 128256, 4096, False, False, False, "lm_head fwd"),
    ]
    for (M, N, K, a_mn, b_mn, acc, label) in shapes:
        a = torch.randn((K, M) if a_mn else (M, K), device=dev, dtype=torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device=dev, dtype=torch.bfloat16)
        out = torch.zeros(M, N, device=dev, dtype=torch.float32 if acc else torch.bfloat16)
        res = {"shape": [M, N, K], "label": label, "a_mn": a_mn, "b_mn": b_mn}
        flops = 2.0 * M * N * K
        for bn in (128, 256):
            t = _time(lambda: ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=acc, bn=bn), flush=flush)
            res[f"ours_bn{bn}_ms"] = round(t, 4)
            res[f"ours_bn{bn}_tflops"] = round(flops / t / 1e9, 1)
        t = _time(lambda: ops.gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=out, accumulate=acc, pair=True), flush=flush)
        res["ours_pair_ms"] = round(t, 4)
        res["ours_pair_tflops"] = round(flops / t / 1e9, 1)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        if acc:  # cuBLAS has no bf16-in / fp32-accumulate-into form through torch: time the plain bf16 product
            t = _time(lambda: torch.matmul(A, B), flush=flush)
        else:
            t = _time(lambda: torch.matmul(A, B, out=out), flush=flush)
        res["cublas_ms"] = round(t, 4)
        res["cublas_tflops"] = round(flops / t / 1e9, 1)
        ops.check_errors()
        print(json.dumps(res), flush=True)
        del a, b, out


def bench_attention(shapes=None):
    """Causal attention forward and backward of this library against torch SDPA (cuDNN / flash) on the same data."""
    import torch.nn.functional as F

    from aicomp_b200.ops import flash
    dev = "cuda"
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for (B, S, hq, hkv) in shapes or [(1, 2048, 32, 8), (4, 2048, 32, 8), (2, 4096, 32, 8), (1, 8192, 32, 8)]:
        D = 128
        qkv = torch.randn(B * S, (hq + 2 * hkv) * D, device=dev, dtype=torch.bfloat16)
        dout = torch.randn(B * S, hq * D, device=dev, dtype=torch.bfloat16)
        fwd_flops = 4.0 * B * hq * S * S * D / 2
        res = {"B": B, "S": S, "hq": hq, "hkv": hkv}
        out, lse = flash.flash_fwd(qkv, B, S, hq, hkv, D, need_lse=True)
        t = _time(lambda: flash.flash_fwd(qkv, B, S, hq, hkv, D, need_lse=True), flush=flush)
        res["ours_fwd_ms"], res["ours_fwd_tflops"] = round(t, 4), round(fwd_flops / t / 1e9, 1)
        t = _time(lambda: flash.flash_bwd(qkv, out, dout, lse, B, S, hq, hkv, D), flush=flush)
        res["ours_bwd_ms"], res["ours_bwd_tflops"] = round(t, 4), round(2.5 * fwd_flops / t / 1e9, 1)
        q = qkv[:, : hq * D].view(B, S, hq, D).transpose(1, 2).detach().requires_grad_(True)
        k = qkv[:, hq * D:(hq + hkv) * D].view(B, S, hkv, D).transpose(1, 2).detach().requires_grad_(True)
        v = qkv[:, (hq + hkv) * D:].view(B, S, hkv, D).transpose(1, 2).detach().requires_grad_(True)
        do4 = dout.view(B, S, hq, D).transpose(1, 2)
        with torch.no_grad():
            t = _time(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True), flush=flush)
        res["sdpa_fwd_ms"], res["sdpa_fwd_tflops"] = round(t, 4), round(fwd_flops / t / 1e9, 1)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
        t = _time(lambda: torch.autograd.grad(o, (q, k, v), do4, retain_graph=True), flush=flush)
        res["sdpa_bwd_ms"], res["sdpa_bwd_tflops"] = round(t, 4), round(2.5 * fwd_flops / t / 1e9, 1)
        ops.check_errors()
        print(json.dumps(res), flush=True)


def small_case(kind: str, launches: int = 3) -> None:
    """A few launches of one kernel on inputs larger than L2 and well under 2 GB: the case a profiler captures."""
    dev = "cuda"
    if kind in ("gemm", "gemm1"):  # gate_up forward of Llama-3-8B on 8192 tokens: A 64 MB, B 224 MB, C 448 MB
        a = torch.randn(8192, 4096, device=dev, dtype=torch.bfloat16)
        b = torch.randn(28672, 4096, device=dev, dtype=torch.bfloat16)
        out = torch.empty(8192, 28672, device=dev, dtype=torch.bfloat16)
        # "gemm": the CTA-pair kernel (default for this size); "gemm1": the single-CTA kernel with 128 x 256 tiles
        fn = (lambda: ops.gemm(a, b, out=out)) if kind == "gemm" else (lambda: ops.gemm(a, b, out=out, bn=256))
        work = 2.0 * 8192 * 28672 * 4096
    elif kind == "wgrad":   # gate_up weight gradient, fp32 accumulate in memory (TMA reduce-add epilogue)
        x = torch.randn(8192, 4096, device=dev, dtype=torch.bfloat16)
        dy = torch.randn(8192, 28672, device=dev, dtype=torch.bfloat16)
        out = torch.zeros(28672, 4096, device=dev, dtype=torch.float32)
        fn = lambda: ops.gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True)
        work = 2.0 * 8192 * 28672 * 4096
    elif kind == "flash":   # causal attention forward on packed QKV: 8 x 4096 tokens, 32 query / 8 KV heads of 128
        from aicomp_b200.ops import flash
        qkv = torch.randn(8 * 4096, (32 + 16) * 128, device=dev, dtype=torch.bfloat16)
        fn = lambda: flash.flash_fwd(qkv, 8, 4096, 32, 8, 128)
        work = 4.0 * 8 * 32 * 4096 * 4096 * 128 / 2
    elif kind == "flashbwd":  # causal attention backward, 4 x 4096 tokens, 32 query / 8 KV heads of 128
        from aicomp_b200.ops import flash
        B, S = 4, 4096
        qkv = torch.randn(B * S, (32 + 16) * 128, device=dev, dtype=torch.bfloat16)
        dout = torch.randn(B * S, 32 * 128, device=dev, dtype=torch.bfloat16)
        out, lse = flash.flash_fwd(qkv, B, S, 32, 8, 128, need_lse=True)
        fn = lambda: flash.flash_bwd(qkv, out, dout, lse, B, S, 32, 8, 128)
        work = 2.5 * 4.0 * B * 32 * S * S * 128 / 2
    elif kind == "rmsnorm":  # 65536 x 4096 bf16: 512 MB in, 512 MB out
        x = torch.randn(65536, 4096, device=dev, dtype=torch.bfloat16)
        w = torch.ones(4096, device=dev, dtype=torch.bfloat16)
        fn = lambda: ops.rmsnorm(x, w, 1e-5)
        work = 2.0 * x.numel() * 2
    else:
        raise SystemExit(f"unknown small case {kind}")
    with torch.no_grad():
        t = _time(fn, iters=launches, warmup=2)
    ops.check_errors()
    print(json.dumps({"case": kind, "ms": round(t, 4), "work_per_s": round(work / t / 1e9, 1),
                      "unit": "GB/s" if kind == "rmsnorm" else "TFLOP/s"}), flush=True)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    if what == "gemm":
        bench_gemm()
    elif what == "attention":
        bench_attention()
    elif what == "small":
        small_case(sys.argv[2] if len(sys.argv) > 2 else "gemm")
    else:
        raise SystemExit(f"unknown benchmark {what}")
