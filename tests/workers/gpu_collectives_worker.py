"""Rank body (one GPU per rank, NCCL): fused peer-memory collectives vs NCCL / PyTorch references."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tests.dist_utils import worker_args, worker_report  # noqa: E402

from aicomp_b200 import ops  # noqa: E402
from aicomp_b200.parallel.comm import Comm  # noqa: E402


def main():
    a = worker_args()
    comm = Comm(use_gpu=True)
    dev = comm.device
    world = comm.world_size
    group = dist.group.WORLD
    out = {}
    torch.manual_seed(100 + comm.rank)

    if "allreduce" in a["tests"]:
        from aicomp_b200.parallel.fused_dp import FusedGradAllReduce
        ar = FusedGradAllReduce(group, world, dev)
        n = 8 * 1024 * 1024 + 64
        arena = ar.alloc_arena(n)
        errs = []
        for it in range(3):
            x = torch.randn(n, device=dev)
            arena.copy_(x)
            ref = x.clone()
            dist.all_reduce(ref)
            ref /= world
            region = arena[1024:n - 28]
            ar.all_reduce_mean_(region)
            torch.cuda.synchronize()
            errs.append((region - ref[1024:n - 28]).abs().max().item())
            assert torch.equal(arena[:1024], x[:1024])  # outside the region untouched
        ops.check_errors()
        # timing vs NCCL on 1 GiB
        n = 256 * 1024 * 1024
        ar2 = FusedGradAllReduce(group, world, dev)
        big = ar2.alloc_arena(n)
        big.normal_()
        nccl_buf = torch.randn(n, device=dev)

        def timed(fn, iters=5):
            fn(); torch.cuda.synchronize(); dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record(); torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()
        t_fused = timed(lambda: ar2.all_reduce_mean_(big))
        t_nccl = timed(lambda: (dist.all_reduce(nccl_buf), nccl_buf.div_(world)))
        ops.check_errors()
        busbw = lambda t: 2 * (world - 1) / world * n * 4 / (t * 1e-3) / 1e9
        out["allreduce"] = {"max_err": max(errs), "fused_ms": t_fused, "nccl_ms": t_nccl, "fused_busbw_GBs": busbw(t_fused),
                            "nccl_busbw_GBs": busbw(t_nccl)}

    if "kv_push" in a["tests"] and world >= 2:
        from aicomp_b200.serve.pd import KVPagePusher
        layers, pages, page_bytes = 4, 64, 16 * 8 * 128 * 2
        pusher = KVPagePusher(group, dev, layers=layers, pool_pages=pages, page_bytes=page_bytes)
        pool = pusher.local_pool  # uint8 [layers, 2, pages, page_bytes]
        if comm.rank == 0:
            pool.copy_(torch.randint(0, 255, pool.shape, dtype=torch.uint8, device=dev))
        dist.barrier()
        src_pages = torch.tensor([3, 7, 11, 60], dtype=torch.int32, device=dev)
        dst_pages = torch.tensor([0, 1, 5, 9], dtype=torch.int32, device=dev)
        if comm.rank == 0:
            pusher.push(dst_rank=1, src_pages=src_pages, dst_pages=dst_pages, request_slot=2, ready_value=77)
            torch.cuda.synchronize()
        ok = True
        if comm.rank == 1:
            ok = pusher.wait_ready(request_slot=2, ready_value=77, timeout_s=20.0)
        dist.barrier()
        gathered = [torch.empty_like(pool) for _ in range(world)] if comm.rank == 1 else None
        full0 = pool.clone()
        dist.broadcast(full0, src=0)
        if comm.rank == 1:
            for s, d in zip(src_pages.tolist(), dst_pages.tolist()):
                ok = ok and torch.equal(pool[:, :, d], full0[:, :, s])
        out["kv_push"] = {"ok": bool(ok)}
        ops.check_errors()

    if "tp_fused" in a["tests"]:
        from aicomp_b200.parallel import fused_tp
        T, H, Nq, I = a.get("T", 4096), 4096, 6144 // world, 14336 // world
        Tl = T // world
        res = {}

        def timed(fn, iters=8):
            for _ in range(3):
                fn()
            torch.cuda.synchronize(); dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(iters):
                fn()
            e.record(); torch.cuda.synchronize()
            t = torch.tensor([s.elapsed_time(e) / iters], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()

        # all-gather -> GEMM (QKV-like and gate/up-like)
        for name, N, K in (("qkv", Nq, H), ("gate_up", 2 * I, H)):
            x_local = torch.randn(Tl, K, device=dev, dtype=torch.bfloat16)
            w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
            y = fused_tp._ag_gemm_raw(x_local, w, group)
            xg = torch.empty(T, K, device=dev, dtype=torch.bfloat16)
            dist.all_gather_into_tensor(xg, x_local)
            ref = xg.float() @ w.float().t()
            res[f"ag_{name}_err"] = ((y.float() - ref).abs().max() / ref.abs().max()).item()
            res[f"ag_{name}_fused_ms"] = timed(lambda: fused_tp._ag_gemm_raw(x_local, w, group))
            res[f"ag_{name}_nccl_ms"] = timed(lambda: (dist.all_gather_into_tensor(xg, x_local), ops.gemm(xg, w)))
            res[f"ag_{name}_gemm_only_ms"] = timed(lambda: ops.gemm(xg, w))
        # GEMM -> reduce-scatter (out-proj-like and down-proj-like)
        for name, N, K in (("o_proj", H, 4096 // world), ("down", H, I)):
            x = torch.randn(T, K, device=dev, dtype=torch.bfloat16)
            w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
            y = fused_tp._gemm_rs_raw(x, w, group)
            full = (x.float() @ w.float().t())
            dist.all_reduce(full)
            ref = full[comm.rank * Tl:(comm.rank + 1) * Tl]
            res[f"rs_{name}_err"] = ((y.float() - ref).abs().max() / ref.abs().max()).item()
            rs_out = torch.empty(Tl, N, device=dev, dtype=torch.bfloat16)
            res[f"rs_{name}_fused_ms"] = timed(lambda: fused_tp._gemm_rs_raw(x, w, group))
            res[f"rs_{name}_nccl_ms"] = timed(lambda: dist.reduce_scatter_tensor(rs_out, ops.gemm(x, w)))
            res[f"rs_{name}_gemm_only_ms"] = timed(lambda: ops.gemm(x, w))
        ops.check_errors()
        out["tp_fused"] = res

    worker_report(out)
    comm.barrier()


if __name__ == "__main__":
    main()
