"""Profile-database generator: measures forward and backward time of every FASOP node type with this framework's
kernels on the local GPU and writes ``{model}_{gpu}_{tp}.npz`` (``data`` = forward ms, ``data_bwd`` = backward ms).

    python -m aicomp_b200.fasop.profile_b200 --model llama3b --tp 1 2 4 8 --mbs 1 2 4 8

The reference profiles whole training runs with module hooks and CUDA events and charges inline ops (norms, RoPE,
attention, residuals) to the next module (fasop/make_profiledb/profile_fx.py:450-746); the same attribution is used
here, but nodes are timed in isolation on tensor-parallel-sharded shapes, so one GPU is enough, and backward is
measured instead of assumed to be twice the forward.  The packed QKV and gate/up GEMMs that the fused layer runs
are timed as such and their time is split over the node types in proportion to their output widths.
"""
from __future__ import annotations

import argparse
import os

import numpy as np
import torch

from .. import ops
from ..ops import attention as attn_ops
from .config import MBS_OPTIONS, MODEL_CONFIGS, NODE_TYPES
from .profiledb import save_profile


def _time(fn, iters=5, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return float(np.median(ts))


def _fwd_bwd(make_inputs, fn):
    """Returns (forward ms, backward ms) of ``fn(*inputs)`` with a random upstream gradient."""
    ins = make_inputs()
    f = _time(lambda: fn(*ins))
    out = fn(*ins)
    g = torch.randn_like(out)

    def bwd():
        o = fn(*ins)
        o.backward(g)
    fb = _time(bwd)
    return f, max(fb - f, 0.0)


def profile_nodes(model, tp: int, mbs: int, dev="cuda"):
    m = model
    T, H, D = mbs * m.seq_len, m.hidden, m.head_dim
    hq, hkv, I = m.heads // tp, m.kv_heads // tp, m.ffn // tp
    bf = torch.bfloat16

    def P(*shape):
        p = (torch.randn(*shape, device=dev, dtype=bf) * 0.02).requires_grad_()
        p.main_grad = torch.zeros(*shape, device=dev, dtype=torch.float32)
        return p

    def X(*shape):
        return lambda: (torch.randn(*shape, device=dev, dtype=bf, requires_grad=True),)
    res = {}
    table = P(m.vocab, H)
    ids = torch.randint(0, m.vocab, (mbs, m.seq_len), device=dev)
    res["embed"] = _fwd_bwd(lambda: (), lambda: ops.embedding(ids, table))
    wn = P(H)
    wqkv = P((hq + 2 * hkv) * D, H)
    f, b = _fwd_bwd(X(T, H), lambda x: ops.linear(ops.rmsnorm(x, wn, 1e-5)[0], wqkv))
    tot = hq + 2 * hkv
    res["attn_q"] = (f * hq / tot, b * hq / tot)
    res["attn_k"] = (f * hkv / tot, b * hkv / tot)
    res["attn_v"] = (f * hkv / tot, b * hkv / tot)
    wo = P(H, hq * D)
    cos, sin = ops.rope_tables(m.seq_len, D, 500000.0, dev)
    pos = torch.arange(m.seq_len, device=dev, dtype=torch.int32).repeat(mbs)

    def attn_o(qkv):
        q = ops.apply_rope_qkv(qkv * 1.0, pos, cos, sin, hq + hkv, D)
        a = attn_ops.causal_attention_packed(q, mbs, m.seq_len, hq, hkv, D)
        return ops.linear(a, wo)
    res["attn_o"] = _fwd_bwd(X(T, (hq + 2 * hkv) * D), attn_o)
    wgu = P(2 * I, H)
    wn2 = P(H)
    f, b = _fwd_bwd(X(T, H), lambda x: ops.linear(ops.rmsnorm(x, wn2, 1e-5)[0], wgu))
    res["mlp_gate"] = (f / 2, b / 2)
    res["mlp_up"] = (f / 2, b / 2)
    res["mlp_act_fn"] = _fwd_bwd(X(T, 2 * I), lambda gu: ops.swiglu(gu))
    wd = P(H, I)
    res["mlp_down"] = _fwd_bwd(X(T, I), lambda a: ops.linear(a, wd))
    wl = P(m.vocab, H)
    wn3 = P(H)
    labels = torch.randint(0, m.vocab, (T,), device=dev)
    res["lm_head"] = _fwd_bwd(X(T, H), lambda x: ops.cross_entropy(ops.linear(ops.rmsnorm(x, wn3, 1e-5)[0], wl), labels).reshape(1))
    ops.check_errors()
    return res


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--model", default="llama3b", choices=sorted(MODEL_CONFIGS))
    ap.add_argument("--tp", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--mbs", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--gpu-name", default="B200")
    ap.add_argument("--out", default=os.path.join(os.path.dirname(os.path.abspath(__file__)), "known_cost"))
    a = ap.parse_args(argv)
    model = MODEL_CONFIGS[a.model]
    os.makedirs(a.out, exist_ok=True)
    for tp in a.tp:
        if model.heads % tp or model.kv_heads % tp or model.ffn % tp:
            continue
        fwd, bwd = [], []
        for mbs in sorted(a.mbs):
            if mbs not in MBS_OPTIONS:
                raise SystemExit(f"mbs must be one of {MBS_OPTIONS}")
            try:
                r = profile_nodes(model, tp, mbs)
            except torch.cuda.OutOfMemoryError:
                torch.cuda.empty_cache()
                break
            fwd.append([r[n][0] for n in NODE_TYPES])
            bwd.append([r[n][1] for n in NODE_TYPES])
            print(f"{a.model} tp{tp} mbs{mbs}: fwd layer {sum(fwd[-1][1:9]):.3f} ms, bwd layer {sum(bwd[-1][1:9]):.3f} ms, "
                  f"lm_head {fwd[-1][9]:.3f}/{bwd[-1][9]:.3f} ms", flush=True)
            torch.cuda.empty_cache()
        if fwd:
            path = os.path.join(a.out, f"{a.model}_{a.gpu_name}_{tp}.npz")
            save_profile(path, np.array(fwd), np.array(bwd))
            print("wrote", path)


if __name__ == "__main__":
    main()
