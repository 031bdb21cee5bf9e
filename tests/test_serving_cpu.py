"""Continuous batching on CPU: scheduler invariants with a fake cache, and token-exact serving vs HF greedy."""
import torch

from tests.models_small import build_model


def test_scheduler_admission_backpressure_and_release():
    from aicomp_b200.serve.paged_kv import PagedKVCache
    from aicomp_b200.serve.scheduler import ContinuousBatchingScheduler, Request
    cache = PagedKVCache(1, 1, 8, num_pages=9, max_seqs=4, max_blocks_per_seq=8, dtype=torch.float32, device="cpu")
    sch = ContinuousBatchingScheduler(cache, max_running=4, max_prefill_per_step=4)
    for i in range(4):
        sch.add_request(Request(rid=i, prompt=list(range(20)), max_new_tokens=12, arrival_s=0.0))  # 32 tokens = 2 pages
    sch.add_request(Request(rid=9, prompt=[1], max_new_tokens=1, arrival_s=100.0))
    plan = sch.plan_step(0.0)
    assert [r.rid for r in plan.prefill] == [0, 1, 2, 3] and cache.alloc.available() == 0
    for r in plan.prefill:
        sch.after_prefill(r, 7, 0.1)
    assert len(sch.running) == 4
    # nothing more can be admitted, and the request from the future stays queued
    assert sch.plan_step(1.0).prefill == []
    for step in range(11):
        sch.after_decode(list(sch.running), [5] * len(sch.running), 1.0 + step)
    assert not sch.running and len(sch.finished) == 4 and cache.alloc.available() == 8
    assert all(len(r.generated) == 12 for r in sch.finished)
    assert [r.rid for r in sch.plan_step(200.0).prefill] == [9]


def test_serving_engine_matches_hf_greedy():
    from aicomp_b200.serve.engine import ServingEngine
    from aicomp_b200.serve.scheduler import Request
    ref = build_model("llama").eval()
    prompts = [[5, 7, 11, 13, 17], [2, 3], [9] * 19, [1, 2, 3, 4, 5, 6, 7]]
    news = [6, 9, 4, 12]
    want = []
    for p, n in zip(prompts, news):
        out = torch.tensor([p])
        with torch.no_grad():
            for _ in range(n):
                out = torch.cat([out, ref(input_ids=out, use_cache=False).logits[:, -1].argmax(-1, keepdim=True)], 1)
        want.append(out[0, len(p):].tolist())
    eng = ServingEngine(build_model("llama"), use_gpu=False, num_pages=64, max_seqs=3, max_seq_len=64)
    reqs = [Request(rid=i, prompt=p, max_new_tokens=n, arrival_s=0.01 * i) for i, (p, n) in enumerate(zip(prompts, news))]
    m = eng.serve(reqs, realtime=False)
    got = {r.rid: r.generated for r in eng.scheduler.finished}
    assert [got[i] for i in range(4)] == want
    assert m["requests"] == 4 and m["unfinished"] == 0 and eng.cache.alloc.available() == 63


def test_pd_disaggregated_protocol_matches_hf_greedy():
    """Prefill worker + decode worker over the loopback transport: pages prefilled in one cache and pushed into the
    other give the tokens of plain greedy decoding, with back-pressure on the decode pool."""
    from aicomp_b200.serve.engine import ServingEngine
    from aicomp_b200.serve.pd_engine import DecodeWorker, LoopbackTransport, PrefillWorker
    from aicomp_b200.serve.scheduler import Request
    ref = build_model("llama").eval()
    prompts = [[5, 7, 11, 13, 17], [2, 3], [9] * 19, [1, 2, 3, 4, 5, 6, 7], [4] * 33]
    news = [6, 9, 4, 12, 3]
    want = []
    for p, n in zip(prompts, news):
        out = torch.tensor([p])
        with torch.no_grad():
            for _ in range(n):
                out = torch.cat([out, ref(input_ids=out, use_cache=False).logits[:, -1].argmax(-1, keepdim=True)], 1)
        want.append(out[0, len(p):].tolist())
    pre = ServingEngine(build_model("llama"), use_gpu=False, num_pages=16, max_seqs=2, max_seq_len=64)
    dec = ServingEngine(build_model("llama"), use_gpu=False, num_pages=7, max_seqs=3, max_seq_len=64)  # 6 usable pages: back-pressure
    tr = LoopbackTransport(pre.cache, dec.cache)
    mk = lambda: [Request(rid=i, prompt=p, max_new_tokens=n, arrival_s=0.01 * i) for i, (p, n) in enumerate(zip(prompts, news))]
    pw, dw = PrefillWorker(pre, tr, mk()), DecodeWorker(dec, tr, mk(), max_running=3)
    now, guard = 0.0, 0
    while (pw.has_work() or dw.has_work()) and guard < 10000:
        dw.step(now)
        pw.step(now)
        now += 0.01
        guard += 1
    assert not pw.has_work() and not dw.has_work()
    got = {r.rid: r.generated for r in dw.finished}
    assert [got[i] for i in range(len(prompts))] == want
    assert dec.cache.alloc.available() == 6 and pre.cache.alloc.available() == 15
    assert all(r.t_first_token is not None and r.t_finished >= r.t_first_token for r in dw.finished)
    assert tr.bytes_pushed > 0


def test_tensor_parallel_serving_keeps_ranks_in_step():
    """A TP2 replica under real-time arrivals: both ranks take the same scheduling decisions (one broadcast clock), so
    the run finishes and gives the tokens of the single-rank engine."""
    from tests.dist_utils import run_workers
    one = run_workers("serve_worker", 1, {"tp": 1}, timeout=240)
    two = run_workers("serve_worker", 2, {"tp": 2}, timeout=240)
    assert two[0]["tokens"] == two[1]["tokens"] == one[0]["tokens"]
    assert two[0]["requests"] == 6 and two[0]["unfinished"] == 0
