"""Host-side utilities: watchdog, metrics, configuration."""
import json
import time

import pytest


def test_watchdog_detects_silent_rank_and_bad_steps():
    from aicomp_b200.utils.watchdog import DictStore, Watchdog
    store = DictStore()
    dogs = [Watchdog(store, r, 3, interval_s=0.05, timeout_s=0.4).start() for r in range(3)]
    time.sleep(0.2)
    assert dogs[0].silent_ranks() == []
    dogs[2].pause()                     # rank 2 stops reporting, as a wedged or dead process would
    time.sleep(0.7)
    assert dogs[0].silent_ranks() == [2] and dogs[1].silent_ranks() == [2]
    w = dogs[0]
    for _ in range(6):
        assert w.end_step(0.10, loss=2.0) is None
    assert w.end_step(0.9, loss=2.0)["kind"] == "slow_step"
    assert w.end_step(0.1, loss=float("nan"))["kind"] == "nonfinite_loss"
    for d in dogs:
        d.stop()


def test_metrics_logger_and_timer(tmp_path):
    import torch
    from aicomp_b200.utils.metrics import MetricsLogger, StepTimer
    t = StepTimer(torch.device("cpu"))
    t.start(); time.sleep(0.01); t.stop()
    assert t.elapsed_ms(max_over_ranks=False) >= 9.0
    log = MetricsLogger(str(tmp_path / "m.jsonl"))
    log.log_train_step(1, 100.0, tokens=2048, loss=2.0)
    log.close()
    rec = json.loads(open(tmp_path / "m.jsonl").read().splitlines()[0])
    assert rec["Train/tokens_per_s"] == pytest.approx(20480.0) and rec["step"] == 1


def test_config_roundtrip_and_validation(tmp_path):
    from aicomp_b200.utils.config import ParallelConfig, TrainConfig, load_config
    p = tmp_path / "c.yaml"
    p.write_text("parallel:\n  pp_size: 2\n  dp_size: 4\n  num_mb: 16\nlr: 0.0003\nschedule: 1f1b\n")
    cfg = load_config(str(p))
    assert cfg.parallel.pp_size == 2 and cfg.lr == 0.0003
    kw = cfg.engine_kwargs()
    assert kw["pp_size"] == 2 and kw["num_mb"] == 16
    assert cfg.optimizer_kwargs()["grad_scale"] == pytest.approx(1 / 16)
    with pytest.raises(ValueError):
        ParallelConfig(pp_size=2, dp_size=2).validate(world_size=8)
    bad = tmp_path / "bad.json"
    bad.write_text('{"learning_rate": 1}')
    with pytest.raises(ValueError):
        load_config(str(bad))


def test_native_data_helpers_match_numpy():
    import numpy as np
    from aicomp_b200.ops import build as kb
    from aicomp_b200.utils import data_helpers as dh
    kb.build()
    rng = np.random.RandomState(0)
    sizes = rng.randint(1, 400, size=300).astype(np.int32)
    sizes[5] = 0                                    # an empty document must be skipped
    epochs = 3
    doc_idx = np.concatenate([rng.permutation(300) for _ in range(epochs)]).astype(np.int32)
    tokens = int(sizes.sum())
    for seq in (8, 128, 1000):
        got = dh.build_sample_idx(sizes, doc_idx, seq, epochs, tokens)
        ref = dh.build_sample_idx_numpy(sizes, doc_idx, seq, dh.num_samples(epochs, tokens, seq))
        assert np.array_equal(got, ref)
        # every boundary points inside its document
        assert (got[:, 1] < sizes[doc_idx[got[:, 0]]]).all()
    ds, si = dh.build_blending_indices([0.5, 0.3, 0.2], 10000)
    frac = np.bincount(ds, minlength=3) / 10000
    assert np.allclose(frac, [0.5, 0.3, 0.2], atol=2e-3)
    for d in range(3):
        assert np.array_equal(si[ds == d], np.arange((ds == d).sum()))


def test_packed_dataset_serves_shifted_windows():
    import numpy as np
    from aicomp_b200.utils.data_helpers import BlendedDataset, PackedTokenDataset
    docs = [np.arange(100 * i, 100 * i + n) for i, n in enumerate([37, 5, 64, 120, 9])]
    ds = PackedTokenDataset(docs, seq_len=16, num_epochs=2)
    assert len(ds) == (2 * 235 - 1) // 16
    x, y = ds[0]
    assert x.shape == (16,) and (x[1:] == y[:-1]).all()
    bl = BlendedDataset([ds, ds], [0.7, 0.3], size=50)
    assert len(bl) == 50 and bl[49][0].shape == (16,)


def test_schedule_in_flight_counts_and_ring_layout():
    """Slots a stage needs for CUDA-graph replay (micro-batches between forward and backward) and the byte layout of
    one pipeline mailbox slot."""
    import torch

    from aicomp_b200.parallel.schedule import Schedule1F1B, ScheduleGPipe

    class _E:
        training = True

    def mk(cls, stage, P, M):
        s = cls.__new__(cls)
        s.e, s.stage, s.P, s.M = _E(), stage, P, M
        return s
    for P, M in ((2, 16), (4, 8), (4, 2), (1, 8)):
        for stage in range(P):
            s = mk(Schedule1F1B, stage, P, M)
            live = peak = 0
            for kind, _ in s.order():
                live += 1 if kind == "F" else -1
                peak = max(peak, live)
            assert peak == s.in_flight() == min(P - stage, M)
            assert mk(ScheduleGPipe, stage, P, M).in_flight() == M
    from aicomp_b200.parallel.p2p import PeerChannel
    ch = PeerChannel.__new__(PeerChannel)
    total = ch._layout([(torch.bfloat16, (1, 2048, 4096), True), (torch.int64, (3,), False), (torch.float32, (5, 7), False)])
    assert ch._offsets == [0, 2048 * 4096 * 2, 2048 * 4096 * 2 + 256]
    assert total == 2048 * 4096 * 2 + 256 + 256 and all(o % 256 == 0 for o in ch._offsets)


def test_conv1d_substitution_keeps_the_function():
    """GPT-2's Conv1D layers rewritten to the [in, out]-weight linear op: same parameters, same outputs and gradients
    (CPU runs the op's PyTorch fallback; the GEMM path is checked on the GPU)."""
    import copy

    import torch
    from transformers import GPT2Config, GPT2LMHeadModel

    from aicomp_b200.graph.rewrite import substitute_kernels
    from aicomp_b200.graph.tracer import trace_model
    torch.manual_seed(0)
    model = GPT2LMHeadModel(GPT2Config(vocab_size=128, n_embd=32, n_layer=2, n_head=4, n_positions=64, resid_pdrop=0.0,
                                       embd_pdrop=0.0, attn_pdrop=0.0))
    ref = copy.deepcopy(model)
    ids = torch.randint(0, 128, (2, 16))
    tr = trace_model(model, ["input_ids"], example_inputs={"input_ids": ids})
    counts = substitute_kernels(tr.gm, model)
    assert counts.get("conv1d") == 8
    out = tr.gm(input_ids=ids)["logits"]
    want = ref(input_ids=ids).logits
    assert torch.allclose(out, want, atol=1e-5)
    out.sum().backward()
    want.sum().backward()
    g = model.transformer.h[0].attn.c_attn.weight.grad
    assert g is not None and torch.allclose(g, ref.transformer.h[0].attn.c_attn.weight.grad, atol=1e-4)
