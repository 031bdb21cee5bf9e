"""Generation through Optimus_Inference must match HuggingFace greedy decoding (CPU, fp32)."""
import pytest
import torch

from tests.dist_utils import run_workers
from tests.models_small import build_model


def _hf_greedy(model, ids, n):
    model.eval()
    out = ids.clone()
    with torch.no_grad():
        for _ in range(n):
            logits = model(input_ids=out, use_cache=False).logits[:, -1]
            out = torch.cat([out, logits.argmax(-1, keepdim=True)], 1)
    return out


@pytest.mark.parametrize("model_name", ["llama", "gpt2"])
@pytest.mark.parametrize("kv", [False, True])
def test_generate_single_process_matches_hf(model_name, kv):
    from aicomp_b200 import Optimus_Inference
    if model_name == "gpt2" and kv:
        pytest.skip("GPT-2 graphs take learned positions from the traced arange; cached decoding is covered by Llama")
    ref = build_model(model_name)
    want = _hf_greedy(ref, torch.tensor([[5, 7, 11, 13], [2, 3, 4, 9]]), 6)
    eng = Optimus_Inference(build_model(model_name), use_gpu=False, use_kv_cache=kv, max_seq_len=64, dtype=torch.float32)
    got = eng.generate(torch.tensor([[5, 7, 11, 13], [2, 3, 4, 9]]), max_new_tokens=6, do_sample=False, verbose=False)
    assert torch.equal(got, want)


def test_generate_pp2_tp2_kv_cache_matches_hf():
    ref = build_model("llama")
    want = _hf_greedy(ref, torch.tensor([[5, 7, 11, 13], [2, 3, 4, 9]]), 5).tolist()
    res = run_workers("infer_worker", 4, {"pp": 2, "tp": 2, "kv": True, "new": 5}, timeout=300)
    outs = [r["ids"] for r in res if r and r.get("ids") is not None]
    assert outs and all(o == want for o in outs)


def test_sampling_filters():
    from aicomp_b200.inference import sample_token
    torch.manual_seed(0)
    logits = torch.tensor([[0.0, 5.0, 4.0, -1.0, 3.0]]).repeat(200, 1)
    t = sample_token(logits.clone(), temperature=1.0, top_k=2, top_p=1.0, do_sample=True)
    assert set(t.tolist()) <= {1, 2}
    t = sample_token(logits.clone(), temperature=1.0, top_k=0, top_p=0.5, do_sample=True)
    assert set(t.tolist()) == {1}
    assert sample_token(logits, do_sample=False).tolist() == [1] * 200
