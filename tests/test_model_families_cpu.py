"""The model families the reference's examples train (opt_prime/examples/pp_train_*.py: GPT-Neo, GPT-J, BERT, ELECTRA,
OPT, ViT, Whisper, GPT-2 sequence classification, Qwen2-MoE; plus Mistral): the traced graph and its two-stage split
reproduce the eager model exactly, also for a batch / sequence length other than the traced example."""
import pytest
import torch

pytest.importorskip("transformers")


def _tiny(name):
    import transformers as T
    if name == "gptneo":
        return T.GPTNeoForCausalLM(T.GPTNeoConfig(vocab_size=128, hidden_size=32, num_layers=4, num_heads=4, window_size=8,
                                                  attention_types=[[["global", "local"], 2]], max_position_embeddings=64)), "ids"
    if name == "gptj":
        return T.GPTJForCausalLM(T.GPTJConfig(vocab_size=128, n_embd=32, n_layer=4, n_head=4, rotary_dim=8, n_positions=64)), "ids"
    if name == "bert":
        return T.BertForMaskedLM(T.BertConfig(vocab_size=128, hidden_size=32, num_hidden_layers=4, num_attention_heads=4,
                                              intermediate_size=64, max_position_embeddings=64)), "ids"
    if name == "electra":
        return T.ElectraForMaskedLM(T.ElectraConfig(vocab_size=128, embedding_size=16, hidden_size=32, num_hidden_layers=4,
                                                    num_attention_heads=4, intermediate_size=64, max_position_embeddings=64)), "ids"
    if name == "opt":
        return T.OPTForCausalLM(T.OPTConfig(vocab_size=128, hidden_size=32, num_hidden_layers=4, num_attention_heads=4, ffn_dim=64,
                                            max_position_embeddings=64, word_embed_proj_dim=32)), "ids"
    if name == "vit":
        return T.ViTForImageClassification(T.ViTConfig(hidden_size=32, num_hidden_layers=4, num_attention_heads=4, intermediate_size=64,
                                                       image_size=32, patch_size=8, num_labels=10)), "pixels"
    if name == "whisper":
        return T.WhisperForConditionalGeneration(T.WhisperConfig(
            vocab_size=128, d_model=32, encoder_layers=2, decoder_layers=2, encoder_attention_heads=4, decoder_attention_heads=4,
            encoder_ffn_dim=64, decoder_ffn_dim=64, num_mel_bins=8, max_source_positions=16, max_target_positions=32, pad_token_id=0,
            bos_token_id=1, eos_token_id=2, decoder_start_token_id=1)), "speech"
    if name == "gpt2cls":
        return T.GPT2ForSequenceClassification(T.GPT2Config(vocab_size=128, n_embd=32, n_layer=4, n_head=4, n_positions=64,
                                                            num_labels=3, pad_token_id=0)), "ids"
    if name == "qwenmoe":
        return T.Qwen2MoeForCausalLM(T.Qwen2MoeConfig(
            vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
            moe_intermediate_size=16, shared_expert_intermediate_size=32, num_experts=4, num_experts_per_tok=2,
            max_position_embeddings=64)), "ids"
    if name == "mistral":
        return T.MistralForCausalLM(T.MistralConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=4,
                                                    num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                                    sliding_window=None)), "ids"
    raise ValueError(name)


def _logits(out):
    return out["logits"] if isinstance(out, dict) else out


@pytest.mark.parametrize("name", ["gptneo", "gptj", "bert", "electra", "opt", "vit", "whisper", "gpt2cls", "qwenmoe", "mistral"])
def test_family_traces_and_splits_exactly(name):
    from aicomp_b200.graph.partition import assign_stages
    from aicomp_b200.graph.split import build_stage_plan, extract_stage
    from aicomp_b200.graph.tracer import trace_model
    torch.manual_seed(0)
    model, kind = _tiny(name)
    model.eval()
    if kind == "ids":
        ex = {"input_ids": torch.randint(1, 128, (2, 16))}
    elif kind == "pixels":
        ex = {"pixel_values": torch.randn(2, 3, 32, 32)}
    else:
        ex = {"input_features": torch.randn(2, 8, 32), "decoder_input_ids": torch.randint(1, 128, (2, 8))}
    with torch.no_grad():
        ref = model(**ex).logits
    tr = trace_model(model, list(ex), example_inputs=ex)
    with torch.no_grad():
        assert torch.equal(_logits(tr.gm(**ex)), ref)
        if kind == "ids":  # dynamic shapes: nothing of the example's batch or length is baked into the graph
            other = {"input_ids": torch.randint(1, 128, (3, 24))}
            assert torch.allclose(_logits(tr.gm(**other)), model(**other).logits, atol=1e-6)
    assign = assign_stages(tr.gm, 2, "simple", False, 1)
    plan = build_stage_plan(tr.gm, assign, 2)
    env, last = dict(ex), None
    with torch.no_grad():
        for s in range(2):
            stage = extract_stage(tr.gm, assign, plan, s)
            last, outs = stage(*[env[n] for n in plan.stage_inputs[s]])
            env.update(dict(zip(plan.stage_outputs[s], outs)))
    assert torch.equal(_logits(last), ref)
    # the stages hold disjoint parameter sets that together cover the model
    p0 = {n for n, _ in extract_stage(tr.gm, assign, plan, 0).named_parameters()}
    p1 = {n for n, _ in extract_stage(tr.gm, assign, plan, 1).named_parameters()}
    assert p0 and p1


@pytest.mark.parametrize("name", ["vit", "whisper", "gpt2cls", "qwenmoe"])
def test_family_trains_through_the_engine(name):
    """Image, speech (two inputs), classification-head and mixture-of-experts models step through ``Optimus_p`` and
    learn (single process, two micro-batches)."""
    from aicomp_b200 import Optimus_p
    torch.manual_seed(0)
    model, kind = _tiny(name)
    kw = {}
    if kind == "ids":
        data = torch.randint(1, 128, (4, 16))
        labels = torch.randint(0, 3, (4,)) if name == "gpt2cls" else data.clone()
    elif kind == "pixels":
        data, labels = torch.randn(4, 3, 32, 32), torch.randint(0, 10, (4,))
    else:
        data = {"input_features": torch.randn(4, 8, 32), "decoder_input_ids": torch.randint(1, 128, (4, 8))}
        labels = torch.randint(1, 128, (4, 8))
        kw = {"input_names": ["input_features", "decoder_input_ids"]}
    e = Optimus_p(model, num_mb=2, use_gpu=False, **kw)
    opt = torch.optim.AdamW(e.parameters(), lr=1e-3)
    losses = []
    for _ in range(3):
        opt.zero_grad()
        e.run(data, labels, mode="1f1b")
        opt.step()
        losses.append(sum(e.get_loss()) / 2)
    assert losses[-1] < losses[0], losses


@pytest.mark.parametrize("name", ["gptneo", "gptj", "bert", "electra", "opt", "vit", "whisper", "gpt2cls", "qwenmoe", "mistral"])
def test_family_export_capture_is_exact(name):
    """The ``dynamo_capture=True`` path (torch.export + unflatten, rebuilt as a module-level graph) on the same families."""
    from aicomp_b200.graph.export_capture import export_to_module_graph
    torch.manual_seed(0)
    model, kind = _tiny(name)
    model.eval()
    if kind == "ids":
        ex = {"input_ids": torch.randint(1, 128, (2, 16))}
    elif kind == "pixels":
        ex = {"pixel_values": torch.randn(2, 3, 32, 32)}
    else:
        ex = {"input_features": torch.randn(2, 8, 32), "decoder_input_ids": torch.randint(1, 128, (2, 8))}
    with torch.no_grad():
        ref = model(**ex).logits
    tr = export_to_module_graph(model, list(ex), example_inputs=ex)
    with torch.no_grad():
        assert torch.allclose(_logits(tr.gm(**ex)), ref, atol=1e-6)
        if kind == "ids":
            other = {"input_ids": torch.randint(1, 128, (3, 24))}
            assert torch.allclose(_logits(tr.gm(**other)), model(**other).logits, atol=1e-6)


@pytest.mark.parametrize("name", ["gptneo", "gptj", "bert", "opt", "gpt2cls", "mistral"])
def test_traced_graph_carries_no_dtype_of_the_trace(name):
    """Traced in fp32, run in bf16: a graph that had baked ``torch.float32`` (from ``x.dtype``, ``torch.finfo``) would fail
    or silently up-cast; it must follow the parameters' dtype like the eager model."""
    from aicomp_b200.graph.tracer import trace_model
    torch.manual_seed(0)
    model, _ = _tiny(name)
    model.eval()
    ex = {"input_ids": torch.randint(1, 128, (2, 16))}
    tr = trace_model(model, ["input_ids"], example_inputs=ex)
    model.to(torch.bfloat16)   # the graph module shares the model's parameters
    with torch.no_grad():
        got = _logits(tr.gm(**ex))
        want = model(**ex).logits
    assert got.dtype == want.dtype == torch.bfloat16
    assert torch.allclose(got.float(), want.float(), atol=5e-2, rtol=5e-2)
