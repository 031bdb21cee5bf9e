"""Pipeline / tensor-parallel generation: ``torchrun --nproc-per-node N examples/pp_inference_llama.py --pp-size P --tp-size T``.

Flags follow the reference's ``pp_inference_llama.py`` (examples/pp_inference_llama.py:95-200): ``--use-kv-cache``,
``--use-kv-manager``, ``--serving-mode``, ``--use-mps`` with ``--num-gpus`` / ``--gpu-ids``.  The MPS helper must run
before torch is imported.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp-size", type=int, default=1)
    ap.add_argument("--tp-size", type=int, default=1)
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--use-kv-cache", action="store_true")
    ap.add_argument("--use-kv-manager", action="store_true")
    ap.add_argument("--serving-mode", action="store_true")
    ap.add_argument("--use-mps", action="store_true")
    ap.add_argument("--num-gpus", type=int, default=None)
    ap.add_argument("--gpu-ids", default=None)
    ap.add_argument("--cpu", action="store_true")
    a = ap.parse_args()
    from opt_prime.mps_manager import setup_mps_for_inference
    mgr = setup_mps_for_inference(a.use_mps, a.num_gpus, a.gpu_ids) if (a.use_mps or a.num_gpus or a.gpu_ids) else None
    import torch
    from transformers import LlamaConfig, LlamaForCausalLM

    from opt_prime.inference import Optimus_Inference
    cfg = LlamaConfig(num_hidden_layers=8, hidden_size=1024, num_attention_heads=8, num_key_value_heads=4, intermediate_size=2816,
                      vocab_size=32000, max_position_embeddings=2048, tie_word_embeddings=False)
    torch.manual_seed(0)
    eng = Optimus_Inference(LlamaForCausalLM(cfg), use_gpu=not a.cpu, pp_size=a.pp_size, tp_size=a.tp_size, use_kv_cache=a.use_kv_cache,
                            use_kv_manager=a.use_kv_manager, serving_mode=a.serving_mode, use_mps=a.use_mps,
                            dtype=torch.float32 if a.cpu else torch.bfloat16)
    prompt = torch.randint(0, cfg.vocab_size, (2, 24)) if eng.is_first_stage() else None
    for round_ in range(2 if a.serving_mode else 1):
        out = eng.generate(prompt, max_new_tokens=a.max_new_tokens, do_sample=False, verbose=False)
        if eng.is_output_rank():
            print(f"round {round_}: generated {out.shape[1] - 24} tokens per sequence; first row tail {out[0, -8:].tolist()}")
    eng.barrier()
    if mgr is not None:
        mgr.stop()


if __name__ == "__main__":
    main()
