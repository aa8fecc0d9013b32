"""Child process of tests/test_zzz_vllm_e2e.py (MLA): one vLLM engine on a tiny
random-weight DeepSeek-V2-shaped model -- latent KV cache of 512 + 64 channels,
16 heads, dense MLPs, no tokenizer, no files beyond a generated config.json --
on vLLM's Triton MLA backend, with or without the LOCKS plugin (which replaces
that backend's decode with page selection + sparse latent attention), greedy-
decoding two prompts.

usage: vllm_mla_worker.py <stock|locks> <model_dir> <out.json> [budget_pages]
"""
import json
import os
import sys

os.environ.setdefault("HF_HUB_OFFLINE", "1")
os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")

mode, model_dir, out_path = sys.argv[1], sys.argv[2], sys.argv[3]
budget_pages = int(sys.argv[4]) if len(sys.argv) > 4 else 100000

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "locks-kv_b200"))

import torch  # noqa: E402

CONFIG = {
    "architectures": ["DeepseekV2ForCausalLM"], "model_type": "deepseek_v2",
    "hidden_size": 1024, "intermediate_size": 2048, "moe_intermediate_size": 512,
    "num_hidden_layers": 2, "num_attention_heads": 16, "num_key_value_heads": 16,
    "kv_lora_rank": 512, "q_lora_rank": None, "qk_nope_head_dim": 128,
    "qk_rope_head_dim": 64, "v_head_dim": 128, "n_routed_experts": 4,
    "n_shared_experts": 1, "num_experts_per_tok": 2, "n_group": 1, "topk_group": 1,
    # every layer below first_k_dense_replace has a dense MLP: no expert is built
    "first_k_dense_replace": 2, "moe_layer_freq": 1, "vocab_size": 32000,
    "max_position_embeddings": 8192, "rms_norm_eps": 1e-06, "rope_theta": 10000.0,
    "rope_scaling": None, "hidden_act": "silu", "tie_word_embeddings": False,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
    "attention_bias": False, "attention_dropout": 0.0,
}
os.makedirs(model_dir, exist_ok=True)
with open(os.path.join(model_dir, "config.json"), "w") as fh:
    json.dump(CONFIG, fh)

if mode.startswith("locks"):
    from locks.backend.register import register
    register({"variant": "fast", "budget_pages": budget_pages, "sink_pages": 1,
              "window_pages": 2})

from vllm import LLM, SamplingParams  # noqa: E402

llm = LLM(model=model_dir, load_format="dummy", skip_tokenizer_init=True,
          dtype="bfloat16", max_model_len=8192, block_size=16, enforce_eager=True,
          gpu_memory_utilization=0.08, enable_prefix_caching=False, seed=0,
          max_num_seqs=4, attention_backend="TRITON_MLA")
g = torch.Generator().manual_seed(1)
prompts = [{"prompt_token_ids": torch.randint(3, 31000, (n,), generator=g).tolist()}
           for n in (3000, 777)]
sp = SamplingParams(max_tokens=24, temperature=0.0, detokenize=False,
                    ignore_eos=True, logprobs=0)
outs = llm.generate(prompts, sp)
ids = [list(o.outputs[0].token_ids) for o in outs]
lps = [[float(step[tok].logprob) for step, tok in zip(o.outputs[0].logprobs,
                                                      o.outputs[0].token_ids)]
       for o in outs]
with open(out_path, "w") as fh:
    json.dump({"ids": ids, "logprobs": lps}, fh)
print("WORKER_DONE", mode, flush=True)
os._exit(0)
