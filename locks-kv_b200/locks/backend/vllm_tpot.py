"""End-to-end decode time per token inside vLLM, stock against the LOCKS plugin.

usage: python locks-kv_b200/locks/backend/vllm_tpot.py <stock|locks> [context_tokens=130560] [decode_tokens=513]

Starts one vLLM engine (in-process engine core, CUDA graphs on) on a
Llama-3.1-8B-shaped model with random weights (32 layers, 32 query / 8 KV heads
of 128, no tokenizer), feeds one prompt of ``context_tokens - 8`` random ids and
times greedy generation of 1 token (prefill, best of two) and of
``decode_tokens`` tokens (best of two); time per output token = the difference
over ``decode_tokens - 1``.  ``stock`` leaves vLLM's own backend choice alone;
``locks`` applies ``register()`` (budget 128 pages + 1 sink + 8 recent, the
benchmark's config 1) and starts vLLM on the FlashAttention backend the plugin
replaces.  Prints one ``RESULT {json}`` line.
"""
import json
import os
import sys
import tempfile
import time

os.environ.setdefault("HF_HUB_OFFLINE", "1")
os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")

mode = sys.argv[1]
ctx = int(sys.argv[2]) if len(sys.argv) > 2 else 130560
n_tok = int(sys.argv[3]) if len(sys.argv) > 3 else 513

PKG_PARENT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, PKG_PARENT)

import torch  # noqa: E402

if mode == "locks":
    from locks.backend.register import register
    register({"variant": "fast", "budget_pages": 128, "sink_pages": 1,
              "window_pages": 8})

from vllm import LLM, SamplingParams  # noqa: E402

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "vocab_size": 128256, "max_position_embeddings": 131072, "rms_norm_eps": 1e-05,
    "rope_theta": 500000.0, "hidden_act": "silu", "tie_word_embeddings": False,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
}
model_dir = tempfile.mkdtemp(prefix="llama8b_shape_")
with open(os.path.join(model_dir, "config.json"), "w") as fh:
    json.dump(CONFIG, fh)

kw = {} if mode == "stock" else {"attention_backend": "FLASH_ATTN"}
t0 = time.time()
llm = LLM(model=model_dir, load_format="dummy", skip_tokenizer_init=True,
          dtype="bfloat16", max_model_len=ctx + 512, block_size=16,
          enforce_eager=False, gpu_memory_utilization=0.40,
          enable_prefix_caching=False, seed=0, max_num_seqs=1,
          max_num_batched_tokens=16384, **kw)
init_s = time.time() - t0
g = torch.Generator().manual_seed(1)
prompt = [{"prompt_token_ids":
           torch.randint(3, 120000, (ctx - 8,), generator=g).tolist()}]


def run(n):
    sp = SamplingParams(max_tokens=n, temperature=0.0, detokenize=False,
                        ignore_eos=True)
    torch.cuda.synchronize()
    t = time.time()
    o = llm.generate(prompt, sp, use_tqdm=False)
    torch.cuda.synchronize()
    return time.time() - t, list(o[0].outputs[0].token_ids)


first, _ = run(1)                       # includes one-time warm-up (summary state)
prefill = min(run(1)[0], run(1)[0])
ta, ids = run(n_tok)
tb, ids = run(n_tok)
res = {"mode": mode, "context_tokens": ctx, "decode_tokens": n_tok,
       "engine_start_s": init_s, "first_prefill_s": first, "prefill_s": prefill,
       "generate_s": [ta, tb],
       "ms_per_output_token": (min(ta, tb) - prefill) / (n_tok - 1) * 1e3,
       "first_ids": ids[:8]}
print("RESULT", json.dumps(res), flush=True)
os._exit(0)       # skip engine teardown: nothing is in flight
