"""Child process of tests/test_zzz_vllm_e2e.py: one vLLM engine on a tiny
random-weight Llama (no tokenizer, no files beyond a generated config.json),
with or without the LOCKS plugin, greedy-decoding two prompts.

usage: vllm_worker.py <stock|locks|locks-graph> <model_dir> <out.json> [budget_pages]
(``locks-graph``: CUDA graphs on, so the decode steps replay FULL graphs that
hold the LOCKS launches; the other modes run eagerly)

``VLLM_WORKER_CHUNK=<tokens>``: chunked prefill with that many batched tokens
per step, so that the second prompt's chunks are co-scheduled with the first
request's decode steps (mixed steps).  ``LOCKS_DUMP_STEP`` / ``LOCKS_DUMP_PATH``
pass through to the plugin (one decode step saved for an outside check).
"""
import json
import os
import sys

os.environ.setdefault("HF_HUB_OFFLINE", "1")
os.environ.setdefault("TRANSFORMERS_OFFLINE", "1")
# engine core in this process: register() below must act on the engine itself
os.environ["VLLM_ENABLE_V1_MULTIPROCESSING"] = "0"
os.environ.setdefault("VLLM_LOGGING_LEVEL", "WARNING")

mode, model_dir, out_path = sys.argv[1], sys.argv[2], sys.argv[3]
budget_pages = int(sys.argv[4]) if len(sys.argv) > 4 else 100000

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "locks-kv_b200"))

import torch  # noqa: E402

if mode.startswith("locks"):
    from locks.backend.register import register
    register({"variant": "fast", "budget_pages": budget_pages, "sink_pages": 1,
              "window_pages": 2})

from vllm import LLM, SamplingParams  # noqa: E402

chunk = int(os.environ.get("VLLM_WORKER_CHUNK", "0"))
extra = dict(enable_chunked_prefill=True, max_num_batched_tokens=chunk) if chunk else {}
llm = LLM(model=model_dir, load_format="dummy", skip_tokenizer_init=True,
          dtype="bfloat16", max_model_len=8192, block_size=16, enforce_eager=(mode != "locks-graph"),
          gpu_memory_utilization=0.08, enable_prefix_caching=False, seed=0,
          max_num_seqs=4, attention_backend="FLASH_ATTN", **extra)
g = torch.Generator().manual_seed(1)
prompts = [{"prompt_token_ids": torch.randint(3, 31000, (n,), generator=g).tolist()}
           for n in (3000, 777)]
sp = SamplingParams(max_tokens=40, temperature=0.0, detokenize=False,
                    ignore_eos=True, logprobs=0)
outs = llm.generate(prompts, sp)
ids = [list(o.outputs[0].token_ids) for o in outs]
# log-probability of every generated token: sensitive to the attention output
# where the greedy token itself is not
lps = [[float(step[tok].logprob) for step, tok in zip(o.outputs[0].logprobs,
                                                      o.outputs[0].token_ids)]
       for o in outs]
act = None
if mode.startswith("locks"):
    from locks.backend import _runtime
    act = _runtime.get_activation()
with open(out_path, "w") as fh:
    json.dump({"ids": ids, "logprobs": lps, "activation": act}, fh)
print("WORKER_DONE", mode, flush=True)
os._exit(0)       # skip engine teardown: nothing is in flight, the ids are on disk
