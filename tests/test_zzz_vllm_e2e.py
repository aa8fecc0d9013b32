"""The plugin inside a real vLLM engine (collected last: it starts two engines).

A two-layer Llama-shaped model with random weights (8 query / 2 KV heads of 128,
block size 16) decodes 40 tokens after 3000- and 777-token prompts, once with
stock vLLM and once with ``locks.backend.register.register()`` applied -- the
registration a ``vllm.general_plugins`` entry point performs.  With a budget
that keeps every page the sparse path (page summaries built by the metadata
builder, score -> select -> sparse decode in ``LocksAttentionImpl.forward``)
must reproduce the stock greedy tokens and their log-probabilities (to 0.05);
the engine's log must show that the
LOCKS path actually ran.  Skipped where vLLM is not installed or cannot start
without the plugin either.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu

CONFIG = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 1024, "intermediate_size": 2048, "num_hidden_layers": 2,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 128,
    "vocab_size": 32000, "max_position_embeddings": 32768, "rms_norm_eps": 1e-05,
    "rope_theta": 500000.0, "hidden_act": "silu", "tie_word_embeddings": False,
    "torch_dtype": "bfloat16", "bos_token_id": 1, "eos_token_id": 2,
}


def _run(mode, model_dir, out, budget=None):
    cmd = [sys.executable, os.path.join(ROOT, "tests", "vllm_worker.py"), mode,
           model_dir, out] + ([str(budget)] if budget is not None else [])
    env = dict(os.environ)
    env.pop("LOCKS_CONFIG", None)
    env.pop("LOCKS_DISABLE", None)
    try:
        p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=480)
    except subprocess.TimeoutExpired as e:
        return None, (e.stdout or "") + (e.stderr or "") if isinstance(
            e.stdout, str) else "timed out"
    log = p.stdout + p.stderr
    if p.returncode != 0 or "WORKER_DONE" not in log or not os.path.exists(out):
        return None, log
    with open(out) as fh:
        return json.load(fh), log


@pytest.fixture(scope="module")
def stock(tmp_path_factory):
    """(model_dir, stock result): one stock engine for both tests."""
    pytest.importorskip("vllm")
    tmp = tmp_path_factory.mktemp("vllm_e2e")
    model_dir = str(tmp / "tiny_llama")
    os.makedirs(model_dir)
    with open(os.path.join(model_dir, "config.json"), "w") as fh:
        json.dump(CONFIG, fh)
    res, log = _run("stock", model_dir, str(tmp / "stock.json"))
    if res is None:
        pytest.skip("stock vLLM did not start here: " + log[-300:])
    return model_dir, res, tmp


def _check(got, log, want):
    assert got is not None, log[-3000:]
    assert "[locks] ACTIVE" in log and "[locks] sparse decode ACTIVE" in log, \
        log[-3000:]
    assert "[locks] state allocated" in log
    assert [len(x) for x in got["ids"]] == [40, 40]
    assert got["ids"] == want["ids"]
    # every page kept: the sparse decode is the dense attention up to bf16
    # rounding of a different summation order
    for a, b in zip(got["logprobs"], want["logprobs"]):
        assert max(abs(x - y) for x, y in zip(a, b)) < 0.05, (a[:5], b[:5])


def test_plugin_reproduces_stock_tokens_inside_vllm(stock):
    model_dir, want, tmp = stock
    got, log = _run("locks", model_dir, str(tmp / "locks.json"))
    _check(got, log, want)


def test_plugin_inside_full_cuda_graphs(stock):
    """Same, with CUDA graphs on: vLLM captures FULL decode graphs with the
    LOCKS launches inside (the builder reports single-token-decode graph
    support) and the 40 decode steps replay them."""
    model_dir, want, tmp = stock
    got, log = _run("locks-graph", model_dir, str(tmp / "locks_graph.json"))
    _check(got, log, want)
    assert "decode, FULL" in log, log[-2000:]
