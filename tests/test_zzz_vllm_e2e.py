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


def _run(mode, model_dir, out, budget=None, env_extra=None):
    cmd = [sys.executable, os.path.join(ROOT, "tests", "vllm_worker.py"), mode,
           model_dir, out] + ([str(budget)] if budget is not None else [])
    env = dict(os.environ)
    env.pop("LOCKS_CONFIG", None)
    env.pop("LOCKS_DISABLE", None)
    env.update(env_extra or {})
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
    assert "[locks] KV write ACTIVE" in log       # do_kv_cache_update -> locks_kv_write
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


def test_selective_step_inside_vllm_matches_the_oracle(stock):
    """A SELECTIVE budget (24 of ~190 pages) inside the engine: the tenth decode
    step of an eager run is dumped by the plugin -- per layer the query, the KV
    cache, block table, lengths, summaries, selection and output as the engine
    had them -- and recomputed outside: the summaries against the oracle's build
    of the dumped K cache, and score / selected pages / attention output against
    the oracle's decode step on the dumped inputs.  A selection bug cannot hide
    here the way it can when every page is kept."""
    import numpy as np
    import torch
    import locks_oracle as orc
    model_dir, _want, tmp = stock
    dump = str(tmp / "dump.pt")
    got, log = _run("locks", model_dir, str(tmp / "locks_sel.json"), budget=24,
                    env_extra={"LOCKS_DUMP_STEP": "10", "LOCKS_DUMP_PATH": dump})
    assert got is not None, log[-3000:]
    assert "[locks] dumped decode step 10" in log, log[-2000:]
    layers = torch.load(dump)
    assert sorted(layers) == [0, 1]
    n_kv, G, page, sink, window = 2, 4, 16, 1, 2
    for l, d in layers.items():
        Kc = d["k_cache"].float().numpy()                # (blocks used, page, n_kv, d)
        Vc = d["v_cache"].float().numpy()
        bt, sl = d["block_table"].numpy(), d["seq_lens"].numpy()
        R = sl.shape[0]
        assert R == 2 and sl.min() > 700
        rec = d["records"].numpy()                       # (NB, n_kv, 832) uint8
        slabs = {
            "v4": rec[..., 0:512].reshape(rec.shape[0], n_kv, 8, 64),
            "mu8": rec[..., 512:640].view(np.int8),
            "c8": rec[..., 640:768].view(np.int8).reshape(rec.shape[0], n_kv, 16, 8),
            "cs": torch.from_numpy(rec[..., 768:800].copy()).view(torch.bfloat16)
                  .float().numpy(),
            "vs": torch.from_numpy(rec[..., 800:816].copy()).view(torch.bfloat16)
                  .float().numpy(),
            "mus": torch.from_numpy(rec[..., 816:818].copy()).view(torch.bfloat16)
                   .float().numpy()[..., 0],
        }
        # (a) the engine-built summaries of the pages in use, against the oracle
        used = np.unique(np.concatenate(
            [bt[r, :(sl[r] - 1) // page] for r in range(R)])).astype(np.int64)
        ref = orc.rki4_build_pages(Kc[used])
        Vr, Vn, Cr, Cn = orc.align_signs(ref, {k: v[used] for k, v in slabs.items()})
        dv, dc = np.abs(Vr - Vn), np.abs(Cr - Cn)
        assert dv.max() <= 1 and (dv > 0).mean() <= 1e-3
        assert dc.max() <= 1 and (dc > 0).mean() <= 1e-3
        # (b) the step itself on the dumped inputs
        q = d["q"].float().numpy()
        step = orc.gqa_decode_step(slabs, q, Kc, Vc, bt, sl, 128 ** -0.5, n_kv=n_kv,
                                   G=G, page=page, window=window, sink=sink,
                                   budget_pages=24, split=8)
        np.testing.assert_array_equal(d["b_fix"].numpy(), step["b"])
        nsh = step["n_sel_hi"]
        for r in range(R):
            np.testing.assert_allclose(d["score_h"].numpy()[r, :, :, :nsh[r]],
                                       step["score_h"][r, :, :, :nsh[r]],
                                       rtol=2e-4, atol=2e-4)
        np.testing.assert_array_equal(d["page_cnt"].numpy(), step["page_cnt"])
        assert int(step["page_cnt"].max()) == 24 + sink + window
        tab, tab_ref = d["page_table"].numpy(), step["page_table"]
        for r in range(R):
            for kh in range(n_kv):
                n = step["page_cnt"][r, kh]
                a, b = set(tab[r, kh, :n].tolist()), set(tab_ref[r, kh, :n].tolist())
                if a != b:         # only pages tied with the threshold (1e-3)
                    sel = [p for p in b if sink <= p < nsh[r]]
                    tau = min(step["score"][r, kh, p] for p in sel)
                    assert all(abs(step["score"][r, kh, p] - tau) <= 1e-3 * abs(tau)
                               for p in a ^ b)
        ref64, _ = orc.attention_over_pages(q, Kc, Vc, bt, tab, d["page_cnt"].numpy(),
                                            sl, 128 ** -0.5, n_kv, G)
        np.testing.assert_allclose(d["out"].float().numpy(), ref64, atol=2e-2,
                                   rtol=1e-2)


def test_mixed_prefill_decode_steps_are_split(stock):
    """Chunked prefill with 512 batched tokens per step: the first request decodes
    while the second prompt's chunks are still being prefilled, so steps carry a
    decode row next to a prefill chunk.  Those decode rows must go through the
    sparse path too (batch-split), not to the dense attention: every decode row
    of the run is counted sparse, and with every page kept the tokens and
    log-probabilities equal stock vLLM's under the same chunking."""
    model_dir, _want, tmp = stock
    env = {"VLLM_WORKER_CHUNK": "512"}
    want, log0 = _run("stock", model_dir, str(tmp / "stock_mixed.json"),
                      env_extra=env)
    if want is None:
        pytest.skip("stock vLLM with chunked prefill did not start: " + log0[-300:])
    got, log = _run("locks", model_dir, str(tmp / "locks_mixed.json"),
                    env_extra=env)
    _check(got, log, want)
    act = got["activation"]
    assert act is not None and act["dense"] == 0, act
    # 2 x 40 decode rows in all; some of them rode along with prefill chunks
    assert act["sparse"] >= 78, act


def _run_mla(mode, model_dir, out, budget=None):
    cmd = [sys.executable, os.path.join(ROOT, "tests", "vllm_mla_worker.py"), mode,
           model_dir, out] + ([str(budget)] if budget is not None else [])
    env = dict(os.environ)
    env.pop("LOCKS_CONFIG", None)
    env.pop("LOCKS_DISABLE", None)
    try:
        p = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=480)
    except subprocess.TimeoutExpired:
        return None, "timed out"
    log = p.stdout + p.stderr
    if p.returncode != 0 or "WORKER_DONE" not in log or not os.path.exists(out):
        return None, log
    with open(out) as fh:
        return json.load(fh), log


def test_mla_hook_inside_a_vllm_engine(tmp_path):
    """The MLA decode hook (``LocksMLAImpl.forward_mqa``: device-side factor
    gate, page scores, selection, sparse latent attention) inside a real vLLM
    engine on a two-layer DeepSeek-V2-shaped model (latent cache 512 + 64, 16
    heads, dense MLPs, random weights), Triton MLA backend replaced by
    ``register()``.  With every page kept the greedy tokens equal stock vLLM's
    (their log-probabilities to 0.05); a run with a selective budget must
    complete.  The numerics of the functions the hook calls are checked against
    the oracle in ``tests/test_gpu_mla.py``; this test is about the hook's place
    in the engine."""
    pytest.importorskip("vllm")
    model_dir = str(tmp_path / "tiny_deepseek_v2")
    want, log = _run_mla("stock", model_dir, str(tmp_path / "stock.json"))
    if want is None:
        pytest.skip("stock vLLM (Triton MLA) did not start here: " + log[-300:])
    got, log = _run_mla("locks", model_dir, str(tmp_path / "locks.json"))
    assert got is not None, log[-3000:]
    assert "[locks] ACTIVE (MLA)" in log, log[-3000:]
    assert [len(x) for x in got["ids"]] == [24, 24]
    assert got["ids"] == want["ids"]
    for a, b in zip(got["logprobs"], want["logprobs"]):
        assert max(abs(x - y) for x, y in zip(a, b)) <= 0.05
    sel, log = _run_mla("locks", model_dir, str(tmp_path / "sel.json"), budget=24)
    assert sel is not None, log[-3000:]
    assert "[locks] ACTIVE (MLA) budget_pages=24" in log
    assert [len(x) for x in sel["ids"]] == [24, 24]
