"""Benchmark of the LOCKS decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload c1|c0|c4] [--ctx TOKENS] [--no-cpu-baseline]

One "step" = the attention hot path of one decode step over all layers of the
workload: per layer  page score -> GQA combine + top-b select -> split-K sparse
paged decode -> merge, replayed as one CUDA graph.  The default workload is the
Llama-3.1-8B-shaped single-sequence decode at 131072 tokens of context
(32 layers, 32 q / 8 kv heads, d 128, page 16, budget 128 + 1 sink + 8 recent
pages).  Inputs are seeded synthetic KV caches of that shape, resident in HBM.
One JSON line is printed by rank 0.

With N > 1 every rank decodes its own sequence of the same shape (sequence
sharding, no data-path collective): weak scaling, value = N sequences' tokens/s.
The same line then carries the two partitioned workloads, run by all N ranks
together: `c2_sharded` (the seeded 64-sequence ragged batch with per-sequence
page budgets, sequences dealt to the ranks by step bytes, no collective) and
`cp` (ONE 1M-token sequence, context parallel over the ranks, exchanges inside
the selector and decode kernels; strong scaling) with `cp_parity`, a small
context-parallel case checked against the single-GPU path inside the run.

`--impl reference` times the CPU restatement of the reference's own path
(oracle/locks_oracle.py, numpy, all host threads) on a bounded sample of the
same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (os.path.join(ROOT, "locks-kv_b200"), os.path.join(ROOT, "oracle")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np  # noqa: E402
import torch  # noqa: E402

REC_ALGO_BYTES = 818           # summary bytes per (page, kv-head) the scorer needs
PAGE_KV_BYTES = 16 * 128 * 2 * 2   # K + V bytes of one attended (page, kv-head)


def score_traffic_per_unit():
    """DRAM bytes (read + write) the scorer moved per (page, kv-head) in the ncu
    capture of the committed profile summary: the line
    ``scorer_dram_bytes_per_unit: <number>`` of the summary file under
    ``profiles/``; None when no such line exists."""
    import glob
    import re
    for f in sorted(glob.glob(os.path.join(ROOT, "profiles", "*.md"))):
        m = re.search(r"^scorer_dram_bytes_per_unit:\s*([0-9.]+)", open(f).read(),
                      re.M)
        if m:
            return float(m.group(1))
    return None


def workload(name: str, ctx: int | None):
    from locks import synth
    if name == "c0":
        sh, c = synth.CONFIG0, 4096
    elif name in ("c1", "c1vt"):
        sh, c = synth.CONFIG1, 131072
    elif name in ("c4", "c4cp"):
        sh, c = synth.CONFIG4, 1048576
    elif name == "c2":
        # ragged continuous batch: 64 sequences, log-uniform in [4096, 262144]
        return synth.CONFIG1, c2_draw()[0]
    else:
        raise SystemExit(f"unknown workload {name}")
    return sh, (ctx or c)


def c2_draw(n_seq: int = 64):
    """The ragged batch of the continuous-batching workload: context lengths
    log-uniform in [4096, 262144] and a page budget per sequence from
    {32, 64, 128, 256}, both from one seed."""
    rng = np.random.default_rng(20260202)
    ctx = [int(x) for x in np.exp(rng.uniform(np.log(4096), np.log(262144), n_seq))]
    budgets = [int(b) for b in rng.choice([32, 64, 128, 256], n_seq)]
    return ctx, budgets


def algo_bytes(sh, seq_len, budgets=None):
    """Algorithmic bytes of one step: summaries scanned + selected K/V pages
    (summed over the sequences of a ragged batch; ``budgets``: one page budget
    per sequence instead of the shape's)."""
    lens = seq_len if isinstance(seq_len, (list, tuple)) else [seq_len]
    score = dec = dense = nsh_t = A_t = 0
    for i, sl in enumerate(lens):
        npg = -(-sl // sh.page)
        nsh = npg - sh.window_pages
        bp = budgets[i] if budgets is not None else sh.budget_pages
        A = min(bp, max(nsh - sh.sink_pages, 0)) + sh.sink_pages \
            + sh.window_pages
        score += sh.n_layers * sh.n_kv * nsh * REC_ALGO_BYTES
        dec += sh.n_layers * sh.n_kv * A * PAGE_KV_BYTES
        dense += sh.n_layers * sh.n_kv * npg * PAGE_KV_BYTES
        nsh_t += nsh
        A_t = max(A_t, A)
    return score, dec, dense, nsh_t, A_t


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampler running beside the timed
    region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                 "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- #
# CPU arm: the oracle restatement of the reference path                        #
# --------------------------------------------------------------------------- #
class CpuArm:
    """The oracle restatement of the reference path on the host cores, on a
    bounded sample of the workload: ONE layer, at 1/4 of the context when the
    context exceeds 32K tokens.  Page scoring and selection are linear in the
    number of pages, so their time is scaled by the page ratio; the decode
    attends the same number of pages at any context, so its time is not.
    Summaries are built once, untimed."""

    def __init__(self, sh, seq_len, seed=1234):
        import locks_oracle as orc
        from locks import synth
        self.orc, self.sh = orc, sh
        ctx = seq_len - 1
        self.ctx_s = ctx // 4 if ctx > 32768 else ctx
        self.page_ratio = (ctx / self.ctx_s)
        case = synth.make_gqa_case(seed, sh, [self.ctx_s + 1], device="cpu",
                                   n_layers=1)
        f = lambda t: t.float().numpy()
        self.bt, self.sl = case.block_table.numpy(), case.seq_lens.numpy()
        self.Kc, self.Vc = f(case.kv_caches[0][:, 0]), f(case.kv_caches[0][:, 1])
        self.q = f(case.q[0])
        self.scale = case.scale
        self.MP = case.max_pages
        self.slabs = orc.rki4_build_pages(self.Kc)
        self.sample = (f"1 of {sh.n_layers} layers at ctx {self.ctx_s} "
                       f"(score+select time x{self.page_ratio:g}, decode x1), "
                       f"scaled x{sh.n_layers}; numpy oracle, summaries prebuilt")

    def step(self):
        """Seconds one full decode step would take (all layers, full ctx)."""
        orc, sh = self.orc, self.sh
        t0 = time.perf_counter()
        npg, nsh, b = orc.derive_page_params(self.sl, sh.page, sh.window_pages,
                                             sh.sink_pages, sh.budget_pages)
        score_h = orc.rki4_score(self.slabs, self.q, self.bt, nsh, self.scale,
                                 sh.n_kv, sh.G, self.MP)
        score = orc.nrm_combine(score_h, nsh)
        tab, cnt = orc.topb_select(score, npg, nsh, b, sh.sink_pages)
        t1 = time.perf_counter()
        m, l, acc = orc.sparse_decode_split(self.q, self.Kc, self.Vc, self.bt,
                                            tab, cnt, self.sl, self.scale,
                                            sh.n_kv, sh.G, 64, 2)
        orc.merge_splits(m, l, acc, cnt, 64, 2)
        t2 = time.perf_counter()
        return sh.n_layers * ((t1 - t0) * self.page_ratio + (t2 - t1))


class RefArm:
    """The reference's OWN CPU code, staged under ``oracle/_ref`` by
    ``oracle/make_ref.py``: its ``Rki4State("cpu")``, ``rki4_build_bulk``
    (LAPACK eigh; untimed set-up), and per step ``derive_page_params`` (its
    Triton kernel, interpreted), ``rki4_score_torch``, the nrm combine (three
    torch lines restating ``select_cuda.py:607-658``, as the golden generator
    does) and ``_topb_select_torch``, at the workload's FULL context.  The
    sparse decode + merge has no CPU implementation in the reference (Triton /
    CUDA only): that part is the numpy restatement.  A step = `layers` layers
    (each with its own seeded K/V), scaled to the workload's layer count."""

    def __init__(self, sh, seq_len, layers=1, seed=1234):
        os.environ.setdefault("TRITON_INTERPRET", "1")
        ref_root = os.path.join(ROOT, "oracle", "_ref")
        if ref_root not in sys.path:
            sys.path.insert(0, ref_root)
        from locks_ref.selection import rki4_build as rb
        from locks_ref.selection.rki4_score_torch import rki4_score_torch
        from locks_ref.selection.rki4_state import Rki4State
        from locks_ref.selection.select import (_topb_select_torch,
                                                derive_page_params)
        import locks_oracle as orc
        from locks import synth
        self.orc, self.sh, self.layers = orc, sh, layers
        self._score, self._select, self._derive = (rki4_score_torch,
                                                   _topb_select_torch,
                                                   derive_page_params)
        case = synth.make_gqa_case(seed, sh, [seq_len], device="cpu",
                                   n_layers=layers)
        self.case = case
        G = sh.G
        if G > 8:          # the reference asserts G <= 8; its CPU code is G-generic
            Rki4State.validate_geometry = staticmethod(lambda **kw: None)
        st = Rki4State("cpu", num_layers=layers, num_blocks=case.num_blocks,
                       n_kv=sh.n_kv, G=G, head_dim=sh.d, page=sh.page, max_reqs=1,
                       max_pages=case.max_pages, budget_pages=sh.budget_pages,
                       sink_pages=sh.sink_pages, window_pages=sh.window_pages,
                       combine="nrm")
        K_layers = [c[:, 0] for c in case.kv_caches]
        settled = case.seq_lens - 1
        rb.rki4_build_bulk(st, K_layers, case.block_table, settled, 1,
                           int((settled // sh.page).max()))
        self.st = st
        f = lambda t: t.float().numpy()
        self.bt, self.sl = case.block_table.numpy(), case.seq_lens.numpy()
        self.Kc = [f(c[:, 0]) for c in case.kv_caches]
        self.Vc = [f(c[:, 1]) for c in case.kv_caches]
        self.qf = [f(case.q[l]) for l in range(layers)]
        self.sample = (f"{layers} of {sh.n_layers} layers at the full context "
                       f"({seq_len - 1} tokens), time x{sh.n_layers / layers:g}; "
                       "reference torch code for page parameters, scoring and "
                       "selection (oracle/_ref), numpy restatement for the "
                       "decode + merge it has no CPU code for; summaries prebuilt")

    def step(self):
        """Seconds the sampled layers took."""
        st, sh, case, orc = self.st, self.sh, self.case, self.orc
        t0 = time.perf_counter()
        self._derive(st, case.seq_lens, 1)
        for l in range(self.layers):
            self._score(st, l, case.q[l], case.block_table, case.seq_lens, 1,
                        case.scale)
            hi = int(st.n_sel_hi[0])
            hm = st.score_h[0, :, :, :hi].amax(-1, keepdim=True)
            acc = torch.zeros(sh.n_kv, hi)
            for g in range(sh.G):
                acc = acc + torch.exp(st.score_h[0, :, g, :hi] - hm[:, g])
            st.score[0, :, :hi] = acc
            self._select(st, 1)
            tab, cnt = st.page_table.numpy(), st.page_cnt.numpy()
            m, lse, a = orc.sparse_decode_split(
                self.qf[l], self.Kc[l], self.Vc[l], self.bt, tab, cnt, self.sl,
                case.scale, sh.n_kv, sh.G, 64, 2)
            orc.merge_splits(m, lse, a, cnt, 64, 2)
        return time.perf_counter() - t0


class RefArmMla:
    """Config 3 on the host cores with the reference's own torch code (staged
    under ``oracle/_ref``): ``build_page_factors`` (untimed set-up, as in the
    engine: factors are built once per prompt), then per step
    ``mla_page_score_ref``, ``topb_middle`` and the attention block of its
    backend (``backend/mla_attn.py:178-201``: gather the kept pages, fp32
    softmax(q kv^T) kv[:, :512]) -- ONE batch row of ONE layer at the full
    context, scaled by rows x layers."""

    def __init__(self, sh, seq_len, rows=8, seed=77):
        ref_root = os.path.join(ROOT, "oracle", "_ref")
        if ref_root not in sys.path:
            sys.path.insert(0, ref_root)
        from locks_ref.selection.mla_score_torch import (mla_page_score_ref,
                                                         topb_middle)
        from locks_ref.selection.mla_select import build_page_factors
        from locks import synth
        self.sh, self.rows = sh, rows
        self._score, self._keep = mla_page_score_ref, topb_middle
        case = synth.make_mla_case(seed, sh, [seq_len], device="cpu", n_layers=1)
        page, Lkv = sh.page, sh.kv_lora_rank
        self.L, self.page, self.Lkv = seq_len, page, Lkv
        n_pages, n_cache = -(-seq_len // page), seq_len // page
        self.n_pages, self.n_cache = n_pages, n_cache
        self.cache, self.bt = case.caches[0], case.block_table[0].long()
        kvb = self.cache.index_select(0, self.bt[:n_pages]).reshape(-1, sh.width)[:seq_len]
        Lf, Rf = build_page_factors(kvb[:n_cache * page, :Lkv].float(), n_cache, page, 8)
        self.C8 = Lf @ Rf
        self.k_rope = kvb[:n_cache * page, Lkv:].float().view(n_cache, page, -1)
        self.q = case.q[0][0].float()
        self.scale = case.scale
        self.sample = (f"1 of {rows} rows, 1 of {sh.n_layers} layers at the full "
                       f"context ({seq_len - 1} tokens), time x{rows * sh.n_layers}; "
                       "reference torch code (oracle/_ref): mla_page_score_ref, "
                       "topb_middle, fp32 attention over the kept pages as in its "
                       "backend; page factors prebuilt")

    def step(self):
        sh, page, Lkv, L = self.sh, self.page, self.Lkv, self.L
        t0 = time.perf_counter()
        valid = torch.full((self.n_cache,), page, dtype=torch.long)
        ps = torch.full((self.n_pages,), float("-inf"))
        ps[:self.n_cache] = self._score(self.q[:, :Lkv], self.q[:, Lkv:], self.C8,
                                        self.k_rope, valid, self.scale)
        keep = self._keep(ps, sh.budget_pages, sh.sink_pages, sh.window_pages)
        idx = keep.nonzero().flatten()
        sel = self.cache.index_select(0, self.bt[idx]).reshape(-1, sh.width).float()
        pos = (idx[:, None] * page + torch.arange(page)[None]).reshape(-1)
        sc = (self.q @ sel.T) * self.scale
        sc = sc.masked_fill(~(pos < L)[None], float("-inf"))
        o = torch.softmax(sc, -1) @ sel[:, :Lkv]
        lse = torch.logsumexp(sc, -1)
        del o, lse
        return time.perf_counter() - t0


def run_reference_mla(args, seq_len):
    from locks import synth
    sh = synth.CONFIG3
    if args.layers:
        import dataclasses
        sh = dataclasses.replace(sh, n_layers=args.layers)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    B = 8
    if not reference_available():
        return {"impl": "reference", "unavailable":
                "oracle/_ref is not staged (run oracle/make_ref.py where the "
                "reference checkout is)"}
    arm = RefArmMla(sh, seq_len, rows=B)
    for _ in range(args.warmup):
        arm.step()
    ts = [arm.step() for _ in range(args.steps)]
    tpot = float(np.mean(ts)) * B * sh.n_layers
    return {
        "impl": "reference", "metric": "sparse_decode_tokens_per_s",
        "value": B / tpot, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": float(np.mean(ts)) * 1e3, "tpot_ms": tpot * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": mla_config(sh, B, seq_len),
        "cpu_baseline": {"value": B / tpot, "unit": "tokens/s", "cores": cores,
                         "kind": "reference", "sample": arm.sample,
                         "tpot_ms": tpot * 1e3},
        "e2e": {"value": B / tpot, "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }


def mla_config(sh, B, seq_len):
    rec_b = 8448 + sh.page * sh.rope_dim * 2
    b_score = sh.n_layers * B * (seq_len // sh.page) * rec_b
    b_dec = sh.n_layers * B * min(sh.budget_pages, -(-seq_len // sh.page)) \
        * sh.page * sh.width * 2
    return {"workload": f"c3: MLA, {sh.n_layers} layers, {sh.n_heads} heads, latent "
                        f"{sh.width}, page {sh.page}, batch {B}, ctx {seq_len - 1}, "
                        f"budget {sh.budget_pages} pages incl. {sh.sink_pages} sink + "
                        f"{sh.window_pages} recent",
            "l2_policy": "inputs larger than L2 "
                         f"({(b_score + b_dec) / 1e9:.2f} GB per step)"}


def reference_available() -> bool:
    return os.path.exists(os.path.join(ROOT, "oracle", "_ref", "locks_ref",
                                       "selection", "rki4_score_torch.py"))


def workload_config(args, sh, seq_len):
    """The `config` object both arms print for a single-sequence workload."""
    A = min(sh.budget_pages, max(-(-seq_len // sh.page) - sh.window_pages
                                 - sh.sink_pages, 0)) + sh.sink_pages \
        + sh.window_pages
    b_score, b_dec, _, _, _ = algo_bytes(sh, seq_len)
    return {"workload": f"{args.workload_name}: {sh.n_layers} layers, "
                        f"{sh.n_kv * sh.G}q/{sh.n_kv}kv, d{sh.d}, page {sh.page}, "
                        f"bs1 per GPU, ctx {seq_len - 1}, budget "
                        f"{sh.budget_pages}+{sh.sink_pages} sink+"
                        f"{sh.window_pages} recent = {A} pages attended",
            "l2_policy": "inputs larger than L2 "
                         f"({(b_score + b_dec) / 1e9:.2f} GB touched per step)",
            "sharding": "whole sequences per GPU, no collective"}


def run_reference(args, sh, seq_len):
    """`--impl reference`: the reference's CPU implementation of the path on the
    host cores.  A step is a bounded sample (see RefArm / CpuArm); `ms_per_step`
    is the measured time of that sample, `value` the tokens/s of the whole
    workload it implies (sample time x layer ratio)."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if isinstance(seq_len, (list, tuple)):
        seq_len = sorted(seq_len)[len(seq_len) // 2]       # ragged: median length
    if reference_available():
        arm, kind = RefArm(sh, seq_len, layers=1), "reference"
        scale = sh.n_layers / arm.layers
        full = lambda t: t * scale
    else:
        arm, kind = CpuArm(sh, seq_len), "port"
        full = lambda t: t                 # CpuArm.step already returns full-job s
        arm_step = arm.step
        # the sample's own wall time, for ms_per_step
        def timed_step():
            t0 = time.perf_counter()
            v = arm_step()
            return time.perf_counter() - t0, v
    for _ in range(args.warmup):
        arm.step()
    samples, fulls = [], []
    for _ in range(args.steps):
        if kind == "reference":
            t = arm.step()
            samples.append(t)
            fulls.append(full(t))
        else:
            t, v = timed_step()
            samples.append(t)
            fulls.append(v)
    tpot = float(np.mean(fulls))
    ms_sample = float(np.mean(samples)) * 1e3
    return {
        "impl": "reference", "metric": "sparse_decode_tokens_per_s",
        "value": 1.0 / tpot, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_sample, "tpot_ms": tpot * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, sh, seq_len),
        "cpu_baseline": {"value": 1.0 / tpot, "unit": "tokens/s",
                         "cores": cores, "kind": kind, "sample": arm.sample,
                         "tpot_ms": tpot * 1e3},
        "e2e": {"value": 1.0 / tpot, "unit": "tokens/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


# --------------------------------------------------------------------------- #
# GPU arm                                                                      #
# --------------------------------------------------------------------------- #
def make_device_case(sh, seq_len, dev, seed, return_needles=False, extra_pages=4,
                     n_slabs=None):
    """Paged caches for one sequence (or a ragged batch: a list of lengths),
    generated on the device layer by layer (the full-size cache does not fit a
    CPU round trip).  All sequences share one block pool; block ids are a seeded
    permutation.  ``n_slabs``: generate only that many distinct layer caches
    (the caller cycles its layer launches over them); q is still per layer."""
    from locks import synth
    page = sh.page
    lens = list(seq_len) if isinstance(seq_len, (list, tuple)) else [seq_len]
    npgs = [-(-sl // page) for sl in lens]
    # every sequence also owns `extra_pages` blocks for the tokens it will
    # decode (the block-table entries after its last page)
    NB = sum(npgs) + extra_pages * len(lens) + 3
    g = torch.Generator().manual_seed(seed * 7 + 3)
    perm = torch.randperm(NB, generator=g)
    bt_cpu = torch.zeros(len(lens), max(npgs) + extra_pages, dtype=torch.int32)
    o = 0
    for r, n in enumerate(npgs):
        bt_cpu[r, :n + extra_pages] = perm[o:o + n + extra_pages].to(torch.int32)
        o += n + extra_pages
    bt = bt_cpu.contiguous().to(dev)
    caches, qs, needles = [], [], []
    for l in range(n_slabs or sh.n_layers):
        kvc = torch.zeros(NB, 2, page, sh.n_kv, sh.d, device=dev,
                          dtype=torch.bfloat16)
        ql, ndl = [], []
        for r, sl in enumerate(lens):
            K, V, q, nd = synth.gqa_tokens(seed, l, r, sl, sh, dev)
            pad = npgs[r] * page - sl
            if pad:
                z = torch.zeros(pad, sh.n_kv, sh.d, device=dev, dtype=torch.bfloat16)
                K, V = torch.cat([K, z]), torch.cat([V, z])
            blocks = bt[r, :npgs[r]].long()
            kvc[blocks, 0] = K.view(npgs[r], page, sh.n_kv, sh.d)
            kvc[blocks, 1] = V.view(npgs[r], page, sh.n_kv, sh.d)
            del K, V
            ql.append(q)
            ndl.append(nd)
        needles.append(ndl[0] if len(lens) == 1 else ndl)
        caches.append(kvc)
        qs.append(torch.stack(ql))
    if n_slabs:
        qs = [qs[l % n_slabs] for l in range(sh.n_layers)]
    sl_t = torch.tensor(lens, dtype=torch.int32, device=dev)
    if return_needles:
        return caches, torch.stack(qs), bt, sl_t, needles
    return caches, torch.stack(qs), bt, sl_t


def timed(fn, iters, stream=None):
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters          # ms per call


def run_gpu(args, sh, seq_len):
    import torch.distributed as dist
    from locks import LocksConfig, _cabi
    from locks.attention import DenseDecodeBuffers, dense_paged_decode
    from locks.hotpath import HotPath
    from locks.selection import rki4_score_only, rki4_select_only
    from locks.attention import (sparse_paged_decode_batched,
                                 sparse_paged_decode_fused)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)

    # ---- set-up (untimed): caches, summaries, page parameters -----------------
    caches, q, bt, sl = make_device_case(sh, seq_len, dev, seed=1234 + rank)
    cfg = LocksConfig(budget_pages=sh.budget_pages, sink_pages=sh.sink_pages,
                      window_pages=sh.window_pages)
    hp = HotPath(caches, bt, sl, n_kv=sh.n_kv, G=sh.G,
                 scale=1.0 / math.sqrt(sh.d), cfg=cfg)
    t_build = timed(lambda: hp.build_all(), 1)
    hp.derive()
    hp.q.copy_(q)
    hp.build_tail()                                # first call loads kernels
    t_tail = timed(lambda: hp.build_tail(), 10)
    hp.capture()
    torch.cuda.synchronize()
    hp.st.check_status()

    # ---- timed region: K graph replays ---------------------------------------
    for _ in range(max(args.warmup, 3)):
        hp.step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        hp.step()
    e1.record()
    torch.cuda.synchronize()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
        dist.barrier()
    ms_step = ms_total / args.steps
    hp.st.check_status()

    # ---- per-stage kernel times: one CUDA graph per stage over all layers, so
    # that host launch overhead is not part of the number ------------------------
    st, R = hp.st, hp.n_req
    L = sh.n_layers
    it = max(args.steps // 4, 8)

    def stage_graph(fn):
        for l in range(L):
            fn(l)                                  # warm-up outside capture
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for l in range(L):
                fn(l)
        return g

    g_score = stage_graph(lambda l: rki4_score_only(
        st, l, hp.q[l, :R], bt, sl, R, hp.scale))
    g_select = stage_graph(lambda l: rki4_select_only(st, R, has_hmax=False))
    g_decode = stage_graph(lambda l: sparse_paged_decode_fused(
        hp.q[l, :R], caches[l], bt, sl, st, hp.out[l], hp.vsources[l],
        scale=hp.scale))
    g_split = stage_graph(lambda l: sparse_paged_decode_batched(
        hp.q[l, :R], caches[l], bt, sl, st, hp.out[l], hp.vsources[l],
        scale=hp.scale))
    ms_score = timed(g_score.replay, it) / L
    ms_select = timed(g_select.replay, it) / L
    ms_decode = timed(g_decode.replay, it) / L
    ms_split = timed(g_split.replay, it) / L
    st.hmax.zero_() if st.hmax is not None else None
    hp.step()                       # leave a consistent selection behind

    # ---- KV-write neighbour: rotate + store one new token per layer; in the
    # second graph the token completes a page, so the page's summaries are built
    # in the same launch (a spare block of the pool takes the writes) ------------
    from locks.attention import rope_and_cache
    NBc = int(caches[0].shape[0])
    used = torch.zeros(NBc, dtype=torch.bool)
    used[bt.cpu().long().flatten()] = True
    spare = int((~used).nonzero()[0])
    kw_key = torch.randn(R, sh.n_kv, sh.d, device=dev).to(torch.bfloat16)
    kw_val = torch.randn(R, sh.n_kv, sh.d, device=dev).to(torch.bfloat16)
    ang = torch.rand(64, sh.d // 2, device=dev) * 6.28
    kw_cs = torch.cat([ang.cos(), ang.sin()], 1).to(torch.bfloat16)
    kw_pos = torch.full((R,), 17, dtype=torch.int64, device=dev)
    slot_mid = torch.full((R,), spare * sh.page + 3, dtype=torch.int64, device=dev)
    slot_end = torch.full((R,), spare * sh.page + sh.page - 1, dtype=torch.int64,
                          device=dev)
    g_kw = stage_graph(lambda l: rope_and_cache(kw_key, kw_val, caches[l], slot_mid,
                                                kw_pos, kw_cs, st=st, lidx=l))
    g_kwb = stage_graph(lambda l: rope_and_cache(kw_key, kw_val, caches[l], slot_end,
                                                 kw_pos, kw_cs, st=st, lidx=l))
    ms_kw = timed(g_kw.replay, it) / L
    ms_kwb = timed(g_kwb.replay, it) / L
    from locks.selection import rki4_build_slots
    ms_slots = timed(lambda: rki4_build_slots(st, hp.K_layers, slot_end), 10)

    # ---- decode loop: the step as a model runs it -- the new token's K/V are
    # rotated and written, page parameters follow the grown lengths, and the
    # summaries of pages completed by the PREVIOUS step are built on a forked
    # branch while this step's layers run (the page stays inside the recent
    # window for many steps, so nothing waits for its summary) -----------------
    loop = None
    try:
        KS = 48                                     # 3 page completions per sequence
        lens0 = hp.seq_lens.clone()
        P = int(lens0.max().item()) + KS + 2
        ang = torch.arange(P, device=dev, dtype=torch.float32)[:, None] * \
            (500000.0 ** (-torch.arange(sh.d // 2, device=dev) / (sh.d // 2)))[None]
        cs_tab = torch.cat([ang.cos(), ang.sin()], 1).to(torch.bfloat16)

        def run_loop(fuse_write):
            hp.seq_lens.copy_(lens0)
            hp.enable_append(cs_tab, fuse_write=fuse_write)
            hp.new_k.copy_(torch.randn(L, R, sh.n_kv, sh.d, device=dev))
            hp.new_v.copy_(torch.randn(L, R, sh.n_kv, sh.d, device=dev))
            for _ in range(4):                       # capture + 3 warm replays
                hp.append_step()
            ms = timed(hp.append_step, KS - 4)
            torch.cuda.synchronize()
            st.check_status()
            return ms

        ms_sep = run_loop(False)
        hp.flush_builds()
        ms_loop = run_loop(True)
        # the pages completed on the way have summaries in every layer
        done = []
        for r in range(R):
            a, b = int(lens0[r].item()) // sh.page, int(hp.seq_lens[r].item() - 1) // sh.page
            done += [int(hp.block_table[r, pg].item()) for pg in range(a, b)]
        built = all(not bool(torch.isnan(st.pp_tag[:, blk].float()).any())
                    for blk in done)
        loop = {"ms_per_step": ms_loop, "ms_per_step_separate_kv_write": ms_sep,
                "steps": KS, "pages_completed": len(done),
                "summaries_of_completed_pages_built": built,
                "note": "graph of: slot/position update, derive, per layer score + "
                        "select (its launch also rotates and stores the new token's "
                        "K/V) + decode, slot-driven summary build of the previous "
                        "step's completed pages on a forked branch"}
        hp.flush_builds()
        hp.seq_lens.copy_(lens0)
        hp.derive()
    except Exception as e:       # an optional measurement must not sink the bench line
        loop = {"failed": f"{type(e).__name__}: {e}"}

    # ---- dense full-KV baseline on the same caches ----------------------------
    dsplit = max(1, min(512, (4 * 148) // (sh.n_kv * R)))
    dbuf = DenseDecodeBuffers(dev, R, sh.n_kv, sh.G, sh.d, dsplit)
    dout = torch.empty_like(hp.out[0])
    g_dense = stage_graph(lambda l: dense_paged_decode(
        hp.q[l, :R], caches[l], bt, sl, dbuf, dout, n_kv=sh.n_kv, G=sh.G,
        scale=hp.scale, status=st.status))
    ms_dense = timed(g_dense.replay, max(it // 4, 3))

    # ---- end to end through the public API with HOST buffers -------------------
    # (HotPath.step_host: pinned host staging in, pinned host buffer out; the
    # copies, the page parameters and the L-layer step are one graph replay)
    hp.enable_host_io()
    hp.host_q.copy_(q.cpu())
    hp.host_seq_lens.copy_(sl.cpu())
    hp.host_block_table.copy_(bt.cpu())
    q_host, sl_host, bt_host, out_host = (hp.host_q, hp.host_seq_lens,
                                          hp.host_block_table, hp.host_out)

    def e2e_step():
        hp.step_host()

    for _ in range(3):
        e2e_step()
    t0 = time.perf_counter()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    h2d = q_host.numel() * 2 + sl_host.numel() * 4 + bt_host.numel() * 4
    d2h = out_host.numel() * 2

    clocks = sampler.stop() if rank == 0 else None

    if rank != 0:
        return None

    # ---- roofline of the dominant kernel (the scorer) --------------------------
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak = float(json.load(open(peaks_path))["hbm_gbs"])
        peak_src = "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = 6650.0, "fallback"
    b_score, b_dec, b_dense, nsh, A = algo_bytes(sh, seq_len)
    score_launch_bytes = b_score / L
    achieved = score_launch_bytes / (ms_score * 1e-3) / 1e9
    step_bytes = b_score + b_dec

    cpu = None
    ragged = isinstance(seq_len, (list, tuple))
    if not args.no_cpu_baseline and world == 1 and not ragged:
        # the reference arm, run as a process of its own on the host cores (its
        # Triton interpreter switch and thread settings stay out of this one)
        try:
            cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference",
                   "--workload", args.workload_name, "--steps", "5", "--warmup",
                   "1"] + (["--ctx", str(args.ctx)] if args.ctx else []) \
                + (["--layers", str(args.layers)] if args.layers else [])
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            ref = json.loads([ln for ln in r.stdout.splitlines()
                              if ln.startswith("{")][-1])
            cpu = ref["cpu_baseline"]
            cpu["sample"] += "; mean of 5"
        except Exception as e:   # the baseline must not sink the GPU number
            cpu = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(),
                   "kind": "port", "sample": f"failed: {type(e).__name__}: {e}"}

    line = {
        "metric": "sparse_decode_tokens_per_s",
        "value": world * R / (ms_step * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "tpot_ms": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, sh, seq_len),
        "clocks": clocks,
        "e2e": {"value": world * R / (ms_e2e * 1e-3), "unit": "tokens/s",
                "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": hp.launches_per_step * args.steps,
        "roofline": {"kernel": "rki4_score_kernel", "bound": "hbm",
                     "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak,
                     # dram__bytes_read + write per (page, kv-head) of the ncu
                     # capture on this shape, scaled by the units of a launch
                     "traffic": (score_traffic_per_unit() or 0) * sh.n_kv * nsh
                     or None,
                     "peak_source": peak_src,
                     "bytes_per_launch": score_launch_bytes,
                     "us_per_launch": ms_score * 1e3},
        "step_roofline": {"algorithmic_bytes": step_bytes,
                          "achieved_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
                          "frac_of_measured_peak":
                              step_bytes / (ms_step * 1e-3) / 1e9 / peak,
                          "frac_of_8tbs": step_bytes / (ms_step * 1e-3) / 8e12},
        "stages_us_per_layer": {"score": ms_score * 1e3,
                                "select": ms_select * 1e3,
                                "decode_fused": ms_decode * 1e3,
                                "decode_split_plus_merge": ms_split * 1e3},
        "dense": {"ms_per_step": ms_dense, "bytes": b_dense,
                  "gbs": b_dense / (ms_dense * 1e-3) / 1e9,
                  "speedup_sparse_over_dense": ms_dense / ms_step},
        "build": {"bulk_ms": t_build, "tail_ms_per_finalize": t_tail,
                  "tail_ms_amortised_per_step": t_tail / sh.page},
        "kv_write": {"us_per_layer": ms_kw * 1e3,
                     "us_per_layer_completing_a_page": ms_kwb * 1e3,
                     "slot_driven_build_all_layers_us": ms_slots * 1e3,
                     "note": "rotate K + store K,V (+ summary build of the "
                             "completed page in the same launch); or one "
                             "slot-driven build launch per step for all layers"},
        "decode_loop": loop,
        "cpu_baseline": cpu,
    }
    return line


def _peak():
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return float(json.load(open(peaks_path))["hbm_gbs"]), \
            "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback"


def _timed_steps(step, steps, warmup, dev, world):
    """K replays bracketed by a barrier and a device synchronise on both sides;
    ms per step, max over ranks."""
    import torch.distributed as dist
    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def cp_record(args, dev, rank, world, layers=8):
    """ONE sequence of the 1M-token shape (40 layers as written; `layers` of them
    are run) whose pages are split over the ranks by contiguous ranges: strong
    scaling.  Three launches per layer on every rank (score, select, decode);
    the three per-layer exchanges happen inside the selector and the decode
    kernel over NVLink peer memory.  Reported: us per layer (max over ranks),
    the same with the exchanges switched off (every rank on its own range with
    no peer: the streaming work alone), their difference (= what the three
    exchanges cost), and the earlier arrangement with one exchange kernel per
    exchange between the single-GPU kernels."""
    import dataclasses
    from locks import LocksConfig, synth
    from locks.cp_hotpath import ContextParallelHotPath, check_against_single_gpu
    from locks.parallel import partition_pages
    sh = dataclasses.replace(synth.CONFIG4, n_layers=layers)
    seq_len = 1048576 + 1
    npg = -(-seq_len // sh.page)
    p0, p1 = partition_pages(npg, world)[rank]
    caches, q, bt = synth.make_gqa_shard(1234, sh, seq_len, p0, p1, device=dev)
    cfg = LocksConfig(budget_pages=sh.budget_pages, sink_pages=sh.sink_pages,
                      window_pages=sh.window_pages)
    scale = 1.0 / math.sqrt(sh.d)
    rec = {"workload": f"c4 context parallel: {layers} of 40 layers, "
                       f"{sh.n_kv * sh.G}q/{sh.n_kv}kv, ONE sequence of ctx "
                       f"{seq_len - 1} split over {world} GPU(s) by contiguous "
                       f"page ranges, budget {sh.budget_pages}+{sh.sink_pages} "
                       f"sink+{sh.window_pages} recent",
           "scaling": "strong", "n_gpus": world, "layers": layers}

    def run(transport, solo=False):
        cp = ContextParallelHotPath(caches, bt, seq_len=seq_len, p0=p0, p1=p1,
                                    n_kv=sh.n_kv, G=sh.G, scale=scale, cfg=cfg,
                                    transport=transport, loopback=solo,
                                    group=None)
        if solo:          # every rank alone on its range: no peer in the links
            for d in cp._links:
                d.world, d.rank = 1, 0
                d.regions[0] = cp.link._peers[cp.link.rank]
        return cp
    cp = run("fused")
    t_build = timed(lambda: cp.build_all(), 1)
    cp.q.copy_(q)
    cp.capture()
    ms = _timed_steps(cp.step, args.steps, args.warmup, dev, world)
    status = int(cp.st.status.item())
    rec.update({"us_per_layer": ms * 1e3 / layers, "ms_per_step": ms,
                "launches_per_layer": 3, "status_word": status,
                "path": ("in-kernel exchanges over NVLink peer memory" if world > 1
                         else "one rank: the single-GPU kernels, nothing to exchange"),
                "build_bulk_ms": t_build})
    recs = cp.st.pp_rec
    # the exchange code with no peer: same kernels, links to the rank itself
    solo = run("fused", solo=True)
    solo.st.pp_rec.copy_(recs)
    solo.q.copy_(q)
    solo.capture()
    ms_solo = _timed_steps(solo.step, args.steps, args.warmup, dev, world)
    rec["us_per_layer_no_exchange"] = ms_solo * 1e3 / layers
    rec["exchange_cost_us_per_layer"] = (ms - ms_solo) * 1e3 / layers
    del solo
    if world > 1:
        old = run("peer")
        old.st.pp_rec.copy_(recs)
        old.q.copy_(q)
        old.capture()
        ms_old = _timed_steps(old.step, args.steps, args.warmup, dev, world)
        rec["us_per_layer_separate_exchange_kernels"] = ms_old * 1e3 / layers
        rec["status_word"] |= int(old.st.status.item())
        del old
    b_score, b_dec, _, _, A = algo_bytes(sh, seq_len)
    peak, _ = _peak()
    rec["step_roofline"] = {
        "algorithmic_bytes": b_score + b_dec,
        "achieved_gbs": (b_score + b_dec) / (ms * 1e-3) / 1e9,
        "frac_of_measured_peak_x_gpus":
            (b_score + b_dec) / (ms * 1e-3) / 1e9 / (peak * world)}
    rec["gpu_launches_per_step"] = 3 * layers + 1
    del cp, caches
    torch.cuda.empty_cache()
    # parity of a small context-parallel case against the single-GPU path,
    # inside this run, on these ranks
    if world > 1:
        ok, err, msgs = check_against_single_gpu(seq_len=40005, n_layers=3)
        rec["cp_parity"] = "ok" if ok else "FAILED: " + "; ".join(msgs)
        rec["cp_parity_max_abs_err"] = err
    else:
        rec["cp_parity"] = "n/a (one rank: checked by the single-GPU tests)"
    return rec


def c2_record(args, dev, rank, world, full_line=False):
    """The continuous-batching workload as the benchmark states it: 64 sequences
    with seeded log-uniform context lengths in [4096, 262144], one page budget
    per sequence from {32, 64, 128, 256}, block tables a random permutation of
    the pool, 32 layers.  Sequences are dealt to the ranks by their step bytes
    (no data-path collective).  The 32 layer launches walk over a few distinct
    layer slabs (each far larger than L2) so that the pool stays within the
    150 GB the workload names."""
    import dataclasses
    import torch.distributed as dist
    from locks import LocksConfig, synth
    from locks.hotpath import HotPath
    from locks.parallel import shard_sequences
    from locks.selection import rki4_score_only
    sh = synth.CONFIG1
    ctx, budgets = c2_draw()
    lens = [c + 1 for c in ctx]
    mine = shard_sequences(lens, budgets, world, sh.sink_pages,
                           sh.window_pages)[rank]
    my_lens = [lens[i] for i in mine]
    my_budgets = [budgets[i] for i in mine]
    tok = sum(my_lens)
    slab_bytes = tok * sh.n_kv * sh.d * 2 * 2 * 1.12
    free, _ = torch.cuda.mem_get_info()
    n_slabs = int(max(1, min(8, (0.80 * free) // slab_bytes)))
    if world > 1:
        t = torch.tensor([n_slabs], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        n_slabs = int(t.item())
    L = sh.n_layers
    caches, q, bt, sl = make_device_case(sh, my_lens, dev, seed=4321 + rank,
                                         n_slabs=n_slabs)
    cfg = LocksConfig(budget_pages=max(budgets), sink_pages=sh.sink_pages,
                      window_pages=sh.window_pages)
    hp = HotPath(caches, bt, sl, n_kv=sh.n_kv, G=sh.G, scale=1.0 / math.sqrt(sh.d),
                 cfg=cfg, budget_pages_req=my_budgets, launch_layers=L)
    t_build = timed(lambda: hp.build_all(), 1)
    hp.derive()
    hp.q.copy_(q)
    hp.capture()
    torch.cuda.synchronize()
    hp.st.check_status()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0 and full_line:
        sampler.start()
    ms = _timed_steps(hp.step, args.steps, args.warmup, dev, world)
    hp.st.check_status()
    clocks = sampler.stop() if (rank == 0 and full_line) else None
    # scorer alone (dominant kernel), graph of the L launches
    st, R = hp.st, hp.n_req
    for l in range(L):
        rki4_score_only(st, l % n_slabs, hp.q[l, :R], bt, sl, R, hp.scale)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for l in range(L):
            rki4_score_only(st, l % n_slabs, hp.q[l, :R], bt, sl, R, hp.scale)
    ms_score = timed(g.replay, max(args.steps // 4, 8)) / L
    st.hmax.zero_()
    # the other two stages the same way (the selector from the scores the last
    # scorer launch left, sweeping the maxima itself)
    from locks.attention import sparse_paged_decode_fused
    from locks.selection import rki4_select_only

    def stage_ms(fn):
        for l in range(L):
            fn(l)
        torch.cuda.synchronize()
        gs = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gs):
            for l in range(L):
                fn(l)
        return timed(gs.replay, max(args.steps // 4, 8)) / L

    ms_sel = stage_ms(lambda l: rki4_select_only(st, R, has_hmax=False))
    ms_dec = stage_ms(lambda l: sparse_paged_decode_fused(
        hp.q[l, :R], caches[l % n_slabs], bt, sl, st, hp.out[l],
        hp.vsources[l % n_slabs], scale=hp.scale))
    hp.step()                       # leave a consistent selection behind
    b_score, b_dec, b_dense, nsh, _ = algo_bytes(sh, my_lens, my_budgets)
    tot = torch.tensor([float(b_score), float(b_dec), float(tok), float(len(mine)),
                        ms_score, float(b_score + b_dec)], device=dev,
                       dtype=torch.float64)
    mx = tot.clone()
    if world > 1:
        dist.all_reduce(tot)
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    peak, peak_src = _peak()
    all_score, all_dec = float(tot[0]), float(tot[1])
    rec = {
        "workload": f"c2: {len(lens)} sequences, ctx {min(ctx)}..{max(ctx)} "
                    f"(log-uniform, seeded), per-sequence budget_pages from "
                    f"{{32,64,128,256}} + {sh.sink_pages} sink + "
                    f"{sh.window_pages} recent, {L} layers cycling over "
                    f"{n_slabs} distinct layer slabs, permuted block tables, "
                    f"pool {n_slabs * slab_bytes * world / 1.12 / 1e9:.0f} GB",
        "scaling": "strong (the same 64 sequences at every N)",
        "n_gpus": world, "sequences_on_rank0": len(mine),
        "tokens_per_s": len(lens) / (ms * 1e-3), "ms_per_step": ms,
        "sharding": "whole sequences per GPU by step bytes "
                    "(locks.parallel.shard_sequences), no collective",
        "step_roofline": {
            "algorithmic_bytes": all_score + all_dec,
            "achieved_gbs": (all_score + all_dec) / (ms * 1e-3) / 1e9,
            "frac_of_measured_peak_x_gpus":
                (all_score + all_dec) / (ms * 1e-3) / 1e9 / (peak * world)},
        "roofline": {"kernel": "rki4_score_kernel", "bound": "hbm",
                     "achieved": b_score / L / (ms_score * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s",
                     "frac": b_score / L / (ms_score * 1e-3) / 1e9 / peak,
                     "traffic": (score_traffic_per_unit() or 0) * sh.n_kv * nsh
                     or None,
                     "peak_source": peak_src, "us_per_launch": ms_score * 1e3,
                     "note": "rank 0's launch"},
        "stages_us_per_layer": {"score": ms_score * 1e3, "select": ms_sel * 1e3,
                                "decode_fused": ms_dec * 1e3,
                                "decode_gbs": b_dec / L / (ms_dec * 1e-3) / 1e9,
                                "note": "rank 0's launches"},
        "load_balance": {"max_rank_bytes": float(mx[5]),
                         "mean_rank_bytes": (all_score + all_dec) / world},
        "gpu_launches_per_step": hp.launches_per_step,
        "build_bulk_ms": t_build,
    }
    if full_line:
        rec["_clocks"] = clocks
        rec["_hp"] = hp
        rec["_case"] = (my_lens, my_budgets, sh)
    else:
        del hp, caches
        torch.cuda.empty_cache()
    return rec


def run_gpu_mla(args, seq_len):
    """Workload c3: MLA decode, DeepSeek-V2-Lite shape (27 layers, 16 heads, one
    latent KV head of 512 + 64 rope dims, page 16, batch 8, 128K tokens each,
    budget 128 pages including 1 sink + 10 recent)."""
    import dataclasses
    from locks import synth
    from locks.selection import mla_select as ms

    sh = synth.CONFIG3
    if args.layers:
        sh = dataclasses.replace(sh, n_layers=args.layers)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B = 8
    case = synth.make_mla_case(77, sh, [seq_len] * B, device=dev)
    L, W = sh.n_layers, sh.width
    MP = int(case.block_table.shape[1])
    NB = int(case.caches[0].shape[0])

    def state(budget):
        st = ms.MlaState(dev, num_layers=L, num_blocks=NB, max_rows=B, max_pages=MP,
                         budget_pages=budget, sink_pages=sh.sink_pages,
                         window_pages=sh.window_pages)
        ms.mla_derive(st, case.seq_lens, B)
        if "LOCKS_MLA_TC" in os.environ:       # A/B switch; default: by tile count
            st.tensor_core = os.environ["LOCKS_MLA_TC"] != "0"
        return st
    st = state(sh.budget_pages)
    t_build = timed(lambda: ms.build_prompt_factors(st, case.caches, case.block_table,
                                                    case.seq_lens), 1)
    dense = state(MP)                      # budget >= pages: every page is kept
    dense.n_cache.copy_(st.n_cache)
    out = torch.zeros(L, B, sh.n_heads, sh.kv_lora_rank, device=dev,
                      dtype=torch.bfloat16)
    lse = torch.zeros(L, B, sh.n_heads, device=dev, dtype=torch.float32)
    scale = case.scale

    def layers():
        for l in range(L):
            ms.mla_forward(st, l, case.q[l], case.caches[l], case.block_table,
                           case.seq_lens, out[l], lse[l], scale)

    def graph_of(fn):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g
    g_step = graph_of(layers)
    for _ in range(max(args.warmup, 3)):
        g_step.replay()
    sampler = ClockSampler(0)
    sampler.start()
    ms_step = timed(g_step.replay, args.steps)
    it = max(args.steps // 4, 8)
    g_score = graph_of(lambda: [ms.mla_page_score(st, l, case.q[l], case.caches[l],
                                                  case.block_table, B, scale)
                                for l in range(L)])
    g_sel = graph_of(lambda: [ms.mla_select_pages(st, B) for l in range(L)])
    g_dec = graph_of(lambda: [ms.mla_decode(st, case.q[l], case.caches[l],
                                            case.block_table, case.seq_lens, out[l],
                                            lse[l], B, scale) for l in range(L)])
    ms_score, ms_sel, ms_dec = (timed(g.replay, it) / L for g in (g_score, g_sel, g_dec))
    ms.mla_select_pages(dense, B)
    g_dense = graph_of(lambda: [ms.mla_decode(dense, case.q[l], case.caches[l],
                                              case.block_table, case.seq_lens,
                                              out[l], lse[l], B, scale)
                                for l in range(L)])
    ms_dense = timed(g_dense.replay, max(it // 4, 3))
    # end to end: q from pinned host memory in, o and lse back
    q_host = case.q.cpu().pin_memory()
    o_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def e2e_step():
        case.q.copy_(q_host, non_blocking=True)
        g_step.replay()
        o_host.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    for _ in range(3):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop()
    st.check_status()
    n_cached = seq_len // sh.page
    npg = -(-seq_len // sh.page)
    rec_b = 8448 + sh.page * sh.rope_dim * 2          # factors + rope keys per page
    page_b = sh.page * W * 2
    b_score = L * B * n_cached * rec_b
    b_dec = L * B * min(sh.budget_pages, npg) * page_b
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    peak = (float(json.load(open(peaks_path))["hbm_gbs"])
            if os.path.exists(peaks_path) else 6650.0)
    ach = (b_score / L) / (ms_score * 1e-3) / 1e9
    cpu = None
    if not args.no_cpu_baseline:
        try:
            cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference",
                   "--workload", "c3", "--steps", "3", "--warmup", "1"] \
                + (["--ctx", str(args.ctx)] if args.ctx else []) \
                + (["--layers", str(args.layers)] if args.layers else [])
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            cpu = json.loads([ln for ln in r.stdout.splitlines()
                              if ln.startswith("{")][-1]).get("cpu_baseline")
        except Exception as e:
            cpu = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(),
                   "kind": "reference", "sample": f"failed: {type(e).__name__}: {e}"}
    return {
        "metric": "sparse_decode_tokens_per_s", "value": B / (ms_step * 1e-3),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "tpot_ms": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": mla_config(sh, B, seq_len),
        "clocks": clocks,
        "e2e": {"value": B / (ms_e2e * 1e-3), "unit": "tokens/s",
                "ms_per_step": ms_e2e, "h2d_bytes_per_step": q_host.numel() * 2,
                "d2h_bytes_per_step": o_host.numel() * 2},
        "gpu_launches": 3 * L * args.steps,
        "roofline": {"kernel": "mla_score_kernel", "bound": "hbm", "achieved": ach,
                     "peak": peak, "unit": "GB/s", "frac": ach / peak,
                     "traffic": None,
                     "bytes_per_launch": b_score / L,
                     "us_per_launch": ms_score * 1e3},
        "step_roofline": {"algorithmic_bytes": b_score + b_dec,
                          "achieved_gbs": (b_score + b_dec) / (ms_step * 1e-3) / 1e9,
                          "frac_of_measured_peak":
                              (b_score + b_dec) / (ms_step * 1e-3) / 1e9 / peak},
        "stages_us_per_layer": {"score": ms_score * 1e3, "select": ms_sel * 1e3,
                                "decode": ms_dec * 1e3},
        "dense": {"ms_per_step": ms_dense, "bytes": L * B * npg * page_b,
                  "gbs": L * B * npg * page_b / (ms_dense * 1e-3) / 1e9,
                  "speedup_sparse_over_dense": ms_dense / ms_step},
        "build": {"factors_ms": t_build},
        "cpu_baseline": cpu,
    }


def c2_line(args, dev, rank, world):
    """`--workload c2`: the ragged batch as a bench line of its own."""
    rec = c2_record(args, dev, rank, world, full_line=True)
    hp, clocks = rec.pop("_hp"), rec.pop("_clocks")
    my_lens, my_budgets, sh = rec.pop("_case")
    # end to end with host buffers: q, lengths and block table in, outputs back
    hp.enable_host_io()
    hp.host_q.copy_(hp.q[:, :hp.n_req].cpu())
    hp.host_seq_lens.copy_(hp.seq_lens.cpu())
    hp.host_block_table.copy_(hp.block_table.cpu())
    for _ in range(3):
        hp.step_host()
    ms_e2e = _timed_steps(hp.step_host, args.steps, 0, dev, world)
    h2d = hp.host_q.numel() * 2 + hp.host_seq_lens.numel() * 4 + \
        hp.host_block_table.numel() * 4
    d2h = hp.host_out.numel() * 2
    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        # the oracle on ONE sampled sequence (the median length) with its own
        # budget, one layer, scaled by the batch's share of step bytes
        try:
            import dataclasses
            order = sorted(range(len(my_lens)), key=lambda i: my_lens[i])
            i = order[len(order) // 2]
            shs = dataclasses.replace(sh, budget_pages=my_budgets[i])
            if reference_available():      # the reference's own CPU code
                arm, kind = RefArm(shs, my_lens[i], layers=1), "reference"
                arm.step()
                t_one = float(np.mean([arm.step() for _ in range(3)])) * sh.n_layers
            else:
                arm, kind = CpuArm(shs, my_lens[i]), "port"
                arm.step()
                t_one = float(np.mean([arm.step() for _ in range(3)]))
            bs, bd, _, _, _ = algo_bytes(shs, my_lens[i])
            share = (bs + bd) / rec["step_roofline"]["algorithmic_bytes"]
            cpu = {"value": 64 / (t_one / share), "unit": "tokens/s",
                   "cores": os.cpu_count(), "kind": kind,
                   "sample": f"sequence of {my_lens[i] - 1} tokens, budget "
                             f"{my_budgets[i]}: " + arm.sample +
                             f"; scaled by its {share:.4f} share of the batch's "
                             "step bytes"}
        except Exception as e:
            cpu = {"value": None, "unit": "tokens/s", "cores": os.cpu_count(),
                   "kind": "port", "sample": f"failed: {type(e).__name__}: {e}"}
    if rank != 0:
        return None
    ms = rec["ms_per_step"]
    return {
        "metric": "sparse_decode_tokens_per_s", "value": rec["tokens_per_s"],
        "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "tpot_ms": ms,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": rec["workload"],
                   "l2_policy": "inputs larger than L2",
                   "sharding": rec["sharding"]},
        "clocks": clocks,
        "e2e": {"value": 64 / (ms_e2e * 1e-3), "unit": "tokens/s",
                "ms_per_step": ms_e2e, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h},
        "gpu_launches": rec["gpu_launches_per_step"] * args.steps,
        "roofline": rec["roofline"], "step_roofline": rec["step_roofline"],
        "stages_us_per_layer": rec["stages_us_per_layer"],
        "load_balance": rec["load_balance"],
        "build": {"bulk_ms": rec["build_bulk_ms"]},
        "cpu_baseline": cpu,
    }


def vtier_line(args, sh, seq_len, dev):
    """Config-1 geometry on a few layers with V behind the two-level tier:
    resident V, tier with every selected block staged (steady state), tier with
    nothing staged (every page read in place over the host link), and the cold
    promotion (copy-engine runs) timed by itself."""
    import dataclasses
    from locks import LocksConfig
    from locks.hotpath import HotPath
    L = args.layers or 16
    sh = dataclasses.replace(sh, n_layers=L)
    caches, qs, bt, sl = make_device_case(sh, seq_len, dev, seed=1)
    cfg = LocksConfig(budget_pages=sh.budget_pages, sink_pages=sh.sink_pages,
                      window_pages=sh.window_pages)

    def mk():
        hp = HotPath(caches, bt, sl, n_kv=sh.n_kv, G=sh.G, scale=sh.d ** -0.5, cfg=cfg)
        hp.build_all(); hp.derive()
        hp.q[:, :1].copy_(qs)
        return hp

    def ms(step, n):
        for _ in range(max(args.warmup, 3)):
            step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            step()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    n = args.steps
    hp = mk()
    resident_ms = ms(hp.step, n)
    want = hp.out.clone()
    # nothing staged, nothing promoted: every V page crosses the host link
    cold = mk()
    cold.enable_vtier(8, max_promote_blocks=0)
    inplace_ms = ms(cold.step, n)
    same_inplace = bool(torch.equal(cold.out, want))
    del cold
    hot = mk()
    tier = hot.enable_vtier(2048)
    hot.step()                                   # notes the misses of the cold step
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    tier.promote(block=True); tier.wait_all(); torch.cuda.synchronize()
    cold_promote_s = time.perf_counter() - t0
    promoted = tier.stats["promoted_blocks"]
    runs = tier.stats["copy_runs"]
    blk_bytes = tier.block_elems * 2
    staged_ms = ms(hot.step, n)
    same_staged = bool(torch.equal(hot.out, want))
    tier.promote(block=True); tier.wait_all(); tier.check()
    return {
        "metric": "sparse_decode_tokens_per_s", "value": 1e3 / staged_ms,
        "unit": "tokens/s", "n_gpus": 1, "steps": n, "warmup": max(args.warmup, 3),
        "ms_per_step": staged_ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"c1 geometry, {L} layers, ctx {seq_len - 1}, V behind "
                   "the two-level tier (pinned host pool + 2048-block staging "
                   "buffer per layer), step = CUDA-graph replay + host-side "
                   "promotion calls"},
        "gpu_launches": hot.launches_per_step * n,
        "vtier": {"resident_v_ms": resident_ms, "staged_ms": staged_ms,
                  "all_pages_in_place_over_host_link_ms": inplace_ms,
                  "bit_equal_staged": same_staged, "bit_equal_in_place": same_inplace,
                  "cold_promotion": {"blocks": promoted, "copy_runs": runs,
                                     "seconds": cold_promote_s,
                                     "gb_per_s": promoted * blk_bytes / cold_promote_s / 1e9},
                  "steady_state_missed_blocks": tier.last_missed},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", dest="workload_name", default="c1")
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-partitioned", action="store_true",
                    help="skip the c2_sharded and cp records of the default run")
    ap.add_argument("--layers", type=int, default=None,
                    help="override the layer count (quick experiments only)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload_name == "c3":
        if rank == 0:
            fn = run_reference_mla if args.impl == "reference" else run_gpu_mla
            print(json.dumps(fn(args, (args.ctx or 131072) + 1)), flush=True)
        return
    sh, ctx = workload(args.workload_name, args.ctx)
    if args.layers:
        import dataclasses
        sh = dataclasses.replace(sh, n_layers=args.layers)
    seq_len = [c + 1 for c in ctx] if isinstance(ctx, list) else ctx + 1
    if args.impl == "reference":
        if rank != 0:
            return
        print(json.dumps(run_reference(args, sh, seq_len)), flush=True)
        return
    import torch.distributed as dist
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.workload_name == "c1vt":
        line = vtier_line(args, sh, seq_len, dev) \
            if rank == 0 else None
    elif args.workload_name == "c2":
        line = c2_line(args, dev, rank, world)
    elif args.workload_name == "c4cp":
        rec = cp_record(args, dev, rank, world, layers=args.layers or 8)
        line = None
        if rank == 0:
            ms = rec["ms_per_step"]
            line = {"metric": "sparse_decode_tokens_per_s", "value": 1e3 / ms,
                    "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                    "warmup": max(args.warmup, 3), "ms_per_step": ms,
                    "higher_is_better": True, "scaling": "strong",
                    "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": {"workload": rec["workload"]},
                    "gpu_launches": rec["gpu_launches_per_step"] * args.steps,
                    "cp": rec}
    else:
        line = run_gpu(args, sh, seq_len)
        if args.workload_name == "c1" and not args.no_partitioned \
                and not args.ctx and not args.layers:
            import gc
            gc.collect()
            torch.cuda.empty_cache()
            extra = {}
            for name, fn in (("cp", cp_record), ("c2_sharded", c2_record)):
                try:
                    extra[name] = fn(args, dev, rank, world)
                except Exception as e:   # a side record must not sink the line
                    extra[name] = {"failed": f"{type(e).__name__}: {e}"}
                gc.collect()
                torch.cuda.empty_cache()
            if line is not None:
                line.update(extra)
    if line is not None:
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    # leave without tearing the process group and the IPC mappings down
    os._exit(0)


if __name__ == "__main__":
    main()
