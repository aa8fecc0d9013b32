"""V tier on the GPU: V in pinned host memory + a bounded staging buffer in
device memory, promoted between steps by copy-engine transfers.  Whatever is
resident, the decode output must equal the all-resident fused decode BIT FOR BIT
(the reference's equality gate for its tier, ``tier/pool.py:104-116``), and the
residency invariants must hold after every step."""
from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _paths(seed, lens, n_slots):
    from locks import LocksConfig, synth
    from locks.hotpath import HotPath
    sh = synth.GqaShape(n_layers=2, n_kv=8, G=4, d=128, page=16, budget_pages=24,
                        sink_pages=1, window_pages=3, n_needles=4, n_outlier=4)
    case = synth.make_gqa_case(seed, sh, lens, device=DEV)
    caches = case.kv_caches
    cfg = LocksConfig(budget_pages=24, sink_pages=1, window_pages=3)
    mk = lambda: HotPath(caches, case.block_table, case.seq_lens, n_kv=8, G=4,
                         scale=1 / math.sqrt(128), cfg=cfg)
    ref, tiered = mk(), mk()
    for hp in (ref, tiered):
        hp.build_all(); hp.derive()
    tier = tiered.enable_vtier(n_slots, miss_cap=2048)
    return case, caches, ref, tiered, tier


def test_tiered_decode_equals_resident_decode_while_selections_move():
    lens = [3001, 517, 16 * 40 + 5]
    case, caches, ref, tiered, tier = _paths(31, lens, n_slots=300)
    g = torch.Generator(device=DEV).manual_seed(5)
    R = len(lens)
    # the resident V halves of the tiered path must not be what is read
    shadow = [c.clone() for c in caches]
    qs = [torch.randn(ref.q.shape, device=DEV, generator=g).to(torch.bfloat16)
          for _ in range(4)]
    hit_steps = 0
    for step in range(14):
        q = qs[step % 2] if step < 8 else qs[2 + step % 2]     # selections move
        ref.q.copy_(q); tiered.q.copy_(q)
        want = ref.step_eager().clone()
        got = tiered.step_eager().clone()
        torch.cuda.synchronize()
        tiered.st.check_status()
        assert torch.equal(got[:, :R], want[:, :R]), f"step {step}"
        tier.promote(block=True)         # bring this step's misses in, then check
        tier.wait_all()
        tier.check()
        if tier.last_missed == 0:
            hit_steps += 1
    assert tier.stats["promoted_blocks"] > 0
    assert tier.stats["copy_runs"] <= tier.stats["promoted_blocks"]
    assert hit_steps >= 4                # repeated queries end up fully staged
    assert all(torch.equal(a, b) for a, b in zip(caches, shadow))


def test_small_staging_buffer_evicts_and_stays_exact():
    lens = [4000, 2500]
    case, caches, ref, tiered, tier = _paths(32, lens, n_slots=20)
    g = torch.Generator(device=DEV).manual_seed(6)
    R = len(lens)
    for step in range(10):
        q = torch.randn(ref.q.shape, device=DEV, generator=g).to(torch.bfloat16)
        ref.q.copy_(q); tiered.q.copy_(q)
        want = ref.step_eager().clone()
        got = tiered.step_eager().clone()
        torch.cuda.synchronize()
        assert torch.equal(got[:, :R], want[:, :R]), f"step {step}"
        tier.promote(block=True); tier.wait_all(); tier.check()
        for l in range(tier.L):
            assert tier.resident_blocks(l) <= 20
    assert tier.stats["missed_blocks"] > tier.stats["promoted_blocks"] > 20


def test_block_handed_to_another_sequence_is_dropped():
    lens = [3001]
    case, caches, ref, tiered, tier = _paths(33, lens, n_slots=200)
    for _ in range(3):                   # stage what the query selects
        ref.q.copy_(case.q); tiered.q.copy_(case.q)
        ref.step_eager(); tiered.step_eager()
    tier.promote(block=True); tier.wait_all(); tier.check()
    l = 0
    staged = (tier.clock[l].slot_of >= 0).nonzero()[0][:5].tolist()
    assert staged
    # the blocks get new content (another sequence's tokens): engine cache and
    # pool are rewritten by the KV-write path, the tier is told
    for b in staged:
        new_v = torch.randn_like(caches[l][b, 1])
        caches[l][b, 1].copy_(new_v)
        tier.pool[l].plane[b].copy_(new_v)
    tier.invalidate_blocks(staged)
    for _ in range(2):
        want = ref.step_eager().clone()
        got = tiered.step_eager().clone()
        torch.cuda.synchronize()
        assert torch.equal(got[:, :1], want[:, :1])
    tier.promote(block=True); tier.wait_all(); tier.check()


def test_tiered_step_as_a_graph_replay():
    lens = [3001, 900]
    case, caches, ref, tiered, tier = _paths(34, lens, n_slots=128)
    ref.q.copy_(case.q); tiered.q.copy_(case.q)
    want = ref.step().clone()
    for _ in range(3):
        got = tiered.step().clone()
        torch.cuda.synchronize()
        assert torch.equal(got[:, :2], want[:, :2])
    tier.promote(block=True); tier.wait_all(); tier.check()
    assert tier.last_missed == 0 or tier.stats["promoted_blocks"] > 0
