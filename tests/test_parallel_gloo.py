"""Context-parallel exchanges and sequence sharding on CPU ranks (gloo,
world_size 2 and 3).  The kernels are stood in for by the numpy oracle; what is
tested is that the three exchanges reproduce the single-process selection and
attention exactly."""
from __future__ import annotations

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import locks_oracle as orc
from locks import parallel as par


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        n_kv, G, d, n_pages, window, sink, b = 2, 3, 16, 301, 4, 2, 20
        nsh = n_pages - window
        # coarse per-head scores -> many ties, some exactly at the threshold
        S = (np.round(rng.standard_normal((n_kv, G, n_pages)) * 4) / 4).astype(np.float32)
        ranges = par.partition_pages(n_pages, world)
        p0, p1 = ranges[rank]
        # exchange 1: global per-head maxima from local ones
        hi_loc = min(p1, nsh)
        hm = torch.full((n_kv, G), float("-inf"))
        if hi_loc > p0:
            hm = torch.from_numpy(S[:, :, p0:hi_loc].max(-1))
        par.cp_allreduce_max(hm)
        assert np.array_equal(hm.numpy(), S[:, :, :nsh].max(-1))
        # local combine with the global maxima
        loc = np.zeros((n_kv, p1 - p0), np.float32)
        for g in range(G):
            loc = loc + np.exp(S[:, g, p0:p1] - hm.numpy()[:, g:g + 1]).astype(np.float32)
        # exchange 2
        mine = par.cp_select(torch.from_numpy(loc), p0, n_pages, nsh, b, sink)
        # single-process answer
        full = orc.nrm_combine(S[None], [nsh])
        # recompute the local slice exactly as the ranks did (same op order)
        tab, cnt = orc.topb_select(full, [n_pages], [nsh], [b], sink)
        for kh in range(n_kv):
            want = tab[0, kh, :cnt[0, kh]]
            want = want[(want >= p0) & (want < p1)]
            assert np.array_equal(mine[kh].numpy(), want), (rank, kh)
        # exchange 3: partials of the pages each rank attends
        K = rng.standard_normal((n_pages, 4, d)).astype(np.float32)
        V = rng.standard_normal((n_pages, 4, d)).astype(np.float32)
        qv = rng.standard_normal((n_kv * G, d)).astype(np.float32)
        H = n_kv * G
        m = torch.full((1, H), float("-inf")); l = torch.zeros(1, H)
        acc = torch.zeros(1, H, d)
        for kh in range(n_kv):
            pg = mine[kh].numpy()
            if pg.size == 0:
                continue
            k_ = K[pg].reshape(-1, d); v_ = V[pg].reshape(-1, d)
            s = qv[kh * G:(kh + 1) * G] @ k_.T
            mm = s.max(-1); p = np.exp(s - mm[:, None])
            m[0, kh * G:(kh + 1) * G] = torch.from_numpy(mm)
            l[0, kh * G:(kh + 1) * G] = torch.from_numpy(p.sum(-1))
            acc[0, kh * G:(kh + 1) * G] = torch.from_numpy(p @ v_)
        out = par.cp_merge(m, l, acc).numpy()
        for kh in range(n_kv):
            pg = tab[0, kh, :cnt[0, kh]]
            k_ = K[pg].reshape(-1, d); v_ = V[pg].reshape(-1, d)
            s = qv[kh * G:(kh + 1) * G] @ k_.T
            p = np.exp(s - s.max(-1, keepdims=True))
            ref = (p / p.sum(-1, keepdims=True)) @ v_
            np.testing.assert_allclose(out[kh * G:(kh + 1) * G], ref, rtol=2e-5, atol=2e-5)
        q.put((rank, "ok"))
    except Exception as e:  # surface the failure to the parent
        q.put((rank, f"{type(e).__name__}: {e}"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_context_parallel_exchanges(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(30)
    assert all(r[1] == "ok" for r in res), res


def test_partition_and_sharding():
    r = par.partition_pages(65537, 8)
    assert r[0][0] == 0 and r[-1][1] == 65537
    assert all(a[1] == b[0] for a, b in zip(r, r[1:]))
    assert max(b - a for a, b in r) - min(b - a for a, b in r) <= 1
    rng = np.random.default_rng(0)
    lens = np.exp(rng.uniform(np.log(4096), np.log(262144), 64)).astype(int).tolist()
    buds = rng.choice([32, 64, 128, 256], 64).tolist()
    sh = par.shard_sequences(lens, buds, 8)
    assert sorted(sum(sh, [])) == list(range(64))
    cost = [sum(par.step_bytes(lens[i], buds[i], 1, 8) for i in s) for s in sh]
    assert max(cost) <= 1.15 * (sum(cost) / 8)


def test_global_select_tie_rule():
    s = torch.tensor([[3., 1., 1., 1., 2., 1.]])
    p = torch.tensor([[10, 7, 3, 9, 1, 5]])
    keep = par.global_select(s, p, 4)
    # 3, 2, then the two lowest pages among the ties at 1: pages 3 and 5
    assert sorted(p[0][keep[0]].tolist()) == [1, 3, 5, 10]


def test_global_page_params_match_the_oracle_rule():
    """The context-parallel driver derives (n_pages, n_sel_hi, b) of the whole
    sequence on the host; it must be the per-request rule of the selector."""
    import numpy as np
    import locks_oracle as orc
    from locks import LocksConfig
    from locks.cp_hotpath import global_page_params
    for seq_len in (1, 15, 16, 17, 4099, 131073, 1048577):
        for kw in (dict(budget_pages=128), dict(budget_pages=1), dict(budget=0.1),
                   dict(budget=0.03)):
            cfg = LocksConfig(sink_pages=1, window_pages=8, **kw)
            npg, nsh, b = global_page_params(seq_len, 16, cfg)
            o = orc.derive_page_params(np.array([seq_len]), 16, 8, 1,
                                       kw.get("budget_pages", 0),
                                       kw.get("budget", 0.1))
            assert (npg, nsh, b) == (int(o[0][0]), int(o[1][0]), int(o[2][0]))
