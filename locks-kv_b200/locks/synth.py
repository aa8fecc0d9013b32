"""Seeded synthetic decode workloads with the shapes of the benchmark configs.

Real-model KV caches are not available offline, so every test and benchmark
draws its inputs from here.  The distributions follow the workload description
of the benchmark configs:

  * keys   N(0,1) per channel, ``n_outlier`` channels per KV head scaled x8,
           RoPE (theta 500000, half-split / NeoX pairing) at positions 0..T-1;
  * values N(0,1);
  * query  N(0,1) with RoPE at the position of the token being decoded;
  * ``n_needles`` "needle" pages per KV head whose 16 keys all equal
           3 x (mean query of that head's group, rescaled to unit RMS) plus
           N(0, 0.1) noise, planted in the stored (post-RoPE) key space so the
           page selector has something to find;
  * block tables are a random permutation of the physical block pool.

Everything is generated with ``torch.Generator`` on the requested device, so a
CPU run is bit-reproducible for a given torch build (used by the parity tests
and by the golden-vector script) and a CUDA run is fast enough for the
full-size benchmark caches.

MLA (latent) workloads: latents N(0,1) of width ``kv_lora_rank + rope_dim`` with
RoPE on the trailing rope dims; absorbed queries N(0, 1/sqrt(width)).
"""
from __future__ import annotations

import dataclasses
import math
from typing import List, Optional

import torch

ROPE_THETA = 500000.0


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)
    return g


def rope_half_split(x: torch.Tensor, pos: torch.Tensor,
                    theta: float = ROPE_THETA) -> torch.Tensor:
    """Rotate ``x (T, H, d)`` (fp32) at integer positions ``pos (T,)``.

    Half-split pairing: channel i pairs with channel i + d/2.
    """
    d = x.shape[-1]
    half = d // 2
    inv = theta ** (-torch.arange(half, device=x.device, dtype=torch.float64)
                    * 2.0 / d)
    ang = pos.to(torch.float64)[:, None] * inv[None, :]
    cos = ang.cos().to(torch.float32)[:, None, :]
    sin = ang.sin().to(torch.float32)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


@dataclasses.dataclass
class GqaShape:
    """Geometry + selection knobs of one GQA workload."""
    n_layers: int
    n_kv: int
    G: int
    d: int = 128
    page: int = 16
    budget_pages: int = 32
    sink_pages: int = 1
    window_pages: int = 4
    n_needles: int = 6
    n_outlier: int = 4


CONFIG0 = GqaShape(n_layers=1, n_kv=8, G=4, budget_pages=32, sink_pages=1,
                   window_pages=4, n_needles=6)
CONFIG1 = GqaShape(n_layers=32, n_kv=8, G=4, budget_pages=128, sink_pages=1,
                   window_pages=8, n_needles=6)
CONFIG4 = GqaShape(n_layers=40, n_kv=2, G=16, budget_pages=128, sink_pages=1,
                   window_pages=8, n_needles=32)


def gqa_tokens(seed: int, layer: int, seq: int, n_tok: int, shape: GqaShape,
               device="cpu", chunk: int = 65536):
    """K, V ``(n_tok, n_kv, d)`` bf16 and q ``(n_kv*G, d)`` bf16 for one
    (layer, sequence).  The last token (position ``n_tok - 1``) is the token
    being decoded; q carries RoPE at that position."""
    n_kv, G, d, page = shape.n_kv, shape.G, shape.d, shape.page
    g = _gen(device, seed * 1000003 + layer * 7919 + seq * 104729 + 17)
    # query first (the needle keys depend on it)
    q = torch.randn(n_kv * G, d, generator=g, device=device,
                    dtype=torch.float32)
    qpos = torch.tensor([n_tok - 1], device=device)
    q = rope_half_split(q[None].reshape(1, n_kv * G, d), qpos)[0]
    out_ch = torch.stack([
        torch.randperm(d, generator=g, device=device)[:shape.n_outlier]
        for _ in range(n_kv)])                                   # (n_kv, n_out)
    K = torch.empty(n_tok, n_kv, d, device=device, dtype=torch.bfloat16)
    V = torch.empty(n_tok, n_kv, d, device=device, dtype=torch.bfloat16)
    gain = torch.ones(n_kv, d, device=device)
    gain.scatter_(1, out_ch, 8.0)
    for t0 in range(0, n_tok, chunk):
        t1 = min(t0 + chunk, n_tok)
        k = torch.randn(t1 - t0, n_kv, d, generator=g, device=device,
                        dtype=torch.float32) * gain[None]
        k = rope_half_split(k, torch.arange(t0, t1, device=device))
        K[t0:t1] = k.to(torch.bfloat16)
        V[t0:t1] = torch.randn(t1 - t0, n_kv, d, generator=g, device=device,
                               dtype=torch.float32).to(torch.bfloat16)
    # needle pages: drawn from the selectable range [sink, n_pages - window)
    n_pages = (n_tok + page - 1) // page
    lo, hi = shape.sink_pages, n_pages - shape.window_pages
    needles = torch.zeros(n_kv, 0, dtype=torch.int64, device=device)
    if hi - lo >= 2 * shape.n_needles and shape.n_needles > 0:
        qm = q.reshape(n_kv, G, d).mean(1)
        qm = qm / qm.pow(2).mean(-1, keepdim=True).sqrt()        # unit RMS
        needles = torch.stack([
            lo + torch.randperm(hi - lo, generator=g,
                                device=device)[:shape.n_needles]
            for _ in range(n_kv)])                               # (n_kv, n)
        for kh in range(n_kv):
            for p in needles[kh].tolist():
                noise = torch.randn(page, d, generator=g, device=device) * 0.1
                K[p * page:(p + 1) * page, kh] = \
                    (3.0 * qm[kh][None] + noise).to(torch.bfloat16)
    return K, V, q.to(torch.bfloat16), needles


@dataclasses.dataclass
class GqaCase:
    """A paged GQA decode problem: one KV cache per layer + request metadata."""
    shape: GqaShape
    kv_caches: List[torch.Tensor]      # per layer (NB, 2, page, n_kv, d) bf16
    q: torch.Tensor                    # (n_layers, R, n_kv*G, d) bf16
    block_table: torch.Tensor          # (R, MB) int32
    seq_lens: torch.Tensor             # (R,) int32, INCLUDING the decoded token
    needles: list                      # [layer][req] -> (n_kv, n_needles) int64
    scale: float

    @property
    def n_req(self) -> int:
        return int(self.seq_lens.shape[0])

    @property
    def num_blocks(self) -> int:
        return int(self.kv_caches[0].shape[0])

    @property
    def max_pages(self) -> int:
        return int(self.block_table.shape[1])


def make_gqa_case(seed: int, shape: GqaShape, seq_lens, *, device="cpu",
                  num_blocks: Optional[int] = None, max_pages=None,
                  n_layers: Optional[int] = None,
                  spare_blocks: int = 3) -> GqaCase:
    """Build paged caches for ``len(seq_lens)`` requests.

    ``seq_lens[r]`` counts the token being decoded (its K/V are in the cache,
    as they are when the attention op runs).  Physical blocks are a random
    permutation of the pool; unused block-table slots hold 0.
    """
    L = shape.n_layers if n_layers is None else n_layers
    page, n_kv, d = shape.page, shape.n_kv, shape.d
    seq_lens = [int(s) for s in seq_lens]
    R = len(seq_lens)
    npg = [(s + page - 1) // page for s in seq_lens]
    MP = max(npg) if max_pages is None else int(max_pages)
    assert MP >= max(npg)
    NB = sum(npg) + spare_blocks if num_blocks is None else int(num_blocks)
    assert NB >= sum(npg)
    g = _gen("cpu", seed * 7 + 3)
    perm = torch.randperm(NB, generator=g)
    bt = torch.zeros(R, MP, dtype=torch.int32)
    o = 0
    for r in range(R):
        bt[r, :npg[r]] = perm[o:o + npg[r]].to(torch.int32)
        o += npg[r]
    caches, qs, needles = [], [], []
    for l in range(L):
        kvc = torch.zeros(NB, 2, page, n_kv, d, device=device,
                          dtype=torch.bfloat16)
        ql, nl = [], []
        for r in range(R):
            K, V, q, nd = gqa_tokens(seed, l, r, seq_lens[r], shape, device)
            pad = npg[r] * page - seq_lens[r]
            if pad:
                z = torch.zeros(pad, n_kv, d, device=device,
                                dtype=torch.bfloat16)
                K, V = torch.cat([K, z]), torch.cat([V, z])
            blocks = bt[r, :npg[r]].to(device=device, dtype=torch.int64)
            kvc[blocks, 0] = K.reshape(npg[r], page, n_kv, d)
            kvc[blocks, 1] = V.reshape(npg[r], page, n_kv, d)
            ql.append(q)
            nl.append(nd)
        caches.append(kvc)
        qs.append(torch.stack(ql))
        needles.append(nl)
    return GqaCase(shape=shape, kv_caches=caches, q=torch.stack(qs),
                   block_table=bt.to(device),
                   seq_lens=torch.tensor(seq_lens, dtype=torch.int32,
                                         device=device),
                   needles=needles, scale=1.0 / math.sqrt(d))


def make_gqa_shard(seed: int, shape: GqaShape, seq_len: int, p0: int, p1: int,
                   *, device, n_layers: Optional[int] = None,
                   spare_blocks: int = 3):
    """Pages ``[p0, p1)`` of the ONE sequence ``make_gqa_case(seed, shape,
    [seq_len])`` describes, as a paged cache of their own (context-parallel
    shard).  Returns ``(kv_caches, q (L, 1, H, d), block_table (1, p1-p0))``;
    local page j is global page p0 + j, blocks are a seeded permutation."""
    L = shape.n_layers if n_layers is None else n_layers
    page, n_kv, d = shape.page, shape.n_kv, shape.d
    npg = (int(seq_len) + page - 1) // page
    assert 0 <= p0 < p1 <= npg
    n_loc = p1 - p0
    NB = n_loc + spare_blocks
    g = _gen("cpu", seed * 7 + 3 + 1009 * p0)
    bt = torch.randperm(NB, generator=g)[:n_loc].to(torch.int32)[None]
    blocks = bt[0].to(device=device, dtype=torch.int64)
    caches, qs = [], []
    for l in range(L):
        K, V, q, _ = gqa_tokens(seed, l, 0, int(seq_len), shape, device)
        t0, t1 = p0 * page, min(p1 * page, int(seq_len))
        K, V = K[t0:t1], V[t0:t1]
        pad = n_loc * page - (t1 - t0)
        if pad:
            z = torch.zeros(pad, n_kv, d, device=device, dtype=torch.bfloat16)
            K, V = torch.cat([K, z]), torch.cat([V, z])
        kvc = torch.zeros(NB, 2, page, n_kv, d, device=device,
                          dtype=torch.bfloat16)
        kvc[blocks, 0] = K.reshape(n_loc, page, n_kv, d)
        kvc[blocks, 1] = V.reshape(n_loc, page, n_kv, d)
        del K, V
        caches.append(kvc)
        qs.append(q[None])
    return caches, torch.stack(qs), bt.to(device).contiguous()


# --------------------------------------------------------------------------- #
# MLA (latent KV) workloads                                                    #
# --------------------------------------------------------------------------- #
@dataclasses.dataclass
class MlaShape:
    n_layers: int = 27
    n_heads: int = 16
    kv_lora_rank: int = 512
    rope_dim: int = 64
    page: int = 16
    budget_pages: int = 128
    sink_pages: int = 1
    window_pages: int = 10

    @property
    def width(self) -> int:
        return self.kv_lora_rank + self.rope_dim


CONFIG3 = MlaShape()


@dataclasses.dataclass
class MlaCase:
    shape: MlaShape
    caches: List[torch.Tensor]         # per layer (NB, page, width) bf16
    q: torch.Tensor                    # (n_layers, B, H, width) bf16
    block_table: torch.Tensor          # (B, MB) int32
    seq_lens: torch.Tensor             # (B,) int32
    scale: float


def mla_tokens(seed: int, layer: int, seq: int, n_tok: int, shape: MlaShape,
               device="cpu"):
    W, Lkv = shape.width, shape.kv_lora_rank
    g = _gen(device, seed * 1000003 + layer * 7919 + seq * 104729 + 91)
    lat = torch.randn(n_tok, W, generator=g, device=device,
                      dtype=torch.float32)
    kr = rope_half_split(lat[:, None, Lkv:].contiguous(),
                         torch.arange(n_tok, device=device), 10000.0)[:, 0]
    lat = torch.cat([lat[:, :Lkv], kr], dim=-1)
    q = torch.randn(shape.n_heads, W, generator=g, device=device,
                    dtype=torch.float32) / math.sqrt(W)
    # a few tokens aligned with the queries so that selection matters
    n_pages = n_tok // shape.page
    if n_pages > 8 * shape.n_heads:
        hot = torch.randperm(n_pages - 2, generator=g,
                             device=device)[:shape.n_heads] + 1
        for h, p in enumerate(hot.tolist()):
            t = p * shape.page + (h % shape.page)
            lat[t] = lat[t] + 6.0 * q[h] / q[h].norm() * math.sqrt(W)
    return lat.to(torch.bfloat16), q.to(torch.bfloat16)


def make_mla_case(seed: int, shape: MlaShape, seq_lens, *, device="cpu",
                  n_layers: Optional[int] = None, max_pages=None,
                  spare_blocks: int = 2) -> MlaCase:
    L = shape.n_layers if n_layers is None else n_layers
    page, W = shape.page, shape.width
    seq_lens = [int(s) for s in seq_lens]
    B = len(seq_lens)
    npg = [(s + page - 1) // page for s in seq_lens]
    MP = max(npg) if max_pages is None else int(max_pages)
    NB = sum(npg) + spare_blocks
    g = _gen("cpu", seed * 11 + 5)
    perm = torch.randperm(NB, generator=g)
    bt = torch.zeros(B, MP, dtype=torch.int32)
    o = 0
    for r in range(B):
        bt[r, :npg[r]] = perm[o:o + npg[r]].to(torch.int32)
        o += npg[r]
    caches, qs = [], []
    for l in range(L):
        c = torch.zeros(NB, page, W, device=device, dtype=torch.bfloat16)
        ql = []
        for r in range(B):
            lat, q = mla_tokens(seed, l, r, seq_lens[r], shape, device)
            pad = npg[r] * page - seq_lens[r]
            if pad:
                lat = torch.cat([lat, torch.zeros(pad, W, device=device,
                                                  dtype=torch.bfloat16)])
            c[bt[r, :npg[r]].to(device=device, dtype=torch.int64)] = \
                lat.reshape(npg[r], page, W)
            ql.append(q)
        caches.append(c)
        qs.append(torch.stack(ql))
    return MlaCase(shape=shape, caches=caches, q=torch.stack(qs),
                   block_table=bt.to(device),
                   seq_lens=torch.tensor(seq_lens, dtype=torch.int32,
                                         device=device),
                   scale=1.0 / math.sqrt(128 + shape.rope_dim))
