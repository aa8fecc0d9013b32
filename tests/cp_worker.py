"""Worker of the context-parallel GPU test: run under torchrun, one rank per GPU.

Every rank builds its page range of one seeded sequence, runs the
context-parallel decode step (eagerly and as a CUDA graph) and rank 0 compares
the result with the single-GPU hot path on the whole sequence: same selected
pages, outputs within the bf16 tolerance of a different merge order.
"""
import math
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "locks-kv_b200"))

from locks import LocksConfig, synth                      # noqa: E402
from locks.cp_hotpath import ContextParallelHotPath       # noqa: E402
from locks.hotpath import HotPath                         # noqa: E402
from locks.parallel import partition_pages                # noqa: E402


def main() -> int:
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    seq_len = int(os.environ.get("CP_SEQ_LEN", "40005"))
    shape = synth.GqaShape(n_layers=3, n_kv=2, G=16, d=128, page=16,
                           budget_pages=64, sink_pages=1, window_pages=8,
                           n_needles=6, n_outlier=4)
    cfg = LocksConfig(budget_pages=shape.budget_pages,
                      sink_pages=shape.sink_pages,
                      window_pages=shape.window_pages)
    scale = 1.0 / math.sqrt(shape.d)
    npg = -(-seq_len // shape.page)
    p0, p1 = partition_pages(npg, world)[rank]
    caches, q, bt = synth.make_gqa_shard(11, shape, seq_len, p0, p1, device=dev)
    cp = ContextParallelHotPath(caches, bt, seq_len=seq_len, p0=p0, p1=p1,
                                n_kv=shape.n_kv, G=shape.G, scale=scale, cfg=cfg,
                                transport=os.environ.get("CP_TRANSPORT", "fused"))
    cp.build_all()
    cp.q.copy_(q)
    out_eager = cp.step_eager().clone()
    torch.cuda.synchronize()
    # the pages this rank attended in the last layer, as global ids
    cnt = cp.st.page_cnt[0].tolist()
    mine = [(cp.st.page_table[0, kh, :cnt[kh]] + p0).tolist()
            for kh in range(shape.n_kv)]
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    out_graph = cp.step().clone()
    cp.step()
    torch.cuda.synchronize()
    ok = True
    if not torch.equal(out_graph, cp.out):
        print(f"[rank {rank}] graph replay is not repeatable"); ok = False
    if (out_graph.float() - out_eager.float()).abs().max().item() > 0:
        print(f"[rank {rank}] graph and eager outputs differ"); ok = False
    status = int(cp.st.status.item())
    if status:
        print(f"[rank {rank}] kernel status word {status}"); ok = False
    if rank == 0:
        fc, fq, fbt = synth.make_gqa_shard(11, shape, seq_len, 0, npg, device=dev)
        sl = torch.tensor([seq_len], dtype=torch.int32, device=dev)
        hp = HotPath(fc, fbt, sl, n_kv=shape.n_kv, G=shape.G, scale=scale, cfg=cfg)
        hp.build_all(); hp.derive(); hp.q.copy_(fq)
        ref = hp.step_eager().clone()
        torch.cuda.synchronize()
        rc = hp.st.page_cnt[0].tolist()
        for kh in range(shape.n_kv):
            want = hp.st.page_table[0, kh, :rc[kh]].tolist()
            got = sorted(p for r in range(world) for p in gathered[r][kh])
            if got != want:
                extra = sorted(set(got) - set(want))[:5]
                miss = sorted(set(want) - set(got))[:5]
                print(f"kv head {kh}: page sets differ ({len(got)} vs {len(want)};"
                      f" extra {extra}, missing {miss})")
                ok = False
        err = (out_eager.float() - ref.float()).abs().max().item()
        print(f"context parallel x{world} ({cp.transport}): seq {seq_len}, {npg} pages, "
              f"max |out - single GPU| = {err:.3e}")
        if not err <= 2e-2:              # bf16 outputs, different merge order
            ok = False
    flag = torch.tensor([0 if ok else 1], device=dev)
    dist.all_reduce(flag)
    rc = int(flag.item() != 0)
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    # leave without tearing NCCL down: communicators that captured graphs still
    # reference can block in their destructor
    os._exit(rc)


if __name__ == "__main__":
    sys.exit(main())
