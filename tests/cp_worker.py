"""Worker of the context-parallel GPU test: run under torchrun, one rank per GPU.

Every rank builds its page range of one seeded sequence, runs the
context-parallel decode step (eagerly and as a CUDA graph) and rank 0 compares
the result with the single-GPU hot path on the whole sequence: same selected
pages, outputs within the bf16 tolerance of a different merge order
(``locks.cp_hotpath.check_against_single_gpu``).
"""
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "locks-kv_b200"))

from locks.cp_hotpath import check_against_single_gpu     # noqa: E402


def main() -> int:
    rank = int(os.environ["RANK"])
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    seq_len = int(os.environ.get("CP_SEQ_LEN", "40005"))
    transport = os.environ.get("CP_TRANSPORT", "fused")
    ok, err, msgs = check_against_single_gpu(seq_len=seq_len, transport=transport)
    for m in msgs:
        print(m)
    if rank == 0:
        print(f"context parallel x{dist.get_world_size()} ({transport}): seq "
              f"{seq_len}, max |out - single GPU| = {err:.3e}, ok = {ok}")
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    # leave without tearing NCCL down: communicators that captured graphs still
    # reference can block in their destructor
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    sys.exit(main())
