"""Target architecture facts.  The reference dispatches between sm_90a and
sm_120a at run time (``arch.py:3-69``); this build targets B200 only."""
from __future__ import annotations

ARCH = "sm_100a"
GENCODE = "arch=compute_100a,code=sm_100a"
SMEM_CAP = 232448          # bytes of opt-in shared memory per CTA (227 KB)


def arch_flag() -> str:
    return "-gencode=" + GENCODE


def smem_cap() -> int:
    return SMEM_CAP


def has_pdl() -> bool:
    return True
