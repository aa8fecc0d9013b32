"""Stage the reference's own CPU code for the timed reference arm.

    python oracle/make_ref.py [SRC]      # SRC, else $LOCKS_REFERENCE_SRC, else the default checkout location

Copies, unmodified, the nine files of the reference package (``locks`` v0.1.3)
that its CPU-runnable selection paths consist of -- ``selection/rki4_state.py``,
``rki4_build.py``, ``build.py``, ``rki4_score_torch.py``, ``select.py``, the two
modules they import (``arch.py``, ``quant.py``) and, for the latent (MLA) path,
``selection/mla_select.py`` and ``mla_score_torch.py`` -- into
``oracle/_ref/locks_ref/`` under the package name ``locks_ref`` (their imports
are relative, so the copy works under another name and does not collide with
this repository's own ``locks`` package).  ``oracle/_ref/`` is git-ignored: the
files are staged, never committed; they travel with the working tree to the
machine the benchmark runs on, where ``bench.py --impl reference`` times them
on the host cores.  Where the reference checkout is absent this script does
nothing, and the benchmark falls back to the numpy restatement
(``oracle/locks_oracle.py``).

This is test / measurement infrastructure: nothing under ``locks-kv_b200/``
imports it.
"""
from __future__ import annotations

import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# where the build container keeps the read-only reference checkout
DEFAULT_SRC = os.path.join(os.sep, "root", "reference", "src")
DST = os.path.join(HERE, "_ref", "locks_ref")
FILES = ["arch.py", "quant.py", "selection/rki4_state.py",
         "selection/rki4_build.py", "selection/build.py",
         "selection/rki4_score_torch.py", "selection/select.py",
         "selection/mla_select.py", "selection/mla_score_torch.py"]


def stage(src_root: str | None = None) -> bool:
    src_root = src_root or os.environ.get("LOCKS_REFERENCE_SRC", DEFAULT_SRC)
    pkg = os.path.join(src_root, "locks")
    if not all(os.path.exists(os.path.join(pkg, f)) for f in FILES):
        print(f"[make_ref] no reference checkout at {pkg}: nothing staged")
        return False
    for f in FILES:
        dst = os.path.join(DST, f)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(pkg, f), dst)
    for d in ("", "selection"):
        with open(os.path.join(DST, d, "__init__.py"), "w") as fh:
            fh.write("# stub written by oracle/make_ref.py: the staged modules "
                     "are imported one by one\n")
    print(f"[make_ref] staged {len(FILES)} reference files under {DST}")
    return True


if __name__ == "__main__":
    sys.exit(0 if stage(sys.argv[1] if len(sys.argv) > 1 else None) else 0)
