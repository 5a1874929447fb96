"""Compile the plain-C oracle into oracle/_build/libsfb_oracle.so (TEST INFRASTRUCTURE).

Run as ``python oracle/build_oracle.py``; also called by ``__graft_entry__.build()``
and lazily by ``oracle.c_oracle`` when the library is missing or stale.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "sfb_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libsfb_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = ["gcc", "-O2", "-fno-fast-math", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC", SRC, "-o", OUT, "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
