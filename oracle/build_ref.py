"""Compile the reference's own golden C kernel for the `_mlir_ciface_*` convention
(TEST INFRASTRUCTURE).

    python oracle/build_ref.py [/path/to/LLM-CompileForge]

Without an argument the checkout is looked for in ``$SFB_REFERENCE_ROOT``, then in a directory
named ``reference`` beside this repository; when neither exists nothing is built and an
already built library is kept.

Source: ``tests/data/golden/rms_norm.c`` of the reference, compiled where it lies
(never copied) into ``oracle/_ref/librms_norm_golden.so``.  The output directory is
git-ignored; the built library travels with the working tree to the GPU box, where the
reference checkout itself does not exist.
"""

from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "librms_norm_golden.so")


def reference_root(explicit: str | None = None) -> str:
    """Where the reference checkout lies: the argument, ``$SFB_REFERENCE_ROOT``, or ``../reference`` beside this repository."""
    if explicit:
        return explicit
    env = os.environ.get("SFB_REFERENCE_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root: str | None = None) -> str | None:
    ref_root = reference_root(ref_root)
    src = os.path.join(ref_root, "tests", "data", "golden", "rms_norm.c")
    if not os.path.exists(src):
        return OUT if os.path.exists(OUT) else None
    os.makedirs(OUT_DIR, exist_ok=True)
    if not os.path.exists(OUT) or os.path.getmtime(OUT) < os.path.getmtime(src):
        subprocess.run(["gcc", "-O2", "-shared", "-fPIC", src, "-o", OUT, "-lm"], check=True)
    return OUT


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
