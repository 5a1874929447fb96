"""Build libsfb.so (the CUDA kernels + C ABI) in-tree for sm_100a.

    python -m llm_compileforge_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU.  Each ``csrc/*.cu`` becomes an object under
``csrc/_obj`` (rebuilt only when it or a header changed) and the objects are
linked, with the static CUDA runtime, into ``llm_compileforge_b200/libsfb.so``.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(PKG, "libsfb.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _headers_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    paths += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile and link.  ``SFB_NVCC_FLAGS`` adds compiler flags and ``SFB_LIB_OUT`` writes such a variant to another path
    (objects beside it), leaving the regular library alone."""
    global OBJ, LIB
    extra = os.environ.get("SFB_NVCC_FLAGS", "").split()
    if os.environ.get("SFB_LIB_OUT"):
        LIB = os.path.abspath(os.environ["SFB_LIB_OUT"])
        OBJ = LIB + "_obj"
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr = _headers_mtime()
    jobs = []
    for src in sources:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), hdr):
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", INCLUDE, "-c", s, "-o", o]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd: list[str]) -> None:
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode:
            sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode:
            raise RuntimeError(f"nvcc failed for {cmd[-3]}")

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(run, jobs))
    objs = [os.path.join(OBJ, s[:-3] + ".o") for s in sources]
    if jobs or force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        run(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
