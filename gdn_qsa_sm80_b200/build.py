"""Build the CUDA library in-tree for sm_100a only.

    python -m gdn_qsa_sm80_b200.build [--force] [--verbose]

Compiles every ``csrc/*.cu`` with nvcc (``-gencode arch=compute_100a,code=sm_100a -lineinfo``)
and links ``lib/libgdn_chunk_sm100.so`` next to this file.  nvcc cross-compiles, so no GPU is
needed to build.  There is no other architecture, no JIT cache and no fallback target.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libgdn_chunk_sm100.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC or add it to PATH)")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps_mtime() -> float:
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    files.append(os.path.join(os.path.dirname(HERE), "include", "gdn_chunk_sm100.h"))
    files.append(os.path.abspath(__file__))
    return max(os.path.getmtime(f) for f in files)


def needs_build() -> bool:
    return (not os.path.exists(LIB_PATH)) or os.path.getmtime(LIB_PATH) < _deps_mtime()


def build(force: bool = False, verbose: bool = False, diagnostics: bool | None = None) -> str:
    """diagnostics (default: environment variable GDN_BUILD_DIAGNOSTICS=1) compiles the kernels' cycle accounting in
    (-DGDN_DIAGNOSTICS); a production build carries none of it."""
    if diagnostics is None:
        diagnostics = os.environ.get("GDN_BUILD_DIAGNOSTICS", "0") == "1"
    if not force and not needs_build() and not diagnostics:
        return LIB_PATH
    nvcc = _nvcc()
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []
    if diagnostics:
        extra.append("-DGDN_DIAGNOSTICS")

    def compile_one(src):
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, r

    with ThreadPoolExecutor(max_workers=4) as ex:
        results = list(ex.map(compile_one, sources()))
    objs = []
    for src, obj, r in results:
        if verbose or r.returncode != 0:
            sys.stderr.write(f"--- {os.path.basename(src)}\n{r.stdout}{r.stderr}\n")
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
        objs.append(obj)
    link = [nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("link failed")
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / shared-memory usage")
    ap.add_argument("--diagnostics", action="store_true", help="compile the kernels' cycle accounting in")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, diagnostics=a.diagnostics or None))
