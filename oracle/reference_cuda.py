"""Builds and loads the REFERENCE project's own gdn_chunk CUDA extension, recompiled for sm_100.

TEST / BENCHMARK INFRASTRUCTURE ONLY.  Nothing in the product imports this; it exists so that the
benchmark's reference arm and a cross-check test can run the reference's unmodified kernels
(CuTe mma.sync / cp.async code written for sm_80) on the same GPU as the library under test.

    python -m oracle.reference_cuda [--force]

The sources are compiled where they lie in the reference checkout (nothing is copied): the seven
files its setup.py lists for ``gdn_qsa_sm80._gdn_chunk`` (setup.py:57-68), with its own flags
(setup.py:18-33) except the target, ``-gencode arch=compute_100,code=sm_100`` instead of
``-arch=sm_80``.  Objects and the linked ``_gdn_chunk.so`` go to ``oracle/_ref/`` (git-ignored; the
built file travels with the tree).  Building needs the reference checkout, nvcc and torch's headers;
loading needs only the built file, torch and a GPU.
"""

from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

_HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(_HERE, "_ref")
SO_PATH = os.path.join(OUT_DIR, "_gdn_chunk.so")
SOURCES = ["gdn_kernel.cu", "gdn_scan_stage1.cu", "gdn_scan_stage1_reset.cu", "gdn_scan_stage2.cu",
           "gdn_scan_stage2_blelloch.cu", "gdn_scan_stage3_reset.cu", "gdn_ops.cu"]
_module = None


def reference_root():
    """Where the reference checkout is, or None (it is absent on a machine that only runs the built file):
    the environment variable GDN_REFERENCE_ROOT, else a directory `reference` beside this repository."""
    beside = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    for cand in (os.environ.get("GDN_REFERENCE_ROOT"), beside):
        if cand and os.path.isdir(os.path.join(cand, "csrc", "gdn_chunk")):
            return cand
    return None


def build(force: bool = False) -> str | None:
    """Compile and link the extension; returns its path, or None when the reference checkout is absent."""
    ref = reference_root()
    if ref is None:
        return SO_PATH if os.path.exists(SO_PATH) else None
    srcs = [os.path.join(ref, "csrc", "gdn_chunk", s) for s in SOURCES]
    if not force and os.path.exists(SO_PATH) and os.path.getmtime(SO_PATH) >= max(os.path.getmtime(s) for s in srcs):
        return SO_PATH
    import torch
    tdir = os.path.dirname(torch.__file__)
    inc = [os.path.join(tdir, "include"), os.path.join(tdir, "include", "torch", "csrc", "api", "include"),
           sysconfig.get_paths()["include"], os.path.join(ref, "third_party", "cutlass", "include")]
    obj_dir = os.path.join(OUT_DIR, "obj")
    os.makedirs(obj_dir, exist_ok=True)
    flags = ["-O3", "--expt-relaxed-constexpr", "--extended-lambda", "-lineinfo", "-std=c++17",
             "-gencode", "arch=compute_100,code=sm_100",
             "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_BFLOAT16_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
             "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "--diag-suppress=1301", "-DTORCH_EXTENSION_NAME=_gdn_chunk",
             "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
             "-Xcompiler", "-fPIC"] + [f"-I{i}" for i in inc]

    def one(src):
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        r = subprocess.run(["nvcc", *flags, "-c", src, "-o", obj], capture_output=True, text=True)
        return obj, r

    with ThreadPoolExecutor(max_workers=4) as ex:
        results = list(ex.map(one, srcs))
    for obj, r in results:
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError(f"nvcc failed on the reference source for {obj}")
    tlib = os.path.join(tdir, "lib")
    link = ["g++", "-shared", "-o", SO_PATH, *[o for o, _ in results], f"-L{tlib}", "-lc10", "-ltorch", "-ltorch_cpu",
            "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-L/usr/local/cuda/lib64", "-lcudart"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("linking the reference extension failed")
    return SO_PATH


def load():
    """The reference's extension module (``forward_gdn_chunk_auto`` and friends), or None when it was not built."""
    global _module
    if _module is None:
        if not os.path.exists(SO_PATH):
            return None
        import torch  # noqa: F401  (the extension links against torch's libraries)
        spec = importlib.util.spec_from_file_location("_gdn_chunk", SO_PATH)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _module = mod
    return _module


def gdn_chunk(q, k, v, g, beta, output_final_state=True):
    """The reference's public call (gdn_qsa_sm80/gdn_chunk_interface.py:35-50) on its own extension:
    contiguous CUDA bf16 tensors in, (out, final_state) out."""
    mod = load()
    if mod is None:
        raise RuntimeError("the reference's CUDA extension has not been built (oracle/_ref/_gdn_chunk.so is missing)")
    q, k, v, g, beta = (x.contiguous() for x in (q, k, v, g, beta))
    r = mod.forward_gdn_chunk_auto(q, k, v, g, beta, output_final_state)
    return r[0], r[1]


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
