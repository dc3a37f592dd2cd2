"""ctypes loader for the C oracle (``gdn_chunk_oracle.c``).

TEST INFRASTRUCTURE ONLY: used by the tests, the smoke check and the CPU-baseline
leg of the benchmark.  Builds the shared library with ``make`` on first use when it
is missing (gcc is the only requirement).
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libgdn_chunk_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "gdn_chunk_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(build())
        fp = ctypes.POINTER(ctypes.c_float)
        lib.gdn_oracle_recurrent_f32.argtypes = [fp] * 8 + [ctypes.c_int] * 5
        lib.gdn_oracle_recurrent_f32.restype = ctypes.c_int
        lib.gdn_oracle_chunk_f32.argtypes = [fp] * 8 + [ctypes.c_int] * 6
        lib.gdn_oracle_chunk_f32.restype = ctypes.c_int
        lib.gdn_oracle_max_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def max_threads() -> int:
    return int(_load().gdn_oracle_max_threads())


def _f32(x):
    return np.ascontiguousarray(np.asarray(x, dtype=np.float32))


def _ptr(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) if a is not None else None


def _run(kind, q, k, v, g, beta, initial_state, chunk_size, nthreads):
    lib = _load()
    q, k, v, g, beta = (_f32(x) for x in (q, k, v, g, beta))
    b, s, hk, d = q.shape
    hv = v.shape[2]
    if d != 128 or v.shape[3] != 128:
        raise ValueError("the C oracle is compiled for D = 128")
    h0 = _f32(initial_state) if initial_state is not None else None
    out = np.empty((b, s, hv, d), dtype=np.float32)
    ht = np.empty((b, hv, d, d), dtype=np.float32)
    if kind == "recurrent":
        rc = lib.gdn_oracle_recurrent_f32(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(h0),
                                          _ptr(out), _ptr(ht), b, s, hk, hv, nthreads)
    else:
        rc = lib.gdn_oracle_chunk_f32(_ptr(q), _ptr(k), _ptr(v), _ptr(g), _ptr(beta), _ptr(h0),
                                      _ptr(out), _ptr(ht), b, s, hk, hv, chunk_size, nthreads)
    if rc != 0:
        raise ValueError(f"C oracle rejected its arguments (rc={rc})")
    return out, ht


def recurrent_f32(q, k, v, g, beta, initial_state=None, nthreads=0):
    """Token-by-token oracle in fp32; returns (out, final_state) as numpy arrays."""
    return _run("recurrent", q, k, v, g, beta, initial_state, 0, nthreads)


def chunk_f32(q, k, v, g, beta, initial_state=None, chunk_size=64, nthreads=0):
    """Chunked WY-form oracle in fp32; returns (out, final_state) as numpy arrays."""
    return _run("chunk", q, k, v, g, beta, initial_state, chunk_size, nthreads)
