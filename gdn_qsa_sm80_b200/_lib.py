"""ctypes binding of ``lib/libgdn_chunk_sm100.so`` (the C ABI in ``include/gdn_chunk_sm100.h``).

The library is the only implementation: when it has not been built, loading raises and every
operator call fails loudly.  There is no fallback path of any kind.
"""

from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libgdn_chunk_sm100.so")

GDN_OK = 0
GDN_ERR_BAD_ARGUMENT = 1
GDN_ERR_SCRATCH = 2
GDN_ERR_CUDA = 3
GDN_ERR_DRIVER = 4
GDN_ERR_DEVICE = 5

GATE_BF16 = 0
GATE_F32 = 1

PATH_AUTO = 0
PATH_SIMT = 1
PATH_TWOPASS_NV64 = 4
PATH_TWOPASS_NV32 = 5
PATH_PREPARE_ONLY = 6
PATH_CHAIN_ONLY = 7
PATH_COOP = 8
PATH_COOP_CHAIN_ONLY = 9
FLAG_QK_L2NORM = 1
FLAG_GATE_ACTIVATIONS = 2

PATHS = {"auto": PATH_AUTO, "simt": PATH_SIMT, 
         "twopass_nv64": PATH_TWOPASS_NV64, "twopass_nv32": PATH_TWOPASS_NV32,
         "prepare_only": PATH_PREPARE_ONLY, "chain_only": PATH_CHAIN_ONLY, "coop": PATH_COOP, "coop_chain_only": PATH_COOP_CHAIN_ONLY, "decode": 11, "twopass_t": 12,
         "prepare_only_t": 13, "chain_only_t": 14}

# Every symbol the public header declares (checked by the CPU tests).
EXPORTS = (
    "gdn_chunk_scratch_bytes",
    "gdn_chunk_workspace_offsets",
    "gdn_chunk_fwd_sm100",
    "gdn_chunk_fwd_sm100_ex",
    "gdn_chunk_host_arena_bytes",
    "gdn_rmsnorm_gated_sm100",
    "gdn_key_norm_sq_max_sm100",
    "gdn_forgetting_horizon_sm100",
    "gdn_chunk_fwd_gated_sm100",
    "gdn_chunk_fwd_host_sm100",
    "gdn_chunk_fwd_sm100_noalloc",
    "gdn_chunk_scan_transfers",
    "gdn_chunk_read_status",
    "gdn_chunk_error_string",
    "gdn_chunk_kernel_launches",
    "gdn_chunk_set_phase_profile",
    "gdn_umma_probe",
)

_lib = None


class GdnLibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the shared library once; raise if it is missing (build it with
    ``python -m gdn_qsa_sm80_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise GdnLibraryError(
            f"{LIB_PATH} is missing: build it with `python -m gdn_qsa_sm80_b200.build` "
            "(sm_100a only; there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    vp, ci, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
    lib.gdn_chunk_scratch_bytes.argtypes = [ci, ci, ci, ci, ci]
    lib.gdn_chunk_scratch_bytes.restype = sz
    lib.gdn_chunk_workspace_offsets.argtypes = [ci, ci, ci, ci, ctypes.POINTER(sz)]
    lib.gdn_chunk_workspace_offsets.restype = ci
    lib.gdn_chunk_fwd_sm100.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, ci, ci, vp]
    lib.gdn_chunk_fwd_sm100.restype = ci
    lib.gdn_chunk_fwd_sm100_ex.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, sz, ci, ci, ci, ci, ci, ci, ctypes.c_uint, vp]
    lib.gdn_chunk_fwd_sm100_ex.restype = ci
    lib.gdn_chunk_host_arena_bytes.argtypes = [ci] * 6
    lib.gdn_chunk_host_arena_bytes.restype = sz
    lib.gdn_chunk_fwd_host_sm100.argtypes = [vp] * 9 + [sz] + [ci] * 6 + [ctypes.c_uint, vp]
    lib.gdn_chunk_fwd_host_sm100.restype = ci
    lib.gdn_key_norm_sq_max_sm100.argtypes = [vp, ctypes.c_longlong, vp, vp]
    lib.gdn_key_norm_sq_max_sm100.restype = ci
    lib.gdn_forgetting_horizon_sm100.argtypes = [vp, vp, ci, ci, ci, ci, vp, vp, vp, vp]
    lib.gdn_forgetting_horizon_sm100.restype = ci
    lib.gdn_rmsnorm_gated_sm100.argtypes = [vp, vp, vp, vp, ctypes.c_longlong, ctypes.c_float, vp]
    lib.gdn_rmsnorm_gated_sm100.restype = ci
    lib.gdn_chunk_fwd_gated_sm100.argtypes = [vp] * 8 + [ctypes.c_float, vp, vp, vp, sz] + [ci] * 6 + [ctypes.c_uint, vp]
    lib.gdn_chunk_fwd_gated_sm100.restype = ci
    lib.gdn_chunk_fwd_sm100_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp]
    lib.gdn_chunk_fwd_sm100_noalloc.restype = ci
    lib.gdn_chunk_scan_transfers.argtypes = [vp, vp, vp, vp, vp, ci, ci, vp]
    lib.gdn_chunk_scan_transfers.restype = ci
    lib.gdn_chunk_read_status.argtypes = [vp, vp, ctypes.POINTER(ci)]
    lib.gdn_chunk_read_status.restype = ci
    lib.gdn_chunk_error_string.argtypes = [ci]
    lib.gdn_chunk_error_string.restype = ctypes.c_char_p
    lib.gdn_chunk_kernel_launches.argtypes = []
    lib.gdn_chunk_kernel_launches.restype = ctypes.c_ulonglong
    lib.gdn_chunk_set_phase_profile.argtypes = [vp]
    lib.gdn_chunk_set_phase_profile.restype = None
    lib.gdn_umma_probe.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp]
    lib.gdn_umma_probe.restype = ci
    _lib = lib
    return lib


def error_string(status: int) -> str:
    return load().gdn_chunk_error_string(int(status)).decode()


def check(status: int, what: str) -> None:
    if status != GDN_OK:
        raise GdnLibraryError(f"{what}: {error_string(status)} (status {status})")


def kernel_launches() -> int:
    return int(load().gdn_chunk_kernel_launches())
