"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol the
public header declares; the Python interface validates arguments like the reference's
(gdn_qsa_sm80/gdn_chunk_interface.py:19-32) and refuses to run without CUDA tensors."""

import ctypes
import os
import re

import pytest
import torch

from gdn_qsa_sm80_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "gdn_chunk_sm100.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(gdn_[a-z0-9_]+)\s*\(", text))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return ctypes.CDLL(_lib.LIB_PATH)


def test_header_and_binding_agree():
    assert _declared_functions() == set(_lib.EXPORTS)


def test_library_exports_every_declared_symbol(lib):
    for name in _declared_functions():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_scratch_size_and_error_strings_need_no_gpu():
    L = _lib.load()
    assert L.gdn_chunk_scratch_bytes(1, 8192, 16, 32, 0) >= 4
    assert _lib.error_string(0) == "ok"
    for code in range(1, 6):
        assert _lib.error_string(code) not in ("ok", "unknown status")
    assert _lib.error_string(99) == "unknown status"


def test_argument_validation_before_any_cuda_call():
    L = _lib.load()
    # bad head ratio, bad gate dtype, bad path, missing scratch: rejected on the host, no device touched
    args = [None] * 8
    assert L.gdn_chunk_fwd_sm100(*args, None, 0, 1, 64, 3, 4, 0, 0, None) == _lib.GDN_ERR_BAD_ARGUMENT
    assert L.gdn_chunk_fwd_sm100(*args, None, 0, 1, 64, 2, 4, 7, 0, None) == _lib.GDN_ERR_BAD_ARGUMENT
    assert L.gdn_chunk_fwd_sm100(*args, None, 0, 1, 64, 2, 4, 0, 99, None) == _lib.GDN_ERR_BAD_ARGUMENT
    assert L.gdn_chunk_fwd_sm100(*args, None, 0, 1, 64, 2, 4, 0, 0, None) == _lib.GDN_ERR_SCRATCH


def _cpu_inputs(B=1, S=64, Hk=2, Hv=4):
    q = torch.zeros(B, S, Hk, 128, dtype=torch.bfloat16)
    v = torch.zeros(B, S, Hv, 128, dtype=torch.bfloat16)
    g = torch.zeros(B, S, Hv)
    return q, q.clone(), v, g, g.clone()


def test_interface_shape_errors_match_reference_conventions():
    from gdn_qsa_sm80 import gdn_chunk
    q, k, v, g, beta = _cpu_inputs()
    with pytest.raises(ValueError, match="q must be"):
        gdn_chunk(q[..., :64], k, v, g, beta)
    with pytest.raises(ValueError, match="k must match q"):
        gdn_chunk(q, k[:, :32], v, g, beta)
    with pytest.raises(ValueError, match="v must be"):
        gdn_chunk(q, k, v[:, :32], g, beta)
    with pytest.raises(ValueError, match="g and beta"):
        gdn_chunk(q, k, v, g[..., :2], beta)
    q3, k3, v3, g3, b3 = _cpu_inputs(Hk=3, Hv=4)
    with pytest.raises(ValueError, match="multiple of Hk"):
        gdn_chunk(q3, k3, v3, g3, b3)


def test_no_cpu_fallback():
    from gdn_qsa_sm80 import gdn_chunk
    with pytest.raises(RuntimeError, match="no CPU path"):
        gdn_chunk(*_cpu_inputs())


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", os.path.join(ROOT, "does", "not", "exist.so"))
    with pytest.raises(_lib.GdnLibraryError, match="no fallback"):
        _lib.load()
