"""CPU-only: the C-ABI library loads and exports exactly what include/ampstein_b200.h declares,
and the ctypes table binds the same set. No compute call is made."""
import ctypes
import os
import re

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "ampstein_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(amp_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from ampstein_b200 import _lib
    names = _declared()
    assert "amp_exl3_gemm" in names and "amp_exl3_reconstruct" in names
    L = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(L, n), "library does not export " + n
    bound = set(_lib.SIGNATURES) | {"amp_b200_last_error"}
    assert set(names) == bound, (sorted(set(names) - bound), sorted(bound - set(names)))
    assert _lib.lib().amp_b200_version() >= 1


def test_bad_arguments_return_codes_without_a_gpu():
    """Argument validation happens before any CUDA call, so it can be exercised here."""
    from ampstein_b200 import _lib
    L = _lib.lib()
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p += (-p) % 16
    # K out of range
    assert L.amp_exl3_reconstruct(p, p, 16, 128, 9, 0, 0, 128, None) < 0
    assert "bitrate" in _lib.last_error()
    # n_out not a multiple of 128
    assert L.amp_exl3_reconstruct(p, p, 16, 128, 4, 0, 0, 64, None) < 0
    # slice out of bounds
    assert L.amp_exl3_reconstruct(p, p, 16, 128, 4, 0, 128, 128, None) < 0
    # gemv: m out of range, k not a multiple of 128, missing scale vectors
    assert L.amp_exl3_gemv(p, p, p, p, p, 17, 128, 128, 4, 0, 0, None) < 0
    assert L.amp_exl3_gemv(p, p, p, p, p, 1, 64, 128, 4, 0, 0, None) < 0
    assert L.amp_exl3_gemv(p, p, p, None, p, 1, 128, 128, 4, 0, 0, None) < 0
    # Hadamard: bad dtype / columns
    assert L.amp_had_r_128(p, p, None, None, 1, 128, 4, 1.0, None) < 0
    assert L.amp_had_r_128(p, p, None, None, 1, 100, 0, 1.0, None) < 0
    # empty problems are a no-op
    assert L.amp_exl3_reconstruct(p, p, 0, 128, 4, 0, 0, 128, None) == 0
    assert L.amp_had_r_128(p, p, None, None, 0, 128, 0, 1.0, None) == 0


def test_python_front_end_rejects_cpu_tensors():
    import pytest
    import torch
    import ampstein_b200 as amp
    t = torch.zeros((8, 8, 64), dtype=torch.int16)
    w = torch.zeros((128, 128), dtype=torch.float16)
    with pytest.raises(RuntimeError):
        amp.exl3_reconstruct(w, t, 4)
    with pytest.raises(TypeError):
        amp.exl3_gemm(w, t, w, None, None)
