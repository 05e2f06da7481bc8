"""The shared library builds, loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

from flagattention_b200 import _C

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "flagattn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_all_declared_symbols(built_lib):
    lib = ctypes.CDLL(built_lib)
    declared = _declared_symbols()
    assert len(declared) >= 18
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(declared) == set(_C.EXPORTED_SYMBOLS)


def test_status_strings_and_version(built_lib):
    lib = _C.load()
    assert lib.fa_version().decode().startswith("flagattn_b200")
    assert lib.fa_status_string(0) == b"ok"
    for code in range(-6, 0):
        assert lib.fa_status_string(code) not in (b"ok", b"unknown status")
    assert lib.fa_status_string(-99) == b"unknown status"


def test_argument_validation_needs_no_gpu(built_lib):
    """Bad arguments are rejected on the host before any CUDA call."""
    lib = _C.load()
    shape = _C.FlashShape(_C.FA_BF16, 1, 2, 2, 16, 16, 48, 0, 1.0)      # head_dim 48 is not built
    t = _C.Tensor4(0x1000, 0, 0, 48)
    assert lib.fa_flash_fwd(ctypes.byref(shape), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t),
                            ctypes.byref(t), ctypes.c_void_p(0x1000), None) == -2
    shape.D = 64
    assert lib.fa_flash_fwd(None, None, None, None, None, None, None) == -1
    bad = _C.Tensor4(0x1004, 0, 0, 64)                                   # misaligned pointer
    assert lib.fa_flash_fwd(ctypes.byref(shape), ctypes.byref(bad), ctypes.byref(t), ctypes.byref(t),
                            ctypes.byref(t), ctypes.c_void_p(0x1000), None) == -3
    shape.Hk = 3                                                         # H % Hk != 0
    assert lib.fa_flash_fwd(ctypes.byref(shape), ctypes.byref(t), ctypes.byref(t), ctypes.byref(t),
                            ctypes.byref(t), ctypes.c_void_p(0x1000), None) == -1
    args = _C.PagedArgs()
    assert lib.fa_paged_decode(ctypes.byref(args), None) == -1
    assert lib.fa_paged_workspace_bytes(ctypes.byref(args)) == 0
