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


def test_one_pass_backward_and_cache_writer_validation_needs_no_gpu(built_lib):
    """Workspace, stage and shape errors of the entries added beside the reference's launch pairs are
    decided on the host, before any CUDA call."""
    lib = _C.load()
    lib.fa_flash_bwd_fused_workspace_bytes.restype = ctypes.c_int64
    shape = _C.FlashShape(_C.FA_BF16, 2, 4, 2, 300, 500, 128, 1, 0.1)
    # (B, H, ceil(M / 128) * 128, D) fp32 + 16 bytes for the work-item counter
    assert lib.fa_flash_bwd_fused_workspace_bytes(ctypes.byref(shape)) == 2 * 4 * 384 * 128 * 4 + 16
    # piecewise: two accumulators (dq1, dq2); needs as many kv heads as query heads
    lib.fa_piecewise_bwd_fused_workspace_bytes.restype = ctypes.c_int64
    assert lib.fa_piecewise_bwd_fused_workspace_bytes(ctypes.byref(shape)) == 0
    mha = _C.FlashShape(_C.FA_BF16, 2, 4, 4, 300, 500, 128, 1, 0.1)
    assert lib.fa_piecewise_bwd_fused_workspace_bytes(ctypes.byref(mha)) == 2 * (2 * 4 * 384 * 128 * 4) + 16
    small = _C.FlashShape(_C.FA_BF16, 2, 4, 2, 300, 500, 32, 1, 0.1)       # head_dim 32: two-kernel path only
    assert lib.fa_flash_bwd_fused_workspace_bytes(ctypes.byref(small)) == 0
    drop = _C.FlashShape(_C.FA_BF16, 2, 4, 2, 300, 500, 128, 1, 0.1, 0.5, 1, 0)   # dropout: not covered
    assert lib.fa_flash_bwd_fused_workspace_bytes(ctypes.byref(drop)) == 0
    t = _C.Tensor4(0x1000, 0, 0, 128)
    tensors = [ctypes.byref(t)] * 4
    outs = [ctypes.byref(t)] * 3
    f = ctypes.c_void_p(0x1000)
    call = lambda ws, nbytes, stages: lib.fa_flash_bwd_fused_stages(
        ctypes.byref(shape), *tensors, f, f, *outs, ws, ctypes.c_int64(nbytes), stages, None)
    assert call(None, 1 << 30, 7) == -5                       # no workspace
    assert call(ctypes.c_void_p(0x1000), 16, 7) == -5         # too small
    assert call(ctypes.c_void_p(0x1004), 1 << 30, 7) == -5    # misaligned
    assert call(ctypes.c_void_p(0x1000), 1 << 30, 0) == -1    # no stage selected
    assert call(ctypes.c_void_p(0x1000), 1 << 30, 8) == -1
    assert lib.fa_flash_bwd_fused(ctypes.byref(small), *tensors, f, f, *outs, ctypes.c_void_p(0x1000),
                                  ctypes.c_int64(1 << 30), None) == -2
    # delta + zero-fill in one launch: the buffer must be there, 16-byte aligned, a multiple of 16 bytes
    dz = lambda ptr, nbytes: lib.fa_flash_bwd_delta_zero(ctypes.byref(shape), ctypes.byref(t), ctypes.byref(t), f,
                                                        ptr, ctypes.c_int64(nbytes), None)
    assert dz(None, 1024) == -1 and dz(ctypes.c_void_p(0x1000), 0) == -1
    assert dz(ctypes.c_void_p(0x1000), 1000) == -1 and dz(ctypes.c_void_p(0x1008), 1024) == -1
    i64 = ctypes.c_int64
    app = lambda dtype, head, key: lib.fa_paged_cache_append(
        dtype, 4, 2, head, 16, key, f, i64(256), i64(128), f, f, i64(4096), i64(2048), i64(128), f, None)
    assert app(7, 128, f) == -1                               # unknown dtype
    assert app(_C.FA_F16, 12, f) == -2                        # head not a multiple of 8
    assert app(_C.FA_F16, 128, None) == -1                    # missing pointer
    assert app(_C.FA_F16, 128, ctypes.c_void_p(0x1008)) == -3 # misaligned
    assert lib.fa_paged_cache_append(_C.FA_F16, 0, 2, 128, 16, None, None, i64(0), i64(0), None, None,
                                     i64(0), i64(0), i64(0), None, None) == 0   # nothing to do


def test_rotary_pair_validation_needs_no_gpu(built_lib):
    lib = _C.load()
    i64 = ctypes.c_int64
    t = _C.Tensor4(0x1000, 0, 128 * 64, 64)
    f = ctypes.c_void_p(0x1000)

    def fwd(dtype=_C.FA_BF16, D=64, table=f, stride=32, x=t, rows=10):
        return lib.fa_rotary_pair_fwd(dtype, 1, 2, 128, D, 0, ctypes.byref(x), table, f, f, f, i64(stride),
                                      rows, None, i64(0), ctypes.byref(t), ctypes.byref(t), None)
    assert fwd(dtype=5) == -1
    assert fwd(D=24) == -2 and fwd(D=1024) == -2              # head_dim rule
    assert fwd(table=None) == -1 and fwd(rows=0) == -1
    assert fwd(stride=16) == -3 and fwd(stride=34) == -3      # rows shorter than D / 2; odd stride
    assert fwd(table=ctypes.c_void_p(0x1004)) == -3
    assert fwd(x=_C.Tensor4(0x1002, 0, 128 * 64, 64)) == -3
    assert lib.fa_rotary_pair_bwd(_C.FA_F16, 0, 2, 128, 64, 1, None, None, f, f, f, f, i64(32), 10, None,
                                  i64(0), None, None) == 0    # empty batch: nothing to do
    assert lib.fa_rotary_pair_bwd(_C.FA_F16, 1, 2, 128, 64, 1, None, ctypes.byref(t), f, f, f, f, i64(32),
                                  10, None, i64(0), ctypes.byref(t), None) == -1
