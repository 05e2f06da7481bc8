"""ctypes binding of libflagattn_b200.so (the C ABI in include/flagattn_b200.h).

The library is loaded lazily on first use.  There is no fallback: when the
shared library is missing or a call returns a non-zero status, a RuntimeError
is raised.
"""
import ctypes
import os
import threading

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libflagattn_b200.so")
_lib = None
_lock = threading.Lock()

FA_F16, FA_BF16 = 0, 1

EXPORTED_SYMBOLS = (
    "fa_flash_fwd", "fa_splitkv_fwd", "fa_splitkv_combine", "fa_splitkv_workspace_bytes",
    "fa_num_splits_heuristic", "fa_total_attention", "fa_flash_bwd_delta", "fa_flash_bwd_delta_zero", "fa_flash_bwd_dkdv",
    "fa_flash_bwd_dq", "fa_piecewise_fwd", "fa_piecewise_bwd_dkdv", "fa_piecewise_bwd_dq",
    "fa_paged_decode", "fa_paged_reduce", "fa_paged_workspace_bytes", "fa_paged_trace_blocks",
    "fa_paged_attention_noalloc", "fa_dropout_mask",
    "fa_flash_bwd_fused", "fa_flash_bwd_fused_stages", "fa_flash_bwd_fused_workspace_bytes", "fa_piecewise_bwd_fused",
    "fa_piecewise_bwd_fused_workspace_bytes",
    "fa_paged_cache_append", "fa_rotary_pair_fwd", "fa_rotary_pair_bwd",
    "fa_device_status", "fa_debug_wait_probe", "fa_set_kernel_family", "fa_status_string", "fa_version",
)


class Tensor4(ctypes.Structure):
    _fields_ = [("ptr", ctypes.c_void_p), ("stride_b", ctypes.c_int64),
                ("stride_h", ctypes.c_int64), ("stride_l", ctypes.c_int64)]


class FlashShape(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("B", ctypes.c_int32), ("H", ctypes.c_int32),
                ("Hk", ctypes.c_int32), ("M", ctypes.c_int32), ("N", ctypes.c_int32),
                ("D", ctypes.c_int32), ("causal", ctypes.c_int32), ("sm_scale", ctypes.c_float),
                ("dropout_p", ctypes.c_float), ("philox_seed", ctypes.c_uint64),
                ("philox_offset", ctypes.c_uint64)]


class PagedArgs(ctypes.Structure):
    _fields_ = [
        ("dtype", ctypes.c_int32), ("num_seqs", ctypes.c_int32), ("num_q_heads", ctypes.c_int32),
        ("num_kv_heads", ctypes.c_int32), ("head_size", ctypes.c_int32),
        ("block_size", ctypes.c_int32), ("max_context_len", ctypes.c_int32),
        ("block_table_is_i64", ctypes.c_int32), ("partition_size", ctypes.c_int32),
        ("attn_scale", ctypes.c_float),
        ("query", ctypes.c_void_p), ("q_stride_s", ctypes.c_int64), ("q_stride_h", ctypes.c_int64),
        ("key_cache", ctypes.c_void_p), ("value_cache", ctypes.c_void_p),
        ("kv_stride_b", ctypes.c_int64), ("kv_stride_h", ctypes.c_int64),
        ("kv_stride_t", ctypes.c_int64),
        ("context_lens", ctypes.c_void_p), ("block_tables", ctypes.c_void_p),
        ("bt_stride_s", ctypes.c_int64),
        ("out", ctypes.c_void_p), ("o_stride_s", ctypes.c_int64), ("o_stride_h", ctypes.c_int64),
        ("part_out", ctypes.c_void_p), ("part_max", ctypes.c_void_p), ("part_sum", ctypes.c_void_p),
        ("causal_rows", ctypes.c_int32),
    ]


def lib_path():
    return _LIB_PATH


def load():
    """Returns the loaded library, raising if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(_LIB_PATH):
                raise RuntimeError(
                    "libflagattn_b200.so is not built (%s). Run `python -m flagattention_b200.build`; "
                    "there is no fallback path." % _LIB_PATH)
            lib = ctypes.CDLL(_LIB_PATH)
            lib.fa_status_string.restype = ctypes.c_char_p
            lib.fa_status_string.argtypes = [ctypes.c_int]
            lib.fa_version.restype = ctypes.c_char_p
            lib.fa_splitkv_workspace_bytes.restype = ctypes.c_int64
            lib.fa_paged_workspace_bytes.restype = ctypes.c_int64
            lib.fa_flash_bwd_fused_workspace_bytes.restype = ctypes.c_int64
            lib.fa_piecewise_bwd_fused_workspace_bytes.restype = ctypes.c_int64
            lib.fa_num_splits_heuristic.restype = ctypes.c_int32
            lib.fa_num_splits_heuristic.argtypes = [ctypes.c_int32] * 8
            lib.fa_debug_wait_probe.argtypes = [ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
            lib.fa_set_kernel_family.argtypes = [ctypes.c_int32]
            lib.fa_set_kernel_family.restype = ctypes.c_int32
            _lib = lib
    return _lib


FA_ERR_UNSUPPORTED = -2


class kernel_family:
    """Context manager around fa_set_kernel_family: `with kernel_family("generic"):` runs the
    flash / piecewise operators on the shape-generic kernels only, "auto" on the tcgen05 kernels
    wherever they cover the call, "one_cta_per_tile" on the tcgen05 kernels but with the forward's
    one-CTA-per-query-tile form where "auto" would take the persistent one.  Process-wide while
    active."""

    def __init__(self, family):
        assert family in ("auto", "generic", "one_cta_per_tile")
        self.family = {"auto": 0, "generic": 1, "one_cta_per_tile": 2}[family]

    def __enter__(self):
        self.previous = load().fa_set_kernel_family(self.family)
        return self

    def __exit__(self, *exc):
        load().fa_set_kernel_family(self.previous)
        return False


def check(status, what):
    if status != 0:
        msg = load().fa_status_string(int(status)).decode()
        raise RuntimeError("%s failed: %s (status %d)" % (what, msg, status))


def dtype_code(dtype):
    if dtype == torch.float16:
        return FA_F16
    if dtype == torch.bfloat16:
        return FA_BF16
    raise AssertionError("only float16 and bfloat16 are supported, got %s" % dtype)


def kernel_ready(x):
    """Returns x, or a contiguous copy when x breaks the kernels' layout rule
    (unit inner stride, 16-byte aligned rows)."""
    if x.stride(-1) != 1:
        return x.contiguous()
    if x.data_ptr() % 16 != 0:
        return x.contiguous()
    for size, stride in zip(x.shape[:-1], x.stride()[:-1]):
        if size > 1 and stride % 8 != 0:
            return x.contiguous()
    return x


def tensor4(x):
    """fa_tensor4 view of a (B, H, L, D) tensor that passed kernel_ready()."""
    sb, sh, sl, _ = x.stride()
    b, h, l, _ = x.shape
    return Tensor4(x.data_ptr(), sb if b > 1 else 0, sh if h > 1 else 0, sl if l > 1 else 0)


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def flash_shape(dtype, B, H, Hk, M, N, D, causal, sm_scale, dropout_p=0.0, seed=0, offset=0):
    return FlashShape(dtype_code(dtype), B, H, Hk, M, N, D, 1 if causal else 0, float(sm_scale),
                      float(dropout_p), int(seed) & (2 ** 64 - 1), int(offset) & (2 ** 64 - 1))


def byref(x):
    return ctypes.byref(x)


def fptr(t):
    return ctypes.c_void_p(t.data_ptr())
