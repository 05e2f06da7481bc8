"""Dropout bookkeeping for flash_attention (counterpart of src/flag_attn/dropout.py:5-15 and
src/flag_attn/testing/dropout.py:18-25).

The kernels draw one Philox-4x32 (6 rounds) number per element of the (B, H, M, N) attention
matrix, with the key taken from torch's CUDA generator seed and the counter starting at the
generator's offset; the generator is then advanced past the numbers used, so consecutive calls
(and torch's own random ops) never reuse a counter.
"""
import ctypes

import torch

from . import _C


def philox_cuda_seed_offset(increment, device=None):
    """Returns (seed, offset) of the device's default CUDA generator and advances its offset by
    `increment` rounded up to a multiple of 4."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    index = device.index if device.index is not None else torch.cuda.current_device()
    gen = torch.cuda.default_generators[index]
    state = gen.get_state()
    words = state.view(torch.int64)
    seed, offset = int(words[0]), int(words[1])
    words[1] += (int(increment) + 3) // 4 * 4
    gen.set_state(state)
    return seed, offset


def recompute_mask(B, H, M, N, dropout_p, seed, offset, device):
    """Boolean (B, H, M, N) keep-mask of a flash_attention call that returned (seed, offset)."""
    mask = torch.ones((B, H, M, N), dtype=torch.bool, device=device)
    if dropout_p == 0:
        return mask
    lib = _C.load()
    with torch.cuda.device(device):
        st = lib.fa_dropout_mask(B, H, M, N, ctypes.c_float(dropout_p),
                                 ctypes.c_uint64(int(seed) & (2 ** 64 - 1)),
                                 ctypes.c_uint64(int(offset) & (2 ** 64 - 1)),
                                 ctypes.c_void_p(mask.data_ptr()), _C.stream_ptr(mask.device))
    _C.check(st, "fa_dropout_mask")
    return mask
