"""CPU restatement of the dropout random stream of flash_attention.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The reference draws `tl.rand(seed, offset + idx, n_rounds=6) > dropout_p` per element of the
(B, H, M, N) attention matrix, idx = ((b*H + h)*M + m)*N + n (src/flag_attn/flash.py:369-371,455-456
and src/flag_attn/testing/dropout.py:6-16).  `tl.rand` is part of the third-party dependency
triton (3.6.0 in this image): Philox-4x32 with the 64-bit seed as the key, the 64-bit offset as
counter words 0 and 1 (words 2 and 3 zero), the first output word mapped to [0, 1) by
`x < 0 ? -x - 1 : x` on the signed word, times 4.6566127342e-10.  This file restates that
published algorithm in numpy; tests/golden/philox.pt (made by tests/golden/make_philox_golden.py,
which runs the reference's own mask kernel under triton's CPU interpreter) pins it.
"""
import numpy as np

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_LO = np.uint64(0xFFFFFFFF)
_S32 = np.uint64(32)


def philox_uniform(seed, counters, n_rounds=6):
    """float32 uniforms in [0, 1) for uint64 `counters` (any shape) under 64-bit `seed`."""
    ctr = np.asarray(counters, dtype=np.uint64)
    seed = int(seed) & (2 ** 64 - 1)
    k0, k1 = seed & 0xFFFFFFFF, seed >> 32
    c0, c1 = ctr & _LO, ctr >> _S32
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    for _ in range(n_rounds):
        pa = _M0 * c0   # 32x32 -> 64-bit products, no overflow in uint64
        pb = _M1 * c2
        c0, c1, c2, c3 = ((pb >> _S32) ^ c1 ^ np.uint64(k0), pb & _LO,
                          (pa >> _S32) ^ c3 ^ np.uint64(k1), pa & _LO)
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    x = c0.astype(np.uint32).view(np.int32).astype(np.int64)
    x = np.where(x < 0, -x - 1, x)
    return x.astype(np.float32) * np.float32(4.6566127342e-10)


def dropout_mask(B, H, M, N, dropout_p, seed, offset):
    """Boolean keep-mask, numpy (B, H, M, N); True = the attention weight is kept."""
    idx = np.arange(B * H * M * N, dtype=np.uint64) + np.uint64(int(offset) & (2 ** 64 - 1))
    return (philox_uniform(seed, idx) > np.float32(dropout_p)).reshape(B, H, M, N)
