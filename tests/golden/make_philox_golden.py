"""Generates tests/golden/philox.pt: dropout keep-masks made by the reference's own mask kernel.

Run once where the reference checkout is available:
    python tests/golden/make_philox_golden.py /path/to/FlagAttention
The reference's recompute_mask_kernel (src/flag_attn/testing/dropout.py:5-16) is a triton
kernel; it is loaded BY FILE PATH and run under triton's CPU interpreter (TRITON_INTERPRET=1),
so no GPU is needed.  The raw `tl.rand(seed, offset, n_rounds=6)` numbers behind the masks are
stored as well.  tests/test_oracle_golden.py pins oracle/dropout.py against this file, and the
GPU tests then pin the kernels' mask against oracle/dropout.py bit for bit.
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import importlib.util  # noqa: E402

import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: python %s /path/to/FlagAttention" % sys.argv[0])
REF = sys.argv[1]


@triton.jit
def _rand_kernel(out, seed, offset, n, BLOCK: tl.constexpr):
    offs = tl.arange(0, BLOCK)
    tl.store(out + offs, tl.rand(seed, offset + offs, n_rounds=6), mask=offs < n)


def main():
    path = os.path.join(REF, "src", "flag_attn", "testing", "dropout.py")
    spec = importlib.util.spec_from_file_location("fa_ref_testing_dropout", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    cases = []
    specs = [
        # B, H, M, N, p, seed, offset
        (1, 2, 5, 37, 0.5, 0, 0),
        (2, 3, 7, 40, 0.2, 12345, 8),
        (1, 1, 3, 1100, 0.8, 2 ** 40 + 17, 2 ** 32 - 64),   # counter crosses 2**32; N > 1024
        (1, 2, 4, 16, 0.1, 2 ** 63 + 5, 4096),
    ]
    for B, H, M, N, p, seed, offset in specs:
        mask = torch.full((B, H, M, N), True, dtype=torch.bool)
        mod.recompute_mask_kernel[(M, B, H)](mask, B, H, M, N, p, seed, offset)
        cases.append(dict(B=B, H=H, M=M, N=N, p=p, seed=seed, offset=offset, mask=mask))

    rands = []
    for seed, offset in [(0, 0), (12345, 7), (2 ** 40 + 17, 2 ** 32 - 16), (2 ** 63 + 5, 10 ** 12)]:
        out = torch.zeros(256, dtype=torch.float32)
        _rand_kernel[(1,)](out, seed, offset, 256, BLOCK=256)
        rands.append(dict(seed=seed, offset=offset, values=out))

    torch.save(dict(triton_version=triton.__version__, masks=cases, rands=rands),
               os.path.join(HERE, "philox.pt"))
    print("wrote philox.pt with triton", triton.__version__)


if __name__ == "__main__":
    main()
