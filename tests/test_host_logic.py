"""Host-side logic that needs no GPU: split heuristics, partition planning, layout normalisation,
operator argument checks."""
import math

import pytest
import torch

import flagattention_b200 as fa
from flagattention_b200 import _C, paged, split_kv


def _heuristic_python(B, H, M, N, BLOCK_M, BLOCK_N, num_sms, max_splits):
    """Independent restatement of the reference rule (src/flag_attn/split_kv.py:234-262 there)."""
    cdiv = lambda a, b: (a + b - 1) // b
    blocks = B * H * cdiv(M, BLOCK_M)
    if blocks >= 0.8 * num_sms:
        return 1
    n_blocks = cdiv(N, BLOCK_N)

    def ok(s):
        per = cdiv(n_blocks, s)
        return s == 1 or per * s - n_blocks < per

    def eff(s):
        waves = blocks * s / num_sms
        return waves / math.ceil(waves)

    plans = [(s, eff(s)) for s in range(1, min(num_sms, n_blocks, max_splits) + 1) if ok(s)]
    best = max([e for _, e in plans], default=0.0)
    for s, e in plans:
        if e >= 0.85 * best:
            return s
    return 1


@pytest.mark.parametrize("sms", [108, 132, 148])
def test_split_heuristic_matches_restatement(built_lib, sms):
    for B, H, M, N in [(2, 4, 1, 612), (2, 4, 1, 4096), (1, 2, 4, 8202), (4, 32, 4096, 4096),
                       (1, 1, 1, 524288), (2, 4, 2, 4000), (1, 2, 1, 8192), (1, 16, 3, 100),
                       (8, 8, 16, 2048), (1, 1, 17, 129)]:
        assert split_kv.num_splits_herustic(B, H, M, N, 16, 128, sms, 128) == \
            _heuristic_python(B, H, M, N, 16, 128, sms, 128)


def test_paged_partition_plan():
    plan = paged.plan_partitions
    # north-star decode config: explicit 64 splits of a 32768 context -> 512-token partitions
    assert plan(64, 8, 16, 32768, 64, 148) == (64, 512)
    # automatic: few CTAs -> 256-token partitions
    assert plan(1, 8, 16, 4096, 0, 148) == (16, 256)
    # automatic: short context or huge blocks -> one pass
    assert plan(1, 8, 16, 512, 0, 148) == (1, 0)
    assert plan(1, 8, 256, 4096, 0, 148) == (1, 0)
    # automatic: many CTAs and short context -> one pass; long context -> partitions
    assert plan(64, 8, 16, 2048, 0, 148) == (1, 0)
    assert plan(64, 8, 16, 4096, 0, 148) == (16, 256)
    # explicit single split
    assert plan(16, 8, 16, 2048, 1, 148) == (1, 0)
    # explicit odd split counts round the partition up to a power of two
    assert plan(16, 8, 16, 2048, 3, 148) == (3, 1024)
    assert plan(16, 8, 16, 2048, 6, 148) == (6, 512)
    assert plan(1, 12, 16, 2, 0, 148) == (1, 0)


def test_kernel_ready_layouts():
    x = torch.zeros(2, 4, 32, 64, dtype=torch.float16)
    assert _C.kernel_ready(x) is x
    bthd = torch.zeros(2, 32, 4, 64, dtype=torch.float16).transpose(1, 2)
    assert _C.kernel_ready(bthd) is bthd                       # arbitrary outer strides are fine
    inner = torch.zeros(2, 4, 64, 32, dtype=torch.float16).transpose(2, 3)
    assert _C.kernel_ready(inner).is_contiguous()              # inner stride must be 1
    odd = torch.zeros(2, 4, 32, 72, dtype=torch.float16)[..., 4:68]
    assert _C.kernel_ready(odd).is_contiguous()                # rows must start 16-byte aligned
    t = _C.tensor4(bthd)
    assert (t.stride_b, t.stride_h, t.stride_l) == (32 * 4 * 64, 64, 4 * 64)


def test_operator_argument_errors_match_reference_convention():
    """Shape violations raise AssertionError before touching the GPU, as in the reference
    (src/flag_attn/flash.py:26-35, src/flag_attn/piecewise.py:29-31, src/flag_attn/paged.py:31-32)."""
    q = torch.zeros(1, 4, 8, 48, dtype=torch.float16)
    with pytest.raises(AssertionError):
        fa.flash_attention(q, q, q)                            # head_dim 48
    q = torch.zeros(1, 4, 8, 64, dtype=torch.float16)
    k = torch.zeros(1, 3, 8, 64, dtype=torch.float16)
    with pytest.raises(AssertionError):
        fa.flash_attention(q, k, k)                            # 4 % 3 != 0
    with pytest.raises(AssertionError):
        fa.flash_attention(q, q, q[..., :32])                  # mismatched head_dim
    with pytest.raises(AssertionError):
        fa.piecewise_attention(q, q, q, q[..., :32], q, 4)
    with pytest.raises(AssertionError):
        fa.paged_attention(torch.zeros(2, 8, 24, dtype=torch.float16),
                           torch.zeros(4, 2, 16, 24, dtype=torch.float16),
                           torch.zeros(4, 2, 16, 24, dtype=torch.float16),
                           torch.ones(2, dtype=torch.int32), torch.zeros(2, 1, dtype=torch.int32),
                           1.0, 16)                            # head_size 24
    with pytest.raises(AssertionError):
        fa.paged_attention(torch.zeros(2, 8, 32, dtype=torch.float16),
                           torch.zeros(4, 2, 8, 32, dtype=torch.float16),
                           torch.zeros(4, 2, 8, 32, dtype=torch.float16),
                           torch.ones(2, dtype=torch.int32), torch.zeros(2, 1, dtype=torch.int32),
                           1.0, 8)                             # group > 1 needs block_size >= 16


def test_public_api_surface():
    for name in ("flash_attention", "piecewise_attention", "paged_attention",
                 "flash_attention_split_kv", "testing"):
        assert hasattr(fa, name)
    for name in ("flash_attention", "piecewise_attention", "paged_attention"):
        assert hasattr(fa.testing, name)
    import inspect
    sig = inspect.signature(fa.flash_attention)
    assert list(sig.parameters) == ["q", "k", "v", "causal", "sm_scale", "dropout_p",
                                    "return_log_normalizer", "return_total_attention",
                                    "return_seed_offset"]
    sig = inspect.signature(fa.piecewise_attention)
    assert list(sig.parameters) == ["q1", "k1", "q2", "k2", "v", "dist_threshold", "causal", "sm_scale"]
    sig = inspect.signature(fa.paged_attention)
    assert list(sig.parameters) == ["query", "key_cache", "value_cache", "context_lens",
                                    "block_tables", "attn_scale", "max_context_len", "num_splits"]


def test_single_query_dispatch_rule():
    """Which (q, k, v) the single-query forward may hand to the paged-decode kernels in place."""
    import torch
    from flagattention_b200 import flash as fl
    q = torch.zeros(2, 8, 1, 64, dtype=torch.float16)
    k = torch.zeros(2, 2, 1024, 64, dtype=torch.float16)
    v = torch.zeros(2, 2, 1024, 64, dtype=torch.float16)
    assert fl._decode_covered(q, k, v)
    assert fl._decode_covered(torch.zeros(2, 8, 2, 64, dtype=torch.float16), k, v)          # two queries per head
    assert not fl._decode_covered(torch.zeros(2, 8, 17, 64, dtype=torch.float16), k, v)     # 4 x 17 rows per kv head
    assert fl._decode_covered(torch.zeros(2, 8, 16, 64, dtype=torch.float16), k, v, True)   # causal, M <= N
    assert not fl._decode_covered(torch.zeros(2, 8, 16, 64, dtype=torch.float16), k[:, :, :0], v[:, :, :0])
    assert not fl._decode_covered(q, k[:, :, :1000], v[:, :, :1000])                        # N % 16 != 0
    kt = torch.zeros(2, 1024, 2, 64, dtype=torch.float16).transpose(1, 2)                   # BTHD view
    assert fl._decode_covered(q, kt, kt.clone(memory_format=torch.preserve_format))
    assert not fl._decode_covered(q, kt, v)                                                 # strides differ
    tab, lens = fl._identity_block_table(2, 4, 16, "cpu")
    assert tab.tolist() == [[0, 1, 2, 3], [16, 17, 18, 19]] and lens.tolist() == [64, 64]


def test_rotary_host_checks_and_table_normalisation():
    """rotary_pair's host side: table dtype / shape checks, re-packing of tables the kernel cannot
    read in place, position broadcasting; and rotary_tables against the angle formula."""
    from flagattention_b200 import rotary
    cos, sin = fa.rotary_tables(10, 32, base=100.0, position_scale=0.5)
    assert cos.shape == sin.shape == (10, 16) and cos.dtype == torch.float32
    ang = 3 * 0.5 * 100.0 ** (-2 * 5 / 32)
    assert abs(cos[3, 5].item() - math.cos(ang)) < 1e-6 and abs(sin[3, 5].item() - math.sin(ang)) < 1e-6

    good = [torch.zeros(10, 16) for _ in range(4)]
    tabs, rows, stride = rotary._tables_ready(good, 16, torch.device("cpu"))
    assert rows == 10 and stride == 16 and all(a is b for a, b in zip(tabs, good))
    wide = [torch.zeros(10, 64) for _ in range(4)]               # more columns than D / 2: read in place
    tabs, rows, stride = rotary._tables_ready(wide, 16, torch.device("cpu"))
    assert stride == 64 and all(a is b for a, b in zip(tabs, wide))
    odd = [torch.zeros(10, 35)[:, :16] for _ in range(4)]         # row stride 35: re-packed
    tabs, rows, stride = rotary._tables_ready(odd, 16, torch.device("cpu"))
    assert stride == 16 and all(t.is_contiguous() for t in tabs)
    with pytest.raises(AssertionError):
        rotary._tables_ready([torch.zeros(10, 16, dtype=torch.float64)] * 4, 16, torch.device("cpu"))
    with pytest.raises(AssertionError):
        rotary._tables_ready([torch.zeros(10, 8)] * 4, 16, torch.device("cpu"))        # fewer than D / 2 columns
    with pytest.raises(AssertionError):
        rotary._tables_ready([torch.zeros(10, 16)] * 3 + [torch.zeros(9, 16)], 16, torch.device("cpu"))

    pos, _, stride_b = rotary._positions_ready(torch.arange(7, dtype=torch.int32), 3, 7, "cpu")
    assert pos.dtype == torch.int64 and pos.shape == (1, 7) and stride_b == 0      # one row for the batch
    pos, _, stride_b = rotary._positions_ready(torch.zeros(3, 7, dtype=torch.int64), 3, 7, "cpu")
    assert stride_b == 7
    assert rotary._positions_ready(None, 3, 7, "cpu")[0] is None
    with pytest.raises(AssertionError):
        rotary._positions_ready(torch.zeros(7), 3, 7, "cpu")                        # floating point
    with pytest.raises(AssertionError):
        rotary._positions_ready(torch.zeros(2, 7, dtype=torch.int64), 3, 7, "cpu")  # wrong batch

    import inspect
    assert list(inspect.signature(fa.rotary_pair).parameters) == [
        "x", "cos1", "sin1", "cos2", "sin2", "positions", "interleaved"]
    assert hasattr(fa.testing, "rotary_pair")


def test_operands_on_the_wrong_device_raise_before_any_launch():
    """Host tensors where device tensors are expected raise AssertionError; nothing is launched
    (a kernel handed a host pointer would fault on the GPU)."""
    from flagattention_b200 import rotary
    x = torch.zeros(1, 2, 8, 32, dtype=torch.float16)
    tabs = fa.rotary_tables(8, 32)                              # default device: CPU
    with pytest.raises(AssertionError):
        fa.rotary_pair(x, *tabs, *tabs)                         # x itself is not a CUDA tensor
    with pytest.raises(AssertionError):
        rotary._tables_ready(list(tabs) * 2, 16, torch.device("cuda", 0))   # tables left on the CPU
    q = torch.zeros(1, 2, 8, 32, dtype=torch.float16)
    with pytest.raises(AssertionError):
        fa.piecewise_attention(q, q, q, q, q, 4)
    with pytest.raises(AssertionError):
        fa.flash_attention(q, q, q)
    with pytest.raises(AssertionError):
        fa.paged_attention(torch.zeros(2, 8, 32, dtype=torch.float16),
                           torch.zeros(4, 8, 16, 32, dtype=torch.float16),
                           torch.zeros(4, 8, 16, 32, dtype=torch.float16),
                           torch.ones(2, dtype=torch.int32), torch.zeros(2, 1, dtype=torch.int32),
                           1.0, 16)
    meta_q = torch.zeros(2, 8, 32, dtype=torch.float16, device="meta")
    with pytest.raises(AssertionError):                         # query elsewhere than its tables
        fa.paged_attention(meta_q, torch.zeros(4, 8, 16, 32, dtype=torch.float16, device="meta"),
                           torch.zeros(4, 8, 16, 32, dtype=torch.float16, device="meta"),
                           torch.ones(2, dtype=torch.int32), torch.zeros(2, 1, dtype=torch.int32),
                           1.0, 16)
    with pytest.raises(AssertionError):
        fa.reshape_and_cache(torch.zeros(2, 8, 32, dtype=torch.float16),
                             torch.zeros(2, 8, 32, dtype=torch.float16),
                             torch.zeros(4, 8, 16, 32, dtype=torch.float16),
                             torch.zeros(4, 8, 16, 32, dtype=torch.float16),
                             torch.zeros(2, dtype=torch.int64))


def test_backward_mode_switch():
    """Which backward kernels run is an API, not an environment variable: explicit modes, a context
    manager, and "auto" following torch's determinism switch."""
    from flagattention_b200 import flash as fl
    assert fl.get_backward_mode() == "auto"
    assert fl.use_one_pass_backward()
    with fl.backward_mode("two_kernel"):
        assert fl.get_backward_mode() == "two_kernel" and not fl.use_one_pass_backward()
        with fl.backward_mode("one_pass"):
            assert fl.use_one_pass_backward()
        assert not fl.use_one_pass_backward()
    assert fl.get_backward_mode() == "auto"
    before = torch.are_deterministic_algorithms_enabled()
    try:
        torch.use_deterministic_algorithms(True)
        assert not fl.use_one_pass_backward()
        with fl.backward_mode("one_pass"):
            assert fl.use_one_pass_backward()
    finally:
        torch.use_deterministic_algorithms(before)
    with pytest.raises(AssertionError):
        fl.set_backward_mode("fast")


def test_kernel_family_switch(built_lib):
    lib = _C.load()
    assert lib.fa_set_kernel_family(0) == 0
    with _C.kernel_family("generic"):
        assert lib.fa_set_kernel_family(1) == 1
    assert lib.fa_set_kernel_family(0) == 0
    with _C.kernel_family("one_cta_per_tile"):      # tcgen05 kernels, forward without its persistent form
        assert lib.fa_set_kernel_family(2) == 2
    assert lib.fa_set_kernel_family(7) == 0          # unknown values mean 0
    assert lib.fa_set_kernel_family(0) == 0
