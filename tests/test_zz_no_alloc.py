"""fa_paged_attention_noalloc: the partitioned decode for hosts that cannot allocate a workspace.

Some users of the library have no memory to give it -- a serving process that reserved all free
HBM for its KV-cache pool, or a decode loop that is not allowed to enter the CUDA allocator.  For
them the split-KV scratch lives in a fixed array inside the library.  This test drives that entry
point through the C ABI, twice in a row with different inputs (the array keeps the first call's
contents, which must not leak into the second result), and compares each output with the ordinary
entry points working on a torch-allocated workspace and with the oracle.  A third call repeats the
first problem's layout with shorter contexts, so that partition slots the first call filled are
left unwritten: the reducer must not read them.  The file name makes pytest collect it last.
"""
import ctypes

import pytest
import torch

import oracle
from flagattention_b200 import _C

pytestmark = pytest.mark.gpu

SCRATCH_BYTES = 17039360   # FA_PAGED_NOALLOC_SCRATCH_BYTES in include/flagattn_b200.h


def _problem(seed, num_seqs, q_heads, kv_heads, head, block, max_len, partition, table_dtype,
             len_cap=None):
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, len_cap or max_len, (num_seqs,), generator=gen, dtype=torch.int32)
    if len_cap is None:
        lens[0] = max_len
    nb = 400
    scale = head ** -0.5
    q = ((torch.rand((num_seqs, q_heads, head), generator=gen) * 2 - 1) * scale).half().cuda()
    kc = ((torch.rand((nb, kv_heads, block, head), generator=gen) * 2 - 1) * scale).half().cuda()
    vc = ((torch.rand((nb, kv_heads, block, head), generator=gen) * 2 - 1) * scale).half().cuda()
    bt = torch.randint(0, nb, (num_seqs, (max_len + block - 1) // block), generator=gen).to(table_dtype).cuda()
    lens = lens.cuda()
    out = torch.empty_like(q)
    a = _C.PagedArgs()
    a.dtype, a.num_seqs, a.num_q_heads, a.num_kv_heads = _C.FA_F16, num_seqs, q_heads, kv_heads
    a.head_size, a.block_size, a.max_context_len = head, block, max_len
    a.block_table_is_i64 = int(table_dtype == torch.int64)
    a.partition_size, a.attn_scale = partition, scale
    a.query, a.q_stride_s, a.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    a.key_cache, a.value_cache = kc.data_ptr(), vc.data_ptr()
    a.kv_stride_b, a.kv_stride_h, a.kv_stride_t = kc.stride()[:3]
    a.context_lens, a.block_tables, a.bt_stride_s = lens.data_ptr(), bt.data_ptr(), bt.stride(0)
    a.out, a.o_stride_s, a.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    keep = (q, kc, vc, bt, lens, scale)   # keeps the device buffers alive
    return a, out, keep


def _with_workspace(a, out_like):
    """The existing path: caller-provided workspace, fa_paged_decode + fa_paged_reduce."""
    lib = _C.load()
    P = (a.max_context_len + a.partition_size - 1) // a.partition_size
    rows = a.num_seqs * a.num_q_heads * P
    part_out = torch.empty(rows * a.head_size, dtype=torch.float32, device="cuda")
    part_max = torch.empty(rows, dtype=torch.float32, device="cuda")
    part_sum = torch.empty(rows, dtype=torch.float32, device="cuda")
    out = torch.empty_like(out_like)
    saved = (a.out, a.part_out, a.part_max, a.part_sum)
    a.out = out.data_ptr()
    a.part_out, a.part_max, a.part_sum = part_out.data_ptr(), part_max.data_ptr(), part_sum.data_ptr()
    stream = _C.stream_ptr(out.device)
    assert lib.fa_paged_decode(ctypes.byref(a), stream) == 0
    assert lib.fa_paged_reduce(ctypes.byref(a), stream) == 0
    torch.cuda.synchronize()
    a.out, a.part_out, a.part_max, a.part_sum = saved
    return out


def test_noalloc_matches_workspace_path_twice_in_a_row():
    lib = _C.load()
    stream = _C.stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    # first call: the first use on this device also resolves the scratch array's address
    problems = [
        _problem(101, 6, 32, 8, 128, 16, 3000, 512, torch.int32),
        _problem(202, 9, 16, 16, 64, 32, 1700, 256, torch.int64),   # other shape, other layout of the array
        _problem(101, 6, 32, 8, 128, 16, 3000, 512, torch.int32),
        # the layout of the call before, contexts of at most 600 tokens: the slots of partitions
        # 2..5 still hold that call's numbers and must stay unread
        _problem(404, 6, 32, 8, 128, 16, 3000, 512, torch.int32, len_cap=600),
    ]
    for a, out, keep in problems:
        out.fill_(float("nan"))
        assert lib.fa_paged_attention_noalloc(ctypes.byref(a), stream) == 0
        torch.cuda.synchronize()
        want = _with_workspace(a, out)
        assert torch.isfinite(out.float()).all()
        assert torch.allclose(out, want, atol=2e-3, rtol=1e-5), (out.float() - want.float()).abs().max()
        q, kc, vc, bt, lens, scale = keep
        ref = oracle.paged_attention_gathered(q, kc, vc, bt, lens, scale)
        assert torch.allclose(out, ref, atol=2e-3, rtol=1e-5), (out.float() - ref.float()).abs().max()


def test_noalloc_rejects_what_does_not_fit_and_one_pass_mode():
    lib = _C.load()
    stream = _C.stream_ptr(torch.device("cuda", torch.cuda.current_device()))
    a, out, _keep = _problem(303, 6, 32, 8, 128, 16, 3000, 512, torch.int32)
    assert lib.fa_paged_workspace_bytes(ctypes.byref(a)) <= SCRATCH_BYTES
    a.num_seqs = 6000                       # 6000 x 32 x 6 slots: far beyond the fixed array
    assert lib.fa_paged_workspace_bytes(ctypes.byref(a)) > SCRATCH_BYTES
    assert lib.fa_paged_attention_noalloc(ctypes.byref(a), stream) == -6      # FA_ERR_TOO_LARGE
    assert b"capacity" in lib.fa_status_string(-6)
    a.num_seqs, a.partition_size = 6, 0     # one-pass decode needs no scratch: not this entry point
    assert lib.fa_paged_attention_noalloc(ctypes.byref(a), stream) == -1      # FA_ERR_BAD_ARG
