"""GPU parity of paged_attention against the oracle: the reference's matrices
(tests/flag_attn/test_paged_attention.py there), bit-exact block-table indexing, golden fixtures."""
import ctypes
import os

import pytest
import torch

import flagattention_b200 as fa
import oracle
from flagattention_b200 import _C
from helpers import GOLDEN, assert_within_2x, max_diff

pytestmark = pytest.mark.gpu
NUM_BLOCKS = 1000


def _make(num_seqs, num_q_heads, group, head, block, max_seq_len, table_dtype=torch.int64, seed=0,
          dtype=torch.float16):
    gen = torch.Generator().manual_seed(seed)
    kv_heads = num_q_heads // group
    lens = torch.randint(1, max(2, max_seq_len), (num_seqs,), generator=gen, dtype=torch.int32)
    lens[0] = max_seq_len
    scale = head ** -0.5
    q = ((torch.rand((num_seqs, num_q_heads, head), generator=gen) * 2 - 1) * scale).to(dtype).cuda()
    kc = ((torch.rand((NUM_BLOCKS, kv_heads, block, head), generator=gen) * 2 - 1) * scale).to(dtype).cuda()
    vc = ((torch.rand((NUM_BLOCKS, kv_heads, block, head), generator=gen) * 2 - 1) * scale).to(dtype).cuda()
    max_blocks = (max_seq_len + block - 1) // block
    bt = torch.randint(0, NUM_BLOCKS, (num_seqs, max_blocks), generator=gen).to(table_dtype).cuda()
    return q, kc, vc, lens.cuda(), bt, scale, int(lens.max())


def _check(q, kc, vc, lens, bt, scale, max_len, num_splits=0):
    out = fa.paged_attention(q, kc, vc, lens, bt, scale, max_len, num_splits)
    ref = oracle.paged_attention_gathered(q, kc, vc, bt, lens, scale)
    assert out.shape == q.shape and out.dtype == q.dtype
    assert torch.allclose(out, ref, atol=2e-3, rtol=1e-5), f"max diff {max_diff(out, ref):.3e}"
    # and the 2x rule of the dense operators: error against unrounded fp32 at most twice that of
    # the same-precision PyTorch path on densely gathered keys / values
    ref32 = oracle.paged_attention_gathered(q, kc, vc, bt, lens, scale, out_dtype=torch.float32)
    same = oracle.paged_attention_same_precision(q, kc, vc, bt, lens, scale)
    assert_within_2x(out, ref32, same, "paged out")
    return out


def test_gathered_oracle_equals_token_loop_oracle():
    args = _make(3, 8, 4, 32, 16, 100, seed=1)
    q, kc, vc, lens, bt, scale, _ = args
    a = oracle.paged_attention(q, kc, vc, bt, lens, scale)
    b = oracle.paged_attention_gathered(q, kc, vc, bt, lens, scale)
    assert max_diff(a, b) <= 2 ** -11 * a.float().abs().max().item()


@pytest.mark.parametrize("num_seqs", [1, 32])
@pytest.mark.parametrize("group", [1, 8])
@pytest.mark.parametrize("head", [64, 128])
@pytest.mark.parametrize("block", [16, 128, 256])
@pytest.mark.parametrize("max_seq_len", [512, 4096])
def test_default(num_seqs, group, head, block, max_seq_len):
    tdt = torch.int64 if (num_seqs + head) % 3 else torch.int32
    _check(*_make(num_seqs, 64, group, head, block, max_seq_len, tdt, seed=head + block))


@pytest.mark.parametrize("num_seqs", [1, 16])
@pytest.mark.parametrize("group", [1, 8])
@pytest.mark.parametrize("head", [32, 64])
@pytest.mark.parametrize("num_splits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_by_num_splits(num_seqs, group, head, num_splits):
    _check(*_make(num_seqs, 64, group, head, 16, 2048, seed=num_splits), num_splits=num_splits)


@pytest.mark.parametrize("num_seqs,heads,group,head,block,max_seq_len,num_splits", [
    (1, 12, 1, 64, 16, 2, 0), (16, 64, 8, 32, 16, 2048, 2), (16, 64, 1, 64, 16, 2048, 6),
    (4, 32, 4, 128, 16, 5000, 0), (2, 40, 20, 128, 32, 700, 0), (3, 8, 2, 256, 16, 300, 2),
    (2, 6, 3, 16, 48, 333, 0),
])
def test_by_case(num_seqs, heads, group, head, block, max_seq_len, num_splits):
    _check(*_make(num_seqs, heads, group, head, block, max_seq_len, seed=heads), num_splits=num_splits)


def test_bf16_and_strided_query():
    q, kc, vc, lens, bt, scale, mx = _make(5, 32, 4, 128, 16, 1500, seed=9, dtype=torch.bfloat16)
    wide = torch.zeros((5, 32, 256), dtype=torch.bfloat16, device="cuda")
    wide[..., :128] = q
    out = fa.paged_attention(wide[..., :128], kc, vc, lens, bt, scale, mx)
    ref = oracle.paged_attention_gathered(q, kc, vc, bt, lens, scale)
    assert torch.allclose(out.float(), ref.float(), atol=2e-2, rtol=1e-2)


def test_block_table_indexing_is_bit_exact():
    """(1) The physical block ids the kernel resolves equal block_tables exactly, for int32 and
    int64 tables; (2) with one-hot value blocks any wrong block would move the output by O(1)."""
    for tdt in (torch.int32, torch.int64):
        q, kc, vc, lens, bt, scale, mx = _make(7, 16, 4, 64, 16, 900, tdt, seed=21)
        lib = _C.load()
        args = _C.PagedArgs()
        args.dtype, args.num_seqs, args.num_q_heads, args.num_kv_heads = 0, 7, 16, 4
        args.head_size, args.block_size, args.max_context_len = 64, 16, mx
        args.block_table_is_i64 = int(tdt == torch.int64)
        args.query, args.q_stride_s, args.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
        args.key_cache, args.value_cache = kc.data_ptr(), vc.data_ptr()
        args.kv_stride_b, args.kv_stride_h, args.kv_stride_t = kc.stride()[:3]
        args.context_lens, args.block_tables = lens.data_ptr(), bt.data_ptr()
        args.bt_stride_s = bt.stride(0)
        out = torch.empty_like(q)
        args.out, args.o_stride_s, args.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
        visited = torch.full((7, bt.shape[1]), -7, dtype=torch.int64, device="cuda")
        st = lib.fa_paged_trace_blocks(ctypes.byref(args), ctypes.c_void_p(visited.data_ptr()),
                                       bt.shape[1], _C.stream_ptr(q.device))
        assert st == 0
        used = (lens.long() + 15) // 16
        cols = torch.arange(bt.shape[1], device="cuda")[None, :]
        want = torch.where(cols < used[:, None], bt.long(), torch.full_like(bt.long(), -1))
        assert torch.equal(visited, want)

    # one-hot values: V of physical block p is the constant p / 1024 in every channel, K is zero
    # so the softmax is uniform -> out = mean over the context of (block id / 1024)
    S, Hq, G, D, BS = 4, 8, 4, 64, 16
    gen = torch.Generator().manual_seed(4)
    lens = torch.tensor([16, 160, 333, 1000], dtype=torch.int32)
    nb = 256
    bt = torch.stack([torch.randperm(nb, generator=gen)[:63] for _ in range(S)]).to(torch.int32).cuda()
    kc = torch.zeros((nb, Hq // G, BS, D), dtype=torch.float16, device="cuda")
    vc = (torch.arange(nb, device="cuda").float() / 1024).half()[:, None, None, None].expand(nb, Hq // G, BS, D).contiguous()
    q = torch.randn((S, Hq, D), generator=gen).half().cuda()
    for splits in (1, 4):
        out = fa.paged_attention(q, kc, vc, lens.cuda(), bt, 1.0, 1000, splits)
        for i in range(S):
            ctx = int(lens[i])
            ids = bt[i].long().cpu()
            per_tok = (ids[torch.arange(ctx) // BS].float() / 1024).half().float()
            want = per_tok.mean().item()
            assert abs(out[i].float().mean().item() - want) < 2e-3


def test_unused_table_entries_are_never_read():
    """Entries past ceil(context_len / block_size) may hold anything.  Here they name a valid block
    whose keys and values are NaN: a kernel that read one of them would return NaN, a failed
    assertion instead of an out-of-range access."""
    q, kc, vc, lens, bt, scale, mx = _make(6, 16, 2, 128, 16, 700, torch.int32, seed=33)
    poison_id = NUM_BLOCKS - 1
    bt = bt.clamp(max=poison_id - 1)                     # no live entry names the poisoned block
    kc, vc = kc.clone(), vc.clone()
    kc[poison_id], vc[poison_id] = float("nan"), float("nan")
    used = (lens.long() + 15) // 16
    cols = torch.arange(bt.shape[1], device="cuda")[None, :]
    poisoned = torch.where(cols < used[:, None], bt, torch.full_like(bt, poison_id))
    assert (poisoned == poison_id).any()
    for splits in (0, 1, 4):
        a = fa.paged_attention(q, kc, vc, lens, bt, scale, mx, splits)
        b = fa.paged_attention(q, kc, vc, lens, poisoned, scale, mx, splits)
        assert torch.isfinite(b.float()).all()
        assert torch.equal(a, b)


def test_golden_fixtures_on_gpu():
    cases = torch.load(os.path.join(GOLDEN, "paged.pt"))["cases"]
    for c in cases:
        out = fa.paged_attention(c["q"].cuda(), c["key_cache"].cuda(), c["value_cache"].cuda(),
                                 c["context_lens"].cuda(), c["block_tables"].cuda(), c["scale"],
                                 int(c["context_lens"].max()))
        assert torch.allclose(out.cpu(), c["out"], atol=2e-3, rtol=1e-5)
