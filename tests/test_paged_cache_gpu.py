"""Writer of the paged KV cache (flagattention_b200.reshape_and_cache): bit-exact against the
token-by-token restatement, and the round trip append -> paged_attention against the read-side
oracle that the golden fixtures pin."""
import pytest
import torch

import flagattention_b200 as fa
import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,kv_heads,head,block,blocks", [(1, 1, 16, 16, 4), (77, 8, 128, 16, 40),
                                                               (300, 2, 64, 32, 20), (513, 4, 256, 128, 8),
                                                               (64, 32, 128, 256, 3)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("slot_dtype", [torch.int64, torch.int32])
def test_append_is_bit_exact(tokens, kv_heads, head, block, blocks, dtype, slot_dtype):
    gen = torch.Generator().manual_seed(tokens + head)
    key = torch.randn((tokens, kv_heads, head), generator=gen).to(dtype)
    value = torch.randn((tokens, kv_heads, head), generator=gen).to(dtype)
    kc = torch.randn((blocks, kv_heads, block, head), generator=gen).to(dtype)
    vc = torch.randn((blocks, kv_heads, block, head), generator=gen).to(dtype)
    slots = torch.randperm(blocks * block, generator=gen)[:tokens].to(slot_dtype)
    slots[::7] = -1                                   # padding tokens are skipped
    kc_ref, vc_ref = kc.clone(), vc.clone()
    oracle.cache_append(key, value, kc_ref, vc_ref, slots)
    kc_d, vc_d = kc.cuda(), vc.cuda()
    fa.reshape_and_cache(key.cuda(), value.cuda(), kc_d, vc_d, slots.cuda())
    assert torch.equal(kc_d.cpu(), kc_ref) and torch.equal(vc_d.cpu(), vc_ref)


def test_append_from_strided_rows_and_empty_batch():
    """key / value as slices of a fused qkv projection (row stride > heads * head); zero tokens."""
    gen = torch.Generator().manual_seed(5)
    T, Hk, D, BS, NB = 40, 4, 64, 16, 6
    qkv = torch.randn((T, 3 * Hk * D), generator=gen).to(torch.float16).cuda()
    key = qkv[:, Hk * D:2 * Hk * D].view(T, Hk, D)
    value = qkv[:, 2 * Hk * D:].view(T, Hk, D)
    kc = torch.zeros((NB, Hk, BS, D), dtype=torch.float16, device="cuda")
    vc = torch.zeros_like(kc)
    slots = torch.arange(T, device="cuda") + 3
    fa.reshape_and_cache(key, value, kc, vc, slots)
    kc_ref, vc_ref = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    oracle.cache_append(key.cpu(), value.cpu(), kc_ref, vc_ref, slots.cpu())
    assert torch.equal(kc.cpu(), kc_ref) and torch.equal(vc.cpu(), vc_ref)
    fa.reshape_and_cache(key[:0], value[:0], kc, vc, slots[:0])     # nothing to do, no error
    assert torch.equal(kc.cpu(), kc_ref)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_append_then_decode_round_trip(dtype):
    """Prefill + three decode steps: tokens are appended through scattered slots, then
    paged_attention over the cache equals the oracle over the same cache and over the plain
    (gathered) keys and values."""
    gen = torch.Generator().manual_seed(9)
    seqs, Hq, Hk, D, BS = 5, 8, 2, 128, 16
    lens = [37, 200, 16, 1, 129]
    max_blocks = (max(lens) + 3 + BS - 1) // BS
    NB = seqs * max_blocks + 7
    perm = torch.randperm(NB, generator=gen)[:seqs * max_blocks].view(seqs, max_blocks)
    bt = perm.to(torch.int32).cuda()
    kc = torch.zeros((NB, Hk, BS, D), dtype=dtype, device="cuda")
    vc = torch.zeros_like(kc)
    keys = [torch.randn((l + 3, Hk, D), generator=gen).to(dtype).cuda() for l in lens]
    vals = [torch.randn((l + 3, Hk, D), generator=gen).to(dtype).cuda() for l in lens]

    def slots_of(s, lo, hi):
        pos = torch.arange(lo, hi)
        return (perm[s, pos // BS] * BS + pos % BS).cuda()

    # prefill: all sequences' tokens in one call
    fa.reshape_and_cache(torch.cat([k[:l] for k, l in zip(keys, lens)]),
                         torch.cat([v[:l] for v, l in zip(vals, lens)]), kc, vc,
                         torch.cat([slots_of(s, 0, l) for s, l in enumerate(lens)]))
    cur = list(lens)
    for step in range(3):
        fa.reshape_and_cache(torch.stack([k[c] for k, c in zip(keys, cur)]),
                             torch.stack([v[c] for v, c in zip(vals, cur)]), kc, vc,
                             torch.cat([slots_of(s, c, c + 1) for s, c in enumerate(cur)]))
        cur = [c + 1 for c in cur]
        q = torch.randn((seqs, Hq, D), generator=gen).to(dtype).cuda()
        ctx = torch.tensor(cur, dtype=torch.int32, device="cuda")
        out = fa.paged_attention(q, kc, vc, ctx, bt, D ** -0.5, max(cur))
        ref = oracle.paged_attention(q, kc, vc, bt, ctx, D ** -0.5)
        # the reference's bar for fp16 (tests/flag_attn/test_paged_attention.py there); one bf16
        # rounding step of an O(1) output is 2^-8
        torch.testing.assert_close(out, ref, atol=2e-3 if dtype == torch.float16 else 8e-3, rtol=1e-5)
        # and against the tokens themselves, never having gone through a cache
        for s in range(seqs):
            k_s = keys[s][:cur[s]].float().repeat_interleave(Hq // Hk, dim=1)   # (ctx, Hq, D)
            v_s = vals[s][:cur[s]].float().repeat_interleave(Hq // Hk, dim=1)
            p = torch.softmax(torch.einsum("hd,thd->ht", q[s].float(), k_s) * D ** -0.5, dim=-1)
            o_s = torch.einsum("ht,thd->hd", p, v_s)
            tol = 1e-2 if dtype == torch.float16 else 4e-2   # one 16-bit rounding step of the output
            torch.testing.assert_close(out[s].float(), o_s, atol=tol, rtol=tol)
