"""Oracle for paged_attention (test infrastructure, see oracle/__init__.py).

`paged_attention` follows src/flag_attn/testing/paged.py:5-52 of the
reference literally: per sequence, token j is fetched from
cache[block_tables[i][j // block_size], :, j % block_size, :] in a Python loop
(:31-37), kv heads are repeated for GQA (:40-43), all arithmetic is fp32
(:45-47), the result is cast to the cache dtype (:48).  Note its argument
order (block_tables before context_lens), which differs from the operator's.

`paged_attention_gathered` computes the same thing with one index_select per
sequence instead of a per-token loop; tests show it equal to the loop on
small cases and then use it where the loop would take minutes.
"""
import torch


def paged_attention(query, key_cache, value_cache, block_tables, context_lens, scale):
    out = torch.empty_like(query)
    n_q_heads = query.shape[1]
    n_kv_heads, block_size, head_size = value_cache.shape[1:]
    group = n_q_heads // n_kv_heads
    tables = block_tables.cpu().tolist()
    lens = context_lens.cpu().tolist()
    for i in range(query.shape[0]):
        ks, vs = [], []
        for j in range(int(lens[i])):
            blk = int(tables[i][j // block_size])
            ks.append(key_cache[blk, :, j % block_size, :])
            vs.append(value_cache[blk, :, j % block_size, :])
        keys, values = torch.stack(ks, 0), torch.stack(vs, 0)      # (ctx, kv_heads, head)
        if group > 1:
            keys = keys.repeat_interleave(group, dim=1)
            values = values.repeat_interleave(group, dim=1)
        qi = query[i].unsqueeze(0).transpose(0, 1).float()           # (heads, 1, head)
        scores = torch.bmm(qi, keys.permute(1, 2, 0).float()) * scale
        probs = torch.softmax(scores, dim=-1)
        oi = torch.bmm(probs, values.transpose(0, 1).float()).transpose(0, 1)
        out[i].copy_(oi.to(values.dtype).view(n_q_heads, head_size))
    return out


def _gather(cache, ids, ctx):
    """(kv_heads, ctx, head) view of one sequence's tokens: blocks `ids` laid end to end."""
    n_kv_heads, _, head_size = cache.shape[1:]
    return cache.index_select(0, ids).permute(1, 0, 2, 3).reshape(n_kv_heads, -1, head_size)[:, :ctx]


def paged_attention_gathered(query, key_cache, value_cache, block_tables, context_lens, scale,
                             out_dtype=None):
    """out_dtype=torch.float32 keeps the fp32 result unrounded (the reference rounds it to the cache
    dtype, src/flag_attn/testing/paged.py:48): the fp32 side of the 2x tolerance rule."""
    out = torch.empty_like(query, dtype=out_dtype or query.dtype)
    n_q_heads = query.shape[1]
    n_kv_heads, block_size, head_size = value_cache.shape[1:]
    group = n_q_heads // n_kv_heads
    lens = context_lens.cpu().tolist()
    for i in range(query.shape[0]):
        ctx = int(lens[i])
        n_blk = (ctx + block_size - 1) // block_size
        ids = block_tables[i, :n_blk].long()
        # (n_blk, kv_heads, block, head) -> (kv_heads, n_blk*block, head)[:ctx]
        keys = key_cache.index_select(0, ids).permute(1, 0, 2, 3).reshape(n_kv_heads, -1, head_size)[:, :ctx]
        values = value_cache.index_select(0, ids).permute(1, 0, 2, 3).reshape(n_kv_heads, -1, head_size)[:, :ctx]
        if group > 1:
            keys = keys.repeat_interleave(group, dim=0)
            values = values.repeat_interleave(group, dim=0)
        qi = query[i].float().unsqueeze(1)                            # (heads, 1, head)
        scores = torch.bmm(qi, keys.float().transpose(1, 2)) * scale
        probs = torch.softmax(scores, dim=-1)
        oi = torch.bmm(probs, values.float()).squeeze(1)
        out[i].copy_(oi.to(out.dtype))
    return out


def paged_attention_same_precision(query, key_cache, value_cache, block_tables, context_lens, scale):
    """The same-precision PyTorch path for paged decode, which the reference does not have (its test
    is an allclose, tests/flag_attn/test_paged_attention.py:62): per sequence, the flash oracle of
    src/flag_attn/testing/flash.py:5-70 with upcast=False on the single query token against the
    densely gathered keys and values, i.e. matmuls in the cache dtype and an fp32 softmax.  With it
    the reference's 2x rule (kernel error <= 2 x error of this path, both against fp32) applies to
    paged_attention too."""
    from .flash import flash_attention
    out = torch.empty_like(query)
    block_size = value_cache.shape[2]
    lens = context_lens.cpu().tolist()
    for i in range(query.shape[0]):
        ctx = int(lens[i])
        ids = block_tables[i, :(ctx + block_size - 1) // block_size].long()
        keys, values = _gather(key_cache, ids, ctx), _gather(value_cache, ids, ctx)
        o = flash_attention(query[i][None, :, None, :], keys[None], values[None], False,
                            sm_scale=scale, upcast=False)
        out[i].copy_(o[0, :, 0, :])
    return out


def cache_append(key, value, key_cache, value_cache, slot_mapping):
    """Token-by-token restatement of the paged-cache writer (the layout paged_attention reads:
    src/flag_attn/testing/paged.py:31-37).  The reference has no writer, so this has no fixture of
    its own; the round trip append -> paged_attention is held to the pinned read-side oracle."""
    block = key_cache.shape[2]
    for i, slot in enumerate(slot_mapping.tolist()):
        if slot < 0:
            continue
        key_cache[slot // block, :, slot % block, :] = key[i]
        value_cache[slot // block, :, slot % block, :] = value[i]
