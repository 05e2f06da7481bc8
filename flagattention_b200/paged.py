"""paged_attention: single-token decode over a block-table KV cache.

Mirrors src/flag_attn/paged.py:6-163: same arguments, same split rule
(num_splits == 0 picks it automatically, 1 disables it, > 1 fixes the count),
returns a new tensor shaped like `query`.
"""
import torch

from . import _C

__all__ = ["attention", "reshape_and_cache"]


def _next_power_of_2(n):
    return 1 << (max(int(n), 1) - 1).bit_length()


def _cdiv(a, b):
    return (a + b - 1) // b


def plan_partitions(num_seqs, num_kv_heads, kv_block_size, max_context_len, num_splits, num_sms):
    """Returns (num_splits, partition_size) by the reference's rule
    (src/flag_attn/paged.py:40-53); partition_size is 0 when there is one pass."""
    partition_size = 0
    if num_splits == 0:
        if num_seqs * num_kv_heads > 2 * num_sms:
            num_splits = 1
            if max_context_len >= 4096:
                partition_size = max(256, kv_block_size)
                num_splits = _cdiv(max_context_len, partition_size)
        else:
            partition_size = max(256, kv_block_size)
            num_splits = _cdiv(max_context_len, partition_size)
            if max_context_len <= 1024 or kv_block_size >= 256:
                num_splits = 1
    elif num_splits > 1:
        partition_size = _next_power_of_2(_cdiv(max_context_len, num_splits))
    if num_splits == 1:
        partition_size = 0
    return num_splits, partition_size


def attention(query, key_cache, value_cache, context_lens, block_tables, attn_scale,
              max_context_len, num_splits=0):
    """query [num_seqs, kv_heads * group, head]; caches [num_blocks, kv_heads, block, head]
    with identical strides; context_lens [num_seqs] int32; block_tables
    [num_seqs, max_blocks] int32 or int64."""
    num_seqs, num_q_heads, head_size = query.shape
    num_kv_heads, kv_block_size = key_cache.shape[1], key_cache.shape[2]
    assert key_cache.shape[3] == head_size
    assert num_q_heads % num_kv_heads == 0
    query_group_size = num_q_heads // num_kv_heads
    assert head_size in (16, 32, 64, 128, 256, 512), f"head_size={head_size}"
    assert head_size <= 256, "head_size 512 is not built for B200 yet"
    assert query_group_size == 1 or kv_block_size >= 16, f"kv_block_size={kv_block_size}"
    assert key_cache.stride() == value_cache.stride(), "key and value cache must share strides"
    assert query.is_cuda and query.dtype == key_cache.dtype == value_cache.dtype
    assert block_tables.dtype in (torch.int32, torch.int64)
    for name, t in (("key_cache", key_cache), ("value_cache", value_cache),
                    ("context_lens", context_lens), ("block_tables", block_tables)):
        assert t.device == query.device, f"{name} is on {t.device}, query on {query.device}"

    if context_lens.dtype != torch.int32:
        context_lens = context_lens.to(torch.int32)
    context_lens = context_lens.contiguous()
    if block_tables.stride(-1) != 1:
        block_tables = block_tables.contiguous()
    if query.stride(-1) != 1 or query.data_ptr() % 16 or query.stride(0) % 8 or query.stride(1) % 8:
        query = query.contiguous()
    if key_cache.stride(-1) != 1 or any(s % 8 for s in key_cache.stride()[:-1]):
        key_cache, value_cache = key_cache.contiguous(), value_cache.contiguous()

    lib = _C.load()
    with torch.cuda.device(query.device):
        num_sms = torch.cuda.get_device_properties(query.device).multi_processor_count
        num_splits, partition_size = plan_partitions(num_seqs, num_kv_heads, kv_block_size,
                                                     max_context_len, num_splits, num_sms)
        if partition_size:
            assert partition_size >= kv_block_size and partition_size % kv_block_size == 0, \
                f"partition_size={partition_size}, kv_block_size={kv_block_size}"
            assert partition_size % 16 == 0, f"partition_size={partition_size}"

        out = torch.empty(query.shape, dtype=query.dtype, device=query.device)
        args = _C.PagedArgs()
        args.dtype = _C.dtype_code(query.dtype)
        args.num_seqs, args.num_q_heads, args.num_kv_heads = num_seqs, num_q_heads, num_kv_heads
        args.head_size, args.block_size = head_size, kv_block_size
        args.max_context_len = int(max_context_len)
        args.block_table_is_i64 = 1 if block_tables.dtype == torch.int64 else 0
        args.partition_size = partition_size
        args.attn_scale = float(attn_scale)
        args.query, args.q_stride_s, args.q_stride_h = query.data_ptr(), query.stride(0), query.stride(1)
        args.key_cache, args.value_cache = key_cache.data_ptr(), value_cache.data_ptr()
        args.kv_stride_b, args.kv_stride_h, args.kv_stride_t = key_cache.stride()[:3]
        args.context_lens = context_lens.data_ptr()
        args.block_tables, args.bt_stride_s = block_tables.data_ptr(), block_tables.stride(0)
        args.out, args.o_stride_s, args.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
        stream = _C.stream_ptr(query.device)

        if partition_size:
            P = _cdiv(int(max_context_len), partition_size)
            part_out = torch.empty((num_seqs, num_q_heads, P, head_size), dtype=torch.float32,
                                   device=query.device)
            part_max = torch.empty((num_seqs, num_q_heads, P), dtype=torch.float32,
                                   device=query.device)
            part_sum = torch.empty_like(part_max)
            args.part_out, args.part_max, args.part_sum = (part_out.data_ptr(), part_max.data_ptr(),
                                                           part_sum.data_ptr())
        _C.check(lib.fa_paged_decode(_C.byref(args), stream), "fa_paged_decode")
        if partition_size:
            _C.check(lib.fa_paged_reduce(_C.byref(args), stream), "fa_paged_reduce")
    return out


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping):
    """Writes new tokens into the paged caches `attention` reads.

    key, value: [num_tokens, kv_heads, head]; caches [num_blocks, kv_heads, block, head];
    slot_mapping [num_tokens] integer: token i goes to block slot // block, position slot % block;
    negative slots are skipped.  The reference has no writer (its tests fill the caches with random
    numbers); a serving loop runs this step right before the decode kernel."""
    import ctypes
    num_tokens, num_kv_heads, head_size = key.shape
    assert value.shape == key.shape and key_cache.shape == value_cache.shape
    assert key_cache.shape[1] == num_kv_heads and key_cache.shape[3] == head_size
    assert key.dtype == value.dtype == key_cache.dtype == value_cache.dtype
    assert key_cache.stride() == value_cache.stride(), "key and value cache must share strides"
    assert key_cache.stride(-1) == 1 and all(s % 8 == 0 for s in key_cache.stride()[:-1]), \
        "caches need unit inner stride and 16-byte aligned rows"
    assert slot_mapping.numel() == num_tokens
    assert key.is_cuda, "inputs must be CUDA tensors"
    for name, t in (("value", value), ("key_cache", key_cache), ("value_cache", value_cache),
                    ("slot_mapping", slot_mapping)):
        assert t.device == key.device, f"{name} is on {t.device}, key on {key.device}"
    if key.stride() != value.stride() or key.stride(-1) != 1 or any(s % 8 for s in key.stride()[:-1]) \
            or key.data_ptr() % 16 or value.data_ptr() % 16:
        key, value = key.contiguous(), value.contiguous()
    slots = slot_mapping.to(torch.int64).contiguous()
    lib = _C.load()
    with torch.cuda.device(key.device):
        st = lib.fa_paged_cache_append(
            _C.dtype_code(key.dtype), num_tokens, num_kv_heads, head_size, key_cache.shape[2],
            _C.fptr(key), _C.fptr(value), ctypes.c_int64(key.stride(0)), ctypes.c_int64(key.stride(1)),
            _C.fptr(key_cache), _C.fptr(value_cache), ctypes.c_int64(key_cache.stride(0)),
            ctypes.c_int64(key_cache.stride(1)), ctypes.c_int64(key_cache.stride(2)),
            _C.fptr(slots), _C.stream_ptr(key.device))
    _C.check(st, "fa_paged_cache_append")
