"""flash_attention: host side of the B200 kernels.

Mirrors the operator interface of the reference (src/flag_attn/flash.py:23-286):
same argument names, same return structure (the output alone, or the 5-tuple
when any return_* flag is set), same AssertionErrors on bad shapes, autograd
through q, k, v only.  The kernels run on the current CUDA stream of the
inputs' device.
"""
import ctypes
import math

import torch

from . import _C
from .dropout import philox_cuda_seed_offset
from .split_kv import get_fwd_config as get_fwd_config_kv_split
from .split_kv import num_splits_herustic, _splitkv_forward

__all__ = ["attention", "set_backward_mode", "get_backward_mode", "backward_mode"]

# Which kernels compute the gradients at head_dim 64 / 128:
#   "one_pass"   one kernel for dq, dk, dv (five matrix products per tile); dq is summed with fp32
#                reductions in global memory, so it is reproducible to fp32 rounding only;
#   "two_kernel" a dK/dV kernel and a dQ kernel without any global reduction or atomic (seven
#                products per tile), the split of the reference (src/flag_attn/flash.py:204-249):
#                every gradient is bitwise reproducible;
#   "auto"       (default) "two_kernel" while torch.are_deterministic_algorithms_enabled(),
#                else "one_pass".
_BACKWARD_MODES = ("auto", "one_pass", "two_kernel")
_backward_mode = "auto"


def set_backward_mode(mode):
    """Selects the backward kernels of flash_attention and piecewise_attention (see above);
    returns the previous mode."""
    global _backward_mode
    assert mode in _BACKWARD_MODES, f"mode must be one of {_BACKWARD_MODES}"
    previous, _backward_mode = _backward_mode, mode
    return previous


def get_backward_mode():
    return _backward_mode


class backward_mode:
    """`with backward_mode("two_kernel"): loss.backward()`"""

    def __init__(self, mode):
        assert mode in _BACKWARD_MODES, f"mode must be one of {_BACKWARD_MODES}"
        self.mode = mode

    def __enter__(self):
        self.previous = set_backward_mode(self.mode)
        return self

    def __exit__(self, *exc):
        set_backward_mode(self.previous)
        return False


def use_one_pass_backward():
    if _backward_mode == "auto":
        return not torch.are_deterministic_algorithms_enabled()
    return _backward_mode == "one_pass"


def get_fwd_config(B, H, M, N, D, causal):
    """Tile shape used by the one-pass forward kernel: (BLOCK_M, BLOCK_N, stages, warps).
    Kept for interface compatibility (src/flag_attn/flash.py:290-322); the tile
    shape is compiled into the kernels, so overriding this has no effect."""
    return (128, 64, 2, 6)


def get_bwd_config(B, H, M, N, D, causal):
    """Counterpart of src/flag_attn/flash.py:493-519; informational only."""
    return (128, 128, 3, 18)


def _forward(q, k, v, causal, sm_scale, dropout_p=0.0, seed=0, offset=0):
    B, H, M, D = q.shape
    N, Hk = k.shape[2], k.shape[1]
    lib = _C.load()
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    L = torch.empty((B, H, M), device=q.device, dtype=torch.float32)
    shape = _C.flash_shape(q.dtype, B, H, Hk, M, N, D, causal, sm_scale, dropout_p, seed, offset)
    tq, tk, tv, to = _C.tensor4(q), _C.tensor4(k), _C.tensor4(v), _C.tensor4(o)
    st = lib.fa_flash_fwd(_C.byref(shape), _C.byref(tq), _C.byref(tk), _C.byref(tv), _C.byref(to),
                          _C.fptr(L), _C.stream_ptr(q.device))
    _C.check(st, "fa_flash_fwd")
    return o, L


_identity_tables = {}


def _identity_block_table(B, blocks_per_batch, id_stride, device):
    """(block_tables, context_lens) with block_tables[b, c] = b * id_stride + c, cached: the block
    table under which a (B, Hk, N, D) key tensor is, in place, a paged cache of 16-token blocks."""
    key = (B, blocks_per_batch, id_stride, str(device))
    tab = _identity_tables.get(key)
    if tab is None:
        if len(_identity_tables) >= 8:
            _identity_tables.clear()
        tab = (torch.arange(B, device=device, dtype=torch.int32)[:, None] * id_stride +
               torch.arange(blocks_per_batch, device=device, dtype=torch.int32)[None, :]).contiguous()
        lens = torch.full((B,), blocks_per_batch * 16, dtype=torch.int32, device=device)
        tab = (tab, lens)
        _identity_tables[key] = tab
    return tab


_DECODE_MAX_ROWS = 64   # query rows (group x queries) per kv head the gather kernel is given


def _decode_covered(q, k, v, causal=False):
    """Decode-shaped forward (a few queries per head, at most _DECODE_MAX_ROWS rows per kv head)
    that the paged-decode kernels can run directly on k and v: the keys of a batch element are then
    a block table of 16-token blocks in place."""
    B, H, M, D = q.shape
    N, Hk = k.shape[2], k.shape[1]
    if M < 1 or N % 16 != 0 or N == 0 or (H // Hk) * M > _DECODE_MAX_ROWS:
        return False
    if causal and M > 1 and N < M:
        return False      # rows that see no key at all: the tile kernels give them their zeros
    if k.stride() != v.stride() or k.stride(3) != 1 or k.data_ptr() % 16 or v.data_ptr() % 16:
        return False
    sb, sh, sl, _ = k.stride()
    if sl % 8 or sh % 8 or sb % (16 * sl) or (B * (sb // (16 * sl))) >= 2 ** 31:
        return False
    return True


def _decode_forward(q, k, v, sm_scale, causal=False):
    """o for a few queries per head through fa_paged_decode / fa_paged_reduce (an HBM-bound gather
    kernel that streams K and V once per 16 query rows of a kv head), instead of the split-KV tile
    kernels.  The M queries of a head go in as M consecutive "query heads" of its kv head."""
    B, H, M, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    BS = 16
    sb, sh, sl, _ = k.stride()
    lib = _C.load()
    num_sms = torch.cuda.get_device_properties(q.device).multi_processor_count
    # partitions of the key axis: enough (batch, kv head, partition) CTAs for about eight waves,
    # each long enough (>= 256 keys) to amortise its pipeline fill
    partition_size = 256
    while partition_size < 8192 and B * Hk * (N // (2 * partition_size)) >= 8 * num_sms:
        partition_size *= 2
    if N <= partition_size:
        partition_size = 0   # one pass, no reduction kernel
    table, ctx_lens = _identity_block_table(B, N // BS, sb // (BS * sl), q.device)
    q2 = q.reshape(B, H * M, D)
    if q2.stride(-1) != 1 or q2.data_ptr() % 16 or q2.stride(0) % 8 or q2.stride(1) % 8:
        q2 = q2.contiguous()
    o = torch.empty((B, H, M, D), dtype=q.dtype, device=q.device)
    args = _C.PagedArgs()
    args.dtype = _C.dtype_code(q.dtype)
    args.num_seqs, args.num_q_heads, args.num_kv_heads = B, H * M, Hk
    args.causal_rows = M if (causal and M > 1) else 0
    args.head_size, args.block_size = D, BS
    args.max_context_len = N
    args.block_table_is_i64 = 0
    args.partition_size = partition_size
    args.attn_scale = float(sm_scale)
    args.query, args.q_stride_s, args.q_stride_h = q2.data_ptr(), q2.stride(0), q2.stride(1)
    args.key_cache, args.value_cache = k.data_ptr(), v.data_ptr()
    args.kv_stride_b, args.kv_stride_h, args.kv_stride_t = BS * sl, sh if Hk > 1 else 0, sl
    args.context_lens = ctx_lens.data_ptr()
    args.block_tables, args.bt_stride_s = table.data_ptr(), table.stride(0)
    args.out, args.o_stride_s, args.o_stride_h = o.data_ptr(), H * M * D, D
    stream = _C.stream_ptr(q.device)
    if partition_size:
        P = (N + partition_size - 1) // partition_size
        part_out = torch.empty((B, H * M, P, D), dtype=torch.float32, device=q.device)
        part_max = torch.empty((B, H * M, P), dtype=torch.float32, device=q.device)
        part_sum = torch.empty_like(part_max)
        args.part_out, args.part_max, args.part_sum = (part_out.data_ptr(), part_max.data_ptr(),
                                                       part_sum.data_ptr())
    _C.check(lib.fa_paged_decode(_C.byref(args), stream), "fa_paged_decode")
    if partition_size:
        _C.check(lib.fa_paged_reduce(_C.byref(args), stream), "fa_paged_reduce")
    return o


def _total_attention(q, k, L, causal, sm_scale):
    B, H, M, D = q.shape
    N, Hk = k.shape[2], k.shape[1]
    lib = _C.load()
    tot = torch.empty((B, H, N), device=q.device, dtype=torch.float32)
    shape = _C.flash_shape(q.dtype, B, H, Hk, M, N, D, causal, sm_scale)
    tq, tk = _C.tensor4(q), _C.tensor4(k)
    st = lib.fa_total_attention(_C.byref(shape), _C.byref(tq), _C.byref(tk), _C.fptr(L),
                                _C.fptr(tot), _C.stream_ptr(q.device))
    _C.check(st, "fa_total_attention")
    return tot


def _backward(q, k, v, o, L, do, causal, sm_scale, mark=None, dropout_p=0.0, seed=0, offset=0):
    """Launches delta, dK/dV and dQ. `mark(name)`, when given, is called before the first launch
    and after each one (the benchmark records CUDA events there)."""
    B, H, M, D = q.shape
    N, Hk = k.shape[2], k.shape[1]
    lib = _C.load()
    do = _C.kernel_ready(do)
    with torch.cuda.device(q.device):
        stream = _C.stream_ptr(q.device)
        shape = _C.flash_shape(q.dtype, B, H, Hk, M, N, D, causal, sm_scale, dropout_p, seed, offset)
        delta = torch.empty_like(L)
        # dk / dv come out with Hk heads: the group sum is done in the kernel
        dk = torch.empty((B, Hk, N, D), dtype=k.dtype, device=q.device)
        dv = torch.empty((B, Hk, N, D), dtype=v.dtype, device=q.device)
        dq = torch.empty((B, H, M, D), dtype=q.dtype, device=q.device)
        tq, tk, tv, to, tdo = (_C.tensor4(x) for x in (q, k, v, o, do))
        tdk, tdv, tdq = _C.tensor4(dk), _C.tensor4(dv), _C.tensor4(dq)
        if mark:
            mark("start")
        ws_bytes = (lib.fa_flash_bwd_fused_workspace_bytes(_C.byref(shape))
                    if use_one_pass_backward() else 0)
        if ws_bytes > 0:
            # one pass over the score tiles; dq is accumulated in an fp32 workspace, which the
            # delta kernel fills with zeros on its way (two memory-bound passes in one launch)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
            st = lib.fa_flash_bwd_delta_zero(_C.byref(shape), _C.byref(to), _C.byref(tdo), _C.fptr(delta),
                                             _C.fptr(ws), ctypes.c_int64(ws_bytes), stream)
            _C.check(st, "fa_flash_bwd_delta_zero")
        else:
            st = lib.fa_flash_bwd_delta(_C.byref(shape), _C.byref(to), _C.byref(tdo),
                                        _C.fptr(delta), stream)
            _C.check(st, "fa_flash_bwd_delta")
        if mark:
            mark("delta")
        if ws_bytes > 0:
            args = (_C.byref(shape), _C.byref(tq), _C.byref(tk), _C.byref(tv), _C.byref(tdo),
                    _C.fptr(L), _C.fptr(delta), _C.byref(tdq), _C.byref(tdk), _C.byref(tdv),
                    _C.fptr(ws), ctypes.c_int64(ws_bytes))
            if mark:
                # the parts of the call one by one, so that each can be timed
                st = 0
                for stage, name in ((2, "dkdvdq"), (4, "dq_convert")):
                    st = lib.fa_flash_bwd_fused_stages(*args, stage, stream)
                    if st != 0:
                        break
                    mark(name)
            else:
                st = lib.fa_flash_bwd_fused_stages(*args, 6, stream)   # kernel + dq conversion
            # a layout the one-pass kernel cannot map (a broadcast stride) goes to the pair below
            if st != _C.FA_ERR_UNSUPPORTED:
                _C.check(st, "fa_flash_bwd_fused")
                return dq, dk, dv
        st = lib.fa_flash_bwd_dkdv(_C.byref(shape), _C.byref(tq), _C.byref(tk), _C.byref(tv),
                                   _C.byref(tdo), _C.fptr(L), _C.fptr(delta), _C.byref(tdk),
                                   _C.byref(tdv), stream)
        _C.check(st, "fa_flash_bwd_dkdv")
        if mark:
            mark("dkdv")
        st = lib.fa_flash_bwd_dq(_C.byref(shape), _C.byref(tq), _C.byref(tk), _C.byref(tv),
                                 _C.byref(tdo), _C.fptr(L), _C.fptr(delta), _C.byref(tdq), stream)
        _C.check(st, "fa_flash_bwd_dq")
        if mark:
            mark("dq")
    return dq, dk, dv


class FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, dropout_p, return_log_normalizer,
                return_total_attention, return_seed_offset):
        Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
        assert Dq == Dk == Dv, "feature size of q, k, v should be equal"
        assert Dk in {16, 32, 64, 128}
        assert 0.0 <= dropout_p < 1.0, f"dropout_p={dropout_p}"
        assert q.is_cuda and k.is_cuda and v.is_cuda, "inputs must be CUDA tensors"
        assert q.dtype == k.dtype == v.dtype

        B, H, M, D = q.shape
        N = k.shape[2]
        Hk, Hv = k.shape[1], v.shape[1]
        assert Hk == Hv, "num of heads in k and v should be equal"
        assert H % Hk == 0, "number of heads in q must be a multiple of that in k & v"

        if sm_scale is None:
            sm_scale = 1. / math.sqrt(D)

        q, k, v = _C.kernel_ready(q), _C.kernel_ready(k), _C.kernel_ready(v)

        has_extra_return = True in (return_log_normalizer, return_total_attention, return_seed_offset)
        if (M <= 16 and dropout_p == 0 and not has_extra_return and not any(ctx.needs_input_grad[:3])
                and _decode_covered(q, k, v, causal)):
            # decode step without gradients: nothing but o is needed.  One query always goes to the
            # gather kernel, which streams K and V once; a few queries go there when the reference
            # would split the keys (src/flag_attn/flash.py:59-61), i.e. when the tile grid alone
            # would leave most of the GPU idle.
            with torch.cuda.device(q.device):
                take = M == 1
                if not take:
                    num_sms = torch.cuda.get_device_properties(q.device).multi_processor_count
                    cfg = get_fwd_config_kv_split(B, H, M, N, D, causal)
                    take = num_splits_herustic(B, H, M, N, cfg[0], cfg[1], num_sms, 128) > 1
                if take:
                    return _decode_forward(q, k, v, sm_scale, causal)

        with torch.cuda.device(q.device):
            # dropout: one Philox counter per element of the (B, H, M, N) attention matrix
            is_dropout = dropout_p > 0
            if is_dropout:
                seed, offset = philox_cuda_seed_offset(B * H * M * N, q.device)
            else:
                seed, offset = 0, 0

            num_sms = torch.cuda.get_device_properties(q.device).multi_processor_count
            cfg = get_fwd_config_kv_split(B, H, M, N, D, causal)
            S = num_splits_herustic(B, H, M, N, cfg[0], cfg[1], num_sms, 128)
            if S > 1:
                assert not is_dropout, "Cannot apply dropout with splitkv."
                o, L = _splitkv_forward(q, k, v, causal, sm_scale, S)
            else:
                o, L = _forward(q, k, v, causal, sm_scale, dropout_p, seed, offset)
            tot_attn = None
            if return_total_attention:
                tot_attn = _total_attention(q, k, L, causal, sm_scale)

        ctx.save_for_backward(q, k, v, o, L)
        ctx.sm_scale = sm_scale
        ctx.causal = causal
        ctx.dropout_p = dropout_p
        ctx.seed = seed
        ctx.offset = offset

        has_extra_return = True in (return_log_normalizer, return_total_attention, return_seed_offset)
        if has_extra_return:
            return (o, L if return_log_normalizer else None, tot_attn,
                    seed if is_dropout and return_seed_offset else None,
                    offset if is_dropout and return_seed_offset else None)
        return o

    @staticmethod
    def backward(ctx, do, *ignored):
        q, k, v, o, L = ctx.saved_tensors
        dq, dk, dv = _backward(q, k, v, o, L, do, ctx.causal, ctx.sm_scale, None, ctx.dropout_p,
                               ctx.seed, ctx.offset)
        return dq, dk, dv, None, None, None, None, None, None


def attention(q, k, v, causal=False, sm_scale=None, dropout_p=0.0,
              return_log_normalizer=False, return_total_attention=False, return_seed_offset=False):
    """FlashAttention forward/backward on B200.

    Arguments:
        q: (batch, heads_q, seqlen_q, headdim); k, v: (batch, heads_k, seqlen_k, headdim),
           fp16 or bf16 CUDA tensors, heads_q a multiple of heads_k, headdim in {16,32,64,128}.
        causal: bottom-right aligned causal mask.
        sm_scale: softmax scale, default 1/sqrt(headdim).
        dropout_p: dropout probability on the attention weights.
        return_log_normalizer / return_total_attention / return_seed_offset: when any is set,
           returns (out, log_normalizer | None, total_attention | None, seed | None, offset | None);
           seed and offset are the Philox seed and starting offset used by dropout (None without).

    Returns out, shape of q; log_normalizer (batch, heads_q, seqlen_q) fp32;
    total_attention (batch, heads_q, seqlen_k) fp32.
    """
    return FlashAttention.apply(q, k, v, causal, sm_scale, dropout_p, return_log_normalizer,
                                return_total_attention, return_seed_offset)
