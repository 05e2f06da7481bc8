"""Multi-GPU helpers: how the operators are sharded over one process per GPU.

The operators are stateless and per-device, and every (batch, head) pair of flash / piecewise
attention and every sequence of paged attention is independent, so a multi-GPU run needs no
collective on the data path: each rank computes its shard, and one all_gather reassembles the
outputs only where a consumer wants the full tensor.

The exception is a sequence too long for one GPU: ring_flash_attention shards the SEQUENCE over
the ranks and passes key / value shards round a ring, forward and backward (the gradients of a
shard travel round the ring with it).
"""
import torch


def shard_batch_heads(B, Hk, world_size, rank):
    """Splits the flattened (batch, kv head) pairs into `world_size` contiguous, near-equal runs and
    returns the run of `rank` as a list of (b, kv_head_begin, kv_head_end).  Sharding by kv head keeps
    every GQA group (the query heads that share one kv head) on one rank."""
    total = B * Hk
    base, extra = divmod(total, world_size)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    out = []
    i = begin
    while i < end:
        b, h = divmod(i, Hk)
        run = min(end - i, Hk - h)
        out.append((b, h, h + run))
        i += run
    return out


def shard_sequences_lpt(context_lens, world_size):
    """Longest-processing-time assignment of decode sequences to ranks: sequences sorted by context
    length (longest first) each go to the currently lightest rank.  Returns a list of index lists."""
    lens = [int(x) for x in context_lens]
    order = sorted(range(len(lens)), key=lambda i: (-lens[i], i))
    loads = [0] * world_size
    shards = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        shards[r].append(i)
        loads[r] += lens[i]
    return [sorted(s) for s in shards]


def all_gather_rows(local, counts, group=None):
    """all_gather of per-rank tensors whose first dimension differs (`counts[r]` rows on rank r);
    returns the list of all ranks' tensors.  Pads to the largest count, so any backend works."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    pad = max(counts)
    buf = torch.zeros((pad,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    buf[: local.shape[0]] = local
    gathered = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(gathered, buf, group=group)
    return [g[: counts[r]] for r, g in enumerate(gathered)]


def max_over_ranks(value, device, group=None):
    """Maximum of a Python float over all ranks (device-side timing is reported as the slowest rank)."""
    import torch.distributed as dist
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def combine_partial_attention(o_a, lse_a, o_b, lse_b):
    """Merges two attention results over disjoint key sets for the same queries, each normalised
    over its own keys with natural-log normaliser `lse` (B, H, M): the softmax over the union is
    o = o_a * exp(lse_a - lse) + o_b * exp(lse_b - lse), lse = logaddexp(lse_a, lse_b).  The rule of
    the reference's split-KV combine (src/flag_attn/split_kv.py:170-227) applied to two parts; rows
    without any key in either part (lse = -inf) stay zero.  fp32 in, fp32 out."""
    lse = torch.logaddexp(lse_a, lse_b)
    safe = torch.where(torch.isinf(lse) & (lse < 0), torch.zeros_like(lse), lse)
    w_a = torch.exp(lse_a - safe).unsqueeze(-1)
    w_b = torch.exp(lse_b - safe).unsqueeze(-1)
    return o_a * w_a + o_b * w_b, lse


def _ring_forward(q, k, v, causal, sm_scale, group, attention):
    """The forward ring: returns (o, log_normalizer) of the local queries over all ranks' keys."""
    world, rank, nxt, prv = _ring_peers(group)
    if causal:
        assert q.shape[2] == k.shape[2], "causal ring attention needs as many queries as keys per rank"
    k_cur, v_cur = k.contiguous(), v.contiguous()
    o_acc = lse_acc = None
    for step in range(world):
        owner = (rank - step) % world            # whose keys / values are in hand
        reqs, kv_nxt = ([], None) if step == world - 1 else _exchange([k_cur, v_cur], nxt, prv, group)
        if not causal or owner <= rank:
            o_j, lse_j = attention(q, k_cur, v_cur, causal and owner == rank, sm_scale)
            o_j, lse_j = o_j.float(), lse_j.float()
            if o_acc is None:
                o_acc, lse_acc = o_j, lse_j
            else:
                o_acc, lse_acc = combine_partial_attention(o_acc, lse_acc, o_j, lse_j)
        for req in reqs:
            req.wait()
        if kv_nxt is not None:
            k_cur, v_cur = kv_nxt
    return o_acc.to(q.dtype), lse_acc


def _ring_peers(group):
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    peer = (lambda i: dist.get_global_rank(group, i)) if group is not None else (lambda i: i)
    return world, rank, peer((rank + 1) % world), peer((rank - 1) % world)


def _exchange(tensors, nxt, prv, group):
    """Posts the sends of `tensors` to the next rank and the receives of their successors from the
    previous one; returns (requests, received tensors)."""
    import torch.distributed as dist
    recv = [torch.empty_like(t) for t in tensors]
    ops = [dist.P2POp(dist.isend, t, nxt, group) for t in tensors] + \
          [dist.P2POp(dist.irecv, t, prv, group) for t in recv]
    return dist.batch_isend_irecv(ops), recv


def _ring_backward(q, k, v, o, lse, do, causal, sm_scale, group, backward):
    """Gradients of the ring forward.  `backward(q, k, v, o, lse, do, causal, sm_scale)` is the
    single-device backward evaluated with the GLOBAL o and log-normaliser of the local rows, so what
    it returns for the shard in hand are that shard's exact contributions: dq is summed locally, and
    the dk / dv of a shard travel round the ring WITH the shard (fp32), arriving back at its owner
    after the last hop."""
    world, rank, nxt, prv = _ring_peers(group)
    k_cur, v_cur = k.contiguous(), v.contiguous()
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    dk_cur = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
    dv_cur = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
    for step in range(world):
        owner = (rank - step) % world
        kv_reqs, kv_nxt = ([], None) if step == world - 1 else _exchange([k_cur, v_cur], nxt, prv, group)
        if not causal or owner <= rank:
            dq_j, dk_j, dv_j = backward(q, k_cur, v_cur, o, lse, do, causal and owner == rank, sm_scale)
            dq += dq_j.float()
            dk_cur += dk_j.float()
            dv_cur += dv_j.float()
        g_reqs = []
        if world > 1:
            g_reqs, (dk_cur, dv_cur) = _exchange([dk_cur, dv_cur], nxt, prv, group)
        for req in kv_reqs + g_reqs:
            req.wait()
        if kv_nxt is not None:
            k_cur, v_cur = kv_nxt
    return dq.to(q.dtype), dk_cur.to(k.dtype), dv_cur.to(v.dtype)


class _RingFlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, sm_scale, group, attention, backward):
        o, lse = _ring_forward(q, k, v, causal, sm_scale, group, attention)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.args = (causal, sm_scale, group, backward)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        causal, sm_scale, group, backward = ctx.args
        dq, dk, dv = _ring_backward(q, k, v, o, lse, do.contiguous(), causal, sm_scale, group, backward)
        return dq, dk, dv, None, None, None, None, None


def ring_flash_attention(q, k, v, causal=False, sm_scale=None, group=None, attention=None, backward=None):
    """flash_attention with the SEQUENCE sharded over the ranks of `group`: every rank passes in ITS
    rows of q and ITS keys / values (equal lengths on all ranks, rank order = sequence order) and gets
    back (o, log_normalizer) of its rows over ALL keys; differentiable with respect to q, k, v.

    The key / value shards travel round a ring, one hop per step (point-to-point sends of the
    process group, posted before the step's attention call so that they overlap it); each step
    attends the local queries to the shard in hand with the ordinary single-device operator and folds
    the result in with the log-normaliser rule of the split-KV combine.  Under `causal` the global
    mask is bottom-right aligned over the whole sequence, which needs as many queries as keys per
    rank: a shard from an earlier rank is fully visible, the rank's own shard is causal, later
    shards are skipped.  The backward makes the same tour with the single-device backward kernels,
    fed the global o and log-normaliser; every rank of the group must call it.

    `attention(q, k, v, causal, sm_scale) -> (o, log_normalizer)` and
    `backward(q, k, v, o, log_normalizer, do, causal, sm_scale) -> (dq, dk, dv)` default to this
    package's kernels; tests inject PyTorch statements of both to run the ring on CPU ranks."""
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    if attention is None:
        from .flash import attention as flash_attention

        def attention(q_, k_, v_, causal_, scale_):
            o_, lse_, *_ = flash_attention(q_, k_, v_, causal=causal_, sm_scale=scale_,
                                           return_log_normalizer=True)
            return o_, lse_
    if backward is None:
        from . import _C
        from .flash import _backward

        def backward(q_, k_, v_, o_, lse_, do_, causal_, scale_):
            q_, k_, v_, o_ = (_C.kernel_ready(t) for t in (q_, k_, v_, o_))
            return _backward(q_, k_, v_, o_, lse_.contiguous(), do_, causal_, scale_)
    return _RingFlashAttention.apply(q, k, v, causal, sm_scale, group, attention, backward)
