"""Multi-GPU helpers: how the operators are sharded over one process per GPU.

The operators are stateless and per-device, and every (batch, head) pair of flash / piecewise
attention and every sequence of paged attention is independent, so a multi-GPU run needs no
collective on the data path: each rank computes its shard, and one all_gather reassembles the
outputs only where a consumer wants the full tensor.
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
