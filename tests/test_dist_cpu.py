"""Multi-rank host logic on CPU: shard helpers, and a world_size-2 gloo run that shards a decode batch,
computes each shard with the oracle (the stand-in for the per-rank GPU operator) and reassembles it."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from flagattention_b200 import dist as fdist


def test_shard_batch_heads_partitions_exactly():
    for B, Hk, world in [(4, 32, 8), (4, 32, 3), (1, 48, 8), (2, 1, 4), (3, 5, 2)]:
        seen = []
        sizes = []
        for r in range(world):
            runs = fdist.shard_batch_heads(B, Hk, world, r)
            n = 0
            for b, h0, h1 in runs:
                assert 0 <= b < B and 0 <= h0 < h1 <= Hk
                seen += [(b, h) for h in range(h0, h1)]
                n += h1 - h0
            sizes.append(n)
        assert sorted(seen) == [(b, h) for b in range(B) for h in range(Hk)]
        assert max(sizes) - min(sizes) <= 1


def test_shard_sequences_lpt_balances():
    gen = torch.Generator().manual_seed(1)
    lens = torch.randint(1024, 32769, (64,), generator=gen).tolist()
    for world in (1, 2, 4, 8):
        shards = fdist.shard_sequences_lpt(lens, world)
        assert sorted(i for s in shards for i in s) == list(range(64))
        loads = [sum(lens[i] for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(lens)          # LPT bound
        assert max(loads) <= 1.1 * sum(lens) / world


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    import torch.distributed as dist
    import oracle
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        gen = torch.Generator().manual_seed(5)                 # same inputs on every rank
        S, Hq, Hk, D, BS, NB = 6, 4, 2, 32, 16, 40
        lens = torch.tensor([100, 17, 64, 1, 90, 33], dtype=torch.int32)
        q = torch.randn((S, Hq, D), generator=gen).half()
        kc = torch.randn((NB, Hk, BS, D), generator=gen).half()
        vc = torch.randn((NB, Hk, BS, D), generator=gen).half()
        bt = torch.randint(0, NB, (S, 7), generator=gen)
        shards = fdist.shard_sequences_lpt(lens.tolist(), world)
        mine = shards[rank]
        idx = torch.tensor(mine, dtype=torch.long)
        local = oracle.paged_attention_gathered(q[idx], kc, vc, bt[idx], lens[idx], D ** -0.5)
        parts = fdist.all_gather_rows(local, [len(s) for s in shards])
        full = torch.empty_like(q)
        for s, part in zip(shards, parts):
            full[torch.tensor(s, dtype=torch.long)] = part
        want = oracle.paged_attention_gathered(q, kc, vc, bt, lens, D ** -0.5)
        assert torch.equal(full, want)
        slowest = fdist.max_over_ranks(1.0 + rank, torch.device("cpu"))
        assert slowest == float(world)
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_shard_and_gather(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def _warmup_worker(rank, world, port, result_dir):
    import importlib.util
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py"))
        bench = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(bench)
        # the ranks ran their first calls at different paces: rank 0 fast, rank 1 slow, rank 2 done already
        spent = [0.01, 0.2, 0.9][rank]
        n = bench.extra_warmup_calls(dist, torch.device("cpu"), 5, 0.5, spent)
        assert n == int((0.5 - 0.01) / (0.01 / 5)) + 1          # the fastest rank's proposal, on every rank
        assert bench.extra_warmup_calls(dist, torch.device("cpu"), 5, 0.5, 0.7) == 0
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_warmup_count_of_the_benchmark_is_the_same_on_every_rank(tmp_path):
    """bench.py warms up "for half a second"; the number of calls that takes must be agreed among the
    ranks, because a timed function may contain a collective (ranks that disagreed hung the 4- and
    8-GPU runs once)."""
    world = 3
    mp.spawn(_warmup_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def _ring_worker(rank, world, port, result_dir):
    import torch.distributed as dist
    from flagattention_b200 import testing
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def attention(q, k, v, causal, sm_scale):
            o, lse, _ = testing.flash_attention(q, k, v, causal, sm_scale=sm_scale,
                                                return_log_normalizer=True, upcast=True)
            return o, lse

        def backward(q, k, v, o, lse, do, causal, sm_scale):
            """The flash backward in plain fp32 torch, given the log-normaliser: P = exp(S - lse),
            dS = P * (dP - rowsum(o * do)); group sums for dk, dv."""
            G = q.shape[1] // k.shape[1]
            kx, vx = k.repeat_interleave(G, dim=1), v.repeat_interleave(G, dim=1)
            S = q @ kx.transpose(-1, -2) * sm_scale
            if causal:
                M, N = S.shape[-2:]
                keep = (torch.arange(M)[:, None] + (N - M)) >= torch.arange(N)
                S = S.masked_fill(~keep, float("-inf"))
            P = torch.exp(S - lse[..., None])
            dS = P * (do @ vx.transpose(-1, -2) - (o * do).sum(-1, keepdim=True)) * sm_scale
            dq, dk, dv = dS @ kx, dS.transpose(-1, -2) @ q, P.transpose(-1, -2) @ do
            fold = lambda t: t.reshape(t.shape[0], k.shape[1], G, *t.shape[2:]).sum(2)
            return dq, fold(dk), fold(dv)

        gen = torch.Generator().manual_seed(7)                 # same full tensors on every rank
        B, Hq, Hk, D, m = 2, 4, 2, 32, 24                     # m rows / keys per rank
        L = m * world
        q = torch.randn((B, Hq, L, D), generator=gen)
        k = torch.randn((B, Hk, L, D), generator=gen)
        v = torch.randn((B, Hk, L, D), generator=gen)
        rows = slice(rank * m, (rank + 1) * m)
        for causal in (False, True):
            o, lse = fdist.ring_flash_attention(q[:, :, rows], k[:, :, rows], v[:, :, rows], causal, None,
                                                attention=attention)
            o_full, lse_full, _ = testing.flash_attention(q, k, v, causal, return_log_normalizer=True,
                                                          upcast=True)
            assert torch.allclose(o, o_full[:, :, rows], atol=1e-5, rtol=1e-5), causal
            assert torch.allclose(lse, lse_full[:, :, rows], atol=1e-5, rtol=1e-5), causal
            # gradients: the ring's tour against autograd through the reference on the full sequence
            do = torch.randn((B, Hq, L, D), generator=torch.Generator().manual_seed(11))
            qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
            o_ref = testing.flash_attention(qf, kf, vf, causal, upcast=True)
            g_full = torch.autograd.grad(o_ref, (qf, kf, vf), do)
            ql, kl, vl = (t[:, :, rows].clone().requires_grad_() for t in (q, k, v))
            o_l, _ = fdist.ring_flash_attention(ql, kl, vl, causal, None, attention=attention,
                                                backward=backward)
            g = torch.autograd.grad(o_l, (ql, kl, vl), do[:, :, rows])
            for name, a, b in zip(("dq", "dk", "dv"), g, g_full):
                assert torch.allclose(a, b[:, :, rows], atol=2e-5, rtol=1e-4), (name, causal)
        # non-causal with more keys than queries per rank (a decode-like shard)
        kk = torch.randn((B, Hk, 40 * world, D), generator=gen)
        vv = torch.randn((B, Hk, 40 * world, D), generator=gen)
        keys = slice(rank * 40, (rank + 1) * 40)
        o, lse = fdist.ring_flash_attention(q[:, :, rows], kk[:, :, keys], vv[:, :, keys], False, 0.2,
                                            attention=attention)
        o_full, lse_full, _ = testing.flash_attention(q[:, :, rows], kk, vv, False, sm_scale=0.2,
                                                      return_log_normalizer=True, upcast=True)
        assert torch.allclose(o, o_full, atol=1e-5, rtol=1e-5)
        assert torch.allclose(lse, lse_full, atol=1e-5, rtol=1e-5)
        open(os.path.join(result_dir, f"ring{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_ring_attention_over_gloo_ranks(tmp_path, world):
    """Context-parallel forward: the ring exchange and the log-normaliser combine on CPU ranks, with
    the PyTorch reference standing in for the single-device operator."""
    mp.spawn(_ring_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ring{r}").exists() for r in range(world))


def test_combine_partial_attention_handles_rows_without_keys():
    o_a, o_b = torch.ones(1, 1, 3, 2), 3 * torch.ones(1, 1, 3, 2)
    lse_a = torch.tensor([[[0.0, float("-inf"), float("-inf")]]])
    lse_b = torch.tensor([[[0.0, 1.0, float("-inf")]]])
    o, lse = fdist.combine_partial_attention(o_a, lse_a, o_b * torch.tensor([1.0, 1.0, 0.0])[None, None, :, None],
                                             lse_b)
    assert torch.allclose(o[0, 0, 0], torch.tensor([2.0, 2.0]))          # equal weights
    assert torch.allclose(o[0, 0, 1], torch.tensor([3.0, 3.0]))          # only part b has keys
    assert torch.equal(o[0, 0, 2], torch.zeros(2)) and lse[0, 0, 2] == float("-inf")
