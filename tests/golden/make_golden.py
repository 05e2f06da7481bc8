"""Generates tests/golden/*.pt by running the reference's own PyTorch oracles.

Run once where the reference checkout is available:
    python tests/golden/make_golden.py /path/to/FlagAttention
It imports src/flag_attn/testing/{flash,piecewise,paged}.py BY FILE PATH (the
package itself needs triton kernels we do not want), runs them on CPU on small
seeded inputs and stores inputs and outputs.  tests/test_oracle_golden.py then
pins oracle/ (and flagattention_b200.testing) against these files on machines
that do not have the reference.
"""
import importlib.util
import math
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    sys.exit("usage: python %s /path/to/FlagAttention" % sys.argv[0])
REF = sys.argv[1]


def _load(name):
    path = os.path.join(REF, "src", "flag_attn", "testing", name + ".py")
    spec = importlib.util.spec_from_file_location("fa_ref_testing_" + name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _randn(gen, shape, dtype, std=1.0):
    return (torch.randn(shape, generator=gen, dtype=torch.float32) * std).to(dtype)


def flash_cases(ref):
    out = []
    specs = [
        # B, Hq, Hk, M, N, D, causal, dtype, std
        (1, 2, 2, 48, 80, 32, True, torch.float16, 1.0),
        (1, 2, 2, 48, 80, 32, False, torch.float16, 2.0),
        (1, 4, 2, 40, 40, 16, True, torch.bfloat16, 1.0),
        (2, 2, 1, 33, 65, 64, False, torch.bfloat16, 1.0),
        (1, 2, 2, 70, 10, 16, True, torch.float16, 1.0),   # M > N: rows without any visible key
        (1, 1, 1, 3, 130, 128, True, torch.bfloat16, 3.0),  # decode-shaped
    ]
    for idx, (B, Hq, Hk, M, N, D, causal, dtype, std) in enumerate(specs):
        gen = torch.Generator().manual_seed(10086 + idx)
        q = _randn(gen, (B, Hq, M, D), dtype, std)
        k = _randn(gen, (B, Hk, N, D), dtype, std)
        v = _randn(gen, (B, Hk, N, D), dtype, std)
        do = _randn(gen, (B, Hq, M, D), dtype, 1.0)
        case = dict(q=q, k=k, v=v, do=do, causal=causal, sm_scale=None)
        for upcast in (True, False):
            qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
            o, lse, tot = ref.attention(qq, kk, vv, causal, return_log_normalizer=True,
                                        return_total_attention=True, upcast=upcast)
            dq, dk, dv = torch.autograd.grad(o, (qq, kk, vv), do)
            tag = "ref" if upcast else "torch"
            case[tag] = dict(o=o.detach(), lse=lse.detach(), tot=tot.detach(), dq=dq, dk=dk, dv=dv)
        out.append(case)
    return out


def cfg1_case(ref):
    """The CPU-runnable benchmark configuration: fp32, B=2, H=4, L=256, D=64, causal."""
    gen = torch.Generator().manual_seed(10086 + 1)
    B, H, L, D = 2, 4, 256, 64
    q, k, v, do = (_randn(gen, (B, H, L, D), torch.float32) for _ in range(4))
    qq, kk, vv = (t.clone().requires_grad_() for t in (q, k, v))
    o, lse, tot = ref.attention(qq, kk, vv, True, sm_scale=0.125, return_log_normalizer=True,
                                return_total_attention=True, upcast=True)
    dq, dk, dv = torch.autograd.grad(o, (qq, kk, vv), do)
    # inputs are regenerated from the seed by the test; keep head (1, 2) of the big tensors
    sl = (1, 2)
    return dict(seed=10086 + 1, shape=(B, H, L, D), sm_scale=0.125, lse=lse.detach(),
                tot=tot.detach(), o=o.detach()[sl].clone(), dq=dq[sl].clone(), dk=dk[sl].clone(),
                dv=dv[sl].clone(), head=sl,
                input_checksum=float(q.double().sum() + k.double().sum() + v.double().sum() + do.double().sum()))


def piecewise_cases(ref):
    out = []
    specs = [
        (1, 2, 64, 96, 32, 20, True, torch.bfloat16, 1.0),
        (1, 2, 64, 96, 32, 20, False, torch.float16, 1.0),
        (2, 1, 50, 50, 16, 25, True, torch.float16, 2.0),
        (1, 2, 80, 30, 64, 65, True, torch.bfloat16, 1.0),   # M > N
    ]
    for idx, (B, H, M, N, D, w, causal, dtype, std) in enumerate(specs):
        gen = torch.Generator().manual_seed(20086 + idx)
        q1, q2 = (_randn(gen, (B, H, M, D), dtype, std) for _ in range(2))
        k1, k2, v = (_randn(gen, (B, H, N, D), dtype, std) for _ in range(3))
        do = _randn(gen, (B, H, M, D), dtype, 1.0)
        case = dict(q1=q1, k1=k1, q2=q2, k2=k2, v=v, do=do, w=w, causal=causal)
        for upcast in (True, False):
            ins = [t.clone().requires_grad_() for t in (q1, k1, q2, k2, v)]
            o = ref.attention(*ins, w, causal, upcast=upcast)
            grads = torch.autograd.grad(o, ins, do)
            tag = "ref" if upcast else "torch"
            case[tag] = dict(o=o.detach(), grads=[g for g in grads])
        sm = 1.0 / math.sqrt(D)
        o32 = case["ref"]["o"]
        case["closed_form"] = list(ref.attention_grad(q1, k1, q2, k2, v, w, causal, sm, o32, do, upcast=True))
        out.append(case)
    return out


def paged_cases(ref):
    out = []
    specs = [
        # seqs, q heads, group, head, block, ctx lens, num blocks, table dtype
        (3, 8, 4, 32, 16, [1, 37, 64], 12, torch.int64),
        (2, 4, 1, 64, 16, [16, 33], 7, torch.int32),
        (2, 16, 8, 16, 32, [70, 5], 9, torch.int64),
    ]
    for idx, (S, Hq, G, D, BS, lens, NB, tdt) in enumerate(specs):
        gen = torch.Generator().manual_seed(30086 + idx)
        scale = D ** -0.5
        q = ((torch.rand((S, Hq, D), generator=gen) * 2 - 1) * scale).to(torch.float16)
        kc = ((torch.rand((NB, Hq // G, BS, D), generator=gen) * 2 - 1) * scale).to(torch.float16)
        vc = ((torch.rand((NB, Hq // G, BS, D), generator=gen) * 2 - 1) * scale).to(torch.float16)
        max_blocks = (max(lens) + BS - 1) // BS
        bt = torch.randint(0, NB, (S, max_blocks), generator=gen).to(tdt)   # repeats allowed
        cl = torch.tensor(lens, dtype=torch.int32)
        o = ref.attention(q, kc, vc, bt, cl, scale)
        out.append(dict(q=q, key_cache=kc, value_cache=vc, block_tables=bt, context_lens=cl,
                        scale=scale, out=o))
    return out


def main():
    flash, piecewise, paged = _load("flash"), _load("piecewise"), _load("paged")
    torch.manual_seed(0)
    torch.set_num_threads(1)
    torch.save(dict(cases=flash_cases(flash), cfg1=cfg1_case(flash)), os.path.join(HERE, "flash.pt"))
    torch.save(dict(cases=piecewise_cases(piecewise)), os.path.join(HERE, "piecewise.pt"))
    torch.save(dict(cases=paged_cases(paged)), os.path.join(HERE, "paged.pt"))
    for f in ("flash.pt", "piecewise.pt", "paged.pt"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
