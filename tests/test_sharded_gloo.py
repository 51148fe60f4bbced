"""The multi-GPU sharding logic on CPU ranks: world_size 2 over gloo, with the CPU oracle injected
as the compute function (the product path itself always uses the CUDA operator)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_matmul_into(out, lhs, tl, rhs, tr, bias=None, activation=None):
    from oracle import oracle
    if lhs.dim() == 3 and rhs.dim() == 2:
        rhs = rhs.expand(lhs.shape[0], *rhs.shape)
    res = oracle.matmul(lhs.contiguous().numpy(), rhs.contiguous().numpy(), 0, tl, tr, threads=1)
    out.copy_(torch.from_numpy(res))
    return out


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import swiftrt_b200 as srt
        g = torch.Generator().manual_seed(0)          # same operands on every rank
        cases = [("n", (24, 16), (16, 40), False, False), ("n", (24, 16), (36, 16), False, True),
                 ("m", (26, 16), (16, 12), False, False), ("m", (16, 26), (16, 12), True, False),
                 ("batch", (6, 8, 5), (6, 5, 7), False, False), ("batch", (5, 8, 5), (5, 7), False, False),
                 ("m", (3, 10, 5), (3, 5, 7), False, False)]
        ok = True
        for axis, ash, bsh, tl, tr in cases:
            a = torch.rand(ash, generator=g) * 2 - 1
            b = torch.rand(bsh, generator=g) * 2 - 1
            nb = max(a.shape[0] if a.dim() == 3 else 1, b.shape[0] if b.dim() == 3 else 1)
            a3 = a if a.dim() == b.dim() else (a if a.dim() == 3 else a.expand(nb, *a.shape))
            b3 = b if a.dim() == b.dim() else (b if b.dim() == 3 else b.expand(nb, *b.shape))
            want = torch.empty(0)
            from oracle import oracle
            want = torch.from_numpy(oracle.matmul(a3.numpy(), b3.numpy(), 0, tl, tr, threads=1))
            full = srt.sharded_matmul(a3, b3, tl, tr, axis=axis, gather=True, matmul_into_fn=_oracle_matmul_into)
            ok &= bool(torch.equal(full, want))
            local = srt.sharded_matmul(a3, b3, tl, tr, axis=axis, gather=False, matmul_into_fn=_oracle_matmul_into)
            total = want.shape[{"batch": 0, "m": want.dim() - 2, "n": want.dim() - 1}[axis]]
            lo, hi = srt.shard_range(total, world, rank, 4 if axis == "n" else 1)
            dim = {"batch": 0, "m": want.dim() - 2, "n": want.dim() - 1}[axis]
            ok &= bool(torch.equal(local, want.narrow(dim, lo, hi - lo)))
        # host-buffer form, axis "n": every rank passes only its row block of lhs and its column block
        # of rhs; the row blocks are all-gathered (gloo here) piece by piece
        a = torch.rand((2 * 300, 24), generator=g) * 2 - 1
        b = torch.rand((24, 40), generator=g) * 2 - 1
        want = torch.from_numpy(oracle.matmul(a.numpy(), b.numpy(), 0, threads=1))
        lo, hi = srt.shard_range(40, world, rank, 4)
        mine = srt.sharded_matmul_host(a[rank * 300:(rank + 1) * 300].contiguous(), b[:, lo:hi].contiguous(), axis="n",
                                       device="cpu", pieces=3, matmul_into_fn=_oracle_matmul_into)
        ok &= bool(torch.equal(mine, want[:, lo:hi]))
        flag = torch.tensor([1 if ok else 0])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            results.put(int(flag.item()))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(300)
def test_sharded_matmul_world_size_2_gloo():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(240)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    assert results.get(timeout=10) == 1


def test_single_rank_needs_no_process_group():
    import swiftrt_b200 as srt
    a, b = torch.rand(8, 4), torch.rand(4, 12)
    full = srt.sharded_matmul(a, b, axis="n", gather=True, matmul_into_fn=_oracle_matmul_into, rank=0, world=1)
    assert torch.allclose(full, a @ b, atol=1e-5)
    part = srt.sharded_matmul(a, b, axis="n", gather=False, matmul_into_fn=_oracle_matmul_into, rank=1, world=3)
    lo, hi = srt.shard_range(12, 3, 1, 4)
    assert torch.allclose(part, (a @ b)[:, lo:hi], atol=1e-5)
