"""srtMatmulAllGather on a B200: the product whose epilogue also stores every tile into the other
ranks' buffers.

On one GPU the "peers" are further buffers of the same device, which exercises the kernel's
extra bulk tensor stores and the copy path exactly as peer-mapped addresses would; the two-process
test at the end runs only where two GPUs are visible."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from _gpu_util import BF16, F16, F32, TOL, TORCH_DTYPE, from_dev, random_bits, to_dev

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def srt():
    import swiftrt_b200 as s
    assert torch.cuda.is_available()
    return s


def _full_buffers(n, shape, dtype):
    return [torch.full(shape, -3.0, dtype=TORCH_DTYPE[dtype], device="cuda:0") for _ in range(n)]


@pytest.mark.parametrize("dtype,M,N,K,expect_fused", [
    (BF16, 512, 1024, 2048, True),        # CTA-pair kernel: tiles stored to every buffer by the epilogue
    (F16, 384, 256, 512, None),           # one CTA per tile
    (F16, 768, 520, 1024, None),          # ragged right edge, clipped by the tensor maps
    (F32, 384, 512, 1024, None),          # Float32 runs the 3xTF32 kernel: product, then copies
    (BF16, 96, 200, 64, None),           # small: one CTA per tile, the same fused epilogue
    (F32, 33, 17, 9, None),              # strided SIMT kernel, then copies
])
def test_block_lands_in_every_buffer(srt, oracle, dtype, M, N, K, expect_fused):
    rng = np.random.default_rng(M + N + K)
    a = to_dev(random_bits(oracle, rng, (M, K), dtype), dtype)
    b = to_dev(random_bits(oracle, rng, (K, N), dtype), dtype)
    want = srt.matmul(a, b)
    # the block is columns [N, 2N) of a [M, 3N] result: a strided view, other columns untouched
    bufs = _full_buffers(3, (M, 3 * N), dtype)
    views = [t.narrow(1, N, N) for t in bufs]
    if expect_fused:
        srt.set_tuning(srt.KERNEL_TCGEN05_PAIR)           # few tiles: the planner alone would take one CTA per tile
    try:
        plan = srt.query_plan(a, b, views[0])
        fused = (plan["kernel"] in (srt.KERNEL_TCGEN05_PAIR, srt.KERNEL_TCGEN05) and plan["splitK"] <= 1 and
                 (N * a.element_size()) % 16 == 0)
        if expect_fused:
            assert fused, plan
        before = srt.launch_count()
        srt.matmul_all_gather_into(views[0], [v.data_ptr() for v in views[1:]], a, False, b, False)
        torch.cuda.synchronize()
        assert srt.check_status() == 0
        if fused:
            assert srt.launch_count() == before + 1          # one kernel wrote all three buffers
        for t in bufs:
            assert torch.allclose(t.narrow(1, N, N).float(), want.float(), rtol=2e-2, atol=2e-2)
            assert torch.equal(t.narrow(1, N, N), views[0])
            assert bool((t.narrow(1, 0, N) == -3.0).all()) and bool((t.narrow(1, 2 * N, N) == -3.0).all())
        first = views[0].clone()
        # twice in a row (cached call) and after the buffers changed
        for t in bufs:
            t.fill_(5.0)
        srt.matmul_all_gather_into(views[0], [v.data_ptr() for v in views[1:]], a, False, b, False)
        torch.cuda.synchronize()
        for t in bufs:
            assert torch.equal(t.narrow(1, N, N), first)
    finally:
        srt.set_tuning()


def test_bias_activation_and_oracle_parity_through_the_gather(srt, oracle):
    rng = np.random.default_rng(11)
    M, K, N = 512, 1024, 768
    x = random_bits(oracle, rng, (M, K), BF16, scale=0.5)
    w = random_bits(oracle, rng, (K, N), BF16, scale=0.1)
    bias = random_bits(oracle, rng, (N,), BF16, scale=0.1)
    ref = oracle.matmul(x, w, BF16, False, False, bias=bias, activation="relu")
    bufs = _full_buffers(2, (M, N), BF16)
    srt.matmul_all_gather_into(bufs[0], [bufs[1].data_ptr()], to_dev(x, BF16), False, to_dev(w, BF16), False,
                               to_dev(bias, BF16), srt.ActivationType.relu)
    torch.cuda.synchronize()
    for t in bufs:
        err = oracle.rel_frobenius(oracle.decode(from_dev(t, BF16), BF16), oracle.decode(ref, BF16))
        assert err <= TOL[BF16], err
    assert torch.equal(bufs[0], bufs[1])


@pytest.mark.parametrize("axis", ["n", "m", "batch"])
def test_four_emulated_ranks_fill_four_buffers(srt, axis):
    """sharded_matmul with peer buffers, the ranks played one after the other on one GPU."""
    torch.manual_seed(0)
    if axis == "batch":
        a = torch.randn(8, 256, 512, device="cuda:0", dtype=torch.bfloat16)
        b = torch.randn(8, 512, 384, device="cuda:0", dtype=torch.bfloat16)
    else:
        a = torch.randn(1024, 1024, device="cuda:0", dtype=torch.bfloat16)
        b = torch.randn(1024, 2048, device="cuda:0", dtype=torch.bfloat16)
    want = srt.matmul(a, b)
    world = 4
    bufs = _full_buffers(world, tuple(want.shape), BF16)

    class Fake:
        def __init__(self, rank):
            self.tensor = bufs[rank]
            self.peer_base = {r: t.data_ptr() for r, t in enumerate(bufs) if r != rank}
            self.nbytes = self.tensor.numel() * self.tensor.element_size()
        peer_pointers = srt.PeerBuffer.peer_pointers

    for rank in range(world):
        srt.sharded_matmul(a, b, axis=axis, rank=rank, world=world, peer_buffer=Fake(rank))
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    for t in bufs:
        # blocks and the whole product may run under different plans: equal up to bf16 rounding,
        # while all buffers must hold the very same bits
        assert torch.allclose(t.float(), want.float(), rtol=2e-2, atol=2e-2)
        assert torch.equal(t, bufs[0])
    assert not bool((bufs[0] == -3.0).all())


def test_peer_buffer_single_rank_and_argument_errors(srt):
    buf = srt.PeerBuffer((64, 128), torch.float32)
    assert buf.tensor.shape == (64, 128) and buf.tensor.is_cuda and buf.peer_base == {}
    a = torch.randn(64, 32, device="cuda:0")
    b = torch.randn(32, 128, device="cuda:0")
    got = srt.sharded_matmul(a, b, axis="m", peer_buffer=buf)
    torch.cuda.synchronize()
    assert torch.equal(got, srt.matmul(a, b))
    with pytest.raises(srt.MatmulError) as e:
        srt.matmul_all_gather_into(buf.tensor, [buf.tensor.data_ptr()] * 8, a, False, b, False)
    assert e.value.code == 1 and "peerCount" in str(e.value)
    buf.close()
    buf.close()                                            # idempotent


_TWO_RANK_SCRIPT = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
dist.init_process_group("nccl", device_id=torch.device(f"cuda:{rank}"))
import swiftrt_b200 as srt
torch.manual_seed(0)                                   # same operands on every rank
ok = True
cases = [(axis, ash, bsh, mc) for mc in (False, True)
         for axis, ash, bsh in (("n", (1024, 1024), (1024, 2048)), ("m", (2048, 512), (512, 640)), ("batch", (4, 256, 256), (4, 256, 384)))]
for axis, ash, bsh, mc in cases:
    a = torch.randn(ash, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(bsh, device="cuda", dtype=torch.bfloat16)
    want = srt.matmul(a, b)
    # mc: buffers bound to one NVLink multicast object; eligible products store each tile once (multimem.st)
    buf = srt.PeerBuffer(tuple(want.shape), torch.bfloat16, multicast=mc)
    if mc and rank == 0:
        print("multicast mapping:", hex(buf.multicast_base), flush=True)
    buf.tensor.fill_(-1.0)
    torch.cuda.synchronize(); dist.barrier()
    for _ in range(2):
        got = srt.sharded_matmul(a, b, axis=axis, peer_buffer=buf)
        buf.ranks_done()
        torch.cuda.synchronize()
        ok &= bool(torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2)) and srt.check_status() == 0
        other = got.clone()
        dist.broadcast(other, src=0)                   # both GPUs must hold the very same bits
        ok &= bool(torch.equal(other, got))
        dist.barrier()
    buf.close()
flag = torch.tensor([1 if ok else 0], device="cuda")
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
if rank == 0:
    print("GATHER_OK" if int(flag.item()) == 1 else "GATHER_MISMATCH", flush=True)
dist.destroy_process_group()
"""


@pytest.mark.timeout(600)
def test_two_processes_two_gpus(tmp_path):
    """Each rank computes half of C and stores it into both GPUs' buffers over NVLink (plain bulk
    tensor stores to peer memory; NVLS off)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "two_rank.py"
    script.write_text(_TWO_RANK_SCRIPT)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    run = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script), ROOT],
                         capture_output=True, text=True, timeout=540, env=env)
    assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-4000:]
    assert "GATHER_OK" in run.stdout, run.stdout[-2000:] + run.stderr[-2000:]
