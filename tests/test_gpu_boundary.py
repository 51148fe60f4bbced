"""Boundary behaviour of the C ABI on a B200: the device of a call comes from its stream, workspaces
grow without waiting and survive CUDA graphs that captured them, and the C-level sharding entry
points (srtMatmulSharded, srtMatmulShardedDevices) place every block where the host mirror does."""
import ctypes

import numpy as np
import pytest
import torch

from _gpu_util import BF16, F32, TORCH_DTYPE, from_dev, random_bits, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def srt():
    import swiftrt_b200 as s
    assert torch.cuda.is_available()
    return s


def _raw_matmul(out, a, b, stream_ptr, bias=None, act=5):
    """srtMatmulBiasActivation through ctypes with an explicit stream handle and NO device switch."""
    from swiftrt_b200 import _lib
    from swiftrt_b200.tensor import Descriptor
    da, db, do = Descriptor(a), Descriptor(b), Descriptor(out)
    dbias = Descriptor(bias) if bias is not None else None
    rc = _lib.lib.srtMatmulBiasActivation(a.data_ptr(), da.ref(), False, b.data_ptr(), db.ref(), False,
                                          bias.data_ptr() if bias is not None else None,
                                          dbias.ref() if dbias is not None else None, act, out.data_ptr(), do.ref(), stream_ptr)
    return rc, _lib.last_error()


def test_call_runs_on_the_device_of_its_stream(srt, oracle):
    """The reference's queues enqueue on their stream without selecting a device
    (platform/cuda/functions/CudaMath.swift:117-125), so a call whose stream belongs to device 1 must
    work while device 0 is current -- split-K workspace, kernel attributes and status word included --
    and must leave device 0 current."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    rng = np.random.default_rng(0)
    cases = [(BF16, 256, 256, 8192),      # split-K: allocates a workspace on the stream's device
             (BF16, 512, 768, 1024),
             (F32, 100, 90, 70)]
    torch.cuda.set_device(0)
    s1 = torch.cuda.Stream(device=1)
    for dtype, M, N, K in cases:
        a_bits, b_bits = random_bits(oracle, rng, (M, K), dtype), random_bits(oracle, rng, (K, N), dtype)
        want = oracle.matmul(a_bits, b_bits, dtype)
        a, b = to_dev(a_bits, dtype, "cuda:1"), to_dev(b_bits, dtype, "cuda:1")
        out = torch.zeros((M, N), dtype=TORCH_DTYPE[dtype], device="cuda:1")
        torch.cuda.synchronize(1)
        assert torch.cuda.current_device() == 0
        rc, err = _raw_matmul(out, a, b, s1.cuda_stream)
        assert rc == 0, err
        assert torch.cuda.current_device() == 0          # restored
        s1.synchronize()
        got = from_dev(out, dtype)
        err = oracle.rel_frobenius(oracle.decode(got, dtype), oracle.decode(want, dtype))
        assert err <= (1e-5 if dtype == F32 else 2e-3), err
    status = ctypes.c_uint32(7)
    from swiftrt_b200 import _lib
    assert _lib.lib.srtMatmulCheckStatus(s1.cuda_stream, ctypes.byref(status)) == 0 and status.value == 0
    assert torch.cuda.current_device() == 0


def test_workspace_growth_keeps_a_captured_graph_valid(srt):
    """A CUDA graph that captured a split-K product has the workspace address baked in.  A later,
    larger split-K call on the same stream handle must not free that buffer: the replay afterwards
    has to give the captured result again."""
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(7)
    a = (torch.rand((256, 8192), device=dev, generator=g) - 0.5).to(torch.bfloat16)
    b = (torch.rand((8192, 256), device=dev, generator=g) - 0.5).to(torch.bfloat16)
    out = torch.empty((256, 256), dtype=torch.bfloat16, device=dev)
    plan = srt.query_plan(a, b, out)
    assert plan["splitK"] > 1, plan
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        srt.matmul_into(out, a, False, b, False)          # allocates this stream's workspace outside the capture
    stream.synchronize()
    want = out.clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        srt.matmul_into(out, a, False, b, False)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    # a much larger split-K product on the SAME stream handle forces the workspace to grow
    a2 = (torch.rand((256, 32768), device=dev, generator=g) - 0.5).to(torch.bfloat16)
    b2 = (torch.rand((32768, 1024), device=dev, generator=g) - 0.5).to(torch.bfloat16)
    out2 = torch.empty((256, 1024), dtype=torch.bfloat16, device=dev)
    plan2 = srt.query_plan(a2, b2, out2)
    assert plan2["workspaceBytes"] > plan["workspaceBytes"], (plan, plan2)
    with torch.cuda.stream(stream):
        srt.matmul_into(out2, a2, False, b2, False)
    stream.synchronize()
    ref2 = (a2.float() @ b2.float())
    assert float((out2.float() - ref2).norm() / ref2.norm()) <= 1e-2
    # scribble over freshly allocated memory, then replay: the graph's buffer must still be its own
    junk = [torch.full((1 << 22,), float("nan"), device=dev) for _ in range(4)]
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    del junk
    assert torch.equal(out, want)
    assert srt.check_status() == 0
    # released buffers come back on demand; captured ones are kept unless asked for
    srt.release_workspaces()
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want)
    with torch.cuda.stream(stream):
        srt.matmul_into(out2, a2, False, b2, False)
    stream.synchronize()
    assert float((out2.float() - ref2).norm() / ref2.norm()) <= 1e-2
    del graph
    srt.release_workspaces(include_captured=True)


def test_growing_workspace_does_not_block_the_caller(srt):
    """Growth frees the old buffer in stream order: results of the smaller product that is still in
    flight when the larger one is enqueued stay correct."""
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(3)
    stream = torch.cuda.Stream(device=dev)
    outs, refs = [], []
    with torch.cuda.stream(stream):
        for k in (4096, 8192, 16384, 32768):
            a = (torch.rand((192, k), device=dev, generator=g) - 0.5).to(torch.bfloat16)
            b = (torch.rand((k, 64 * (k // 2048)), device=dev, generator=g) - 0.5).to(torch.bfloat16)
            outs.append(srt.matmul(a, b))
            refs.append((a, b))
    stream.synchronize()
    for o, (a, b) in zip(outs, refs):
        ref = a.float() @ b.float()
        assert float((o.float() - ref).norm() / ref.norm()) <= 1e-2
    assert srt.check_status() == 0


def _shard_call(axis, world, rank, out, a, ta, b, tb, bias=None, act=5, peers=()):
    from swiftrt_b200 import _lib
    from swiftrt_b200.tensor import Descriptor
    da, db, do = Descriptor(a), Descriptor(b), Descriptor(out)
    dbias = Descriptor(bias) if bias is not None else None
    arr = (ctypes.c_void_p * max(1, len(peers)))(*peers) if peers else None
    rc = _lib.lib.srtMatmulSharded(axis, world, rank, a.data_ptr(), da.ref(), ta, b.data_ptr(), db.ref(), tb,
                                   bias.data_ptr() if bias is not None else None, dbias.ref() if dbias is not None else None,
                                   act, out.data_ptr(), do.ref(), len(peers), arr, None,
                                   torch.cuda.current_stream().cuda_stream)
    return rc, _lib.last_error()


@pytest.mark.parametrize("axis,world", [(0, 4), (1, 3), (2, 4), (2, 8), (1, 8)])
def test_sharded_entry_point_places_every_block(srt, oracle, axis, world):
    """All ranks' calls issued one after another on one GPU fill the full result exactly as one
    unsharded call does; with `peers`, every block also lands in the second and third buffer."""
    torch.cuda.set_device(0)
    rng = np.random.default_rng(axis * 10 + world)
    if axis == 0:
        a = to_dev(random_bits(oracle, rng, (6, 96, 64), BF16), BF16)
        b = to_dev(random_bits(oracle, rng, (6, 200, 64), BF16), BF16)
        ta, tb, bias = False, True, None
        want = srt.matmul(a, b, False, True)
    else:
        a = to_dev(random_bits(oracle, rng, (520, 256), BF16), BF16)
        b = to_dev(random_bits(oracle, rng, (256, 776), BF16), BF16)
        bias = to_dev(random_bits(oracle, rng, (776,), BF16), BF16)
        ta, tb = False, False
        want = srt.matmul(a, b, bias=bias, activation=srt.ActivationType.relu)
    bufs = [torch.full_like(want, -3.0) for _ in range(3)]
    for rank in range(world):
        rc, err = _shard_call(axis, world, rank, bufs[0], a, ta, b, tb, bias, 1 if bias is not None else 5,
                              peers=[bufs[1].data_ptr(), bufs[2].data_ptr()])
        assert rc == 0, err
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    for t in bufs:
        assert torch.equal(t, want)


def test_sharded_devices_entry_point_from_one_process(srt, oracle):
    """srtMatmulShardedDevices: one process, one stream per device; with gather every device's buffer
    holds the whole result afterwards.  On one GPU the same device stands for both 'devices'."""
    from swiftrt_b200 import _lib
    from swiftrt_b200.tensor import Descriptor
    n_dev = 2
    devs = [torch.device("cuda", i % torch.cuda.device_count()) for i in range(n_dev)]
    rng = np.random.default_rng(21)
    a_bits, b_bits = random_bits(oracle, rng, (512, 512), BF16), random_bits(oracle, rng, (512, 1024), BF16)
    want = oracle.matmul(a_bits, b_bits, BF16)
    a = [to_dev(a_bits, BF16, d) for d in devs]
    b = [to_dev(b_bits, BF16, d) for d in devs]
    out = [torch.zeros((512, 1024), dtype=torch.bfloat16, device=d) for d in devs]
    streams = [torch.cuda.Stream(device=d) for d in devs]
    torch.cuda.synchronize()
    da, db, do = Descriptor(a[0]), Descriptor(b[0]), Descriptor(out[0])
    vp = ctypes.c_void_p * n_dev
    rc = _lib.lib.srtMatmulShardedDevices(2, n_dev, vp(*[s.cuda_stream for s in streams]), vp(*[t.data_ptr() for t in a]), da.ref(), False,
                                          vp(*[t.data_ptr() for t in b]), db.ref(), False, None, None, 5,
                                          vp(*[t.data_ptr() for t in out]), do.ref(), True, None)
    assert rc == 0, _lib.last_error()
    for s in streams:
        s.synchronize()
    for t in out:
        err = oracle.rel_frobenius(oracle.decode(from_dev(t, BF16), BF16), oracle.decode(want, BF16))
        assert err <= 2e-3, err
    assert torch.equal(out[0].cpu(), out[1].cpu())


def test_multicast_buffers_from_one_process(srt, oracle):
    """srtMulticastAlloc: one process binds a buffer of every GPU to one NVLink multicast object; the
    sharded product then stores each tile once (multimem.st) and every GPU's buffer holds all of C."""
    from swiftrt_b200 import _lib
    from swiftrt_b200.peer import _RawDeviceMemory
    from swiftrt_b200.tensor import Descriptor
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    n_dev, M, N, K = 2, 512, 1024, 1024
    nbytes = M * N * 2
    devs = (ctypes.c_int32 * n_dev)(0, 1)
    local = (ctypes.c_void_p * n_dev)()
    mc, handle = ctypes.c_void_p(), ctypes.c_void_p()
    rc = _lib.lib.srtMulticastAlloc(n_dev, devs, nbytes, local, ctypes.byref(mc), ctypes.byref(handle))
    if rc == 801:
        pytest.skip("no NVLink multicast on this machine: " + _lib.last_error())
    assert rc == 0, _lib.last_error()
    try:
        rng = np.random.default_rng(5)
        a_bits, b_bits = random_bits(oracle, rng, (M, K), BF16), random_bits(oracle, rng, (K, N), BF16)
        want = oracle.matmul(a_bits, b_bits, BF16)
        out = []
        for i in range(n_dev):
            raw = torch.as_tensor(_RawDeviceMemory(local[i], nbytes), device=f"cuda:{i}")
            out.append(raw.view(torch.bfloat16).reshape(M, N))
            out[-1].fill_(-2.0)
        a = [to_dev(a_bits, BF16, f"cuda:{i}") for i in range(n_dev)]
        b = [to_dev(b_bits, BF16, f"cuda:{i}") for i in range(n_dev)]
        streams = [torch.cuda.Stream(device=i) for i in range(n_dev)]
        torch.cuda.synchronize(0)
        torch.cuda.synchronize(1)
        da, db, do = Descriptor(a[0]), Descriptor(b[0]), Descriptor(out[0])
        vp = ctypes.c_void_p * n_dev
        before = srt.launch_count()
        rc = _lib.lib.srtMatmulShardedDevices(2, n_dev, vp(*[s.cuda_stream for s in streams]), vp(*[t.data_ptr() for t in a]), da.ref(), False,
                                              vp(*[t.data_ptr() for t in b]), db.ref(), False, None, None, 5,
                                              vp(*[t.data_ptr() for t in out]), do.ref(), True, mc)
        assert rc == 0, _lib.last_error()
        for s in streams:
            s.synchronize()
        assert srt.launch_count() - before == n_dev       # one fused kernel per device, no copies
        for i, t in enumerate(out):
            err = oracle.rel_frobenius(oracle.decode(from_dev(t, BF16), BF16), oracle.decode(want, BF16))
            assert err <= 2e-3, (i, err)
        assert torch.equal(out[0].cpu(), out[1].cpu())
        for i in range(n_dev):
            st = ctypes.c_uint32(9)
            assert _lib.lib.srtMatmulCheckStatus(streams[i].cuda_stream, ctypes.byref(st)) == 0 and st.value == 0
        del out
    finally:
        assert _lib.lib.srtMulticastFree(handle) == 0
