"""srtMatmulNoAlloc: the matmul entry point for callers that may not allocate device memory.

Some hosts cannot call cudaMalloc where they need the product -- a real-time loop, a callback from
a runtime that owns all device memory, a process whose pool was handed out in full at start-up.
For them the split-K scratch (fp32 partial sums) is a 16 MiB array compiled into the library.
The test drives the entry point through the C ABI, twice in a row on the same scratch with
different inputs, and checks each result against the regular srtMatmul entry point.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

SPLIT_3XTF32, TENSOR_CORE = 4, 2
TOL = {torch.float32: 1e-5, torch.bfloat16: 1e-2, torch.float16: 1e-2}     # the path's tolerances


def _no_alloc(srt, out, a, ta, b, tb):
    """out = op(a) . op(b) through srtMatmulNoAlloc on torch's current stream."""
    from swiftrt_b200 import _lib
    from swiftrt_b200.tensor import Descriptor
    da, db, do = Descriptor(a), Descriptor(b), Descriptor(out)
    stream = torch.cuda.current_stream(out.device).cuda_stream
    rc = _lib.lib.srtMatmulNoAlloc(a.data_ptr(), da.ref(), ta, b.data_ptr(), db.ref(), tb,
                                   out.data_ptr(), do.ref(), stream)
    return rc, _lib.last_error()


def _rel(x, ref):
    return float((x.double() - ref.double()).norm() / ref.double().norm())


@pytest.mark.parametrize("dtype,M,N,K,tb", [
    (torch.bfloat16, 256, 256, 8192, False),       # few tiles, long reduction: split for occupancy
    (torch.float16, 130, 200, 4096, True),         # ragged edges
    (torch.float32, 512, 256, 4096, False),        # Float32 beyond K = 2048: split for accuracy
    (torch.bfloat16, 32, 1024, 2048, False),       # a few rows against a wide operand: planned transposed,
                                                   # the reduce pass turns the tile (splitk_reduce_transposed_kernel)
])
def test_no_alloc_matches_regular_entry_point_on_two_calls_in_a_row(dtype, M, N, K, tb):
    import swiftrt_b200 as srt
    dev = torch.device("cuda:0")
    srt.set_tuning(0, 0, 0, 0)
    srt.set_split_k(0)
    g = torch.Generator(device=dev).manual_seed(1234)
    for call in range(2):                           # second call: new inputs, same scratch
        a = (torch.rand((M, K), device=dev, generator=g) * 2 - 1).to(dtype)
        b = (torch.rand((N, K) if tb else (K, N), device=dev, generator=g) * 2 - 1).to(dtype)
        want = srt.matmul(a, b, False, tb)                                   # regular entry point
        plan = srt.query_plan(a, b, want, False, tb)
        assert plan["splitK"] > 1 and plan["workspaceBytes"] <= 16 << 20, plan   # the scratch is really used
        if M == 32:
            assert plan["swapped"] == 1, plan
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc, err = _no_alloc(srt, got, a, False, b, tb)
        assert rc == 0, err
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] >= free_before, "the call took device memory"
        assert srt.check_status() == 0
        assert _rel(got, want) <= TOL[dtype], (call, _rel(got, want))
        assert torch.equal(got, want), "same plan and kernels: the two entry points should agree exactly"
        # and against an independent fp64 product, so that a wrong pair of equal results cannot pass
        ref = a.double() @ (b.double().t() if tb else b.double())
        assert _rel(got, ref) <= (2e-3 if dtype != torch.float32 else 1e-5)


def test_no_alloc_refuses_products_beyond_the_static_scratch():
    import swiftrt_b200 as srt
    dev = torch.device("cuda:0")
    srt.set_tuning(TENSOR_CORE, 0, 0, 0)
    srt.set_split_k(4)                               # 4 x 2048 x 2048 x 4 bytes = 64 MiB of partial sums
    try:
        a = torch.ones((2048, 4096), dtype=torch.bfloat16, device=dev)
        b = torch.ones((4096, 2048), dtype=torch.bfloat16, device=dev)
        out = torch.zeros((2048, 2048), dtype=torch.bfloat16, device=dev)
        launches = srt.launch_count()
        rc, err = _no_alloc(srt, out, a, False, b, False)
        assert rc == 1 and "static scratch" in err and "67108864" in err, (rc, err)
        assert srt.launch_count() == launches           # nothing was launched
        torch.cuda.synchronize()
        assert float(out.float().abs().sum()) == 0.0
        # a product that is not split needs no scratch and is never refused for its size
        srt.set_split_k(1)
        rc, err = _no_alloc(srt, out, a, False, b, False)
        assert rc == 0, err
        torch.cuda.synchronize()
        assert bool((out == 4096).all())
    finally:
        srt.set_tuning(0, 0, 0, 0)
        srt.set_split_k(0)


def test_no_alloc_first_call_for_a_kernel_variant_and_second_device():
    """The very first launch of a kernel variant loads its code (CUDA loads modules lazily), which takes
    device memory inside the driver: the header asks for that first call to happen where allocation is
    allowed.  Here srtMatmulNoAlloc is the first to run a shape and element type no other test uses;
    the memory the cold call took is printed, the warm call must take none, and both must be right.
    With two GPUs the same is repeated on the second one (its own copy of the scratch array)."""
    import swiftrt_b200 as srt
    srt.set_tuning(0, 0, 0, 0)
    srt.set_split_k(0)
    for index in range(min(2, torch.cuda.device_count())):
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            g = torch.Generator(device=dev).manual_seed(99 + index)
            a = (torch.rand((96, 6144), device=dev, generator=g) * 2 - 1).to(torch.float16)
            b = (torch.rand((6144, 72), device=dev, generator=g) * 2 - 1).to(torch.float16)
            got = torch.zeros((96, 72), dtype=torch.float16, device=dev)
            ref = a.double() @ b.double()
            torch.cuda.synchronize(dev)
            for attempt in ("cold", "warm"):
                got.zero_()
                torch.cuda.synchronize(dev)
                free_before = torch.cuda.mem_get_info(dev)[0]
                rc, err = _no_alloc(srt, got, a, False, b, False)
                assert rc == 0, err
                torch.cuda.synchronize(dev)
                taken = free_before - torch.cuda.mem_get_info(dev)[0]
                print(f"srtMatmulNoAlloc {attempt} call on {dev}: {taken} bytes of device memory taken")
                if attempt == "warm":
                    assert taken <= 0, taken
                assert _rel(got, ref) <= 2e-3
            assert srt.check_status(dev) == 0
