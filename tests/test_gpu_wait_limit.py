"""The bounded waits of the tensor-core kernels on a B200.

Every pipeline wait inside the kernels has a limit; a wait that runs out ends its kernel in an orderly
way (outstanding loads and MMAs are waited for, tensor memory is released) and sets a status word
instead of hanging the GPU.  The tests shorten the limit to one nanosecond on small VALID products, so
that the first wait that does not succeed at once gives up: nothing faults, nothing hangs, the status
word reports it, and the same context then computes the same products correctly with the default limit."""
import numpy as np
import pytest
import torch

from _gpu_util import BF16, F32, TOL, from_dev, random_bits, to_dev

pytestmark = pytest.mark.gpu

TC, PAIR, SPLIT, X3 = 2, 3, 4, 5


@pytest.fixture()
def srt():
    import swiftrt_b200 as s
    assert torch.cuda.is_available()
    s.set_tuning(0, 0, 0, 0)
    s.set_split_k(0)
    s.set_wait_limit(0)
    yield s
    s.set_wait_limit(0)
    s.set_tuning(0, 0, 0, 0)
    torch.cuda.synchronize()
    s.check_status()


@pytest.mark.parametrize("kernel,dtype,M,N,K", [
    (TC, BF16, 384, 256, 2048),        # one CTA per tile
    (SPLIT, F32, 256, 256, 512),       # 3 x TF32 with transform warps
    (PAIR, BF16, 1024, 512, 2048),     # CTA pairs: the abort is raised in both CTAs, loads are evened out
    (X3, F32, 1024, 256, 512),         # CTA pairs with a pack pass and worker warps
])
def test_a_wait_that_runs_out_ends_the_kernel_and_leaves_the_context_usable(srt, oracle, kernel, dtype, M, N, K):
    rng = np.random.default_rng(kernel * 100 + M)
    a_bits, b_bits = random_bits(oracle, rng, (M, K), dtype), random_bits(oracle, rng, (K, N), dtype)
    want = oracle.matmul(a_bits, b_bits, dtype)
    a, b = to_dev(a_bits, dtype), to_dev(b_bits, dtype)
    out = torch.zeros((M, N), dtype=a.dtype, device="cuda:0")
    srt.set_tuning(kernel, 0, 0, 0)
    assert srt.query_plan(a, b, out)["kernel"] == kernel
    srt.matmul_into(out, a, False, b, False)                 # loads the kernel with the default limit
    torch.cuda.synchronize()
    assert srt.check_status() == 0

    srt.set_wait_limit(1)                                    # one nanosecond: the first wait that has to wait gives up
    gave_up = 0
    for _ in range(3):
        srt.matmul_into(out, a, False, b, False)
        torch.cuda.synchronize()                             # returns: the kernel ended by itself
        gave_up |= srt.check_status()                        # reads and clears the status word
    assert gave_up != 0, "no wait ran out although the limit was one nanosecond"
    assert gave_up & ~0xF == 0                               # only the documented bits

    srt.set_wait_limit(0)                                    # back to the default
    out.zero_()
    srt.matmul_into(out, a, False, b, False)
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    got = from_dev(out, dtype)
    err = oracle.rel_frobenius(oracle.decode(got, dtype), oracle.decode(want, dtype))
    assert err <= (TOL[F32] if dtype == F32 else 2e-3), err
