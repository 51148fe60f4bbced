"""srtMatmulTune and the plan table on a B200: the tuner times the candidate kernels for one call
signature, later calls with that signature run the winner, and the table survives a save / load."""
import numpy as np
import pytest
import torch

from _gpu_util import BF16, F32, TOL, from_dev, random_bits, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture()
def srt():
    import swiftrt_b200 as s
    assert torch.cuda.is_available()
    s.set_tuning()
    s.set_split_k(0)
    s.clear_plan_cache()
    yield s
    s.clear_plan_cache()
    s.set_tuning()


def _time_us(fn, reps=20):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / reps


@pytest.mark.parametrize("dtype,M,N,K", [(BF16, 512, 768, 1024), (BF16, 128, 4096, 4096), (F32, 512, 512, 512)])
def test_tuned_plan_is_used_correct_and_not_slower(srt, oracle, dtype, M, N, K, tmp_path):
    rng = np.random.default_rng(M + N + K)
    a, b = random_bits(oracle, rng, (M, K), dtype), random_bits(oracle, rng, (K, N), dtype)
    da, db = to_dev(a, dtype), to_dev(b, dtype)
    out = torch.empty((M, N), dtype=da.dtype, device="cuda:0")
    op = srt.MatmulOp(out, da, False, db, False)
    default_plan = srt.query_plan(da, db, out)
    other_before = srt.query_plan(da[: M // 2], db, out[: M // 2])
    default_us = _time_us(op)
    best = srt.tune(da, db, out)
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    ref = oracle.matmul(a, b, dtype)
    assert oracle.rel_frobenius(oracle.decode(from_dev(out, dtype), dtype), oracle.decode(ref, dtype)) <= TOL[dtype]
    # the same signature now plans as the winner did ...
    plan = srt.query_plan(da, db, out)
    for key in ("kernel", "tileN", "stages", "splitK"):
        assert plan[key] == best[key], (key, plan, best)
    # ... on other buffers too, and a different signature is untouched
    da2, db2 = to_dev(a, dtype), to_dev(b, dtype)
    assert srt.query_plan(da2, db2, torch.empty_like(out))["kernel"] == best["kernel"]
    assert srt.query_plan(da[: M // 2], db, out[: M // 2]) == other_before
    tuned_us = _time_us(op)
    assert tuned_us <= default_us * 1.10 + 1.0, (default_plan, best, default_us, tuned_us)
    out.zero_()
    op()
    torch.cuda.synchronize()
    assert oracle.rel_frobenius(oracle.decode(from_dev(out, dtype), dtype), oracle.decode(ref, dtype)) <= TOL[dtype]
    # process-wide tuning still overrides the table
    srt.set_tuning(1)
    assert srt.query_plan(da, db, out)["kernel"] == 1
    srt.set_tuning()
    # save, clear (back to the cost model), load (back to the tuned plan)
    path = tmp_path / "plans.txt"
    srt.save_plan_cache(str(path))
    srt.clear_plan_cache()
    assert srt.query_plan(da, db, out) == default_plan
    assert srt.load_plan_cache(str(path)) == 1
    assert srt.query_plan(da, db, out)["kernel"] == best["kernel"]
