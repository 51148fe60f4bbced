"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Bit-exact where the arithmetic order is the reference's (the strided SIMT kernel); within the
path's tolerances (relative Frobenius error <= 1e-5 Float32, <= 1e-2 Float16 / BFloat16 with
fp32 accumulation) on the tensor-core kernel, whose accumulation order differs."""
import json
import os

import numpy as np
import pytest
import torch

from _gpu_util import BF16, F16, F32, TOL, TORCH_DTYPE, from_dev, random_bits, to_dev

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "matmul_kat.json")
SIMT, TC, PAIR, SPLIT = 1, 2, 3, 4
TRANSPOSES = [(False, False), (False, True), (True, False), (True, True)]


@pytest.fixture(scope="module")
def srt():
    import swiftrt_b200 as s
    assert torch.cuda.is_available(), "these tests need a GPU"
    yield s
    s.set_tuning(0, 0, 0, 0)


@pytest.fixture(autouse=True)
def _reset_tuning_and_check_status(srt):
    srt.set_tuning(0, 0, 0, 0)
    srt.set_split_k(0)
    yield
    srt.set_split_k(0)
    assert srt.check_status() == 0, "a pipeline wait of the tensor-core kernel timed out"
    srt.set_tuning(0, 0, 0, 0)


def _shapes(M, N, K, ta, tb, batch=0):
    ash = (K, M) if ta else (M, K)
    bsh = (N, K) if tb else (K, N)
    if batch:
        ash, bsh = (batch,) + ash, (batch,) + bsh
    return ash, bsh


def _run(srt, oracle, dtype, a, b, ta, tb, bias=None, act=None, expect_kernel=None, out=None, da=None, db=None):
    """a, b, bias: numpy stored bits (any strides); da, db: the same operands already on the device
    (for views whose base offset matters).  Returns (gpu bits, oracle bits)."""
    ref = oracle.matmul(a, b, dtype, ta, tb, bias=bias, activation=act)
    da = to_dev(a, dtype) if da is None else da
    db = to_dev(b, dtype) if db is None else db
    dbias = to_dev(bias, dtype) if bias is not None else None
    activation = srt.ActivationType[act] if act else None
    if out is None:
        c = srt.matmul(da, db, ta, tb, bias=dbias, activation=activation)
    else:
        c = srt.matmul_into(out, da, ta, db, tb, dbias, activation)
    if expect_kernel is not None:
        assert srt.query_plan(da, db, c, ta, tb)["kernel"] == expect_kernel
    torch.cuda.synchronize()
    return from_dev(c, dtype), ref


# ------------------------------------------------------------------ the reference's known answers
def test_known_answers_on_gpu(srt):
    cases = json.load(open(GOLDEN))["cases"]
    dev = "cuda:0"
    for name, case in cases.items():
        a = torch.arange(int(np.prod(case["a_shape"])), dtype=torch.float32, device=dev).reshape(case["a_shape"])
        b = torch.arange(int(np.prod(case["b_shape"])), dtype=torch.float32, device=dev).reshape(case["b_shape"])
        c = srt.matmul(a, b)
        if "c" in case:
            assert c.cpu().tolist() == case["c"], name
        else:
            assert c[0].cpu().tolist() == case["c_first_item"], name
    # gradients of test_matmul through matmulGradients' two extra matmul calls
    case = cases["test_matmul"]
    a = torch.arange(6.0, device=dev).reshape(3, 2)
    b = torch.arange(8.0, device=dev).reshape(2, 4)
    ga, gb = srt.matmul_gradients(torch.ones(3, 4, device=dev), a, False, b, False)
    assert ga.cpu().tolist() == case["grad_a"] and gb.cpu().tolist() == case["grad_b"]
    # batched gradients: per-item products, literal by literal
    case = cases["test_batchMatmul"]
    a = torch.arange(12.0, device=dev).reshape(2, 3, 2)
    b = torch.arange(16.0, device=dev).reshape(2, 2, 4)
    ones = torch.ones(2, 3, 4, device=dev)
    assert srt.matmul(ones, b, False, True).cpu().tolist() == case["grad_a"]
    assert srt.matmul(a, ones, True, False).cpu().tolist() == case["grad_b"]


# ------------------------------------------------------------------ strided kernel: bit-exact
@pytest.mark.parametrize("dtype", [F32, BF16, F16])
@pytest.mark.parametrize("ta,tb", TRANSPOSES)
@pytest.mark.parametrize("M,N,K,batch", [(1, 1, 1, 0), (3, 4, 2, 0), (65, 70, 33, 0), (64, 64, 64, 3), (130, 17, 257, 2), (1, 50, 300, 0), (40, 1, 77, 0)])
def test_strided_kernel_is_bit_exact(srt, oracle, dtype, ta, tb, M, N, K, batch):
    srt.set_tuning(SIMT, 0, 0, 0)
    rng = np.random.default_rng(M * 1000 + N * 10 + K + dtype)
    ash, bsh = _shapes(M, N, K, ta, tb, batch)
    a, b = random_bits(oracle, rng, ash, dtype), random_bits(oracle, rng, bsh, dtype)
    got, ref = _run(srt, oracle, dtype, a, b, ta, tb, expect_kernel=SIMT)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
def test_strided_kernel_views_bias_relu_bit_exact(srt, oracle, dtype):
    srt.set_tuning(SIMT, 0, 0, 0)
    rng = np.random.default_rng(11 + dtype)
    big_a, big_b = random_bits(oracle, rng, (70, 90), dtype), random_bits(oracle, rng, (90, 80), dtype)
    a, b = big_a[3:63:2, 5:85:3], big_b[10:37, 1:61:4]          # no unit stride, odd offsets
    bias = random_bits(oracle, rng, (30,), dtype)[::2]            # strided bias
    got, ref = _run(srt, oracle, dtype, a, b, False, False, bias=bias, act="relu", expect_kernel=SIMT)
    assert np.array_equal(got, ref)
    got, ref = _run(srt, oracle, dtype, a, b, False, False, bias=bias, act="identity")
    assert np.array_equal(got, ref)


def test_output_view_is_honoured_and_nothing_else_is_written(srt, oracle):
    rng = np.random.default_rng(12)
    a, b = random_bits(oracle, rng, (33, 20), F32), random_bits(oracle, rng, (20, 15), F32)
    canvas = torch.full((40, 64), 7.0, device="cuda:0")
    view = canvas[2:35, 3:48:3]                                  # 33 x 15, column stride 3
    got, ref = _run(srt, oracle, F32, a, b, False, False, out=view, expect_kernel=SIMT)
    assert np.array_equal(got, ref)
    mask = torch.ones_like(canvas, dtype=torch.bool)
    mask[2:35, 3:48:3] = False
    assert bool((canvas[mask] == 7.0).all())


def test_broadcast_operands_left_and_right_batch(srt, oracle):
    rng = np.random.default_rng(13)
    a3, b2 = random_bits(oracle, rng, (4, 9, 6), F32), random_bits(oracle, rng, (6, 5), F32)
    ref = oracle.matmul(a3, np.broadcast_to(b2, (4, 6, 5)), F32)
    c = srt.matmul(to_dev(a3, F32), to_dev(b2, F32))
    assert np.array_equal(from_dev(c, F32), ref)
    a2, b3 = random_bits(oracle, rng, (9, 6), F32), random_bits(oracle, rng, (4, 6, 5), F32)
    ref = oracle.matmul(np.broadcast_to(a2, (4, 9, 6)), b3, F32)
    c = srt.matmul(to_dev(a2, F32), to_dev(b3, F32))
    assert np.array_equal(from_dev(c, F32), ref)


@pytest.mark.parametrize("act", ["sigmoid", "tanh", "gelu", "geluTanh"])
def test_transcendental_activations(srt, oracle, act):
    rng = np.random.default_rng(14)
    a, b = random_bits(oracle, rng, (50, 40), F32, scale=2.0), random_bits(oracle, rng, (40, 30), F32)
    bias = random_bits(oracle, rng, (30,), F32)
    got, ref = _run(srt, oracle, F32, a, b, False, False, bias=bias, act=act)
    assert oracle.rel_frobenius(got, ref) <= TOL[F32]


# ------------------------------------------------------------------ tensor-core kernel
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("ta,tb", TRANSPOSES)
@pytest.mark.parametrize("M,N,K,batch,tile_n", [
    (128, 256, 64, 0, 0), (1000, 520, 200, 0, 0), (8, 8, 8, 0, 256), (136, 264, 72, 0, 128),
    (512, 384, 1024, 0, 64), (256, 512, 64, 5, 0), (2048, 1024, 4096, 0, 0)])
def test_tensor_core_kernel_within_tolerance(srt, oracle, dtype, ta, tb, M, N, K, batch, tile_n):
    srt.set_tuning(TC, tile_n, 0, 0)
    rng = np.random.default_rng(M + 3 * N + 7 * K + dtype + 2 * ta + tb)
    ash, bsh = _shapes(M, N, K, ta, tb, batch)
    a, b = random_bits(oracle, rng, ash, dtype), random_bits(oracle, rng, bsh, dtype)
    got, ref = _run(srt, oracle, dtype, a, b, ta, tb, expect_kernel=TC)
    err = oracle.rel_frobenius(oracle.decode(got, dtype), oracle.decode(ref, dtype))
    assert err <= TOL[dtype]
    assert err <= 2e-3          # far inside the tolerance: only the final rounding can differ


@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("ta,tb", TRANSPOSES)
@pytest.mark.parametrize("M,N,K,batch,tile_n", [
    (256, 256, 64, 0, 0), (1000, 520, 200, 0, 0), (8, 8, 8, 0, 0), (264, 136, 72, 0, 128),
    (512, 384, 1024, 0, 128), (512, 512, 64, 5, 0), (2048, 1024, 4096, 0, 0), (4096, 4096, 512, 0, 0)])
def test_cta_pair_kernel_within_tolerance(srt, oracle, dtype, ta, tb, M, N, K, batch, tile_n):
    srt.set_tuning(PAIR, tile_n, 0, 0)
    rng = np.random.default_rng(M + 3 * N + 7 * K + dtype + 2 * ta + tb + 1)
    ash, bsh = _shapes(M, N, K, ta, tb, batch)
    a, b = random_bits(oracle, rng, ash, dtype), random_bits(oracle, rng, bsh, dtype)
    got, ref = _run(srt, oracle, dtype, a, b, ta, tb, expect_kernel=PAIR)
    err = oracle.rel_frobenius(oracle.decode(got, dtype), oracle.decode(ref, dtype))
    assert err <= TOL[dtype] and err <= 2e-3


@pytest.mark.parametrize("ta,tb", TRANSPOSES)
@pytest.mark.parametrize("M,N,K,batch,tile_n", [
    (128, 256, 32, 0, 0), (1000, 520, 200, 0, 0), (4, 4, 4, 0, 256), (136, 264, 72, 0, 128),
    (512, 384, 1024, 0, 64), (256, 512, 64, 5, 0), (2048, 512, 2048, 0, 0)])
def test_float32_3xtf32_kernel_within_tolerance(srt, oracle, ta, tb, M, N, K, batch, tile_n):
    """Float32 on the tensor cores (hi/lo split, three TF32 products) must stay within 1e-5."""
    srt.set_tuning(SPLIT, tile_n, 0, 0)
    rng = np.random.default_rng(M + 3 * N + 7 * K + 2 * ta + tb + 5)
    ash, bsh = _shapes(M, N, K, ta, tb, batch)
    a, b = random_bits(oracle, rng, ash, F32), random_bits(oracle, rng, bsh, F32)
    got, ref = _run(srt, oracle, F32, a, b, ta, tb, expect_kernel=SPLIT)
    assert oracle.rel_frobenius(got, ref) <= TOL[F32]


def test_float32_3xtf32_epilogue_and_special_values(srt, oracle):
    srt.set_tuning(SPLIT, 0, 0, 0)
    rng = np.random.default_rng(41)
    a, b = random_bits(oracle, rng, (300, 256), F32), random_bits(oracle, rng, (256, 520), F32)
    bias = random_bits(oracle, rng, (520,), F32)
    got, ref = _run(srt, oracle, F32, a, b, False, False, bias=bias, act="relu", expect_kernel=SPLIT)
    assert oracle.rel_frobenius(got, ref) <= TOL[F32]
    # values spanning many binades and a NaN: the NaN must poison exactly its row, like in the reference
    # (an infinity times an operand whose low part is zero gives NaN instead of infinity on this
    # kernel: the split evaluates inf . 0 for the missing low part)
    a2 = a.copy()
    a2[:, 0] *= 2.0 ** 60
    a2[:, 1] *= 2.0 ** -60
    a2[9, 5] = np.nan
    got, ref = _run(srt, oracle, F32, a2, b, False, False, expect_kernel=SPLIT)
    fin = np.isfinite(ref)
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    assert oracle.rel_frobenius(got[fin], ref[fin]) <= TOL[F32]


X3 = 5      # srtMatmulKernelTf32x3Pair


@pytest.mark.parametrize("M,N,K,batch,tb,col_out", [
    (512, 256, 1024, 0, False, False),        # whole tiles
    (4096, 256, 256, 0, False, False),        # more tiles than CTA pairs: the persistent loop and its phases
    (1000, 200, 100, 0, False, False),        # ragged M, N and K (K not a multiple of a k-block: zero filled)
    (1536, 384, 2048, 0, True, False),        # two column tiles, K-contiguous op(b), the longest allowed reduction
    (640, 136, 72, 3, False, False),          # batched
    (640, 136, 72, 3, True, False),
    (768, 264, 512, 0, False, True),          # column-order result: planned as the transposed problem
])
@pytest.mark.parametrize("tile_n", [0, 128])
def test_float32_pair_kernel_with_bf16_corrections_within_tolerance(srt, oracle, M, N, K, batch, tb, col_out, tile_n):
    """Float32 as one TF32 pass plus BFloat16 correction terms, op(b) pre-split by the pack pass:
    within 1e-5 of the reference loop.  Both tile widths: 256 (the default) and 128 (double-buffered
    accumulators)."""
    srt.set_tuning(X3, tile_n, 0, 0)
    rng = np.random.default_rng(M + 3 * N + 7 * K + batch + tb)
    if col_out:
        # out^T = b^T . a^T: the library sees op(a') = b^T (K-contiguous when b is stored [N x K] ... use tb)
        a, b = random_bits(oracle, rng, (N, K), F32), random_bits(oracle, rng, (M, K), F32)
        da, db = to_dev(a, F32), to_dev(b, F32)
        out = srt.empty((N, M), torch.float32, "cuda:0", srt.Order.col)
        srt.matmul_into(out, da, False, db, True)
        plan = srt.query_plan(da, db, out, False, True)
        assert plan["kernel"] == X3 and plan["swapped"] == 1 and plan["tileN"] == (tile_n or 256), plan
        ref = oracle.matmul(a, b, F32, False, True)
        torch.cuda.synchronize()
        assert oracle.rel_frobenius(out.cpu().numpy(), ref) <= TOL[F32]
        return
    ash, bsh = _shapes(M, N, K, False, tb, batch)
    a, b = random_bits(oracle, rng, ash, F32), random_bits(oracle, rng, bsh, F32)
    got, ref = _run(srt, oracle, F32, a, b, False, tb, expect_kernel=X3)
    err = oracle.rel_frobenius(got, ref)
    assert err <= TOL[F32], err


def test_float32_pair_kernel_epilogue_views_and_special_values(srt, oracle):
    srt.set_tuning(X3, 0, 0, 0)
    rng = np.random.default_rng(43)
    a, b = random_bits(oracle, rng, (900, 256), F32), random_bits(oracle, rng, (256, 520), F32)
    bias = random_bits(oracle, rng, (520,), F32)
    got, ref = _run(srt, oracle, F32, a, b, False, False, bias=bias, act="relu", expect_kernel=X3)
    assert oracle.rel_frobenius(got, ref) <= TOL[F32]
    # a strided (but TMA-addressable) view of a wider operand, and a result view with guard columns
    wide = random_bits(oracle, rng, (900, 512), F32)
    av = wide[:, 128:384]
    big = torch.full((900, 1024), -7.0, device="cuda:0")
    out = big[:, 256:776]
    dwide = to_dev(wide, F32)
    srt.matmul_into(out, dwide[:, 128:384], False, to_dev(b, F32), False)
    assert srt.query_plan(dwide[:, 128:384], to_dev(b, F32), out)["kernel"] == X3
    torch.cuda.synchronize()
    assert oracle.rel_frobenius(out.cpu().numpy(), oracle.matmul(av, b, F32)) <= TOL[F32]
    assert bool((big[:, :256] == -7.0).all()) and bool((big[:, 776:] == -7.0).all())
    # many binades, a NaN and infinities: the NaN poisons exactly its row; an infinity times a value whose
    # low part is zero (1.0, 0.5, small integers) stays an infinity, as in the reference loop
    a2 = a.copy()
    a2[:, 0] *= 2.0 ** 60
    a2[:, 1] *= 2.0 ** -60
    a2[9, 5] = np.nan
    a2[17, 3] = np.inf
    a2[33, 7] = -np.inf
    b2 = b.copy()
    b2[3, :] = 1.0
    b2[7, ::2] = 0.5
    b2[7, 1::2] = -3.0
    got, ref = _run(srt, oracle, F32, a2, b2, False, False, expect_kernel=X3)
    fin = np.isfinite(ref)
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    assert np.array_equal(got[~fin & ~np.isnan(ref)], ref[~fin & ~np.isnan(ref)])      # +inf / -inf in the same places
    assert oracle.rel_frobenius(got[fin], ref[fin]) <= TOL[F32]
    # the same special values through the 3 x TF32 kernel (one CTA per tile)
    srt.set_tuning(SPLIT, 0, 0, 0)
    got, ref = _run(srt, oracle, F32, a2, b2, False, False, expect_kernel=SPLIT)
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    assert np.array_equal(got[~fin & ~np.isnan(ref)], ref[~fin & ~np.isnan(ref)])
    assert oracle.rel_frobenius(got[fin], ref[fin]) <= TOL[F32]


def test_float32_kernel_choice_follows_size_and_k(srt):
    dev = "cuda:0"
    small = torch.zeros((256, 256), device=dev)
    assert srt.query_plan(small, small, small)["kernel"] == SIMT
    a, b = torch.zeros((8192, 1024), device=dev), torch.zeros((1024, 256), device=dev)
    assert srt.query_plan(a, b, torch.zeros((8192, 256), device=dev))["kernel"] == X3          # streamed a, small b
    a, b = torch.zeros((1024, 1024), device=dev), torch.zeros((1024, 4096), device=dev)
    assert srt.query_plan(a, b, torch.zeros((1024, 4096), device=dev))["kernel"] == SPLIT      # b is the larger operand
    a, b = torch.zeros((1024, 8192), device=dev).t(), torch.zeros((1024, 256), device=dev)
    assert srt.query_plan(a, b, torch.zeros((8192, 256), device=dev), False, False)["kernel"] == SPLIT   # a not K-contiguous
    a, b = torch.zeros((1024, 4096), device=dev), torch.zeros((4096, 256), device=dev)
    plan = srt.query_plan(a, b, torch.zeros((1024, 256), device=dev))
    assert plan["kernel"] == SPLIT and plan["splitK"] >= 2                                 # K > 2048


@pytest.mark.parametrize("kernel", [TC, PAIR])
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("act,with_bias", [("relu", True), ("identity", True), ("relu", False), ("gelu", True)])
def test_tensor_core_fused_epilogue(srt, oracle, dtype, act, with_bias, kernel):
    srt.set_tuning(kernel, 0, 0, 0)
    rng = np.random.default_rng(21 + dtype)
    a = random_bits(oracle, rng, (300, 256), dtype, scale=0.05)
    w = random_bits(oracle, rng, (256, 520), dtype, scale=0.05)
    bias = random_bits(oracle, rng, (520,), dtype, scale=0.05) if with_bias else None
    got, ref = _run(srt, oracle, dtype, a, w, False, False, bias=bias, act=act, expect_kernel=kernel)
    assert oracle.rel_frobenius(oracle.decode(got, dtype), oracle.decode(ref, dtype)) <= 2e-3


def test_tensor_core_views_alignment_decides_the_kernel(srt, oracle):
    rng = np.random.default_rng(22)
    big_a, big_b = random_bits(oracle, rng, (300, 512), BF16), random_bits(oracle, rng, (512, 400), BF16)
    dev_a, dev_b = to_dev(big_a, BF16), to_dev(big_b, BF16)
    # 16-byte aligned sub-views with legal strides stay on the tensor cores
    got, ref = _run(srt, oracle, BF16, big_a[4:260, 64:448], big_b[64:448, 8:392], False, False, expect_kernel=TC,
                    da=dev_a[4:260, 64:448], db=dev_b[64:448, 8:392])
    assert oracle.rel_frobenius(oracle.decode(got, BF16), oracle.decode(ref, BF16)) <= 2e-3
    # an odd element offset breaks the 16-byte base alignment: strided kernel, bit-exact
    got, ref = _run(srt, oracle, BF16, big_a[4:260, 63:447], big_b[63:447, 8:392], False, False, expect_kernel=SIMT,
                    da=dev_a[4:260, 63:447], db=dev_b[63:447, 8:392])
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("dtype", [BF16, F16])
def test_col_order_output_runs_transposed_problem_with_row_bias(srt, oracle, dtype):
    """A col-order lhs gives a col-order result (Matmul.swift:36-38): computed as out^T = B^T . A^T."""
    srt.set_tuning(TC, 0, 0, 0)
    rng = np.random.default_rng(23)
    a, b = random_bits(oracle, rng, (264, 200), dtype), random_bits(oracle, rng, (200, 136), dtype)
    bias = random_bits(oracle, rng, (136,), dtype)
    ref = oracle.matmul(a, b, dtype, bias=bias, activation="relu")
    a_col = to_dev(np.asfortranarray(a), dtype)                  # logical [264 x 200], strides (1, 264)
    assert srt.order_of(a_col) == srt.Order.col
    c = srt.matmul(a_col, to_dev(b, dtype), bias=to_dev(bias, dtype), activation=srt.ActivationType.relu)
    assert srt.order_of(c) == srt.Order.col and c.stride() == (1, 264)
    plan = srt.query_plan(a_col, to_dev(b, dtype), c)
    assert plan["kernel"] in (TC, PAIR) and plan["swapped"] == 1
    got = from_dev(c, dtype)
    assert oracle.rel_frobenius(oracle.decode(got, dtype), oracle.decode(ref, dtype)) <= 2e-3


def test_identity_and_permutation_products_are_exact_at_full_size(srt):
    """Size-independent property at the large-square configuration's size: A . I == A and
    A . P permutes columns, bit for bit (every sum has one non-zero term)."""
    n = 16384
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)
    a = (torch.rand((n, n), device=dev, generator=g) * 2 - 1).to(torch.bfloat16)
    eye = torch.eye(n, dtype=torch.bfloat16, device=dev)
    c = srt.matmul(a, eye)
    assert torch.equal(c, a)
    perm = torch.randperm(n, device=dev, generator=g)
    c = srt.matmul(a, eye[:, perm].contiguous())
    assert torch.equal(c, a[:, perm])
    c = srt.matmul(eye, a, False, True)                          # I . A^T
    assert torch.equal(c, a.t())


# ------------------------------------------------------------------ split-K
@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("M,N,K,batch,ta,tb,splits", [
    (256, 256, 4096, 0, False, False, 4), (300, 200, 1000, 0, False, False, 3), (130, 203, 1024, 0, False, True, 8),
    (128, 64, 2048, 3, True, False, 2), (64, 512, 8192, 0, False, True, 0), (128, 128, 8192, 0, False, False, 0)])
def test_split_k_sixteen_bit(srt, oracle, dtype, M, N, K, batch, ta, tb, splits):
    """Reduction cut into parts (forced, or chosen automatically for few tiles and a long K):
    fp32 partial sums + reduce pass must give the same result within tolerance."""
    srt.set_tuning(TC, 0, 0, 0)
    srt.set_split_k(splits)
    rng = np.random.default_rng(M + 3 * N + 7 * K + dtype + 11)
    ash, bsh = _shapes(M, N, K, ta, tb, batch)
    a, b = random_bits(oracle, rng, ash, dtype), random_bits(oracle, rng, bsh, dtype)
    bias = random_bits(oracle, rng, (N,), dtype)
    ref = oracle.matmul(a, b, dtype, ta, tb, bias=bias, activation="relu")
    da, db, dbias = to_dev(a, dtype), to_dev(b, dtype), to_dev(bias, dtype)
    c = srt.matmul(da, db, ta, tb, bias=dbias, activation=srt.ActivationType.relu)
    plan = srt.query_plan(da, db, c, ta, tb)
    assert plan["kernel"] == TC and plan["splitK"] > 1
    assert plan["workspaceBytes"] == plan["splitK"] * max(batch, 1) * M * N * 4
    got = from_dev(c, dtype)
    assert oracle.rel_frobenius(oracle.decode(got, dtype), oracle.decode(ref, dtype)) <= 2e-3


def test_call_cache_slot_reused_by_another_kernel(srt):
    """The per-thread call cache has 64 slots.  Fill them with split-K launches, then run many
    distinct strided-kernel calls that land in the same slots: each must behave like a fresh call
    (no reduce pass of the slot's previous owner)."""
    torch.manual_seed(3)
    srt.set_tuning(TC, 0, 0, 0)
    srt.set_split_k(4)
    keep = []
    for i in range(96):
        a = torch.randn(128, 1024 + 64 * (i % 8), device="cuda:0", dtype=torch.bfloat16)
        b = torch.randn(a.shape[1], 64 + 8 * (i // 8), device="cuda:0", dtype=torch.bfloat16)
        keep.append((a, b, srt.matmul(a, b)))
    srt.set_tuning(SIMT, 0, 0, 0)
    srt.set_split_k(0)
    for i in range(192):
        a = torch.randn(1 + i % 7, 30 + i, device="cuda:0")
        b = torch.randn(30 + i, 5 + i % 11, device="cuda:0")
        c = srt.matmul(a, b)
        ref = a.double() @ b.double()
        assert torch.allclose(c.double(), ref, rtol=1e-4, atol=1e-4), i
    torch.cuda.synchronize()


def test_split_k_col_order_output_and_strided_view(srt, oracle):
    srt.set_tuning(TC, 0, 0, 0)
    srt.set_split_k(4)
    rng = np.random.default_rng(51)
    a, b = random_bits(oracle, rng, (264, 2048), BF16), random_bits(oracle, rng, (2048, 136), BF16)
    bias = random_bits(oracle, rng, (136,), BF16)
    ref = oracle.matmul(a, b, BF16, bias=bias, activation="relu")
    a_col = to_dev(np.asfortranarray(a), BF16)
    c = srt.matmul(a_col, to_dev(b, BF16), bias=to_dev(bias, BF16), activation=srt.ActivationType.relu)
    plan = srt.query_plan(a_col, to_dev(b, BF16), c)
    assert plan["swapped"] == 1 and plan["splitK"] > 1 and c.stride() == (1, 264)
    assert oracle.rel_frobenius(oracle.decode(from_dev(c, BF16), BF16), oracle.decode(ref, BF16)) <= 2e-3
    # a strided output view: only the view is written
    canvas = torch.full((300, 512), 7.0, dtype=torch.bfloat16, device="cuda:0")
    view = canvas[10:274, 64:200]
    srt.matmul_into(view, to_dev(a, BF16), False, to_dev(b, BF16), False)
    ref2 = oracle.matmul(a, b, BF16)
    assert oracle.rel_frobenius(oracle.decode(from_dev(view, BF16), BF16), oracle.decode(ref2, BF16)) <= 2e-3
    mask = torch.ones_like(canvas, dtype=torch.bool)
    mask[10:274, 64:200] = False
    assert bool((canvas[mask] == 7.0).all())


@pytest.mark.parametrize("M,N,K,ta,tb", [(512, 256, 4096, False, False), (256, 384, 8192, False, True), (1000, 520, 2056, True, False)])
def test_float32_large_k_uses_split_k_and_holds_tolerance(srt, oracle, M, N, K, ta, tb):
    """Beyond K = 2048 the 3 x TF32 kernel sums chunks of 2048 separately (accumulator truncation
    grows with K); the result must stay within 1e-5 for any K."""
    rng = np.random.default_rng(M + N + K)
    ash, bsh = _shapes(M, N, K, ta, tb)
    a, b = random_bits(oracle, rng, ash, F32), random_bits(oracle, rng, bsh, F32)
    ref = oracle.matmul(a, b, F32, ta, tb)
    da, db = to_dev(a, F32), to_dev(b, F32)
    c = srt.matmul(da, db, ta, tb)
    plan = srt.query_plan(da, db, c, ta, tb)
    assert plan["kernel"] == SPLIT and plan["splitK"] >= -(-K // 2048)
    assert oracle.rel_frobenius(from_dev(c, F32), ref) <= TOL[F32]


# ------------------------------------------------------------------ the five named configurations
def _sample_rows(M, count, tile=128):
    """Rows covering both matrix edges and every residue class of the tile height."""
    rng = np.random.default_rng(0)
    rows = {0, M - 1, tile - 1 if M >= tile else 0, min(M - 1, tile)}
    while len(rows) < min(count, M):
        rows.add(int(rng.integers(0, M)))
    return sorted(rows)


def test_config1_float32_256_cubed(srt, oracle):
    rng = np.random.default_rng(0)
    a, b = random_bits(oracle, rng, (256, 256), F32), random_bits(oracle, rng, (256, 256), F32)
    got, ref = _run(srt, oracle, F32, a, b, False, False)
    assert oracle.rel_frobenius(got, ref) <= TOL[F32]
    assert np.array_equal(got, ref)           # the fp32 path keeps the reference's arithmetic order


def test_config2_dense_bf16_bias_relu(srt, oracle):
    rng = np.random.default_rng(0)
    x = random_bits(oracle, rng, (1024, 4096), BF16, scale=0.05)
    w = random_bits(oracle, rng, (4096, 4096), BF16, scale=0.05)
    bias = random_bits(oracle, rng, (4096,), BF16, scale=0.05)
    layer = srt.Dense(to_dev(w, BF16), to_dev(bias, BF16), srt.ActivationType.relu)
    dx = to_dev(x, BF16)
    y = layer(dx)
    assert srt.query_plan(dx, layer.weight, y)["kernel"] in (TC, PAIR)
    ref = oracle.matmul(x, w, BF16, bias=bias, activation="relu")
    got = from_dev(y, BF16)
    err = oracle.rel_frobenius(oracle.decode(got, BF16), oracle.decode(ref, BF16))
    assert err <= TOL[BF16] and err <= 2e-3


def test_config3_batched_fp16_attention_score_shape(srt, oracle):
    rng = np.random.default_rng(0)
    a = random_bits(oracle, rng, (64, 512, 64), F16, dist="normal")
    b = random_bits(oracle, rng, (64, 512, 64), F16, dist="normal")
    got, ref = _run(srt, oracle, F16, a, b, False, True)
    err = oracle.rel_frobenius(oracle.decode(got, F16), oracle.decode(ref, F16))
    assert err <= TOL[F16] and err <= 2e-3


def test_config4_tall_skinny_float32(srt, oracle):
    rng = np.random.default_rng(0)
    a, b = random_bits(oracle, rng, (65536, 1024), F32), random_bits(oracle, rng, (1024, 256), F32)
    da, db = to_dev(a, F32), to_dev(b, F32)
    c = srt.matmul(da, db)
    assert srt.query_plan(da, db, c)["kernel"] == X3
    got = from_dev(c, F32)
    rows = _sample_rows(65536, 2048)
    ref = oracle.matmul(np.ascontiguousarray(a[rows]), b, F32)
    assert oracle.rel_frobenius(got[rows], ref) <= TOL[F32]
    # column checksums over ALL rows against float64: sum_i C_ij = (sum_i A_i.) . B_.j ; a lost or
    # duplicated tile row would move a column sum by hundreds, rounding moves it by ~1e-2
    want = a.astype(np.float64).sum(axis=0) @ b.astype(np.float64)
    assert float(np.abs(got.astype(np.float64).sum(axis=0) - want).max()) < 1.0


def test_config5_large_square_bf16(srt, oracle):
    n = 16384
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(0)
    a = (torch.rand((n, n), device=dev, generator=g) * 2 - 1).to(torch.bfloat16)
    b = (torch.rand((n, n), device=dev, generator=g) * 2 - 1).to(torch.bfloat16)
    c = srt.matmul(a, b)
    assert srt.query_plan(a, b, c)["kernel"] in (TC, 3)
    # sampled rows against the CPU oracle on the same stored bits
    rows = _sample_rows(n, 24)
    idx = torch.tensor(rows, device=dev)
    a_rows = from_dev(a[idx], BF16)
    b_host = from_dev(b, BF16)
    ref = oracle.matmul(a_rows, b_host, BF16)
    got = from_dev(c[idx], BF16)
    err = oracle.rel_frobenius(oracle.decode(got, BF16), oracle.decode(ref, BF16))
    assert err <= TOL[BF16] and err <= 2e-3
    # a band of 1024 full rows against the reference-ordered strided kernel (itself bit-exact with the oracle)
    srt.set_tuning(SIMT, 0, 0, 0)
    band = slice(7 * 1024 + 64, 8 * 1024 + 64)
    exact = srt.matmul(a[band].contiguous(), b)
    diff = (c[band].float() - exact.float()).norm() / exact.float().norm()
    assert float(diff) <= 2e-3


# ------------------------------------------------------------------ host buffers and bookkeeping
def test_host_buffer_entry_and_launch_counter(srt, oracle):
    rng = np.random.default_rng(31)
    a, b = random_bits(oracle, rng, (256, 384), BF16), random_bits(oracle, rng, (384, 512), BF16)
    ha = torch.from_numpy(a).view(torch.bfloat16).pin_memory()
    hb = torch.from_numpy(b).view(torch.bfloat16).pin_memory()
    before = srt.launch_count()
    hc = srt.matmul_host(ha, hb)
    assert srt.launch_count() == before + 1
    assert not hc.is_cuda
    ref = oracle.matmul(a, b, BF16)
    got = hc.view(torch.uint16).numpy()
    assert oracle.rel_frobenius(oracle.decode(got, BF16), oracle.decode(ref, BF16)) <= 2e-3


def test_host_buffer_entry_pipelined_over_row_blocks(srt, oracle):
    """Large host products are cut into row blocks whose copies overlap the math: same result."""
    rng = np.random.default_rng(32)
    M, K, N = 4096 + 200, 4096, 2048
    a, b = random_bits(oracle, rng, (M, K), BF16), random_bits(oracle, rng, (K, N), BF16)
    bias = random_bits(oracle, rng, (N,), BF16)
    ha = torch.from_numpy(a).view(torch.bfloat16).pin_memory()
    hb = torch.from_numpy(b).view(torch.bfloat16).pin_memory()
    hbias = torch.from_numpy(bias).view(torch.bfloat16).pin_memory()
    before = srt.launch_count()
    hc = srt.matmul_host(ha, hb, bias=hbias, activation=srt.ActivationType.relu)
    assert 2 <= srt.launch_count() - before <= 16        # one launch per row block
    whole = srt.matmul_host(ha, hb, bias=hbias, activation=srt.ActivationType.relu, chunks=1)
    # row blocks and the whole product may run under different plans (tile width, split-K): equal up to
    # the last bit of a BFloat16 here and there, not bit for bit
    assert oracle.rel_frobenius(hc.float().numpy(), whole.float().numpy()) <= 1e-3
    rows = _sample_rows(M, 48)
    ref = oracle.matmul(np.ascontiguousarray(a[rows]), b, BF16, bias=bias, activation="relu")
    got = hc.view(torch.uint16).numpy()[rows]
    assert oracle.rel_frobenius(oracle.decode(got, BF16), oracle.decode(ref, BF16)) <= 2e-3


def test_unsupported_inputs_return_not_supported(srt):
    a = torch.zeros((4, 4), dtype=torch.float64, device="cuda:0")
    with pytest.raises(srt.MatmulError) as e:
        srt.matmul(a, a)
    assert e.value.code == 801


def test_empty_results_and_empty_reductions(srt):
    """Edge cases of the loop nest (CpuMath.swift:1141-1186): no rows, no columns or no batch items
    write nothing; a reduction over no terms gives 0 (+ bias, activation) in every element."""
    dev = "cuda:0"
    before = srt.launch_count()
    for ash, bsh in (((0, 8), (8, 5)), ((4, 8), (8, 0)), ((0, 3, 8), (0, 8, 5))):
        c = srt.matmul(torch.zeros(ash, device=dev), torch.zeros(bsh, device=dev))
        assert tuple(c.shape) == tuple(ash[:-1]) + (bsh[-1],) and c.numel() == 0
    assert srt.launch_count() == before                                   # nothing was launched
    for dtype in (torch.float32, torch.bfloat16):
        a, b = torch.zeros((6, 0), device=dev, dtype=dtype), torch.zeros((0, 10), device=dev, dtype=dtype)
        out = torch.full((6, 10), 7.0, device=dev, dtype=dtype)
        srt.matmul_into(out, a, False, b, False)
        assert bool((out == 0).all())
        bias = torch.arange(-5, 5, device=dev).to(dtype)
        y = srt.matmul(a, b, bias=bias, activation=srt.ActivationType.relu)
        assert torch.equal(y, torch.relu(bias).expand(6, 10))
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype,kernel", [(F32, SIMT), (BF16, TC), (F16, PAIR), (F32, SPLIT)])
def test_small_shape_sweep_with_guard_bands(srt, oracle, dtype, kernel):
    """Every combination of M, N, K from {1, 2, 3, 5, 8, 9, 16, 17, 31, 32, 33}: the strided kernel
    bit-exact, the tensor-core kernels (which take the shapes TMA can address and leave the rest
    to the strided kernel) within tolerance; sentinels before and after the result stay intact."""
    sizes = (1, 2, 3, 5, 8, 9, 16, 17, 31, 32, 33)
    rng = np.random.default_rng(dtype * 7 + kernel)
    srt.set_tuning(kernel, 0, 0, 0)
    tdt = {F32: torch.float32, BF16: torch.bfloat16, F16: torch.float16}[dtype]
    a_all = random_bits(oracle, rng, (33, 33), dtype)
    b_all = random_bits(oracle, rng, (33, 33), dtype)
    guard = 32
    worst = 0.0
    for M in sizes:
        for K in sizes:
            a = np.ascontiguousarray(a_all[:M, :K])
            da = to_dev(a, dtype)
            for N in sizes:
                b = np.ascontiguousarray(b_all[:K, :N])
                canvas = torch.full((guard + M * N + guard,), 3.0, dtype=tdt, device="cuda:0")
                out = canvas[guard:guard + M * N].view(M, N)
                srt.matmul_into(out, da, False, to_dev(b, dtype), False)
                ref = oracle.matmul(a, b, dtype, threads=1)
                got = from_dev(out, dtype)
                if kernel == SIMT:
                    assert np.array_equal(got, ref), (M, N, K)
                else:
                    err = oracle.rel_frobenius(oracle.decode(got, dtype), oracle.decode(ref, dtype))
                    worst = max(worst, err)
                    assert err <= TOL[dtype], (M, N, K, err)
                assert bool((canvas[:guard] == 3.0).all()) and bool((canvas[guard + M * N:] == 3.0).all()), (M, N, K)
    assert srt.check_status() == 0


@pytest.mark.parametrize("dtype", [BF16, F16])
@pytest.mark.parametrize("M,K,N,transposed", [(1, 1024, 512, False), (1, 4096, 4096, True), (8, 4096, 4096, True),
                                              (33, 2048, 1000, True), (64, 4096, 4096, True), (64, 1024, 8192, False),
                                              (100, 4096, 2048, True), (256, 4096, 4096, True)])
def test_small_batch_runs_transposed_with_split_k(srt, oracle, dtype, M, K, N, transposed):
    """A few rows against a wide weight are planned as the transposed problem (the wide dimension
    fills the MMA's 128 rows) with split-K, whose reduce pass writes the row-major result; bias and
    activation follow the columns of the result as usual."""
    rng = np.random.default_rng(M + K + N + dtype)
    a, b = random_bits(oracle, rng, (M, K), dtype, scale=0.5), random_bits(oracle, rng, (K, N), dtype, scale=0.5)
    bias = random_bits(oracle, rng, (N,), dtype)
    ref = oracle.matmul(a, b, dtype, bias=bias, activation="relu")
    da, db, dbias = to_dev(a, dtype), to_dev(b, dtype), to_dev(bias, dtype)
    canvas = torch.full((M + 2, N), 9.0, dtype=da.dtype, device="cuda:0")
    out = canvas[1:M + 1]
    srt.matmul_into(out, da, False, db, False, dbias, srt.ActivationType.relu)
    plan = srt.query_plan(da, db, out)
    if transposed:
        assert plan["kernel"] == TC and plan["swapped"] == 1 and plan["splitK"] > 1, plan
        assert plan["tileN"] == (64 if M <= 64 else 128 if M <= 128 else 256), plan
    else:
        assert plan["swapped"] == 0, plan          # too short a reduction to split: the given orientation
    err = oracle.rel_frobenius(oracle.decode(from_dev(out, dtype), dtype), oracle.decode(ref, dtype))
    assert err <= 2e-3, err
    assert bool((canvas[0] == 9.0).all()) and bool((canvas[M + 1] == 9.0).all())
    # more than 256 rows keep the given orientation
    big = torch.zeros((257, K), dtype=da.dtype, device="cuda:0")
    assert srt.query_plan(big, db, torch.zeros((257, N), dtype=da.dtype, device="cuda:0"))["swapped"] == 0


@pytest.mark.parametrize("ta,tb", TRANSPOSES)
def test_small_batch_transposed_plan_all_transposes(srt, oracle, ta, tb):
    rng = np.random.default_rng(5 + 2 * ta + tb)
    M, K, N = 24, 2048, 1536
    ash, bsh = _shapes(M, N, K, ta, tb)
    a, b = random_bits(oracle, rng, ash, BF16, scale=0.5), random_bits(oracle, rng, bsh, BF16, scale=0.5)
    bias = random_bits(oracle, rng, (N,), BF16)
    got, ref = _run(srt, oracle, BF16, a, b, ta, tb, bias=bias, act="gelu")
    assert oracle.rel_frobenius(oracle.decode(got, BF16), oracle.decode(ref, BF16)) <= 2e-3
    da, db = to_dev(a, BF16), to_dev(b, BF16)
    plan = srt.query_plan(da, db, torch.empty((M, N), dtype=torch.bfloat16, device="cuda:0"), ta, tb)
    assert plan["swapped"] == 1 and plan["splitK"] > 1, plan
