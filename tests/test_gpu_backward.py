"""Backward of the Dense path on a B200, through the C ABI, against the CPU oracle.

dz = dy * act'(y) is elementwise with one rounding, so it must match the oracle bit for bit;
dbias is a column sum whose order differs from the oracle's sequential sum, so it is compared
within the path's tolerances (1e-5 Float32, 1e-2 16-bit)."""
import numpy as np
import pytest
import torch

from _gpu_util import BF16, F16, F32, TOL, from_dev, random_bits, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def srt():
    import swiftrt_b200 as s
    assert torch.cuda.is_available()
    return s


def _forward_like(oracle, rng, shape, dtype, act):
    """A plausible forward output y for the activation (range matters for the derivative)."""
    z = rng.standard_normal(shape)
    y = {"relu": np.maximum(z, 0), "sigmoid": 1 / (1 + np.exp(-z)), "tanh": np.tanh(z), "identity": z}[act]
    return oracle.encode(y.astype(np.float32), dtype)


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
@pytest.mark.parametrize("act", ["identity", "relu", "sigmoid", "tanh"])
@pytest.mark.parametrize("M,N", [(1, 8), (300, 17), (1024, 4096), (777, 520)])
def test_bias_activation_backward_matches_oracle(srt, oracle, dtype, act, M, N):
    rng = np.random.default_rng(M * 7 + N + dtype)
    dy = random_bits(oracle, rng, (M, N), dtype, dist="normal")
    y = _forward_like(oracle, rng, (M, N), dtype, act)
    dz_ref, db_ref = oracle.bias_activation_backward(dy, y, dtype, act)
    before = srt.launch_count()
    dz, db = srt.bias_activation_backward(to_dev(dy, dtype), to_dev(y, dtype), srt.ActivationType[act])
    torch.cuda.synchronize()
    assert srt.launch_count() == before + 2
    assert np.array_equal(from_dev(dz, dtype), dz_ref)
    err = oracle.rel_frobenius(oracle.decode(from_dev(db, dtype), dtype), oracle.decode(db_ref, dtype))
    assert err <= TOL[dtype], err


def test_backward_strided_views_batches_and_optional_outputs(srt, oracle):
    rng = np.random.default_rng(3)
    big_dy = random_bits(oracle, rng, (3, 40, 70), F32, dist="normal")
    big_y = _forward_like(oracle, rng, (3, 40, 70), F32, "relu")
    dy, y = big_dy[:, 2:35, 5:64:3], big_y[:, 2:35, 5:64:3]            # rank 3, column stride 3
    flat_dy = np.ascontiguousarray(dy).reshape(-1, dy.shape[-1])
    flat_y = np.ascontiguousarray(y).reshape(-1, y.shape[-1])
    dz_ref, db_ref = oracle.bias_activation_backward(flat_dy, flat_y, F32, "relu")
    dz, db = srt.bias_activation_backward(to_dev(dy, F32), to_dev(y, F32), srt.ActivationType.relu)
    assert np.array_equal(from_dev(dz, F32).reshape(-1, dy.shape[-1]), dz_ref)
    assert oracle.rel_frobenius(from_dev(db, F32), db_ref) <= TOL[F32]
    only_db = srt.bias_activation_backward(to_dev(dy, F32), to_dev(y, F32), srt.ActivationType.relu, want_dz=False)
    assert only_db[0] is None and torch.equal(only_db[1], db)
    only_dz = srt.bias_activation_backward(to_dev(dy, F32), to_dev(y, F32), srt.ActivationType.relu, want_dbias=False)
    assert only_dz[1] is None and torch.equal(only_dz[0], dz)
    with pytest.raises(srt.MatmulError) as e:
        srt.bias_activation_backward(to_dev(dy, F32), to_dev(y, F32), srt.ActivationType.elu)
    assert e.value.code == 801


@pytest.mark.parametrize("dtype", [BF16, F32])
def test_dense_layer_backward_against_oracle_composition(srt, oracle, dtype):
    """dx = dz . W^T, dW = x^T . dz, db = column sums of dz for y = relu(x . W + b): every piece
    against the oracle fed with the same stored bits."""
    rng = np.random.default_rng(4)
    M, K, N = 384, 512, 264
    x = random_bits(oracle, rng, (M, K), dtype, scale=0.5)
    w = random_bits(oracle, rng, (K, N), dtype, scale=0.1)
    b = random_bits(oracle, rng, (N,), dtype, scale=0.1)
    dy = random_bits(oracle, rng, (M, N), dtype, dist="normal")
    layer = srt.Dense(to_dev(w, dtype), to_dev(b, dtype), srt.ActivationType.relu)
    dx_in = to_dev(x, dtype)
    y = layer(dx_in)
    y_bits = from_dev(y, dtype)
    dx, dw, db = layer.backward(dx_in, y, to_dev(dy, dtype))
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    dz_ref, db_ref = oracle.bias_activation_backward(dy, y_bits, dtype, "relu")     # same y as the GPU used
    dx_ref = oracle.matmul(dz_ref, w, dtype, False, True)
    dw_ref = oracle.matmul(x, dz_ref, dtype, True, False)
    tol = 2e-3 if dtype != F32 else TOL[F32]
    for got, ref in ((dx, dx_ref), (dw, dw_ref), (db, db_ref)):
        assert oracle.rel_frobenius(oracle.decode(from_dev(got, dtype), dtype), oracle.decode(ref, dtype)) <= tol


def test_matmul_gradient_literals_with_bias_sum(srt):
    """The reference's gradient literals for the batched cases need a sum over the batch for the
    broadcast operand (Tests/SwiftRTCoreTests/test_AlgebraicField.swift:601-645); the column-sum
    kernel provides it: grad of the rank-2 rhs of test_leftBatchMatmul = sum over the batch of A^T . 1."""
    dev = "cuda:0"
    a = torch.arange(12.0, device=dev).reshape(2, 3, 2)
    ones = torch.ones((2, 3, 4), device=dev)
    per_item = srt.matmul(a, ones, True, False)                      # [2, 2, 4]
    # sum over the batch = column sums of the [batch x (2*4)] matrix of flattened items
    _, total = srt.bias_activation_backward(per_item.reshape(2, 8), None, srt.ActivationType.identity, want_dz=False)
    assert total.reshape(2, 4).cpu().tolist() == [[30.0] * 4, [36.0] * 4]


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
@pytest.mark.parametrize("act", ["gelu", "geluTanh"])
@pytest.mark.parametrize("M,N", [(300, 17), (1024, 4096)])
def test_gelu_backward_from_pre_activation_values(srt, oracle, dtype, act, M, N):
    """GELU's derivative is evaluated at the pre-activation values z (the reference leaves it as
    fatalError, MathDerivatives.swift:520-554).  erff / tanhf differ by a few ulp between the device
    and libm, so dz is compared within the path's tolerances rather than bit for bit."""
    rng = np.random.default_rng(M + N + dtype)
    dy = random_bits(oracle, rng, (M, N), dtype, dist="normal")
    z = random_bits(oracle, rng, (M, N), dtype, dist="normal", scale=1.0)
    dz_ref, db_ref = oracle.bias_activation_backward(dy, z, dtype, act)
    dz, db = srt.bias_activation_backward(to_dev(dy, dtype), to_dev(z, dtype), srt.ActivationType[act])
    torch.cuda.synchronize()
    tol = 1e-5 if dtype == F32 else TOL[dtype]
    assert oracle.rel_frobenius(oracle.decode(from_dev(dz, dtype), dtype), oracle.decode(dz_ref, dtype)) <= tol
    assert oracle.rel_frobenius(oracle.decode(from_dev(db, dtype), dtype), oracle.decode(db_ref, dtype)) <= TOL[dtype]
    # and against the analytic derivative in float64
    zf = oracle.decode(z, dtype).astype(np.float64)
    if act == "gelu":
        from math import erf
        cdf = 0.5 * (1 + np.vectorize(erf)(zf[:64] / np.sqrt(2)))
        want = oracle.decode(dy, dtype)[:64] * (cdf + zf[:64] * np.exp(-0.5 * zf[:64] ** 2) / np.sqrt(2 * np.pi))
        assert oracle.rel_frobenius(oracle.decode(from_dev(dz, dtype), dtype)[:64], want) <= (1e-5 if dtype == F32 else 1e-2)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("act", ["gelu", "geluTanh", "relu", "tanh"])
def test_activation_forward_matches_oracle(srt, oracle, dtype, act):
    rng = np.random.default_rng(11)
    big = random_bits(oracle, rng, (2, 70, 136), dtype, dist="normal")
    for z in (big, big[:, 3:61, 8:128], big[0, :, ::3]):            # dense, aligned view, strided view
        want = oracle.activation_forward(np.ascontiguousarray(z), dtype, act)
        got = srt.activation_forward(to_dev(z, dtype), srt.ActivationType[act])
        tol = 1e-6 if dtype == F32 else TOL[dtype]
        assert oracle.rel_frobenius(oracle.decode(from_dev(got, dtype), dtype), oracle.decode(want, dtype)) <= tol


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_gelu_dense_layer_trains(srt, oracle, dtype):
    """A GELU Dense: forward_keep keeps z, backward gives dx, dW, db; every piece against the oracle."""
    rng = np.random.default_rng(5)
    M, K, N = 256, 384, 264
    x = random_bits(oracle, rng, (M, K), dtype, scale=0.5)
    w = random_bits(oracle, rng, (K, N), dtype, scale=0.1)
    b = random_bits(oracle, rng, (N,), dtype, scale=0.1)
    dy = random_bits(oracle, rng, (M, N), dtype, dist="normal")
    layer = srt.Dense(to_dev(w, dtype), to_dev(b, dtype), srt.ActivationType.gelu)
    dx_in = to_dev(x, dtype)
    y, saved = layer.forward_keep(dx_in)
    z_ref = oracle.matmul(x, w, dtype, bias=b)
    tol = 2e-3 if dtype != F32 else TOL[F32]
    assert oracle.rel_frobenius(oracle.decode(from_dev(saved, dtype), dtype), oracle.decode(z_ref, dtype)) <= tol
    y_fused = layer(dx_in)                                                # the inference path: one fused launch
    assert oracle.rel_frobenius(oracle.decode(from_dev(y, dtype), dtype), oracle.decode(from_dev(y_fused, dtype), dtype)) <= (1e-6 if dtype == F32 else 1e-2)
    dx, dw, db = layer.backward(dx_in, saved, to_dev(dy, dtype))
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    z_bits = from_dev(saved, dtype)
    dz_ref, db_ref = oracle.bias_activation_backward(dy, z_bits, dtype, "gelu")
    dx_ref = oracle.matmul(dz_ref, w, dtype, False, True)
    dw_ref = oracle.matmul(x, dz_ref, dtype, True, False)
    for got, ref in ((dx, dx_ref), (dw, dw_ref), (db, db_ref)):
        assert oracle.rel_frobenius(oracle.decode(from_dev(got, dtype), dtype), oracle.decode(ref, dtype)) <= tol
