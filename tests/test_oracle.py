"""The CPU oracle against the reference's own known-answer vectors and against itself.

The vectors are the literals of Tests/SwiftRTCoreTests/test_AlgebraicField.swift:551-645
(tests/golden/matmul_kat.json, written by tests/golden/make_kat.py)."""
import json
import os

import numpy as np
import pytest
import torch

F32, F16, BF16 = 0, 2, 14
GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "matmul_kat.json")


def _kat():
    with open(GOLDEN) as f:
        return json.load(f)["cases"]


def _range(shape):
    return np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)


def _bcast3(x, nb):
    return x if x.ndim == 3 else np.broadcast_to(x, (nb,) + x.shape)


@pytest.mark.parametrize("name", ["test_matmul", "test_batchMatmul", "test_leftBatchMatmul", "test_rightBatchMatmul"])
@pytest.mark.parametrize("mode", [0, 1])
def test_known_answers_forward(oracle, name, mode):
    case = _kat()[name]
    a, b = _range(case["a_shape"]), _range(case["b_shape"])
    if a.ndim != b.ndim:                       # left / right batch forms: stride-0 broadcast view
        nb = max(a.shape[0] if a.ndim == 3 else 1, b.shape[0] if b.ndim == 3 else 1)
        a, b = _bcast3(a, nb), _bcast3(b, nb)
    c = oracle.matmul(a, b, F32, mode=mode)
    if "c" in case:
        assert np.array_equal(c, np.array(case["c"], dtype=np.float32))
    else:
        assert np.array_equal(c[0], np.array(case["c_first_item"], dtype=np.float32))


@pytest.mark.parametrize("name", ["test_matmul", "test_batchMatmul", "test_leftBatchMatmul", "test_rightBatchMatmul"])
def test_known_answers_gradients(oracle, name):
    """matmulGradients' (false, false) case: lhsGrad = dC . B^T, rhsGrad = A^T . dC
    (MathDerivatives.swift:468-470) with dC = ones; a broadcast operand sums over the batch."""
    case = _kat()[name]
    a, b = _range(case["a_shape"]), _range(case["b_shape"])
    nb = max(a.shape[0] if a.ndim == 3 else 1, b.shape[0] if b.ndim == 3 else 1)
    batched = a.ndim == 3 or b.ndim == 3
    a3, b3 = (_bcast3(a, nb), _bcast3(b, nb)) if batched else (a, b)
    c = oracle.matmul(a3, b3, F32)
    ones = np.ones_like(c)
    ga = oracle.matmul(ones, b3, F32, False, True)
    gb = oracle.matmul(a3, ones, F32, True, False)
    if batched and a.ndim == 2:
        ga = ga.sum(axis=0)
    if batched and b.ndim == 2:
        gb = gb.sum(axis=0)
    assert np.array_equal(ga, np.array(case["grad_a"], dtype=np.float32))
    assert np.array_equal(gb, np.array(case["grad_b"], dtype=np.float32))


def test_bf16_codec_matches_round_to_nearest_even(oracle):
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-30, 30, 20000),
                        np.array([0.0, -0.0, 1.0, np.inf, -np.inf, 65504.0, 3.3895314e38, 1e-45], dtype=np.float32)])
    x = x.astype(np.float32)
    got = oracle.encode(x, BF16)
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(got, want)
    assert np.array_equal(oracle.decode(got, BF16), torch.from_numpy(want).view(torch.bfloat16).float().numpy())
    # ties: exactly halfway patterns round to even
    ties = np.array([0x3f808000, 0x3f818000, 0xbf808000], dtype=np.uint32).view(np.float32)
    assert list(oracle.encode(ties, BF16)) == [0x3f80, 0x3f82, 0xbf80]
    # the reference maps every NaN to 0x7fff (BFloat16.swift:71-73)
    assert list(oracle.encode(np.array([np.nan, -np.nan], dtype=np.float32), BF16)) == [0x7fff, 0x7fff]


def test_f16_codec_matches_ieee(oracle):
    rng = np.random.default_rng(2)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 10.0 ** rng.integers(-9, 6, 20000),
                        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.9604645e-8, 2.9802322e-8,
                                  2.98023224e-8 * 1.0000001, 6.1035156e-5, np.inf, -np.inf], dtype=np.float32)])
    x = x.astype(np.float32)
    got = oracle.encode(x, F16)
    want = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)
    allbits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    finite = allbits[(allbits & 0x7c00) != 0x7c00]
    assert np.array_equal(oracle.decode(finite, F16), finite.view(np.float16).astype(np.float32))
    assert np.array_equal(oracle.encode(oracle.decode(finite, F16), F16), finite)
    assert list(oracle.encode(np.array([np.nan], dtype=np.float32), F16)) == [0x7fff]


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_fast_loop_is_bit_identical_to_faithful_loop(oracle, dtype, ta, tb):
    rng = np.random.default_rng(3)
    M, N, K, nb = 37, 29, 53, 3
    a = oracle.encode(rng.uniform(-1, 1, (nb, K, M) if ta else (nb, M, K)), dtype)
    b = oracle.encode(rng.uniform(-1, 1, (nb, N, K) if tb else (nb, K, N)), dtype)
    bias = oracle.encode(rng.uniform(-1, 1, (N,)), dtype)
    c0 = oracle.matmul(a, b, dtype, ta, tb, bias=bias, activation="relu", mode=0)
    c1 = oracle.matmul(a, b, dtype, ta, tb, bias=bias, activation="relu", mode=1, threads=4)
    assert np.array_equal(c0, c1)


def test_matches_float64_and_handles_views(oracle):
    rng = np.random.default_rng(4)
    big_a = rng.uniform(-1, 1, (40, 90)).astype(np.float32)
    big_b = rng.uniform(-1, 1, (90, 70)).astype(np.float32)
    a = big_a[3:35:2, 5:85:3]        # 16 x 27, strides (180, 3)
    b = big_b[10:37, 1:61:4]         # 27 x 15
    out = np.zeros((16, 40), dtype=np.float32)
    view = out[:, 2:32:2]            # strided output view
    oracle.matmul(a, b, F32, out=view)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert oracle.rel_frobenius(view, ref) < 1e-6
    assert np.all(out[:, 1::2] == 0) and np.all(out[:, 32:] == 0)      # nothing outside the view
    # column-order storage is a strided view of the same logical matrix (Shape.swift:292-297)
    a_col = np.asfortranarray(a)
    assert np.array_equal(oracle.matmul(a_col, b, F32), oracle.matmul(np.ascontiguousarray(a), b, F32))


def test_sequential_fp32_accumulation_order(oracle):
    """1 + 2^-24 + 2^-24 in k order stays 1 in fp32 (each add rounds back), whereas a pairwise
    or wider accumulation would give 1 + 2^-23: pins the reference's strictly sequential sum."""
    a = np.array([[1.0, 2.0 ** -24, 2.0 ** -24]], dtype=np.float32)
    b = np.ones((3, 1), dtype=np.float32)
    assert oracle.matmul(a, b, F32)[0, 0] == np.float32(1.0)
    a2 = np.array([[2.0 ** -24, 2.0 ** -24, 1.0]], dtype=np.float32)
    assert oracle.matmul(a2, b, F32)[0, 0] == np.float32(1.0 + 2.0 ** -23)


def test_f16_native_accumulation_variant_is_within_tolerance(oracle):
    """The reference has two Float16 value types (Float16.swift:12-16 native, :173-211 emulated with
    fp32 accumulation).  The graded oracle is the fp32-accumulate one; the native variant stays
    inside the 1e-2 tolerance at the attention-score shape's K = 64."""
    rng = np.random.default_rng(5)
    a = oracle.encode(rng.standard_normal((2, 64, 64)), F16)
    b = oracle.encode(rng.standard_normal((2, 48, 64)), F16)
    c32 = oracle.matmul(a, b, F16, False, True)
    c16 = oracle.matmul(a, b, F16, False, True, f16_native=True)
    d = oracle.rel_frobenius(oracle.decode(c16, F16), oracle.decode(c32, F16))
    assert 0 < d < 1e-2


def test_fused_dense_epilogue_is_within_tolerance_of_unfused_ops(oracle):
    rng = np.random.default_rng(6)
    x = oracle.encode(rng.uniform(-0.05, 0.05, (64, 512)), BF16)
    w = oracle.encode(rng.uniform(-0.05, 0.05, (512, 96)), BF16)
    bias = oracle.encode(rng.uniform(-0.05, 0.05, (96,)), BF16)
    fused = oracle.matmul(x, w, BF16, bias=bias, activation="relu")
    unfused = oracle.matmul(x, w, BF16)
    oracle.lib().oracle_bias_activation_unfused(BF16, unfused.ctypes.data, 64, 96, bias.ctypes.data, oracle.ACT["relu"])
    assert oracle.rel_frobenius(oracle.decode(unfused, BF16), oracle.decode(fused, BF16)) < 1e-2
    # plain matmul(bias:) of the reference ignores the bias (Matmul.swift:70): has_epilogue = 0
    assert np.array_equal(oracle.matmul(x, w, BF16), oracle.matmul(x, w, BF16, bias=None, activation=None))


def test_relu_maps_nan_to_zero_like_cpu_max(oracle):
    a = np.array([[np.nan, 1.0]], dtype=np.float32)
    b = np.array([[1.0], [1.0]], dtype=np.float32)
    assert oracle.matmul(a, b, F32, activation="relu")[0, 0] == 0.0
    assert np.isnan(oracle.matmul(a, b, F32, activation="identity")[0, 0])


def test_row_window_leaves_other_rows_untouched(oracle):
    rng = np.random.default_rng(7)
    a = rng.uniform(-1, 1, (20, 8)).astype(np.float32)
    b = rng.uniform(-1, 1, (8, 5)).astype(np.float32)
    full = oracle.matmul(a, b, F32)
    part = np.full((20, 5), 7.0, dtype=np.float32)
    oracle.matmul(a, b, F32, out=part, rows=(4, 9))
    assert np.array_equal(part[4:9], full[4:9]) and np.all(part[:4] == 7) and np.all(part[9:] == 7)


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
@pytest.mark.parametrize("act", ["identity", "relu", "sigmoid", "tanh"])
def test_bias_activation_backward_restatement(oracle, dtype, act):
    """dz = dy * act'(y) and dbias = column sums, against float64; the reference-style row-by-row
    rounding of the running sum (cpu_sum keeps it in the output tensor) is recorded next to the
    graded fp32 running sum."""
    rng = np.random.default_rng(8)
    y = oracle.encode(np.tanh(rng.standard_normal((300, 17))) if act != "sigmoid" else rng.uniform(0, 1, (300, 17)), dtype)
    dy = oracle.encode(rng.standard_normal((300, 17)), dtype)
    dz, db = oracle.bias_activation_backward(dy, y, dtype, act)
    yf, gf = oracle.decode(y, dtype).astype(np.float64), oracle.decode(dy, dtype).astype(np.float64)
    grad = {"identity": np.ones_like(yf), "relu": (yf > 0).astype(np.float64), "sigmoid": yf * (1 - yf),
            "tanh": 1 - yf * yf}[act]
    tol = 1e-6 if dtype == F32 else 1e-2
    assert oracle.rel_frobenius(oracle.decode(dz, dtype), gf * grad) <= tol
    assert oracle.rel_frobenius(oracle.decode(db, dtype), oracle.decode(dz, dtype).astype(np.float64).sum(axis=0)) <= tol
    _, db_step = oracle.bias_activation_backward(dy, y, dtype, act, stepwise=True)
    if dtype == F32:
        assert np.array_equal(db_step, db)          # fp32 elements: rounding every row IS the fp32 running sum
    else:
        assert oracle.rel_frobenius(oracle.decode(db_step, dtype), oracle.decode(db, dtype)) < 0.1


# ------------------------------------------------------------------ LSTM cell: the reference's golden data
def _lstm_kat():
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "lstm_kat.json")) as f:
        return json.load(f)


def test_lstm_cell_restatement_reproduces_reference_golden_states(oracle):
    """Four time steps with the reference's weights, bias and initial state
    (Tests/SwiftRTLayerTests/test_Recurrent.swift:97-167): hidden state after every step and the
    final cell state, to the reference's own accuracy of 1e-6.  This pins matmul(bias:)."""
    k = _lstm_kat()
    w = np.array(k["fused_weight"], np.float32)
    b = np.array(k["fused_bias"], np.float32)
    c = np.array([k["initial_cell"]], np.float32)
    h = np.array([k["initial_hidden"]], np.float32)
    for step, x in enumerate(k["inputs"]):
        c, h = oracle.lstm_cell(np.array([x], np.float32), h, c, w, b, 0)
        assert np.abs(h[0] - np.array(k["expected_hidden_per_step"][step], np.float32)).max() <= k["accuracy"]
    assert np.abs(c[0] - np.array(k["expected_final_cell"], np.float32)).max() <= k["accuracy"]
    # Float32: rounding every intermediate changes nothing
    c2, h2 = oracle.lstm_cell(np.array([k["inputs"][0]], np.float32), np.array([k["initial_hidden"]], np.float32),
                              np.array([k["initial_cell"]], np.float32), w, b, 0, stepwise=True)
    c1, h1 = oracle.lstm_cell(np.array([k["inputs"][0]], np.float32), np.array([k["initial_hidden"]], np.float32),
                              np.array([k["initial_cell"]], np.float32), w, b, 0)
    assert np.array_equal(c1, c2) and np.array_equal(h1, h2)


def test_lstm_golden_gradients_pin_the_backward_restatements(oracle):
    """Back-propagation through the four steps, built from the oracle's own pieces -- the two
    transposed products of matmulGradients and the bias gradient as a column sum
    (oracle_bias_activation_backward) -- must reproduce the reference's golden gradients of
    sum(final cell) (test_Recurrent.swift:169-240)."""
    k = _lstm_kat()
    F32 = 0
    w = np.array(k["fused_weight"], np.float32)
    b = np.array(k["fused_bias"], np.float32)
    H, I = 4, 4
    c = np.array([k["initial_cell"]], np.float32)
    h = np.array([k["initial_hidden"]], np.float32)
    sig = lambda v: (1 / (1 + np.exp(-v.astype(np.float64)))).astype(np.float32)
    saved = []
    for x in k["inputs"]:
        gate_in = np.concatenate([np.array([x], np.float32), h], axis=1)
        fused = oracle.matmul(np.ascontiguousarray(gate_in), w, F32, bias=b)
        gi, gu, gf, go = sig(fused[:, :H]), np.tanh(fused[:, H:2 * H]), sig(fused[:, 2 * H:3 * H]), sig(fused[:, 3 * H:])
        c_new = c * gf + gi * gu
        saved.append((gate_in, gi, gu, gf, go, c, c_new))
        h = np.tanh(c_new) * go
        c = c_new
    dc = np.ones((1, H), np.float32)
    dh = np.zeros((1, H), np.float32)
    dw = np.zeros_like(w)
    db = np.zeros_like(b)
    dxs = []
    for gate_in, gi, gu, gf, go, c_prev, c_new in reversed(saved):
        t = np.tanh(c_new)
        dc = dc + dh * go * (1 - t * t)
        dfused = np.concatenate([dc * gu * gi * (1 - gi), dc * gi * (1 - gu * gu), dc * c_prev * gf * (1 - gf),
                                 dh * t * go * (1 - go)], axis=1).astype(np.float32)
        dw += oracle.matmul(np.ascontiguousarray(gate_in), dfused, F32, True, False)        # x^T . dz
        _, step_db = oracle.bias_activation_backward(dfused, dfused, F32, "identity")       # column sums
        db += step_db
        dgate = oracle.matmul(dfused, w, F32, False, True)                                  # dz . W^T
        dxs.append(dgate[0, :I])
        dh = dgate[:, I:]
        dc = dc * gf
    dxs.reverse()
    tol = 2e-6
    assert np.abs(dw - np.array(k["grad_fused_weight"], np.float32)).max() <= tol
    assert np.abs(db - np.array(k["grad_fused_bias"], np.float32)).max() <= tol
    assert np.abs(np.array(dxs) - np.array(k["grad_inputs"], np.float32)).max() <= tol
    assert np.abs(dc[0] - np.array(k["grad_initial_cell"], np.float32)).max() <= tol
    assert np.abs(dh[0] - np.array(k["grad_initial_hidden"], np.float32)).max() <= tol
