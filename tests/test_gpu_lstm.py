"""The LSTM cell step on a B200 (srtLstmCell: concatenation, fused product with bias, gate pass)
against the reference's golden data and against the CPU oracle."""
import json
import os

import numpy as np
import pytest
import torch

from _gpu_util import BF16, F16, F32, TOL, from_dev, random_bits, to_dev

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def srt():
    import swiftrt_b200 as s
    assert torch.cuda.is_available()
    return s


@pytest.fixture(scope="module")
def kat():
    with open(os.path.join(HERE, "golden", "lstm_kat.json")) as f:
        return json.load(f)


def _t(x):
    return torch.tensor(x, dtype=torch.float32, device="cuda:0")


def test_reference_golden_sequence(srt, kat):
    """Tests/SwiftRTLayerTests/test_Recurrent.swift:47-66 with its data (:97-167): the hidden state
    after each of the four steps and the final cell state, to the reference's accuracy of 1e-6."""
    cell = srt.LSTMCell(_t(kat["fused_weight"]), _t(kat["fused_bias"]))
    assert cell.hidden_size == 4
    state = srt.LSTMState(_t([kat["initial_cell"]]), _t([kat["initial_hidden"]]))
    before = srt.launch_count()
    outputs = srt.run_sequence(cell, [_t([x]) for x in kat["inputs"]], state)
    torch.cuda.synchronize()
    assert srt.launch_count() - before == 4 * 3          # concatenation, product, gates per step
    assert len(outputs) == 4
    hidden = torch.cat([s.hidden for s in outputs]).cpu().numpy()
    assert np.abs(hidden - np.array(kat["expected_hidden_per_step"], np.float32)).max() <= kat["accuracy"]
    assert np.abs(outputs[-1].cell.cpu().numpy()[0] - np.array(kat["expected_final_cell"], np.float32)).max() <= kat["accuracy"]


def test_reference_golden_gradients_through_the_gpu_operators(srt, kat):
    """Back-propagation through the four steps with the library's own pieces -- srtMatmul with
    transpose flags for x^T.dz and dz.W^T, srtBiasActivationBackward for the bias gradient -- must give
    the reference's golden gradients of sum(final cell) (test_Recurrent.swift:169-240)."""
    w, b = _t(kat["fused_weight"]), _t(kat["fused_bias"])
    H, I = 4, 4
    c, h = _t([kat["initial_cell"]]), _t([kat["initial_hidden"]])
    saved = []
    for x in kat["inputs"]:
        gate_in = torch.cat([_t([x]), h], dim=1)
        fused = srt.matmul(gate_in, w, bias=b)
        gi, gu = torch.sigmoid(fused[:, :H]), torch.tanh(fused[:, H:2 * H])
        gf, go = torch.sigmoid(fused[:, 2 * H:3 * H]), torch.sigmoid(fused[:, 3 * H:])
        c_new = c * gf + gi * gu
        saved.append((gate_in, gi, gu, gf, go, c, c_new))
        h, c = torch.tanh(c_new) * go, c_new
    dc, dh = torch.ones_like(c), torch.zeros_like(c)
    dw, db, dxs = torch.zeros_like(w), torch.zeros_like(b), []
    for gate_in, gi, gu, gf, go, c_prev, c_new in reversed(saved):
        t = torch.tanh(c_new)
        dc = dc + dh * go * (1 - t * t)
        dfused = torch.cat([dc * gu * gi * (1 - gi), dc * gi * (1 - gu * gu), dc * c_prev * gf * (1 - gf),
                            dh * t * go * (1 - go)], dim=1).contiguous()
        dgate, step_dw = srt.matmul_gradients(dfused, gate_in, False, w, False)
        _, step_db = srt.bias_activation_backward(dfused, None, srt.ActivationType.identity, want_dz=False)
        dw += step_dw
        db += step_db
        dxs.append(dgate[0, :I].clone())
        dh = dgate[:, I:]
        dc = dc * gf
    dxs.reverse()
    tol = 2e-6
    assert (dw.cpu().numpy() - np.array(kat["grad_fused_weight"], np.float32)).__abs__().max() <= tol
    assert (db.cpu().numpy() - np.array(kat["grad_fused_bias"], np.float32)).__abs__().max() <= tol
    assert (torch.stack(dxs).cpu().numpy() - np.array(kat["grad_inputs"], np.float32)).__abs__().max() <= tol
    assert (dc.cpu().numpy()[0] - np.array(kat["grad_initial_cell"], np.float32)).__abs__().max() <= tol
    assert (dh.cpu().numpy()[0] - np.array(kat["grad_initial_hidden"], np.float32)).__abs__().max() <= tol


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
@pytest.mark.parametrize("batch,nx,nh", [(3, 5, 7), (64, 96, 128), (256, 512, 512), (1, 1024, 256)])
def test_cell_step_matches_oracle(srt, oracle, dtype, batch, nx, nh):
    rng = np.random.default_rng(batch + 3 * nx + 7 * nh + dtype)
    x = random_bits(oracle, rng, (batch, nx), dtype)
    h = random_bits(oracle, rng, (batch, nh), dtype)
    c = random_bits(oracle, rng, (batch, nh), dtype, dist="normal")
    w = random_bits(oracle, rng, (nx + nh, 4 * nh), dtype, scale=1.0 / np.sqrt(nx + nh))
    b = random_bits(oracle, rng, (4 * nh,), dtype, scale=0.5)
    ref_c, ref_h = oracle.lstm_cell(x, h, c, w, b, dtype)
    cell = srt.LSTMCell(to_dev(w, dtype), to_dev(b, dtype))
    out = cell(to_dev(x, dtype), srt.LSTMState(to_dev(c, dtype), to_dev(h, dtype)))
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    for got, ref in ((out.cell, ref_c), (out.hidden, ref_h)):
        err = oracle.rel_frobenius(oracle.decode(from_dev(got, dtype), dtype), oracle.decode(ref, dtype))
        assert err <= TOL[dtype], err
    if dtype != F32:
        # rounding every intermediate, as the composed reference operators would, stays inside the tolerance too
        step_c, step_h = oracle.lstm_cell(x, h, c, w, b, dtype, stepwise=True)
        assert oracle.rel_frobenius(oracle.decode(from_dev(out.hidden, dtype), dtype), oracle.decode(step_h, dtype)) <= TOL[dtype]


def test_strided_state_views_no_bias_and_argument_errors(srt, oracle):
    rng = np.random.default_rng(9)
    batch, nx, nh = 10, 12, 16
    x = random_bits(oracle, rng, (batch, nx), F32)
    big_h = random_bits(oracle, rng, (batch, 2 * nh), F32)
    big_c = random_bits(oracle, rng, (2 * batch, nh), F32)
    h, c = big_h[:, ::2], big_c[::2]                                   # column stride 2, row stride 2
    w = random_bits(oracle, rng, (nx + nh, 4 * nh), F32, scale=0.2)
    ref_c, ref_h = oracle.lstm_cell(x, np.ascontiguousarray(h), np.ascontiguousarray(c), w, None, F32)
    cell = srt.LSTMCell(to_dev(w, F32), None)
    out = cell(to_dev(x, F32), srt.LSTMState(to_dev(c, F32), to_dev(h, F32)))
    assert oracle.rel_frobenius(from_dev(out.cell, F32), ref_c) <= TOL[F32]
    assert oracle.rel_frobenius(from_dev(out.hidden, F32), ref_h) <= TOL[F32]
    zero = cell.zero_state(to_dev(x, F32))
    assert zero.cell.shape == (batch, nh) and float(zero.hidden.abs().sum()) == 0.0
    with pytest.raises(srt.MatmulError) as e:
        cell(to_dev(x[:, :5].copy(), F32), srt.LSTMState(to_dev(c, F32), to_dev(h, F32)))      # inputSize mismatch
    assert e.value.code == 1 and "fusedWeight" in str(e.value)
    with pytest.raises(ValueError):
        srt.LSTMCell(to_dev(w[:, :30].copy(), F32), None)


def test_sequence_captured_in_a_cuda_graph(srt, kat):
    """The golden four-step sequence replayed from a CUDA graph gives the same bits as the eager
    launches, follows new inputs, and enqueues faster than 12 separate launches."""
    cell = srt.LSTMCell(_t(kat["fused_weight"]), _t(kat["fused_bias"]))
    state = srt.LSTMState(_t([kat["initial_cell"]]), _t([kat["initial_hidden"]]))
    inputs = [_t([x]) for x in kat["inputs"]]
    eager = srt.run_sequence(cell, inputs, state)
    graphed = srt.GraphedSequence(cell, steps=4, batch=1, input_size=4, dtype=torch.float32)
    before = srt.launch_count()
    out = graphed(inputs, state)
    torch.cuda.synchronize()
    assert srt.launch_count() == before                      # a replay makes no library call
    for a, b in zip(eager, out):
        assert torch.equal(a.cell, b.cell) and torch.equal(a.hidden, b.hidden)
    hidden = torch.cat([s.hidden for s in out]).cpu().numpy()
    assert np.abs(hidden - np.array(kat["expected_hidden_per_step"], np.float32)).max() <= kat["accuracy"]
    # other inputs through the same graph
    shifted = [x + 0.25 for x in inputs]
    want = srt.run_sequence(cell, shifted, state)
    got = graphed(shifted, state)
    torch.cuda.synchronize()
    assert torch.equal(want[-1].hidden, got[-1].hidden) and srt.check_status() == 0
    with pytest.raises(ValueError):
        graphed(inputs[:2], state)

    def wall(fn, reps=50):
        import time
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps * 1e6

    t_eager = wall(lambda: srt.run_sequence(cell, inputs, state))
    t_graph = wall(lambda: graphed.graph.replay())
    print(f"4-step LSTM sequence: eager {t_eager:.1f} us, graph replay {t_graph:.1f} us")
    assert t_graph < t_eager


@pytest.mark.parametrize("dtype", [F32, BF16, F16])
@pytest.mark.parametrize("batch,nx,nh,bias_rank", [(3, 5, 7, 2), (64, 96, 128, 1), (32, 1024, 1024, 2)])
def test_basic_rnn_cell_matches_oracle(srt, oracle, dtype, batch, nx, nh, bias_rank):
    """BasicRNNCell (Recurrent.swift:110-161): tanh(matmul(concatenate(input, state), weight) + bias) with the
    bias as the reference keeps it ([1 x hiddenSize]) or as a vector."""
    rng = np.random.default_rng(batch + nx + nh + dtype)
    x = random_bits(oracle, rng, (batch, nx), dtype)
    h = random_bits(oracle, rng, (batch, nh), dtype)
    w = random_bits(oracle, rng, (nx + nh, nh), dtype, scale=1.0 / np.sqrt(nx + nh))
    b = random_bits(oracle, rng, (nh,), dtype, scale=0.5)
    ref = oracle.matmul(np.ascontiguousarray(np.concatenate([x, h], axis=1)), w, dtype, bias=b, activation="tanh")
    dbias = to_dev(b, dtype)
    cell = srt.BasicRNNCell(to_dev(w, dtype), dbias.reshape(1, nh) if bias_rank == 2 else dbias)
    before = srt.launch_count()
    out = cell(to_dev(x, dtype), to_dev(h, dtype))
    torch.cuda.synchronize()
    assert srt.check_status() == 0 and 2 <= srt.launch_count() - before <= 3
    err = oracle.rel_frobenius(oracle.decode(from_dev(out, dtype), dtype), oracle.decode(ref, dtype))
    assert err <= TOL[dtype], err
    assert cell.zero_state(to_dev(x, dtype)).shape == (batch, nh)
    with pytest.raises(srt.MatmulError):
        srt.BasicRNNCell(to_dev(w, dtype), to_dev(b[:-1].copy(), dtype))(to_dev(x, dtype), to_dev(h, dtype))


def test_sequence_without_per_step_concatenation(srt, kat, oracle):
    """The hidden state lives inside the next step's gate input: same results, two launches per step."""
    cell = srt.LSTMCell(_t(kat["fused_weight"]), _t(kat["fused_bias"]))
    state = srt.LSTMState(_t([kat["initial_cell"]]), _t([kat["initial_hidden"]]))
    inputs = [_t([x]) for x in kat["inputs"]]
    eager = srt.run_sequence(cell, inputs, state)
    before = srt.launch_count()
    fused = srt.run_sequence_preconcatenated(cell, inputs, state)
    torch.cuda.synchronize()
    assert srt.launch_count() - before == 4 * 2
    for a, b in zip(eager, fused):
        assert torch.equal(a.cell, b.cell) and torch.equal(a.hidden, b.hidden)
    # a larger bf16 case through the tensor-core kernels, strided gate input and hidden views included
    rng = np.random.default_rng(3)
    batch, nx, nh, steps = 128, 256, 512, 3
    w = to_dev(random_bits(oracle, rng, (nx + nh, 4 * nh), BF16, scale=0.04), BF16)
    b = to_dev(random_bits(oracle, rng, (4 * nh,), BF16, scale=0.5), BF16)
    cell2 = srt.LSTMCell(w, b)
    xs = [to_dev(random_bits(oracle, rng, (batch, nx), BF16), BF16) for _ in range(steps)]
    ref = srt.run_sequence(cell2, xs)
    got = srt.run_sequence_preconcatenated(cell2, xs)
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    for a, c in zip(ref, got):
        assert torch.equal(a.cell, c.cell) and torch.equal(a.hidden, c.hidden)


@pytest.mark.parametrize("dtype,batch,nx,nh", [(F32, 5, 7, 6), (F32, 64, 96, 128), (BF16, 256, 256, 256), (F16, 33, 40, 24)])
def test_gru_cell_matches_operator_by_operator_composition(srt, oracle, dtype, batch, nx, nh):
    """srtGruCell (two fused products) against GRUCell.callAsFunction composed operator by operator on
    the CPU (Sources/SwiftRTLayers/Recurrent.swift:328-337).  The reference holds no GRU test data, so
    the oracle composition is the pin; the fused products round once where the composition rounds per
    operator, hence the path's tolerances rather than bit equality."""
    rng = np.random.default_rng(batch + nx + nh)
    sc = 1.0 / np.sqrt(nx + nh)
    w = {name: random_bits(oracle, rng, shape, dtype, scale=sc) for name, shape in (
        ("resetW1", (nx, nh)), ("resetW2", (nh, nh)), ("updateW1", (nx, nh)), ("updateW2", (nh, nh)),
        ("outputW1", (nx, nh)), ("outputW2", (nh, nh)))}
    for name in ("resetB", "updateB", "outputB"):
        w[name] = random_bits(oracle, rng, (nh,), dtype, scale=0.5)
    x = random_bits(oracle, rng, (batch, nx), dtype)
    h = random_bits(oracle, rng, (batch, nh), dtype)
    want = oracle.gru_cell(x, h, w, dtype)
    d = {k: to_dev(v, dtype) for k, v in w.items()}
    cell = srt.GRUCell(d["resetW1"], d["resetW2"], d["resetB"], d["updateW1"], d["updateW2"], d["updateB"],
                       d["outputW1"], d["outputW2"], d["outputB"])
    before = srt.launch_count()
    got = cell(to_dev(x, dtype), to_dev(h, dtype))
    torch.cuda.synchronize()
    assert srt.launch_count() - before == 5
    assert srt.check_status() == 0
    tol = 1e-5 if dtype == F32 else TOL[dtype]
    assert oracle.rel_frobenius(oracle.decode(from_dev(got, dtype), dtype), oracle.decode(want, dtype)) <= tol
    # a second step from the new state, in place (newHidden aliases hidden)
    want2 = oracle.gru_cell(x, want, w, dtype)
    got2 = cell(to_dev(x, dtype), got)
    assert oracle.rel_frobenius(oracle.decode(from_dev(got2, dtype), dtype), oracle.decode(want2, dtype)) <= 2 * tol


@pytest.mark.parametrize("dtype,batch,nx,nh", [(BF16, 512, 256, 256), (F16, 300, 136, 72), (BF16, 4096, 1024, 1024)])
def test_lstm_step_with_gates_in_the_product_epilogue(srt, oracle, dtype, batch, nx, nh):
    """srtLstmCellFused: the gate pass runs on the accumulators of the product over an interleaved
    weight; new cell and hidden states against the oracle (which rounds the fused product to the element
    type first, as the reference's matmul(bias:) does: tolerance, not bit equality) and against the
    three-launch step."""
    rng = np.random.default_rng(batch + nx + nh)
    w = to_dev(random_bits(oracle, rng, (nx + nh, 4 * nh), dtype, scale=1.0 / np.sqrt(nx + nh)), dtype)
    b = to_dev(random_bits(oracle, rng, (4 * nh,), dtype, scale=0.5), dtype)
    x_bits, h_bits, c_bits = (random_bits(oracle, rng, (batch, n), dtype) for n in (nx, nh, nh))
    plain = srt.LSTMCell(w, b)
    fused = srt.LSTMCell(w, b, fuse_gates=True)
    wi, bi = fused.interleaved()
    torch.cuda.synchronize()
    assert torch.equal(wi, w.reshape(nx + nh, 4, nh).transpose(1, 2).reshape(nx + nh, 4 * nh))
    assert torch.equal(bi, b.reshape(4, nh).t().reshape(4 * nh))
    x, state = to_dev(x_bits, dtype), srt.LSTMState(to_dev(c_bits, dtype), to_dev(h_bits, dtype))
    ref = plain(x, state)
    before = srt.launch_count()
    got = fused(x, state)
    torch.cuda.synchronize()
    assert srt.launch_count() - before == 2              # concatenation + the product with its gate epilogue
    assert srt.check_status() == 0
    if batch <= 512:
        want_c, want_h = oracle.lstm_cell(x_bits, h_bits, c_bits, from_dev(w, dtype), from_dev(b, dtype), dtype)
        for g, wnt in ((got.cell, want_c), (got.hidden, want_h)):
            assert oracle.rel_frobenius(oracle.decode(from_dev(g, dtype), dtype), oracle.decode(wnt, dtype)) <= TOL[dtype]
    for g, r in ((got.cell, ref.cell), (got.hidden, ref.hidden)):
        assert oracle.rel_frobenius(oracle.decode(from_dev(g, dtype), dtype), oracle.decode(from_dev(r, dtype), dtype)) <= TOL[dtype]
    # a sequence with the hidden state kept inside the next step's gate input: one launch per step
    xs = [to_dev(random_bits(oracle, rng, (batch, nx), dtype), dtype) for _ in range(3)]
    before = srt.launch_count()
    seq = srt.run_sequence_preconcatenated(fused, xs)
    torch.cuda.synchronize()
    assert srt.launch_count() - before == 3
    seq_ref = srt.run_sequence(plain, xs)
    for a, r in zip(seq, seq_ref):
        assert oracle.rel_frobenius(oracle.decode(from_dev(a.hidden, dtype), dtype), oracle.decode(from_dev(r.hidden, dtype), dtype)) <= 2 * TOL[dtype]
    assert srt.check_status() == 0


def test_fused_lstm_step_falls_back_when_not_eligible(srt, oracle):
    rng = np.random.default_rng(9)
    batch, nx, nh = 64, 40, 12                       # hiddenSize not a multiple of 8
    w = to_dev(random_bits(oracle, rng, (nx + nh, 4 * nh), BF16, scale=0.1), BF16)
    b = to_dev(random_bits(oracle, rng, (4 * nh,), BF16, scale=0.5), BF16)
    x = to_dev(random_bits(oracle, rng, (batch, nx), BF16), BF16)
    state = srt.LSTMState(to_dev(random_bits(oracle, rng, (batch, nh), BF16), BF16), to_dev(random_bits(oracle, rng, (batch, nh), BF16), BF16))
    ref = srt.LSTMCell(w, b)(x, state)
    before = srt.launch_count()
    got = srt.LSTMCell(w, b, fuse_gates=True)(x, state)
    torch.cuda.synchronize()
    assert srt.launch_count() - before >= 3 + 2      # the two interleave passes, then the ordinary three-launch step
    assert torch.equal(got.cell, ref.cell) and torch.equal(got.hidden, ref.hidden)
