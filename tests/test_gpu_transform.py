"""srtMatrixTransform on a B200, through the C ABI, against the numpy restatement of the reference's storage
orders (oracle/layouts.py).  A pure re-layout (alpha = 1, beta = 0) and integer-valued sums must match bit for
bit, padding elements of the destination buffer must stay untouched; general alpha / beta sums are compared
to 1e-6 relative (the oracle's fused multiply-add is formed in float64)."""
import itertools

import numpy as np
import pytest
import torch

from oracle import layouts as L

pytestmark = pytest.mark.gpu

F32, F16, I8, BF16 = 0, 2, 3, 14
ORDERS = [L.ROW, L.COL, L.COL_TILED32, L.COL_TILED_TC32X32]
TORCH = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16, I8: torch.int8}


@pytest.fixture(scope="module")
def srt():
    import swiftrt_b200 as s
    assert torch.cuda.is_available()
    return s


def _dev(bits: np.ndarray, dtype: int) -> torch.Tensor:
    t = torch.from_numpy(bits)
    if dtype in (F16, BF16):
        t = t.view(TORCH[dtype])
    return t.cuda()


def _host(t: torch.Tensor, dtype: int) -> np.ndarray:
    t = t.cpu()
    return t.view(torch.uint16).numpy() if dtype in (F16, BF16) else t.numpy()


def _mirror(srt, lay: L.Layout):
    return srt.MatrixLayout(lay.dtype, lay.order, lay.rows, lay.cols, lay.ld, lay.batch_count, lay.batch_stride)


def _sentinel(lay: L.Layout) -> np.ndarray:
    return np.full(lay.elements, 0x7b if lay.dtype == I8 else (0x7b7b if lay.dtype != F32 else 123.0),
                   dtype=np.int8 if lay.dtype == I8 else (np.uint16 if lay.dtype != F32 else np.float32))


def _run(srt, alpha, a, la, ta, beta, b, lb, tb, lc):
    init = _sentinel(lc)
    out = _dev(init.copy(), lc.dtype)
    srt.matrix_transform(_dev(a, la.dtype), _mirror(srt, la), _mirror(srt, lc), alpha, ta, beta,
                         _dev(b, lb.dtype) if b is not None else None, _mirror(srt, lb) if lb is not None else None, tb, out=out)
    torch.cuda.synchronize()
    assert srt.check_status() == 0
    return _host(out, lc.dtype), L.matrix_transform(alpha, a, la, ta, beta, b, lb, tb, lc, c_init=init)


def _padded(dtype, order, rows, cols, batch, vector_friendly):
    """A layout whose leading dimension and batch stride are multiples of 16 elements (so that the kernels take
    their 16-byte accesses, with ragged run ends), or the smallest ones (element-wise accesses)."""
    if not vector_friendly:
        return L.Layout(dtype, order, rows, cols, batch_count=batch)
    ld = (L.leading_dimension(order, rows, cols) + 15) // 16 * 16
    stride = (L.element_count(order, rows, cols, ld) + 15) // 16 * 16
    return L.Layout(dtype, order, rows, cols, ld=ld, batch_count=batch, batch_stride=stride)


@pytest.mark.parametrize("src,dst", list(itertools.product(ORDERS, ORDERS)))
@pytest.mark.parametrize("trans", [False, True])
@pytest.mark.parametrize("dtype,vector_friendly", [(F32, False), (F32, True), (BF16, True), (I8, True)])
def test_relayout_every_order_pair_is_bit_exact(srt, src, dst, trans, dtype, vector_friendly):
    rng = np.random.default_rng(src * 16 + dst * 2 + trans)
    rows, cols, batch = 75, 133, 2                       # ragged against the 64-element tiles and the 32-wide groups
    la = _padded(dtype, src, cols if trans else rows, rows if trans else cols, batch, vector_friendly)
    lc = _padded(dtype, dst, rows, cols, batch, vector_friendly)
    a = L.to_storage(rng.integers(-100, 100, (batch, la.rows, la.cols)), la, fill=7)
    got, ref = _run(srt, 1.0, a, la, trans, 0.0, None, None, False, lc)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("src,dst", list(itertools.product(ORDERS, ORDERS)))
@pytest.mark.parametrize("trans", [False, True])
@pytest.mark.parametrize("dtype", [I8, BF16, F16])
def test_whole_tile_relayouts_of_small_elements_are_bit_exact(srt, src, dst, trans, dtype):
    """Extents that are multiples of 128: transpositions of 1- and 2-byte elements take the packed-word kernel."""
    rng = np.random.default_rng(src * 16 + dst * 2 + trans + 1000)
    rows, cols, batch = 256, 384, 2
    la = _padded(dtype, src, cols if trans else rows, rows if trans else cols, batch, True)
    lc = _padded(dtype, dst, rows, cols, batch, True)
    a = L.to_storage(rng.integers(-100, 100, (batch, la.rows, la.cols)), la, fill=7)
    got, ref = _run(srt, 1.0, a, la, trans, 0.0, None, None, False, lc)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("ta,tc", [(F32, I8), (I8, F32), (I8, I8), (BF16, F16), (F16, BF16), (F32, BF16), (I8, BF16)])
@pytest.mark.parametrize("src,dst", [(L.ROW, L.COL_TILED_TC32X32), (L.COL_TILED_TC32X32, L.COL), (L.COL, L.COL_TILED32), (L.COL_TILED32, L.ROW)])
def test_element_types_convert_with_one_rounding(srt, ta, tc, src, dst):
    rng = np.random.default_rng(ta * 100 + tc)
    rows, cols = 96, 160
    la, lc = L.Layout(ta, src, rows, cols), L.Layout(tc, dst, rows, cols)
    vals = rng.uniform(-200, 200, (1, rows, cols)) if tc == I8 and ta != I8 else rng.uniform(-100, 100, (1, rows, cols))
    a = L.to_storage(vals, la)                            # Int8 sources round here; Int8 destinations saturate in the transform
    got, ref = _run(srt, 1.0, a, la, False, 0.0, None, None, False, lc)
    assert np.array_equal(got, ref)


def test_int8_sum_saturates_and_rounds_to_even(srt):
    la = L.Layout(I8, L.ROW, 4, 32)
    lc = L.Layout(I8, L.COL_TILED32, 4, 32)
    a = np.arange(-64, 64, dtype=np.int8)
    b = np.full(128, 3, dtype=np.int8)
    got, ref = _run(srt, 2.5, a, la, False, 0.5, b, la, False, lc)      # 2.5 a + 1.5: halves round to even, |a| > 51 saturates
    assert np.array_equal(got, ref)
    vals = L.from_storage(got, lc)[0]
    assert vals.max() == 127 and vals.min() == -128


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_alpha_beta_sum_with_transposes_and_batches(srt, dtype, ta, tb):
    rng = np.random.default_rng(5 + ta * 2 + tb)
    rows, cols, batch = 130, 70, 3
    la = L.Layout(dtype, L.COL_TILED_TC32X32, cols if ta else rows, rows if ta else cols, batch_count=batch)
    lb = L.Layout(dtype, L.COL, cols if tb else rows, rows if tb else cols, ld=(cols if tb else rows) + 5, batch_count=batch)
    lc = L.Layout(dtype, L.ROW, rows, cols, ld=cols + 3, batch_count=batch, batch_stride=rows * (cols + 3) + 11)
    a = L.to_storage(rng.standard_normal((batch, la.rows, la.cols)), la)
    b = L.to_storage(rng.standard_normal((batch, lb.rows, lb.cols)), lb)
    got, ref = _run(srt, 0.75, a, la, ta, -1.25, b, lb, tb, lc)
    g, r = L.from_storage(got, lc), L.from_storage(ref, lc)
    if dtype == F32:
        assert np.allclose(g, r, rtol=1e-6, atol=1e-7)
    else:
        assert np.mean(g != r) < 1e-3 and np.allclose(g, r, rtol=8e-3)   # a double-rounding tie may differ by one bf16 ulp
    # padding (between rows, between matrices) keeps the sentinel
    mask = np.ones(lc.elements, dtype=bool)
    off = L.offsets(lc.order, lc.ld, rows, cols).ravel()
    for bt in range(batch):
        mask[bt * lc.batch_stride + off] = False
    assert np.array_equal(got[mask], _sentinel(lc)[mask])


def test_large_relayout_round_trip_and_one_launch(srt):
    rows, cols = 4096, 8192
    x = torch.randint(-128, 128, (rows, cols), dtype=torch.int8, device="cuda")
    lx = srt.MatrixLayout.of(x)
    lt = srt.MatrixLayout(srt.DataType.real8I, srt.Order.colTiledTC32x32, rows, cols)
    before = srt.launch_count()
    tiled = srt.matrix_transform(x.view(-1), lx, lt)
    back = srt.matrix_transform(tiled, lt, lx)
    torch.cuda.synchronize()
    assert srt.launch_count() - before == 2
    assert torch.equal(back.view(rows, cols), x)
    # a few elements against the order's formula
    q = 37
    t = ((q % 8) // 2 * 4 + q // 8 % 4) * 2 + q % 2
    r, c = 32 * 5 + q, 32 * 9 + 3
    q = r % 32
    t = ((q % 8) // 2 * 4 + q // 8) * 2 + q % 2
    assert tiled[(c // 32) * lt.leading_dimension + (r // 32) * 1024 + t * 32 + c % 32].item() == x[r, c].item()
    # transposed view of a torch tensor is the col order
    lt2 = srt.MatrixLayout.of(x.t())
    assert lt2.order == srt.Order.col and lt2.rows == cols and lt2.leading_dimension == cols
    y = srt.matrix_transform(x.view(-1), lt2, srt.MatrixLayout(srt.DataType.real8I, srt.Order.row, cols, rows))
    assert torch.equal(y.view(cols, rows), x.t())
