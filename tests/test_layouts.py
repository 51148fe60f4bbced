"""Storage orders of the reference (Order, Sources/SwiftRTCore/tensor/Tensor.swift:177-231): the oracle's
restatement against the figures the reference's documentation gives, and the C helpers and argument checks
of srtMatrixTransform (no compute: nothing here needs a GPU)."""
import ctypes

import numpy as np
import pytest

from oracle import layouts as L

ORDERS = [L.ROW, L.COL, L.COL_TILED32, L.COL_TILED_TC32X32]


def test_leading_dimensions_of_the_reference_documentation():
    # Tensor.swift:188-192: "if the matrix has 33 columns and 2 rows, then the leading dimension must be at least (32) * 2 = 64"
    assert L.leading_dimension(L.COL_TILED32, 2, 33) == 64
    # Tensor.swift:219-231: "if matrix has 33 columns and 1 row, ld must be at least (32*32)*1 = 1024"
    assert L.leading_dimension(L.COL_TILED_TC32X32, 1, 33) == 1024
    assert L.leading_dimension(L.ROW, 5, 7) == 7 and L.leading_dimension(L.COL, 5, 7) == 5


def test_tc32x32_row_permutation_of_the_reference_formula():
    # index = (((row%8) / 2 * 4 + row / 8) * 2 + row % 2) * 32 + col   (Tensor.swift:222)
    off = L.offsets(L.COL_TILED_TC32X32, 1024, 32, 32)
    for row in range(32):
        for col in (0, 5, 31):
            assert off[row, col] == (((row % 8) // 2 * 4 + row // 8) * 2 + row % 2) * 32 + col
    assert sorted(off.ravel().tolist()) == list(range(1024))            # a permutation of the tile
    assert off[1, 0] == 32 and off[2, 0] == 256 and off[8, 0] == 64     # rows 0,1 adjacent; rows 0,8 two slots apart


@pytest.mark.parametrize("order", ORDERS)
@pytest.mark.parametrize("rows,cols", [(1, 1), (2, 33), (33, 2), (40, 70), (64, 64), (65, 31)])
def test_offsets_are_distinct_and_inside_the_buffer(order, rows, cols):
    ld = L.leading_dimension(order, rows, cols) + (0 if order in (L.COL_TILED32, L.COL_TILED_TC32X32) else 3)
    off = L.offsets(order, ld, rows, cols).ravel()
    assert len(set(off.tolist())) == rows * cols
    assert off.min() >= 0 and off.max() < L.element_count(order, rows, cols, ld)


@pytest.mark.parametrize("order", ORDERS)
@pytest.mark.parametrize("dtype", [0, 2, 14, 3])
def test_storage_round_trip(order, dtype):
    rng = np.random.default_rng(order * 10 + dtype)
    lay = L.Layout(dtype, order, 37, 45, batch_count=2)
    vals = rng.integers(-100, 100, (2, 37, 45)).astype(np.float32)      # exact in every element type
    assert np.array_equal(L.from_storage(L.to_storage(vals, lay), lay), vals)


def test_oracle_transform_is_linear_and_transposes():
    rng = np.random.default_rng(1)
    a = rng.integers(-8, 8, (1, 6, 40)).astype(np.float32)
    b = rng.integers(-8, 8, (1, 40, 6)).astype(np.float32)
    la, lb = L.Layout(0, L.ROW, 6, 40), L.Layout(3, L.COL_TILED_TC32X32, 40, 6)
    lc = L.Layout(0, L.COL_TILED32, 6, 40)
    out = L.matrix_transform(2.0, L.to_storage(a, la), la, False, -3.0, L.to_storage(b, lb), lb, True, lc)
    assert np.array_equal(L.from_storage(out, lc), 2 * a - 3 * b.transpose(0, 2, 1))


# ---- the C side, without a device: helpers and argument checks run before anything touches CUDA
@pytest.fixture(scope="module")
def lib():
    from swiftrt_b200 import _lib
    return _lib


@pytest.mark.parametrize("order", ORDERS)
def test_c_layout_helpers_agree_with_the_oracle(lib, order):
    for rows, cols in [(1, 1), (2, 33), (33, 2), (100, 100), (31, 65), (0, 5)]:
        ld = L.leading_dimension(order, rows, cols)
        assert lib.lib.srtMatrixLayoutLeadingDimension(order, rows, cols) == ld
        assert lib.lib.srtMatrixLayoutElementCount(order, rows, cols, ld + 32) == L.element_count(order, rows, cols, ld + 32)
    assert lib.lib.srtMatrixLayoutLeadingDimension(L.COL_TILED_TC32X8, 8, 32) == 0      # not computed


def _layout(lib, dtype, order, rows, cols, ld=None, batch=1):
    ld = L.leading_dimension(order, rows, cols) if ld is None else ld
    stride = L.element_count(order, rows, cols, ld) if rows and cols and order != L.COL_TILED_TC32X8 else 0
    return lib.MatrixLayoutStruct(dtype, order, rows, cols, ld, batch, stride)


def test_argument_checks_need_no_device(lib):
    one, zero = ctypes.c_float(1.0), ctypes.c_float(0.0)
    buf = (ctypes.c_float * 4096)()
    p = ctypes.addressof(buf)
    call = lambda la, lc, ta=False, a=p, beta=zero, b=None, lb=None: lib.lib.srtMatrixTransform(
        ctypes.byref(one), a, ctypes.byref(la), ta, ctypes.byref(beta), b, ctypes.byref(lb) if lb is not None else None, False,
        p, ctypes.byref(lc), None)
    row = _layout(lib, 0, L.ROW, 8, 8)
    assert call(row, row, a=None) == lib.cudaErrorInvalidValue
    assert call(_layout(lib, 0, L.COL_TILED_TC32X8, 8, 8, ld=256), row) == lib.cudaErrorNotSupported
    assert "colTiledTC32x8" in lib.last_error()
    assert call(_layout(lib, 1, L.ROW, 8, 8), row) == lib.cudaErrorNotSupported              # Float64
    assert call(_layout(lib, 0, L.COL_TILED32, 8, 8, ld=8), row) == lib.cudaErrorInvalidValue     # ld below 32 rows
    assert "leading dimension" in lib.last_error()
    assert call(_layout(lib, 0, L.ROW, 8, 4), row) == lib.cudaErrorInvalidValue              # shape mismatch
    assert call(_layout(lib, 0, L.ROW, 4, 8), _layout(lib, 0, L.ROW, 8, 4)) == lib.cudaErrorInvalidValue
    assert call(_layout(lib, 0, L.ROW, 8, 8, batch=2), row) == lib.cudaErrorInvalidValue     # batch mismatch
    assert call(row, row, beta=one) == lib.cudaErrorInvalidValue                             # beta != 0 without B
    empty = _layout(lib, 0, L.ROW, 0, 8, ld=8)
    assert call(empty, empty) == lib.cudaSuccess                                             # nothing to do, no launch


def test_host_mirror_layouts_without_a_device():
    import torch
    import swiftrt_b200 as srt
    x = torch.empty((3, 5), dtype=torch.int8)
    lx = srt.MatrixLayout.of(x)
    assert (lx.order, lx.rows, lx.cols, lx.leading_dimension, lx.type) == (srt.Order.row, 3, 5, 5, srt.DataType.real8I)
    lt = srt.MatrixLayout.of(x.t())                       # a transposed view is the col order (strides (1, rows))
    assert (lt.order, lt.rows, lt.cols, lt.leading_dimension) == (srt.Order.col, 5, 3, 5)
    lb = srt.MatrixLayout.of(torch.empty((4, 6, 8), dtype=torch.bfloat16))
    assert (lb.batch_count, lb.batch_stride, lb.elements) == (4, 48, 4 * 48)
    tiled = srt.MatrixLayout(srt.DataType.real8I, srt.Order.colTiledTC32x32, 33, 70)
    assert tiled.leading_dimension == 32 * 64 and tiled.elements == 2 * 2048 + 2048
    with pytest.raises(srt.MatmulError):
        srt.MatrixLayout(srt.DataType.real8I, srt.Order.colTiledTC32x8, 8, 32)
    with pytest.raises(ValueError):
        srt.matrix_transform(x.view(-1), lx, lx)          # host tensors are refused: there is no CPU path
