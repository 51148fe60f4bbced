"""TEST INFRASTRUCTURE ONLY: numpy restatement of the reference's storage orders and of the
matrix re-layout  C = alpha . op(A) + beta . op(B)  (cublasLtMatrixTransform, whose descriptors
Sources/SwiftRTCore/platform/cuda/cublaslt/MatrixTransform.swift:21-129 and MatrixLayout.swift:21-204
wrap; the reference never runs it, so this checker is pinned by the order definitions only:
parity unpinned beyond them).

Order values are cublasLtOrder_t's (Order.cublas, MatrixLayout.swift:221-231).  Element offsets follow
Order's documentation, Sources/SwiftRTCore/tensor/Tensor.swift:177-231:
  col (:177-181), row (:183-186), colTiled32 (:188-192: tiles of 32 columns, ld >= 32 rows),
  colTiledTC32x32 (:219-231: 32 x 32 tiles, row q of a tile at ((q%8)/2*4 + q/8)*2 + q%2).
colTiledTC32x8 (:204-217) has no stated element formula and is not restated.

Only tests and bench_configs.py's checks import this module; the product package never does.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import oracle

COL, ROW, COL_TILED32, COL_TILED_TC32X8, COL_TILED_TC32X32 = 0, 1, 2, 3, 4
I8 = 3                                # srtDataType real8I (tensor_api.h:31-38)


@dataclass
class Layout:
    """The fields of MatrixLayout (MatrixLayout.swift:89-186)."""
    dtype: int
    order: int
    rows: int
    cols: int
    ld: int = 0
    batch_count: int = 1
    batch_stride: int = 0

    def __post_init__(self):
        if self.ld == 0:
            self.ld = leading_dimension(self.order, self.rows, self.cols)
        if self.batch_stride == 0:
            self.batch_stride = element_count(self.order, self.rows, self.cols, self.ld)

    @property
    def elements(self) -> int:
        return (self.batch_count - 1) * self.batch_stride + element_count(self.order, self.rows, self.cols, self.ld)


def leading_dimension(order: int, rows: int, cols: int) -> int:
    """Smallest valid ld.  Tensor.leadingDimension (cuda/device/CudaPlatform.swift:298-311) gives the
    same rule for the tiled orders: 32 x the tile-rounded extent of the dimension that runs down a tile."""
    if order == ROW:
        return cols
    if order == COL:
        return rows
    if order == COL_TILED32:
        return 32 * rows
    if order == COL_TILED_TC32X32:
        return 32 * ((rows + 31) // 32 * 32)
    raise ValueError(f"order {order} is not restated")


def element_count(order: int, rows: int, cols: int, ld: int) -> int:
    if rows == 0 or cols == 0:
        return 0
    if order == ROW:
        return (rows - 1) * ld + cols
    if order == COL:
        return (cols - 1) * ld + rows
    if order == COL_TILED32:
        return ((cols - 1) // 32) * ld + 32 * rows
    if order == COL_TILED_TC32X32:
        return ((cols - 1) // 32) * ld + 32 * ((rows + 31) // 32 * 32)
    raise ValueError(f"order {order} is not restated")


def offsets(order: int, ld: int, rows: int, cols: int) -> np.ndarray:
    """int64 [rows, cols]: where element (r, c) of a stored matrix lives."""
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(cols, dtype=np.int64)[None, :]
    if order == ROW:
        return r * ld + c
    if order == COL:
        return c * ld + r
    if order == COL_TILED32:
        return (c // 32) * ld + r * 32 + c % 32
    if order == COL_TILED_TC32X32:
        q = r % 32
        t = ((q % 8) // 2 * 4 + q // 8) * 2 + q % 2
        return (c // 32) * ld + (r // 32) * 1024 + t * 32 + c % 32
    raise ValueError(f"order {order} is not restated")


def _np_dtype(dtype: int):
    return np.int8 if dtype == I8 else oracle.np_dtype(dtype)


def _decode(bits: np.ndarray, dtype: int) -> np.ndarray:
    return bits.astype(np.float32) if dtype == I8 else oracle.decode(bits, dtype)


def _encode(values: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == I8:
        r = np.rint(values.astype(np.float32))              # to nearest even
        r = np.where(np.isnan(r), 0.0, r)
        return np.clip(r, -128, 127).astype(np.int8)
    return oracle.encode(values, dtype)


def to_storage(values: np.ndarray, layout: Layout, fill=0) -> np.ndarray:
    """[batch, rows, cols] float32 values -> the flat stored buffer (bits of layout.dtype)."""
    values = np.asarray(values, dtype=np.float32).reshape(layout.batch_count, layout.rows, layout.cols)
    buf = np.full(layout.elements, fill, dtype=_np_dtype(layout.dtype))
    off = offsets(layout.order, layout.ld, layout.rows, layout.cols)
    for b in range(layout.batch_count):
        buf[b * layout.batch_stride + off] = _encode(values[b], layout.dtype)
    return buf


def from_storage(buf: np.ndarray, layout: Layout) -> np.ndarray:
    """the flat stored buffer -> [batch, rows, cols] float32 values."""
    off = offsets(layout.order, layout.ld, layout.rows, layout.cols)
    out = np.empty((layout.batch_count, layout.rows, layout.cols), dtype=np.float32)
    for b in range(layout.batch_count):
        out[b] = _decode(np.asarray(buf)[b * layout.batch_stride + off], layout.dtype)
    return out


def matrix_transform(alpha: float, a: np.ndarray, a_layout: Layout, trans_a: bool,
                     beta: float, b, b_layout, trans_b: bool, c_layout: Layout, c_init=None) -> np.ndarray:
    """The stored buffer of C.  fp32 arithmetic: fl(alpha a), then one fused multiply-add with beta b
    (computed in float64 and rounded, which differs from a true fma only in double-rounding cases),
    then one rounding to C's element type.  Elements of the buffer that belong to no (r, c) keep c_init."""
    va = from_storage(a, a_layout)
    if trans_a:
        va = va.transpose(0, 2, 1)
    acc = (np.float32(alpha) * va).astype(np.float32)
    if beta != 0.0:
        vb = from_storage(b, b_layout)
        if trans_b:
            vb = vb.transpose(0, 2, 1)
        acc = (np.float64(np.float32(beta)) * vb.astype(np.float64) + acc.astype(np.float64)).astype(np.float32)
    if acc.shape != (c_layout.batch_count, c_layout.rows, c_layout.cols):
        raise ValueError("op(A), op(B) and C differ in shape")
    out = np.array(c_init, dtype=_np_dtype(c_layout.dtype)) if c_init is not None else np.zeros(c_layout.elements, _np_dtype(c_layout.dtype))
    off = offsets(c_layout.order, c_layout.ld, c_layout.rows, c_layout.cols)
    for bt in range(c_layout.batch_count):
        out[bt * c_layout.batch_stride + off] = _encode(acc[bt], c_layout.dtype)
    return out
