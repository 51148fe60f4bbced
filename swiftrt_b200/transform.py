"""Matrix re-layout between the reference's storage orders: C = alpha . op(A) + beta . op(B).

Host mirror of the reference's cublasLt wrappers for this operation -- `MatrixLayout`
(Sources/SwiftRTCore/platform/cuda/cublaslt/MatrixLayout.swift:21-204: type, order, rows, cols,
leadingDimension, batchCount, batchStride) and `MatrixTransform` (cublaslt/MatrixTransform.swift:21-129:
transA, transB, host scalars) -- over srtMatrixTransform.  Buffers are flat device tensors holding the
stored elements; a layout says where element (r, c) lives in them (Order, tensor/Tensor.swift:177-231).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import lib
from .matmul import MatmulError
from .tensor import DataType, Order

_TORCH2SRT = {torch.float32: DataType.real32F, torch.float16: DataType.real16F,
              torch.bfloat16: DataType.real16BF, torch.int8: DataType.real8I}
_SRT2TORCH = {v: k for k, v in _TORCH2SRT.items()}


def leading_dimension(order: Order, rows: int, cols: int) -> int:
    """Smallest valid leading dimension (srtMatrixLayoutLeadingDimension; the rule of
    Tensor.leadingDimension, cuda/device/CudaPlatform.swift:298-311)."""
    ld = int(lib.srtMatrixLayoutLeadingDimension(int(order), rows, cols))
    if ld == 0 and rows and cols:
        raise MatmulError(_lib.cudaErrorNotSupported, f"order {Order(order).name} is not computed")
    return ld


@dataclass
class MatrixLayout:
    """Same properties as the reference's MatrixLayout (MatrixLayout.swift:89-186)."""
    type: DataType
    order: Order
    rows: int
    cols: int
    leading_dimension: int = 0          # 0: the smallest valid one
    batch_count: int = 1
    batch_stride: int = 0               # 0: matrices back to back

    def __post_init__(self):
        self.type, self.order = DataType(self.type), Order(self.order)
        if self.leading_dimension == 0:
            self.leading_dimension = leading_dimension(self.order, self.rows, self.cols)
        if self.batch_stride == 0:
            self.batch_stride = self.matrix_elements

    @property
    def matrix_elements(self) -> int:
        return int(lib.srtMatrixLayoutElementCount(int(self.order), self.rows, self.cols, self.leading_dimension))

    @property
    def elements(self) -> int:
        """Elements a buffer for this layout must hold."""
        return (self.batch_count - 1) * self.batch_stride + self.matrix_elements

    def empty(self, device) -> torch.Tensor:
        return torch.empty(self.elements, dtype=_SRT2TORCH[self.type], device=device)

    def struct(self) -> _lib.MatrixLayoutStruct:
        return _lib.MatrixLayoutStruct(int(self.type), int(self.order), self.rows, self.cols, self.leading_dimension,
                                       self.batch_count, self.batch_stride)

    @staticmethod
    def of(t: torch.Tensor) -> "MatrixLayout":
        """Layout of a row- or col-ordered torch matrix ([rows, cols] or [batch, rows, cols]) as it lies in memory
        (MatrixLayout.init(_ tensor:), MatrixLayout.swift:27-47)."""
        if t.dim() not in (2, 3):
            raise ValueError("rank 2 or 3 expected")
        rows, cols = t.shape[-2], t.shape[-1]
        if t.stride(-1) == 1 or cols == 1:
            order, ld = Order.row, t.stride(-2)
        elif t.stride(-2) == 1 or rows == 1:
            order, ld = Order.col, t.stride(-1)
        else:
            raise ValueError("one of the last two dimensions must be contiguous")
        batch = t.shape[0] if t.dim() == 3 else 1
        return MatrixLayout(_TORCH2SRT[t.dtype], order, rows, cols, max(ld, 1), batch,
                            t.stride(0) if t.dim() == 3 and batch > 1 else 0)


def matrix_transform(a: torch.Tensor, a_layout: MatrixLayout, c_layout: MatrixLayout, alpha: float = 1.0,
                     trans_a: bool = False, beta: float = 0.0, b: torch.Tensor | None = None,
                     b_layout: MatrixLayout | None = None, trans_b: bool = False,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """C = alpha . op(A) + beta . op(B) on the current stream of A's device; returns C's buffer."""
    if not a.is_cuda:
        raise ValueError("device tensors expected")
    c = out if out is not None else c_layout.empty(a.device)
    if c.numel() < c_layout.elements or a.numel() < a_layout.elements or (b is not None and b_layout is not None and b.numel() < b_layout.elements):
        raise ValueError("a buffer is smaller than its layout")
    if _TORCH2SRT.get(a.dtype) != a_layout.type or _TORCH2SRT.get(c.dtype) != c_layout.type or \
            (b is not None and b_layout is not None and _TORCH2SRT.get(b.dtype) != b_layout.type):
        raise ValueError("a buffer's element type differs from its layout's")
    fa, fb = ctypes.c_float(alpha), ctypes.c_float(beta)
    sa, sc = a_layout.struct(), c_layout.struct()
    sb = b_layout.struct() if b_layout is not None else None
    with torch.cuda.device(a.device):
        rc = lib.srtMatrixTransform(ctypes.byref(fa), a.data_ptr(), ctypes.byref(sa), trans_a,
                                    ctypes.byref(fb), b.data_ptr() if b is not None else None,
                                    ctypes.byref(sb) if sb is not None else None, trans_b,
                                    c.data_ptr(), ctypes.byref(sc), torch.cuda.current_stream(a.device).cuda_stream)
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())
    return c
