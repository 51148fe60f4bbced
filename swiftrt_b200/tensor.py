"""Host-side mirror of the pieces of the reference's tensor model that the matmul path
touches: element types, storage order, and the stack descriptor passed across the C ABI.

torch tensors stand in for SwiftRT's Tensor<Shape, Element> (device memory + shape +
strides); torch is plumbing here, it computes nothing on this path.
"""
from __future__ import annotations

import ctypes
import enum

import torch

from ._lib import TensorDescriptor


class DataType(enum.IntEnum):
    """srtDataType values (Modules/SwiftRTCuda/tensor_api.h:31-38)."""
    real32F = 0
    real16F = 2
    real8I = 3
    real16BF = 14


class Order(enum.IntEnum):
    """Storage order with cublasLtOrder_t values (Sources/SwiftRTCore/tensor/Tensor.swift:177-236)."""
    col = 0
    row = 1
    colTiled32 = 2          # tiled orders: storage of MatrixLayout buffers only (transform.py), not of torch tensors
    colTiledTC32x8 = 3
    colTiledTC32x32 = 4


class ActivationType(enum.IntEnum):
    """Raw values of ActivationType (platform/common/FunctionProperties.swift:44-51) plus gelu."""
    sigmoid = 0
    relu = 1
    tanh = 2
    clippedRelu = 3
    elu = 4
    identity = 5
    gelu = 6
    geluTanh = 7


_TORCH2SRT = {torch.float32: DataType.real32F, torch.float16: DataType.real16F,
              torch.bfloat16: DataType.real16BF}


def data_type(t: torch.Tensor) -> int:
    """srtDataType of a tensor; unknown element types map to -1 (the C ABI rejects them)."""
    return int(_TORCH2SRT.get(t.dtype, -1))


def order_of(t: torch.Tensor) -> Order:
    """Order of a tensor's last two dims as SwiftRT would label it: col when the row index
    is the contiguous one (strides (1, rows), tensor/Shape.swift:292-297), row otherwise."""
    if t.dim() >= 2 and t.stride(-2) == 1 and t.stride(-1) != 1:
        return Order.col
    return Order.row


def empty(shape, dtype: torch.dtype, device, order: Order = Order.row) -> torch.Tensor:
    """A dense tensor of the given logical shape stored in `order` (col order keeps the
    logical shape and transposes the last two dims of the storage)."""
    shape = tuple(int(s) for s in shape)
    if order == Order.row or len(shape) < 2:
        return torch.empty(shape, dtype=dtype, device=device)
    phys = shape[:-2] + (shape[-1], shape[-2])
    return torch.empty(phys, dtype=dtype, device=device).transpose(-1, -2)


class Descriptor:
    """Owns the ctypes arrays behind one srtTensorDescriptor for the duration of a call,
    as withTensor does on the Swift side (cuda/device/CudaExtensions.swift:24-84)."""

    def __init__(self, t: torch.Tensor):
        n = t.dim()
        sz = ctypes.c_size_t
        for s in t.stride():
            if s < 0:
                raise ValueError("negative strides cannot be described")
        self._shape = (sz * max(n, 1))(*t.shape)
        self._strides = (sz * max(n, 1))(*t.stride())
        span = 1 + sum((d - 1) * s for d, s in zip(t.shape, t.stride())) if t.numel() else 0
        self.struct = TensorDescriptor(data_type(t), n, int(order_of(t)), t.numel(), span,
                                       self._shape, self._strides, self._strides)

    def ref(self):
        return ctypes.byref(self.struct)
