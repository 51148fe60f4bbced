"""Dense layer: y = activation(x . W + b), the semantics that the reference's Dense declares
(Sources/SwiftRTLayers/Dense.swift:21-71: fields activation / weight / bias, weight
[inputSize x outputSize], bias [outputSize], init assertion bias.shape[0] == weight.shape[1])
but does not compute (callAsFunction returns its input, Dense.swift:36-39).  One fused kernel
launch per call."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import lib
from .matmul import MatmulError, _descriptor, matmul
from .tensor import ActivationType, order_of


def bias_activation_backward(out_grad: torch.Tensor, output: torch.Tensor | None, activation: ActivationType,
                             want_dz: bool = True, want_dbias: bool = True):
    """(dz, dbias) of the fused epilogue: dz = out_grad * activation'(output), dbias = column sums of dz.

    The derivatives that the reference leaves unimplemented for matmul(bias:)
    (differentiable/MathDerivatives.swift:520-554), written in terms of the forward output like the
    reference's cuDNN activation backward (cuda/layers/CudaActivation.swift:101-127).  One pass over
    out_grad and output on torch's current stream."""
    if not out_grad.is_cuda:
        raise ValueError("device tensors expected")
    activation = ActivationType(activation)
    dz = torch.empty_like(out_grad, memory_format=torch.contiguous_format) if want_dz else None
    dbias = torch.empty((out_grad.shape[-1],), dtype=out_grad.dtype, device=out_grad.device) if want_dbias else None
    d_dy = _descriptor(out_grad)
    d_y = _descriptor(output) if output is not None else None
    d_dz = _descriptor(dz) if dz is not None else None
    d_db = _descriptor(dbias) if dbias is not None else None
    with torch.cuda.device(out_grad.device):
        rc = lib.srtBiasActivationBackward(
            out_grad.data_ptr(), d_dy.ref(), output.data_ptr() if output is not None else None,
            d_y.ref() if d_y is not None else None, int(activation),
            dz.data_ptr() if dz is not None else None, d_dz.ref() if d_dz is not None else None,
            dbias.data_ptr() if dbias is not None else None, d_db.ref() if d_db is not None else None,
            torch.cuda.current_stream(out_grad.device).cuda_stream)
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())
    return dz, dbias


class Dense:
    def __init__(self, weight: torch.Tensor, bias: torch.Tensor, activation: ActivationType):
        # Dense.swift:48-49
        assert order_of(weight) == order_of(bias) or bias.dim() == 1
        assert bias.shape[0] == weight.shape[-1], "bias.shape[0] must equal weight.shape[1]"
        self.weight = weight
        self.bias = bias
        self.activation = ActivationType(activation)
        self.plan = None            # Dense.plan (Dense.swift:29): the plan is chosen per call

    def __call__(self, input: torch.Tensor) -> torch.Tensor:
        return matmul(input, self.weight, bias=self.bias, activation=self.activation)

    def backward(self, input: torch.Tensor, output: torch.Tensor, out_grad: torch.Tensor):
        """(input gradient, weight gradient, bias gradient) for y = activation(x . W + b).

        dz and db come from one fused pass; dx = dz . W^T and dW = x^T . dz are the two transposed
        products that matmulGradients composes (MathDerivatives.swift:460-482, case (false, false))."""
        dz, db = bias_activation_backward(out_grad, output, self.activation)
        dx = matmul(dz, self.weight, False, True)
        dw = matmul(input, dz, True, False)
        return dx, dw, db
