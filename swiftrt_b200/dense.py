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
    For gelu and geluTanh `output` is the PRE-activation tensor (see Dense.forward_keep).

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


def activation_forward(pre_activation: torch.Tensor, activation: ActivationType, out: torch.Tensor | None = None) -> torch.Tensor:
    """y = activation(z), elementwise (srtActivationForward): the layer output of a Dense that kept
    its pre-activation values for the backward pass."""
    if not pre_activation.is_cuda:
        raise ValueError("device tensors expected")
    y = out if out is not None else torch.empty_like(pre_activation, memory_format=torch.contiguous_format)
    dz, dy = _descriptor(pre_activation), _descriptor(y)
    with torch.cuda.device(pre_activation.device):
        rc = lib.srtActivationForward(pre_activation.data_ptr(), dz.ref(), int(ActivationType(activation)), y.data_ptr(), dy.ref(),
                                      torch.cuda.current_stream(pre_activation.device).cuda_stream)
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())
    return y


_NEEDS_PRE_ACTIVATION = (ActivationType.gelu, ActivationType.geluTanh)


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

    def forward_keep(self, input: torch.Tensor):
        """(output, saved) for training: `saved` is what backward() needs in place of the output.  For
        activations whose derivative is a function of the output (identity, relu, sigmoid, tanh) this is
        the fused call and saved is the output itself; GELU's derivative needs the pre-activation
        values, so the product runs with the identity epilogue, its result is kept, and the activation
        is a second elementwise pass."""
        if self.activation in _NEEDS_PRE_ACTIVATION:
            z = matmul(input, self.weight, bias=self.bias, activation=ActivationType.identity)
            return activation_forward(z, self.activation), z
        y = self(input)
        return y, y

    def backward(self, input: torch.Tensor, output: torch.Tensor, out_grad: torch.Tensor):
        """(input gradient, weight gradient, bias gradient) for y = activation(x . W + b); `output` is
        the second value of forward_keep (the layer output, or the pre-activation values for GELU).

        dz and db come from one fused pass; dx = dz . W^T and dW = x^T . dz are the two transposed
        products that matmulGradients composes (MathDerivatives.swift:460-482, case (false, false))."""
        dz, db = bias_activation_backward(out_grad, output, self.activation)
        dx = matmul(dz, self.weight, False, True)
        dw = matmul(input, dz, True, False)
        return dx, dw, db
