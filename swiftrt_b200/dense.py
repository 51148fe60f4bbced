"""Dense layer: y = activation(x . W + b), the semantics that the reference's Dense declares
(Sources/SwiftRTLayers/Dense.swift:21-71: fields activation / weight / bias, weight
[inputSize x outputSize], bias [outputSize], init assertion bias.shape[0] == weight.shape[1])
but does not compute (callAsFunction returns its input, Dense.swift:36-39).  One fused kernel
launch per call."""
from __future__ import annotations

import torch

from .matmul import matmul
from .tensor import ActivationType, order_of


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
