"""Recurrent cells that call the fused product: the host mirror of LSTMCell and of the time-step
loop of RecurrentLayer (Sources/SwiftRTLayers/Recurrent.swift:165-266, 346-370).

Only what sits on the matmul path is mirrored: the cell step (concatenate, matmul(bias:), gates)
runs as srtLstmCell; parameter initialisers, the derivative plumbing and the GRU cell, whose
reference weights are [inputSize x 1] placeholders (Recurrent.swift:311-323), are not."""
from __future__ import annotations

from typing import NamedTuple, Sequence

import torch

from . import _lib
from ._lib import lib
from .matmul import MatmulError, _descriptor


class LSTMState(NamedTuple):
    """LSTMCell.State (Recurrent.swift:222-241)."""
    cell: torch.Tensor
    hidden: torch.Tensor


class LSTMCell:
    """fusedWeight [(inputSize + hiddenSize) x 4 hiddenSize], fusedBias [4 hiddenSize]; the four
    column blocks are the input, update, forget and output gates (Part, Recurrent.swift:173)."""

    def __init__(self, fused_weight: torch.Tensor, fused_bias: torch.Tensor | None, hidden_size: int | None = None):
        if fused_weight.dim() != 2 or fused_weight.shape[1] % 4:
            raise ValueError("fusedWeight must be [(inputSize + hiddenSize) x 4 hiddenSize]")
        self.fused_weight = fused_weight
        self.fused_bias = fused_bias
        self.hidden_size = int(hidden_size if hidden_size is not None else fused_weight.shape[1] // 4)
        if fused_weight.shape[1] != 4 * self.hidden_size:
            raise ValueError("fusedWeight has 4 hiddenSize columns")
        if fused_bias is not None and tuple(fused_bias.shape) != (4 * self.hidden_size,):
            raise ValueError("fusedBias has 4 hiddenSize elements")

    def zero_state(self, input: torch.Tensor) -> LSTMState:
        """zeroState(for:) (Recurrent.swift:245-248)."""
        shape = (input.shape[0], self.hidden_size)
        return LSTMState(torch.zeros(shape, dtype=input.dtype, device=input.device),
                         torch.zeros(shape, dtype=input.dtype, device=input.device))

    def __call__(self, input: torch.Tensor, state: LSTMState) -> LSTMState:
        """One time step; returns the new state (output and state are the same value in the
        reference, Recurrent.swift:264-265).  Asynchronous on torch's current stream."""
        if not input.is_cuda:
            raise ValueError("device tensors expected")
        new_cell = torch.empty_like(state.cell, memory_format=torch.contiguous_format)
        new_hidden = torch.empty_like(state.hidden, memory_format=torch.contiguous_format)
        tensors = (input, state.hidden, state.cell, self.fused_weight, self.fused_bias, new_cell, new_hidden)
        descs = [_descriptor(t) if t is not None else None for t in tensors]
        args = []
        for t, d in zip(tensors, descs):
            args += [t.data_ptr() if t is not None else None, d.ref() if d is not None else None]
        with torch.cuda.device(input.device):
            rc = lib.srtLstmCell(*args, torch.cuda.current_stream(input.device).cuda_stream)
        if rc != _lib.cudaSuccess:
            raise MatmulError(rc, _lib.last_error())
        return LSTMState(new_cell, new_hidden)


def run_sequence(cell: LSTMCell, inputs: Sequence[torch.Tensor], initial_state: LSTMState | None = None) -> list[LSTMState]:
    """RecurrentLayer.callAsFunction(_:initialState:) (Recurrent.swift:356-370): the cell applied to
    every time step in order, each step's state feeding the next; returns the state after every step."""
    if not inputs:
        return []
    state = initial_state if initial_state is not None else cell.zero_state(inputs[0])
    outputs = []
    for x in inputs:
        state = cell(x, state)
        outputs.append(state)
    return outputs
