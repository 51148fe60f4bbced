"""Recurrent cells that call the fused product: the host mirror of LSTMCell and of the time-step
loop of RecurrentLayer (Sources/SwiftRTLayers/Recurrent.swift:165-266, 346-370).

Only what sits on the matmul path is mirrored: the cell step (concatenate, matmul(bias:), gates)
runs as srtLstmCell, the GRU step as srtGruCell; parameter initialisers and the derivative plumbing
are not mirrored."""
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

    def __init__(self, fused_weight: torch.Tensor, fused_bias: torch.Tensor | None, hidden_size: int | None = None,
                 fuse_gates: bool = False):
        """`fuse_gates`: run the gate pass inside the product's epilogue (srtLstmCellFused) when the step is
        eligible -- 16-bit elements, hiddenSize a multiple of 8, a one-pass tensor-core product -- and fall
        back to the three-launch step otherwise.  The interleaved copies of weight and bias are made once, here."""
        self.fuse_gates = bool(fuse_gates)
        self._interleaved = None
        if fused_weight.dim() != 2 or fused_weight.shape[1] % 4:
            raise ValueError("fusedWeight must be [(inputSize + hiddenSize) x 4 hiddenSize]")
        self.fused_weight = fused_weight
        self.fused_bias = fused_bias
        self.hidden_size = int(hidden_size if hidden_size is not None else fused_weight.shape[1] // 4)
        if fused_weight.shape[1] != 4 * self.hidden_size:
            raise ValueError("fusedWeight has 4 hiddenSize columns")
        if fused_bias is not None and tuple(fused_bias.shape) != (4 * self.hidden_size,):
            raise ValueError("fusedBias has 4 hiddenSize elements")

    def interleaved(self):
        """(weight, bias) with the four gate columns of every hidden unit side by side (srtLstmInterleaveGates)."""
        if self._interleaved is None:
            w = torch.empty_like(self.fused_weight, memory_format=torch.contiguous_format)
            b = torch.empty_like(self.fused_bias, memory_format=torch.contiguous_format) if self.fused_bias is not None else None
            with torch.cuda.device(w.device):
                stream = torch.cuda.current_stream(w.device).cuda_stream
                for src, dst in ((self.fused_weight, w), (self.fused_bias, b)):
                    if src is None:
                        continue
                    ds, dd = _descriptor(src), _descriptor(dst)
                    rc = lib.srtLstmInterleaveGates(src.data_ptr(), ds.ref(), dst.data_ptr(), dd.ref(), stream)
                    if rc != _lib.cudaSuccess:
                        raise MatmulError(rc, _lib.last_error())
            self._interleaved = (w, b)
        return self._interleaved

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
        _lstm_call(self, input, state.hidden, state.cell, new_cell, new_hidden)
        return LSTMState(new_cell, new_hidden)


def _lstm_call(cell: "LSTMCell", input, hidden, cell_state, new_cell, new_hidden) -> None:
    if cell.fuse_gates and input.dtype in (torch.float16, torch.bfloat16):
        w, b = cell.interleaved()
        tensors = (input, hidden, cell_state, w, b, new_cell, new_hidden)
        descs = [_descriptor(t) if t is not None else None for t in tensors]
        args = []
        for t, d in zip(tensors, descs):
            args += [t.data_ptr() if t is not None else None, d.ref() if d is not None else None]
        with torch.cuda.device(input.device):
            rc = lib.srtLstmCellFused(*args, torch.cuda.current_stream(input.device).cuda_stream)
        if rc == _lib.cudaSuccess:
            return
        if rc != _lib.cudaErrorNotSupported:
            raise MatmulError(rc, _lib.last_error())
    tensors = (input, hidden, cell_state, cell.fused_weight, cell.fused_bias, new_cell, new_hidden)
    descs = [_descriptor(t) if t is not None else None for t in tensors]
    args = []
    for t, d in zip(tensors, descs):
        args += [t.data_ptr() if t is not None else None, d.ref() if d is not None else None]
    with torch.cuda.device(input.device):
        rc = lib.srtLstmCell(*args, torch.cuda.current_stream(input.device).cuda_stream)
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())


def run_sequence_preconcatenated(cell: "LSTMCell", inputs: Sequence[torch.Tensor],
                                 initial_state: "LSTMState | None" = None) -> list:
    """run_sequence without the per-step concatenation: one buffer [T][batch][inputSize + hiddenSize]
    holds every step's gate input, the inputs are copied into its left columns once, and each
    step writes its hidden state straight into the right columns of the next step's row block
    (srtLstmCell with hidden = NULL).  Two launches per step instead of three; the returned hidden
    states are views into that buffer."""
    if not inputs:
        return []
    x0 = inputs[0]
    batch, nx, nh, steps = x0.shape[0], x0.shape[1], cell.hidden_size, len(inputs)
    state = initial_state if initial_state is not None else cell.zero_state(x0)
    gate = torch.empty((steps, batch, nx + nh), dtype=x0.dtype, device=x0.device)
    gate[:, :, :nx].copy_(torch.stack(list(inputs)))
    gate[0, :, nx:].copy_(state.hidden)
    outputs, c = [], state.cell
    for t in range(steps):
        new_cell = torch.empty_like(c, memory_format=torch.contiguous_format)
        new_hidden = gate[t + 1, :, nx:] if t + 1 < steps else torch.empty((batch, nh), dtype=x0.dtype, device=x0.device)
        _lstm_call(cell, gate[t], None, c, new_cell, new_hidden)
        outputs.append(LSTMState(new_cell, new_hidden))
        c = new_cell
    return outputs


class BasicRNNCell:
    """BasicRNNCell (Recurrent.swift:110-161): weight [(inputSize + hiddenSize) x hiddenSize], bias
    [1 x hiddenSize] (or a vector); newState = tanh(matmul(concatenate(input, state), weight) + bias)."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None):
        if weight.dim() != 2:
            raise ValueError("weight must be [(inputSize + hiddenSize) x hiddenSize]")
        self.weight = weight
        self.bias = bias
        self.hidden_size = int(weight.shape[1])

    def zero_state(self, input: torch.Tensor) -> torch.Tensor:
        """zeroState(for:) (Recurrent.swift:146-150)."""
        return torch.zeros((input.shape[0], self.hidden_size), dtype=input.dtype, device=input.device)

    def __call__(self, input: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        new_state = torch.empty_like(state, memory_format=torch.contiguous_format)
        tensors = (input, state, self.weight, self.bias, new_state)
        descs = [_descriptor(t) if t is not None else None for t in tensors]
        args = []
        for t, d in zip(tensors, descs):
            args += [t.data_ptr() if t is not None else None, d.ref() if d is not None else None]
        with torch.cuda.device(input.device):
            rc = lib.srtRnnCell(*args, torch.cuda.current_stream(input.device).cuda_stream)
        if rc != _lib.cudaSuccess:
            raise MatmulError(rc, _lib.last_error())
        return new_state


class GRUCell:
    """GRUCell (Recurrent.swift:271-342) with weights of the sizes its formulas need (the
    reference's initialiser allocates [inputSize x 1] placeholders, Recurrent.swift:311-323):
    reset / update / output Weight1 [inputSize x hiddenSize], Weight2 [hiddenSize x hiddenSize],
    biases [hiddenSize].  The six products of callAsFunction (Recurrent.swift:328-337) are fused
    into two at construction: gate weight [[resetW1 | updateW1], [resetW2 | updateW2]] and output
    weight [[outputW1], [outputW2]]."""

    def __init__(self, reset_w1, reset_w2, reset_bias, update_w1, update_w2, update_bias, output_w1, output_w2, output_bias):
        self.hidden_size = int(reset_w2.shape[0])
        self.gate_weight = torch.cat([torch.cat([reset_w1, update_w1], dim=1), torch.cat([reset_w2, update_w2], dim=1)], dim=0).contiguous()
        self.gate_bias = torch.cat([reset_bias, update_bias]).contiguous() if reset_bias is not None else None
        self.output_weight = torch.cat([output_w1, output_w2], dim=0).contiguous()
        self.output_bias = output_bias

    def zero_state(self, input: torch.Tensor) -> torch.Tensor:
        return torch.zeros((input.shape[0], self.hidden_size), dtype=input.dtype, device=input.device)

    def __call__(self, input: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
        new_state = torch.empty_like(state, memory_format=torch.contiguous_format)
        tensors = (input, state, self.gate_weight, self.gate_bias, self.output_weight, self.output_bias, new_state)
        descs = [_descriptor(t) if t is not None else None for t in tensors]
        args = []
        for t, d in zip(tensors, descs):
            args += [t.data_ptr() if t is not None else None, d.ref() if d is not None else None]
        with torch.cuda.device(input.device):
            rc = lib.srtGruCell(*args, torch.cuda.current_stream(input.device).cuda_stream)
        if rc != _lib.cudaSuccess:
            raise MatmulError(rc, _lib.last_error())
        return new_state


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


class GraphedSequence:
    """A fixed number of time steps of one cell captured into a CUDA graph: short sequences of
    small cells are bound by their 3 launches per step, and a replay enqueues all of them at once.

    The cell's weights, the step count, batch and sizes are fixed at construction.  Inputs and the
    initial state are copied into the graph's static buffers on every call; the returned states
    are the graph's static outputs (overwritten by the next call).  The capture runs on a private
    side stream, which also owns the library workspace the captured launches use."""

    def __init__(self, cell: LSTMCell, steps: int, batch: int, input_size: int, dtype: torch.dtype,
                 device: torch.device | str | None = None):
        device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.cell = cell
        self.inputs = [torch.zeros((batch, input_size), dtype=dtype, device=device) for _ in range(steps)]
        self.initial = LSTMState(torch.zeros((batch, cell.hidden_size), dtype=dtype, device=device),
                                 torch.zeros((batch, cell.hidden_size), dtype=dtype, device=device))
        self._stream = torch.cuda.Stream(device=device)
        current = torch.cuda.current_stream(device)
        self._stream.wait_stream(current)
        with torch.cuda.stream(self._stream):
            # everything that allocates or sets attributes happens here, outside the capture:
            # the workspace of this stream, kernel attributes, the planner's device query
            run_sequence(cell, self.inputs, self.initial)
        self._stream.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self._stream):
            self.outputs = run_sequence(cell, self.inputs, self.initial)
        current.wait_stream(self._stream)

    def __call__(self, inputs: Sequence[torch.Tensor], initial_state: LSTMState | None = None) -> list[LSTMState]:
        if len(inputs) != len(self.inputs):
            raise ValueError(f"captured for {len(self.inputs)} time steps")
        for dst, src in zip(self.inputs, inputs):
            dst.copy_(src)
        if initial_state is None:
            self.initial.cell.zero_()
            self.initial.hidden.zero_()
        else:
            self.initial.cell.copy_(initial_state.cell)
            self.initial.hidden.copy_(initial_state.hidden)
        self.graph.replay()
        return self.outputs
