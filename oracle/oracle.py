"""TEST INFRASTRUCTURE ONLY: ctypes wrapper around the CPU oracle (oracle/cpu_matmul.c).

Only tests, the smoke check and the benchmark's CPU arms import this module; the product
package never does.  16-bit tensors travel as numpy uint16 arrays holding the raw bf16 /
fp16 bit patterns, fp32 tensors as float32 arrays.  Arrays may be arbitrarily strided
views: strides are forwarded in elements, as the reference's srtTensorDescriptor does
(Modules/SwiftRTCuda/tensor_api.h:70-87).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

F32, F16, BF16 = 0, 2, 14            # srtDataType values (tensor_api.h:34-38)
ACT = {"sigmoid": 0, "relu": 1, "tanh": 2, "clippedRelu": 3, "elu": 4, "identity": 5,
       "gelu": 6, "geluTanh": 7}     # ActivationType raw values (FunctionProperties.swift:44-51) + gelu

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file; returns its path."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "cpu_matmul.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s"], check=True)
    return so


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        sz = ctypes.c_size_t
        L.oracle_matmul.restype = ctypes.c_int
        L.oracle_matmul.argtypes = [
            ctypes.c_int, ctypes.c_int,
            ctypes.c_void_p, ctypes.POINTER(sz), ctypes.POINTER(sz), ctypes.c_int,
            ctypes.c_void_p, ctypes.POINTER(sz), ctypes.POINTER(sz), ctypes.c_int,
            ctypes.c_void_p, ctypes.POINTER(sz), ctypes.POINTER(sz),
            ctypes.c_void_p, sz, ctypes.c_int, ctypes.c_int,
            ctypes.c_int, ctypes.c_int, ctypes.c_int, sz, sz]
        L.oracle_convert_f32_to.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, sz]
        L.oracle_convert_to_f32.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, sz]
        L.oracle_bias_activation_unfused.argtypes = [ctypes.c_int, ctypes.c_void_p, sz, sz,
                                                     ctypes.c_void_p, ctypes.c_int]
        L.oracle_bias_activation_backward.restype = ctypes.c_int
        L.oracle_bias_activation_backward.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, sz, sz, ctypes.c_int,
                                                      ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        L.oracle_activation_forward.restype = ctypes.c_int
        L.oracle_activation_forward.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, sz, ctypes.c_int]
        L.oracle_max_threads.restype = ctypes.c_int
        _LIB = L
    return _LIB


def np_dtype(dtype: int):
    return np.float32 if dtype == F32 else np.uint16


def encode(x, dtype: int) -> np.ndarray:
    """float32 values -> stored bits of `dtype` (RNE, NaN rule of the reference)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if dtype == F32:
        return x.copy()
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_convert_f32_to(dtype, x.ctypes.data, out.ctypes.data, x.size)
    return out


def decode(x: np.ndarray, dtype: int) -> np.ndarray:
    """stored bits of `dtype` -> float32 values (exact)."""
    if dtype == F32:
        return np.array(x, dtype=np.float32)
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().oracle_convert_to_f32(dtype, x.ctypes.data, out.ctypes.data, x.size)
    return out


def _desc(arr: np.ndarray):
    sz = ctypes.c_size_t
    item = arr.dtype.itemsize
    for s in arr.strides:
        if s < 0 or s % item:
            raise ValueError("negative or unaligned strides are not representable")
    shape = (sz * arr.ndim)(*arr.shape)
    strides = (sz * arr.ndim)(*[s // item for s in arr.strides])
    return shape, strides


def matmul(a: np.ndarray, b: np.ndarray, dtype: int, trans_a: bool = False, trans_b: bool = False,
           bias: np.ndarray | None = None, activation: str | None = None,
           out: np.ndarray | None = None, f16_native: bool = False,
           mode: int = 1, threads: int | None = None,
           rows: tuple[int, int] | None = None) -> np.ndarray:
    """C = op(A) . op(B) [+ bias, activation] exactly as the reference CPU loop computes it.

    a, b: rank 2, or rank 3 with the batch first; views with any non-negative strides.
    `out` may be a preallocated (possibly strided) view; otherwise a dense row-major result
    is created.  `rows=(r0, r1)` limits the computed output rows (bounded samples of large
    problems); other rows of `out` are left untouched.
    """
    L = lib()
    rank = a.ndim
    if rank not in (2, 3) or b.ndim != rank:
        raise ValueError("rank 2 or 3 operands of equal rank expected")
    q = rank - 2
    M = a.shape[q + 1] if trans_a else a.shape[q]
    N = b.shape[q] if trans_b else b.shape[q + 1]
    if out is None:
        oshape = (a.shape[0], M, N) if rank == 3 else (M, N)
        out = np.zeros(oshape, dtype=np_dtype(dtype))
    ash, ast = _desc(a)
    bsh, bst = _desc(b)
    osh, ost = _desc(out)
    has_epi = int(bias is not None or activation is not None)
    bias_p, bias_s = None, 0
    if bias is not None:
        bias_p = bias.ctypes.data
        bias_s = bias.strides[0] // bias.dtype.itemsize
    act = ACT[activation] if activation is not None else ACT["identity"]
    if threads is None:
        threads = L.oracle_max_threads()
    r0, r1 = rows if rows is not None else (0, M)
    rc = L.oracle_matmul(dtype, rank, a.ctypes.data, ash, ast, int(trans_a),
                         b.ctypes.data, bsh, bst, int(trans_b),
                         out.ctypes.data, osh, ost, bias_p, bias_s, act, has_epi,
                         int(f16_native), mode, threads, r0, r1)
    if rc != 0:
        raise ValueError(f"oracle_matmul failed with code {rc}")
    return out


def bias_activation_backward(dy: np.ndarray, y: np.ndarray, dtype: int, activation: str = "identity",
                             stepwise: bool = False):
    """(dz, dbias) for dense row-major [M x N] dy and forward output y: dz = dy * act'(y),
    dbias = column sums of dz (fp32 running sum rounded once; `stepwise` rounds after every row as
    the reference's cpu_sum does)."""
    dy = np.ascontiguousarray(dy)
    y = np.ascontiguousarray(y)
    M, N = dy.shape
    dz = np.empty_like(dy)
    dbias = np.zeros((N,), dtype=dy.dtype)
    rc = lib().oracle_bias_activation_backward(dtype, dy.ctypes.data, y.ctypes.data, M, N, ACT[activation],
                                               dz.ctypes.data, dbias.ctypes.data, int(stepwise))
    if rc != 0:
        raise ValueError(f"oracle_bias_activation_backward failed with code {rc}")
    return dz, dbias


def activation_forward(z: np.ndarray, dtype: int, activation: str) -> np.ndarray:
    """y = activation(z) on stored bits, fp32 arithmetic, one rounding."""
    z = np.ascontiguousarray(z)
    y = np.empty_like(z)
    rc = lib().oracle_activation_forward(dtype, z.ctypes.data, y.ctypes.data, z.size, ACT[activation])
    if rc != 0:
        raise ValueError(f"oracle_activation_forward failed with code {rc}")
    return y


def gru_cell(x: np.ndarray, hidden: np.ndarray, w: dict, dtype: int) -> np.ndarray:
    """One step of GRUCell.callAsFunction (Sources/SwiftRTLayers/Recurrent.swift:328-337) on stored
    bits, composed operator by operator as the reference does (every operator result rounded to the
    element type):
        reset  = sigmoid(matmul(x, resetW1) + matmul(h, resetW2, bias: resetB))
        update = sigmoid(matmul(x, updateW1) + matmul(h, updateW2, bias: updateB))
        output = tanh(matmul(x, outputW1, bias: outputB) + matmul(reset * h, outputW2))
        new    = (1 - update) * h + (1 - update) * output
    `w` maps resetW1, resetW2, resetB, updateW1, ... to stored bits.  Returns the new state's bits."""
    rnd = lambda v: decode(encode(v.astype(np.float32), dtype), dtype)          # noqa: E731
    mm = lambda a, b, bias=None: decode(matmul(np.ascontiguousarray(a), np.ascontiguousarray(b), dtype, bias=bias), dtype)   # noqa: E731
    h = decode(hidden, dtype)
    reset = rnd(_sigmoid32(rnd(mm(x, w["resetW1"]) + mm(hidden, w["resetW2"], w["resetB"]))))
    update = rnd(_sigmoid32(rnd(mm(x, w["updateW1"]) + mm(hidden, w["updateW2"], w["updateB"]))))
    rh = encode(rnd(reset * h), dtype)
    output = rnd(np.tanh(rnd(mm(x, w["outputW1"], w["outputB"]) + mm(rh, w["outputW2"])), dtype=np.float32))
    keep = rnd(np.float32(1) - update)
    return encode(rnd(keep * h) + rnd(keep * output), dtype)


def _sigmoid32(x: np.ndarray) -> np.ndarray:
    """1 / (1 + exp(-x)) in Float32, the reference's definition (cpu/functions/CpuMath.swift:1369-1377)."""
    x = x.astype(np.float32)
    return (np.float32(1) / (np.float32(1) + np.exp(-x, dtype=np.float32))).astype(np.float32)


def lstm_cell(x: np.ndarray, hidden: np.ndarray, cell: np.ndarray, fused_weight: np.ndarray,
              fused_bias: np.ndarray | None, dtype: int, stepwise: bool = False):
    """One step of LSTMCell.callAsFunction (Sources/SwiftRTLayers/Recurrent.swift:255-266) on stored
    bits: fused = matmul(concatenate(x, hidden), fusedWeight, bias:) through the restated CPU loop,
    gates i, u, f, o = sigmoid, tanh, sigmoid, sigmoid of its four column blocks, cell' = cell * f +
    i * u, hidden' = tanh(cell') * o.  Returns (cell', hidden') as stored bits.

    stepwise=False rounds only the tensors the step stores (fused, cell', hidden'); stepwise=True
    rounds every intermediate tensor to the element type, which is what composing the reference's
    separate operators does for 16-bit elements (identical for Float32)."""
    H = hidden.shape[1]
    gate_in = np.ascontiguousarray(np.concatenate([x, hidden], axis=1))
    fused = decode(matmul(gate_in, np.ascontiguousarray(fused_weight), dtype, bias=fused_bias), dtype)
    rnd = (lambda v: decode(encode(v, dtype), dtype)) if stepwise else (lambda v: v.astype(np.float32))
    gi = rnd(_sigmoid32(fused[:, 0:H]))
    gu = rnd(np.tanh(fused[:, H:2 * H], dtype=np.float32))
    gf = rnd(_sigmoid32(fused[:, 2 * H:3 * H]))
    go = rnd(_sigmoid32(fused[:, 3 * H:4 * H]))
    c = decode(cell, dtype)
    new_cell = encode(rnd(c * gf) + rnd(gi * gu), dtype)
    new_hidden = encode(rnd(np.tanh(decode(new_cell, dtype), dtype=np.float32)) * go, dtype)
    return new_cell, new_hidden


def rel_frobenius(x: np.ndarray, ref: np.ndarray) -> float:
    """||x - ref||_F / ||ref||_F in float64."""
    x = np.asarray(x, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = float(np.linalg.norm(ref.ravel()))
    num = float(np.linalg.norm((x - ref).ravel()))
    return num / den if den > 0 else num
