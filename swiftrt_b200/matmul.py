"""Host-side mirror of the reference's matmul operators over the C ABI.

Same names, argument meaning and error behaviour as
  matmul(_:transposed:_:transposed:)        Sources/SwiftRTCore/operators/Matmul.swift:29-45
  matmul(_:transposed:_:transposed:bias:)   Matmul.swift:57-72
  matmulGradients                           differentiable/MathDerivatives.swift:460-482
and the queue-level rank-3 (batched) form   platform/cpu/functions/CpuMath.swift:363-369.
Every call goes to the CUDA library; there is no other path.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import lib
from .tensor import ActivationType, Descriptor, Order, empty, order_of


class MatmulError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"srtMatmul failed with cudaError {code}: {what}")
        self.code = code


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _result_shape(lhs, transpose_lhs, rhs, transpose_rhs):
    ls = tuple(lhs.shape[-2:])[::-1] if transpose_lhs else tuple(lhs.shape[-2:])
    rs = tuple(rhs.shape[-2:])[::-1] if transpose_rhs else tuple(rhs.shape[-2:])
    # the reference asserts here (Matmul.swift:35)
    assert ls[1] == rs[0], "matmul inner dimensions must be equal"
    batch = ()
    if lhs.dim() == 3 or rhs.dim() == 3:
        nb = max(lhs.shape[0] if lhs.dim() == 3 else 1, rhs.shape[0] if rhs.dim() == 3 else 1)
        batch = (nb,)
    return batch + (ls[0], rs[1])


_DESC_CACHE: dict = {}
_DESC_CACHE_MAX = 512


def _descriptor(t: torch.Tensor) -> Descriptor:
    """Descriptor for a tensor's geometry; built once per (shape, strides, dtype) and reused --
    descriptors hold no pointer, so tensors with equal geometry share one."""
    key = (t.dtype, tuple(t.shape), t.stride())
    d = _DESC_CACHE.get(key)
    if d is None:
        if len(_DESC_CACHE) >= _DESC_CACHE_MAX:
            _DESC_CACHE.clear()
        d = _DESC_CACHE[key] = Descriptor(t)
    return d


class MatmulOp:
    """A prepared call: descriptors and arguments are marshalled once, `op()` only enqueues.
    The object form of the operator, as DeviceMatmul2 / CudaMatmul2 is in the reference
    (cpu/functions/CpuMatmul.swift:21-58, cuda/functions/CudaMatmul.swift:71-120).  The tensors
    must stay alive and keep their geometry while the op is used."""

    def __init__(self, out: torch.Tensor, lhs: torch.Tensor, transpose_lhs: bool, rhs: torch.Tensor,
                 transpose_rhs: bool, bias: torch.Tensor | None = None,
                 activation: ActivationType | None = None, peer_pointers=None, multicast_pointer: int | None = None):
        """`peer_pointers`: device addresses of the same output view in other GPUs' buffers
        (PeerBuffer.peer_pointers); the result block is then delivered to them as well
        (srtMatmulAllGather).  `multicast_pointer`: address of the view in an NVLink multicast
        mapping instead (PeerBuffer.multicast_pointer, srtMatmulAllGatherMulticast)."""
        if not (lhs.is_cuda and rhs.is_cuda and out.is_cuda):
            raise ValueError("device tensors expected; use matmul_host for host buffers")
        self.out = out
        self._keep = (lhs, rhs, bias)
        self._device = out.device
        self._index = out.device.index if out.device.index is not None else torch.cuda.current_device()
        da, db, do = _descriptor(lhs), _descriptor(rhs), _descriptor(out)
        self._descs = (da, db, do)
        if multicast_pointer:
            dbias = _descriptor(bias) if bias is not None else None
            self._descs += (dbias,)
            self._fn = lib.srtMatmulAllGatherMulticast
            self._args = (lhs.data_ptr(), da.ref(), bool(transpose_lhs), rhs.data_ptr(), db.ref(), bool(transpose_rhs),
                          bias.data_ptr() if bias is not None else None, dbias.ref() if dbias is not None else None,
                          int(activation if activation is not None else ActivationType.identity),
                          out.data_ptr(), do.ref(), int(multicast_pointer))
        elif peer_pointers:
            dbias = _descriptor(bias) if bias is not None else None
            self._descs += (dbias,)
            self._peers = (ctypes.c_void_p * len(peer_pointers))(*peer_pointers)
            self._fn = lib.srtMatmulAllGather
            self._args = (lhs.data_ptr(), da.ref(), bool(transpose_lhs), rhs.data_ptr(), db.ref(), bool(transpose_rhs),
                          bias.data_ptr() if bias is not None else None, dbias.ref() if dbias is not None else None,
                          int(activation if activation is not None else ActivationType.identity),
                          out.data_ptr(), do.ref(), len(peer_pointers), self._peers)
        elif bias is None and activation is None:
            self._fn = lib.srtMatmul
            self._args = (lhs.data_ptr(), da.ref(), bool(transpose_lhs), rhs.data_ptr(), db.ref(), bool(transpose_rhs),
                          out.data_ptr(), do.ref())
        else:
            dbias = _descriptor(bias) if bias is not None else None
            self._descs += (dbias,)
            self._fn = lib.srtMatmulBiasActivation
            self._args = (lhs.data_ptr(), da.ref(), bool(transpose_lhs), rhs.data_ptr(), db.ref(), bool(transpose_rhs),
                          bias.data_ptr() if bias is not None else None, dbias.ref() if dbias is not None else None,
                          int(activation if activation is not None else ActivationType.identity),
                          out.data_ptr(), do.ref())

    def __call__(self) -> torch.Tensor:
        """Enqueues the product on torch's current stream of the output's device."""
        idx = self._index
        if torch.cuda.current_device() != idx:
            with torch.cuda.device(idx):
                rc = self._fn(*self._args, torch.cuda.current_stream(idx).cuda_stream)
        else:
            rc = self._fn(*self._args, torch.cuda.current_stream(idx).cuda_stream)
        if rc != _lib.cudaSuccess:
            raise MatmulError(rc, _lib.last_error())
        return self.out


def matmul_into(out: torch.Tensor, lhs: torch.Tensor, transpose_lhs: bool, rhs: torch.Tensor,
                transpose_rhs: bool, bias: torch.Tensor | None = None,
                activation: ActivationType | None = None) -> torch.Tensor:
    """The queue-level call: writes op(lhs).op(rhs) [+ bias, activation] into `out`, which may be a
    strided view (CpuMath.swift:355-369 takes the result inout).  Asynchronous on torch's current
    stream of out's device."""
    return MatmulOp(out, lhs, transpose_lhs, rhs, transpose_rhs, bias, activation)()


def matmul_all_gather_into(out: torch.Tensor, peer_pointers, lhs: torch.Tensor, transpose_lhs: bool, rhs: torch.Tensor,
                           transpose_rhs: bool, bias: torch.Tensor | None = None,
                           activation: ActivationType | None = None) -> torch.Tensor:
    """matmul_into whose result block also lands at `peer_pointers` (the same view in the other
    ranks' buffers).  The peers' copies are complete when this rank's stream has drained; order
    the ranks (PeerBuffer.ranks_done) before reading blocks that others wrote."""
    return MatmulOp(out, lhs, transpose_lhs, rhs, transpose_rhs, bias, activation, peer_pointers)()


def matmul_all_gather_multicast_into(out: torch.Tensor, multicast_pointer: int, lhs: torch.Tensor, transpose_lhs: bool,
                                     rhs: torch.Tensor, transpose_rhs: bool, bias: torch.Tensor | None = None,
                                     activation: ActivationType | None = None) -> torch.Tensor:
    """matmul_into whose result block is stored once to an NVLink multicast mapping and replicated
    into every rank's buffer by the NVSwitch (srtMatmulAllGatherMulticast).  Raises MatmulError
    with code 801 when the product is not eligible; use matmul_all_gather_into then."""
    return MatmulOp(out, lhs, transpose_lhs, rhs, transpose_rhs, bias, activation, None, multicast_pointer)()


def matmul(lhs: torch.Tensor, rhs: torch.Tensor, transposed_lhs: bool = False, transposed_rhs: bool = False,
           bias: torch.Tensor | None = None, activation: ActivationType | None = None) -> torch.Tensor:
    """result = op(lhs) . op(rhs), allocated dense in lhs's order (Matmul.swift:36-38).

    With `bias` (rank 1, one value per output column) the sum is added before the single
    rounding to the element type -- what matmul(bias:) declares.  Rank-3 operands are batched
    over dimension 0; a rank-2 operand next to a rank-3 one is used for every batch item."""
    shape = _result_shape(lhs, transposed_lhs, rhs, transposed_rhs)
    out = empty(shape, lhs.dtype, lhs.device, order_of(lhs))
    return matmul_into(out, lhs, transposed_lhs, rhs, transposed_rhs, bias, activation)


def matmul_gradients(out_grad: torch.Tensor, lhs: torch.Tensor, transpose_lhs: bool, rhs: torch.Tensor,
                     transpose_rhs: bool):
    """(lhsGrad, rhsGrad) exactly as matmulGradients composes them from two more matmul calls
    (MathDerivatives.swift:460-482), including its formulas for the transposed cases."""
    if not transpose_lhs and not transpose_rhs:
        return (matmul(out_grad, rhs, False, True), matmul(lhs, out_grad, True, False))
    if not transpose_lhs and transpose_rhs:
        return (matmul(out_grad, rhs), matmul(lhs, out_grad, True, False))
    if transpose_lhs and not transpose_rhs:
        return (matmul(out_grad, rhs, False, True), matmul(lhs, out_grad))
    return (matmul(out_grad, rhs, True, True), matmul(lhs, out_grad, True, True))


_HOST_STREAMS: dict = {}
_HOST_CHUNK_BYTES = 32 << 20       # below this much of lhs + result, one copy each way is as fast


def _side_streams(dev: torch.device):
    """(copy-in stream, copy-out stream) of a device, created once."""
    key = (dev.type, dev.index)
    if key not in _HOST_STREAMS:
        _HOST_STREAMS[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _HOST_STREAMS[key]


def matmul_host(lhs: torch.Tensor, rhs: torch.Tensor, transposed_lhs: bool = False, transposed_rhs: bool = False,
                bias: torch.Tensor | None = None, activation: ActivationType | None = None,
                device="cuda:0", out_host: torch.Tensor | None = None, chunks: int = 16) -> torch.Tensor:
    """The same operator for HOST tensors: inputs are copied to `device`, multiplied there and the
    result is copied back; the call returns when the result is in host memory.  This is what the
    reference's storage does around a queue call (host replicas migrate on deviceRead,
    DiscreteStorage.swift:310-381).  Pinned host memory makes the copies asynchronous.

    Large rank-2 products with a row-major, untransposed lhs are pipelined over `chunks` blocks of
    rows: rhs is copied first, then the copy-in of row block i + 1, the product of block i and the
    copy-out of block i - 1 overlap (the two copy directions use separate DMA engines)."""
    dev = torch.device(device)
    M = lhs.shape[-1] if transposed_lhs else lhs.shape[-2]
    N = rhs.shape[-2] if transposed_rhs else rhs.shape[-1]
    pipelined = (lhs.dim() == 2 and rhs.dim() == 2 and not transposed_lhs and lhs.is_contiguous() and chunks > 1
                 and M >= 128 * chunks
                 and (lhs.numel() + M * N) * lhs.element_size() >= _HOST_CHUNK_BYTES
                 and (out_host is None or out_host.is_contiguous()))
    if not pipelined:
        a = lhs.to(dev, non_blocking=True)
        b = rhs.to(dev, non_blocking=True)
        bz = bias.to(dev, non_blocking=True) if bias is not None else None
        c = matmul(a, b, transposed_lhs, transposed_rhs, bz, activation)
        if out_host is None:
            out_host = torch.empty(c.shape, dtype=c.dtype, pin_memory=True)
        out_host.copy_(c, non_blocking=True)
        torch.cuda.current_stream(dev).synchronize()
        return out_host

    if out_host is None:
        out_host = torch.empty((M, N), dtype=lhs.dtype, pin_memory=True)
    main = torch.cuda.current_stream(dev)
    s_in, s_out = _side_streams(dev)
    s_in.wait_stream(main)
    s_out.wait_stream(main)
    with torch.cuda.device(dev):
        a = torch.empty(lhs.shape, dtype=lhs.dtype, device=dev)
        c = torch.empty((M, N), dtype=lhs.dtype, device=dev)
        with torch.cuda.stream(s_in):
            b = rhs.to(dev, non_blocking=True)
            bz = bias.to(dev, non_blocking=True) if bias is not None else None
        rows = -(-M // chunks)
        rows = -(-rows // 128) * 128                      # whole tiles per block
        for r0 in range(0, M, rows):
            r1 = min(M, r0 + rows)
            with torch.cuda.stream(s_in):
                a[r0:r1].copy_(lhs[r0:r1], non_blocking=True)
                arrived = s_in.record_event()
            main.wait_event(arrived)
            matmul_into(c[r0:r1], a[r0:r1], False, b, transposed_rhs, bz, activation)
            done = main.record_event()
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                out_host[r0:r1].copy_(c[r0:r1], non_blocking=True)
        # the device buffers must outlive the side streams' work
        for t in (a, b, c) + ((bz,) if bz is not None else ()):
            t.record_stream(main)
            t.record_stream(s_in)
            t.record_stream(s_out)
    s_out.synchronize()
    return out_host


def query_plan(lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor, transposed_lhs: bool = False,
               transposed_rhs: bool = False) -> dict:
    """What a call with these tensors would launch (stands in for MatmulAlgorithm.query,
    cublaslt/MatmulAlgorithmSearch.swift:51-100)."""
    plan = _lib.MatmulPlan()
    da, db, do = Descriptor(lhs), Descriptor(rhs), Descriptor(out)
    with torch.cuda.device(out.device):
        rc = lib.srtMatmulQueryPlan(lhs.data_ptr(), da.ref(), transposed_lhs, rhs.data_ptr(), db.ref(), transposed_rhs,
                                    out.data_ptr(), do.ref(), ctypes.byref(plan))
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())
    return {name: getattr(plan, name) for name, _ in plan._fields_}


def tune(lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor, transposed_lhs: bool = False,
         transposed_rhs: bool = False, bias: torch.Tensor | None = None,
         activation: ActivationType | None = None) -> dict:
    """Times every kernel / tile width for this call and keeps the fastest for later calls with the
    same signature (srtMatmulTune; stands in for MatmulAlgorithm.search,
    cublaslt/MatmulAlgorithmSearch.swift:128-216).  Returns the winning plan plus its time
    ("microseconds"); `out` holds the product afterwards."""
    plan = _lib.MatmulPlan()
    us = ctypes.c_float()
    da, db, do = Descriptor(lhs), Descriptor(rhs), Descriptor(out)
    dbias = Descriptor(bias) if bias is not None else None
    with torch.cuda.device(out.device):
        rc = lib.srtMatmulTune(lhs.data_ptr(), da.ref(), transposed_lhs, rhs.data_ptr(), db.ref(), transposed_rhs,
                               bias.data_ptr() if bias is not None else None, dbias.ref() if dbias is not None else None,
                               int(activation if activation is not None else ActivationType.identity),
                               out.data_ptr(), do.ref(), torch.cuda.current_stream(out.device).cuda_stream,
                               ctypes.byref(plan), ctypes.byref(us))
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())
    result = {name: getattr(plan, name) for name, _ in plan._fields_}
    result["microseconds"] = float(us.value)
    return result


def save_plan_cache(path: str) -> None:
    """Writes the tuned plans to a text file (srtMatmulPlanCacheSave)."""
    if lib.srtMatmulPlanCacheSave(str(path).encode()) != _lib.cudaSuccess:
        raise MatmulError(_lib.cudaErrorInvalidValue, _lib.last_error())


def load_plan_cache(path: str) -> int:
    """Merges a plan cache file into the process's table; returns the number of entries read."""
    n = ctypes.c_int32()
    if lib.srtMatmulPlanCacheLoad(str(path).encode(), ctypes.byref(n)) != _lib.cudaSuccess:
        raise MatmulError(_lib.cudaErrorInvalidValue, _lib.last_error())
    return int(n.value)


def clear_plan_cache() -> None:
    lib.srtMatmulPlanCacheClear()


def set_tuning(force_kernel: int = 0, tile_n: int = 0, stages: int = 0, max_ctas: int = 0) -> None:
    rc = lib.srtMatmulSetTuning(force_kernel, tile_n, stages, max_ctas)
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())


def set_split_k(splits: int = 0) -> None:
    """0 = automatic, 1 = never, n > 1 = cut the reduction into up to n parts (srtMatmulSetSplitK)."""
    rc = lib.srtMatmulSetSplitK(splits)
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())


def check_status(device=None) -> int:
    """Synchronises the current stream and returns the tensor-core kernels' status word
    (0 = every pipeline wait completed)."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    status = ctypes.c_uint32(0)
    with torch.cuda.device(dev):
        rc = lib.srtMatmulCheckStatus(_stream_ptr(dev), ctypes.byref(status))
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())
    return status.value


def release_workspaces(include_captured: bool = False) -> None:
    """Frees the library's per-(device, stream) scratch buffers (srtMatmulReleaseWorkspaces)."""
    rc = lib.srtMatmulReleaseWorkspaces(bool(include_captured))
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())


def set_wait_limit(nanoseconds: int = 0, device=None) -> None:
    """Limit of every pipeline wait inside the tensor-core kernels of `device` (0 = the default)."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        rc = lib.srtMatmulSetWaitLimit(int(nanoseconds))
    if rc != _lib.cudaSuccess:
        raise MatmulError(rc, _lib.last_error())


def launch_count() -> int:
    return int(lib.srtMatmulLaunchCount())
