"""Multi-GPU sharding of one matmul: one process per GPU, independent output blocks, no
reduction, at most one exchange step (an all-gather of the output shards).

This is the reference's only data-parallel idea -- pmap splits axis 0 into partitions whose
results land in views of one shared output (Sources/SwiftRTCore/platform/common/pmap.swift:
26-72, 77-86) -- moved from CPU threads to GPUs:

  axis "batch": rank r multiplies batch items [b0, b1)            (batched matmul)
  axis "m":     rank r multiplies rows [m0, m1) of op(lhs)          (tall-skinny matmul)
  axis "n":     rank r multiplies columns [n0, n1) of op(rhs)       (large square matmul)

Every rank passes the full logical operands (or at least the slices it owns: only the owned
slices are read).  The local result is written straight into this rank's view of `out` when the
full output is wanted, so the gather needs no staging copy for the batch and m axes.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

AXES = ("batch", "m", "n")


def shard_range(total: int, world: int, rank: int, align: int = 1) -> tuple[int, int]:
    """Contiguous, balanced [start, stop) of `total` items for `rank` of `world`.

    Shard boundaries are multiples of `align` (the last shard takes the remainder), so that
    column slices of 16-bit matrices stay 16-byte aligned for TMA."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    units = -(-total // align)
    base, extra = divmod(units, world)
    start_u = rank * base + min(rank, extra)
    stop_u = start_u + base + (1 if rank < extra else 0)
    return min(start_u * align, total), min(stop_u * align, total)


def _slice_operands(lhs, transposed_lhs, rhs, transposed_rhs, axis, lo, hi):
    if axis == "batch":
        a = lhs[lo:hi] if lhs.dim() == 3 else lhs
        b = rhs[lo:hi] if rhs.dim() == 3 else rhs
        return a, b
    if axis == "m":
        # rows of op(lhs): dim -2 of lhs, or dim -1 when it is used transposed
        a = lhs.narrow(-1 if transposed_lhs else -2, lo, hi - lo)
        return a, rhs
    b = rhs.narrow(-2 if transposed_rhs else -1, lo, hi - lo)
    return lhs, b


def sharded_matmul(lhs: torch.Tensor, rhs: torch.Tensor, transposed_lhs: bool = False,
                   transposed_rhs: bool = False, axis: str = "n", gather: bool = False,
                   out: Optional[torch.Tensor] = None, group=None,
                   matmul_into_fn: Optional[Callable] = None,
                   rank: Optional[int] = None, world: Optional[int] = None,
                   peer_buffer=None, gather_fn: Optional[Callable] = None) -> torch.Tensor:
    """Computes this rank's block of op(lhs).op(rhs).

    Returns the local block (a dense tensor) when `gather` is False, else the full result on
    every rank.  `out`, if given, is the full-size result tensor to fill (gather) or the local
    block.  `matmul_into_fn(out, lhs, tl, rhs, tr)` defaults to the CUDA operator; tests on CPU
    ranks inject their own.

    With `peer_buffer` (a swiftrt_b200.peer.PeerBuffer of the full result's shape) the gather is
    fused into the product: this rank's block is written into its view of every rank's buffer
    by the product's own kernel (srtMatmulAllGather), there is no collective and no staging copy
    for any axis, and the call returns peer_buffer.tensor.  Blocks from other ranks are complete
    after peer_buffer.ranks_done().  `gather_fn(out_view, peer_pointers, lhs, tl, rhs, tr)`
    defaults to the CUDA operator."""
    if axis not in AXES:
        raise ValueError(f"axis must be one of {AXES}")
    if matmul_into_fn is None:
        from .matmul import matmul_into as matmul_into_fn
    if world is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
    if rank is None:
        rank = dist.get_rank(group) if dist.is_initialized() else 0

    a_rows = lhs.shape[-1] if transposed_lhs else lhs.shape[-2]
    b_cols = rhs.shape[-2] if transposed_rhs else rhs.shape[-1]
    batched = lhs.dim() == 3 or rhs.dim() == 3
    nb = max(lhs.shape[0] if lhs.dim() == 3 else 1, rhs.shape[0] if rhs.dim() == 3 else 1)
    if axis == "batch" and not batched:
        raise ValueError("batch sharding needs a rank-3 operand")
    total = {"batch": nb, "m": a_rows, "n": b_cols}[axis]
    align = 8 if axis == "n" and lhs.element_size() == 2 else (4 if axis == "n" else 1)
    lo, hi = shard_range(total, world, rank, align)
    a, b = _slice_operands(lhs, transposed_lhs, rhs, transposed_rhs, axis, lo, hi)

    full_shape = ((nb,) if batched else ()) + (a_rows, b_cols)
    dim = {"batch": 0, "m": len(full_shape) - 2, "n": len(full_shape) - 1}[axis]
    local_shape = list(full_shape)
    local_shape[dim] = hi - lo

    if peer_buffer is not None:
        if tuple(peer_buffer.tensor.shape) != tuple(full_shape):
            raise ValueError(f"peer buffer of shape {tuple(peer_buffer.tensor.shape)}, result is {tuple(full_shape)}")
        if hi > lo:
            view = peer_buffer.tensor.narrow(dim, lo, hi - lo)
            if gather_fn is None:
                from .matmul import MatmulError, matmul_all_gather_into, matmul_all_gather_multicast_into
                # between two GPUs there is nothing for the switch to replicate: the per-peer form is faster there
                mc = peer_buffer.multicast_pointer(view) if (getattr(peer_buffer, "multicast_base", 0) and world > 2) else 0
                if mc:
                    try:        # one multimem store per tile; products it does not take (code 801) go peer by peer
                        matmul_all_gather_multicast_into(view, mc, a, transposed_lhs, b, transposed_rhs)
                        return peer_buffer.tensor
                    except MatmulError as e:
                        if e.code != 801:
                            raise
                gather_fn = matmul_all_gather_into
            gather_fn(view, peer_buffer.peer_pointers(view), a, transposed_lhs, b, transposed_rhs)
        return peer_buffer.tensor

    if not gather:
        local = out if out is not None else torch.empty(local_shape, dtype=lhs.dtype, device=lhs.device)
        if hi > lo:
            matmul_into_fn(local, a, transposed_lhs, b, transposed_rhs)
        return local

    full = out if out is not None else torch.empty(full_shape, dtype=lhs.dtype, device=lhs.device)
    if world == 1:
        matmul_into_fn(full, a, transposed_lhs, b, transposed_rhs)
        return full
    if dim == 0 and full.is_contiguous() and total % world == 0 and (total // world) % align == 0:
        # equal contiguous blocks along the outermost dim: compute in place, gather in place
        if hi > lo:
            matmul_into_fn(full.narrow(0, lo, hi - lo), a, transposed_lhs, b, transposed_rhs)
        dist.all_gather_into_tensor(full, full.narrow(0, lo, hi - lo), group=group)
        return full
    # general case (inner-dim blocks, ragged shards): every rank contributes a dense block padded
    # to the longest shard, the blocks are gathered into a staging tensor and placed
    longest = max(shard_range(total, world, r, align)[1] - shard_range(total, world, r, align)[0]
                  for r in range(world))
    pad_shape = list(full_shape)
    pad_shape[dim] = longest
    staging = torch.empty([world] + pad_shape, dtype=lhs.dtype, device=lhs.device)
    mine = staging[rank]
    if hi > lo:
        matmul_into_fn(mine.narrow(dim, 0, hi - lo), a, transposed_lhs, b, transposed_rhs)
    dist.all_gather_into_tensor(staging.flatten(0, 1), mine, group=group)   # blocks concatenated along dim 0
    for r in range(world):
        r_lo, r_hi = shard_range(total, world, r, align)
        if r_hi > r_lo:
            full.narrow(dim, r_lo, r_hi - r_lo).copy_(staging[r].narrow(dim, 0, r_hi - r_lo))
    return full


_HOST_STREAMS: dict = {}


class _InlineStream:
    """Stands in for a CUDA stream on CPU ranks (the gloo tests): everything runs in program order."""

    def wait_stream(self, other):
        pass

    def wait_event(self, event):
        pass

    def record_event(self):
        return None

    def synchronize(self):
        pass


def _on(stream):
    import contextlib
    return contextlib.nullcontext() if isinstance(stream, _InlineStream) else torch.cuda.stream(stream)


def _host_streams(dev: torch.device):
    """(main, copy-in, all-gather, copy-out) streams of a device; the side streams are created once."""
    if dev.type != "cuda":
        return _InlineStream(), _InlineStream(), _InlineStream(), _InlineStream()
    key = (dev.type, dev.index)
    if key not in _HOST_STREAMS:
        _HOST_STREAMS[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return (torch.cuda.current_stream(dev),) + _HOST_STREAMS[key]


def sharded_matmul_host(lhs: torch.Tensor, rhs: torch.Tensor, transposed_lhs: bool = False, transposed_rhs: bool = False,
                        axis: str = "n", bias: Optional[torch.Tensor] = None, activation=None,
                        out_host: Optional[torch.Tensor] = None, device=None, group=None, pieces: int = 4,
                        rank: Optional[int] = None, world: Optional[int] = None,
                        matmul_into_fn: Optional[Callable] = None, matmul_host_fn: Optional[Callable] = None) -> torch.Tensor:
    """sharded_matmul for HOST tensors, one process per GPU: every rank passes only ITS OWN share of
    the host data and receives its block of the result in host memory, so that each operand byte
    crosses PCIe once whatever the number of GPUs (the reference migrates whole replicas on
    deviceRead, Sources/SwiftRTCore/tensor/DiscreteStorage.swift:310-381).

      axis "batch"  lhs, rhs: this rank's batch items          -> its batch items of the result
      axis "m"      lhs: this rank's rows, rhs: all of it       -> its rows of the result
      axis "n"      lhs: this rank's ROW block [M / world x K] of the operand every rank needs,
                    rhs: this rank's column block [K x n_local] -> its column block [M x n_local]

    For axis "n" the row blocks of lhs are all-gathered over NVLink (NCCL) into every rank's device
    copy, piece by piece: the copy-in of piece p + 1, the all-gather of piece p, the product of the
    rows already gathered and the copy-out of finished rows overlap.  The product kernel reads local
    HBM only.  Row blocks must be equal on all ranks; lhs rank 2, not transposed."""
    if axis not in AXES:
        raise ValueError(f"axis must be one of {AXES}")
    if world is None:
        world = dist.get_world_size(group) if dist.is_initialized() else 1
    if rank is None:
        rank = dist.get_rank(group) if dist.is_initialized() else 0
    if matmul_host_fn is None:
        from .matmul import matmul_host as matmul_host_fn
    dev = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
    on_gpu = dev.type == "cuda"
    if axis != "n" or world == 1:
        return matmul_host_fn(lhs, rhs, transposed_lhs, transposed_rhs, bias=bias, activation=activation, device=dev,
                              out_host=out_host)
    if lhs.dim() != 2 or rhs.dim() != 2 or transposed_lhs:
        raise ValueError("axis 'n' with host buffers takes a rank-2, untransposed lhs row block")
    if matmul_into_fn is None:
        from .matmul import matmul_into as matmul_into_fn
    mb, k = lhs.shape
    n_local = rhs.shape[0] if transposed_rhs else rhs.shape[1]
    m = mb * world
    if out_host is None:
        out_host = torch.empty((m, n_local), dtype=lhs.dtype, pin_memory=on_gpu)
    pieces = max(1, min(pieces, mb))
    step = -(-mb // pieces)
    step = min(mb, -(-step // 128) * 128)                     # whole tiles per piece
    import contextlib
    main, s_in, s_ag, s_out = _host_streams(dev)
    for s in (s_in, s_ag, s_out):
        s.wait_stream(main)
    with (torch.cuda.device(dev) if on_gpu else contextlib.nullcontext()):
        with _on(s_in):
            b = rhs.to(dev, non_blocking=True)
            bz = bias.to(dev, non_blocking=True) if bias is not None else None
            b_ready = s_in.record_event()
        c = torch.empty((world, mb, n_local), dtype=lhs.dtype, device=dev)
        keep = [b, c] + ([bz] if bz is not None else [])
        main.wait_event(b_ready)
        for r0 in range(0, mb, step):
            r1 = min(mb, r0 + step)
            g = torch.empty((world, r1 - r0, k), dtype=lhs.dtype, device=dev)     # rows [r0, r1) of every rank's block
            keep.append(g)
            with _on(s_in):
                g[rank].copy_(lhs[r0:r1], non_blocking=True)
                arrived = s_in.record_event()
            with _on(s_ag):
                s_ag.wait_event(arrived)
                dist.all_gather_into_tensor(g.view(world * (r1 - r0), k), g[rank], group=group)
                gathered = s_ag.record_event()
            main.wait_event(gathered)
            # one batched product: item r = the rows of rank r's block, against this rank's columns
            matmul_into_fn(c[:, r0:r1], g, False, b, transposed_rhs, bz, activation)
            done = main.record_event()
            with _on(s_out):
                s_out.wait_event(done)
                for r in range(world):
                    out_host[r * mb + r0:r * mb + r1].copy_(c[r, r0:r1], non_blocking=True)
        if on_gpu:
            for t in keep:
                for s in (main, s_in, s_ag, s_out):
                    t.record_stream(s)
    s_out.synchronize()
    return out_host
