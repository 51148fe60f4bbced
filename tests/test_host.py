"""Host-side mirror of the reference's operator interface: shapes, orders, descriptors, sharding."""
import pytest
import torch

import swiftrt_b200 as srt
from swiftrt_b200.matmul import _result_shape
from swiftrt_b200.tensor import Descriptor


def test_order_and_col_storage():
    t = srt.empty((2, 3), torch.float32, "cpu", srt.Order.col)
    assert tuple(t.shape) == (2, 3) and t.stride() == (1, 2)      # strides (1, rows): Shape.swift:292-297
    assert srt.order_of(t) == srt.Order.col
    r = srt.empty((2, 3), torch.float32, "cpu", srt.Order.row)
    assert r.stride() == (3, 1) and srt.order_of(r) == srt.Order.row
    # reference fixture: logical [[0,1,2],[3,4,5]] in col order is stored [0,3,1,4,2,5] (test_Shape.swift:85-101)
    t.copy_(torch.arange(6.0).reshape(2, 3))
    assert t.t().contiguous().flatten().tolist() == [0, 3, 1, 4, 2, 5]


def test_result_shape_follows_transposes_and_batch():
    a, b = torch.empty(3, 2), torch.empty(2, 4)
    assert _result_shape(a, False, b, False) == (3, 4)
    assert _result_shape(a.t(), True, b, False) == (3, 4)
    assert _result_shape(a, False, b.t(), True) == (3, 4)
    assert _result_shape(torch.empty(5, 3, 2), False, b, False) == (5, 3, 4)
    assert _result_shape(a, False, torch.empty(7, 2, 4), False) == (7, 3, 4)
    with pytest.raises(AssertionError):
        _result_shape(a, False, torch.empty(3, 4), False)


def test_descriptor_carries_view_geometry():
    base = torch.empty(10, 12, dtype=torch.bfloat16)
    v = base[2:8:2, 1:9]
    d = Descriptor(v).struct
    assert d.type == 14 and d.rank == 2 and d.count == 24
    assert [d.shape[i] for i in range(2)] == [3, 8]
    assert [d.strides[i] for i in range(2)] == [24, 1]
    assert d.spanCount == 2 * 24 + 7 + 1
    assert Descriptor(torch.empty(2, dtype=torch.int32)).struct.type == -1


def test_host_tensors_are_rejected_by_the_device_operator():
    with pytest.raises(ValueError):
        srt.matmul(torch.empty(3, 2), torch.empty(2, 4))


def test_dense_checks_shapes_like_the_reference_init():
    w, b = torch.empty(8, 4), torch.empty(4)
    layer = srt.Dense(w, b, srt.ActivationType.relu)
    assert layer.activation == srt.ActivationType.relu
    with pytest.raises(AssertionError):
        srt.Dense(w, torch.empty(5), srt.ActivationType.relu)


@pytest.mark.parametrize("total,world,align", [(16384, 8, 8), (64, 8, 1), (65536, 4, 1), (100, 8, 8), (5, 8, 1), (520, 3, 8)])
def test_shard_ranges_partition_the_axis(total, world, align):
    ranges = [srt.shard_range(total, world, r, align) for r in range(world)]
    assert ranges[0][0] == 0 and ranges[-1][1] == total
    for (lo, hi), (lo2, _) in zip(ranges, ranges[1:]):
        assert hi == lo2 and lo <= hi
    assert all(lo % align == 0 for lo, _ in ranges)
    sizes = [hi - lo for lo, hi in ranges]
    assert max(sizes) - min(s for s in sizes if s or True) <= 2 * align or min(sizes) == 0


class _FakePeerBuffer:
    """The part of PeerBuffer that sharded_matmul uses, over host tensors of one process: the
    'addresses' of the peers' buffers are the data pointers of the other ranks' tensors."""

    def __init__(self, tensors, rank):
        self.tensor = tensors[rank]
        self.peer_base = {r: t.data_ptr() for r, t in enumerate(tensors) if r != rank}
        self.nbytes = self.tensor.numel() * self.tensor.element_size()

    peer_pointers = __import__("swiftrt_b200").PeerBuffer.peer_pointers


@pytest.mark.parametrize("axis,ash,bsh,tl,tr", [("n", (24, 16), (16, 40), False, False),
                                                 ("m", (26, 16), (16, 12), False, False),
                                                 ("m", (16, 26), (12, 16), True, True),
                                                 ("batch", (6, 8, 5), (6, 5, 7), False, False)])
def test_sharded_matmul_with_peer_buffers_fills_every_rank(axis, ash, bsh, tl, tr):
    """Every rank's block must land at the same place in every rank's buffer: the view offsets
    handed to the gathering product are checked by writing through them."""
    import ctypes
    import swiftrt_b200 as srt
    g = torch.Generator().manual_seed(1)
    a = torch.rand(ash, generator=g)
    b = torch.rand(bsh, generator=g)
    want = torch.matmul(a.transpose(-1, -2) if tl else a, b.transpose(-1, -2) if tr else b)
    world = 3
    buffers = [torch.full(want.shape, -1.0) for _ in range(world)]

    def gather_fn(view, peer_ptrs, lhs, tl_, rhs, tr_):
        block = torch.matmul(lhs.transpose(-1, -2) if tl_ else lhs, rhs.transpose(-1, -2) if tr_ else rhs)
        view.copy_(block)
        assert len(peer_ptrs) == world - 1
        for ptr in peer_ptrs:                       # the same view, re-based on a peer's buffer
            span = 1 + sum((n - 1) * s for n, s in zip(view.shape, view.stride()))
            raw = (ctypes.c_float * span).from_address(ptr)
            peer = torch.as_strided(torch.frombuffer(raw, dtype=torch.float32), view.shape, view.stride())
            peer.copy_(block)

    for rank in range(world):
        got = srt.sharded_matmul(a, b, tl, tr, axis=axis, rank=rank, world=world,
                                 peer_buffer=_FakePeerBuffer(buffers, rank), gather_fn=gather_fn)
        assert got is buffers[rank]
    for buf in buffers:
        assert torch.allclose(buf, want, rtol=1e-6, atol=1e-6)
    with pytest.raises(ValueError):
        srt.sharded_matmul(a, b, tl, tr, axis=axis, rank=0, world=world,
                           peer_buffer=_FakePeerBuffer([torch.zeros(2, 2)] * 2, 0), gather_fn=gather_fn)


def test_plan_cache_file_round_trip_without_a_gpu(tmp_path):
    """The plan table's file form: load merges entries (bad lines are skipped, a wrong header is
    refused), save writes them back, clear empties the table."""
    import swiftrt_b200 as srt
    srt.clear_plan_cache()
    src = tmp_path / "plans.txt"
    src.write_text("srt_matmul_plan_cache v1\n# comment\n"
                   "14 85 1024 4096 4096 1 3 256 4 0 1 29.5\n"
                   "0 21 65536 256 1024 1 4 128 3 0 1 184.0\n"
                   "not a plan line\n"
                   "14 85 1024 4096 4096 1 2 128 6 0 1 31.0\n")       # same signature again: the later line wins
    assert srt.load_plan_cache(str(src)) == 3
    dst = tmp_path / "out.txt"
    srt.save_plan_cache(str(dst))
    lines = [l for l in dst.read_text().splitlines() if l and not l.startswith("#")]
    assert lines[0] == "srt_matmul_plan_cache v1"
    assert sorted(lines[1:]) == sorted(["14 85 1024 4096 4096 1 2 128 6 0 1 31.000", "0 21 65536 256 1024 1 4 128 3 0 1 184.000"])
    bad = tmp_path / "bad.txt"
    bad.write_text("something else\n1 2 3\n")
    with pytest.raises(srt.MatmulError):
        srt.load_plan_cache(str(bad))
    with pytest.raises(srt.MatmulError):
        srt.load_plan_cache(str(tmp_path / "missing.txt"))
    srt.clear_plan_cache()
    srt.save_plan_cache(str(dst))
    assert [l for l in dst.read_text().splitlines() if l and not l.startswith("#")] == ["srt_matmul_plan_cache v1"]
