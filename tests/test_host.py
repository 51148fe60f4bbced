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
