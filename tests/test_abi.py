"""The C-ABI library: it loads, exports every symbol the header declares, keeps the reference's
descriptor layout, validates arguments before touching CUDA, and has no CPU fallback."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "srt_matmul_api.h")


def _declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(srt[A-Z]\w*)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import swiftrt_b200 as srt
    declared = _declared_symbols()
    assert declared, "no declarations found in the header"
    lib = ctypes.CDLL(srt.SO)
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert sorted(srt.EXPORTS) == declared


def test_library_exports_nothing_but_its_entry_points():
    """Every dynamic symbol the library defines is an srt* entry point: helpers and state stay
    internal, so they can neither collide with nor be interposed by a host program's symbols."""
    import subprocess
    import swiftrt_b200 as srt
    out = subprocess.run(["nm", "-D", "--defined-only", srt.SO], capture_output=True, text=True, check=True).stdout
    names = [line.split()[-1] for line in out.splitlines() if line.strip()]
    own = [n for n in names if not n.startswith("_") and not n.startswith("cuda") and not n.startswith("__")]
    leaked = [n for n in own if not n.startswith("srt")]
    assert not leaked, leaked
    assert sorted(n for n in own if n.startswith("srt")) == sorted(srt.EXPORTS)


@pytest.mark.parametrize("total,world,align", [(64, 8, 1), (65536, 8, 1), (16384, 8, 8), (10, 4, 1), (100, 8, 8), (3, 8, 1), (0, 2, 1)])
def test_shard_range_of_the_library_equals_the_host_mirror(total, world, align):
    """srtShardRange (C) and sharded.shard_range (Python) are one arithmetic; blocks are contiguous,
    cover everything once and start on multiples of `align`."""
    from swiftrt_b200 import _lib
    from swiftrt_b200.sharded import shard_range
    covered = 0
    for rank in range(world):
        lo, hi = ctypes.c_size_t(), ctypes.c_size_t()
        assert _lib.lib.srtShardRange(total, world, rank, align, ctypes.byref(lo), ctypes.byref(hi)) == 0
        assert (lo.value, hi.value) == shard_range(total, world, rank, align)
        assert lo.value == covered and (lo.value % align == 0 or lo.value == total)
        covered = hi.value
    assert covered == total
    lo, hi = ctypes.c_size_t(), ctypes.c_size_t()
    assert _lib.lib.srtShardRange(8, 2, 2, 1, ctypes.byref(lo), ctypes.byref(hi)) == 1


def test_descriptor_layout_matches_reference_struct():
    # srtTensorDescriptor: {int32 type; uint32 rank; int32 order; size_t count, spanCount; 3 pointers}
    # (Modules/SwiftRTCuda/tensor_api.h:70-87) -> 56 bytes, count at offset 16 on LP64
    from swiftrt_b200._lib import MatmulPlan, TensorDescriptor
    assert ctypes.sizeof(TensorDescriptor) == 56
    assert TensorDescriptor.count.offset == 16 and TensorDescriptor.shape.offset == 32
    assert TensorDescriptor.logicalStrides.offset == 48
    assert ctypes.sizeof(MatmulPlan) == 64


def test_enum_values_match_reference():
    import swiftrt_b200 as srt
    assert (srt.DataType.real32F, srt.DataType.real16F, srt.DataType.real16BF) == (0, 2, 14)
    assert (srt.Order.col, srt.Order.row) == (0, 1)
    names = ["sigmoid", "relu", "tanh", "clippedRelu", "elu", "identity"]      # FunctionProperties.swift:44-51
    assert [srt.ActivationType[n].value for n in names] == list(range(6))


def _desc(dtype, shape, strides=None):
    from swiftrt_b200._lib import TensorDescriptor
    sz = ctypes.c_size_t
    if strides is None:
        strides, acc = [], 1
        for d in reversed(shape):
            strides.insert(0, acc)
            acc *= d
    sh, st = (sz * len(shape))(*shape), (sz * len(shape))(*strides)
    n = 1
    for d in shape:
        n *= d
    d = TensorDescriptor(dtype, len(shape), 1, n, n, sh, st, st)
    d._keep = (sh, st)
    return d


FAKE = 0x10000   # non-null, never dereferenced: validation fails before any CUDA call


@pytest.mark.parametrize("a_shape,b_shape,o_shape,ta,tb,dt,code,needle", [
    ((3, 2), (3, 4), (3, 4), False, False, (0, 0, 0), 1, "inner dimensions"),
    ((3, 2), (2, 4), (3, 5), False, False, (0, 0, 0), 1, "does not match"),
    ((3, 2), (2, 4), (3, 4), False, False, (0, 14, 0), 1, "same element type"),
    ((3, 2), (2, 4), (3, 4), False, False, (1, 1, 1), 801, "not computed"),       # real64F
    ((3, 2), (2, 4), (3, 4), True, False, (0, 0, 0), 1, "inner dimensions"),
    ((2, 3, 2), (3, 2, 4), (2, 3, 4), False, False, (0, 0, 0), 1, "batch size"),
])
def test_argument_errors_are_reported_without_a_gpu(a_shape, b_shape, o_shape, ta, tb, dt, code, needle):
    from swiftrt_b200 import _lib
    da, db, do = _desc(dt[0], a_shape), _desc(dt[1], b_shape), _desc(dt[2], o_shape)
    rc = _lib.lib.srtMatmul(FAKE, ctypes.byref(da), ta, FAKE, ctypes.byref(db), tb, FAKE, ctypes.byref(do), None)
    assert rc == code
    assert needle in _lib.last_error()


def test_null_arguments_and_bad_bias_and_activation():
    from swiftrt_b200 import _lib
    da, db, do = _desc(0, (3, 2)), _desc(0, (2, 4)), _desc(0, (3, 4))
    assert _lib.lib.srtMatmul(None, ctypes.byref(da), False, FAKE, ctypes.byref(db), False, FAKE, ctypes.byref(do), None) == 1
    bad_bias = _desc(0, (5,))
    rc = _lib.lib.srtMatmulBiasActivation(FAKE, ctypes.byref(da), False, FAKE, ctypes.byref(db), False,
                                          FAKE, ctypes.byref(bad_bias), 1, FAKE, ctypes.byref(do), None)
    assert rc == 1 and "bias" in _lib.last_error()
    ok_bias = _desc(0, (4,))
    for act, code in ((3, 801), (4, 801), (99, 1)):        # clippedRelu, elu, unknown
        rc = _lib.lib.srtMatmulBiasActivation(FAKE, ctypes.byref(da), False, FAKE, ctypes.byref(db), False,
                                              FAKE, ctypes.byref(ok_bias), act, FAKE, ctypes.byref(do), None)
        assert rc == code
    assert _lib.lib.srtMatmulSetTuning(7, 0, 0, 0) == 1
    assert _lib.lib.srtMatmulSetTuning(0, 96, 0, 0) == 1
    assert _lib.lib.srtMatmulSetTuning(0, 0, 0, 0) == 0


def test_no_cpu_fallback_when_no_device_is_present():
    """With valid arguments and no usable GPU the call must fail loudly, not compute elsewhere."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from swiftrt_b200 import _lib
    da, db, do = _desc(0, (3, 2)), _desc(0, (2, 4)), _desc(0, (3, 4))
    rc = _lib.lib.srtMatmul(FAKE, ctypes.byref(da), False, FAKE, ctypes.byref(db), False, FAKE, ctypes.byref(do), None)
    assert rc != 0
    assert _lib.lib.srtMatmulLaunchCount() == 0


def test_product_code_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "swiftrt_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "liboracle" not in text and "import oracle" not in text and "from oracle" not in text, f
