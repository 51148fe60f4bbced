"""ctypes binding of libsrt_b200.so (the C ABI declared in include/srt_matmul_api.h).

There is no fallback: if the compiled CUDA library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os

PKG = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(PKG, "libsrt_b200.so")

cudaSuccess = 0
cudaErrorInvalidValue = 1
cudaErrorNotSupported = 801


class TensorDescriptor(ctypes.Structure):
    """Field-for-field srtTensorDescriptor (Modules/SwiftRTCuda/tensor_api.h:70-87)."""
    _fields_ = [("type", ctypes.c_int),
                ("rank", ctypes.c_uint32),
                ("order", ctypes.c_int),
                ("count", ctypes.c_size_t),
                ("spanCount", ctypes.c_size_t),
                ("shape", ctypes.POINTER(ctypes.c_size_t)),
                ("strides", ctypes.POINTER(ctypes.c_size_t)),
                ("logicalStrides", ctypes.POINTER(ctypes.c_size_t))]


class MatmulPlan(ctypes.Structure):
    """srtMatmulPlan."""
    _fields_ = [("kernel", ctypes.c_int32),
                ("tileM", ctypes.c_int32), ("tileN", ctypes.c_int32), ("tileK", ctypes.c_int32),
                ("stages", ctypes.c_int32), ("ctas", ctypes.c_int32), ("tiles", ctypes.c_int32),
                ("swapped", ctypes.c_int32), ("aMajor", ctypes.c_int32), ("bMajor", ctypes.c_int32),
                ("fp32Split", ctypes.c_int32), ("splitK", ctypes.c_int32),
                ("workspaceBytes", ctypes.c_size_t), ("dynamicSmemBytes", ctypes.c_size_t)]


# every symbol include/srt_matmul_api.h declares
EXPORTS = ["srtMatmul", "srtMatmulBiasActivation", "srtMatmulQueryPlan", "srtMatmulSetTuning", "srtMatmulSetSplitK", "srtMatmulNoAlloc", "srtBiasActivationBackward",
           "srtMatmulCheckStatus", "srtMatmulLaunchCount", "srtMatmulGetLastErrorString",
           "srtMatmulAllGather", "srtPeerMemAlloc", "srtPeerMemOpen", "srtPeerMemClose", "srtPeerMemFree", "srtLstmCell", "srtRnnCell",
           "srtMatmulAllGatherMulticast", "srtMatmulTune", "srtMatmulPlanCacheSave", "srtMatmulPlanCacheLoad", "srtMatmulPlanCacheClear",
           "srtActivationForward", "srtMatmulReleaseWorkspaces", "srtGruCell", "srtShardRange", "srtMatmulSharded",
           "srtMatmulShardedDevices", "srtMatmulSetWaitLimit", "srtLstmCellFused", "srtLstmInterleaveGates", "srtPeerSignal", "srtPeerWait", "srtMulticastAlloc", "srtMulticastFree",
           "srtMatrixTransform", "srtMatrixLayoutLeadingDimension", "srtMatrixLayoutElementCount"]

if not os.path.exists(SO):
    raise ImportError(
        f"{SO} is missing: the CUDA library has not been built. Run "
        "`python swiftrt_b200/build.py` (needs nvcc); there is no CPU or PyTorch fallback.")

lib = ctypes.CDLL(SO)

_D = ctypes.POINTER(TensorDescriptor)
_P = ctypes.c_void_p
lib.srtMatmul.restype = ctypes.c_int
lib.srtMatmul.argtypes = [_P, _D, ctypes.c_bool, _P, _D, ctypes.c_bool, _P, _D, _P]
lib.srtBiasActivationBackward.restype = ctypes.c_int
lib.srtBiasActivationBackward.argtypes = [_P, _D, _P, _D, ctypes.c_int, _P, _D, _P, _D, _P]
lib.srtMatmulNoAlloc.restype = ctypes.c_int
lib.srtMatmulNoAlloc.argtypes = [_P, _D, ctypes.c_bool, _P, _D, ctypes.c_bool, _P, _D, _P]
lib.srtMatmulBiasActivation.restype = ctypes.c_int
lib.srtMatmulBiasActivation.argtypes = [_P, _D, ctypes.c_bool, _P, _D, ctypes.c_bool, _P, _D, ctypes.c_int, _P, _D, _P]
lib.srtMatmulQueryPlan.restype = ctypes.c_int
lib.srtMatmulQueryPlan.argtypes = [_P, _D, ctypes.c_bool, _P, _D, ctypes.c_bool, _P, _D, ctypes.POINTER(MatmulPlan)]
lib.srtMatmulSetTuning.restype = ctypes.c_int
lib.srtMatmulSetTuning.argtypes = [ctypes.c_int32] * 4
lib.srtMatmulSetSplitK.restype = ctypes.c_int
lib.srtMatmulSetSplitK.argtypes = [ctypes.c_int32]
lib.srtMatmulCheckStatus.restype = ctypes.c_int
lib.srtMatmulCheckStatus.argtypes = [_P, ctypes.POINTER(ctypes.c_uint32)]
lib.srtMatmulLaunchCount.restype = ctypes.c_uint64
lib.srtMatmulLaunchCount.argtypes = []
lib.srtMatmulGetLastErrorString.restype = ctypes.c_char_p
lib.srtMatmulGetLastErrorString.argtypes = []



class PeerMemHandle(ctypes.Structure):
    """srtPeerMemHandle (64 opaque bytes)."""
    _fields_ = [("bytes", ctypes.c_ubyte * 64)]


lib.srtMatmulAllGather.restype = ctypes.c_int
lib.srtMatmulAllGather.argtypes = [_P, _D, ctypes.c_bool, _P, _D, ctypes.c_bool, _P, _D, ctypes.c_int, _P, _D,
                                   ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p), _P]
lib.srtMatmulAllGatherMulticast.restype = ctypes.c_int
lib.srtMatmulAllGatherMulticast.argtypes = [_P, _D, ctypes.c_bool, _P, _D, ctypes.c_bool, _P, _D, ctypes.c_int, _P, _D, _P, _P]
lib.srtPeerMemAlloc.restype = ctypes.c_int
lib.srtPeerMemAlloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(PeerMemHandle)]
lib.srtPeerMemOpen.restype = ctypes.c_int
lib.srtPeerMemOpen.argtypes = [ctypes.POINTER(PeerMemHandle), ctypes.POINTER(ctypes.c_void_p)]
lib.srtPeerSignal.restype = ctypes.c_int
lib.srtPeerSignal.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64, _P]
lib.srtPeerWait.restype = ctypes.c_int
lib.srtPeerWait.argtypes = [_P, ctypes.c_int32, ctypes.c_int32, ctypes.c_uint64, ctypes.c_uint64, _P]
lib.srtPeerMemClose.restype = ctypes.c_int
lib.srtPeerMemClose.argtypes = [_P]
lib.srtPeerMemFree.restype = ctypes.c_int
lib.srtPeerMemFree.argtypes = [_P]

lib.srtLstmCell.restype = ctypes.c_int
lib.srtLstmCell.argtypes = [_P, _D] * 7 + [_P]
lib.srtLstmCellFused.restype = ctypes.c_int
lib.srtLstmCellFused.argtypes = [_P, _D] * 7 + [_P]
lib.srtLstmInterleaveGates.restype = ctypes.c_int
lib.srtLstmInterleaveGates.argtypes = [_P, _D, _P, _D, _P]
lib.srtRnnCell.restype = ctypes.c_int
lib.srtRnnCell.argtypes = [_P, _D] * 5 + [_P]
lib.srtMatmulTune.restype = ctypes.c_int
lib.srtMatmulTune.argtypes = [_P, _D, ctypes.c_bool, _P, _D, ctypes.c_bool, _P, _D, ctypes.c_int, _P, _D, _P,
                              ctypes.POINTER(MatmulPlan), ctypes.POINTER(ctypes.c_float)]
lib.srtMatmulPlanCacheSave.restype = ctypes.c_int
lib.srtMatmulPlanCacheSave.argtypes = [ctypes.c_char_p]
lib.srtMatmulPlanCacheLoad.restype = ctypes.c_int
lib.srtMatmulPlanCacheLoad.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int32)]
lib.srtMatmulPlanCacheClear.restype = ctypes.c_int
lib.srtMatmulPlanCacheClear.argtypes = []


class MatrixLayoutStruct(ctypes.Structure):
    """srtMatrixLayout of include/srt_matmul_api.h."""
    _fields_ = [("type", ctypes.c_int), ("order", ctypes.c_int), ("rows", ctypes.c_uint64), ("cols", ctypes.c_uint64),
                ("leadingDimension", ctypes.c_int64), ("batchCount", ctypes.c_int32), ("batchStride", ctypes.c_int64)]


lib.srtMatrixTransform.restype = ctypes.c_int
lib.srtMatrixTransform.argtypes = [ctypes.POINTER(ctypes.c_float), _P, ctypes.POINTER(MatrixLayoutStruct), ctypes.c_bool,
                                   ctypes.POINTER(ctypes.c_float), _P, ctypes.POINTER(MatrixLayoutStruct), ctypes.c_bool,
                                   _P, ctypes.POINTER(MatrixLayoutStruct), _P]
lib.srtMatrixLayoutLeadingDimension.restype = ctypes.c_uint64
lib.srtMatrixLayoutLeadingDimension.argtypes = [ctypes.c_int, ctypes.c_uint64, ctypes.c_uint64]
lib.srtMatrixLayoutElementCount.restype = ctypes.c_uint64
lib.srtMatrixLayoutElementCount.argtypes = [ctypes.c_int, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64]
lib.srtActivationForward.restype = ctypes.c_int
lib.srtActivationForward.argtypes = [_P, _D, ctypes.c_int, _P, _D, _P]
lib.srtMatmulReleaseWorkspaces.restype = ctypes.c_int
lib.srtMatmulReleaseWorkspaces.argtypes = [ctypes.c_bool]
lib.srtGruCell.restype = ctypes.c_int
lib.srtGruCell.argtypes = [_P, _D] * 7 + [_P]
lib.srtShardRange.restype = ctypes.c_int
lib.srtShardRange.argtypes = [ctypes.c_size_t, ctypes.c_int32, ctypes.c_int32, ctypes.c_size_t,
                              ctypes.POINTER(ctypes.c_size_t), ctypes.POINTER(ctypes.c_size_t)]
lib.srtMatmulSharded.restype = ctypes.c_int
lib.srtMatmulSharded.argtypes = [ctypes.c_int, ctypes.c_int32, ctypes.c_int32, _P, _D, ctypes.c_bool, _P, _D, ctypes.c_bool,
                                 _P, _D, ctypes.c_int, _P, _D, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p), _P, _P]
lib.srtMatmulShardedDevices.restype = ctypes.c_int
lib.srtMatmulShardedDevices.argtypes = [ctypes.c_int, ctypes.c_int32, ctypes.POINTER(ctypes.c_void_p),
                                        ctypes.POINTER(ctypes.c_void_p), _D, ctypes.c_bool,
                                        ctypes.POINTER(ctypes.c_void_p), _D, ctypes.c_bool,
                                        ctypes.POINTER(ctypes.c_void_p), _D, ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_void_p), _D, ctypes.c_bool, _P]
lib.srtMulticastAlloc.restype = ctypes.c_int
lib.srtMulticastAlloc.argtypes = [ctypes.c_int32, ctypes.POINTER(ctypes.c_int32), ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p),
                                  ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p)]
lib.srtMulticastFree.restype = ctypes.c_int
lib.srtMulticastFree.argtypes = [_P]
lib.srtMatmulSetWaitLimit.restype = ctypes.c_int
lib.srtMatmulSetWaitLimit.argtypes = [ctypes.c_uint64]


def last_error() -> str:
    return lib.srtMatmulGetLastErrorString().decode()
