"""ctypes loader for libhiptensor_b200.so (the flat C ABI in include/hiptensor_b200.h)."""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libhiptensor_b200.so")

_lib = None

_vp, _i32p, _i64p = ctypes.c_void_p, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int64)
_u32, _u64, _int = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int

# name -> (restype, argtypes); the same list is what tests check against the header
SIGNATURES = {
    "htCreate": (_int, [ctypes.POINTER(_vp)]),
    "htDestroy": (_int, [_vp]),
    "htGetErrorString": (ctypes.c_char_p, [_int]),
    "htCreateTensorDescriptor": (_int, [_vp, ctypes.POINTER(_vp), _u32, _i64p, _i64p, _int, _int]),
    "htDestroyTensorDescriptor": (_int, [_vp]),
    "htGetAlignmentRequirement": (_int, [_vp, _vp, _vp, ctypes.POINTER(_u32)]),
    "htPermutation": (_int, [_vp, _vp, _vp, _vp, _i32p, _vp, _vp, _i32p, _int, _vp]),
    "htCreateContractionDescriptor": (_int, [_vp, ctypes.POINTER(_vp), _vp, _i32p, _u32, _vp, _i32p, _u32, _vp, _i32p,
                                             _u32, _vp, _i32p, _u32, _int]),
    "htDestroyContractionDescriptor": (_int, [_vp]),
    "htCreateContractionFind": (_int, [_vp, ctypes.POINTER(_vp), _int]),
    "htDestroyContractionFind": (_int, [_vp]),
    "htContractionGetWorkspaceSize": (_int, [_vp, _vp, _vp, _int, ctypes.POINTER(_u64)]),
    "htCreateContractionPlan": (_int, [_vp, ctypes.POINTER(_vp), _vp, _vp, _u64]),
    "htDestroyContractionPlan": (_int, [_vp]),
    "htContraction": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _vp]),
    "htReduction": (_int, [_vp, _vp, _vp, _vp, _i32p, _vp, _vp, _vp, _i32p, _vp, _vp, _i32p, _int, _int, _vp, _u64,
                           _vp]),
    "htReductionNoAlloc": (_int, [_vp, _vp, _vp, _vp, _i32p, _vp, _vp, _vp, _i32p, _vp, _vp, _i32p, _int, _int, _vp]),
    "htReductionGetWorkspaceSize": (_int, [_vp, _vp, _vp, _i32p, _vp, _vp, _i32p, _vp, _vp, _i32p, _int, _int,
                                           ctypes.POINTER(_u64)]),
    "htLoggerSetMask": (_int, [ctypes.c_int32]),
    "htLoggerOpenFile": (_int, [ctypes.c_char_p]),
    "htDescribePermutationPlan": (_int, [_u32, _i64p, _i32p, _i32p, _int, _int, ctypes.c_char_p, _u64]),
    "htDescribeReductionPlan": (_int, [_u32, _i64p, _i64p, _i32p, _u32, _i64p, _i64p, _i32p, _int, ctypes.c_char_p,
                                       _u64]),
    "htDescribeContractionPlan": (_int, [_u32, _i64p, _i64p, _i32p, _int, _u32, _i64p, _i64p, _i32p, _int, _u32,
                                         _i64p, _i64p, _i32p, _int, _int, _int, ctypes.c_char_p, _u64]),
    "htLastKernelName": (ctypes.c_char_p, []),
    "htGetDeviceStatus": (_int, [_vp, ctypes.POINTER(ctypes.c_int32)]),
    "htInjectDeviceStatus": (_int, [_vp, ctypes.c_int32]),
    "htKernelLaunchCount": (_u64, []),
    "htReloadSwitches": (None, []),
    "htReductionFinish": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _vp]),
}


def lib():
    """Loads the shared library; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libhiptensor_b200.so is missing: run `python -m hiptensor_b200.build` "
                              "(needs nvcc); this package has no other execution path")
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def i64(v):
    if v is None:
        return None
    return (ctypes.c_int64 * len(v))(*[int(x) for x in v])


def i32(v):
    if v is None:
        return None
    return (ctypes.c_int32 * len(v))(*[int(x) for x in v])
