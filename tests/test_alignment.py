"""hiptensorGetAlignmentRequirement: the largest power of two in [element size, 16] that divides the address
(reference: library/src/hiptensor.cpp:256-321). Pure host arithmetic: the function reads neither the handle's
contents nor the pointer's target, so these checks need no GPU (a zeroed block stands in for the handle)."""
import ctypes

import pytest


@pytest.fixture(scope="module")
def L():
    from hiptensor_b200 import _lib, build

    build.build()
    return _lib.lib()


def _desc(L, handle, dtype):
    from hiptensor_b200 import _lib

    d = ctypes.c_void_p(0)
    assert L.htCreateTensorDescriptor(handle, ctypes.byref(d), 2, _lib.i64([4, 4]), None, dtype, 1) == 0
    return d


def test_alignment_values(L):
    import hiptensor_b200 as ht

    handle = ctypes.cast(ctypes.create_string_buffer(512), ctypes.c_void_p)
    out = ctypes.c_uint32(99)
    base = 0x7F0000001000  # 4 KiB aligned
    cases = [
        (ht.R_32F, base, 16), (ht.R_32F, base + 8, 8), (ht.R_32F, base + 4, 4), (ht.R_32F, base + 12, 4),
        (ht.R_16F, base, 16), (ht.R_16F, base + 2, 2), (ht.R_16F, base + 4, 4), (ht.R_16F, base + 6, 2),
        (ht.R_16BF, base + 2, 2), (ht.R_64F, base, 16), (ht.R_64F, base + 8, 8), (ht.C_32F, base + 8, 8),
        (ht.C_64F, base, 16),
    ]
    for dtype, addr, want in cases:
        d = _desc(L, handle, dtype)
        assert L.htGetAlignmentRequirement(handle, ctypes.c_void_p(addr), d, ctypes.byref(out)) == 0
        assert out.value == want, (dtype, hex(addr), out.value)
        L.htDestroyTensorDescriptor(d)


def test_misaligned_pointer_is_invalid(L):
    import hiptensor_b200 as ht

    handle = ctypes.cast(ctypes.create_string_buffer(512), ctypes.c_void_p)
    out = ctypes.c_uint32(99)
    for dtype, addr in [(ht.R_32F, 0x1001), (ht.R_32F, 0x1002), (ht.R_16F, 0x1001), (ht.R_64F, 0x1004),
                        (ht.C_64F, 0x1008)]:
        d = _desc(L, handle, dtype)
        assert L.htGetAlignmentRequirement(handle, ctypes.c_void_p(addr), d, ctypes.byref(out)) == ht.STATUS_INVALID_VALUE
        assert out.value == 0
        L.htDestroyTensorDescriptor(d)


def test_null_arguments(L):
    import hiptensor_b200 as ht

    handle = ctypes.cast(ctypes.create_string_buffer(512), ctypes.c_void_p)
    out = ctypes.c_uint32(0)
    d = _desc(L, handle, ht.R_32F)
    assert L.htGetAlignmentRequirement(None, ctypes.c_void_p(0x1000), d, ctypes.byref(out)) == ht.STATUS_NOT_INITIALIZED
    assert L.htGetAlignmentRequirement(handle, ctypes.c_void_p(0x1000), None, ctypes.byref(out)) == ht.STATUS_NOT_INITIALIZED
    assert L.htGetAlignmentRequirement(handle, ctypes.c_void_p(0x1000), d, None) == ht.STATUS_INVALID_VALUE
    L.htDestroyTensorDescriptor(d)
