"""ctypes binding of the CPU oracle (oracle/oracle.cpp).

Test infrastructure only: imported by tests/, by __graft_entry__.smoke() and by the
cpu_baseline / reference legs of bench.py. The shipped package never imports it.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

# hipDataType / cudaDataType codes
F32, F64, F16, BF16 = 0, 1, 2, 14
# hiptensorComputeType_t
COMPUTE_16F, COMPUTE_32F, COMPUTE_64F, COMPUTE_16BF = 1, 4, 16, 1024
# hiptensorOperator_t
OP_IDENTITY, OP_SQRT, OP_ADD, OP_MUL, OP_MAX, OP_MIN = 1, 2, 3, 5, 6, 7

_NP = {F32: np.float32, F64: np.float64, F16: np.float16, BF16: np.uint16}


def build(force=False):
    """Compile oracle.cpp with g++ (seconds)."""
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "liboracle.so"])
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        L = ctypes.CDLL(_SO)
        L.orc_max_rel_error.restype = ctypes.c_double
        L.orc_max_rel_error.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64]
        L.orc_fill_uniform.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_uint32]
        L.orc_fill_normal.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_uint32,
                                      ctypes.c_float]
        _lib = L
    return _lib


def np_dtype(dt):
    return _NP[dt]


def _i64(v):
    return (ctypes.c_int64 * len(v))(*[int(x) for x in v])


def _i32(v):
    return (ctypes.c_int32 * len(v))(*[int(x) for x in v])


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data) if a is not None else ctypes.c_void_p(0)


def scalar_buffer(value, compute_type):
    """Host scalar laid out as the given compute type (what alpha/beta must point to)."""
    if compute_type == COMPUTE_32F:
        return np.array([value], dtype=np.float32)
    if compute_type == COMPUTE_64F:
        return np.array([value], dtype=np.float64)
    if compute_type == COMPUTE_16F:
        return np.array([value], dtype=np.float16)
    if compute_type == COMPUTE_16BF:
        return f32_to_bf16_bits(np.array([value], dtype=np.float32))
    raise ValueError(compute_type)


def f32_to_bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b):
    return (b.astype(np.uint32) << 16).view(np.float32)


def to_f64(a, dt):
    """Any oracle array -> float64 numpy array."""
    if dt == BF16:
        return bf16_bits_to_f32(a).astype(np.float64)
    return a.astype(np.float64)


def fill_uniform(n, dt, seed):
    """The reference harness' generator (test/device/common.hpp:68-108)."""
    out = np.empty(int(n), dtype=_NP[dt])
    lib().orc_fill_uniform(_ptr(out), dt, int(n), int(seed) & 0xFFFFFFFF)
    return out


def fill_normal(n, dt, seed, sigma):
    out = np.empty(int(n), dtype=_NP[dt])
    lib().orc_fill_normal(_ptr(out), dt, int(n), int(seed) & 0xFFFFFFFF, float(sigma))
    return out


def contraction(alpha, A, lenA, strA, modeA, typeA, B, lenB, strB, modeB, typeB, beta, C, D, lenD, strD,
                modeD, typeD, compute_type, sample=None, nthreads=0):
    """D (numpy, modified in place) = alpha*A*B + beta*C by the reference's CPU algorithm."""
    a = scalar_buffer(alpha, compute_type)
    b = scalar_buffer(beta, compute_type)
    smp = None
    ns = 0
    if sample is not None:
        smp = np.ascontiguousarray(sample, dtype=np.int64)
        ns = smp.size
    rc = lib().orc_contraction(
        _ptr(a), _ptr(A), len(lenA), _i64(lenA), _i64(strA), _i32(modeA), typeA,
        _ptr(B), len(lenB), _i64(lenB), _i64(strB), _i32(modeB), typeB,
        _ptr(b), _ptr(C), _ptr(D), len(lenD), _i64(lenD), _i64(strD), _i32(modeD), typeD,
        compute_type, _ptr(smp), ctypes.c_int64(ns), int(nthreads))
    if rc != 0:
        raise RuntimeError("oracle contraction rejected the problem (code %d)" % rc)
    return D


C32F, C64F = 4, 5
COMPUTE_C32F, COMPUTE_C64F = 2048, 4096


def contraction_complex(alpha, A, lenA, strA, modeA, B, lenB, strB, modeB, beta, C, D, lenD, strD, modeD, dtype,
                        nthreads=0):
    """Complex contraction by the reference's CPU algorithm; A, B, C, D are numpy complex64 / complex128
    arrays (dtype C32F / C64F), alpha and beta Python complex numbers."""
    ct = np.complex64 if dtype == C32F else np.complex128
    a = np.array([alpha], dtype=ct)
    b = np.array([beta], dtype=ct)
    rc = lib().orc_contraction_complex(
        _ptr(a), _ptr(A), len(lenA), _i64(lenA), _i64(strA), _i32(modeA),
        _ptr(B), len(lenB), _i64(lenB), _i64(strB), _i32(modeB),
        _ptr(b), _ptr(C), _ptr(D), len(lenD), _i64(lenD), _i64(strD), _i32(modeD), int(dtype), int(nthreads))
    if rc != 0:
        raise RuntimeError("oracle complex contraction rejected the problem (code %d)" % rc)
    return D


def permutation(alpha, type_scalar, A, lenA, modeA, typeA, B, modeB, typeB, opA=OP_IDENTITY, opB=OP_IDENTITY,
                nthreads=1):
    a = np.array([alpha], dtype=np.float32 if type_scalar == F32 else np.float16)
    rc = lib().orc_permutation(_ptr(a), type_scalar, _ptr(A), len(lenA), _i64(lenA), _i32(modeA), typeA, opA,
                               _ptr(B), _i32(modeB), typeB, opB, int(nthreads))
    if rc != 0:
        raise RuntimeError("oracle permutation rejected the problem (code %d)" % rc)
    return B


def reduction(alpha, A, lenA, strA, modeA, typeA, beta, C, D, lenD, strD, modeD, typeD, op, compute_type,
              nthreads=0):
    a = scalar_buffer(alpha, compute_type)
    b = scalar_buffer(beta, compute_type)
    rc = lib().orc_reduction(_ptr(a), _ptr(A), len(lenA), _i64(lenA), _i64(strA), _i32(modeA), typeA,
                             _ptr(b), _ptr(C), _ptr(D), len(lenD), _i64(lenD), _i64(strD), _i32(modeD), typeD,
                             op, compute_type, int(nthreads))
    if rc != 0:
        raise RuntimeError("oracle reduction rejected the problem (code %d)" % rc)
    return D


def max_rel_error(dev, host, dt):
    """max |d-h|/(|d|+|h|+1); -1.0 when a NaN/Inf is met (reference: test/utils.hpp:285-383)."""
    assert dev.size == host.size
    return float(lib().orc_max_rel_error(_ptr(np.ascontiguousarray(dev)), _ptr(np.ascontiguousarray(host)),
                                         dt, dev.size))


def packed_strides(lens, first_fastest):
    """util.hpp:45-69 stridesFromLengths: first_fastest=False is the NULL-stride default."""
    n = len(lens)
    st = [1] * n
    if first_fastest:
        for i in range(1, n):
            st[i] = st[i - 1] * lens[i - 1]
    else:
        for i in range(n - 2, -1, -1):
            st[i] = st[i + 1] * lens[i + 1]
    return st
