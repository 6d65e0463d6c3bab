"""Python mirror of the hipTensor entry points (reference: library/include/hiptensor/hiptensor.hpp).

Data arguments are device pointers: pass a torch CUDA tensor, an int address or None.
alpha/beta are Python numbers; they are laid out as the type the reference expects
(typeScalar for permutation, the compute type for contraction and reduction).
Every non-zero status raises HiptensorError.
"""
import ctypes
import struct

from . import _lib

__all__ = [
    "HiptensorError", "Handle", "TensorDescriptor",
    "R_32F", "R_64F", "R_16F", "R_16BF", "C_32F", "C_64F",
    "COMPUTE_16F", "COMPUTE_32F", "COMPUTE_64F", "COMPUTE_16BF", "COMPUTE_C32F", "COMPUTE_C64F",
    "OP_IDENTITY", "OP_SQRT", "OP_ADD", "OP_MUL", "OP_MAX", "OP_MIN",
    "ALGO_DEFAULT", "ALGO_DEFAULT_PATIENT", "ALGO_ACTOR_CRITIC",
    "WORKSPACE_MIN", "WORKSPACE_RECOMMENDED", "WORKSPACE_MAX",
    "STATUS_SUCCESS", "STATUS_NOT_INITIALIZED", "STATUS_INVALID_VALUE", "STATUS_ARCH_MISMATCH",
    "STATUS_INTERNAL_ERROR", "STATUS_NOT_SUPPORTED", "STATUS_HIP_ERROR", "STATUS_INSUFFICIENT_WORKSPACE",
    "STATUS_EXECUTION_FAILED",
    "error_string", "last_kernel_name", "kernel_launch_count", "reload_switches",
    "describe_permutation_plan", "describe_reduction_plan", "describe_contraction_plan", "dtype_size",
]

# hipDataType (hiptensor_types.hpp uses hipDataType; values equal cudaDataType)
R_32F, R_64F, R_16F, R_16BF = 0, 1, 2, 14
C_32F, C_64F = 4, 5
# hiptensorComputeType_t (hiptensor_types.hpp:74-99)
COMPUTE_16F, COMPUTE_32F, COMPUTE_64F, COMPUTE_16BF = 1, 4, 16, 1024
COMPUTE_C32F, COMPUTE_C64F = 2048, 4096
# hiptensorOperator_t (hiptensor_types.hpp:102-124)
OP_IDENTITY, OP_SQRT, OP_ADD, OP_MUL, OP_MAX, OP_MIN = 1, 2, 3, 5, 6, 7
# hiptensorAlgo_t (hiptensor_types.hpp:127-136)
ALGO_DEFAULT, ALGO_DEFAULT_PATIENT, ALGO_ACTOR_CRITIC = -1, -6, -8
# hiptensorWorksizePreference_t (hiptensor_types.hpp:139-148)
WORKSPACE_MIN, WORKSPACE_RECOMMENDED, WORKSPACE_MAX = 1, 2, 3
# hiptensorStatus_t (hiptensor_types.hpp:42-71)
STATUS_SUCCESS, STATUS_NOT_INITIALIZED, STATUS_INVALID_VALUE, STATUS_ARCH_MISMATCH = 0, 1, 7, 8
STATUS_INTERNAL_ERROR, STATUS_NOT_SUPPORTED, STATUS_HIP_ERROR, STATUS_INSUFFICIENT_WORKSPACE = 14, 15, 18, 19
STATUS_EXECUTION_FAILED = 13

_DTYPE_SIZE = {R_32F: 4, R_64F: 8, R_16F: 2, R_16BF: 2, C_32F: 8, C_64F: 16}


def dtype_size(dt):
    return _DTYPE_SIZE[dt]


def error_string(status):
    return _lib.lib().htGetErrorString(int(status)).decode()


class HiptensorError(RuntimeError):
    def __init__(self, status, where):
        self.status = int(status)
        super().__init__("%s failed: %s (%d)" % (where, error_string(status), status))


def _check(status, where):
    if status != 0:
        raise HiptensorError(status, where)


def _ptr(x):
    if x is None:
        return ctypes.c_void_p(0)
    if isinstance(x, int):
        return ctypes.c_void_p(x)
    return ctypes.c_void_p(int(x.data_ptr()))


def _f32_to_bf16_bits(v):
    u = struct.unpack("<I", struct.pack("<f", float(v)))[0]
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF


def _scalar_for_compute(value, compute_type):
    """Host buffer holding `value` as the given compute type."""
    if compute_type == COMPUTE_32F:
        return ctypes.create_string_buffer(struct.pack("<f", float(value)), 8)
    if compute_type == COMPUTE_64F:
        return ctypes.create_string_buffer(struct.pack("<d", float(value)), 8)
    if compute_type == COMPUTE_16F:
        return ctypes.create_string_buffer(struct.pack("<e", float(value)), 8)
    if compute_type == COMPUTE_16BF:
        return ctypes.create_string_buffer(struct.pack("<H", _f32_to_bf16_bits(value)), 8)
    if compute_type == COMPUTE_C32F:  # hipFloatComplex
        v = complex(value)
        return ctypes.create_string_buffer(struct.pack("<ff", v.real, v.imag), 8)
    if compute_type == COMPUTE_C64F:  # hipDoubleComplex
        v = complex(value)
        return ctypes.create_string_buffer(struct.pack("<dd", v.real, v.imag), 16)
    raise HiptensorError(STATUS_NOT_SUPPORTED, "scalar conversion")


def _stream_ptr(stream):
    if stream is None:
        return ctypes.c_void_p(0)
    if isinstance(stream, int):
        return ctypes.c_void_p(stream)
    return ctypes.c_void_p(int(stream.cuda_stream))


class TensorDescriptor:
    """hiptensorTensorDescriptor_t, made by Handle.tensor_descriptor (hiptensorInitTensorDescriptor)."""

    def __init__(self, ptr, lens, dtype):
        self._p = ptr
        self.lens = list(lens)
        self.dtype = dtype

    def __del__(self):
        try:
            if self._p:
                _lib.lib().htDestroyTensorDescriptor(self._p)
        except Exception:
            pass


class _Owned:
    def __init__(self, ptr, destroy):
        self._p = ptr
        self._destroy = destroy

    def __del__(self):
        try:
            if self._p:
                getattr(_lib.lib(), self._destroy)(self._p)
        except Exception:
            pass


class Handle:
    """hiptensorHandle_t bound to the CUDA device current at construction (hiptensorCreate)."""

    def __init__(self):
        self._L = _lib.lib()
        h = ctypes.c_void_p(0)
        _check(self._L.htCreate(ctypes.byref(h)), "hiptensorCreate")
        self._h = h

    def destroy(self):
        if self._h:
            self._L.htDestroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    # hiptensorInitTensorDescriptor: strides=None means packed with the LAST mode fastest
    def tensor_descriptor(self, lens, strides=None, dtype=R_32F, unary_op=OP_IDENTITY):
        d = ctypes.c_void_p(0)
        _check(self._L.htCreateTensorDescriptor(self._h, ctypes.byref(d), len(lens), _lib.i64(lens),
                                                _lib.i64(strides), int(dtype), int(unary_op)),
               "hiptensorInitTensorDescriptor")
        return TensorDescriptor(d, lens, dtype)

    def alignment_requirement(self, ptr, desc):
        out = ctypes.c_uint32(0)
        _check(self._L.htGetAlignmentRequirement(self._h, _ptr(ptr), desc._p, ctypes.byref(out)),
               "hiptensorGetAlignmentRequirement")
        return out.value

    # hiptensorPermutation: B[modeB] = opB(alpha * opA(A[modeA]))
    def permutation(self, alpha, A, descA, modeA, B, descB, modeB, type_scalar=R_32F, stream=None):
        if type_scalar == R_32F:
            a = ctypes.create_string_buffer(struct.pack("<f", float(alpha)), 8)
        elif type_scalar == R_16F:
            a = ctypes.create_string_buffer(struct.pack("<e", float(alpha)), 8)
        else:
            a = ctypes.create_string_buffer(8)  # rejected by the library with NOT_SUPPORTED
        _check(self._L.htPermutation(self._h, a, _ptr(A), descA._p, _lib.i32(modeA), _ptr(B), descB._p,
                                     _lib.i32(modeB), int(type_scalar), _stream_ptr(stream)), "hiptensorPermutation")

    # hiptensorReduction: D = alpha * reduce(A) + beta * C
    def reduction(self, alpha, A, descA, modeA, beta, C, descC, modeC, D, descD, modeD, op_reduce, type_compute,
                  workspace=None, workspace_size=0, stream=None):
        a = _scalar_for_compute(alpha, type_compute)
        b = _scalar_for_compute(beta, type_compute)
        _check(self._L.htReduction(self._h, a, _ptr(A), descA._p, _lib.i32(modeA), b, _ptr(C), descC._p,
                                   _lib.i32(modeC), _ptr(D), descD._p, _lib.i32(modeD), int(op_reduce),
                                   int(type_compute), _ptr(workspace), int(workspace_size), _stream_ptr(stream)),
               "hiptensorReduction")

    def device_status(self):
        """The handle's device status word: 0, or the code left by a kernel whose bounded device-side wait ran out."""
        out = ctypes.c_int32(0)
        _check(self._L.htGetDeviceStatus(self._h, ctypes.byref(out)), "htGetDeviceStatus")
        return out.value

    def reduction_no_alloc(self, alpha, A, descA, modeA, beta, C, descC, modeC, D, descD, modeD, op_reduce,
                           type_compute, stream=None):
        """htReductionNoAlloc: the same reduction for callers that may not allocate device memory (hosts
        that own the device heap, latency-critical loops, services with an allocation ban after start-up). Scratch is an 8 KiB array inside
        the library, shared by all calls on the device: do not overlap two such calls on one device; a
        reduction of long contiguous rows that needs more raises STATUS_INSUFFICIENT_WORKSPACE (other plans use the
        slices that fit, or one pass). The first call per device does a
        one-time address lookup and belongs outside stream capture."""
        a = _scalar_for_compute(alpha, type_compute)
        b = _scalar_for_compute(beta, type_compute)
        _check(self._L.htReductionNoAlloc(self._h, a, _ptr(A), descA._p, _lib.i32(modeA), b, _ptr(C), descC._p,
                                          _lib.i32(modeC), _ptr(D), descD._p, _lib.i32(modeD), int(op_reduce),
                                          int(type_compute), _stream_ptr(stream)), "htReductionNoAlloc")

    def reduction_finish(self, alpha, partial, beta, C, D, descD, type_compute, stream=None):
        """htReductionFinish: D = alpha * partial + beta * C over descD's layout. `partial` holds the results of
        per-device reductions (alpha 1, beta 0) of a reduced mode that was split over devices, already combined
        across devices by one all-reduce with the reduction's operator."""
        a = _scalar_for_compute(alpha, type_compute)
        b = _scalar_for_compute(beta, type_compute)
        _check(self._L.htReductionFinish(self._h, a, _ptr(partial), b, _ptr(C), _ptr(D), descD._p, int(type_compute),
                                         _stream_ptr(stream)), "htReductionFinish")

    def reduction_workspace_size(self, A, descA, modeA, C, descC, modeC, D, descD, modeD, op_reduce, type_compute):
        out = ctypes.c_uint64(0)
        _check(self._L.htReductionGetWorkspaceSize(self._h, _ptr(A), descA._p, _lib.i32(modeA), _ptr(C), descC._p,
                                                   _lib.i32(modeC), _ptr(D), descD._p, _lib.i32(modeD),
                                                   int(op_reduce), int(type_compute), ctypes.byref(out)),
               "hiptensorReductionGetWorkspaceSize")
        return out.value

    # hiptensorInitContractionDescriptor: descC=None selects D = alpha*A*B
    def contraction_descriptor(self, descA, modeA, descB, modeB, descC, modeC, descD, modeD, type_compute,
                               align=(16, 16, 16, 16)):
        d = ctypes.c_void_p(0)
        _check(self._L.htCreateContractionDescriptor(
            self._h, ctypes.byref(d), descA._p, _lib.i32(modeA), align[0], descB._p, _lib.i32(modeB), align[1],
            descC._p if descC is not None else None, _lib.i32(modeC) if modeC is not None else None, align[2],
            descD._p, _lib.i32(modeD), align[3], int(type_compute)), "hiptensorInitContractionDescriptor")
        o = _Owned(d, "htDestroyContractionDescriptor")
        o.type_compute = type_compute
        o.keep = (descA, descB, descC, descD)
        return o

    def contraction_find(self, algo=ALGO_DEFAULT):
        f = ctypes.c_void_p(0)
        _check(self._L.htCreateContractionFind(self._h, ctypes.byref(f), int(algo)), "hiptensorInitContractionFind")
        return _Owned(f, "htDestroyContractionFind")

    def contraction_workspace_size(self, desc, find, pref=WORKSPACE_RECOMMENDED):
        out = ctypes.c_uint64(0)
        _check(self._L.htContractionGetWorkspaceSize(self._h, desc._p, find._p, int(pref), ctypes.byref(out)),
               "hiptensorContractionGetWorkspaceSize")
        return out.value

    def contraction_plan(self, desc, find, workspace_size=0):
        p = ctypes.c_void_p(0)
        _check(self._L.htCreateContractionPlan(self._h, ctypes.byref(p), desc._p, find._p, int(workspace_size)),
               "hiptensorInitContractionPlan")
        o = _Owned(p, "htDestroyContractionPlan")
        o.type_compute = desc.type_compute
        return o

    # hiptensorContraction: D = alpha*A*B + beta*C, alpha/beta typed by the plan's compute type
    def contraction(self, plan, alpha, A, B, beta, C, D, workspace=None, workspace_size=0, stream=None):
        a = _scalar_for_compute(alpha, plan.type_compute)
        b = _scalar_for_compute(beta, plan.type_compute)
        _check(self._L.htContraction(self._h, plan._p, a, _ptr(A), _ptr(B), b, _ptr(C), _ptr(D), _ptr(workspace),
                                     int(workspace_size), _stream_ptr(stream)), "hiptensorContraction")


def last_kernel_name():
    return _lib.lib().htLastKernelName().decode()


def reload_switches():
    """Re-reads the HTB_* variant switches from the environment (the library reads them once when loaded)."""
    _lib.lib().htReloadSwitches()


def kernel_launch_count():
    return int(_lib.lib().htKernelLaunchCount())


def describe_permutation_plan(lensA, modeA, modeB, dtypeA=R_32F, dtypeB=None):
    buf = ctypes.create_string_buffer(1024)
    _check(_lib.lib().htDescribePermutationPlan(len(lensA), _lib.i64(lensA), _lib.i32(modeA), _lib.i32(modeB),
                                                int(dtypeA), int(dtypeA if dtypeB is None else dtypeB), buf, 1024),
           "describe_permutation_plan")
    return buf.value.decode()


def describe_reduction_plan(lensA, stridesA, modeA, lensD, stridesD, modeD, dtype=R_32F):
    buf = ctypes.create_string_buffer(1024)
    _check(_lib.lib().htDescribeReductionPlan(len(lensA), _lib.i64(lensA), _lib.i64(stridesA), _lib.i32(modeA),
                                              len(lensD), _lib.i64(lensD), _lib.i64(stridesD), _lib.i32(modeD),
                                              int(dtype), buf, 1024), "describe_reduction_plan")
    return buf.value.decode()


def describe_contraction_plan(lensA, stridesA, modeA, dtypeA, lensB, stridesB, modeB, dtypeB, lensD, stridesD, modeD,
                              dtypeD, has_c, type_compute):
    buf = ctypes.create_string_buffer(2048)
    _check(_lib.lib().htDescribeContractionPlan(
        len(lensA), _lib.i64(lensA), _lib.i64(stridesA), _lib.i32(modeA), int(dtypeA),
        len(lensB), _lib.i64(lensB), _lib.i64(stridesB), _lib.i32(modeB), int(dtypeB),
        len(lensD), _lib.i64(lensD), _lib.i64(stridesD), _lib.i32(modeD), int(dtypeD),
        1 if has_c else 0, int(type_compute), buf, 2048), "describe_contraction_plan")
    return buf.value.decode()
