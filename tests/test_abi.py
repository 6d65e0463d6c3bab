"""CPU-only checks of the drop-in boundary: the shared library loads without a GPU or driver,
exports every symbol include/hiptensor_b200.h declares, and refuses to work without a device."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from hiptensor_b200 import build

    return build.build()


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "hiptensor_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ht[A-Z]\w+)\s*\(", text)))


def test_header_symbols_are_exported(built):
    from hiptensor_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 24
    L = ctypes.CDLL(built)
    for n in names:
        assert hasattr(L, n), n
    assert sorted(_lib.SIGNATURES) == names


def test_cpp_api_symbols_are_exported(built):
    out = subprocess.check_output(["nm", "-D", "--defined-only", built], text=True)
    for fn in ["hiptensorCreate", "hiptensorDestroy", "hiptensorInitTensorDescriptor", "hiptensorGetErrorString",
               "hiptensorGetAlignmentRequirement", "hiptensorInitContractionDescriptor",
               "hiptensorInitContractionFind", "hiptensorContractionGetWorkspaceSize", "hiptensorInitContractionPlan",
               "hiptensorContraction", "hiptensorPermutation", "hiptensorReduction",
               "hiptensorReductionGetWorkspaceSize", "hiptensorLoggerSetMask"]:
        assert re.search(r" T _Z\d+%s[A-Za-z0-9]" % fn, out), fn


def test_no_driver_dependency(built):
    out = subprocess.check_output(["ldd", built], text=True)
    assert "libcuda.so" not in out and "libcudart" not in out


def test_error_strings(built):
    import hiptensor_b200 as ht

    assert ht.error_string(0) == "HIPTENSOR_STATUS_SUCCESS"
    assert ht.error_string(19) == "HIPTENSOR_STATUS_INSUFFICIENT_WORKSPACE"
    assert ht.error_string(99) == "HIPTENSOR_STATUS_UNKNOWN"


def test_fails_loudly_without_a_gpu(built):
    import torch

    import hiptensor_b200 as ht

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(ht.HiptensorError) as e:
        ht.Handle()
    assert e.value.status == ht.STATUS_HIP_ERROR


def test_null_handle_is_rejected(built):
    from hiptensor_b200 import _lib

    L = _lib.lib()
    d = ctypes.c_void_p(0)
    lens = _lib.i64([2, 3])
    assert L.htCreateTensorDescriptor(None, ctypes.byref(d), 2, lens, None, 0, 1) == 1
    assert L.htPermutation(None, None, None, None, None, None, None, None, 0, None) == 1
    assert L.htReduction(None, None, None, None, None, None, None, None, None, None, None, None, 3, 4, None, 0,
                         None) == 1
    assert L.htContraction(None, None, None, None, None, None, None, None, None, 0, None) == 1
