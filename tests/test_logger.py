"""CPU-only tests of the logger entry points of the C ABI (reference: library/src/logger.cpp, mask and
file selection through hiptensorLoggerSetMask / hiptensorLoggerOpenFile, library/include/hiptensor/hiptensor.hpp)."""
import os

import pytest


@pytest.fixture(scope="module")
def lib():
    from hiptensor_b200 import build

    build.build()
    from hiptensor_b200 import _lib

    return _lib.lib()


def test_mask_accepts_bit_combinations_and_rejects_out_of_range(lib):
    for mask in (0, 1, 2, 4, 8, 16, 1 | 16, 31):
        assert lib.htLoggerSetMask(mask) == 0
    for mask in (-1, 32, 1 << 20):
        assert lib.htLoggerSetMask(mask) != 0
    assert lib.htLoggerSetMask(0) == 0


def test_errors_go_to_the_opened_file(lib, tmp_path):
    path = tmp_path / "ht.log"
    assert lib.htLoggerOpenFile(str(path).encode()) == 0
    assert lib.htLoggerSetMask(1) == 0  # errors only
    # a permutation called with null arguments is refused with NOT_INITIALIZED and logged at error level
    status = lib.htPermutation(None, None, None, None, None, None, None, None, 0, None)
    assert status != 0
    assert lib.htLoggerSetMask(0) == 0
    # an unwritable path is refused
    assert lib.htLoggerOpenFile(os.path.join(str(tmp_path), "no_such_dir", "x.log").encode()) != 0
    text = path.read_text()
    assert "[Error]" in text and "hiptensorPermutation" in text and "nullptr" in text, text
