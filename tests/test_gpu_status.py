"""Device-side waits are bounded: a kernel whose wait runs out writes the handle's status word (pinned host memory)
and exits; the next operation on the handle reports EXECUTION_FAILED once. The failure is injected on the host
(htInjectDeviceStatus writes the word as such a kernel would); no kernel is made to wait."""
import ctypes

import numpy as np
import pytest

from helpers import run_permutation
from oracle import binding as orc

pytestmark = pytest.mark.gpu


def test_timeout_status_is_reported_once_and_the_handle_stays_usable():
    import hiptensor_b200 as ht
    from hiptensor_b200 import _lib

    h = ht.Handle()
    assert h.device_status() == 0
    got, exp = run_permutation(ht, h, [40, 24, 20], [0, 1, 2], [2, 0, 1])
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))
    assert h.device_status() == 0  # normal runs leave it alone

    assert _lib.lib().htInjectDeviceStatus(h._h, 3) == 0
    assert h.device_status() == 3
    with pytest.raises(ht.HiptensorError) as e:
        run_permutation(ht, h, [40, 24, 20], [0, 1, 2], [2, 0, 1])
    assert e.value.status == ht.STATUS_EXECUTION_FAILED
    assert h.device_status() == 0  # reported once, then cleared
    got, exp = run_permutation(ht, h, [40, 24, 20], [0, 1, 2], [2, 0, 1])
    assert np.array_equal(got.view(np.uint32), exp.view(np.uint32))
