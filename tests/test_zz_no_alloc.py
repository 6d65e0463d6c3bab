"""htReductionNoAlloc: the reduction entry point for callers that may not allocate device memory
(plug-ins of hosts that own the device heap, latency-critical loops, services that forbid device
allocations after start-up). Called through the C ABI and compared with htReduction on the same inputs, twice in a row
because the built-in scratch is shared between calls and keeps its old contents.
This file sorts last on purpose: a run that stops at the first failure has then seen every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _pair(ht, h, lens, kept, op, dt, ct, alpha, beta, seed, want_oracle=False):
    """(result of htReductionNoAlloc, result of htReduction with a caller workspace, kernel names[, the CPU
    oracle's result on the same inputs])."""
    import torch

    from helpers import to_device, to_host
    from oracle import binding as orc

    modeA = list(range(len(lens)))
    lensD = [lens[m] for m in kept]
    A = orc.fill_uniform(int(np.prod(lens)), dt, seed)
    C = orc.fill_uniform(max(int(np.prod(lensD)), 1), dt, seed + 2)
    dA = h.tensor_descriptor(lens, None, dt)
    dD = h.tensor_descriptor(lensD, None, dt)
    A_d, C_d = to_device(A, dt), to_device(C, dt)
    D1 = torch.zeros_like(C_d)
    D2 = torch.zeros_like(C_d)
    h.reduction_no_alloc(alpha, A_d, dA, modeA, beta, C_d, dD, kept, D1, dD, kept, op, ct)
    k1 = ht.last_kernel_name()
    ws_size = h.reduction_workspace_size(A_d, dA, modeA, C_d, dD, kept, D2, dD, kept, op, ct)
    ws = torch.empty(max(ws_size, 1), dtype=torch.uint8, device="cuda")
    h.reduction(alpha, A_d, dA, modeA, beta, C_d, dD, kept, D2, dD, kept, op, ct, ws, ws_size)
    k2 = ht.last_kernel_name()
    torch.cuda.synchronize()
    if not want_oracle:
        return to_host(D1, dt), to_host(D2, dt), k1, k2
    exp = np.zeros(C.size, dtype=orc.np_dtype(dt))
    orc.reduction(alpha, A, lens, orc.packed_strides(lens, False), modeA, dt, beta, C, exp, lensD,
                  orc.packed_strides(lensD, False), kept, dt, op, ct)
    return to_host(D1, dt), to_host(D2, dt), k1, k2, exp


def test_matches_the_workspace_entry_point_twice_in_a_row():
    import hiptensor_b200 as ht
    from oracle import binding as orc

    h = ht.Handle()
    # few outputs, long reduced range: the two-pass path, whose partial sums go through the scratch;
    # the second call has other values, other extents and another operator, and finds the first
    # call's partials still in the scratch
    cases = [([3, 512, 1024], [0], orc.OP_ADD, 17), ([2, 300, 2048], [0], orc.OP_MAX, 23),
             ([700, 64, 64], [], orc.OP_ADD, 29)]
    for lens, kept, op, seed in cases:
        got, ref, k1, k2, exp = _pair(ht, h, lens, kept, op, orc.F32, orc.COMPUTE_32F, 2.0, 0.5, seed, want_oracle=True)
        assert k1 == "red_finalize" and k2 == "red_finalize"
        # against the CPU oracle (both entry points run the same kernels, so agreement between them alone would
        # not show a fault they share): the reference's own bound for a sequential fp32 reduction, reduce_len * eps
        n_red = int(np.prod(lens)) // max(int(np.prod([lens[m] for m in kept])), 1)
        bound = n_red * float(np.finfo(np.float32).eps) if op == orc.OP_ADD else 1e-7
        from helpers import rel_error as _rel

        assert 0 <= _rel(got, exp, orc.F32) < bound
        # same kernels, same slicing, same order of operations: identical bits; the stated tolerance
        # of the reduction tests (1e-5 under the reference's metric) is the bound
        from helpers import rel_error

        assert 0 <= rel_error(got, ref, orc.F32) < 1e-5
        assert np.array_equal(got, ref)
    # single-pass shapes take no scratch at all and go through the same entry point
    got, ref, k1, _ = _pair(ht, h, [64, 16, 32, 8], [0, 1], orc.OP_ADD, orc.F32, orc.COMPUTE_32F, 1.0, 0.5, 31)
    assert k1 == "red_row" and np.array_equal(got, ref)


def test_rejects_what_does_not_fit_the_built_in_scratch():
    import torch

    import hiptensor_b200 as ht

    h = ht.Handle()
    # fp64, 591 outputs, 16384 reduced elements each: three slices of 591 doubles = 14184 bytes > 8 KiB
    lens = [591, 16384]
    A = torch.zeros(lens[0] * lens[1], dtype=torch.float64, device="cuda")
    D = torch.zeros(lens[0], dtype=torch.float64, device="cuda")
    dA = h.tensor_descriptor(lens, None, ht.R_64F)
    dD = h.tensor_descriptor([lens[0]], None, ht.R_64F)
    assert h.reduction_workspace_size(A, dA, [0, 1], D, dD, [0], D, dD, [0], ht.OP_ADD, ht.COMPUTE_64F) > 8192
    with pytest.raises(ht.HiptensorError) as e:
        h.reduction_no_alloc(1.0, A, dA, [0, 1], 0.0, D, dD, [0], D, dD, [0], ht.OP_ADD, ht.COMPUTE_64F)
    assert e.value.status == ht.STATUS_INSUFFICIENT_WORKSPACE


def test_plans_sliced_by_thread_count_fit_the_built_in_scratch():
    """Short rows and contiguous kept modes are sliced by thread or block count, far beyond 8 KiB of partial results with
    a caller workspace: without one the call uses the slices that fit (or one pass) and agrees with htReduction."""
    import hiptensor_b200 as ht
    from oracle import binding as orc

    h = ht.Handle()
    # 130 outputs along the contiguous kept mode under 20000 reduced rows; 24 outputs of rows of 4 under 3000 outer rows
    for lens, kept in (([20000, 130], [1]), ([3000, 24, 4], [1])):
        from helpers import rel_error

        got, ref, k1, k2, exp = _pair(ht, h, lens, kept, orc.OP_ADD, orc.F32, orc.COMPUTE_32F, 1.5, 0.5, 41,
                                      want_oracle=True)
        assert k1 == "red_finalize" and k2 == "red_finalize"
        n_red = int(np.prod(lens)) // int(np.prod([lens[m] for m in kept]))
        # the reference's bound for a sequential fp32 reduction against the oracle; the two entry points differ in
        # the number of slices only (stated tolerance of the reduction tests between them)
        assert 0 <= rel_error(got, exp, orc.F32) < n_red * float(np.finfo(np.float32).eps)
        assert 0 <= rel_error(ref, exp, orc.F32) < n_red * float(np.finfo(np.float32).eps)
        assert 0 <= rel_error(got, ref, orc.F32) < 1e-5


def test_a_warm_call_allocates_no_device_memory():
    """After the first call on the device (which looks the scratch address up), a call must leave the device's
    free memory and the caching allocator of the test harness untouched."""
    import torch

    import hiptensor_b200 as ht
    from helpers import to_device
    from oracle import binding as orc

    h = ht.Handle()
    lens, kept = [3, 512, 1024], [0]
    A_d = to_device(orc.fill_uniform(int(np.prod(lens)), orc.F32, 41), orc.F32)
    C_d = to_device(orc.fill_uniform(3, orc.F32, 43), orc.F32)
    D_d = torch.zeros_like(C_d)
    dA = h.tensor_descriptor(lens, None, ht.R_32F)
    dD = h.tensor_descriptor([3], None, ht.R_32F)
    call = lambda: h.reduction_no_alloc(2.0, A_d, dA, [0, 1, 2], 0.5, C_d, dD, kept, D_d, dD, kept, ht.OP_ADD,  # noqa: E731
                                        ht.COMPUTE_32F)
    import gc

    call()  # first call on this device: one-time address lookup
    gc.collect()  # tensors of earlier tests that are still waiting for the collector go now, not between the readings
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    events0 = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert ht.last_kernel_name() == "red_finalize"
    assert free1 >= free0  # nothing taken from the device (cudaMalloc by the library would show here)
    assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == events0  # nor from the harness' allocator
    assert torch.cuda.memory_allocated() <= alloc0 and torch.cuda.memory_reserved() <= reserved0
