"""GPU parity: hiptensorReduction through the C ABI against the CPU oracle.
Metric: the reference's max|d-h|/(|d|+|h|+1) (test/device/common.hpp:122-151). Short reductions are
held to 1e-5 against the oracle directly; long fp32 ADD reductions are held to the reference's own
bound reduce_len*eps (test/03_reduction/reduction_test.cpp:518-543) against the oracle and to 1e-5
against the exact (fp64) result, see helpers.check_f32. f16 / bf16 outputs: 2*2^-10 / 2*2^-7."""
import itertools
import json
import os

import numpy as np
import pytest

from helpers import check_f32, rel_error, run_reduction
from oracle import binding as orc


def bits(a):
    return a.view({8: np.uint64, 4: np.uint32, 2: np.uint16}[a.dtype.itemsize])

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = {orc.F32: 1e-5, orc.F64: 1e-5, orc.F16: 2 * 2.0 ** -10, orc.BF16: 2 * 2.0 ** -7}


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


@pytest.mark.parametrize("dt", [orc.F32, orc.F64])
def test_golden_vector(env, dt):
    ht, h = env
    g = json.load(open(os.path.join(GOLD, "reduction_mhkv_kv.json")))
    modeA, modeC = [ord(c) for c in g["modeA"]], [ord(c) for c in g["modeC"]]
    lensA = [g["extent"][c] for c in g["modeA"]]
    import torch

    from helpers import to_device, to_host

    A = np.arange(int(np.prod(lensA)), dtype=orc.np_dtype(dt))
    lensC = [g["extent"][c] for c in g["modeC"]]
    D = np.full(int(np.prod(lensC)), g["C"], dtype=orc.np_dtype(dt))
    dA, dC = h.tensor_descriptor(lensA, None, dt), h.tensor_descriptor(lensC, None, dt)
    A_d, D_d = to_device(A, dt), to_device(D, dt)
    ct = orc.COMPUTE_64F if dt == orc.F64 else orc.COMPUTE_32F
    h.reduction(g["alpha"], A_d, dA, modeA, g["beta"], D_d, dC, modeC, D_d, dC, modeC, ht.OP_ADD, ct)
    got = to_host(D_d, dt)
    exp = np.array(g["expected_default_build"], dtype=orc.np_dtype(dt))
    assert 0 <= rel_error(got, exp, dt) < 1e-6


@pytest.mark.parametrize("op", [orc.OP_ADD, orc.OP_MUL, orc.OP_MIN, orc.OP_MAX])
def test_rank4_every_output_subset(env, op):
    """All subsets of kept modes incl. the full reduction and the identity (reference:
    test/03_reduction/configs/validation/rank4_test_params.yaml:21-39)."""
    ht, h = env
    lens, modeA = [6, 5, 9, 8], [0, 1, 2, 3]
    for r in range(0, 5):
        for kept in itertools.combinations(modeA, r):
            got, exp = run_reduction(ht, h, lens, modeA, list(kept), op=op, alpha=1.0, beta=0.0)
            err = rel_error(got, exp, orc.F32)
            assert 0 <= err < 1e-5, (op, kept, err, ht.last_kernel_name())


@pytest.mark.parametrize("first_fastest", [False, True])
@pytest.mark.parametrize("kept", [[0, 1], [2, 3], [0, 3], [1], [3]])
def test_layouts_and_beta(env, first_fastest, kept):
    ht, h = env
    lens, modeA = [36, 20, 24, 40], [0, 1, 2, 3]
    sA = orc.packed_strides(lens, first_fastest)
    lensD = [lens[m] for m in kept]
    sD = orc.packed_strides(lensD, first_fastest)
    terms = int(np.prod(lens)) // int(np.prod(lensD))
    for alias in (False, True):
        got, exp, exact = run_reduction(ht, h, lens, modeA, kept, alpha=1.2, beta=2.1, stridesA=sA, stridesD=sD,
                                        alias=alias, want_exact=True)
        check_f32(got, exp, exact, terms)


@pytest.mark.parametrize("op", [orc.OP_ADD, orc.OP_MAX, orc.OP_MUL])
@pytest.mark.parametrize("dt,lens", [(orc.F32, [37, 5, 256]), (orc.F32, [9, 11, 8, 32]), (orc.F32, [70, 3, 512]),
                                     (orc.F16, [37, 5, 512]), (orc.F16, [13, 7, 1024]), (orc.F64, [37, 5, 128])])
def test_short_rows_eight_lanes_per_output(env, op, dt, lens):
    """Contiguous reduced rows of at most 2 KiB run with eight lanes per output, four outputs per warp; the number of
    outputs is not a multiple of 32, so the last block has idle groups. ADD and MUL within the reference's bound, MAX
    bit-exact."""
    ht, h = env
    modeA = list(range(len(lens)))
    kept = modeA[:2]
    A = None
    if op == orc.OP_MUL:  # values near 1 keep the product in range
        A = (1.0 + orc.fill_uniform(int(np.prod(lens)), orc.F64, 3) * 1e-3).astype({orc.F32: np.float32, orc.F16: np.float16,
                                                                                 orc.F64: np.float64}[dt])
    got, exp = run_reduction(ht, h, lens, modeA, kept, dt=dt, op=op, alpha=1.5, beta=0.5, A=A)
    assert ht.last_kernel_name() == "red_row"
    terms = int(np.prod(lens[2:]))
    if op == orc.OP_MAX:
        assert np.array_equal(bits(got), bits(exp))
    else:
        eps = {orc.F32: np.finfo(np.float32).eps, orc.F16: np.finfo(np.float16).eps, orc.F64: np.finfo(np.float64).eps}[dt]
        assert 0 <= rel_error(got, exp, dt) < max(terms * float(eps), 1e-6)


EPS = {orc.F32: float(np.finfo(np.float32).eps), orc.F16: float(np.finfo(np.float16).eps),
       orc.F64: float(np.finfo(np.float64).eps), orc.BF16: 2.0 ** -8}


def check_reduction(got, exp, dt, op, terms):
    if op in (orc.OP_MAX, orc.OP_MIN):
        assert np.array_equal(bits(got), bits(exp))
    else:
        assert 0 <= rel_error(got, exp, dt) < max(terms * EPS[dt], 1e-6)


@pytest.mark.parametrize("op", [orc.OP_ADD, orc.OP_MAX])
@pytest.mark.parametrize("dt", [orc.F32, orc.F16, orc.F64, orc.BF16])
@pytest.mark.parametrize("row", [2, 3, 4, 8, 12, 24, 33, 64, 130])
def test_short_contiguous_rows(env, op, dt, row):
    """Contiguous reduced rows of 2 to 130 elements, alone and under a further reduced mode: 1 to 32 lanes per output
    (one load per lane up to 16 loads a row, several beyond), neighbouring lanes on neighbouring rows. The output
    count is not a multiple of the outputs per block."""
    ht, h = env
    # last mode contiguous: [kept 37][kept 5][row]
    got, exp = run_reduction(ht, h, [37, 5, row], [0, 1, 2], [0, 1], dt=dt, op=op, alpha=1.5, beta=0.5)
    size = {orc.F32: 4, orc.F16: 2, orc.F64: 8, orc.BF16: 2}[dt]
    # rows of more than 16 full 16-byte loads and no further reduced mode stay on the row kernel's eight lanes
    assert ht.last_kernel_name() == ("red_short" if row * size <= 256 or row * size % 16 else "red_row")
    check_reduction(got, exp, dt, op, row)
    # [reduced 9][kept 21][kept 3][row]: the outer reduced mode is walked without divisions
    got, exp = run_reduction(ht, h, [9, 21, 3, row], [0, 1, 2, 3], [1, 2], dt=dt, op=op, alpha=-0.5, beta=2.0)
    assert ht.last_kernel_name() == "red_short"
    check_reduction(got, exp, dt, op, 9 * row)
    # two outer reduced modes of odd extents around the kept ones
    got, exp = run_reduction(ht, h, [7, 10, 5, 3, row], [0, 1, 2, 3, 4], [1, 3], dt=dt, op=op)
    assert ht.last_kernel_name() == "red_short"
    check_reduction(got, exp, dt, op, 35 * row)


@pytest.mark.parametrize("op", [orc.OP_ADD, orc.OP_MIN])
@pytest.mark.parametrize("dt", [orc.F32, orc.F16])
@pytest.mark.parametrize("lens,kept", [([3000, 24, 4], [1]), ([5000, 3, 6], [1]), ([2048, 7, 16], [1]),
                                       ([4096, 33, 130], [1])])
def test_short_rows_few_outputs_are_sliced(env, op, dt, lens, kept):
    """A few outputs with short rows and a long outer reduced mode: slices of the outer mode fill the GPU, a second
    pass folds them; without a workspace one pass gives the same values within the bound."""
    ht, h = env
    got, exp = run_reduction(ht, h, lens, [0, 1, 2], kept, dt=dt, op=op, alpha=1.25, beta=0.75)
    assert ht.last_kernel_name() == "red_finalize"
    check_reduction(got, exp, dt, op, lens[0] * lens[2])
    got, exp = run_reduction(ht, h, lens, [0, 1, 2], kept, dt=dt, op=op, alpha=1.25, beta=0.75, use_workspace=False)
    assert ht.last_kernel_name() == "red_short"
    check_reduction(got, exp, dt, op, lens[0] * lens[2])


@pytest.mark.parametrize("op", [orc.OP_ADD, orc.OP_MAX])
@pytest.mark.parametrize("dt", [orc.F32, orc.F16, orc.F64])
@pytest.mark.parametrize("lens,kept", [([300, 40, 2], [1, 2]), ([300, 40, 4], [2]), ([64, 9, 50, 6], [1, 3]),
                                       ([500, 16], [1]), ([12, 70, 3, 8], [1, 3]), ([8, 100, 100], [1, 2]),
                                       ([40000, 8], [1])])
def test_short_contiguous_kept_mode(env, op, dt, lens, kept):
    """The contiguous mode is kept and short (2 to 16 elements): the column kernel's lanes run over the flattened outputs,
    or along the rows of the innermost reduced mode when those follow the kept run without a gap; few outputs are
    sliced."""
    ht, h = env
    modes = list(range(len(lens)))
    got, exp = run_reduction(ht, h, lens, modes, kept, dt=dt, op=op, alpha=1.5, beta=0.5)
    assert ht.last_kernel_name() in ("red_col", "red_finalize")
    terms = int(np.prod([lens[i] for i in modes if i not in kept]))
    check_reduction(got, exp, dt, op, terms)
    got, exp = run_reduction(ht, h, lens, modes, kept, dt=dt, op=op, alpha=1.5, beta=0.5, use_workspace=False)
    assert ht.last_kernel_name() == "red_col"
    check_reduction(got, exp, dt, op, terms)


def test_permuted_output_strides(env):
    """Output extents in A's order, permutation expressed by strides
    (test/03_reduction/reduction_test.cpp:334-372)."""
    ht, h = env
    lens, modeA, kept = [3, 5, 8], [0, 1, 2], [1, 2]
    got, exp = run_reduction(ht, h, lens, modeA, kept, stridesD=[1, 5], alpha=1.0, beta=0.0)
    assert 0 <= rel_error(got, exp, orc.F32) < 1e-5


@pytest.mark.parametrize("dt,ct", [(orc.F16, orc.COMPUTE_16F), (orc.F16, orc.COMPUTE_32F),
                                   (orc.BF16, orc.COMPUTE_16BF), (orc.BF16, orc.COMPUTE_32F),
                                   (orc.F64, orc.COMPUTE_64F)])
def test_other_types(env, dt, ct):
    ht, h = env
    for kept in ([0], [2], [0, 2]):
        for op in (orc.OP_ADD, orc.OP_MAX):
            got, exp = run_reduction(ht, h, [24, 16, 40], [0, 1, 2], kept, dt=dt, compute=ct, op=op, alpha=0.5,
                                     beta=1.0)
            err = rel_error(got, exp, dt)
            assert 0 <= err < TOL[dt], (dt, ct, kept, op, err)


def test_nan_propagates_through_max_and_min(env):
    ht, h = env
    lens = [8, 64]
    A = orc.fill_uniform(8 * 64, orc.F32, 17)
    A[3 * 64 + 11] = np.nan
    for op in (orc.OP_MAX, orc.OP_MIN):
        got, exp = run_reduction(ht, h, lens, [0, 1], [0], op=op, A=A.copy())
        assert np.isnan(got[3]) and np.isnan(exp[3])
        keep = np.arange(8) != 3
        assert np.array_equal(got[keep], exp[keep])


def test_few_outputs_long_reduction_two_pass(env):
    """Few outputs and a long reduced range: the sliced two-pass path through the workspace, and
    the single-pass path when the caller gives no workspace."""
    ht, h = env
    lens, modeA = [3, 512, 1024], [0, 1, 2]
    for kept in ([0], []):
        for op in (orc.OP_ADD, orc.OP_MAX):
            terms = 512 * 1024 * (1 if kept else 3)
            got, exp, exact = run_reduction(ht, h, lens, modeA, kept, op=op, alpha=2.0, beta=0.5, use_workspace=True,
                                            want_exact=True)
            assert ht.last_kernel_name() == "red_finalize"
            check_f32(got, exp, exact, terms)
            got2, exp2, exact2 = run_reduction(ht, h, lens, modeA, kept, op=op, alpha=2.0, beta=0.5,
                                               use_workspace=False, want_exact=True)
            assert ht.last_kernel_name() != "red_finalize"
            check_f32(got2, exp2, exact2, terms)


def test_rejects_mismatched_descriptors(env):
    import torch

    ht, h = env
    x = torch.zeros(64, device="cuda")
    dA = h.tensor_descriptor([8, 8], None, ht.R_32F)
    dC = h.tensor_descriptor([8], None, ht.R_32F)
    dD = h.tensor_descriptor([8], [2], ht.R_32F)
    with pytest.raises(ht.HiptensorError) as e:
        h.reduction(1.0, x, dA, [0, 1], 0.0, x, dC, [0], x, dD, [0], ht.OP_ADD, ht.COMPUTE_32F)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED
    with pytest.raises(ht.HiptensorError) as e:
        h.reduction(1.0, x, dA, [0, 1], 0.0, x, dC, [5], x, dC, [5], ht.OP_ADD, ht.COMPUTE_32F)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED
    with pytest.raises(ht.HiptensorError) as e:
        h.reduction(1.0, x, dA, [0, 1], 0.0, x, dC, [0], x, dC, [0], ht.OP_ADD, ht.COMPUTE_64F)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED


@pytest.mark.parametrize("first_fastest", [False, True])
def test_config3_full_size(env, first_fastest):
    """A[m,n,k,h] = {4096,64,64,32} fp32 (2 GiB) reduced over {k,h}: D = 1.0*reduce + 0.5*C, ADD then MAX,
    against the oracle on the full tensor. first_fastest=False is the NULL-stride layout (contiguous
    2048-element rows), True the strided-column layout."""
    import torch

    from helpers import to_host

    ht, h = env
    lens, modeA, kept = [4096, 64, 64, 32], [0, 1, 2, 3], [0, 1]
    sA = orc.packed_strides(lens, first_fastest)
    sD = orc.packed_strides(lens[:2], first_fastest)
    n = int(np.prod(lens))
    A = orc.fill_uniform(n, orc.F32, 17)
    C = orc.fill_uniform(4096 * 64, orc.F32, 19)
    A_d, C_d = torch.from_numpy(A).cuda(), torch.from_numpy(C).cuda()
    dA = h.tensor_descriptor(lens, sA, ht.R_32F)
    dD = h.tensor_descriptor(lens[:2], sD, ht.R_32F)
    for op in (orc.OP_ADD, orc.OP_MAX):
        D_d = torch.zeros(4096 * 64, device="cuda")
        h.reduction(1.0, A_d, dA, modeA, 0.5, C_d, dD, kept, D_d, dD, kept, op, ht.COMPUTE_32F)
        exp = np.zeros(4096 * 64, dtype=np.float32)
        orc.reduction(1.0, A, lens, sA, modeA, orc.F32, 0.5, C, exp, lens[:2], sD, kept, orc.F32, op,
                      orc.COMPUTE_32F)
        got = to_host(D_d, orc.F32)
        if op == orc.OP_MAX:  # max is order independent: bit-exact
            assert np.array_equal(got, exp)
        else:
            exact = np.zeros(4096 * 64, dtype=np.float64)
            orc.reduction(1.0, A.astype(np.float64), lens, sA, modeA, orc.F64, 0.5, C.astype(np.float64), exact,
                          lens[:2], sD, kept, orc.F64, op, orc.COMPUTE_64F)
            check_f32(got, exp, exact, 2048)


@pytest.mark.parametrize("rank", [1, 2, 3, 5, 6])
def test_other_ranks(env, rank):
    """Ranks 1 to 6 (reference: test/03_reduction/configs/validation/rank{1..6}_test_params.yaml): the full
    reduction, each single kept mode, and a split in the middle, both memory orders."""
    ht, h = env
    lens = [7, 4, 6, 3, 5, 2][:rank]
    modeA = list(range(rank))
    keeps = [[]] + [[m] for m in modeA] + ([modeA[: rank // 2]] if rank > 1 else []) + ([modeA[rank // 2:]] if rank > 1 else [])
    for kept in keeps:
        if len(kept) == rank:
            continue
        for first in (False, True):
            sA = orc.packed_strides(lens, first)
            lensD = [lens[m] for m in kept]
            sD = orc.packed_strides(lensD, first)
            got, exp, exact = run_reduction(ht, h, lens, modeA, kept, op=orc.OP_ADD, alpha=1.5, beta=0.0, stridesA=sA,
                                            stridesD=sD, want_exact=True)
            reduce_len = int(np.prod(lens)) // max(int(np.prod(lensD)), 1)
            check_f32(got, exp, exact, reduce_len)
