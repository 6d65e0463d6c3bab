"""GPU parity of complex contractions (cf32 / cf64, compute C32F / C64F) through the C ABI against the CPU
oracle (reference algorithm: contraction_cpu_reference_impl.hpp:166-323).

The library runs a complex contraction as ONE real contraction of doubled N and K extents on its real
kernels (FP64 tensor pipe, TF32-split tensor cores or FMA), after copying the smaller operand, scaled by
alpha, in expanded form into the workspace; the reference runs four real contractions on planes it unpacks into
device memory it allocates (device_contraction_bilinear_complex.hpp:454-470,535-558).

The problem lists the reference's harness sweeps
(test/01_contraction/configs/validation/complex_{bilinear,scale}_test_params_rank{1..6}.yaml) run in
test_gpu_contraction_validation.py through this module's run(); here are larger problems that reach the
tensor-core kernels, aliasing, workspace rules. Tolerances: the reference accepts 2*K*eps(float) under
max|d-h|/(|d|+|h|+1) for both precisions (contraction_test.cpp:882-905); here cf32 is held to that bound
against the oracle and to 2e-5 against the fp64 evaluation of the same values, cf64 to 1e-12."""
import numpy as np
import pytest

from helpers import rel_error, span
from oracle import binding as orc

pytestmark = pytest.mark.gpu
EPS = float(np.finfo(np.float32).eps)
SEEDS = (255, 256, 257)  # contraction_test.cpp:381-441


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


def cfill(n, dtype, seed):
    """n complex elements with independent real and imaginary parts from the harness' generator."""
    real = orc.F32 if dtype == orc.C32F else orc.F64
    return orc.fill_uniform(2 * n, real, seed).view(np.complex64 if dtype == orc.C32F else np.complex128)


def run(env, ext, modeA, modeB, modeD, dtype, alpha, beta, with_c=True, first_fastest=False, alias=False,
        pref=None, same_parts=False):
    import torch

    ht, h = env
    ct = np.complex64 if dtype == orc.C32F else np.complex128
    hdt = ht.C_32F if dtype == orc.C32F else ht.C_64F
    compute = ht.COMPUTE_C32F if dtype == orc.C32F else ht.COMPUTE_C64F
    lA, lB, lD = ([ext[m] for m in ms] for ms in (modeA, modeB, modeD))
    sA, sB, sD = (orc.packed_strides(l, first_fastest) for l in (lA, lB, lD))
    nA, nB, nD = span(lA, sA), span(lB, sB), span(lD, sD)
    A, B, C = cfill(nA, dtype, SEEDS[0]), cfill(nB, dtype, SEEDS[1]), cfill(nD, dtype, SEEDS[2])
    if same_parts:  # the harness' own fill: real and imaginary part equal (test/device/common.hpp:92-100)
        A, B, C = ((x.real + 1j * x.real).astype(ct) for x in (A, B, C))
    dA, dB, dD = (h.tensor_descriptor(l, s, hdt) for l, s in ((lA, sA), (lB, sB), (lD, sD)))
    cd = h.contraction_descriptor(dA, modeA, dB, modeB, dD if with_c else None, modeD if with_c else None, dD, modeD,
                                  compute)
    find = h.contraction_find()
    ws_size = h.contraction_workspace_size(cd, find, ht.WORKSPACE_RECOMMENDED if pref is None else pref)
    assert ws_size >= 4 * min(nA, nB) * (4 if dtype == orc.C32F else 8)
    plan = h.contraction_plan(cd, find, ws_size)
    ws = torch.empty(ws_size, dtype=torch.uint8, device="cuda")
    A_d, B_d = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    C_d = torch.from_numpy(C).cuda() if with_c else None
    D_d = C_d if (alias and with_c) else torch.from_numpy(np.full(nD, np.nan + 1j * np.nan, dtype=ct)).cuda()
    h.contraction(plan, alpha, A_d, B_d, beta, C_d, D_d, ws, ws_size)
    torch.cuda.synchronize()
    assert h.device_status() == 0
    got = D_d.cpu().numpy()
    exp = np.full(nD, np.nan + 1j * np.nan, dtype=ct)
    orc.contraction_complex(alpha, A, lA, sA, modeA, B, lB, sB, modeB, beta, C if with_c else None, exp, lD, sD, modeD,
                            dtype)
    K = int(np.prod([ext[m] for m in modeA if m in modeB]))
    real = orc.F32 if dtype == orc.C32F else orc.F64
    g, e = got.view(ct(0).real.dtype), exp.view(ct(0).real.dtype)
    assert not np.isnan(g).any()
    if dtype == orc.C64F:
        err = rel_error(g, e, real)
        assert 0 <= err < 1e-12, err
    else:
        err = rel_error(g, e, real)
        assert 0 <= err < max(2 * 2 * K * EPS, 1e-6), ("vs reference algorithm", err)
        exact = np.full(nD, np.nan + 1j * np.nan, dtype=np.complex128)
        orc.contraction_complex(complex(np.complex64(alpha)), A.astype(np.complex128), lA, sA, modeA,
                                B.astype(np.complex128), lB, sB, modeB, complex(np.complex64(beta)),
                                C.astype(np.complex128) if with_c else None, exact, lD, sD, modeD, orc.C64F)
        err2 = rel_error(g.astype(np.float64), exact.view(np.float64), orc.F64)
        # twice the bound of the real fp32 tests: a complex output accumulates two sums of K products each,
        # of magnitude up to 2 for inputs in [-1, 1)
        assert 0 <= err2 < 2e-5, ("vs exact", err2)
    return ht.last_kernel_name()


@pytest.mark.parametrize("dtype", [orc.C32F, orc.C64F])
def test_real_beta_uses_the_kernel_epilogue_and_alias(env, dtype):
    """beta real and exactly representable: no pass over C; C aliasing D (the reference's samples call it so);
    complex beta with C aliasing D: the pass runs in place."""
    ext = {0: 24, 1: 20, 2: 12, 3: 16, 4: 8, 5: 10}
    mA, mB, mD = [0, 1, 4, 5], [2, 3, 4, 5], [0, 1, 2, 3]
    ht = env[0]
    n0 = ht.kernel_launch_count()
    run(env, ext, mA, mB, mD, dtype, 1.5 + 0j, 0.5 + 0j)
    assert ht.kernel_launch_count() - n0 == 2  # the copy and the contraction
    run(env, ext, mA, mB, mD, dtype, 1.5 - 0.5j, 0.5 + 0j, alias=True)
    n0 = ht.kernel_launch_count()
    run(env, ext, mA, mB, mD, dtype, 1.5 - 0.5j, 0.5 + 0.25j, alias=True)
    assert ht.kernel_launch_count() - n0 == 3


@pytest.mark.parametrize("first_fastest", [False, True])
def test_cf32_on_the_tensor_cores(env, first_fastest):
    """Extents that give 16-byte aligned strides: the real problem runs on the TF32 big/small split kernel with
    fp32-grade accuracy. With the contracted modes innermost (NULL strides) the larger operand is read where it
    lies; with the first mode fastest its real view is neither K-major nor M-major (the (re, im) pairs sit between
    consecutive rows), so it is copied too."""
    ext = {0: 16, 1: 24, 2: 12, 3: 16, 4: 8, 5: 12}
    name = run(env, ext, [0, 1, 4, 5], [2, 3, 4, 5], [0, 1, 2, 3], orc.C32F, 1.1 + 1.2j, 2.2 + 2.3j,
               first_fastest=first_fastest)
    assert name.startswith("contraction_tf32x3"), name
    ht = env[0]
    n0 = ht.kernel_launch_count()
    run(env, ext, [0, 1, 4, 5], [2, 3, 4, 5], [0, 1, 2, 3], orc.C32F, 1.0 + 0j, 0j, with_c=False,
        first_fastest=first_fastest)
    assert ht.kernel_launch_count() - n0 == (3 if first_fastest else 2)


def test_cf64_on_the_fp64_tensor_pipe_and_operand_choice(env):
    """The smaller operand is the one copied, whichever side it is on; interleaved mode orders."""
    ext = {0: 12, 1: 10, 2: 6, 3: 14, 4: 9, 5: 7}
    assert run(env, ext, [0, 4, 1, 5], [5, 2, 4, 3], [0, 2, 1, 3], orc.C64F, 2 + 0.5j, 0.5 - 1j) == "contraction_tiled_dmma"
    big = dict(ext)
    big.update({2: 30, 3: 28})  # now A is the smaller one
    assert run(env, big, [0, 4, 1, 5], [5, 2, 4, 3], [3, 0, 2, 1], orc.C64F, 2 + 0.5j, 0.5 - 1j) == "contraction_tiled_dmma"


def test_workspace_rules(env):
    """The copy's space is required at every preference; without it the call reports INSUFFICIENT_WORKSPACE."""
    import torch

    ht, h = env
    l = [32, 32]
    d = h.tensor_descriptor(l, None, ht.C_32F)
    cd = h.contraction_descriptor(d, [0, 2], d, [1, 2], d, [0, 1], d, [0, 1], ht.COMPUTE_C32F)
    find = h.contraction_find()
    need = h.contraction_workspace_size(cd, find, ht.WORKSPACE_MIN)
    assert need == 32 * 32 * 16
    assert h.contraction_workspace_size(cd, find, ht.WORKSPACE_MAX) >= need
    plan = h.contraction_plan(cd, find, 0)
    t = torch.zeros(32 * 32, dtype=torch.complex64, device="cuda")
    with pytest.raises(ht.HiptensorError) as e:
        h.contraction(plan, 1 + 0j, t, t, 0j, t, t, None, 0)
    assert e.value.status == ht.STATUS_INSUFFICIENT_WORKSPACE
    # complex tensors with a real compute type, or the other precision's: rejected when the plan is made
    cd = h.contraction_descriptor(d, [0, 2], d, [1, 2], d, [0, 1], d, [0, 1], ht.COMPUTE_32F)
    with pytest.raises(ht.HiptensorError) as e:
        h.contraction_plan(cd, find, 1 << 20)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED
