"""CPU checks of the complex contraction: the oracle against an independent evaluation (numpy einsum in
complex128), and the planner's rewriting of a complex contraction as one real contraction.

Reference: contraction_cpu_reference_impl.hpp:166-323 (CPU algorithm),
device_contraction_bilinear_complex.hpp:454-470 (the four real contractions this library replaces by one)."""
import numpy as np
import pytest

from oracle import binding as orc


def packed(lens, first_fastest=False):
    return orc.packed_strides(lens, first_fastest)


@pytest.mark.parametrize("dtype", [orc.C32F, orc.C64F])
@pytest.mark.parametrize("bilinear", [False, True])
def test_oracle_against_einsum(dtype, bilinear):
    ct = np.complex64 if dtype == orc.C32F else np.complex128
    rng = np.random.default_rng(5)
    lA, lB, lD = [5, 6, 3, 4], [2, 3, 3, 4], [5, 6, 2, 3]  # A[m0,m1,k0,k1] B[n0,n1,k0,k1] D[m0,m1,n0,n1]
    A = (rng.uniform(-1, 1, lA) + 1j * rng.uniform(-1, 1, lA)).astype(ct)
    B = (rng.uniform(-1, 1, lB) + 1j * rng.uniform(-1, 1, lB)).astype(ct)
    C = (rng.uniform(-1, 1, lD) + 1j * rng.uniform(-1, 1, lD)).astype(ct)
    alpha, beta = 1.1 + 1.2j, 2.2 + 2.3j
    D = np.full(lD, np.nan + 0j, dtype=ct)
    orc.contraction_complex(alpha, A.ravel(), lA, packed(lA), [0, 1, 4, 5], B.ravel(), lB, packed(lB), [2, 3, 4, 5],
                            beta, C.ravel() if bilinear else None, D.reshape(-1), lD, packed(lD), [0, 1, 2, 3], dtype)
    want = alpha * np.einsum("abkl,cdkl->abcd", A.astype(np.complex128), B.astype(np.complex128))
    if bilinear:
        want = want + beta * C.astype(np.complex128)
    tol = 1e-5 if dtype == orc.C32F else 1e-13
    assert np.max(np.abs(D - want)) < tol


def test_oracle_strided_and_first_fastest():
    """First-mode-fastest strides and a mode order where the contracted modes are not innermost."""
    rng = np.random.default_rng(6)
    ext = {0: 4, 1: 3, 2: 5, 3: 2, 4: 6}
    mA, mB, mD = [4, 0, 1], [2, 4, 3], [0, 2, 1, 3]
    lA, lB, lD = ([ext[m] for m in ms] for ms in (mA, mB, mD))
    sA, sB, sD = (packed(l, True) for l in (lA, lB, lD))
    A = (rng.uniform(-1, 1, int(np.prod(lA))) + 1j * rng.uniform(-1, 1, int(np.prod(lA)))).astype(np.complex128)
    B = (rng.uniform(-1, 1, int(np.prod(lB))) + 1j * rng.uniform(-1, 1, int(np.prod(lB)))).astype(np.complex128)
    D = np.zeros(int(np.prod(lD)), dtype=np.complex128)
    orc.contraction_complex(1.0, A, lA, sA, mA, B, lB, sB, mB, 0.0, None, D, lD, sD, mD, orc.C64F)
    # first-fastest memory = Fortran order
    An = A.reshape(lA[::-1]).transpose(range(len(lA) - 1, -1, -1))
    Bn = B.reshape(lB[::-1]).transpose(range(len(lB) - 1, -1, -1))
    want = np.einsum("kab,ckd->acbd", An, Bn)
    got = D.reshape(lD[::-1]).transpose(range(len(lD) - 1, -1, -1))
    assert np.max(np.abs(got - want)) < 1e-13


@pytest.fixture(scope="module")
def ht():
    import hiptensor_b200

    return hiptensor_b200


def test_planner_rewrites_complex_as_one_real_contraction(ht):
    """cf64 A[m0,m1,k0,k1] (96 x 96 x 32 x 32) times the smaller B[n0,n1,k0,k1]: B is copied (four reals per
    element), the real problem has N and K doubled and runs on the FP64 tensor-pipe kernel; cf32 with 16-byte
    aligned strides runs on the TF32-split tensor-core kernel."""
    lA, lB, lD = [96, 96, 32, 32], [16, 24, 32, 32], [96, 96, 16, 24]
    args = (lA, packed(lA), [0, 1, 4, 5])
    d = ht.describe_contraction_plan(*args, ht.C_64F, lB, packed(lB), [2, 3, 4, 5], ht.C_64F, lD, packed(lD),
                                     [0, 1, 2, 3], ht.C_64F, True, ht.COMPUTE_C64F)
    nB = int(np.prod(lB))
    assert "complex contraction (copy of B: %d bytes)" % (nB * 32) in d, d
    assert "kind=tiled_dmma" in d and "M=9216 N=768 K=2048" in d, d
    d = ht.describe_contraction_plan(*args, ht.C_32F, lB, packed(lB), [2, 3, 4, 5], ht.C_32F, lD, packed(lD),
                                     [0, 1, 2, 3], ht.C_32F, False, ht.COMPUTE_C32F)
    assert "copy of B: %d bytes" % (nB * 16) in d and "kind=tf32x3" in d and "M=9216 N=768 K=2048" in d, d
    # first mode fastest: the in-place operand's real view has no stride-1 row or K mode, so cf32 copies both
    d = ht.describe_contraction_plan(lA, packed(lA, True), [0, 1, 4, 5], ht.C_32F, lB, packed(lB, True), [2, 3, 4, 5],
                                     ht.C_32F, lD, packed(lD, True), [0, 1, 2, 3], ht.C_32F, False, ht.COMPUTE_C32F)
    assert "copy of A and B: %d bytes" % (nB * 16 + int(np.prod(lA)) * 8) in d and "kind=tf32x3" in d, d
    d = ht.describe_contraction_plan(lA, packed(lA, True), [0, 1, 4, 5], ht.C_64F, lB, packed(lB, True), [2, 3, 4, 5],
                                     ht.C_64F, lD, packed(lD, True), [0, 1, 2, 3], ht.C_64F, False, ht.COMPUTE_C64F)
    assert "copy of B:" in d and "kind=tiled_dmma" in d, d
    # the smaller operand is the one copied
    d = ht.describe_contraction_plan(lB, packed(lB), [2, 3, 4, 5], ht.C_32F, lA, packed(lA), [0, 1, 4, 5], ht.C_32F,
                                     lD, packed(lD), [0, 1, 2, 3], ht.C_32F, False, ht.COMPUTE_C32F)
    assert "copy of A" in d, d


def test_planner_complex_type_rules(ht):
    l, s, m = [4, 4], [4, 1], [0, 1]
    ok = dict(lensA=l, stridesA=s, modeA=[0, 2], dtypeA=ht.C_32F, lensB=l, stridesB=s, modeB=[1, 2], dtypeB=ht.C_32F,
              lensD=l, stridesD=s, modeD=m, dtypeD=ht.C_32F, has_c=True, type_compute=ht.COMPUTE_C32F)
    assert "complex contraction" in ht.describe_contraction_plan(**ok)
    for bad in (dict(ok, type_compute=ht.COMPUTE_C64F), dict(ok, dtypeB=ht.C_64F), dict(ok, dtypeD=ht.R_32F),
                dict(ok, type_compute=ht.COMPUTE_32F)):
        with pytest.raises(ht.HiptensorError) as e:
            ht.describe_contraction_plan(**bad)
        assert e.value.status == ht.STATUS_NOT_SUPPORTED
