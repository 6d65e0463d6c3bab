"""Pins the CPU oracle against the known-answer vectors of the reference's own tests
(tests/golden/*.json, extracted by tests/golden/extract_golden.py) and against
closed-form identities."""
import json
import os

import numpy as np

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_permutation_golden_f32(oracle):
    g = json.load(open(os.path.join(GOLD, "permutation_whcn_cnhw.json")))
    ext = g["extent"]
    modeA = [ord(c) for c in g["modeA"]]
    modeB = [ord(c) for c in g["modeB"]]
    lenA = [ext[c] for c in g["modeA"]]
    A = np.arange(120, dtype=np.float32)
    B = np.full(120, np.nan, dtype=np.float32)
    oracle.permutation(g["alpha"], oracle.F32, A, lenA, modeA, oracle.F32, B, modeB, oracle.F32)
    exp = np.array(g["expected_first_mode_fastest"], dtype=np.float32)
    # the reference compares with a relative metric; float(2.1f * i) vs decimal literal
    assert oracle.max_rel_error(B, exp, oracle.F32) < 1e-6
    assert np.allclose(B, exp, rtol=2e-7, atol=0)


def test_permutation_golden_f16(oracle):
    g = json.load(open(os.path.join(GOLD, "permutation_whcn_cnhw.json")))
    ext = g["extent"]
    modeA = [ord(c) for c in g["modeA"]]
    modeB = [ord(c) for c in g["modeB"]]
    lenA = [ext[c] for c in g["modeA"]]
    A = np.arange(120, dtype=np.float16)
    B = np.zeros(120, dtype=np.float16)
    oracle.permutation(g["alpha"], oracle.F16, A, lenA, modeA, oracle.F16, B, modeB, oracle.F16)
    exp = np.array(g["expected_first_mode_fastest"], dtype=np.float16)
    # reference tolerance for f16: 2 * 2^-10 (test/utils.hpp:353-370), scaled by 10 in its CPU test
    assert 0 <= oracle.max_rel_error(B, exp, oracle.F16) < 2 * 2.0 ** -10


def _reduction_case(oracle, dt, ct):
    g = json.load(open(os.path.join(GOLD, "reduction_mhkv_kv.json")))
    ext = g["extent"]
    modeA = [ord(c) for c in g["modeA"]]
    modeC = [ord(c) for c in g["modeC"]]
    lenA = [ext[c] for c in g["modeA"]]
    lenC = [ext[c] for c in g["modeC"]]
    npdt = oracle.np_dtype(dt)
    A = np.arange(int(np.prod(lenA)), dtype=npdt)
    D = np.full(int(np.prod(lenC)), g["C"], dtype=npdt)
    # NULL strides in hiptensorInitTensorDescriptor = last mode fastest (hiptensor.cpp:205)
    oracle.reduction(g["alpha"], A, lenA, oracle.packed_strides(lenA, False), modeA, dt, g["beta"], None, D, lenC,
                     oracle.packed_strides(lenC, False), modeC, dt, oracle.OP_ADD, ct)
    return D, np.array(g["expected_default_build"], dtype=npdt)


def test_reduction_golden_f32(oracle):
    D, exp = _reduction_case(oracle, oracle.F32, oracle.COMPUTE_32F)
    err = oracle.max_rel_error(D, exp, oracle.F32)
    assert 0 <= err < 24 * 15 * np.finfo(np.float32).eps  # reduce_len * eps (reduction_test.cpp:518-543)
    assert np.allclose(D, exp, rtol=1e-6)


def test_reduction_golden_f64(oracle):
    D, exp = _reduction_case(oracle, oracle.F64, oracle.COMPUTE_64F)
    assert np.allclose(D, exp, rtol=1e-12)


def test_fill_generator_known_values(oracle):
    # pcg_hash restated independently in numpy (test/device/common.hpp:68-80)
    def pcg(x):
        x = np.asarray(x, dtype=np.uint64)
        state = (x * 747796405 + 2891336453) & 0xFFFFFFFF
        word = (((state >> ((state >> 28) + 4)) ^ state) * 277803737) & 0xFFFFFFFF
        return ((word >> 22) ^ word) & 0xFFFFFFFF

    n, seed = 1000, 255
    got = oracle.fill_uniform(n, oracle.F32, seed)
    h = pcg((np.arange(n, dtype=np.uint64) + seed) & 0xFFFFFFFF).astype(np.float32)
    exp = (h / np.float32(4294967295.0) - np.float32(0.5)) * np.float32(2.0)
    assert np.array_equal(got, exp.astype(np.float32))
    assert got.min() >= -1.0 and got.max() <= 1.0


def test_contraction_matches_einsum(oracle):
    rng = np.random.default_rng(0)
    # D[m0,m1,n0,n1] = a*A[m0,m1,k0,k1]*B[n0,n1,k0,k1] + b*C  (first-mode-fastest strides)
    e = 5
    lens = [e, e + 1, e + 2, e + 3]
    m0, m1, n0, n1, k0, k1 = 0, 1, 2, 3, 4, 5
    ext = {m0: 3, m1: 4, n0: 5, n1: 2, k0: 6, k1: 3}
    mA, mB, mD = [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1]
    lA, lB, lD = [ext[m] for m in mA], [ext[m] for m in mB], [ext[m] for m in mD]
    sA, sB, sD = (oracle.packed_strides(l, True) for l in (lA, lB, lD))
    A = rng.uniform(-1, 1, int(np.prod(lA))).astype(np.float64)
    B = rng.uniform(-1, 1, int(np.prod(lB))).astype(np.float64)
    C = rng.uniform(-1, 1, int(np.prod(lD))).astype(np.float64)
    D = np.full_like(C, np.nan)
    oracle.contraction(2.0, A, lA, sA, mA, oracle.F64, B, lB, sB, mB, oracle.F64, 0.5, C, D, lD, sD, mD,
                       oracle.F64, oracle.COMPUTE_64F)
    At = A.reshape(lA[::-1]).transpose(3, 2, 1, 0)  # index [m0,m1,k0,k1]
    Bt = B.reshape(lB[::-1]).transpose(3, 2, 1, 0)
    Ct = C.reshape(lD[::-1]).transpose(3, 2, 1, 0)
    ref = 2.0 * np.einsum("abkl,cdkl->abcd", At, Bt) + 0.5 * Ct
    got = D.reshape(lD[::-1]).transpose(3, 2, 1, 0)
    assert np.allclose(got, ref, rtol=1e-12, atol=1e-12)
    # sampled evaluation agrees with the full one
    D2 = np.full_like(C, np.nan)
    smp = np.array([0, 7, 33, len(C) - 1])
    oracle.contraction(2.0, A, lA, sA, mA, oracle.F64, B, lB, sB, mB, oracle.F64, 0.5, C, D2, lD, sD, mD,
                       oracle.F64, oracle.COMPUTE_64F, sample=smp)
    assert np.array_equal(D2[smp], D[smp]) and np.isnan(D2).sum() == len(C) - len(smp)


def test_reduction_max_and_nan(oracle):
    lenA, modeA, modeD = [4, 3, 5], [0, 1, 2], [0]
    A = np.arange(60, dtype=np.float32)
    A[17] = np.nan
    D = np.zeros(4, dtype=np.float32)
    C = np.ones(4, dtype=np.float32)
    oracle.reduction(1.0, A, lenA, oracle.packed_strides(lenA, False), modeA, oracle.F32, 0.5, C, D, [4], [1],
                     modeD, oracle.F32, oracle.OP_MAX, oracle.COMPUTE_32F)
    assert D[0] == 14.5 and np.isnan(D[1]) and D[2] == 44.5 and D[3] == 59.5
