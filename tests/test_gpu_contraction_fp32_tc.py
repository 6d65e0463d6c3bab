"""GPU parity of the fp32 tensor-core contraction (big/small TF32 split, three MMAs per K step) through the
C ABI against the CPU oracle.

The reference runs fp32 contractions on its matrix cores with fp32 accuracy
(library/src/contraction/device/*f32_f32_f32_f32*_instance.cpp) and accepts 2*K*eps under its metric
max|d-h|/(|d|+|h|+1) (test/01_contraction/contraction_test.cpp:882-905). The split path is held to the same
tolerance as the FMA kernel: the reference's bound 2*K*eps against the reference's CPU algorithm, and 1e-5
against the exact (fp64) result. (The tensor cores add product groups to an fp32 accumulator with truncation;
the kernel keeps that harmless by accumulating the main product over 64 K elements at a time and summing
those segments in registers with round-to-nearest, see contraction_tf32x3.cu.)

Layouts: the reference's kernels come in four variants by which of A/B has K or M/N fastest
(contraction_solution_instances.cpp:40-106); all four are exercised here, with rows gathered over
several modes, ragged extents and K tails."""
import os

import numpy as np
import pytest

from helpers import SEED_CONTRACTION, check_f32, rel_error, run_contraction, set_switch
from oracle import binding as orc

pytestmark = pytest.mark.gpu
EPS = float(np.finfo(np.float32).eps)


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


def exact_f64(ext, modeA, modeB, modeD, alpha, beta, first_fastest):
    """The same seeded fp32 problem evaluated by the oracle with fp64 data and accumulation."""
    lA, lB, lD = ([ext[m] for m in ms] for ms in (modeA, modeB, modeD))
    sA, sB, sD = (orc.packed_strides(l, first_fastest) for l in (lA, lB, lD))
    n = [int(np.prod(l)) for l in (lA, lB, lD)]
    A = orc.to_f64(orc.fill_uniform(n[0], orc.F32, SEED_CONTRACTION[0]), orc.F32)
    B = orc.to_f64(orc.fill_uniform(n[1], orc.F32, SEED_CONTRACTION[1]), orc.F32)
    C = orc.to_f64(orc.fill_uniform(n[2], orc.F32, SEED_CONTRACTION[2]), orc.F32)
    D = np.full(n[2], np.nan)
    orc.contraction(alpha, A, lA, sA, modeA, orc.F64, B, lB, sB, modeB, orc.F64, beta, C, D, lD, sD, modeD, orc.F64,
                    orc.COMPUTE_64F)
    return D


def run_and_check(env, ext, modeA, modeB, modeD, K, alpha=1.0, beta=0.0, first_fastest=False, kernel=None):
    ht, h = env
    got, exp, td = run_contraction(ht, h, ext, modeA, modeB, modeD, typeAB=orc.F32, alpha=alpha, beta=beta,
                                   with_c=beta != 0.0, first_fastest=first_fastest)
    name = ht.last_kernel_name()
    assert name == kernel if kernel else name.startswith("contraction_tf32x3"), name
    assert not np.isnan(got).any()
    exact = exact_f64(ext, modeA, modeB, modeD, alpha, beta, first_fastest)
    return check_f32(got, exp, exact, 2 * K)


# A / B mode orders (last mode fastest) for the four layout variants of D[m, n]
LAYOUTS = {"kk": ([0, 2], [1, 2]), "mn_mn": ([2, 0], [2, 1]), "k_mn": ([0, 2], [2, 1]), "mn_k": ([2, 0], [1, 2])}


@pytest.mark.parametrize("layout", sorted(LAYOUTS))
@pytest.mark.parametrize("shape", [(128, 64, 32), (256, 320, 96), (384, 1000, 136), (200, 132, 72)])
def test_plain_matrices(env, layout, shape):
    """All four operand layouts; ragged M, N and a K tail (extents stay multiples of 4: TMA needs 16-byte
    strides). Single CTAs or CTA pairs as the launcher sees fit."""
    M, N, K = shape
    modeA, modeB = LAYOUTS[layout]
    run_and_check(env, {0: M, 1: N, 2: K}, modeA, modeB, [0, 1], K, alpha=1.5, beta=0.5)
    # M-fastest output: the planner exchanges the operands
    if N >= 128:
        run_and_check(env, {0: M, 1: N, 2: K}, modeA, modeB, [1, 0], K, alpha=1.0, beta=0.0)


def test_config1_layout_runs_on_tensor_cores(env):
    """All extents 24, first mode fastest (folded 576^3, both operands and D M/N-major)."""
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m: 24 for m in range(6)}
    run_and_check(env, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], 576, alpha=1.0, beta=1.0,
                  first_fastest=True)


def test_gathered_rows_k_major(env):
    """K-major operands whose tile rows span two modes (power-of-two inner mode, ragged outer mode), interleaved
    output modes: one TMA box gathers the rows."""
    m0, m1, n0, n1, k0 = range(5)
    ext = {m0: 12, m1: 16, n0: 32, n1: 6, k0: 200}
    run_and_check(env, ext, [m0, m1, k0], [n1, n0, k0], [m1, n1, m0, n0], 200, alpha=1.5, beta=0.5)


def test_chunked_rows_two_k_modes(env):
    """M/N-major operands: 32-row chunks along a ragged stride-1 mode (40, 72), a second row mode, and two K modes
    that do not fold (16 x 6, gathered by a two-dimensional K box)."""
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m0: 40, m1: 5, n0: 72, n1: 3, k0: 16, k1: 6}
    run_and_check(env, ext, [k1, m1, k0, m0], [k1, n1, k0, n0], [m1, n1, m0, n0], 96, alpha=2.0, beta=0.25)
    # the same with D's stride-1 mode on the other operand (operands exchanged by the planner)
    run_and_check(env, ext, [k1, m1, k0, m0], [k1, n1, k0, n0], [n1, m1, n0, m0], 96, alpha=1.0, beta=1.0)


@pytest.mark.parametrize("layout", sorted(LAYOUTS))
def test_cta_pair_kernel_forced(env, layout):
    """256 x 256 tiles on CTA pairs, forced on a problem with an odd number of 128-row sub-tiles along M and N
    (the last pair repeats a sub-tile and must not store it twice)."""
    modeA, modeB = LAYOUTS[layout]
    set_switch("HTB_TF32_PAIR", True)
    try:
        run_and_check(env, {0: 640, 1: 896, 2: 104}, modeA, modeB, [0, 1], 104, alpha=0.5, beta=2.0,
                      kernel="contraction_tf32x3_pair")
    finally:
        set_switch("HTB_TF32_PAIR", False)


@pytest.mark.parametrize("layout", ["kk", "mn_mn"])
@pytest.mark.parametrize("pair", [False, True])
def test_large_sampled(env, layout, pair):
    """Several tiles per CTA (the rings, segment accumulators and correction accumulators wrap around many times);
    checked on 4096 sampled outputs. Single CTAs (the default) and CTA pairs."""
    ht, h = env
    M, N, K = 2048, 2560, 512
    modeA, modeB = LAYOUTS[layout]
    smp = np.random.default_rng(11).integers(0, M * N, 4096)
    if pair:
        set_switch("HTB_TF32_PAIR", True)
    try:
        got, exp, td = run_contraction(ht, h, {0: M, 1: N, 2: K}, modeA, modeB, [0, 1], typeAB=orc.F32, alpha=1.0,
                                       beta=0.5, sample=smp)
    finally:
        set_switch("HTB_TF32_PAIR", False)
    assert ht.last_kernel_name() == ("contraction_tf32x3_pair" if pair else "contraction_tf32x3")
    assert not np.isnan(got).any()
    err = rel_error(got, exp, td)
    assert 0 <= err < 2 * K * EPS, err


def test_unaligned_or_small_problems_keep_the_fma_kernel(env):
    """Strides that are not multiples of 16 bytes, or tiles too small, stay on the gathered FMA kernel."""
    ht, h = env
    got, exp, td = run_contraction(ht, h, {0: 130, 1: 70, 2: 34}, [0, 2], [1, 2], [0, 1], typeAB=orc.F32)
    assert ht.last_kernel_name() == "contraction_tiled_simt"
    assert 0 <= rel_error(got, exp, td) < 1e-5
    got, exp, td = run_contraction(ht, h, {0: 64, 1: 64, 2: 64}, [0, 2], [1, 2], [0, 1], typeAB=orc.F32)
    assert ht.last_kernel_name() == "contraction_tiled_simt"
    assert 0 <= rel_error(got, exp, td) < 1e-5


@pytest.mark.parametrize("compute", [orc.COMPUTE_16F, orc.COMPUTE_16BF])
@pytest.mark.parametrize("layout", sorted(LAYOUTS))
def test_f32_data_with_half_precision_compute(env, compute, layout):
    """fp32 tensors with compute type f16 / bf16 (reference tuples f32,f32,f32 with ComputeT half / bhalf,
    contraction_cpu_reference_instances.cpp): every element is rounded to the compute type, products and sums are
    fp32. The kernel rounds in its converter and issues one TF32 MMA per K step (the rounded values are exact in
    TF32), so only the summation order differs from the reference's CPU loop."""
    ht, h = env
    modeA, modeB = LAYOUTS[layout]
    for M, N, K in ((256, 320, 96), (384, 1000, 136)):
        got, exp, td = run_contraction(ht, h, {0: M, 1: N, 2: K}, modeA, modeB, [0, 1], typeAB=orc.F32, compute=compute,
                                       alpha=1.5, beta=0.5)
        assert ht.last_kernel_name().startswith("contraction_tf32x3"), ht.last_kernel_name()
        assert not np.isnan(got).any()
        err = rel_error(got, exp, td)
        assert 0 <= err < 1e-5, (compute, layout, (M, N, K), err)


@pytest.mark.parametrize("layout", sorted(LAYOUTS))
def test_k_split_of_small_problems(env, layout):
    """Few tiles and a long K: every tile is cut into K ranges (the CTAs of one cluster), the partial sums travel
    through the owner's shared memory and are added in a fixed order; no workspace is involved. Split and whole
    results must both satisfy the bounds; the split one must be reproducible bit for bit."""
    ht, h = env
    modeA, modeB = LAYOUTS[layout]
    M, N, K = 256, 192, 1024
    ext = {0: M, 1: N, 2: K}
    lA, lB, lD = ([ext[m] for m in ms] for ms in (modeA, modeB, [0, 1]))
    dA, dB, dD = (h.tensor_descriptor(l, None, ht.R_32F) for l in (lA, lB, lD))
    cd = h.contraction_descriptor(dA, modeA, dB, modeB, dD, [0, 1], dD, [0, 1], ht.COMPUTE_32F)
    find = h.contraction_find()
    assert h.contraction_workspace_size(cd, find, ht.WORKSPACE_RECOMMENDED) == 0
    assert "splitK=4" in ht.describe_contraction_plan(lA, orc.packed_strides(lA, False), modeA, ht.R_32F, lB,
                                                      orc.packed_strides(lB, False), modeB, ht.R_32F, lD,
                                                      orc.packed_strides(lD, False), [0, 1], ht.R_32F, True,
                                                      ht.COMPUTE_32F)
    first = None
    for _ in range(2):
        got, exp, td = run_contraction(ht, h, ext, modeA, modeB, [0, 1], typeAB=orc.F32, alpha=1.5, beta=0.5)
        assert ht.last_kernel_name() == "contraction_tf32x3"
        assert not np.isnan(got).any()
        exact = exact_f64(ext, modeA, modeB, [0, 1], 1.5, 0.5, False)
        check_f32(got, exp, exact, 2 * K)
        if first is None:
            first = got.copy()
    assert np.array_equal(first.view(np.uint32), got.view(np.uint32))
    set_switch("HTB_TF32_NOSPLIT", True)
    try:
        whole, exp, td = run_contraction(ht, h, ext, modeA, modeB, [0, 1], typeAB=orc.F32, alpha=1.5, beta=0.5)
    finally:
        set_switch("HTB_TF32_NOSPLIT", False)
    assert 0 <= rel_error(whole, first, orc.F32) < 1e-5
