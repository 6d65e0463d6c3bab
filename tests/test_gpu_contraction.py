"""GPU parity: hiptensorContraction through the C ABI against the CPU oracle.

Metric: the reference's max|d-h|/(|d|+|h|+1) (test/device/common.hpp:122-151).
Tolerances: 1e-5 for fp32/fp64 accumulation, 1e-2 for f16/bf16 inputs;
next to them the reference's own bound 2*K*eps (+2*2^-10 f16, +2*2^-7 bf16 outputs),
test/01_contraction/contraction_test.cpp:882-905, is checked where it is the stricter one.
Mode lists and extents of the shuffled cases are those of
test/01_contraction/configs/mode_test_params.yaml:15-59."""
import os

import numpy as np
import pytest

from helpers import check_f32, rel_error, run_contraction, set_switch
from oracle import binding as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def pairs_wherever_possible():
    """The library takes CTA pairs (256 x 256 tiles) only from about two waves of pairs on; this module runs the
    pair kernel on small problems too (odd tile counts, K split, half tiles), as HTB_TC_PAIR allows."""
    set_switch("HTB_TC_PAIR", True)
    yield
    set_switch("HTB_TC_PAIR", False)


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


def ext_of(modes, lens):
    return {m: l for ms, ls in zip(modes, lens) for m, l in zip(ms, ls)}



def exact_f64(ext, modeA, modeB, modeD, dt, alpha, beta, first_fastest, fill="uniform"):
    """The same seeded problem evaluated by the oracle with fp64 data and accumulation."""
    from helpers import SEED_CONTRACTION as S

    lA, lB, lD = ([ext[m] for m in ms] for ms in (modeA, modeB, modeD))
    sA, sB, sD = (orc.packed_strides(l, first_fastest) for l in (lA, lB, lD))
    n = [int(np.prod(l)) for l in (lA, lB, lD)]
    gen = (lambda k, d, s: orc.fill_uniform(k, d, s)) if fill == "uniform" else (
        lambda k, d, s: orc.fill_normal(k, d, s, 0.5))
    A = orc.to_f64(gen(n[0], dt, S[0]), dt)
    B = orc.to_f64(gen(n[1], dt, S[1]), dt)
    C = orc.to_f64(orc.fill_uniform(n[2], dt, S[2]), dt)
    D = np.full(n[2], np.nan)
    orc.contraction(alpha, A, lA, sA, modeA, orc.F64, B, lB, sB, modeB, orc.F64, beta, C, D, lD, sD, modeD, orc.F64,
                    orc.COMPUTE_64F)
    return D


# (lengths of A, B, D) and (modes of A, B, D)
MODE_CASES = [
    ([[3, 2, 3, 3, 4, 3, 1, 2, 4, 5, 3, 5], [2, 4, 3, 3, 1, 4, 1, 2, 4, 5, 3, 5], [3, 2, 3, 3, 4, 3, 2, 4, 3, 3, 1, 4]],
     [[0, 1, 2, 3, 4, 5, 12, 13, 14, 15, 16, 17], [6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17],
      [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]]),
    ([[3, 2, 3, 3, 4, 3, 3], [2, 4, 3, 3, 1, 4, 3], [3, 2, 3, 3, 4, 3, 2, 4, 3, 3, 1, 4]],
     [[0, 1, 2, 3, 4, 5, 16], [6, 7, 8, 9, 10, 11, 16], [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]]),
    ([[3, 3], [2, 3], [3, 2]], [[0, 16], [6, 16], [0, 6]]),
    ([[3, 1, 2, 2, 3, 4, 3, 5, 4, 3, 3, 5], [2, 1, 4, 2, 3, 4, 3, 5, 1, 3, 4, 5], [3, 2, 2, 4, 3, 3, 3, 3, 4, 1, 3, 4]],
     [[0, 12, 1, 13, 2, 14, 3, 15, 4, 16, 5, 17], [6, 12, 7, 13, 8, 14, 9, 15, 10, 16, 11, 17],
      [0, 6, 1, 7, 2, 8, 3, 9, 4, 10, 5, 11]]),
    ([[3, 3, 4, 3, 2, 5, 1, 2, 5, 3, 3, 4], [2, 5, 1, 4, 4, 2, 4, 5, 3, 3, 1, 3], [3, 4, 3, 1, 3, 3, 3, 4, 3, 2, 4, 2]],
     [[5, 2, 14, 16, 13, 15, 12, 1, 17, 3, 0, 4], [13, 15, 12, 11, 7, 6, 14, 17, 16, 8, 10, 9],
      [8, 4, 9, 10, 2, 5, 3, 7, 0, 1, 11, 6]]),
]


@pytest.mark.parametrize("case", range(len(MODE_CASES)))
@pytest.mark.parametrize("dt", [orc.F32, orc.F64])
def test_mode_orders(env, case, dt):
    ht, h = env
    lens, modes = MODE_CASES[case]
    ext = ext_of(modes, lens)
    K = int(np.prod([ext[m] for m in modes[0] if m in modes[1]]))
    for ab in ((1.0, 2.0), (1.0, 0.0), (0.0, 2.0)):
        got, exp, td = run_contraction(ht, h, ext, modes[0], modes[1], modes[2], typeAB=dt, alpha=ab[0], beta=ab[1])
        if dt == orc.F32:
            exact = exact_f64(ext, modes[0], modes[1], modes[2], dt, ab[0], ab[1], False)
            check_f32(got, exp, exact, 2 * K)
        else:
            err = rel_error(got, exp, td)
            assert 0 <= err < 1e-5, (case, dt, ab, err, ht.last_kernel_name())


@pytest.mark.parametrize("dt,ct", [(orc.F32, orc.COMPUTE_32F), (orc.F32, orc.COMPUTE_16F), (orc.F32, orc.COMPUTE_16BF),
                                   (orc.F64, orc.COMPUTE_64F), (orc.F64, orc.COMPUTE_32F)])
@pytest.mark.parametrize("with_c", [True, False])
def test_rank2_type_tuples(env, dt, ct, with_c):
    """2M2N2K shapes of the reference's validation lists (bilinear/scale_test_params_rank2.yaml)."""
    ht, h = env
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m0: 5, m1: 6, n0: 3, n1: 4, k0: 7, k1: 8}
    for ff in (False, True):
        got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=dt,
                                       compute=ct, alpha=1.1, beta=2.2 if with_c else 0.0, with_c=with_c,
                                       first_fastest=ff)
        err = rel_error(got, exp, td)
        # f64 data with f32 compute accumulates in float on both sides
        assert 0 <= err < 1e-5, (dt, ct, with_c, ff, err)


@pytest.mark.parametrize("dt", [orc.F16, orc.BF16])
@pytest.mark.parametrize("out32", [False, True])
def test_half_inputs_small(env, dt, out32):
    ht, h = env
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m0: 6, m1: 5, n0: 4, n1: 7, k0: 8, k1: 3}
    got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=dt,
                                   typeD=orc.F32 if out32 else dt, alpha=1.0, beta=1.0)
    err = rel_error(got, exp, td)
    tol = 1e-5 if out32 else (2 * 2.0 ** -10 if dt == orc.F16 else 2 * 2.0 ** -7)
    assert 0 <= err < tol, (dt, out32, err)


def test_config1_fp32_bilinear(env):
    """D[m0,m1,n0,n1] = 1.0*A[m0,m1,k0,k1]*B[n0,n1,k0,k1] + 1.0*C, all extents 24, first mode fastest.

    Two statements. Against the reference's CPU algorithm (fp32 accumulation in its own k order) the
    reference's own bound 2*K*eps holds; two fp32 summation orders of 576 terms differ by more than
    1e-5 under the metric, so the 1e-5 bound is checked against the same contraction evaluated by
    the oracle in fp64 (inputs widened exactly), i.e. against the exact product."""
    ht, h = env
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m: 24 for m in range(6)}
    got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=orc.F32,
                                   alpha=1.0, beta=1.0, first_fastest=True)
    exact = exact_f64(ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], orc.F32, 1.0, 1.0, True)
    check_f32(got, exp, exact, 2 * 576)


def test_config5_scaled_down(env):
    """fp64 3M2N2K with interleaved modes at extents m=4, n=12, k=12: whole tensor against the oracle."""
    ht, h = env
    m0, m1, m2, n0, n1, k0, k1 = range(7)
    ext = {m0: 4, m1: 4, m2: 4, n0: 12, n1: 12, k0: 12, k1: 12}
    got, exp, td = run_contraction(ht, h, ext, [m0, k0, m1, k1, m2], [k1, n0, k0, n1], [m0, m1, m2, n0, n1],
                                   typeAB=orc.F64, alpha=2.0, beta=0.5)
    err = rel_error(got, exp, td)
    assert 0 <= err < 1e-12, err
    assert ht.last_kernel_name() == "contraction_tiled_dmma"


F64_LAYOUTS = {"kk": ([0, 2], [1, 2]), "mn_mn": ([2, 0], [2, 1]), "k_mn": ([0, 2], [2, 1]), "mn_k": ([2, 0], [1, 2])}


@pytest.mark.parametrize("layout", sorted(F64_LAYOUTS))
@pytest.mark.parametrize("shape", [(256, 192, 96), (200, 132, 72), (130, 70, 34), (129, 67, 35), (64, 64, 8),
                                   (200, 132, 520), (129, 67, 131), (520, 260, 2050)])
def test_fp64_operand_layouts(env, layout, shape):
    """fp64 on the FP64 tensor pipe with each operand contiguous along K or along its rows. Even extents take the
    16-byte asynchronous copies (pairs along the contiguous direction), odd ones the 8-byte copies; ragged M, N
    and K tails (K not a multiple of the 16-wide step, shorter than the copy ring) are zero-filled. The last three
    shapes have few tiles and a long K: their K steps are cut over clusters of four or two CTAs (uneven ranges,
    ragged last step) that exchange accumulators through shared memory."""
    ht, h = env
    M, N, K = shape
    modeA, modeB = F64_LAYOUTS[layout]
    got, exp, td = run_contraction(ht, h, {0: M, 1: N, 2: K}, modeA, modeB, [0, 1], typeAB=orc.F64, alpha=1.5, beta=0.5)
    assert ht.last_kernel_name() == "contraction_tiled_dmma"
    assert not np.isnan(got).any()
    err = rel_error(got, exp, td)
    assert 0 <= err < 1e-12, (layout, shape, err)
    # D contiguous along M: the planner exchanges the operands
    got, exp, td = run_contraction(ht, h, {0: M, 1: N, 2: K}, modeA, modeB, [1, 0], typeAB=orc.F64, alpha=1.0, beta=0.0)
    err = rel_error(got, exp, td)
    assert 0 <= err < 1e-12, (layout, shape, err)


def test_fp64_unaligned_base_and_strided_rows(env):
    """Operands that start 8 bytes past a 16-byte boundary (8-byte copies) and rows with padding between them
    (even strides: 16-byte copies stay legal)."""
    import torch

    from helpers import to_device

    ht, h = env
    M, N, K = 96, 80, 48
    for pad, shift in ((0, 1), (2, 0), (3, 0)):
        sA, sB, sD = [K + pad, 1], [K + pad, 1], [N, 1]
        nA, nB = M * (K + pad), N * (K + pad)
        A = orc.fill_uniform(nA + shift, orc.F64, 255)
        B = orc.fill_uniform(nB + shift, orc.F64, 256)
        dA, dB, dD = (h.tensor_descriptor(l, s, ht.R_64F) for l, s in (([M, K], sA), ([N, K], sB), ([M, N], sD)))
        cd = h.contraction_descriptor(dA, [0, 2], dB, [1, 2], None, None, dD, [0, 1], ht.COMPUTE_64F)
        find = h.contraction_find()
        plan = h.contraction_plan(cd, find, 0)
        A_d, B_d = to_device(A, orc.F64), to_device(B, orc.F64)
        D_d = torch.full((M * N,), float("nan"), dtype=torch.float64, device="cuda")
        h.contraction(plan, 2.0, A_d[shift:], B_d[shift:], 0.0, None, D_d)
        exp = np.full(M * N, np.nan)
        orc.contraction(2.0, A[shift:], [M, K], sA, [0, 2], orc.F64, B[shift:], [N, K], sB, [1, 2], orc.F64, 0.0, None,
                        exp, [M, N], sD, [0, 1], orc.F64, orc.COMPUTE_64F)
        err = rel_error(D_d.cpu().numpy(), exp, orc.F64)
        assert 0 <= err < 1e-12, (pad, shift, err)


def test_config5_full_size_sampled(env):
    """fp64 M=4096, N=K=2304: 4096 sampled outputs against the exact-order oracle."""
    ht, h = env
    m0, m1, m2, n0, n1, k0, k1 = range(7)
    ext = {m0: 16, m1: 16, m2: 16, n0: 48, n1: 48, k0: 48, k1: 48}
    rng = np.random.default_rng(5)
    smp = rng.integers(0, 16 ** 3 * 48 ** 2, 4096)
    got, exp, td = run_contraction(ht, h, ext, [m0, k0, m1, k1, m2], [k1, n0, k0, n1], [m0, m1, m2, n0, n1],
                                   typeAB=orc.F64, alpha=2.0, beta=0.5, sample=smp)
    err = rel_error(got, exp, td)
    assert 0 <= err < 2 * 2304 * np.finfo(np.float64).eps, err
    assert not np.isnan(got).any()


def test_config4_scaled_down(env):
    """f16 x f16 -> f32, k modes innermost, extents 16 (M=N=K=256): whole tensor."""
    ht, h = env
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m: 16 for m in range(6)}
    got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=orc.F16,
                                   typeD=orc.F32, alpha=1.0, beta=0.0, with_c=False, fill="normal")
    err = rel_error(got, exp, td)
    assert 0 <= err < 1e-2, err
    assert err < 1e-4


def test_config4_full_size_sampled(env):
    """f16 inputs, fp32 output, extents 64 (M=N=K=4096): 8192 sampled outputs, plus linearity in alpha."""
    ht, h = env
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m: 64 for m in range(6)}
    rng = np.random.default_rng(4)
    smp = rng.integers(0, 64 ** 4, 8192)
    got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=orc.F16,
                                   typeD=orc.F32, alpha=1.0, beta=0.0, with_c=False, fill="normal", sample=smp)
    err = rel_error(got, exp, td)
    assert 0 <= err < 1e-2, err
    assert not np.isnan(got).any()
    assert ht.last_kernel_name() == "contraction_tcgen05_pair_wide"
    got2, _, _ = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=orc.F16,
                                 typeD=orc.F32, alpha=2.0, beta=0.0, with_c=False, fill="normal", sample=smp[:8])
    assert np.array_equal(got2, 2.0 * got)  # scaling by a power of two is exact


def test_argument_errors(env):
    import torch

    ht, h = env
    d = h.tensor_descriptor([4, 4], None, ht.R_32F)
    x = torch.zeros(16, device="cuda")
    # a mode of D that neither A nor B has
    cd = h.contraction_descriptor(d, [0, 1], d, [2, 1], d, [0, 3], d, [0, 3], ht.COMPUTE_32F)
    with pytest.raises(ht.HiptensorError) as e:
        h.contraction_plan(cd, h.contraction_find())
    assert e.value.status == ht.STATUS_INVALID_VALUE
    # unsupported type tuple: f32 data with f64 compute
    cd = h.contraction_descriptor(d, [0, 1], d, [2, 1], d, [0, 2], d, [0, 2], ht.COMPUTE_64F)
    with pytest.raises(ht.HiptensorError) as e:
        h.contraction_plan(cd, h.contraction_find())
    assert e.value.status == ht.STATUS_NOT_SUPPORTED
    with pytest.raises(ht.HiptensorError) as e:
        h.contraction_find(123)
    assert e.value.status == ht.STATUS_INVALID_VALUE
    cd = h.contraction_descriptor(d, [0, 1], d, [2, 1], d, [0, 2], d, [0, 2], ht.COMPUTE_32F)
    plan = h.contraction_plan(cd, h.contraction_find())
    with pytest.raises(ht.HiptensorError) as e:
        h.contraction(plan, 1.0, None, x, 0.0, x, x)
    assert e.value.status == ht.STATUS_INVALID_VALUE


@pytest.mark.parametrize("dt", [orc.F16, orc.BF16])
def test_tensor_core_path_gathered_tiles(env, dt):
    """K-major operands whose tile rows span two modes (power-of-two inner mode, ragged outer mode),
    K not a multiple of the 64-wide K block, interleaved output modes: the TMA boxes gather the rows."""
    ht, h = env
    m0, m1, n0, n1, k0 = range(5)
    ext = {m0: 12, m1: 16, n0: 32, n1: 6, k0: 192 + 8}
    for out32 in (True, False):
        got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0], [n1, n0, k0], [m1, n1, m0, n0], typeAB=dt,
                                       typeD=orc.F32 if out32 else dt, alpha=1.5, beta=0.5, fill="normal")
        assert ht.last_kernel_name() == "contraction_tcgen05"
        err = rel_error(got, exp, td)
        tol = 1e-4 if out32 else (2 * 2.0 ** -10 if dt == orc.F16 else 2 * 2.0 ** -7)
        assert 0 <= err < tol, (dt, out32, err)


@pytest.mark.parametrize("shape", [(256, 320, 96), (128, 64, 64), (384, 1000, 520), (640, 896, 200), (1024, 512, 64)])
def test_tensor_core_path_plain_matrices(env, shape):
    ht, h = env
    M, N, K = shape
    m, n, k = 0, 1, 2
    ext = {m: M, n: N, k: K}
    for with_c in (True, False):
        got, exp, td = run_contraction(ht, h, ext, [m, k], [n, k], [m, n], typeAB=orc.F16, typeD=orc.F16, alpha=1.0,
                                       beta=2.0 if with_c else 0.0, with_c=with_c, fill="normal")
        assert ht.last_kernel_name() == ("contraction_tcgen05_pair" if min(M, N) >= 512 else "contraction_tcgen05")
        err = rel_error(got, exp, td)
        assert 0 <= err < 2 * 2.0 ** -10, (shape, with_c, err)
    # M-major output: the planner exchanges the operands
    got, exp, td = run_contraction(ht, h, ext, [m, k], [n, k], [n, m], typeAB=orc.BF16, typeD=orc.F32, alpha=1.0,
                                   beta=1.0, fill="normal")
    if N >= 128:  # after the exchange the 128-row tile runs along the original N
        assert ht.last_kernel_name().startswith("contraction_tcgen05")
    assert 0 <= rel_error(got, exp, td) < 1e-4


@pytest.mark.parametrize("shape", [(256, 256, 2048), (384, 200, 1096), (128, 1000, 776), (640, 384, 520)])
@pytest.mark.parametrize("out", [orc.F32, orc.F16])
def test_single_cta_kernel_k_split_over_a_cluster(env, shape, out):
    """Few tiles and a long K on the single-CTA kernel: the K blocks of a tile are cut over the 2-4 CTAs of a
    cluster (uneven ranges, ragged last block), parts 1.. hand their accumulators to part 0 through its shared
    memory. Results must satisfy the usual bounds, be reproducible bit for bit, and agree with the unsplit run."""
    ht, h = env
    M, N, K = shape
    ext = {0: M, 1: N, 2: K}
    runs = []
    for _ in range(2):
        got, exp, td = run_contraction(ht, h, ext, [0, 2], [1, 2], [0, 1], typeAB=orc.F16, typeD=out, alpha=1.5, beta=0.5,
                                       fill="normal")
        assert ht.last_kernel_name() == "contraction_tcgen05"
        err = rel_error(got, exp, td)
        assert 0 <= err < (1e-4 if out == orc.F32 else 2 * 2.0 ** -10), (shape, out, err)
        runs.append(got)
    assert runs[0].tobytes() == runs[1].tobytes()
    set_switch("HTB_TC_NOSPLIT", True)
    try:
        whole, exp, td = run_contraction(ht, h, ext, [0, 2], [1, 2], [0, 1], typeAB=orc.F16, typeD=out, alpha=1.5, beta=0.5,
                                         fill="normal")
    finally:
        set_switch("HTB_TC_NOSPLIT", False)
    # two summation orders of the tensor cores' fp32 accumulation: the bound of the comparison with the oracle
    assert 0 <= rel_error(whole, runs[0], td) < (1e-4 if out == orc.F32 else 2 * 2.0 ** -10)


@pytest.mark.parametrize("dt", [orc.F16, orc.BF16])
def test_cta_pair_kernel_gathered_odd_tiles(env, dt):
    """256 x 256 tiles over CTA pairs with an odd number of 128-row sub-tiles along M and N (the last
    pair repeats a sub-tile and must not store it twice) and rows gathered from two modes."""
    ht, h = env
    m0, m1, n0, n1, k0 = range(5)
    ext = {m0: 40, m1: 16, n0: 32, n1: 20, k0: 136}
    got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0], [n1, n0, k0], [m1, n1, m0, n0], typeAB=dt,
                                   typeD=orc.F32, alpha=0.5, beta=2.0, fill="normal")
    assert ht.last_kernel_name() == "contraction_tcgen05_pair"
    err = rel_error(got, exp, td)
    assert 0 <= err < 1e-4, (dt, err)
    assert not np.isnan(got).any()


@pytest.mark.parametrize("shape", [(512, 768, 4096), (640, 896, 4104), (512, 512, 8192), (768, 1280, 2048)])
@pytest.mark.parametrize("wide", [False, True])
def test_cta_pair_kernel_k_split(env, shape, wide):
    """Few tiles and a long K on the pair kernel: a cluster is four CTAs, each pair takes half of the K blocks of the
    tile (uneven halves, ragged last block, odd sub-tile counts), and the CTAs that hold the same rows exchange
    halves of their partial sums through shared memory. No workspace is involved. The result must match the oracle,
    be reproducible bit for bit, and agree closely with the unsplit run."""
    ht, h = env
    M, N, K = shape
    m, n, k = 0, 1, 2
    ext = {m: M, n: N, k: K}
    smp = np.random.default_rng(7).integers(0, M * N, 4096)
    name = "contraction_tcgen05_pair_wide" if wide else "contraction_tcgen05_pair"
    set_switch("HTB_TC_KSPLIT", True)
    set_switch("HTB_TC_WIDE" if wide else "HTB_TC_NARROW", True)
    try:
        runs = []
        for _ in range(2):
            got, exp, td = run_contraction(ht, h, ext, [m, k], [n, k], [m, n], typeAB=orc.F16, typeD=orc.F32, alpha=1.5,
                                           beta=0.5, fill="normal", sample=smp)
            assert ht.last_kernel_name() == name
            assert not np.isnan(got).any()
            # stated tolerance for f16 inputs is 1e-2; over 2048-8192 terms the tensor cores' truncating fp32
            # accumulation stays within 5e-4 of the reference's sequential fp32 sum
            assert 0 <= rel_error(got, exp, td) < 5e-4
            runs.append(got)
        assert runs[0].tobytes() == runs[1].tobytes()
        assert h.device_status() == 0
        set_switch("HTB_TC_NOSPLIT", True)
        unsplit, _, _ = run_contraction(ht, h, ext, [m, k], [n, k], [m, n], typeAB=orc.F16, typeD=orc.F32, alpha=1.5,
                                        beta=0.5, fill="normal", sample=smp[:1])
        assert ht.last_kernel_name() == name
    finally:
        for sw in ("HTB_TC_KSPLIT", "HTB_TC_WIDE", "HTB_TC_NARROW", "HTB_TC_NOSPLIT"):
            set_switch(sw, False)
    # regrouping 2048-8192 terms of the truncating fp32 accumulation moves results by up to 5e-4 under the metric
    assert 0 <= rel_error(runs[0], unsplit, orc.F32) < 1e-3
    assert runs[0].tobytes() != unsplit.tobytes()  # the split really ran another summation order


def test_contraction_needs_no_workspace(env):
    """Every real contraction runs without scratch: the K splits of the tensor-core kernels meet in shared memory."""
    ht, h = env
    for dt, dtD in ((ht.R_16F, ht.R_32F), (ht.R_32F, ht.R_32F), (ht.R_64F, ht.R_64F)):
        dA, dB = (h.tensor_descriptor([512, 4096], None, dt) for _ in range(2))
        dD = h.tensor_descriptor([512, 512], None, dtD)
        cd = h.contraction_descriptor(dA, [0, 2], dB, [1, 2], dD, [0, 1], dD, [0, 1],
                                      ht.COMPUTE_64F if dt == ht.R_64F else ht.COMPUTE_32F)
        find = h.contraction_find()
        for pref in (ht.WORKSPACE_MIN, ht.WORKSPACE_RECOMMENDED, ht.WORKSPACE_MAX):
            assert h.contraction_workspace_size(cd, find, pref) == 0


HALF_LAYOUTS = {"kk": ([0, 2], [1, 2]), "mn_mn": ([2, 0], [2, 1]), "k_mn": ([0, 2], [2, 1]), "mn_k": ([2, 0], [1, 2])}
HALF_OUT = {"f32": orc.F32, "f16": orc.F16}


@pytest.mark.parametrize("layout", ["kk", "mn_mn", "k_mn", "mn_k"])
@pytest.mark.parametrize("shape", [(640, 896, 200), (512, 1024, 72), (1280, 2560, 328)])
@pytest.mark.parametrize("out", sorted(HALF_OUT))
def test_cta_pair_kernel_wide_tiles(env, layout, shape, out):
    """256 x 512 tiles (two MMAs per K step sharing A, one accumulator of 512 columns, eight epilogue warps), forced on
    problems with odd numbers of 128-row sub-tiles (a tile's last sub-tiles are missing), for the four operand
    layouts and both output types; several tiles per CTA pair in the largest case."""
    ht, h = env
    M, N, K = shape
    modeA, modeB = HALF_LAYOUTS[layout]
    smp = np.random.default_rng(9).integers(0, M * N, 8192) if M * N > 1 << 20 else None
    set_switch("HTB_TC_WIDE", True)
    try:
        got, exp, td = run_contraction(ht, h, {0: M, 1: N, 2: K}, modeA, modeB, [0, 1], typeAB=orc.F16, typeD=HALF_OUT[out],
                                       alpha=1.5, beta=0.5, fill="normal", sample=smp)
    finally:
        set_switch("HTB_TC_WIDE", False)
    assert ht.last_kernel_name() == "contraction_tcgen05_pair_wide"
    assert not np.isnan(got.astype(np.float32)).any()
    assert 0 <= rel_error(got, exp, td) < (1e-4 if out == "f32" else 2 * 2.0 ** -10)
    assert h.device_status() == 0


# A / B mode orders (last mode fastest) of D[m, n] = A x B for the reference's four layout variants
# (which of A/B has K or M/N fastest, contraction_solution_instances.cpp:40-106)


@pytest.mark.parametrize("layout", sorted(HALF_LAYOUTS))
@pytest.mark.parametrize("shape", [(256, 320, 96), (384, 1000, 520), (640, 896, 200), (1024, 512, 72)])
def test_tensor_core_path_operand_layouts(env, layout, shape):
    """f16/bf16 operands that are contiguous along M/N instead of K run on the tensor cores as well: rows are
    taken in 64-element chunks of the stride-1 mode and the shared-memory descriptors are the transposed form.
    Ragged M, N (1000 = 15.6 chunks) and K tails; single CTAs and CTA pairs."""
    ht, h = env
    M, N, K = shape
    modeA, modeB = HALF_LAYOUTS[layout]
    for dt, td in ((orc.F16, orc.F32), (orc.BF16, orc.BF16)):
        got, exp, tdo = run_contraction(ht, h, {0: M, 1: N, 2: K}, modeA, modeB, [0, 1], typeAB=dt, typeD=td, alpha=1.5,
                                        beta=0.5, fill="normal")
        assert ht.last_kernel_name() == ("contraction_tcgen05_pair" if min(M, N) >= 512 else "contraction_tcgen05")
        assert not np.isnan(orc.to_f64(got, tdo)).any()
        err = rel_error(got, exp, tdo)
        assert 0 <= err < (1e-4 if td == orc.F32 else 2 * 2.0 ** -7), (layout, shape, dt, err)


@pytest.mark.parametrize("dt", [orc.F16, orc.BF16])
def test_tensor_core_path_chunked_rows(env, dt):
    """M/N-major half-precision operands whose row groups hold a ragged stride-1 mode (40, 72: chunks of 64 with a
    zero-filled rest) and a second mode; D's stride-1 mode on either operand."""
    ht, h = env
    m0, m1, n0, n1, k0 = range(5)
    ext = {m0: 40, m1: 5, n0: 72, n1: 3, k0: 136}
    for modeD in ([m1, n1, m0, n0], [n1, m1, n0, m0]):
        got, exp, td = run_contraction(ht, h, ext, [m1, k0, m0], [n1, k0, n0], modeD, typeAB=dt, typeD=orc.F32, alpha=2.0,
                                       beta=0.25, fill="normal")
        assert ht.last_kernel_name() == "contraction_tcgen05"
        assert not np.isnan(got).any()
        err = rel_error(got, exp, td)
        assert 0 <= err < 1e-4, (dt, modeD, err)


@pytest.mark.parametrize("layout", sorted(HALF_LAYOUTS))
def test_cta_pair_kernel_half_tiles_in_last_wave(env, layout):
    """More tiles than CTA pairs with a last wave that is at most half full (80 tiles on 74 pairs): its tiles are
    cut into 256 x 128 halves. Checked on sampled outputs and, against the same problem with the cut disabled,
    bit for bit (each output is accumulated in the same order either way)."""
    import torch

    ht, h = env
    M, N, K = 2560, 2048, 136
    modeA, modeB = HALF_LAYOUTS[layout]
    smp = np.random.default_rng(5).integers(0, M * N, 8192)
    set_switch("HTB_TC_NARROW", True)
    try:
        got, exp, td = run_contraction(ht, h, {0: M, 1: N, 2: K}, modeA, modeB, [0, 1], typeAB=orc.F16, typeD=orc.F32,
                                       alpha=1.5, beta=0.5, fill="normal", sample=smp)
    finally:
        set_switch("HTB_TC_NARROW", False)
    assert ht.last_kernel_name() == "contraction_tcgen05_pair"
    assert not np.isnan(got).any()
    assert 0 <= rel_error(got, exp, td) < 1e-4
    set_switch("HTB_TC_NOHALF", True)
    set_switch("HTB_TC_NARROW", True)
    try:
        whole, _, _ = run_contraction(ht, h, {0: M, 1: N, 2: K}, modeA, modeB, [0, 1], typeAB=orc.F16, typeD=orc.F32,
                                      alpha=1.5, beta=0.5, fill="normal", sample=smp[:1])
    finally:
        set_switch("HTB_TC_NOHALF", False)
        set_switch("HTB_TC_NARROW", False)
    assert np.array_equal(got.view(np.uint32), whole.view(np.uint32))


@pytest.mark.parametrize("case", ["f16_single", "f16_pair", "f32_tensor", "f32_fma", "f64"])
def test_c_may_alias_d(env, case):
    """D = alpha*A*B + beta*C with C and D the same buffer, as the reference's sample calls it
    (samples/01_contraction/simple_bilinear_contraction.hpp:270-271): every kernel family reads an element of C
    before the same thread overwrites it."""
    ht, h = env
    shapes = {"f16_single": (orc.F16, orc.F32, (256, 320, 96), "contraction_tcgen05"),
              "f16_pair": (orc.F16, orc.F32, (640, 768, 136), "contraction_tcgen05_pair"),
              "f32_tensor": (orc.F32, orc.F32, (256, 192, 96), "contraction_tf32x3"),
              "f32_fma": (orc.F32, orc.F32, (70, 50, 33), "contraction_tiled_simt"),
              "f64": (orc.F64, orc.F64, (96, 80, 40), "contraction_tiled_dmma")}
    dt, td, (M, N, K), kernel = shapes[case]
    got, exp, tdo = run_contraction(ht, h, {0: M, 1: N, 2: K}, [0, 2], [1, 2], [0, 1], typeAB=dt, typeD=td, alpha=1.5,
                                    beta=0.5, fill="normal" if dt == orc.F16 else "uniform", alias=True)
    assert ht.last_kernel_name() == kernel
    err = rel_error(got, exp, tdo)
    assert 0 <= err < (1e-4 if dt == orc.F16 else 1e-5), (case, err)


def test_measurement_switches_are_not_in_the_default_build(env):
    """The switches that make a kernel skip loads, MMAs or conversion exist only in measurement builds
    (-DHTB_MEASURE): in the shipped library an environment variable cannot make a result wrong."""
    ht, h = env
    os.environ["HTB_TC_PROBE"] = "7"
    os.environ["HTB_TF32_PROBE"] = "11"
    ht.reload_switches()
    try:
        for dt, k in ((orc.F16, 256), (orc.F32, 136)):
            got, exp, td = run_contraction(ht, h, {0: 512, 1: 512, 2: k}, [0, 2], [1, 2], [0, 1], typeAB=dt,
                                           typeD=orc.F32, alpha=1.0, beta=0.0, with_c=False, fill="normal")
            assert ht.last_kernel_name().startswith("contraction_tcgen05" if dt == orc.F16 else "contraction_tf32x3")
            assert 0 <= rel_error(got, exp, td) < 1e-4
    finally:
        del os.environ["HTB_TC_PROBE"], os.environ["HTB_TF32_PROBE"]
        ht.reload_switches()



# Several K modes that do not fold (the reference's kernels take up to six K modes, contraction_meta_traits.hpp:41-43;
# its mode tests interleave K with M and N, test/01_contraction/configs/mode_test_params.yaml:15-59). Mode lists are
# given last-mode-fastest; the K block of the tensor-core kernels runs along one K mode, the others are iterated.
MULTI_K = {
    # both operands contiguous along k0; k1 slower
    "kk_2": ({"m": 256, "n": 192, "k1": 3, "k0": 48}, ["m", "k1", "k0"], ["k1", "n", "k0"], ["m", "n"]),
    # K modes interleaved with the M modes of A, ragged block mode (136 = 2 x 64 + 8)
    "kk_interleaved": ({"m0": 8, "m1": 32, "n": 320, "k1": 4, "k0": 136}, ["m0", "k1", "m1", "k0"], ["n", "k1", "k0"],
                       ["m0", "m1", "n"]),
    # three K modes in different orders in A and B
    "kk_3": ({"m": 384, "n": 128, "k2": 2, "k1": 3, "k0": 32}, ["m", "k2", "k1", "k0"], ["n", "k1", "k2", "k0"], ["m", "n"]),
    # A contiguous along k0, B contiguous along n
    "k_mn_2": ({"m": 256, "n": 256, "k1": 5, "k0": 64}, ["k1", "m", "k0"], ["k1", "k0", "n"], ["m", "n"]),
    # both operands contiguous along a row mode, two K modes
    "mn_mn_2": ({"m": 192, "n": 256, "k1": 3, "k0": 40}, ["k1", "k0", "m"], ["k0", "k1", "n"], ["m", "n"]),
    # large enough for the CTA-pair kernel
    "kk_2_pair": ({"m": 1024, "n": 1536, "k1": 6, "k0": 96}, ["m", "k1", "k0"], ["k1", "n", "k0"], ["m", "n"]),
}


@pytest.mark.parametrize("case", sorted(MULTI_K))
@pytest.mark.parametrize("dt", [orc.F16, orc.BF16])
def test_tensor_core_path_several_k_modes(env, case, dt):
    ht, h = env
    ext_named, mA, mB, mD = MULTI_K[case]
    names = sorted(ext_named)
    idx = {nm: i for i, nm in enumerate(names)}
    ext = {idx[nm]: e for nm, e in ext_named.items()}
    K = int(np.prod([e for nm, e in ext_named.items() if nm.startswith("k")]))
    smp = None
    if case == "kk_2_pair":
        smp = np.random.default_rng(3).integers(0, 1024 * 1536, 8192)
    got, exp, td = run_contraction(ht, h, ext, [idx[x] for x in mA], [idx[x] for x in mB], [idx[x] for x in mD],
                                   typeAB=dt, typeD=orc.F32, alpha=1.5, beta=0.5, fill="normal", sample=smp)
    assert ht.last_kernel_name().startswith("contraction_tcgen05"), ht.last_kernel_name()
    if case == "kk_2_pair":
        assert ht.last_kernel_name() == "contraction_tcgen05_pair"
    assert not np.isnan(got).any()
    assert 0 <= rel_error(got, exp, td) < 1e-4, (case, K)
    assert h.device_status() == 0


def test_config5_layout_in_half_precision(env):
    """The mode layout of configuration 5, D[m0,m1,m2,n0,n1] = A[m0,k0,m1,k1,m2] B[k1,n0,k0,n1], with f16 data: neither
    operand is contiguous along a K mode and the K group does not fold, so both are taken MN-major with two K modes
    (A in chunks along m2, B along n1). It must run on the tensor cores, not on the FMA kernel."""
    ht, h = env
    m0, m1, m2, n0, n1, k0, k1 = range(7)
    ext = {m0: 16, m1: 16, m2: 16, n0: 48, n1: 48, k0: 48, k1: 48}
    smp = np.random.default_rng(5).integers(0, 16 ** 3 * 48 ** 2, 4096)
    got, exp, td = run_contraction(ht, h, ext, [m0, k0, m1, k1, m2], [k1, n0, k0, n1], [m0, m1, m2, n0, n1],
                                   typeAB=orc.F16, typeD=orc.F32, alpha=2.0, beta=0.5, fill="normal", sample=smp)
    assert ht.last_kernel_name().startswith("contraction_tcgen05"), ht.last_kernel_name()
    assert not np.isnan(got).any()
    assert 0 <= rel_error(got, exp, td) < 5e-4


@pytest.mark.parametrize("case", range(len(MODE_CASES)))
def test_mode_orders_half_precision(env, case):
    """The reference's shuffled mode lists with f16 data and fp32 output (whatever kernel the planner picks)."""
    ht, h = env
    lens, modes = MODE_CASES[case]
    ext = ext_of(modes, lens)
    got, exp, td = run_contraction(ht, h, ext, modes[0], modes[1], modes[2], typeAB=orc.F16, typeD=orc.F32, alpha=1.0,
                                   beta=2.0, fill="normal")
    assert 0 <= rel_error(got, exp, td) < 1e-4


def test_f64_data_with_f32_compute_runs_on_the_fp64_tensor_pipe(env):
    """f64 tensors with compute type f32 (a reference tuple): the FP64 tensor-pipe kernel runs it (more precision than
    asked for, and faster than rounding to float for the FMA kernel). It must satisfy the reference's criterion
    against the oracle, whose algorithm accumulates in float, and agree with the FMA kernel to float rounding."""
    ht, h = env
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m0: 12, m1: 11, n0: 9, n1: 14, k0: 13, k1: 10}
    got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=orc.F64,
                                   compute=orc.COMPUTE_32F, alpha=1.1, beta=2.2)
    assert ht.last_kernel_name() == "contraction_tiled_dmma"
    assert 0 <= rel_error(got, exp, td) < 1e-5
    set_switch("HTB_F64_COMPUTE32_FMA", True)
    try:
        fma, _, _ = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=orc.F64,
                                    compute=orc.COMPUTE_32F, alpha=1.1, beta=2.2)
        assert ht.last_kernel_name() == "contraction_tiled_simt"
    finally:
        set_switch("HTB_F64_COMPUTE32_FMA", False)
    assert 0 <= rel_error(got, fma, td) < 1e-5
