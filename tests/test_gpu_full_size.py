"""Benchmark configurations 2, 4 and 5 at full size with every output element checked (configuration 3 at full
size is in tests/test_gpu_reduction.py), and the slabs that an N-way split of configurations 2, 3 and 4
hands to one GPU (N = 2, 4, 8), each against the CPU oracle, with the kernel the planner picked asserted.

Configurations 4 and 5 fold to plain matrices, so the whole-tensor reference is a blocked fp64
matrix product of the folded host views (numpy, all host cores); the oracle's sequential
k-order algorithm stays the reference on sampled outputs (tests/test_gpu_contraction.py).
Whole-tensor comparison with the output pre-filled with NaN follows the reference's own
contraction test (test/01_contraction/contraction_test.cpp:852-945)."""
import numpy as np
import pytest

from helpers import rel_error, run_contraction, run_reduction
from oracle import binding as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


def bits(a):
    return a.view(np.uint32 if a.dtype.itemsize == 4 else np.uint16)


def test_config4_full_size_every_output(env):
    """f16 x f16 -> f32, extents 64 (M = N = K = 4096): all 16.7 M outputs against the fp64 product of the same
    f16 values. Tolerance: 1e-2 stated for half-precision inputs, 1e-3 asserted: the products are exact, the
    tensor cores add them to the fp32 accumulator with truncation, so the error grows with K (1e-5 at K = 256,
    1.6e-4 observed at K = 4096 as the maximum over all outputs)."""
    ht, h = env
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m: 64 for m in range(6)}
    inp = {}
    got, _, td = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=orc.F16,
                                 typeD=orc.F32, alpha=1.0, beta=0.0, with_c=False, fill="normal", oracle=False,
                                 inputs=inp)
    assert ht.last_kernel_name() == "contraction_tcgen05_pair_wide"
    assert not np.isnan(got).any()  # D was pre-filled with NaN: every element has been written
    A = inp["A"].astype(np.float64).reshape(4096, 4096)  # [m0 m1][k0 k1], last mode fastest
    B = inp["B"].astype(np.float64).reshape(4096, 4096)  # [n0 n1][k0 k1]
    ref = A @ B.T
    err = rel_error(got.astype(np.float64), ref.reshape(-1), orc.F64)
    assert 0 <= err < 1e-2, err
    assert err < 1e-3, err


def test_config5_full_size_every_output(env):
    """fp64, D[m0,m1,m2,n0,n1] = 2 A[m0,k0,m1,k1,m2] B[k1,n0,k0,n1] + 0.5 C (M = 4096, N = K = 2304): all 9.4 M
    outputs against the blocked fp64 product of the folded views. Tolerance: the reference's 2 K eps."""
    ht, h = env
    m0, m1, m2, n0, n1, k0, k1 = range(7)
    ext = {m0: 16, m1: 16, m2: 16, n0: 48, n1: 48, k0: 48, k1: 48}
    inp = {}
    got, _, td = run_contraction(ht, h, ext, [m0, k0, m1, k1, m2], [k1, n0, k0, n1], [m0, m1, m2, n0, n1],
                                 typeAB=orc.F64, alpha=2.0, beta=0.5, oracle=False, inputs=inp)
    assert ht.last_kernel_name() == "contraction_tiled_dmma"
    assert not np.isnan(got).any()
    A = inp["A"].reshape(16, 48, 16, 48, 16).transpose(0, 2, 4, 1, 3).reshape(4096, 2304)  # [m0 m1 m2][k0 k1]
    B = inp["B"].reshape(48, 48, 48, 48).transpose(1, 3, 2, 0).reshape(2304, 2304)  # [n0 n1][k0 k1]
    ref = 2.0 * (np.ascontiguousarray(A) @ np.ascontiguousarray(B).T) + 0.5 * inp["C"].reshape(4096, 2304)
    err = rel_error(got, ref.reshape(-1), orc.F64)
    assert 0 <= err < 2 * 2304 * np.finfo(np.float64).eps, err


def test_config2_full_size_against_the_oracle(env):
    """fp32 B[d,c,b,a] = A[a,b,c,d], extents 128 (1 GiB in, 1 GiB out): bit-exact against the CPU oracle run
    on the whole tensor with every host core."""
    import torch

    ht, h = env
    e = 128
    n = e ** 4
    A = orc.fill_uniform(n, orc.F32, 256)
    A_d = torch.from_numpy(A).cuda()
    B_d = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    d = h.tensor_descriptor([e] * 4, None, ht.R_32F)
    h.permutation(1.0, A_d, d, [0, 1, 2, 3], B_d, d, [3, 2, 1, 0], ht.R_32F)
    assert ht.last_kernel_name() == "perm_tma"
    got = B_d.cpu().numpy()
    del A_d, B_d
    exp = np.empty(n, dtype=np.float32)
    orc.permutation(1.0, orc.F32, A, [e] * 4, [0, 1, 2, 3], orc.F32, exp, [3, 2, 1, 0], orc.F32, nthreads=0)
    assert np.array_equal(bits(got), bits(exp))


def test_short_mode_permutation_above_l2(env):
    """fp32 B[d,c,b,a] = A[a,b,c,d] with a contiguous mode of 6 elements on the input side (192 MiB in, 192 MiB out): the
    box kernel, bit-exact against the oracle on the whole tensor."""
    from helpers import run_permutation

    ht, h = env
    got, exp = run_permutation(ht, h, [512, 128, 128, 6], [0, 1, 2, 3], [3, 2, 1, 0])
    assert ht.last_kernel_name() == "perm_box"
    assert np.array_equal(bits(got), bits(exp))


def test_short_row_reduction_above_l2(env):
    """fp32 rows of 4 contiguous elements reduced under 2^24 outputs (256 MiB in, 64 MiB out): the short-row kernel, one
    lane per output."""
    ht, h = env
    for op in (orc.OP_ADD, orc.OP_MAX):
        got, exp = run_reduction(ht, h, [4096, 64, 64, 4], [0, 1, 2, 3], [0, 1, 2], op=op, alpha=1.0, beta=0.5)
        assert ht.last_kernel_name() == "red_short"
        if op == orc.OP_MAX:
            assert np.array_equal(bits(got), bits(exp))
        else:
            assert 0 <= rel_error(got, exp, orc.F32) < 4 * float(np.finfo(np.float32).eps)


# ---------------------------------------------------------------------------------------- slabs of an N-way split
@pytest.mark.parametrize("m0_local", [8, 16, 32])
def test_config4_slab(env, m0_local):
    """The slab of configuration 4 that one of 8 / 4 / 2 GPUs owns (m0 = 64 / N, folded M = 512 / 1024 / 2048,
    N = K = 4096): whole slab against the fp64 product, sampled outputs against the oracle's k order."""
    ht, h = env
    m0, m1, n0, n1, k0, k1 = range(6)
    ext = {m: 64 for m in range(6)}
    ext[m0] = m0_local
    M = m0_local * 64
    inp = {}
    smp = np.random.default_rng(m0_local).integers(0, M * 4096, 2048)
    got, exp, td = run_contraction(ht, h, ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], typeAB=orc.F16,
                                   typeD=orc.F32, alpha=1.0, beta=0.0, with_c=False, fill="normal", sample=smp,
                                   inputs=inp)
    # 2048 rows: 256 x 512 tiles; 1024: 256 x 256 tiles; 512: 256 x 256 tiles with every tile's K range cut over two
    # CTA pairs
    assert ht.last_kernel_name() == ("contraction_tcgen05_pair_wide" if m0_local == 32 else "contraction_tcgen05_pair")
    assert not np.isnan(got).any()
    assert 0 <= rel_error(got, exp, td) < 1e-3  # two fp32 summation orders of 4096 products
    ref = inp["A"].astype(np.float64).reshape(M, 4096) @ inp["B"].astype(np.float64).reshape(4096, 4096).T
    assert 0 <= rel_error(got.astype(np.float64), ref.reshape(-1), orc.F64) < 1e-3


@pytest.mark.parametrize("d_local", [16, 32, 64])
def test_config2_slab(env, d_local):
    """The slab of configuration 2 that one of 8 / 4 / 2 GPUs owns (d = 128 / N): bit-exact against the oracle."""
    from helpers import run_permutation

    ht, h = env
    got, exp = run_permutation(ht, h, [128, 128, 128, d_local], [0, 1, 2, 3], [3, 2, 1, 0])
    assert ht.last_kernel_name() == "perm_tma"
    assert np.array_equal(bits(got), bits(exp))


@pytest.mark.parametrize("m_local", [512, 1024, 2048])
@pytest.mark.parametrize("op", [orc.OP_ADD, orc.OP_MAX])
def test_config3_slab(env, m_local, op):
    """The slab of configuration 3 that one of 8 / 4 / 2 GPUs owns (m = 4096 / N)."""
    ht, h = env
    got, exp, exact = run_reduction(ht, h, [m_local, 64, 64, 32], [0, 1, 2, 3], [0, 1], op=op, alpha=1.0, beta=0.5,
                                    want_exact=True)
    assert ht.last_kernel_name() == "red_row"
    if op == orc.OP_MAX:
        assert np.array_equal(bits(got), bits(exp))
    else:
        assert 0 <= rel_error(got, exp, orc.F32) < 2048 * float(np.finfo(np.float32).eps)
        assert 0 <= rel_error(got.astype(np.float64), exact, orc.F64) < 1e-5


@pytest.mark.parametrize("k_local", [8, 16, 32])
@pytest.mark.parametrize("op", [orc.OP_ADD, orc.OP_MAX])
def test_config3_reduced_mode_split_and_finish(env, k_local, op):
    """Configuration 3 with the REDUCED mode k split N ways, the N partial reductions run one after the other on
    this GPU (alpha 1, beta 0), combined with the operator as the all-reduce would, and finished by
    htReductionFinish: equals the oracle on the whole tensor."""
    import torch

    ht, h = env
    lens = [256, 64, 64, 32]  # 256 of the 4096 rows: the oracle on the whole of A stays short
    n = int(np.prod(lens))
    A = orc.fill_uniform(n, orc.F32, 17)
    C = orc.fill_uniform(lens[0] * lens[1], orc.F32, 19)
    sA = orc.packed_strides(lens, False)
    lD, sD = lens[:2], orc.packed_strides(lens[:2], False)
    exp = np.zeros(lD[0] * lD[1], dtype=np.float32)
    orc.reduction(1.5, A, lens, sA, [0, 1, 2, 3], orc.F32, 0.5, C, exp, lD, sD, [0, 1], orc.F32, op, orc.COMPUTE_32F)
    A_d, C_d = torch.from_numpy(A).cuda(), torch.from_numpy(C).cuda()
    dD = h.tensor_descriptor(lD, sD, ht.R_32F)
    parts = []
    for r in range(64 // k_local):
        loc = [lens[0], lens[1], k_local, lens[3]]
        dA = h.tensor_descriptor(loc, sA, ht.R_32F)  # a strided view of the whole tensor
        P = torch.zeros(lD[0] * lD[1], device="cuda")
        h.reduction(1.0, A_d[r * k_local * sA[2]:], dA, [0, 1, 2, 3], 0.0, P, dD, [0, 1], P, dD, [0, 1], op,
                    ht.COMPUTE_32F)
        parts.append(P)
    total = parts[0]
    for P in parts[1:]:
        total = total + P if op == orc.OP_ADD else torch.maximum(total, P)
    D = torch.full_like(total, float("nan"))
    h.reduction_finish(1.5, total, 0.5, C_d, D, dD, ht.COMPUTE_32F)
    assert ht.last_kernel_name() == "red_finish"
    got = D.cpu().numpy()
    assert 0 <= rel_error(got, exp, orc.F32) < 2048 * float(np.finfo(np.float32).eps)
    # in place (partial aliases D) gives the same bits
    h.reduction_finish(1.5, total, 0.5, C_d, total, dD, ht.COMPUTE_32F)
    assert np.array_equal(bits(total.cpu().numpy()), bits(got))
