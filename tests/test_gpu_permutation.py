"""GPU parity: hiptensorPermutation through the C ABI against the CPU oracle, bit-exact.
Cases follow the reference harness (test/02_permutation/permutation_test.cpp:251-453 and
configs/validation/rank{2..6}_test_params.yaml: every order at small ranks, alpha != 1, both unary ops)."""
import itertools
import json
import os

import numpy as np
import pytest

from helpers import run_permutation
from oracle import binding as orc

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


def bits(a):
    return a.view(np.uint16 if a.dtype.itemsize == 2 else np.uint32)


def test_golden_vector_f32(env):
    ht, h = env
    g = json.load(open(os.path.join(GOLD, "permutation_whcn_cnhw.json")))
    modeA, modeB = [ord(c) for c in g["modeA"]], [ord(c) for c in g["modeB"]]
    lensA = [g["extent"][c] for c in g["modeA"]]
    got, exp = run_permutation(ht, h, lensA, modeA, modeB, alpha=g["alpha"], A=np.arange(120, dtype=np.float32))
    assert np.array_equal(bits(got), bits(exp))
    assert np.allclose(got, np.array(g["expected_first_mode_fastest"], dtype=np.float32), rtol=2e-7)


def test_golden_vector_f16(env):
    ht, h = env
    g = json.load(open(os.path.join(GOLD, "permutation_whcn_cnhw.json")))
    modeA, modeB = [ord(c) for c in g["modeA"]], [ord(c) for c in g["modeB"]]
    lensA = [g["extent"][c] for c in g["modeA"]]
    got, exp = run_permutation(ht, h, lensA, modeA, modeB, typeA=orc.F16, alpha=g["alpha"],
                               A=np.arange(120, dtype=np.float16))
    assert np.array_equal(bits(got), bits(exp))


@pytest.mark.parametrize("lens", [[5, 3, 7, 2], [33, 17, 9, 65], [1, 6, 1, 70]])
def test_all_rank4_orders_ragged(env, lens):
    ht, h = env
    modeA = [0, 1, 2, 3]
    for perm in itertools.permutations(modeA):
        got, exp = run_permutation(ht, h, lens, modeA, list(perm), alpha=1.0)
        assert np.array_equal(bits(got), bits(exp)), (lens, perm, ht.last_kernel_name())


def test_all_rank4_orders_tma_shapes(env):
    ht, h = env
    lens, modeA = [64, 20, 36, 72], [0, 1, 2, 3]
    kernels = set()
    for perm in itertools.permutations(modeA):
        got, exp = run_permutation(ht, h, lens, modeA, list(perm), alpha=1.0)
        kernels.add(ht.last_kernel_name())
        assert np.array_equal(bits(got), bits(exp)), (perm, ht.last_kernel_name())
    assert "perm_tma" in kernels and "perm_copy" in kernels


@pytest.mark.parametrize("lens", [[64, 24, 40, 72], [128, 8, 8, 136]])
def test_all_rank4_orders_tma_shapes_f16(env, lens):
    """f16 elements through the TMA kernel (both contiguous extents multiples of 8): every order bit-exact."""
    ht, h = env
    modeA = [0, 1, 2, 3]
    kernels = set()
    for perm in itertools.permutations(modeA):
        got, exp = run_permutation(ht, h, lens, modeA, list(perm), typeA=orc.F16, alpha=1.0)
        kernels.add(ht.last_kernel_name())
        assert np.array_equal(bits(got), bits(exp)), (perm, ht.last_kernel_name())
    assert "perm_tma" in kernels


@pytest.mark.parametrize("alpha,ops", [(0.5, (orc.OP_IDENTITY, orc.OP_IDENTITY)), (1.0, (orc.OP_SQRT, orc.OP_IDENTITY)),
                                       (2.0, (orc.OP_IDENTITY, orc.OP_SQRT))])
def test_tma_f16_alpha_and_unary_ops(env, alpha, ops):
    ht, h = env
    A = np.abs(orc.fill_uniform(64 * 32 * 16 * 72, orc.F16, 5))
    got, exp = run_permutation(ht, h, [64, 32, 16, 72], [0, 1, 2, 3], [3, 1, 2, 0], typeA=orc.F16, alpha=alpha,
                               opA=ops[0], opB=ops[1], A=A)
    assert ht.last_kernel_name() == "perm_tma"
    assert np.array_equal(bits(got), bits(exp))


def test_config2_full_size_f16(env):
    """Configuration 2 with f16 elements (512 MiB in, 512 MiB out): bit-exact against an independent transpose."""
    import torch

    ht, h = env
    e = 128
    n = e ** 4
    A = torch.from_numpy(orc.fill_uniform(n, orc.F16, 256)).cuda()
    B = torch.full((n,), float("nan"), dtype=torch.float16, device="cuda")
    d = h.tensor_descriptor([e] * 4, None, ht.R_16F)
    h.permutation(1.0, A, d, [0, 1, 2, 3], B, d, [3, 2, 1, 0], ht.R_16F)
    assert ht.last_kernel_name() == "perm_tma"
    ref = A.view(e, e, e, e).permute(3, 2, 1, 0).contiguous().view(-1)
    assert torch.equal(B.view(torch.int16), ref.view(torch.int16))


@pytest.mark.parametrize("typeA", [orc.F32, orc.F16])
@pytest.mark.parametrize("lens,perm", [([128, 24, 40, 16], [3, 2, 1, 0]), ([64, 10, 38, 32], [3, 2, 1, 0]),
                                       ([96, 50, 16], [2, 1, 0]), ([64, 6, 37, 8], [3, 2, 0, 1]),
                                       ([128, 16, 7, 16], [3, 1, 0, 2]), ([64, 33, 16, 5], [2, 1, 3, 0]),
                                       ([128, 12, 9, 8], [3, 2, 1, 0]), ([64, 5, 22, 4], [3, 2, 1, 0]),
                                       ([256, 3, 130, 8], [3, 2, 0, 1])])
def test_tma_short_contiguous_output_mode(env, typeA, lens, perm):
    """B's contiguous mode is shorter than a tile: the TMA kernel merges it with the mode that follows it in B when the
    two are one contiguous run there (the slab of an output mode split over several GPUs), with whole and ragged
    numbers of runs per tile; otherwise it runs the short mode alone. Bit-exact either way."""
    ht, h = env
    got, exp = run_permutation(ht, h, lens, list(range(len(lens))), perm, typeA=typeA, alpha=1.0)
    assert np.array_equal(bits(got), bits(exp)), (lens, perm, ht.last_kernel_name())
    got, exp = run_permutation(ht, h, lens, list(range(len(lens))), perm, typeA=typeA, alpha=0.5)
    assert np.array_equal(bits(got), bits(exp)), (lens, perm, ht.last_kernel_name())


@pytest.mark.parametrize("typeA", [orc.F32, orc.F16])
@pytest.mark.parametrize("lens,perm", [([16, 40, 24, 128], [3, 2, 1, 0]), ([32, 38, 10, 64], [3, 2, 1, 0]),
                                       ([16, 50, 96], [2, 1, 0]), ([8, 37, 6, 64], [3, 0, 1, 2]),
                                       ([16, 7, 16, 128], [3, 2, 0, 1]), ([4, 22, 5, 64], [3, 2, 1, 0]),
                                       ([16, 24, 40, 16], [3, 2, 1, 0]), ([8, 128, 8], [2, 1, 0]),
                                       ([16, 20, 30, 8], [3, 1, 2, 0])])
def test_tma_short_contiguous_input_mode(env, typeA, lens, perm):
    """A's contiguous mode is shorter than a tile (the mirror image of the test above, e.g. the way back from a slab),
    alone and together with a short contiguous mode of B. Bit-exact."""
    ht, h = env
    got, exp = run_permutation(ht, h, lens, list(range(len(lens))), perm, typeA=typeA, alpha=1.0)
    assert np.array_equal(bits(got), bits(exp)), (lens, perm, ht.last_kernel_name())
    got, exp = run_permutation(ht, h, lens, list(range(len(lens))), perm, typeA=typeA, alpha=2.0)
    assert np.array_equal(bits(got), bits(exp)), (lens, perm, ht.last_kernel_name())


@pytest.mark.parametrize("typeA,typeB", [(orc.F16, orc.F16), (orc.F16, orc.F32), (orc.F32, orc.F32)])
@pytest.mark.parametrize("lens,perm", [([4, 128, 64, 6], [1, 2, 3, 0]), ([6, 24, 40, 12], [3, 2, 1, 0]),
                                       ([2, 6, 130, 66], [0, 1, 3, 2]), ([2, 2, 2, 2, 2, 2], [5, 4, 3, 2, 1, 0]),
                                       ([3, 5, 67, 31], [2, 0, 3, 1]), ([16, 32, 24, 20], [1, 0, 2, 3]),
                                       ([6, 1000], [1, 0]), ([5, 3, 7, 129], [3, 1, 0, 2])])
@pytest.mark.parametrize("alpha,ops", [(1.0, (orc.OP_IDENTITY, orc.OP_IDENTITY)), (0.5, (orc.OP_SQRT, orc.OP_SQRT))])
def test_box_kernel_short_contiguous_modes(env, typeA, typeB, lens, perm, alpha, ops):
    """Contiguous modes of a few elements on either side (input, output or both, odd extents included): one block moves
    a box of up to 2048 elements that spans several leading modes of A and of B."""
    ht, h = env
    modes = list(range(len(lens)))
    got, exp = run_permutation(ht, h, lens, modes, [modes[i] for i in perm], typeA=typeA, typeB=typeB, alpha=alpha,
                               type_scalar=typeA, opA=ops[0], opB=ops[1])
    assert ht.last_kernel_name() == "perm_box"
    assert np.array_equal(bits(got), bits(exp))


@pytest.mark.parametrize("typeA,typeB", [(orc.F16, orc.F16), (orc.F16, orc.F32), (orc.F32, orc.F32)])
@pytest.mark.parametrize("lens", [[8, 6, 130, 66], [16, 3, 67, 31], [32, 33, 65, 9], [12, 6, 130, 66], [6, 6, 130, 66]])
@pytest.mark.parametrize("alpha", [1.0, 0.5])
def test_box_kernel_short_rows_move_as_words(env, typeA, typeB, lens, alpha):
    """Rows of at most 128 bytes shared by A and B: the box kernel moves them as words of 4 to 16 bytes."""
    ht, h = env
    for perm in ([0, 2, 1, 3], [0, 3, 2, 1], [0, 3, 1, 2]):
        got, exp = run_permutation(ht, h, lens, [0, 1, 2, 3], perm, typeA=typeA, typeB=typeB, alpha=alpha,
                                   type_scalar=typeA)
        if lens[0] * (2 if typeA == orc.F16 else 4) <= 128:
            assert ht.last_kernel_name() == "perm_box"
        assert np.array_equal(bits(got), bits(exp)), (lens, perm)


@pytest.mark.parametrize("offA,offB", [(1, 0), (0, 1), (2, 2), (4, 0)])
def test_box_kernel_words_respect_pointer_alignment(env, offA, offB):
    """The same short rows from pointers that are aligned to an element only: narrower words, same result."""
    import torch

    ht, h = env
    lens, perm = [8, 5, 67, 33], [0, 2, 1, 3]
    n = int(np.prod(lens))
    A = orc.fill_uniform(n, orc.F16, 77)
    exp = np.zeros(n, dtype=np.float16)
    orc.permutation(1.0, orc.F16, A, lens, [0, 1, 2, 3], orc.F16, exp, perm, orc.F16, nthreads=0)
    A_d = torch.zeros(n + 8, dtype=torch.float16, device="cuda")
    A_d[offA:offA + n] = torch.from_numpy(A).cuda()
    B_d = torch.zeros(n + 8, dtype=torch.float16, device="cuda")
    dA = h.tensor_descriptor(lens, None, ht.R_16F)
    dB = h.tensor_descriptor([lens[i] for i in perm], None, ht.R_16F)
    h.permutation(1.0, A_d[offA:], dA, [0, 1, 2, 3], B_d[offB:], dB, perm, ht.R_16F)
    assert ht.last_kernel_name() == "perm_box"
    got = B_d.cpu().numpy()
    assert np.array_equal(bits(got[offB:offB + n]), bits(exp))
    assert not got[:offB].any() and not got[offB + n:].any()


@pytest.mark.parametrize("rank", [2, 3, 5, 6])
def test_other_ranks(env, rank):
    ht, h = env
    base = [12, 5, 8, 3, 4, 6][:rank]
    modeA = list(range(rank))
    rng = np.random.default_rng(rank)
    orders = [list(reversed(modeA))] + [list(rng.permutation(rank)) for _ in range(6)]
    for perm in orders:
        got, exp = run_permutation(ht, h, base, modeA, [int(x) for x in perm], alpha=1.0)
        assert np.array_equal(bits(got), bits(exp)), (rank, perm)


@pytest.mark.parametrize("alpha", [0.0, 2.1, -0.5])
@pytest.mark.parametrize("ops", [(1, 1), (2, 1), (1, 2), (2, 2)])
def test_alpha_and_unary_ops(env, alpha, ops):
    ht, h = env
    for lens in ([40, 24, 20], [7, 9, 11]):
        got, exp = run_permutation(ht, h, lens, [0, 1, 2], [2, 0, 1], alpha=alpha, opA=ops[0], opB=ops[1])
        assert np.array_equal(bits(got), bits(exp)), (lens, alpha, ops, ht.last_kernel_name())


@pytest.mark.parametrize("typeB", [orc.F16, orc.F32])
def test_f16_inputs(env, typeB):
    ht, h = env
    for perm in ([1, 0, 2], [2, 1, 0], [0, 2, 1]):
        got, exp = run_permutation(ht, h, [70, 33, 12], [0, 1, 2], perm, typeA=orc.F16, typeB=typeB, alpha=1.5,
                                   type_scalar=orc.F16)
        assert np.array_equal(bits(got), bits(exp)), (perm, typeB)


@pytest.mark.parametrize("typeA,typeB", [(orc.F16, orc.F16), (orc.F16, orc.F32), (orc.F32, orc.F32)])
@pytest.mark.parametrize("lens", [[63, 34, 12, 7], [129, 65, 3, 5], [1, 67, 131, 2]])
def test_generic_tile_kernel_plain_moves(env, typeA, typeB, lens):
    """alpha = 1 and identity operators on odd extents: the element kernel's path that moves values unchanged
    (tiles inside the tensor without bounds checks, ragged tiles at the edges)."""
    ht, h = env
    for perm in ([3, 2, 1, 0], [1, 0, 2, 3], [2, 3, 0, 1]):
        got, exp = run_permutation(ht, h, lens, [0, 1, 2, 3], perm, typeA=typeA, typeB=typeB, alpha=1.0,
                                   type_scalar=typeA)
        assert np.array_equal(bits(got), bits(exp)), (lens, perm, ht.last_kernel_name())


@pytest.mark.parametrize("typeA,typeB", [(orc.F16, orc.F16), (orc.F16, orc.F32), (orc.F32, orc.F32)])
@pytest.mark.parametrize("lens", [[70, 34, 12, 6], [66, 130, 2, 10], [64, 3, 128, 5], [63, 34, 12, 7]])
def test_generic_tile_kernel_even_and_odd(env, typeA, typeB, lens):
    """The shared-memory tile kernel moves 2 x 2 blocks when every extent and stride involved is even (edge tiles
    that are not multiples of 64, odd extents in the other modes) and single elements otherwise; with scale and
    unary operators, all three type pairs, orders that transpose different mode pairs."""
    ht, h = env
    for perm in ([3, 2, 1, 0], [1, 0, 2, 3], [2, 3, 0, 1], [1, 3, 0, 2]):
        got, exp = run_permutation(ht, h, lens, [0, 1, 2, 3], perm, typeA=typeA, typeB=typeB, alpha=2.1,
                                   type_scalar=typeA, opA=orc.OP_SQRT, opB=orc.OP_IDENTITY)
        assert np.array_equal(bits(got), bits(exp)), (lens, perm, ht.last_kernel_name())


@pytest.mark.parametrize("typeB", [orc.F16, orc.F32])
@pytest.mark.parametrize("lens", [[132, 8, 68, 12], [256, 4, 128, 4], [64, 3, 128, 5], [4, 4, 4, 4]])
def test_f16_tile_kernel_blocks_of_four(env, typeB, lens):
    """f16 tensors whose extents and strides are multiples of 4 take 128 x 128 tiles with 4 x 4 register blocks
    (ragged tiles: 132 = 128 + 4, 68; tiny tensors); scale and unary operators; both output types."""
    ht, h = env
    for perm in ([3, 2, 1, 0], [1, 0, 2, 3], [2, 3, 0, 1], [2, 0, 3, 1]):
        for opA, opB, alpha in ((orc.OP_IDENTITY, orc.OP_IDENTITY, 1.0), (orc.OP_SQRT, orc.OP_SQRT, 0.5)):
            got, exp = run_permutation(ht, h, lens, [0, 1, 2, 3], perm, typeA=orc.F16, typeB=typeB, alpha=alpha,
                                       type_scalar=orc.F16, opA=opA, opB=opB)
            assert np.array_equal(bits(got), bits(exp)), (lens, perm, opA, ht.last_kernel_name())


def test_rejects_unsupported(env):
    ht, h = env
    dA = h.tensor_descriptor([4, 4], None, ht.R_64F)
    import torch

    x = torch.zeros(16, dtype=torch.float64, device="cuda")
    with pytest.raises(ht.HiptensorError) as e:
        h.permutation(1.0, x, dA, [0, 1], x, dA, [1, 0], ht.R_32F)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED


def test_config2_full_size(env):
    """fp32 B[d,c,b,a] = A[a,b,c,d], extents 128 (1 GiB): bit-exact against an independent
    transpose, and the inverse permutation restores A."""
    import torch

    ht, h = env
    e = 128
    n = e ** 4
    A = torch.from_numpy(orc.fill_uniform(n, orc.F32, 256)).cuda()
    B = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    d = h.tensor_descriptor([e] * 4, None, ht.R_32F)
    h.permutation(1.0, A, d, [0, 1, 2, 3], B, d, [3, 2, 1, 0], ht.R_32F)
    assert ht.last_kernel_name() == "perm_tma"
    # first mode fastest: memory image viewed as [d][c][b][a]; B as [a][b][c][d]
    ref = A.view(e, e, e, e).permute(3, 2, 1, 0).contiguous().view(-1)
    assert torch.equal(B.view(torch.int32), ref.view(torch.int32))
    del ref
    A2 = torch.empty_like(A)
    h.permutation(1.0, B, d, [3, 2, 1, 0], A2, d, [0, 1, 2, 3], ht.R_32F)
    assert torch.equal(A2.view(torch.int32), A.view(torch.int32))
    # oracle on a slab small enough to finish in seconds: d restricted to 2
    lens = [e, e, e, 2]
    from helpers import run_permutation as rp

    got, exp = rp(ht, h, lens, [0, 1, 2, 3], [3, 2, 1, 0])
    assert np.array_equal(bits(got), bits(exp))
