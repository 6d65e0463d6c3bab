"""GPU parity of the packed-operand path: real contractions whose operands the tensor-core kernels cannot read in
place (strides that are not multiples of 16 bytes, contracted modes interleaved with free ones) and that are large
enough (about a GFLOP) are run on packed copies in the caller's workspace. Every output against the fp64 contraction
of the same values (numpy), sampled outputs against the CPU oracle's k order; without a workspace the same problem
runs on the gathered FMA kernel and agrees."""
import numpy as np
import pytest

from helpers import rel_error, run_contraction, to_device, to_host, nan_like
from oracle import binding as orc

pytestmark = pytest.mark.gpu

TENSOR_CORE = ("contraction_tcgen05", "contraction_tcgen05_pair", "contraction_tcgen05_pair_wide", "contraction_tf32x3")


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


def einsum_ref(inp, modeA, modeB, modeD, typeAB, alpha, beta, typeD):
    """fp64 contraction of the host images (strided views of the flat arrays)."""
    def view(flat, lens, strides, dt):
        a = orc.to_f64(flat, dt)
        return np.lib.stride_tricks.as_strided(a, shape=lens, strides=[s * 8 for s in strides])

    letters = {m: chr(ord("a") + i) for i, m in enumerate(sorted(set(modeA) | set(modeB)))}
    sub = lambda ms: "".join(letters[m] for m in ms)
    A = view(inp["A"], inp["lA"], inp["sA"], typeAB)
    B = view(inp["B"], inp["lB"], inp["sB"], typeAB)
    ref = alpha * np.einsum("%s,%s->%s" % (sub(modeA), sub(modeB), sub(modeD)), A, B, optimize=True)
    if inp["C"] is not None and beta != 0.0:
        ref = ref + beta * view(inp["C"], inp["lD"], inp["sD"], typeD)
    return ref


def written(got, inp, typeD):
    g = orc.to_f64(got, typeD)
    return np.lib.stride_tricks.as_strided(g, shape=inp["lD"], strides=[s * 8 for s in inp["sD"]])


CASES = [
    # (typeAB, typeD, extents, modeA, modeB, modeD): rank 4 x rank 4 -> rank 4
    ("f16 extents of 30: strides of 60 bytes", orc.F16, orc.F32, 30, [0, 1, 4, 5], [2, 3, 4, 5], [0, 1, 2, 3]),
    ("f16 interleaved modes", orc.F16, orc.F32, 32, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3]),
    ("bf16 extents of 30, interleaved", orc.BF16, orc.F32, 30, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3]),
    ("f16 in and out, extents of 33", orc.F16, orc.F16, 33, [4, 0, 5, 1], [2, 4, 3, 5], [2, 3, 0, 1]),
    ("f32 interleaved modes", orc.F32, orc.F32, 30, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3]),
    ("f32 extents of 33, interleaved", orc.F32, orc.F32, 33, [0, 4, 1, 5], [5, 2, 4, 3], [3, 2, 1, 0]),
]


@pytest.mark.parametrize("name,typeAB,typeD,e,modeA,modeB,modeD", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("alpha,beta", [(1.0, 0.0), (1.5, 0.5)])
def test_packed_operands_every_output(env, name, typeAB, typeD, e, modeA, modeB, modeD, alpha, beta):
    ht, h = env
    ext = {m: e for m in range(6)}
    inp = {}
    smp = np.random.default_rng(e).integers(0, e ** 4, 512)
    got, exp, td = run_contraction(ht, h, ext, modeA, modeB, modeD, typeAB=typeAB, typeD=typeD, alpha=alpha, beta=beta,
                                   with_c=beta != 0.0, fill="normal", sample=smp, inputs=inp)
    assert ht.last_kernel_name() in TENSOR_CORE, ht.last_kernel_name()
    half_out = typeD in (orc.F16, orc.BF16)
    # tolerances: f16 / bf16 products are exact and summed in fp32 (tensor cores truncate: 1e-3 over 900 to 1089 terms);
    # fp32 data runs as three TF32 products (1e-5, the reference's fp32 criterion); a half-precision D rounds once more
    tol = 4e-3 if half_out else (1e-3 if typeAB != orc.F32 else 1e-5)
    assert 0 <= rel_error(got, exp, td) < tol
    ref = einsum_ref(inp, modeA, modeB, modeD, typeAB, alpha, beta, typeD)
    out = written(got, inp, typeD)
    assert not np.isnan(out).any()
    err = float(np.max(np.abs(out - ref) / (np.abs(out) + np.abs(ref) + 1.0)))
    assert err < tol, err


def test_without_a_workspace_the_fma_kernel_gives_the_same(env):
    """The plan made for a workspace of 0 bytes copies nothing: same problem, gathered FMA kernel, results within the
    two paths' summation orders."""
    import torch

    ht, h = env
    e, modeA, modeB, modeD = 30, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3]
    lens = [e] * 4
    A = orc.fill_normal(e ** 4, orc.F16, 11, 0.5)
    B = orc.fill_normal(e ** 4, orc.F16, 12, 0.5)
    d16 = h.tensor_descriptor(lens, None, ht.R_16F)
    d32 = h.tensor_descriptor(lens, None, ht.R_32F)
    cd = h.contraction_descriptor(d16, modeA, d16, modeB, None, None, d32, modeD, ht.COMPUTE_32F)
    find = h.contraction_find(ht.ALGO_DEFAULT)
    assert h.contraction_workspace_size(cd, find, ht.WORKSPACE_MIN) == 0
    need = h.contraction_workspace_size(cd, find, ht.WORKSPACE_RECOMMENDED)
    assert need >= 2 * e ** 4 * 2  # room for both copies
    A_d, B_d = to_device(A, orc.F16), to_device(B, orc.F16)
    outs = []
    for ws_size in (0, need):
        plan = h.contraction_plan(cd, find, ws_size)
        D_d = to_device(nan_like(e ** 4, orc.F32), orc.F32)
        ws = torch.empty(ws_size, dtype=torch.uint8, device="cuda") if ws_size else None
        h.contraction(plan, 1.0, A_d, B_d, 0.0, None, D_d, ws, ws_size)
        outs.append((ht.last_kernel_name(), to_host(D_d, orc.F32)))
    assert outs[0][0] == "contraction_tiled_simt" and outs[1][0] in TENSOR_CORE
    assert 0 <= rel_error(outs[1][1], outs[0][1], orc.F32) < 1e-3
    # a workspace pointer that is aligned to 2 bytes only: the copies move to the next multiple of 256 bytes
    plan = h.contraction_plan(cd, find, need)
    D_d = to_device(nan_like(e ** 4, orc.F32), orc.F32)
    ws = torch.empty(need + 2, dtype=torch.uint8, device="cuda")
    h.contraction(plan, 1.0, A_d, B_d, 0.0, None, D_d, ws[2:], need)
    assert ht.last_kernel_name() in TENSOR_CORE
    assert np.array_equal(to_host(D_d, orc.F32).view(np.uint32), outs[1][1].view(np.uint32))
    # a plan made for the copies refuses a smaller workspace at execution
    plan = h.contraction_plan(cd, find, need)
    D_d = to_device(nan_like(e ** 4, orc.F32), orc.F32)
    with pytest.raises(ht.HiptensorError) as err:
        h.contraction(plan, 1.0, A_d, B_d, 0.0, None, D_d, None, 0)
    assert err.value.status == ht.STATUS_INSUFFICIENT_WORKSPACE


def test_two_dimensional_odd_k(env):
    """A[m,k] B[n,k] with K = 999 (rows of 1998 bytes): packed rows are padded to 1000 elements with zeros."""
    ht, h = env
    ext = {0: 1001, 1: 1003, 2: 999}
    inp = {}
    got, _, td = run_contraction(ht, h, ext, [0, 2], [1, 2], [0, 1], typeAB=orc.F16, typeD=orc.F32, alpha=1.0, beta=0.0,
                                 with_c=False, fill="normal", oracle=False, inputs=inp)
    assert ht.last_kernel_name() in TENSOR_CORE
    ref = einsum_ref(inp, [0, 2], [1, 2], [0, 1], orc.F16, 1.0, 0.0, orc.F32)
    out = written(got, inp, orc.F32)
    assert not np.isnan(out).any()
    assert float(np.max(np.abs(out - ref) / (np.abs(out) + np.abs(ref) + 1.0))) < 1e-3


def test_strided_operands(env):
    """Operands that are views with gaps (row pitches of 34 and 37 elements for extents of 30), first-mode-fastest D."""
    ht, h = env
    e = 30
    ext = {m: e for m in range(6)}
    modeA, modeB, modeD = [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3]
    sA = orc.packed_strides([e, e, e, 34], False)
    sB = orc.packed_strides([e, e, 37, e], False)
    inp = {}
    got, _, td = run_contraction(ht, h, ext, modeA, modeB, modeD, typeAB=orc.F16, typeD=orc.F32, alpha=2.0, beta=-1.0,
                                 with_c=True, fill="normal", oracle=False, stridesA=sA, stridesB=sB, first_fastest=True,
                                 inputs=inp)
    assert ht.last_kernel_name() in TENSOR_CORE
    ref = einsum_ref(inp, modeA, modeB, modeD, orc.F16, 2.0, -1.0, orc.F32)
    out = written(got, inp, orc.F32)
    assert not np.isnan(out).any()
    assert float(np.max(np.abs(out - ref) / (np.abs(out) + np.abs(ref) + 1.0))) < 1e-3


@pytest.mark.parametrize("typeAB", [orc.F16, orc.F32])
@pytest.mark.parametrize("M,N,K,kfirst", [(64, 64, 8192, False), (16, 256, 4096, False), (24, 40, 16384, True),
                                          (128, 32, 1024, False), (64, 64, 1016, False), (100, 30, 8192, False),
                                          (100, 30, 8192, True), (33, 33, 4096, True), (1000, 30, 1024, True)])
def test_small_outputs_under_a_long_contraction(env, typeAB, M, N, K, kfirst):
    """M < 128 or N < 64 with K >= 1024: one ragged tensor-core tile (rows beyond M and N zero-filled by TMA, masked in
    the epilogue) with its K range cut over a cluster, instead of one FMA tile walking all of K. Row extents that are
    not powers of two take a box that reaches past the tensor; with K first and odd extents (strides of 200 or 66 bytes)
    the operands are packed first. Every output against the oracle's k order; K = 1016 stays below the threshold on the
    FMA kernel."""
    ht, h = env
    ext = {0: M, 1: N, 2: K}
    modeA, modeB = ([2, 0], [2, 1]) if kfirst else ([0, 2], [1, 2])
    inp = {}
    got, exp, td = run_contraction(ht, h, ext, modeA, modeB, [0, 1], typeAB=typeAB, typeD=orc.F32, alpha=1.25, beta=0.5,
                                   with_c=True, fill="normal", inputs=inp)
    if K >= 1024:
        assert ht.last_kernel_name() in TENSOR_CORE, ht.last_kernel_name()
    else:
        assert ht.last_kernel_name() == "contraction_tiled_simt"
    assert not np.isnan(got).any()
    # against the oracle: two fp32 summation orders of K terms (the oracle adds sequentially in fp32)
    assert 0 <= rel_error(got, exp, td) < max(1e-3 if typeAB == orc.F16 else 0.0, K * float(np.finfo(np.float32).eps))
    # against the fp64 contraction of the same values: f16 products are exact, the tensor cores' fp32 adds truncate;
    # fp32 data runs as three TF32 products (the reference's fp32 criterion)
    ref = einsum_ref(inp, modeA, modeB, [0, 1], typeAB, 1.25, 0.5, orc.F32)
    out = written(got, inp, orc.F32)
    err = float(np.max(np.abs(out - ref) / (np.abs(out) + np.abs(ref) + 1.0)))
    # (1e-5 up to K = 4096, growing with K: the fp32 accumulator rounds once per 8-element MMA step)
    assert err < (1e-3 if typeAB == orc.F16 else 1e-5 * max(1.0, K / 4096.0)), err


@pytest.mark.parametrize("typeAB", [orc.F16, orc.F32])
@pytest.mark.parametrize("M,N,K", [(4096, 2048, 8), (2048, 2048, 24), (2048, 4096, 40)])
def test_short_contraction_under_a_large_output(env, typeAB, M, N, K):
    """K below one K block (64 f16 / 32 f32 elements) with four million outputs or more: the tensor-core kernels run
    with the block's tail zero-filled by TMA; the stores of D bound the time. Every output against fp64."""
    ht, h = env
    inp = {}
    got, _, td = run_contraction(ht, h, {0: M, 1: N, 2: K}, [0, 2], [1, 2], [0, 1], typeAB=typeAB, typeD=orc.F32,
                                 alpha=1.0, beta=0.0, with_c=False, fill="normal", oracle=False, inputs=inp)
    assert ht.last_kernel_name() in TENSOR_CORE, ht.last_kernel_name()
    ref = einsum_ref(inp, [0, 2], [1, 2], [0, 1], typeAB, 1.0, 0.0, orc.F32)
    out = written(got, inp, orc.F32)
    assert not np.isnan(out).any()
    assert float(np.max(np.abs(out - ref) / (np.abs(out) + np.abs(ref) + 1.0))) < (1e-3 if typeAB == orc.F16 else 1e-5)
