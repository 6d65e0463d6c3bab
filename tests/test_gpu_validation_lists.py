"""The permutation and reduction problem lists of the reference's validation harness, run through the C ABI
against the CPU oracle (lists read as text from test/02_permutation/configs/validation/rank{2..6}_test_params.yaml
and test/03_reduction/configs/validation/rank{1..6}_test_params.yaml into tests/golden/*_validation_lists.json by
tests/golden/extract_shapes.py).

Permutation (permutation_test.cpp:257-340): modeB[i] = modeA[permuted_dims[i]], NULL strides, the second data type
is the scalar's; results must be bit-exact. Ranks 2-4 run the whole cross product; ranks 5 and 6 (120 and 720
orders) run every order once while the data types, alphas and operator pairs rotate.
Reduction (reduction_test.cpp:306-375,518-543): modeC = modeD = the listed output dims in the listed order, D's extents
are those of the SORTED dims and its strides say where each dim lies when the listed order is the memory order (last
listed fastest); pass criterion: reduced size * eps of the compute type for f32 / f64, 2*2^-10 / 2*2^-7 for f16 / bf16."""
import itertools
import json
import os

import numpy as np
import pytest

from helpers import SEED_REDUCTION, rel_error, run_permutation, to_device, to_host
from oracle import binding as orc

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
PERM = json.load(open(os.path.join(GOLD, "permutation_validation_lists.json")))
RED = json.load(open(os.path.join(GOLD, "reduction_validation_lists.json")))
DT = {"HIP_R_16F": orc.F16, "HIP_R_16BF": orc.BF16, "HIP_R_32F": orc.F32, "HIP_R_64F": orc.F64}
CT = {"HIP_R_16F": orc.COMPUTE_16F, "HIP_R_16BF": orc.COMPUTE_16BF, "HIP_R_32F": orc.COMPUTE_32F,
      "HIP_R_64F": orc.COMPUTE_64F}
OPS = {"HIPTENSOR_OP_IDENTITY": orc.OP_IDENTITY, "HIPTENSOR_OP_SQRT": orc.OP_SQRT, "HIPTENSOR_OP_ADD": orc.OP_ADD,
       "HIPTENSOR_OP_MUL": orc.OP_MUL, "HIPTENSOR_OP_MIN": orc.OP_MIN, "HIPTENSOR_OP_MAX": orc.OP_MAX}


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


@pytest.mark.parametrize("rank", range(2, 7))
def test_permutation_lists(env, rank):
    ht, h = env
    L = PERM["rank%d" % rank]
    modeA = list(range(rank))
    combos = list(itertools.product(L["types"], L["alphas"], L["operators"]))
    turn = 0
    for lens in L["lengths"]:
        for dims in L["permuted_dims"]:
            modeB = [modeA[d] for d in dims]
            # whole cross product at ranks 2-4, one rotating combination per order above
            chosen = combos if rank <= 4 else [combos[turn % len(combos)]]
            turn += 1
            for (tdata, tscalar), alpha, (opA, opB) in chosen:
                got, exp = run_permutation(ht, h, lens, modeA, modeB, typeA=DT[tdata], alpha=float(alpha),
                                           type_scalar=DT[tscalar], opA=OPS[opA], opB=OPS[opB])
                assert got.tobytes() == exp.tobytes(), (rank, lens, dims, tdata, tscalar, alpha, opA, opB)


def output_layout(lens, dims):
    """D's extents and strides as the reference's harness builds them (reduction_test.cpp:334-371)."""
    srt = sorted(dims)
    ext = [lens[d] for d in srt]
    if list(dims) == srt:
        return ext, orc.packed_strides(ext, False)
    where, s = {}, 1
    for d in reversed(dims):
        where[d] = s
        s *= lens[d]
    return ext, [where[d] for d in srt]


def reduce_once(env, lens, dims, dt, compute, op, alpha, beta):
    import torch

    ht, h = env
    modeA = list(range(len(lens)))
    modeD = [modeA[d] for d in dims]
    extD, sD = output_layout(lens, dims)
    nA, nD = int(np.prod(lens)), int(np.prod(extD)) if extD else 1
    A = orc.fill_uniform(nA, dt, SEED_REDUCTION[0])
    C = orc.fill_uniform(nD, dt, SEED_REDUCTION[1])
    dA = h.tensor_descriptor(lens, None, dt)
    dD = h.tensor_descriptor(extD, sD if extD else None, dt)
    A_d, C_d = to_device(A, dt), to_device(C, dt)
    D_d = to_device(np.zeros(nD, dtype=orc.np_dtype(dt)), dt)
    ws_size = h.reduction_workspace_size(A_d, dA, modeA, C_d, dD, modeD, D_d, dD, modeD, op, compute)
    ws = torch.empty(ws_size, dtype=torch.uint8, device="cuda") if ws_size else None
    h.reduction(alpha, A_d, dA, modeA, beta, C_d, dD, modeD, D_d, dD, modeD, op, compute, ws, ws_size)
    got = to_host(D_d, dt)
    exp = np.zeros(nD, dtype=orc.np_dtype(dt))
    orc.reduction(alpha, A, lens, orc.packed_strides(lens, False), modeA, dt, beta, C, exp, extD, sD, modeD, dt, op,
                  compute)
    return A, got, exp, nA // nD


@pytest.mark.parametrize("rank", range(1, 7))
def test_reduction_lists(env, rank):
    L = RED["rank%d" % rank]
    for (tdata, tcomp), lens, opname, dims in itertools.product(L["types"], L["lengths"], L["operators"],
                                                                L["output_dims"]):
        if len(dims) >= len(lens):
            continue  # the harness skips these (reduction_test.cpp:216)
        dt, compute = DT[tdata], CT[tcomp]
        for alpha, beta in itertools.product(L["alphas"], L["betas"]):
            A, got, exp, reduced = reduce_once(env, lens, dims, dt, compute, OPS[opname], float(alpha), float(beta))
            if dt == orc.BF16 or compute == orc.COMPUTE_16BF:
                tol = 2 * 2.0 ** -7
            elif dt == orc.F16 or compute == orc.COMPUTE_16F:
                tol = 2 * 2.0 ** -10
            else:
                tol = reduced * float(np.finfo(np.float64 if compute == orc.COMPUTE_64F else np.float32).eps)
            err = rel_error(got, exp, dt)
            assert 0 <= err <= max(tol, 1e-7), (rank, tdata, tcomp, lens, opname, dims, err)


@pytest.mark.parametrize("dims", [[2, 1], [3, 0], [2, 0, 1], [3, 1, 2]])
def test_unsorted_output_dims_against_numpy(env, dims):
    """The layout rule for output dims listed out of order, checked against numpy instead of the oracle: the
    memory image of D is the sum over the other axes, transposed to the listed order, C-contiguous."""
    lens = [5, 4, 6, 3]
    A, got, exp, _ = reduce_once(env, lens, dims, orc.F64, orc.COMPUTE_64F, orc.OP_ADD, 1.0, 0.0)
    R = A.reshape(lens).sum(axis=tuple(d for d in range(4) if d not in dims))  # axes = sorted dims
    srt = sorted(dims)
    want = R.transpose([srt.index(d) for d in dims]).ravel()
    assert np.max(np.abs(got - want)) < 1e-12
