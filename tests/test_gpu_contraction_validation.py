"""The contraction problem lists of the reference's validation harness, run through the C ABI against the CPU
oracle: test/01_contraction/configs/validation/{bilinear,scale,complex_bilinear,complex_scale}_test_params_rank{1..6}.yaml
(ranks 1-6 = one to six modes per group, seven real type tuples, two complex ones; the lists were read as text into
tests/golden/contraction_validation_shapes.json by tests/golden/extract_shapes.py).

Pass criterion: the reference's own (contraction_test.cpp:882-905): max|d-h|/(|d|+|h|+1) < 2*K*eps, eps of
float unless the compute type is 64F, plus 2*2^-10 / 2*2^-7 when the compute or output type is f16 / bf16. The
complex lists go through test_gpu_contraction_complex.run, which holds cf64 to 1e-12 and cf32 also to 2e-5 against
the fp64 evaluation."""
import json
import os

import numpy as np
import pytest

from helpers import rel_error, run_contraction
from oracle import binding as orc
from test_gpu_contraction_complex import run as run_complex

pytestmark = pytest.mark.gpu
LISTS = json.load(open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden",
                                    "contraction_validation_shapes.json")))
DT = {"HIP_R_16F": orc.F16, "HIP_R_16BF": orc.BF16, "HIP_R_32F": orc.F32, "HIP_R_64F": orc.F64}
CT = {"HIP_R_16F": orc.COMPUTE_16F, "HIP_R_16BF": orc.COMPUTE_16BF, "HIP_R_32F": orc.COMPUTE_32F,
      "HIP_R_64F": orc.COMPUTE_64F}


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


def ext_of(lens, modes):
    ext = {}
    for l, m in zip(lens, modes):
        assert len(l) == len(m)
        for x, y in zip(l, m):
            assert ext.setdefault(y, x) == x, "inconsistent extents in the list"
    return ext


@pytest.mark.parametrize("rank", range(1, 7))
@pytest.mark.parametrize("kind", ["bilinear", "scale"])
def test_real_lists(env, kind, rank):
    ht, h = env
    L = LISTS["%s_rank%d" % (kind, rank)]
    mA, mB, mD = L["modes"]
    betas = L["betas"] or [[0]] * len(L["alphas"])
    for tA, tB, tC, tD, tcomp in L["types"]:
        assert tA == tB and (tC == tD or kind == "scale")
        for lens in L["lengths"]:
            ext = ext_of(lens, (mA, mB, mD))
            K = int(np.prod([ext[m] for m in mA if m in mB]))
            eps = np.finfo(np.float64).eps if tcomp == "HIP_R_64F" else np.finfo(np.float32).eps
            tol = 2 * K * float(eps)
            if "HIP_R_16BF" in (tD, tcomp):
                tol += 2 * 2.0 ** -7
            elif "HIP_R_16F" in (tD, tcomp):
                tol += 2 * 2.0 ** -10
            for al, be in zip(L["alphas"], betas):
                got, exp, td = run_contraction(ht, h, ext, mA, mB, mD, typeAB=DT[tA], typeD=DT[tD], compute=CT[tcomp],
                                               alpha=float(al[0]), beta=float(be[0]), with_c=(kind == "bilinear"))
                err = rel_error(got, exp, td)
                assert 0 <= err < max(tol, 1e-7), (kind, rank, tA, tD, tcomp, lens, al, be, err, ht.last_kernel_name())


@pytest.mark.parametrize("rank", range(1, 7))
@pytest.mark.parametrize("kind", ["complex_bilinear", "complex_scale"])
def test_complex_lists(env, kind, rank):
    L = LISTS["%s_rank%d" % (kind, rank)]
    mA, mB, mD = L["modes"]
    betas = L["betas"] or [[0, 0]] * len(L["alphas"])
    for types in L["types"]:
        dtype = orc.C32F if types[0] == "HIP_C_32F" else orc.C64F
        assert types[0] in ("HIP_C_32F", "HIP_C_64F") and types[0] == types[1] == types[3] == types[4]
        for lens in L["lengths"]:
            ext = ext_of(lens, (mA, mB, mD))
            for al, be in zip(L["alphas"], betas):
                run_complex(env, ext, mA, mB, mD, dtype, complex(al[0], al[1]), complex(be[0], be[1]),
                            with_c=(kind == "complex_bilinear"))
    # the harness' own fill: real and imaginary parts equal (test/device/common.hpp:92-100)
    ext = ext_of(L["lengths"][0], (mA, mB, mD))
    run_complex(env, ext, mA, mB, mD, orc.C32F, 1 + 1j, 2.2 + 2.3j, with_c=(kind == "complex_bilinear"),
                same_parts=True)
