"""Shared helpers of the GPU parity tests: run one operation through the library (flat C ABI via
hiptensor_b200) on seeded inputs, run the CPU oracle on the same inputs, hand both results back."""
import numpy as np

from oracle import binding as orc

# seeds of the reference harness: contraction A/B/C (test/01_contraction/contraction_test.cpp:381-441),
# permutation A (test/02_permutation/permutation_resource.cpp:97-110),
# reduction A/C (test/03_reduction/reduction_resource.cpp:111-123)
SEED_CONTRACTION = (255, 256, 257)
SEED_PERMUTATION = 256
SEED_REDUCTION = (17, 19)


def set_switch(name, on):
    """Sets or clears one of the library's HTB_* variant switches and has the library read them again
    (it reads the environment once when it is loaded)."""
    import os

    import hiptensor_b200 as ht

    if on:
        os.environ[name] = "1"
    else:
        os.environ.pop(name, None)
    ht.reload_switches()


def torch_dtype(dt):
    import torch

    return {orc.F32: torch.float32, orc.F64: torch.float64, orc.F16: torch.float16, orc.BF16: torch.bfloat16}[dt]


def to_device(a, dt):
    """numpy oracle array -> torch CUDA tensor of the matching dtype (bf16 travels as uint16 bits)."""
    import torch

    t = torch.from_numpy(a)
    if dt == orc.BF16:
        t = t.view(torch.bfloat16)
    return t.cuda()


def to_host(t, dt):
    import torch

    t = t.detach().cpu()
    if dt == orc.BF16:
        return t.view(torch.uint16).numpy().copy()
    return t.numpy().copy()


def span(lens, strides):
    """Elements a strided tensor spans in memory."""
    return 1 + sum((l - 1) * s for l, s in zip(lens, strides))


def nan_like(n, dt):
    a = np.empty(n, dtype=orc.np_dtype(dt))
    if dt == orc.BF16:
        a[:] = 0x7FC0
    else:
        a[:] = np.nan
    return a


def run_permutation(ht, h, lensA, modeA, modeB, typeA=orc.F32, typeB=None, alpha=1.0, type_scalar=None,
                    opA=orc.OP_IDENTITY, opB=orc.OP_IDENTITY, seed=SEED_PERMUTATION, A=None):
    typeB = typeA if typeB is None else typeB
    type_scalar = typeA if type_scalar is None else type_scalar
    n = int(np.prod(lensA))
    if A is None:
        A = orc.fill_uniform(n, typeA, seed)
    lensB = [lensA[modeA.index(m)] for m in modeB]
    dA = h.tensor_descriptor(lensA, None, typeA, opA)
    dB = h.tensor_descriptor(lensB, None, typeB, opB)
    A_d = to_device(A, typeA)
    B_d = to_device(nan_like(n, typeB), typeB)
    h.permutation(alpha, A_d, dA, modeA, B_d, dB, modeB, type_scalar)
    got = to_host(B_d, typeB)
    exp = nan_like(n, typeB)
    orc.permutation(alpha, type_scalar, A, lensA, modeA, typeA, exp, modeB, typeB, opA, opB, nthreads=0)
    return got, exp


def run_reduction(ht, h, lensA, modeA, modeD, dt=orc.F32, compute=None, op=orc.OP_ADD, alpha=1.0, beta=0.0,
                  stridesA=None, stridesD=None, alias=False, seeds=SEED_REDUCTION, A=None, use_workspace=True,
                  want_exact=False):
    """modeD lists the kept modes; extents of D follow A's order (positional contract).
    want_exact adds a third result: the oracle run on the same values widened to fp64."""
    import torch

    compute = compute if compute is not None else (orc.COMPUTE_64F if dt == orc.F64 else orc.COMPUTE_32F)
    kept = [m for m in modeA if m in modeD]
    lensD = [lensA[modeA.index(m)] for m in kept]
    sA = stridesA if stridesA is not None else orc.packed_strides(lensA, False)
    sD = stridesD if stridesD is not None else orc.packed_strides(lensD, False)
    nA = span(lensA, sA)
    nD = span(lensD, sD) if lensD else 1
    if A is None:
        A = orc.fill_uniform(nA, dt, seeds[0])
    C = orc.fill_uniform(nD, dt, seeds[1])
    dA = h.tensor_descriptor(lensA, stridesA, dt)
    dD = h.tensor_descriptor(lensD, sD if lensD else None, dt)
    A_d = to_device(A, dt)
    C_d = to_device(C, dt)
    D_d = C_d if alias else to_device(np.zeros(nD, dtype=orc.np_dtype(dt)), dt)
    ws, ws_size = None, 0
    if use_workspace:
        ws_size = h.reduction_workspace_size(A_d, dA, modeA, C_d, dD, kept, D_d, dD, kept, op, compute)
        if ws_size:
            ws = torch.empty(ws_size, dtype=torch.uint8, device="cuda")
    h.reduction(alpha, A_d, dA, modeA, beta, C_d, dD, kept, D_d, dD, kept, op, compute, ws, ws_size)
    got = to_host(D_d, dt)
    exp = C.copy() if alias else np.zeros(nD, dtype=orc.np_dtype(dt))
    orc.reduction(alpha, A, lensA, sA, modeA, dt, beta, None if alias else C, exp, lensD, sD, kept, dt, op, compute)
    if not want_exact:
        return got, exp
    A64, C64 = orc.to_f64(A, dt), orc.to_f64(C, dt)
    exact = C64.copy() if alias else np.zeros(nD, dtype=np.float64)
    orc.reduction(alpha, A64, lensA, sA, modeA, orc.F64, beta, None if alias else C64, exact, lensD, sD, kept,
                  orc.F64, op, orc.COMPUTE_64F)
    return got, exp, exact


def check_f32(got, exp, exact, terms):
    """fp32 results. Against the reference's CPU algorithm (sequential fp32 accumulation) the
    reference's own bound terms*eps (reduction_test.cpp:518-543; 2*K*eps for contraction,
    contraction_test.cpp:882-905) holds; two fp32 summation orders of thousands of terms differ by
    more than 1e-5 under the metric, so the 1e-5 bound is checked against the same operation
    evaluated by the oracle in fp64 on the same values, i.e. against the exact result."""
    e1 = rel_error(got, exp, orc.F32)
    assert 0 <= e1 < max(terms * float(np.finfo(np.float32).eps), 1e-6), ("vs reference algorithm", e1)
    e2 = rel_error(got.astype(np.float64), exact, orc.F64)
    assert 0 <= e2 < 1e-5, ("vs exact", e2)
    return e1, e2


def run_contraction(ht, h, extent, modeA, modeB, modeD, typeAB=orc.F32, typeD=None, compute=None, alpha=1.0,
                    beta=0.0, with_c=True, first_fastest=False, stridesA=None, stridesB=None, stridesD=None,
                    fill="uniform", sample=None, seeds=SEED_CONTRACTION, algo=None, alias=False, oracle=True,
                    inputs=None):
    """extent: dict mode -> extent. Returns (got, expected, typeD) as flat memory images of D.
    alias: C and D are the same device buffer (the reference's samples call it that way).
    oracle=False skips the CPU oracle (expected is None) for callers that check the result another way;
    inputs, a dict, receives the host arrays A, B, C and the strides that were used."""
    typeD = typeAB if typeD is None else typeD
    if compute is None:
        compute = orc.COMPUTE_64F if typeAB == orc.F64 else orc.COMPUTE_32F
    lA, lB, lD = ([extent[m] for m in ms] for ms in (modeA, modeB, modeD))
    sA = stridesA if stridesA is not None else orc.packed_strides(lA, first_fastest)
    sB = stridesB if stridesB is not None else orc.packed_strides(lB, first_fastest)
    sD = stridesD if stridesD is not None else orc.packed_strides(lD, first_fastest)
    nA, nB, nD = span(lA, sA), span(lB, sB), span(lD, sD)
    if fill == "uniform":
        A = orc.fill_uniform(nA, typeAB, seeds[0])
        B = orc.fill_uniform(nB, typeAB, seeds[1])
    else:  # normal(0, 0.5), defined by the oracle's Box-Muller generator
        A = orc.fill_normal(nA, typeAB, seeds[0], 0.5)
        B = orc.fill_normal(nB, typeAB, seeds[1], 0.5)
    C = orc.fill_uniform(nD, typeD, seeds[2]) if with_c else None
    dA = h.tensor_descriptor(lA, sA, typeAB)
    dB = h.tensor_descriptor(lB, sB, typeAB)
    dD = h.tensor_descriptor(lD, sD, typeD)
    dC = dD if with_c else None
    cd = h.contraction_descriptor(dA, modeA, dB, modeB, dC, modeD if with_c else None, dD, modeD, compute)
    find = h.contraction_find(ht.ALGO_DEFAULT if algo is None else algo)
    ws_size = h.contraction_workspace_size(cd, find, ht.WORKSPACE_RECOMMENDED)
    plan = h.contraction_plan(cd, find, ws_size)
    A_d, B_d = to_device(A, typeAB), to_device(B, typeAB)
    C_d = to_device(C, typeD) if with_c else None
    D_d = C_d if (alias and with_c) else to_device(nan_like(nD, typeD), typeD)
    ws = None
    if ws_size:
        import torch

        ws = torch.empty(ws_size, dtype=torch.uint8, device="cuda")
    h.contraction(plan, alpha, A_d, B_d, beta, C_d, D_d, ws, ws_size)
    got = to_host(D_d, typeD)
    if inputs is not None:
        inputs.update(A=A, B=B, C=C, sA=sA, sB=sB, sD=sD, lA=lA, lB=lB, lD=lD)
    if not oracle:
        return got, None, typeD
    exp = nan_like(nD, typeD)
    orc.contraction(alpha, A, lA, sA, modeA, typeAB, B, lB, sB, modeB, typeAB, beta, C, exp, lD, sD, modeD, typeD,
                    compute, sample=sample)
    return got, exp, typeD


def rel_error(got, exp, dt, mask=None):
    """The reference's metric max |d-h|/(|d|+|h|+1) over the written elements; -1 on NaN/Inf."""
    g = orc.to_f64(got, dt)
    e = orc.to_f64(exp, dt)
    if mask is None:
        mask = ~np.isnan(e)
    g, e = g[mask], e[mask]
    if g.size == 0:
        return 0.0
    if not (np.all(np.isfinite(g)) and np.all(np.isfinite(e))):
        return -1.0
    return float(np.max(np.abs(g - e) / (np.abs(g) + np.abs(e) + 1.0)))
