"""Seeded random shapes through the planner's form rules, checked against references that share nothing with the
library or the oracle: an fp64 matrix product for mid-size f16 / bf16 contractions (CTA pairs, half tiles, K split,
single CTAs; all four operand layouts, with and without C), torch.permute for permutations (the TMA kernel with short
and long contiguous modes, the copy kernel, the shared-memory kernels), bit-exact there; numpy in fp64 for reductions."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import hiptensor_b200 as ht

    return ht, ht.Handle()


def test_random_mid_size_half_precision_contractions(env):
    import torch

    ht, h = env
    rng = np.random.default_rng(12345)
    kernels = set()
    for _ in range(32):
        M, N, K = int(rng.integers(64, 330)) * 8, int(rng.integers(64, 330)) * 8, int(rng.integers(16, 560)) * 8
        bf, with_c = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        mn_a, mn_b = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        tdt, t = (torch.bfloat16, ht.R_16BF) if bf else (torch.float16, ht.R_16F)
        A = torch.randn(M, K, device="cuda").to(tdt)
        B = torch.randn(N, K, device="cuda").to(tdt)
        C = torch.randn(M, N, device="cuda")
        D = torch.full((M, N), float("nan"), device="cuda")
        As = A.t().contiguous() if mn_a else A.contiguous()  # storage: [K][rows] or [rows][K]
        Bs = B.t().contiguous() if mn_b else B.contiguous()
        dA = h.tensor_descriptor([M, K], [1, M] if mn_a else [K, 1], t)
        dB = h.tensor_descriptor([N, K], [1, N] if mn_b else [K, 1], t)
        dD = h.tensor_descriptor([M, N], [N, 1], ht.R_32F)
        desc = h.contraction_descriptor(dA, [0, 2], dB, [1, 2], dD if with_c else None, [0, 1] if with_c else None, dD,
                                        [0, 1], ht.COMPUTE_32F)
        plan = h.contraction_plan(desc, h.contraction_find(ht.ALGO_DEFAULT), 0)
        alpha, beta = 1.25, (0.5 if with_c else 0.0)
        h.contraction(plan, alpha, As, Bs, beta, C if with_c else None, D, None, 0)
        torch.cuda.synchronize()
        kernels.add(ht.last_kernel_name())
        ref = alpha * (A.double() @ B.double().t()) + (beta * C.double() if with_c else 0)
        assert not torch.isnan(D).any().item(), (M, N, K, ht.last_kernel_name())
        # half-precision inputs: 1e-2 stated; the tensor cores' truncating fp32 accumulation stays below 2e-3 at these K
        err = ((D.double() - ref).abs().max() / ref.abs().max()).item()
        assert err < 2e-3, (M, N, K, bf, with_c, mn_a, mn_b, ht.last_kernel_name(), err)
    assert "contraction_tcgen05_pair" in kernels and "contraction_tcgen05" in kernels


def test_random_permutations(env):
    import torch

    ht, h = env
    rng = np.random.default_rng(777)
    choices = [4, 8, 16, 32, 64, 128, 12, 20, 24, 40, 3, 5, 7, 36, 100]
    kernels = set()
    for _ in range(160):
        rank = int(rng.integers(3, 6))
        lens = [int(rng.choice(choices)) for _ in range(rank)]
        while np.prod(lens) > 4e6:
            lens[int(rng.integers(0, rank))] = 4
        perm = [int(p) for p in rng.permutation(rank)]
        f16 = bool(rng.integers(0, 2))
        tdt, t = (torch.float16, ht.R_16F) if f16 else (torch.float32, ht.R_32F)
        n = int(np.prod(lens))
        A = torch.randn(n, device="cuda").to(tdt)
        B = torch.full((n,), float("nan"), device="cuda", dtype=tdt)
        dA = h.tensor_descriptor(lens, None, t)
        dB = h.tensor_descriptor([lens[p] for p in perm], None, t)
        h.permutation(1.0, A, dA, list(range(rank)), B, dB, perm, t)
        kernels.add(ht.last_kernel_name())
        # first mode fastest: the memory image of A is a torch tensor with the extents reversed
        rp = [rank - 1 - perm[rank - 1 - i] for i in range(rank)]
        ref = A.view(*lens[::-1]).permute(*rp).contiguous().view(-1)
        it = torch.int16 if f16 else torch.int32
        assert torch.equal(B.view(it), ref.view(it)), (lens, perm, f16, ht.last_kernel_name())
    assert {"perm_tma", "perm_copy", "perm_box"} <= kernels  # short contiguous modes take the box kernel


def test_random_reductions(env):
    """Random f32 reductions (ranks 2-5, every kind of kept subset, ADD and MAX, alpha and beta) against numpy in
    fp64: MAX exactly, ADD within 1e-5 of the exact result."""
    import torch

    ht, h = env
    rng = np.random.default_rng(4242)
    choices = [2, 3, 5, 8, 16, 32, 64, 128, 256, 7, 12, 40]
    kernels = set()
    for _ in range(120):
        rank = int(rng.integers(2, 6))
        lens = [int(rng.choice(choices)) for _ in range(rank)]
        while np.prod(lens) > 3e6:
            lens[int(rng.integers(0, rank))] = 2
        nkept = int(rng.integers(0, rank))
        kept = sorted(int(x) for x in rng.choice(rank, size=nkept, replace=False))
        op = ht.OP_MAX if rng.integers(0, 2) else ht.OP_ADD
        A = rng.standard_normal(lens).astype(np.float32)
        lensD = [lens[m] for m in kept] if kept else [1]
        C = rng.standard_normal(lensD).astype(np.float32)
        red = tuple(m for m in range(rank) if m not in kept)
        A64 = A.astype(np.float64)
        r = (A64.max(axis=red) if op == ht.OP_MAX else A64.sum(axis=red)) if red else A64
        ref = 1.5 * np.asarray(r, dtype=np.float64).reshape(lensD) + 0.25 * C.astype(np.float64)
        A_d, C_d = torch.from_numpy(A).cuda(), torch.from_numpy(C).cuda()
        D_d = torch.full(lensD, float("nan"), device="cuda")
        dA = h.tensor_descriptor(lens, None, ht.R_32F)
        dD = h.tensor_descriptor(lensD if kept else [], None, ht.R_32F)  # no kept mode: a rank-0 output
        h.reduction(1.5, A_d, dA, list(range(rank)), 0.25, C_d, dD, kept, D_d, dD, kept, op, ht.COMPUTE_32F)
        kernels.add(ht.last_kernel_name())
        got = D_d.cpu().numpy().astype(np.float64)
        if op == ht.OP_MAX:
            exp32 = (np.float32(1.5) * A.max(axis=red).reshape(lensD) if red else np.float32(1.5) * A.reshape(lensD))
            exp32 = exp32 + np.float32(0.25) * C
            assert np.array_equal(got.astype(np.float32), exp32.astype(np.float32)), (lens, kept, ht.last_kernel_name())
        else:
            scale = max(np.abs(ref).max(), 1e-30)
            assert np.abs(got - ref).max() / scale < 1e-5, (lens, kept, ht.last_kernel_name())
    assert "red_row" in kernels and len(kernels) >= 2
