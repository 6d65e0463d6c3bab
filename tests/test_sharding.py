"""Multi-rank host logic on CPU: two gloo ranks run the slab arithmetic of hiptensor_b200.sharding, compute
their slabs with the CPU oracle, and the assembled result must equal the oracle on the whole problem."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _view(flat, shard):
    """numpy strided view of a slab inside the flat global array."""
    itemsize = flat.itemsize
    return np.lib.stride_tricks.as_strided(flat[shard.offset:], shape=shard.lens,
                                           strides=[s * itemsize for s in shard.strides])


def _worker(rank, world, port, out):
    import torch
    import torch.distributed as dist

    from hiptensor_b200 import sharding as sh
    from oracle import binding as orc

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # ---- contraction sharded along free mode m0: slabs of D are disjoint, B is replicated
        m0, m1, n0, k0 = 0, 1, 2, 3
        ext = {m0: 5, m1: 3, n0: 4, k0: 6}
        mA, mB, mD = [m0, m1, k0], [n0, k0], [m0, m1, n0]
        lA, lB, lD = ([ext[m] for m in ms] for ms in (mA, mB, mD))
        sA, sB, sD = (sh.packed_strides(l, False) for l in (lA, lB, lD))
        A = orc.fill_uniform(int(np.prod(lA)), orc.F64, 255)
        B = orc.fill_uniform(int(np.prod(lB)), orc.F64, 256)
        C = orc.fill_uniform(int(np.prod(lD)), orc.F64, 257)
        full = np.zeros_like(C)
        orc.contraction(2.0, A, lA, sA, mA, orc.F64, B, lB, sB, mB, orc.F64, 0.5, C, full, lD, sD, mD, orc.F64,
                        orc.COMPUTE_64F)
        va, vb, vd = sh.shard_contraction(lA, sA, mA, lB, sB, mB, lD, sD, mD, m0, rank, world)
        D = np.zeros_like(C)
        if va.lens[0] > 0:
            orc.contraction(2.0, A[va.offset:], va.lens, va.strides, mA, orc.F64, B[vb.offset:], vb.lens, vb.strides,
                            mB, orc.F64, 0.5, C[vd.offset:], D[vd.offset:], vd.lens, vd.strides, mD, orc.F64,
                            orc.COMPUTE_64F)
        t = torch.from_numpy(D)
        dist.all_reduce(t)  # disjoint slabs: the sum assembles D (test-side gather only)
        ok1 = np.allclose(t.numpy(), full, rtol=1e-13, atol=1e-13)

        # ---- reduction: kept mode sharded (no exchange) and reduced mode sharded (one all-reduce)
        lens, modes, kept = [6, 5, 4], [0, 1, 2], [0, 2]
        sAr = sh.packed_strides(lens, False)
        lDr = [6, 4]
        sDr = sh.packed_strides(lDr, False)
        Ar = orc.fill_uniform(120, orc.F64, 17)
        Cr = orc.fill_uniform(24, orc.F64, 19)
        oks = []
        for op in (orc.OP_ADD, orc.OP_MAX):
            ref = np.zeros(24)
            orc.reduction(1.5, Ar, lens, sAr, modes, orc.F64, 0.5, Cr, ref, lDr, sDr, kept, orc.F64, op,
                          orc.COMPUTE_64F)
            # kept mode 0
            va, vd, exch = sh.shard_reduction(lens, sAr, modes, lDr, sDr, kept, 0, rank, world)
            assert not exch
            Dk = np.zeros(24)
            orc.reduction(1.5, Ar[va.offset:], va.lens, va.strides, modes, orc.F64, 0.5, Cr[vd.offset:],
                          Dk[vd.offset:], vd.lens, vd.strides, kept, orc.F64, op, orc.COMPUTE_64F)
            tk = torch.from_numpy(Dk)
            dist.all_reduce(tk)
            oks.append(np.allclose(tk.numpy(), ref, rtol=1e-13))
            # reduced mode 1: partials with alpha=1, beta=0, then the exchange and the epilogue once
            va, vd, exch = sh.shard_reduction(lens, sAr, modes, lDr, sDr, kept, 1, rank, world)
            assert exch and vd.lens == lDr
            P = np.zeros(24)
            orc.reduction(1.0, Ar[va.offset:], va.lens, va.strides, modes, orc.F64, 0.0, None, P, lDr, sDr, kept,
                          orc.F64, op, orc.COMPUTE_64F)
            # CPU ranks: the epilogue (the reference's order) is the test's own arithmetic
            res = sh.reduce_partials(torch.from_numpy(P), op, 1.5, 0.5, None,
                                     finish=lambda r: r.numpy() * 1.5 + Cr * 0.5)
            oks.append(np.allclose(res, ref, rtol=1e-13))

        # ---- permutation sharded on mode d of B[d,c,b,a] = A[a,b,c,d]
        lensA, modeA, modeB = [4, 3, 2, 6], [0, 1, 2, 3], [3, 2, 1, 0]
        Ap = orc.fill_uniform(144, orc.F32, 256)
        refp = np.zeros(144, dtype=np.float32)
        orc.permutation(1.0, orc.F32, Ap, lensA, modeA, orc.F32, refp, modeB, orc.F32)
        av, bv = sh.shard_permutation(lensA, modeA, modeB, 3, rank, world)
        localA = np.ascontiguousarray(_view(Ap, av).transpose(3, 2, 1, 0)).reshape(-1)  # packed, first mode fastest
        localB = np.zeros_like(localA)
        orc.permutation(1.0, orc.F32, localA, av.lens, modeA, orc.F32, localB, modeB, orc.F32)
        Bp = np.zeros(144, dtype=np.float32)
        _view(Bp, bv)[...] = localB.reshape(bv.lens[::-1]).transpose(3, 2, 1, 0)
        tp = torch.from_numpy(Bp)
        dist.all_reduce(tp)
        ok3 = np.array_equal(tp.numpy(), refp)
        out[rank] = bool(ok1 and all(oks) and ok3)
    finally:
        dist.destroy_process_group()


def test_slab_is_balanced_and_complete():
    from hiptensor_b200.sharding import slab

    for extent in (1, 7, 8, 128, 4096):
        for world in (1, 2, 3, 8):
            parts = [slab(extent, r, world) for r in range(world)]
            assert sum(p.count for p in parts) == extent
            assert parts[0].start == 0
            for a, b in zip(parts, parts[1:]):
                assert b.start == a.start + a.count and a.count - b.count in (0, 1)


def test_two_gloo_ranks():
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}
