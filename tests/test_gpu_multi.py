"""Two GPUs, one process each: a reduction whose REDUCED mode is sharded finishes with one NCCL all-reduce
of the partial results (hiptensor_b200.sharding.reduce_partials), a reduction sharded on a kept mode and
a contraction sharded on a free mode need no exchange. Skipped when fewer than two GPUs are visible."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import hiptensor_b200 as ht
        from hiptensor_b200 import sharding as sh
        from oracle import binding as orc

        h = ht.Handle()
        lens, modes, kept = [64, 96, 128], [0, 1, 2], [0, 2]
        sA = sh.packed_strides(lens, False)
        lD = [64, 128]
        sD = sh.packed_strides(lD, False)
        A = orc.fill_uniform(int(np.prod(lens)), orc.F32, 17)
        C = orc.fill_uniform(64 * 128, orc.F32, 19)
        A_d, C_d = torch.from_numpy(A).cuda(), torch.from_numpy(C).cuda()
        ok = []
        for op in (ht.OP_ADD, ht.OP_MAX):
            ref = np.zeros(64 * 128, dtype=np.float64)
            orc.reduction(1.5, A.astype(np.float64), lens, sA, modes, orc.F64, 0.5, C.astype(np.float64), ref, lD, sD,
                          kept, orc.F64, op, orc.COMPUTE_64F)
            # reduced mode 1 sharded: partial results, one all-reduce, epilogue applied once
            va, vd, exch = sh.shard_reduction(lens, sA, modes, lD, sD, kept, 1, rank, world)
            assert exch
            dA = h.tensor_descriptor(va.lens, va.strides, ht.R_32F)
            dD = h.tensor_descriptor(vd.lens, vd.strides, ht.R_32F)
            P = torch.zeros(64 * 128, device="cuda")
            h.reduction(1.0, A_d[va.offset:], dA, modes, 0.0, P, dD, kept, P, dD, kept, op, ht.COMPUTE_32F)
            res = sh.reduce_partials(P, op, 1.5, 0.5, C_d, handle=h, descD=dD, type_compute=ht.COMPUTE_32F)
            ok.append(ht.last_kernel_name() == "red_finish")
            ok.append(np.allclose(res.cpu().numpy(), ref, rtol=2e-5, atol=2e-5))
            # kept mode 0 sharded: disjoint slabs of D, no exchange
            va, vd, exch = sh.shard_reduction(lens, sA, modes, lD, sD, kept, 0, rank, world)
            assert not exch
            dA = h.tensor_descriptor(va.lens, va.strides, ht.R_32F)
            dD = h.tensor_descriptor(vd.lens, vd.strides, ht.R_32F)
            D = torch.zeros(64 * 128, device="cuda")
            h.reduction(1.5, A_d[va.offset:], dA, modes, 0.5, C_d[vd.offset:], dD, kept, D[vd.offset:], dD, kept, op,
                        ht.COMPUTE_32F)
            dist.all_reduce(D)  # test-side gather of the disjoint slabs
            ok.append(np.allclose(D.cpu().numpy(), ref, rtol=2e-5, atol=2e-5))
        # ---- contraction sharded along the free mode m0: every rank computes its slab of D from its slab of A (offset
        # views of the global tensors with the global strides) and the whole of B; no exchange
        m0, m1, n0, k0 = 0, 1, 2, 3
        ext = {m0: 6, m1: 64, n0: 192, k0: 136}
        mA, mB, mD = [m0, m1, k0], [n0, k0], [m0, m1, n0]
        lA, lB, lD = ([ext[m] for m in ms] for ms in (mA, mB, mD))
        sA2, sB2, sD2 = (sh.packed_strides(l, False) for l in (lA, lB, lD))
        A2 = orc.fill_normal(int(np.prod(lA)), orc.F16, 255, 0.5)
        B2 = orc.fill_normal(int(np.prod(lB)), orc.F16, 256, 0.5)
        C2 = orc.fill_uniform(int(np.prod(lD)), orc.F32, 257)
        full = np.zeros_like(C2)
        orc.contraction(1.5, A2, lA, sA2, mA, orc.F16, B2, lB, sB2, mB, orc.F16, 0.5, C2, full, lD, sD2, mD, orc.F32,
                        orc.COMPUTE_32F)
        va, vb, vd = sh.shard_contraction(lA, sA2, mA, lB, sB2, mB, lD, sD2, mD, m0, rank, world)
        A2_d, B2_d, C2_d = torch.from_numpy(A2).cuda(), torch.from_numpy(B2).cuda(), torch.from_numpy(C2).cuda()
        D2_d = torch.zeros_like(C2_d)
        dA2 = h.tensor_descriptor(va.lens, va.strides, ht.R_16F)
        dB2 = h.tensor_descriptor(vb.lens, vb.strides, ht.R_16F)
        dD2 = h.tensor_descriptor(vd.lens, vd.strides, ht.R_32F)
        cd = h.contraction_descriptor(dA2, mA, dB2, mB, dD2, mD, dD2, mD, ht.COMPUTE_32F)
        find = h.contraction_find()
        plan = h.contraction_plan(cd, find, 0)
        h.contraction(plan, 1.5, A2_d[va.offset:], B2_d[vb.offset:], 0.5, C2_d[vd.offset:], D2_d[vd.offset:])
        ok.append(ht.last_kernel_name().startswith("contraction_tcgen05"))
        dist.all_reduce(D2_d)  # test-side gather of the disjoint slabs
        got2 = D2_d.cpu().numpy().astype(np.float64)
        ok.append(float(np.max(np.abs(got2 - full) / (np.abs(got2) + np.abs(full) + 1.0))) < 1e-4)
        out[rank] = all(ok)
    finally:
        dist.destroy_process_group()


def test_two_gpus_sharded_reduction_and_contraction():
    import torch
    import torch.multiprocessing as mp

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    assert dict(out) == {0: True, 1: True}
