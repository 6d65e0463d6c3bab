#!/usr/bin/env python
"""Benchmark of the three hot paths on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c1|c2|c3|c4|c5|c4f32|c2f16|c3col] [--impl reference]

One step = one pass of the hot path over one batch of seeded synthetic input, called through the
library's C ABI. The default workload is the second of the five benchmark configurations (c2): the fp32 rank-4 permutation
B[d,c,b,a] = A[a,b,c,d] with all extents 128 (1 GiB in, 1 GiB out), metric HBM GB/s.
With N > 1 (launched by torch.distributed.run) every rank owns one slab of the sharded mode and
runs the same problem on it; no data-path collective is involved ("scaling": "weak").

Printed by rank 0: ONE JSON line with the whole-job throughput (`value`, inputs resident in HBM),
the same metric end to end with pinned host buffers and both copies inside the timed region (`e2e`),
the roofline of the dominant kernel, the CPU baseline measured beside it, the SM clocks sampled
during the timed region and the number of kernels this library launched.

`--impl reference` times the reference's CPU algorithm for the same workload (the CPU oracle in
oracle/, a restatement of hipTensor's own CPU reference; the reference itself needs hipcc and
Composable Kernel and cannot be built here) on the host cores, on a bounded sample of the workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NOMINAL_FP64_TFLOPS = 40.0  # FP64 tensor pipe, nominal: no measured figure exists for it

# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum from the
# ncu captures summarised under profiles/, full-size workloads, one launch each).
NCU_TRAFFIC_BYTES = {"c2": 2113114000, "c3": 2153492640, "c4": 127901952, "c1": 4088320, "c5": 357141760,
                     "c4f32": 637814528, "c2f16": 1025741312, "c3col": 2155740184}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm": float(p["hbm_gbs"]), "bf16": float(p["bf16_tflops"]),
                "bf16_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm": FALLBACK_HBM_GBS, "bf16": FALLBACK_BF16_TFLOPS, "bf16_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load: at or above the median of what was seen
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------- workloads
def packed(lens, first_fastest):
    n = len(lens)
    s = [1] * n
    if first_fastest:
        for i in range(1, n):
            s[i] = s[i - 1] * lens[i - 1]
    else:
        for i in range(n - 2, -1, -1):
            s[i] = s[i + 1] * lens[i + 1]
    return s


class Workload:
    """setup() builds device inputs from the seeded generator; step(stream) enqueues one pass."""
    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "hbm"

    def __init__(self, ht, handle, rank, world):
        self.ht, self.h, self.rank, self.world = ht, handle, rank, world

    def units_per_step(self):  # bytes (hbm) or flops (tensor) one step processes on this rank
        raise NotImplementedError

    # End-to-end pieces. h2d() and d2h() enqueue the copies of one step on the current torch stream and return
    # the bytes moved; twin() gives a second buffer set (own device tensors and host result, shared pinned inputs)
    # so that consecutive steps can overlap.
    DEVICE_BUFFERS = ()
    HOST_RESULTS = ()

    def h2d(self):
        raise NotImplementedError

    def d2h(self):
        raise NotImplementedError

    def twin(self):
        import copy
        import torch
        t = copy.copy(self)
        for name in self.DEVICE_BUFFERS:
            v = getattr(self, name)
            setattr(t, name, None if v is None else torch.empty_like(v))
        for name in self.HOST_RESULTS:
            v = getattr(self, name)
            setattr(t, name, torch.empty_like(v).pin_memory())
        return t

    def e2e_step(self, stream):
        import torch
        with torch.cuda.stream(stream):
            nin = self.h2d()
            self.step(stream)
            nout = self.d2h()
        return nin, nout

    def host_inputs(self):  # list of pinned host tensors that feed the step
        raise NotImplementedError

    def device_inputs(self):
        raise NotImplementedError

    def result(self):
        raise NotImplementedError


def _fill(n, dt, seed, normal=False):
    """Seeded inputs from the reference harness' generator (test/device/common.hpp:68-108), made on
    the host by the oracle's generator and returned as a torch CPU tensor."""
    import numpy as np
    import torch
    from oracle import binding as orc

    a = orc.fill_normal(n, dt, seed, 0.5) if normal else orc.fill_uniform(n, dt, seed)
    t = torch.from_numpy(a)
    return t


class PermutationC2(Workload):
    name, metric, unit, dtype, bound = "c2", "permutation_hbm_gbs", "GB/s", "f32", "hbm"
    E = 128

    def setup(self):
        import torch
        ht = self.ht
        e = self.E
        n = e ** 4
        # rank r owns slab d in [r*128, (r+1)*128) of a tensor whose mode d has extent 128*world
        self.A_host = _fill(n, 0, 256 + self.rank).pin_memory()
        self.A = self.A_host.cuda(non_blocking=True)
        self.B = torch.empty(n, dtype=torch.float32, device="cuda")
        self.B_host = torch.empty(n, dtype=torch.float32).pin_memory()
        self.desc = self.h.tensor_descriptor([e] * 4, None, ht.R_32F)
        self.bytes = 2 * n * 4

    def step(self, stream):
        self.h.permutation(1.0, self.A, self.desc, [0, 1, 2, 3], self.B, self.desc, [3, 2, 1, 0], self.ht.R_32F, stream)

    def units_per_step(self):
        return self.bytes

    DEVICE_BUFFERS = ("A", "B")
    HOST_RESULTS = ("B_host",)

    def h2d(self):
        self.A.copy_(self.A_host, non_blocking=True)
        return self.A_host.numel() * self.A_host.element_size()

    def d2h(self):
        self.B_host.copy_(self.B, non_blocking=True)
        return self.B_host.numel() * self.B_host.element_size()

    def config(self):
        return {"workload": "c2: fp32 permutation B[d,c,b,a]=A[a,b,c,d], extents 128, 1 GiB in + 1 GiB out per GPU",
                "parallelism": "mode d sharded, one slab of 128 per GPU, no collective",
                "cache": "inputs (1 GiB) larger than L2 (126 MB), no flush needed", "alpha": 1.0}

    def cpu_sample(self, nthreads):
        """Oracle permutation on a slab of the same problem (d restricted to 64): same access pattern."""
        import numpy as np
        from oracle import binding as orc
        lens = [self.E, self.E, self.E, 64]
        n = int(np.prod(lens))
        A = orc.fill_uniform(n, orc.F32, 256)
        B = np.empty(n, dtype=np.float32)
        t0 = time.perf_counter()
        orc.permutation(1.0, orc.F32, A, lens, [0, 1, 2, 3], orc.F32, B, [3, 2, 1, 0], orc.F32, nthreads=nthreads)
        dt = time.perf_counter() - t0
        return 2 * n * 4 / dt / 1e9, "oracle permutation of the slab extents [128,128,128,64] (512 MiB in + 512 MiB out)"


class PermutationC2F16(PermutationC2):
    """Not one of the five benchmark configurations: config 2 with f16 elements (the generic shared-memory tile kernel)."""
    name, dtype = "c2f16", "f16"

    def setup(self):
        import torch
        ht = self.ht
        e = self.E
        n = e ** 4
        self.A_host = _fill(n, 2, 256 + self.rank).pin_memory()
        self.A = self.A_host.cuda(non_blocking=True)
        self.B = torch.empty(n, dtype=torch.float16, device="cuda")
        self.B_host = torch.empty(n, dtype=torch.float16).pin_memory()
        self.desc = self.h.tensor_descriptor([e] * 4, None, ht.R_16F)
        self.bytes = 2 * n * 2

    def step(self, stream):
        self.h.permutation(1.0, self.A, self.desc, [0, 1, 2, 3], self.B, self.desc, [3, 2, 1, 0], self.ht.R_16F, stream)

    def config(self):
        return {"workload": "c2f16: f16 permutation B[d,c,b,a]=A[a,b,c,d], extents 128, 512 MiB in + 512 MiB out per GPU",
                "parallelism": "mode d sharded, one slab of 128 per GPU, no collective",
                "cache": "inputs (512 MiB) larger than L2 (126 MB), no flush needed", "alpha": 1.0}

    def cpu_sample(self, nthreads):
        import numpy as np
        from oracle import binding as orc
        lens = [self.E, self.E, self.E, 64]
        n = int(np.prod(lens))
        A = orc.fill_uniform(n, orc.F16, 256)
        B = np.empty(n, dtype=np.float16)
        t0 = time.perf_counter()
        orc.permutation(1.0, orc.F16, A, lens, [0, 1, 2, 3], orc.F16, B, [3, 2, 1, 0], orc.F16, nthreads=nthreads)
        dt = time.perf_counter() - t0
        return 2 * n * 2 / dt / 1e9, "oracle permutation of the slab extents [128,128,128,64] (256 MiB in + 256 MiB out)"


class ReductionC3(Workload):
    name, metric, unit, dtype, bound = "c3", "reduction_hbm_gbs", "GB/s", "f32", "hbm"
    LENS = [4096, 64, 64, 32]

    def setup(self, op=None):
        import numpy as np
        import torch
        ht = self.ht
        self.op = ht.OP_ADD if op is None else op
        lens = self.LENS
        n = int(np.prod(lens))
        self.A_host = _fill(n, 0, 17 + self.rank).pin_memory()
        self.A = self.A_host.cuda(non_blocking=True)
        self.C_host = _fill(lens[0] * lens[1], 0, 19).pin_memory()
        self.C = self.C_host.cuda()
        self.D = torch.zeros(lens[0] * lens[1], dtype=torch.float32, device="cuda")
        self.D_host = torch.empty(lens[0] * lens[1], dtype=torch.float32).pin_memory()
        self.dA = self.h.tensor_descriptor(lens, None, ht.R_32F)
        self.dD = self.h.tensor_descriptor(lens[:2], None, ht.R_32F)
        self.bytes = n * 4 + 2 * lens[0] * lens[1] * 4

    def step(self, stream):
        ht = self.ht
        self.h.reduction(1.0, self.A, self.dA, [0, 1, 2, 3], 0.5, self.C, self.dD, [0, 1], self.D, self.dD, [0, 1],
                         self.op, ht.COMPUTE_32F, None, 0, stream)

    def units_per_step(self):
        return self.bytes

    DEVICE_BUFFERS = ("A", "C", "D")
    HOST_RESULTS = ("D_host",)

    def h2d(self):
        self.A.copy_(self.A_host, non_blocking=True)
        self.C.copy_(self.C_host, non_blocking=True)
        return (self.A_host.numel() + self.C_host.numel()) * 4

    def d2h(self):
        self.D_host.copy_(self.D, non_blocking=True)
        return self.D_host.numel() * 4

    def config(self):
        return {"workload": "c3: fp32 reduction A[4096,64,64,32] over {k,h} -> D[4096,64] = 1.0*sum + 0.5*C (ADD), "
                            "NULL strides (contiguous 2048-element rows), 2 GiB in per GPU",
                "parallelism": "mode m sharded, one slab of 4096 per GPU, no collective",
                "cache": "input (2 GiB) larger than L2 (126 MB), no flush needed"}

    def cpu_sample(self, nthreads):
        import numpy as np
        from oracle import binding as orc
        lens = [512, 64, 64, 32]
        n = int(np.prod(lens))
        A = orc.fill_uniform(n, orc.F32, 17)
        C = orc.fill_uniform(lens[0] * lens[1], orc.F32, 19)
        D = np.zeros(lens[0] * lens[1], dtype=np.float32)
        t0 = time.perf_counter()
        orc.reduction(1.0, A, lens, packed(lens, False), [0, 1, 2, 3], orc.F32, 0.5, C, D, lens[:2],
                      packed(lens[:2], False), [0, 1], orc.F32, orc.OP_ADD, orc.COMPUTE_32F, nthreads=nthreads)
        dt = time.perf_counter() - t0
        return (n * 4 + 2 * D.size * 4) / dt / 1e9, "oracle reduction of the slab m=512 (256 MiB in)"


class ReductionC3Col(ReductionC3):
    """Not a separate benchmark configuration: config 3 with explicit first-mode-fastest strides (m contiguous), the
    strided "column" reduction."""
    name = "c3col"

    def setup(self, op=None):
        super().setup(op)
        ht = self.ht
        lens = self.LENS
        self.dA = self.h.tensor_descriptor(lens, packed(lens, True), ht.R_32F)
        self.dD = self.h.tensor_descriptor(lens[:2], packed(lens[:2], True), ht.R_32F)

    def config(self):
        c = super().config()
        c["workload"] = ("c3col: fp32 reduction A[4096,64,64,32] over {k,h} -> D[4096,64] = 1.0*sum + 0.5*C (ADD), "
                         "first mode fastest (m contiguous, reduced elements 1 MiB apart), 2 GiB in per GPU")
        return c

    def cpu_sample(self, nthreads):
        import numpy as np
        from oracle import binding as orc
        lens = [512, 64, 64, 32]
        n = int(np.prod(lens))
        A = orc.fill_uniform(n, orc.F32, 17)
        C = orc.fill_uniform(lens[0] * lens[1], orc.F32, 19)
        D = np.zeros(lens[0] * lens[1], dtype=np.float32)
        t0 = time.perf_counter()
        orc.reduction(1.0, A, lens, packed(lens, True), [0, 1, 2, 3], orc.F32, 0.5, C, D, lens[:2],
                      packed(lens[:2], True), [0, 1], orc.F32, orc.OP_ADD, orc.COMPUTE_32F, nthreads=nthreads)
        dt = time.perf_counter() - t0
        return (n * 4 + 2 * D.size * 4) / dt / 1e9, "oracle reduction of the slab m=512 (256 MiB in), first mode fastest"


class ContractionBase(Workload):
    bound = "tensor"
    unit = "TFLOP/s"

    def _setup(self, ext, mA, mB, mD, dt, dtD, compute, alpha, beta, with_c, first_fastest, normal, seeds):
        import numpy as np
        import torch
        ht = self.ht
        lA, lB, lD = ([ext[m] for m in ms] for ms in (mA, mB, mD))
        sA, sB, sD = (packed(l, first_fastest) for l in (lA, lB, lD))
        tdt = {0: torch.float32, 1: torch.float64, 2: torch.float16}
        self.A_host = _fill(int(np.prod(lA)), dt, seeds[0] + self.rank, normal).pin_memory()
        self.B_host = _fill(int(np.prod(lB)), dt, seeds[1], normal).pin_memory()
        self.C_host = _fill(int(np.prod(lD)), dtD, seeds[2]).pin_memory() if with_c else None
        self.A, self.B = self.A_host.cuda(), self.B_host.cuda()
        self.C = self.C_host.cuda() if with_c else None
        self.D = torch.empty(int(np.prod(lD)), dtype=tdt[dtD], device="cuda")
        self.D_host = torch.empty(int(np.prod(lD)), dtype=tdt[dtD]).pin_memory()
        dA = self.h.tensor_descriptor(lA, sA, dt)
        dB = self.h.tensor_descriptor(lB, sB, dt)
        dD = self.h.tensor_descriptor(lD, sD, dtD)
        cd = self.h.contraction_descriptor(dA, mA, dB, mB, dD if with_c else None, mD if with_c else None, dD, mD,
                                           compute)
        find = self.h.contraction_find(ht.ALGO_DEFAULT)
        self.ws_size = self.h.contraction_workspace_size(cd, find, ht.WORKSPACE_RECOMMENDED)
        self.ws = torch.empty(max(self.ws_size, 1), dtype=torch.uint8, device="cuda")
        self.plan = self.h.contraction_plan(cd, find, self.ws_size)
        self.alpha, self.beta = alpha, beta
        self.keep = (dA, dB, dD, cd, find)

    def step(self, stream):
        self.h.contraction(self.plan, self.alpha, self.A, self.B, self.beta, self.C, self.D, self.ws, self.ws_size,
                           stream)

    def units_per_step(self):
        return self.flops

    DEVICE_BUFFERS = ("A", "B", "C", "D", "ws")
    HOST_RESULTS = ("D_host",)

    def h2d(self):
        self.A.copy_(self.A_host, non_blocking=True)
        self.B.copy_(self.B_host, non_blocking=True)
        nb = self.A_host.numel() * self.A_host.element_size() + self.B_host.numel() * self.B_host.element_size()
        if self.C is not None:
            self.C.copy_(self.C_host, non_blocking=True)
            nb += self.C_host.numel() * self.C_host.element_size()
        return nb

    def d2h(self):
        self.D_host.copy_(self.D, non_blocking=True)
        return self.D_host.numel() * self.D_host.element_size()


class ContractionC4(ContractionBase):
    name, metric, dtype = "c4", "contraction_tflops", "f16 inputs, f32 accumulate and output"

    def setup(self):
        m0, m1, n0, n1, k0, k1 = range(6)
        self._setup({m: 64 for m in range(6)}, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], 2, 0,
                    self.ht.COMPUTE_32F, 1.0, 0.0, False, False, True, (255, 256, 257))
        self.flops = 2 * 4096 ** 3

    def config(self):
        return {"workload": "c4: f16 x f16 -> f32 contraction D[m0,m1,n0,n1]=A[m0,m1,k0,k1]*B[n0,n1,k0,k1], extents 64 "
                            "(folded M=N=K=4096), k modes innermost, alpha=1, beta=0, values normal(0,0.5)",
                "parallelism": "mode m0 sharded, one slab of 64 per GPU, B replicated, no collective",
                "cache": "operands (64 MiB) fit L2 (126 MB); a 256 MiB buffer is written between steps to flush it"}

    flush_l2 = True

    def cpu_sample(self, nthreads):
        import numpy as np
        from oracle import binding as orc
        m0, m1, n0, n1, k0, k1 = range(6)
        l = [64] * 4
        s = packed(l, False)
        A = orc.fill_normal(64 ** 4, orc.F16, 255, 0.5)
        B = orc.fill_normal(64 ** 4, orc.F16, 256, 0.5)
        D = np.empty(64 ** 4, dtype=np.float32)
        smp = np.random.default_rng(0).integers(0, 64 ** 4, 65536)
        t0 = time.perf_counter()
        orc.contraction(1.0, A, l, s, [m0, m1, k0, k1], orc.F16, B, l, s, [n0, n1, k0, k1], orc.F16, 0.0, None, D, l, s,
                        [m0, m1, n0, n1], orc.F32, orc.COMPUTE_32F, sample=smp, nthreads=nthreads)
        dt = time.perf_counter() - t0
        return 2 * 65536 * 4096 / dt / 1e12, "oracle on 65536 sampled outputs (268 M multiply-adds), exact k order"


class ContractionC4F32(ContractionBase):
    """Not one of the five benchmark configurations: config 4's shape with fp32 operands, the large case of the fp32 tensor-core kernel."""
    name, metric, dtype = "c4f32", "contraction_tflops", "f32 (TF32 big/small split, three MMAs per product)"

    def setup(self):
        m0, m1, n0, n1, k0, k1 = range(6)
        self._setup({m: 64 for m in range(6)}, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], 0, 0,
                    self.ht.COMPUTE_32F, 1.0, 0.0, False, False, True, (255, 256, 257))
        self.flops = 2 * 4096 ** 3

    def config(self):
        return {"workload": "c4f32: config 4 with fp32 operands, D[m0,m1,n0,n1]=A[m0,m1,k0,k1]*B[n0,n1,k0,k1], extents 64 "
                            "(folded M=N=K=4096), k modes innermost, alpha=1, beta=0, values normal(0,0.5)",
                "parallelism": "mode m0 sharded, one slab of 64 per GPU, B replicated, no collective",
                "cache": "operands (128 MiB) about fill L2 (126 MB); a 256 MiB buffer is written between steps to flush it"}

    flush_l2 = True

    def cpu_sample(self, nthreads):
        import numpy as np
        from oracle import binding as orc
        m0, m1, n0, n1, k0, k1 = range(6)
        l = [64] * 4
        s = packed(l, False)
        A = orc.fill_normal(64 ** 4, orc.F32, 255, 0.5)
        B = orc.fill_normal(64 ** 4, orc.F32, 256, 0.5)
        D = np.empty(64 ** 4, dtype=np.float32)
        smp = np.random.default_rng(0).integers(0, 64 ** 4, 65536)
        t0 = time.perf_counter()
        orc.contraction(1.0, A, l, s, [m0, m1, k0, k1], orc.F32, B, l, s, [n0, n1, k0, k1], orc.F32, 0.0, None, D, l, s,
                        [m0, m1, n0, n1], orc.F32, orc.COMPUTE_32F, sample=smp, nthreads=nthreads)
        dt = time.perf_counter() - t0
        return 2 * 65536 * 4096 / dt / 1e12, "oracle on 65536 sampled outputs (268 M multiply-adds), exact k order"


class ContractionC1(ContractionBase):
    name, metric, dtype = "c1", "contraction_tflops", "f32"

    def setup(self):
        m0, m1, n0, n1, k0, k1 = range(6)
        self._setup({m: 24 for m in range(6)}, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], 0, 0,
                    self.ht.COMPUTE_32F, 1.0, 1.0, True, True, False, (255, 256, 257))
        self.flops = 2 * 576 ** 3

    flush_l2 = True

    def config(self):
        return {"workload": "c1: fp32 bilinear contraction, all extents 24 (folded M=N=K=576), first mode fastest, "
                            "alpha=beta=1 (0.38 GFLOP: latency bound)",
                "parallelism": "replicas", "cache": "5 MiB problem; L2 flushed between steps"}

    def cpu_sample(self, nthreads):
        import numpy as np
        from oracle import binding as orc
        m0, m1, n0, n1, k0, k1 = range(6)
        l = [24] * 4
        s = packed(l, True)
        A = orc.fill_uniform(24 ** 4, orc.F32, 255)
        B = orc.fill_uniform(24 ** 4, orc.F32, 256)
        C = orc.fill_uniform(24 ** 4, orc.F32, 257)
        D = np.empty(24 ** 4, dtype=np.float32)
        t0 = time.perf_counter()
        orc.contraction(1.0, A, l, s, [m0, m1, k0, k1], orc.F32, B, l, s, [n0, n1, k0, k1], orc.F32, 1.0, C, D, l, s,
                        [m0, m1, n0, n1], orc.F32, orc.COMPUTE_32F, nthreads=nthreads)
        dt = time.perf_counter() - t0
        return 2 * 576 ** 3 / dt / 1e12, "oracle on the whole problem"


class ContractionC5(ContractionBase):
    name, metric, dtype = "c5", "contraction_tflops", "f64"

    def setup(self):
        m0, m1, m2, n0, n1, k0, k1 = range(7)
        ext = {m0: 16, m1: 16, m2: 16, n0: 48, n1: 48, k0: 48, k1: 48}
        self._setup(ext, [m0, k0, m1, k1, m2], [k1, n0, k0, n1], [m0, m1, m2, n0, n1], 1, 1, self.ht.COMPUTE_64F, 2.0,
                    0.5, True, False, False, (255, 256, 257))
        self.flops = 2 * 4096 * 2304 * 2304

    flush_l2 = True

    def config(self):
        return {"workload": "c5: fp64 contraction D[m0,m1,m2,n0,n1]=2.0*A[m0,k0,m1,k1,m2]*B[k1,n0,k0,n1]+0.5*C, "
                            "m=16, n=k=48 (folded M=4096, N=K=2304), packed last-mode-fastest",
                "parallelism": "replicas", "cache": "L2 flushed between steps"}

    def cpu_sample(self, nthreads):
        import numpy as np
        from oracle import binding as orc
        m0, m1, m2, n0, n1, k0, k1 = range(7)
        lA, lB, lD = [16, 48, 16, 48, 16], [48, 48, 48, 48], [16, 16, 16, 48, 48]
        A = orc.fill_uniform(int(np.prod(lA)), orc.F64, 255)
        B = orc.fill_uniform(int(np.prod(lB)), orc.F64, 256)
        C = orc.fill_uniform(int(np.prod(lD)), orc.F64, 257)
        D = np.empty(int(np.prod(lD)), dtype=np.float64)
        smp = np.random.default_rng(0).integers(0, int(np.prod(lD)), 65536)
        t0 = time.perf_counter()
        orc.contraction(2.0, A, lA, packed(lA, False), [m0, k0, m1, k1, m2], orc.F64, B, lB, packed(lB, False),
                        [k1, n0, k0, n1], orc.F64, 0.5, C, D, lD, packed(lD, False), [m0, m1, m2, n0, n1], orc.F64,
                        orc.COMPUTE_64F, sample=smp, nthreads=nthreads)
        dt = time.perf_counter() - t0
        return 2 * 65536 * 2304 / dt / 1e12, "oracle on 65536 sampled outputs (151 M multiply-adds), exact k order"


WORKLOADS = {"c1": ContractionC1, "c2": PermutationC2, "c3": ReductionC3, "c4": ContractionC4, "c5": ContractionC5,
             "c4f32": ContractionC4F32, "c2f16": PermutationC2F16, "c3col": ReductionC3Col}


# --------------------------------------------------------------------------------------------- timing
def time_steps(wl, steps, warmup, stream, flusher=None):
    """Device time of `steps` passes (ms, total) measured with CUDA events on the launch stream.
    With a flusher the L2-flush write runs between steps, outside the per-step event pairs."""
    import torch
    for _ in range(warmup):
        if flusher is not None:
            flusher()
        wl.step(stream)
    torch.cuda.synchronize()
    if flusher is None:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(steps):
            wl.step(stream)
        stop.record(stream)
        torch.cuda.synchronize()
        return start.elapsed_time(stop)
    total = 0.0
    pairs = []
    for _ in range(steps):
        flusher()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        wl.step(stream)
        e.record(stream)
        pairs.append((s, e))
    torch.cuda.synchronize()
    for s, e in pairs:
        total += s.elapsed_time(e)
    return total


def run_gpu(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import hiptensor_b200 as ht
    h = ht.Handle()
    wl = WORKLOADS[args.workload](ht, h, rank, world)
    wl.setup()
    stream = torch.cuda.current_stream()
    flusher = None
    if getattr(wl, "flush_l2", False):
        scratch = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device="cuda")
        flusher = lambda: scratch.fill_(1.0)  # noqa: E731

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput
    time_steps(wl, 0, args.warmup, stream, flusher)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = ht.kernel_launch_count()
    ms = time_steps(wl, args.steps, 0, stream, flusher)
    launches = ht.kernel_launch_count() - launches0
    barrier()
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    units = wl.units_per_step() * args.steps * world
    scale = 1e9 if wl.bound == "hbm" else 1e12
    value = units / (ms_max / 1e3) / scale

    # ---- end to end: pinned host buffers, H2D of the inputs and D2H of the result of EVERY step inside the region.
    # Two buffer sets and three streams let the copy-in of step i+1, the kernel of step i and the copy-out of step
    # i-1 overlap (PCIe is full duplex), as an application streaming batches through the library would run it.
    e2e_steps = max(2, min(args.steps, 8))
    sets = [wl, wl.twin()]
    for w in sets:
        w.e2e_step(stream)
    barrier()
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_cmp, ev_out = [None, None], [None, None]
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(s_in)
    for i in range(e2e_steps):
        j = i % 2
        w = sets[j]
        if ev_cmp[j] is not None:
            s_in.wait_event(ev_cmp[j])  # the set's inputs are free once its previous kernel has run
        with torch.cuda.stream(s_in):
            h2d = w.h2d()
        ev_in = torch.cuda.Event()
        ev_in.record(s_in)
        s_cmp.wait_event(ev_in)
        if ev_out[j] is not None:
            s_cmp.wait_event(ev_out[j])  # its result buffer is free once the previous copy-out is done
        w.step(s_cmp)
        ev_cmp[j] = torch.cuda.Event()
        ev_cmp[j].record(s_cmp)
        s_out.wait_event(ev_cmp[j])
        with torch.cuda.stream(s_out):
            d2h = w.d2h()
        ev_out[j] = torch.cuda.Event()
        ev_out[j].record(s_out)
    e.record(s_out)  # the last copy-out ends the region
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = wl.units_per_step() * e2e_steps * world / (float(t.item()) / 1e3) / scale

    if rank == 0:
        pk = peaks()
        per_launch_ms = ms / max(args.steps, 1)  # rank 0's own kernel time; one launch of the dominant kernel per step
        achieved = wl.units_per_step() / (per_launch_ms / 1e3) / scale
        if wl.bound == "hbm":
            peak, punit = pk["hbm"], "GB/s"
        elif wl.name == "c5":
            peak, punit = NOMINAL_FP64_TFLOPS, "TFLOP/s"
        elif wl.name in ("c1", "c4f32"):
            # fp32 on the tensor cores: TF32 runs at half the bf16 rate and every product takes three MMAs
            peak, punit = round(pk["bf16"] / 6.0, 1), "TFLOP/s"
        else:
            peak, punit = pk["bf16"], "TFLOP/s"
        roof = {"bound": wl.bound, "achieved": round(achieved, 2), "peak": peak, "unit": punit,
                "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC_BYTES.get(wl.name),
                "peak_source": "nominal FP64 tensor pipe (no measured figure)" if wl.name == "c5" else
                (("of measured (MEASURED_PEAKS.json)" if pk["source"] == "measured" else "of fallback")
                 + ("; bf16 rate / 2 for TF32 / 3 MMAs per product" if wl.name in ("c1", "c4f32") else "")),
                "kernel": ht.last_kernel_name()}
        ncores = os.cpu_count() or 1
        cpu_value, sample = wl.cpu_sample(ncores)
        line = {
            "metric": wl.metric, "value": round(value, 2), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_max / max(args.steps, 1), 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic", "config": wl.config(),
            "roofline": roof,
            "cpu_baseline": {"value": round(cpu_value, 4), "unit": wl.unit, "cores": ncores, "kind": "port",
                             "sample": sample},
            "e2e": {"value": round(e2e_value, 3), "unit": wl.unit, "h2d_bytes_per_step": int(h2d),
                    "d2h_bytes_per_step": int(d2h), "steps": e2e_steps,
                    "overlap": "two buffer sets, three streams: copy-in, kernel and copy-out of consecutive steps overlap"},
            "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU algorithm for the workload, timed on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from oracle import binding as orc
    orc.build()
    cls = WORKLOADS[args.workload]
    wl = cls(None, None, 0, 1)
    ncores = os.cpu_count() or 1
    for _ in range(min(args.warmup, 1)):
        wl.cpu_sample(ncores)
    vals = []
    t0 = time.perf_counter()
    sample = ""
    for _ in range(max(1, min(args.steps, 5))):
        v, sample = wl.cpu_sample(ncores)
        vals.append(v)
    wall = time.perf_counter() - t0
    value = statistics.median(vals)
    line = {
        "impl": "reference", "metric": cls.metric, "value": round(value, 4), "unit": cls.unit, "n_gpus": world,
        "steps": len(vals), "warmup": min(args.warmup, 1), "ms_per_step": round(wall / len(vals) * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": cls.dtype, "data": "synthetic",
        "config": dict(cls.config(wl), note="CPU restatement of hipTensor's own CPU reference (the reference needs "
                                            "hipcc + Composable Kernel and cannot be built here); each step is a "
                                            "bounded sample of the workload: " + sample),
        "cpu_baseline": {"value": round(value, 4), "unit": cls.unit, "cores": ncores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
