#!/usr/bin/env python
"""Benchmark of the three hot paths on B200: the five benchmark configurations in one run.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--only c4,c2,...] [--impl reference]

One step = one pass of a hot path over one batch of seeded synthetic input, called through the
library's C ABI. One run measures all five configurations and prints ONE JSON line:

  top level   configuration 4: the f16 x f16 -> f32 contraction D[m0,m1,n0,n1] = A[m0,m1,k0,k1] B[n0,n1,k0,k1],
              extents 64 (folded M = N = K = 4096), metric TFLOP/s;
  "configs"   c1 (fp32 bilinear contraction, extents 24), c2 (fp32 permutation, 1 GiB), c3 and c3max
              (fp32 reduction, ADD and MAX), c5 (fp64 contraction), each with the same sub-fields; with
              N > 1 also c3k (configuration 3 with the REDUCED mode k split over the ranks: partial
              reductions, one NCCL all-reduce of 1 MiB, htReductionFinish).

With N > 1 (launched by torch.distributed.run, one rank per GPU) the FIXED tensors of configurations 2, 3
and 4 are split over the ranks along d, m and m0 ("scaling": "strong"; no data-path collective, B of
configuration 4 replicated); `value` is whole-problem work divided by the slowest rank's time. The number
with every rank running the whole problem is kept as `weak_value`. Configurations 1 and 5 do not shard
(replicas).

Per workload: `value` = device-resident throughput (CUDA events on the launch stream around exactly K
steps, K steps captured once in a CUDA graph and replayed so that kernels run back to back; the buffer
sets rotate so that no step finds its operands in L2; the K-step region is repeated until 200 ms have run
and the median is reported); `e2e` = the same metric through the C ABI with pinned HOST buffers, the H2D
copy of every step's inputs and the D2H copy of its result inside the timed region; `roofline` of the
dominant kernel; `cpu_baseline` (N = 1 only) = the CPU oracle on the host cores; `clocks` sampled during
the timed region.

`--impl reference` times the reference's CPU algorithm (the CPU oracle in oracle/, a restatement of
hipTensor's own CPU reference; the reference itself needs hipcc and Composable Kernel and cannot be built
here) for the same configurations, on all host cores, rank 0 only.
"""
import argparse
import json
import math
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
NOMINAL_BF16_TFLOPS = 2250.0
L2_BYTES = 126 * 1000 * 1000
MIN_LOAD_MS = 200.0  # the K-step region is repeated until this much device time has run

# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture
# of the full-size single-GPU workload) and the summary under profiles/ that holds the capture. Updated together
# with the profile when a kernel changes.
NCU_TRAFFIC = {
    "c1": (4088320, "profiles/contraction_tf32x3_c4f32_c1.md"),
    "c2": (2113114000, "profiles/perm_tma_c2.md"),
    "c2f16": (1031170304, "profiles/perm_tma_c2f16.md"),
    "c3": (2153492640, "profiles/red_row_c3.md"),
    "c3max": (2153492640, "profiles/red_row_c3.md"),
    "c4": (128962816, "profiles/contraction_tcgen05_pair_c4.md"),
    "c5": (398871808, "profiles/contraction_dmma_c5.md"),
}


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
            time.sleep(0.05)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
                power.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # under load: the samples whose power draw is in the upper half of what was seen
        cut = (min(power) + max(power)) / 2.0
        load = [s for s, p in zip(sm, power) if p >= cut] or sm
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "samples": len(sm),
                "samples_under_load": len(load), "power_w_max": max(power), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------- helpers
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


def prod(v):
    r = 1
    for x in v:
        r *= int(x)
    return r


def _fill(n, dt, seed, normal=False):
    """Seeded inputs from the reference harness' generator (test/device/common.hpp:68-108), made on
    the host by the oracle's generator and returned as a torch CPU tensor."""
    import torch
    from oracle import binding as orc

    a = orc.fill_normal(n, dt, seed, 0.5) if normal else orc.fill_uniform(n, dt, seed)
    return torch.from_numpy(a)


class BufferSet:
    """Device tensors of one step plus the pinned host result."""

    def __init__(self, **tensors):
        self.__dict__.update(tensors)


class Workload:
    """setup() builds the host inputs and `nsets` device buffer sets; step(stream, s) enqueues one pass on set s."""
    name = metric = unit = dtype = ""
    bound = "hbm"
    sharded = False  # True: the fixed problem is split over the ranks (strong scaling)

    def __init__(self, ht, handle, rank, world, weak=False):
        self.ht, self.h, self.rank, self.world = ht, handle, rank, world
        # ranks the problem is split over (1: every rank runs the whole problem)
        self.split = world if (self.sharded and not weak) else 1
        self.sets = []

    # work of the WHOLE job per step (all ranks), in bytes or flops
    def units_job(self):
        return self.units_local() * self.world if self.split == 1 else self.units_whole()

    def footprint(self):  # bytes one step touches on this rank
        raise NotImplementedError

    def nsets(self):
        return max(1, min(64, math.ceil(3.0 * L2_BYTES / max(self.footprint(), 1))))

    def release(self):
        import torch

        self.sets = []
        for k in list(self.__dict__):
            if k.endswith("_host") or k in ("ws",):
                self.__dict__.pop(k)
        torch.cuda.empty_cache()


# ----------------------------------------------------------------------------------------------- c2: permutation
class PermutationC2(Workload):
    name, metric, unit, dtype, bound, sharded = "c2", "permutation_hbm_gbs", "GB/s", "f32", "hbm", True
    E = 128

    def setup(self):
        import torch
        ht = self.ht
        e = self.E
        self.d_local = e // self.split
        n = e ** 3 * self.d_local
        self.n = n
        # d is A's slowest mode: a rank's slab is a contiguous range of the global A; its B slab is packed locally
        self.A_host = _fill(n, 0, 256 + (self.rank if self.split > 1 else 0)).pin_memory()
        self.descA = self.h.tensor_descriptor([e, e, e, self.d_local], None, ht.R_32F)
        self.descB = self.h.tensor_descriptor([self.d_local, e, e, e], None, ht.R_32F)
        for _ in range(self.nsets()):
            self.sets.append(BufferSet(A=self.A_host.cuda(non_blocking=True),
                                       B=torch.empty(n, dtype=torch.float32, device="cuda"),
                                       B_host=torch.empty(n, dtype=torch.float32).pin_memory()))

    def step(self, stream, s):
        b = self.sets[s]
        self.h.permutation(1.0, b.A, self.descA, [0, 1, 2, 3], b.B, self.descB, [3, 2, 1, 0], self.ht.R_32F, stream)

    def units_local(self):
        return 2 * self.n * 4

    def units_whole(self):
        return 2 * self.E ** 4 * 4

    def footprint(self):
        return 2 * self.E ** 3 * (self.E // self.split) * 4

    def h2d(self, b):
        b.A.copy_(self.A_host, non_blocking=True)
        return self.n * 4

    def d2h(self, b):
        b.B_host.copy_(b.B, non_blocking=True)
        return self.n * 4

    @classmethod
    def config(cls, world):
        c = {"workload": "c2: fp32 permutation B[d,c,b,a]=A[a,b,c,d], extents 128 (1 GiB in + 1 GiB out), alpha 1",
             "cache": "operands exceed L2 (126 MB); buffer sets rotate so that 3 x L2 is touched between reuses"}
        c["parallelism"] = ("1 GPU" if world == 1 else
                            "mode d split over %d ranks (d = %d each), no collective" % (world, cls.E // world))
        return c

    @classmethod
    def cpu_step(cls, nthreads, state):
        """Oracle permutation of the WHOLE tensor."""
        import numpy as np
        from oracle import binding as orc
        e = cls.E
        if "A" not in state:
            state["A"] = orc.fill_uniform(e ** 4, orc.F32, 256)
            state["B"] = np.empty(e ** 4, dtype=np.float32)
        t0 = time.perf_counter()
        orc.permutation(1.0, orc.F32, state["A"], [e] * 4, [0, 1, 2, 3], orc.F32, state["B"], [3, 2, 1, 0], orc.F32,
                        nthreads=nthreads)
        return 2 * e ** 4 * 4, time.perf_counter() - t0, "oracle permutation of the whole tensor (1 GiB in + 1 GiB out)"


class PermutationC2F16(PermutationC2):
    """Not one of the five configurations: configuration 2 with f16 elements (512 MiB in + 512 MiB out)."""
    name, dtype, sharded = "c2f16", "f16", False

    def setup(self):
        import torch
        ht = self.ht
        e = self.E
        self.d_local = e
        n = e ** 4
        self.n = n
        self.A_host = _fill(n, 2, 256).pin_memory()
        self.descA = self.h.tensor_descriptor([e] * 4, None, ht.R_16F)
        self.descB = self.descA
        for _ in range(self.nsets()):
            self.sets.append(BufferSet(A=self.A_host.cuda(non_blocking=True),
                                       B=torch.empty(n, dtype=torch.float16, device="cuda"),
                                       B_host=torch.empty(n, dtype=torch.float16).pin_memory()))

    def step(self, stream, s):
        b = self.sets[s]
        self.h.permutation(1.0, b.A, self.descA, [0, 1, 2, 3], b.B, self.descB, [3, 2, 1, 0], self.ht.R_16F, stream)

    def units_local(self):
        return 2 * self.n * 2

    def units_whole(self):
        return 2 * self.E ** 4 * 2

    def footprint(self):
        return 2 * self.E ** 4 * 2

    def h2d(self, b):
        b.A.copy_(self.A_host, non_blocking=True)
        return self.n * 2

    def d2h(self, b):
        b.B_host.copy_(b.B, non_blocking=True)
        return self.n * 2

    @classmethod
    def config(cls, world):
        return {"workload": "c2f16: configuration 2 with f16 elements, B[d,c,b,a]=A[a,b,c,d], extents 128 (512 MiB in + "
                            "512 MiB out), alpha 1",
                "cache": "operands exceed L2 (126 MB)",
                "parallelism": "1 GPU" if world == 1 else "%d replicas" % world}

    @classmethod
    def cpu_step(cls, nthreads, state):
        import numpy as np
        from oracle import binding as orc
        e = cls.E
        if "A" not in state:
            state["A"] = orc.fill_uniform(e ** 4, orc.F16, 256)
            state["B"] = np.empty(e ** 4, dtype=np.float16)
        t0 = time.perf_counter()
        orc.permutation(1.0, orc.F16, state["A"], [e] * 4, [0, 1, 2, 3], orc.F16, state["B"], [3, 2, 1, 0], orc.F16,
                        nthreads=nthreads)
        return 2 * e ** 4 * 2, time.perf_counter() - t0, "oracle permutation of the whole tensor (512 MiB in + 512 MiB out)"


# ----------------------------------------------------------------------------------------------- c3: reduction
class ReductionC3(Workload):
    name, metric, unit, dtype, bound, sharded = "c3", "reduction_hbm_gbs", "GB/s", "f32", "hbm", True
    LENS = [4096, 64, 64, 32]
    OP = "ADD"

    def setup(self):
        import torch
        ht = self.ht
        self.op = ht.OP_ADD if self.OP == "ADD" else ht.OP_MAX
        self.lens = [self.LENS[0] // self.split] + self.LENS[1:]
        n = prod(self.lens)
        nd = self.lens[0] * self.lens[1]
        self.n, self.nd = n, nd
        self.A_host = _fill(n, 0, 17 + (self.rank if self.split > 1 else 0)).pin_memory()
        self.C_host = _fill(nd, 0, 19).pin_memory()
        self.dA = self.h.tensor_descriptor(self.lens, None, ht.R_32F)
        self.dD = self.h.tensor_descriptor(self.lens[:2], None, ht.R_32F)
        for _ in range(self.nsets()):
            self.sets.append(BufferSet(A=self.A_host.cuda(non_blocking=True), C=self.C_host.cuda(non_blocking=True),
                                       D=torch.zeros(nd, dtype=torch.float32, device="cuda"),
                                       D_host=torch.empty(nd, dtype=torch.float32).pin_memory()))

    def step(self, stream, s):
        ht, b = self.ht, self.sets[s]
        self.h.reduction(1.0, b.A, self.dA, [0, 1, 2, 3], 0.5, b.C, self.dD, [0, 1], b.D, self.dD, [0, 1],
                         self.op, ht.COMPUTE_32F, None, 0, stream)

    def units_local(self):
        return self.n * 4 + 2 * self.nd * 4

    def units_whole(self):
        return prod(self.LENS) * 4 + 2 * self.LENS[0] * self.LENS[1] * 4

    def footprint(self):
        return (prod(self.LENS) * 4 + 2 * self.LENS[0] * self.LENS[1] * 4) // self.split

    def h2d(self, b):
        b.A.copy_(self.A_host, non_blocking=True)
        b.C.copy_(self.C_host, non_blocking=True)
        return (self.n + self.nd) * 4

    def d2h(self, b):
        b.D_host.copy_(b.D, non_blocking=True)
        return self.nd * 4

    @classmethod
    def config(cls, world):
        c = {"workload": "%s: fp32 reduction A[4096,64,64,32] over {k,h} -> D[4096,64] = 1.0*%s + 0.5*C, NULL "
                         "strides (contiguous 2048-element rows), 2 GiB in" % (cls.name, "sum" if cls.OP == "ADD" else "max"),
             "cache": "input exceeds L2 (126 MB); buffer sets rotate so that 3 x L2 is touched between reuses"}
        c["parallelism"] = ("1 GPU" if world == 1 else
                            "mode m split over %d ranks (m = %d each), no collective" % (world, cls.LENS[0] // world))
        return c

    @classmethod
    def cpu_step(cls, nthreads, state):
        import numpy as np
        from oracle import binding as orc
        lens = cls.LENS
        if "A" not in state:
            state["A"] = orc.fill_uniform(prod(lens), orc.F32, 17)
            state["C"] = orc.fill_uniform(lens[0] * lens[1], orc.F32, 19)
            state["D"] = np.zeros(lens[0] * lens[1], dtype=np.float32)
        t0 = time.perf_counter()
        orc.reduction(1.0, state["A"], lens, packed(lens, False), [0, 1, 2, 3], orc.F32, 0.5, state["C"], state["D"],
                      lens[:2], packed(lens[:2], False), [0, 1], orc.F32, orc.OP_ADD if cls.OP == "ADD" else orc.OP_MAX,
                      orc.COMPUTE_32F, nthreads=nthreads)
        return prod(lens) * 4 + 2 * lens[0] * lens[1] * 4, time.perf_counter() - t0, \
            "oracle reduction of the whole tensor (2 GiB in)"


class ReductionC3Max(ReductionC3):
    name, OP = "c3max", "MAX"


# ----------------------------------------------------------------------------------------------- contractions
class ContractionBase(Workload):
    bound, unit, metric = "tensor", "TFLOP/s", "contraction_tflops"
    TORCH_DT = None

    def _setup(self, ext, mA, mB, mD, dt, dtD, compute, alpha, beta, with_c, first_fastest, normal, seeds):
        import torch
        ht = self.ht
        lA, lB, lD = ([ext[m] for m in ms] for ms in (mA, mB, mD))
        sA, sB, sD = (packed(l, first_fastest) for l in (lA, lB, lD))
        tdt = {0: torch.float32, 1: torch.float64, 2: torch.float16}
        self.A_host = _fill(prod(lA), dt, seeds[0] + (self.rank if self.split > 1 else 0), normal).pin_memory()
        self.B_host = _fill(prod(lB), dt, seeds[1], normal).pin_memory()
        self.C_host = _fill(prod(lD), dtD, seeds[2]).pin_memory() if with_c else None
        dA = self.h.tensor_descriptor(lA, sA, dt)
        dB = self.h.tensor_descriptor(lB, sB, dt)
        dD = self.h.tensor_descriptor(lD, sD, dtD)
        cd = self.h.contraction_descriptor(dA, mA, dB, mB, dD if with_c else None, mD if with_c else None, dD, mD,
                                           compute)
        find = self.h.contraction_find(ht.ALGO_DEFAULT)
        self.ws_size = self.h.contraction_workspace_size(cd, find, ht.WORKSPACE_RECOMMENDED)
        self.plan = self.h.contraction_plan(cd, find, self.ws_size)
        self.alpha, self.beta = alpha, beta
        self.keep = (dA, dB, dD, cd, find)
        self.bytes_in = (self.A_host.numel() * self.A_host.element_size() + self.B_host.numel() * self.B_host.element_size()
                         + (self.C_host.numel() * self.C_host.element_size() if with_c else 0))
        nD = prod(lD)
        self.bytes_out = nD * (8 if dtD == 1 else 4)
        self._fp = self.bytes_in + self.bytes_out
        self.ws = torch.empty(max(self.ws_size, 1), dtype=torch.uint8, device="cuda")
        for _ in range(self.nsets()):
            self.sets.append(BufferSet(A=self.A_host.cuda(non_blocking=True), B=self.B_host.cuda(non_blocking=True),
                                       C=self.C_host.cuda(non_blocking=True) if with_c else None,
                                       D=torch.empty(nD, dtype=tdt[dtD], device="cuda"),
                                       D_host=torch.empty(nD, dtype=tdt[dtD]).pin_memory()))

    def step(self, stream, s):
        b = self.sets[s]
        self.h.contraction(self.plan, self.alpha, b.A, b.B, self.beta, b.C, b.D, self.ws, self.ws_size, stream)

    def units_local(self):
        return self.flops_local

    def units_whole(self):
        return self.FLOPS

    def footprint(self):
        return self._fp

    def h2d(self, b):
        b.A.copy_(self.A_host, non_blocking=True)
        b.B.copy_(self.B_host, non_blocking=True)
        if b.C is not None:
            b.C.copy_(self.C_host, non_blocking=True)
        return self.bytes_in

    def d2h(self, b):
        b.D_host.copy_(b.D, non_blocking=True)
        return self.bytes_out


class ContractionC4(ContractionBase):
    name, dtype, sharded = "c4", "f16 inputs, f32 accumulate and output", True
    FLOPS = 2 * 4096 ** 3

    def setup(self):
        m0, m1, n0, n1, k0, k1 = range(6)
        ext = {m: 64 for m in range(6)}
        ext[m0] = 64 // self.split
        self.flops_local = self.FLOPS // self.split
        self._setup(ext, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], 2, 0, self.ht.COMPUTE_32F, 1.0, 0.0,
                    False, False, True, (255, 256, 257))

    @classmethod
    def config(cls, world):
        c = {"workload": "c4: f16 x f16 -> f32 contraction D[m0,m1,n0,n1]=A[m0,m1,k0,k1]*B[n0,n1,k0,k1], extents 64 "
                         "(folded M=N=K=4096), k modes innermost, alpha=1, beta=0, values normal(0,0.5)",
             "cache": "operand sets rotate so that 3 x L2 (126 MB) is touched between reuses: no step finds its "
                      "operands in L2"}
        c["parallelism"] = ("1 GPU" if world == 1 else
                            "mode m0 split over %d ranks (m0 = %d each, folded M = %d), B replicated, no collective"
                            % (world, 64 // world, 4096 // world))
        return c

    @classmethod
    def cpu_step(cls, nthreads, state):
        import numpy as np
        from oracle import binding as orc
        m0, m1, n0, n1, k0, k1 = range(6)
        l = [64] * 4
        s = packed(l, False)
        if "A" not in state:
            state["A"] = orc.fill_normal(64 ** 4, orc.F16, 255, 0.5)
            state["B"] = orc.fill_normal(64 ** 4, orc.F16, 256, 0.5)
            state["D"] = np.empty(64 ** 4, dtype=np.float32)
            state["smp"] = np.random.default_rng(0).integers(0, 64 ** 4, 65536)
        t0 = time.perf_counter()
        orc.contraction(1.0, state["A"], l, s, [m0, m1, k0, k1], orc.F16, state["B"], l, s, [n0, n1, k0, k1], orc.F16,
                        0.0, None, state["D"], l, s, [m0, m1, n0, n1], orc.F32, orc.COMPUTE_32F, sample=state["smp"],
                        nthreads=nthreads)
        return 2 * 65536 * 4096, time.perf_counter() - t0, \
            "oracle on 65536 sampled outputs of the whole problem (268 M multiply-adds, exact k order); the rate is " \
            "extrapolated to the whole problem"


class ContractionC1(ContractionBase):
    name, dtype = "c1", "f32"
    FLOPS = 2 * 576 ** 3

    def setup(self):
        m0, m1, n0, n1, k0, k1 = range(6)
        self.flops_local = self.FLOPS
        self._setup({m: 24 for m in range(6)}, [m0, m1, k0, k1], [n0, n1, k0, k1], [m0, m1, n0, n1], 0, 0,
                    self.ht.COMPUTE_32F, 1.0, 1.0, True, True, False, (255, 256, 257))

    @classmethod
    def config(cls, world):
        return {"workload": "c1: fp32 bilinear contraction D[m0,m1,n0,n1]=A[m0,m1,k0,k1]*B[n0,n1,k0,k1]+C, all extents "
                            "24 (folded M=N=K=576), first mode fastest, alpha=beta=1 (0.38 GFLOP: latency bound)",
                "cache": "64 operand sets (5 MiB each) rotate so that 3 x L2 is touched between reuses",
                "parallelism": "1 GPU" if world == 1 else "%d replicas (the problem does not shard)" % world}

    @classmethod
    def cpu_step(cls, nthreads, state):
        import numpy as np
        from oracle import binding as orc
        m0, m1, n0, n1, k0, k1 = range(6)
        l = [24] * 4
        s = packed(l, True)
        if "A" not in state:
            state["A"] = orc.fill_uniform(24 ** 4, orc.F32, 255)
            state["B"] = orc.fill_uniform(24 ** 4, orc.F32, 256)
            state["C"] = orc.fill_uniform(24 ** 4, orc.F32, 257)
            state["D"] = np.empty(24 ** 4, dtype=np.float32)
        t0 = time.perf_counter()
        orc.contraction(1.0, state["A"], l, s, [m0, m1, k0, k1], orc.F32, state["B"], l, s, [n0, n1, k0, k1], orc.F32,
                        1.0, state["C"], state["D"], l, s, [m0, m1, n0, n1], orc.F32, orc.COMPUTE_32F, nthreads=nthreads)
        return cls.FLOPS, time.perf_counter() - t0, "oracle on the whole problem"


class ContractionC5(ContractionBase):
    name, dtype = "c5", "f64"
    FLOPS = 2 * 4096 * 2304 * 2304

    def setup(self):
        m0, m1, m2, n0, n1, k0, k1 = range(7)
        ext = {m0: 16, m1: 16, m2: 16, n0: 48, n1: 48, k0: 48, k1: 48}
        self.flops_local = self.FLOPS
        self._setup(ext, [m0, k0, m1, k1, m2], [k1, n0, k0, n1], [m0, m1, m2, n0, n1], 1, 1, self.ht.COMPUTE_64F, 2.0,
                    0.5, True, False, False, (255, 256, 257))

    @classmethod
    def config(cls, world):
        return {"workload": "c5: fp64 contraction D[m0,m1,m2,n0,n1]=2.0*A[m0,k0,m1,k1,m2]*B[k1,n0,k0,n1]+0.5*C, "
                            "m=16, n=k=48 (folded M=4096, N=K=2304), packed last-mode-fastest",
                "cache": "operand sets rotate so that 3 x L2 is touched between reuses",
                "parallelism": "1 GPU" if world == 1 else "%d replicas (not a sharded configuration)" % world}

    @classmethod
    def cpu_step(cls, nthreads, state):
        import numpy as np
        from oracle import binding as orc
        m0, m1, m2, n0, n1, k0, k1 = range(7)
        lA, lB, lD = [16, 48, 16, 48, 16], [48, 48, 48, 48], [16, 16, 16, 48, 48]
        if "A" not in state:
            state["A"] = orc.fill_uniform(prod(lA), orc.F64, 255)
            state["B"] = orc.fill_uniform(prod(lB), orc.F64, 256)
            state["C"] = orc.fill_uniform(prod(lD), orc.F64, 257)
            state["D"] = np.empty(prod(lD), dtype=np.float64)
            state["smp"] = np.random.default_rng(0).integers(0, prod(lD), 65536)
        t0 = time.perf_counter()
        orc.contraction(2.0, state["A"], lA, packed(lA, False), [m0, k0, m1, k1, m2], orc.F64, state["B"], lB,
                        packed(lB, False), [k1, n0, k0, n1], orc.F64, 0.5, state["C"], state["D"], lD, packed(lD, False),
                        [m0, m1, m2, n0, n1], orc.F64, orc.COMPUTE_64F, sample=state["smp"], nthreads=nthreads)
        return 2 * 65536 * 2304, time.perf_counter() - t0, \
            "oracle on 65536 sampled outputs of the whole problem (151 M multiply-adds, exact k order); the rate is " \
            "extrapolated to the whole problem"


class ContractionC5F16(ContractionBase):
    """Not one of the five configurations: the mode layout of configuration 5 (no operand contiguous along a K mode,
    a K group that does not fold) with f16 data and fp32 output, on the tensor-core path for several K modes."""
    name, dtype = "c5f16", "f16 inputs, f32 accumulate and output"
    FLOPS = 2 * 4096 * 2304 * 2304

    def setup(self):
        m0, m1, m2, n0, n1, k0, k1 = range(7)
        ext = {m0: 16, m1: 16, m2: 16, n0: 48, n1: 48, k0: 48, k1: 48}
        self.flops_local = self.FLOPS
        self._setup(ext, [m0, k0, m1, k1, m2], [k1, n0, k0, n1], [m0, m1, m2, n0, n1], 2, 0, self.ht.COMPUTE_32F, 2.0,
                    0.5, True, False, True, (255, 256, 257))

    @classmethod
    def config(cls, world):
        return {"workload": "c5f16: configuration 5's layout D[m0,m1,m2,n0,n1]=2.0*A[m0,k0,m1,k1,m2]*B[k1,n0,k0,n1]+0.5*C "
                            "with f16 data and fp32 output (folded M=4096, N=K=2304): in place both operands are MN-major in "
                            "chunks of 16 (m2) and 48 (n1) valid rows out of 64 with two K modes, so each step first "
                            "copies them into the workspace as packed K-major matrices (two copy kernels, timed with "
                            "the contraction)",
                "cache": "operand sets rotate so that 3 x L2 is touched between reuses",
                "parallelism": "1 GPU" if world == 1 else "%d replicas (not a sharded configuration)" % world}

    @classmethod
    def cpu_step(cls, nthreads, state):
        import numpy as np
        from oracle import binding as orc
        m0, m1, m2, n0, n1, k0, k1 = range(7)
        lA, lB, lD = [16, 48, 16, 48, 16], [48, 48, 48, 48], [16, 16, 16, 48, 48]
        if "A" not in state:
            state["A"] = orc.fill_normal(prod(lA), orc.F16, 255, 0.5)
            state["B"] = orc.fill_normal(prod(lB), orc.F16, 256, 0.5)
            state["C"] = orc.fill_uniform(prod(lD), orc.F32, 257)
            state["D"] = np.empty(prod(lD), dtype=np.float32)
            state["smp"] = np.random.default_rng(0).integers(0, prod(lD), 65536)
        t0 = time.perf_counter()
        orc.contraction(2.0, state["A"], lA, packed(lA, False), [m0, k0, m1, k1, m2], orc.F16, state["B"], lB,
                        packed(lB, False), [k1, n0, k0, n1], orc.F16, 0.5, state["C"], state["D"], lD, packed(lD, False),
                        [m0, m1, m2, n0, n1], orc.F32, orc.COMPUTE_32F, sample=state["smp"], nthreads=nthreads)
        return 2 * 65536 * 2304, time.perf_counter() - t0, \
            "oracle on 65536 sampled outputs of the whole problem (151 M multiply-adds, exact k order); the rate is " \
            "extrapolated to the whole problem"


WORKLOADS = {"c1": ContractionC1, "c2": PermutationC2, "c3": ReductionC3, "c3max": ReductionC3Max,
             "c4": ContractionC4, "c5": ContractionC5, "c5f16": ContractionC5F16, "c2f16": PermutationC2F16}
ORDER = ["c4", "c1", "c2", "c3", "c3max", "c5", "c5f16", "c2f16"]


# --------------------------------------------------------------------------------------------- timing
def measure_device(wl, steps, warmup, stream, barrier, world, dist, local_rank, sample_clocks):
    """Median (over repeats) of the slowest rank's device time for exactly `steps` steps, in ms; the launch mode; the
    repeats; this rank's own median; the library's kernel launches per K-step region; the clock record."""
    import torch

    ht = wl.ht
    nsets = len(wl.sets)
    for i in range(max(warmup, 3)):
        wl.step(stream, i % nsets)
    torch.cuda.synchronize()
    l0 = ht.kernel_launch_count()
    wl.step(stream, 0)
    per_step = ht.kernel_launch_count() - l0
    torch.cuda.synchronize()

    # K steps captured once per group of buffer sets, replayed: kernels run back to back, the host is out of the way
    ngraphs = max(1, math.ceil(nsets / steps))
    graphs, mode = [], "cuda-graph"
    try:
        for g in range(ngraphs):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                cs = torch.cuda.current_stream()
                for i in range(steps):
                    wl.step(cs, (g * steps + i) % nsets)
            graphs.append(gr)
    except Exception as e:  # capture refused: enqueue the steps directly
        graphs, mode = [], "direct (graph capture failed: %s)" % str(e).splitlines()[0][:80]
        torch.cuda.synchronize()

    def region(r):
        if graphs:
            graphs[r % ngraphs].replay()
        else:
            for i in range(steps):
                wl.step(stream, (r * steps + i) % nsets)

    def timed(r):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        region(r)
        e.record(stream)
        torch.cuda.synchronize()
        return s.elapsed_time(e)

    timed(0)
    first = timed(1)
    t = torch.tensor([first], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    repeats = int(min(400, max(5, math.ceil(MIN_LOAD_MS / max(float(t.item()), 1e-3)))))
    sampler = ClockSampler(local_rank) if sample_clocks else None
    times = [timed(r) for r in range(repeats)]
    clocks = sampler.stop() if sampler else None
    tt = torch.tensor(times, dtype=torch.float64, device="cuda")
    own = statistics.median(times)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)  # every repeat is bracketed by a barrier: same index, same repeat
    ms = statistics.median(tt.tolist())
    return ms, mode, repeats, own, per_step * steps, clocks


def measure_e2e(wl, steps, stream, barrier, world, dist):
    """End to end through the C ABI: pinned host buffers, H2D of the inputs and D2H of the result of EVERY step
    inside the region. Two buffer sets and three streams let the copy-in of step i+1, the kernel of step i and the
    copy-out of step i-1 overlap (PCIe is full duplex), as an application streaming batches through the library
    would run it."""
    import torch

    n = max(2, min(steps, 8))
    sets = [0, 1 % len(wl.sets)]
    if sets[0] == sets[1]:
        import copy

        b = wl.sets[0]
        twin = copy.copy(b)
        for k, v in b.__dict__.items():
            if v is not None:
                setattr(twin, k, torch.empty_like(v).pin_memory() if k.endswith("_host") else torch.empty_like(v))
        wl.sets.append(twin)
        sets = [0, len(wl.sets) - 1]
    with torch.cuda.stream(stream):
        for s in sets:
            wl.h2d(wl.sets[s])
            wl.step(stream, s)
            wl.d2h(wl.sets[s])
    barrier()
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_cmp, ev_out = [None, None], [None, None]
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(s_in)
    h2d = d2h = 0
    for i in range(n):
        j = i % 2
        b = wl.sets[sets[j]]
        if ev_cmp[j] is not None:
            s_in.wait_event(ev_cmp[j])  # the set's inputs are free once its previous kernel has run
        with torch.cuda.stream(s_in):
            h2d = wl.h2d(b)
        ev_in = torch.cuda.Event()
        ev_in.record(s_in)
        s_cmp.wait_event(ev_in)
        if ev_out[j] is not None:
            s_cmp.wait_event(ev_out[j])  # its result buffer is free once the previous copy-out is done
        wl.step(s_cmp, sets[j])
        ev_cmp[j] = torch.cuda.Event()
        ev_cmp[j].record(s_cmp)
        s_out.wait_event(ev_cmp[j])
        with torch.cuda.stream(s_out):
            d2h = wl.d2h(b)
        ev_out[j] = torch.cuda.Event()
        ev_out[j].record(s_out)
    e.record(s_out)  # the last copy-out ends the region
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), n, int(h2d), int(d2h)


def roofline_of(wl, per_launch_ms, pk, kernel):
    scale = 1e9 if wl.bound == "hbm" else 1e12
    achieved = wl.units_local() / (per_launch_ms / 1e3) / scale
    measured = "of measured (MEASURED_PEAKS.json)" if pk["source"] == "measured" else "of fallback"
    if wl.bound == "hbm":
        peak, punit, src = pk["hbm"], "GB/s", measured + ": copy bandwidth"
    elif wl.name == "c5":
        peak, punit, src = NOMINAL_FP64_TFLOPS, "TFLOP/s", "nominal FP64 tensor pipe (no measured figure)"
    elif wl.name == "c1":
        # fp32 on the tensor cores: TF32 runs at half the bf16 rate and every product takes three MMAs
        peak, punit, src = round(pk["bf16_sustained"] / 6.0, 1), "TFLOP/s", \
            measured + ": bf16 sustained / 2 for TF32 / 3 MMAs per product"
    else:
        # the kernel is timed inside a loop that keeps the GPU under load for 200 ms and more (the power cap, not the
        # burst clock, sets the rate): the sustained cuBLAS figure is the like-for-like denominator
        peak, punit, src = pk["bf16_sustained"], "TFLOP/s", measured + ": cuBLAS bf16 sustained (back-to-back launches)"
    traffic, tsrc = NCU_TRAFFIC.get(wl.name, (None, None))
    if wl.split > 1:
        traffic, tsrc = None, None  # the captures are of the whole single-GPU problem
    r = {"bound": wl.bound, "achieved": round(achieved, 2), "peak": peak, "unit": punit,
         "frac": round(achieved / peak, 4), "traffic": traffic, "traffic_source": tsrc, "peak_source": src,
         "kernel": kernel}
    if wl.name in ("c4", "c5f16"):
        r["frac_of_nominal_2250"] = round(achieved / NOMINAL_BF16_TFLOPS, 4)
        r["frac_of_burst"] = round(achieved / pk["bf16"], 4)
    return r


def cpu_baseline_of(cls, ncores, budget_s=6.0):
    state = {}
    units, dt, sample = cls.cpu_step(ncores, state)
    runs = [(units, dt)]
    t0 = time.perf_counter()
    while time.perf_counter() - t0 + dt < budget_s and len(runs) < 5:
        u, d, _ = cls.cpu_step(ncores, state)
        runs.append((u, d))
    scale = 1e9 if cls.bound == "hbm" else 1e12
    rate = statistics.median(u / d for u, d in runs) / scale
    return {"value": round(rate, 5), "unit": cls.unit, "cores": ncores, "kind": "port",
            "sample": sample + "; %d passes, median" % len(runs)}


def run_workload(cls, ht, h, args, rank, world, local, dist, barrier, pk, weak=False, light=False):
    """One configuration: device-resident throughput, end to end, roofline, CPU baseline. Returns the record (rank 0)
    or None."""
    import torch

    stream = torch.cuda.current_stream()
    wl = cls(ht, h, rank, world, weak=weak)
    wl.setup()
    torch.cuda.synchronize()
    ms, mode, repeats, own_ms, launches, clocks = measure_device(wl, args.steps, args.warmup, stream, barrier, world, dist,
                                                                 local, rank == 0 and not light)
    kernel = ht.last_kernel_name()
    scale = 1e9 if wl.bound == "hbm" else 1e12
    value = wl.units_job() * args.steps / (ms / 1e3) / scale
    rec = {"metric": wl.metric, "value": round(value, 2), "unit": wl.unit, "ms_per_step": round(ms / args.steps, 6)}
    if light:
        wl.release()
        return rec if rank == 0 else None
    e2e_ms, e2e_steps, h2d, d2h = measure_e2e(wl, args.steps, stream, barrier, world, dist)
    e2e_value = wl.units_job() * e2e_steps / (e2e_ms / 1e3) / scale
    nsets = len(wl.sets)
    split = wl.split
    out = None
    if rank == 0:
        rec.update({
            "dtype": wl.dtype, "scaling": "strong" if split > 1 else ("replicas" if world > 1 else "strong"),
            "config": cls.config(world),
            "roofline": roofline_of(wl, own_ms / args.steps, pk, kernel),
            "e2e": {"value": round(e2e_value, 3), "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps,
                    "overlap": "two buffer sets, three streams: copy-in, kernel and copy-out of consecutive steps overlap"},
            "gpu_launches": int(launches), "clocks": clocks,
            "protocol": {"launch": mode, "buffer_sets": nsets, "repeats_of_k_steps": repeats,
                         "statistic": "median over repeats of the slowest rank's CUDA-event time for K steps"},
        })
        if clocks and clocks.get("sm_mhz"):
            rec["sm_cycles_per_step"] = round(ms / args.steps * 1e-3 * clocks["sm_mhz"] * 1e6)
        out = rec
    wl.release()
    return out


def run_c3k(ht, h, args, rank, world, local, dist, barrier):
    """Configuration 3 with the REDUCED mode k split over the ranks: every rank reduces its share of k (alpha 1,
    beta 0), one NCCL all-reduce of the 1 MiB of partial results, htReductionFinish applies alpha and beta*C.
    ADD and MAX; the all-reduce's own time is reported; rank 0 checks the result against the CPU oracle."""
    import numpy as np
    import torch

    from hiptensor_b200 import sharding as sh

    lens = [4096, 64, 64, 32]
    sA = packed(lens, False)
    lD, sD = lens[:2], packed(lens[:2], False)
    A_host = _fill(prod(lens), 0, 17)
    C_host = _fill(lD[0] * lD[1], 0, 19)
    A, C = A_host.cuda(), C_host.cuda()
    va, vd, exch = sh.shard_reduction(lens, sA, [0, 1, 2, 3], lD, sD, [0, 1], 2, rank, world)
    dA = h.tensor_descriptor(va.lens, va.strides, ht.R_32F)
    dD = h.tensor_descriptor(lD, sD, ht.R_32F)
    stream = torch.cuda.current_stream()
    res = {}
    for opname, op, dop in (("add", ht.OP_ADD, dist.ReduceOp.SUM), ("max", ht.OP_MAX, dist.ReduceOp.MAX)):
        P = torch.zeros(lD[0] * lD[1], device="cuda")
        D = torch.zeros_like(P)

        def once(timing):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record(stream)
            h.reduction(1.0, A[va.offset:], dA, [0, 1, 2, 3], 0.0, P, dD, [0, 1], P, dD, [0, 1], op, ht.COMPUTE_32F,
                        None, 0, stream)
            ev[1].record(stream)
            dist.all_reduce(P, op=dop)
            ev[2].record(stream)
            h.reduction_finish(1.0, P, 0.5, C, D, dD, ht.COMPUTE_32F, stream)
            ev[3].record(stream)
            torch.cuda.synchronize()
            return [ev[i].elapsed_time(ev[i + 1]) for i in range(3)] + [ev[0].elapsed_time(ev[3])]

        for _ in range(max(args.warmup, 3)):
            once(False)
        rows = []
        for _ in range(args.steps):
            barrier()
            rows.append(once(True))
        t = torch.tensor(rows, dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        med = [statistics.median(col) for col in zip(*t.tolist())]
        whole = prod(lens) * 4 + 2 * lD[0] * lD[1] * 4
        ok = None
        if rank == 0:
            from oracle import binding as orc

            exp = np.zeros(lD[0] * lD[1], dtype=np.float32)
            orc.reduction(1.0, A_host.numpy(), lens, sA, [0, 1, 2, 3], orc.F32, 0.5, C_host.numpy(), exp, lD, sD, [0, 1],
                          orc.F32, orc.OP_ADD if opname == "add" else orc.OP_MAX, orc.COMPUTE_32F, nthreads=0)
            got = D.cpu().numpy().astype(np.float64)
            err = float(np.max(np.abs(got - exp) / (np.abs(got) + np.abs(exp) + 1.0)))
            ok = bool(err < 2048 * float(np.finfo(np.float32).eps))
            res[opname] = {"value": round(whole / (med[3] / 1e3) / 1e9, 2), "unit": "GB/s",
                           "ms_per_step": round(med[3], 5), "ms_partial_reduction": round(med[0], 5),
                           "ms_all_reduce": round(med[1], 5), "ms_finish": round(med[2], 5),
                           "all_reduce_bytes": lD[0] * lD[1] * 4, "matches_oracle": ok, "max_rel_error": err}
    del A, C
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {"metric": "reduction_hbm_gbs", "unit": "GB/s", "scaling": "strong",
            "config": {"workload": "c3k: configuration 3 with the reduced mode k split over %d ranks (k = %d each): "
                                   "partial reduction, one NCCL all-reduce of 1 MiB, htReductionFinish" % (world, 64 // world),
                       "parallelism": "reduced mode k split, one all-reduce"},
            "add": res["add"], "max": res["max"], "steps": args.steps,
            "statistic": "median over steps of the slowest rank's CUDA-event times"}


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
    pk = peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    names = [n for n in ORDER if (not args.only or n in args.only)]
    recs = {}
    ncores = os.cpu_count() or 1
    if args.slab_of > 1 and world == 1:
        # one GPU plays rank 0 of an N-way split: device-resident timing of the slab kernels only
        for name in names:
            cls = WORKLOADS[name]
            if not cls.sharded:
                continue
            wl = cls(ht, h, 0, args.slab_of)
            wl.setup()
            ms, mode, repeats, own, launches, clocks = measure_device(wl, args.steps, args.warmup,
                                                                      torch.cuda.current_stream(), barrier, 1, dist, local, True)
            scale = 1e9 if wl.bound == "hbm" else 1e12
            recs[name] = {"slab_of": args.slab_of, "ms_per_step": round(ms / args.steps, 6),
                          "value_of_this_gpu": round(wl.units_local() * args.steps / (ms / 1e3) / scale, 2), "unit": wl.unit,
                          "kernel": ht.last_kernel_name(), "clocks": clocks, "config": cls.config(args.slab_of)}
            wl.release()
        print(json.dumps({"slab_of": args.slab_of, "n_gpus": 1, "steps": args.steps, "configs": recs}), flush=True)
        return
    for name in names:
        cls = WORKLOADS[name]
        rec = run_workload(cls, ht, h, args, rank, world, local, dist, barrier, pk)
        if world > 1 and cls.sharded:
            weak = run_workload(cls, ht, h, args, rank, world, local, dist, barrier, pk, weak=True, light=True)
            if rank == 0:
                rec["weak_value"] = weak["value"]
                rec["weak_ms_per_step"] = weak["ms_per_step"]
        if rank == 0:
            # the CPU baseline is measured at N = 1 only (rank 0's host cores are shared with the other ranks otherwise)
            rec["cpu_baseline"] = cpu_baseline_of(cls, ncores) if world == 1 else None
            recs[name] = rec
    if world > 1 and (not args.only or "c3k" in args.only):
        r = run_c3k(ht, h, args, rank, world, local, dist, barrier)
        if rank == 0:
            recs["c3k"] = r
    if rank == 0:
        head = "c4" if "c4" in recs else names[0]
        top = recs.pop(head)
        line = {"metric": top["metric"], "value": top["value"], "unit": top["unit"], "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": top["ms_per_step"],
                "higher_is_better": True, "scaling": top["scaling"] if world > 1 else "strong", "vs_baseline": None,
                "dtype": top["dtype"], "data": "synthetic"}
        for k in ("config", "roofline", "cpu_baseline", "e2e", "gpu_launches", "clocks", "protocol",
                  "sm_cycles_per_step", "weak_value", "weak_ms_per_step"):
            if k in top:
                line[k] = top[k]
        line["configs"] = recs
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU algorithm for every configuration, timed on the host cores (rank 0 only). One step is one
    oracle pass over the whole of c1, c2, c3 and over a fixed sample of the outputs of c4 and c5."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from oracle import binding as orc
    orc.build()
    ncores = os.cpu_count() or 1
    names = [n for n in ORDER if (not args.only or n in args.only)]
    recs = {}
    for name in names:
        cls = WORKLOADS[name]
        state = {}
        sample = ""
        for _ in range(args.warmup):
            cls.cpu_step(ncores, state)
        runs = []
        for _ in range(args.steps):
            u, d, sample = cls.cpu_step(ncores, state)
            runs.append((u, d))
        scale = 1e9 if cls.bound == "hbm" else 1e12
        value = sum(u for u, _ in runs) / sum(d for _, d in runs) / scale
        recs[name] = {
            "metric": cls.metric, "value": round(value, 5), "unit": cls.unit,
            "ms_per_step": round(sum(d for _, d in runs) / len(runs) * 1e3, 3), "dtype": cls.dtype,
            "config": cls.config(world),
            "cpu_baseline": {"value": round(value, 5), "unit": cls.unit, "cores": ncores, "kind": "port",
                             "sample": "CPU restatement of hipTensor's own CPU reference (the reference needs hipcc + "
                                       "Composable Kernel and cannot be built here); each step: " + sample},
            "e2e": {"value": round(value, 5), "unit": cls.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
    head = "c4" if "c4" in recs else names[0]
    top = recs.pop(head)
    line = {"impl": "reference", "metric": top["metric"], "value": top["value"], "unit": top["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": top["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": top["dtype"], "data": "synthetic",
            "config": top["config"], "cpu_baseline": top["cpu_baseline"], "e2e": top["e2e"], "gpu_launches": 0,
            "configs": recs}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--only", default="", help="comma-separated subset of c4,c1,c2,c3,c3max,c5,c5f16,c2f16,c3k")
    ap.add_argument("--slab-of", type=int, default=0,
                    help="single GPU only: run rank 0's share of an N-way split of the sharded configurations (the "
                         "kernels and sizes one GPU of N sees), for profiling")
    ap.add_argument("--min-load-ms", type=float, default=MIN_LOAD_MS,
                    help="device time over which the K-step region is repeated (profiling runs pass a small value)")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    args = ap.parse_args()
    args.only = [x for x in args.only.split(",") if x]
    globals()["MIN_LOAD_MS"] = args.min_load_ms
    args.steps = max(args.steps, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_gpu(args)


if __name__ == "__main__":
    main()
