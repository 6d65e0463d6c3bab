"""Slab arithmetic for running the three operations on several GPUs, one process per GPU.

The reference has no multi-device support (a handle is bound to one device,
library/src/contraction/hiptensor_contraction.cpp:263-277); the partitioning below follows the
problem structure: every operation splits along one *kept* (free) mode into independent slabs,
with no exchange between ranks. Only a reduction whose *reduced* mode is split needs one
all-reduce of the small partial results, after which alpha and beta*C are applied once.

All functions are pure host arithmetic on extents/strides (elements, not bytes).
"""
from dataclasses import dataclass
from typing import List, Optional, Sequence


@dataclass
class Slab:
    start: int  # first index of the sharded mode owned by this rank
    count: int  # number of indices owned (0 if the rank has no work)


def slab(extent: int, rank: int, world: int) -> Slab:
    """Balanced contiguous split of range(extent): the first extent % world ranks get one more."""
    base, rem = divmod(extent, world)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return Slab(start, count)


def packed_strides(lens: Sequence[int], first_fastest: bool) -> List[int]:
    n = len(lens)
    s = [1] * n
    if first_fastest:
        for i in range(1, n):
            s[i] = s[i - 1] * lens[i - 1]
    else:
        for i in range(n - 2, -1, -1):
            s[i] = s[i + 1] * lens[i + 1]
    return s


@dataclass
class TensorShard:
    lens: List[int]  # local extents (sharded mode shortened)
    strides: List[int]  # strides of the GLOBAL tensor (the slab is a strided view of it)
    offset: int  # element offset of the slab's origin in the global tensor


def shard_tensor(lens: Sequence[int], strides: Sequence[int], modes: Sequence[int], mode: int, s: Slab) -> TensorShard:
    """The slab of a strided tensor along `mode` (a tensor that lacks the mode is replicated)."""
    lens, strides = list(lens), list(strides)
    if mode not in modes:
        return TensorShard(lens, strides, 0)
    i = list(modes).index(mode)
    local = list(lens)
    local[i] = s.count
    return TensorShard(local, strides, s.start * strides[i])


def shard_contraction(lensA, stridesA, modeA, lensB, stridesB, modeB, lensD, stridesD, modeD, mode, rank, world):
    """Split along a free mode (one that appears in D and in exactly one of A, B). Returns the
    per-rank views of A, B and D (C shares D's view); the contracted modes are untouched."""
    in_a, in_b = mode in modeA, mode in modeB
    if mode not in modeD or in_a == in_b:
        raise ValueError("contractions shard along a free mode of A or of B")
    extent = lensD[list(modeD).index(mode)]
    s = slab(extent, rank, world)
    return (shard_tensor(lensA, stridesA, modeA, mode, s), shard_tensor(lensB, stridesB, modeB, mode, s),
            shard_tensor(lensD, stridesD, modeD, mode, s))


def shard_reduction(lensA, stridesA, modeA, lensD, stridesD, modeD, mode, rank, world):
    """Split along `mode` of A. A kept mode gives independent slabs of D; a reduced mode gives every
    rank a partial result for the whole of D (combine with reduce_partials). Returns
    (view of A, view of D, needs_exchange)."""
    if mode not in modeA:
        raise ValueError("the sharded mode must be a mode of A")
    s = slab(lensA[list(modeA).index(mode)], rank, world)
    kept = [m for m in modeA if m in modeD]  # D's extents follow A's order (positional contract)
    return (shard_tensor(lensA, stridesA, modeA, mode, s), shard_tensor(lensD, stridesD, kept, mode, s),
            mode not in modeD)


def shard_permutation(lensA, modeA, modeB, mode, rank, world):
    """Permutation tensors are packed with the first mode fastest on both sides
    (library/src/permutation/permutation_solution_impl.hpp:125-128), so each rank runs a self-contained
    permutation on local packed buffers. Returns (local extents of A, gather/scatter description):
    the local A is the slab A[..., mode in slab, ...] and the local B the slab of B along the same mode;
    `a_view` / `b_view` are those slabs as strided views of the global packed tensors."""
    s = slab(lensA[list(modeA).index(mode)], rank, world)
    lensB = [lensA[list(modeA).index(m)] for m in modeB]
    a_view = shard_tensor(lensA, packed_strides(lensA, True), modeA, mode, s)
    b_view = shard_tensor(lensB, packed_strides(lensB, True), modeB, mode, s)
    return a_view, b_view


_REDUCE_OPS = {3: "SUM", 5: "PRODUCT", 6: "MAX", 7: "MIN"}


def reduce_partials(partial, op: int, alpha: float, beta: float, C, handle=None, D=None, descD=None,
                    type_compute=None, group=None, stream=None, finish=None):
    """Finish a reduction whose reduced mode was sharded: one all-reduce of the partial results
    (torch tensor laid out like D, raw reduce values computed with alpha=1, beta=0) with the reduction's
    operator, then alpha*r + beta*C applied ONCE by the library's own kernel (htReductionFinish, through
    `handle`, into D or in place when D is None) on `stream`.

    `finish`, when given, is called with the combined partial results instead of the library: ranks without
    a GPU (host-logic tests on gloo) have no device to run the kernel on and bring their own arithmetic.
    There is no built-in CPU path."""
    import torch.distributed as dist

    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=getattr(dist.ReduceOp, _REDUCE_OPS[op]), group=group)
    if finish is not None:
        return finish(partial)
    if handle is None or descD is None or type_compute is None:
        raise RuntimeError("reduce_partials needs a hiptensor_b200.Handle, D's descriptor and the compute type: "
                           "alpha and beta*C are applied by the library's CUDA kernel, there is no CPU path")
    out = partial if D is None else D
    handle.reduction_finish(alpha, partial, beta, C, out, descD, type_compute, stream)
    return out
