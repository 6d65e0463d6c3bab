"""CPU-only tests of the host-side planner (mode classification, stride folding, kernel choice)
through the introspection entry points of the C ABI."""
import re

import pytest


@pytest.fixture(scope="module")
def ht():
    from hiptensor_b200 import build

    build.build()
    import hiptensor_b200

    return hiptensor_b200


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


def test_permutation_config2_uses_tma(ht):
    d = ht.describe_permutation_plan([128] * 4, [0, 1, 2, 3], [3, 2, 1, 0])
    assert "kind=tma" in d and "ndim=4" in d and "q=3" in d


def test_permutation_folding(ht):
    # B[a,b,d,c] = A[a,b,c,d]: a and b fold, inner mode shared -> row copy
    d = ht.describe_permutation_plan([8, 4, 6, 10], [0, 1, 2, 3], [0, 1, 3, 2])
    assert "kind=copy" in d and "dims=32:1/1 6:32/320 10:192/32" in d
    # identity folds to one mode
    d = ht.describe_permutation_plan([8, 4, 6, 10], [0, 1, 2, 3], [0, 1, 2, 3])
    assert "ndim=1" in d and "dims=1920:1/1" in d
    # golden-vector case: c and n fold
    d = ht.describe_permutation_plan([3, 2, 4, 5], [ord(c) for c in "whcn"], [ord(c) for c in "cnhw"])
    assert "kind=tile" in d and "dims=3:1/40 2:3/20 20:6/1" in d
    # extent-1 modes vanish
    d = ht.describe_permutation_plan([1, 6, 1, 70], [0, 1, 2, 3], [3, 2, 1, 0])
    assert "ndim=2" in d


def test_permutation_short_contiguous_modes_stay_on_tma(ht):
    """A contiguous mode shorter than 64 bytes keeps the TMA kernel when the mode after it in the same tensor makes one
    contiguous run with it (the slab of an output mode split over 8 GPUs, and the way back); it must still be a
    multiple of 16 bytes."""
    assert "kind=tma" in ht.describe_permutation_plan([128, 128, 128, 16], [0, 1, 2, 3], [3, 2, 1, 0])
    assert "kind=tma" in ht.describe_permutation_plan([128, 128, 128, 16], [0, 1, 2, 3], [3, 2, 1, 0], ht.R_16F, ht.R_16F)
    assert "kind=tma" in ht.describe_permutation_plan([16, 128, 128, 128], [0, 1, 2, 3], [3, 2, 1, 0])
    assert "kind=tma" in ht.describe_permutation_plan([128, 24, 40, 4], [0, 1, 2, 3], [3, 2, 1, 0])
    assert "kind=tile" in ht.describe_permutation_plan([128, 128, 12], [0, 1, 2], [2, 1, 0])  # 12: not a power of two
    assert "kind=tile" in ht.describe_permutation_plan([128, 128, 128, 4], [0, 1, 2, 3], [3, 2, 1, 0], ht.R_16F, ht.R_16F)


def test_permutation_rejects(ht):
    with pytest.raises(ht.HiptensorError) as e:
        ht.describe_permutation_plan([4, 4], [0, 1], [0, 2])
    assert e.value.status == ht.STATUS_INVALID_VALUE
    with pytest.raises(ht.HiptensorError) as e:
        ht.describe_permutation_plan([4, 4], [0, 1], [1, 0], ht.R_64F)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED
    with pytest.raises(ht.HiptensorError) as e:
        ht.describe_permutation_plan([4, 4], [0, 1], [1, 0], ht.R_32F, ht.R_16F)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED


def test_reduction_config3_layouts(ht):
    lens = [4096, 64, 64, 32]
    d = ht.describe_reduction_plan(lens, packed(lens, False), [0, 1, 2, 3], lens[:2], packed(lens[:2], False), [0, 1])
    assert "kind=row" in d and "vec=4" in d and "nOut=262144" in d and "red=[2048:1]" in d
    d = ht.describe_reduction_plan(lens, packed(lens, True), [0, 1, 2, 3], lens[:2], packed(lens[:2], True), [0, 1])
    assert "kind=col" in d and "keep=[262144:1/1]" in d and "red=[2048:262144]" in d


def test_reduction_short_rows_and_short_kept_runs(ht):
    """Lanes per output follow the length of the contiguous reduced row; few outputs get optional slices; a kept
    contiguous mode decides the column kernel's block shape."""
    def plan(lens, kept, dtype=None):
        lD = [lens[i] for i in kept]
        return ht.describe_reduction_plan(lens, packed(lens, False), list(range(len(lens))), lD, packed(lD, False), kept,
                                          dtype if dtype is not None else ht.R_32F)

    # rows of 4, 24 and 64 floats: 1, 8 and 16 lanes of 16-byte loads; 130 floats: 8-byte loads, eight per lane
    assert "short=1x4" in plan([4096, 128, 4], [0, 1])
    assert "short=8x4" in plan([4096, 128, 24], [0, 1])
    assert "short=16x4" in plan([4096, 128, 64], [0, 1])
    assert "short=16x2" in plan([4096, 128, 130], [0, 1])
    # 1 KiB rows of full vectors: the row kernel alone, the short-row kernel under a further reduced mode
    assert "short=" not in plan([4096, 128, 256], [0, 1])
    assert "short=8x4" in plan([64, 4096, 256], [1])
    # configuration 3 keeps its plan
    d = plan([4096, 64, 64, 32], [0, 1])
    assert "kind=row" in d and "short=" not in d and "split=1 " in d
    # few outputs under a long outer mode: slices that a caller without scratch may drop
    d = plan([3000, 24, 4], [1])
    assert "short=1x4" in d and "optional-split" in d and int(re.search(r"split=(\d+)", d).group(1)) > 16
    # kept contiguous mode: many outputs and a short reduction take all lanes on outputs and no exchange
    assert "col=256x1 vec=4" in plan([8, 4096, 8192], [1, 2])
    # a kept run of 32 floats followed by the rows of the reduced mode: lanes along those rows
    d = plan([4096, 64, 64, 32], [3])
    assert "col=8x32 vec=4" in d and int(re.search(r"split=(\d+)", d).group(1)) > 16
    # a kept run below a sector: lanes over the flattened outputs
    assert "col=256x1 vec=1" in plan([4096, 128, 128, 4], [1, 3], ht.R_16F)


def test_reduction_split_and_errors(ht):
    lens = [3, 512, 1024]
    d = ht.describe_reduction_plan(lens, packed(lens, False), [0, 1, 2], [3], [1], [0])
    assert "kind=row" in d and int(re.search(r"split=(\d+)", d).group(1)) > 1
    d = ht.describe_reduction_plan(lens, packed(lens, False), [0, 1, 2], [], [], [])
    assert "nOut=1" in d and "nRed=1572864" in d
    with pytest.raises(ht.HiptensorError) as e:  # extent of D does not match the kept mode of A
        ht.describe_reduction_plan(lens, packed(lens, False), [0, 1, 2], [4], [1], [0])
    assert e.value.status == ht.STATUS_INVALID_VALUE
    with pytest.raises(ht.HiptensorError) as e:  # mode of D missing from A
        ht.describe_reduction_plan(lens, packed(lens, False), [0, 1, 2], [3], [1], [9])
    assert e.value.status == ht.STATUS_NOT_SUPPORTED


def test_contraction_config1(ht):
    e = 24
    s = packed([e] * 4, True)
    d = ht.describe_contraction_plan([e] * 4, s, [0, 1, 4, 5], ht.R_32F, [e] * 4, s, [2, 3, 4, 5], ht.R_32F, [e] * 4, s,
                                     [0, 1, 2, 3], ht.R_32F, True, ht.COMPUTE_32F)
    # D is contiguous along m0: operands are exchanged so that the kernel sees it along N
    assert "M=576 N=576 K=576" in d and "swapped=1" in d and "n[576:1/1]" in d and "k[576:576/576]" in d
    # fp32 with 16-byte aligned strides: tensor-core path, both operands taken MN-major in 32-row chunks
    assert "kind=tf32x3" in d and "major=mn/mn" in d and "boxK=[32 1]" in d


def test_contraction_fp32_tensor_core_layouts(ht):
    """The four K-/MN-major operand layouts of plain matrices, a two-mode K box, and the cases that stay on the
    FMA kernel (strides that are not multiples of 16 bytes, tiles smaller than 128 x 64)."""
    f = ht.R_32F

    def plan(lA, mA, lB, mB, lD, mD, compute=None):
        return ht.describe_contraction_plan(lA, packed(lA, False), mA, f, lB, packed(lB, False), mB, f, lD,
                                            packed(lD, False), mD, f, True, compute or ht.COMPUTE_32F)

    M, N, K = 384, 1000, 136
    assert "kind=tf32x3" in plan([M, K], [0, 2], [N, K], [1, 2], [M, N], [0, 1]) and "major=k/k" in plan(
        [M, K], [0, 2], [N, K], [1, 2], [M, N], [0, 1])
    assert "major=mn/mn" in plan([K, M], [2, 0], [K, N], [2, 1], [M, N], [0, 1])
    assert "major=k/mn" in plan([M, K], [0, 2], [K, N], [2, 1], [M, N], [0, 1])
    assert "major=mn/k" in plan([K, M], [2, 0], [N, K], [1, 2], [M, N], [0, 1])
    # two K modes that do not fold: 16 x 2 box
    d = plan([6, 5, 16, 40], [5, 1, 4, 0], [6, 3, 16, 72], [5, 3, 4, 2], [5, 3, 40, 72], [1, 3, 0, 2])
    assert "kind=tf32x3" in d and "boxK=[16 2]" in d and "M=200 N=216 K=96" in d
    # not eligible
    assert "kind=tiled_simt" in plan([130, 34], [0, 2], [70, 34], [1, 2], [130, 70], [0, 1])
    assert "kind=tiled_simt" in plan([64, 64], [0, 2], [64, 64], [1, 2], [64, 64], [0, 1])
    # f16 / bf16 compute on fp32 data: the same kernel with rounding instead of the split
    assert "kind=tf32x3" in plan([M, K], [0, 2], [N, K], [1, 2], [M, N], [0, 1], ht.COMPUTE_16F)
    assert "kind=tf32x3" in plan([K, M], [2, 0], [K, N], [2, 1], [M, N], [0, 1], ht.COMPUTE_16BF)


def test_contraction_packed_operands(ht):
    """Operands TMA cannot describe: large problems are planned on packed copies (contracted modes merged, rows padded
    to 16 bytes, free modes in D's order); small ones and f64 keep the gathered kernels."""
    def plan(e, modeA, modeB, modeD, t=None, tD=None):
        t = ht.R_16F if t is None else t
        tD = ht.R_32F if tD is None else tD
        s = packed([e] * 4, False)
        return ht.describe_contraction_plan([e] * 4, s, modeA, t, [e] * 4, s, modeB, t, [e] * 4, s, modeD, tD, False,
                                            ht.COMPUTE_64F if t == ht.R_64F else ht.COMPUTE_32F)

    # extents of 50 halves: strides of 100 bytes; K = 2500 padded to 2504
    d = plan(50, [0, 1, 4, 5], [2, 3, 4, 5], [0, 1, 2, 3])
    assert "kind=tcgen05" in d and "packed K=2500 Kp=2504" in d and "M=2500 N=2500 K=2504" in d
    assert "copies=%d" % (2 * ((2500 * 2504 * 2 + 255) // 256 * 256) + 256) in d
    # contracted modes interleaved with free ones, in different orders in A and B
    d = plan(48, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3])
    assert "kind=tcgen05" in d and "packed K=2304 Kp=2304" in d
    d = plan(48, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3], ht.R_32F)
    assert "kind=tf32x3" in d and "packed K=2304 Kp=2304" in d
    # below about a GFLOP the copies do not pay; f64 gathers in place on the FP64 tensor pipe
    assert "kind=tiled_simt" in plan(20, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3]) and "packed" not in plan(20, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3])
    d = plan(48, [0, 4, 1, 5], [5, 2, 4, 3], [0, 1, 2, 3], ht.R_64F, ht.R_64F)
    assert "kind=tiled_dmma" in d and "packed" not in d
    # what the tensor-core kernels read in place is not copied
    assert "packed" not in plan(64, [0, 1, 4, 5], [2, 3, 4, 5], [0, 1, 2, 3])
    # ... unless it is read in mostly empty chunks: configuration 5's layout with f16 data (chunks of 16 and 48 of 64,
    # K blocks of 48 of 64: 0.14 of the MMA work useful); with m2 = n1 = k = 64 every chunk is full
    m0, m1, m2, n0, n1, k0, k1 = range(7)

    def c5(ext):
        mA, mB, mD = [m0, k0, m1, k1, m2], [k1, n0, k0, n1], [m0, m1, m2, n0, n1]
        lA, lB, lD = ([ext[m] for m in ms] for ms in (mA, mB, mD))
        return ht.describe_contraction_plan(lA, packed(lA, False), mA, ht.R_16F, lB, packed(lB, False), mB, ht.R_16F, lD,
                                            packed(lD, False), mD, ht.R_32F, True, ht.COMPUTE_32F)

    d = c5({m0: 16, m1: 16, m2: 16, n0: 48, n1: 48, k0: 48, k1: 48})
    assert "kind=tcgen05" in d and "packed K=2304 Kp=2304" in d and "major=k/k" in d
    d = c5({m0: 8, m1: 8, m2: 64, n0: 32, n1: 64, k0: 32, k1: 64})
    assert "kind=tcgen05" in d and "packed" not in d and "major=mn/mn" in d


def test_contraction_ragged_tiles_and_short_k(ht):
    """Outside M >= 128, N >= 64, K >= one K block: small outputs under a long contraction take a ragged tensor-core
    tile, short contractions under a large output too; the rest stays on the FMA kernel."""
    def plan(M, N, K, t):
        return ht.describe_contraction_plan([M, K], [K, 1], [0, 2], t, [N, K], [K, 1], [1, 2], t, [M, N], [N, 1], [0, 1],
                                            ht.R_32F, False, ht.COMPUTE_32F)

    assert "kind=tcgen05" in plan(64, 64, 65536, ht.R_16F) and "kind=tf32x3" in plan(64, 64, 65536, ht.R_32F)
    assert "kind=tcgen05" in plan(16, 256, 1024, ht.R_16F)
    assert "kind=tiled_simt" in plan(64, 64, 1016, ht.R_16F)  # K below 1024
    assert "kind=tiled_simt" in plan(8, 64, 65536, ht.R_16F)  # M below 16
    # the last row mode may be shorter than the tile whatever its extent: the box reaches past the tensor
    d = plan(100, 30, 8192, ht.R_16F)
    assert "kind=tcgen05" in d and "rows=128/64" in d
    # K = 8 under 8192 x 8192 outputs; not under 1024 x 1024
    assert "kind=tcgen05" in plan(8192, 8192, 8, ht.R_16F) and "kind=tf32x3" in plan(8192, 8192, 8, ht.R_32F)
    assert "kind=tiled_simt" in plan(1024, 1024, 8, ht.R_16F)


def test_contraction_k_split_plans(ht):
    """Few tiles and a long K: the fp32 tensor-core plan cuts K into up to four ranges (at least four K blocks
    each, never more CTAs than SMs), one CTA of a cluster each; the sums meet in shared memory, so no workspace is
    asked for. Many tiles or a short K do not split."""
    import re

    def plan(M, N, K, t):
        return ht.describe_contraction_plan([M, K], [K, 1], [0, 2], t, [N, K], [K, 1], [1, 2], t, [M, N], [N, 1],
                                            [0, 1], t, True, ht.COMPUTE_32F)

    d = plan(256, 192, 1024, ht.R_32F)  # 2 x 3 tiles of 128 x 64, 32 K blocks
    m = re.search(r"splitK=(\d+) workspace=(\d+)", d)
    assert "kind=tf32x3" in d and m, d
    assert int(m.group(1)) == 4 and int(m.group(2)) == 0
    d = plan(576, 576, 576, ht.R_32F)  # 5 x 9 tiles of 128 x 64: three ranges fit the SM count
    m = re.search(r"splitK=(\d+)", d)
    assert m and int(m.group(1)) == 3, d
    assert "splitK" not in plan(256, 192, 96, ht.R_32F)  # too few K blocks
    assert "splitK" not in plan(4096, 4096, 1024, ht.R_32F)  # enough tiles for every SM
    assert "splitK" not in plan(256, 256, 4096, ht.R_16F)


def test_contraction_pair_kernel_variants(ht):
    """f16 problems on the CTA-pair kernel: tile width and K split by measured rules. The slabs of an N-way split
    of a 4096^3 problem (M = 4096 / N): 256 x 512 tiles from one and a half rounds of 256 x 256 tiles on,
    256 x 256 tiles for one round, 256 x 256 tiles with every tile's K range cut over two pairs when the tiles fill
    at most half of the pairs; small problems stay on single CTAs."""
    def plan(M, N, K):
        return ht.describe_contraction_plan([M, K], [K, 1], [0, 2], ht.R_16F, [N, K], [K, 1], [1, 2], ht.R_16F, [M, N],
                                            [N, 1], [0, 1], ht.R_32F, False, ht.COMPUTE_32F)

    d = plan(4096, 4096, 4096)
    assert "pair 256x512" in d and "ksplit" not in d, d
    d = plan(2048, 4096, 4096)
    assert "pair 256x512" in d and "ksplit" not in d, d
    d = plan(1024, 4096, 4096)
    assert "pair 256x256" in d and "ksplit" not in d, d
    d = plan(512, 4096, 4096)
    assert "pair 256x256 ksplit=2" in d, d
    assert "pair" not in plan(512, 512, 4096)  # four tiles: single CTAs with their own cluster K split
    assert "ksplit" not in plan(1024, 4096, 512)  # a short K is not worth the exchange
    # no contraction asks for workspace
    assert "workspace" not in d


def test_contraction_config4(ht):
    e = 64
    s = packed([e] * 4, False)
    d = ht.describe_contraction_plan([e] * 4, s, [0, 1, 4, 5], ht.R_16F, [e] * 4, s, [2, 3, 4, 5], ht.R_16F, [e] * 4, s,
                                     [0, 1, 2, 3], ht.R_32F, False, ht.COMPUTE_32F)
    assert "kind=tcgen05" in d and "M=4096 N=4096 K=4096" in d and "k[4096:1/1]" in d and "swapped=0" in d
    assert "major=k/k" in d and "pair" in d
    # the same extents with the first mode fastest: both operands contiguous along M/N, still the tensor-core path
    s = packed([e] * 4, True)
    d = ht.describe_contraction_plan([e] * 4, s, [0, 1, 4, 5], ht.R_16F, [e] * 4, s, [2, 3, 4, 5], ht.R_16F, [e] * 4, s,
                                     [0, 1, 2, 3], ht.R_32F, False, ht.COMPUTE_32F)
    assert "kind=tcgen05" in d and "major=mn/mn" in d and "swapped=1" in d and "pair" in d


def test_contraction_f16_tile_choice_by_size(ht):
    """Small problems take narrow tiles on single CTAs (more CTAs, shorter epilogues); CTA pairs with 256 x 256
    tiles are kept for problems whose tiles occupy most of the pairs."""
    def plan(M, N, K):
        return ht.describe_contraction_plan([M, K], [K, 1], [0, 2], ht.R_16F, [N, K], [K, 1], [1, 2], ht.R_16F, [M, N],
                                            [N, 1], [0, 1], ht.R_32F, False, ht.COMPUTE_32F)

    d = plan(512, 512, 512)
    assert "tile=128x64x64" in d and " pair" not in d, d
    d = plan(2048, 2048, 2048)
    assert "tile=128x256x64" in d and " pair " in d, d  # 64 tiles of 256 x 256: CTA pairs
    d = plan(1280, 1280, 4096)
    assert " pair " in d and "ksplit=2" in d, d  # 25 tiles of 256 x 256 and a long K: pairs with the K cut
    d = plan(1536, 1536, 4096)
    assert " pair " in d and "ksplit" not in d, d  # 36 tiles: plain pairs (an under-filled wave runs in half tiles)
    d = plan(768, 768, 512)
    assert " pair" not in d, d  # nine tiles, short K: single CTAs
    assert " pair 256x512" in plan(4096, 4096, 4096)
    # measured mid-size rules: from a quarter of the SMs' worth of 256 x 256 tiles on, CTA pairs; below that, pairs with
    # the K range of every tile cut in two from K = 2048 on; short K on few tiles stays with single CTAs
    assert " pair " in plan(2048, 1536, 1024) and "ksplit" not in plan(2048, 1536, 1024)  # 48 tiles
    assert " pair " in plan(1536, 1536, 512) and "ksplit" not in plan(1536, 1536, 512)  # 36 tiles, short K
    assert "ksplit=2" in plan(1024, 1024, 2048)  # 16 tiles
    assert "ksplit=2" in plan(1024, 768, 4096)  # 12 tiles
    d = plan(1024, 1024, 1024)
    assert " pair " in d and "ksplit" not in d, d  # 16 tiles, K too short for the exchange: pairs (in half tiles)
    assert " pair" not in plan(1024, 1024, 512)  # 16 tiles and a short K: single CTAs
    assert " pair" not in plan(512, 1024, 4096)  # 8 tiles: single CTAs with their own cluster K split


def test_contraction_config5(ht):
    lA, lB, lD = [16, 48, 16, 48, 16], [48, 48, 48, 48], [16, 16, 16, 48, 48]
    m0, m1, m2, n0, n1, k0, k1 = range(7)
    d = ht.describe_contraction_plan(lA, packed(lA, False), [m0, k0, m1, k1, m2], ht.R_64F, lB, packed(lB, False),
                                     [k1, n0, k0, n1], ht.R_64F, lD, packed(lD, False), [m0, m1, m2, n0, n1],
                                     ht.R_64F, True, ht.COMPUTE_64F)
    assert "kind=tiled_dmma" in d and "M=4096 N=2304 K=2304" in d
    assert "m[16:1/2304 16:768/36864 16:589824/589824]" in d and "k[48:16/110592 48:12288/48]" in d


def test_contraction_errors(ht):
    s = [4, 1]
    args = dict(lensA=[4, 4], stridesA=s, modeA=[0, 1], dtypeA=ht.R_32F, lensB=[4, 4], stridesB=s, modeB=[2, 1],
                dtypeB=ht.R_32F, lensD=[4, 4], stridesD=s, modeD=[0, 2], dtypeD=ht.R_32F, has_c=True,
                type_compute=ht.COMPUTE_32F)
    assert "M=4 N=4 K=4" in ht.describe_contraction_plan(**args)
    bad = dict(args, modeD=[0, 3])
    with pytest.raises(ht.HiptensorError) as e:
        ht.describe_contraction_plan(**bad)
    assert e.value.status == ht.STATUS_INVALID_VALUE
    bad = dict(args, modeB=[2, 0], modeD=[0, 2])  # mode 0 in A, B and D: batch mode
    with pytest.raises(ht.HiptensorError) as e:
        ht.describe_contraction_plan(**bad)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED
    bad = dict(args, lensB=[4, 5])  # contracted extents differ
    with pytest.raises(ht.HiptensorError) as e:
        ht.describe_contraction_plan(**bad)
    assert e.value.status == ht.STATUS_INVALID_VALUE
    bad = dict(args, type_compute=ht.COMPUTE_64F)
    with pytest.raises(ht.HiptensorError) as e:
        ht.describe_contraction_plan(**bad)
    assert e.value.status == ht.STATUS_NOT_SUPPORTED
