// Host-side planner: mode-label parsing, stride folding and kernel selection for the
// three operations. Pure C++ (no CUDA calls) so that it can be tested without a GPU.
// The structs are plain data and are passed by value to the kernels.
//
// It replaces, in the reference:
//   contraction : normalizeTensorModes (library/src/contraction/contraction_solution.cpp:34-160)
//                 and the CK instance selection (contraction_selection.cpp:44-195,1687-2214)
//   permutation : PermutationSolutionImpl::initArgs (permutation_solution_impl.hpp:103-145)
//   reduction   : ReductionSolutionImpl::initArgs (reduction_solution_impl.hpp:105-163)
#pragma once

#include <cstdint>
#include <string>

namespace htb
{
    constexpr int kMaxRank  = 12; // reference limit: 6 M + 6 N or 6 K modes per tensor
    constexpr int kMaxGroup = 6; // modes per group (contraction_meta_traits.hpp:41-43)

    enum PlanStatus : int
    {
        PLAN_OK            = 0,
        PLAN_INVALID       = 7, // HIPTENSOR_STATUS_INVALID_VALUE
        PLAN_NOT_SUPPORTED = 15 // HIPTENSOR_STATUS_NOT_SUPPORTED
    };

    // ------------------------------------------------------------------ permutation
    enum PermKind : int
    {
        PERM_COPY = 0, // A's and B's fastest folded modes coincide: row copy
        PERM_TILE = 1, // 2-D tiled transpose through shared memory, plain loads/stores
        PERM_TMA  = 2 // same tiling, TMA box loads/stores with 128B-swizzled staging
    };

    struct PermPlan
    {
        int     ndim; // folded modes, in A's order; dim 0 has strideA == 1
        int     q; // folded mode whose strideB == 1
        int     kind;
        int     elemSize; // bytes of A's element
        int64_t ext[kMaxGroup];
        int64_t sA[kMaxGroup];
        int64_t sB[kMaxGroup];
        int64_t total;
        // B-side view for the TMA store map: folded modes sorted by ascending strideB
        int orderB[kMaxGroup];
    };

    // lens/modeA describe A; B's extents follow from modeB. Strides are recomputed
    // packed with the first mode fastest, as the reference does.
    int planPermutation(int rank, const int64_t* lensA, const int32_t* modeA, const int32_t* modeB,
                        int typeA, int typeB, bool pointersAligned16, PermPlan* out);
    std::string describe(const PermPlan& p);

    // ------------------------------------------------------------------ reduction
    enum ReduceKind : int
    {
        RED_ROW     = 0, // a reduced mode is contiguous in A: lanes run along the reduced axis
        RED_COL     = 1, // a kept mode is contiguous in A: lanes run along the kept axis
        RED_GENERIC = 2 // neither has stride 1
    };

    struct ReducePlan
    {
        int     nk, nr; // folded kept / reduced modes, each sorted by ascending strideA
        int     kind;
        int     vec; // elements per vector load along the contiguous axis (a power of two, 16 bytes at most)
        int64_t kext[kMaxGroup], ksA[kMaxGroup], ksD[kMaxGroup];
        int64_t rext[kMaxGroup], rsA[kMaxGroup];
        int64_t nOut, nRed;
        int     split; // >1: the reduced range is cut into this many slices (two-pass, needs scratch)
        // Short contiguous reduced rows (RED_ROW with at most 16 loads of shortVec elements per row): lanes per output of
        // the short-row kernel (1, 2, 4, 8 or 16), else 0.
        int     shortLanes, shortVec;
        // RED_COL: outputs per thread along the contiguous kept mode (16-byte loads, or 1) and the block shape: colTx
        // threads over the outputs, colTy over the innermost reduced mode (colTx * colTy <= 256).
        int     colVec, colTx, colTy;
        // 1: the split only fills the GPU better; a caller without enough scratch runs the single pass instead
        int     splitOptional;
    };

    int planReduction(int rankA, const int64_t* lensA, const int64_t* stridesA, const int32_t* modeA, int rankD,
                      const int64_t* lensD, const int64_t* stridesD, const int32_t* modeD, int elemSize,
                      bool pointersAligned16, int smCount, ReducePlan* out);
    std::string describe(const ReducePlan& p);

    // ------------------------------------------------------------------ contraction
    enum ContractionKind : int
    {
        CK_TILED_SIMT = 0, // shared-memory tiled FMA kernel with gathered operands (f32 accumulate)
        CK_TILED_DMMA = 1, // same tiling, FP64 tensor-pipe MMA
        CK_TCGEN05    = 2, // TMA + tcgen05.mma with TMEM accumulators (f16/bf16 inputs)
        CK_TF32X3     = 3 // fp32 inputs on the tensor cores: big/small TF32 split, three tcgen05.mma per K step
    };

    struct ModeDim
    {
        int64_t ext;
        int64_t s0; // stride in the group's first tensor
        int64_t s1; // stride in the group's second tensor
    };

    struct ContractionPlan
    {
        // groups after classification and folding; first/second tensor per group:
        //   m: (A, D)   n: (B, D)   k: (A, B)
        int     nm, nn, nk;
        ModeDim m[kMaxGroup], n[kMaxGroup], k[kMaxGroup];
        int64_t M, N, K;
        int     typeA, typeB, typeC, typeD; // cudaDataType; typeC < 0 when there is no C
        int     computeType;
        int     bilinear;
        int     swapped; // A and B (and M and N) exchanged so that D is contiguous along N
        int     kind;
        // tcgen05 path only
        int tileM, tileN, tileK, stages;
        int boxM[4], boxN[4]; // TMA box extent per folded M / N mode (product = rows gathered per tile)
        int rowsM, rowsN; // rows of the tile that the boxes fill (<= tileM / tileN)
        int pair; // 256 x 256 tile over a CTA pair (tcgen05 cta_group::2), each CTA loading 128 rows of B
        int pairOk; // CK_TCGEN05: the pair kernel can run this problem (pair says whether it is the better choice)
        int wide; // CK_TCGEN05 pair kernel: 256 x 512 tiles (one accumulator filling tensor memory) instead of 256 x 256
        int ksplit; // CK_TCGEN05 pair kernel: 2 = every tile's K range cut over the two CTA pairs of a four-CTA cluster
        int boxN128[4], rowsN128; // N boxes of one CTA's sub-tile in the pair kernels (128 rows; 64 for CK_TF32X3)
        int aKContig, bKContig; // operand has its K group folded to one stride-1 mode
        // CK_TF32X3 only: 0 = operand K-major (rows gathered by boxM / boxN), 1 = MN-major (32-row chunks along
        // the row group's stride-1 mode: m[0] for A, n[nFast] for B; K rows gathered by boxK)
        int aMajor, bMajor, nFast;
        int boxK[2];
        // split of the K range over several CTAs (needs workspace); 1 = none
        int      splitK;
        uint64_t workspaceBytes;
        // Complex contraction run as one real contraction (planComplexContraction); the fields above then
        // describe the real problem. 0: real; 1 / 2: operand A / B is replaced by its expanded real copy, which
        // occupies the first expandBytes of the workspace (required), followed by workspaceBytes (optional).
        int      complexKind;
        int      xRank, xFree; // modes of the copied operand in the copy's order: xFree free modes, then contracted
        int      dRank;
        int64_t  xExt[kMaxRank], xStride[kMaxRank]; // extents and source strides (complex elements)
        int64_t  dExt[kMaxRank], dStride[kMaxRank]; // D's modes (complex elements), for the beta pass over C
        uint64_t expandBytes;
        // cf32 only: the other operand is copied too (plain, contracted modes innermost) when the tensor-core
        // kernel cannot read it where it lies; its copy follows the first one at byte offset yOffset
        int      yCopy, yRank, yFree;
        int64_t  yExt[kMaxRank], yStride[kMaxRank];
        uint64_t yOffset;
        // Real f16 / bf16 / f32 contraction whose operands the tensor-core kernels cannot read where they lie (a stride
        // that is not a multiple of 16 bytes, a contracted mode contiguous in one operand and a free mode in the other
        // ...): both operands are first copied into the workspace as packed matrices, one row per free index, the
        // contracted modes merged into one mode of packK elements padded with zeros to packKp (a multiple of 16 bytes),
        // and the fields above describe the contraction of the copies. A's copy is described by x*, B's by y* (extents
        // and source strides in the copy's order: free modes, then contracted ones); B's copy lies at yOffset;
        // expandBytes covers both.
        int      packReal;
        int64_t  packK, packKp;
        // 0 from the planner. The library's plan registry gives every plan it keeps a process-wide unique
        // number, which the launchers use as the key of their tensor-map caches (0 = do not cache).
        uint64_t cacheId;
    };

    struct TensorView
    {
        int            rank;
        const int64_t* lens;
        const int64_t* strides;
        const int32_t* modes;
        int            type;
    };

    // D's modes are looked up in A first, then in B (as the reference does); C, when
    // present, is addressed with D's strides (contraction_solution_impl.hpp:125-140).
    // workspaceLimit: bytes of scratch the caller can give; a plan that needs packed copies of the operands is made only
    // when the copies fit.
    int planContraction(const TensorView& A, const TensorView& B, const TensorView& D, int typeC, bool bilinear,
                        int computeType, int smCount, ContractionPlan* out, uint64_t workspaceLimit = 0);
    // cf32 / cf64 tensors with compute type C32F / C64F: see planner.cpp
    int planComplexContraction(const TensorView& A, const TensorView& B, const TensorView& D, int typeC, bool bilinear,
                               int computeType, int smCount, ContractionPlan* out);
    std::string describe(const ContractionPlan& p);

    // Whether an M x N x K half-precision problem that the CTA-pair tensor-core kernel can run should run on it
    // (*pair), with 256 x 512 instead of 256 x 256 tiles (*wide), and with every tile's K range cut over the two CTA
    // pairs of a four-CTA cluster (*ksplit = 2). Rules from measurements: see planner.cpp.
    void pairKernelForm(int64_t M, int64_t N, int64_t K, int sms, int* pair, int* wide, int* ksplit);

    // Splits `tile` rows over the folded modes of a group, fastest mode first: a mode is taken
    // whole while it is a power of two smaller than what is left, the first mode at least as
    // large as what is left takes the rest (ragged ends are zero-filled by TMA), and so does the last mode
    // whatever its extent; later modes get 1. Returns the rows covered (0 if the group cannot be boxed).
    int boxDecompose(const ModeDim* dims, int n, int tile, int* box);

    // Shared helper: fold adjacent modes of one group. dims must already be sorted by
    // ascending s0 (or any order the caller wants to keep); two neighbours merge when
    // both strides of the second equal stride*extent of the first. Extent-1 modes are
    // dropped. Returns the new count (at least 1: a group that folds away becomes {1,0,0}).
    int foldGroup(ModeDim* dims, int n);
} // namespace htb
