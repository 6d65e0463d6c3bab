// Launch entry points of the CUDA kernels (one translation unit per operation).
#pragma once

#include <cuda.h>
#include <cuda_runtime_api.h>

#include "common.hpp"
#include "planner.hpp"

namespace htb
{
    // cuTensorMapEncodeTiled, resolved through the runtime so that the library does not
    // link against libcuda (it must load on machines without a driver).
    typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                        const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                        CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                        CUtensorMapFloatOOBfill);
    PFN_encodeTiled tensorMapEncoder();

    cudaError_t launchPermutation(const PermPlan& plan, int typeA, int typeB, const void* A, void* B, float alpha,
                                  int opA, int opB, int smCount, int* deviceStatus, cudaStream_t stream);

    // alpha/beta already widened to double; C may alias D or be null (beta then ignored).
    // workspace is used only when plan.split > 1.
    cudaError_t launchReduction(const ReducePlan& plan, int typeA, int computeType, int op, double alpha,
                                const void* A, double beta, const void* C, void* D, void* workspace,
                                cudaStream_t stream);
    uint64_t    reductionWorkspaceBytes(const ReducePlan& plan, int computeType);

    // Same reduction, with the two-pass scratch taken from a fixed array inside the library
    // instead of from the caller (no allocation anywhere on this path). The first call on a
    // device looks the array's device address up.
    constexpr uint64_t kStaticScratchBytes = 8192;
    constexpr int      kMaxDevices         = 64;
    cudaError_t launchReductionStaticScratch(const ReducePlan& plan, int typeA, int computeType, int op, double alpha,
                                             const void* A, double beta, const void* C, void* D, int device,
                                             cudaStream_t stream);

    // Finish of a reduction whose reduced mode was split over devices: D = alpha * partial + beta * C over D's
    // layout (lens / strides in elements), `partial` laid out like D. Body of htReductionFinish.
    cudaError_t launchReductionFinish(int typeD, double alpha, const void* partial, double beta, const void* C, void* D,
                                      int rank, const int64_t* lens, const int64_t* strides, cudaStream_t stream);
    int         reductionFinish(const hiptensorHandle_t* handle, const void* alpha, const void* partial, const void* beta,
                                const void* C, void* D, const hiptensorTensorDescriptor_t* descD, int typeCompute,
                                void* stream);

    // body of the flat entry point htReductionNoAlloc (api.cpp)
    int reductionNoAlloc(const hiptensorHandle_t* handle, const void* alpha, const void* A,
                         const hiptensorTensorDescriptor_t* descA, const int32_t* modeA, const void* beta,
                         const void* C, const hiptensorTensorDescriptor_t* descC, const int32_t* modeC, void* D,
                         const hiptensorTensorDescriptor_t* descD, const int32_t* modeD, int opReduce,
                         int typeCompute, void* stream);

    // A/B are the caller's operands in the caller's order; the plan says whether to swap.
    cudaError_t launchContraction(const ContractionPlan& plan, float alpha, const void* A, const void* B,
                                  float beta, const void* C, void* D, void* workspace, uint64_t workspaceBytes,
                                  int smCount, int* deviceStatus, cudaStream_t stream);

    // Plans with plan.packReal: copies both operands into the first plan.expandBytes of the workspace (required) as
    // packed matrices and contracts the copies (contraction_pack.cu).
    cudaError_t launchPackedContraction(const ContractionPlan& plan, float alpha, const void* A, const void* B, float beta,
                                        const void* C, void* D, void* workspace, uint64_t workspaceBytes, int smCount,
                                        int* deviceStatus, cudaStream_t stream);

    // Complex plans (plan.complexKind != 0): alpha and beta as (re, im); the first plan.expandBytes of the
    // workspace are required, plan.workspaceBytes more are optional.
    cudaError_t launchComplexContraction(const ContractionPlan& plan, double alphaRe, double alphaIm, const void* A,
                                         const void* B, double betaRe, double betaIm, const void* C, void* D,
                                         void* workspace, uint64_t workspaceBytes, int smCount, int* deviceStatus,
                                         cudaStream_t stream);

    // Encoded tensor maps of recent launches, per host thread: a repeated hiptensorContraction with the same plan
    // on the same operand buffers encodes nothing. The key holds everything a map depends on: the plan (by the
    // registry's unique number; plans without one are never found again), the two base addresses and the kernel
    // variant (family and tile form).
    struct MapCacheEntry
    {
        uint64_t    id;
        const void *A, *B;
        int         variant;
        int         half; // f16 pair kernel, 64-row B map of the half tiles: 0 not made yet, 1 made, 2 cannot be made
        const void* D; // f16 pair kernel: the output that mapD was encoded for (null: none yet)
        CUtensorMap mapA, mapB, mapB64, mapD;
    };
    // The entry for this key; *hit says whether its maps are already encoded. On a miss the caller encodes into
    // the entry (and sets id = 0 if that fails).
    MapCacheEntry* mapCacheFind(uint64_t id, const void* A, const void* B, int variant, bool* hit);

    // Raises a kernel's dynamic shared-memory limit to `bytes` on the current device unless an earlier call
    // already did (the attribute belongs to one device; a launch then costs a table lookup, not a runtime call).
    cudaError_t ensureDynamicSmem(const void* kernel, int bytes);
} // namespace htb
