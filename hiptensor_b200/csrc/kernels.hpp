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

    // Complex plans (plan.complexKind != 0): alpha and beta as (re, im); the first plan.expandBytes of the
    // workspace are required, plan.workspaceBytes more are optional.
    cudaError_t launchComplexContraction(const ContractionPlan& plan, double alphaRe, double alphaIm, const void* A,
                                         const void* B, double betaRe, double betaIm, const void* C, void* D,
                                         void* workspace, uint64_t workspaceBytes, int smCount, int* deviceStatus,
                                         cudaStream_t stream);

    // Function attributes (dynamic shared-memory limit) belong to one device: true the first time the calling
    // site is reached with the current device, so that a process that drives several GPUs sets them on each.
    inline bool firstUseOnDevice(unsigned char (&seen)[kMaxDevices])
    {
        int dev = 0;
        if(cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
            return true;
        if(seen[dev])
            return false;
        seen[dev] = 1;
        return true;
    }
} // namespace htb
