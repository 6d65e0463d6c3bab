// Type definitions of the hipTensor-compatible C++ interface, CUDA edition.
//
// Enumerator values and struct member order match ROCm/hipTensor 1.4.0
// (library/include/hiptensor/hiptensor_types.hpp:42-236) so that code written
// against that header recompiles unchanged against this one. The HIP names
// (hipDataType, hipStream_t, HIP_R_32F ...) are aliases of their CUDA twins,
// whose numeric values coincide (R_32F=0, R_64F=1, R_16F=2, R_16BF=14).
#ifndef HIPTENSOR_TYPES_HPP
#define HIPTENSOR_TYPES_HPP

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <vector>

#include <cuComplex.h>
#include <cuda_runtime_api.h>
#include <library_types.h>

using hipDataType = cudaDataType;
using hipStream_t = cudaStream_t;
// element types of HIP_C_32F / HIP_C_64F tensors and of their alpha / beta (hip/hip_complex.h in the reference)
using hipFloatComplex  = cuFloatComplex;
using hipDoubleComplex = cuDoubleComplex;
#define HIP_R_16F CUDA_R_16F
#define HIP_R_16BF CUDA_R_16BF
#define HIP_R_32F CUDA_R_32F
#define HIP_R_64F CUDA_R_64F
#define HIP_C_32F CUDA_C_32F
#define HIP_C_64F CUDA_C_64F

typedef enum
{
    HIPTENSOR_STATUS_SUCCESS                = 0,
    HIPTENSOR_STATUS_NOT_INITIALIZED        = 1, // null handle / descriptor / plan
    HIPTENSOR_STATUS_ALLOC_FAILED           = 3,
    HIPTENSOR_STATUS_INVALID_VALUE          = 7, // user error in an argument
    HIPTENSOR_STATUS_ARCH_MISMATCH          = 8, // wrong device, or device is not sm_100
    HIPTENSOR_STATUS_EXECUTION_FAILED       = 13, // a kernel reported an error
    HIPTENSOR_STATUS_INTERNAL_ERROR         = 14,
    HIPTENSOR_STATUS_NOT_SUPPORTED          = 15,
    HIPTENSOR_STATUS_CK_ERROR               = 17, // kept for source compatibility, never returned
    HIPTENSOR_STATUS_HIP_ERROR              = 18, // a CUDA runtime call failed
    HIPTENSOR_STATUS_INSUFFICIENT_WORKSPACE = 19,
    HIPTENSOR_STATUS_INSUFFICIENT_DRIVER    = 20,
    HIPTENSOR_STATUS_IO_ERROR               = 21,
} hiptensorStatus_t;

typedef enum
{
    HIPTENSOR_COMPUTE_NONE = 0,
    HIPTENSOR_COMPUTE_16F  = (1U << 0U),
    HIPTENSOR_COMPUTE_32F  = (1U << 2U),
    HIPTENSOR_COMPUTE_64F  = (1U << 4U),
    HIPTENSOR_COMPUTE_8U   = (1U << 6U), // reserved
    HIPTENSOR_COMPUTE_32U  = (1U << 7U), // reserved
    HIPTENSOR_COMPUTE_8I   = (1U << 8U), // reserved
    HIPTENSOR_COMPUTE_32I  = (1U << 9U), // reserved
    HIPTENSOR_COMPUTE_16BF = (1U << 10U),
    HIPTENSOR_COMPUTE_C32F = (1U << 11U),
    HIPTENSOR_COMPUTE_C64F = (1U << 12U),
} hiptensorComputeType_t;

typedef enum
{
    HIPTENSOR_OP_IDENTITY = 1,
    HIPTENSOR_OP_SQRT     = 2, // evaluates x*x, as the reference does
    HIPTENSOR_OP_ADD      = 3,
    HIPTENSOR_OP_MUL      = 5,
    HIPTENSOR_OP_MAX      = 6,
    HIPTENSOR_OP_MIN      = 7,
    HIPTENSOR_OP_UNKNOWN  = 126,
} hiptensorOperator_t;

typedef enum
{
    HIPTENSOR_ALGO_ACTOR_CRITIC    = -8,
    HIPTENSOR_ALGO_DEFAULT_PATIENT = -6,
    HIPTENSOR_ALGO_DEFAULT         = -1,
} hiptensorAlgo_t;

typedef enum
{
    HIPTENSOR_WORKSPACE_MIN         = 1,
    HIPTENSOR_WORKSPACE_RECOMMENDED = 2,
    HIPTENSOR_WORKSPACE_MAX         = 3,
} hiptensorWorksizePreference_t;

typedef enum
{
    HIPTENSOR_LOG_LEVEL_OFF              = 0,
    HIPTENSOR_LOG_LEVEL_ERROR            = 1,
    HIPTENSOR_LOG_LEVEL_PERF_TRACE       = 2,
    HIPTENSOR_LOG_LEVEL_PERF_HINT        = 4,
    HIPTENSOR_LOG_LEVEL_HEURISTICS_TRACE = 8,
    HIPTENSOR_LOG_LEVEL_API_TRACE        = 16,
} hiptensorLogLevel_t;

// 4 KiB opaque library context, allocated by hiptensorCreate.
struct hiptensorHandle_t
{
    int64_t fields[512];
};

struct hiptensorTensorDescriptor_t
{
    hipDataType              mType;
    std::vector<std::size_t> mLengths;
    std::vector<std::size_t> mStrides;
    hiptensorOperator_t      mUnaryOp;
};

struct hiptensorContractionDescriptor_t
{
    int32_t                                  mContractionOpId; // 0 scale, 1 bilinear
    hiptensorComputeType_t                   mComputeType;
    std::vector<hiptensorTensorDescriptor_t> mTensorDesc; // A, B, C, D
    std::vector<uint32_t>                    mAlignmentReq;
    std::vector<std::vector<int32_t>>        mTensorMode; // A, B, C (bilinear) or A, B, D (scale)
};

struct hiptensorContractionFind_t
{
    hiptensorAlgo_t    mSelectionAlgorithm;
    std::vector<void*> mCandidates;
};

struct hiptensorContractionPlan_t
{
    void*                            mSolution; // kernel choice made at plan time
    hiptensorContractionDescriptor_t mContractionDesc;
};

typedef void (*hiptensorLoggerCallback_t)(int32_t logContext, const char* funcName, const char* msg);

#endif // HIPTENSOR_TYPES_HPP
