// hipTensor-compatible C++ entry points, implemented for NVIDIA B200 (sm_100a).
//
// Signatures follow ROCm/hipTensor 1.4.0, library/include/hiptensor/hiptensor.hpp
// (line numbers below refer to that file). Like the reference, the functions have
// C++ linkage because the descriptor structs carry std::vector members; a flat
// extern "C" twin for FFI callers is declared in include/hiptensor_b200.h.
#ifndef HIPTENSOR_API_HPP
#define HIPTENSOR_API_HPP

#include "hiptensor_types.hpp"

// :41, :46  library context bound to the device that is current at creation
hiptensorStatus_t hiptensorCreate(hiptensorHandle_t** handle);
hiptensorStatus_t hiptensorDestroy(hiptensorHandle_t* handle);

// :60-66  strides == NULL means packed with the LAST mode fastest
hiptensorStatus_t hiptensorInitTensorDescriptor(const hiptensorHandle_t* handle, hiptensorTensorDescriptor_t* desc,
                                                const uint32_t numModes, const int64_t lens[],
                                                const int64_t strides[], hipDataType dataType,
                                                hiptensorOperator_t unaryOp);

// :71
const char* hiptensorGetErrorString(const hiptensorStatus_t error);

// :89-98  B[modeB] = opB(alpha * opA(A[modeA])); both tensors packed, FIRST mode fastest
hiptensorStatus_t hiptensorPermutation(const hiptensorHandle_t* handle, const void* alpha, const void* A,
                                       const hiptensorTensorDescriptor_t* descA, const int32_t modeA[], void* B,
                                       const hiptensorTensorDescriptor_t* descB, const int32_t modeB[],
                                       const hipDataType typeScalar, const hipStream_t stream);

// :108-111
hiptensorStatus_t hiptensorGetAlignmentRequirement(const hiptensorHandle_t* handle, const void* ptr,
                                                   const hiptensorTensorDescriptor_t* desc,
                                                   uint32_t*                          alignmentRequirement);

// :131-145  descC == NULL selects D = alpha*A*B, otherwise D = alpha*A*B + beta*C
hiptensorStatus_t hiptensorInitContractionDescriptor(
    const hiptensorHandle_t* handle, hiptensorContractionDescriptor_t* desc,
    const hiptensorTensorDescriptor_t* descA, const int32_t modeA[], const uint32_t alignmentRequirementA,
    const hiptensorTensorDescriptor_t* descB, const int32_t modeB[], const uint32_t alignmentRequirementB,
    const hiptensorTensorDescriptor_t* descC, const int32_t modeC[], const uint32_t alignmentRequirementC,
    const hiptensorTensorDescriptor_t* descD, const int32_t modeD[], const uint32_t alignmentRequirementD,
    hiptensorComputeType_t typeCompute);

// :157-159
hiptensorStatus_t hiptensorInitContractionFind(const hiptensorHandle_t* handle, hiptensorContractionFind_t* find,
                                               const hiptensorAlgo_t algo);

// :170-174
hiptensorStatus_t hiptensorContractionGetWorkspaceSize(const hiptensorHandle_t*                handle,
                                                       const hiptensorContractionDescriptor_t* desc,
                                                       const hiptensorContractionFind_t*       find,
                                                       const hiptensorWorksizePreference_t     pref,
                                                       uint64_t*                               workspaceSize);

// :191-195
hiptensorStatus_t hiptensorInitContractionPlan(const hiptensorHandle_t* handle, hiptensorContractionPlan_t* plan,
                                               const hiptensorContractionDescriptor_t* desc,
                                               const hiptensorContractionFind_t* find, const uint64_t workspaceSize);

// :218-228  alpha/beta: host pointers typed by the plan's compute type
hiptensorStatus_t hiptensorContraction(const hiptensorHandle_t* handle, const hiptensorContractionPlan_t* plan,
                                       const void* alpha, const void* A, const void* B, const void* beta,
                                       const void* C, void* D, void* workspace, uint64_t workspaceSize,
                                       hipStream_t stream);

// :255-271  D = alpha * reduce(A over the modes absent from modeC) + beta * C
hiptensorStatus_t hiptensorReduction(const hiptensorHandle_t* handle, const void* alpha, const void* A,
                                     const hiptensorTensorDescriptor_t* descA, const int32_t modeA[],
                                     const void* beta, const void* C, const hiptensorTensorDescriptor_t* descC,
                                     const int32_t modeC[], void* D, const hiptensorTensorDescriptor_t* descD,
                                     const int32_t modeD[], hiptensorOperator_t opReduce,
                                     hiptensorComputeType_t typeCompute, void* workspace, uint64_t workspaceSize,
                                     hipStream_t stream);

// :290-302
hiptensorStatus_t hiptensorReductionGetWorkspaceSize(
    const hiptensorHandle_t* handle, const void* A, const hiptensorTensorDescriptor_t* descA, const int32_t modeA[],
    const void* C, const hiptensorTensorDescriptor_t* descC, const int32_t modeC[], const void* D,
    const hiptensorTensorDescriptor_t* descD, const int32_t modeD[], hiptensorOperator_t opReduce,
    hiptensorComputeType_t typeCompute, uint64_t* workspaceSize);

// :308-338  logger controls (sink: stdout, FILE*, file name or callback)
hiptensorStatus_t hiptensorLoggerSetCallback(hiptensorLoggerCallback_t callback);
hiptensorStatus_t hiptensorLoggerSetFile(FILE* file);
hiptensorStatus_t hiptensorLoggerOpenFile(const char* logFile);
hiptensorStatus_t hiptensorLoggerSetLevel(hiptensorLogLevel_t level);
hiptensorStatus_t hiptensorLoggerSetMask(int32_t mask);
hiptensorStatus_t hiptensorLoggerForceDisable();

// :343  reports the CUDA runtime version here
int hiptensorGetHiprtVersion();

#endif // HIPTENSOR_API_HPP
