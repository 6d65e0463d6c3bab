// Flat extern "C" twin of the C++ API (include/hiptensor_b200.h): opaque handles around the
// std::vector-bearing structs, plain pointers and integers otherwise. Every function
// forwards to the C++ entry point of the same name in api.cpp.
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include <hiptensor/hiptensor.hpp>
#include <hiptensor_b200.h>

#include "kernels.hpp"

struct htHandle
{
    hiptensorHandle_t h;
};
struct htTensorDescriptor
{
    hiptensorTensorDescriptor_t d;
};
struct htContractionDesc
{
    hiptensorContractionDescriptor_t d;
};
struct htContractionFind
{
    hiptensorContractionFind_t f;
};
struct htContractionPlan
{
    hiptensorContractionPlan_t p;
};

namespace
{
    // a handle made by hiptensorCreate is a bare hiptensorHandle_t; htHandle has it as its
    // only member, so the pointers are interchangeable
    const hiptensorHandle_t* H(const htHandle* h)
    {
        return reinterpret_cast<const hiptensorHandle_t*>(h);
    }
    const hiptensorTensorDescriptor_t* TD(const htTensorDescriptor* d)
    {
        return d ? &d->d : nullptr;
    }
    int copyOut(const std::string& s, char* buf, uint64_t n)
    {
        if(!buf || n == 0)
            return HIPTENSOR_STATUS_INVALID_VALUE;
        std::strncpy(buf, s.c_str(), n - 1);
        buf[n - 1] = 0;
        return HIPTENSOR_STATUS_SUCCESS;
    }
} // namespace

extern "C" {

int htCreate(htHandle** handle)
{
    return hiptensorCreate(reinterpret_cast<hiptensorHandle_t**>(handle));
}
int htDestroy(htHandle* handle)
{
    return hiptensorDestroy(reinterpret_cast<hiptensorHandle_t*>(handle));
}
const char* htGetErrorString(int status)
{
    return hiptensorGetErrorString(hiptensorStatus_t(status));
}

int htCreateTensorDescriptor(const htHandle* handle, htTensorDescriptor** desc, uint32_t numModes,
                             const int64_t* lens, const int64_t* strides, int dataType, int unaryOp)
{
    if(!desc)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    *desc   = nullptr;
    auto* d = new(std::nothrow) htTensorDescriptor;
    if(!d)
        return HIPTENSOR_STATUS_ALLOC_FAILED;
    int rc = hiptensorInitTensorDescriptor(H(handle), &d->d, numModes, lens, strides, hipDataType(dataType),
                                           hiptensorOperator_t(unaryOp));
    if(rc != HIPTENSOR_STATUS_SUCCESS)
    {
        delete d;
        return rc;
    }
    *desc = d;
    return rc;
}
int htDestroyTensorDescriptor(htTensorDescriptor* desc)
{
    delete desc;
    return HIPTENSOR_STATUS_SUCCESS;
}

int htGetAlignmentRequirement(const htHandle* handle, const void* ptr, const htTensorDescriptor* desc,
                              uint32_t* alignmentRequirement)
{
    return hiptensorGetAlignmentRequirement(H(handle), ptr, TD(desc), alignmentRequirement);
}

int htPermutation(const htHandle* handle, const void* alpha, const void* A, const htTensorDescriptor* descA,
                  const int32_t* modeA, void* B, const htTensorDescriptor* descB, const int32_t* modeB,
                  int typeScalar, void* stream)
{
    return hiptensorPermutation(H(handle), alpha, A, TD(descA), modeA, B, TD(descB), modeB, hipDataType(typeScalar),
                                hipStream_t(stream));
}

int htCreateContractionDescriptor(const htHandle* handle, htContractionDesc** desc,
                                  const htTensorDescriptor* descA, const int32_t* modeA, uint32_t alignA,
                                  const htTensorDescriptor* descB, const int32_t* modeB, uint32_t alignB,
                                  const htTensorDescriptor* descC, const int32_t* modeC, uint32_t alignC,
                                  const htTensorDescriptor* descD, const int32_t* modeD, uint32_t alignD,
                                  int typeCompute)
{
    if(!desc)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    *desc   = nullptr;
    auto* d = new(std::nothrow) htContractionDesc;
    if(!d)
        return HIPTENSOR_STATUS_ALLOC_FAILED;
    int rc = hiptensorInitContractionDescriptor(H(handle), &d->d, TD(descA), modeA, alignA, TD(descB), modeB, alignB,
                                                TD(descC), modeC, alignC, TD(descD), modeD, alignD,
                                                hiptensorComputeType_t(typeCompute));
    if(rc != HIPTENSOR_STATUS_SUCCESS)
    {
        delete d;
        return rc;
    }
    *desc = d;
    return rc;
}
int htDestroyContractionDescriptor(htContractionDesc* desc)
{
    delete desc;
    return HIPTENSOR_STATUS_SUCCESS;
}

int htCreateContractionFind(const htHandle* handle, htContractionFind** find, int algo)
{
    if(!find)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    *find   = nullptr;
    auto* f = new(std::nothrow) htContractionFind;
    if(!f)
        return HIPTENSOR_STATUS_ALLOC_FAILED;
    int rc = hiptensorInitContractionFind(H(handle), &f->f, hiptensorAlgo_t(algo));
    if(rc != HIPTENSOR_STATUS_SUCCESS)
    {
        delete f;
        return rc;
    }
    *find = f;
    return rc;
}
int htDestroyContractionFind(htContractionFind* find)
{
    delete find;
    return HIPTENSOR_STATUS_SUCCESS;
}

int htContractionGetWorkspaceSize(const htHandle* handle, const htContractionDesc* desc,
                                  const htContractionFind* find, int pref, uint64_t* workspaceSize)
{
    return hiptensorContractionGetWorkspaceSize(H(handle), desc ? &desc->d : nullptr, find ? &find->f : nullptr,
                                                hiptensorWorksizePreference_t(pref), workspaceSize);
}

int htCreateContractionPlan(const htHandle* handle, htContractionPlan** plan, const htContractionDesc* desc,
                            const htContractionFind* find, uint64_t workspaceSize)
{
    if(!plan)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    *plan   = nullptr;
    auto* p = new(std::nothrow) htContractionPlan;
    if(!p)
        return HIPTENSOR_STATUS_ALLOC_FAILED;
    p->p.mSolution = nullptr;
    int rc = hiptensorInitContractionPlan(H(handle), &p->p, desc ? &desc->d : nullptr, find ? &find->f : nullptr,
                                          workspaceSize);
    if(rc != HIPTENSOR_STATUS_SUCCESS)
    {
        delete p;
        return rc;
    }
    *plan = p;
    return rc;
}
int htDestroyContractionPlan(htContractionPlan* plan)
{
    delete plan;
    return HIPTENSOR_STATUS_SUCCESS;
}

int htContraction(const htHandle* handle, const htContractionPlan* plan, const void* alpha, const void* A,
                  const void* B, const void* beta, const void* C, void* D, void* workspace,
                  uint64_t workspaceSize, void* stream)
{
    return hiptensorContraction(H(handle), plan ? &plan->p : nullptr, alpha, A, B, beta, C, D, workspace,
                                workspaceSize, hipStream_t(stream));
}

int htReduction(const htHandle* handle, const void* alpha, const void* A, const htTensorDescriptor* descA,
                const int32_t* modeA, const void* beta, const void* C, const htTensorDescriptor* descC,
                const int32_t* modeC, void* D, const htTensorDescriptor* descD, const int32_t* modeD,
                int opReduce, int typeCompute, void* workspace, uint64_t workspaceSize, void* stream)
{
    return hiptensorReduction(H(handle), alpha, A, TD(descA), modeA, beta, C, TD(descC), modeC, D, TD(descD), modeD,
                              hiptensorOperator_t(opReduce), hiptensorComputeType_t(typeCompute), workspace,
                              workspaceSize, hipStream_t(stream));
}

int htReductionNoAlloc(const htHandle* handle, const void* alpha, const void* A, const htTensorDescriptor* descA,
                       const int32_t* modeA, const void* beta, const void* C, const htTensorDescriptor* descC,
                       const int32_t* modeC, void* D, const htTensorDescriptor* descD, const int32_t* modeD,
                       int opReduce, int typeCompute, void* stream)
{
    return htb::reductionNoAlloc(H(handle), alpha, A, TD(descA), modeA, beta, C, TD(descC), modeC, D, TD(descD),
                                 modeD, opReduce, typeCompute, stream);
}

int htReductionGetWorkspaceSize(const htHandle* handle, const void* A, const htTensorDescriptor* descA,
                                const int32_t* modeA, const void* C, const htTensorDescriptor* descC,
                                const int32_t* modeC, const void* D, const htTensorDescriptor* descD,
                                const int32_t* modeD, int opReduce, int typeCompute, uint64_t* workspaceSize)
{
    return hiptensorReductionGetWorkspaceSize(H(handle), A, TD(descA), modeA, C, TD(descC), modeC, D, TD(descD), modeD,
                                              hiptensorOperator_t(opReduce), hiptensorComputeType_t(typeCompute),
                                              workspaceSize);
}

int htLoggerSetMask(int32_t mask)
{
    return hiptensorLoggerSetMask(mask);
}
int htLoggerOpenFile(const char* logFile)
{
    return hiptensorLoggerOpenFile(logFile);
}

int htDescribePermutationPlan(uint32_t numModes, const int64_t* lensA, const int32_t* modeA, const int32_t* modeB,
                              int dataTypeA, int dataTypeB, char* buf, uint64_t bufSize)
{
    htb::PermPlan p;
    int           rc = htb::planPermutation(int(numModes), lensA, modeA, modeB, dataTypeA, dataTypeB, true, &p);
    if(rc != htb::PLAN_OK)
        return rc;
    return copyOut(htb::describe(p), buf, bufSize);
}

int htDescribeReductionPlan(uint32_t numModesA, const int64_t* lensA, const int64_t* stridesA,
                            const int32_t* modeA, uint32_t numModesD, const int64_t* lensD,
                            const int64_t* stridesD, const int32_t* modeD, int dataType, char* buf,
                            uint64_t bufSize)
{
    htb::ReducePlan p;
    int rc = htb::planReduction(int(numModesA), lensA, stridesA, modeA, int(numModesD), lensD, stridesD, modeD,
                                htb::dtypeSize(dataType), true, 148, &p);
    if(rc != htb::PLAN_OK)
        return rc;
    return copyOut(htb::describe(p), buf, bufSize);
}

int htDescribeContractionPlan(uint32_t numModesA, const int64_t* lensA, const int64_t* stridesA,
                              const int32_t* modeA, int dataTypeA, uint32_t numModesB, const int64_t* lensB,
                              const int64_t* stridesB, const int32_t* modeB, int dataTypeB, uint32_t numModesD,
                              const int64_t* lensD, const int64_t* stridesD, const int32_t* modeD, int dataTypeD,
                              int hasC, int typeCompute, char* buf, uint64_t bufSize)
{
    if(!lensA || !stridesA || !modeA || !lensB || !stridesB || !modeB || !lensD || !stridesD || !modeD)
        return HIPTENSOR_STATUS_INVALID_VALUE;
    htb::TensorView      A{int(numModesA), lensA, stridesA, modeA, dataTypeA};
    htb::TensorView      B{int(numModesB), lensB, stridesB, modeB, dataTypeB};
    htb::TensorView      D{int(numModesD), lensD, stridesD, modeD, dataTypeD};
    htb::ContractionPlan p;
    const bool cplx = typeCompute == HIPTENSOR_COMPUTE_C32F || typeCompute == HIPTENSOR_COMPUTE_C64F;
    int        rc   = cplx ? htb::planComplexContraction(A, B, D, dataTypeD, hasC != 0, typeCompute, 148, &p)
                           : htb::planContraction(A, B, D, dataTypeD, hasC != 0, typeCompute, 148, &p, ~uint64_t(0));
    if(rc != htb::PLAN_OK)
        return rc;
    return copyOut(htb::describe(p), buf, bufSize);
}

const char* htLastKernelName(void)
{
    return htb::lastKernelName();
}
int htGetDeviceStatus(const htHandle* handle, int32_t* status)
{
    if(!handle || !status)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    const htb::HandleState* st = htb::stateOf(H(handle));
    if(!st)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    *status = st->hostStatus ? *st->hostStatus : 0;
    return HIPTENSOR_STATUS_SUCCESS;
}

int htInjectDeviceStatus(const htHandle* handle, int32_t code)
{
    if(!handle)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    const htb::HandleState* st = htb::stateOf(H(handle));
    if(!st || !st->hostStatus)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    *st->hostStatus = code;
    return HIPTENSOR_STATUS_SUCCESS;
}

int htReductionFinish(const htHandle* handle, const void* alpha, const void* partial, const void* beta, const void* C,
                      void* D, const htTensorDescriptor* descD, int typeCompute, void* stream)
{
    return htb::reductionFinish(H(handle), alpha, partial, beta, C, D, TD(descD), typeCompute, stream);
}

void htReloadSwitches(void)
{
    htb::reloadSwitches();
}

uint64_t htKernelLaunchCount(void)
{
    return htb::launchCount();
}

} // extern "C"
