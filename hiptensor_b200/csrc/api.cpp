// The hipTensor-compatible C++ entry points (include/hiptensor/hiptensor.hpp) for the three
// hot paths. Validation order, status codes and scalar decoding follow the reference
// (library/src/hiptensor.cpp, library/src/contraction/hiptensor_contraction.cpp,
// library/src/permutation/hiptensor_permutation.cpp, library/src/reduction/hiptensor_reduction.cpp);
// kernel selection is the closed-form planner in planner.cpp and the kernels are this
// library's own. Unlike the reference nothing here exits the process or blocks the host:
// CUDA failures come back as HIPTENSOR_STATUS_HIP_ERROR.
#include <iterator>
#include <list>
#include <memory>
#include <mutex>
#include <set>
#include <unordered_map>
#include <vector>

#include <cuda_runtime_api.h>

#include <hiptensor/hiptensor.hpp>

#include "kernels.hpp"

using namespace htb;

namespace
{
    HandleState* mutableState(hiptensorHandle_t* h)
    {
        return reinterpret_cast<HandleState*>(h->fields);
    }

    // ARCH_MISMATCH unless the current device is the one the handle was made on
    // (hiptensor_contraction.cpp:263-277).
    hiptensorStatus_t checkDevice(const char* func, const HandleState* st)
    {
        int dev = -1;
        if(cudaGetDevice(&dev) != cudaSuccess)
            return HIPTENSOR_STATUS_HIP_ERROR;
        if(dev != st->device)
        {
            HTB_LOG_ERROR(func, "Device mismatch error: current device id: %d, handle device id: %d (%s)", dev,
                          st->device, hiptensorGetErrorString(HIPTENSOR_STATUS_ARCH_MISMATCH));
            return HIPTENSOR_STATUS_ARCH_MISMATCH;
        }
        // A kernel of an earlier call gave up a bounded wait (it skipped its remaining work, so that call's
        // output is incomplete): reported once, on the next call, then cleared. The kernels exit cleanly, the
        // handle stays usable.
        if(st->hostStatus && *st->hostStatus != 0)
        {
            const int code = *st->hostStatus;
            *st->hostStatus = 0;
            HTB_LOG_ERROR(func, "an earlier kernel on this handle timed out in a device-side wait (code %d) (%s)", code,
                          hiptensorGetErrorString(HIPTENSOR_STATUS_EXECUTION_FAILED));
            return HIPTENSOR_STATUS_EXECUTION_FAILED;
        }
        return HIPTENSOR_STATUS_SUCCESS;
    }

    std::vector<int64_t> toI64(const std::vector<std::size_t>& v)
    {
        return std::vector<int64_t>(v.begin(), v.end());
    }

    // Plans are owned by the library and shared between identical problems, like the
    // singleton-owned solutions the reference's plan points to
    // (hiptensor_contraction.cpp:600-601). Look-ups are hashed (by content when a plan is made, by
    // address when it is used). The registry keeps the kCapacity most recently used plans; a caller's
    // hiptensorContractionPlan_t whose plan has been dropped is planned again from the descriptor it
    // carries (see hiptensorContraction), so that a service that plans ever new shapes does not grow
    // without bound.
    struct PlanRegistry
    {
        static constexpr std::size_t kCapacity = 4096;
        struct Node
        {
            ContractionPlan plan;
            uint64_t        hash;
        };
        using Iter = std::list<Node>::iterator;
        std::mutex                                        mutex;
        std::list<Node>                                   lru; // most recently used first; nodes never move
        std::unordered_map<const void*, Iter>             byAddress;
        std::unordered_multimap<uint64_t, Iter>           byContent;
        uint64_t                                          nextId = 1;

        static uint64_t hashOf(const ContractionPlan& p)
        {
            // FNV-1a over the plan's bytes (planned with cacheId = 0; the struct is memset before it is filled)
            const unsigned char* b = reinterpret_cast<const unsigned char*>(&p);
            uint64_t             h = 1469598103934665603ull;
            for(std::size_t i = 0; i < sizeof(p); i++)
                h = (h ^ b[i]) * 1099511628211ull;
            return h;
        }
        const ContractionPlan* intern(const ContractionPlan& fresh)
        {
            ContractionPlan p = fresh;
            p.cacheId         = 0;
            const uint64_t h  = hashOf(p);
            std::lock_guard<std::mutex> lock(mutex);
            auto range = byContent.equal_range(h);
            for(auto it = range.first; it != range.second; ++it)
            {
                p.cacheId = it->second->plan.cacheId;
                if(std::memcmp(&it->second->plan, &p, sizeof(p)) == 0)
                {
                    lru.splice(lru.begin(), lru, it->second);
                    return &it->second->plan;
                }
            }
            p.cacheId = nextId++;
            lru.push_front(Node{p, h});
            byAddress.emplace(&lru.front().plan, lru.begin());
            byContent.emplace(h, lru.begin());
            while(lru.size() > kCapacity)
            {
                Iter last  = std::prev(lru.end());
                auto range2 = byContent.equal_range(last->hash);
                for(auto it = range2.first; it != range2.second; ++it)
                    if(it->second == last)
                    {
                        byContent.erase(it);
                        break;
                    }
                byAddress.erase(&last->plan);
                lru.pop_back();
            }
            return &lru.front().plan;
        }
        // the plan at this address if the registry still keeps it (marks it as used)
        const ContractionPlan* find(const void* ptr)
        {
            std::lock_guard<std::mutex> lock(mutex);
            auto it = byAddress.find(ptr);
            if(it == byAddress.end())
                return nullptr;
            lru.splice(lru.begin(), lru, it->second);
            return &it->second->plan;
        }
    };
    PlanRegistry& registry()
    {
        static PlanRegistry r;
        return r;
    }

    int buildContractionPlan(const hiptensorContractionDescriptor_t* desc, int smCount, ContractionPlan* out,
                             uint64_t workspaceLimit)
    {
        if(desc->mTensorDesc.size() != 4 || desc->mTensorMode.size() < 3)
            return HIPTENSOR_STATUS_INVALID_VALUE;
        // operation ids: 0 scale, 1 bilinear, 2 / 3 the same with complex compute types
        // (hiptensor_contraction.cpp:161-188)
        const bool bilinear = (desc->mContractionOpId & 1) != 0;
        const bool cplx     = desc->mContractionOpId >= 2;
        if(desc->mContractionOpId < 0 || desc->mContractionOpId > 3)
            return HIPTENSOR_STATUS_NOT_SUPPORTED;
        auto lA = toI64(desc->mTensorDesc[0].mLengths), sA = toI64(desc->mTensorDesc[0].mStrides);
        auto lB = toI64(desc->mTensorDesc[1].mLengths), sB = toI64(desc->mTensorDesc[1].mStrides);
        // D is described by descriptor 3 and the mode list stored at index 2
        // (hiptensor_contraction.cpp:772-775: modeD is never read)
        auto lD = toI64(desc->mTensorDesc[3].mLengths), sD = toI64(desc->mTensorDesc[3].mStrides);
        const auto& mA = desc->mTensorMode[0];
        const auto& mB = desc->mTensorMode[1];
        const auto& mD = desc->mTensorMode[2];
        if(mA.size() != lA.size() || mB.size() != lB.size() || mD.size() != lD.size() || sA.size() != lA.size()
           || sB.size() != lB.size() || sD.size() != lD.size())
            return HIPTENSOR_STATUS_INVALID_VALUE;
        TensorView A{int(lA.size()), lA.data(), sA.data(), mA.data(), int(desc->mTensorDesc[0].mType)};
        TensorView B{int(lB.size()), lB.data(), sB.data(), mB.data(), int(desc->mTensorDesc[1].mType)};
        TensorView D{int(lD.size()), lD.data(), sD.data(), mD.data(), int(desc->mTensorDesc[3].mType)};
        if(cplx)
            return planComplexContraction(A, B, D, int(desc->mTensorDesc[2].mType), bilinear, int(desc->mComputeType),
                                          smCount, out);
        return planContraction(A, B, D, int(desc->mTensorDesc[2].mType), bilinear, int(desc->mComputeType), smCount,
                               out, workspaceLimit);
    }
} // namespace

// ---------------------------------------------------------------------------- core
hiptensorStatus_t hiptensorCreate(hiptensorHandle_t** handle)
{
    HTB_LOG_API("hiptensorCreate", "handle=%p", (void*)handle);
    if(handle == nullptr)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    *handle = nullptr;
    int dev = -1;
    if(cudaGetDevice(&dev) != cudaSuccess)
    {
        cudaGetLastError();
        HTB_LOG_ERROR("hiptensorCreate", "Initialization error: no CUDA device (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_HIP_ERROR));
        return HIPTENSOR_STATUS_HIP_ERROR;
    }
    int major = 0, minor = 0, sms = 0, smem = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if(major != 10)
    {
        // the kernels are built for sm_100a only (the reference exits the process on an
        // unsupported GPU, library/src/hip_device.cpp:130-148; this returns a status)
        HTB_LOG_ERROR("hiptensorCreate", "Unsupported device: compute capability %d.%d, need 10.x (%s)", major,
                      minor, hiptensorGetErrorString(HIPTENSOR_STATUS_ARCH_MISMATCH));
        return HIPTENSOR_STATUS_ARCH_MISMATCH;
    }
    auto* h = new(std::nothrow) hiptensorHandle_t;
    if(h == nullptr)
        return HIPTENSOR_STATUS_ALLOC_FAILED;
    std::memset(h->fields, 0, sizeof(h->fields));
    HandleState* st  = mutableState(h);
    st->device       = dev;
    st->smCount      = sms;
    st->ccMajor      = major;
    st->ccMinor      = minor;
    st->maxSmemOptin = smem;
    // The status word lives in pinned host memory mapped into the device: a kernel that gives up a bounded wait
    // writes it, the next call on the handle reads it without synchronising.
    void* hostWord = nullptr;
    if(cudaHostAlloc(&hostWord, 256, cudaHostAllocMapped) != cudaSuccess
       || cudaHostGetDevicePointer((void**)&st->deviceStatus, hostWord, 0) != cudaSuccess)
    {
        cudaGetLastError();
        if(hostWord)
            cudaFreeHost(hostWord);
        delete h;
        return HIPTENSOR_STATUS_ALLOC_FAILED;
    }
    std::memset(hostWord, 0, 256);
    st->hostStatus = static_cast<volatile int*>(hostWord);
    st->magic = kHandleMagic;
    *handle   = h;
    return HIPTENSOR_STATUS_SUCCESS;
}

hiptensorStatus_t hiptensorDestroy(hiptensorHandle_t* handle)
{
    HTB_LOG_API("hiptensorDestroy", "handle=%p", (void*)handle);
    if(handle == nullptr)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    HandleState* st = mutableState(handle);
    if(st->magic == kHandleMagic)
    {
        if(st->hostStatus)
            cudaFreeHost(const_cast<int*>(st->hostStatus));
        st->magic = 0;
    }
    delete handle;
    return HIPTENSOR_STATUS_SUCCESS;
}

const char* hiptensorGetErrorString(const hiptensorStatus_t error)
{
    switch(error)
    {
    case HIPTENSOR_STATUS_SUCCESS: return "HIPTENSOR_STATUS_SUCCESS";
    case HIPTENSOR_STATUS_NOT_INITIALIZED: return "HIPTENSOR_STATUS_NOT_INITIALIZED";
    case HIPTENSOR_STATUS_ALLOC_FAILED: return "HIPTENSOR_STATUS_ALLOC_FAILED";
    case HIPTENSOR_STATUS_INVALID_VALUE: return "HIPTENSOR_STATUS_INVALID_VALUE";
    case HIPTENSOR_STATUS_ARCH_MISMATCH: return "HIPTENSOR_STATUS_ARCH_MISMATCH";
    case HIPTENSOR_STATUS_EXECUTION_FAILED: return "HIPTENSOR_STATUS_EXECUTION_FAILED";
    case HIPTENSOR_STATUS_INTERNAL_ERROR: return "HIPTENSOR_STATUS_INTERNAL_ERROR";
    case HIPTENSOR_STATUS_NOT_SUPPORTED: return "HIPTENSOR_STATUS_NOT_SUPPORTED";
    case HIPTENSOR_STATUS_CK_ERROR: return "HIPTENSOR_STATUS_CK_ERROR";
    case HIPTENSOR_STATUS_HIP_ERROR: return "HIPTENSOR_STATUS_HIP_ERROR";
    case HIPTENSOR_STATUS_INSUFFICIENT_WORKSPACE: return "HIPTENSOR_STATUS_INSUFFICIENT_WORKSPACE";
    case HIPTENSOR_STATUS_INSUFFICIENT_DRIVER: return "HIPTENSOR_STATUS_INSUFFICIENT_DRIVER";
    case HIPTENSOR_STATUS_IO_ERROR: return "HIPTENSOR_STATUS_IO_ERROR";
    }
    return "HIPTENSOR_STATUS_UNKNOWN";
}

hiptensorStatus_t hiptensorInitTensorDescriptor(const hiptensorHandle_t* handle, hiptensorTensorDescriptor_t* desc,
                                                const uint32_t numModes, const int64_t lens[],
                                                const int64_t strides[], hipDataType dataType,
                                                hiptensorOperator_t unaryOp)
{
    HTB_LOG_API("hiptensorInitTensorDescriptor", "handle=%p, desc=%p, numModes=%u, lens=%p, strides=%p, dataType=%d, unaryOp=%d",
                (const void*)handle, (void*)desc, numModes, (const void*)lens, (const void*)strides, int(dataType),
                int(unaryOp));
    if(handle == nullptr || desc == nullptr)
    {
        HTB_LOG_ERROR("hiptensorInitTensorDescriptor", "Initialization Error : %s = nullptr (%s)",
                      handle ? "descriptor" : "handle", hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_INITIALIZED));
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    }
    const bool typeOk = dataType == HIP_R_16F || dataType == HIP_R_16BF || dataType == HIP_R_32F
                        || dataType == HIP_R_64F || dataType == HIP_C_32F || dataType == HIP_C_64F;
    const bool opOk = unaryOp == HIPTENSOR_OP_IDENTITY || unaryOp == HIPTENSOR_OP_SQRT;
    if((lens == nullptr && strides != nullptr) || !typeOk || !opOk || (lens == nullptr && numModes > 0))
    {
        HTB_LOG_ERROR("hiptensorInitTensorDescriptor", "Tensor Initialization Error : bad lens/strides, data type or operator (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_INVALID_VALUE));
        return HIPTENSOR_STATUS_INVALID_VALUE;
    }
    desc->mType    = dataType;
    desc->mUnaryOp = unaryOp;
    desc->mLengths.assign(lens, lens + numModes);
    if(strides)
    {
        desc->mStrides.assign(strides, strides + numModes);
    }
    else
    {
        // packed with the LAST mode fastest (library/src/hiptensor.cpp:205,
        // library/src/include/util.hpp:45-69 with col_major = false)
        desc->mStrides.assign(numModes, 1);
        for(int i = int(numModes) - 2; i >= 0; i--)
            desc->mStrides[i] = desc->mStrides[i + 1] * desc->mLengths[i + 1];
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

hiptensorStatus_t hiptensorGetAlignmentRequirement(const hiptensorHandle_t* handle, const void* ptr,
                                                   const hiptensorTensorDescriptor_t* desc,
                                                   uint32_t*                          alignmentRequirement)
{
    if(!handle || !desc)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    if(!alignmentRequirement)
        return HIPTENSOR_STATUS_INVALID_VALUE;
    // largest power of two in [element size, 16] that divides the pointer
    *alignmentRequirement = 0u;
    for(uint32_t i = uint32_t(dtypeSize(desc->mType)); i > 0 && i <= 16u; i *= 2)
        if(std::size_t(ptr) % std::size_t(i) == 0)
            *alignmentRequirement = i;
    if(*alignmentRequirement == 0)
    {
        HTB_LOG_ERROR("hiptensorGetAlignmentRequirement", "Error : alignment requirement is 0 (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_INVALID_VALUE));
        return HIPTENSOR_STATUS_INVALID_VALUE;
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------- permutation
hiptensorStatus_t hiptensorPermutation(const hiptensorHandle_t* handle, const void* alpha, const void* A,
                                       const hiptensorTensorDescriptor_t* descA, const int32_t modeA[], void* B,
                                       const hiptensorTensorDescriptor_t* descB, const int32_t modeB[],
                                       const hipDataType typeScalar, const hipStream_t stream)
{
    const char* fn = "hiptensorPermutation";
    HTB_LOG_API(fn, "handle=%p, alpha=%p, A=%p, descA=%p, modeA=%p, B=%p, descB=%p, modeB=%p, typeScalar=%d, stream=%p",
                (const void*)handle, alpha, A, (const void*)descA, (const void*)modeA, B, (const void*)descB,
                (const void*)modeB, int(typeScalar), (void*)stream);
    if(!handle || !alpha || !A || !descA || !modeA || !B || !descB || !modeB)
    {
        HTB_LOG_ERROR(fn, "Initialization Error : a required argument is nullptr (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_INITIALIZED));
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    }
    const HandleState* st = stateOf(handle);
    if(!st)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    if(descA->mType != HIP_R_16F && descA->mType != HIP_R_32F)
    {
        HTB_LOG_ERROR(fn, "Unsupported Data Type Error : The supported data types of A are f16 and f32 (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_SUPPORTED));
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    }
    if(typeScalar != HIP_R_16F && typeScalar != HIP_R_32F)
    {
        HTB_LOG_ERROR(fn, "Unsupported Data Type Error : The supported scalar types are f16 and f32 (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_SUPPORTED));
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    }
    if(descA->mLengths.size() != descB->mLengths.size())
        return HIPTENSOR_STATUS_INVALID_VALUE;
    if(auto s = checkDevice(fn, st); s != HIPTENSOR_STATUS_SUCCESS)
        return s;

    const int rank = int(descA->mLengths.size());
    auto      lA   = toI64(descA->mLengths);
    // B's extents must be A's extents under the mode mapping
    for(int i = 0; i < rank; i++)
    {
        int ia = -1;
        for(int j = 0; j < rank; j++)
            if(modeA[j] == modeB[i])
                ia = j;
        if(ia < 0 || descB->mLengths[i] != descA->mLengths[ia])
        {
            HTB_LOG_ERROR(fn, "Invalid Value Error : extents of B do not match the permuted extents of A (%s)",
                          hiptensorGetErrorString(HIPTENSOR_STATUS_INVALID_VALUE));
            return HIPTENSOR_STATUS_INVALID_VALUE;
        }
    }
    PermPlan   plan;
    const bool aligned = ((uintptr_t(A) | uintptr_t(B)) & 15) == 0;
    int        rc = planPermutation(rank, lA.data(), modeA, modeB, int(descA->mType), int(descB->mType), aligned, &plan);
    if(rc != PLAN_OK)
    {
        HTB_LOG_ERROR(fn, "The permutation cannot be planned (%s)", hiptensorGetErrorString(hiptensorStatus_t(rc)));
        return hiptensorStatus_t(rc);
    }
    // alpha is read as typeScalar and widened to float (permutation_solution_impl.hpp:104-108)
    float alphaF = (typeScalar == HIP_R_32F) ? *(const float*)alpha : __half2float(*(const __half*)alpha);
    HTB_LOG_HEUR(fn, "%s", describe(plan).c_str());
    cudaError_t e = launchPermutation(plan, int(descA->mType), int(descB->mType), A, B, alphaF, int(descA->mUnaryOp),
                                      int(descB->mUnaryOp), st->smCount, st->deviceStatus, stream);
    if(e != cudaSuccess)
    {
        HTB_LOG_ERROR(fn, "kernel launch failed: %s (%s)", cudaGetErrorString(e),
                      hiptensorGetErrorString(HIPTENSOR_STATUS_HIP_ERROR));
        return HIPTENSOR_STATUS_HIP_ERROR;
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------- reduction
namespace
{
    hiptensorStatus_t checkReduction(const char* fn, const hiptensorHandle_t* handle, const void* alpha, const void* A,
                                     const hiptensorTensorDescriptor_t* descA, const int32_t* modeA, const void* beta,
                                     const hiptensorTensorDescriptor_t* descC, const int32_t* modeC, const void* D,
                                     const hiptensorTensorDescriptor_t* descD, hiptensorComputeType_t typeCompute)
    {
        if(!handle || !alpha || !A || !descA || !modeA || !beta || !descC || !D || !descD)
        {
            HTB_LOG_ERROR(fn, "Initialization Error : a required argument is nullptr (%s)",
                          hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_INITIALIZED));
            return HIPTENSOR_STATUS_NOT_INITIALIZED;
        }
        // the six legal (A, C, D, compute) tuples (hiptensor_reduction.cpp:132-139)
        const auto tA = descA->mType, tC = descC->mType, tD = descD->mType;
        bool       ok = (tA == tC && tA == tD)
                  && ((tA == HIP_R_16F && (typeCompute == HIPTENSOR_COMPUTE_16F || typeCompute == HIPTENSOR_COMPUTE_32F))
                      || (tA == HIP_R_16BF
                          && (typeCompute == HIPTENSOR_COMPUTE_16BF || typeCompute == HIPTENSOR_COMPUTE_32F))
                      || (tA == HIP_R_32F && typeCompute == HIPTENSOR_COMPUTE_32F)
                      || (tA == HIP_R_64F && typeCompute == HIPTENSOR_COMPUTE_64F));
        if(!ok)
        {
            HTB_LOG_ERROR(fn,
                          "Unsupported Data Type Error : The combination of data types of A, C and D and compute type "
                          "is not supported. (%s)",
                          hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_SUPPORTED));
            return HIPTENSOR_STATUS_NOT_SUPPORTED;
        }
        const std::size_t rankC = descC->mLengths.size();
        bool same = descC->mType == descD->mType && descC->mLengths == descD->mLengths
                    && descC->mStrides == descD->mStrides && descC->mUnaryOp == descD->mUnaryOp;
        bool subset = (rankC == 0) || (modeC != nullptr);
        if(subset)
        {
            std::set<int32_t> setA(modeA, modeA + descA->mLengths.size());
            for(std::size_t i = 0; i < rankC; i++)
                if(!setA.count(modeC[i]))
                    subset = false;
        }
        if(descA->mLengths.size() < rankC || !same || !subset)
        {
            HTB_LOG_ERROR(fn,
                          "Unsupported Data Error : The descriptor of C and D should be same and modes of C should be "
                          "subset of modes A. (%s)",
                          hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_SUPPORTED));
            return HIPTENSOR_STATUS_NOT_SUPPORTED;
        }
        return HIPTENSOR_STATUS_SUCCESS;
    }

    int planFor(const HandleState* st, const void* A, const hiptensorTensorDescriptor_t* descA, const int32_t* modeA,
                const void* C, const void* D, const hiptensorTensorDescriptor_t* descD, const int32_t* modeD,
                ReducePlan* plan)
    {
        auto       lA = toI64(descA->mLengths), sA = toI64(descA->mStrides);
        auto       lD = toI64(descD->mLengths), sD = toI64(descD->mStrides);
        const bool aligned = ((uintptr_t(A) | uintptr_t(C) | uintptr_t(D)) & 15) == 0;
        return planReduction(int(lA.size()), lA.data(), sA.data(), modeA, int(lD.size()), lD.data(), sD.data(), modeD,
                             dtypeSize(descA->mType), aligned, st ? st->smCount : 148, plan);
    }
} // namespace

hiptensorStatus_t hiptensorReduction(const hiptensorHandle_t* handle, const void* alpha, const void* A,
                                     const hiptensorTensorDescriptor_t* descA, const int32_t modeA[],
                                     const void* beta, const void* C, const hiptensorTensorDescriptor_t* descC,
                                     const int32_t modeC[], void* D, const hiptensorTensorDescriptor_t* descD,
                                     const int32_t modeD[], hiptensorOperator_t opReduce,
                                     hiptensorComputeType_t typeCompute, void* workspace, uint64_t workspaceSize,
                                     hipStream_t stream)
{
    const char* fn = "hiptensorReduction";
    HTB_LOG_API(fn, "handle=%p, alpha=%p, A=%p, descA=%p, beta=%p, C=%p, descC=%p, D=%p, descD=%p, opReduce=%d, typeCompute=%d, workspace=%p, workspaceSize=%llu, stream=%p",
                (const void*)handle, alpha, A, (const void*)descA, beta, C, (const void*)descC, D, (const void*)descD,
                int(opReduce), int(typeCompute), workspace, (unsigned long long)workspaceSize, (void*)stream);
    if(auto s = checkReduction(fn, handle, alpha, A, descA, modeA, beta, descC, modeC, D, descD, typeCompute);
       s != HIPTENSOR_STATUS_SUCCESS)
        return s;
    const HandleState* st = stateOf(handle);
    if(!st)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    if(opReduce != HIPTENSOR_OP_ADD && opReduce != HIPTENSOR_OP_MUL && opReduce != HIPTENSOR_OP_MIN
       && opReduce != HIPTENSOR_OP_MAX)
    {
        HTB_LOG_ERROR(fn, "Internal Error : no kernel for this reduction operator (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_INTERNAL_ERROR));
        return HIPTENSOR_STATUS_INTERNAL_ERROR; // the reference finds no instance (hiptensor_reduction.cpp:276-285)
    }
    if(auto s = checkDevice(fn, st); s != HIPTENSOR_STATUS_SUCCESS)
        return s;
    ReducePlan plan;
    // the reference hands D's descriptor with modeD to its kernels (hiptensor_reduction.cpp:325-336);
    // modeD == modeC by contract, and a null modeD falls back to modeC
    const int32_t* modesOut = modeD ? modeD : modeC;
    int            rc       = planFor(st, A, descA, modeA, C, D, descD, modesOut, &plan);
    if(rc != PLAN_OK)
    {
        HTB_LOG_ERROR(fn, "No kernel is able to solve the problem (%s)", hiptensorGetErrorString(hiptensorStatus_t(rc)));
        return hiptensorStatus_t(rc);
    }
    // alpha/beta: read as the given compute type, widened to double (hiptensor_reduction.cpp:287-296)
    double alphaD = 0, betaD = 0;
    if(!readScalar(alpha, int(typeCompute), &alphaD) || !readScalar(beta, int(typeCompute), &betaD))
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    // f16/bf16 compute is promoted to f32 (hiptensor_reduction.cpp:259-264)
    const int internalCompute = (typeCompute == HIPTENSOR_COMPUTE_64F) ? HIPTENSOR_COMPUTE_64F : HIPTENSOR_COMPUTE_32F;
    // the two-pass form needs scratch; without enough of it the single-pass kernels run
    const uint64_t need = reductionWorkspaceBytes(plan, internalCompute);
    void*          ws   = (need > 0 && workspace != nullptr && workspaceSize >= need) ? workspace : nullptr;
    if(ws == nullptr)
        plan.split = 1;
    HTB_LOG_HEUR(fn, "%s", describe(plan).c_str());
    // The reference copies C over D and then accumulates in place (hiptensor_reduction.cpp:298-307);
    // reading C at D's offsets inside the kernel gives the same result without the extra pass.
    cudaError_t e = launchReduction(plan, int(descA->mType), internalCompute, int(opReduce), alphaD, A, betaD,
                                    C ? C : D, D, ws, stream);
    if(e != cudaSuccess)
    {
        HTB_LOG_ERROR(fn, "kernel launch failed: %s (%s)", cudaGetErrorString(e),
                      hiptensorGetErrorString(HIPTENSOR_STATUS_HIP_ERROR));
        return HIPTENSOR_STATUS_HIP_ERROR;
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

hiptensorStatus_t hiptensorReductionGetWorkspaceSize(
    const hiptensorHandle_t* handle, const void* A, const hiptensorTensorDescriptor_t* descA, const int32_t modeA[],
    const void* C, const hiptensorTensorDescriptor_t* descC, const int32_t modeC[], const void* D,
    const hiptensorTensorDescriptor_t* descD, const int32_t modeD[], hiptensorOperator_t opReduce,
    hiptensorComputeType_t typeCompute, uint64_t* workspaceSize)
{
    (void)opReduce;
    (void)descC;
    if(!handle)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    if(!workspaceSize || !descA || !descD || !modeA)
        return HIPTENSOR_STATUS_INVALID_VALUE;
    *workspaceSize = 0; // the reference always reports 0 (hiptensor_reduction.cpp:383-399)
    ReducePlan plan;
    if(planFor(stateOf(handle), A, descA, modeA, C, D, descD, modeD ? modeD : modeC, &plan) == PLAN_OK)
    {
        const int internalCompute
            = (typeCompute == HIPTENSOR_COMPUTE_64F) ? HIPTENSOR_COMPUTE_64F : HIPTENSOR_COMPUTE_32F;
        *workspaceSize = reductionWorkspaceBytes(plan, internalCompute);
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------- allocation-free reduction
// Body of htReductionNoAlloc (include/hiptensor_b200.h). Same operation and argument meaning as hiptensorReduction,
// for callers that must not trigger any allocation while they run: real-time loops (cudaMalloc
// synchronises the device), plug-ins of hosts that own the whole device heap (cudaMalloc fails),
// and services that forbid device allocations after start-up.
// The two-pass scratch comes from a fixed array inside the library (htb::kStaticScratchBytes per
// device, resident for the life of the process); no cudaMalloc, cudaFree or allocating routine
// is called, and the host side (descriptor reading, planning) works on stack arrays only.
int htb::reductionNoAlloc(const hiptensorHandle_t* handle, const void* alpha, const void* A,
                          const hiptensorTensorDescriptor_t* descA, const int32_t* modeA, const void* beta,
                          const void* C, const hiptensorTensorDescriptor_t* descC, const int32_t* modeC, void* D,
                          const hiptensorTensorDescriptor_t* descD, const int32_t* modeD, int opReduce,
                          int typeComputeI, void* stream)
{
    const char* fn = "htReductionNoAlloc";
    const auto typeCompute = hiptensorComputeType_t(typeComputeI);
    if(!handle || !alpha || !A || !descA || !modeA || !beta || !descC || !D || !descD)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    const HandleState* st = stateOf(handle);
    if(!st)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    const auto tA = descA->mType;
    const bool typesOk
        = (tA == descC->mType && tA == descD->mType)
          && ((tA == HIP_R_16F && (typeCompute == HIPTENSOR_COMPUTE_16F || typeCompute == HIPTENSOR_COMPUTE_32F))
              || (tA == HIP_R_16BF && (typeCompute == HIPTENSOR_COMPUTE_16BF || typeCompute == HIPTENSOR_COMPUTE_32F))
              || (tA == HIP_R_32F && typeCompute == HIPTENSOR_COMPUTE_32F)
              || (tA == HIP_R_64F && typeCompute == HIPTENSOR_COMPUTE_64F));
    if(!typesOk)
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    const int rankA = int(descA->mLengths.size()), rankD = int(descD->mLengths.size());
    if(rankA < 1 || rankA > kMaxGroup || rankD > rankA || descC->mLengths != descD->mLengths
       || descC->mStrides != descD->mStrides || (rankD > 0 && !modeD && !modeC))
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    if(opReduce != HIPTENSOR_OP_ADD && opReduce != HIPTENSOR_OP_MUL && opReduce != HIPTENSOR_OP_MIN
       && opReduce != HIPTENSOR_OP_MAX)
        return HIPTENSOR_STATUS_INTERNAL_ERROR;
    if(auto s = checkDevice(fn, st); s != HIPTENSOR_STATUS_SUCCESS)
        return s;
    int64_t lA[kMaxGroup], sA[kMaxGroup], lD[kMaxGroup], sD[kMaxGroup];
    for(int i = 0; i < rankA; i++)
    {
        lA[i] = int64_t(descA->mLengths[i]);
        sA[i] = int64_t(descA->mStrides[i]);
    }
    for(int i = 0; i < rankD; i++)
    {
        lD[i] = int64_t(descD->mLengths[i]);
        sD[i] = int64_t(descD->mStrides[i]);
    }
    ReducePlan plan;
    const bool aligned = ((uintptr_t(A) | uintptr_t(C) | uintptr_t(D)) & 15) == 0;
    int rc = planReduction(rankA, lA, sA, modeA, rankD, lD, sD, modeD ? modeD : modeC, dtypeSize(tA), aligned,
                           st->smCount, &plan);
    if(rc != PLAN_OK)
        return rc;
    const int internalCompute = (typeCompute == HIPTENSOR_COMPUTE_64F) ? HIPTENSOR_COMPUTE_64F : HIPTENSOR_COMPUTE_32F;
    uint64_t need = reductionWorkspaceBytes(plan, internalCompute);
    if(need > kStaticScratchBytes && (plan.splitOptional || plan.kind == RED_COL || plan.shortLanes > 0))
    {
        // these plans are sliced by thread or block count, with many more slices than the built-in scratch holds: as
        // many slices as fit, or one pass
        const uint64_t acc = (internalCompute == HIPTENSOR_COMPUTE_64F) ? 8 : 4;
        const uint64_t fit = kStaticScratchBytes / (uint64_t(plan.nOut) * acc);
        plan.split         = fit >= 2 ? int(std::min<uint64_t>(fit, uint64_t(plan.split))) : 1;
        need               = reductionWorkspaceBytes(plan, internalCompute);
    }
    if(need > kStaticScratchBytes)
    {
        HTB_LOG_ERROR(fn, "this reduction needs %llu bytes of scratch, the built-in scratch holds %llu: use "
                          "hiptensorReduction with a caller workspace (%s)",
                      (unsigned long long)need, (unsigned long long)kStaticScratchBytes,
                      hiptensorGetErrorString(HIPTENSOR_STATUS_INSUFFICIENT_WORKSPACE));
        return HIPTENSOR_STATUS_INSUFFICIENT_WORKSPACE;
    }
    double alphaD = 0, betaD = 0;
    if(!readScalar(alpha, int(typeCompute), &alphaD) || !readScalar(beta, int(typeCompute), &betaD))
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    cudaError_t e = launchReductionStaticScratch(plan, int(tA), internalCompute, opReduce, alphaD, A, betaD, C ? C : D,
                                                 D, st->device, cudaStream_t(stream));
    if(e != cudaSuccess)
    {
        HTB_LOG_ERROR(fn, "launch failed: %s (%s)", cudaGetErrorString(e),
                      hiptensorGetErrorString(HIPTENSOR_STATUS_HIP_ERROR));
        return HIPTENSOR_STATUS_HIP_ERROR;
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------- reduction split over devices
// Body of htReductionFinish (include/hiptensor_b200.h). The reference binds a handle to one device and has no
// multi-device path; when a REDUCED mode is split over several devices, each device calls hiptensorReduction
// on its share with alpha = 1 and beta = 0, the partial results are combined with one all-reduce that uses
// the reduction's operator, and this call applies alpha and beta * C once, in the order of the reference's
// epilogue (library/src/reduction/reduction_cpu_reference_impl.hpp:45-64).
int htb::reductionFinish(const hiptensorHandle_t* handle, const void* alpha, const void* partial, const void* beta,
                         const void* C, void* D, const hiptensorTensorDescriptor_t* descD, int typeComputeI,
                         void* stream)
{
    const char* fn = "htReductionFinish";
    if(!handle || !alpha || !beta || !partial || !D || !descD)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    const HandleState* st = stateOf(handle);
    if(!st)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    const auto typeCompute = hiptensorComputeType_t(typeComputeI);
    const auto tD          = descD->mType;
    const bool typesOk
        = (tD == HIP_R_16F && (typeCompute == HIPTENSOR_COMPUTE_16F || typeCompute == HIPTENSOR_COMPUTE_32F))
          || (tD == HIP_R_16BF && (typeCompute == HIPTENSOR_COMPUTE_16BF || typeCompute == HIPTENSOR_COMPUTE_32F))
          || (tD == HIP_R_32F && typeCompute == HIPTENSOR_COMPUTE_32F)
          || (tD == HIP_R_64F && typeCompute == HIPTENSOR_COMPUTE_64F);
    if(!typesOk || descD->mLengths.size() > std::size_t(kMaxGroup))
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    if(auto s = checkDevice(fn, st); s != HIPTENSOR_STATUS_SUCCESS)
        return s;
    double alphaD = 0, betaD = 0;
    if(!readScalar(alpha, typeComputeI, &alphaD) || !readScalar(beta, typeComputeI, &betaD))
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    int64_t   lens[kMaxGroup], strides[kMaxGroup];
    const int rank = int(descD->mLengths.size());
    for(int i = 0; i < rank; i++)
    {
        lens[i]    = int64_t(descD->mLengths[i]);
        strides[i] = int64_t(descD->mStrides[i]);
    }
    cudaError_t e = launchReductionFinish(int(tD), alphaD, partial, betaD, C, D, rank, lens, strides, cudaStream_t(stream));
    if(e != cudaSuccess)
    {
        HTB_LOG_ERROR(fn, "launch failed: %s (%s)", cudaGetErrorString(e), hiptensorGetErrorString(HIPTENSOR_STATUS_HIP_ERROR));
        return HIPTENSOR_STATUS_HIP_ERROR;
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------- contraction
hiptensorStatus_t hiptensorInitContractionDescriptor(
    const hiptensorHandle_t* handle, hiptensorContractionDescriptor_t* desc,
    const hiptensorTensorDescriptor_t* descA, const int32_t modeA[], const uint32_t alignmentRequirementA,
    const hiptensorTensorDescriptor_t* descB, const int32_t modeB[], const uint32_t alignmentRequirementB,
    const hiptensorTensorDescriptor_t* descC, const int32_t modeC[], const uint32_t alignmentRequirementC,
    const hiptensorTensorDescriptor_t* descD, const int32_t modeD[], const uint32_t alignmentRequirementD,
    hiptensorComputeType_t typeCompute)
{
    const char* fn = "hiptensorInitContractionDescriptor";
    HTB_LOG_API(fn, "handle=%p, desc=%p, descA=%p, descB=%p, descC=%p, descD=%p, typeCompute=%d", (const void*)handle,
                (void*)desc, (const void*)descA, (const void*)descB, (const void*)descC, (const void*)descD,
                int(typeCompute));
    if(!handle || !desc || !descA || !descB || !descD)
    {
        HTB_LOG_ERROR(fn, "Initialization Error : %s = nullptr (%s)",
                      !handle ? "handle" : (!desc ? "contraction descriptor" : "Tensor descriptors"),
                      hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_INITIALIZED));
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    }
    if(!modeA || !modeB || !modeD)
        return HIPTENSOR_STATUS_INVALID_VALUE;
    if(descA->mUnaryOp != HIPTENSOR_OP_IDENTITY || descB->mUnaryOp != HIPTENSOR_OP_IDENTITY
       || descD->mUnaryOp != HIPTENSOR_OP_IDENTITY || (descC && descC->mUnaryOp != HIPTENSOR_OP_IDENTITY))
    {
        HTB_LOG_ERROR(fn, "Unsupported Operator Type Error : The supported Operator is HIPTENSOR_OP_IDENTITY (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_SUPPORTED));
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    }
    const bool complexCompute = typeCompute == HIPTENSOR_COMPUTE_C32F || typeCompute == HIPTENSOR_COMPUTE_C64F;
    std::vector<int32_t> mA(modeA, modeA + descA->mLengths.size());
    std::vector<int32_t> mB(modeB, modeB + descB->mLengths.size());
    std::vector<int32_t> mD(modeD, modeD + descD->mLengths.size());
    desc->mComputeType = typeCompute;
    if(descC == nullptr || modeC == nullptr)
    {
        // scale form: the C slot holds a typeless placeholder, mode list 2 is D's
        desc->mContractionOpId = complexCompute ? 2 : 0;
        hiptensorTensorDescriptor_t none{hipDataType(31), std::vector<std::size_t>(descD->mLengths.size(), 0),
                                         std::vector<std::size_t>(descD->mStrides.size(), 0), HIPTENSOR_OP_IDENTITY};
        desc->mTensorDesc   = {*descA, *descB, none, *descD};
        desc->mAlignmentReq = {alignmentRequirementA, alignmentRequirementB, 0, alignmentRequirementD};
        desc->mTensorMode   = {mA, mB, mD};
    }
    else
    {
        desc->mContractionOpId = complexCompute ? 3 : 1;
        std::vector<int32_t> mC(modeC, modeC + descC->mLengths.size());
        desc->mTensorDesc   = {*descA, *descB, *descC, *descD};
        desc->mAlignmentReq = {alignmentRequirementA, alignmentRequirementB, alignmentRequirementC,
                               alignmentRequirementD};
        desc->mTensorMode   = {mA, mB, mC, mD};
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

hiptensorStatus_t hiptensorInitContractionFind(const hiptensorHandle_t* handle, hiptensorContractionFind_t* find,
                                               const hiptensorAlgo_t algo)
{
    const char* fn = "hiptensorInitContractionFind";
    HTB_LOG_API(fn, "handle=%p, find=%p, algo=%d", (const void*)handle, (void*)find, int(algo));
    if(!handle || !find)
    {
        HTB_LOG_ERROR(fn, "Initialization Error : %s = nullptr (%s)", handle ? "contraction find" : "handle",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_INITIALIZED));
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    }
    const HandleState* st = stateOf(handle);
    if(!st)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    if(auto s = checkDevice(fn, st); s != HIPTENSOR_STATUS_SUCCESS)
        return s;
    if(algo != HIPTENSOR_ALGO_DEFAULT && algo != HIPTENSOR_ALGO_DEFAULT_PATIENT && algo != HIPTENSOR_ALGO_ACTOR_CRITIC)
        return HIPTENSOR_STATUS_INVALID_VALUE;
    // Every algorithm id selects the same closed-form planner: there is no instance list
    // to enumerate, so the candidate vector stays empty.
    find->mSelectionAlgorithm = algo;
    find->mCandidates.clear();
    return HIPTENSOR_STATUS_SUCCESS;
}

hiptensorStatus_t hiptensorContractionGetWorkspaceSize(const hiptensorHandle_t*                handle,
                                                       const hiptensorContractionDescriptor_t* desc,
                                                       const hiptensorContractionFind_t*       find,
                                                       const hiptensorWorksizePreference_t     pref,
                                                       uint64_t*                               workspaceSize)
{
    if(!handle || !desc || !find || !workspaceSize)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    *workspaceSize = 0;
    ContractionPlan    plan;
    const HandleState* st = stateOf(handle);
    // every real kernel runs without scratch (WORKSPACE_MIN = 0); the recommended size lets the
    // tensor-core kernels split tiles along K. Complex contractions need room for the expanded copy
    // of their smaller operand at every preference.
    // (Operands that the tensor-core kernels cannot read in place are copied into the workspace when there is one:
    // the recommended size has room for the copies, the minimum stays 0 and leaves such problems on the FMA kernel.)
    if(buildContractionPlan(desc, st ? st->smCount : 148, &plan, pref != HIPTENSOR_WORKSPACE_MIN ? ~uint64_t(0) : 0)
       == HIPTENSOR_STATUS_SUCCESS)
        *workspaceSize = plan.expandBytes + (pref != HIPTENSOR_WORKSPACE_MIN ? plan.workspaceBytes : 0);
    return HIPTENSOR_STATUS_SUCCESS;
}

hiptensorStatus_t hiptensorInitContractionPlan(const hiptensorHandle_t* handle, hiptensorContractionPlan_t* plan,
                                               const hiptensorContractionDescriptor_t* desc,
                                               const hiptensorContractionFind_t* find, const uint64_t workspaceSize)
{
    const char* fn = "hiptensorInitContractionPlan";
    HTB_LOG_API(fn, "handle=%p, plan=%p, desc=%p, find=%p, workspaceSize=%llu", (const void*)handle, (void*)plan,
                (const void*)desc, (const void*)find, (unsigned long long)workspaceSize);
    if(!handle || !plan || !desc || !find)
    {
        HTB_LOG_ERROR(fn, "Initialization Error : %s = nullptr (%s)",
                      !handle ? "handle" : (!plan ? "plan" : (!desc ? "contraction descriptor" : "contraction find")),
                      hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_INITIALIZED));
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    }
    const HandleState* st = stateOf(handle);
    if(!st)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    if(auto s = checkDevice(fn, st); s != HIPTENSOR_STATUS_SUCCESS)
        return s;
    ContractionPlan cp;
    int             rc = buildContractionPlan(desc, st->smCount, &cp, workspaceSize);
    if(rc != HIPTENSOR_STATUS_SUCCESS)
    {
        // the reference ends with EXECUTION_FAILED when no candidate survives its type
        // query (contraction_selection.cpp:185-190); the cause is reported more precisely here
        HTB_LOG_ERROR(fn, "No kernel can run this contraction (%s)", hiptensorGetErrorString(hiptensorStatus_t(rc)));
        return hiptensorStatus_t(rc);
    }
    if(cp.expandBytes + cp.workspaceBytes > workspaceSize)
        cp.workspaceBytes = 0; // planned for the workspace the caller said it has: no split
    HTB_LOG_HEUR(fn, "%s", describe(cp).c_str());
    plan->mSolution        = const_cast<ContractionPlan*>(registry().intern(cp));
    plan->mContractionDesc = *desc;
    return HIPTENSOR_STATUS_SUCCESS;
}

hiptensorStatus_t hiptensorContraction(const hiptensorHandle_t* handle, const hiptensorContractionPlan_t* plan,
                                       const void* alpha, const void* A, const void* B, const void* beta,
                                       const void* C, void* D, void* workspace, uint64_t workspaceSize,
                                       hipStream_t stream)
{
    const char* fn = "hiptensorContraction";
    HTB_LOG_API(fn, "handle=%p, plan=%p, alpha=%p, A=%p, B=%p, beta=%p, C=%p, D=%p, workspace=%p, workspaceSize=%llu, stream=%p",
                (const void*)handle, (const void*)plan, alpha, A, B, beta, C, D, workspace,
                (unsigned long long)workspaceSize, (void*)stream);
    if(!handle || !plan)
    {
        HTB_LOG_ERROR(fn, "Initialization Error : %s = nullptr (%s)", handle ? "plan" : "handle",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_NOT_INITIALIZED));
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    }
    if(!alpha || !A || !B || !D)
    {
        HTB_LOG_ERROR(fn, "Input Parameter Error : %s = nullptr (%s)", alpha ? "A/B/D" : "alpha",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_INVALID_VALUE));
        return HIPTENSOR_STATUS_INVALID_VALUE;
    }
    const HandleState* st = stateOf(handle);
    if(!st)
        return HIPTENSOR_STATUS_NOT_INITIALIZED;
    const ContractionPlan* cp = plan->mSolution ? registry().find(plan->mSolution) : nullptr;
    if(cp == nullptr && plan->mSolution != nullptr)
    {
        // the registry has dropped this plan (more than kCapacity other plans were used since): plan again
        // from the descriptor the caller's plan carries
        ContractionPlan again;
        if(buildContractionPlan(&plan->mContractionDesc, st->smCount, &again, workspaceSize) == HIPTENSOR_STATUS_SUCCESS)
        {
            if(again.expandBytes + again.workspaceBytes > workspaceSize)
                again.workspaceBytes = 0;
            cp = registry().intern(again);
        }
    }
    if(cp == nullptr)
    {
        HTB_LOG_ERROR(fn, "Internal Error : solution = nullptr (%s)",
                      hiptensorGetErrorString(HIPTENSOR_STATUS_INTERNAL_ERROR));
        return HIPTENSOR_STATUS_INTERNAL_ERROR;
    }
    if(auto s = checkDevice(fn, st); s != HIPTENSOR_STATUS_SUCCESS)
        return s;
    const uint64_t needBytes = cp->expandBytes + cp->workspaceBytes;
    if(needBytes > workspaceSize || (needBytes > 0 && workspace == nullptr))
    {
        HTB_LOG_ERROR(fn, "Insufficient workspace: req: %llu alloc: %llu (%s)", (unsigned long long)needBytes,
                      (unsigned long long)workspaceSize,
                      hiptensorGetErrorString(HIPTENSOR_STATUS_INSUFFICIENT_WORKSPACE));
        return HIPTENSOR_STATUS_INSUFFICIENT_WORKSPACE;
    }
    // alpha/beta are typed by the compute type and held as float by the epilogue
    // (contraction_solution_impl.hpp:110-123)
    const bool bilinear = cp->bilinear != 0;
    if(cp->complexKind)
    {
        // alpha / beta point to hipFloatComplex / hipDoubleComplex (data_types.cpp:187-196)
        const bool c32 = cp->typeD == CUDA_R_32F;
        double     al[2], be[2] = {0, 0};
        if(bilinear && (!beta || !C))
        {
            HTB_LOG_ERROR(fn, "Input Parameter Error : beta/C = nullptr for a bilinear contraction (%s)",
                          hiptensorGetErrorString(HIPTENSOR_STATUS_INVALID_VALUE));
            return HIPTENSOR_STATUS_INVALID_VALUE;
        }
        for(int i = 0; i < 2; i++)
        {
            al[i] = c32 ? double(((const float*)alpha)[i]) : ((const double*)alpha)[i];
            if(bilinear)
                be[i] = c32 ? double(((const float*)beta)[i]) : ((const double*)beta)[i];
        }
        cudaError_t e = launchComplexContraction(*cp, al[0], al[1], A, B, be[0], be[1], bilinear ? C : nullptr, D,
                                                 workspace, needBytes, st->smCount, st->deviceStatus, stream);
        if(e != cudaSuccess)
        {
            HTB_LOG_ERROR(fn, "kernel launch failed: %s (%s)", cudaGetErrorString(e),
                          hiptensorGetErrorString(HIPTENSOR_STATUS_HIP_ERROR));
            return HIPTENSOR_STATUS_HIP_ERROR;
        }
        return HIPTENSOR_STATUS_SUCCESS;
    }
    double alphaD = 0, betaD = 0;
    if(!readScalar(alpha, cp->computeType, &alphaD))
        return HIPTENSOR_STATUS_NOT_SUPPORTED;
    if(bilinear)
    {
        if(!beta || !C)
        {
            HTB_LOG_ERROR(fn, "Input Parameter Error : beta/C = nullptr for a bilinear contraction (%s)",
                          hiptensorGetErrorString(HIPTENSOR_STATUS_INVALID_VALUE));
            return HIPTENSOR_STATUS_INVALID_VALUE;
        }
        readScalar(beta, cp->computeType, &betaD);
    }
    // scratch is used only up to what the plan was made for
    cudaError_t e = cp->packReal
                        ? launchPackedContraction(*cp, float(alphaD), A, B, float(betaD), bilinear ? C : nullptr, D, workspace,
                                                  needBytes, st->smCount, st->deviceStatus, stream)
                        : launchContraction(*cp, float(alphaD), A, B, float(betaD), bilinear ? C : nullptr, D,
                                            cp->workspaceBytes ? workspace : nullptr, cp->workspaceBytes, st->smCount,
                                            st->deviceStatus, stream);
    if(e != cudaSuccess)
    {
        HTB_LOG_ERROR(fn, "kernel launch failed: %s (%s)", cudaGetErrorString(e),
                      hiptensorGetErrorString(HIPTENSOR_STATUS_HIP_ERROR));
        return HIPTENSOR_STATUS_HIP_ERROR;
    }
    return HIPTENSOR_STATUS_SUCCESS;
}

// ---------------------------------------------------------------------------- logger, version
hiptensorStatus_t hiptensorLoggerSetCallback(hiptensorLoggerCallback_t callback)
{
    return hiptensorStatus_t(Logger::instance().setCallback(callback));
}
hiptensorStatus_t hiptensorLoggerSetFile(FILE* file)
{
    return hiptensorStatus_t(Logger::instance().setFile(file));
}
hiptensorStatus_t hiptensorLoggerOpenFile(const char* logFile)
{
    return hiptensorStatus_t(Logger::instance().openFile(logFile));
}
hiptensorStatus_t hiptensorLoggerSetLevel(hiptensorLogLevel_t level)
{
    return hiptensorStatus_t(Logger::instance().setLevel(int32_t(level)));
}
hiptensorStatus_t hiptensorLoggerSetMask(int32_t mask)
{
    return hiptensorStatus_t(Logger::instance().setMask(mask));
}
hiptensorStatus_t hiptensorLoggerForceDisable()
{
    Logger::instance().disable();
    return HIPTENSOR_STATUS_SUCCESS;
}
int hiptensorGetHiprtVersion()
{
    int v = -1;
    if(cudaRuntimeGetVersion(&v) != cudaSuccess)
        return -1;
    return v;
}
