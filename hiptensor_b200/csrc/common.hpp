// Shared host-side definitions of libhiptensor_b200: data-type helpers, the state
// kept inside the opaque handle, the logger and the launch bookkeeping.
#pragma once

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <hiptensor/hiptensor_types.hpp>

namespace htb
{
    inline int dtypeSize(int dt)
    {
        switch(dt)
        {
        case CUDA_R_32F: return 4;
        case CUDA_R_64F: return 8;
        case CUDA_R_16F: return 2;
        case CUDA_R_16BF: return 2;
        case CUDA_C_32F: return 8;
        case CUDA_C_64F: return 16;
        default: return 0;
        }
    }

    inline const char* dtypeName(int dt)
    {
        switch(dt)
        {
        case CUDA_R_32F: return "f32";
        case CUDA_R_64F: return "f64";
        case CUDA_R_16F: return "f16";
        case CUDA_R_16BF: return "bf16";
        case CUDA_C_32F: return "cf32";
        case CUDA_C_64F: return "cf64";
        default: return "none";
        }
    }

    // Host scalar -> double. The pointer is typed by the compute type
    // (reference: library/src/data_types.cpp:152-205 readVal).
    inline bool readScalar(const void* p, int computeType, double* out)
    {
        switch(computeType)
        {
        case HIPTENSOR_COMPUTE_32F: *out = double(*(const float*)p); return true;
        case HIPTENSOR_COMPUTE_64F: *out = *(const double*)p; return true;
        case HIPTENSOR_COMPUTE_16F: *out = double(__half2float(*(const __half*)p)); return true;
        case HIPTENSOR_COMPUTE_16BF: *out = double(__bfloat162float(*(const __nv_bfloat16*)p)); return true;
        default: return false;
        }
    }

    // State placed inside hiptensorHandle_t::fields (reference: library/src/handle.cpp:31-48
    // places a Handle{HipDevice} there).
    struct HandleState
    {
        uint64_t magic;
        int      device;
        int      smCount;
        int      ccMajor;
        int      ccMinor;
        int      maxSmemOptin;
        int      reserved;
        int*     deviceStatus; // device address of the status word that kernels raise when a bounded wait runs out
        volatile int* hostStatus; // the same word as the host sees it (pinned, mapped memory)
    };
    constexpr uint64_t kHandleMagic = 0x4854423230300001ull;

    inline const HandleState* stateOf(const hiptensorHandle_t* h)
    {
        auto* s = reinterpret_cast<const HandleState*>(h->fields);
        return s->magic == kHandleMagic ? s : nullptr;
    }

    // ---- logger (subset of library/src/logger.cpp: mask, FILE*/file/callback sinks,
    //      line format "[pid][time][hipTensor][ctx][func] msg") ----
    class Logger
    {
    public:
        static Logger& instance();
        void           log(int32_t context, const char* func, const char* fmt, ...);
        bool           enabled(int32_t context) const
        {
            return !mDisabled && (mMask.load(std::memory_order_relaxed) & context);
        }
        int  setMask(int32_t mask);
        int  setLevel(int32_t level);
        int  setFile(FILE* f);
        int  openFile(const char* name);
        int  setCallback(hiptensorLoggerCallback_t cb);
        void disable()
        {
            mDisabled = true;
        }

    private:
        Logger() = default;
        std::mutex                mMutex;
        std::atomic<int32_t>      mMask{HIPTENSOR_LOG_LEVEL_ERROR};
        bool                      mDisabled = false;
        FILE*                     mFile     = nullptr; // nullptr = stdout
        bool                      mOwnsFile = false;
        hiptensorLoggerCallback_t mCallback = nullptr;
    };

#define HTB_LOG_ERROR(func, ...)                                                      \
    do                                                                                \
    {                                                                                 \
        if(::htb::Logger::instance().enabled(HIPTENSOR_LOG_LEVEL_ERROR))              \
            ::htb::Logger::instance().log(HIPTENSOR_LOG_LEVEL_ERROR, func, __VA_ARGS__); \
    } while(0)
#define HTB_LOG_API(func, ...)                                                            \
    do                                                                                    \
    {                                                                                     \
        if(::htb::Logger::instance().enabled(HIPTENSOR_LOG_LEVEL_API_TRACE))              \
            ::htb::Logger::instance().log(HIPTENSOR_LOG_LEVEL_API_TRACE, func, __VA_ARGS__); \
    } while(0)
#define HTB_LOG_HEUR(func, ...)                                                                  \
    do                                                                                           \
    {                                                                                            \
        if(::htb::Logger::instance().enabled(HIPTENSOR_LOG_LEVEL_HEURISTICS_TRACE))              \
            ::htb::Logger::instance().log(HIPTENSOR_LOG_LEVEL_HEURISTICS_TRACE, func, __VA_ARGS__); \
    } while(0)

    // ---- variant switches ----
    // Environment variables that choose between shipped kernels or variants of them (tests of a
    // variant on problems the planner would give to another one, and measurements). None of them
    // changes a result beyond the order of summation. They are read once when the library is loaded
    // and again on htReloadSwitches(); a launch reads no environment variable.
    // Switches that make a kernel skip part of its work (timing one pipeline role alone) exist only in
    // builds made with -DHTB_MEASURE and are absent from the default build.
    struct Switches
    {
        bool tcSingle, tcPair, tcNoHalf, tcNoSplit, tcNarrow, tcWide, tcKsplit, tcNoTmaStore, tcNoPdl; // f16/bf16 tensor-core kernels
        bool noTf32x3, tf32Pair, tf32NoInplace, tf32NoSplit; // fp32 tensor-core kernel
        bool dmmaNoVec, dmmaNoSplit, f64Compute32Fma; // FP64 tensor-pipe kernel; f64 data with compute f32 on the FMA kernel
        int  tcProbe, tf32Probe; // HTB_MEASURE builds only, else 0
        int  permTile, permStages, permCtas; // HTB_MEASURE builds only, else 0
    };
    const Switches& switches();
    void            reloadSwitches();

    // ---- launch bookkeeping (which kernel family ran; how many launches) ----
    void        noteLaunch(const char* kernelFamily, int launches = 1);
    const char* lastKernelName();
    uint64_t    launchCount();
} // namespace htb
