// Runtime support shared by the API layer and the kernels: logger, launch bookkeeping
// and the driver entry point needed to build TMA tensor maps.
#include <cstdlib>
#include <ctime>
#include <unistd.h>

#include <cuda.h>
#include <cuda_runtime_api.h>

#include "kernels.hpp"

namespace htb
{
    // ------------------------------------------------------------------ logger
    Logger& Logger::instance()
    {
        static Logger inst;
        return inst;
    }

    void Logger::log(int32_t context, const char* func, const char* fmt, ...)
    {
        char    msg[2048];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(msg, sizeof(msg), fmt, ap);
        va_end(ap);

        const char* ctx = "";
        switch(context)
        {
        case HIPTENSOR_LOG_LEVEL_ERROR: ctx = "Error"; break;
        case HIPTENSOR_LOG_LEVEL_PERF_TRACE: ctx = "Performance"; break;
        case HIPTENSOR_LOG_LEVEL_PERF_HINT: ctx = "Performance Hint"; break;
        case HIPTENSOR_LOG_LEVEL_HEURISTICS_TRACE: ctx = "Heuristics"; break;
        case HIPTENSOR_LOG_LEVEL_API_TRACE: ctx = "API"; break;
        }
        std::lock_guard<std::mutex> lock(mMutex);
        if(mCallback)
        {
            mCallback(context, func, msg);
            return;
        }
        char       stamp[32];
        time_t     now = time(nullptr);
        struct tm  tmv;
        localtime_r(&now, &tmv);
        strftime(stamp, sizeof(stamp), "%Y-%m-%d %H:%M:%S", &tmv);
        FILE* f = mFile ? mFile : stdout;
        fprintf(f, "[%d][%s][hipTensor][%s][%s] %s\n", int(getpid()), stamp, ctx, func, msg);
        fflush(f);
    }

    int Logger::setMask(int32_t mask)
    {
        if(mask < 0 || mask > 31)
            return HIPTENSOR_STATUS_INVALID_VALUE;
        mMask = mask;
        return HIPTENSOR_STATUS_SUCCESS;
    }

    int Logger::setLevel(int32_t level)
    {
        switch(level)
        {
        case HIPTENSOR_LOG_LEVEL_OFF:
        case HIPTENSOR_LOG_LEVEL_ERROR:
        case HIPTENSOR_LOG_LEVEL_PERF_TRACE:
        case HIPTENSOR_LOG_LEVEL_PERF_HINT:
        case HIPTENSOR_LOG_LEVEL_HEURISTICS_TRACE:
        case HIPTENSOR_LOG_LEVEL_API_TRACE: mMask = level; return HIPTENSOR_STATUS_SUCCESS;
        }
        return HIPTENSOR_STATUS_INVALID_VALUE;
    }

    int Logger::setFile(FILE* f)
    {
        std::lock_guard<std::mutex> lock(mMutex);
        if(mOwnsFile && mFile)
            fclose(mFile);
        mOwnsFile = false;
        mFile     = nullptr;
        if(f == nullptr)
            return HIPTENSOR_STATUS_IO_ERROR;
        mFile = f;
        return HIPTENSOR_STATUS_SUCCESS;
    }

    int Logger::openFile(const char* name)
    {
        std::lock_guard<std::mutex> lock(mMutex);
        if(mOwnsFile && mFile)
            fclose(mFile);
        mOwnsFile = false;
        mFile     = nullptr;
        if(!name)
            return HIPTENSOR_STATUS_IO_ERROR;
        FILE* f = fopen(name, "w");
        if(!f)
            return HIPTENSOR_STATUS_IO_ERROR;
        mFile     = f;
        mOwnsFile = true;
        return HIPTENSOR_STATUS_SUCCESS;
    }

    int Logger::setCallback(hiptensorLoggerCallback_t cb)
    {
        if(cb == nullptr)
            return HIPTENSOR_STATUS_INVALID_VALUE;
        std::lock_guard<std::mutex> lock(mMutex);
        mCallback = cb;
        return HIPTENSOR_STATUS_SUCCESS;
    }

    // ------------------------------------------------------------------ launch bookkeeping
    static std::atomic<uint64_t>    gLaunches{0};
    static thread_local const char* tLastKernel = "";

    void noteLaunch(const char* kernelFamily, int launches)
    {
        tLastKernel = kernelFamily;
        gLaunches.fetch_add(uint64_t(launches), std::memory_order_relaxed);
    }
    const char* lastKernelName()
    {
        return tLastKernel;
    }
    uint64_t launchCount()
    {
        return gLaunches.load(std::memory_order_relaxed);
    }

    // ------------------------------------------------------------------ tensor map encoder
    PFN_encodeTiled tensorMapEncoder()
    {
        static PFN_encodeTiled fn = []() -> PFN_encodeTiled {
            void*                           p = nullptr;
            cudaDriverEntryPointQueryResult q;
            if(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess
               || q != cudaDriverEntryPointSuccess)
                return nullptr;
            return reinterpret_cast<PFN_encodeTiled>(p);
        }();
        return fn;
    }
} // namespace htb
