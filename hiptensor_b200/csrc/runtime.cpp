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

    // ------------------------------------------------------------------ variant switches
    namespace
    {
        Switches gSwitches;
        bool     envSet(const char* name)
        {
            const char* e = getenv(name);
            return e != nullptr && e[0] != '\0' && !(e[0] == '0' && e[1] == '\0');
        }
#ifdef HTB_MEASURE
        int envInt(const char* name)
        {
            const char* e = getenv(name);
            return e ? atoi(e) : 0;
        }
#endif
        void readSwitches(Switches& s)
        {
            std::memset(&s, 0, sizeof(s));
            s.tcSingle      = envSet("HTB_TC_SINGLE");
            s.tcPair        = envSet("HTB_TC_PAIR");
            s.tcNoHalf      = envSet("HTB_TC_NOHALF");
            s.tcNoSplit     = envSet("HTB_TC_NOSPLIT");
            s.tcNarrow      = envSet("HTB_TC_NARROW");
            s.tcWide        = envSet("HTB_TC_WIDE");
            s.tcKsplit      = envSet("HTB_TC_KSPLIT");
            s.tcNoTmaStore  = envSet("HTB_TC_NOTMASTORE");
            s.tcNoPdl       = envSet("HTB_TC_NOPDL");
            s.noTf32x3      = envSet("HTB_NO_TF32X3");
            s.tf32Pair      = envSet("HTB_TF32_PAIR");
            s.tf32NoInplace = envSet("HTB_TF32_NOINPLACE");
            s.tf32NoSplit   = envSet("HTB_TF32_NOSPLIT");
            s.dmmaNoVec     = envSet("HTB_DMMA_NOVEC");
            s.dmmaNoSplit   = envSet("HTB_DMMA_NOSPLIT");
            s.f64Compute32Fma = envSet("HTB_F64_COMPUTE32_FMA");
#ifdef HTB_MEASURE
            s.tcProbe    = envInt("HTB_TC_PROBE");
            s.tf32Probe  = envInt("HTB_TF32_PROBE");
            s.permTile   = envInt("HTB_PERM_TILE");
            s.permStages = envInt("HTB_PERM_STAGES");
            s.permCtas   = envInt("HTB_PERM_CTAS");
#endif
        }
        struct SwitchesInit
        {
            SwitchesInit()
            {
                readSwitches(gSwitches);
            }
        } gSwitchesInit;
    } // namespace
    const Switches& switches()
    {
        return gSwitches;
    }
    void reloadSwitches()
    {
        readSwitches(gSwitches);
    }

    // ------------------------------------------------------------------ per-device function attributes
    cudaError_t ensureDynamicSmem(const void* kernel, int bytes)
    {
        struct Entry
        {
            const void* fn;
            int         bytes[kMaxDevices];
        };
        static std::mutex mutex;
        static Entry      table[64];
        static int        used = 0;
        int               dev  = 0;
        if(cudaGetDevice(&dev) != cudaSuccess)
            return cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(mutex);
        Entry*                      e = nullptr;
        for(int i = 0; i < used && !e; i++)
            if(table[i].fn == kernel)
                e = &table[i];
        if(!e && used < 64)
        {
            e     = &table[used++];
            e->fn = kernel;
            std::memset(e->bytes, 0, sizeof(e->bytes));
        }
        if(e && dev >= 0 && dev < kMaxDevices && e->bytes[dev] >= bytes)
            return cudaSuccess;
        const cudaError_t rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if(rc == cudaSuccess && e && dev >= 0 && dev < kMaxDevices)
            e->bytes[dev] = bytes;
        return rc;
    }

    // ------------------------------------------------------------------ tensor-map cache
    MapCacheEntry* mapCacheFind(uint64_t id, const void* A, const void* B, int variant, bool* hit)
    {
        constexpr int              kEntries = 8;
        thread_local MapCacheEntry entries[kEntries];
        thread_local MapCacheEntry uncached;
        thread_local int           next = 0;
        *hit                            = false;
        if(id == 0)
        {
            uncached.id   = 0;
            uncached.half = 0;
            uncached.D    = nullptr;
            return &uncached;
        }
        for(int i = 0; i < kEntries; i++)
            if(entries[i].id == id && entries[i].A == A && entries[i].B == B && entries[i].variant == variant)
            {
                *hit = true;
                return &entries[i];
            }
        MapCacheEntry* e = &entries[next];
        next             = (next + 1) % kEntries;
        e->id            = id;
        e->A             = A;
        e->B             = B;
        e->variant       = variant;
        e->half          = 0;
        e->D             = nullptr;
        return e;
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
