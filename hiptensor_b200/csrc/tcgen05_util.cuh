// Device helpers shared by the tensor-core contraction kernels: mbarrier arrive / bounded wait,
// TMA box loads, shared-memory matrix descriptors, cluster addressing. Every wait is bounded by a
// clock limit and reports failure instead of spinning for ever.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace htb
{
    namespace
    {
        constexpr long long kWaitCycles = 4000000000ll; // about two seconds

        __device__ __forceinline__ uint32_t smemAddr(const void* p)
        {
            return uint32_t(__cvta_generic_to_shared(p));
        }

        // starts fetching a tensor map (a kernel parameter) so that the first TMA instruction does not wait for it
        __device__ __forceinline__ void prefetchTensorMap(const CUtensorMap* map)
        {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
        }

        __device__ __forceinline__ void mbarInit(uint32_t bar, uint32_t count)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
        }
        __device__ __forceinline__ void mbarArriveExpectTx(uint32_t bar, uint32_t bytes)
        {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        }
        __device__ __forceinline__ void mbarArrive(uint32_t bar)
        {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
        }
        // bounded wait; false when the limit ran out or another role already gave up
        __device__ __forceinline__ bool mbarWait(uint32_t bar, uint32_t parity, volatile int* abortFlag)
        {
            const long long t0 = clock64();
            for(;;)
            {
                uint32_t done;
                asm volatile("{\n\t.reg .pred p;\n\t"
                             "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                             "selp.u32 %0, 1, 0, p;\n\t}"
                             : "=r"(done)
                             : "r"(bar), "r"(parity)
                             : "memory");
                if(done)
                    return true;
                if(*abortFlag)
                    return false;
                if(clock64() - t0 > kWaitCycles)
                {
                    *abortFlag = 1;
                    return false;
                }
            }
        }

        // shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
        __device__ __forceinline__ uint64_t smemDesc(uint32_t addr)
        {
            uint64_t d = 0;
            d |= uint64_t((addr & 0x3FFFF) >> 4); // start address
            d |= uint64_t(1) << 16; // leading byte offset (unused for swizzled K-major)
            d |= uint64_t(1024 >> 4) << 32; // stride byte offset
            d |= uint64_t(1) << 46; // descriptor version of sm_100
            d |= uint64_t(2) << 61; // SWIZZLE_128B
            return d;
        }

        // shared-memory matrix descriptor of an MN-major half-precision operand: the tile is a row of chunks, each
        // chunk [64 k][64 rows = 128 bytes] with 128-byte swizzle; chunks (leading dimension) 8192 bytes apart,
        // 8-k groups (stride dimension) 1024 bytes apart. A 16-wide K step advances the start by 2048 bytes.
        __device__ __forceinline__ uint64_t smemDescMn(uint32_t addr)
        {
            uint64_t d = 0;
            d |= uint64_t((addr & 0x3FFFF) >> 4);
            d |= uint64_t(8192 >> 4) << 16;
            d |= uint64_t(1024 >> 4) << 32;
            d |= uint64_t(1) << 46;
            d |= uint64_t(2) << 61;
            return d;
        }

        template <int RANK>
        __device__ __forceinline__ void tmaLoad(uint32_t dst, const CUtensorMap* map, uint32_t bar, const int* c)
        {
            if constexpr(RANK == 2)
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
                             "{%3, %4}], [%2];" ::"r"(dst),
                             "l"(map), "r"(bar), "r"(c[0]), "r"(c[1])
                             : "memory");
            else if constexpr(RANK == 3)
                asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
                             "{%3, %4, %5}], [%2];" ::"r"(dst),
                             "l"(map), "r"(bar), "r"(c[0]), "r"(c[1]), "r"(c[2])
                             : "memory");
            else if constexpr(RANK == 4)
                asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
                             "{%3, %4, %5, %6}], [%2];" ::"r"(dst),
                             "l"(map), "r"(bar), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3])
                             : "memory");
            else
                asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
                             "{%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
                             "l"(map), "r"(bar), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(c[4])
                             : "memory");
        }
        __device__ __forceinline__ void tmaLoadRank(int rank, uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                    const int* c)
        {
            switch(rank)
            {
            case 2: tmaLoad<2>(dst, map, bar, c); break;
            case 3: tmaLoad<3>(dst, map, bar, c); break;
            case 4: tmaLoad<4>(dst, map, bar, c); break;
            default: tmaLoad<5>(dst, map, bar, c); break;
            }
        }

        __device__ __forceinline__ uint32_t clusterRank()
        {
            uint32_t r;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
            return r;
        }
        __device__ __forceinline__ uint32_t mapToRank(uint32_t addr, uint32_t rank)
        {
            uint32_t r;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
            return r;
        }
        __device__ __forceinline__ void clusterSync()
        {
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        }

        // bounded wait for the two single-thread roles: a tight try_wait loop, the clock is read
        // only every 256th unsuccessful poll
#ifndef HTB_TC_SPIN
#define HTB_TC_SPIN 0
#endif
        constexpr bool kSpinWaits = HTB_TC_SPIN != 0; // poll with test_wait instead of the suspending try_wait
        __device__ __forceinline__ bool mbarWaitTight(uint32_t bar, uint32_t parity, volatile int* abortFlag)
        {
            long long t0 = 0;
            for(uint32_t it = 1;; it++)
            {
                uint32_t done;
                if(kSpinWaits)
                    asm volatile("{\n\t.reg .pred p;\n\t"
                                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                                 "selp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(done)
                                 : "r"(bar), "r"(parity)
                                 : "memory");
                else
                    asm volatile("{\n\t.reg .pred p;\n\t"
                                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                                 "selp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(done)
                                 : "r"(bar), "r"(parity)
                                 : "memory");
                if(done)
                    return true;
                if((it & 255) == 0)
                {
                    if(t0 == 0)
                        t0 = clock64();
                    if(*abortFlag)
                        return false;
                    if(clock64() - t0 > kWaitCycles)
                    {
                        *abortFlag = 1;
                        return false;
                    }
                }
            }
        }

        __device__ __forceinline__ void tmaLoadPair5(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                                     int c2, int c3, int c4)
        {
            asm volatile("cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
                         "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
                         "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
                         : "memory");
        }
    } // namespace
} // namespace htb
