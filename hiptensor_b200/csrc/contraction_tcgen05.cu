// Tensor-core contraction for sm_100a: f16/bf16 operands, fp32 accumulation in tensor memory.
//
//   D[m, n] = alpha * sum_k A[m, k] * B[n, k]  (+ beta * C[m, n])
//
// on the folded view of the mode lists. Both operands are K-major: their K group folds to one
// stride-1 mode. The M (N) rows of a tile may span several folded modes of the strided tensor:
// one multi-dimensional TMA tensor map per operand gathers a [rows x 64] box straight from the
// tensor into 128-byte-swizzled shared memory, no transposed or packed copy is made.
//
// Persistent, warp-specialised CTA (192 threads, one CTA per SM):
//   warp 0      TMA producer: waits for a free stage, arms the stage's mbarrier with the
//               expected byte count, issues the A and B box loads.
//   warp 1      allocates tensor memory; one lane issues tcgen05.mma (128 x tileN x 16, four
//               per 64-wide K block) from shared-memory descriptors, commits each stage back
//               to the producer and each finished accumulator to the epilogue.
//   warps 2-5   epilogue: tcgen05.ld of their 32-lane quadrant, alpha/beta, rounding to the
//               output type, stores to the strided D. Two accumulators in tensor memory let
//               the epilogue of tile i overlap the main loop of tile i+1.
// Every mbarrier wait is bounded by a clock limit; when it runs out the kernel raises the
// device status word, skips the remaining work and still frees its tensor memory.
//
// A second kernel (further down) runs 256 x 256 tiles on pairs of CTAs. Neither uses multicast loads:
// every CTA fetches its own operands.
// It stands where the reference instantiates CK's xdl contraction kernels for f16/bf16
// (library/src/contraction/device/*f16*_instance.cpp, *bf16*_instance.cpp).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "kernels.hpp"
#include "tcgen05_util.cuh"
#include "row_groups.cuh"

namespace htb
{
    namespace
    {
        constexpr int kThreads   = 192;
        constexpr int kTileM     = 128;
        constexpr int kTileK     = 64; // 64 half-precision elements = one 128-byte swizzle row
        constexpr int kMaxStages = 8;

        struct TcArgs
        {
            int     nm, nn; // folded modes per group
            int     boxM[4], boxN[4];
            int     tilesPerDimM[4], tilesPerDimN[4];
            int64_t extM[4], extN[4], sDm[4], sDn[4];
            int     tilesM, tilesN;
            // K group: a 64-wide block runs along the block mode (dimension "K" of the tensor maps), at one index of
            // each of the other K modes (at most two; extent 1 when absent). Block kb: chunk kb % kfChunks of the block
            // mode, the rest of kb enumerates the other modes, first one fastest. kPosA / kPosB: coordinate index of
            // the first other K mode in the operand's tensor map (the second follows).
            int     kfChunks, kExt1, kExt2, kPosA, kPosB;
            int     kBlocks;
            int     stages;
            int     tileN;
            uint32_t stageBytes;
            float   alpha, beta;
            int     bilinear;
            int     nContig; // N is one folded mode with stride 1 in D and D is 16-byte aligned
            int     parts; // single-CTA kernel: K ranges per tile (CTAs of one cluster); 0 or 1 = no split
#ifdef HTB_MEASURE
            int     probe; // measurement builds only, bit mask: 1 = producer skips the loads, 2 = issuer skips the
                           // MMAs, 4 = the pair kernel's epilogue skips its stores (results invalid)
            unsigned long long* trace; // measurement builds only: time stamps (ns) of cluster 0's roles, or null
#endif
            int*    status;
            // chunked row groups of MN-major operands (kernel instantiations with LAYOUT != 0 only)
            TfGroup gm, gn;
        };

        template <typename T>
        __device__ __forceinline__ float outToFloat(T v);
        template <>
        __device__ __forceinline__ float outToFloat<float>(float v)
        {
            return v;
        }
        template <>
        __device__ __forceinline__ float outToFloat<__half>(__half v)
        {
            return __half2float(v);
        }
        template <>
        __device__ __forceinline__ float outToFloat<__nv_bfloat16>(__nv_bfloat16 v)
        {
            return __bfloat162float(v);
        }

        // round the accumulator to the output type first, then alpha*x + beta*c in float
        // (contraction_cpu_reference_impl.hpp:406-425)
        template <typename TD>
        __device__ __forceinline__ TD finish(float acc, float alpha, float beta, bool bilinear, const TD* C, int64_t off)
        {
            float x = outToFloat<TD>(TD(acc));
            float y = __fmul_rn(alpha, x);
            if(bilinear)
                y = __fadd_rn(y, __fmul_rn(beta, outToFloat<TD>(C[off])));
            return TD(y);
        }

        // tile index -> per-mode tile coordinates (first folded mode fastest)
        __device__ __forceinline__ void tileCoords(int t, const int* tilesPerDim, const int* box, int n, int* coord)
        {
            for(int d = 0; d < n; d++)
            {
                const int q = t % tilesPerDim[d];
                t /= tilesPerDim[d];
                coord[d] = q * box[d];
            }
        }
        // row r of a tile -> offset in D along this group, or -1 outside the tensor
        __device__ __forceinline__ int64_t rowOffset(int r, const int* coord, const int* box, const int64_t* ext,
                                                     const int64_t* sD, int n)
        {
            int64_t off = 0;
            for(int d = 0; d < n; d++)
            {
                const int     i = r % box[d];
                r /= box[d];
                const int64_t g = int64_t(coord[d]) + i;
                if(g >= ext[d])
                    return -1;
                off += g * sD[d];
            }
            return (r == 0) ? off : -1; // rows beyond the boxes' product do not exist
        }

        // K block kb -> first element along the block mode and indices of the other K modes
        struct KCoord
        {
            int k0, i1, i2;
        };
        __device__ __forceinline__ KCoord kCoordOf(const TcArgs& a, int kb)
        {
            KCoord c;
            c.k0 = kb * kTileK;
            c.i1 = c.i2 = 0;
            if(a.kExt1 > 1 || a.kExt2 > 1)
            {
                const int r = kb / a.kfChunks;
                c.k0        = (kb - r * a.kfChunks) * kTileK;
                c.i2        = r / a.kExt1; // beyond the last block: outside the map, the box is zero-filled
                c.i1        = r - c.i2 * a.kExt1;
            }
            return c;
        }
        // coordinate j (1 .. 4) of a tensor map: the indices of the other K modes from position kPos on, else `row`
        __device__ __forceinline__ int kPlace(int j, int kPos, const KCoord& c, int row)
        {
            return j == kPos ? c.i1 : (j == kPos + 1 ? c.i2 : row);
        }

#ifdef HTB_MEASURE
        // time stamp k of CTA 0 of the single-CTA kernel (measurement builds): trace[k]
#define HTB_STAMP1(k)                                                             \
    do                                                                            \
    {                                                                             \
        if(a.trace && blockIdx.x == 0)                                            \
        {                                                                         \
            unsigned long long t_;                                                \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                \
            a.trace[k] = t_;                                                      \
        }                                                                         \
    } while(0)
#else
#define HTB_STAMP1(k)
#endif

        // LAYOUT: bit 0 = A is MN-major, bit 1 = B is MN-major (64-row chunks instead of boxes, transposed
        // shared-memory descriptors); 0 = both K-major.
        template <typename TD, int LAYOUT>
        __global__ void __launch_bounds__(kThreads, 1)
            contraction_tcgen05_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                       const TD* C, TD* D, TcArgs a, uint32_t idesc) // C may alias D
        {
            extern __shared__ unsigned char smemRaw[];
            unsigned char* tiles = (unsigned char*)((uintptr_t(smemRaw) + 1023) & ~uintptr_t(1023));

            __shared__ __align__(8) unsigned long long fullBar[kMaxStages], emptyBar[kMaxStages];
            __shared__ __align__(8) unsigned long long tmemFullBar[2], tmemEmptyBar[2];
            __shared__ uint32_t tmemBase;
            __shared__ int      abortFlag;
            __shared__ int64_t  colOff[4][256]; // one table per epilogue warp

            const int      warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const int      tileN      = a.tileN;
            const uint32_t aBytes     = kTileM * kTileK * 2; // the stage always reserves a full A tile
            const uint32_t stageStride = aBytes + uint32_t(tileN) * kTileK * 2;
            const int      numTiles   = a.tilesM * a.tilesN;
            // K split of problems with few tiles: `parts` CTAs per tile (one thread-block cluster), each with a range
            // of the K blocks; unit u = part (u % parts) of tile (u / parts). Parts 1.. hand their accumulators to
            // part 0 through its shared memory (see the epilogue). With parts > 1 every CTA has exactly one unit.
            const int      parts      = a.parts > 1 ? a.parts : 1;
            const int      numUnits   = numTiles * parts;
            auto           kRange     = [&](int u, int& kb0, int& kb1) {
                const int part = u % parts;
                kb0            = int((long long)a.kBlocks * part / parts);
                kb1            = int((long long)a.kBlocks * (part + 1) / parts);
            };
            const uint32_t tmemCols   = (2 * tileN <= 128) ? 128 : (2 * tileN <= 256 ? 256 : 512);

            if(threadIdx.x == 0)
                HTB_STAMP1(0);
            // Programmatic dependent launch, as in the CTA-pair kernel below: the next kernel's set-up may overlap this
            // grid's tail. Every thread that touches global memory runs griddepcontrol.wait right before its first
            // access (the producer before its first load, the epilogue threads before C and D), so that the tile
            // arithmetic ahead of it, on a cold instruction cache 1.4 us, also runs while the grid ahead drains.
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            if(threadIdx.x == 32)
            {
                prefetchTensorMap(&mapA);
                prefetchTensorMap(&mapB);
            }
            if(threadIdx.x == 0)
            {
                abortFlag = 0;
                for(int s = 0; s < a.stages; s++)
                {
                    mbarInit(smemAddr(&fullBar[s]), 1);
                    mbarInit(smemAddr(&emptyBar[s]), 1);
                }
                for(int i = 0; i < 2; i++)
                {
                    mbarInit(smemAddr(&tmemFullBar[i]), 1);
                    mbarInit(smemAddr(&tmemEmptyBar[i]), 128);
                }
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            if(warp == 1)
            {
                asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemBase)),
                             "r"(tmemCols)
                             : "memory");
                asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if(threadIdx.x == 0)
                HTB_STAMP1(1);
            const uint32_t tmem = tmemBase;
            volatile int*  abortP = &abortFlag;

            if(warp == 0)
            {
                // ---------------------------------------------------------------- TMA producer
                // (a second thread issuing the loads of B was measured and changed nothing: a K block's period is what
                // the SM's path from L2 delivers, 0.2 us for the 24 KiB of a 128 x 64 tile)
                if(lane == 0)
                {
                    int      stage = 0;
                    uint32_t phase = 0;
                    bool     ok    = true, waited = false;
                    for(int u = blockIdx.x; u < numUnits && ok; u += gridDim.x)
                    {
                        const int t  = u / parts;
                        const int tm = t % a.tilesM, tn = t / a.tilesM;
                        int       kb0, kb1;
                        kRange(u, kb0, kb1);
                        int       cA[5] = {0, 0, 0, 0, 0}, cB[5] = {0, 0, 0, 0, 0};
                        TfChunks  qA{}, qB{};
                        if constexpr(LAYOUT & 1)
                            qA = tfChunksOf(a.gm, tfTileOf(a.gm, tm));
                        else
                            tileCoords(tm, a.tilesPerDimM, a.boxM, a.nm, cA + 1);
                        if constexpr(LAYOUT & 2)
                            qB = tfChunksOf(a.gn, tfTileOf(a.gn, tn));
                        else
                            tileCoords(tn, a.tilesPerDimN, a.boxN, a.nn, cB + 1);
                        for(int kb = kb0; kb < kb1; kb++)
                        {
                            ok = mbarWaitTight(smemAddr(&emptyBar[stage]), phase ^ 1, abortP);
                            if(!ok)
                                break;
                            const uint32_t bar = smemAddr(&fullBar[stage]);
                            mbarArriveExpectTx(bar, a.stageBytes);
                            const KCoord   kc   = kCoordOf(a, kb);
                            const uint32_t dstA = smemAddr(tiles + size_t(stage) * stageStride);
                            if(!waited)
                            {
                                // the first read of global memory: the grid ahead of this one must be complete
                                asm volatile("griddepcontrol.wait;" ::: "memory");
                                waited = true;
                                HTB_STAMP1(2);
                            }
                            if constexpr(LAYOUT & 1)
                            {
                                // MN-major map {mode0, K, mode1, mode2, ..}: one [64 k][64 rows] box per chunk
#pragma unroll
                                for(int j = 0; j < kTileM / 64; j++)
                                {
                                    const int c[5] = {qA.c0[j], kc.k0, kPlace(2, a.kPosA, kc, qA.i1[j]), kPlace(3, a.kPosA, kc, qA.i2[j]),
                                                      kPlace(4, a.kPosA, kc, 0)};
                                    tmaLoad<5>(dstA + uint32_t(j) * 8192, &mapA, bar, c);
                                }
                            }
                            else
                            {
                                const int c[5] = {kc.k0, kPlace(1, a.kPosA, kc, cA[1]), kPlace(2, a.kPosA, kc, cA[2]),
                                                  kPlace(3, a.kPosA, kc, cA[3]), kPlace(4, a.kPosA, kc, cA[4])};
                                tmaLoad<5>(dstA, &mapA, bar, c);
                            }
                            if constexpr(LAYOUT & 2)
                            {
                                for(int j = 0; j < (tileN >> 6); j++)
                                {
                                    const int c[5] = {qB.c0[j], kc.k0, kPlace(2, a.kPosB, kc, qB.i1[j]), kPlace(3, a.kPosB, kc, qB.i2[j]),
                                                      kPlace(4, a.kPosB, kc, 0)};
                                    tmaLoad<5>(dstA + aBytes + uint32_t(j) * 8192, &mapB, bar, c);
                                }
                            }
                            else
                            {
                                const int c[5] = {kc.k0, kPlace(1, a.kPosB, kc, cB[1]), kPlace(2, a.kPosB, kc, cB[2]),
                                                  kPlace(3, a.kPosB, kc, cB[3]), kPlace(4, a.kPosB, kc, cB[4])};
                                tmaLoad<5>(dstA + aBytes, &mapB, bar, c);
                            }
                            if(kb == kb0)
                                HTB_STAMP1(3);
                            if(kb == kb1 - 1)
                                HTB_STAMP1(9);
                            if(++stage == a.stages)
                            {
                                stage = 0;
                                phase ^= 1;
                            }
                        }
                    }
                }
                if(parts > 1)
                {
                    __syncwarp();
                    clusterSync(); // the two meeting points of the K-split hand-over (see the epilogue)
                    clusterSync();
                }
            }
            else if(warp == 1)
            {
                // ---------------------------------------------------------------- MMA issuer
                if(lane == 0)
                {
                    int      stage = 0;
                    uint32_t phase = 0;
                    int      local = 0;
                    bool     ok    = true;
                    for(int u = blockIdx.x; u < numUnits && ok; u += gridDim.x, local++)
                    {
                        const int      acc      = local & 1;
                        const uint32_t accPhase = (local >> 1) & 1;
                        int            kb0, kb1;
                        kRange(u, kb0, kb1);
                        ok = mbarWaitTight(smemAddr(&tmemEmptyBar[acc]), accPhase ^ 1, abortP);
                        if(!ok)
                            break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t dTmem = tmem + uint32_t(acc * tileN);
                        for(int kb = kb0; kb < kb1; kb++)
                        {
                            ok = mbarWaitTight(smemAddr(&fullBar[stage]), phase, abortP);
                            if(!ok)
                                break;
                            if(kb == kb0)
                                HTB_STAMP1(4);
                            if(kb == kb1 - 1)
                                HTB_STAMP1(10);
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            const uint32_t sa    = smemAddr(tiles + size_t(stage) * stageStride);
                            const uint64_t descA = (LAYOUT & 1) ? smemDescMn(sa) : smemDesc(sa);
                            const uint64_t descB = (LAYOUT & 2) ? smemDescMn(sa + aBytes) : smemDesc(sa + aBytes);
                            // a 16-wide K step: 32 bytes = 2 address units along a K-major row, 16 rows of 128 bytes = 128
                            // units down an MN-major chunk
                            constexpr uint64_t stepA = (LAYOUT & 1) ? 128 : 2, stepB = (LAYOUT & 2) ? 128 : 2;
#pragma unroll
                            for(int k = 0; k < kTileK / 16; k++)
                            {
                                const uint32_t accumulate = (kb != kb0 || k) ? 1u : 0u;
                                asm volatile("{\n\t.reg .pred p;\n\t"
                                             "setp.ne.b32 p, %4, 0;\n\t"
                                             "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(dTmem),
                                             "l"(descA + stepA * uint64_t(k)), "l"(descB + stepB * uint64_t(k)), "r"(idesc),
                                             "r"(accumulate)
                                             : "memory");
                            }
                            // the stage is free once these MMAs have read it
                            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                             smemAddr(&emptyBar[stage]))
                                         : "memory");
                            if(++stage == a.stages)
                            {
                                stage = 0;
                                phase ^= 1;
                            }
                        }
                        if(ok)
                            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                                             smemAddr(&tmemFullBar[acc]))
                                         : "memory");
                        HTB_STAMP1(5);
                    }
                }
                if(parts > 1)
                {
                    __syncwarp();
                    clusterSync();
                    clusterSync();
                }
            }
            else
            {
                // ---------------------------------------------------------------- epilogue
                const int quad = warp & 3; // TMEM lane quadrant this warp may read
                const int row  = quad * 32 + lane;
                int64_t*  cols = colOff[quad];
                int       local = 0;
                int       syncs = 0; // cluster meeting points of the K-split hand-over passed so far
                auto      loadChunk = [&](uint32_t addr, uint32_t(&v)[32]) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
                          "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
                          "=r"(v[30]), "=r"(v[31])
                        : "r"(addr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                };
                for(int u = blockIdx.x; u < numUnits; u += gridDim.x, local++)
                {
                    const int      t = u / parts, part = u % parts;
                    const int      acc      = local & 1;
                    const uint32_t accPhase = (local >> 1) & 1;
                    const int      tm = t % a.tilesM, tn = t / a.tilesM;
                    int            cM[4], cN[4];
                    tileCoords(tm, a.tilesPerDimM, a.boxM, a.nm, cM);
                    tileCoords(tn, a.tilesPerDimN, a.boxN, a.nn, cN);
                    // this warp's table of column offsets for the tile
                    __syncwarp();
                    if constexpr(LAYOUT & 2)
                    {
                        const TfTile wn = tfTileOf(a.gn, tn);
                        for(int c = lane; c < tileN; c += 32)
                            cols[c] = tfRowOffset(a.gn, wn, c);
                    }
                    else
                    {
                        for(int c = lane; c < tileN; c += 32)
                            cols[c] = rowOffset(c, cN, a.boxN, a.extN, a.sDn, a.nn);
                    }
                    __syncwarp();
                    const int64_t offM = (LAYOUT & 1) ? tfRowOffset(a.gm, tfTileOf(a.gm, tm), row)
                                                      : rowOffset(row, cM, a.boxM, a.extM, a.sDm, a.nm);

                    // one lane waits, the warp follows its verdict
                    int ok = 1;
                    if(lane == 0)
                        ok = mbarWait(smemAddr(&tmemFullBar[acc]), accPhase, abortP) ? 1 : 0;
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if(!ok)
                        break;
                    // C is read and D written from here on (the sums exist, so the producer's own wait has long returned)
                    asm volatile("griddepcontrol.wait;" ::: "memory");
                    if(threadIdx.x == 64)
                        HTB_STAMP1(6);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16) + uint32_t(acc * tileN);
                    // K split: parts 1.. store their raw accumulators into part 0's stage memory (idle once every CTA of
                    // the cluster has its sums), layout [part - 1][32-column chunk][column group of four][128 rows] of
                    // 16 bytes; part 0 adds them chunk by chunk before its usual epilogue
                    const uint32_t zone = smemAddr(tiles) + uint32_t(row) * 16u;
                    if(parts > 1)
                    {
                        clusterSync();
                        syncs++;
                        if(part > 0)
                        {
                            for(int c0 = 0; c0 < tileN; c0 += 32)
                            {
                                uint32_t v[32];
                                loadChunk(taddr + uint32_t(c0), v);
                                const uint32_t dst
                                    = mapToRank(zone + uint32_t(((part - 1) * (tileN >> 5) + (c0 >> 5)) * 8) * 2048u, 0);
#pragma unroll
                                for(int j = 0; j < 8; j++)
                                    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + uint32_t(j) * 2048u),
                                                 "r"(v[4 * j]), "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                                                 : "memory");
                            }
                            clusterSync();
                            syncs++;
                            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                            mbarArrive(smemAddr(&tmemEmptyBar[acc]));
                            continue;
                        }
                        clusterSync();
                        syncs++;
                    }
                    for(int c0 = 0; c0 < tileN; c0 += 32)
                    {
                        uint32_t v[32];
                        loadChunk(taddr + uint32_t(c0), v);
                        for(int q = 0; q + 1 < parts; q++)
                        {
                            const uint32_t src = zone + uint32_t((q * (tileN >> 5) + (c0 >> 5)) * 8) * 2048u;
#pragma unroll
                            for(int j = 0; j < 8; j++)
                            {
                                float4 p4;
                                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                             : "=f"(p4.x), "=f"(p4.y), "=f"(p4.z), "=f"(p4.w)
                                             : "r"(src + uint32_t(j) * 2048u));
                                v[4 * j]     = __float_as_uint(__uint_as_float(v[4 * j]) + p4.x);
                                v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + p4.y);
                                v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + p4.z);
                                v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + p4.w);
                            }
                        }
                        if(offM < 0)
                            continue;
                        const int64_t first = cols[c0];
                        const bool    fullChunk = a.nContig && first >= 0 && cols[c0 + 31] == first + 31;
                        if(fullChunk && sizeof(TD) == 4 && ((offM + first) & 3) == 0)
                        {
                            // 32 consecutive floats of this row: eight 128-bit stores
                            float*       dst = (float*)D + offM + first;
                            const float* src = (const float*)C + offM + first;
                            // C may be D, so every load of C stays ahead of the stores that follow it: the loads are
                            // taken four at a time before their stores (one memory round trip per sixteen columns)
#pragma unroll
                            for(int j0 = 0; j0 < 32; j0 += 16)
                            {
                                float4 c4[4];
                                if(a.bilinear)
                                {
#pragma unroll
                                    for(int q = 0; q < 4; q++)
                                        c4[q] = *(const float4*)(src + j0 + 4 * q);
                                }
#pragma unroll
                                for(int q = 0; q < 4; q++)
                                {
                                    const int j = j0 + 4 * q;
                                    float4    o;
                                    o.x = __fmul_rn(a.alpha, __uint_as_float(v[j]));
                                    o.y = __fmul_rn(a.alpha, __uint_as_float(v[j + 1]));
                                    o.z = __fmul_rn(a.alpha, __uint_as_float(v[j + 2]));
                                    o.w = __fmul_rn(a.alpha, __uint_as_float(v[j + 3]));
                                    if(a.bilinear)
                                    {
                                        o.x = __fadd_rn(o.x, __fmul_rn(a.beta, c4[q].x));
                                        o.y = __fadd_rn(o.y, __fmul_rn(a.beta, c4[q].y));
                                        o.z = __fadd_rn(o.z, __fmul_rn(a.beta, c4[q].z));
                                        o.w = __fadd_rn(o.w, __fmul_rn(a.beta, c4[q].w));
                                    }
                                    *(float4*)(dst + j) = o;
                                }
                            }
                        }
                        else
                        {
#pragma unroll
                            for(int j = 0; j < 32; j++)
                            {
                                const int64_t oc = cols[c0 + j];
                                if(oc >= 0)
                                    D[offM + oc] = finish<TD>(__uint_as_float(v[j]), a.alpha, a.beta, a.bilinear != 0, C,
                                                              offM + oc);
                            }
                        }
                    }
                    // hand the accumulator back to the MMA warp
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    mbarArrive(smemAddr(&tmemEmptyBar[acc]));
                    if(threadIdx.x == 64)
                        HTB_STAMP1(7);
                }
                for(; parts > 1 && syncs < 2; syncs++)
                    clusterSync(); // a role that gave up still meets the others
            }

            // ---------------------------------------------------------------- teardown
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if(threadIdx.x == 0)
                HTB_STAMP1(8);
            if(threadIdx.x == 0 && abortFlag && a.status)
                atomicExch(a.status, 2);
            if(warp == 1)
            {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmemCols) : "memory");
                if(lane == 0)
                    HTB_STAMP1(11);
            }
        }

        // ------------------------------------------------------------------ CTA-pair kernel
        // Two CTAs of a cluster (two neighbouring SMs) work on one output tile of 256 rows with
        // tcgen05.mma.cta_group::2: each CTA loads its own 128 rows of A and its half of the rows of B,
        // the leader CTA (even cluster rank) issues the MMAs for both, and each CTA's tensor memory
        // receives the accumulators of its own 128 rows. Against the single-CTA kernel this halves the
        // B traffic per SM (L2 and shared memory).
        //   * the TMA loads of both CTAs complete on the LEADER's full barrier (cta_group::2 form,
        //     barrier address mapped to the leader), which expects the bytes of both;
        //   * tcgen05.commit with a CTA mask releases a stage, or publishes an accumulator, in both
        //     CTAs at once;
        //   * the epilogue threads of both CTAs arrive on the leader's accumulator-empty barrier.
        // Loads carry no multicast qualifier: every CTA fetches its own operands.
        //
        // Tile width (template NSUB). The kernel is bound by the operand bytes that enter the SMs from
        // L2 (about 10 TB/s for the whole chip), i.e. by (1 / tile rows + 1 / tile columns) per flop:
        //   NSUB = 1  256 x 256 tiles, two accumulators in tensor memory (the epilogue of a tile overlaps the
        //             main loop of the next), three stages of two 64-wide K blocks (64 KiB each);
        //   NSUB = 2  256 x 512 tiles, two MMAs (N = 256) per 16-wide K step sharing the A operand, ONE
        //             accumulator of 512 columns (all of tensor memory: the epilogue is not overlapped, eight
        //             epilogue warps keep it short), four stages of one K block (48 KiB each). A quarter fewer
        //             operand bytes per flop.
        //
        // K split (ksplit = 2). When the tiles number at most half of the CTA pairs the machine can hold, a
        // cluster is FOUR CTAs: pair 0 (ranks 0, 1) takes the first half of the K blocks of the tile, pair 1
        // (ranks 2, 3) the second. CTA r and CTA r ^ 2 then hold partial sums of the same 128 rows; each sends
        // the half of its columns that the other one finishes into the other's (by then idle) stage memory
        // (st.shared::cluster), between two cluster barriers, adds what it received to what it kept, applies
        // alpha / beta and stores: no scratch in global memory, the exchange and the stores are spread over all
        // four SMs, and a + b = b + a keeps the result independent of which CTA adds.
#ifdef HTB_MEASURE
        // time stamp k of `role` (0 producer, 1 issuer, 2 first epilogue thread, 3 thread 0) in work unit `unit`,
        // cluster 0 only: trace[((rank * 4 + role) * 8 + unit) * 8 + k]
#define HTB_STAMP(role, unit, k)                                                                                  \
    do                                                                                                            \
    {                                                                                                             \
        if(a.trace && clusterId == 0 && (unit) < 8)                                                               \
        {                                                                                                         \
            unsigned long long t_;                                                                                \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                                \
            a.trace[((rank * 4 + (role)) * 8 + (unit)) * 8 + (k)] = t_;                                           \
        }                                                                                                         \
    } while(0)
#else
#define HTB_STAMP(role, unit, k)
#endif

        struct TcPairArgs
        {
            TcArgs base; // boxN / tilesPerDimN / tilesN describe 128-row N sub-tiles here
            int    pairsM, groupsN; // tiles: pairsM x groupsN; a tile is 256 rows x (2 * NSUB) N sub-tiles
            int    iters; // pipeline stages per whole tile: ceil(K blocks / blocks per stage)
            int    numUnits;
            int    ksplit; // 1, or 2: clusters of four CTAs, pair (rank >> 1) takes K range (rank >> 1)
            // Half tiles (NSUB = 1 only). With several waves of tiles, the tiles of a last wave that fills at most
            // half of the CTA pairs are cut into two 256 x 128 halves along N, one unit each (halves = 1): the last
            // wave then takes half as long. A half unit loads 64 rows of B per CTA and issues MMAs with N = 128.
            int      fullUnits, halves;
            uint32_t idescHalf;
            // A 128-column sub-tile can run alone: 64 rows of B per CTA (K-major B: second tensor map with 64-row boxes),
            // MMAs with N = 128. Without it an odd sub-tile at the edge is paired with a repeat of itself.
            int      singleOk;
            // Output by TMA (fp32 D whose rows and columns are one folded mode each, columns contiguous, no C): the
            // epilogue warps write their 32 x 32 blocks into 128-byte-swizzled shared memory and one lane per warp
            // issues a bulk tensor store, which leaves the SM asynchronously (plain st.global of a 128 x 256 block
            // was measured to take 4-7 us and cannot overlap anything). storeBufs 4 KiB slots per warp.
            int      tmaStore, storeBufs;
            uint32_t storeOffset; // of the slots (tmaStore) or of the column-offset table (otherwise) in the tile memory
        };

        struct TcUnit
        {
            int pm, s0, cnt; // row block (256 rows), first N sub-tile, number of N sub-tiles (1 .. 2 * NSUB)
            int kbBegin, kbEnd; // stage range [kbBegin, kbEnd)
        };
        struct TcSched
        {
            int u;
        };
        __device__ __forceinline__ TcSched schedInit(const TcPairArgs&, int clusterId, int)
        {
            TcSched sc;
            sc.u = clusterId;
            return sc;
        }
        // the next work unit of this cluster; false when there is none
        template <int NSUB>
        __device__ __forceinline__ bool schedNext(const TcPairArgs& pa, int numClusters, int kpart, TcSched& sc, TcUnit& w)
        {
            const int S = pa.base.tilesN;
            w.kbBegin   = 0;
            w.kbEnd     = pa.iters;
            if(sc.u >= pa.numUnits)
                return false;
            const int u = sc.u;
            sc.u += numClusters;
            if(pa.ksplit > 1)
            {
                w.kbBegin = int((long long)pa.iters * kpart / pa.ksplit);
                w.kbEnd   = int((long long)pa.iters * (kpart + 1) / pa.ksplit);
            }
            int tile = u, half = -1;
            if(pa.halves && u >= pa.fullUnits)
            {
                const int x = u - pa.fullUnits;
                tile        = pa.fullUnits + (x >> 1);
                half        = x & 1;
            }
            w.pm         = tile % pa.pairsM;
            const int pn = tile / pa.pairsM;
            w.s0         = 2 * NSUB * pn + (half >= 0 ? half : 0);
            w.cnt        = half >= 0 ? 1 : min(2 * NSUB, S - w.s0);
            return true;
        }
        // sub-tiles of accumulator half h of a unit: valid ones, and loaded ones (an odd one that cannot run alone
        // is paired with a repeat)
        __device__ __forceinline__ int subValid(const TcUnit& w, int h)
        {
            return max(0, min(2, w.cnt - 2 * h));
        }
        __device__ __forceinline__ int subLoaded(const TcPairArgs& pa, const TcUnit& w, int h)
        {
            const int v = subValid(w, h);
            return (v == 1 && !pa.singleOk) ? 2 : v;
        }

        // barrier of the epilogue warps of one CTA (named barrier 1) that also tells every thread whether any of
        // them raised `flag`
        template <int THREADS>
        __device__ __forceinline__ bool epiBarrierAny(bool flag)
        {
            uint32_t any;
            asm volatile("{\n\t.reg .pred p, q;\n\t"
                         "setp.ne.u32 q, %1, 0;\n\t"
                         "bar.red.or.pred p, 1, %2, q;\n\t"
                         "selp.u32 %0, 1, 0, p;\n\t}"
                         : "=r"(any)
                         : "r"(flag ? 1u : 0u), "r"(THREADS)
                         : "memory");
            return any != 0;
        }

        // LAYOUT as in the single-CTA kernel: bit 0 = A MN-major, bit 1 = B MN-major
        template <typename TD, int LAYOUT, int NSUB>
        __global__ void __launch_bounds__(64 + 128 * NSUB, 1)
            contraction_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap mapA,
                                            const __grid_constant__ CUtensorMap mapB,
                                            const __grid_constant__ CUtensorMap mapB64,
                                            const __grid_constant__ CUtensorMap mapD, const TD* C, TD* D, TcPairArgs pa,
                                            uint32_t idesc) // C may alias D
        {
            constexpr int KSUB = (NSUB == 1) ? 2 : 1; // 64-wide K blocks per pipeline stage
            constexpr int EPI  = 128 * NSUB; // epilogue threads per CTA
            constexpr int NACC = 2 / NSUB; // accumulators in tensor memory
            constexpr int W    = 256 * NSUB; // accumulator columns = tile columns
            const TcArgs& a = pa.base;
            extern __shared__ unsigned char smemRaw[];
            unsigned char* tiles = (unsigned char*)((uintptr_t(smemRaw) + 1023) & ~uintptr_t(1023));

            __shared__ __align__(8) unsigned long long fullBar[kMaxStages], emptyBar[kMaxStages];
            __shared__ __align__(8) unsigned long long tmemFullBar[2], tmemEmptyBar[2];
            __shared__ uint32_t tmemBase;
            __shared__ int      abortFlag;
            // D offset of every column of the tile, shared by the epilogue warps (plain stores only): W entries that
            // live behind the pipeline stages, where the TMA-store slots lie otherwise
            int64_t* colOff = (int64_t*)(tiles + pa.storeOffset);

            const int      warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t rank = clusterRank();
            const uint32_t pairRank = rank & 1u, leaderRank = rank & ~1u;
            const int      kpart  = int(rank >> 1); // K range of this pair (ksplit = 2), else 0
            const bool     leader = (pairRank == 0);
            constexpr uint32_t kHalfBytes = 128 * kTileK * 2; // 16 KiB: 128 rows of one 64-wide K block
            constexpr uint32_t kStage     = KSUB * (1 + NSUB) * kHalfBytes; // A blocks, then this CTA's B blocks
            const int      csize       = 2 * pa.ksplit;
            const int      clusterId   = blockIdx.x / csize;
            const int      numClusters = gridDim.x / csize;

            if(threadIdx.x == 0)
                HTB_STAMP(3, 0, 0);
            // Programmatic dependent launch: the next kernel of the stream (when it was launched with that attribute)
            // may bring its CTAs up as soon as every CTA of this grid is here, so that its barrier set-up, tensor-memory
            // allocation, cluster meeting and first tile arithmetic overlap this grid's tail; its threads read or write
            // global memory only after their own griddepcontrol.wait (the producer right before its first load, the
            // epilogue threads before C and D), i.e. once this grid is complete.
            asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
            if(threadIdx.x == 32)
            {
                prefetchTensorMap(&mapA);
                prefetchTensorMap(&mapB);
                prefetchTensorMap(&mapB64);
                if(pa.tmaStore)
                    prefetchTensorMap(&mapD);
            }
            if(threadIdx.x == 0)
            {
                abortFlag = 0;
                for(int s = 0; s < a.stages; s++)
                {
                    mbarInit(smemAddr(&fullBar[s]), 1);
                    mbarInit(smemAddr(&emptyBar[s]), 1);
                }
                for(int i = 0; i < 2; i++)
                {
                    mbarInit(smemAddr(&tmemFullBar[i]), 1);
                    mbarInit(smemAddr(&tmemEmptyBar[i]), 2 * EPI);
                }
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            if(warp == 1)
            {
                asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemBase)),
                             "r"(512u)
                             : "memory");
                asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            clusterSync(); // the peers' barriers exist before anything signals them
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem   = tmemBase;
            volatile int*  abortP = &abortFlag;
            const uint32_t tilesAddr = smemAddr(tiles);
            const uint32_t fullAddr = smemAddr(&fullBar[0]), emptyAddr = smemAddr(&emptyBar[0]);
            if(threadIdx.x == 0)
                HTB_STAMP(3, 0, 1);

            if(warp == 0)
            {
                // ---------------------------------------------------------------- TMA producer
                if(lane == 0)
                {
                    int            unitNo = 0;
                    const uint32_t leaderFull = mapToRank(fullAddr, leaderRank);
                    uint32_t       stage = 0, phase = 0;
                    bool           ok = true;
                    TcSched        sched = schedInit(pa, clusterId, numClusters);
                    TcUnit         w;
                    bool           waited = false;
                    while(ok && schedNext<NSUB>(pa, numClusters, kpart, sched, w))
                    {
                        const int    tm = min(2 * w.pm + int(pairRank), a.tilesM - 1);
                        // B rows of this CTA, per accumulator half h: two sub-tiles -> the 128 rows of sub-tile
                        // s0 + 2 h + pairRank; one sub-tile -> its 64-row piece `pairRank` (K-major: second tensor map
                        // with 64-row boxes; MN-major: one chunk instead of two)
                        int          cA[4] = {0, 0, 0, 0}, cB[NSUB][4], nl[NSUB];
                        TfChunks     qA{}, qB[NSUB];
                        uint32_t     txBytes = 2 * KSUB * 16384; // both CTAs' A rows
                        if constexpr(LAYOUT & 1)
                            qA = tfChunksOf(a.gm, tfTileOf(a.gm, tm));
                        else
                            tileCoords(tm, a.tilesPerDimM, a.boxM, a.nm, cA);
#pragma unroll
                        for(int h = 0; h < NSUB; h++)
                        {
                            nl[h]        = subLoaded(pa, w, h);
                            const int tn = nl[h] == 1 ? w.s0 + 2 * h : min(w.s0 + 2 * h + int(pairRank), a.tilesN - 1);
                            txBytes += uint32_t(nl[h]) * KSUB * 16384;
                            cB[h][0] = cB[h][1] = cB[h][2] = cB[h][3] = 0;
                            qB[h] = TfChunks{};
                            if(nl[h] == 0)
                                continue;
                            if constexpr(LAYOUT & 2)
                                qB[h] = tfChunksOf(a.gn, tfTileOf(a.gn, tn));
                            else
                                tileCoords(tn, a.tilesPerDimN, a.boxN, a.nn, cB[h]);
                            if(nl[h] == 1)
                            {
                                cB[h][0] += int(pairRank) * 64;
                                qB[h].c0[0] = qB[h].c0[pairRank];
                                qB[h].i1[0] = qB[h].i1[pairRank];
                                qB[h].i2[0] = qB[h].i2[pairRank];
                            }
                        }
                        const int a1 = cA[0], a2 = cA[1], a3 = cA[2], a4 = cA[3];
                        HTB_STAMP(0, unitNo, 0);
                        for(int it = w.kbBegin; it < w.kbEnd; it++)
                        {
                            ok = mbarWaitTight(emptyAddr + 8 * stage, phase ^ 1, abortP);
                            if(!ok)
                                break;
                            if(it == w.kbBegin)
                                HTB_STAMP(0, unitNo, 1);
#ifdef HTB_MEASURE
                            if(a.probe & 1)
                            {
                                if(leader)
                                    mbarArrive(fullAddr + 8 * stage);
                            }
                            else
#endif
                            {
                                if(leader)
                                    mbarArriveExpectTx(fullAddr + 8 * stage, txBytes);
                                const uint32_t bar = leaderFull + 8 * stage;
                                const uint32_t dst = tilesAddr + stage * kStage;
                                if(!waited)
                                {
                                    // the first read of global memory: the grid ahead of this one must be complete
                                    asm volatile("griddepcontrol.wait;" ::: "memory");
                                    waited = true;
                                }
#pragma unroll
                                for(int q = 0; q < KSUB; q++)
                                {
                                    // beyond the last K block the coordinates fall outside the map: the box is zero-filled
                                    const KCoord kc = kCoordOf(a, it * KSUB + q);
                                    const int    k0 = kc.k0;
                                    if constexpr(LAYOUT & 1)
                                    {
                                        // MN-major map {mode0, K, mode1, mode2, ..}: two [64 k][64 rows] boxes
                                        tmaLoadPair5(dst + q * kHalfBytes, &mapA, bar, qA.c0[0], k0, kPlace(2, a.kPosA, kc, qA.i1[0]),
                                                     kPlace(3, a.kPosA, kc, qA.i2[0]), kPlace(4, a.kPosA, kc, 0));
                                        tmaLoadPair5(dst + q * kHalfBytes + 8192, &mapA, bar, qA.c0[1], k0,
                                                     kPlace(2, a.kPosA, kc, qA.i1[1]), kPlace(3, a.kPosA, kc, qA.i2[1]),
                                                     kPlace(4, a.kPosA, kc, 0));
                                    }
                                    else
                                        tmaLoadPair5(dst + q * kHalfBytes, &mapA, bar, k0, kPlace(1, a.kPosA, kc, a1),
                                                     kPlace(2, a.kPosA, kc, a2), kPlace(3, a.kPosA, kc, a3), kPlace(4, a.kPosA, kc, a4));
#pragma unroll
                                    for(int h = 0; h < NSUB; h++)
                                    {
                                        if(nl[h] == 0)
                                            continue;
                                        const uint32_t db = dst + (KSUB * (1 + h) + q) * kHalfBytes;
                                        if constexpr(LAYOUT & 2)
                                        {
                                            tmaLoadPair5(db, &mapB, bar, qB[h].c0[0], k0, kPlace(2, a.kPosB, kc, qB[h].i1[0]),
                                                         kPlace(3, a.kPosB, kc, qB[h].i2[0]), kPlace(4, a.kPosB, kc, 0));
                                            if(nl[h] == 2)
                                                tmaLoadPair5(db + 8192, &mapB, bar, qB[h].c0[1], k0, kPlace(2, a.kPosB, kc, qB[h].i1[1]),
                                                             kPlace(3, a.kPosB, kc, qB[h].i2[1]), kPlace(4, a.kPosB, kc, 0));
                                        }
                                        else
                                            tmaLoadPair5(db, nl[h] == 2 ? &mapB : &mapB64, bar, k0, kPlace(1, a.kPosB, kc, cB[h][0]),
                                                         kPlace(2, a.kPosB, kc, cB[h][1]), kPlace(3, a.kPosB, kc, cB[h][2]),
                                                         kPlace(4, a.kPosB, kc, cB[h][3]));
                                    }
                                }
                            }
                            if(++stage == uint32_t(a.stages))
                            {
                                stage = 0;
                                phase ^= 1;
                            }
                        }
                        HTB_STAMP(0, unitNo, 2);
                        unitNo++;
                    }
                }
                if(pa.ksplit > 1)
                {
                    __syncwarp();
                    clusterSync(); // the two meeting points of the K-split exchange (see the epilogue)
                    clusterSync();
                }
            }
            else if(warp == 1)
            {
                // ---------------------------------------------------------------- MMA issuer (leader CTA of the pair)
                if(lane == 0 && leader)
                {
                    const uint64_t descBaseA = (LAYOUT & 1) ? smemDescMn(tilesAddr) : smemDesc(tilesAddr);
                    const uint64_t descBaseB = (LAYOUT & 2) ? smemDescMn(tilesAddr) : smemDesc(tilesAddr);
                    // a 16-wide K step: 2 address units along a K-major row, 128 down an MN-major chunk
                    constexpr int  stepA = (LAYOUT & 1) ? 128 : 2, stepB = (LAYOUT & 2) ? 128 : 2;
                    const unsigned short pairMask = (unsigned short)(3u << leaderRank);
                    uint32_t       stage = 0, phase = 0;
                    int            local = 0;
                    bool           ok    = true;
                    TcSched        sched = schedInit(pa, clusterId, numClusters);
                    TcUnit         w;
                    for(; ok && schedNext<NSUB>(pa, numClusters, kpart, sched, w); local++)
                    {
                        const int      acc      = local % NACC;
                        const uint32_t accPhase = (local / NACC) & 1;
                        int            nl[NSUB];
#pragma unroll
                        for(int h = 0; h < NSUB; h++)
                            nl[h] = subLoaded(pa, w, h);
                        HTB_STAMP(1, local, 0);
                        ok = mbarWaitTight(smemAddr(&tmemEmptyBar[acc]), accPhase ^ 1, abortP);
                        if(!ok)
                            break;
                        HTB_STAMP(1, local, 1);
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const uint32_t dTmem = tmem + uint32_t(acc * 256);
                        for(int it = w.kbBegin; it < w.kbEnd; it++)
                        {
                            ok = mbarWaitTight(fullAddr + 8 * stage, phase, abortP);
                            if(!ok)
                                break;
                            if(it == w.kbBegin)
                                HTB_STAMP(1, local, 2);
                            if(it == w.kbBegin + 1)
                                HTB_STAMP(1, local, 3);
                            if(it == w.kbEnd - 1)
                                HTB_STAMP(1, local, 4);
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                            // descriptor address field counts 16-byte units
                            const uint64_t descA = descBaseA + uint64_t((stage * kStage) >> 4);
                            const uint64_t descB = descBaseB + uint64_t((stage * kStage + KSUB * kHalfBytes) >> 4);
#ifdef HTB_MEASURE
                            if(!(a.probe & 2))
#endif
                            {
#pragma unroll
                                for(int k = 0; k < KSUB * (kTileK / 16); k++)
                                {
                                    // 64-wide K blocks are 16 KiB apart
                                    const uint64_t offA = uint64_t((k / 4) * (kHalfBytes >> 4) + stepA * (k % 4));
                                    const uint64_t offB = uint64_t((k / 4) * (kHalfBytes >> 4) + stepB * (k % 4));
                                    const uint32_t accumulate = (it != w.kbBegin || k != 0) ? 1u : 0u;
#pragma unroll
                                    for(int h = 0; h < NSUB; h++)
                                    {
                                        if(nl[h] == 0)
                                            continue;
                                        // N = 256 for two sub-tiles, 128 for a single one
                                        asm volatile("{\n\t.reg .pred p;\n\t"
                                                     "setp.ne.b32 p, %4, 0;\n\t"
                                                     "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(dTmem + uint32_t(h * 256)),
                                                     "l"(descA + offA), "l"(descB + offB + uint64_t(h * KSUB * (kHalfBytes >> 4))),
                                                     "r"(nl[h] == 2 ? idesc : pa.idescHalf), "r"(accumulate)
                                                     : "memory");
                                    }
                                }
                            }
                            // frees the stage in both CTAs of the pair once these MMAs have read it
                            asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
                                         "[%0], %1;" ::"r"(emptyAddr + 8 * stage),
                                         "h"(pairMask)
                                         : "memory");
                            if(++stage == uint32_t(a.stages))
                            {
                                stage = 0;
                                phase ^= 1;
                            }
                        }
                        if(ok)
                            asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
                                         "[%0], %1;" ::"r"(smemAddr(&tmemFullBar[acc])),
                                         "h"(pairMask)
                                         : "memory");
                        HTB_STAMP(1, local, 5);
                    }
                }
                if(pa.ksplit > 1)
                {
                    __syncwarp();
                    clusterSync();
                    clusterSync();
                }
            }
            else
            {
                // ---------------------------------------------------------------- epilogue (both CTAs)
                const int quad = warp & 3; // TMEM lane quadrant this warp may read
                const int row  = quad * 32 + lane;
                const int et   = int(threadIdx.x) - 64; // index among the epilogue threads
                const int colGroup = (warp - 2) >> 2; // NSUB = 2: which half of the columns this warp takes
                int       local = 0;
                int       syncs = 0; // cluster meeting points of the K-split exchange passed so far
                int       storeSeq = 0; // bulk stores this warp has issued (they rotate over its slots)
                auto      loadChunk = [&](uint32_t addr, uint32_t(&v)[32]) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
                          "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
                          "=r"(v[30]), "=r"(v[31])
                        : "r"(addr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                };
                TcSched sched = schedInit(pa, clusterId, numClusters);
                TcUnit  w;
                for(; schedNext<NSUB>(pa, numClusters, kpart, sched, w); local++)
                {
                    const int      acc      = local % NACC;
                    const uint32_t accPhase = (local / NACC) & 1;
                    const int      tmRaw = 2 * w.pm + int(pairRank);
                    // accumulator column c belongs to sub-tile s0 + 2 (c / 256) + (c % 256) / 128 when that one is part
                    // of the unit
                    auto subOf = [&](int c) { return w.s0 + 2 * (c >> 8) + ((c & 255) >> 7); };
                    auto inUnit = [&](int c) { return ((c & 255) >> 7) < subValid(w, c >> 8); };
                    const bool     dupM  = tmRaw >= a.tilesM; // this CTA repeats its peer's rows: no stores
                    const int      tm    = min(tmRaw, a.tilesM - 1);
                    int            cM[4];
                    tileCoords(tm, a.tilesPerDimM, a.boxM, a.nm, cM);
                    // the table of column offsets, filled by all epilogue threads once nobody reads the previous one
                    epiBarrierAny<EPI>(false);
                    for(int c = et; c < W && !pa.tmaStore; c += EPI)
                    {
                        const int tnRaw = subOf(c);
                        int64_t   off   = -1;
                        if(inUnit(c) && tnRaw < a.tilesN)
                        {
                            if constexpr(LAYOUT & 2)
                                off = tfRowOffset(a.gn, tfTileOf(a.gn, tnRaw), c & 127);
                            else
                            {
                                int cN[4];
                                tileCoords(tnRaw, a.tilesPerDimN, a.boxN, a.nn, cN);
                                off = rowOffset(c & 127, cN, a.boxN, a.extN, a.sDn, a.nn);
                            }
                        }
                        colOff[c] = off;
                    }
                    const int64_t offM = dupM ? -1
                                              : ((LAYOUT & 1) ? tfRowOffset(a.gm, tfTileOf(a.gm, tm), row)
                                                              : rowOffset(row, cM, a.boxM, a.extM, a.sDm, a.nm));
                    // one lane waits for the accumulator; the barrier completes the table and tells every epilogue
                    // thread of the CTA whether a wait ran out (all of them then leave together)
                    bool failed = false;
                    if(et == 0)
                        HTB_STAMP(2, local, 0);
                    if(lane == 0)
                        failed = !mbarWait(smemAddr(&tmemFullBar[acc]), accPhase, abortP);
                    if(et == 0)
                        HTB_STAMP(2, local, 1);
                    __syncwarp();
                    if(epiBarrierAny<EPI>(failed))
                        break;
                    // C is read and D written from here on (the sums exist, so the producer's own wait has long returned)
                    asm volatile("griddepcontrol.wait;" ::: "memory");
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t taddr = tmem + (uint32_t(quad * 32) << 16) + uint32_t(acc * 256);
                    // D offsets of the eight rows of this lane's group of eight lanes (for the line-wise stores below)
                    int64_t rowOff[8];
#pragma unroll
                    for(int k = 0; k < 8; k++)
                        rowOff[k] = __shfl_sync(0xffffffffu, offM, (lane & ~7) + k);

                    // alpha / beta and the stores of 32 accumulator columns c0 .. c0 + 31 of this thread's row
                    auto storeChunk = [&](uint32_t(&v)[32], int c0) {
#ifdef HTB_MEASURE
                        if(a.probe & 4)
                            return;
#endif
                        if(pa.tmaStore)
                        {
                            // the chunk's sub-tile; sub-tiles beyond the tensor and the rows of a CTA that repeats its
                            // peer's rows are dropped, ragged edges are clipped by the bulk store itself
                            const int tnRaw = subOf(c0);
                            if(dupM || !inUnit(c0) || tnRaw >= a.tilesN)
                                return;
                            const uint32_t slot = tilesAddr + pa.storeOffset
                                                  + uint32_t(((warp - 2) * pa.storeBufs + storeSeq % pa.storeBufs) * 4096);
                            storeSeq++;
                            // the slot is free once the bulk stores issued before its last use have read their data
                            if(lane == 0)
                            {
                                if(pa.storeBufs >= 4)
                                    asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
                                else if(pa.storeBufs == 2)
                                    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                                else
                                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                            }
                            __syncwarp();
                            // row `lane` of the 32 x 32 block: 128 bytes, its 16-byte units permuted by the 128-byte swizzle
                            const uint32_t rowAddr = slot + uint32_t(lane) * 128u;
#pragma unroll
                            for(int j = 0; j < 8; j++)
                            {
                                const float x0 = __fmul_rn(a.alpha, __uint_as_float(v[4 * j])),
                                            x1 = __fmul_rn(a.alpha, __uint_as_float(v[4 * j + 1])),
                                            x2 = __fmul_rn(a.alpha, __uint_as_float(v[4 * j + 2])),
                                            x3 = __fmul_rn(a.alpha, __uint_as_float(v[4 * j + 3]));
                                asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(rowAddr + uint32_t((j ^ (lane & 7)) << 4)),
                                             "f"(x0), "f"(x1), "f"(x2), "f"(x3)
                                             : "memory");
                            }
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            __syncwarp();
                            if(lane == 0)
                            {
                                const int col = tnRaw * 128 + (c0 & 127), rowC = tm * 128 + quad * 32;
                                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(&mapD),
                                             "r"(slot), "r"(col), "r"(rowC)
                                             : "memory");
                                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            }
                            return;
                        }
                        const int64_t first     = colOff[c0];
                        const bool    fullChunk = a.nContig && first >= 0 && colOff[c0 + 31] == first + 31;
                        if constexpr(sizeof(TD) == 4)
                        {
                            // Line-wise stores. A lane holds 32 consecutive floats of its own row; stored as they are, one
                            // instruction touches 32 different lines, and that request stream was measured to slow the
                            // MMAs of the next tile: the first stages of a tile took twice as long while the previous
                            // tile was being stored. The eight lanes of a group therefore transpose their 8 x 8 blocks of
                            // four floats with three rounds of shuffles, after which lane m holds quarter-line m of each
                            // of the group's eight rows and one store instruction writes four whole 128-byte lines.
                            if(fullChunk && __all_sync(0xffffffffu, offM < 0 || ((offM + first) & 3) == 0))
                            {
                                float4 o[8];
#pragma unroll
                                for(int c = 0; c < 8; c++)
                                {
                                    o[c].x = __fmul_rn(a.alpha, __uint_as_float(v[4 * c]));
                                    o[c].y = __fmul_rn(a.alpha, __uint_as_float(v[4 * c + 1]));
                                    o[c].z = __fmul_rn(a.alpha, __uint_as_float(v[4 * c + 2]));
                                    o[c].w = __fmul_rn(a.alpha, __uint_as_float(v[4 * c + 3]));
                                }
                                const int m = lane & 7;
#pragma unroll
                                for(int sft = 4; sft >= 1; sft >>= 1)
                                {
                                    const bool hi = (m & sft) != 0;
#pragma unroll
                                    for(int c = 0; c < 8; c++)
                                    {
                                        if(c & sft)
                                            continue;
                                        // the lane with the bit clear gives its o[c | sft] and takes the partner's o[c]
                                        const float4 snd = hi ? o[c] : o[c | sft];
                                        float4       rcv;
                                        rcv.x = __shfl_xor_sync(0xffffffffu, snd.x, sft);
                                        rcv.y = __shfl_xor_sync(0xffffffffu, snd.y, sft);
                                        rcv.z = __shfl_xor_sync(0xffffffffu, snd.z, sft);
                                        rcv.w = __shfl_xor_sync(0xffffffffu, snd.w, sft);
                                        if(hi)
                                            o[c] = rcv;
                                        else
                                            o[c | sft] = rcv;
                                    }
                                }
                                // o[k] is now quarter-line m of row k of the group
                                if(a.bilinear)
                                {
                                    float4 c4[8]; // all loads of C ahead of the stores (C may be D)
#pragma unroll
                                    for(int k = 0; k < 8; k++)
                                        c4[k] = rowOff[k] >= 0 ? *(const float4*)((const float*)C + rowOff[k] + first + 4 * m)
                                                               : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                                    for(int k = 0; k < 8; k++)
                                    {
                                        o[k].x = __fadd_rn(o[k].x, __fmul_rn(a.beta, c4[k].x));
                                        o[k].y = __fadd_rn(o[k].y, __fmul_rn(a.beta, c4[k].y));
                                        o[k].z = __fadd_rn(o[k].z, __fmul_rn(a.beta, c4[k].z));
                                        o[k].w = __fadd_rn(o[k].w, __fmul_rn(a.beta, c4[k].w));
                                    }
                                }
#pragma unroll
                                for(int k = 0; k < 8; k++)
                                    if(rowOff[k] >= 0)
                                        *(float4*)((float*)D + rowOff[k] + first + 4 * m) = o[k];
                                return;
                            }
                        }
                        if(offM < 0)
                            return;
                        if(fullChunk && sizeof(TD) == 4 && ((offM + first) & 3) == 0)
                        {
                            float*       dst = (float*)D + offM + first;
                            const float* src = (const float*)C + offM + first;
                            // C may be D, so every load of C stays ahead of the stores that follow it: the loads are
                            // taken four at a time before their stores (one memory round trip per sixteen columns)
#pragma unroll
                            for(int j0 = 0; j0 < 32; j0 += 16)
                            {
                                float4 c4[4];
                                if(a.bilinear)
                                {
#pragma unroll
                                    for(int q = 0; q < 4; q++)
                                        c4[q] = *(const float4*)(src + j0 + 4 * q);
                                }
#pragma unroll
                                for(int q = 0; q < 4; q++)
                                {
                                    const int j = j0 + 4 * q;
                                    float4    o;
                                    o.x = __fmul_rn(a.alpha, __uint_as_float(v[j]));
                                    o.y = __fmul_rn(a.alpha, __uint_as_float(v[j + 1]));
                                    o.z = __fmul_rn(a.alpha, __uint_as_float(v[j + 2]));
                                    o.w = __fmul_rn(a.alpha, __uint_as_float(v[j + 3]));
                                    if(a.bilinear)
                                    {
                                        o.x = __fadd_rn(o.x, __fmul_rn(a.beta, c4[q].x));
                                        o.y = __fadd_rn(o.y, __fmul_rn(a.beta, c4[q].y));
                                        o.z = __fadd_rn(o.z, __fmul_rn(a.beta, c4[q].z));
                                        o.w = __fadd_rn(o.w, __fmul_rn(a.beta, c4[q].w));
                                    }
                                    *(float4*)(dst + j) = o;
                                }
                            }
                        }
                        else
                        {
#pragma unroll
                            for(int j = 0; j < 32; j++)
                            {
                                const int64_t oc = colOff[c0 + j];
                                if(oc >= 0)
                                    D[offM + oc] = finish<TD>(__uint_as_float(v[j]), a.alpha, a.beta, a.bilinear != 0, C,
                                                              offM + oc);
                            }
                        }
                    };

                    if(pa.ksplit > 1)
                    {
                        // K-split exchange. This CTA finishes the half `kpart` of the tile's columns and sends the other
                        // half of its partial sums to CTA rank ^ 2 (same rows, other K range). Each warp sends 128 columns
                        // and finishes 128: layout in the receiver's stage memory [32-column chunk][column group of
                        // four][128 rows] of 16 bytes.
                        constexpr int kHalfW = W / 2;
                        const int     keep = kpart * kHalfW + colGroup * 128, send = (1 - kpart) * kHalfW + colGroup * 128;
                        const uint32_t zone = tilesAddr + uint32_t(row) * 16u + uint32_t(colGroup * 4) * 16384u;
                        clusterSync(); // every CTA of the cluster has its sums: all stage memory is idle
                        syncs++;
                        if(et == 0)
                            HTB_STAMP(2, local, 2);
                        const uint32_t remote = mapToRank(zone, rank ^ 2u);
#pragma unroll 1
                        for(int c0 = 0; c0 < 128; c0 += 32)
                        {
                            uint32_t v[32];
                            loadChunk(taddr + uint32_t(send + c0), v);
                            const uint32_t dst = remote + uint32_t(c0 >> 5) * 16384u;
#pragma unroll
                            for(int j = 0; j < 8; j++)
                                asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + uint32_t(j) * 2048u),
                                             "r"(v[4 * j]), "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                                             : "memory");
                        }
                        if(et == 0)
                            HTB_STAMP(2, local, 3);
                        clusterSync(); // the partner's sums have arrived
                        syncs++;
                        if(et == 0)
                            HTB_STAMP(2, local, 4);
#pragma unroll 1
                        for(int c0 = 0; c0 < 128; c0 += 32)
                        {
                            uint32_t v[32];
                            loadChunk(taddr + uint32_t(keep + c0), v);
                            if(et == 0 && c0 == 0)
                                HTB_STAMP(2, local, 6);
                            const uint32_t src = zone + uint32_t(c0 >> 5) * 16384u;
#pragma unroll
                            for(int j = 0; j < 8; j++)
                            {
                                float4 p4;
                                asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                             : "=f"(p4.x), "=f"(p4.y), "=f"(p4.z), "=f"(p4.w)
                                             : "r"(src + uint32_t(j) * 2048u));
                                v[4 * j]     = __float_as_uint(__uint_as_float(v[4 * j]) + p4.x);
                                v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + p4.y);
                                v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + p4.z);
                                v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + p4.w);
                            }
                            storeChunk(v, keep + c0);
                            if(et == 0 && c0 == 0)
                                HTB_STAMP(2, local, 7);
                        }
                    }
                    else
                    {
                        // whole tile: the two warps of a lane quadrant (NSUB = 2) take 256 columns each
                        const int cBegin = (NSUB == 2) ? colGroup * 256 : 0;
                        const int cEnd   = cBegin + 256;
#pragma unroll 1
                        for(int c0 = cBegin; c0 < cEnd; c0 += 32)
                        {
                            if(!inUnit(c0))
                                continue;
                            uint32_t v[32];
                            loadChunk(taddr + uint32_t(c0), v);
                            if(et == 0 && c0 == cBegin)
                                HTB_STAMP(2, local, 6);
                            storeChunk(v, c0);
                            if(et == 0 && c0 == cBegin)
                                HTB_STAMP(2, local, 7);
                        }
                    }
                    if(et == 0)
                        HTB_STAMP(2, local, 5);
                    // hand the accumulator back: every epilogue thread of the pair arrives on the leader's barrier
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    const uint32_t emptyBarAddr = mapToRank(smemAddr(&tmemEmptyBar[acc]), leaderRank);
                    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(emptyBarAddr) : "memory");
                }
                for(; pa.ksplit > 1 && syncs < 2; syncs++)
                    clusterSync(); // a CTA whose wait ran out still meets the others
                // the bulk stores of this warp have read their shared-memory slots (the end of the grid makes their
                // writes visible, as for any store)
                if(pa.tmaStore && lane == 0)
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            }

            // ---------------------------------------------------------------- teardown
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if(threadIdx.x == 0)
                HTB_STAMP(3, 0, 2);
            clusterSync(); // all CTAs are done with tensor memory and with each other's barriers and shared memory
            if(threadIdx.x == 0)
                HTB_STAMP(3, 0, 3);
            if(threadIdx.x == 0 && abortFlag && a.status)
                atomicExch(a.status, 3);
            if(warp == 1)
            {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
            }
        }

        // Tensor map of a K-major operand: dimension 0 is the block K mode (contiguous), dimensions 1 .. n the folded
        // modes of the row group, then the other K modes (box 1). The map always has rank 5 (missing dimensions have
        // extent 1) so that the kernels use one fixed form of the load instruction with register coordinates.
        // kOther: the K modes after the block mode, `second` selects their stride (s0: operand A, s1: operand B).
        bool encodeOperand(PFN_encodeTiled encode, CUtensorMap* map, const void* base, bool bf16, const ModeDim* kModes,
                           int nk, bool second, const ModeDim* dims, int n, const int* box)
        {
            cuuint64_t gdim[5], gstr[4];
            cuuint32_t bx[5], estr[5] = {1, 1, 1, 1, 1};
            gdim[0] = cuuint64_t(kModes[0].ext);
            bx[0]   = kTileK;
            if(n + nk - 1 > 4)
                return false;
            for(int d = 0; d < 4; d++)
            {
                const bool    row  = d < n, kdim = !row && d - n < nk - 1;
                const int64_t ext  = row ? dims[d].ext : (kdim ? kModes[1 + d - n].ext : 1);
                const int64_t str  = row ? dims[d].s0 : (kdim ? (second ? kModes[1 + d - n].s1 : kModes[1 + d - n].s0) : 0);
                gdim[d + 1]        = ext > 1 ? cuuint64_t(ext) : 1;
                // a degenerate mode may carry stride 0: any 16-byte multiple is legal for extent 1
                gstr[d]   = ext > 1 ? cuuint64_t(str) * 2 : 16;
                bx[d + 1] = row ? cuuint32_t(box[d]) : 1;
                if(gstr[d] % 16 != 0 || gstr[d] == 0)
                    return false;
            }
            return encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                          const_cast<void*>(base), gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                   == CUDA_SUCCESS;
        }

        // Tensor map of an MN-major operand: {mode0 (stride 1), block K mode, mode1, mode2 (those the group has), the
        // other K modes}; one box is [64 k][64 rows]
        bool encodeOperandMn(PFN_encodeTiled encode, CUtensorMap* map, const void* base, bool bf16, const RowGroupView& g,
                             const ModeDim* kModes, int nk, bool second)
        {
            auto kStride = [&](int i) { return second ? kModes[i].s1 : kModes[i].s0; };
            cuuint64_t gdim[5] = {cuuint64_t(g.ext[0]), cuuint64_t(kModes[0].ext), 1, 1, 1},
                       gstr[4] = {cuuint64_t(kStride(0)) * 2, 16, 16, 16};
            cuuint32_t bx[5] = {64, kTileK, 1, 1, 1}, estr[5] = {1, 1, 1, 1, 1};
            if(g.n > 3 || (g.n - 1) + (nk - 1) > 3)
                return false;
            for(int d = 1; d < g.n; d++)
                if(g.ext[d] > 1)
                {
                    gdim[1 + d] = cuuint64_t(g.ext[d]);
                    gstr[d]     = cuuint64_t(g.sOp[d]) * 2;
                }
            for(int i = 1; i < nk; i++)
                if(kModes[i].ext > 1)
                {
                    gdim[g.n + i]     = cuuint64_t(kModes[i].ext);
                    gstr[g.n + i - 1] = cuuint64_t(kStride(i)) * 2;
                }
            for(int d = 0; d < 4; d++)
                if(gstr[d] % 16 != 0 || gstr[d] == 0)
                    return false;
            return encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                          const_cast<void*>(base), gdim, gstr, bx, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                   == CUDA_SUCCESS;
        }

        void fillGroupArgs(const ModeDim* dims, int n, const int* box, int* boxOut, int64_t* ext, int64_t* sD,
                           int* tilesPerDim, int& tiles)
        {
            tiles = 1;
            for(int d = 0; d < n; d++)
            {
                boxOut[d]      = box[d];
                ext[d]         = dims[d].ext;
                sD[d]          = dims[d].s1;
                tilesPerDim[d] = int((dims[d].ext + box[d] - 1) / box[d]);
                tiles *= tilesPerDim[d];
            }
        }

        template <typename TD>
        cudaError_t launchTyped(const ContractionPlan& p, float alpha, const void* A, const void* B, float beta,
                                const void* C, void* D, void* workspace, uint64_t workspaceBytes, int smCount,
                                int* status, cudaStream_t stream)
        {
            PFN_encodeTiled encode = tensorMapEncoder();
            if(!encode)
                return cudaErrorNotSupported;
            const bool  bf16 = (p.typeA == CUDA_R_16BF);
            // HTB_TC_PAIR: CTA pairs wherever they can run, not only where they pay off (tests of the pair kernel on
            // small problems)
            const Switches& sw = switches();
            const bool  pair = (p.pair != 0 || (p.pairOk != 0 && sw.tcPair)) && !sw.tcSingle;
            const int*  boxN = pair ? p.boxN128 : p.boxN;
            const int   layout = (p.aMajor ? 1 : 0) | (p.bMajor ? 2 : 0);
            const RowGroupView vm = viewOf(p.m, p.nm, p.aMajor ? 0 : -1), vn = viewOf(p.n, p.nn, p.bMajor ? p.nFast : -1);
            bool           cached = false;
            MapCacheEntry* maps   = mapCacheFind(p.cacheId, A, B, pair ? 1 : 0, &cached);
            CUtensorMap &  mapA = maps->mapA, &mapB = maps->mapB;
            if(!cached)
            {
                const bool okA = p.aMajor ? encodeOperandMn(encode, &mapA, A, bf16, vm, p.k, p.nk, false)
                                          : encodeOperand(encode, &mapA, A, bf16, p.k, p.nk, false, p.m, p.nm, p.boxM);
                const bool okB = p.bMajor ? encodeOperandMn(encode, &mapB, B, bf16, vn, p.k, p.nk, true)
                                          : encodeOperand(encode, &mapB, B, bf16, p.k, p.nk, true, p.n, p.nn, boxN);
                if(!okA || !okB)
                {
                    maps->id = 0; // not a usable entry
                    return cudaErrorNotSupported;
                }
            }

            TcArgs a{};
            a.nm = p.nm;
            a.nn = p.nn;
            const int ones[4] = {1, 1, 1, 1}; // MN-major groups have no boxes
            fillGroupArgs(p.m, p.nm, p.aMajor ? ones : p.boxM, a.boxM, a.extM, a.sDm, a.tilesPerDimM, a.tilesM);
            fillGroupArgs(p.n, p.nn, p.bMajor ? ones : boxN, a.boxN, a.extN, a.sDn, a.tilesPerDimN, a.tilesN);
            // chunked description of MN-major groups (64 half-precision elements per chunk)
            fillGroup(a.gm, vm, p.aMajor, 128, p.boxM, 6);
            fillGroup(a.gn, vn, p.bMajor, pair ? 128 : p.tileN, boxN, 6);
            if(p.aMajor)
                a.tilesM = a.gm.tiles;
            if(p.bMajor)
                a.tilesN = a.gn.tiles;
            // K blocks: 64-wide chunks of the block mode k[0], times the extents of the other K modes
            a.kfChunks = int((p.k[0].ext + kTileK - 1) / kTileK);
            a.kExt1    = p.nk > 1 ? int(p.k[1].ext) : 1;
            a.kExt2    = p.nk > 2 ? int(p.k[2].ext) : 1;
            a.kPosA    = p.nk > 1 ? (p.aMajor ? 1 + vm.n : 1 + p.nm) : 8;
            a.kPosB    = p.nk > 1 ? (p.bMajor ? 1 + vn.n : 1 + p.nn) : 8;
            if(p.nk > 3 || int64_t(a.kfChunks) * a.kExt1 * a.kExt2 > 0x7fffffffll)
                return cudaErrorNotSupported;
            a.kBlocks  = a.kfChunks * a.kExt1 * a.kExt2;
            a.tileN      = pair ? 256 : p.tileN;
            a.stages     = pair ? 6 : p.stages;
            a.stageBytes = uint32_t((p.aMajor ? 128 : p.rowsM) + (p.bMajor ? (pair ? 128 : p.tileN) : (pair ? p.rowsN128 : p.rowsN)))
                           * kTileK * 2;
            a.alpha      = alpha;
            a.beta       = beta;
            a.bilinear   = (p.bilinear && C != nullptr) ? 1 : 0;
            a.nContig    = (((p.bMajor && vn.sD[0] == 1) || (p.nn == 1 && p.n[0].s1 == 1)) && (uintptr_t(D) & 15) == 0
                         && (!a.bilinear || (uintptr_t(C) & 15) == 0))
                               ? 1
                               : 0;
            a.status     = status;
#ifdef HTB_MEASURE
            a.probe = sw.tcProbe;
            if(const char* env = getenv("HTB_TC_TRACE_PTR")) // device buffer of 4 * 4 * 8 * 8 words, made by the caller
                a.trace = (unsigned long long*)strtoull(env, nullptr, 0);
#endif
            if(int64_t(a.tilesM) * a.tilesN > 0x7fffffffll || a.stages > kMaxStages)
                return cudaErrorInvalidConfiguration;

            // instruction descriptor: fp32 accumulate, A/B format, transposed (MN-major) A / B, N/8, M/16
            const uint32_t fmt = bf16 ? 1u : 0u;
            const uint32_t majors = (p.aMajor ? (1u << 15) : 0u) | (p.bMajor ? (1u << 16) : 0u);
            const int      sms = smCount > 0 ? smCount : 148;
            if(pair)
            {
                // tile width and K split: the planner's choice (cost model in planner.cpp), narrowed here by what the
                // device grants (resident clusters) and by the variant switches
                const int  nsub   = ((p.wide || sw.tcWide) && !sw.tcNarrow) ? 2 : 1;
                const int  ksub   = nsub == 1 ? 2 : 1;
                TcPairArgs pa{};
                a.stages     = 192 * 1024 / int(ksub * (1 + nsub) * 16384);
                a.stageBytes = uint32_t(128 + nsub * 128) * kTileK * 2;
                pa.base      = a;
                pa.pairsM    = (a.tilesM + 1) / 2;
                pa.groupsN   = (a.tilesN + 2 * nsub - 1) / (2 * nsub);
                pa.iters     = (a.kBlocks + ksub - 1) / ksub;
                pa.ksplit    = 1;
                const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | majors | (uint32_t(256 >> 3) << 17)
                                       | (uint32_t(256 >> 4) << 24);
                using PairKernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const CUtensorMap, const TD*,
                                            TD*, TcPairArgs, uint32_t);
                static const PairKernel kernels[2][4] = {
                    {contraction_tcgen05_pair_kernel<TD, 0, 1>, contraction_tcgen05_pair_kernel<TD, 1, 1>,
                     contraction_tcgen05_pair_kernel<TD, 2, 1>, contraction_tcgen05_pair_kernel<TD, 3, 1>},
                    {contraction_tcgen05_pair_kernel<TD, 0, 2>, contraction_tcgen05_pair_kernel<TD, 1, 2>,
                     contraction_tcgen05_pair_kernel<TD, 2, 2>, contraction_tcgen05_pair_kernel<TD, 3, 2>}};
                PairKernel kernel = kernels[nsub - 1][layout];
                // pipeline stages, alignment slack, and 32 KiB behind the stages for the TMA-store slots (or the table of
                // column offsets of the plain stores)
                const size_t smem = size_t(192) * 1024 + 1024 + 32 * 1024;
                cudaError_t  e    = ensureDynamicSmem((const void*)kernel, int(smem));
                if(e != cudaSuccess)
                    return e;
                cudaLaunchConfig_t cfg{};
                cudaLaunchAttribute attr[2];
                attr[0].id               = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = 2;
                attr[0].val.clusterDim.y = 1;
                attr[0].val.clusterDim.z = 1;
                // this kernel may start while the kernel before it in the stream drains (see griddepcontrol in the kernel)
                attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
                attr[1].val.programmaticStreamSerializationAllowed = 1;
                cfg.blockDim             = dim3(unsigned(64 + 128 * nsub));
                cfg.dynamicSmemBytes     = smem;
                cfg.stream               = stream;
                cfg.attrs                = attr;
                cfg.numAttrs             = sw.tcNoPdl ? 1 : 2;
                // clusters of two and of four CTAs that can be resident at once (GPCs with an odd SM count lose an SM);
                // per device, the same for every instantiation: one CTA per SM
                static std::atomic<int> clustersOf[kMaxDevices][2];
                int                     dev = 0;
                cudaGetDevice(&dev);
                const bool devOk  = dev >= 0 && dev < kMaxDevices;
                auto       resident = [&](int csize) {
                    const int slot = csize == 2 ? 0 : 1;
                    int       n    = devOk ? clustersOf[dev][slot].load(std::memory_order_relaxed) : 0;
                    if(n == 0)
                    {
                        attr[0].val.clusterDim.x = unsigned(csize);
                        cfg.gridDim              = dim3(unsigned(sms / csize * csize));
                        if(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0)
                        {
                            cudaGetLastError();
                            n = csize == 2 ? sms / 2 : sms / 8; // a cautious guess for clusters of four
                        }
                        if(devOk)
                            clustersOf[dev][slot].store(n, std::memory_order_relaxed);
                    }
                    return n;
                };
                const int     maxClusters = resident(2);
                const int64_t tiles       = int64_t(pa.pairsM) * pa.groupsN;
                pa.fullUnits = int(tiles);
                pa.numUnits  = int(tiles);
                // K split over clusters of four CTAs: every tile gets two pairs, all of them resident at once, each
                // K range at least eight stages long
                if((p.ksplit == 2 || sw.tcKsplit) && !sw.tcNoSplit && pa.iters >= (sw.tcKsplit ? 2 : 16) && tiles <= resident(4))
                    pa.ksplit = 2;
                // A 128-column sub-tile on its own (64 rows of B per CTA, MMAs with N = 128). K-major B needs its 128-row
                // sub-tile to be one box along the first N mode, so that rows 64.. are a coordinate offset, and a second
                // tensor map with 64-row boxes; an MN-major B loads one 64-row chunk instead of two.
                CUtensorMap mapB64 = mapB; // stays a copy of B's map (unused by the kernel) when single sub-tiles cannot run
                pa.singleOk        = p.bMajor ? 1 : 0;
                if(!p.bMajor)
                {
                    if(maps->half == 0)
                    {
                        const int box64[4] = {64, 1, 1, 1};
                        maps->half = (p.boxN128[0] == 128 && encodeOperand(encode, &maps->mapB64, B, bf16, p.k, p.nk, true, p.n, p.nn, box64))
                                         ? 1
                                         : 2;
                    }
                    if(maps->half == 1)
                    {
                        mapB64      = maps->mapB64;
                        pa.singleOk = 1;
                    }
                }
                pa.idescHalf = (1u << 4) | (fmt << 7) | (fmt << 10) | majors | (uint32_t(128 >> 3) << 17)
                               | (uint32_t(256 >> 4) << 24);
                // Half tiles (256 x 256 tiles): a last wave (or the only one) that is at most half full: its tiles run as
                // two units of one sub-tile each. The N sub-tiles must pair up evenly.
                if(nsub == 1 && pa.ksplit == 1 && !sw.tcNoHalf && a.tilesN % 2 == 0 && pa.singleOk)
                {
                    const int64_t tail = tiles % maxClusters;
                    if(tail > 0 && 2 * tail <= maxClusters)
                    {
                        pa.halves    = 1;
                        pa.fullUnits = int(tiles - tail);
                        pa.numUnits  = int(tiles + tail);
                    }
                }
                const int64_t clustersUsed = pa.ksplit > 1 ? int64_t(pa.numUnits) : std::min<int64_t>(pa.numUnits, maxClusters);
                // Output by bulk tensor stores: fp32 D with one folded row mode and one contiguous column mode, no C
                // (a tensor map needs 16-byte aligned base and row stride)
                pa.storeOffset = uint32_t(192 * 1024);
                pa.storeBufs   = 1;
                CUtensorMap mapD = mapA; // a valid map even when unused
                if(sizeof(TD) == 4 && p.typeD == CUDA_R_32F && !a.bilinear && !sw.tcNoTmaStore && p.nm == 1 && p.nn == 1
                   && p.n[0].s1 == 1 && (p.m[0].s1 % 4) == 0 && (uintptr_t(D) & 15) == 0 && p.N < (int64_t(1) << 31)
                   && p.M < (int64_t(1) << 31) && (p.m[0].ext == 1 || p.m[0].s1 >= p.N))
                {
                    if(maps->D != D)
                    {
                        cuuint64_t gdim[2] = {cuuint64_t(p.N), cuuint64_t(p.M)}, gstr[1] = {cuuint64_t(p.m[0].s1) * 4};
                        cuuint32_t bx[2] = {32, 32}, estr[2] = {1, 1};
                        if(gstr[0] == 0)
                            gstr[0] = cuuint64_t(p.N) * 4;
                        const bool ok = encode(&maps->mapD, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, D, gdim, gstr, bx, estr,
                                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                               CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                                        == CUDA_SUCCESS;
                        maps->D = ok ? D : nullptr;
                    }
                    if(maps->D == D)
                    {
                        mapD        = maps->mapD;
                        pa.tmaStore = 1;
                        if(pa.ksplit > 1)
                        {
                            // the exchange zone takes the first (tile columns / 2) x 512 bytes of the idle stage memory
                            pa.storeOffset = uint32_t(128 * nsub * 512);
                            pa.storeBufs   = nsub == 1 ? 4 : 2;
                        }
                        else
                            pa.storeBufs = nsub == 1 ? 2 : 1;
                    }
                }
                HTB_LOG_HEUR("hiptensorContraction",
                             "pair kernel: %lld tiles of 256 x %d on %d CTA pairs, K split %d, %s, %d work units",
                             (long long)tiles, 256 * nsub, maxClusters, pa.ksplit, pa.halves ? "last wave in half tiles" : "whole tiles",
                             pa.numUnits);
                // one cluster per work unit, as many as can be resident
                attr[0].val.clusterDim.x = unsigned(2 * pa.ksplit);
                cfg.gridDim = dim3(unsigned(2 * pa.ksplit * clustersUsed));
                e           = cudaLaunchKernelEx(&cfg, kernel, mapA, mapB, mapB64, mapD, (const TD*)C, (TD*)D, pa, idesc);
                if(e == cudaSuccess)
                    noteLaunch(nsub == 2 ? "contraction_tcgen05_pair_wide" : "contraction_tcgen05_pair");
                return e;
            }
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | majors | (uint32_t(p.tileN >> 3) << 17)
                                   | (uint32_t(kTileM >> 4) << 24);
            const size_t smem = size_t(a.stages) * (size_t(kTileM) + p.tileN) * kTileK * 2 + 1024;
            using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const TD*, TD*, TcArgs, uint32_t);
            static const Kernel kernels[4] = {contraction_tcgen05_kernel<TD, 0>, contraction_tcgen05_kernel<TD, 1>,
                                              contraction_tcgen05_kernel<TD, 2>, contraction_tcgen05_kernel<TD, 3>};
            Kernel      kernel = kernels[layout];
            cudaError_t e = ensureDynamicSmem((const void*)kernel, int(smem));
            if(e != cudaSuccess)
                return e;
            // Few tiles and a long K: up to four CTAs per tile (one cluster), at least eight K blocks each (with fewer the
            // hand-over costs more than it saves: 512^3 11.3 us whole, 13.3 split), every unit on
            // its own SM; the accumulators of parts 1.. must fit into part 0's stages.
            const int64_t numTiles = int64_t(a.tilesM) * a.tilesN;
            a.parts                = 1;
            if(!sw.tcNoSplit)
            {
                const int64_t byTiles = sms / std::max<int64_t>(numTiles, 1), byK = a.kBlocks / 8;
                const int64_t byRoom  = 1 + int64_t(size_t(a.stages) * (size_t(kTileM) + p.tileN) * kTileK * 2)
                                               / (int64_t(kTileM) * p.tileN * 4);
                const int64_t q = std::min<int64_t>(std::min<int64_t>(4, byTiles), std::min<int64_t>(byK, byRoom));
                if(q >= 2)
                    a.parts = int(q);
            }
            // a cluster per tile when K is split (else clusters of one CTA), programmatic dependent launch
            cudaLaunchConfig_t  cfg{};
            cudaLaunchAttribute attr[2];
            attr[0].id                                         = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x                           = unsigned(a.parts);
            attr[0].val.clusterDim.y                           = 1;
            attr[0].val.clusterDim.z                           = 1;
            attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.gridDim          = dim3(unsigned(a.parts > 1 ? numTiles * a.parts : std::min<int64_t>(numTiles, sms)));
            cfg.blockDim         = dim3(kThreads);
            cfg.dynamicSmemBytes = smem;
            cfg.stream           = stream;
            cfg.attrs            = attr;
            cfg.numAttrs         = sw.tcNoPdl ? 1 : 2;
            e                    = cudaLaunchKernelEx(&cfg, kernel, mapA, mapB, (const TD*)C, (TD*)D, a, idesc);
            if(e == cudaSuccess)
                noteLaunch("contraction_tcgen05");
            return e;
        }
    } // namespace

    cudaError_t launchContractionTcgen05(const ContractionPlan& plan, float alpha, const void* A, const void* B,
                                         float beta, const void* C, void* D, void* workspace, uint64_t workspaceBytes,
                                         int smCount, int* deviceStatus, cudaStream_t stream)
    {
        switch(plan.typeD)
        {
        case CUDA_R_32F:
            return launchTyped<float>(plan, alpha, A, B, beta, C, D, workspace, workspaceBytes, smCount, deviceStatus,
                                      stream);
        case CUDA_R_16F:
            return launchTyped<__half>(plan, alpha, A, B, beta, C, D, workspace, workspaceBytes, smCount, deviceStatus,
                                       stream);
        case CUDA_R_16BF:
            return launchTyped<__nv_bfloat16>(plan, alpha, A, B, beta, C, D, workspace, workspaceBytes, smCount,
                                              deviceStatus, stream);
        }
        return cudaErrorNotSupported;
    }
} // namespace htb
