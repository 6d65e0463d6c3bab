// Tensor-core contraction for fp32 operands on sm_100a with fp32-grade accuracy (the "3xTF32" split):
//
//   D[m, n] = alpha * sum_k A[m, k] * B[n, k]  (+ beta * C[m, n]),   A, B, C, D fp32, compute type fp32.
//
// Every operand element x is split into big = tf32(x) and small = tf32(x - big); the tensor cores
// accumulate  small_a*big_b + big_a*small_b + big_a*big_b  in fp32 in tensor memory. The dropped
// small*small term is below 2^-22 of the product, i.e. below fp32 rounding of the sum.
//
// With compute type f16 or bf16 (fp32 data whose elements the reference first converts to the compute type,
// contraction_cpu_reference_impl.hpp:359-384) the converter rounds each element to that type instead: the result
// is exactly representable in TF32, so one MMA per K step multiplies exactly what the reference multiplies.
//
// kind::tf32 takes K-major shared-memory operands only, so the split doubles as the layout change:
//   TMA            strided tensor -> staging tile, in whichever order the operand is contiguous:
//                    K-major operand  : one box  [rows x 32 k], 128-byte swizzle, rows gathered over the
//                                       folded modes of the row group;
//                    MN-major operand : one box per 32 rows [32 k x 32 rows], the 32 rows being
//                                       consecutive elements of the group's stride-1 mode;
//   converter      8 warps, two threads per tile row (16 k each): read from staging (conflict-free in
//                  both orders), split, write the big and the small half row into the K-major,
//                  128-byte-swizzled operand ring;
//   tcgen05.mma    three MMAs per 8-wide K step from the ring: the main product into a segment accumulator that
//                  the epilogue drains every 64 K elements, the two correction products into their own;
//   epilogue       tcgen05.ld, running sums in registers, alpha/beta, stores to the strided D.
// When both operands are K-major the staging step is skipped (INPLACE): TMA writes into the ring's big tiles and
// the converter only adds the small ones. Small problems are cut along K over the CTAs of a thread-block cluster
// (parts); the partial sums go to the owner's shared memory over the cluster network.
//
// Warp roles (576 threads): 0 TMA producer, 1 MMA issuer + tensor-memory owner, 2-9 epilogue (two warps
// per tensor-memory lane quadrant, 64 columns each), 10-17 converter. PAIR = true runs a 256 x 128 tile
// on a cluster of two CTAs (cta_group::2): each CTA stages and converts its own 128 rows of A and 64 of
// the 128 rows of B; the leader CTA issues the MMAs for both. Loads carry no multicast qualifier.
//
// All mbarrier waits are bounded; on a timeout the kernel raises the device status word, skips the
// remaining work and frees its tensor memory.
//
// It stands where the reference instantiates CK's xdl contraction kernels for f32
// (library/src/contraction/device/*f32_f32_f32_f32*_instance.cpp, compute type f32).
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
        constexpr int      kTfThreads    = 576;
        constexpr int      kEpiWarps = 8, kConvWarps = 8; // warps 2..9 and 10..17
        constexpr int      kTfK          = 32; // fp32 elements per K block = one 128-byte swizzle row
        constexpr uint32_t kTileBytes    = 128 * kTfK * 4; // 16 KiB: 128 rows of one K block
        constexpr int      kMaxSlots     = 4;

        // Shared-memory rings. A staging slot holds the raw A rows and B rows of one K block, an operand slot
        // A big, A small, B big, B small. A CTA of a pair carries 64 rows of B and so affords three slots of each.
        // INPLACE (both operands K-major, compute f32): TMA writes the raw rows straight into the "big" tiles of an
        // operand slot - the tensor cores read fp32 bits as TF32 by dropping the low 13 mantissa bits - and the
        // converter adds only the small tiles. No staging ring, three operand slots, a third less conversion traffic.
        template <bool PAIR, bool INPLACE>
        struct TfRing
        {
            static constexpr uint32_t kBBytes       = PAIR ? kTileBytes / 2 : kTileBytes;
            static constexpr int      kStagingSlots = INPLACE ? 0 : (PAIR ? 3 : 2), kOpSlots = (PAIR || INPLACE) ? 3 : 2;
            static constexpr uint32_t kStagingBytes = kTileBytes + kBBytes;
            static constexpr uint32_t kOpBytes      = 2 * kTileBytes + 2 * kBBytes;
            static constexpr uint32_t kTotal        = kStagingSlots * kStagingBytes + kOpSlots * kOpBytes;
        };

        struct TfArgs
        {
            TfGroup  gm, gn;
            int      boxK[2], kTilesPerDim[2]; // K block -> coordinates of the (at most two) folded K modes
            int      kBlocks;
            uint32_t bytesA, bytesB; // TMA bytes per K block into one CTA's staging slot
            float    alpha, beta;
            int      bilinear;
            int      nContig; // 32 consecutive columns of a tile are 32 consecutive, 16-byte aligned floats of D
            int      pairsM, pairsN; // PAIR only
            // K split of small problems (single CTAs only): every tile is cut into `parts` ranges of K blocks, one CTA
            // each, launched as one thread-block cluster per tile. Part 0 owns the tile: when every part has its sums,
            // parts 1.. store theirs into part 0's (by then idle) shared-memory rings over the cluster network, and part 0
            // adds them in order and applies alpha/beta.
            int      parts;
            int      round; // 0: big/small split (compute f32); 1 / 2: elements rounded to f16 / bf16, one MMA per K step
#ifdef HTB_MEASURE
            int      probe; // measurement builds only, bit mask: 1 = converter skips its work, 2 = issuer skips the
                            // MMAs, 8 = producer skips the loads (results invalid)
#define HTB_TF_PROBE(args, bit) ((args).probe & (bit))
#else
#define HTB_TF_PROBE(args, bit) 0
#endif
            int*     status;
        };

        // TMA loads of one operand's rows of one K block into a staging tile
        //   major 0 map: {K, mode0, mode1, mode2, mode3}         one box
        //   major 1 map: {mode0, k0, k1, mode1, mode2}           one box per 32-row chunk
        __device__ __forceinline__ void tfLoadRows(const TfGroup& g, const TfTile& w, const TfChunks& q, const CUtensorMap* map,
                                                   uint32_t dst, uint32_t bar, int kb, int kc0, int kc1)
        {
            if(g.major == 0)
            {
                const int c[5] = {kb * kTfK, w.c[0], w.c[1], w.c[2], w.c[3]};
                tmaLoad<5>(dst, map, bar, c);
                return;
            }
#pragma unroll
            for(int j = 0; j < 4; j++)
            {
                if(j < (g.rows >> 5))
                {
                    const int c[5] = {q.c0[j], kc0, kc1, q.i1[j], q.i2[j]};
                    tmaLoad<5>(dst + uint32_t(j) * (kTfK * 128), map, bar, c);
                }
            }
        }

        // big = x rounded to TF32 (nearest, ties away: add half an ulp to the magnitude, drop 13 bits),
        // small = x - big, exact in fp32; the tensor cores drop the last bits of small, 2^-21 of x.
        __device__ __forceinline__ float tfBig(float x)
        {
            return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
        }
        // elements rounded to f16 (ROUND == 1) or bf16 (ROUND == 2) and widened again; no small part
        template <int ROUND>
        __device__ __forceinline__ float tfRound(float x)
        {
            if(ROUND == 1)
                return __half2float(__float2half_rn(x));
            return __bfloat162float(__float2bfloat16_rn(x));
        }
        template <int ROUND>
        __device__ __forceinline__ float4 tfRound4(const float4& v)
        {
            return make_float4(tfRound<ROUND>(v.x), tfRound<ROUND>(v.y), tfRound<ROUND>(v.z), tfRound<ROUND>(v.w));
        }
        __device__ __forceinline__ void tfSplit4(const float4& v, float4& b, float4& s)
        {
            b.x = tfBig(v.x);
            b.y = tfBig(v.y);
            b.z = tfBig(v.z);
            b.w = tfBig(v.w);
            s.x = v.x - b.x;
            s.y = v.y - b.y;
            s.z = v.z - b.z;
            s.w = v.w - b.w;
            // an infinite big (x infinite, or rounded up past the largest finite value) must not make a NaN small
            if(!(fabsf(b.x) + fabsf(b.y) + fabsf(b.z) + fabsf(b.w) < INFINITY))
            {
                s.x = (fabsf(b.x) < INFINITY) ? s.x : 0.f;
                s.y = (fabsf(b.y) < INFINITY) ? s.y : 0.f;
                s.z = (fabsf(b.z) < INFINITY) ? s.z : 0.f;
                s.w = (fabsf(b.w) < INFINITY) ? s.w : 0.f;
            }
        }

        __device__ __forceinline__ float4 lds128(uint32_t addr)
        {
            float4 v;
            asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
            return v;
        }
        __device__ __forceinline__ float lds32(uint32_t addr)
        {
            float v;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
            return v;
        }
        __device__ __forceinline__ void sts128(uint32_t addr, float4 v)
        {
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
        }

        // Conversion of a rows x 32 tile by the 256 converter threads (thread: row r = 0..127, K half h):
        // staging -> (big, small) in the K-major ring layout, where the 16-byte piece j of row r sits at
        // r*128 + ((j ^ (r & 7)) << 4).
        // round: 0 = big/small split, 1 = round to f16, 2 = round to bf16 (big tile only)
        __device__ __forceinline__ void tfConvertRow(int major, uint32_t src, uint32_t dstBig, uint32_t dstSmall, int r, int h, int rows,
                                                     int round)
        {
            const uint32_t rowOff = uint32_t(r) * 128;
            if(major == 0)
            {
                // Staging has the ring layout already (TMA 128-byte swizzle): the copy is position by position. Eight
                // consecutive threads take the eight 16-byte pieces of one row, a warp four rows, the 256 converter
                // threads 32 rows per pass.
                const int t = r + 128 * h; // converter thread index
#pragma unroll
                for(int pass = 0; pass < 4; pass++)
                {
                    if(pass * 32 >= rows)
                        break;
                    const uint32_t off = uint32_t(pass * 32 + (t >> 3)) * 128 + (uint32_t(t & 7) << 4);
                    const float4   v   = lds128(src + off);
                    if(round == 0)
                    {
                        float4 b, s;
                        tfSplit4(v, b, s);
                        sts128(dstBig + off, b);
                        sts128(dstSmall + off, s);
                    }
                    else
                        sts128(dstBig + off, round == 1 ? tfRound4<1>(v) : tfRound4<2>(v));
                }
            }
            else if(r < rows)
            {
                // staging: chunk r/32 holds [32 k][32 rows], unswizzled; the lanes of a warp read 32 consecutive floats
                const uint32_t col = src + uint32_t(r >> 5) * (kTfK * 128) + uint32_t(r & 31) * 4 + uint32_t(h) * (16 * 128);
                float          x[16];
#pragma unroll
                for(int k = 0; k < 16; k++)
                    x[k] = lds32(col + uint32_t(k) * 128);
#pragma unroll
                for(int jj = 0; jj < 4; jj++)
                {
                    const uint32_t off = rowOff + (uint32_t((4 * h + jj) ^ (r & 7)) << 4);
                    const float4   v   = make_float4(x[4 * jj], x[4 * jj + 1], x[4 * jj + 2], x[4 * jj + 3]);
                    if(round == 0)
                    {
                        float4 b, s;
                        tfSplit4(v, b, s);
                        sts128(dstBig + off, b);
                        sts128(dstSmall + off, s);
                    }
                    else
                        sts128(dstBig + off, round == 1 ? tfRound4<1>(v) : tfRound4<2>(v));
                }
            }
        }

        // In-place variant: the tile at `big` holds the raw fp32 rows (K-major, TMA-swizzled); write the small tile.
        // The tensor cores will use big = x with the low 13 mantissa bits dropped, so small = x - that, rounded to
        // TF32 (nearest, by integer add-and-mask) so that their truncation of it loses nothing more.
        __device__ __forceinline__ void tfConvertSmall(uint32_t big, uint32_t dstSmall, int t, int rows)
        {
#pragma unroll
            for(int pass = 0; pass < 4; pass++)
            {
                if(pass * 32 >= rows)
                    break;
                const uint32_t off = uint32_t(pass * 32 + (t >> 3)) * 128 + (uint32_t(t & 7) << 4);
                const float4   v   = lds128(big + off);
                const float    x[4] = {v.x, v.y, v.z, v.w};
                float          sm[4];
#pragma unroll
                for(int e = 0; e < 4; e++)
                {
                    const float b = __uint_as_float(__float_as_uint(x[e]) & 0xFFFFE000u);
                    const float r = x[e] - b; // exact
                    sm[e]         = tfBig(r);
                }
                // infinite or NaN elements: keep them in the big part only
                if(!(fabsf(v.x) + fabsf(v.y) + fabsf(v.z) + fabsf(v.w) < INFINITY))
                {
#pragma unroll
                    for(int e = 0; e < 4; e++)
                        sm[e] = (fabsf(x[e]) < INFINITY) ? sm[e] : 0.f;
                }
                sts128(dstSmall + off, make_float4(sm[0], sm[1], sm[2], sm[3]));
            }
        }

        // Bounded wait, executed by every thread of the waiting warp: a tight try_wait loop, the clock is read only
        // every 256th unsuccessful poll.
        __device__ __forceinline__ bool tfWait(uint32_t bar, uint32_t parity, volatile int* abortFlag)
        {
            long long t0 = 0;
            for(uint32_t it = 1;; it++)
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

        // Accumulation. The tensor cores add each 8-wide group of products to the fp32 accumulator with
        // truncation, which over a long K would cost several digits. So
        //   * the two correction products (small*big, big*small), whose sum is 2^-11 of the result and whose
        //     truncation error is therefore negligible, go to an accumulator of their own for the whole tile;
        //   * the main product (big*big) is accumulated over kSegBlocks K blocks only, then the epilogue warps
        //     add that segment to running sums held in registers (round to nearest) while the tensor cores
        //     fill the other segment accumulator.
        // Tensor memory, 512 columns per CTA: segment accumulators at columns 0 and 128, correction
        // accumulators (double buffered across tiles) at 256 and 384.
        constexpr int kSegBlocks = 2;

        template <bool PAIR, bool INPLACE>
        __global__ void __launch_bounds__(kTfThreads, 1)
            contraction_tf32x3_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                      const float* C, float* D, TfArgs a, uint32_t idesc) // C may alias D
        {
            extern __shared__ unsigned char smemRaw[];
            unsigned char* tiles = (unsigned char*)((uintptr_t(smemRaw) + 1023) & ~uintptr_t(1023));

            using Ring = TfRing<PAIR, INPLACE>;
            static_assert(!(PAIR && INPLACE), "the in-place ring is built for single CTAs");
            constexpr int      kStagingSlots = Ring::kStagingSlots, kOpSlots = Ring::kOpSlots;
            constexpr int      kLoadSlots = INPLACE ? kOpSlots : kStagingSlots; // slots that TMA writes
            constexpr uint32_t kStagingBytes = Ring::kStagingBytes, kOpBytes = Ring::kOpBytes, kBBytes = Ring::kBBytes;
            __shared__ __align__(8) unsigned long long stFullBar[kMaxSlots], stEmptyBar[kMaxSlots];
            __shared__ __align__(8) unsigned long long opFullBar[kMaxSlots], opEmptyBar[kMaxSlots];
            __shared__ __align__(8) unsigned long long segFullBar[2], segEmptyBar[2], corrFullBar[2], corrEmptyBar[2];
            __shared__ uint32_t tmemBase;
            __shared__ int      abortFlag;
            __shared__ int64_t  colOff[kEpiWarps][64]; // one table per epilogue warp

            const int      warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
            const uint32_t rank   = PAIR ? clusterRank() : 0u;
            const bool     leader = (rank == 0);
            const int      ctas   = PAIR ? 2 : 1;
            const int      worker = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x); // CTA or CTA pair
            const int      numWorkers = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);
            const int      parts      = PAIR ? 1 : a.parts;
            const int      numUnits   = PAIR ? a.pairsM * a.pairsN : a.gm.tiles * a.gn.tiles * parts;
            const int      unitsM     = PAIR ? a.pairsM : a.gm.tiles;
            const int      accCols    = ctas * a.gn.rows; // accumulator columns per tile (a pair: two 64-row B tiles)
            // K blocks of a unit: part (u % parts) of tile (u / parts)
            auto kRange = [&](int u, int& kb0, int& kb1) {
                const int part = u % parts;
                kb0            = int((long long)a.kBlocks * part / parts);
                kb1            = int((long long)a.kBlocks * (part + 1) / parts);
            };
            constexpr uint32_t kTmemCols = 512;

            if(threadIdx.x == 32)
            {
                prefetchTensorMap(&mapA);
                prefetchTensorMap(&mapB);
            }
            if(threadIdx.x == 0)
            {
                abortFlag = 0;
                for(int s = 0; s < kLoadSlots; s++)
                {
                    mbarInit(smemAddr(&stFullBar[s]), 1);
                    mbarInit(smemAddr(&stEmptyBar[s]), kConvWarps);
                }
                for(int s = 0; s < kOpSlots; s++)
                {
                    mbarInit(smemAddr(&opFullBar[s]), kConvWarps * ctas); // converter warps of the whole pair (leader's copy is used)
                    mbarInit(smemAddr(&opEmptyBar[s]), 1);
                }
                for(int i = 0; i < 2; i++)
                {
                    mbarInit(smemAddr(&segFullBar[i]), 1);
                    mbarInit(smemAddr(&segEmptyBar[i]), kEpiWarps * ctas); // one arrival per epilogue warp
                    mbarInit(smemAddr(&corrFullBar[i]), 1);
                    mbarInit(smemAddr(&corrEmptyBar[i]), kEpiWarps * ctas);
                }
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            if(warp == 1)
            {
                if(PAIR)
                {
                    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemBase)),
                                 "r"(kTmemCols)
                                 : "memory");
                    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
                }
                else
                {
                    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(&tmemBase)),
                                 "r"(kTmemCols)
                                 : "memory");
                    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if(PAIR)
                clusterSync(); // the peer's barriers exist before anything signals them
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem      = tmemBase;
            volatile int*  abortP    = &abortFlag;
            const uint32_t stagingAddr = smemAddr(tiles);
            const uint32_t opAddr      = stagingAddr + kStagingSlots * kStagingBytes;
            const uint32_t stFull = smemAddr(&stFullBar[0]), stEmpty = smemAddr(&stEmptyBar[0]);
            const uint32_t opFull = smemAddr(&opFullBar[0]), opEmpty = smemAddr(&opEmptyBar[0]);
            const uint32_t segFull = smemAddr(&segFullBar[0]), segEmpty = smemAddr(&segEmptyBar[0]);
            const uint32_t corrFull = smemAddr(&corrFullBar[0]), corrEmpty = smemAddr(&corrEmptyBar[0]);

            // this CTA's row tiles of a unit (a pair's second CTA takes the next tile of each group;
            // past the edge it repeats the last one and its results are not stored)
            auto tilesOf = [&](int u, int& tm, int& tn) {
                const int t  = u / parts;
                const int um = t % unitsM, un = t / unitsM;
                tm = PAIR ? min(2 * um + int(rank), a.gm.tiles - 1) : um;
                tn = PAIR ? min(2 * un + int(rank), a.gn.tiles - 1) : un;
            };
            // signal a barrier of the issuing CTA from any CTA of the pair / commit MMAs to both CTAs
            auto arriveIssuer = [&](uint32_t bar) {
                if(PAIR)
                    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(mapToRank(bar, 0)) : "memory");
                else
                    mbarArrive(bar);
            };
            auto commitTo = [&](uint32_t bar) {
                if(PAIR)
                    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
                                 "h"((unsigned short)3)
                                 : "memory");
                else
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
            };
            auto mma = [&](uint32_t d, uint64_t da, uint64_t db, uint32_t accumulate) {
                if(PAIR)
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
                                 "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
                                 : "memory");
                else
                    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d),
                                 "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
                                 : "memory");
            };

            if(warp == 0)
            {
                // ---------------------------------------------------------------- TMA producer
                // The whole warp waits (a warp that waits converged is woken promptly; a single diverged lane is not),
                // lane 0 issues.
                {
                    uint32_t slot = 0, phase = 0;
                    bool     ok = true;
                    for(int u = worker; u < numUnits && ok; u += numWorkers)
                    {
                        int tm, tn;
                        tilesOf(u, tm, tn);
                        const TfTile   wm = tfTileOf(a.gm, tm), wn = tfTileOf(a.gn, tn);
                        const TfChunks qm = tfChunksOf(a.gm, wm), qn = tfChunksOf(a.gn, wn);
                        int kb0, kb1;
                        kRange(u, kb0, kb1);
                        // K coordinates of the block (MN-major operands)
                        int kq = kb0 % a.kTilesPerDim[0], kc0 = kq * a.boxK[0], kc1 = (kb0 / a.kTilesPerDim[0]) * a.boxK[1];
                        for(int kb = kb0; kb < kb1; kb++)
                        {
                            // a free slot: of the staging ring (released by the converter) or, in place, of the operand
                            // ring (released by the MMAs that read it)
                            ok = __all_sync(0xffffffffu, tfWait((INPLACE ? opEmpty : stEmpty) + 8 * slot, phase ^ 1, abortP));
                            if(!ok)
                                break;
                            if(lane == 0)
                            {
                                const uint32_t bar = stFull + 8 * slot;
                                if(HTB_TF_PROBE(a, 8))
                                    mbarArrive(bar);
                                else
                                {
                                    mbarArriveExpectTx(bar, a.bytesA + a.bytesB);
                                    const uint32_t dst  = INPLACE ? opAddr + slot * kOpBytes : stagingAddr + slot * kStagingBytes;
                                    const uint32_t dstB = dst + (INPLACE ? 2 * kTileBytes : kTileBytes);
                                    tfLoadRows(a.gm, wm, qm, &mapA, dst, bar, kb, kc0, kc1);
                                    tfLoadRows(a.gn, wn, qn, &mapB, dstB, bar, kb, kc0, kc1);
                                }
                            }
                            __syncwarp();
                            kc0 += a.boxK[0];
                            if(++kq == a.kTilesPerDim[0])
                            {
                                kq  = 0;
                                kc0 = 0;
                                kc1 += a.boxK[1];
                            }
                            if(++slot == kLoadSlots)
                            {
                                slot = 0;
                                phase ^= 1;
                            }
                        }
                    }
                }
                if(parts > 1)
                {
                    clusterSync(); // the two meeting points of the K-split hand-over (see the epilogue)
                    clusterSync();
                }
            }
            else if(warp == 1)
            {
                // ---------------------------------------------------------------- MMA issuer (leader CTA of a pair)
                // the whole warp waits, lane 0 issues
                if(leader)
                {
                    const uint64_t descBase = smemDesc(opAddr);
                    const uint32_t descLo = uint32_t(descBase), descHi = uint32_t(descBase >> 32);
                    auto           descOf = [&](uint32_t lo) { return (uint64_t(descHi) << 32) | lo; };
                    uint32_t       slot = 0, phase = 0;
                    uint32_t       seg = 0; // running count of segments: buffer seg & 1, use (seg >> 1)
                    int            local = 0;
                    bool           ok    = true;
                    for(int u = worker; u < numUnits && ok; u += numWorkers, local++)
                    {
                        const int      cb     = local & 1;
                        const uint32_t dCorr  = tmem + 256u + uint32_t(cb) * 128u;
                        bool           corrReady = false;
                        int            kb0, kb1;
                        kRange(u, kb0, kb1);
                        for(int kb = kb0; kb < kb1; kb++)
                        {
                            const bool     segStart = ((kb - kb0) % kSegBlocks) == 0;
                            const uint32_t sb       = seg & 1;
                            if(segStart)
                            {
                                ok = __all_sync(0xffffffffu, tfWait(segEmpty + 8 * sb, ((seg >> 1) & 1) ^ 1, abortP));
                                if(!ok)
                                    break;
                            }
                            if(!corrReady)
                            {
                                // the epilogue must have read this correction accumulator's previous tile
                                ok = __all_sync(0xffffffffu, tfWait(corrEmpty + 8 * cb, ((local >> 1) & 1) ^ 1, abortP));
                                if(!ok)
                                    break;
                                corrReady = true;
                            }
                            ok = __all_sync(0xffffffffu, tfWait(opFull + 8 * slot, phase, abortP));
                            if(!ok)
                                break;
                            if(lane == 0)
                            {
                                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                                const uint32_t dMain = tmem + sb * 128u;
                                // Descriptors differ in their low word only (the start address in 16-byte units, which
                                // cannot carry out of its field): four running low words, advanced by 2 units (8 fp32 =
                                // 32 bytes) per K step, keep the issue loop short. The tensor cores need 64 cycles per
                                // MMA; a longer issue sequence would leave them idle.
                                uint32_t aBig = descLo + slot * (kOpBytes >> 4);
                                uint32_t aSml = aBig + (kTileBytes >> 4), bBig = aBig + (2 * kTileBytes >> 4),
                                         bSml = bBig + (kBBytes >> 4);
                                if(!(HTB_TF_PROBE(a, 2)))
                                {
#pragma unroll
                                    for(int k = 0; k < kTfK / 8; k++)
                                    {
                                        mma(dMain, descOf(aBig), descOf(bBig), (!segStart || k) ? 1u : 0u);
                                        if(a.round == 0)
                                        {
                                            mma(dCorr, descOf(aSml), descOf(bBig), ((kb - kb0) | k) ? 1u : 0u);
                                            mma(dCorr, descOf(aBig), descOf(bSml), 1u);
                                        }
                                        aBig += 2;
                                        aSml += 2;
                                        bBig += 2;
                                        bSml += 2;
                                    }
                                }
                                commitTo(opEmpty + 8 * slot); // the ring slot is free (in both CTAs) once these MMAs have read it
                                if(((kb - kb0) % kSegBlocks) == kSegBlocks - 1 || kb == kb1 - 1)
                                    commitTo(segFull + 8 * sb);
                                if(kb == kb1 - 1)
                                    commitTo(corrFull + 8 * cb);
                            }
                            __syncwarp();
                            if(++slot == kOpSlots)
                            {
                                slot = 0;
                                phase ^= 1;
                            }
                            if(((kb - kb0) % kSegBlocks) == kSegBlocks - 1 || kb == kb1 - 1)
                                seg++;
                        }
                    }
                }
                if(parts > 1)
                {
                    clusterSync();
                    clusterSync();
                }
            }
            else if(warp < 2 + kEpiWarps)
            {
                // ---------------------------------------------------------------- epilogue (every CTA: its own rows)
                const int      quad  = warp & 3; // tensor-memory lane quadrant this warp may read
                const int      half  = (warp - 2) >> 2; // which 64 accumulator columns
                const int      row   = quad * 32 + lane;
                const int      cbase = half * 64;
                const bool     active = cbase < accCols; // a 64-column tile leaves the second half idle
                int64_t*       cols  = colOff[warp - 2];
                const uint32_t lanes = tmem + (uint32_t(quad * 32) << 16) + uint32_t(cbase);
                uint32_t       seg   = 0;
                int            local = 0;
                int            syncs = 0; // cluster meeting points of the K-split hand-over passed so far
                bool           alive = true;
                auto waitWarp = [&](uint32_t bar, uint32_t parity) {
                    return __all_sync(0xffffffffu, tfWait(bar, parity, abortP)) != 0;
                };
                auto loadChunk = [&](uint32_t taddr, uint32_t(&v)[32]) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),
                          "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
                          "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                };
                for(int u = worker; u < numUnits && alive; u += numWorkers, local++)
                {
                    const int    cb = local & 1;
                    const int    um = (u / parts) % unitsM, un = (u / parts) / unitsM;
                    const int    tmRaw = PAIR ? 2 * um + int(rank) : um;
                    const bool   dupM  = tmRaw >= a.gm.tiles; // this CTA repeats its peer's rows: no stores
                    const TfTile wm    = tfTileOf(a.gm, min(tmRaw, a.gm.tiles - 1));
                    // D offsets of this warp's 64 columns: a pair's accumulator holds the two CTAs' 64-row B tiles side
                    // by side, a single CTA's holds one B tile of 64 or 128 rows
                    __syncwarp();
                    {
                        const int    tnRaw = PAIR ? 2 * un + half : un;
                        const TfTile wn    = tfTileOf(a.gn, min(tnRaw, a.gn.tiles - 1));
                        const int    first = PAIR ? 0 : cbase;
                        for(int c = lane; c < 64; c += 32)
                            cols[c] = (tnRaw < a.gn.tiles && first + c < a.gn.rows) ? tfRowOffset(a.gn, wn, first + c) : -1;
                    }
                    __syncwarp();
                    const int64_t offM = (dupM || !active) ? -1 : tfRowOffset(a.gm, wm, row);
                    // the tile's owner will read C at the very end: start bringing its rows into L2 now
                    if(a.bilinear && offM >= 0 && (u % parts) == 0)
                    {
#pragma unroll
                        for(int c0 = 0; c0 < 64; c0 += 32)
                        {
                            const int64_t f = cols[c0], l = cols[c0 + 31];
                            if(f >= 0)
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(C + offM + f));
                            if(l >= 0)
                                asm volatile("prefetch.global.L2 [%0];" ::"l"(C + offM + l));
                        }
                    }

                    // running sums of the main product, one segment at a time
                    float sum[64];
#pragma unroll
                    for(int j = 0; j < 64; j++)
                        sum[j] = 0.f;
                    int kb0, kb1;
                    kRange(u, kb0, kb1);
                    const int numSegs = (kb1 - kb0 + kSegBlocks - 1) / kSegBlocks;
                    for(int s = 0; s < numSegs && alive; s++, seg++)
                    {
                        const uint32_t sb = seg & 1;
                        alive = waitWarp(segFull + 8 * sb, (seg >> 1) & 1);
                        if(!alive)
                            break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        if(active)
                        {
#pragma unroll
                            for(int c0 = 0; c0 < 64; c0 += 32)
                            {
                                uint32_t v[32];
                                loadChunk(lanes + sb * 128u + uint32_t(c0), v);
#pragma unroll
                                for(int j = 0; j < 32; j++)
                                    sum[c0 + j] = __fadd_rn(sum[c0 + j], __uint_as_float(v[j]));
                            }
                        }
                        // the warp's loads have completed (wait::ld); one lane hands the buffer back for all
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        __syncwarp();
                        if(lane == 0)
                            arriveIssuer(segEmpty + 8 * sb);
                    }
                    if(!alive)
                        break;
                    alive = waitWarp(corrFull + 8 * cb, (local >> 1) & 1);
                    if(!alive)
                        break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    // the correction products complete the sums
                    if(active && a.round == 0)
                    {
#pragma unroll
                        for(int c0 = 0; c0 < 64; c0 += 32)
                        {
                            uint32_t v[32];
                            loadChunk(lanes + 256u + uint32_t(cb) * 128u + uint32_t(c0), v);
#pragma unroll
                            for(int j = 0; j < 32; j++)
                                sum[c0 + j] = __fadd_rn(sum[c0 + j], __uint_as_float(v[j]));
                        }
                    }
                    // K split: every part has its sums; parts 1.. hand theirs to part 0, which adds them in order
                    const int part = u % parts;
                    if(parts > 1)
                    {
                        // zone of part q in the owner's ring memory: [q - 1][column groups of four][128 rows] of float4
                        // (a warp's 32 rows of one column group are 512 contiguous bytes)
                        const uint32_t zone = stagingAddr + uint32_t(cbase >> 2) * 2048u + uint32_t(row) * 16u;
                        const uint32_t zoneBytes = 128u * uint32_t(accCols) * 4u;
                        clusterSync(); // the owner's MMAs have read the last operands: its rings are free
                        syncs++;
                        if(part > 0 && active)
                        {
                            const uint32_t dst = mapToRank(zone + uint32_t(part - 1) * zoneBytes, 0);
#pragma unroll
                            for(int j = 0; j < 16; j++)
                                asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(dst + uint32_t(j) * 2048u),
                                             "f"(sum[4 * j]), "f"(sum[4 * j + 1]), "f"(sum[4 * j + 2]), "f"(sum[4 * j + 3])
                                             : "memory");
                        }
                        clusterSync(); // the sums have arrived
                        syncs++;
                        if(part == 0 && active)
                        {
                            for(int q = 0; q < parts - 1; q++)
                            {
#pragma unroll
                                for(int j = 0; j < 16; j++)
                                {
                                    float4 p4;
                                    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
                                                 : "=f"(p4.x), "=f"(p4.y), "=f"(p4.z), "=f"(p4.w)
                                                 : "r"(zone + uint32_t(q) * zoneBytes + uint32_t(j) * 2048u));
                                    sum[4 * j]     = __fadd_rn(sum[4 * j], p4.x);
                                    sum[4 * j + 1] = __fadd_rn(sum[4 * j + 1], p4.y);
                                    sum[4 * j + 2] = __fadd_rn(sum[4 * j + 2], p4.z);
                                    sum[4 * j + 3] = __fadd_rn(sum[4 * j + 3], p4.w);
                                }
                            }
                        }
                    }
                    if(active && part == 0 && alive)
                    {
                        // D offsets of the eight rows of this lane's group of eight lanes
                        int64_t rowOff[8];
#pragma unroll
                        for(int k = 0; k < 8; k++)
                            rowOff[k] = __shfl_sync(0xffffffffu, offM, (lane & ~7) + k);
#pragma unroll
                        for(int c0 = 0; c0 < 64; c0 += 32)
                        {
                            const int64_t first     = cols[c0];
                            const bool    fullChunk = a.nContig && first >= 0 && cols[c0 + 31] == first + 31;
                            if(fullChunk && __all_sync(0xffffffffu, offM < 0 || ((offM + first) & 3) == 0))
                            {
                                // Line-wise: the eight lanes of a group exchange quarter lines (three rounds of
                                // shuffles, in place in the sums) so that lane m ends up with quarter-line m of each of
                                // the group's eight rows; a load or store instruction then covers four whole 128-byte
                                // lines instead of 32 different ones.
                                const int m = lane & 7;
#pragma unroll
                                for(int j = 0; j < 32; j++)
                                    sum[c0 + j] = __fmul_rn(a.alpha, sum[c0 + j]);
#pragma unroll
                                for(int sft = 4; sft >= 1; sft >>= 1)
                                {
                                    const bool hi = (m & sft) != 0;
#pragma unroll
                                    for(int c = 0; c < 8; c++)
                                    {
                                        if(c & sft)
                                            continue;
#pragma unroll
                                        for(int e = 0; e < 4; e++)
                                        {
                                            float&      lo  = sum[c0 + 4 * c + e];
                                            float&      up  = sum[c0 + 4 * (c | sft) + e];
                                            const float rcv = __shfl_xor_sync(0xffffffffu, hi ? lo : up, sft);
                                            if(hi)
                                                lo = rcv;
                                            else
                                                up = rcv;
                                        }
                                    }
                                }
                                // sum[c0 + 4 k + e] is now element e of quarter-line m of row k of the group
#pragma unroll
                                for(int k0 = 0; k0 < 8; k0 += 4)
                                {
                                    float4 c4[4]; // loads of C ahead of the stores (C may be D)
                                    if(a.bilinear)
                                    {
#pragma unroll
                                        for(int q = 0; q < 4; q++)
                                            c4[q] = rowOff[k0 + q] >= 0 ? *(const float4*)(C + rowOff[k0 + q] + first + 4 * m)
                                                                        : make_float4(0.f, 0.f, 0.f, 0.f);
                                    }
#pragma unroll
                                    for(int q = 0; q < 4; q++)
                                    {
                                        const int k = k0 + q;
                                        float4    o = make_float4(sum[c0 + 4 * k], sum[c0 + 4 * k + 1], sum[c0 + 4 * k + 2],
                                                                  sum[c0 + 4 * k + 3]);
                                        if(a.bilinear)
                                        {
                                            o.x = __fadd_rn(o.x, __fmul_rn(a.beta, c4[q].x));
                                            o.y = __fadd_rn(o.y, __fmul_rn(a.beta, c4[q].y));
                                            o.z = __fadd_rn(o.z, __fmul_rn(a.beta, c4[q].z));
                                            o.w = __fadd_rn(o.w, __fmul_rn(a.beta, c4[q].w));
                                        }
                                        if(rowOff[k] >= 0)
                                            *(float4*)(D + rowOff[k] + first + 4 * m) = o;
                                    }
                                }
                                continue;
                            }
                            if(offM < 0)
                                continue;
                            if(fullChunk && ((offM + first) & 3) == 0)
                            {
                                // 32 consecutive floats of this row: eight 128-bit stores
                                float*       dst = D + offM + first;
                                const float* src = C + offM + first;
                                // C may be D: the compiler must keep every load of C before the stores that follow it,
                                // so the loads are taken four at a time ahead of their stores (one memory round trip
                                // per sixteen columns instead of one per four)
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
                                        o.x = __fmul_rn(a.alpha, sum[c0 + j]);
                                        o.y = __fmul_rn(a.alpha, sum[c0 + j + 1]);
                                        o.z = __fmul_rn(a.alpha, sum[c0 + j + 2]);
                                        o.w = __fmul_rn(a.alpha, sum[c0 + j + 3]);
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
                                    {
                                        float y = __fmul_rn(a.alpha, sum[c0 + j]);
                                        if(a.bilinear)
                                            y = __fadd_rn(y, __fmul_rn(a.beta, C[offM + oc]));
                                        D[offM + oc] = y;
                                    }
                                }
                            }
                        }
                    }
                    // hand the correction accumulator back
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if(lane == 0)
                        arriveIssuer(corrEmpty + 8 * cb);
                }
                for(; parts > 1 && syncs < 2; syncs++)
                    clusterSync(); // a role that gave up still meets the others
            }
            else
            {
                // ---------------------------------------------------------------- converter (every CTA: its own rows)
                const int  ct   = int(threadIdx.x) - 32 * (2 + kEpiWarps);
                const int  r    = ct & 127, kh = ct >> 7; // tile row, half of the K block
                uint32_t   sSlot = 0, sPhase = 0, oSlot = 0, oPhase = 0;
                bool       ok = true;
                for(int u = worker; u < numUnits && ok; u += numWorkers)
                {
                    int kb0, kb1;
                    kRange(u, kb0, kb1);
                    for(int kb = kb0; kb < kb1; kb++)
                    {
                        if constexpr(INPLACE)
                        {
                            // the loads of this operand slot have landed (its producer had waited for the slot to be free)
                            ok = __all_sync(0xffffffffu, tfWait(stFull + 8 * oSlot, oPhase, abortP));
                            if(!ok)
                                break;
                            const uint32_t op = opAddr + oSlot * kOpBytes;
                            if(!(HTB_TF_PROBE(a, 1)))
                            {
                                tfConvertSmall(op, op + kTileBytes, ct, 128);
                                tfConvertSmall(op + 2 * kTileBytes, op + 2 * kTileBytes + kBBytes, ct, a.gn.rows);
                            }
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            __syncwarp();
                            if(lane == 0)
                                arriveIssuer(opFull + 8 * oSlot);
                        }
                        else
                        {
                            ok = tfWait(stFull + 8 * sSlot, sPhase, abortP) && tfWait(opEmpty + 8 * oSlot, oPhase ^ 1, abortP);
                            ok = __all_sync(0xffffffffu, ok);
                            if(!ok)
                                break;
                            const uint32_t st = stagingAddr + sSlot * kStagingBytes;
                            const uint32_t op = opAddr + oSlot * kOpBytes;
                            if(!(HTB_TF_PROBE(a, 1)))
                            {
                                tfConvertRow(a.gm.major, st, op, op + kTileBytes, r, kh, 128, a.round);
                                tfConvertRow(a.gn.major, st + kTileBytes, op + 2 * kTileBytes, op + 2 * kTileBytes + kBBytes, r, kh,
                                             a.gn.rows, a.round);
                            }
                            // the ring is read by the tensor cores (async proxy): order this thread's stores before it
                            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                            __syncwarp();
                            if(lane == 0)
                            {
                                mbarArrive(stEmpty + 8 * sSlot);
                                arriveIssuer(opFull + 8 * oSlot);
                            }
                            if(++sSlot == (kStagingSlots > 0 ? kStagingSlots : 1))
                            {
                                sSlot = 0;
                                sPhase ^= 1;
                            }
                        }
                        if(++oSlot == kOpSlots)
                        {
                            oSlot = 0;
                            oPhase ^= 1;
                        }
                    }
                }
                if(parts > 1)
                {
                    clusterSync();
                    clusterSync();
                }
            }

            // ---------------------------------------------------------------- teardown
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncthreads();
            if(PAIR)
                clusterSync(); // both CTAs are done with tensor memory and with each other's barriers
            if(threadIdx.x == 0 && abortFlag && a.status)
                atomicExch(a.status, 4);
            if(warp == 1)
            {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if(PAIR)
                    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
                else
                    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
            }
        }

        // ------------------------------------------------------------------ host side
        // K-major operand: {K, mode0 .. mode3}, one [rows x 32] box, 128-byte swizzle
        bool encodeKMajor(PFN_encodeTiled encode, CUtensorMap* map, const void* base, int64_t K, const RowGroupView& g,
                          const int* box)
        {
            cuuint64_t gdim[5], gstr[4];
            cuuint32_t bx[5], estr[5] = {1, 1, 1, 1, 1};
            gdim[0] = cuuint64_t(K);
            bx[0]   = kTfK;
            for(int d = 0; d < 4; d++)
            {
                const bool real = d < g.n && g.ext[d] > 1;
                gdim[d + 1]     = real ? cuuint64_t(g.ext[d]) : 1;
                gstr[d]         = real ? cuuint64_t(g.sOp[d]) * 4 : 16; // extent 1: any 16-byte multiple is legal
                bx[d + 1]       = (d < g.n) ? cuuint32_t(box[d]) : 1;
                if(gstr[d] % 16 != 0 || gstr[d] == 0)
                    return false;
            }
            return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<void*>(base), gdim, gstr, bx, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                   == CUDA_SUCCESS;
        }

        // MN-major operand: {mode0 (stride 1), k0, k1, mode1, mode2}, one [32 k x 32 rows] box per chunk, unswizzled
        bool encodeMnMajor(PFN_encodeTiled encode, CUtensorMap* map, const void* base, const RowGroupView& g, int nk,
                           const int64_t* extK, const int64_t* sK, const int* boxK)
        {
            cuuint64_t gdim[5], gstr[4];
            cuuint32_t bx[5] = {32, 1, 1, 1, 1}, estr[5] = {1, 1, 1, 1, 1};
            gdim[0] = cuuint64_t(g.ext[0]);
            for(int d = 0; d < 2; d++)
            {
                const bool real = d < nk && extK[d] > 1;
                gdim[1 + d]     = real ? cuuint64_t(extK[d]) : 1;
                gstr[d]         = real ? cuuint64_t(sK[d]) * 4 : 16;
                bx[1 + d]       = (d < nk) ? cuuint32_t(boxK[d]) : 1;
            }
            for(int d = 1; d < 3; d++)
            {
                const bool real = d < g.n && g.ext[d] > 1;
                gdim[2 + d]     = real ? cuuint64_t(g.ext[d]) : 1;
                gstr[1 + d]     = real ? cuuint64_t(g.sOp[d]) * 4 : 16;
            }
            for(int d = 0; d < 4; d++)
                if(gstr[d] % 16 != 0 || gstr[d] == 0)
                    return false;
            return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<void*>(base), gdim, gstr, bx, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
                   == CUDA_SUCCESS;
        }

        template <bool PAIR, bool INPLACE>
        cudaError_t launchKernel(const CUtensorMap& mapA, const CUtensorMap& mapB, const float* C, float* D, TfArgs& a, int sms,
                                 cudaStream_t stream)
        {
            auto         kernel = contraction_tf32x3_kernel<PAIR, INPLACE>;
            const size_t smem   = size_t(TfRing<PAIR, INPLACE>::kTotal) + 1024;
            if(cudaError_t e = ensureDynamicSmem((const void*)kernel, int(smem)); e != cudaSuccess)
                return e;
            const int      accCols = PAIR ? 128 : a.gn.rows;
            const uint32_t idesc   = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(accCols >> 3) << 17)
                                   | (uint32_t((PAIR ? 256 : 128) >> 4) << 24); // fp32 accumulate, tf32 x tf32, K-major
            // the cluster: one CTA when there is none. (Programmatic dependent launch, which the f16 CTA-pair kernel uses,
            // was measured on this kernel and is not used: configuration 1 back to back took 32.9 us per launch with it
            // and 21.7 us without.)
            cudaLaunchConfig_t  cfg{};
            cudaLaunchAttribute attr[1];
            attr[0].id               = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.blockDim             = dim3(kTfThreads);
            cfg.dynamicSmemBytes     = smem;
            cfg.stream               = stream;
            cfg.attrs                = attr;
            cfg.numAttrs             = 1;
            if(!PAIR)
            {
                // with a K split one cluster per tile: its CTAs are the K ranges (the caller made sure every unit gets a CTA)
                const int grid = int(std::min<int64_t>(int64_t(a.gm.tiles) * a.gn.tiles * std::max(a.parts, 1), sms));
                attr[0].val.clusterDim.x = unsigned(std::max(a.parts, 1));
                cfg.gridDim              = dim3(unsigned(grid));
                cudaError_t e            = cudaLaunchKernelEx(&cfg, kernel, mapA, mapB, C, D, a, idesc);
                if(e == cudaSuccess)
                    noteLaunch("contraction_tf32x3");
                return e;
            }
            attr[0].val.clusterDim.x = 2;
            // CTA pairs that can be resident at once: per device, the same for every instantiation
            static std::atomic<int> clustersOf[kMaxDevices];
            int                     dev = 0;
            cudaGetDevice(&dev);
            const bool devOk       = dev >= 0 && dev < kMaxDevices;
            int        maxClusters = devOk ? clustersOf[dev].load(std::memory_order_relaxed) : 0;
            if(maxClusters == 0)
            {
                cfg.gridDim = dim3(unsigned(sms / 2 * 2));
                int n       = 0;
                if(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0)
                {
                    cudaGetLastError();
                    n = sms / 2;
                }
                maxClusters = n;
                if(devOk)
                    clustersOf[dev].store(n, std::memory_order_relaxed);
            }
            const int64_t pairs = int64_t(a.pairsM) * a.pairsN;
            cfg.gridDim         = dim3(unsigned(2 * std::min<int64_t>(pairs, maxClusters)));
            cudaError_t e       = cudaLaunchKernelEx(&cfg, kernel, mapA, mapB, C, D, a, idesc);
            if(e == cudaSuccess)
                noteLaunch("contraction_tf32x3_pair");
            return e;
        }
    } // namespace

    cudaError_t launchContractionTf32x3(const ContractionPlan& p, float alpha, const void* A, const void* B, float beta,
                                        const void* C, void* D, void* workspace, uint64_t workspaceBytes, int smCount,
                                        int* deviceStatus, cudaStream_t stream)
    {
        (void)workspace; // this kernel needs no scratch
        (void)workspaceBytes;
        PFN_encodeTiled encode = tensorMapEncoder();
        if(!encode)
            return cudaErrorNotSupported;
        const int          sms = smCount > 0 ? smCount : 148;
        const RowGroupView vm = viewOf(p.m, p.nm, p.aMajor ? 0 : -1), vn = viewOf(p.n, p.nn, p.bMajor ? p.nFast : -1);
        int64_t            extK[2] = {1, 1}, sKa[2] = {0, 0}, sKb[2] = {0, 0};
        for(int i = 0; i < p.nk && i < 2; i++)
        {
            extK[i] = p.k[i].ext;
            sKa[i]  = p.k[i].s0;
            sKb[i]  = p.k[i].s1;
        }
        // Single CTAs with 128 x 128 tiles by default. CTA pairs (256 x 128 tiles, each CTA loading 64 rows of B,
        // three ring slots instead of two) measured slower on 4096^3 (1.53 ms against 1.14 ms): the kernel is
        // bound by the latency around its rings, which the cross-CTA signalling lengthens, not by the shared-memory
        // bandwidth that a pair saves. HTB_TF32_PAIR=1 selects them.
        const Switches& sw   = switches();
        const bool      pair = p.pair != 0 && sw.tf32Pair;
        TfArgs a{};
        fillGroup(a.gm, vm, p.aMajor, 128, p.boxM, 5);
        fillGroup(a.gn, vn, p.bMajor, pair ? 64 : p.tileN, pair ? p.boxN128 : p.boxN, 5);
        bool           cached = false;
        MapCacheEntry* maps   = mapCacheFind(p.cacheId, A, B, pair ? 3 : 2, &cached);
        CUtensorMap &  mapA = maps->mapA, &mapB = maps->mapB;
        if(!cached)
        {
            const bool okA = p.aMajor ? encodeMnMajor(encode, &mapA, A, vm, p.nk, extK, sKa, p.boxK)
                                      : encodeKMajor(encode, &mapA, A, p.K, vm, p.boxM);
            const bool okB = p.bMajor ? encodeMnMajor(encode, &mapB, B, vn, p.nk, extK, sKb, p.boxK)
                                      : encodeKMajor(encode, &mapB, B, p.K, vn, pair ? p.boxN128 : p.boxN);
            if(!okA || !okB)
            {
                maps->id = 0;
                return cudaErrorNotSupported;
            }
        }
        a.boxK[0] = p.boxK[0];
        a.boxK[1] = p.boxK[1];
        a.kTilesPerDim[0] = int((extK[0] + a.boxK[0] - 1) / a.boxK[0]);
        a.kTilesPerDim[1] = int((extK[1] + a.boxK[1] - 1) / a.boxK[1]);
        a.kBlocks  = (p.aMajor || p.bMajor) ? a.kTilesPerDim[0] * a.kTilesPerDim[1] : int((p.K + kTfK - 1) / kTfK);
        a.bytesA   = uint32_t(p.aMajor ? 128 : p.rowsM) * kTfK * 4;
        a.bytesB   = uint32_t(p.bMajor ? a.gn.rows : (pair ? p.rowsN128 : p.rowsN)) * kTfK * 4;
        a.alpha    = alpha;
        a.beta     = beta;
        a.bilinear = (p.bilinear && C != nullptr) ? 1 : 0;
        a.nContig  = (vn.sD[0] == 1 && (uintptr_t(D) & 15) == 0 && (!a.bilinear || (uintptr_t(C) & 15) == 0)) ? 1 : 0;
        a.pairsM   = (a.gm.tiles + 1) / 2;
        a.pairsN   = (a.gn.tiles + 1) / 2;
        a.status   = deviceStatus;
        a.round    = (p.computeType == HIPTENSOR_COMPUTE_16F) ? 1 : (p.computeType == HIPTENSOR_COMPUTE_16BF ? 2 : 0);
#ifdef HTB_MEASURE
        a.probe = sw.tf32Probe;
#endif
        if(int64_t(a.gm.tiles) * a.gn.tiles > 0x7fffffffll)
            return cudaErrorInvalidConfiguration;
        HTB_LOG_HEUR("hiptensorContraction", "tf32x3: %d x %d row tiles (%d B rows each), %d K blocks, %s", a.gm.tiles,
                     a.gn.tiles, a.gn.rows, a.kBlocks, pair ? "CTA pairs" : "single CTAs");
        if(pair)
            return launchKernel<true, false>(mapA, mapB, (const float*)C, (float*)D, a, sms, stream);
        // K split, if the plan asks for it and every unit gets a CTA (one cluster of `parts` CTAs per tile)
        a.parts = 1;
        {
            const int64_t tiles = int64_t(a.gm.tiles) * a.gn.tiles;
            const int     parts = p.splitK;
            if(parts > 1 && parts <= 4 && tiles * parts <= sms && a.kBlocks >= 4 * parts && !sw.tf32NoSplit)
                a.parts = parts;
        }
        // both operands K-major and no rounding: TMA loads straight into the operand ring
        const bool inplace = !p.aMajor && !p.bMajor && a.round == 0 && !sw.tf32NoInplace;
        return inplace ? launchKernel<false, true>(mapA, mapB, (const float*)C, (float*)D, a, sms, stream)
                       : launchKernel<false, false>(mapA, mapB, (const float*)C, (float*)D, a, sms, stream);
    }
} // namespace htb
