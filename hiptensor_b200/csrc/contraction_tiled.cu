// Gathered tiled contraction kernel for sm_100a:  D = alpha * (A x B) + beta * C  on the
// folded (M, N, K) view of arbitrary mode lists.
//
// One CTA owns a tile of the folded output. Row/column offsets of the tile (M and N
// multi-indices decomposed over the folded modes) are computed once into shared memory; K
// offsets are computed per K step. Operand tiles are gathered from the strided tensors
// straight into shared memory (converted through the compute type), double buffered with
// a register prefetch, and consumed either by
//   - an FMA micro-kernel, 64x64 tile, 4x4 register tile per thread (fp32 accumulate), or
//   - the FP64 tensor pipe (mma.sync m8n8k4 f64), 128x64 tile, 32x32 warp tiles.
// The epilogue rounds the accumulator to the output type first and then applies
// alpha*x + beta*c, which is the order of the reference's CPU implementation
// (library/src/contraction/contraction_cpu_reference_impl.hpp:406-425).
//
// It stands where the reference enumerates CK DeviceContractionMultipleD_Xdl_CShuffle
// instances (library/src/contraction/device/*_instance.cpp) and covers every mode layout,
// including those a TMA box cannot describe.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "kernels.hpp"
#include "tcgen05_util.cuh"

namespace htb
{
    cudaError_t launchContractionTcgen05(const ContractionPlan& plan, float alpha, const void* A, const void* B,
                                         float beta, const void* C, void* D, void* workspace, uint64_t workspaceBytes,
                                         int smCount, int* deviceStatus, cudaStream_t stream);
    cudaError_t launchContractionTf32x3(const ContractionPlan& plan, float alpha, const void* A, const void* B, float beta,
                                        const void* C, void* D, void* workspace, uint64_t workspaceBytes, int smCount,
                                        int* deviceStatus, cudaStream_t stream);

    namespace
    {
        constexpr int BM = 64, BN = 64, BK = 32, PAD = 4, THREADS = 256;
        constexpr int NL     = BM * BK / THREADS; // elements of each operand tile gathered per thread and K step
        constexpr int KSLOTS = 4; // ring of K-offset tables (steps kt .. kt+3 are live at once)

        struct CtrArgs
        {
            int     nm, nn, nk;
            ModeDim m[kMaxGroup], n[kMaxGroup], k[kMaxGroup];
            int64_t M, N, K;
            float   alpha, beta;
            int     bilinear;
            int     aKfast, bKfast;
            int     tilesN;
        };

        template <typename T>
        __device__ __forceinline__ float toFloat(T v);
        template <>
        __device__ __forceinline__ float toFloat<float>(float v)
        {
            return v;
        }
        template <>
        __device__ __forceinline__ float toFloat<double>(double v)
        {
            return float(v);
        }
        template <>
        __device__ __forceinline__ float toFloat<__half>(__half v)
        {
            return __half2float(v);
        }
        template <>
        __device__ __forceinline__ float toFloat<__nv_bfloat16>(__nv_bfloat16 v)
        {
            return __bfloat162float(v);
        }

        // element -> accumulate type through the compute type (ROUND: 0 none, 1 f16, 2 bf16)
        template <typename TAcc, typename T, int ROUND>
        __device__ __forceinline__ TAcc loadConv(const T* p, int64_t off)
        {
            if constexpr(sizeof(TAcc) == 8)
            {
                return TAcc(p[off]);
            }
            else
            {
                float v = toFloat<T>(p[off]);
                if(ROUND == 1)
                    v = __half2float(__float2half_rn(v));
                if(ROUND == 2)
                    v = __bfloat162float(__float2bfloat16_rn(v));
                return v;
            }
        }

        template <typename TD, typename TAcc>
        __device__ __forceinline__ void storeEpilogue(TD* D, const TD* C, int64_t off, TAcc acc, float alpha, float beta,
                                                      int bilinear)
        {
            if constexpr(sizeof(TD) == 8)
            {
                double x = double(acc);
                double y = __dmul_rn(double(alpha), x);
                if(bilinear)
                    y = __dadd_rn(y, __dmul_rn(double(beta), C[off]));
                D[off] = y;
            }
            else if constexpr(sizeof(TD) == 4)
            {
                float x = float(acc);
                float y = __fmul_rn(alpha, x);
                if(bilinear)
                    y = __fadd_rn(y, __fmul_rn(beta, C[off]));
                D[off] = y;
            }
            else
            {
                TD    xr = TD(float(acc)); // round to the output type first
                float y  = __fmul_rn(alpha, toFloat<TD>(xr));
                if(bilinear)
                    y = __fadd_rn(y, __fmul_rn(beta, toFloat<TD>(C[off])));
                D[off] = TD(y);
            }
        }

        __device__ __forceinline__ void decompose2(const ModeDim* dims, int nd, int64_t idx, int64_t& o0, int64_t& o1)
        {
            o0 = 0;
            o1 = 0;
            for(int d = 0; d < nd; d++)
            {
                int64_t c = idx % dims[d].ext;
                idx /= dims[d].ext;
                o0 += c * dims[d].s0;
                o1 += c * dims[d].s1;
            }
        }

        // ------------------------------------------------------------------ FMA kernel
        // 64 x 64 output tile per CTA, 256 threads, a contiguous 4 x 4 register tile per thread read
        // from shared memory with 128-bit loads. The K loop runs in steps of 32 with two shared
        // buffers and two register sets: the gather of step kt+2 is issued before the arithmetic of
        // step kt and is stored to shared memory after the arithmetic of step kt+1, so that every
        // global load has two compute phases to land in.
        template <typename TA, typename TD, int ROUND>
        __global__ void __launch_bounds__(THREADS)
            contraction_simt_kernel(const TA* __restrict__ A, const TA* __restrict__ B, const TD* C, TD* D, CtrArgs a)
        {
            __shared__ __align__(16) float sA[2][BK][BM + PAD];
            __shared__ __align__(16) float sB[2][BK][BN + PAD];
            __shared__ int64_t             offAm[BM], offDm[BM], offBn[BN], offDn[BN];
            __shared__ int64_t             offAk[KSLOTS][BK], offBk[KSLOTS][BK];

            const int     tid   = threadIdx.x;
            const int64_t tileM = blockIdx.x / a.tilesN, tileN = blockIdx.x % a.tilesN;
            const int64_t m0 = tileM * BM, n0 = tileN * BN;

            auto computeK = [&](int slot, int64_t k0, int t) {
                const int64_t kk = k0 + t;
                int64_t       oa = -1, ob = -1;
                if(kk < a.K)
                    decompose2(a.k, a.nk, kk, oa, ob);
                offAk[slot][t] = oa;
                offBk[slot][t] = ob;
            };
            if(tid < BM)
            {
                const int64_t mm = m0 + tid;
                int64_t       oa = -1, od = -1;
                if(mm < a.M)
                    decompose2(a.m, a.nm, mm, oa, od);
                offAm[tid] = oa;
                offDm[tid] = od;
            }
            else if(tid < BM + BN)
            {
                const int     t  = tid - BM;
                const int64_t nn = n0 + t;
                int64_t       ob = -1, od = -1;
                if(nn < a.N)
                    decompose2(a.n, a.nn, nn, ob, od);
                offBn[t] = ob;
                offDn[t] = od;
            }
            else if(tid < BM + BN + 3 * BK)
            {
                const int t = tid - BM - BN; // K offsets of the first three steps
                computeK(t / BK, int64_t(t / BK) * BK, t % BK);
            }
            __syncthreads();

            auto gload = [&](int64_t step, float(&ra)[NL], float(&rb)[NL]) {
                const int slot = int(step & (KSLOTS - 1));
#pragma unroll
                for(int j = 0; j < NL; j++)
                {
                    const int     idx = tid + THREADS * j;
                    const int     mi  = a.aKfast ? idx / BK : idx % BM;
                    const int     ki  = a.aKfast ? idx % BK : idx / BM;
                    const int64_t om = offAm[mi], ok = offAk[slot][ki];
                    ra[j]            = (om >= 0 && ok >= 0) ? loadConv<float, TA, ROUND>(A, om + ok) : 0.f;
                    const int     ni  = a.bKfast ? idx / BK : idx % BN;
                    const int     kj  = a.bKfast ? idx % BK : idx / BN;
                    const int64_t on = offBn[ni], ok2 = offBk[slot][kj];
                    rb[j]            = (on >= 0 && ok2 >= 0) ? loadConv<float, TA, ROUND>(B, on + ok2) : 0.f;
                }
            };
            auto sstore = [&](int buf, const float(&ra)[NL], const float(&rb)[NL]) {
#pragma unroll
                for(int j = 0; j < NL; j++)
                {
                    const int idx = tid + THREADS * j;
                    if(a.aKfast)
                        sA[buf][idx % BK][idx / BK] = ra[j];
                    else
                        sA[buf][idx / BM][idx % BM] = ra[j];
                    if(a.bKfast)
                        sB[buf][idx % BK][idx / BK] = rb[j];
                    else
                        sB[buf][idx / BN][idx % BN] = rb[j];
                }
            };

            const int64_t nkt = (a.K + BK - 1) / BK;
            const int     tx = tid & 15, ty = tid >> 4;
            float         r0a[NL], r0b[NL], r1a[NL], r1b[NL];
            float         acc[4][4];
#pragma unroll
            for(int i = 0; i < 4; i++)
#pragma unroll
                for(int j = 0; j < 4; j++)
                    acc[i][j] = 0.f;

            gload(0, r0a, r0b);
            sstore(0, r0a, r0b);
            if(nkt > 1)
                gload(1, r1a, r1b);
            __syncthreads();

            // one K step: `held` carries step kt+1 (loaded one iteration ago), `fresh` receives kt+2
            auto iteration = [&](int64_t kt, int cur, float(&heldA)[NL], float(&heldB)[NL], float(&freshA)[NL],
                                 float(&freshB)[NL]) {
                if(kt + 2 < nkt)
                    gload(kt + 2, freshA, freshB);
                // the 32 products of a K step are summed on their own and then added to the running
                // total: short partial sums keep the fp32 rounding error of long contractions well
                // below that of one sequential sum
                float part[4][4];
#pragma unroll
                for(int i = 0; i < 4; i++)
#pragma unroll
                    for(int j = 0; j < 4; j++)
                        part[i][j] = 0.f;
#pragma unroll
                for(int kk = 0; kk < BK; kk++)
                {
                    const float4 av4   = *reinterpret_cast<const float4*>(&sA[cur][kk][ty * 4]);
                    const float4 bv4   = *reinterpret_cast<const float4*>(&sB[cur][kk][tx * 4]);
                    const float  av[4] = {av4.x, av4.y, av4.z, av4.w};
                    const float  bv[4] = {bv4.x, bv4.y, bv4.z, bv4.w};
#pragma unroll
                    for(int i = 0; i < 4; i++)
#pragma unroll
                        for(int j = 0; j < 4; j++)
                            part[i][j] += av[i] * bv[j];
                }
#pragma unroll
                for(int i = 0; i < 4; i++)
#pragma unroll
                    for(int j = 0; j < 4; j++)
                        acc[i][j] += part[i][j];
                if(kt + 1 < nkt)
                    sstore(cur ^ 1, heldA, heldB);
                if(kt + 3 < nkt && tid >= BM + BN && tid < BM + BN + BK)
                    computeK(int((kt + 3) & (KSLOTS - 1)), (kt + 3) * BK, tid - BM - BN);
                __syncthreads();
            };
            for(int64_t kt = 0; kt < nkt; kt += 2)
            {
                iteration(kt, 0, r1a, r1b, r0a, r0b);
                if(kt + 1 < nkt)
                    iteration(kt + 1, 1, r0a, r0b, r1a, r1b);
            }

            // epilogue: four consecutive N positions per thread, written as one 128-bit store when
            // D (and C) are contiguous and aligned there
#pragma unroll
            for(int i = 0; i < 4; i++)
            {
                const int64_t om = offDm[ty * 4 + i];
                if(om < 0)
                    continue;
                const int64_t on0 = offDn[tx * 4], on3 = offDn[tx * 4 + 3];
                if constexpr(sizeof(TD) == 4)
                {
                    const int64_t off = om + on0;
                    bool          vec = on0 >= 0 && on3 == on0 + 3 && ((uintptr_t(D + off) & 15) == 0);
                    if(a.bilinear)
                        vec = vec && ((uintptr_t(C + off) & 15) == 0);
                    if(vec)
                    {
                        float4 y;
                        y.x = __fmul_rn(a.alpha, acc[i][0]);
                        y.y = __fmul_rn(a.alpha, acc[i][1]);
                        y.z = __fmul_rn(a.alpha, acc[i][2]);
                        y.w = __fmul_rn(a.alpha, acc[i][3]);
                        if(a.bilinear)
                        {
                            const float4 c = *reinterpret_cast<const float4*>(C + off);
                            y.x            = __fadd_rn(y.x, __fmul_rn(a.beta, c.x));
                            y.y            = __fadd_rn(y.y, __fmul_rn(a.beta, c.y));
                            y.z            = __fadd_rn(y.z, __fmul_rn(a.beta, c.z));
                            y.w            = __fadd_rn(y.w, __fmul_rn(a.beta, c.w));
                        }
                        *reinterpret_cast<float4*>(D + off) = y;
                        continue;
                    }
                }
#pragma unroll
                for(int j = 0; j < 4; j++)
                {
                    const int64_t on = offDn[tx * 4 + j];
                    if(on >= 0)
                        storeEpilogue<TD, float>(D, C, om + on, acc[i][j], a.alpha, a.beta, a.bilinear);
                }
            }
        }

        CtrArgs makeArgs(const ContractionPlan& p, float alpha, float beta, const void* C)
        {
            CtrArgs a{};
            a.nm = p.nm;
            a.nn = p.nn;
            a.nk = p.nk;
            for(int i = 0; i < kMaxGroup; i++)
            {
                a.m[i] = p.m[i];
                a.n[i] = p.n[i];
                a.k[i] = p.k[i];
            }
            a.M        = p.M;
            a.N        = p.N;
            a.K        = p.K;
            a.alpha    = alpha;
            a.beta     = beta;
            a.bilinear = (p.bilinear && C != nullptr) ? 1 : 0;
            a.aKfast   = (p.k[0].s0 == 1 && p.k[0].ext > 1) ? 1 : 0;
            a.bKfast   = (p.k[0].s1 == 1 && p.k[0].ext > 1) ? 1 : 0;
            return a;
        }

        // ------------------------------------------------------------------ FP64 tensor-pipe kernel
        // 128 x 64 output tile per CTA, 16-wide K steps, eight MMA warps in a 4 x 2 grid, each warp a 32 x 32 tile
        // made of 4 x 4 mma.sync.m8n8k4.f64 fragments (16 MMAs for 8 shared-memory loads per 4-wide K step).
        // Operands are gathered through offset tables (row offsets once per CTA, K offsets per step), so any mode
        // structure is read in place. The gathers are cp.async copies straight from global to shared memory into
        // a ring of three stages, 16 bytes at a time when the operand's layout allows (two elements that are
        // neighbours in memory: along M/N for an operand whose rows are contiguous, along K for a K-contiguous
        // one), else 8 bytes. Shared layout per operand: rows contiguous in memory -> [k][rows + 4]; K contiguous
        // -> [row][k + 4] (both free of bank conflicts for the fragment loads: 8 rows x 4 k per instruction).
        constexpr int DM = 128, DN = 64;
        constexpr int kDmmaStages = 3;
        constexpr int kDmmaK      = 16;
        constexpr int kDmmaATile  = DM * (kDmmaK + PAD); // doubles per stage, the larger of the two layouts
        constexpr int kDmmaBTile  = DN * (kDmmaK + PAD);

        __device__ __forceinline__ void cpAsync16(uint32_t dst, const void* src, bool valid)
        {
            const int n = valid ? 16 : 0; // 0: the destination is filled with zeros
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
        }
        __device__ __forceinline__ void cpAsync8(uint32_t dst, const void* src, bool valid)
        {
            const int n = valid ? 8 : 0;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
        }

        struct DmmaArgs
        {
            CtrArgs base;
            int     vecA, vecB; // 16-byte copies are legal for this operand
            int     k32; // K fits 32 bits: the producers decompose K indices with 32-bit divisions
            // K split of problems with few tiles: a tile's K steps are cut over the 2 or 4 CTAs of a thread-block
            // cluster. Afterwards the CTAs exchange accumulators over the cluster network so that each ends up with the
            // full sums of its share of the tile's row blocks (summed in a fixed order) and stores that share.
            int     parts;
            int*    status; // the handle's device status word (raised when a bounded wait runs out)
        };

        // Warp-specialised: eight MMA warps that execute nothing but fragment loads and MMAs, and two producer warps that own the
        // gathers: they compute the K offsets of a tile, issue all of the tile's cp.async copies (24 sixteen-byte
        // copies per lane, or 48 eight-byte ones) into a ring of three stages and let them arrive on the stage's
        // "full" mbarrier; each MMA warp waits for that barrier, consumes the stage and arrives on its "empty"
        // barrier. There is no CTA-wide barrier in the K loop. Waits are clock-bounded: when one runs out the
        // kernel raises the status word and every role leaves its loop.
        constexpr int kWsProducers = 2; // two producer warps cost nothing: registers are granted per pair of warps
        constexpr int kWsThreads   = THREADS + 32 * kWsProducers;

        __device__ __forceinline__ void decompose2u(const ModeDim* dims, int nd, uint32_t idx, int64_t& o0, int64_t& o1)
        {
            o0 = 0;
            o1 = 0;
            for(int d = 0; d < nd; d++)
            {
                const uint32_t e = uint32_t(dims[d].ext), q = idx / e, c = idx - q * e;
                idx = q;
                o0 += int64_t(c) * dims[d].s0;
                o1 += int64_t(c) * dims[d].s1;
            }
        }

        __global__ void __launch_bounds__(kWsThreads, 2)
            contraction_dmma_kernel(const double* __restrict__ A, const double* __restrict__ B, const double* C,
                                       double* D, DmmaArgs args)
        {
            const CtrArgs& a = args.base;
            constexpr int  DK = kDmmaK, S = kDmmaStages;
            extern __shared__ __align__(16) unsigned char dsmem[];
            double* sA = reinterpret_cast<double*>(dsmem); // [S][kDmmaATile]
            double* sB = sA + S * kDmmaATile; // [S][kDmmaBTile]
            __shared__ int64_t offAm[DM], offDm[DM], offBn[DN], offDn[DN];
            __shared__ int64_t offAkAll[kWsProducers][S][DK], offBkAll[kWsProducers][S][DK]; // one table per producer warp
            __shared__ __align__(8) unsigned long long fullBar[S], emptyBar[S];
            __shared__ int abortFlag;

            const int     tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
            const int     parts = args.parts, part = int(blockIdx.x) % parts; // part = rank in the tile's cluster
            const int64_t tile  = blockIdx.x / parts;
            const int64_t tileM = tile / a.tilesN, tileN = tile % a.tilesN;
            const int64_t m0 = tileM * DM, n0 = tileN * DN;
            const int     nktAll = int((a.K + DK - 1) / DK); // the launcher refuses K beyond 2^31 steps
            const int     kt0 = int(int64_t(nktAll) * part / parts), nkt = int(int64_t(nktAll) * (part + 1) / parts) - kt0;

            if(tid < DM)
            {
                const int64_t mm = m0 + tid;
                int64_t       oa = -1, od = -1;
                if(mm < a.M)
                    decompose2(a.m, a.nm, mm, oa, od);
                offAm[tid] = oa;
                offDm[tid] = od;
            }
            else if(tid < DM + DN)
            {
                const int     t  = tid - DM;
                const int64_t nn = n0 + t;
                int64_t       ob = -1, od = -1;
                if(nn < a.N)
                    decompose2(a.n, a.nn, nn, ob, od);
                offBn[t] = ob;
                offDn[t] = od;
            }
            else if(tid == DM + DN)
            {
                abortFlag = 0;
                for(int s = 0; s < S; s++)
                {
                    mbarInit(smemAddr(&fullBar[s]), 32 * kWsProducers); // the producers' lanes, each when its copies have landed
                    mbarInit(smemAddr(&emptyBar[s]), THREADS / 32); // one arrival per MMA warp
                }
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            __syncthreads();
            volatile int*  abortP    = &abortFlag;
            const uint32_t fullAddr  = smemAddr(&fullBar[0]), emptyAddr = smemAddr(&emptyBar[0]);
            const int      aRS = a.aKfast ? DK + PAD : 1, aKS = a.aKfast ? 1 : DM + PAD;
            const int      bRS = a.bKfast ? DK + PAD : 1, bKS = a.bKfast ? 1 : DN + PAD;

            if(warp >= THREADS / 32)
            {
                // ---------------------------------------------------------------- producer warps
                const int      pw = warp - THREADS / 32; // takes every kWsProducers-th group of 32 copies
                int64_t(*offAk)[DK] = offAkAll[pw];
                int64_t(*offBk)[DK] = offBkAll[pw];
                const int      first = lane + 32 * pw, step = 32 * kWsProducers;
                const uint32_t sAaddr = smemAddr(sA), sBaddr = smemAddr(sB);
                int      st = 0;
                uint32_t ph = 0; // parity of the stage's current use
                for(int kt = 0; kt < nkt; kt++)
                {
                    // the stage's previous use must have been consumed by every MMA warp
                    if(kt >= S && !mbarWaitTight(emptyAddr + 8 * st, ph ^ 1u, abortP))
                        break;
                    if(lane < DK)
                    {
                        const int64_t kk = int64_t(kt0 + kt) * DK + lane;
                        int64_t       oa = -1, ob = -1;
                        if(kk < a.K)
                        {
                            if(args.k32)
                                decompose2u(a.k, a.nk, uint32_t(kk), oa, ob);
                            else
                                decompose2(a.k, a.nk, kk, oa, ob);
                        }
                        offAk[st][lane] = oa;
                        offBk[st][lane] = ob;
                    }
                    __syncwarp();
                    const uint32_t dA = sAaddr + 8u * uint32_t(st * kDmmaATile), dB = sBaddr + 8u * uint32_t(st * kDmmaBTile);
                    if(args.vecA)
                    {
                        // step is a multiple of DM / 2 and of DK / 2: a lane keeps its row pair (rows contiguous) or its
                        // K pair (K contiguous) for the whole stage, so that table entry is read once (the first
                        // version read both tables for every copy: two shared loads per cp.async, with bank conflicts)
                        if(!a.aKfast)
                        {
                            const int     r  = 2 * (first % (DM / 2));
                            const int64_t om = offAm[r];
#pragma unroll 4
                            for(int k = first / (DM / 2); k < DK; k += step / (DM / 2))
                            {
                                const int64_t ok = offAk[st][k];
                                const bool    v  = om >= 0 && ok >= 0;
                                cpAsync16(dA + 8u * uint32_t(r * aRS + k * aKS), v ? A + om + ok : A, v);
                            }
                        }
                        else
                        {
                            const int     k  = 2 * (first % (DK / 2));
                            const int64_t ok = offAk[st][k];
#pragma unroll 4
                            for(int r = first / (DK / 2); r < DM; r += step / (DK / 2))
                            {
                                const int64_t om = offAm[r];
                                const bool    v  = om >= 0 && ok >= 0;
                                cpAsync16(dA + 8u * uint32_t(r * aRS + k * aKS), v ? A + om + ok : A, v);
                            }
                        }
                    }
                    else
                    {
#pragma unroll 4
                        for(int idx = first; idx < DM * DK; idx += step)
                        {
                            const int r = a.aKfast ? idx / DK : idx % DM;
                            const int k = a.aKfast ? idx % DK : idx / DM;
                            const int64_t om = offAm[r], ok = offAk[st][k];
                            const bool    v  = om >= 0 && ok >= 0;
                            cpAsync8(dA + 8u * uint32_t(r * aRS + k * aKS), v ? A + om + ok : A, v);
                        }
                    }
                    if(args.vecB)
                    {
                        if(!a.bKfast)
                        {
                            const int     r  = 2 * (first % (DN / 2));
                            const int64_t on = offBn[r];
#pragma unroll 4
                            for(int k = first / (DN / 2); k < DK; k += step / (DN / 2))
                            {
                                const int64_t ok = offBk[st][k];
                                const bool    v  = on >= 0 && ok >= 0;
                                cpAsync16(dB + 8u * uint32_t(r * bRS + k * bKS), v ? B + on + ok : B, v);
                            }
                        }
                        else
                        {
                            const int     k  = 2 * (first % (DK / 2));
                            const int64_t ok = offBk[st][k];
#pragma unroll 4
                            for(int r = first / (DK / 2); r < DN; r += step / (DK / 2))
                            {
                                const int64_t on = offBn[r];
                                const bool    v  = on >= 0 && ok >= 0;
                                cpAsync16(dB + 8u * uint32_t(r * bRS + k * bKS), v ? B + on + ok : B, v);
                            }
                        }
                    }
                    else
                    {
#pragma unroll 4
                        for(int idx = first; idx < DN * DK; idx += step)
                        {
                            const int r = a.bKfast ? idx / DK : idx % DN;
                            const int k = a.bKfast ? idx % DK : idx / DN;
                            const int64_t on = offBn[r], ok = offBk[st][k];
                            const bool    v  = on >= 0 && ok >= 0;
                            cpAsync8(dB + 8u * uint32_t(r * bRS + k * bKS), v ? B + on + ok : B, v);
                        }
                    }
                    // this lane's arrival on the stage's barrier happens when its copies above have landed
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(fullAddr + 8 * st) : "memory");
                    if(++st == S)
                    {
                        st = 0;
                        ph ^= 1u;
                    }
                }
                asm volatile("cp.async.wait_all;" ::: "memory");
                if(lane == 0 && *abortP && args.status)
                    atomicExch(args.status, 3);
                if(parts > 1)
                {
                    clusterSync(); // the two meeting points of the accumulator exchange (see the MMA warps)
                    clusterSync();
                }
                return;
            }

            // -------------------------------------------------------------------- MMA warps
            double acc[4][4][2];
#pragma unroll
            for(int i = 0; i < 4; i++)
#pragma unroll
                for(int j = 0; j < 4; j++)
                    acc[i][j][0] = acc[i][j][1] = 0.0;
            const int wm = warp & 3, wn = warp >> 2;
            const int aFrag = (wm * 32 + (lane >> 2)) * aRS + (lane & 3) * aKS;
            const int bFrag = (wn * 32 + (lane >> 2)) * bRS + (lane & 3) * bKS;
            bool      ok    = true;
            int       st    = 0;
            uint32_t  ph    = 0;
            for(int kt = 0; kt < nkt; kt++)
            {
                ok = mbarWaitTight(fullAddr + 8 * st, ph, abortP);
                if(!ok)
                    break;
                const double* tA = sA + st * kDmmaATile + aFrag;
                const double* tB = sB + st * kDmmaBTile + bFrag;
#pragma unroll
                for(int k4 = 0; k4 < DK / 4; k4++)
                {
                    double af[4], bf[4];
#pragma unroll
                    for(int i = 0; i < 4; i++)
                        af[i] = tA[i * 8 * aRS + k4 * 4 * aKS];
#pragma unroll
                    for(int j = 0; j < 4; j++)
                        bf[j] = tB[j * 8 * bRS + k4 * 4 * bKS];
#pragma unroll
                    for(int i = 0; i < 4; i++)
#pragma unroll
                        for(int j = 0; j < 4; j++)
                            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                                         : "+d"(acc[i][j][0]), "+d"(acc[i][j][1])
                                         : "d"(af[i]), "d"(bf[j]));
                }
                __syncwarp();
                if(lane == 0)
                    mbarArrive(emptyAddr + 8 * st);
                if(++st == S)
                {
                    st = 0;
                    ph ^= 1u;
                }
            }
            if(!ok && lane == 0 && args.status)
                atomicExch(args.status, 3);
            if(parts > 1)
            {
                // Row block i of every warp tile belongs to part i * parts / 4. Each thread sends the eight sums of a
                // foreign row block to its owner's shared memory (the copy ring, idle once every CTA of the cluster has
                // left its K loop), slot [sender][i % (4 / parts)][thread]; then every owner adds the parts in order.
                const int      per  = 4 / parts; // row blocks per part
                const uint32_t zone = smemAddr(sA);
                clusterSync();
#pragma unroll
                for(int i = 0; i < 4; i++)
                {
                    const int owner = i / per;
                    if(owner == part)
                        continue;
                    const uint32_t dst = mapToRank(zone + uint32_t(((part * per + i % per) * THREADS + tid) * 64), uint32_t(owner));
#pragma unroll
                    for(int j = 0; j < 4; j++)
                        asm volatile("st.shared::cluster.v2.f64 [%0], {%1, %2};" ::"r"(dst + 16u * uint32_t(j)), "d"(acc[i][j][0]),
                                     "d"(acc[i][j][1])
                                     : "memory");
                }
                clusterSync();
#pragma unroll
                for(int i = 0; i < 4; i++)
                {
                    if(i / per != part)
                        continue;
                    double tot[4][2];
#pragma unroll
                    for(int j = 0; j < 4; j++)
                        tot[j][0] = tot[j][1] = 0.0;
                    for(int q = 0; q < parts; q++)
                    {
                        const double2* src = reinterpret_cast<const double2*>(
                            reinterpret_cast<const unsigned char*>(sA) + size_t((q * per + i % per) * THREADS + tid) * 64);
#pragma unroll
                        for(int j = 0; j < 4; j++)
                        {
                            const double2 v = (q == part) ? make_double2(acc[i][j][0], acc[i][j][1]) : src[j];
                            tot[j][0] += v.x;
                            tot[j][1] += v.y;
                        }
                    }
#pragma unroll
                    for(int j = 0; j < 4; j++)
                    {
                        acc[i][j][0] = tot[j][0];
                        acc[i][j][1] = tot[j][1];
                    }
                }
            }
            if(!ok)
                return;
            // C may be D, so a load of C cannot move above an earlier store to D: the eight values of C that a row
            // block needs are loaded first, then the eight results are stored (4 memory round trips instead of 32)
#pragma unroll
            for(int i = 0; i < 4; i++)
            {
                if(parts > 1 && i / (4 / parts) != part)
                    continue; // another CTA of the cluster holds and stores this row block
                const int64_t om = offDm[wm * 32 + i * 8 + (lane >> 2)];
                if(om < 0)
                    continue;
                int64_t off[4][2];
                double  cv[4][2];
#pragma unroll
                for(int j = 0; j < 4; j++)
#pragma unroll
                    for(int e = 0; e < 2; e++)
                    {
                        const int64_t on = offDn[wn * 32 + j * 8 + 2 * (lane & 3) + e];
                        off[j][e]        = on >= 0 ? om + on : -1;
                        cv[j][e]         = (a.bilinear && on >= 0) ? C[om + on] : 0.0;
                    }
#pragma unroll
                for(int j = 0; j < 4; j++)
#pragma unroll
                    for(int e = 0; e < 2; e++)
                        if(off[j][e] >= 0)
                        {
                            double y = __dmul_rn(double(a.alpha), acc[i][j][e]);
                            if(a.bilinear)
                                y = __dadd_rn(y, __dmul_rn(double(a.beta), cv[j][e]));
                            D[off[j][e]] = y;
                        }
            }
        }

        // 16-byte copies along the operand's contiguous direction: the direction's extent and every other stride
        // of the operand even, base address 16-byte aligned. (Tiles start at even indices, so pairs never
        // straddle the end of the contiguous mode.)
        bool dmmaVectorOk(const void* base, const ModeDim* rows, int nrows, const ModeDim* ks, int nks, bool second, bool kFast)
        {
            if(uintptr_t(base) & 15)
                return false;
            auto strideOf = [&](const ModeDim& d, bool kGroup) { return kGroup ? (second ? d.s1 : d.s0) : d.s0; };
            const ModeDim& unit = kFast ? ks[0] : rows[0];
            if(strideOf(unit, kFast) != 1 || (unit.ext & 1))
                return false;
            for(int i = 0; i < nrows; i++)
                if(!(i == 0 && !kFast) && rows[i].ext > 1 && (strideOf(rows[i], false) & 1))
                    return false;
            for(int i = 0; i < nks; i++)
                if(!(i == 0 && kFast) && ks[i].ext > 1 && (strideOf(ks[i], true) & 1))
                    return false;
            return true;
        }

        cudaError_t launchDmma(const ContractionPlan& p, float alpha, const void* A, const void* B, float beta,
                               const void* C, void* D, int smCountIn, int* deviceStatus, cudaStream_t stream)
        {
            const int smCount = smCountIn > 0 ? smCountIn : 148;
            DmmaArgs  args{};
            args.base            = makeArgs(p, alpha, beta, C);
            CtrArgs&      a      = args.base;
            const int64_t tilesM = (p.M + DM - 1) / DM, tilesN = (p.N + DN - 1) / DN;
            if(tilesM * tilesN > 0x7fffffffll || p.K / kDmmaK >= 0x7fffffffll)
                return cudaErrorInvalidConfiguration;
            a.tilesN = int(tilesN);
            // operand A's rows are the M group (first strides), B's the N group (first strides); K strides: A first, B second
            args.vecA = dmmaVectorOk(A, p.m, p.nm, p.k, p.nk, false, a.aKfast != 0) ? 1 : 0;
            args.vecB = dmmaVectorOk(B, p.n, p.nn, p.k, p.nk, true, a.bKfast != 0) ? 1 : 0;
            if(switches().dmmaNoVec)
                args.vecA = args.vecB = 0;
            args.k32    = p.K < (int64_t(1) << 31) ? 1 : 0;
            args.status = deviceStatus;
            // few tiles and a long K: 4 or 2 CTAs per tile, at least four K steps each, never more CTAs than fit at once
            // (two per SM)
            const int64_t tiles = tilesM * tilesN, steps = (p.K + kDmmaK - 1) / kDmmaK;
            args.parts          = 1;
            for(int q = 4; q >= 2; q >>= 1)
                if(tiles * q <= 2 * int64_t(smCount) && steps >= 4 * q && !switches().dmmaNoSplit)
                {
                    args.parts = q;
                    break;
                }
            const size_t smem = sizeof(double) * kDmmaStages * (kDmmaATile + kDmmaBTile);
            if(cudaError_t e = ensureDynamicSmem((const void*)contraction_dmma_kernel, int(smem)); e != cudaSuccess)
                return e;
            if(args.parts > 1)
            {
                cudaLaunchConfig_t  cfg{};
                cudaLaunchAttribute attr[1];
                attr[0].id               = cudaLaunchAttributeClusterDimension;
                attr[0].val.clusterDim.x = unsigned(args.parts);
                attr[0].val.clusterDim.y = 1;
                attr[0].val.clusterDim.z = 1;
                cfg.gridDim              = dim3(unsigned(tiles * args.parts));
                cfg.blockDim             = dim3(kWsThreads);
                cfg.dynamicSmemBytes     = smem;
                cfg.stream               = stream;
                cfg.attrs                = attr;
                cfg.numAttrs             = 1;
                cudaError_t e = cudaLaunchKernelEx(&cfg, contraction_dmma_kernel, (const double*)A, (const double*)B,
                                                   (const double*)C, (double*)D, args);
                if(e == cudaSuccess)
                    noteLaunch("contraction_tiled_dmma");
                return e;
            }
            contraction_dmma_kernel<<<unsigned(tiles), kWsThreads, smem, stream>>>(
                (const double*)A, (const double*)B, (const double*)C, (double*)D, args);
            noteLaunch("contraction_tiled_dmma");
            return cudaGetLastError();
        }

        template <typename TA, typename TD, int ROUND>
        cudaError_t launchTiled(const ContractionPlan& p, float alpha, const void* A, const void* B, float beta,
                                const void* C, void* D, cudaStream_t stream)
        {
            CtrArgs a{};
            a.nm = p.nm;
            a.nn = p.nn;
            a.nk = p.nk;
            for(int i = 0; i < kMaxGroup; i++)
            {
                a.m[i] = p.m[i];
                a.n[i] = p.n[i];
                a.k[i] = p.k[i];
            }
            a.M        = p.M;
            a.N        = p.N;
            a.K        = p.K;
            a.alpha    = alpha;
            a.beta     = beta;
            a.bilinear = (p.bilinear && C != nullptr) ? 1 : 0;
            a.aKfast   = (p.k[0].s0 == 1 && p.k[0].ext > 1) ? 1 : 0;
            a.bKfast   = (p.k[0].s1 == 1 && p.k[0].ext > 1) ? 1 : 0;
            const int64_t tilesM = (p.M + BM - 1) / BM, tilesN = (p.N + BN - 1) / BN;
            if(tilesM * tilesN > 0x7fffffffll)
                return cudaErrorInvalidConfiguration;
            a.tilesN = int(tilesN);
            contraction_simt_kernel<TA, TD, ROUND>
                <<<unsigned(tilesM * tilesN), THREADS, 0, stream>>>((const TA*)A, (const TA*)B, (const TD*)C, (TD*)D, a);
            noteLaunch("contraction_tiled_simt");
            return cudaGetLastError();
        }
    } // namespace

    cudaError_t launchContraction(const ContractionPlan& plan, float alpha, const void* A0, const void* B0,
                                  float beta, const void* C, void* D, void* workspace, uint64_t workspaceBytes,
                                  int smCount, int* deviceStatus, cudaStream_t stream)
    {
        if(plan.M == 0 || plan.N == 0)
            return cudaSuccess;
        const void* A = plan.swapped ? B0 : A0;
        const void* B = plan.swapped ? A0 : B0;
        if(plan.kind == CK_TCGEN05)
        {
            const bool aligned = ((uintptr_t(A) | uintptr_t(B)) & 15) == 0;
            if(aligned)
                return launchContractionTcgen05(plan, alpha, A, B, beta, C, D, workspace, workspaceBytes, smCount,
                                                deviceStatus, stream);
        }
        if(plan.kind == CK_TF32X3 && !switches().noTf32x3)
        {
            const bool aligned = ((uintptr_t(A) | uintptr_t(B)) & 15) == 0;
            if(aligned)
                return launchContractionTf32x3(plan, alpha, A, B, beta, C, D, workspace, workspaceBytes, smCount, deviceStatus,
                                               stream);
        }
        const int ct = plan.computeType;
        switch(plan.typeA)
        {
        case CUDA_R_32F:
            if(ct == HIPTENSOR_COMPUTE_16F)
                return launchTiled<float, float, 1>(plan, alpha, A, B, beta, C, D, stream);
            if(ct == HIPTENSOR_COMPUTE_16BF)
                return launchTiled<float, float, 2>(plan, alpha, A, B, beta, C, D, stream);
            return launchTiled<float, float, 0>(plan, alpha, A, B, beta, C, D, stream);
        case CUDA_R_64F:
            // compute type f64, and f32 unless the switch asks for the FMA kernel (float accumulation, as the reference)
            if(ct == HIPTENSOR_COMPUTE_64F || !switches().f64Compute32Fma)
                return launchDmma(plan, alpha, A, B, beta, C, D, smCount, deviceStatus, stream);
            return launchTiled<double, double, 0>(plan, alpha, A, B, beta, C, D, stream);
        case CUDA_R_16F:
            if(plan.typeD == CUDA_R_32F)
                return launchTiled<__half, float, 0>(plan, alpha, A, B, beta, C, D, stream);
            return launchTiled<__half, __half, 0>(plan, alpha, A, B, beta, C, D, stream);
        case CUDA_R_16BF:
            if(plan.typeD == CUDA_R_32F)
                return launchTiled<__nv_bfloat16, float, 0>(plan, alpha, A, B, beta, C, D, stream);
            return launchTiled<__nv_bfloat16, __nv_bfloat16, 0>(plan, alpha, A, B, beta, C, D, stream);
        }
        return cudaErrorInvalidValue;
    }
} // namespace htb
