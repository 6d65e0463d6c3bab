// Reduction kernels for sm_100a: D = alpha * reduce_op(A over the reduced modes) + beta * C.
//
//   red_row_kernel : a reduced mode is contiguous in A. A group of G threads (one warp or
//                    one block) owns one output; lanes stride along the contiguous run with
//                    128-bit loads and four independent accumulators, then warp shuffles and
//                    (for G=256) a shared-memory step combine them.
//   red_col_kernel : a kept mode is contiguous in A. Lanes run along the kept mode
//                    (coalesced), threadIdx.y cuts the reduced range, shared memory combines.
//   red_gen_kernel : no stride-1 mode: G threads per output over the flattened reduced range.
//   red_finalize_kernel : second pass when the reduced range was cut into slices (few outputs,
//                    long reductions); partial results live in caller-provided scratch.
//
// Semantics follow CK's host ReferenceReduce as used by the reference
// (library/src/reduction/reduction_cpu_reference_impl.hpp:45-64): accumulate in the compute
// type, NaN propagates through MIN/MAX, then "if alpha != 1: acc *= alpha; if beta != 0:
// acc += C * beta". They replace CK's DeviceReduceMultiBlock instances
// (library/src/reduction/reduction_solution_impl.hpp:224-267: 256 threads, vector width 1).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cfloat>
#include <mutex>
#include <type_traits>

#include "kernels.hpp"

namespace htb
{
    namespace
    {
        struct RedArgs
        {
            int     nk, nr;
            int64_t kext[kMaxGroup], ksA[kMaxGroup], ksD[kMaxGroup];
            int64_t rext[kMaxGroup], rsA[kMaxGroup];
            int64_t nOut, nRed;
            int     split; // slices of the reduced range (1 = single pass)
            int     sliceOuter; // 1: slices cut the outer reduced index, 0: the innermost reduced mode
            int64_t sliceLen;
            int64_t outer; // nRed / rext[0]: iterations over the outer reduced modes
        };

        enum
        {
            OP_ADD = 3,
            OP_MUL = 5,
            OP_MAX = 6,
            OP_MIN = 7
        };

        template <typename T>
        __device__ __forceinline__ T lowestOf();
        template <>
        __device__ __forceinline__ float lowestOf<float>()
        {
            return -FLT_MAX;
        }
        template <>
        __device__ __forceinline__ double lowestOf<double>()
        {
            return -DBL_MAX;
        }

        template <typename T, int OP>
        struct Op
        {
            static __device__ __forceinline__ T identity()
            {
                if(OP == OP_ADD)
                    return T(0);
                if(OP == OP_MUL)
                    return T(1);
                if(OP == OP_MAX)
                    return lowestOf<T>();
                return -lowestOf<T>();
            }
            static __device__ __forceinline__ T combine(T acc, T v)
            {
                if(OP == OP_ADD)
                    return acc + v;
                if(OP == OP_MUL)
                    return acc * v;
                // MAX / MIN propagate NaN (PropagateNan = true in the reference's host reduction)
                if constexpr(sizeof(T) == 4)
                {
                    // one instruction: the result is NaN when either operand is
                    float r;
                    if(OP == OP_MAX)
                        asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(acc), "f"(v));
                    else
                        asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(acc), "f"(v));
                    return r;
                }
                if(OP == OP_MAX)
                    return (v != v || acc < v) ? ((acc != acc) ? acc : v) : acc;
                return (v != v || acc > v) ? ((acc != acc) ? acc : v) : acc;
            }
        };

        // Two-level accumulator of one thread. Four independent running values take the
        // elements in turn; every 8 rounds (32 elements) they are folded into a top-level value.
        // For fp32 sums the top level is fp64, so that the rounding error of a long sum stays
        // that of its short fp32 partial sums (the reference accumulates sequentially in fp32;
        // its own tolerance is reduce_len * eps). The other operators fold only once, at the end.
        template <typename TAcc, int OP>
        struct Accum
        {
            using Top = typename std::conditional<(OP == OP_ADD && sizeof(TAcc) == 4), double, TAcc>::type;
            static constexpr bool kTwoLevel = !std::is_same<Top, TAcc>::value;
            TAcc a0, a1, a2, a3;
            Top  top;
            int  cnt;
            __device__ __forceinline__ void init()
            {
                a0 = a1 = a2 = a3 = Op<TAcc, OP>::identity();
                top               = Op<Top, OP>::identity();
                cnt               = 0;
            }
            __device__ __forceinline__ void fold()
            {
                TAcc s = Op<TAcc, OP>::combine(Op<TAcc, OP>::combine(a0, a1), Op<TAcc, OP>::combine(a2, a3));
                top    = Op<Top, OP>::combine(top, Top(s));
                a0 = a1 = a2 = a3 = Op<TAcc, OP>::identity();
                cnt               = 0;
            }
            __device__ __forceinline__ void add4(TAcc v0, TAcc v1, TAcc v2, TAcc v3)
            {
                a0 = Op<TAcc, OP>::combine(a0, v0);
                a1 = Op<TAcc, OP>::combine(a1, v1);
                a2 = Op<TAcc, OP>::combine(a2, v2);
                a3 = Op<TAcc, OP>::combine(a3, v3);
                if(kTwoLevel && ++cnt == 8)
                    fold();
            }
            __device__ __forceinline__ void add1(TAcc v)
            {
                a0 = Op<TAcc, OP>::combine(a0, v);
                if(kTwoLevel && ++cnt == 8)
                    fold();
            }
            __device__ __forceinline__ Top result()
            {
                fold();
                return top;
            }
        };

        template <typename TAcc, typename TIn>
        __device__ __forceinline__ TAcc widen(TIn v);
        template <>
        __device__ __forceinline__ float widen<float, float>(float v)
        {
            return v;
        }
        template <>
        __device__ __forceinline__ double widen<double, double>(double v)
        {
            return v;
        }
        template <>
        __device__ __forceinline__ float widen<float, __half>(__half v)
        {
            return __half2float(v);
        }
        template <>
        __device__ __forceinline__ float widen<float, __nv_bfloat16>(__nv_bfloat16 v)
        {
            return __bfloat162float(v);
        }
        template <typename TOut, typename TAcc>
        __device__ __forceinline__ TOut narrow(TAcc v);
        template <>
        __device__ __forceinline__ float narrow<float, float>(float v)
        {
            return v;
        }
        template <>
        __device__ __forceinline__ double narrow<double, double>(double v)
        {
            return v;
        }
        template <>
        __device__ __forceinline__ __half narrow<__half, float>(float v)
        {
            return __float2half_rn(v);
        }
        template <>
        __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, float>(float v)
        {
            return __float2bfloat16_rn(v);
        }

        __device__ __forceinline__ float mulRn(float a, float b)
        {
            return __fmul_rn(a, b);
        }
        __device__ __forceinline__ double mulRn(double a, double b)
        {
            return __dmul_rn(a, b);
        }
        __device__ __forceinline__ float addRn(float a, float b)
        {
            return __fadd_rn(a, b);
        }
        __device__ __forceinline__ double addRn(double a, double b)
        {
            return __dadd_rn(a, b);
        }

        template <typename TIn, typename TAcc>
        __device__ __forceinline__ void epilogue(TAcc acc, TAcc alpha, TAcc beta, const TIn* C, TIn* D, int64_t offD)
        {
            if(alpha != TAcc(1))
                acc = mulRn(acc, alpha);
            if(beta != TAcc(0) && C != nullptr)
                acc = addRn(acc, mulRn(widen<TAcc, TIn>(C[offD]), beta));
            D[offD] = narrow<TIn, TAcc>(acc);
        }

        // 16-byte vector of TIn
        template <typename TIn, int VEC>
        struct alignas(sizeof(TIn) * VEC) Vec
        {
            TIn v[VEC];
        };

        __device__ __forceinline__ void keptOffsets(const RedArgs& a, int64_t o, int64_t& offA, int64_t& offD)
        {
            offA = 0;
            offD = 0;
            for(int d = 0; d < a.nk; d++)
            {
                int64_t c = o % a.kext[d];
                o /= a.kext[d];
                offA += c * a.ksA[d];
                offD += c * a.ksD[d];
            }
        }
        // the same with 32-bit divisions, for kernels launched only when the output count fits 31 bits
        __device__ __forceinline__ void keptOffsets32(const RedArgs& a, int64_t o, int64_t& offA, int64_t& offD)
        {
            offA       = 0;
            offD       = 0;
            uint32_t r = uint32_t(o);
            for(int d = 0; d < a.nk; d++)
            {
                const uint32_t e = uint32_t(a.kext[d]), q = r / e, c = r - q * e;
                r = q;
                offA += int64_t(c) * a.ksA[d];
                offD += int64_t(c) * a.ksD[d];
            }
        }
        // offset of outer reduced index ro (reduced modes 1..nr-1)
        __device__ __forceinline__ int64_t outerRedOffset(const RedArgs& a, int64_t ro)
        {
            int64_t off = 0;
            for(int d = 1; d < a.nr; d++)
            {
                int64_t c = ro % a.rext[d];
                ro /= a.rext[d];
                off += c * a.rsA[d];
            }
            return off;
        }

        template <typename TAcc, int OP, int G>
        __device__ __forceinline__ TAcc groupReduce(TAcc acc, TAcc* smem)
        {
            // groups of 8 lanes (short rows) fold within the group only
#pragma unroll
            for(int s = (G < 32 ? G / 2 : 16); s > 0; s >>= 1)
                acc = Op<TAcc, OP>::combine(acc, __shfl_xor_sync(0xffffffffu, acc, s));
            if(G > 32)
            {
                const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
                if(lane == 0)
                    smem[warp] = acc;
                __syncthreads();
                if(warp == 0)
                {
                    acc = (lane < G / 32) ? smem[lane] : Op<TAcc, OP>::identity();
#pragma unroll
                    for(int s = 16; s > 0; s >>= 1)
                        acc = Op<TAcc, OP>::combine(acc, __shfl_xor_sync(0xffffffffu, acc, s));
                }
            }
            return acc;
        }

        // ------------------------------------------------------------ row kernel
        // blockDim.x = 256. G = 32: eight outputs per block; G = 256: one output per block; G = 8: 32 outputs
        // per block for short rows (a warp per 1 KiB row was bound by the instructions around the loads: offsets,
        // shuffle tree, epilogue). gridDim.y = split.
        template <typename TIn, typename TAcc, int OP, int G, int VEC>
        __global__ void __launch_bounds__(256)
            red_row_kernel(const TIn* __restrict__ A, const TIn* C, TIn* D, TAcc* __restrict__ partial, RedArgs a,
                           TAcc alpha, TAcc beta)
        {
            __shared__ double smem[8];
            constexpr int   perBlock = 256 / G;
            const int       sub = threadIdx.x / G, lane = threadIdx.x % G;
            const int64_t   o = int64_t(blockIdx.x) * perBlock + sub;
            if(G == 32 && o >= a.nOut)
                return;
            const bool    idle = G < 32 && o >= a.nOut; // a sub-warp group beyond the last output stays for the shuffles
            const int64_t L0 = a.rext[0], RO = a.nRed / L0;
            int64_t       roLo = 0, roHi = idle ? 0 : RO, iLo = 0, iHi = L0;
            if(a.split > 1)
            {
                const int64_t s = blockIdx.y;
                if(a.sliceOuter)
                {
                    roLo = s * a.sliceLen;
                    roHi = min(RO, roLo + a.sliceLen);
                }
                else
                {
                    iLo = s * a.sliceLen;
                    iHi = min(L0, iLo + a.sliceLen);
                }
            }
            int64_t offA, offD;
            keptOffsets(a, idle ? 0 : o, offA, offD);
            Accum<TAcc, OP> accum;
            accum.init();
            for(int64_t ro = roLo; ro < roHi; ro++)
            {
                const TIn*    row  = A + offA + outerRedOffset(a, ro);
                const int64_t step = int64_t(G) * VEC;
                int64_t       i    = iLo + int64_t(lane) * VEC;
                // four loads in flight per thread
                for(; i + 3 * step < iHi; i += 4 * step)
                {
                    Vec<TIn, VEC> v0 = *(const Vec<TIn, VEC>*)(row + i);
                    Vec<TIn, VEC> v1 = *(const Vec<TIn, VEC>*)(row + i + step);
                    Vec<TIn, VEC> v2 = *(const Vec<TIn, VEC>*)(row + i + 2 * step);
                    Vec<TIn, VEC> v3 = *(const Vec<TIn, VEC>*)(row + i + 3 * step);
#pragma unroll
                    for(int e = 0; e < VEC; e++)
                        accum.add4(widen<TAcc, TIn>(v0.v[e]), widen<TAcc, TIn>(v1.v[e]), widen<TAcc, TIn>(v2.v[e]),
                                   widen<TAcc, TIn>(v3.v[e]));
                }
                for(; i < iHi; i += step)
                {
                    Vec<TIn, VEC> v0 = *(const Vec<TIn, VEC>*)(row + i);
#pragma unroll
                    for(int e = 0; e < VEC; e++)
                        accum.add1(widen<TAcc, TIn>(v0.v[e]));
                }
            }
            using Top = typename Accum<TAcc, OP>::Top;
            Top acc   = groupReduce<Top, OP, G>(accum.result(), (Top*)smem);
            if(lane == 0 && o < a.nOut)
            {
                if(a.split > 1)
                    partial[int64_t(blockIdx.y) * a.nOut + o] = TAcc(acc);
                else
                    epilogue<TIn, TAcc>(TAcc(acc), alpha, beta, C, D, offD);
            }
        }

        // ------------------------------------------------------------ short-row kernel
        // Contiguous reduced rows of at most 2 KiB: g lanes per output (g = 1, 2, 4, .. 32, a launch argument). Up to 32
        // vector loads a row takes one load per lane, so neighbouring lanes read neighbouring rows and a warp's load
        // covers 32 / g outputs; longer rows take several loads per lane. With further reduced modes a group walks them like an odometer (no division per row), four
        // rows in flight. gridDim.y = split (slices of the outer reduced index).
        template <typename TIn, typename TAcc, int OP, int VEC>
        __global__ void __launch_bounds__(256)
            red_short_kernel(const TIn* __restrict__ A, const TIn* C, TIn* D, TAcc* __restrict__ partial, RedArgs a,
                             TAcc alpha, TAcc beta, int lgG)
        {
            // (a thread may own a single 16-byte load: no division on its way, 64-bit ones least of all)
            const int     g = 1 << lgG, lane = threadIdx.x & (g - 1), sub = threadIdx.x >> lgG;
            const int64_t o    = (int64_t(blockIdx.x) << (8 - lgG)) + sub;
            const bool    idle = o >= a.nOut; // stays for the shuffles
            const int64_t L0 = a.rext[0], RO = a.outer;
            int64_t       roLo = 0, roHi = RO;
            if(a.split > 1)
            {
                roLo = int64_t(blockIdx.y) * a.sliceLen;
                roHi = min(RO, roLo + a.sliceLen);
            }
            const bool has = !idle && int64_t(lane) * VEC < L0;
            int64_t    offA, offD;
            keptOffsets32(a, idle ? 0 : o, offA, offD);
            // coordinates of the outer reduced modes at roLo
            int64_t c[kMaxGroup], off = 0;
            for(int d = 1; d < a.nr; d++)
                c[d] = 0;
            if(roLo != 0) // slices only
            {
                int64_t r = roLo;
                for(int d = 1; d < a.nr; d++)
                {
                    c[d] = r % a.rext[d];
                    r /= a.rext[d];
                    off += c[d] * a.rsA[d];
                }
            }
            auto next = [&]() {
                for(int d = 1; d < a.nr; d++)
                {
                    off += a.rsA[d];
                    if(++c[d] < a.rext[d])
                        return;
                    off -= a.rext[d] * a.rsA[d];
                    c[d] = 0;
                }
            };
            using V        = Vec<TIn, VEC>;
            const TIn* row = A + offA + int64_t(lane) * VEC;
            Accum<TAcc, OP> accum;
            accum.init();
            if(!idle && L0 > int64_t(g) * VEC)
            {
                // several loads per lane and row (rows of up to 2 KiB): four in flight within the row
                const int64_t step = int64_t(g) * VEC;
                for(int64_t ro = roLo; ro < roHi; ro++)
                {
                    const TIn* r = A + offA + off;
                    next();
                    // the loads of a batch are issued together, the last batch of a row with predicates
                    for(int64_t i = int64_t(lane) * VEC; i < L0; i += 4 * step)
                    {
                        const bool p1 = i + step < L0, p2 = i + 2 * step < L0, p3 = i + 3 * step < L0;
                        V          v0 = *reinterpret_cast<const V*>(r + i), v1, v2, v3;
                        if(p1)
                            v1 = *reinterpret_cast<const V*>(r + i + step);
                        if(p2)
                            v2 = *reinterpret_cast<const V*>(r + i + 2 * step);
                        if(p3)
                            v3 = *reinterpret_cast<const V*>(r + i + 3 * step);
                        if(p3)
                        {
#pragma unroll
                            for(int e = 0; e < VEC; e++)
                                accum.add4(widen<TAcc, TIn>(v0.v[e]), widen<TAcc, TIn>(v1.v[e]), widen<TAcc, TIn>(v2.v[e]),
                                           widen<TAcc, TIn>(v3.v[e]));
                        }
                        else
                        {
#pragma unroll
                            for(int e = 0; e < VEC; e++)
                            {
                                accum.add1(widen<TAcc, TIn>(v0.v[e]));
                                if(p1)
                                    accum.add1(widen<TAcc, TIn>(v1.v[e]));
                                if(p2)
                                    accum.add1(widen<TAcc, TIn>(v2.v[e]));
                            }
                        }
                    }
                }
            }
            else if(has)
            {
                int64_t ro = roLo;
                for(; ro + 3 < roHi; ro += 4)
                {
                    const int64_t o0 = off;
                    next();
                    const int64_t o1 = off;
                    next();
                    const int64_t o2 = off;
                    next();
                    const int64_t o3 = off;
                    next();
                    const V v0 = *reinterpret_cast<const V*>(row + o0);
                    const V v1 = *reinterpret_cast<const V*>(row + o1);
                    const V v2 = *reinterpret_cast<const V*>(row + o2);
                    const V v3 = *reinterpret_cast<const V*>(row + o3);
#pragma unroll
                    for(int e = 0; e < VEC; e++)
                        accum.add4(widen<TAcc, TIn>(v0.v[e]), widen<TAcc, TIn>(v1.v[e]), widen<TAcc, TIn>(v2.v[e]),
                                   widen<TAcc, TIn>(v3.v[e]));
                }
                for(; ro < roHi; ro++)
                {
                    const V v0 = *reinterpret_cast<const V*>(row + off);
                    next();
#pragma unroll
                    for(int e = 0; e < VEC; e++)
                        accum.add1(widen<TAcc, TIn>(v0.v[e]));
                }
            }
            using Top = typename Accum<TAcc, OP>::Top;
            Top acc   = accum.result();
            for(int s = g >> 1; s > 0; s >>= 1)
                acc = Op<Top, OP>::combine(acc, __shfl_xor_sync(0xffffffffu, acc, s));
            if(lane == 0 && !idle)
            {
                if(a.split > 1)
                    partial[int64_t(blockIdx.y) * a.nOut + o] = TAcc(acc);
                else
                    epilogue<TIn, TAcc>(TAcc(acc), alpha, beta, C, D, offD);
            }
        }

        // ------------------------------------------------------------ column kernel
        // blockDim = (TX, TY); x runs over the flattened outputs (kept modes by ascending stride in A, so that lanes stay
        // on neighbouring addresses across a short contiguous kept mode too); gridDim.x = ceil(nOut / TX); gridDim.y = split
        template <typename TIn, typename TAcc, int OP>
        __global__ void __launch_bounds__(256)
            red_col_kernel(const TIn* __restrict__ A, const TIn* C, TIn* D, TAcc* __restrict__ partial, RedArgs a,
                           TAcc alpha, TAcc beta)
        {
            __shared__ double smemRaw[256];
            const int       tx = threadIdx.x, ty = threadIdx.y, TX = blockDim.x, TY = blockDim.y;
            const int64_t   o  = int64_t(blockIdx.x) * TX + tx;
            const bool      ok = o < a.nOut;
            int64_t         offA, offD;
            keptOffsets32(a, ok ? o : 0, offA, offD);
            const int64_t L0 = a.rext[0], RO = a.nRed / L0, s0 = a.rsA[0];
            int64_t       roLo = 0, roHi = RO, iLo = 0, iHi = L0;
            if(a.split > 1)
            {
                const int64_t s = blockIdx.y;
                if(a.sliceOuter)
                {
                    roLo = s * a.sliceLen;
                    roHi = min(RO, roLo + a.sliceLen);
                }
                else
                {
                    iLo = s * a.sliceLen;
                    iHi = min(L0, iLo + a.sliceLen);
                }
            }
            Accum<TAcc, OP> accum;
            accum.init();
            if(ok)
            {
                for(int64_t ro = roLo; ro < roHi; ro++)
                {
                    const TIn* col = A + offA + outerRedOffset(a, ro);
                    int64_t    i   = iLo + ty;
                    for(; i + 3 * TY < iHi; i += 4 * TY)
                    {
                        TIn v0 = col[i * s0], v1 = col[(i + TY) * s0], v2 = col[(i + 2 * TY) * s0],
                            v3 = col[(i + 3 * TY) * s0];
                        accum.add4(widen<TAcc, TIn>(v0), widen<TAcc, TIn>(v1), widen<TAcc, TIn>(v2),
                                   widen<TAcc, TIn>(v3));
                    }
                    for(; i < iHi; i += TY)
                        accum.add1(widen<TAcc, TIn>(col[i * s0]));
                }
            }
            using Top          = typename Accum<TAcc, OP>::Top;
            Top* smem          = (Top*)smemRaw;
            Top  acc           = accum.result();
            smem[ty * TX + tx] = acc;
            __syncthreads();
            // TY is a power of two
            for(int h = TY >> 1; h > 0; h >>= 1)
            {
                if(ty < h)
                {
                    acc                = Op<Top, OP>::combine(acc, smem[(ty + h) * TX + tx]);
                    smem[ty * TX + tx] = acc;
                }
                __syncthreads();
            }
            if(ty == 0 && ok)
            {
                if(a.split > 1)
                    partial[int64_t(blockIdx.y) * a.nOut + o] = TAcc(acc);
                else
                    epilogue<TIn, TAcc>(TAcc(acc), alpha, beta, C, D, offD);
            }
        }

        // ------------------------------------------------------------ column kernel, 16-byte loads
        // The same decomposition with VEC consecutive kept elements per thread: one 16-byte load per row, four rows
        // in flight, VEC accumulators. Needs the kept extent, every other stride of A and the base address to be
        // multiples of VEC elements.
        template <typename TIn, typename TAcc, int OP, int VEC>
        __global__ void __launch_bounds__(256)
            red_colv_kernel(const TIn* __restrict__ A, const TIn* C, TIn* D, TAcc* __restrict__ partial, RedArgs a,
                            TAcc alpha, TAcc beta)
        {
            using Top = typename Accum<TAcc, OP>::Top;
            extern __shared__ __align__(16) unsigned char smemDyn[];
            Top*          smem = (Top*)smemDyn; // [TY][TX][VEC]
            const int     tx = threadIdx.x, ty = threadIdx.y, TX = blockDim.x, TY = blockDim.y;
            // VEC neighbouring outputs of the contiguous kept mode (its extent is a multiple of VEC)
            const int64_t o  = (int64_t(blockIdx.x) * TX + tx) * VEC;
            const bool    ok = o < a.nOut;
            int64_t       offA, offD;
            keptOffsets32(a, ok ? o : 0, offA, offD);
            const int64_t L0 = a.rext[0], RO = a.nRed / L0, s0 = a.rsA[0];
            int64_t       roLo = 0, roHi = RO, iLo = 0, iHi = L0;
            if(a.split > 1)
            {
                const int64_t s = blockIdx.y;
                if(a.sliceOuter)
                {
                    roLo = s * a.sliceLen;
                    roHi = min(RO, roLo + a.sliceLen);
                }
                else
                {
                    iLo = s * a.sliceLen;
                    iHi = min(L0, iLo + a.sliceLen);
                }
            }
            using V = Vec<TIn, VEC>;
            Accum<TAcc, OP> accum[VEC];
#pragma unroll
            for(int e = 0; e < VEC; e++)
                accum[e].init();
            if(ok)
            {
                for(int64_t ro = roLo; ro < roHi; ro++)
                {
                    const TIn* col = A + offA + outerRedOffset(a, ro);
                    int64_t    i   = iLo + ty;
                    for(; i + 3 * TY < iHi; i += 4 * TY)
                    {
                        const V v0 = *reinterpret_cast<const V*>(col + i * s0);
                        const V v1 = *reinterpret_cast<const V*>(col + (i + TY) * s0);
                        const V v2 = *reinterpret_cast<const V*>(col + (i + 2 * TY) * s0);
                        const V v3 = *reinterpret_cast<const V*>(col + (i + 3 * TY) * s0);
#pragma unroll
                        for(int e = 0; e < VEC; e++)
                            accum[e].add4(widen<TAcc, TIn>(v0.v[e]), widen<TAcc, TIn>(v1.v[e]), widen<TAcc, TIn>(v2.v[e]),
                                          widen<TAcc, TIn>(v3.v[e]));
                    }
                    for(; i < iHi; i += TY)
                    {
                        const V v = *reinterpret_cast<const V*>(col + i * s0);
#pragma unroll
                        for(int e = 0; e < VEC; e++)
                            accum[e].add1(widen<TAcc, TIn>(v.v[e]));
                    }
                }
            }
            Top acc[VEC];
#pragma unroll
            for(int e = 0; e < VEC; e++)
            {
                acc[e]                             = accum[e].result();
                smem[(ty * TX + tx) * VEC + e] = acc[e];
            }
            __syncthreads();
            for(int h = TY >> 1; h > 0; h >>= 1)
            {
                if(ty < h)
                {
#pragma unroll
                    for(int e = 0; e < VEC; e++)
                    {
                        acc[e]                         = Op<Top, OP>::combine(acc[e], smem[((ty + h) * TX + tx) * VEC + e]);
                        smem[(ty * TX + tx) * VEC + e] = acc[e];
                    }
                }
                __syncthreads();
            }
            if(ty == 0 && ok)
            {
#pragma unroll
                for(int e = 0; e < VEC; e++)
                {
                    if(a.split > 1)
                        partial[int64_t(blockIdx.y) * a.nOut + o + e] = TAcc(acc[e]);
                    else
                        epilogue<TIn, TAcc>(TAcc(acc[e]), alpha, beta, C, D, offD + e * a.ksD[0]);
                }
            }
        }

        // ------------------------------------------------------------ generic kernel
        // G threads per output over the flattened reduced range [lo, hi).
        template <typename TIn, typename TAcc, int OP, int G>
        __global__ void __launch_bounds__(256)
            red_gen_kernel(const TIn* __restrict__ A, const TIn* C, TIn* D, TAcc* __restrict__ partial, RedArgs a,
                           TAcc alpha, TAcc beta)
        {
            __shared__ double smem[8];
            constexpr int   perBlock = 256 / G;
            const int       sub = threadIdx.x / G, lane = threadIdx.x % G;
            const int64_t   o = int64_t(blockIdx.x) * perBlock + sub;
            if(G == 32 && o >= a.nOut)
                return;
            int64_t lo = 0, hi = a.nRed;
            if(a.split > 1)
            {
                lo = int64_t(blockIdx.y) * a.sliceLen;
                hi = min(a.nRed, lo + a.sliceLen);
            }
            int64_t offA, offD;
            keptOffsets(a, o, offA, offD);
            Accum<TAcc, OP> accum;
            accum.init();
            for(int64_t r = lo + lane; r < hi; r += G)
            {
                int64_t rem = r, off = 0;
                for(int d = 0; d < a.nr; d++)
                {
                    int64_t c = rem % a.rext[d];
                    rem /= a.rext[d];
                    off += c * a.rsA[d];
                }
                accum.add1(widen<TAcc, TIn>(A[offA + off]));
            }
            using Top = typename Accum<TAcc, OP>::Top;
            Top acc   = groupReduce<Top, OP, G>(accum.result(), (Top*)smem);
            if(lane == 0 && o < a.nOut)
            {
                if(a.split > 1)
                    partial[int64_t(blockIdx.y) * a.nOut + o] = TAcc(acc);
                else
                    epilogue<TIn, TAcc>(TAcc(acc), alpha, beta, C, D, offD);
            }
        }

        // ------------------------------------------------------------ second pass
        template <typename TIn, typename TAcc, int OP>
        __global__ void __launch_bounds__(256)
            red_finalize_kernel(const TAcc* __restrict__ partial, const TIn* C, TIn* D, RedArgs a, TAcc alpha,
                                TAcc beta)
        {
            const int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
            if(o >= a.nOut)
                return;
            Accum<TAcc, OP> accum;
            accum.init();
            for(int s = 0; s < a.split; s++)
                accum.add1(partial[int64_t(s) * a.nOut + o]);
            int64_t offA, offD;
            keptOffsets(a, o, offA, offD);
            epilogue<TIn, TAcc>(TAcc(accum.result()), alpha, beta, C, D, offD);
        }

        // ------------------------------------------------------------ finish of a reduction split over devices
        // Every device reduced its share of a reduced mode with alpha = 1, beta = 0 and the partial results
        // were combined across devices (one all-reduce with the reduction's operator). This pass applies
        // alpha and beta * C once, element by element over D's layout, in the order of the single-device
        // epilogue. `partial` is laid out like D.
        struct FinishArgs
        {
            int     n; // folded modes of D
            int64_t ext[kMaxGroup], stride[kMaxGroup];
            int64_t total;
        };
        template <typename TIn, typename TAcc>
        __global__ void __launch_bounds__(256)
            red_finish_kernel(const TIn* partial, const TIn* C, TIn* D, FinishArgs a, TAcc alpha, TAcc beta)
        {
            for(int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < a.total;
                i += int64_t(gridDim.x) * blockDim.x)
            {
                int64_t off = 0, r = i;
                for(int d = 0; d < a.n; d++)
                {
                    off += (r % a.ext[d]) * a.stride[d];
                    r /= a.ext[d];
                }
                epilogue<TIn, TAcc>(widen<TAcc, TIn>(partial[off]), alpha, beta, C, D, off);
            }
        }
        template <typename TIn, typename TAcc>
        cudaError_t launchFinish(const FinishArgs& a, double alpha, const void* partial, double beta, const void* C,
                                 void* D, cudaStream_t stream)
        {
            const int64_t blocks = std::min<int64_t>((a.total + 255) / 256, 148 * 8);
            red_finish_kernel<TIn, TAcc><<<unsigned(blocks), 256, 0, stream>>>((const TIn*)partial, (const TIn*)C, (TIn*)D, a,
                                                                               TAcc(alpha), TAcc(beta));
            noteLaunch("red_finish");
            return cudaGetLastError();
        }

        template <typename TIn, typename TAcc, int OP>
        cudaError_t launchTyped(const ReducePlan& p, TAcc alpha, const void* Av, TAcc beta, const void* Cv, void* Dv,
                                void* workspace, cudaStream_t stream)
        {
            const TIn* A = (const TIn*)Av;
            const TIn* C = (const TIn*)Cv;
            TIn*       D = (TIn*)Dv;
            RedArgs    a{};
            a.nk = p.nk;
            a.nr = p.nr;
            for(int i = 0; i < kMaxGroup; i++)
            {
                a.kext[i] = p.kext[i];
                a.ksA[i]  = p.ksA[i];
                a.ksD[i]  = p.ksD[i];
                a.rext[i] = p.rext[i];
                a.rsA[i]  = p.rsA[i];
            }
            a.nOut  = p.nOut;
            a.nRed  = p.nRed;
            a.split = (workspace != nullptr) ? p.split : 1;
            TAcc*         partial = (TAcc*)workspace;
            const int64_t L0 = p.rext[0], RO = p.nRed / L0;
            a.outer          = RO;
            if(a.split > 1)
            {
                if(p.kind == RED_GENERIC)
                {
                    a.sliceLen = (p.nRed + a.split - 1) / a.split;
                }
                else if(RO >= a.split)
                {
                    a.sliceOuter = 1;
                    a.sliceLen   = (RO + a.split - 1) / a.split;
                }
                else
                {
                    a.sliceOuter = 0;
                    int64_t len  = (L0 + a.split - 1) / a.split;
                    len          = (len + 15) / 16 * 16; // keeps vector loads aligned
                    a.sliceLen   = len;
                    a.split      = int((L0 + len - 1) / len);
                }
            }
            const unsigned gy = unsigned(a.split);
            if(p.nOut > 0x7fffffffll)
                return cudaErrorInvalidConfiguration;
            if(p.kind == RED_ROW && p.shortLanes > 0)
            {
                int g = p.shortLanes, lgG = 0;
                while((1 << lgG) < g)
                    lgG++;
                const dim3 grid(unsigned((p.nOut + 256 / g - 1) / (256 / g)), gy);
                if(a.split > 1 && !a.sliceOuter)
                    return cudaErrorInvalidConfiguration; // the planner slices the outer reduced index only
                constexpr int full = 16 / int(sizeof(TIn));
                if(p.shortVec == full)
                    red_short_kernel<TIn, TAcc, OP, full><<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta, lgG);
                else if(full >= 4 && p.shortVec == full / 2)
                    red_short_kernel<TIn, TAcc, OP, (full >= 4 ? full / 2 : 1)>
                        <<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta, lgG);
                else if(full >= 8 && p.shortVec == full / 4)
                    red_short_kernel<TIn, TAcc, OP, (full >= 8 ? full / 4 : 1)>
                        <<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta, lgG);
                else if(p.shortVec == 1)
                    red_short_kernel<TIn, TAcc, OP, 1><<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta, lgG);
                else
                    return cudaErrorInvalidConfiguration;
                noteLaunch("red_short");
            }
            else if(p.kind == RED_ROW)
            {
                const bool perBlock = (p.nRed >= 8192 && p.nOut < 4096) || a.split > 1;
                if(perBlock)
                {
                    dim3 grid(unsigned(p.nOut), gy);
                    if(p.vec == 16 / int(sizeof(TIn)))
                        red_row_kernel<TIn, TAcc, OP, 256, 16 / sizeof(TIn)>
                            <<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta);
                    else
                        red_row_kernel<TIn, TAcc, OP, 256, 1><<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta);
                }
                else if(p.vec == 16 / int(sizeof(TIn)) && p.nr == 1 && p.rext[0] * int64_t(sizeof(TIn)) <= 2048)
                {
                    // a row of at most 2 KiB: eight lanes per output, four outputs per warp
                    dim3 grid(unsigned((p.nOut + 31) / 32), gy);
                    red_row_kernel<TIn, TAcc, OP, 8, 16 / sizeof(TIn)><<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta);
                }
                else
                {
                    dim3 grid(unsigned((p.nOut + 7) / 8), gy);
                    if(p.vec == 16 / int(sizeof(TIn)))
                        red_row_kernel<TIn, TAcc, OP, 32, 16 / sizeof(TIn)>
                            <<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta);
                    else
                        red_row_kernel<TIn, TAcc, OP, 32, 1><<<grid, 256, 0, stream>>>(A, C, D, partial, a, alpha, beta);
                }
                noteLaunch("red_row");
            }
            else if(p.kind == RED_COL)
            {
                // block shape and vector width come with the plan
                constexpr int VEC = 16 / int(sizeof(TIn));
                const int     tx = p.colTx, ty = p.colTy;
                if(p.colVec == VEC && VEC > 1 && (uintptr_t(A) & 15) == 0)
                {
                    const int64_t blocks = (p.nOut / VEC + tx - 1) / tx;
                    if(blocks > 0x7fffffffll)
                        return cudaErrorInvalidConfiguration;
                    using Top         = typename Accum<TAcc, OP>::Top;
                    const size_t smem = size_t(tx) * ty * VEC * sizeof(Top);
                    red_colv_kernel<TIn, TAcc, OP, VEC>
                        <<<dim3(unsigned(blocks), gy), dim3(tx, ty), smem, stream>>>(A, C, D, partial, a, alpha, beta);
                }
                else
                {
                    // colTx counts vectors when the plan has them; without (a pointer the planner did not see) lanes are
                    // single outputs
                    const int     txs    = p.colVec > 1 ? 32 : tx;
                    const int     tys    = p.colVec > 1 ? std::min(ty, 8) : ty;
                    const int64_t blocks = (p.nOut + txs - 1) / txs;
                    if(blocks > 0x7fffffffll)
                        return cudaErrorInvalidConfiguration;
                    red_col_kernel<TIn, TAcc, OP>
                        <<<dim3(unsigned(blocks), gy), dim3(txs, tys), 0, stream>>>(A, C, D, partial, a, alpha, beta);
                }
                noteLaunch("red_col");
            }
            else
            {
                if(p.nRed >= 4096 || a.split > 1)
                    red_gen_kernel<TIn, TAcc, OP, 256>
                        <<<dim3(unsigned(p.nOut), gy), 256, 0, stream>>>(A, C, D, partial, a, alpha, beta);
                else
                    red_gen_kernel<TIn, TAcc, OP, 32>
                        <<<dim3(unsigned((p.nOut + 7) / 8), gy), 256, 0, stream>>>(A, C, D, partial, a, alpha, beta);
                noteLaunch("red_generic");
            }
            cudaError_t e = cudaGetLastError();
            if(e != cudaSuccess)
                return e;
            if(a.split > 1)
            {
                red_finalize_kernel<TIn, TAcc, OP>
                    <<<unsigned((p.nOut + 255) / 256), 256, 0, stream>>>(partial, C, D, a, alpha, beta);
                noteLaunch("red_finalize");
                e = cudaGetLastError();
            }
            return e;
        }

        template <typename TIn, typename TAcc>
        cudaError_t launchOp(const ReducePlan& p, int op, double alpha, const void* A, double beta, const void* C,
                             void* D, void* ws, cudaStream_t s)
        {
            switch(op)
            {
            case OP_ADD: return launchTyped<TIn, TAcc, OP_ADD>(p, TAcc(alpha), A, TAcc(beta), C, D, ws, s);
            case OP_MUL: return launchTyped<TIn, TAcc, OP_MUL>(p, TAcc(alpha), A, TAcc(beta), C, D, ws, s);
            case OP_MAX: return launchTyped<TIn, TAcc, OP_MAX>(p, TAcc(alpha), A, TAcc(beta), C, D, ws, s);
            case OP_MIN: return launchTyped<TIn, TAcc, OP_MIN>(p, TAcc(alpha), A, TAcc(beta), C, D, ws, s);
            }
            return cudaErrorInvalidValue;
        }
    } // namespace

    // ------------------------------------------------------------------ built-in scratch
    // Scratch for the two-pass reduction that lives inside the library image instead of in
    // memory the caller allocates. Every device that loads the library carries these bytes
    // until the process exits; all calls on a device share them.
    static __device__ __align__(256) unsigned char gReduceScratch[kStaticScratchBytes];

    cudaError_t launchReductionStaticScratch(const ReducePlan& plan, int typeA, int computeType, int op, double alpha,
                                             const void* A, double beta, const void* C, void* D, int device,
                                             cudaStream_t stream)
    {
        // In host code the array's name is only a handle for the runtime, not a device address.
        // The address is looked up once per device, with that device current, and kept.
        static std::mutex lock;
        static void*      address[kMaxDevices] = {};
        if(device < 0 || device >= kMaxDevices)
            return cudaErrorInvalidDevice;
        void* scratch = nullptr;
        {
            std::lock_guard<std::mutex> guard(lock);
            if(address[device] == nullptr)
            {
                void*       p = nullptr;
                cudaError_t e = cudaGetSymbolAddress(&p, gReduceScratch);
                if(e != cudaSuccess)
                    return e;
                address[device] = p;
            }
            scratch = address[device];
        }
        // pass 1 writes every partial slot that pass 2 reads, so nothing has to start at zero
        return launchReduction(plan, typeA, computeType, op, alpha, A, beta, C, D, plan.split > 1 ? scratch : nullptr,
                               stream);
    }

    cudaError_t launchReductionFinish(int typeD, double alpha, const void* partial, double beta, const void* C, void* D,
                                      int rank, const int64_t* lens, const int64_t* strides, cudaStream_t stream)
    {
        if(rank < 0 || rank > kMaxGroup)
            return cudaErrorInvalidValue;
        // D's modes by ascending stride, neighbours merged where they are contiguous
        FinishArgs a{};
        int        order[kMaxGroup];
        int        n = 0;
        a.total      = 1;
        for(int i = 0; i < rank; i++)
        {
            if(lens[i] <= 0)
                return cudaSuccess; // an empty tensor
            a.total *= lens[i];
            if(lens[i] == 1)
                continue;
            int j = n++;
            for(; j > 0 && strides[order[j - 1]] > strides[i]; j--)
                order[j] = order[j - 1];
            order[j] = i;
        }
        for(int j = 0; j < n; j++)
        {
            const int64_t e = lens[order[j]], st = strides[order[j]];
            if(a.n > 0 && a.stride[a.n - 1] * a.ext[a.n - 1] == st)
                a.ext[a.n - 1] *= e;
            else
            {
                a.ext[a.n]    = e;
                a.stride[a.n] = st;
                a.n++;
            }
        }
        switch(typeD)
        {
        case CUDA_R_32F: return launchFinish<float, float>(a, alpha, partial, beta, C, D, stream);
        case CUDA_R_64F: return launchFinish<double, double>(a, alpha, partial, beta, C, D, stream);
        case CUDA_R_16F: return launchFinish<__half, float>(a, alpha, partial, beta, C, D, stream);
        case CUDA_R_16BF: return launchFinish<__nv_bfloat16, float>(a, alpha, partial, beta, C, D, stream);
        }
        return cudaErrorInvalidValue;
    }

    uint64_t reductionWorkspaceBytes(const ReducePlan& plan, int computeType)
    {
        if(plan.split <= 1)
            return 0;
        const uint64_t accSize = (computeType == HIPTENSOR_COMPUTE_64F) ? 8 : 4;
        return uint64_t(plan.split) * uint64_t(plan.nOut) * accSize;
    }

    cudaError_t launchReduction(const ReducePlan& plan, int typeA, int computeType, int op, double alpha,
                                const void* A, double beta, const void* C, void* D, void* workspace,
                                cudaStream_t stream)
    {
        if(plan.nOut == 0)
            return cudaSuccess;
        switch(typeA)
        {
        case CUDA_R_32F: return launchOp<float, float>(plan, op, alpha, A, beta, C, D, workspace, stream);
        case CUDA_R_64F: return launchOp<double, double>(plan, op, alpha, A, beta, C, D, workspace, stream);
        case CUDA_R_16F: return launchOp<__half, float>(plan, op, alpha, A, beta, C, D, workspace, stream);
        case CUDA_R_16BF: return launchOp<__nv_bfloat16, float>(plan, op, alpha, A, beta, C, D, workspace, stream);
        }
        (void)computeType;
        return cudaErrorInvalidValue;
    }
} // namespace htb
