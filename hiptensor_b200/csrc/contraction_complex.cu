// Complex contraction (cf32 / cf64) on the real contraction kernels.
//
// The reference splits A, B, C and D into real and imaginary planes in freshly allocated device memory, runs
// four real contractions and recombines with alpha and beta in a last kernel
// (library/src/contraction/device/device_contraction_bilinear_complex.hpp:454-470,535-558,
// library/src/contraction/contraction_pack_util.hpp:40-120). Here the work is ONE real contraction of twice
// the N and twice the K extent (planner.cpp, planComplexContraction): a complex tensor already is a real tensor
// with an innermost mode of extent 2, so the larger operand and D are used where they lie; only the smaller
// operand X is copied, once, into the caller's workspace as
//     X2[free.., 0, k.., :] = ( re, -im )      X2[free.., 1, k.., :] = ( im, re )      of alpha * X.
// alpha is applied during the copy. beta * C is either the real epilogue of the contraction kernel (beta real)
// or a pass D = beta * C before it (the kernel then adds D to the sums: C may alias D in every kernel).
// The real kernels are the FP64 tensor-pipe kernel for cf64 and the TF32 big/small split kernel (or the FMA
// kernel) for cf32, so accuracy is that of the real paths. For cf32 the other operand is copied as well (packed,
// contracted modes innermost) when its layout would otherwise keep the problem off the tensor cores.
#include <cuda_runtime.h>

#include <algorithm>

#include "kernels.hpp"

namespace htb
{
    namespace
    {
        struct CxDims
        {
            int     rank, nFree;
            int64_t ext[kMaxRank], stride[kMaxRank];
        };

        template <typename T>
        struct Vec2;
        template <>
        struct Vec2<float>
        {
            using type = float2;
        };
        template <>
        struct Vec2<double>
        {
            using type = double2;
        };

        // One thread per complex element of X, contracted index fastest (the copy's rows are written contiguously;
        // the reads follow X's strides). PLAIN: a packed copy of the elements as they are (one row per free index).
        template <typename T, bool PLAIN>
        __global__ void __launch_bounds__(256) complex_expand_kernel(const typename Vec2<T>::type* __restrict__ X,
                                                                     typename Vec2<T>::type* __restrict__ X2, CxDims d,
                                                                     int64_t F, int64_t K, T ar, T ai, int unitAlpha)
        {
            using V             = typename Vec2<T>::type;
            const int64_t total = F * K;
            for(int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
            {
                const int64_t k = i % K, f = i / K;
                int64_t       off = 0, rem = k;
                for(int m = d.rank - 1; m >= d.nFree; m--)
                {
                    off += (rem % d.ext[m]) * d.stride[m];
                    rem /= d.ext[m];
                }
                rem = f;
                for(int m = d.nFree - 1; m >= 0; m--)
                {
                    off += (rem % d.ext[m]) * d.stride[m];
                    rem /= d.ext[m];
                }
                const V x = X[off];
                if(PLAIN)
                {
                    X2[i] = x;
                    continue;
                }
                T       pr = x.x, pi = x.y;
                if(!unitAlpha)
                {
                    pr = ar * x.x - ai * x.y;
                    pi = ar * x.y + ai * x.x;
                }
                V lo, hi;
                lo.x = pr;
                lo.y = -pi;
                hi.x = pi;
                hi.y = pr;
                X2[f * 2 * K + k]     = lo; // row (f, 0)
                X2[f * 2 * K + K + k] = hi; // row (f, 1)
            }
        }

        // D = beta * C over D's index space (C is addressed with D's strides, as everywhere in the contraction).
        // Dimensions are sorted by ascending stride, dimension 0 fastest.
        template <typename T>
        __global__ void __launch_bounds__(256) complex_scale_kernel(const typename Vec2<T>::type* C,
                                                                    typename Vec2<T>::type* D, CxDims d, int64_t total,
                                                                    T br, T bi)
        {
            using V = typename Vec2<T>::type;
            for(int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
            {
                int64_t off = 0, rem = i;
                for(int m = 0; m < d.rank; m++)
                {
                    off += (rem % d.ext[m]) * d.stride[m];
                    rem /= d.ext[m];
                }
                const V c = C[off];
                V       o;
                o.x    = c.x * br - c.y * bi;
                o.y    = c.y * br + c.x * bi;
                D[off] = o;
            }
        }

        template <typename T>
        cudaError_t runTyped(const ContractionPlan& p, double ar, double ai, const void* A, const void* B, double br,
                             double bi, const void* C, void* D, void* workspace, uint64_t workspaceBytes, int smCount,
                             int* deviceStatus, cudaStream_t stream)
        {
            using V        = typename Vec2<T>::type;
            const void* X  = (p.complexKind == 1) ? A : B;
            void*       X2 = workspace;
            CxDims      d{};
            d.rank  = p.xRank;
            d.nFree = p.xFree;
            int64_t F = 1, K = 1;
            for(int i = 0; i < p.xRank; i++)
            {
                d.ext[i]    = p.xExt[i];
                d.stride[i] = p.xStride[i];
                (i < p.xFree ? F : K) *= p.xExt[i];
            }
            const int     sms   = smCount > 0 ? smCount : 148;
            const int64_t total = F * K;
            int           grid  = int(std::min<int64_t>((total + 255) / 256, int64_t(sms) * 8));
            const int     unit  = (ar == 1.0 && ai == 0.0) ? 1 : 0;
            complex_expand_kernel<T, false><<<grid, 256, 0, stream>>>((const V*)X, (V*)X2, d, F, K, T(ar), T(ai), unit);
            cudaError_t e = cudaGetLastError();
            if(e != cudaSuccess)
                return e;
            noteLaunch("complex_expand");
            const void* Y = (p.complexKind == 1) ? B : A;
            if(p.yCopy)
            {
                CxDims dy{};
                dy.rank  = p.yRank;
                dy.nFree = p.yFree;
                int64_t FY = 1, KY = 1;
                for(int i = 0; i < p.yRank; i++)
                {
                    dy.ext[i]    = p.yExt[i];
                    dy.stride[i] = p.yStride[i];
                    (i < p.yFree ? FY : KY) *= p.yExt[i];
                }
                void* Y2 = (char*)workspace + p.yOffset;
                grid     = int(std::min<int64_t>((FY * KY + 255) / 256, int64_t(sms) * 8));
                complex_expand_kernel<T, true><<<grid, 256, 0, stream>>>((const V*)Y, (V*)Y2, dy, FY, KY, T(0), T(0), 1);
                e = cudaGetLastError();
                if(e != cudaSuccess)
                    return e;
                noteLaunch("complex_copy");
                Y = Y2;
            }

            const bool bilinear = p.bilinear != 0 && C != nullptr;
            float      betaReal = 0.f;
            const void* Cin     = nullptr;
            if(bilinear)
            {
                const bool direct = (bi == 0.0) && double(float(br)) == br; // the real epilogue holds beta as float
                if(direct)
                {
                    betaReal = float(br);
                    Cin      = C;
                }
                else
                {
                    CxDims  dd{};
                    int64_t n = 1;
                    int     r = 0;
                    for(int i = 0; i < p.dRank; i++)
                        if(p.dExt[i] > 1)
                        {
                            dd.ext[r]    = p.dExt[i];
                            dd.stride[r] = p.dStride[i];
                            r++;
                            n *= p.dExt[i];
                        }
                    for(int i = 1; i < r; i++) // insertion sort by stride
                        for(int j = i; j > 0 && dd.stride[j] < dd.stride[j - 1]; j--)
                        {
                            std::swap(dd.stride[j], dd.stride[j - 1]);
                            std::swap(dd.ext[j], dd.ext[j - 1]);
                        }
                    dd.rank = r;
                    grid    = int(std::min<int64_t>((n + 255) / 256, int64_t(sms) * 8));
                    complex_scale_kernel<T><<<grid, 256, 0, stream>>>((const V*)C, (V*)D, dd, n, T(br), T(bi));
                    e = cudaGetLastError();
                    if(e != cudaSuccess)
                        return e;
                    noteLaunch("complex_scale");
                    betaReal = 1.f;
                    Cin      = D;
                }
            }
            void*          inner      = p.workspaceBytes ? (char*)workspace + p.expandBytes : nullptr;
            const uint64_t innerBytes = workspaceBytes > p.expandBytes ? workspaceBytes - p.expandBytes : 0;
            return launchContraction(p, 1.0f, p.complexKind == 1 ? X2 : Y, p.complexKind == 1 ? Y : X2, betaReal, Cin, D,
                                     inner, std::min<uint64_t>(innerBytes, p.workspaceBytes), smCount, deviceStatus, stream);
        }
    } // namespace

    cudaError_t launchComplexContraction(const ContractionPlan& plan, double alphaRe, double alphaIm, const void* A,
                                         const void* B, double betaRe, double betaIm, const void* C, void* D,
                                         void* workspace, uint64_t workspaceBytes, int smCount, int* deviceStatus,
                                         cudaStream_t stream)
    {
        if(plan.complexKind == 0 || workspace == nullptr || workspaceBytes < plan.expandBytes)
            return cudaErrorInvalidValue;
        if(uintptr_t(workspace) & 15)
            return cudaErrorMisalignedAddress;
        if(plan.typeD == CUDA_R_32F)
            return runTyped<float>(plan, alphaRe, alphaIm, A, B, betaRe, betaIm, C, D, workspace, workspaceBytes, smCount,
                                   deviceStatus, stream);
        if(plan.typeD == CUDA_R_64F)
            return runTyped<double>(plan, alphaRe, alphaIm, A, B, betaRe, betaIm, C, D, workspace, workspaceBytes,
                                    smCount, deviceStatus, stream);
        return cudaErrorNotSupported;
    }
} // namespace htb
