// Packed copies of the operands of a real contraction (plan.packReal).
//
// The tensor-core kernels read an operand through TMA: every stride but one must be a multiple of 16 bytes, and the
// contracted modes must form a block mode both operands can be walked along. Operands that do not fit (extents of
// 50 f16 elements, contracted modes interleaved with free ones in different orders, ...) used to run on the gathered
// FMA kernel at 10-18 TFLOP/s whatever their size. From about a GFLOP on (planner.cpp, planContraction) each operand
// is first copied into the caller's workspace as a matrix with one row per free index and the contracted modes
// merged, in the same order for both operands, into one innermost mode padded with zeros to a multiple of 16 bytes;
// the contraction of the copies runs on the tensor cores. The copies cost one pass over A and B (M K + N K elements
// against M N K multiply-adds).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "kernels.hpp"

namespace htb
{
    namespace
    {
        struct PackDims
        {
            int      rank, nFree;
            uint32_t ext[kMaxRank];
            int64_t  stride[kMaxRank];
        };

        // One thread per 16 bytes of the copy (V elements), the merged contracted index fastest: the writes are contiguous
        // 16-byte stores, the reads follow the source strides. The row and the first contracted index are decoded once
        // per thread (32-bit divisions: the copy has fewer than 2^32 vectors), the following indices by stepping the
        // contracted coordinates like an odometer. Rows are padded with zeros from K to Kp (a multiple of V).
        template <typename T>
        __global__ void __launch_bounds__(256)
            contraction_pack_kernel(const T* __restrict__ X, T* __restrict__ X2, PackDims d, uint32_t total, uint32_t K, uint32_t Kp)
        {
            constexpr int  V      = 16 / int(sizeof(T));
            const uint32_t perRow = Kp / V;
            for(uint32_t i = blockIdx.x * 256u + threadIdx.x; i < total; i += gridDim.x * 256u)
            {
                const uint32_t f = i / perRow, k0 = (i - f * perRow) * V;
                int64_t        off = 0;
                uint32_t       c[kMaxRank];
                uint32_t       rem = k0;
                for(int m = d.rank - 1; m >= d.nFree; m--)
                {
                    const uint32_t q = rem / d.ext[m];
                    c[m]             = rem - q * d.ext[m];
                    off += int64_t(c[m]) * d.stride[m];
                    rem = q;
                }
                rem = f;
                for(int m = d.nFree - 1; m >= 0; m--)
                {
                    const uint32_t q = rem / d.ext[m];
                    off += int64_t(rem - q * d.ext[m]) * d.stride[m];
                    rem = q;
                }
                union
                {
                    uint4 w;
                    T     e[V];
                } v;
                v.w = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for(int e = 0; e < V; e++)
                {
                    if(k0 + e < K)
                        v.e[e] = X[off];
                    // next contracted index
                    for(int m = d.rank - 1; m >= d.nFree; m--)
                    {
                        off += d.stride[m];
                        if(++c[m] < d.ext[m])
                            break;
                        off -= int64_t(d.ext[m]) * d.stride[m];
                        c[m] = 0;
                    }
                }
                *reinterpret_cast<uint4*>(X2 + int64_t(f) * Kp + k0) = v.w;
            }
        }

        template <typename T>
        cudaError_t packOne(const void* X, void* X2, int rank, int nFree, const int64_t* ext, const int64_t* stride,
                            int64_t K, int64_t Kp, int smCount, cudaStream_t stream)
        {
            PackDims d{};
            d.rank  = rank;
            d.nFree = nFree;
            int64_t rows = 1;
            for(int i = 0; i < rank; i++)
            {
                if(ext[i] >= (int64_t(1) << 31))
                    return cudaErrorInvalidValue;
                d.ext[i]    = uint32_t(ext[i]);
                d.stride[i] = stride[i];
                if(i < nFree)
                    rows *= ext[i];
            }
            if(K >= (int64_t(1) << 31) || Kp >= (int64_t(1) << 31))
                return cudaErrorInvalidValue;
            const int64_t total = rows * (Kp / (16 / int64_t(sizeof(T))));
            if(total >= (int64_t(1) << 32) - 65536)
                return cudaErrorInvalidValue; // more than 64 GiB of copy
            const int sms  = smCount > 0 ? smCount : 148;
            const int grid = int(std::min<int64_t>((total + 255) / 256, int64_t(sms) * 32));
            contraction_pack_kernel<T><<<grid, 256, 0, stream>>>((const T*)X, (T*)X2, d, uint32_t(total), uint32_t(K), uint32_t(Kp));
            return cudaGetLastError();
        }
    } // namespace

    cudaError_t launchPackedContraction(const ContractionPlan& plan, float alpha, const void* A, const void* B, float beta,
                                        const void* C, void* D, void* workspace, uint64_t workspaceBytes, int smCount,
                                        int* deviceStatus, cudaStream_t stream)
    {
        if(!plan.packReal || workspace == nullptr || workspaceBytes < plan.expandBytes)
            return cudaErrorInvalidValue;
        // plan.typeA / typeB follow the plan's swap; both operands have the same type
        const int type = plan.typeA;
        // the copies are written with 16-byte stores and read by TMA: they start at a multiple of 256 bytes whatever the
        // caller's pointer (plan.expandBytes has 256 bytes of slack for that)
        unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 255u) & ~uintptr_t(255));
        void*          A2   = base;
        void*          B2   = base + plan.yOffset;
        cudaError_t e;
        if(type == CUDA_R_32F)
        {
            e = packOne<float>(A, A2, plan.xRank, plan.xFree, plan.xExt, plan.xStride, plan.packK, plan.packKp, smCount, stream);
            if(e == cudaSuccess)
                e = packOne<float>(B, B2, plan.yRank, plan.yFree, plan.yExt, plan.yStride, plan.packK, plan.packKp, smCount, stream);
        }
        else
        {
            // f16 and bf16 are moved as 16-bit words
            e = packOne<unsigned short>(A, A2, plan.xRank, plan.xFree, plan.xExt, plan.xStride, plan.packK, plan.packKp, smCount,
                                        stream);
            if(e == cudaSuccess)
                e = packOne<unsigned short>(B, B2, plan.yRank, plan.yFree, plan.yExt, plan.yStride, plan.packK, plan.packKp,
                                            smCount, stream);
        }
        if(e != cudaSuccess)
            return e;
        noteLaunch("contraction_pack", 2);
        unsigned char* rest = static_cast<unsigned char*>(workspace) + plan.expandBytes;
        rest                = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(rest) + 255u) & ~uintptr_t(255));
        if(plan.workspaceBytes && rest + plan.workspaceBytes > static_cast<unsigned char*>(workspace) + workspaceBytes)
            return cudaErrorInvalidValue;
        return launchContraction(plan, alpha, A2, B2, beta, C, D, plan.workspaceBytes ? rest : nullptr, plan.workspaceBytes,
                                 smCount, deviceStatus, stream);
    }
} // namespace htb
