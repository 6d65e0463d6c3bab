// Permutation kernels for sm_100a: B[perm(i)] = opB(alpha * opA(A[i])).
//
// Three kernels, chosen by the planner (planner.hpp PermKind):
//   perm_copy_kernel : A's and B's fastest folded modes coincide; coalesced row copy.
//   perm_tile_kernel : 64x64 tile through padded shared memory, plain loads/stores;
//                      any extents, f32 and f16.
//   perm_tma_kernel  : f32, extents multiple of 4: TMA box loads into 128B-swizzled
//                      shared memory, a 4x4 register transpose per thread with a
//                      diagonal thread->chunk assignment that is bank-conflict free on
//                      both sides, 128-bit shared accesses, TMA box stores.
//
// They replace the CK DeviceElementwiseImpl instances the reference enumerates
// (library/src/permutation/device/permutation_scale_f32_instances.hpp:47-87).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "kernels.hpp"

namespace htb
{
    namespace
    {
        struct PermArgs
        {
            int     ndim, q;
            int64_t ext[kMaxGroup], sA[kMaxGroup], sB[kMaxGroup];
            float   alpha;
            int     opA, opB; // 1 identity, 2 square
        };

        // f32 path: everything in float. f16 path: intermediates stay in half, the scale is
        // a half*half product (CK's Scale functor for half, which the reference applies).
        template <typename T>
        struct Elem;
        template <>
        struct Elem<float>
        {
            static __device__ __forceinline__ float apply(float x, float alpha, int opA, int opB)
            {
                if(opA == 2)
                    x = __fmul_rn(x, x);
                x = __fmul_rn(alpha, x);
                if(opB == 2)
                    x = __fmul_rn(x, x);
                return x;
            }
        };
        template <>
        struct Elem<__half>
        {
            static __device__ __forceinline__ __half apply(__half x, float alpha, int opA, int opB)
            {
                if(opA == 2)
                    x = __hmul(x, x);
                x = __hmul(__float2half_rn(alpha), x);
                if(opB == 2)
                    x = __hmul(x, x);
                return x;
            }
        };
        template <typename TO, typename TI>
        __device__ __forceinline__ TO convertOut(TI v);
        template <>
        __device__ __forceinline__ float convertOut<float, float>(float v)
        {
            return v;
        }
        template <>
        __device__ __forceinline__ __half convertOut<__half, __half>(__half v)
        {
            return v;
        }
        template <>
        __device__ __forceinline__ float convertOut<float, __half>(__half v)
        {
            return __half2float(v);
        }

        // ------------------------------------------------------------ copy kernel
        // grid.x covers rows (all folded modes but the first); blockDim = (TX, 256/TX).
        template <typename TI, typename TO>
        __global__ void __launch_bounds__(256) perm_copy_kernel(const TI* __restrict__ A, TO* __restrict__ B,
                                                                PermArgs a, int64_t rows)
        {
            const int     tx  = threadIdx.x;
            const int64_t row = int64_t(blockIdx.x) * blockDim.y + threadIdx.y;
            if(row >= rows)
                return;
            int64_t rem = row, offA = 0, offB = 0;
            for(int d = 1; d < a.ndim; d++)
            {
                int64_t c = rem % a.ext[d];
                rem /= a.ext[d];
                offA += c * a.sA[d];
                offB += c * a.sB[d];
            }
            for(int64_t i = tx; i < a.ext[0]; i += blockDim.x)
            {
                TI v          = A[offA + i];
                B[offB + i] = convertOut<TO, TI>(Elem<TI>::apply(v, a.alpha, a.opA, a.opB));
            }
        }

        // ------------------------------------------------------------ padded-tile kernel
        constexpr int kTile = 64;

        template <typename TI, typename TO>
        __global__ void __launch_bounds__(256)
            perm_tile_kernel(const TI* __restrict__ A, TO* __restrict__ B, PermArgs a, int tilesP, int tilesQ)
        {
            __shared__ TI tile[kTile][kTile + 1];
            int64_t       bid = blockIdx.x;
            const int     tp  = int(bid % tilesP);
            bid /= tilesP;
            const int tq = int(bid % tilesQ);
            bid /= tilesQ;
            int64_t offA = 0, offB = 0;
            for(int d = 1; d < a.ndim; d++)
            {
                if(d == a.q)
                    continue;
                int64_t c = bid % a.ext[d];
                bid /= a.ext[d];
                offA += c * a.sA[d];
                offB += c * a.sB[d];
            }
            const int64_t p0 = int64_t(tp) * kTile, q0 = int64_t(tq) * kTile;
            const int     tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
            const int64_t sAq = a.sA[a.q], sBp = a.sB[0];
            // load: lanes run along p (contiguous in A)
            {
                const int64_t p     = p0 + tx;
                const bool    pok   = p < a.ext[0];
                const TI*     src   = A + offA + p;
#pragma unroll
                for(int j = 0; j < kTile / 4; j++)
                {
                    const int     ql = ty + 4 * j;
                    const int64_t qq = q0 + ql;
                    if(pok && qq < a.ext[a.q])
                        tile[ql][tx] = src[qq * sAq];
                }
            }
            __syncthreads();
            // store: lanes run along q (contiguous in B)
            {
                const int64_t qq  = q0 + tx;
                const bool    qok = qq < a.ext[a.q];
                TO*           dst = B + offB + qq;
#pragma unroll
                for(int j = 0; j < kTile / 4; j++)
                {
                    const int     pl = ty + 4 * j;
                    const int64_t p  = p0 + pl;
                    if(qok && p < a.ext[0])
                        dst[p * sBp] = convertOut<TO, TI>(Elem<TI>::apply(tile[tx][pl], a.alpha, a.opA, a.opB));
                }
            }
        }

        // ------------------------------------------------------------ TMA kernel (f32)
        // Tile = (32*NP) x (32*NQ) elements of the (p, q) plane. Input boxes: NP boxes of
        // [32*NQ rows of q][32 floats of p]; output boxes: NQ boxes of [32*NP rows of p]
        // [32 floats of q]. Rows are 128 bytes, swizzled by TMA (16-byte chunk index XOR
        // row index mod 8), buffers 1024-byte aligned.
        struct PermTmaArgs
        {
            int     ndim, q;
            int     posP_B, posQ_B; // position of folded modes 0 and q in B's tensor map
            int     mapPosB[kMaxGroup]; // folded mode -> position in B's tensor map
            int64_t ext[kMaxGroup];
            float   alpha;
            int     opA, opB;
            int     tilesP, tilesQ;
            int*    status;
        };

        __device__ __forceinline__ uint32_t smemAddr(const void* p)
        {
            return uint32_t(__cvta_generic_to_shared(p));
        }

        template <int NP, int NQ>
        __global__ void __launch_bounds__(64 * NP * NQ)
            perm_tma_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                            PermTmaArgs a)
        {
            constexpr int TP = 32 * NP, TQ = 32 * NQ;
            extern __shared__ unsigned char smemRaw[];
            // 1024-byte alignment for the 128B swizzle pattern
            unsigned char* base = (unsigned char*)((uintptr_t(smemRaw) + 1023) & ~uintptr_t(1023));
            float*         in   = (float*)base; // NP boxes * TQ rows * 32 floats
            float*         outb = in + NP * TQ * 32; // NQ boxes * TP rows * 32 floats
            __shared__ __align__(8) unsigned long long bar;

            int64_t   bid = blockIdx.x;
            const int tp  = int(bid % a.tilesP);
            bid /= a.tilesP;
            const int tq = int(bid % a.tilesQ);
            bid /= a.tilesQ;
            int coordA[5] = {0, 0, 0, 0, 0};
            int coordB[5] = {0, 0, 0, 0, 0};
            for(int d = 1; d < a.ndim; d++)
            {
                if(d == a.q)
                    continue;
                int c = int(bid % a.ext[d]);
                bid /= a.ext[d];
                coordA[d]            = c;
                coordB[a.mapPosB[d]] = c;
            }
            const int p0 = tp * TP, q0 = tq * TQ;

            const uint32_t barAddr = smemAddr(&bar);
            if(threadIdx.x == 0)
            {
                asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(barAddr));
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            __syncthreads();
            if(threadIdx.x == 0)
            {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(barAddr),
                             "r"(uint32_t(NP * TQ * 128))
                             : "memory");
#pragma unroll
                for(int i = 0; i < NP; i++)
                {
                    coordA[0]   = p0 + 32 * i;
                    coordA[a.q] = q0;
                    const uint32_t dst = smemAddr(in + i * TQ * 32);
                    if(a.ndim == 2)
                        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
                                     "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                                     "l"(&mapA), "r"(barAddr), "r"(coordA[0]), "r"(coordA[1])
                                     : "memory");
                    else if(a.ndim == 3)
                        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
                                     "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
                                     "l"(&mapA), "r"(barAddr), "r"(coordA[0]), "r"(coordA[1]), "r"(coordA[2])
                                     : "memory");
                    else if(a.ndim == 4)
                        asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
                                     "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
                                     "l"(&mapA), "r"(barAddr), "r"(coordA[0]), "r"(coordA[1]), "r"(coordA[2]),
                                     "r"(coordA[3])
                                     : "memory");
                    else
                        asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes "
                                     "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
                                     "l"(&mapA), "r"(barAddr), "r"(coordA[0]), "r"(coordA[1]), "r"(coordA[2]),
                                     "r"(coordA[3]), "r"(coordA[4])
                                     : "memory");
                }
            }
            // bounded wait for the boxes to land
            {
                uint32_t done = 0;
                for(int spin = 0; spin < (1 << 22) && !done; spin++)
                {
                    asm volatile("{\n\t.reg .pred p;\n\t"
                                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                                 "selp.u32 %0, 1, 0, p;\n\t}"
                                 : "=r"(done)
                                 : "r"(barAddr), "r"(0u)
                                 : "memory");
                }
                if(!done)
                {
                    if(a.status)
                        atomicExch(a.status, 1);
                    return; // no store is issued; the loads complete on their own
                }
            }

            // 4x4 register transpose; 64 threads per 32x32 sub-tile
            const int t   = threadIdx.x;
            const int sub = t >> 6; // sub-tile index: pi = sub % NP, qj = sub / NP
            const int pi = sub % NP, qj = sub / NP;
            const int e = t & 7, kk = (t >> 3) & 7;
            const int c = e, g = (e + kk) & 7;
            float4    v[4];
            const unsigned char* inBox = (const unsigned char*)(in + pi * TQ * 32);
#pragma unroll
            for(int i = 0; i < 4; i++)
            {
                const int r = 32 * qj + 4 * g + i;
                v[i]        = *(const float4*)(inBox + r * 128 + ((c ^ (r & 7)) << 4));
            }
            unsigned char* outBox = (unsigned char*)(outb + qj * TP * 32);
#pragma unroll
            for(int j = 0; j < 4; j++)
            {
                float4 w;
                w.x = Elem<float>::apply(((const float*)&v[0])[j], a.alpha, a.opA, a.opB);
                w.y = Elem<float>::apply(((const float*)&v[1])[j], a.alpha, a.opA, a.opB);
                w.z = Elem<float>::apply(((const float*)&v[2])[j], a.alpha, a.opA, a.opB);
                w.w = Elem<float>::apply(((const float*)&v[3])[j], a.alpha, a.opA, a.opB);
                const int rr = 32 * pi + 4 * c + j;
                *(float4*)(outBox + rr * 128 + ((g ^ (rr & 7)) << 4)) = w;
            }
            // make the generic-proxy writes visible to the async proxy, then store
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            if(threadIdx.x == 0)
            {
#pragma unroll
                for(int j = 0; j < NQ; j++)
                {
                    coordB[a.posQ_B] = q0 + 32 * j;
                    coordB[a.posP_B] = p0;
                    const uint32_t src = smemAddr(outb + j * TP * 32);
                    if(a.ndim == 2)
                        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                                         &mapB),
                                     "r"(src), "r"(coordB[0]), "r"(coordB[1])
                                     : "memory");
                    else if(a.ndim == 3)
                        asm volatile(
                            "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                                &mapB),
                            "r"(src), "r"(coordB[0]), "r"(coordB[1]), "r"(coordB[2])
                            : "memory");
                    else if(a.ndim == 4)
                        asm volatile(
                            "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                                &mapB),
                            "r"(src), "r"(coordB[0]), "r"(coordB[1]), "r"(coordB[2]), "r"(coordB[3])
                            : "memory");
                    else
                        asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, "
                                     "%6}], [%1];" ::"l"(&mapB),
                                     "r"(src), "r"(coordB[0]), "r"(coordB[1]), "r"(coordB[2]), "r"(coordB[3]),
                                     "r"(coordB[4])
                                     : "memory");
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                // shared memory must stay valid until the stores have read it
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            }
        }

        template <int NP, int NQ>
        cudaError_t launchTma(const PermPlan& p, const void* A, void* B, float alpha, int opA, int opB,
                              int* status, cudaStream_t stream)
        {
            constexpr int TP = 32 * NP, TQ = 32 * NQ;
            PFN_encodeTiled encode = tensorMapEncoder();
            if(!encode)
                return cudaErrorNotSupported;
            CUtensorMap mapA, mapB;
            cuuint64_t  gdim[5], gstr[4];
            cuuint32_t  box[5], estr[5] = {1, 1, 1, 1, 1};
            // A: folded modes in A's order
            for(int d = 0; d < p.ndim; d++)
            {
                gdim[d] = cuuint64_t(p.ext[d]);
                box[d]  = 1;
                if(d > 0)
                    gstr[d - 1] = cuuint64_t(p.sA[d]) * 4;
            }
            box[0]   = 32;
            box[p.q] = TQ;
            if(encode(&mapA, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.ndim, const_cast<void*>(A), gdim, gstr, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               != CUDA_SUCCESS)
                return cudaErrorInvalidValue;
            // B: folded modes by ascending stride in B
            PermTmaArgs a{};
            for(int i = 0; i < p.ndim; i++)
            {
                const int d  = p.orderB[i];
                gdim[i]      = cuuint64_t(p.ext[d]);
                box[i]       = 1;
                a.mapPosB[d] = i;
                if(i > 0)
                    gstr[i - 1] = cuuint64_t(p.sB[d]) * 4;
            }
            a.posP_B     = a.mapPosB[0];
            a.posQ_B     = a.mapPosB[p.q];
            box[a.posQ_B] = 32;
            box[a.posP_B] = TP;
            if(encode(&mapB, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.ndim, B, gdim, gstr, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               != CUDA_SUCCESS)
                return cudaErrorInvalidValue;
            a.ndim = p.ndim;
            a.q    = p.q;
            for(int d = 0; d < p.ndim; d++)
                a.ext[d] = p.ext[d];
            a.alpha  = alpha;
            a.opA    = opA;
            a.opB    = opB;
            a.tilesP = int((p.ext[0] + TP - 1) / TP);
            a.tilesQ = int((p.ext[p.q] + TQ - 1) / TQ);
            a.status = status;
            int64_t blocks = int64_t(a.tilesP) * a.tilesQ;
            for(int d = 1; d < p.ndim; d++)
                if(d != p.q)
                    blocks *= p.ext[d];
            if(blocks > 0x7fffffffll)
                return cudaErrorInvalidConfiguration;
            const int   smem = 2 * TP * TQ * 4 + 1024;
            static bool attrSet = false;
            if(!attrSet)
            {
                cudaFuncSetAttribute(perm_tma_kernel<NP, NQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
                attrSet = true;
            }
            perm_tma_kernel<NP, NQ><<<unsigned(blocks), 64 * NP * NQ, smem, stream>>>(mapA, mapB, a);
            return cudaGetLastError();
        }

        template <typename TI, typename TO>
        cudaError_t launchPlain(const PermPlan& p, const void* A, void* B, float alpha, int opA, int opB,
                                cudaStream_t stream)
        {
            PermArgs a{};
            a.ndim = p.ndim;
            a.q    = p.q;
            for(int d = 0; d < p.ndim; d++)
            {
                a.ext[d] = p.ext[d];
                a.sA[d]  = p.sA[d];
                a.sB[d]  = p.sB[d];
            }
            a.alpha = alpha;
            a.opA   = opA;
            a.opB   = opB;
            if(p.kind == PERM_COPY)
            {
                int tx = 32;
                while(tx < 256 && tx < p.ext[0])
                    tx <<= 1;
                const int     ty   = 256 / tx;
                const int64_t rows = p.total / p.ext[0];
                const int64_t grid = (rows + ty - 1) / ty;
                if(grid > 0x7fffffffll)
                    return cudaErrorInvalidConfiguration;
                perm_copy_kernel<TI, TO>
                    <<<unsigned(grid), dim3(tx, ty), 0, stream>>>((const TI*)A, (TO*)B, a, rows);
                noteLaunch("perm_copy");
            }
            else
            {
                const int tilesP = int((p.ext[0] + kTile - 1) / kTile);
                const int tilesQ = int((p.ext[p.q] + kTile - 1) / kTile);
                int64_t   blocks = int64_t(tilesP) * tilesQ;
                for(int d = 1; d < p.ndim; d++)
                    if(d != p.q)
                        blocks *= p.ext[d];
                if(blocks > 0x7fffffffll)
                    return cudaErrorInvalidConfiguration;
                perm_tile_kernel<TI, TO><<<unsigned(blocks), 256, 0, stream>>>((const TI*)A, (TO*)B, a, tilesP, tilesQ);
                noteLaunch("perm_tile");
            }
            return cudaGetLastError();
        }
    } // namespace

    cudaError_t launchPermutation(const PermPlan& plan, int typeA, int typeB, const void* A, void* B, float alpha,
                                  int opA, int opB, int* deviceStatus, cudaStream_t stream)
    {
        if(plan.total == 0)
            return cudaSuccess;
        if(plan.kind == PERM_TMA)
        {
            cudaError_t e = launchTma<2, 2>(plan, A, B, alpha, opA, opB, deviceStatus, stream);
            if(e == cudaSuccess)
                noteLaunch("perm_tma");
            return e;
        }
        if(typeA == CUDA_R_32F)
            return launchPlain<float, float>(plan, A, B, alpha, opA, opB, stream);
        if(typeB == CUDA_R_16F)
            return launchPlain<__half, __half>(plan, A, B, alpha, opA, opB, stream);
        return launchPlain<__half, float>(plan, A, B, alpha, opA, opB, stream);
    }
} // namespace htb
