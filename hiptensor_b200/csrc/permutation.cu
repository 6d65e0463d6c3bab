// Permutation kernels for sm_100a: B[perm(i)] = opB(alpha * opA(A[i])).
//
// Kernels, chosen by the planner (planner.hpp PermKind) and, within PERM_TILE, by alignment:
//   perm_copy_kernel : A's and B's fastest folded modes coincide; coalesced row copy.
//   perm_tile_kernel : 64x64 tile through padded shared memory, plain loads/stores; any extents, f32 and
//                      f16; 2x2 register blocks when everything is even, else element by element.
//   perm_tile4_half_kernel : f16 with extents and strides that are multiples of 4: 128x128 tiles, 4x4 blocks.
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

#include <algorithm>
#include <cstdlib>

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
        // A's and B's contiguous folded mode coincide (mode 0): rows of ext[0] elements move
        // unchanged, only the outer modes are permuted. A block copies a tile of T0 elements of
        // mode 0 by T1 rows of mode 1 with 16-byte accesses (VEC elements) and four independent
        // accesses per thread; the outer modes are decomposed once per block.
        template <typename T, int N>
        struct alignas(sizeof(T) * N) VecT
        {
            T v[N];
        };

        template <typename TI, typename TO, int VEC>
        __global__ void __launch_bounds__(256)
            perm_copy_kernel(const TI* __restrict__ A, TO* __restrict__ B, PermArgs a, int chunks0Log2, int tiles0,
                             int tiles1, int64_t flatTotal)
        {
            const int chunks0 = 1 << chunks0Log2; // 16-byte chunks of mode 0 per tile
            const int T1      = 1024 >> chunks0Log2; // rows of mode 1 per tile
            // (32-bit divisions: the grid, and with it every extent met here, is below 2^31)
            uint32_t  bid     = blockIdx.x;
            const int t0      = int(bid % uint32_t(tiles0));
            bid /= uint32_t(tiles0);
            const int t1 = int(bid % uint32_t(tiles1));
            bid /= uint32_t(tiles1);
            int64_t offA = 0, offB = 0;
            for(int d = 2; d < a.ndim; d++)
            {
                const uint32_t e = uint32_t(a.ext[d]), c = bid % e;
                bid /= e;
                offA += int64_t(c) * a.sA[d];
                offB += int64_t(c) * a.sB[d];
            }
            const int64_t ext1 = (a.ndim > 1) ? a.ext[1] : 1;
            const int64_t sA1 = (a.ndim > 1) ? a.sA[1] : 0, sB1 = (a.ndim > 1) ? a.sB[1] : 0;
            VecT<TI, VEC> v[4];
            bool          ok[4];
#pragma unroll
            for(int k = 0; k < 4; k++)
            {
                const int     item = threadIdx.x + 256 * k;
                const int64_t i0   = (int64_t(t0) * chunks0 + (item & (chunks0 - 1))) * VEC;
                const int64_t i1   = int64_t(t1) * T1 + (item >> chunks0Log2);
                ok[k]              = (i0 < a.ext[0]) && (i1 < ext1) && (flatTotal == 0 || i1 * sA1 + i0 < flatTotal);
                if(ok[k])
                    v[k] = *(const VecT<TI, VEC>*)(A + offA + i1 * sA1 + i0);
            }
#pragma unroll
            for(int k = 0; k < 4; k++)
            {
                const int     item = threadIdx.x + 256 * k;
                const int64_t i0   = (int64_t(t0) * chunks0 + (item & (chunks0 - 1))) * VEC;
                const int64_t i1   = int64_t(t1) * T1 + (item >> chunks0Log2);
                if(ok[k])
                {
                    VecT<TO, VEC> w;
#pragma unroll
                    for(int e = 0; e < VEC; e++)
                        w.v[e] = convertOut<TO, TI>(Elem<TI>::apply(v[k].v[e], a.alpha, a.opA, a.opB));
                    *(VecT<TO, VEC>*)(B + offB + i1 * sB1 + i0) = w;
                }
            }
        }

        // ------------------------------------------------------------ padded-tile kernel
        // 64 x 64 tile of the (p, q) plane through shared memory: p is A's contiguous folded mode, q is B's.
        // PACK = 2 (every extent, stride and base address even): a thread moves 2 x 2 blocks - two 2-element
        // loads along p from rows q and q+1, a register transpose, two 2-element shared stores along q - so global
        // and shared accesses are 4 bytes (f16) or 8 bytes (f32) wide. PACK = 1: element by element, any extents.
        // Tiles that lie inside the tensor take a path without bounds checks; row pointers advance by addition.
        constexpr int kTile = 64;

        template <typename T>
        struct Pair;
        template <>
        struct Pair<float>
        {
            using type = float2;
            static __device__ __forceinline__ void transpose(float2 a, float2 b, float2& o0, float2& o1)
            {
                o0 = make_float2(a.x, b.x);
                o1 = make_float2(a.y, b.y);
            }
        };
        template <>
        struct Pair<__half>
        {
            using type = uint32_t;
            static __device__ __forceinline__ void transpose(uint32_t a, uint32_t b, uint32_t& o0, uint32_t& o1)
            {
                o0 = __byte_perm(a, b, 0x5410);
                o1 = __byte_perm(a, b, 0x7632);
            }
        };

        template <typename TI, typename TO>
        __device__ __forceinline__ void storePair(TO* dst, typename Pair<TI>::type v, float alpha, int opA, int opB)
        {
            if constexpr(sizeof(TI) == 4)
            {
                float2 o;
                o.x = Elem<float>::apply(v.x, alpha, opA, opB);
                o.y = Elem<float>::apply(v.y, alpha, opA, opB);
                *reinterpret_cast<float2*>(dst) = o;
            }
            else
            {
                // both halves at once: the paired multiply rounds each lane like the scalar one
                __half2 h = *reinterpret_cast<const __half2*>(&v);
                if(opA == 2)
                    h = __hmul2(h, h);
                h = __hmul2(__float2half2_rn(alpha), h);
                if(opB == 2)
                    h = __hmul2(h, h);
                if constexpr(sizeof(TO) == 2)
                    *reinterpret_cast<__half2*>(dst) = h;
                else
                    *reinterpret_cast<float2*>(dst) = __half22float2(h);
            }
        }

        // PLAIN (PACK = 1 only): alpha is 1 and both element operators are the identity, elements move unchanged.
        template <typename TI, typename TO, int PACK, bool PLAIN = false>
        __global__ void __launch_bounds__(256)
            perm_tile_kernel(const TI* __restrict__ A, TO* __restrict__ B, PermArgs a, int tilesP, int tilesQ)
        {
            // the grid is below 2^31 blocks, so every extent met here fits 32 bits: 32-bit divisions (the 64-bit ones
            // of this decoding cost as many instructions as moving a thread's sixteen elements)
            uint32_t  bid = blockIdx.x;
            const int tp  = int(bid % uint32_t(tilesP));
            bid /= uint32_t(tilesP);
            const int tq = int(bid % uint32_t(tilesQ));
            bid /= uint32_t(tilesQ);
            int64_t offA = 0, offB = 0;
            for(int d = 1; d < a.ndim; d++)
            {
                if(d == a.q)
                    continue;
                const uint32_t e = uint32_t(a.ext[d]), c = bid % e;
                bid /= e;
                offA += int64_t(c) * a.sA[d];
                offB += int64_t(c) * a.sB[d];
            }
            const int64_t p0 = int64_t(tp) * kTile, q0 = int64_t(tq) * kTile;
            const int64_t sAq = a.sA[a.q], sBp = a.sB[0];
            const bool    inside = p0 + kTile <= a.ext[0] && q0 + kTile <= a.ext[a.q];
            if constexpr(PACK == 2)
            {
                using P2 = typename Pair<TI>::type;
                // transposed tile: row = p, 64 elements of q; the pitch of 33 pairs keeps the column-wise stores
                // of a warp (rows 2l) on 16 different 8-byte banks twice over
                __shared__ P2 tile[kTile][kTile / 2 + 1];
                const int lx = threadIdx.x & 31, ly = threadIdx.x >> 5;
                {
                    // lanes along p: pair lx of the row; rows q0 + 2*(ly + 8j) and the next
                    const TI* src = A + offA + p0 + 2 * lx + (q0 + 2 * ly) * sAq;
                    const bool pok = inside || p0 + 2 * lx < a.ext[0];
#pragma unroll
                    for(int j = 0; j < 4; j++)
                    {
                        const int ql = 2 * (ly + 8 * j);
                        if(pok && (inside || q0 + ql < a.ext[a.q]))
                        {
                            const P2 r0 = *reinterpret_cast<const P2*>(src);
                            const P2 r1 = *reinterpret_cast<const P2*>(src + sAq);
                            P2       o0, o1;
                            Pair<TI>::transpose(r0, r1, o0, o1);
                            tile[2 * lx][ql >> 1]     = o0;
                            tile[2 * lx + 1][ql >> 1] = o1;
                        }
                        src += 16 * sAq;
                    }
                }
                __syncthreads();
                {
                    // lanes along q: pair lx of the output row; rows p0 + ly + 8j
                    TO*        dst = B + offB + q0 + 2 * lx + (p0 + ly) * sBp;
                    const bool qok = inside || q0 + 2 * lx < a.ext[a.q];
#pragma unroll
                    for(int j = 0; j < 8; j++)
                    {
                        const int pl = ly + 8 * j;
                        if(qok && (inside || p0 + pl < a.ext[0]))
                            storePair<TI, TO>(dst, tile[pl][lx], a.alpha, a.opA, a.opB);
                        dst += 8 * sBp;
                    }
                }
            }
            else
            {
                // Element by element. The kernel was bound by instruction issue, not by memory (3.6 TB/s with the issue
                // slots 85 % busy), so the loops of tiles inside the tensor carry no bounds checks, the extents, the
                // scale and the operators are read once, and PLAIN tensors skip the arithmetic.
                __shared__ TI tile[kTile][kTile + 1];
                const int     tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
                const int64_t ext0 = a.ext[0], extQ = a.ext[a.q];
                const float   alpha = a.alpha;
                const int     opA = a.opA, opB = a.opB;
                {
                    // load: lanes run along p (contiguous in A)
                    const TI*     src  = A + offA + p0 + tx + (q0 + ty) * sAq;
                    const int64_t step = 4 * sAq;
                    if(inside)
                    {
#pragma unroll
                        for(int j = 0; j < kTile / 4; j++)
                        {
                            tile[ty + 4 * j][tx] = *src;
                            src += step;
                        }
                    }
                    else if(p0 + tx < ext0)
                    {
                        const int rows = int(min(int64_t(kTile), extQ - q0));
#pragma unroll 4
                        for(int ql = ty; ql < rows; ql += 4)
                        {
                            tile[ql][tx] = *src;
                            src += step;
                        }
                    }
                }
                __syncthreads();
                {
                    // store: lanes run along q (contiguous in B)
                    TO*           dst  = B + offB + q0 + tx + (p0 + ty) * sBp;
                    const int64_t step = 4 * sBp;
                    auto          out  = [&](TI v) -> TO {
                        if constexpr(PLAIN)
                            return convertOut<TO, TI>(v);
                        else
                            return convertOut<TO, TI>(Elem<TI>::apply(v, alpha, opA, opB));
                    };
                    if(inside)
                    {
#pragma unroll
                        for(int j = 0; j < kTile / 4; j++)
                        {
                            *dst = out(tile[tx][ty + 4 * j]);
                            dst += step;
                        }
                    }
                    else if(q0 + tx < extQ)
                    {
                        const int rows = int(min(int64_t(kTile), ext0 - p0));
#pragma unroll 4
                        for(int pl = ty; pl < rows; pl += 4)
                        {
                            *dst = out(tile[tx][pl]);
                            dst += step;
                        }
                    }
                }
            }
        }

        // ------------------------------------------------------------ box kernel for short contiguous modes
        // When A's or B's contiguous folded mode is shorter than a tile side, a (p, q) tile is mostly empty (a store
        // instruction of the tile kernel wrote 2 of 64 lanes for an extent of 2: 0.16 TB/s). The box kernel
        // moves a box over SEVERAL modes instead: the leading modes of A until their tile extents multiply to 64 (a
        // contiguous run of A), the leading modes of B likewise (a contiguous run of B), every tile extent a power
        // of two. A block reads its box in A's order (consecutive threads along A's run) into shared memory and
        // writes it in B's order (consecutive threads along B's run); the coordinates of an element follow from its
        // index in the box by shifts.
        constexpr int kBoxMaxDims = 6;
        constexpr int kBoxBits    = 13; // a box holds at most 8192 elements
        constexpr int kBoxRounds  = 1 << (kBoxBits - 8); // elements per thread of a block of 256
        struct PermBoxArgs
        {
            int      nb; // modes of the box
            int      no; // other modes (walked by the grid)
            // box modes in A's order (ascending stride in A): log2 of the tile extent, extent, strides
            int      lgA[kBoxMaxDims];
            uint32_t extA[kBoxMaxDims];
            int64_t  sAofA[kBoxMaxDims], sBofA[kBoxMaxDims];
            uint32_t tilesOf[kBoxMaxDims]; // tiles along each box mode (A's order)
            uint32_t extO[kBoxMaxDims];
            int64_t  sAO[kBoxMaxDims], sBO[kBoxMaxDims];
            int      lgBox; // log2 of the box size
            // Every tile extent is a power of two, so an element's offsets are sums over the BITS of its index in
            // the box: bit k of the index in A's order adds wA[k] to the offset in A; bit k of the index in B's order
            // adds wB[k] to the offset in B, slotB[k] to the index in A's order (where the element lies in shared
            // memory) and belongs to box mode dimB[k] with value valB[k] there (for the bounds of an edge box).
            int64_t  wA[kBoxBits], wB[kBoxBits];
            uint32_t slotB[kBoxBits];
            // the same sums for every value of the index bits above the low eight (a thread's elements differ in those)
            int64_t  hiA[kBoxRounds], hiB[kBoxRounds];
            uint32_t hiS[kBoxRounds];
            // pairs kernel only: position (A's order) of the lowest index bit of B's contiguous mode, and its weight in A
            // in 4-byte words
            int      betaBit;
            int64_t  betaW;
            float    alpha;
            int      opA, opB;
        };

        // slot of box element i in shared memory: the low five bits are mixed with the bits above them, so that the
        // strided reads of the write phase (strides of 32, 64, .. 4096 elements) spread over the banks
        __device__ __forceinline__ uint32_t boxSlot(uint32_t i)
        {
            return i ^ (((i >> 5) ^ (i >> 10)) & 31u);
        }

        // A unit of the box kernel: PACK neighbouring elements of the contiguous mode moved as one word of 2 to 16 bytes
        // (PACK > 1 only when that mode is the contiguous one of A and of B).
        template <int BYTES>
        struct BoxWord;
        template <>
        struct BoxWord<2>
        {
            using type = unsigned short;
        };
        template <>
        struct BoxWord<4>
        {
            using type = uint32_t;
        };
        template <>
        struct BoxWord<8>
        {
            using type = uint2;
        };
        template <>
        struct BoxWord<16>
        {
            using type = uint4;
        };

        template <typename TI, typename TO, int PACK, bool PLAIN>
        __global__ void __launch_bounds__(256, 5) perm_box_kernel(const void* __restrict__ Av, void* __restrict__ Bv, PermBoxArgs a)
        {
            using UI = typename BoxWord<sizeof(TI) * PACK>::type;
            using UO = typename BoxWord<sizeof(TO) * PACK>::type;
            const UI* A = reinterpret_cast<const UI*>(Av);
            UO*       B = reinterpret_cast<UO*>(Bv);
            extern __shared__ __align__(16) unsigned char boxRaw[];
            UI*      box = reinterpret_cast<UI*>(boxRaw);
            // origin of the box and offsets of the other modes (32-bit divisions: the grid is below 2^31 blocks)
            uint32_t bid = blockIdx.x;
            uint32_t org[kBoxMaxDims];
            int64_t  offA = 0, offB = 0;
            uint32_t cut = 0; // box modes that the tensor's edge cuts in this block
#pragma unroll
            for(int d = 0; d < kBoxMaxDims; d++)
            {
                org[d] = 0;
                if(d < a.nb)
                {
                    const uint32_t t = bid % a.tilesOf[d];
                    bid /= a.tilesOf[d];
                    org[d] = t << a.lgA[d];
                    offA += int64_t(org[d]) * a.sAofA[d];
                    offB += int64_t(org[d]) * a.sBofA[d];
                    if(org[d] + (1u << a.lgA[d]) > a.extA[d])
                        cut |= 1u << d;
                }
            }
            const bool inside = cut == 0;
            for(int d = 0; d < a.no; d++)
            {
                const uint32_t c = bid % a.extO[d];
                bid /= a.extO[d];
                offA += int64_t(c) * a.sAO[d];
                offB += int64_t(c) * a.sBO[d];
            }
            const uint32_t size = 1u << a.lgBox;
            // An element of an edge box lies in the tensor when its coordinate in every cut mode does (index i in A's
            // order). A cut mode whose index bits all belong to the part of the index that a thread keeps through a phase
            // (fixed) is checked once per thread (ok); the others (rest) once per element. A short odd contiguous mode cuts
            // EVERY box, and its bits are fixed in both phases.
            // The first two of the others are kept as (shift, mask, room left above the thread's share of the coordinate):
            // the share of an element's other index bits is the same for every thread, which leaves a shift, a mask and a
            // compare per element and mode.
            uint32_t sh0 = 0, m0 = 0, room0 = 1, sh1 = 0, m1 = 0, room1 = 1;
            int      restN = 0;
            auto     splitChecks = [&](uint32_t fixed, uint32_t part, bool& ok, uint32_t& rest) {
                ok     = true;
                rest   = 0;
                restN  = 0;
                sh0 = sh1 = m0 = m1 = 0;
                room0 = room1 = 1;
                int sh = 0;
#pragma unroll
                for(int d = 0; d < kBoxMaxDims; d++)
                    if(d < a.nb)
                    {
                        const uint32_t m = (1u << a.lgA[d]) - 1u;
                        if((cut >> d) & 1u)
                        {
                            if(((m << sh) & ~fixed) == 0)
                                ok = ok && org[d] + ((part >> sh) & m) < a.extA[d];
                            else if(restN < 2)
                            {
                                // what the element's other bits may add to the thread's share of the coordinate
                                const uint32_t mine = (part >> sh) & m, lim = a.extA[d] - org[d];
                                ok = ok && mine < lim;
                                if(restN == 0)
                                {
                                    sh0   = uint32_t(sh);
                                    m0    = m;
                                    room0 = lim - mine;
                                }
                                else
                                {
                                    sh1   = uint32_t(sh);
                                    m1    = m;
                                    room1 = lim - mine;
                                }
                                restN++;
                            }
                            else
                                rest |= 1u << d;
                        }
                        sh += a.lgA[d];
                    }
            };
            // others: the index bits of the element that the thread does not fix (disjoint from the thread's)
            auto restOk = [&](uint32_t others) {
                // (with no such mode the masks are zero and the rooms one)
                return ((others >> sh0) & m0) < room0 && ((others >> sh1) & m1) < room1;
            };
            auto valid = [&](uint32_t i, uint32_t rest) {
                if(rest == 0)
                    return true;
                bool ok = true;
                int  sh = 0;
#pragma unroll
                for(int d = 0; d < kBoxMaxDims; d++)
                    if(d < a.nb)
                    {
                        if((rest >> d) & 1u)
                            ok = ok && org[d] + ((i >> sh) & ((1u << a.lgA[d]) - 1u)) < a.extA[d];
                        sh += a.lgA[d];
                    }
                return ok;
            };
            // A thread's elements share the low eight bits of their index (blockDim.x = 256): that part of the offsets
            // is summed once per thread; the part of the bits above comes from the launch arguments (constant memory:
            // no load instruction competes with the element moves).
            const uint32_t t = threadIdx.x;
            int64_t  lowA = offA, lowB = offB;
            uint32_t lowI = 0, fixedB = 0;
#pragma unroll
            for(int k = 0; k < 8; k++)
            {
                fixedB |= a.slotB[k];
                if((t >> k) & 1u)
                {
                    lowA += a.wA[k];
                    lowB += a.wB[k];
                    lowI += a.slotB[k];
                }
            }
            const uint32_t rounds = max(size >> 8, 1u);
            const bool     mine   = t < size; // boxes of fewer than 256 elements
            const UI*      src    = A + lowA;
            if(inside)
            {
                // eight loads in flight per thread: with elements of two or four bytes the bytes in flight bound the rate
#pragma unroll
                for(uint32_t k0 = 0; k0 < kBoxRounds; k0 += 8)
                    if(k0 < rounds)
                    {
                        UI v[8];
#pragma unroll
                        for(uint32_t j = 0; j < 8; j++)
                            if(mine && k0 + j < rounds)
                                v[j] = src[a.hiA[k0 + j]];
#pragma unroll
                        for(uint32_t j = 0; j < 8; j++)
                            if(mine && k0 + j < rounds)
                                box[boxSlot(t | ((k0 + j) << 8))] = v[j];
                    }
            }
            else
            {
                bool     ok;
                uint32_t rest;
                splitChecks(0xffu, t, ok, rest);
                ok = ok && mine;
                // (not unrolled over the batches: with the inside path the kernel would outgrow the instruction cache)
                if(rest == 0)
                {
#pragma unroll 1
                    for(uint32_t k0 = 0; k0 < rounds; k0 += 8)
                    {
                        // the table entry of k0 + j is the sum of those of k0 and j (disjoint bits): one indexed
                        // constant load per batch, the rest are immediate operands
                        const UI* base = src + a.hiA[k0];
                        UI        v[8];
                        bool      in[8];
#pragma unroll
                        for(uint32_t j = 0; j < 8; j++)
                        {
                            in[j] = ok && k0 + j < rounds && restOk((k0 + j) << 8);
                            if(in[j])
                                v[j] = base[a.hiA[j]];
                        }
#pragma unroll
                        for(uint32_t j = 0; j < 8; j++)
                            if(in[j])
                                box[boxSlot(t | ((k0 + j) << 8))] = v[j];
                    }
                }
                else
                {
#pragma unroll 1
                    for(uint32_t k = 0; k < rounds; k++)
                        if(ok && restOk(k << 8) && valid(t | (k << 8), rest))
                            box[boxSlot(t | (k << 8))] = src[a.hiA[k]];
                }
            }
            __syncthreads();
            UO*  dst = B + lowB;
            auto out = [&](UI u) -> UO {
                if constexpr(PLAIN && sizeof(TI) == sizeof(TO))
                    return u;
                else
                {
                    union
                    {
                        UI w;
                        TI e[PACK];
                    } in;
                    union
                    {
                        UO w;
                        TO e[PACK];
                    } res;
                    in.w = u;
#pragma unroll
                    for(int e = 0; e < PACK; e++)
                    {
                        if constexpr(PLAIN)
                            res.e[e] = convertOut<TO, TI>(in.e[e]);
                        else
                            res.e[e] = convertOut<TO, TI>(Elem<TI>::apply(in.e[e], a.alpha, a.opA, a.opB));
                    }
                    return res.w;
                }
            };
            if(inside)
            {
#pragma unroll
                for(uint32_t k0 = 0; k0 < kBoxRounds; k0 += 8)
                    if(k0 < rounds)
                    {
#pragma unroll
                        for(uint32_t j = 0; j < 8; j++)
                            if(mine && k0 + j < rounds)
                                dst[a.hiB[k0 + j]] = out(box[boxSlot(lowI + a.hiS[k0 + j])]);
                    }
            }
            else
            {
                bool     ok;
                uint32_t rest;
                splitChecks(fixedB, lowI, ok, rest);
                ok = ok && mine;
                if(rest == 0)
                {
#pragma unroll 1
                    for(uint32_t k0 = 0; k0 < rounds; k0 += 8)
                    {
                        UO*            base = dst + a.hiB[k0];
                        const uint32_t hs0  = a.hiS[k0];
#pragma unroll
                        for(uint32_t j = 0; j < 8; j++)
                        {
                            const uint32_t hs = hs0 + a.hiS[j];
                            if(ok && k0 + j < rounds && restOk(hs))
                                base[a.hiB[j]] = out(box[boxSlot(lowI + hs)]);
                        }
                    }
                }
                else
                {
#pragma unroll 1
                    for(uint32_t k = 0; k < rounds; k++)
                    {
                        const uint32_t i = lowI + a.hiS[k];
                        if(ok && restOk(a.hiS[k]) && valid(i, rest))
                            dst[a.hiB[k]] = out(box[boxSlot(i)]);
                    }
                }
            }
        }

        // ------------------------------------------------------------ 128 x 128 tile kernel for f16, 4 x 4 blocks
        // Every extent and stride involved is a multiple of 4 elements: a thread loads four rows of 8 bytes
        // (4 halves along p from rows q .. q+3), transposes the 4 x 4 block in registers (eight byte permutes) and
        // stores four 8-byte units along q into the transposed shared tile [128 p][32 units]. Units are swizzled
        // (unit ^ (p / 4)) so that both the column-wise stores and the row-wise loads of a half warp touch 16
        // different 8-byte banks. A warp moves 256 contiguous bytes per row on both sides.
        constexpr int kTile4 = 128;

        __device__ __forceinline__ void transpose4x4Half(const uint2 (&r)[4], uint2 (&o)[4])
        {
            // r[i] = row q+i: halves p0..p3 (x: p0 p1, y: p2 p3);  o[j] = row p+j: halves q0..q3
            o[0].x = __byte_perm(r[0].x, r[1].x, 0x5410);
            o[0].y = __byte_perm(r[2].x, r[3].x, 0x5410);
            o[1].x = __byte_perm(r[0].x, r[1].x, 0x7632);
            o[1].y = __byte_perm(r[2].x, r[3].x, 0x7632);
            o[2].x = __byte_perm(r[0].y, r[1].y, 0x5410);
            o[2].y = __byte_perm(r[2].y, r[3].y, 0x5410);
            o[3].x = __byte_perm(r[0].y, r[1].y, 0x7632);
            o[3].y = __byte_perm(r[2].y, r[3].y, 0x7632);
        }

        template <typename TO>
        __global__ void __launch_bounds__(256)
            perm_tile4_half_kernel(const __half* __restrict__ A, TO* __restrict__ B, PermArgs a, int tilesP, int tilesQ)
        {
            __shared__ uint2 tile[kTile4][32];
            uint32_t         bid = blockIdx.x; // 32-bit divisions, as in perm_tile_kernel
            const int        tp  = int(bid % uint32_t(tilesP));
            bid /= uint32_t(tilesP);
            const int tq = int(bid % uint32_t(tilesQ));
            bid /= uint32_t(tilesQ);
            int64_t offA = 0, offB = 0;
            for(int d = 1; d < a.ndim; d++)
            {
                if(d == a.q)
                    continue;
                const uint32_t e = uint32_t(a.ext[d]), c = bid % e;
                bid /= e;
                offA += int64_t(c) * a.sA[d];
                offB += int64_t(c) * a.sB[d];
            }
            const int64_t p0 = int64_t(tp) * kTile4, q0 = int64_t(tq) * kTile4;
            const int64_t sAq = a.sA[a.q], sBp = a.sB[0];
            const bool    inside = p0 + kTile4 <= a.ext[0] && q0 + kTile4 <= a.ext[a.q];
            const int     lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
            {
                // lanes along p: halves 4*lane .. 4*lane+3; the warp takes q blocks warp, warp+8, warp+16, warp+24
                const __half* src = A + offA + p0 + 4 * lane + (q0 + 4 * warp) * sAq;
                const bool    pok = inside || p0 + 4 * lane < a.ext[0];
#pragma unroll
                for(int j = 0; j < 4; j++)
                {
                    const int qb = warp + 8 * j;
                    if(pok && (inside || q0 + 4 * qb < a.ext[a.q]))
                    {
                        uint2 r[4], o[4];
#pragma unroll
                        for(int i = 0; i < 4; i++)
                            r[i] = *reinterpret_cast<const uint2*>(src + i * sAq);
                        transpose4x4Half(r, o);
#pragma unroll
                        for(int i = 0; i < 4; i++)
                            tile[4 * lane + i][qb ^ lane] = o[i];
                    }
                    src += 32 * sAq;
                }
            }
            __syncthreads();
            {
                // lanes along q: unit `lane` (halves 4*lane .. +3) of the output row; the warp takes rows warp + 8j
                TO*        dst = B + offB + q0 + 4 * lane + (p0 + warp) * sBp;
                const bool qok = inside || q0 + 4 * lane < a.ext[a.q];
                const __half2 alpha2 = __float2half2_rn(a.alpha);
#pragma unroll 4
                for(int j = 0; j < 16; j++)
                {
                    const int pl = warp + 8 * j;
                    if(qok && (inside || p0 + pl < a.ext[0]))
                    {
                        const uint2 v  = tile[pl][lane ^ ((pl >> 2) & 31)];
                        __half2     h0 = *reinterpret_cast<const __half2*>(&v.x), h1 = *reinterpret_cast<const __half2*>(&v.y);
                        if(a.opA == 2)
                        {
                            h0 = __hmul2(h0, h0);
                            h1 = __hmul2(h1, h1);
                        }
                        h0 = __hmul2(alpha2, h0);
                        h1 = __hmul2(alpha2, h1);
                        if(a.opB == 2)
                        {
                            h0 = __hmul2(h0, h0);
                            h1 = __hmul2(h1, h1);
                        }
                        if constexpr(sizeof(TO) == 2)
                        {
                            uint2 o;
                            o.x = *reinterpret_cast<const uint32_t*>(&h0);
                            o.y = *reinterpret_cast<const uint32_t*>(&h1);
                            *reinterpret_cast<uint2*>(dst) = o;
                        }
                        else
                        {
                            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
                            *reinterpret_cast<float4*>(dst) = make_float4(f0.x, f0.y, f1.x, f1.y);
                        }
                    }
                    dst += 8 * sBp;
                }
            }
        }

        // ------------------------------------------------------------ TMA kernel (f32)
        // Tile = (32*NP) x (32*NQ) elements of the (p, q) plane, p = A's fastest folded mode,
        // q = B's fastest folded mode. Input stage: NP boxes of [32*NQ rows of q][32 floats of p];
        // output stage: NQ boxes of [32*NP rows of p][32 floats of q]. Rows are 128 bytes, swizzled
        // by TMA (16-byte chunk index XOR row index mod 8), stages 1024-byte aligned.
        //
        // Persistent CTA: a producer warp keeps the input stages' tile loads in flight (full/empty
        // mbarriers per stage); 64*NP*NQ consumer threads transpose 4x4 blocks in registers and
        // hand finished tiles to TMA stores that drain asynchronously from kOutStages buffers.
        constexpr int kMaxInStages = 8, kOutStages = 2;

        struct PermTmaArgs
        {
            int       ndim, q;
            int       posP_B, posQ_B; // position of folded modes 0 and q in B's tensor map
            int       mapPosB[kMaxGroup]; // folded mode -> position in B's tensor map
            uint32_t  ext[kMaxGroup];
            float     alpha;
            int       opA, opB;
            uint32_t  tilesP, tilesQ;
            int       inStages; // input stages in flight per CTA
            int       wide; // 1: modes p and q are split 32 x (extent/32) in the tensor maps (see launchTma)
            // > 0: mode q stands for two modes of A that are adjacent in B (see launchTma): its first qInner elements
            // are A's map dimension q, the rest one more dimension at the end of A's map
            int       qInner;
            // the same for mode p (A's contiguous mode) and the mode that follows it in A: B's map has the extra dimension
            int       pInner;
            uint32_t  numTiles;
            int*      status;
        };

        __device__ __forceinline__ uint32_t smemAddr(const void* p)
        {
            return uint32_t(__cvta_generic_to_shared(p));
        }

        __device__ __forceinline__ bool mbarWaitBounded(uint32_t bar, uint32_t parity, volatile int* abortFlag)
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
                if(clock64() - t0 > 4000000000ll)
                {
                    *abortFlag = 1;
                    return false;
                }
            }
        }

        __device__ __forceinline__ void tmaLoadN(int ndim, uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 const int* c)
        {
            if(ndim == 2)
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
                             "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                             "l"(map), "r"(bar), "r"(c[0]), "r"(c[1])
                             : "memory");
            else if(ndim == 3)
                asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
                             "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
                             "l"(map), "r"(bar), "r"(c[0]), "r"(c[1]), "r"(c[2])
                             : "memory");
            else if(ndim == 4)
                asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes "
                             "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
                             "l"(map), "r"(bar), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3])
                             : "memory");
            else
                asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes "
                             "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
                             "l"(map), "r"(bar), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(c[4])
                             : "memory");
        }

        __device__ __forceinline__ void tmaStoreN(int ndim, const CUtensorMap* map, uint32_t src, const int* c)
        {
            if(ndim == 2)
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                             "r"(src), "r"(c[0]), "r"(c[1])
                             : "memory");
            else if(ndim == 3)
                asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
                             "r"(src), "r"(c[0]), "r"(c[1]), "r"(c[2])
                             : "memory");
            else if(ndim == 4)
                asm volatile(
                    "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(map),
                    "r"(src), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3])
                    : "memory");
            else
                asm volatile(
                    "cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];" ::"l"(map),
                    "r"(src), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(c[4])
                    : "memory");
        }

        // tile index -> TMA coordinates of the tile's origin in A's map and in B's map.
        // Narrow maps: one dimension per folded mode (A's order / ascending stride in B).
        // Wide maps: the contiguous mode of each tensor is split into (32, extent/32), which
        // shifts every other dimension up by one.
        __device__ __forceinline__ void permTileCoords(const PermTmaArgs& a, uint32_t tile, int NP, int NQ, int E, int* cA,
                                                       int* cB)
        {
            const int tp = int(tile % a.tilesP);
            tile /= a.tilesP;
            const int tq = int(tile % a.tilesQ);
            tile /= a.tilesQ;
            const int sh = a.wide ? 1 : 0;
            for(int d = 0; d < 5; d++)
            {
                cA[d] = 0;
                cB[d] = 0;
            }
            for(int d = 1; d < a.ndim; d++)
            {
                if(d == a.q)
                    continue;
                const int c = int(tile % a.ext[d]);
                tile /= a.ext[d];
                cA[d + sh]            = c;
                cB[a.mapPosB[d] + sh] = c;
            }
            if(a.qInner > 0 || a.pInner > 0)
            {
                // a tile's rows of a merged mode are whole runs of its inner mode: coordinate 0 there, the run index
                // in the extra dimension at the end of the other tensor's map
                if(a.wide)
                {
                    cA[1] = tp * NP;
                    cB[1] = tq * NQ;
                }
                else
                {
                    cA[0]        = tp * NP * E;
                    cB[a.posQ_B] = tq * NQ * E;
                }
                if(a.qInner > 0)
                {
                    cA[a.q + sh]    = 0;
                    cA[a.ndim + sh] = tq * (NQ * E / a.qInner);
                }
                else
                    cA[a.q + sh] = tq * NQ * E;
                if(a.pInner > 0)
                {
                    cB[a.posP_B + sh] = 0;
                    cB[a.ndim + sh]   = tp * (NP * E / a.pInner);
                }
                else
                    cB[a.posP_B + sh] = tp * NP * E;
            }
            else if(a.wide)
            {
                cA[1]            = tp * NP; // p: 128-byte group index
                cA[a.q + 1]      = tq * NQ * E; // q: rows of the input tile
                cB[1]            = tq * NQ; // q: 128-byte group index
                cB[a.posP_B + 1] = tp * NP * E; // p: rows of the output tile
            }
            else
            {
                cA[0]        = tp * NP * E;
                cA[a.q]      = tq * NQ * E;
                cB[a.posQ_B] = tq * NQ * E;
                cB[a.posP_B] = tp * NP * E;
            }
        }

        // ESZ: element size in bytes (4: fp32, 2: f16). A 128-byte row holds E = 128 / ESZ elements, a thread moves
        // VEC x VEC blocks (VEC = 16 / ESZ elements per 16-byte access), sub-tiles are E x E elements.
        template <int NP, int NQ, int ESZ>
        __global__ void __launch_bounds__(64 * NP * NQ + 32)
            perm_tma_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                            PermTmaArgs a)
        {
            constexpr int E = 128 / ESZ, VEC = 16 / ESZ;
            constexpr int TP = E * NP, TQ = E * NQ;
            constexpr int kConsumers = 64 * NP * NQ;
            constexpr int kStageFloats = TP * TQ * ESZ / 4; // stage size in 4-byte words
            extern __shared__ unsigned char smemRaw[];
            float* in   = (float*)((uintptr_t(smemRaw) + 1023) & ~uintptr_t(1023));
            float* outb = in + a.inStages * kStageFloats;
            __shared__ __align__(8) unsigned long long fullBar[kMaxInStages], emptyBar[kMaxInStages];
            __shared__ int abortFlag;
            __shared__ int coordB[kMaxInStages][5], coordOut[kOutStages][5];

            if(threadIdx.x == 32)
            {
                // start fetching the tensor maps (kernel parameters) before the first copy needs them
                asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mapA)) : "memory");
                asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&mapB)) : "memory");
            }
            if(threadIdx.x == 0)
            {
                abortFlag = 0;
                for(int s = 0; s < a.inStages; s++)
                {
                    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smemAddr(&fullBar[s])));
                    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(&emptyBar[s])),
                                 "r"(kConsumers / 32));
                }
                asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            }
            __syncthreads();
            volatile int* abortP = &abortFlag;

            if(threadIdx.x >= kConsumers)
            {
                // ---------------------------------------------------------------- producer warp
                if(threadIdx.x == kConsumers)
                {
                    int      stage = 0;
                    uint32_t phase = 0;
                    for(uint32_t tile = blockIdx.x; tile < a.numTiles; tile += gridDim.x)
                    {
                        int cA[5], cB[5];
                        permTileCoords(a, tile, NP, NQ, E, cA, cB);
                        if(!mbarWaitBounded(smemAddr(&emptyBar[stage]), phase ^ 1, abortP))
                            break;
                        // the storing thread reads the tile's B coordinates from shared memory
#pragma unroll
                        for(int d = 0; d < 5; d++)
                            coordB[stage][d] = cB[d];
                        const uint32_t bar = smemAddr(&fullBar[stage]);
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                                     "r"(uint32_t(kStageFloats * 4))
                                     : "memory");
                        if(a.wide)
                        {
                            // one box [32][NP][..][TQ]: the NP 128-byte pieces of a row arrive together
                            tmaLoadN(a.ndim + 1 + (a.qInner > 0 ? 1 : 0), smemAddr(in + stage * kStageFloats), &mapA, bar, cA);
                        }
                        else
                        {
                            const int p0 = cA[0];
#pragma unroll
                            for(int i = 0; i < NP; i++)
                            {
                                cA[0] = p0 + E * i;
                                tmaLoadN(a.ndim + (a.qInner > 0 ? 1 : 0), smemAddr(in + stage * kStageFloats + i * TQ * 32), &mapA, bar, cA);
                            }
                        }
                        if(++stage == a.inStages)
                        {
                            stage = 0;
                            phase ^= 1;
                        }
                    }
                }
                return;
            }

            // -------------------------------------------------------------------- consumers
            const int t   = threadIdx.x;
            const int sub = t >> 6; // sub-tile: pi = sub % NP, qj = sub / NP
            const int pi = sub % NP, qj = sub / NP;
            const int e = t & 7, kk = (t >> 3) & 7;
            const int c = e, g = (e + kk) & 7; // diagonal assignment: conflict free on both sides
            int      stage = 0, ostage = 0;
            uint32_t phase = 0;
            for(uint32_t tile = blockIdx.x; tile < a.numTiles; tile += gridDim.x)
            {
                // one lane per warp waits for the tile, the warp follows its verdict
                int ok = 1;
                if((t & 31) == 0)
                    ok = mbarWaitBounded(smemAddr(&fullBar[stage]), phase, abortP) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                // the output buffer about to be written must have been read by its last store
                if(t == 0)
                    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kOutStages - 1) : "memory");
                asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
                if(!ok || *abortP)
                    break;

                // the tile's B coordinates move to a slot of the output stage before this input
                // stage is handed back to the producer
                if(t == 0)
                {
#pragma unroll
                    for(int d = 0; d < 5; d++)
                        coordOut[ostage][d] = coordB[stage][d];
                }
                // row of (sub-tile pi, tile-local q index ql) in the input stage, and of
                // (sub-tile qj, tile-local p index pl) in the output stage
                uint4                v[VEC];
                const unsigned char* inStage = (const unsigned char*)(in + stage * kStageFloats);
#pragma unroll
                for(int i = 0; i < VEC; i++)
                {
                    const int ql = E * qj + VEC * g + i;
                    const int r  = a.wide ? (pi + NP * ql) : (pi * TQ + ql);
                    v[i]         = *(const uint4*)(inStage + r * 128 + ((c ^ (r & 7)) << 4));
                }
                // this warp is done with the input stage
                __syncwarp();
                if((t & 31) == 0)
                    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(&emptyBar[stage])) : "memory");

                unsigned char* outStage = (unsigned char*)(outb + ostage * kStageFloats);
                if constexpr(ESZ == 4)
                {
#pragma unroll
                    for(int j = 0; j < 4; j++)
                    {
                        float4 w;
                        w.x = Elem<float>::apply(__uint_as_float(((const uint32_t*)&v[0])[j]), a.alpha, a.opA, a.opB);
                        w.y = Elem<float>::apply(__uint_as_float(((const uint32_t*)&v[1])[j]), a.alpha, a.opA, a.opB);
                        w.z = Elem<float>::apply(__uint_as_float(((const uint32_t*)&v[2])[j]), a.alpha, a.opA, a.opB);
                        w.w = Elem<float>::apply(__uint_as_float(((const uint32_t*)&v[3])[j]), a.alpha, a.opA, a.opB);
                        const int pl = E * pi + VEC * c + j;
                        const int rr = a.wide ? (qj + NQ * pl) : (qj * TP + pl);
                        *(float4*)(outStage + rr * 128 + ((g ^ (rr & 7)) << 4)) = w;
                    }
                }
                else
                {
                    // 8 x 8 block of 16-bit elements: output row j takes element j of each of the eight input rows; one
                    // byte permute builds a word from the same half of the same word of two neighbouring rows
                    // (one loop per case, so that none carries a branch: plain move, scale only, scale and squares)
                    const __half2 alpha2 = __float2half2_rn(a.alpha);
                    auto          block  = [&](auto f) {
#pragma unroll
                        for(int j = 0; j < 8; j++)
                        {
                            uint32_t w[4];
#pragma unroll
                            for(int x = 0; x < 4; x++)
                            {
                                const uint32_t lo = ((const uint32_t*)&v[2 * x])[j >> 1], hi = ((const uint32_t*)&v[2 * x + 1])[j >> 1];
                                w[x] = f(__byte_perm(lo, hi, (j & 1) ? 0x7632 : 0x5410));
                            }
                            const int pl = E * pi + VEC * c + j;
                            const int rr = a.wide ? (qj + NQ * pl) : (qj * TP + pl);
                            *(uint4*)(outStage + rr * 128 + ((g ^ (rr & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    };
                    // both halves of a word at once: the paired multiply rounds each lane like the scalar one
                    if(a.opA == 2 || a.opB == 2)
                        block([&](uint32_t u) {
                            __half2 hh = *reinterpret_cast<__half2*>(&u);
                            if(a.opA == 2)
                                hh = __hmul2(hh, hh);
                            hh = __hmul2(alpha2, hh);
                            if(a.opB == 2)
                                hh = __hmul2(hh, hh);
                            return *reinterpret_cast<uint32_t*>(&hh);
                        });
                    else if(a.alpha != 1.0f)
                        block([&](uint32_t u) {
                            const __half2 hh = __hmul2(alpha2, *reinterpret_cast<__half2*>(&u));
                            return *reinterpret_cast<const uint32_t*>(&hh);
                        });
                    else
                        block([](uint32_t u) { return u; });
                }
                // generic-proxy writes -> async proxy, then one thread stores the tile
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
                if(t == 0)
                {
                    int cB[5];
#pragma unroll
                    for(int d = 0; d < 5; d++)
                        cB[d] = coordOut[ostage][d];
                    if(a.wide)
                    {
                        tmaStoreN(a.ndim + 1 + (a.pInner > 0 ? 1 : 0), &mapB, smemAddr(outb + ostage * kStageFloats), cB);
                    }
                    else
                    {
                        const int q0 = cB[a.posQ_B];
#pragma unroll
                        for(int j = 0; j < NQ; j++)
                        {
                            cB[a.posQ_B] = q0 + E * j;
                            tmaStoreN(a.ndim + (a.pInner > 0 ? 1 : 0), &mapB, smemAddr(outb + ostage * kStageFloats + j * TP * 32), cB);
                        }
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                if(++stage == a.inStages)
                {
                    stage = 0;
                    phase ^= 1;
                }
                if(++ostage == kOutStages)
                    ostage = 0;
            }
            if(t == 0)
            {
                // shared memory must stay valid until the stores have read it
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                if(abortFlag && a.status)
                    atomicExch(a.status, 1);
            }
        }

        // Launch-time choices of the TMA kernel. Measured on B200 over the rank-4 orders of a
        // 128^4 fp32 tensor: 64x64 tiles with TWO input stages and two CTAs per SM gave the highest
        // bandwidth on every order (deeper pipelines or more CTAs per SM lost 5-25%: more tiles in
        // flight mix more read and write streams in DRAM).
        struct PermTune
        {
            int shape     = 22; // NP*10 + NQ
            int inStages  = 2;
            int ctasPerSm = 2;
        };

        template <int NP, int NQ, int ESZ>
        cudaError_t launchTma(const PermPlan& plan, const void* A, void* B, float alpha, int opA, int opB,
                              const PermTune& tune, int smCount, int* status, cudaStream_t stream)
        {
            constexpr int E = 128 / ESZ, TP = E * NP, TQ = E * NQ;
            // Merged q. When B's contiguous mode q is shorter than a tile's TQ rows, a tile would be mostly empty
            // and B would be written in pieces of ext[q] elements (the slab of an output mode split over 8 GPUs:
            // 16 floats). If the next mode of B, q2, follows q without a gap, the two form one contiguous run in B:
            // the kernel then sees ONE mode of ext[q] * ext[q2] elements with stride 1 in B, and only A's tensor
            // map knows that it is two of A's modes (dimension q with box ext[q], and one more dimension at the
            // end of the map with box TQ / ext[q]: the rows of the shared tile then come in B's order).
            PermPlan p      = plan;
            int      qInner = 0;
            int64_t  q2Ext = 0, q2StrideA = 0;
            if(p.ndim >= 3 && p.ndim <= 4 && p.ext[p.q] < TQ && TQ % p.ext[p.q] == 0 && p.orderB[0] == p.q)
            {
                const int q2 = p.orderB[1];
                if(q2 != 0 && p.sB[q2] == p.ext[p.q])
                {
                    qInner    = int(p.ext[p.q]);
                    q2Ext     = p.ext[q2];
                    q2StrideA = p.sA[q2];
                    // drop q2 from the modes the kernel walks; q takes the merged extent
                    PermPlan m = p;
                    m.ndim     = 0;
                    int remap[kMaxGroup];
                    for(int d = 0; d < p.ndim; d++)
                    {
                        remap[d] = -1;
                        if(d == q2)
                            continue;
                        remap[d]     = m.ndim;
                        m.ext[m.ndim] = p.ext[d] * (d == p.q ? q2Ext : 1);
                        m.sA[m.ndim]  = p.sA[d];
                        m.sB[m.ndim]  = p.sB[d];
                        m.ndim++;
                    }
                    m.q = remap[p.q];
                    int n = 0;
                    for(int i = 0; i < p.ndim; i++)
                        if(p.orderB[i] != q2)
                            m.orderB[n++] = remap[p.orderB[i]];
                    p = m;
                }
            }
            // Merged p: the mirror image. A's contiguous mode p (folded mode 0) is shorter than a tile's TP rows and the
            // next mode of A follows it without a gap: the kernel sees one contiguous mode of A, and B's map carries
            // the two as dimension p (box ext[p]) and one more dimension at its end (box TP / ext[p]).
            int     pInner = 0;
            int64_t p2Ext = 0, p2StrideB = 0;
            if(p.ndim >= 3 && p.ndim <= 4 && p.ext[0] < TP && TP % p.ext[0] == 0 && p.q != 1 && p.sA[1] == p.ext[0])
            {
                pInner     = int(p.ext[0]);
                p2Ext      = p.ext[1];
                p2StrideB  = p.sB[1];
                PermPlan m = p;
                m.ndim     = 0;
                int remap[kMaxGroup];
                for(int d = 0; d < p.ndim; d++)
                {
                    remap[d] = -1;
                    if(d == 1)
                        continue;
                    remap[d]      = m.ndim;
                    m.ext[m.ndim] = p.ext[d] * (d == 0 ? p2Ext : 1);
                    m.sA[m.ndim]  = p.sA[d];
                    m.sB[m.ndim]  = p.sB[d];
                    m.ndim++;
                }
                m.q   = remap[p.q];
                int n = 0;
                for(int i = 0; i < p.ndim; i++)
                    if(p.orderB[i] != 1)
                        m.orderB[n++] = remap[p.orderB[i]];
                p = m;
            }
            constexpr CUtensorMapDataType kType = ESZ == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16;
            PFN_encodeTiled encode = tensorMapEncoder();
            if(!encode)
                return cudaErrorNotSupported;
            CUtensorMap mapA, mapB;
            cuuint64_t  gdim[5], gstr[4];
            cuuint32_t  box[5], estr[5] = {1, 1, 1, 1, 1};
            PermTmaArgs a{};
            // Wide maps: the contiguous mode is described as (32, extent/32) so that ONE box
            // [32][NP] covers NP consecutive 128-byte pieces of a row; the pieces of one row are
            // then requested back to back and DRAM serves them from one open page.
            const bool wide = (NP > 1 || NQ > 1) && p.ndim + ((qInner || pInner) ? 1 : 0) <= 4 && p.ext[0] % E == 0
                              && p.ext[p.q] % E == 0;
            a.wide          = wide ? 1 : 0;
            a.qInner        = qInner;
            a.pInner        = pInner;
            const int sh    = wide ? 1 : 0;
            // A: folded modes in A's order
            for(int d = 0; d < p.ndim; d++)
            {
                gdim[d + sh] = cuuint64_t(d == p.q && qInner ? qInner : p.ext[d]);
                box[d + sh]  = 1;
                if(d > 0)
                    gstr[d - 1 + sh] = cuuint64_t(p.sA[d]) * ESZ;
            }
            if(qInner)
            {
                // the second mode of a merged q: last dimension of A's map
                gdim[p.ndim + sh]     = cuuint64_t(q2Ext);
                gstr[p.ndim - 1 + sh] = cuuint64_t(q2StrideA) * ESZ;
                box[p.ndim + sh]      = cuuint32_t(TQ / qInner);
            }
            if(wide)
            {
                gdim[0] = E;
                gdim[1] = cuuint64_t(p.ext[0] / E);
                gstr[0] = 128;
                box[0]  = E;
                box[1]  = NP;
            }
            else
                box[0] = E;
            box[p.q + sh] = qInner ? cuuint32_t(qInner) : cuuint32_t(TQ);
            if(encode(&mapA, kType, p.ndim + sh + (qInner ? 1 : 0), const_cast<void*>(A), gdim, gstr, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               != CUDA_SUCCESS)
                return cudaErrorInvalidValue;
            // B: folded modes by ascending stride in B
            for(int i = 0; i < p.ndim; i++)
            {
                const int d  = p.orderB[i];
                gdim[i + sh] = cuuint64_t(d == 0 && pInner ? pInner : p.ext[d]);
                box[i + sh]  = 1;
                a.mapPosB[d] = i;
                if(i > 0)
                    gstr[i - 1 + sh] = cuuint64_t(p.sB[d]) * ESZ;
            }
            if(pInner)
            {
                // the second mode of a merged p: last dimension of B's map
                gdim[p.ndim + sh]     = cuuint64_t(p2Ext);
                gstr[p.ndim - 1 + sh] = cuuint64_t(p2StrideB) * ESZ;
                box[p.ndim + sh]      = cuuint32_t(TP / pInner);
            }
            a.posP_B = a.mapPosB[0];
            a.posQ_B = a.mapPosB[p.q];
            if(wide)
            {
                gdim[0] = E;
                gdim[1] = cuuint64_t(p.ext[p.q] / E);
                gstr[0] = 128;
                box[0]  = E;
                box[1]  = NQ;
            }
            else
                box[a.posQ_B] = E;
            box[a.posP_B + sh] = pInner ? cuuint32_t(pInner) : cuuint32_t(TP);
            if(encode(&mapB, kType, p.ndim + sh + (pInner ? 1 : 0), B, gdim, gstr, box, estr,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE)
               != CUDA_SUCCESS)
                return cudaErrorInvalidValue;
            a.ndim = p.ndim;
            a.q    = p.q;
            for(int d = 0; d < p.ndim; d++)
                a.ext[d] = uint32_t(p.ext[d]);
            a.alpha  = alpha;
            a.opA    = opA;
            a.opB    = opB;
            a.tilesP = uint32_t((p.ext[0] + TP - 1) / TP);
            a.tilesQ = uint32_t((p.ext[p.q] + TQ - 1) / TQ);
            a.status = status;
            long long tiles = (long long)a.tilesP * a.tilesQ;
            for(int d = 1; d < p.ndim; d++)
                if(d != p.q)
                    tiles *= p.ext[d];
            if(tiles > 0x7fffffffll)
                return cudaErrorInvalidConfiguration;
            a.numTiles = uint32_t(tiles);
            a.inStages  = tune.inStages;
            const int   smem = (a.inStages + kOutStages) * TP * TQ * ESZ + 1024;
            // the limit is a property of the function on the current device; the stage count can change between calls
            if(cudaError_t e = ensureDynamicSmem((const void*)perm_tma_kernel<NP, NQ, ESZ>, smem); e != cudaSuccess)
                return e;
            const int       fit   = std::max(1, (227 * 1024) / (smem + 1024));
            const int       perSm = std::min(fit, tune.ctasPerSm);
            const long long grid  = std::min<long long>(tiles, (long long)(smCount > 0 ? smCount : 148) * perSm);
            perm_tma_kernel<NP, NQ, ESZ><<<unsigned(grid), 64 * NP * NQ + 32, smem, stream>>>(mapA, mapB, a);
            return cudaGetLastError();
        }

        // The box kernel for f16 transpositions with even contiguous extents: a thread loads two 4-byte words (two
        // neighbours along A's contiguous mode, at two neighbouring coordinates of B's contiguous mode), exchanges their
        // halves and keeps two words that are pairs along B's contiguous mode, so shared memory and the stores to B move 4-byte
        // words as well: half the load/store instructions per element of the element-wise kernel. Index spaces, all in
        // A's order: element index i (lgBox bits); word index j = i without bit betaBit (what shared memory holds); unit
        // index u = j without bit 0 (what a thread loads: 2 x 2 elements).
        template <bool PLAIN>
        __global__ void __launch_bounds__(256) perm_box_pairs_kernel(const uint32_t* __restrict__ A, uint32_t* __restrict__ B, PermBoxArgs a)
        {
            extern __shared__ __align__(16) unsigned char boxRaw[];
            uint32_t* box = reinterpret_cast<uint32_t*>(boxRaw);
            uint32_t  bid = blockIdx.x;
            uint32_t  org[kBoxMaxDims];
            int64_t   offA = 0, offB = 0;
            uint32_t  cut = 0;
#pragma unroll
            for(int d = 0; d < kBoxMaxDims; d++)
            {
                org[d] = 0;
                if(d < a.nb)
                {
                    const uint32_t t = bid % a.tilesOf[d];
                    bid /= a.tilesOf[d];
                    org[d] = t << a.lgA[d];
                    offA += int64_t(org[d]) * a.sAofA[d];
                    offB += int64_t(org[d]) * a.sBofA[d];
                    if(org[d] + (1u << a.lgA[d]) > a.extA[d])
                        cut |= 1u << d;
                }
            }
            for(int d = 0; d < a.no; d++)
            {
                const uint32_t c = bid % a.extO[d];
                bid /= a.extO[d];
                offA += int64_t(c) * a.sAO[d];
                offB += int64_t(c) * a.sBO[d];
            }
            // the element offsets are even: every stride but the contiguous one is, and the contiguous extents are
            const uint32_t words = 1u << (a.lgBox - 1), units = words >> 1;
            const uint32_t t = threadIdx.x;
            // Both elements of a pair are inside the tensor or outside (even extents): one check per word, on the element
            // index with the pair's bit zero. Cut modes are split as in the element-wise kernel: those whose index bits
            // the thread fixes for a phase are checked once, up to two others with an add and a compare per word.
            const uint32_t bm     = (1u << a.betaBit) - 1u;
            auto           expand = [&](uint32_t j) { return (j & bm) | ((j & ~bm) << 1); };
            uint32_t       sh0 = 0, m0 = 0, room0 = 1, sh1 = 0, m1 = 0, room1 = 1;
            int            restN       = 0;
            auto           splitChecks = [&](uint32_t fixed, uint32_t part, bool& ok, uint32_t& rest) {
                ok     = true;
                rest   = 0;
                restN  = 0;
                sh0 = sh1 = m0 = m1 = 0;
                room0 = room1 = 1;
                int sh = 0;
#pragma unroll
                for(int d = 0; d < kBoxMaxDims; d++)
                    if(d < a.nb)
                    {
                        const uint32_t m = (1u << a.lgA[d]) - 1u;
                        if((cut >> d) & 1u)
                        {
                            if(((m << sh) & ~fixed) == 0)
                                ok = ok && org[d] + ((part >> sh) & m) < a.extA[d];
                            else if(restN < 2)
                            {
                                // what the element's other bits may add to the thread's share of the coordinate
                                const uint32_t mine = (part >> sh) & m, lim = a.extA[d] - org[d];
                                ok = ok && mine < lim;
                                if(restN == 0)
                                {
                                    sh0   = uint32_t(sh);
                                    m0    = m;
                                    room0 = lim - mine;
                                }
                                else
                                {
                                    sh1   = uint32_t(sh);
                                    m1    = m;
                                    room1 = lim - mine;
                                }
                                restN++;
                            }
                            else
                                rest |= 1u << d;
                        }
                        sh += a.lgA[d];
                    }
            };
            auto restOk = [&](uint32_t others) {
                // (with no such mode the masks are zero and the rooms one)
                return ((others >> sh0) & m0) < room0 && ((others >> sh1) & m1) < room1;
            };
            auto valid = [&](uint32_t i, uint32_t rest) {
                if(rest == 0)
                    return true;
                bool ok = true;
                int  sh = 0;
#pragma unroll
                for(int d = 0; d < kBoxMaxDims; d++)
                    if(d < a.nb)
                    {
                        if((rest >> d) & 1u)
                            ok = ok && org[d] + ((i >> sh) & ((1u << a.lgA[d]) - 1u)) < a.extA[d];
                        sh += a.lgA[d];
                    }
                return ok;
            };
            // slot of word j: bit 0 stays (a thread stores two neighbouring words at once), bits 1-4 are mixed with the
            // bits above them against bank conflicts of the strided reads
            auto slot = [](uint32_t j) { return j ^ (((j >> 5) ^ (j >> 10)) & 30u); };
            int64_t  lowA = offA >> 1, lowB = offB >> 1;
            uint32_t lowJ = 0, fixedJ = 0;
#pragma unroll
            for(int k = 0; k < 8; k++)
            {
                fixedJ |= a.slotB[k];
                if((t >> k) & 1u)
                {
                    lowA += a.wA[k];
                    lowB += a.wB[k];
                    lowJ += a.slotB[k];
                }
            }
            const uint32_t  loadRounds = max(units >> 8, 1u), storeRounds = max(words >> 8, 1u);
            const uint32_t* src = A + lowA;
            auto            put = [&](uint32_t r, uint32_t w0, uint32_t w1) {
                const uint32_t j = (t | (r << 8)) << 1;
                *reinterpret_cast<uint2*>(box + slot(j)) = make_uint2(__byte_perm(w0, w1, 0x5410), __byte_perm(w0, w1, 0x7632));
            };
            if(cut == 0)
            {
#pragma unroll
                for(uint32_t k0 = 0; k0 < kBoxRounds / 4; k0 += 8)
                    if(k0 < loadRounds)
                    {
                        uint32_t w0[8], w1[8];
#pragma unroll
                        for(uint32_t n = 0; n < 8; n++)
                            if(t < units && k0 + n < loadRounds)
                            {
                                w0[n] = src[a.hiA[k0 + n]];
                                w1[n] = src[a.hiA[k0 + n] + a.betaW];
                            }
#pragma unroll
                        for(uint32_t n = 0; n < 8; n++)
                            if(t < units && k0 + n < loadRounds)
                                put(k0 + n, w0[n], w1[n]);
                    }
            }
            else
            {
                bool     ok;
                uint32_t rest;
                splitChecks(expand(0x1ffu) | (1u << a.betaBit), expand(t << 1), ok, rest);
                ok = ok && t < units;
                {
                    // at most eight rounds of loads (2048 units of 2 x 2 elements)
                    uint32_t w0[8], w1[8];
                    bool     in[8];
#pragma unroll
                    for(uint32_t n = 0; n < 8; n++)
                    {
                        const uint32_t others = expand(n << 9);
                        in[n] = ok && n < loadRounds && restOk(others) && valid(expand(t << 1) | others, rest);
                        if(in[n])
                        {
                            w0[n] = src[a.hiA[n]];
                            w1[n] = src[a.hiA[n] + a.betaW];
                        }
                    }
#pragma unroll
                    for(uint32_t n = 0; n < 8; n++)
                        if(in[n])
                            put(n, w0[n], w1[n]);
                }
            }
            __syncthreads();
            uint32_t* dst = B + lowB;
            auto      out = [&](uint32_t w) -> uint32_t {
                if constexpr(PLAIN)
                    return w;
                else
                {
                    union
                    {
                        uint32_t w;
                        __half   e[2];
                    } v;
                    v.w    = w;
                    v.e[0] = Elem<__half>::apply(v.e[0], a.alpha, a.opA, a.opB);
                    v.e[1] = Elem<__half>::apply(v.e[1], a.alpha, a.opA, a.opB);
                    return v.w;
                }
            };
            if(cut == 0)
            {
#pragma unroll
                for(uint32_t k0 = 0; k0 < kBoxRounds / 2; k0 += 8)
                    if(k0 < storeRounds)
                    {
#pragma unroll
                        for(uint32_t n = 0; n < 8; n++)
                            if(t < words && k0 + n < storeRounds)
                                dst[a.hiB[k0 + n]] = out(box[slot(lowJ + a.hiS[k0 + n])]);
                    }
            }
            else
            {
                bool     ok;
                uint32_t rest;
                splitChecks(expand(fixedJ) | (1u << a.betaBit), expand(lowJ), ok, rest);
                ok = ok && t < words;
#pragma unroll 1
                for(uint32_t k0 = 0; k0 < storeRounds; k0 += 8)
                {
                    // the table entry of k0 + n is the sum of those of k0 and n (disjoint bits)
                    uint32_t*      base = dst + a.hiB[k0];
                    const uint32_t hs0  = a.hiS[k0];
#pragma unroll
                    for(uint32_t n = 0; n < 8; n++)
                    {
                        const uint32_t hs = hs0 + a.hiS[n], others = expand(hs);
                        if(ok && k0 + n < storeRounds && restOk(others) && valid(expand(lowJ) | others, rest))
                            base[a.hiB[n]] = out(box[slot(lowJ + hs)]);
                    }
                }
            }
        }

        // Box of the box kernel: A's leading modes until their tile extents multiply to 64, B's leading modes likewise,
        // then more of A's modes until the box holds 2048 to 8192 elements. False when the grid would not fit.
        template <typename TI, typename TO, int PACK>
        bool launchBoxPacked(const PermPlan& p, const void* A, void* B, float alpha, int opA, int opB, bool pairs,
                             cudaStream_t stream, cudaError_t* err)
        {
            auto lgCeil = [](int64_t v) {
                int l = 0;
                while((int64_t(1) << l) < v)
                    l++;
                return l;
            };
            if constexpr(PACK * sizeof(TI) > 16 || PACK * sizeof(TO) > 16)
                return false;
            else
            {
            int lg[kMaxGroup] = {0, 0, 0, 0, 0, 0};
            // A's run
            // 64 elements of 2 or 4 bytes; packed words need fewer for the same bytes
            constexpr int runBits = PACK >= 8 ? 3 : PACK == 4 ? 4 : PACK == 2 ? 5 : 6;
            for(int d = 0, need = runBits; d < p.ndim && need > 0; d++)
            {
                const int l = std::min(lgCeil(p.ext[d]), need);
                lg[d]       = std::max(lg[d], l);
                need -= l;
            }
            // B's run
            for(int i = 0, need = runBits; i < p.ndim && need > 0; i++)
            {
                const int d = p.orderB[i], l = std::min(lgCeil(p.ext[d]), need);
                lg[d]       = std::max(lg[d], l);
                need -= l;
            }
            int total = 0;
            for(int d = 0; d < p.ndim; d++)
                total += lg[d];
            // grow along A's order up to the target size
            // larger boxes amortise a block's set-up (2.9 TB/s with 8192 elements of two bytes against 1.7 with 2048);
            // smaller ones keep at least eight blocks per SM on tensors of a few million elements
            int64_t count = 1;
            for(int d = 0; d < p.ndim; d++)
                count *= p.ext[d];
            int target = 11;
            while(target < kBoxBits && (count >> (target + 1)) >= 8 * 148 && (sizeof(TI) * PACK << (target + 1)) <= 32768)
                target++;
            for(int d = 0; d < p.ndim && total < target; d++)
                while(total < target && lg[d] < lgCeil(p.ext[d]))
                {
                    lg[d]++;
                    total++;
                }
            if(total > kBoxBits || (sizeof(TI) * PACK << total) > 48 * 1024)
                return false;
            PermBoxArgs a{};
            int64_t     grid = 1;
            for(int d = 0; d < p.ndim; d++)
            {
                if(lg[d] > 0)
                {
                    const int k = a.nb++;
                    a.lgA[k]    = lg[d];
                    a.extA[k]   = uint32_t(p.ext[d]);
                    a.sAofA[k]  = p.sA[d];
                    a.sBofA[k]  = p.sB[d];
                    a.tilesOf[k] = uint32_t((p.ext[d] + (int64_t(1) << lg[d]) - 1) >> lg[d]);
                    grid *= a.tilesOf[k];
                }
                else
                {
                    const int k = a.no++;
                    a.extO[k]   = uint32_t(p.ext[d]);
                    a.sAO[k]    = p.sA[d];
                    a.sBO[k]    = p.sB[d];
                    grid *= p.ext[d];
                }
                if(p.ext[d] >= (int64_t(1) << 31) || grid > 0x7fffffffll)
                    return false;
            }
            // weights of the index bits: A's order follows the folded modes, B's order their ascending stride in B
            int shiftOf[kMaxGroup], bit = 0;
            for(int d = 0; d < p.ndim; d++)
            {
                shiftOf[d] = bit;
                for(int k = 0; k < lg[d]; k++, bit++)
                    a.wA[bit] = p.sA[d] << k;
            }
            bit = 0;
            for(int i = 0; i < p.ndim; i++)
            {
                const int d = p.orderB[i];
                for(int k = 0; k < lg[d]; k++, bit++)
                {
                    a.wB[bit]    = p.sB[d] << k;
                    a.slotB[bit] = 1u << (shiftOf[d] + k);
                }
            }
            if(pairs)
            {
                // from element indices to unit indices (loads) and word indices (shared memory, stores); weights in words
                const int beta = shiftOf[p.q];
                int64_t   wA2[kBoxBits] = {}, wB2[kBoxBits] = {};
                uint32_t  s2[kBoxBits] = {};
                for(int k = 0; k + 2 < total; k++)
                    wA2[k] = a.wA[k + 1 < beta ? k + 1 : k + 2] / 2;
                for(int k = 0; k + 1 < total; k++)
                {
                    int pos = 0;
                    while((a.slotB[k + 1] >> pos) != 1u)
                        pos++;
                    s2[k]  = 1u << (pos < beta ? pos : pos - 1);
                    wB2[k] = a.wB[k + 1] / 2;
                }
                a.betaBit = beta;
                a.betaW   = a.wA[beta] / 2;
                for(int k = 0; k < kBoxBits; k++)
                {
                    a.wA[k]    = wA2[k];
                    a.wB[k]    = wB2[k];
                    a.slotB[k] = s2[k];
                }
            }
            for(int r = 0; r < kBoxRounds; r++)
                for(int k = 8; k < kBoxBits; k++)
                    if((r >> (k - 8)) & 1)
                    {
                        a.hiA[r] += a.wA[k];
                        a.hiB[r] += a.wB[k];
                        a.hiS[r] += a.slotB[k];
                    }
            a.lgBox = total;
            a.alpha = alpha;
            a.opA   = opA;
            a.opB   = opB;
            const size_t smem = (size_t(1) << total) * sizeof(TI) * PACK;
            if(pairs)
            {
                if(alpha == 1.0f && opA != 2 && opB != 2)
                    perm_box_pairs_kernel<true><<<unsigned(grid), 256, smem, stream>>>((const uint32_t*)A, (uint32_t*)B, a);
                else
                    perm_box_pairs_kernel<false><<<unsigned(grid), 256, smem, stream>>>((const uint32_t*)A, (uint32_t*)B, a);
            }
            else if(alpha == 1.0f && opA != 2 && opB != 2)
                perm_box_kernel<TI, TO, PACK, true><<<unsigned(grid), 256, smem, stream>>>(A, B, a);
            else
                perm_box_kernel<TI, TO, PACK, false><<<unsigned(grid), 256, smem, stream>>>(A, B, a);
            *err = cudaGetLastError();
            if(*err == cudaSuccess)
                noteLaunch("perm_box");
            return true;
            }
        }

        // Picks the word the box kernel moves and launches it.
        template <typename TI, typename TO>
        bool launchBox(const PermPlan& p, const void* A, void* B, float alpha, int opA, int opB, cudaStream_t stream,
                       cudaError_t* err)
        {
            // Rows shared by A and B move as words of up to 16 bytes: the same permutation of fewer, larger elements.
            int pack = 1;
            if(p.kind == PERM_COPY && p.sA[0] == 1 && p.sB[0] == 1)
            {
                constexpr int wide = int(sizeof(TI) > sizeof(TO) ? sizeof(TI) : sizeof(TO));
                for(int c = 16 / wide; c > 1 && pack == 1; c /= 2)
                {
                    bool ok = p.ext[0] % c == 0 && (uintptr_t)A % (c * sizeof(TI)) == 0 && (uintptr_t)B % (c * sizeof(TO)) == 0;
                    for(int d = 1; d < p.ndim; d++)
                        ok = ok && p.sA[d] % c == 0 && p.sB[d] % c == 0;
                    if(ok)
                        pack = c;
                }
            }
            if(pack > 1)
            {
                PermPlan w = p;
                w.kind     = PERM_TILE; // not packed again
                w.ext[0] /= pack;
                for(int d = 1; d < w.ndim; d++)
                {
                    w.sA[d] /= pack;
                    w.sB[d] /= pack;
                }
                switch(pack)
                {
                case 2: return launchBoxPacked<TI, TO, 2>(w, A, B, alpha, opA, opB, false, stream, err);
                case 4: return launchBoxPacked<TI, TO, 4>(w, A, B, alpha, opA, opB, false, stream, err);
                default: return launchBoxPacked<TI, TO, 8>(w, A, B, alpha, opA, opB, false, stream, err);
                }
            }
            // f16 transpositions whose contiguous extents and other strides are even: 2 x 2 elements per thread
            bool pairs = false;
            if constexpr(std::is_same<TI, __half>::value && std::is_same<TO, __half>::value)
            {
                pairs = p.kind != PERM_COPY && p.q != 0 && p.orderB[0] == p.q && p.sA[0] == 1 && p.sB[p.q] == 1 && p.ext[0] % 2 == 0
                        && p.ext[p.q] % 2 == 0 && (uintptr_t)A % 4 == 0 && (uintptr_t)B % 4 == 0;
                for(int d = 0; d < p.ndim; d++)
                    pairs = pairs && (d == 0 || p.sA[d] % 2 == 0) && (d == p.q || p.sB[d] % 2 == 0);
            }
            return launchBoxPacked<TI, TO, 1>(p, A, B, alpha, opA, opB, pairs, stream, err);
        }


        template <typename TI, typename TO>
        cudaError_t launchPlain(const PermPlan& p, const void* A, void* B, float alpha, int opA, int opB, bool preferBox,
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
            // short contiguous modes: a box over several modes instead of a (p, q) tile or a (mode 0, mode 1) tile
            {
                const bool shortTile = p.kind != PERM_COPY && p.ndim >= 2 && (preferBox || p.ext[0] < 32 || p.ext[p.q] < 32);
                // copies: rows of at most 128 bytes, of 256 or 512 (a power of two of 16-byte words), or rows of at most 1 KiB with very few of them per tile
                const bool shortCopy = p.kind == PERM_COPY && p.ndim >= 2
                                       && (p.ext[0] * int64_t(sizeof(TI)) <= 128
                                           || p.ext[0] * int64_t(sizeof(TI)) == 256 || p.ext[0] * int64_t(sizeof(TI)) == 512
                                           || (p.ndim >= 3 && p.ext[1] <= 8 && p.ext[0] * int64_t(sizeof(TI)) <= 1024));
                cudaError_t e;
                if((shortTile || shortCopy) && launchBox<TI, TO>(p, A, B, alpha, opA, opB, stream, &e))
                    return e;
            }
            if(p.kind == PERM_COPY)
            {
                // widest vector that keeps every access aligned
                int vec = 16 / int(sizeof(TI));
                if(sizeof(TO) > sizeof(TI))
                    vec /= 2; // 16-byte stores of the wider output type
                auto aligned = [&](int v) {
                    if((uintptr_t(A) % (sizeof(TI) * v)) || (uintptr_t(B) % (sizeof(TO) * v)) || p.ext[0] % v)
                        return false;
                    for(int d = 1; d < p.ndim; d++)
                        if(p.sA[d] % v || p.sB[d] % v)
                            return false;
                    return true;
                };
                while(vec > 1 && !aligned(vec))
                    vec >>= 1;
                // a single folded mode (plain scaled copy) is viewed as rows of 256 vectors
                int64_t flatTotal = 0;
                if(p.ndim == 1 && p.ext[0] > 256 * vec)
                {
                    flatTotal = p.ext[0];
                    a.ndim    = 2;
                    a.ext[0]  = 256 * vec;
                    a.ext[1]  = (flatTotal + a.ext[0] - 1) / a.ext[0];
                    a.sA[1] = a.sB[1] = a.ext[0];
                }
                const PermArgs& q = a; // extents as the kernel sees them
                const int64_t chunks = (q.ext[0] + vec - 1) / vec;
                int           log2c  = 0;
                while(log2c < 8 && (int64_t(1) << log2c) < chunks)
                    log2c++;
                const int     T1     = 1024 >> log2c;
                const int64_t ext1   = (q.ndim > 1) ? q.ext[1] : 1;
                const int64_t tiles0 = (chunks + (int64_t(1) << log2c) - 1) >> log2c;
                const int64_t tiles1 = (ext1 + T1 - 1) / T1;
                int64_t       grid   = tiles0 * tiles1;
                for(int d = 2; d < q.ndim; d++)
                    grid *= q.ext[d];
                if(grid > 0x7fffffffll || tiles0 > 0x7fffffffll || tiles1 > 0x7fffffffll)
                    return cudaErrorInvalidConfiguration;
                const TI* Ap = (const TI*)A;
                TO*       Bp = (TO*)B;
                switch(vec)
                {
                case 8:
                    if constexpr(sizeof(TI) == 2 && sizeof(TO) == 2)
                        perm_copy_kernel<TI, TO, 8>
                            <<<unsigned(grid), 256, 0, stream>>>(Ap, Bp, a, log2c, int(tiles0), int(tiles1), flatTotal);
                    break;
                case 4:
                    perm_copy_kernel<TI, TO, 4><<<unsigned(grid), 256, 0, stream>>>(Ap, Bp, a, log2c, int(tiles0), int(tiles1), flatTotal);
                    break;
                case 2:
                    perm_copy_kernel<TI, TO, 2><<<unsigned(grid), 256, 0, stream>>>(Ap, Bp, a, log2c, int(tiles0), int(tiles1), flatTotal);
                    break;
                default:
                    perm_copy_kernel<TI, TO, 1><<<unsigned(grid), 256, 0, stream>>>(Ap, Bp, a, log2c, int(tiles0), int(tiles1), flatTotal);
                    break;
                }
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
                // f16 with everything a multiple of 4 elements: 128 x 128 tiles, 4 x 4 blocks, 8-byte accesses
                if constexpr(sizeof(TI) == 2)
                {
                    bool quad = (uintptr_t(A) % 8) == 0 && (uintptr_t(B) % (4 * sizeof(TO))) == 0 && p.ext[0] % 4 == 0
                                && p.ext[p.q] % 4 == 0;
                    for(int d = 0; d < p.ndim && quad; d++)
                        quad = (d == 0 || p.sA[d] % 4 == 0) && (d == p.q || p.sB[d] % 4 == 0);
                    if(quad)
                    {
                        const int tP = int((p.ext[0] + kTile4 - 1) / kTile4), tQ = int((p.ext[p.q] + kTile4 - 1) / kTile4);
                        int64_t   nb = int64_t(tP) * tQ;
                        for(int d = 1; d < p.ndim; d++)
                            if(d != p.q)
                                nb *= p.ext[d];
                        if(nb > 0x7fffffffll)
                            return cudaErrorInvalidConfiguration;
                        perm_tile4_half_kernel<TO><<<unsigned(nb), 256, 0, stream>>>((const __half*)A, (TO*)B, a, tP, tQ);
                        noteLaunch("perm_tile");
                        return cudaGetLastError();
                    }
                }
                // 2 x 2 blocks when every extent, stride and base address is even (2-element accesses stay aligned)
                bool even = (uintptr_t(A) % (2 * sizeof(TI))) == 0 && (uintptr_t(B) % (2 * sizeof(TO))) == 0;
                for(int d = 0; d < p.ndim && even; d++)
                    even = (d == 0 || p.sA[d] % 2 == 0) && (d == p.q || p.sB[d] % 2 == 0);
                even = even && p.ext[0] % 2 == 0 && p.ext[p.q] % 2 == 0;
                if(even)
                    perm_tile_kernel<TI, TO, 2><<<unsigned(blocks), 256, 0, stream>>>((const TI*)A, (TO*)B, a, tilesP, tilesQ);
                else
                {
                    if(a.alpha == 1.0f && a.opA != 2 && a.opB != 2)
                        perm_tile_kernel<TI, TO, 1, true><<<unsigned(blocks), 256, 0, stream>>>((const TI*)A, (TO*)B, a, tilesP, tilesQ);
                    else
                        perm_tile_kernel<TI, TO, 1><<<unsigned(blocks), 256, 0, stream>>>((const TI*)A, (TO*)B, a, tilesP, tilesQ);
                }
                noteLaunch("perm_tile");
            }
            return cudaGetLastError();
        }
    } // namespace

    cudaError_t launchPermutation(const PermPlan& plan, int typeA, int typeB, const void* A, void* B, float alpha,
                                  int opA, int opB, int smCount, int* deviceStatus, cudaStream_t stream)
    {
        if(plan.total == 0)
            return cudaSuccess;
        // A TMA tile is 2E x 2E elements (E = 128 bytes of elements). A contiguous mode much shorter than that leaves it
        // mostly empty unless the kernel can merge the mode with its neighbour (launchTma); at a quarter full or less the box
        // kernel is faster (4.8 TB/s against 2.0 to 2.3 on 4-byte elements, 2.9 against 2.2 to 2.4 on 2-byte ones).
        bool sparseTiles = false;
        if(plan.kind == PERM_TMA)
        {
            const int64_t side = 2 * (128 / std::max(plan.elemSize, 1));
            const bool    pow2P = (plan.ext[0] & (plan.ext[0] - 1)) == 0, pow2Q = (plan.ext[plan.q] & (plan.ext[plan.q] - 1)) == 0;
            const bool    rank34 = plan.ndim >= 3 && plan.ndim <= 4;
            const bool    mergeP = rank34 && pow2P && plan.q != 1;
            const bool    mergeQ = rank34 && pow2Q && plan.orderB[0] == plan.q && plan.orderB[1] != 0;
            const double  fillP = mergeP ? 1.0 : double(std::min(plan.ext[0], side)) / double(side);
            const double  fillQ = mergeQ ? 1.0 : double(std::min(plan.ext[plan.q], side)) / double(side);
            sparseTiles         = fillP * fillQ <= 0.25;
        }
        if(plan.kind == PERM_TMA && !sparseTiles)
        {
            // tile shape: long runs on the store side (rows of the output tile are 32*NQ... wide)
            PermTune tune;
#ifdef HTB_MEASURE
            // measurement builds only: tile shape (22, 14, 41, 24, 42), input stages and CTAs per SM of a tuning run
            const Switches& sw = switches();
            if(sw.permTile)
                tune.shape = sw.permTile;
            if(sw.permStages)
                tune.inStages = sw.permStages;
            if(sw.permCtas)
                tune.ctasPerSm = sw.permCtas;
#endif
            tune.inStages = std::min(std::max(tune.inStages, 1), kMaxInStages);
            cudaError_t e;
            if(typeA == CUDA_R_16F)
            {
                // 2-byte elements: 128-byte rows hold 64 elements; 128 x 128 tiles by default
                switch(tune.shape)
                {
                case 11: e = launchTma<1, 1, 2>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                case 12: e = launchTma<1, 2, 2>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                case 21: e = launchTma<2, 1, 2>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                default: e = launchTma<2, 2, 2>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                }
            }
            else
            {
                switch(tune.shape)
                {
                case 14: e = launchTma<1, 4, 4>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                case 41: e = launchTma<4, 1, 4>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                case 24: e = launchTma<2, 4, 4>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                case 42: e = launchTma<4, 2, 4>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                default: e = launchTma<2, 2, 4>(plan, A, B, alpha, opA, opB, tune, smCount, deviceStatus, stream); break;
                }
            }
            if(e == cudaSuccess)
                noteLaunch("perm_tma");
            // a tensor map that the driver refuses (nothing was launched) leaves the shared-memory tile kernel
            if(e != cudaErrorInvalidValue)
                return e;
            cudaGetLastError();
        }
        if(typeA == CUDA_R_32F)
            return launchPlain<float, float>(plan, A, B, alpha, opA, opB, sparseTiles, stream);
        if(typeB == CUDA_R_16F)
            return launchPlain<__half, __half>(plan, A, B, alpha, opA, opB, sparseTiles, stream);
        return launchPlain<__half, float>(plan, A, B, alpha, opA, opB, sparseTiles, stream);
    }
} // namespace htb
