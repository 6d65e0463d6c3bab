// Row groups of a contraction tile, shared by the tensor-core contraction kernels.
//
// A tile takes its rows (of A and D, or of B and the columns of D) from one group of folded modes in one of
// two ways:
//   major 0  the operand is K-major: the rows are gathered by a multi-dimensional TMA box over the folded modes
//            (boxDecompose in the planner);
//   major 1  the operand is MN-major: the group's stride-1 mode is cut into chunks of 128 bytes (32 fp32 or 64
//            half-precision elements); a tile is a run of consecutive chunks, chunk index = (chunk along mode 0)
//            + chunks0 * (index over the remaining modes).
// Device code turns (tile, row) into an element offset of D and into TMA coordinates; host code fills the
// descriptions from the planner's groups.
#pragma once

#include <cstdint>

#include "planner.hpp"

namespace htb
{
    namespace
    {
        // One row group of the tile: the M side (rows of A and D) or the N side (rows of B, columns of D).
        struct TfGroup
        {
            int     major; // 0: operand K-major, rows gathered by a TMA box over the folded modes
                           // 1: operand MN-major, rows taken in chunks of 2^chunkShift (32 fp32 or 64 half elements =
                           //    128 bytes) along the stride-1 mode 0
            int     n; // folded modes
            int     rows; // rows of this group per CTA tile (128, or 64 for a narrow N tile)
            int     tiles;
            int     box[4], tilesPerDim[4]; // major 0
            int     chunkShift; // major 1: log2 of the rows per chunk
            int     chunks0; // major 1: chunks along mode 0
            int64_t restExt; // major 1: product of the extents of modes 1..
            int64_t ext[4], sD[4];
        };


        // position of a tile inside its group
        struct TfTile
        {
            int c[4]; // major 0: first coordinate per mode
            int chunkBase; // major 1: first chunk
        };

        __device__ __forceinline__ TfTile tfTileOf(const TfGroup& g, int t)
        {
            TfTile w;
            w.chunkBase = t * (g.rows >> g.chunkShift);
#pragma unroll
            for(int d = 0; d < 4; d++)
            {
                const int per = (d < g.n) ? g.tilesPerDim[d] : 1;
                w.c[d]        = (t % per) * ((d < g.n) ? g.box[d] : 1);
                t /= per;
            }
            return w;
        }

        // row r of a tile -> offset in D along this group, or -1 outside the tensor
        __device__ __forceinline__ int64_t tfRowOffset(const TfGroup& g, const TfTile& w, int r)
        {
            if(g.major == 0)
            {
                int64_t off = 0;
                for(int d = 0; d < g.n; d++)
                {
                    const int i = r % g.box[d];
                    r /= g.box[d];
                    const int64_t x = int64_t(w.c[d]) + i;
                    if(x >= g.ext[d])
                        return -1;
                    off += x * g.sD[d];
                }
                return (r == 0) ? off : -1;
            }
            const int     chunk = w.chunkBase + (r >> g.chunkShift);
            const int64_t i0    = (int64_t(chunk % g.chunks0) << g.chunkShift) + (r & ((1 << g.chunkShift) - 1));
            int64_t       rest  = chunk / g.chunks0;
            if(i0 >= g.ext[0] || rest >= g.restExt)
                return -1;
            int64_t off = i0 * g.sD[0];
            for(int d = 1; d < g.n; d++)
            {
                off += (rest % g.ext[d]) * g.sD[d];
                rest /= g.ext[d];
            }
            return off;
        }

        // TMA coordinates of a tile's chunks (MN-major operands), fixed for the whole K loop
        struct TfChunks
        {
            int c0[4], i1[4], i2[4];
        };
        __device__ __forceinline__ TfChunks tfChunksOf(const TfGroup& g, const TfTile& w)
        {
            TfChunks       q;
            const uint32_t e1 = (g.n > 1) ? uint32_t(g.ext[1]) : 1u; // extents fit 32 bits (tensor-map limit)
#pragma unroll
            for(int j = 0; j < 4; j++)
            {
                const uint32_t chunk = uint32_t(w.chunkBase + j);
                const uint32_t rest  = chunk / uint32_t(g.chunks0);
                // beyond the tensor the coordinates fall outside the map and the box is zero-filled
                q.c0[j] = int((chunk - rest * uint32_t(g.chunks0)) << g.chunkShift);
                q.i2[j] = int(rest / e1);
                q.i1[j] = int(rest - uint32_t(q.i2[j]) * e1);
            }
            return q;
        }


        // ------------------------------------------------------------------ host side
        struct RowGroupView
        {
            int     n;
            int64_t ext[4], sOp[4], sD[4]; // extent, stride in the operand, stride in D; mode 0 first
        };


        // planner group -> view with the chunked (stride-1) mode first
        RowGroupView viewOf(const ModeDim* dims, int n, int fast)
        {
            RowGroupView v{};
            int          k = 0;
            auto         put = [&](int i) {
                v.ext[k] = dims[i].ext;
                v.sOp[k] = dims[i].s0;
                v.sD[k]  = dims[i].s1;
                k++;
            };
            if(fast >= 0)
                put(fast);
            for(int i = 0; i < n && k < 4; i++)
                if(i != fast)
                    put(i);
            v.n = k;
            return v;
        }

        void fillGroup(TfGroup& g, const RowGroupView& v, int major, int rows, const int* box, int chunkShift)
        {
            g.major = major;
            g.n     = v.n;
            g.rows  = rows;
            g.tiles = 1;
            g.restExt = 1;
            for(int d = 0; d < 4; d++)
            {
                g.ext[d]         = d < v.n ? v.ext[d] : 1;
                g.sD[d]          = d < v.n ? v.sD[d] : 0;
                g.box[d]         = (major == 0 && d < v.n) ? box[d] : 1;
                g.tilesPerDim[d] = int((g.ext[d] + g.box[d] - 1) / g.box[d]);
                if(major == 0)
                    g.tiles *= g.tilesPerDim[d];
                else if(d >= 1)
                    g.restExt *= g.ext[d];
            }
            g.chunkShift = chunkShift;
            g.chunks0    = int((g.ext[0] + (int64_t(1) << chunkShift) - 1) >> chunkShift);
            if(major == 1)
            {
                const int64_t chunks = int64_t(g.chunks0) * g.restExt, per = rows >> chunkShift;
                g.tiles              = int((chunks + per - 1) / per);
            }
        }
    } // namespace
} // namespace htb
