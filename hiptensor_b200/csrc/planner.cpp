// Host-side planner (see planner.hpp). No CUDA calls in this file.
#include "planner.hpp"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <library_types.h>

namespace htb
{
    namespace
    {
        int findMode(const int32_t* modes, int n, int32_t m)
        {
            for(int i = 0; i < n; i++)
                if(modes[i] == m)
                    return i;
            return -1;
        }

        bool hasDuplicates(const int32_t* modes, int n)
        {
            for(int i = 0; i < n; i++)
                for(int j = i + 1; j < n; j++)
                    if(modes[i] == modes[j])
                        return true;
            return false;
        }

        int elemSizeOf(int dt)
        {
            switch(dt)
            {
            case CUDA_R_32F: return 4;
            case CUDA_R_64F: return 8;
            case CUDA_R_16F: return 2;
            case CUDA_R_16BF: return 2;
            default: return 0;
            }
        }

        const char* typeName(int dt)
        {
            switch(dt)
            {
            case CUDA_R_32F: return "f32";
            case CUDA_R_64F: return "f64";
            case CUDA_R_16F: return "f16";
            case CUDA_R_16BF: return "bf16";
            default: return "none";
            }
        }

        void appendDims(std::string& s, const char* name, const ModeDim* d, int n)
        {
            char buf[96];
            s += name;
            s += "[";
            for(int i = 0; i < n; i++)
            {
                snprintf(buf, sizeof(buf), "%s%lld:%lld/%lld", i ? " " : "", (long long)d[i].ext,
                         (long long)d[i].s0, (long long)d[i].s1);
                s += buf;
            }
            s += "]";
        }

        // stable insertion sort of the few (at most kMaxRank + 2) entries of a mode group: no heap buffer,
        // unlike std::stable_sort, so that planning allocates nothing
        template <typename T, typename Less>
        void sortSmall(T* v, int n, Less less)
        {
            for(int i = 1; i < n; i++)
            {
                T   x = v[i];
                int j = i;
                for(; j > 0 && less(x, v[j - 1]); j--)
                    v[j] = v[j - 1];
                v[j] = x;
            }
        }

        bool isPow2(int64_t v)
        {
            return v > 0 && (v & (v - 1)) == 0;
        }
    } // namespace

    int foldGroup(ModeDim* dims, int n)
    {
        int w = 0;
        for(int i = 0; i < n; i++)
        {
            if(dims[i].ext == 1)
                continue;
            if(w > 0 && dims[i].s0 == dims[w - 1].s0 * dims[w - 1].ext
               && dims[i].s1 == dims[w - 1].s1 * dims[w - 1].ext)
            {
                dims[w - 1].ext *= dims[i].ext;
            }
            else
            {
                dims[w++] = dims[i];
            }
        }
        if(w == 0)
        {
            dims[0] = ModeDim{1, 0, 0};
            w       = 1;
        }
        return w;
    }

    // Form of the CTA-pair tensor-core kernel for an M x N x K problem, from measurements on B200 (f16, N = K =
    // 4096, kernels back to back, microseconds; "tiles" counts 256 x 256 tiles, 74 CTA pairs fit the chip):
    //   tiles  M     single CTAs  256x256  256x256 K/2  256x512  256x512 K/2
    //    32    512      30.4        30.5      23.7         -          -
    //    64   1024       -          33-35      -          49.6      36-39
    //   128   2048       -          65.5       -          61-64       -
    //   256   4096       -         107-123     -         115-123      -
    // The main loops run at the same rate per flop (a pipeline stage turns around in 2.3 - 2.7 us whatever it holds),
    // so the wider tile only pays where it saves rounds or operand traffic, and a K split only where the tiles fill
    // at most half of the pairs (each part must still be 16 stages long to pay for the exchange).
    // Mid-size problems, same protocol (single CTAs / pairs, an under-filled wave in half tiles / pairs with the K split):
    //   tiles   M x N        K = 512          1024             2048             4096
    //     9    768 x 768    6.8/6.7/8.8     9.9/9.0/10.1    12.7/13.5/12.5   18.6/22.8/18.3
    //    16   1024 x 1024   6.9/6.8/8.8     9.6/9.2/10.1    15.1/14.0/13.1   25.8/23.1/18.4
    //    25   1280 x 1280   8.9/8.2/10.5   11.7/10.7/12.0   17.5/15.4/14.9   28.4/24.4/20.0
    //    32    512 x 4096   8.6/9.0/11.4   11.7/11.5/13.2   17.1/16.0/16.0   27.9/25.5/21.5
    //    36   1536 x 1536  10.2/9.2/9.1    13.2/11.7/11.9   18.8/16.3/17.0   29.7/25.4/27.2
    //    48   2048 x 1536  14.6/10.5/-     17.3/13.1/-      23.3/18.2/-      35.2/28.4/-
    //    64   2048 x 2048  13.2/11.8/-     15.0/13.9/-      21.1/19.1/-      37.0/34.8/-
    //   100   2560 x 2560  31.7/14.5/-     31.6/18.2/-      43.9/28.1/-      69.5/53.0/-
    // A single CTA's tile shares no operand with a neighbour and an SM takes 64 bytes per clock from L2, so the pairs win
    // from nine tiles on unless K is short; up to 32 tiles and from K = 2048 on the K split is better still.
    void pairKernelForm(int64_t M, int64_t N, int64_t K, int sms, int* pair, int* wide, int* ksplit)
    {
        const int64_t tiles = ((M + 255) / 256) * ((N + 255) / 256), pairs = sms / 2, quads = sms / 4 - 1;
        *pair   = 0;
        *wide   = 0;
        *ksplit = 1;
        if(tiles >= sms / 16 && tiles <= (int64_t(sms) * 7) / 32 && K >= 2048)
        {
            *pair   = 1;
            *ksplit = 2;
        }
        else if(tiles >= quads || (tiles >= sms / 16 && K >= 1024))
        {
            *pair = 1;
            *wide = tiles > (3 * pairs) / 2 ? 1 : 0;
        }
    }

    int boxDecompose(const ModeDim* dims, int n, int tile, int* box)
    {
        int64_t remaining = tile;
        for(int i = 0; i < n; i++)
        {
            if(remaining == 1)
                box[i] = 1;
            else if(dims[i].ext >= remaining)
            {
                box[i]    = int(remaining);
                remaining = 1;
            }
            else if(isPow2(dims[i].ext))
            {
                box[i] = int(dims[i].ext);
                remaining /= dims[i].ext;
            }
            else if(i == n - 1)
            {
                // the slowest mode may be shorter than what is left of the tile: its box reaches past the tensor, TMA fills
                // those rows with zeros and the epilogue masks them like any ragged end
                box[i]    = int(remaining);
                remaining = 1;
            }
            else
                return 0;
        }
        return int(tile / remaining);
    }

    // ------------------------------------------------------------------ permutation
    int planPermutation(int rank, const int64_t* lensA, const int32_t* modeA, const int32_t* modeB,
                        int typeA, int typeB, bool pointersAligned16, PermPlan* out)
    {
        std::memset(out, 0, sizeof(*out));
        if(rank < 1 || rank > kMaxGroup || !lensA || !modeA || !modeB)
            return PLAN_INVALID;
        // reference type rules: f16->f16, f16->f32, f32->f32
        // (docs/api-reference/api-reference.rst:77-81, hiptensor_permutation.cpp:123-144)
        const bool typesOk = (typeA == CUDA_R_32F && typeB == CUDA_R_32F)
                             || (typeA == CUDA_R_16F && (typeB == CUDA_R_16F || typeB == CUDA_R_32F));
        if(!typesOk)
            return PLAN_NOT_SUPPORTED;
        if(hasDuplicates(modeA, rank) || hasDuplicates(modeB, rank))
            return PLAN_INVALID;
        for(int i = 0; i < rank; i++)
        {
            if(lensA[i] <= 0)
                return PLAN_INVALID;
            if(findMode(modeA, rank, modeB[i]) < 0)
                return PLAN_INVALID;
        }

        ModeDim dims[kMaxGroup];
        int64_t s = 1;
        for(int i = 0; i < rank; i++)
        {
            dims[i].ext = lensA[i];
            dims[i].s0  = s;
            s *= lensA[i];
        }
        out->total = s;
        s          = 1;
        for(int i = 0; i < rank; i++)
        {
            int ia      = findMode(modeA, rank, modeB[i]);
            dims[ia].s1 = s;
            s *= lensA[ia];
        }
        int n     = foldGroup(dims, rank);
        out->ndim = n;
        out->q    = 0;
        for(int i = 0; i < n; i++)
        {
            out->ext[i] = dims[i].ext;
            out->sA[i]  = dims[i].s0;
            out->sB[i]  = dims[i].s1;
            if(dims[i].s1 == 1 && dims[i].ext > 1)
                out->q = i;
        }
        if(n == 1 && dims[0].ext == 1)
        {
            out->sA[0] = out->sB[0] = 1;
        }
        for(int i = 0; i < n; i++)
            out->orderB[i] = i;
        std::sort(out->orderB, out->orderB + n, [&](int a, int b) { return out->sB[a] < out->sB[b]; });
        out->elemSize = elemSizeOf(typeA);

        if(out->q == 0)
        {
            out->kind = PERM_COPY;
        }
        else
        {
            // TMA path: fp32 -> fp32 and f16 -> f16, every stride a multiple of 16 bytes (extents of the two
            // contiguous modes multiples of 4 / 8 elements)
            const int64_t per16 = 16 / std::max(out->elemSize, 1);
            // a short contiguous mode of B (a power of two from 16 bytes on) will do when the mode after it in B makes
            // one contiguous run with it: the kernel merges the two (launchTma, "merged q")
            const int64_t extQ      = out->ext[out->q];
            const bool    mergeable = n >= 3 && n <= 4 && isPow2(extQ) && out->orderB[0] == out->q && out->orderB[1] != 0
                                   && out->sB[out->orderB[1]] == extQ;
            // and the same for A's contiguous mode and the mode after it in A ("merged p")
            const bool mergeableP = n >= 3 && n <= 4 && isPow2(out->ext[0]) && out->q != 1 && out->sA[1] == out->ext[0];
            bool tma = ((typeA == CUDA_R_32F && typeB == CUDA_R_32F) || (typeA == CUDA_R_16F && typeB == CUDA_R_16F))
                       && pointersAligned16 && n <= 5 && out->ext[0] % per16 == 0 && extQ % per16 == 0
                       && (out->ext[0] >= 4 * per16 || mergeableP) && (extQ >= 4 * per16 || mergeable);
            for(int i = 0; i < n && tma; i++)
            {
                // cuTensorMapEncodeTiled limits: extent < 2^32, byte stride < 2^40
                if(out->ext[i] >= (int64_t(1) << 32) || out->sA[i] * out->elemSize >= (int64_t(1) << 40)
                   || out->sB[i] * out->elemSize >= (int64_t(1) << 40))
                    tma = false;
            }
            out->kind = tma ? PERM_TMA : PERM_TILE;
        }
        return PLAN_OK;
    }

    std::string describe(const PermPlan& p)
    {
        static const char* kinds[] = {"copy", "tile", "tma"};
        std::string        s       = "permutation kind=";
        s += kinds[p.kind];
        char buf[128];
        snprintf(buf, sizeof(buf), " ndim=%d q=%d total=%lld dims=", p.ndim, p.q, (long long)p.total);
        s += buf;
        for(int i = 0; i < p.ndim; i++)
        {
            snprintf(buf, sizeof(buf), "%s%lld:%lld/%lld", i ? " " : "", (long long)p.ext[i], (long long)p.sA[i],
                     (long long)p.sB[i]);
            s += buf;
        }
        return s;
    }

    // ------------------------------------------------------------------ reduction
    int planReduction(int rankA, const int64_t* lensA, const int64_t* stridesA, const int32_t* modeA, int rankD,
                      const int64_t* lensD, const int64_t* stridesD, const int32_t* modeD, int elemSize,
                      bool pointersAligned16, int smCount, ReducePlan* out)
    {
        std::memset(out, 0, sizeof(*out));
        if(rankA < 1 || rankA > kMaxGroup || rankD < 0 || rankD > rankA || !lensA || !stridesA || !modeA)
            return PLAN_INVALID;
        if(rankD > 0 && (!lensD || !stridesD || !modeD))
            return PLAN_INVALID;
        if(hasDuplicates(modeA, rankA) || hasDuplicates(modeD, rankD))
            return PLAN_INVALID;
        for(int j = 0; j < rankD; j++)
            if(findMode(modeA, rankA, modeD[j]) < 0)
                return PLAN_NOT_SUPPORTED; // modes of D must be a subset of A's

        ModeDim keep[kMaxGroup], red[kMaxGroup];
        int     nk = 0, nr = 0;
        for(int i = 0; i < rankA; i++)
        {
            if(lensA[i] <= 0)
                return PLAN_INVALID;
            if(findMode(modeD, rankD, modeA[i]) >= 0)
            {
                // positional contract of the reference: D's j-th extent/stride belongs to
                // the j-th kept mode of A (reduction_solution_impl.hpp:105-143)
                if(lensD[nk] != lensA[i])
                    return PLAN_INVALID;
                keep[nk] = ModeDim{lensA[i], stridesA[i], stridesD[nk]};
                nk++;
            }
            else
            {
                red[nr++] = ModeDim{lensA[i], stridesA[i], 0};
            }
        }
        auto byS0 = [](const ModeDim& a, const ModeDim& b) { return a.s0 < b.s0; };
        sortSmall(keep, nk, byS0);
        sortSmall(red, nr, byS0);
        nk = foldGroup(keep, nk);
        nr = foldGroup(red, nr);
        out->nk   = nk;
        out->nr   = nr;
        out->nOut = 1;
        out->nRed = 1;
        for(int i = 0; i < nk; i++)
        {
            out->kext[i] = keep[i].ext;
            out->ksA[i]  = keep[i].s0;
            out->ksD[i]  = keep[i].s1;
            out->nOut *= keep[i].ext;
        }
        for(int i = 0; i < nr; i++)
        {
            out->rext[i] = red[i].ext;
            out->rsA[i]  = red[i].s0;
            out->nRed *= red[i].ext;
        }
        const bool redContig  = (out->rext[0] > 1 && out->rsA[0] == 1);
        const bool keepContig = (out->kext[0] > 1 && out->ksA[0] == 1);
        out->kind             = redContig ? RED_ROW : (keepContig ? RED_COL : RED_GENERIC);
        if(out->nRed == 1 && out->kind == RED_GENERIC && out->nOut > 1)
            out->kind = keepContig ? RED_COL : RED_GENERIC;

        // vector width along the contiguous reduced axis (row kernel only)
        out->vec = 1;
        if(out->kind == RED_ROW && pointersAligned16)
        {
            int v = 16 / elemSize;
            for(; v > 1; v >>= 1)
            {
                bool ok = (out->rext[0] % v == 0);
                for(int i = 1; i < nr && ok; i++)
                    ok = (out->rsA[i] % v == 0);
                for(int i = 0; i < nk && ok; i++)
                    ok = (out->kext[i] == 1) || (out->ksA[i] % v == 0);
                if(ok)
                    break;
            }
            out->vec = v;
        }
        // A short contiguous reduced row: one load per lane covers it, 1 to 32 lanes per output; up to 2 KiB a few loads.
        out->shortLanes = 0;
        out->shortVec   = 1;
        if(out->kind == RED_ROW)
        {
            const int     v     = std::max(out->vec, 1); // a power of two up to 16 bytes
            const int64_t loads = (out->rext[0] + v - 1) / v;
            // rows of up to 2 KiB with further reduced modes, or without full vectors, take a warp per output here too
            // (several loads per lane); full vectors and no further reduced mode keep the row kernel's eight lanes
            const bool medium = out->rext[0] * int64_t(elemSize) <= 2048 && !(v == 16 / elemSize && nr == 1);
            if(loads <= 16 || medium)
            {
                // one load per lane up to 16 loads; beyond, eight per lane
                const int64_t lanes = loads <= 16 ? loads : (loads + 7) / 8;
                int           g     = 1;
                while(g < lanes && g < 32)
                    g <<= 1;
                out->shortLanes = g;
                out->shortVec   = v;
            }
        }
        // Few outputs and a long reduction: cut the reduced range into slices so that the
        // whole GPU works on it (two passes through a scratch buffer).
        out->split         = 1;
        out->splitOptional = 0;
        // A contiguous kept mode: threads along the outputs (16-byte loads when extents, strides and pointers allow), the
        // rest of the block along the innermost reduced mode. Few outputs leave few blocks: slices make up for them.
        out->colVec = out->colTx = out->colTy = 1;
        if(out->kind == RED_COL)
        {
            const int full = 16 / elemSize;
            bool      vecOk = full > 1 && pointersAligned16 && out->ksA[0] == 1 && out->kext[0] % full == 0;
            for(int d = 1; d < nk && vecOk; d++)
                vecOk = out->ksA[d] % full == 0;
            for(int d = 0; d < nr && vecOk; d++)
                vecOk = out->rsA[d] % full == 0;
            out->colVec         = vecOk ? full : 1;
            const int64_t units = out->nOut / out->colVec;
            // Lanes first along the contiguous kept run (kext[0]: neighbours were folded into it). When the innermost
            // reduced mode follows that run without a gap, the next lanes go along it (neighbouring rows are
            // neighbouring memory); what is left of the block takes further outputs.
            // (Runs below a 32-byte sector do better with all lanes on outputs: a thread's next rows are in the sectors
            // that its warp has just fetched. 0.7 against 1.5 TB/s with a run of four f16.)
            const bool    rowsAdjacent = out->rsA[0] == out->kext[0] && out->kext[0] * int64_t(elemSize) >= 32;
            int           tx           = 1;
            while(tx < 256 && tx < (rowsAdjacent ? out->kext[0] / out->colVec : units))
                tx <<= 1;
            // lanes along the innermost reduced mode: what the outputs leave of the block, at most its extent, and at
            // least eight loads per thread (a short reduction is cheaper without the exchange through shared memory)
            // (four loads in flight per thread come from one pass over that mode: a quarter of its extent at most)
            int ty = 256 / tx;
            while(ty > 1 && (ty * 4 > out->rext[0] || out->nRed / ty < 8))
                ty >>= 1;
            while(tx * ty < 256 && tx < units)
                tx <<= 1;
            out->colTx = tx;
            out->colTy = ty;
            const int64_t blocks = (units + tx - 1) / tx;
            if(smCount > 0 && blocks < int64_t(smCount) * 2)
            {
                const int64_t want  = (int64_t(smCount) * 4 + blocks - 1) / blocks;
                const int64_t maxBy = out->nRed / (int64_t(ty) * 16); // sixteen loads per thread at least
                out->split          = int(std::max<int64_t>(1, std::min<int64_t>(std::min(want, maxBy), 1024)));
                out->splitOptional  = out->split > 1 && out->nOut >= int64_t(smCount) * 4;
            }
        }
        else if(smCount > 0 && out->nOut < int64_t(smCount) * 4 && out->nRed >= 16384 && out->shortLanes == 0)
        {
            int64_t want  = (int64_t(smCount) * 8 + out->nOut - 1) / out->nOut;
            int64_t maxBy = out->nRed / 4096;
            out->split    = int(std::max<int64_t>(1, std::min<int64_t>(std::min(want, maxBy), 1024)));
        }
        // The short-row kernel has few lanes per output and needs many outputs to fill the GPU; with fewer, slices of
        // the outer reduced modes supply the threads.
        if(smCount > 0 && out->split == 1 && out->shortLanes > 0)
        {
            const int64_t lanes   = out->shortLanes;
            const int64_t threads = out->nOut * lanes;
            const int64_t outer   = out->rext[0] > 0 ? out->nRed / out->rext[0] : 1; // outer reduced iterations
            if(threads < int64_t(smCount) * 1024 && outer >= 64)
            {
                const int64_t want = (int64_t(smCount) * 2048 + threads - 1) / threads;
                out->split         = int(std::max<int64_t>(1, std::min<int64_t>(std::min(want, outer / 16), 1024)));
                out->splitOptional = out->split > 1;
            }
        }
        return PLAN_OK;
    }

    std::string describe(const ReducePlan& p)
    {
        static const char* kinds[] = {"row", "col", "generic"};
        std::string        s       = "reduction kind=";
        s += kinds[p.kind];
        char buf[128];
        snprintf(buf, sizeof(buf), " vec=%d split=%d nOut=%lld nRed=%lld keep=[", p.vec, p.split,
                 (long long)p.nOut, (long long)p.nRed);
        s += buf;
        for(int i = 0; i < p.nk; i++)
        {
            snprintf(buf, sizeof(buf), "%s%lld:%lld/%lld", i ? " " : "", (long long)p.kext[i],
                     (long long)p.ksA[i], (long long)p.ksD[i]);
            s += buf;
        }
        s += "] red=[";
        for(int i = 0; i < p.nr; i++)
        {
            snprintf(buf, sizeof(buf), "%s%lld:%lld", i ? " " : "", (long long)p.rext[i], (long long)p.rsA[i]);
            s += buf;
        }
        s += "]";
        if(p.shortLanes > 0)
        {
            snprintf(buf, sizeof(buf), " short=%dx%d", p.shortLanes, p.shortVec);
            s += buf;
        }
        if(p.kind == RED_COL)
        {
            snprintf(buf, sizeof(buf), " col=%dx%d vec=%d", p.colTx, p.colTy, p.colVec);
            s += buf;
        }
        if(p.splitOptional)
            s += " optional-split";
        return s;
    }

    // ------------------------------------------------------------------ contraction
    namespace
    {
        // two more modes than the interface allows: the real view of a complex tensor has one mode more, its
        // expanded copy two (planComplexContraction)
        constexpr int kPlanRank = kMaxRank + 2;
        int planReal(const TensorView& A, const TensorView& B, const TensorView& D, int typeC, bool bilinear,
                     int computeType, int smCount, int rankLimit, ContractionPlan* out);
    } // namespace

    int planContraction(const TensorView& A, const TensorView& B, const TensorView& D, int typeC, bool bilinear,
                        int computeType, int smCount, ContractionPlan* out, uint64_t workspaceLimit)
    {
        const int rc = planReal(A, B, D, typeC, bilinear, computeType, smCount, kMaxRank, out);
        if(rc != PLAN_OK || workspaceLimit == 0)
            return rc;
        // Operands that the f16 tensor-core kernel reads in place but in mostly empty pieces are packed too: an MN-major
        // operand is cut into 64-element chunks of its stride-1 mode, K into blocks of 64 along the block mode, and a mode
        // of 16 or 48 elements fills a quarter or three quarters of each (configuration 5's layout with f16 data: 0.14
        // of the MMA work is useful).
        double fill = 1.0;
        if(out->kind == CK_TCGEN05)
        {
            auto chunkFill = [](int64_t e) { return double(e) / double((e + 63) / 64 * 64); };
            if(out->aMajor == 1)
                fill *= chunkFill(out->m[0].ext);
            if(out->bMajor == 1)
                fill *= chunkFill(out->n[out->nFast].ext);
            fill *= chunkFill(out->k[0].ext);
        }
        // (The copies cost about 3200 / min(M, N) times the packed contraction's own time: they pay from a quarter of
        // useful work down, on outputs of a thousand rows and columns or more.)
        const bool sparse = out->kind == CK_TCGEN05 && fill < 0.25 && out->M >= 1024 && out->N >= 1024;
        if(out->kind != CK_TILED_SIMT && !sparse)
            return rc;
        // The gathered FMA kernel reads anything but runs at a fiftieth of the tensor cores' rate. From about a GFLOP
        // on, two passes that copy the operands into packed matrices (contracted modes merged and innermost, rows
        // padded to 16 bytes) cost less than they save.
        const bool tensorType = A.type == CUDA_R_16F || A.type == CUDA_R_16BF || A.type == CUDA_R_32F;
        // ... and under a long contraction whatever the size: the FMA kernel's tiles walk K at about 0.1 us per element
        // (100 x 30 x 8192: 763 us against 10 us of copies and 37 us on a ragged tensor-core tile).
        const bool large = out->M >= 128 && out->N >= 128 && out->K >= 64
                           && 2.0 * double(out->M) * double(out->N) * double(out->K) >= 1e9;
        const bool longK = out->K >= 1024 && out->M >= 16 && out->N >= 16;
        if(!tensorType || !(large || (longK && !sparse)))
            return rc;
        const int elem = A.type == CUDA_R_32F ? 4 : 2, per16 = 16 / elem;
        int       freeA[kMaxRank], freeB[kMaxRank], conA[kMaxRank], conB[kMaxRank], nfa = 0, nfb = 0, nc = 0;
        for(int i = 0; i < A.rank; i++)
        {
            const int ib = findMode(B.modes, B.rank, A.modes[i]);
            if(ib >= 0)
            {
                conA[nc] = i;
                conB[nc] = ib;
                nc++;
            }
            else
                freeA[nfa++] = i;
        }
        for(int i = 0; i < B.rank; i++)
            if(findMode(A.modes, A.rank, B.modes[i]) < 0)
                freeB[nfb++] = i;
        if(nc == 0 || nfa == 0 || nfb == 0 || nfa + 1 > kMaxRank || nfb + 1 > kMaxRank)
            return rc;
        // the rows of a copy follow D's order (slowest mode of D first): free modes that are neighbours in D are
        // neighbours in the copy and fold into one mode of the row group
        auto strideInD = [&](const TensorView& T, int pos) {
            const int id = findMode(D.modes, D.rank, T.modes[pos]);
            return id >= 0 ? D.strides[id] : int64_t(0);
        };
        sortSmall(freeA, nfa, [&](int x, int y) { return strideInD(A, x) > strideInD(A, y); });
        sortSmall(freeB, nfb, [&](int x, int y) { return strideInD(B, x) > strideInD(B, y); });
        int64_t K = 1;
        for(int i = 0; i < nc; i++)
            K *= A.lens[conA[i]];
        const int64_t Kp = (K + per16 - 1) / per16 * per16;
        // a label for the merged contracted mode that no tensor uses
        int32_t kLabel = 0;
        for(bool clash = true; clash; )
        {
            clash = findMode(A.modes, A.rank, kLabel) >= 0 || findMode(B.modes, B.rank, kLabel) >= 0
                    || findMode(D.modes, D.rank, kLabel) >= 0;
            if(clash)
                kLabel++;
        }
        int64_t lA[kMaxRank], sA[kMaxRank], lB[kMaxRank], sB[kMaxRank];
        int32_t mA[kMaxRank], mB[kMaxRank];
        int64_t rowsA = 1, rowsB = 1;
        lA[nfa] = Kp;
        sA[nfa] = 1;
        mA[nfa] = kLabel;
        for(int i = nfa - 1; i >= 0; i--)
        {
            lA[i] = A.lens[freeA[i]];
            mA[i] = A.modes[freeA[i]];
            sA[i] = (i == nfa - 1) ? Kp : sA[i + 1] * lA[i + 1];
            rowsA *= lA[i];
        }
        lB[nfb] = Kp;
        sB[nfb] = 1;
        mB[nfb] = kLabel;
        for(int i = nfb - 1; i >= 0; i--)
        {
            lB[i] = B.lens[freeB[i]];
            mB[i] = B.modes[freeB[i]];
            sB[i] = (i == nfb - 1) ? Kp : sB[i + 1] * lB[i + 1];
            rowsB *= lB[i];
        }
        const uint64_t bytesA = (uint64_t(rowsA) * uint64_t(Kp) * elem + 255u) & ~uint64_t(255);
        const uint64_t bytesB = (uint64_t(rowsB) * uint64_t(Kp) * elem + 255u) & ~uint64_t(255);
        if(bytesA + bytesB + 256 > workspaceLimit)
            return rc;
        const TensorView A2{nfa + 1, lA, sA, mA, A.type}, B2{nfb + 1, lB, sB, mB, B.type};
        ContractionPlan  packed;
        if(planReal(A2, B2, D, typeC, bilinear, computeType, smCount, kMaxRank, &packed) != PLAN_OK
           || (packed.kind != CK_TCGEN05 && packed.kind != CK_TF32X3))
            return rc;
        packed.packReal = 1;
        packed.packK    = K;
        packed.packKp   = Kp;
        packed.xRank    = nfa + nc;
        packed.xFree    = nfa;
        packed.yRank    = nfb + nc;
        packed.yFree    = nfb;
        if(packed.xRank > kMaxRank || packed.yRank > kMaxRank)
            return rc;
        for(int i = 0; i < nfa; i++)
        {
            packed.xExt[i]    = A.lens[freeA[i]];
            packed.xStride[i] = A.strides[freeA[i]];
        }
        for(int i = 0; i < nfb; i++)
        {
            packed.yExt[i]    = B.lens[freeB[i]];
            packed.yStride[i] = B.strides[freeB[i]];
        }
        for(int i = 0; i < nc; i++)
        {
            packed.xExt[nfa + i]    = A.lens[conA[i]];
            packed.xStride[nfa + i] = A.strides[conA[i]];
            packed.yExt[nfb + i]    = B.lens[conB[i]];
            packed.yStride[nfb + i] = B.strides[conB[i]];
        }
        packed.yOffset     = bytesA;
        packed.expandBytes = bytesA + bytesB + 256; // the copies start at the next multiple of 256 bytes in the workspace
        if(packed.expandBytes + packed.workspaceBytes > workspaceLimit)
            packed.workspaceBytes = 0;
        *out = packed;
        return PLAN_OK;
    }

    namespace
    {
    int planReal(const TensorView& A, const TensorView& B, const TensorView& D, int typeC, bool bilinear,
                 int computeType, int smCount, int rankLimit, ContractionPlan* out)
    {
        std::memset(out, 0, sizeof(*out));
        if(A.rank < 1 || B.rank < 1 || D.rank < 1 || A.rank > rankLimit || B.rank > rankLimit
           || D.rank > rankLimit)
            return PLAN_INVALID;
        if(hasDuplicates(A.modes, A.rank) || hasDuplicates(B.modes, B.rank) || hasDuplicates(D.modes, D.rank))
            return PLAN_INVALID;

        // ---- type tuples of the reference (contraction_solution_instances.cpp:36-284,
        //      contraction_cpu_reference_instances.cpp:32-298) plus f16/bf16 inputs with f32 output
        const int  tA = A.type, tB = B.type, tD = D.type;
        const bool half = (tA == CUDA_R_16F || tA == CUDA_R_16BF);
        bool       ok   = false;
        if(tA == tB)
        {
            if(half && computeType == 4 /*32F*/ && (tD == tA || tD == CUDA_R_32F))
                ok = true;
            if(tA == CUDA_R_32F && tD == CUDA_R_32F
               && (computeType == 4 || computeType == 1 /*16F*/ || computeType == 1024 /*16BF*/))
                ok = true;
            if(tA == CUDA_R_64F && tD == CUDA_R_64F && (computeType == 16 /*64F*/ || computeType == 4))
                ok = true;
        }
        if(bilinear && typeC != tD)
            ok = false;
        if(!ok)
            return PLAN_NOT_SUPPORTED;

        ModeDim gm[kPlanRank], gn[kPlanRank], gk[kPlanRank];
        int     nm = 0, nn = 0, nk = 0;
        for(int i = 0; i < D.rank; i++)
        {
            if(D.lens[i] <= 0)
                return PLAN_INVALID;
            int ia = findMode(A.modes, A.rank, D.modes[i]);
            int ib = findMode(B.modes, B.rank, D.modes[i]);
            if(ia >= 0 && ib >= 0)
                return PLAN_NOT_SUPPORTED; // batch mode (the reference mis-classifies it)
            if(ia >= 0)
            {
                if(A.lens[ia] != D.lens[i])
                    return PLAN_INVALID;
                gm[nm++] = ModeDim{A.lens[ia], A.strides[ia], D.strides[i]};
            }
            else if(ib >= 0)
            {
                if(B.lens[ib] != D.lens[i])
                    return PLAN_INVALID;
                gn[nn++] = ModeDim{B.lens[ib], B.strides[ib], D.strides[i]};
            }
            else
                return PLAN_INVALID; // a mode of D that neither A nor B carries
        }
        for(int i = 0; i < A.rank; i++)
        {
            if(A.lens[i] <= 0)
                return PLAN_INVALID;
            int ib = findMode(B.modes, B.rank, A.modes[i]);
            int id = findMode(D.modes, D.rank, A.modes[i]);
            if(ib >= 0)
            {
                if(A.lens[i] != B.lens[ib])
                    return PLAN_INVALID;
                gk[nk++] = ModeDim{A.lens[i], A.strides[i], B.strides[ib]};
            }
            else if(id < 0)
                return PLAN_INVALID; // a mode of A that is neither contracted nor kept
        }
        for(int i = 0; i < B.rank; i++)
        {
            if(B.lens[i] <= 0)
                return PLAN_INVALID;
            if(findMode(A.modes, A.rank, B.modes[i]) < 0 && findMode(D.modes, D.rank, B.modes[i]) < 0)
                return PLAN_INVALID;
        }
        // ---- make D contiguous along N when it is contiguous along some M mode
        int64_t minM = INT64_MAX, minN = INT64_MAX;
        for(int i = 0; i < nm; i++)
            if(gm[i].ext > 1)
                minM = std::min(minM, gm[i].s1);
        for(int i = 0; i < nn; i++)
            if(gn[i].ext > 1)
                minN = std::min(minN, gn[i].s1);
        out->swapped = (minM < minN) ? 1 : 0;
        if(out->swapped)
        {
            std::swap_ranges(gm, gm + kPlanRank, gn);
            std::swap(nm, nn);
            for(int i = 0; i < nk; i++)
                std::swap(gk[i].s0, gk[i].s1);
        }
        out->typeA = out->swapped ? tB : tA;
        out->typeB = out->swapped ? tA : tB;
        out->typeC = bilinear ? typeC : -1;
        out->typeD = tD;
        out->computeType = computeType;
        out->bilinear    = bilinear ? 1 : 0;

        // ---- order and fold: M by its stride in A, N by its stride in D, K by its stride in A
        sortSmall(gm, nm, [](const ModeDim& a, const ModeDim& b) { return a.s0 < b.s0; });
        sortSmall(gn, nn, [](const ModeDim& a, const ModeDim& b) { return a.s1 < b.s1; });
        sortSmall(gk, nk, [](const ModeDim& a, const ModeDim& b) { return a.s0 < b.s0; });
        nm = foldGroup(gm, nm);
        nn = foldGroup(gn, nn);
        nk = foldGroup(gk, nk);
        if(nm > kMaxGroup || nn > kMaxGroup || nk > kMaxGroup)
            return PLAN_NOT_SUPPORTED; // the reference's limit of six modes per group, applied after folding
        out->nm = nm;
        out->nn = nn;
        out->nk = nk;
        out->M = out->N = out->K = 1;
        for(int i = 0; i < nm; i++)
        {
            out->m[i] = gm[i];
            out->M *= gm[i].ext;
        }
        for(int i = 0; i < nn; i++)
        {
            out->n[i] = gn[i];
            out->N *= gn[i].ext;
        }
        for(int i = 0; i < nk; i++)
        {
            out->k[i] = gk[i];
            out->K *= gk[i].ext;
        }

        out->aKContig = (nk == 1 && gk[0].s0 == 1) ? 1 : 0;
        out->bKContig = (nk == 1 && gk[0].s1 == 1) ? 1 : 0;
        out->splitK   = 1;
        out->workspaceBytes = 0;

        // ---- kernel family
        if(tA == CUDA_R_64F && (computeType == 16 || computeType == 4))
        {
            // f64 data. Compute type f32 (a reference tuple, contraction_solution_instances.cpp:124-146) asks for
            // accumulation in AT LEAST single precision: the FP64 tensor pipe gives more at 1.7 times the rate of the
            // fp32 FMA kernel, which first rounds every element to float (results agree to the float rounding the
            // reference itself commits, far inside its 1e-5 criterion).
            out->kind = CK_TILED_DMMA;
        }
        else if(half)
        {
            // tcgen05 path. The K group may keep several folded modes (the reference's kernels take up to six,
            // contraction_meta_traits.hpp:41-43): a 64-wide K block runs along ONE of them, the block mode kf, at
            // one index of each of the others (at most two others fit the five dimensions of a tensor map beside the
            // row modes). An operand is taken K-major (stride 1 along kf, rows gathered by a TMA box over the folded
            // modes of its row group) or MN-major (a stride-1 mode in its row group, rows taken in 64-element chunks
            // of that mode). All other strides must be multiples of 16 bytes. Among the K modes that give both
            // operands a form, the one with more K-major operands wins, then the longer one.
            int nFastB = -1;
            for(int i = 0; i < nn && nFastB < 0; i++)
                if(gn[i].s0 == 1 && gn[i].ext > 1)
                    nFastB = i;
            const bool aMn = gm[0].s0 == 1 && gm[0].ext > 1;
            int        kf = -1, kfScore = -1;
            for(int f = 0; f < nk; f++)
            {
                const int am = gk[f].s0 == 1 ? 0 : (aMn ? 1 : -1), bm = gk[f].s1 == 1 ? 0 : (nFastB >= 0 ? 1 : -1);
                if(am < 0 || bm < 0 || (nk > 1 && gk[f].ext < 16))
                    continue;
                const int score = (am == 0) + (bm == 0);
                if(score > kfScore || (score == kfScore && gk[f].ext > gk[kf].ext))
                {
                    kf      = f;
                    kfScore = score;
                }
            }
            out->aMajor = out->bMajor = -1;
            out->nFast  = 0;
            if(kf >= 0)
            {
                // the block mode goes first, the others keep their order
                const ModeDim block = gk[kf];
                for(int i = kf; i > 0; i--)
                    gk[i] = gk[i - 1];
                gk[0] = block;
                for(int i = 0; i < nk; i++)
                    out->k[i] = gk[i];
                out->aMajor = gk[0].s0 == 1 ? 0 : 1;
                out->bMajor = gk[0].s1 == 1 ? 0 : 1;
                if(out->bMajor == 1)
                    out->nFast = nFastB;
            }
            out->aKContig = out->aMajor == 0 ? 1 : 0;
            out->bKContig = out->bMajor == 0 ? 1 : 0;
            const int kOthers = nk - 1;
            // a short contraction under a large output is bound by the stores of D: the K block's zero-filled tail costs MMA
            // steps that hide behind them (8192 x 8192 x 8: 0.33 ms on the FMA kernel)
            const bool bigOutput = double(out->M) * double(out->N) >= double(1 << 22);
            bool tc = out->aMajor >= 0 && out->bMajor >= 0 && (out->K >= 64 || (out->K >= 8 && bigOutput)) && kOthers <= 2 && nm + kOthers <= 4
                      && nn + kOthers <= 4 && nm <= (out->aMajor == 1 ? 3 : 4) && nn <= (out->bMajor == 1 ? 3 : 4);
            if(tc && nk == 1 && (out->aMajor == 0 || out->bMajor == 0))
                tc = out->K % 8 == 0;
            if(tc && out->aMajor == 1)
                tc = gk[0].s0 % 8 == 0;
            if(tc && out->bMajor == 1)
                tc = gk[0].s1 % 8 == 0;
            for(int i = 0; i < nk && tc; i++)
                tc = gk[i].ext < (int64_t(1) << 31) && (i == 0 || (gk[i].s0 % 8 == 0 && gk[i].s1 % 8 == 0));
            for(int i = 0; i < nm && tc; i++)
                tc = ((gm[i].s0 % 8 == 0 || (out->aMajor == 1 && i == 0)) && gm[i].ext < (int64_t(1) << 31));
            for(int i = 0; i < nn && tc; i++)
                tc = ((gn[i].s0 % 8 == 0 || (out->bMajor == 1 && i == out->nFast)) && gn[i].ext < (int64_t(1) << 31));
            // small problems do not fill the machine with 128-row tiles: leave them to the
            // gathered tiled kernel
            // (except under a long contraction: a single FMA tile walks K = 65536 in 6.5 ms, a ragged tensor-core tile
            // with its K range cut over a cluster in tens of microseconds)
            tc = tc && ((out->M >= 128 && out->N >= 64) || (out->K >= 1024 && out->M >= 16 && out->N >= 16));
            if(tc)
            {
                out->tileM = 128;
                out->tileK = 64;
                out->rowsM = out->aMajor ? 128 : boxDecompose(gm, nm, 128, out->boxM);
                out->rowsN = 0;
                // the widest tile that still gives half of the SMs one (small problems are latency bound: more,
                // smaller tiles shorten the loads and the epilogue of each CTA)
                const int64_t smsH = smCount > 0 ? smCount : 148;
                int           tn0  = out->N >= 256 ? 256 : (out->N >= 128 ? 128 : 64);
                while(tn0 > 64 && ((out->M + 127) / 128) * ((out->N + tn0 - 1) / tn0) < smsH / 2)
                    tn0 >>= 1;
                for(int tn = tn0; tn >= 64 && out->rowsN == 0; tn >>= 1)
                {
                    out->tileN = tn;
                    out->rowsN = out->bMajor ? tn : boxDecompose(gn, nn, tn, out->boxN);
                }
                tc = out->rowsM > 0 && out->rowsN > 0;
                out->stages = (out->tileN == 256) ? 4 : 6;
                // large problems: 256 x 256 tiles over CTA pairs
                out->rowsN128 = out->bMajor ? 128 : boxDecompose(gn, nn, 128, out->boxN128);
                // (possible from 512 x 512 on; they pay off once the 256 x 256 tiles occupy most of the CTA pairs:
                // measured with K = 4096, 32 tiles 34 us on single CTAs against 47 on pairs, 64 tiles 40 against 40,
                // 128 tiles 71 against 63, 256 tiles 124 against 106)
                out->pairOk = (tc && out->N >= 256 && out->rowsN128 == 128 && out->rowsM == 128 && out->M >= 512
                               && out->N >= 512)
                                  ? 1
                                  : 0;
                out->pair   = 0;
                out->wide   = 0;
                out->ksplit = 1;
                if(out->pairOk)
                    pairKernelForm(out->M, out->N, out->K, int(smsH), &out->pair, &out->wide, &out->ksplit);
            }
            out->kind = tc ? CK_TCGEN05 : CK_TILED_SIMT;
        }
        else if(tA == CUDA_R_32F && (computeType == 4 || computeType == 1 || computeType == 1024))
        {
            // fp32 data on the tensor cores (compute f32: TF32 big/small split; compute f16 / bf16: elements
            // rounded to that type, one MMA). An operand is taken K-major (one stride-1 K mode) or MN-major (a
            // stride-1 mode in its row group); all other strides must be multiples of 16 bytes for TMA.
            const bool bigOutput = double(out->M) * double(out->N) >= double(1 << 22);
            bool tf = (out->K >= 32 || (out->K >= 4 && bigOutput)) && ((out->M >= 128 && out->N >= 64) || (out->K >= 1024 && out->M >= 16 && out->N >= 16))
                      && nk <= 2;
            out->aMajor = out->aKContig ? 0 : ((gm[0].s0 == 1 && gm[0].ext > 1) ? 1 : -1);
            out->bMajor = out->bKContig ? 0 : -1;
            out->nFast  = 0;
            for(int i = 0; i < nn && out->bMajor < 0; i++)
                if(gn[i].s0 == 1 && gn[i].ext > 1)
                {
                    out->bMajor = 1;
                    out->nFast  = i;
                }
            tf = tf && out->aMajor >= 0 && out->bMajor >= 0;
            auto stridesOk = [](const ModeDim* g, int n, int skip) {
                for(int i = 0; i < n; i++)
                    if(i != skip && g[i].ext > 1 && (g[i].s0 % 4 != 0 || g[i].ext >= (int64_t(1) << 31)))
                        return false;
                return true;
            };
            if(tf)
            {
                tf = stridesOk(gm, nm, out->aMajor ? 0 : -1) && stridesOk(gn, nn, out->bMajor ? out->nFast : -1);
                tf = tf && nm <= (out->aMajor ? 3 : 4) && nn <= (out->bMajor ? 3 : 4);
                for(int i = 0; i < nm && tf; i++)
                    tf = gm[i].ext < (int64_t(1) << 31);
                for(int i = 0; i < nn && tf; i++)
                    tf = gn[i].ext < (int64_t(1) << 31);
            }
            if(tf)
            {
                out->boxK[0] = 32;
                out->boxK[1] = 1;
                if(out->aMajor || out->bMajor)
                {
                    int bk[kMaxGroup] = {1, 1, 1, 1, 1, 1};
                    tf = boxDecompose(gk, nk, 32, bk) == 32;
                    out->boxK[0] = bk[0];
                    out->boxK[1] = bk[1];
                    for(int i = 0; i < nk && tf; i++)
                        tf = (!out->aMajor || gk[i].s0 % 4 == 0) && (!out->bMajor || gk[i].s1 % 4 == 0)
                             && gk[i].ext < (int64_t(1) << 31);
                }
            }
            if(tf)
            {
                out->tileM = 128;
                out->tileK = 32;
                // 128 x 128 tiles; 128 x 64 when those would leave SMs without a tile (576^3: 34 us instead of 39,
                // 1024^3: 47 instead of 60)
                out->tileN = out->N >= 128 ? 128 : 64;
                if(((out->M + 127) / 128) * ((out->N + 127) / 128) < int64_t(smCount > 0 ? smCount : 148))
                    out->tileN = 64;
                out->rowsM = out->aMajor ? 128 : boxDecompose(gm, nm, 128, out->boxM);
                out->rowsN = out->bMajor ? out->tileN : boxDecompose(gn, nn, out->tileN, out->boxN);
                if(out->rowsN == 0 && out->tileN == 128)
                {
                    out->tileN = 64;
                    out->rowsN = boxDecompose(gn, nn, 64, out->boxN);
                }
                tf          = out->rowsM > 0 && out->rowsN > 0;
                out->stages = 2;
                // CTA pairs work on 256 x 128 tiles, each CTA loading 64 rows of B
                out->rowsN128 = out->bMajor ? 64 : boxDecompose(gn, nn, 64, out->boxN128);
                out->pair     = (tf && out->N >= 128 && out->rowsM == 128 && out->rowsN128 == 64 && out->M >= 256) ? 1 : 0;
            }
            if(tf)
            {
                // Small problems: cut every tile into ranges of K blocks so that more SMs work (the per-CTA chain of K
                // blocks, each paying the ring latency, is what bounds them). All work units must be resident at once.
                int64_t tilesM = 1, tilesN = 1, kBlocks = (out->K + 31) / 32;
                if(out->aMajor)
                    tilesM = (((gm[0].ext + 31) / 32) * (out->M / gm[0].ext) + 3) / 4;
                else
                    for(int i = 0; i < nm; i++)
                        tilesM *= (gm[i].ext + out->boxM[i] - 1) / out->boxM[i];
                if(out->bMajor)
                {
                    const int64_t per = out->tileN / 32;
                    tilesN            = (((gn[out->nFast].ext + 31) / 32) * (out->N / gn[out->nFast].ext) + per - 1) / per;
                }
                else
                    for(int i = 0; i < nn; i++)
                        tilesN *= (gn[i].ext + out->boxN[i] - 1) / out->boxN[i];
                if(out->aMajor || out->bMajor)
                {
                    kBlocks = 1;
                    for(int i = 0; i < nk; i++)
                        kBlocks *= (gk[i].ext + out->boxK[i < 2 ? i : 1] - 1) / out->boxK[i < 2 ? i : 1];
                }
                const int64_t sms   = smCount > 0 ? smCount : 148;
                const int64_t tiles = tilesM * tilesN;
                int           parts = int(std::min<int64_t>(std::min<int64_t>(4, sms / std::max<int64_t>(tiles, 1)), kBlocks / 4));
                if(parts >= 2)
                    out->splitK = parts; // a cluster of `parts` CTAs per tile; the sums meet in shared memory: no scratch
            }
            out->kind = tf ? CK_TF32X3 : CK_TILED_SIMT;
        }
        else
        {
            out->kind = CK_TILED_SIMT;
        }
        (void)smCount;
        return PLAN_OK;
    }
    } // namespace

    // Complex contraction as ONE real contraction. A complex tensor is, in memory, a real tensor with one more
    // mode c of extent 2 and stride 1 (all other strides doubled). With Y the operand that stays in place and X
    // the one that is copied,
    //   Re D = sum_k Yr Xr - Yi Xi      Im D = sum_k Yr Xi + Yi Xr
    // is the real contraction D'[.., cOut] = sum_{k, cK} Y'[.., k, cK] * X2[.., cOut, k, cK] with
    //   X2[.., 0, k, :] = (Xr, -Xi)     X2[.., 1, k, :] = (Xi, Xr),
    // i.e. M*2N*2K real multiply-adds, the same count as the four real contractions of the reference
    // (device_contraction_bilinear_complex.hpp:454-470), on the real tensor-core kernels, with no
    // split of Y or D into real and imaginary planes. X2 is packed: free modes of X (slowest, ordered by
    // their stride in D), cOut, the contracted modes (ordered by their stride in Y), cK (fastest).
    int planComplexContraction(const TensorView& A, const TensorView& B, const TensorView& D, int typeC, bool bilinear,
                               int computeType, int smCount, ContractionPlan* out)
    {
        std::memset(out, 0, sizeof(*out));
        if(A.rank < 1 || B.rank < 1 || D.rank < 1 || A.rank > kMaxRank || B.rank > kMaxRank || D.rank > kMaxRank)
            return PLAN_INVALID;
        if(hasDuplicates(A.modes, A.rank) || hasDuplicates(B.modes, B.rank) || hasDuplicates(D.modes, D.rank))
            return PLAN_INVALID;
        // reference tuples: cf32 with compute C32F, cf64 with compute C64F
        // (contraction_solution_instances.cpp:108-121,152-165,240-253,284-297)
        const bool c32 = A.type == CUDA_C_32F && computeType == 2048, c64 = A.type == CUDA_C_64F && computeType == 4096;
        if(!(c32 || c64) || B.type != A.type || D.type != A.type || (bilinear && typeC != A.type))
            return PLAN_NOT_SUPPORTED;
        const int realType = c32 ? CUDA_R_32F : CUDA_R_64F, realSize = c32 ? 4 : 8;
        int64_t   nA = 1, nB = 1;
        for(int i = 0; i < A.rank; i++)
            nA *= A.lens[i];
        for(int i = 0; i < B.rank; i++)
            nB *= B.lens[i];
        if(nA <= 0 || nB <= 0)
            return PLAN_INVALID;
        const bool        expandA = nA < nB; // copy the smaller operand
        const TensorView& X = expandA ? A : B;
        const TensorView& Y = expandA ? B : A;

        // two mode labels that no tensor uses
        int32_t fresh[2];
        {
            int32_t cand = 0x40000000;
            for(int f = 0; f < 2; f++, cand++)
            {
                while(findMode(A.modes, A.rank, cand) >= 0 || findMode(B.modes, B.rank, cand) >= 0
                      || findMode(D.modes, D.rank, cand) >= 0)
                    cand++;
                fresh[f] = cand;
            }
        }
        const int32_t cK = fresh[0], cOut = fresh[1];

        // X's modes in the copy's order: free modes by descending stride in D, then contracted modes by
        // descending stride in Y
        struct XMode
        {
            int     pos; // position in X
            int64_t key; // stride in D (free) or in Y (contracted)
        };
        XMode freeM[kMaxRank], conM[kMaxRank];
        int   nFree = 0, nCon = 0;
        for(int i = 0; i < X.rank; i++)
        {
            if(X.lens[i] <= 0)
                return PLAN_INVALID;
            const int iy = findMode(Y.modes, Y.rank, X.modes[i]);
            const int id = findMode(D.modes, D.rank, X.modes[i]);
            if(iy >= 0 && id >= 0)
                return PLAN_NOT_SUPPORTED; // batch mode
            if(iy >= 0)
                conM[nCon++] = XMode{i, Y.strides[iy]};
            else if(id >= 0)
                freeM[nFree++] = XMode{i, D.strides[id]};
            else
                return PLAN_INVALID;
        }
        auto byKey = [](const XMode& a, const XMode& b) { return a.key > b.key; };
        sortSmall(freeM, nFree, byKey);
        sortSmall(conM, nCon, byKey);

        // Y's modes for a packed copy: free modes by descending stride in D, contracted modes in the order of X2's
        XMode yFreeM[kMaxRank];
        int   nYFree = 0;
        for(int i = 0; i < Y.rank; i++)
        {
            if(Y.lens[i] <= 0)
                return PLAN_INVALID;
            if(findMode(X.modes, X.rank, Y.modes[i]) >= 0)
                continue;
            const int id = findMode(D.modes, D.rank, Y.modes[i]);
            if(id < 0)
                return PLAN_INVALID;
            yFreeM[nYFree++] = XMode{i, D.strides[id]};
        }
        sortSmall(yFreeM, nYFree, byKey);

        auto planWith = [&](bool copyY, ContractionPlan* plan) -> int {
        int64_t lX[kPlanRank], sX[kPlanRank], lY[kPlanRank], sY[kPlanRank], lD[kPlanRank], sD[kPlanRank];
        int32_t mX[kPlanRank], mY[kPlanRank], mD[kPlanRank];
        int     r = 0;
        for(int i = 0; i < nFree; i++, r++)
        {
            lX[r] = X.lens[freeM[i].pos];
            mX[r] = X.modes[freeM[i].pos];
        }
        lX[r]   = 2;
        mX[r++] = cOut;
        for(int i = 0; i < nCon; i++, r++)
        {
            lX[r] = X.lens[conM[i].pos];
            mX[r] = X.modes[conM[i].pos];
        }
        lX[r]   = 2;
        mX[r++] = cK;
        const int rankX2 = r;
        sX[rankX2 - 1]   = 1;
        for(int i = rankX2 - 2; i >= 0; i--)
            sX[i] = sX[i + 1] * lX[i + 1];
        int posY[kMaxRank]; // Y's modes in the copy's order
        if(copyY)
        {
            int q = 0;
            for(int i = 0; i < nYFree; i++)
                posY[q++] = yFreeM[i].pos;
            for(int i = 0; i < nCon; i++)
                posY[q++] = findMode(Y.modes, Y.rank, X.modes[conM[i].pos]);
            for(int i = 0; i < Y.rank; i++)
            {
                lY[i] = Y.lens[posY[i]];
                mY[i] = Y.modes[posY[i]];
            }
            sY[Y.rank] = 1;
            sY[Y.rank - 1] = 2;
            for(int i = Y.rank - 2; i >= 0; i--)
                sY[i] = sY[i + 1] * lY[i + 1];
        }
        else
        {
            for(int i = 0; i < Y.rank; i++)
            {
                lY[i] = Y.lens[i];
                sY[i] = 2 * Y.strides[i];
                mY[i] = Y.modes[i];
            }
            sY[Y.rank] = 1;
        }
        lY[Y.rank] = 2;
        mY[Y.rank] = cK;
        for(int i = 0; i < D.rank; i++)
        {
            lD[i] = D.lens[i];
            sD[i] = 2 * D.strides[i];
            mD[i] = D.modes[i];
        }
        lD[D.rank] = 2;
        sD[D.rank] = 1;
        mD[D.rank] = cOut;
        const TensorView X2{rankX2, lX, sX, mX, realType}, Y2{Y.rank + 1, lY, sY, mY, realType},
            D2{D.rank + 1, lD, sD, mD, realType};
        const int rc = planReal(expandA ? X2 : Y2, expandA ? Y2 : X2, D2, realType, bilinear, c32 ? 4 : 16, smCount,
                                kPlanRank, plan);
        if(rc != PLAN_OK)
            return rc;
        plan->complexKind = expandA ? 1 : 2;
        plan->xRank       = nFree + nCon;
        plan->xFree       = nFree;
        for(int i = 0; i < nFree; i++)
        {
            plan->xExt[i]    = X.lens[freeM[i].pos];
            plan->xStride[i] = X.strides[freeM[i].pos];
        }
        for(int i = 0; i < nCon; i++)
        {
            plan->xExt[nFree + i]    = X.lens[conM[i].pos];
            plan->xStride[nFree + i] = X.strides[conM[i].pos];
        }
        plan->dRank = D.rank;
        for(int i = 0; i < D.rank; i++)
        {
            plan->dExt[i]    = D.lens[i];
            plan->dStride[i] = D.strides[i];
        }
        const uint64_t bytes = uint64_t(expandA ? nA : nB) * 4u * uint64_t(realSize);
        plan->expandBytes     = (bytes + 255u) & ~uint64_t(255);
        if(copyY)
        {
            plan->yCopy   = 1;
            plan->yRank   = Y.rank;
            plan->yFree   = nYFree;
            plan->yOffset = plan->expandBytes;
            for(int i = 0; i < Y.rank; i++)
            {
                plan->yExt[i]    = Y.lens[posY[i]];
                plan->yStride[i] = Y.strides[posY[i]];
            }
            const uint64_t bytesY = uint64_t(expandA ? nB : nA) * 2u * uint64_t(realSize);
            plan->expandBytes += (bytesY + 255u) & ~uint64_t(255);
        }
        return PLAN_OK;
        };

        const int rc = planWith(false, out);
        if(rc != PLAN_OK)
            return rc;
        if(c32 && out->kind != CK_TF32X3)
        {
            // Y as it lies is neither K-major nor MN-major in its real view (e.g. first-mode-fastest strides: the
            // (re, im) pairs sit between consecutive rows). A packed copy with the contracted modes innermost
            // costs one pass over Y and puts the problem on the tensor cores.
            ContractionPlan alt;
            if(planWith(true, &alt) == PLAN_OK && alt.kind == CK_TF32X3)
                *out = alt;
        }
        return PLAN_OK;
    }

    std::string describe(const ContractionPlan& p)
    {
        static const char* kinds[] = {"tiled_simt", "tiled_dmma", "tcgen05", "tf32x3"};
        std::string        s       = p.complexKind ? "complex contraction (copy of " : "contraction kind=";
        if(p.complexKind)
        {
            char cb[96];
            snprintf(cb, sizeof(cb), "%s: %lld bytes) kind=", p.yCopy ? "A and B" : (p.complexKind == 1 ? "A" : "B"),
                     (long long)p.expandBytes);
            s += cb;
        }
        s += kinds[p.kind];
        char buf[192];
        snprintf(buf, sizeof(buf), " M=%lld N=%lld K=%lld types=%s,%s,%s->%s compute=%d swapped=%d ",
                 (long long)p.M, (long long)p.N, (long long)p.K, typeName(p.typeA), typeName(p.typeB),
                 p.bilinear ? typeName(p.typeC) : "-", typeName(p.typeD), p.computeType, p.swapped);
        s += buf;
        appendDims(s, "m", p.m, p.nm);
        appendDims(s, " n", p.n, p.nn);
        appendDims(s, " k", p.k, p.nk);
        if(p.kind == CK_TF32X3)
        {
            snprintf(buf, sizeof(buf), " major=%s/%s boxK=[%d %d]", p.aMajor ? "mn" : "k", p.bMajor ? "mn" : "k", p.boxK[0],
                     p.boxK[1]);
            s += buf;
        }
        if(p.kind == CK_TCGEN05)
        {
            snprintf(buf, sizeof(buf), " major=%s/%s", p.aMajor ? "mn" : "k", p.bMajor ? "mn" : "k");
            s += buf;
        }
        if(p.kind == CK_TCGEN05 || p.kind == CK_TF32X3)
        {
            snprintf(buf, sizeof(buf), " tile=%dx%dx%d stages=%d rows=%d/%d boxM=[", p.tileM, p.tileN, p.tileK,
                     p.stages, p.rowsM, p.rowsN);
            s += buf;
            for(int i = 0; i < p.nm; i++)
            {
                snprintf(buf, sizeof(buf), "%s%d", i ? " " : "", p.boxM[i]);
                s += buf;
            }
            s += "] boxN=[";
            for(int i = 0; i < p.nn; i++)
            {
                snprintf(buf, sizeof(buf), "%s%d", i ? " " : "", p.boxN[i]);
                s += buf;
            }
            s += p.pair ? (p.wide ? "] pair 256x512" : "] pair 256x256") : "]";
            if(p.pair && p.ksplit > 1)
                s += " ksplit=2";
        }
        if(p.packReal)
        {
            snprintf(buf, sizeof(buf), " packed K=%lld Kp=%lld copies=%llu", (long long)p.packK, (long long)p.packKp,
                     (unsigned long long)p.expandBytes);
            s += buf;
        }
        if(p.splitK > 1)
        {
            snprintf(buf, sizeof(buf), " splitK=%d workspace=%lld", p.splitK, (long long)p.workspaceBytes);
            s += buf;
        }
        return s;
    }
} // namespace htb
