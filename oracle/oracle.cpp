// CPU oracle: a plain C++17 restatement of hipTensor's own CPU reference
// implementations of contraction, permutation and reduction.
//
// THIS IS TEST INFRASTRUCTURE. It is the checker that the CUDA library is
// compared with; nothing in the shipped library links, loads or calls it.
//
// Parity status
//   permutation : pinned by the golden vector of
//                 test/02_permutation/permutation_cpu_impl_test.cpp:82-93
//   reduction   : ADD with alpha and beta pinned by the golden vector of
//                 test/03_reduction/reduction_cpu_impl_test.cpp:73-83;
//                 MUL/MIN/MAX and NaN propagation: parity unpinned
//                 (the arithmetic lives in Composable Kernel's host
//                 ReferenceReduce, a third-party dependency that is not
//                 vendored; floor version composable_kernel 1.0.0,
//                 library/src/CMakeLists.txt:27).
//   contraction : parity unpinned (the reference holds no golden vector;
//                 its tests only compare its GPU path with its CPU path);
//                 the same holds for the complex form.
//
// Every function cites the reference file:line whose behaviour it restates.
// No reference source is copied: loop structure is re-expressed with
// pre-computed offset tables, the arithmetic order is kept.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <thread>
#include <vector>

namespace
{
    // ---- data type codes (same numeric values as hipDataType / cudaDataType) ----
    enum : int
    {
        DT_F32  = 0,
        DT_F64  = 1,
        DT_F16  = 2,
        DT_BF16 = 14
    };
    // ---- hiptensorComputeType_t values (hiptensor_types.hpp:74-99) ----
    enum : int
    {
        CT_16F  = 1,
        CT_32F  = 4,
        CT_64F  = 16,
        CT_16BF = 1024
    };
    // ---- hiptensorOperator_t values (hiptensor_types.hpp:102-124) ----
    enum : int
    {
        OP_IDENTITY = 1,
        OP_SQRT     = 2,
        OP_ADD      = 3,
        OP_MUL      = 5,
        OP_MAX      = 6,
        OP_MIN      = 7
    };

    using f16 = _Float16;

    struct bf16
    {
        uint16_t bits;
    };

    inline float bf16_to_float(bf16 v)
    {
        uint32_t u = uint32_t(v.bits) << 16;
        float    f;
        std::memcpy(&f, &u, 4);
        return f;
    }
    // round-to-nearest-even, NaN kept quiet (CK's default float->bhalf conversion)
    inline bf16 float_to_bf16(float f)
    {
        uint32_t u;
        std::memcpy(&u, &f, 4);
        if((u & 0x7fffffffu) > 0x7f800000u)
        {
            return bf16{uint16_t((u >> 16) | 0x40)};
        }
        uint32_t lsb = (u >> 16) & 1u;
        u += 0x7fffu + lsb;
        return bf16{uint16_t(u >> 16)};
    }

    int dtype_size(int dt)
    {
        switch(dt)
        {
        case DT_F32: return 4;
        case DT_F64: return 8;
        case DT_F16: return 2;
        case DT_BF16: return 2;
        default: return 0;
        }
    }

    inline double load_as_double(const void* p, int dt, int64_t i)
    {
        switch(dt)
        {
        case DT_F32: return double(((const float*)p)[i]);
        case DT_F64: return ((const double*)p)[i];
        case DT_F16: return double(float(((const f16*)p)[i]));
        case DT_BF16: return double(bf16_to_float(((const bf16*)p)[i]));
        }
        return 0.0;
    }
    inline float load_as_float(const void* p, int dt, int64_t i)
    {
        switch(dt)
        {
        case DT_F32: return ((const float*)p)[i];
        case DT_F64: return float(((const double*)p)[i]);
        case DT_F16: return float(((const f16*)p)[i]);
        case DT_BF16: return bf16_to_float(((const bf16*)p)[i]);
        }
        return 0.f;
    }
    inline void store_from_float(void* p, int dt, int64_t i, float v)
    {
        switch(dt)
        {
        case DT_F32: ((float*)p)[i] = v; break;
        case DT_F64: ((double*)p)[i] = double(v); break;
        case DT_F16: ((f16*)p)[i] = f16(v); break;
        case DT_BF16: ((bf16*)p)[i] = float_to_bf16(v); break;
        }
    }

    // The reference test generator: test/device/common.hpp:68-108.
    inline uint32_t pcg_hash(uint32_t input)
    {
        uint32_t state = input * 747796405u + 2891336453u;
        uint32_t word  = ((state >> ((state >> 28u) + 4u)) ^ state) * 277803737u;
        return (word >> 22u) ^ word;
    }
    inline float uniform_pm1(uint32_t seeded_index)
    {
        return (float(pcg_hash(seeded_index)) / float(0xffffffffu) - 0.5f) * 2.0f;
    }

    // Scalar decode: alpha/beta arrive typed by the compute type and the
    // reference squeezes them through a float-holding functor
    // (contraction_solution_impl.hpp:110-123, data_types.cpp:152-205).
    double read_scalar(const void* p, int computeType)
    {
        switch(computeType)
        {
        case CT_32F: return double(*(const float*)p);
        case CT_64F: return *(const double*)p;
        case CT_16F: return double(float(*(const f16*)p));
        case CT_16BF: return double(bf16_to_float(*(const bf16*)p));
        }
        return 0.0;
    }

    template <class F>
    void parallel_for(int64_t n, int nthreads, F&& body)
    {
        if(nthreads <= 0)
            nthreads = int(std::thread::hardware_concurrency());
        if(nthreads < 1)
            nthreads = 1;
        if(n < 1024 || nthreads == 1)
        {
            body(int64_t(0), n);
            return;
        }
        std::vector<std::thread> pool;
        int64_t                  chunk = (n + nthreads - 1) / nthreads;
        for(int t = 0; t < nthreads; t++)
        {
            int64_t lo = t * chunk, hi = std::min(n, lo + chunk);
            if(lo >= hi)
                break;
            pool.emplace_back([=, &body] { body(lo, hi); });
        }
        for(auto& th : pool)
            th.join();
    }

    // One group of modes (M, N or K) of a normalised contraction.
    struct ModeGroup
    {
        std::vector<int64_t> len, s0, s1; // extents, stride in first tensor, stride in second
        int64_t              total() const
        {
            int64_t t = 1;
            for(auto l : len)
                t *= l;
            return t;
        }
    };

    // Offsets of a group enumerated with the LAST mode of the group fastest,
    // i.e. the nesting order of the reference's loop nest (k0 outermost,
    // contraction_cpu_reference_impl.hpp:347-404) and of its parallel functor
    // over (m0..m5,n0..n5).
    void enumerate(const ModeGroup& g, std::vector<int64_t>& o0, std::vector<int64_t>& o1)
    {
        int64_t tot = g.total();
        o0.resize(tot);
        o1.resize(tot);
        int                  r = int(g.len.size());
        std::vector<int64_t> idx(r, 0);
        for(int64_t i = 0; i < tot; i++)
        {
            int64_t a = 0, b = 0;
            for(int d = 0; d < r; d++)
            {
                a += idx[d] * g.s0[d];
                b += idx[d] * g.s1[d];
            }
            o0[i] = a;
            o1[i] = b;
            for(int d = r - 1; d >= 0; d--)
            {
                if(++idx[d] < g.len[d])
                    break;
                idx[d] = 0;
            }
        }
    }

    int find_mode(const int32_t* modes, int n, int32_t m)
    {
        for(int i = 0; i < n; i++)
            if(modes[i] == m)
                return i;
        return -1;
    }

    template <class AccT>
    inline AccT to_compute(const void* p, int dt, int64_t i, int computeType)
    {
        // contraction_cpu_reference_impl.hpp:386-398: the element is converted to
        // ComputeDataType first, then widened to AccDataType.
        if constexpr(std::is_same_v<AccT, double>)
        {
            return load_as_double(p, dt, i);
        }
        else
        {
            float v = load_as_float(p, dt, i); // f64 data with compute f32: rounds to float
            if(computeType == CT_16F)
                v = float(f16(v));
            else if(computeType == CT_16BF)
                v = bf16_to_float(float_to_bf16(v));
            return v;
        }
    }

    // Epilogue: the reference rounds the accumulator to the OUTPUT type, then applies
    // CK's Scale / Bilinear functor (contraction_cpu_reference_impl.hpp:406-425).
    // The functors evaluate alpha*x (+ beta*c) in float for f16/bf16/f32 outputs and
    // in double for f64 outputs, with alpha/beta held as float
    // (contraction_solution_impl.hpp:110).
    template <class AccT>
    inline void epilogue(void* D, int typeD, int64_t offD, AccT acc, bool bilinear, const void* C,
                         int64_t offC, float alpha, float beta)
    {
        switch(typeD)
        {
        case DT_F32:
        {
            float x = float(acc);
            float y = alpha * x;
            if(bilinear)
                y = alpha * x + beta * ((const float*)C)[offC];
            ((float*)D)[offD] = y;
            break;
        }
        case DT_F64:
        {
            double x = double(acc);
            double y = double(alpha) * x;
            if(bilinear)
                y = double(alpha) * x + double(beta) * ((const double*)C)[offC];
            ((double*)D)[offD] = y;
            break;
        }
        case DT_F16:
        {
            float x = float(f16(float(acc)));
            float y = alpha * x;
            if(bilinear)
                y = alpha * x + beta * float(((const f16*)C)[offC]);
            ((f16*)D)[offD] = f16(y);
            break;
        }
        case DT_BF16:
        {
            float x = bf16_to_float(float_to_bf16(float(acc)));
            float y = alpha * x;
            if(bilinear)
                y = alpha * x + beta * bf16_to_float(((const bf16*)C)[offC]);
            ((bf16*)D)[offD] = float_to_bf16(y);
            break;
        }
        }
    }
} // namespace

extern "C" {

int orc_dtype_size(int dt)
{
    return dtype_size(dt);
}

// test/device/common.hpp:82-108 (fillKernel): element i <- uniform[-1,1) of
// pcg_hash((i + seed) mod UINT_MAX), computed in float, then cast.
void orc_fill_uniform(void* dst, int dt, uint64_t n, uint32_t seed)
{
    parallel_for(int64_t(n), 0, [&](int64_t lo, int64_t hi) {
        for(int64_t i = lo; i < hi; i++)
        {
            uint32_t index  = uint32_t(i);
            uint32_t seeded = uint32_t(uint64_t(uint32_t(index + seed)) % 0xffffffffull);
            float    v      = uniform_pm1(seeded);
            store_from_float(dst, dt, i, v);
        }
    });
}

// Not in the reference (it has no normal generator): Box-Muller over two
// PCG-hash draws per element; element i uses hash inputs 2i+seed and 2i+1+seed.
void orc_fill_normal(void* dst, int dt, uint64_t n, uint32_t seed, float sigma)
{
    parallel_for(int64_t(n), 0, [&](int64_t lo, int64_t hi) {
        for(int64_t i = lo; i < hi; i++)
        {
            uint32_t h1 = pcg_hash(uint32_t(2 * i) + seed);
            uint32_t h2 = pcg_hash(uint32_t(2 * i + 1) + seed);
            float    u1 = (float(h1 >> 8) + 1.0f) * (1.0f / 16777216.0f); // (0,1]
            float    u2 = float(h2 >> 8) * (1.0f / 16777216.0f); // [0,1)
            float    r  = std::sqrt(-2.0f * std::log(u1));
            float    v  = sigma * r * std::cos(6.28318530717958647692f * u2);
            store_from_float(dst, dt, i, v);
        }
    });
}

// Contraction oracle.
//   contraction_solution.cpp:34-160  : M = modes of D found in A (D's order), N = the
//       other modes of D (looked up in B), K = modes of A also in B (A's order).
//   contraction_solution_impl.hpp:125-140 : C is addressed with D's strides.
//   contraction_cpu_reference_impl.hpp:326-441 : per output element a sequential
//       K nest, accumulate in AccDataType, round to the output type, CDE functor.
//   contraction_cpu_reference_instances.cpp:32-298 : (A,B,Acc,E,Compute) tuples;
//       f64 data with compute f32 accumulates in float (:124-136).
// sample: optional list of logical output indices (first mode of D fastest) to
// evaluate instead of the whole tensor (used for the problems that are too large
// to evaluate in full). Returns 0 on success.
int orc_contraction(const void* alphaP, const void* A, int nA, const int64_t* lenA,
                    const int64_t* strA, const int32_t* modeA, int typeA, const void* B, int nB,
                    const int64_t* lenB, const int64_t* strB, const int32_t* modeB, int typeB,
                    const void* betaP, const void* C, void* D, int nD, const int64_t* lenD,
                    const int64_t* strD, const int32_t* modeD, int typeD, int computeType,
                    const int64_t* sample, int64_t nsample, int nthreads)
{
    ModeGroup gm, gn, gk; // M: (A,D)   N: (B,D)   K: (A,B)
    for(int i = 0; i < nD; i++)
    {
        int ia = find_mode(modeA, nA, modeD[i]);
        if(ia >= 0)
        {
            gm.len.push_back(lenA[ia]);
            gm.s0.push_back(strA[ia]);
            gm.s1.push_back(strD[i]);
        }
        else
        {
            int ib = find_mode(modeB, nB, modeD[i]);
            if(ib < 0)
                return 1;
            gn.len.push_back(lenB[ib]);
            gn.s0.push_back(strB[ib]);
            gn.s1.push_back(strD[i]);
        }
    }
    for(int i = 0; i < nA; i++)
    {
        int ib = find_mode(modeB, nB, modeA[i]);
        if(ib >= 0)
        {
            if(find_mode(modeD, nD, modeA[i]) >= 0)
                return 2; // batch mode: mis-classified by the reference, not evaluated here
            gk.len.push_back(lenA[i]);
            gk.s0.push_back(strA[i]);
            gk.s1.push_back(strB[ib]);
        }
    }
    std::vector<int64_t> aM, dM, bN, dN, aK, bK;
    enumerate(gm, aM, dM);
    enumerate(gn, bN, dN);
    enumerate(gk, aK, bK);
    const int64_t M = gm.total(), N = gn.total(), K = gk.total();

    const bool  bilinear = (C != nullptr);
    const float alpha    = float(read_scalar(alphaP, computeType));
    const float beta     = (bilinear && betaP) ? float(read_scalar(betaP, computeType)) : 0.f;
    const bool  accDouble = (typeA == DT_F64 && computeType == CT_64F);

    // logical D index (first listed mode fastest) -> (m, n) linear indices
    std::vector<int64_t> smn;
    if(sample)
    {
        // position of each D mode within its group, and group multipliers (last fastest)
        std::vector<int> isM(nD), pos(nD);
        int              cm = 0, cn = 0;
        for(int i = 0; i < nD; i++)
        {
            bool inA = find_mode(modeA, nA, modeD[i]) >= 0;
            isM[i]   = inA;
            pos[i]   = inA ? cm++ : cn++;
        }
        std::vector<int64_t> mulM(gm.len.size(), 1), mulN(gn.len.size(), 1);
        for(int d = int(gm.len.size()) - 2; d >= 0; d--)
            mulM[d] = mulM[d + 1] * gm.len[d + 1];
        for(int d = int(gn.len.size()) - 2; d >= 0; d--)
            mulN[d] = mulN[d + 1] * gn.len[d + 1];
        smn.resize(2 * nsample);
        for(int64_t s = 0; s < nsample; s++)
        {
            int64_t rem = sample[s], m = 0, n = 0;
            for(int i = 0; i < nD; i++)
            {
                int64_t c = rem % lenD[i];
                rem /= lenD[i];
                if(isM[i])
                    m += c * mulM[pos[i]];
                else
                    n += c * mulN[pos[i]];
            }
            smn[2 * s]     = m;
            smn[2 * s + 1] = n;
        }
    }

    const int64_t total = sample ? nsample : M * N;
    parallel_for(total, nthreads, [&](int64_t lo, int64_t hi) {
        for(int64_t t = lo; t < hi; t++)
        {
            int64_t m, n;
            if(sample)
            {
                m = smn[2 * t];
                n = smn[2 * t + 1];
            }
            else
            {
                m = t / N;
                n = t % N;
            }
            const int64_t oa = aM[m], ob = bN[n], od = dM[m] + dN[n];
            if(accDouble)
            {
                double acc = 0;
                for(int64_t k = 0; k < K; k++)
                    acc += to_compute<double>(A, typeA, oa + aK[k], computeType)
                           * to_compute<double>(B, typeB, ob + bK[k], computeType);
                epilogue<double>(D, typeD, od, acc, bilinear, C, od, alpha, beta);
            }
            else
            {
                float acc = 0;
                for(int64_t k = 0; k < K; k++)
                    acc += to_compute<float>(A, typeA, oa + aK[k], computeType)
                           * to_compute<float>(B, typeB, ob + bK[k], computeType);
                epilogue<float>(D, typeD, od, acc, bilinear, C, od, alpha, beta);
            }
        }
    });
    return 0;
}

// Complex contraction oracle (cf32: typeCode 4, cf64: typeCode 5; alpha/beta point to two floats / two doubles).
//   contraction_cpu_reference_impl.hpp:166-323 : acc = (0,0); for k0..k5: acc = acc + a*b with the complex
//       product (ar*br - ai*bi, ai*br + ar*bi) evaluated in the accumulator type (float for cf32, double for
//       cf64: contraction_cpu_reference_instances.cpp:108-121,152-165); BilinearComplex:
//       E = alpha*acc + beta*D, ScaleComplex: E = alpha*acc, complex products in the element type with alpha,
//       beta narrowed to it.
//   Parity unpinned: the reference holds no golden vector for complex contractions either.
int orc_contraction_complex(const void* alphaP, const void* A, int nA, const int64_t* lenA, const int64_t* strA,
                            const int32_t* modeA, const void* B, int nB, const int64_t* lenB, const int64_t* strB,
                            const int32_t* modeB, const void* betaP, const void* C, void* D, int nD,
                            const int64_t* lenD, const int64_t* strD, const int32_t* modeD, int typeCode, int nthreads)
{
    if(typeCode != 4 && typeCode != 5)
        return 3;
    ModeGroup gm, gn, gk;
    for(int i = 0; i < nD; i++)
    {
        int ia = find_mode(modeA, nA, modeD[i]);
        if(ia >= 0)
        {
            gm.len.push_back(lenA[ia]);
            gm.s0.push_back(strA[ia]);
            gm.s1.push_back(strD[i]);
        }
        else
        {
            int ib = find_mode(modeB, nB, modeD[i]);
            if(ib < 0)
                return 1;
            gn.len.push_back(lenB[ib]);
            gn.s0.push_back(strB[ib]);
            gn.s1.push_back(strD[i]);
        }
    }
    for(int i = 0; i < nA; i++)
    {
        int ib = find_mode(modeB, nB, modeA[i]);
        if(ib >= 0)
        {
            if(find_mode(modeD, nD, modeA[i]) >= 0)
                return 2;
            gk.len.push_back(lenA[i]);
            gk.s0.push_back(strA[i]);
            gk.s1.push_back(strB[ib]);
        }
    }
    std::vector<int64_t> aM, dM, bN, dN, aK, bK;
    enumerate(gm, aM, dM);
    enumerate(gn, bN, dN);
    enumerate(gk, aK, bK);
    const int64_t M = gm.total(), N = gn.total(), K = gk.total();
    const bool    bilinear = (C != nullptr);
    auto run = [&](auto zero) {
        using T        = decltype(zero);
        const T*  a    = (const T*)A;
        const T*  b    = (const T*)B;
        const T*  c    = (const T*)C;
        T*        d    = (T*)D;
        const T   ar = ((const T*)alphaP)[0], ai = ((const T*)alphaP)[1];
        const T   br = (bilinear && betaP) ? ((const T*)betaP)[0] : T(0), bi = (bilinear && betaP) ? ((const T*)betaP)[1] : T(0);
        parallel_for(M * N, nthreads, [&](int64_t lo, int64_t hi) {
            for(int64_t t = lo; t < hi; t++)
            {
                const int64_t m = t / N, n = t % N;
                const int64_t oa = aM[m], ob = bN[n], od = dM[m] + dN[n];
                T             sr = 0, si = 0;
                for(int64_t k = 0; k < K; k++)
                {
                    const T xr = a[2 * (oa + aK[k])], xi = a[2 * (oa + aK[k]) + 1];
                    const T yr = b[2 * (ob + bK[k])], yi = b[2 * (ob + bK[k]) + 1];
                    const T pr = xr * yr - xi * yi, pi = xi * yr + xr * yi;
                    sr = sr + pr;
                    si = si + pi;
                }
                T er = ar * sr - ai * si, ei = ai * sr + ar * si;
                if(bilinear)
                {
                    const T cr = c[2 * od], ci = c[2 * od + 1];
                    er = er + (br * cr - bi * ci);
                    ei = ei + (bi * cr + br * ci);
                }
                d[2 * od]     = er;
                d[2 * od + 1] = ei;
            }
        });
    };
    if(typeCode == 4)
        run(0.0f);
    else
        run(0.0);
    return 0;
}

// Permutation oracle.
//   permutation_solution_impl.hpp:103-145 : alpha widened to float; the descriptor's
//       strides are ignored and packed strides are recomputed with the FIRST mode
//       fastest (HIPTENSOR_DATA_LAYOUT_COL_MAJOR, default ON); B's strides are
//       re-indexed into A's mode order.
//   permutation_cpu_reference_impl.hpp:112-145 : single-threaded odometer over A's
//       index space, B[off_b] = Bop(alpha * Aop(A[off_a])).
//   permutation_types_impl.hpp:45-49 : HIPTENSOR_OP_SQRT is the SQUARE x*x.
// Scale on f16 data multiplies in half precision (CK's Scale functor, third-party).
int orc_permutation(const void* alphaP, int typeScalar, const void* A, int nmode,
                    const int64_t* lenA, const int32_t* modeA, int typeA, int opA, void* B,
                    const int32_t* modeB, int typeB, int opB, int nthreads)
{
    float alpha;
    if(typeScalar == DT_F32)
        alpha = *(const float*)alphaP;
    else if(typeScalar == DT_F16)
        alpha = float(*(const f16*)alphaP);
    else
        return 1;

    std::vector<int64_t> sa(nmode), sb(nmode), lenB(nmode);
    int64_t              s = 1;
    for(int i = 0; i < nmode; i++)
    {
        sa[i] = s;
        s *= lenA[i];
    }
    const int64_t total = s;
    for(int i = 0; i < nmode; i++)
    {
        int ia = find_mode(modeA, nmode, modeB[i]);
        if(ia < 0)
            return 2;
        lenB[i] = lenA[ia];
    }
    s = 1;
    for(int i = 0; i < nmode; i++)
    {
        int ia = find_mode(modeA, nmode, modeB[i]);
        sb[ia] = s;
        s *= lenB[i];
    }

    auto unary = [](float x, int op) { return op == OP_SQRT ? x * x : x; };

    parallel_for(total, nthreads, [&](int64_t lo, int64_t hi) {
        // odometer with the last A index fastest, as the reference iterates
        std::vector<int64_t> idx(nmode, 0);
        int64_t              rem = lo;
        for(int d = nmode - 1; d >= 0; d--)
        {
            idx[d] = rem % lenA[d];
            rem /= lenA[d];
        }
        for(int64_t e = lo; e < hi; e++)
        {
            int64_t oa = 0, ob = 0;
            for(int d = 0; d < nmode; d++)
            {
                oa += idx[d] * sa[d];
                ob += idx[d] * sb[d];
            }
            if(typeA == DT_F32)
            {
                float x = unary(((const float*)A)[oa], opA);
                x       = alpha * x;
                x       = unary(x, opB);
                ((float*)B)[ob] = x;
            }
            else // f16 input: intermediates stay in half
            {
                f16 x = ((const f16*)A)[oa];
                if(opA == OP_SQRT)
                    x = f16(float(x) * float(x));
                x = f16(float(f16(alpha)) * float(x));
                if(opB == OP_SQRT)
                    x = f16(float(x) * float(x));
                if(typeB == DT_F16)
                    ((f16*)B)[ob] = x;
                else
                    ((float*)B)[ob] = float(x);
            }
            for(int d = nmode - 1; d >= 0; d--)
            {
                if(++idx[d] < lenA[d])
                    break;
                idx[d] = 0;
            }
        }
    });
    return 0;
}

// Reduction oracle.
//   hiptensor_reduction.cpp:254-307 / reduction_cpu_reference.cpp:46-88 : compute type
//       f16/bf16 promoted to f32; alpha/beta read as the compute type and widened to
//       double; C copied over D when they differ; then D = alpha*reduce(A) + beta*D.
//   reduction_solution_impl.hpp:105-163 : reduced dims = positions in A of modes absent
//       from D; D's j-th extent/stride belongs to the j-th kept mode of A (positional).
//   CK host ReferenceReduce (third-party, described in words): per kept index,
//       acc = identity; acc = op(acc, Acc(a)) sequentially with the last reduced mode
//       fastest; NaN propagates through MIN/MAX; if alpha != 1: acc *= alpha;
//       if beta != 0: acc += Acc(D_old) * beta; D = Out(acc).
int orc_reduction(const void* alphaP, const void* A, int nA, const int64_t* lenA,
                  const int64_t* strA, const int32_t* modeA, int typeA, const void* betaP,
                  const void* C, void* D, int nD, const int64_t* lenD, const int64_t* strD,
                  const int32_t* modeD, int typeD, int opReduce, int computeType, int nthreads)
{
    (void)lenD;
    const double alphaD = read_scalar(alphaP, computeType);
    const double betaD  = read_scalar(betaP, computeType);
    const bool   accF64 = (computeType == CT_64F);

    ModeGroup keep, red; // keep: (A, D)   red: (A, -)
    int       j = 0;
    for(int i = 0; i < nA; i++)
    {
        if(find_mode(modeD, nD, modeA[i]) >= 0)
        {
            keep.len.push_back(lenA[i]);
            keep.s0.push_back(strA[i]);
            keep.s1.push_back(strD[j]);
            j++;
        }
        else
        {
            red.len.push_back(lenA[i]);
            red.s0.push_back(strA[i]);
            red.s1.push_back(0);
        }
    }
    std::vector<int64_t> aKeep, dKeep, aRed, unused;
    enumerate(keep, aKeep, dKeep);
    enumerate(red, aRed, unused);
    const int64_t nOut = keep.total(), nRed = red.total();

    auto body = [&](auto accTag) {
        using Acc = decltype(accTag);
        const Acc alpha = Acc(alphaD), beta = Acc(betaD);
        parallel_for(nOut, nthreads, [&](int64_t lo, int64_t hi) {
            for(int64_t o = lo; o < hi; o++)
            {
                Acc acc;
                switch(opReduce)
                {
                case OP_ADD: acc = Acc(0); break;
                case OP_MUL: acc = Acc(1); break;
                case OP_MAX: acc = std::numeric_limits<Acc>::lowest(); break;
                case OP_MIN: acc = std::numeric_limits<Acc>::max(); break;
                default: acc = Acc(0);
                }
                const int64_t base = aKeep[o];
                for(int64_t r = 0; r < nRed; r++)
                {
                    Acc v;
                    if constexpr(std::is_same_v<Acc, double>)
                        v = load_as_double(A, typeA, base + aRed[r]);
                    else
                        v = load_as_float(A, typeA, base + aRed[r]);
                    switch(opReduce)
                    {
                    case OP_ADD: acc = acc + v; break;
                    case OP_MUL: acc = acc * v; break;
                    case OP_MAX:
                        if(std::isnan(v) || acc < v)
                            acc = (std::isnan(acc) ? acc : v);
                        break;
                    case OP_MIN:
                        if(std::isnan(v) || acc > v)
                            acc = (std::isnan(acc) ? acc : v);
                        break;
                    }
                }
                if(alpha != Acc(1))
                    acc *= alpha;
                if(beta != Acc(0))
                {
                    const void* src = (C != nullptr) ? C : (const void*)D;
                    Acc         old;
                    if constexpr(std::is_same_v<Acc, double>)
                        old = load_as_double(src, typeD, dKeep[o]);
                    else
                        old = load_as_float(src, typeD, dKeep[o]);
                    acc += old * beta;
                }
                if constexpr(std::is_same_v<Acc, double>)
                    ((double*)D)[dKeep[o]] = acc;
                else
                    store_from_float(D, typeD, dKeep[o], acc);
            }
        });
    };
    if(accF64)
        body(double{});
    else
        body(float{});
    return 0;
}

// test/device/common.hpp:122-151 + test/utils.hpp:285-383: max over elements of
// |d-h| / (|d|+|h|+1); NaN or Inf anywhere makes the comparison fail (returned as -1).
double orc_max_rel_error(const void* dev, const void* host, int dt, uint64_t n)
{
    double worst = 0;
    for(uint64_t i = 0; i < n; i++)
    {
        double d = load_as_double(dev, dt, int64_t(i)), h = load_as_double(host, dt, int64_t(i));
        double num = std::fabs(d - h), den = std::fabs(d) + std::fabs(h) + 1.0;
        if(std::isnan(num) || std::isnan(den) || std::isinf(num) || std::isinf(den))
            return -1.0;
        worst = std::max(worst, num / den);
    }
    return worst;
}

} // extern "C"
