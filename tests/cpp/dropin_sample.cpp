// A caller written against the reference's C++ API (hiptensor.hpp), compiled unchanged against this
// library's header: permutation, reduction, a bilinear contraction and a complex one, following the call sequences of
// samples/02_permutation/permutation.cpp:107-130, samples/03_reduction/reduction.cpp:116-171 and
// samples/01_contraction/simple_bilinear_contraction.hpp:86-271 of the reference. Each result is checked
// on the host with plain loops. Prints "DROPIN OK" and returns 0 on success.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_runtime.h>
#include <hiptensor/hiptensor.hpp>

#define CHECK_HT(x)                                                                       \
    do                                                                                    \
    {                                                                                     \
        hiptensorStatus_t s_ = (x);                                                       \
        if(s_ != HIPTENSOR_STATUS_SUCCESS)                                                \
        {                                                                                 \
            printf("%s failed: %s (line %d)\n", #x, hiptensorGetErrorString(s_), __LINE__); \
            return 1;                                                                     \
        }                                                                                 \
    } while(0)
#define CHECK_CUDA(x)                                                        \
    do                                                                       \
    {                                                                        \
        cudaError_t e_ = (x);                                                \
        if(e_ != cudaSuccess)                                                \
        {                                                                    \
            printf("%s failed: %s\n", #x, cudaGetErrorString(e_));           \
            return 1;                                                        \
        }                                                                    \
    } while(0)

static float frand()
{
    return float(rand()) / float(RAND_MAX) * 2.f - 1.f;
}

int main()
{
    hiptensorHandle_t* handle = nullptr;
    CHECK_HT(hiptensorCreate(&handle));

    // ---------------------------------------------------------------- permutation B[c,n,h,w] = 2.1 * A[w,h,c,n]
    {
        std::vector<int32_t> modeA{'w', 'h', 'c', 'n'}, modeB{'c', 'n', 'h', 'w'};
        std::vector<int64_t> extA{36, 20, 16, 8}, extB{16, 8, 20, 36};
        const size_t         n = 36 * 20 * 16 * 8;
        std::vector<float>   A(n), B(n, -1.f);
        for(auto& v : A)
            v = frand();
        float *dA = nullptr, *dB = nullptr;
        CHECK_CUDA(cudaMalloc(&dA, n * 4));
        CHECK_CUDA(cudaMalloc(&dB, n * 4));
        CHECK_CUDA(cudaMemcpy(dA, A.data(), n * 4, cudaMemcpyHostToDevice));
        hiptensorTensorDescriptor_t descA, descB;
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descA, 4, extA.data(), NULL, HIP_R_32F, HIPTENSOR_OP_IDENTITY));
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descB, 4, extB.data(), NULL, HIP_R_32F, HIPTENSOR_OP_IDENTITY));
        const float alpha = 2.1f;
        CHECK_HT(hiptensorPermutation(handle, &alpha, dA, &descA, modeA.data(), dB, &descB, modeB.data(), HIP_R_32F, 0));
        CHECK_CUDA(cudaMemcpy(B.data(), dB, n * 4, cudaMemcpyDeviceToHost));
        for(int w = 0; w < 36; w++)
            for(int h = 0; h < 20; h++)
                for(int c = 0; c < 16; c++)
                    for(int nn = 0; nn < 8; nn++)
                    {
                        // both tensors packed with the first mode fastest
                        float a = A[w + 36 * (h + 20 * (c + 16 * nn))];
                        float b = B[c + 16 * (nn + 8 * (h + 20 * w))];
                        if(b != alpha * a)
                        {
                            printf("permutation mismatch\n");
                            return 1;
                        }
                    }
        cudaFree(dA);
        cudaFree(dB);
    }

    // ---------------------------------------------------------------- reduction D[k,v] = 1.2 * sum_{m,h} A[m,h,k,v] + 2.1 * D
    {
        std::vector<int32_t> modeA{'m', 'h', 'k', 'v'}, modeC{'k', 'v'};
        std::vector<int64_t> extA{3, 5, 6, 4}, extC{6, 4};
        std::vector<double>  A(360), C(24, 1.0);
        for(size_t i = 0; i < A.size(); i++)
            A[i] = double(i);
        double *dA = nullptr, *dC = nullptr;
        CHECK_CUDA(cudaMalloc(&dA, 360 * 8));
        CHECK_CUDA(cudaMalloc(&dC, 24 * 8));
        CHECK_CUDA(cudaMemcpy(dA, A.data(), 360 * 8, cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(dC, C.data(), 24 * 8, cudaMemcpyHostToDevice));
        hiptensorTensorDescriptor_t descA, descC;
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descA, 4, extA.data(), NULL, HIP_R_64F, HIPTENSOR_OP_IDENTITY));
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descC, 2, extC.data(), NULL, HIP_R_64F, HIPTENSOR_OP_IDENTITY));
        uint64_t worksize = 0;
        CHECK_HT(hiptensorReductionGetWorkspaceSize(handle, dA, &descA, modeA.data(), dC, &descC, modeC.data(), dC, &descC,
                                                    modeC.data(), HIPTENSOR_OP_ADD, HIPTENSOR_COMPUTE_64F, &worksize));
        const double alpha = 1.2, beta = 2.1;
        CHECK_HT(hiptensorReduction(handle, &alpha, dA, &descA, modeA.data(), &beta, dC, &descC, modeC.data(), dC, &descC,
                                    modeC.data(), HIPTENSOR_OP_ADD, HIPTENSOR_COMPUTE_64F, nullptr, 0, 0));
        CHECK_CUDA(cudaMemcpy(C.data(), dC, 24 * 8, cudaMemcpyDeviceToHost));
        // first known answer of the reference's CPU test: 1.2 * (24 * 105) + 2.1
        if(std::fabs(C[0] - 3026.1) > 1e-9 || std::fabs(C[23] - 3440.1) > 1e-9)
        {
            printf("reduction mismatch %f %f\n", C[0], C[23]);
            return 1;
        }
        cudaFree(dA);
        cudaFree(dC);
    }

    // ---------------------------------------------------------------- contraction C[m,n,u,v] = 1.1*A[m,n,h,k]*B[u,v,h,k] + 2.2*C
    {
        std::vector<int32_t> modeC{'m', 'n', 'u', 'v'}, modeA{'m', 'n', 'h', 'k'}, modeB{'u', 'v', 'h', 'k'};
        std::vector<int64_t> ext{5, 6, 3, 4}, extA{5, 6, 3, 4}, extB{3, 4, 3, 4}, extC{5, 6, 3, 4};
        const size_t         nA = 5 * 6 * 3 * 4, nB = 3 * 4 * 3 * 4, nC = 5 * 6 * 3 * 4;
        std::vector<float>   A(nA), B(nB), C(nC), D(nC);
        for(auto& v : A)
            v = frand();
        for(auto& v : B)
            v = frand();
        for(auto& v : C)
            v = frand();
        float *dA, *dB, *dC;
        CHECK_CUDA(cudaMalloc(&dA, nA * 4));
        CHECK_CUDA(cudaMalloc(&dB, nB * 4));
        CHECK_CUDA(cudaMalloc(&dC, nC * 4));
        CHECK_CUDA(cudaMemcpy(dA, A.data(), nA * 4, cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(dB, B.data(), nB * 4, cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(dC, C.data(), nC * 4, cudaMemcpyHostToDevice));
        hiptensorTensorDescriptor_t descA, descB, descC;
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descA, 4, extA.data(), NULL, HIP_R_32F, HIPTENSOR_OP_IDENTITY));
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descB, 4, extB.data(), NULL, HIP_R_32F, HIPTENSOR_OP_IDENTITY));
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descC, 4, extC.data(), NULL, HIP_R_32F, HIPTENSOR_OP_IDENTITY));
        uint32_t alA, alB, alC;
        CHECK_HT(hiptensorGetAlignmentRequirement(handle, dA, &descA, &alA));
        CHECK_HT(hiptensorGetAlignmentRequirement(handle, dB, &descB, &alB));
        CHECK_HT(hiptensorGetAlignmentRequirement(handle, dC, &descC, &alC));
        hiptensorContractionDescriptor_t desc;
        CHECK_HT(hiptensorInitContractionDescriptor(handle, &desc, &descA, modeA.data(), alA, &descB, modeB.data(), alB,
                                                    &descC, modeC.data(), alC, &descC, modeC.data(), alC,
                                                    HIPTENSOR_COMPUTE_32F));
        hiptensorContractionFind_t find;
        CHECK_HT(hiptensorInitContractionFind(handle, &find, HIPTENSOR_ALGO_DEFAULT));
        uint64_t worksize = 0;
        CHECK_HT(hiptensorContractionGetWorkspaceSize(handle, &desc, &find, HIPTENSOR_WORKSPACE_RECOMMENDED, &worksize));
        void* work = nullptr;
        if(worksize > 0)
            CHECK_CUDA(cudaMalloc(&work, worksize));
        hiptensorContractionPlan_t plan;
        CHECK_HT(hiptensorInitContractionPlan(handle, &plan, &desc, &find, worksize));
        const float alpha = 1.1f, beta = 2.2f;
        // C aliases D, as in the reference's sample
        CHECK_HT(hiptensorContraction(handle, &plan, &alpha, dA, dB, &beta, dC, dC, work, worksize, 0));
        CHECK_CUDA(cudaMemcpy(D.data(), dC, nC * 4, cudaMemcpyDeviceToHost));
        // NULL strides: last mode fastest
        double worst = 0;
        for(int m = 0; m < 5; m++)
            for(int n = 0; n < 6; n++)
                for(int u = 0; u < 3; u++)
                    for(int v = 0; v < 4; v++)
                    {
                        double acc = 0;
                        for(int h = 0; h < 3; h++)
                            for(int k = 0; k < 4; k++)
                                acc += double(A[((m * 6 + n) * 3 + h) * 4 + k]) * double(B[((u * 4 + v) * 3 + h) * 4 + k]);
                        const size_t i   = ((m * 6 + n) * 3 + u) * 4 + v;
                        const double ref = 1.1f * acc + 2.2f * double(C[i]);
                        worst            = std::fmax(worst, std::fabs(ref - D[i]) / (std::fabs(ref) + std::fabs(D[i]) + 1));
                    }
        if(worst > 1e-5)
        {
            printf("contraction mismatch %g\n", worst);
            return 1;
        }
        cudaFree(dA);
        cudaFree(dB);
        cudaFree(dC);
        if(work)
            cudaFree(work);
    }

    // ---------------------------------------------------------------- complex: C[m,u] = (1.1+1.2i) * A[m,h,k]*B[u,h,k] + (2.2+2.3i) * C
    {
        std::vector<int32_t> modeC{'m', 'u'}, modeA{'m', 'h', 'k'}, modeB{'u', 'h', 'k'};
        std::vector<int64_t> extA{7, 3, 4}, extB{5, 3, 4}, extC{7, 5};
        const size_t         nA = 7 * 3 * 4, nB = 5 * 3 * 4, nC = 7 * 5;
        std::vector<hipDoubleComplex> A(nA), B(nB), C(nC), D(nC);
        for(auto& v : A)
            v = make_cuDoubleComplex(frand(), frand());
        for(auto& v : B)
            v = make_cuDoubleComplex(frand(), frand());
        for(auto& v : C)
            v = make_cuDoubleComplex(frand(), frand());
        hipDoubleComplex *dA, *dB, *dC;
        CHECK_CUDA(cudaMalloc(&dA, nA * 16));
        CHECK_CUDA(cudaMalloc(&dB, nB * 16));
        CHECK_CUDA(cudaMalloc(&dC, nC * 16));
        CHECK_CUDA(cudaMemcpy(dA, A.data(), nA * 16, cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(dB, B.data(), nB * 16, cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(dC, C.data(), nC * 16, cudaMemcpyHostToDevice));
        hiptensorTensorDescriptor_t descA, descB, descC;
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descA, 3, extA.data(), NULL, HIP_C_64F, HIPTENSOR_OP_IDENTITY));
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descB, 3, extB.data(), NULL, HIP_C_64F, HIPTENSOR_OP_IDENTITY));
        CHECK_HT(hiptensorInitTensorDescriptor(handle, &descC, 2, extC.data(), NULL, HIP_C_64F, HIPTENSOR_OP_IDENTITY));
        hiptensorContractionDescriptor_t desc;
        CHECK_HT(hiptensorInitContractionDescriptor(handle, &desc, &descA, modeA.data(), 16, &descB, modeB.data(), 16, &descC,
                                                    modeC.data(), 16, &descC, modeC.data(), 16, HIPTENSOR_COMPUTE_C64F));
        hiptensorContractionFind_t find;
        CHECK_HT(hiptensorInitContractionFind(handle, &find, HIPTENSOR_ALGO_DEFAULT));
        uint64_t worksize = 0;
        CHECK_HT(hiptensorContractionGetWorkspaceSize(handle, &desc, &find, HIPTENSOR_WORKSPACE_RECOMMENDED, &worksize));
        void* work = nullptr;
        if(worksize > 0)
            CHECK_CUDA(cudaMalloc(&work, worksize));
        hiptensorContractionPlan_t plan;
        CHECK_HT(hiptensorInitContractionPlan(handle, &plan, &desc, &find, worksize));
        const hipDoubleComplex alpha = make_cuDoubleComplex(1.1, 1.2), beta = make_cuDoubleComplex(2.2, 2.3);
        CHECK_HT(hiptensorContraction(handle, &plan, &alpha, dA, dB, &beta, dC, dC, work, worksize, 0));
        CHECK_CUDA(cudaMemcpy(D.data(), dC, nC * 16, cudaMemcpyDeviceToHost));
        double worst = 0;
        for(int m = 0; m < 7; m++)
            for(int u = 0; u < 5; u++)
            {
                hipDoubleComplex acc = make_cuDoubleComplex(0, 0);
                for(int hk = 0; hk < 12; hk++)
                    acc = cuCadd(acc, cuCmul(A[m * 12 + hk], B[u * 12 + hk]));
                const hipDoubleComplex ref = cuCadd(cuCmul(alpha, acc), cuCmul(beta, C[m * 5 + u]));
                worst = std::fmax(worst, cuCabs(cuCsub(ref, D[m * 5 + u])));
            }
        if(worst > 1e-12)
        {
            printf("complex contraction mismatch %g\n", worst);
            return 1;
        }
        cudaFree(dA);
        cudaFree(dB);
        cudaFree(dC);
        if(work)
            cudaFree(work);
    }

    CHECK_HT(hiptensorDestroy(handle));
    printf("DROPIN OK\n");
    return 0;
}
