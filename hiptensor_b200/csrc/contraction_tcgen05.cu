// placeholder, replaced below
#include "kernels.hpp"
namespace htb
{
    cudaError_t launchContractionTcgen05(const ContractionPlan&, float, const void*, const void*, float, const void*,
                                         void*, int, int*, cudaStream_t)
    {
        return cudaErrorNotSupported;
    }
}
