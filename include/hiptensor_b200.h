/* Flat C ABI of libhiptensor_b200.so.
 *
 * The reference library (ROCm/hipTensor 1.4.0) exposes its API with C++ linkage and
 * std::vector-bearing structs, which no FFI can bind. Each function below is the
 * extern "C" twin of one of those entry points: plain pointers, sizes and integers,
 * descriptors behind opaque handles that the library allocates and frees. Argument
 * meaning, status codes and error behaviour are those of the C++ function named in
 * the comment (file:line inside the reference project).
 *
 * Data pointers (A, B, C, D, workspace) are device pointers; alpha/beta are host
 * pointers; all work is enqueued on `stream` (a cudaStream_t passed as void*).
 * Status codes: the hiptensorStatus_t values (0 success, 1 not initialised,
 * 7 invalid value, 8 arch mismatch, 13 execution failed, 14 internal error,
 * 15 not supported, 18 CUDA error, 19 insufficient workspace).
 */
#ifndef HIPTENSOR_B200_H
#define HIPTENSOR_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct htHandle           htHandle;           /* hiptensorHandle_t */
typedef struct htTensorDescriptor htTensorDescriptor; /* hiptensorTensorDescriptor_t */
typedef struct htContractionDesc  htContractionDesc;  /* hiptensorContractionDescriptor_t */
typedef struct htContractionFind  htContractionFind;  /* hiptensorContractionFind_t */
typedef struct htContractionPlan  htContractionPlan;  /* hiptensorContractionPlan_t */

/* library/include/hiptensor/hiptensor.hpp:41,46 (library/src/hiptensor.cpp:35-104) */
int htCreate(htHandle** handle);
int htDestroy(htHandle* handle);

/* hiptensor.hpp:71 (hiptensor.cpp:216-254) */
const char* htGetErrorString(int status);

/* hiptensor.hpp:60-66 (hiptensor.cpp:106-214). strides == NULL: packed, LAST mode fastest.
 * dataType: 0 f32, 1 f64, 2 f16, 14 bf16. unaryOp: 1 identity, 2 "sqrt" (= square). */
int htCreateTensorDescriptor(const htHandle* handle, htTensorDescriptor** desc, uint32_t numModes,
                             const int64_t* lens, const int64_t* strides, int dataType, int unaryOp);
int htDestroyTensorDescriptor(htTensorDescriptor* desc);

/* hiptensor.hpp:108-111 (hiptensor.cpp:256-321) */
int htGetAlignmentRequirement(const htHandle* handle, const void* ptr, const htTensorDescriptor* desc,
                              uint32_t* alignmentRequirement);

/* hiptensor.hpp:89-98 (library/src/permutation/hiptensor_permutation.cpp:43-279).
 * typeScalar: 0 f32, 2 f16 (type alpha points to). */
int htPermutation(const htHandle* handle, const void* alpha, const void* A, const htTensorDescriptor* descA,
                  const int32_t* modeA, void* B, const htTensorDescriptor* descB, const int32_t* modeB,
                  int typeScalar, void* stream);

/* hiptensor.hpp:131-145 (library/src/contraction/hiptensor_contraction.cpp:71-219).
 * descC == NULL selects the scale form D = alpha*A*B.
 * typeCompute: 1 f16, 4 f32, 16 f64, 1024 bf16 (hiptensorComputeType_t). */
int htCreateContractionDescriptor(const htHandle* handle, htContractionDesc** desc,
                                  const htTensorDescriptor* descA, const int32_t* modeA, uint32_t alignA,
                                  const htTensorDescriptor* descB, const int32_t* modeB, uint32_t alignB,
                                  const htTensorDescriptor* descC, const int32_t* modeC, uint32_t alignC,
                                  const htTensorDescriptor* descD, const int32_t* modeD, uint32_t alignD,
                                  int typeCompute);
int htDestroyContractionDescriptor(htContractionDesc* desc);

/* hiptensor.hpp:157-159 (hiptensor_contraction.cpp:221-316). algo: -1 default, -6 patient, -8 actor-critic. */
int htCreateContractionFind(const htHandle* handle, htContractionFind** find, int algo);
int htDestroyContractionFind(htContractionFind* find);

/* hiptensor.hpp:170-174 (hiptensor_contraction.cpp:318-419). pref: 1 min, 2 recommended, 3 max. */
int htContractionGetWorkspaceSize(const htHandle* handle, const htContractionDesc* desc,
                                  const htContractionFind* find, int pref, uint64_t* workspaceSize);

/* hiptensor.hpp:191-195 (hiptensor_contraction.cpp:421-604) */
int htCreateContractionPlan(const htHandle* handle, htContractionPlan** plan, const htContractionDesc* desc,
                            const htContractionFind* find, uint64_t workspaceSize);
int htDestroyContractionPlan(htContractionPlan* plan);

/* hiptensor.hpp:218-228 (hiptensor_contraction.cpp:606-855). alpha/beta typed by the compute type. */
int htContraction(const htHandle* handle, const htContractionPlan* plan, const void* alpha, const void* A,
                  const void* B, const void* beta, const void* C, void* D, void* workspace,
                  uint64_t workspaceSize, void* stream);

/* hiptensor.hpp:255-271 (library/src/reduction/hiptensor_reduction.cpp:174-381).
 * opReduce: 3 add, 5 mul, 6 max, 7 min. */
int htReduction(const htHandle* handle, const void* alpha, const void* A, const htTensorDescriptor* descA,
                const int32_t* modeA, const void* beta, const void* C, const htTensorDescriptor* descC,
                const int32_t* modeC, void* D, const htTensorDescriptor* descD, const int32_t* modeD,
                int opReduce, int typeCompute, void* workspace, uint64_t workspaceSize, void* stream);

/* hiptensor.hpp:290-302 (hiptensor_reduction.cpp:383-399) */
int htReductionGetWorkspaceSize(const htHandle* handle, const void* A, const htTensorDescriptor* descA,
                                const int32_t* modeA, const void* C, const htTensorDescriptor* descC,
                                const int32_t* modeC, const void* D, const htTensorDescriptor* descD,
                                const int32_t* modeD, int opReduce, int typeCompute, uint64_t* workspaceSize);

/* No counterpart in the reference. hiptensorReduction for callers that are not allowed to allocate
 * device memory while they work: a plug-in inside a host application that has claimed the whole device
 * heap, a latency-critical loop where cudaMalloc's implicit device synchronisation is not acceptable, a
 * service whose policy forbids device allocations once start-up is over. The scratch of the two-pass reduction (few outputs, long reduced
 * range) is a fixed 8 KiB array inside the library, present on every device that loads the library until
 * the process ends; the call makes no cudaMalloc / cudaFree and uses no caller workspace. Inputs and
 * outputs are still the caller's. Limits and rules:
 *  - a reduction of long contiguous rows whose two-pass scratch would exceed 8 KiB returns 19
 *    (INSUFFICIENT_WORKSPACE) and does nothing; use htReduction with a workspace for it (on B200 this only
 *    concerns fp64 reductions with several hundred outputs). Reductions of short rows or with a contiguous kept
 *    mode use as many slices as the 8 KiB hold, or a single pass;
 *  - the first call on a device looks up the array's device address; make that first call outside any
 *    stream capture;
 *  - all calls on one device share the array, and it keeps the last call's contents. Nothing in it needs
 *    clearing (the first pass overwrites every slot the second pass reads), but two such calls that run
 *    at the same time on one device (different streams) race on it: keep them on one stream or order
 *    them with events. */
int htReductionNoAlloc(const htHandle* handle, const void* alpha, const void* A, const htTensorDescriptor* descA,
                       const int32_t* modeA, const void* beta, const void* C, const htTensorDescriptor* descC,
                       const int32_t* modeC, void* D, const htTensorDescriptor* descD, const int32_t* modeD,
                       int opReduce, int typeCompute, void* stream);

/* No counterpart in the reference, whose handle is bound to one device (hiptensor_contraction.cpp:263-277).
 * Finishes a reduction whose REDUCED mode is split over several devices: every device calls htReduction on
 * its share of A with alpha = 1 and beta = 0, the partial results (laid out like D) are combined by one
 * all-reduce that uses the reduction's operator (sum, product, min, max), and this call then writes
 * D = alpha * partial + beta * C once, in the order of the single-device epilogue
 * (library/src/reduction/reduction_cpu_reference_impl.hpp:45-64). partial, C and D share descD; C may be
 * NULL (beta is then ignored) and partial may alias D. */
int htReductionFinish(const htHandle* handle, const void* alpha, const void* partial, const void* beta, const void* C,
                      void* D, const htTensorDescriptor* descD, int typeCompute, void* stream);

/* hiptensor.hpp:308-338 (library/src/logger.cpp). mask: OR of 1 error, 2 perf, 4 hint, 8 heuristics, 16 api. */
int htLoggerSetMask(int32_t mask);
int htLoggerOpenFile(const char* logFile);

/* Introspection of the host-side planner (no device work; usable without a GPU).
 * Each writes a short human-readable description of the plan the library would run
 * (folded extents, kernel family, tile shape) into buf and returns a status code.
 * They replace nothing in the reference: its selection is CK instance enumeration
 * (library/src/contraction/contraction_selection.cpp:44-195,1687-2214). */
int htDescribePermutationPlan(uint32_t numModes, const int64_t* lensA, const int32_t* modeA, const int32_t* modeB,
                              int dataTypeA, int dataTypeB, char* buf, uint64_t bufSize);
int htDescribeReductionPlan(uint32_t numModesA, const int64_t* lensA, const int64_t* stridesA,
                            const int32_t* modeA, uint32_t numModesD, const int64_t* lensD,
                            const int64_t* stridesD, const int32_t* modeD, int dataType, char* buf,
                            uint64_t bufSize);
int htDescribeContractionPlan(uint32_t numModesA, const int64_t* lensA, const int64_t* stridesA,
                              const int32_t* modeA, int dataTypeA, uint32_t numModesB, const int64_t* lensB,
                              const int64_t* stridesB, const int32_t* modeB, int dataTypeB, uint32_t numModesD,
                              const int64_t* lensD, const int64_t* stridesD, const int32_t* modeD, int dataTypeD,
                              int hasC, int typeCompute, char* buf, uint64_t bufSize);

/* Name of the kernel family the last call on this thread launched ("" if none).
 * For tests and the bench, to show which CUDA path ran. */
const char* htLastKernelName(void);
/* Device status word of the handle: 0, or the code a kernel left when one of its bounded device-side waits ran
 * out (1 permutation, 2 single-CTA f16 kernel, 3 CTA-pair f16 kernel, 4 fp32 tensor-core kernel). Reading does not
 * clear it; the next operation on the handle reports HIPTENSOR_STATUS_EXECUTION_FAILED once and clears it. No
 * reference counterpart: the reference's kernels have no device-side waits. */
int htGetDeviceStatus(const htHandle* handle, int32_t* status);
/* Test aid (host-side fault injection): writes the status word as a timed-out kernel would, so that the error
 * path of the next operation can be exercised without making a kernel wait. */
int htInjectDeviceStatus(const htHandle* handle, int32_t code);
/* The library reads its variant switches (environment variables HTB_*, which choose between shipped kernel
 * variants and never change a result beyond the order of summation) once when it is loaded; this reads them
 * again. For tests that set a switch after loading the library. */
void htReloadSwitches(void);
/* Number of kernel launches made by this library since load (all threads). */
uint64_t htKernelLaunchCount(void);

#ifdef __cplusplus
}
#endif
#endif /* HIPTENSOR_B200_H */
