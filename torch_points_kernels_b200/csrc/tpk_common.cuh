// Shared helpers of the tpk_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/tpk_b200.h"

namespace tpk
{

// Records the text returned by tpk_last_error() for the calling thread.
void set_error(const char* fmt, ...);

// Adds to the process-wide count of kernels this library has launched (or recorded into a
// stream capture); every launch site calls it.
void count_launches(int k);

// Test hook: is `name` (or `name=value`) listed in the environment variable TPK_B200_TEST?
// The only environment variable the library reads; it selects kernels the size heuristics
// would not pick, for tests that compare kernel families.
bool test_path(const char* name);
bool test_value(const char* name, char* out, size_t cap);

// Bits of the sticky device status word reported by tpk_device_status().
constexpr int kStatusWaitAbandoned = 1;  // a bounded wait (cluster exchange, bulk copy) ran out
constexpr int kStatusBadIndex = 2;       // an index outside its tensor was skipped

typedef cudaError_t (*StatusReader)(int* value, int reset);
struct StatusRegistrar
{
    explicit StatusRegistrar(StatusReader r);
};

// Gives the including .cu file its own device status word `g_dev_status` and hooks it into
// tpk_device_status().  Use once per file, at namespace tpk scope.
#define TPK_DEFINE_STATUS_WORD()                                                                   \
    namespace                                                                                      \
    {                                                                                              \
    __device__ int g_dev_status = 0;                                                               \
    cudaError_t read_status_word(int* value, int reset)                                            \
    {                                                                                              \
        cudaError_t err = cudaMemcpyFromSymbol(value, g_dev_status, sizeof(int));                  \
        if (err == cudaSuccess && reset && *value != 0)                                            \
        {                                                                                          \
            const int zero = 0;                                                                    \
            err = cudaMemcpyToSymbol(g_dev_status, &zero, sizeof(int));                            \
        }                                                                                          \
        return err;                                                                                \
    }                                                                                              \
    StatusRegistrar g_status_registrar(read_status_word);                                          \
    }

// gather.cu: gradient of grouping with atomics; gbs = batch stride of grad_out in floats
int grouping_grad_atomic(int b, int c, int n, int npoint, int nsample, const float* grad_out, long long gbs,
                         const int64_t* idx, float* grad_features, cudaStream_t s);

constexpr unsigned kFullMask = 0xffffffffu;
// Dynamic shared memory from which a launcher raises the kernel's limit
// (cudaFuncAttributeMaxDynamicSharedMemorySize).  Well below the 48 KB a launch may use without
// that: the limit counts a kernel's static shared memory too, so a request of exactly 48 KB by a
// kernel with one static mbarrier fails with "invalid argument" unless the limit was raised.
constexpr size_t kDynSmemOptIn = 32 * 1024;
constexpr int kNumSmsB200 = 148;

inline int num_sms()
{
    static int cached = 0;
    if (cached == 0)
    {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
            cached = v;
        else
            cached = kNumSmsB200;
    }
    return cached;
}

// Turns the sticky launch error into a status; never exits the process
// (the reference prints and calls exit(-1), cuda/include/cuda_utils.h:53-63).
inline int check_launch(const char* what)
{
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess)
    {
        set_error("%s: %s", what, cudaGetErrorString(err));
        return TPK_ERR_CUDA;
    }
    return TPK_OK;
}

// Every kernel of the library asks for the same (largest) shared-memory carve-out.  An
// SM changes its L1/shared split only when it is idle, so kernels with different
// preferences cannot share an SM; with one common setting the long-running FPS clusters,
// the search kernels and the row-resident gather kernels co-reside freely.
template <class K>
inline void prefer_max_shared(K kernel)
{
    (void)cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
}

#define TPK_REQUIRE(cond, ...)                                                                     \
    do                                                                                             \
    {                                                                                              \
        if (!(cond))                                                                               \
        {                                                                                          \
            ::tpk::set_error(__VA_ARGS__);                                                         \
            return TPK_ERR_INVALID_ARGUMENT;                                                       \
        }                                                                                          \
    } while (0)

// a*a + b*b + c*c exactly as nvcc's default contraction evaluates the reference's
// left-associated expression: one rounded product, two fused multiply-adds.
// Used by dense ball query (ball_query_gpu.cu:35-36), three_nn (interpolate_gpu.cu:34),
// chamfer (chamfer_dist_gpu.cu:41) and FPS (sampling_gpu.cu:52,56).
__device__ __forceinline__ float sumsq_abc(float a, float b, float c)
{
    return __fmaf_rn(c, c, __fmaf_rn(a, a, __fmul_rn(b, b)));
}

// dist = 0; dist += a*a; dist += b*b; dist += c*c as contracted for the
// partial_dense loop (ball_query_gpu.cu:78-82): three chained fused multiply-adds.
__device__ __forceinline__ float sumsq_loop(float a, float b, float c)
{
    return __fmaf_rn(c, c, __fmaf_rn(b, b, __fmul_rn(a, a)));
}

// ((a*a) + b*b) + c*c with every operation rounded: the arithmetic of the reference's
// CPU kd-tree metric (cpu/include/nanoflann.hpp:488-497, built without FMA).
__device__ __forceinline__ float sumsq_unfused(float a, float b, float c)
{
    return __fadd_rn(__fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b)), __fmul_rn(c, c));
}

__device__ __forceinline__ double sumsq_abc(double a, double b, double c)
{
    return __fma_rn(c, c, __fma_rn(a, a, __dmul_rn(b, b)));
}

}  // namespace tpk
