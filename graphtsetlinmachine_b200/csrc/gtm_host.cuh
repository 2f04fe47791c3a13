// Host-side helpers shared by the translation unit: last-error text, status macros, device allocation.
#pragma once
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/gtm_b200.h"

// ----------------------------------------------------------------------------------------------- errors
inline std::string &gtm_error_text()
{
    static thread_local std::string text;
    return text;
}

inline int fail(int code, const char *fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    gtm_error_text() = buf;
    return code;
}

#define GTM_CU(call)                                                                              \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess)                                                                    \
            return fail(e_ == cudaErrorMemoryAllocation ? GTM_ERR_OOM : GTM_ERR_CUDA, "%s failed: %s", #call, \
                        cudaGetErrorString(e_));                                                  \
    } while (0)

#define GTM_TRY(call)            \
    do {                         \
        int s_ = (call);         \
        if (s_ != GTM_OK) return s_; \
    } while (0)

template <class T>
inline int dev_alloc(T **p, size_t count)
{
    *p = nullptr;
    if (count == 0) count = 1;
    GTM_CU(cudaMalloc((void **)p, count * sizeof(T)));
    return GTM_OK;
}


// Stream-ordered allocation from the device's default memory pool, whose release threshold is raised once per
// device so that freed blocks stay cached: graph sets and result buffers that come and go with every scoring call
// then cost no cudaMalloc / cudaFree (both of which synchronise the device).
inline int pool_prepare(int device)
{
    static bool done[64];
    if (device < 0 || device >= 64 || done[device]) return GTM_OK;
    cudaMemPool_t pool;
    GTM_CU(cudaDeviceGetDefaultMemPool(&pool, device));
    unsigned long long keep = ~0ull;
    GTM_CU(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
    done[device] = true;
    return GTM_OK;
}

template <class T>
inline int pool_alloc(T **p, size_t count, cudaStream_t s)
{
    *p = nullptr;
    if (count == 0) count = 1;
    GTM_CU(cudaMallocAsync((void **)p, count * sizeof(T), s));
    return GTM_OK;
}
