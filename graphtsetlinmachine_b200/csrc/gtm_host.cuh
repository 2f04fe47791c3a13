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


// Stream-ordered allocation from a memory pool that belongs to this library (one per device, created on first use):
// freed blocks stay cached in it, so graph sets and result buffers that come and go with every scoring call cost no
// cudaMalloc / cudaFree (both of which synchronise the device).  The device's default pool, which other allocators of
// the process share, is left as it is.
inline cudaMemPool_t *gtm_pools()
{
    static cudaMemPool_t pools[64];
    return pools;
}

inline int pool_prepare(int device)
{
    if (device < 0 || device >= 64) return fail(GTM_ERR_ARG, "device ordinal %d beyond the 64 this library keeps a memory pool for", device);
    if (gtm_pools()[device]) return GTM_OK;
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = device;
    cudaMemPool_t pool;
    GTM_CU(cudaMemPoolCreate(&pool, &props));
    unsigned long long keep = ~0ull;
    GTM_CU(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
    gtm_pools()[device] = pool;
    return GTM_OK;
}

// Allocates on the CURRENT device (every entry point binds the model's device first).
template <class T>
inline int pool_alloc(T **p, size_t count, cudaStream_t s)
{
    *p = nullptr;
    if (count == 0) count = 1;
    int device = 0;
    GTM_CU(cudaGetDevice(&device));
    GTM_TRY(pool_prepare(device));
    GTM_CU(cudaMallocFromPoolAsync((void **)p, count * sizeof(T), gtm_pools()[device], s));
    return GTM_OK;
}
