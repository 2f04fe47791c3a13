// TEST INFRASTRUCTURE ONLY (checker, never the product path).
//
// A minimal stand-in for the CUDA execution model so that the reference's kernel source
// (GraphTsetlinMachine/kernels.py, read verbatim at build time by oracle/build_ref.py and never copied into
// this repository) compiles as plain C++ with g++ and runs on the host, one "thread" at a time.
//
//  * __global__/__device__ vanish; blockIdx/threadIdx/blockDim/gridDim are thread_local structs that the
//    launchers below set before each call, so a "launch" is a loop over thread indices.  The reference kernels
//    are grid-stride loops, so any launch shape gives the same result; the launchers use one block of
//    `nthreads` threads.
//  * curandState is replaced by a counter-based stream: draw i of stream s is component (i & 3) of
//    Philox4x32-10(counter = (i >> 2, 0, s, 0), key = (seed_lo, seed_hi)), or word i of a caller-supplied
//    recorded buffer.  curand() returns the raw 32-bit draw; curand_uniform() maps it to (0, 1] exactly as
//    curand_uniform.h does (x * 2^-32 + 2^-33 in float; the product is exact, so FMA contraction cannot
//    change the value).  The engine under test consumes the very same streams, which is what makes
//    Tsetlin-automaton updates comparable bit for bit.
#pragma once
#include <climits>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>

#define __global__
#define __device__
#define __host__

struct ref_dim3 { unsigned int x, y, z; };
static thread_local ref_dim3 blockIdx = {0, 0, 0};
static thread_local ref_dim3 threadIdx = {0, 0, 0};
static thread_local ref_dim3 blockDim = {1, 1, 1};
static thread_local ref_dim3 gridDim = {1, 1, 1};

static inline int __popc(unsigned int v) { return __builtin_popcount(v); }
static inline int atomicAdd(int *addr, int v) { int old = *addr; *addr = old + v; return old; }
static inline int max(int a, int b) { return a > b ? a : b; }
static inline int min(int a, int b) { return a < b ? a : b; }

// ---- Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) ----
static inline void ref_philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                     uint32_t k0, uint32_t k1, uint32_t out[4])
{
    for (int r = 0; r < 10; ++r) {
        uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        uint32_t n1 = (uint32_t)p1;
        uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

struct curandState {
    uint64_t stream;        // = clause index in every harness launch
    uint64_t pos;           // draws consumed so far
    uint32_t seed_lo, seed_hi;
    const uint32_t *rec;    // optional recorded draws for this stream (rec_len words), else NULL
    uint64_t rec_len;
};

static inline unsigned int curand(curandState *s)
{
    uint64_t i = s->pos++;
    if (s->rec) return s->rec[i % s->rec_len];
    uint32_t o[4];
    ref_philox4x32_10((uint32_t)(i >> 2), (uint32_t)(i >> 34), (uint32_t)s->stream, (uint32_t)(s->stream >> 32),
                      s->seed_lo, s->seed_hi, o);
    return o[i & 3];
}

static inline float curand_uniform(curandState *s)
{
    unsigned int x = curand(s);
    return (float)x * 2.3283064365386963e-10f + 1.1641532182693481e-10f;   // 2^-32, 2^-33
}
