// Phase time stamps for a build made with -DBRAID_TRACE (BRAIDINFER_TRACE=1 in the environment
// of the process that builds the library).  A kernel that wants to be traced declares a
// buffer with BRAID_TRACE_BUFFER(name, ctas) at file scope, takes a row at its top with
// braid_trace_open() and stamps %globaltimer (nanoseconds) into the row's eight slots at the
// boundaries of its phases; the host reads all rows with braid_<name>_trace_read().  Row
// [launch][cta]: every CTA counts its own launches, so no ordering between CTAs is needed.
// Without the flag everything here compiles to nothing.  The reference has cycle counters per
// op behind a build flag for the same purpose (kernels/op_profile.h).
#pragma once
#include "common.cuh"

#define BRAID_TRACE_SLOTS 8
#define BRAID_TRACE_LAUNCHES 64

#ifdef BRAID_TRACE
__device__ __forceinline__ unsigned long long braid_trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#define BRAID_TRACE_BUFFER(name, ctas)                                                                     \
    static __device__ unsigned long long name##_trace[BRAID_TRACE_LAUNCHES * (ctas) * BRAID_TRACE_SLOTS];  \
    static __device__ unsigned int name##_trace_count[ctas];                                               \
    static unsigned long long name##_trace_zero[BRAID_TRACE_LAUNCHES * (ctas) * BRAID_TRACE_SLOTS];        \
    extern "C" int braid_##name##_trace_ctas(void) { return ctas; }                                        \
    /* copies every row to `host` after the device has gone idle; `reset` clears rows and counts */        \
    extern "C" int braid_##name##_trace_read(unsigned long long* host, int reset) {                        \
        cudaError_t e = cudaDeviceSynchronize();                                                           \
        if (e == cudaSuccess && host) e = cudaMemcpyFromSymbol(host, name##_trace, sizeof(name##_trace));  \
        if (e == cudaSuccess && reset) {                                                                   \
            e = cudaMemcpyToSymbol(name##_trace, name##_trace_zero, sizeof(name##_trace));                 \
            if (e == cudaSuccess) e = cudaMemcpyToSymbol(name##_trace_count, name##_trace_zero, sizeof(unsigned int) * (ctas)); \
        }                                                                                                  \
        return (int)e;                                                                                     \
    }
// The row of this CTA's current launch, or null when the buffer is full or the CTA beyond it.  One thread calls it.
#define braid_trace_open(name, ctas)                                                                       \
    ((blockIdx.x < (ctas) && name##_trace_count[blockIdx.x] < BRAID_TRACE_LAUNCHES)                        \
         ? &name##_trace[((size_t)(name##_trace_count[blockIdx.x]++) * (ctas) + blockIdx.x) * BRAID_TRACE_SLOTS] \
         : nullptr)
#define BRAID_STAMP(row, slot) do { if (row) (row)[slot] = braid_trace_now(); } while (0)
#define BRAID_STAMP_ONCE(row, slot) do { if ((row) && (row)[slot] == 0) (row)[slot] = braid_trace_now(); } while (0)
#else
#define BRAID_TRACE_BUFFER(name, ctas)
#define braid_trace_open(name, ctas) nullptr
#define BRAID_STAMP(row, slot) do { } while (0)
#define BRAID_STAMP_ONCE(row, slot) do { } while (0)
#endif
