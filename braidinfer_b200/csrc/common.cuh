// Shared helpers of the sm_100a kernels: element types, conversions, error reporting.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

// Element type codes used across the C interface.
#define BRAID_F32 0
#define BRAID_BF16 1

// Error codes returned by every entry point: 0 is success, a positive value is a
// cudaError_t, a negative value is a refusal by the entry point itself whose text
// braid_last_error() returns.
#define BRAID_OK 0
#define BRAID_REFUSED (-1)

#ifdef __cplusplus
extern "C" {
#endif
const char* braid_last_error(void);
#ifdef __cplusplus
}
#endif

void braid_set_error(const char* fmt, ...);

#define BRAID_REFUSE(...)            \
    do {                             \
        braid_set_error(__VA_ARGS__); \
        return BRAID_REFUSED;        \
    } while (0)

#define BRAID_LAUNCH_CHECK()                         \
    do {                                             \
        cudaError_t e__ = cudaGetLastError();        \
        if (e__ != cudaSuccess) {                    \
            braid_set_error("%s:%d: %s", __FILE__, __LINE__, cudaGetErrorString(e__)); \
            return (int)e__;                         \
        }                                            \
        return BRAID_OK;                             \
    } while (0)

// Programmatic dependent launch.  Every kernel of the library is launched with the
// attribute that lets it begin while its predecessor in the stream drains, calls
// pdl_trigger() at its top (so that its own successor may be scheduled early) and
// pdl_wait() before its first access to memory that an earlier kernel may have written
// (or may still read).  What comes before pdl_wait() must touch only weights and the
// kernel's own shared or tensor memory.  BRAIDINFER_PDL=0 in the environment turns the
// attribute off; the two instructions are then no-ops.
int braid_pdl_enabled(void);

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t braid_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = braid_pdl_enabled();
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads, same order every time; all threads get the result.
__device__ __forceinline__ float block_sum(float v, float* smem32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[warp] = v;
    __syncthreads();
    const int nw = (blockDim.x + 31) >> 5;
    float t = (lane < nw) ? smem32[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
