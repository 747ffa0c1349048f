// Shared host/device helpers for the quartz_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/quartz_b200.h"

namespace qz {

// ggml type ids (src/gguf.rs:172-188 in the reference; 2, 3 and 18 are additions)
enum : uint32_t {
    T_F32 = 0, T_F16 = 1, T_Q4_0 = 2, T_Q4_1 = 3, T_Q5_0 = 6, T_Q5_1 = 7, T_Q8_0 = 8,
    T_Q2_K = 10, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ2_XXS = 16, T_IQ2_XS = 17,
    T_IQ3_XXS = 18, T_IQ4_NL = 20, T_IQ3_S = 21, T_IQ2_S = 22, T_BF16 = 30
};

// Sticky error codes (QZ_OK, QZ_ERR_*) come from include/quartz_b200.h.

void set_error(int code, const char *what);
cudaStream_t stream();   // stream every launch of this library goes to
int sm_count();

#define QZ_CUDA_CHECK(expr)                                                        \
    do {                                                                           \
        cudaError_t e__ = (expr);                                                  \
        if (e__ != cudaSuccess) ::qz::set_error(QZ_ERR_CUDA, cudaGetErrorString(e__)); \
    } while (0)

extern long long g_launch_count;   // kernels launched by this library so far
#define QZ_LAUNCH_CHECK()                  \
    do {                                   \
        ::qz::g_launch_count++;            \
        QZ_CUDA_CHECK(cudaGetLastError()); \
    } while (0)

// Programmatic dependent launch: a kernel launched with the "programmatic stream serialization"
// attribute may begin while its predecessor in the stream is still running; pdl_wait() blocks until
// the predecessor has completed and its writes are visible (a no-op for ordinary launches), and
// pdl_trigger() lets the successor begin.  Code before pdl_wait() may touch only data no kernel writes
// (weights, codebooks).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ float h2f(uint16_t bits)
{
    return __half2float(__ushort_as_half(bits));
}

__device__ __forceinline__ uint16_t ld_u16(const uint8_t *p)
{
    return (uint16_t)(p[0] | (p[1] << 8));
}

__device__ __forceinline__ uint32_t ld_u32_bytes(const uint8_t *p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    return v;
}

// Streaming 128-bit load: weights are read exactly once, keep them out of L1.
__device__ __forceinline__ uint4 ld_stream(const void *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ uint32_t ld_stream_u32(const void *p)
{
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ uint16_t ld_stream_u16(const void *p)
{
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

}  // namespace qz
