// Row-sharded layers over the GPUs of one box: the exchange of output slices without a collective
// library call.  The reference is single-GPU (src/cuda.rs has one device, stream 0); this is the
// multi-GPU form of its GEMV for layers sharded over the output dimension.
//
// Every rank owns a "window": one cudaMalloc'ed buffer whose first 256 bytes hold control words and
// whose rest holds f32 data.  Windows are mapped into every other rank's address space (CUDA IPC),
// so a kernel on rank r can store straight into rank p's window over NVLink.
//
//   push:  the kernel that produced a slice of y stores it at the same offset of EVERY rank's
//          window (its own included), fences at system scope, and the last CTA to finish bumps
//          this rank's push counter and stores it, with release semantics, into slot [r] of every
//          rank's flag array.
//   wait:  every rank issues the same sequence of pushes, so "all slices of the exchanges I have
//          pushed so far have landed" is: every slot of my flag array has reached MY OWN push
//          counter.  The poll runs in a one-CTA kernel, or in the prologue of the kernel that
//          consumes the data (the activation conversion of the next GEMV, whose weight stream has
//          then already started).  It is bounded; when it runs out the status word is set and the
//          kernel carries on to its end.
//
// The counters live in device memory, so a recorded graph can be replayed.  A region of the window
// may be rewritten only after a wait that followed an exchange into a different region (a rank
// can run at most one wait ahead of the slowest one).
#pragma once

#include "common.cuh"

namespace qz {

constexpr int MGPU_MAX_RANKS = 8;
constexpr int MGPU_CTRL_BYTES = 256;   // flags[8] | cta counter | pushes
constexpr long long MGPU_WAIT_CYCLES = 1000000000LL;   // ~0.5 s

struct MgpuCtrl {
    int flags[MGPU_MAX_RANKS];   // flags[r] = number of exchanges rank r has completed into this window
    int cta_counter;             // CTAs of the running push kernel that have finished
    int pushes;                  // exchanges this rank has pushed
};

struct PushArgs {
    float *data[MGPU_MAX_RANKS];      // data area of every rank's window
    MgpuCtrl *ctrl[MGPU_MAX_RANKS];   // control words of every rank's window
    int n;                            // ranks (0 = no push: plain local store)
    int rank;
    long long dst_off;                // element offset of row 0 of this slice inside the data area
    int wait_after;                   // 1: the thread that publishes then waits (bounded) until every rank has published
                                      //    as many exchanges, so the kernel's end is the exchange's end (no wait launch)
};

__device__ __forceinline__ int ld_acquire_sys(const int *p)
{
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(int *p, int v)
{
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by ONE thread of a CTA after a CTA-level barrier that follows all of the CTA's remote
// stores.  The count is a release/acquire read-modify-write at GPU scope: through the barrier it is
// cumulative over the other threads' stores, and the last CTA to count in has thereby acquired every
// CTA's stores.  That CTA publishes the exchange: one system-scope fence, then the new counter
// stored into every rank's flag array.
__device__ __forceinline__ void push_publish(const PushArgs &p, int total_ctas, int *status = nullptr, bool may_wait = false)
{
    MgpuCtrl *mine = p.ctrl[p.rank];
    int prev;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(&mine->cta_counter) : "memory");
    if (prev == total_ctas - 1) {
        mine->cta_counter = 0;
        const int e = mine->pushes + 1;
        mine->pushes = e;
        // ONE system-scope fence, then the flag stores: a release store per peer would repeat the fence
        // (a few microseconds each) once per rank
        __threadfence_system();
        for (int r = 0; r < p.n; r++) st_relaxed_sys(&p.ctrl[r]->flags[p.rank], e);
        if (may_wait && p.wait_after) {
            // the exchange is complete once every rank's flag has reached this rank's own count; bounded like every wait
            const long long t0 = clock64();
            for (int r = 0; r < p.n; r++) {
                while (ld_acquire_sys(&mine->flags[r]) - e < 0) {
                    if (clock64() - t0 > MGPU_WAIT_CYCLES) {
                        if (status) atomicExch(status, QZ_ERR_TIMEOUT);
                        return;
                    }
                    __nanosleep(64);
                }
            }
        }
    }
}

// Any-shape push: src is this rank's [M x n_local] block (row stride n_local); it lands in every
// window at dst_off + m * dst_ld + j.  Used for GEMM outputs and for GEMVs the fused epilogue
// does not cover.
__global__ void mgpu_push_rows_kernel(const float *__restrict__ src, int M, int n_local, long long dst_ld, PushArgs p)
{
    const long long total = (long long)M * n_local;
    // 16 bytes per thread and store when rows, leading dimension, offset and pointers allow it (the usual case:
    // row counts and offsets that are multiples of four); a warp then writes 512 contiguous bytes per rank
    const bool vec = (n_local & 3) == 0 && (dst_ld & 3) == 0 && (p.dst_off & 3) == 0 && (((uintptr_t)src) & 15) == 0;
    if (vec) {
        const long long total4 = total >> 2;
        const int n4 = n_local >> 2;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
            const long long m = i / n4, j = (i - m * n4) << 2;
            const float4 v = __ldcs((const float4 *)src + i);
            for (int r = 0; r < p.n; r++) *(float4 *)(p.data[r] + p.dst_off + m * dst_ld + j) = v;
        }
    } else {
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
            const long long m = i / n_local, j = i - m * n_local;
            const float v = src[i];
            for (int r = 0; r < p.n; r++) p.data[r][p.dst_off + m * dst_ld + j] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) push_publish(p, gridDim.x);
}

// Lanes 0..n-1 of the calling CTA poll this rank's flags until every rank has published as many
// exchanges as this rank has pushed; the caller follows with __syncthreads().
__device__ __forceinline__ void mgpu_poll(const MgpuCtrl *mine, int n, int *status)
{
    if ((int)threadIdx.x < n) {
        const int expected = *(volatile const int *)&mine->pushes;
        const long long t0 = clock64();
        while (ld_acquire_sys(&mine->flags[threadIdx.x]) < expected) {
            if (clock64() - t0 > MGPU_WAIT_CYCLES) {
                atomicExch(status, QZ_ERR_TIMEOUT);
                break;
            }
            __nanosleep(64);
        }
    }
}

__global__ void mgpu_wait_kernel(const MgpuCtrl *mine, int n, int *status)
{
    mgpu_poll(mine, n, status);
}

}  // namespace qz
