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
//   wait:  a one-CTA kernel on each rank bumps its own wait counter and polls its local flag array
//          until every slot has reached that count: all slices of the current exchange have landed.
//          The poll is bounded; when it runs out the status word is set and the kernel returns.
//
// Both counters live in device memory, so a recorded graph can be replayed: the n-th wait always
// pairs with the n-th push of every rank.  A region of the window may be rewritten only after an
// exchange into a different region has completed in between (ranks run at most one exchange
// ahead of one another, because the next push depends on data of the previous wait).
#pragma once

#include "common.cuh"

namespace qz {

constexpr int MGPU_MAX_RANKS = 8;
constexpr int MGPU_CTRL_BYTES = 256;   // flags[8] | cta counter | pushes | waits
constexpr long long MGPU_WAIT_CYCLES = 1000000000LL;   // ~0.5 s

struct MgpuCtrl {
    int flags[MGPU_MAX_RANKS];   // flags[r] = number of exchanges rank r has completed into this window
    int cta_counter;             // CTAs of the running push kernel that have finished
    int pushes;                  // exchanges this rank has pushed
    int waits;                   // exchanges this rank has waited for
};

struct PushArgs {
    float *data[MGPU_MAX_RANKS];      // data area of every rank's window
    MgpuCtrl *ctrl[MGPU_MAX_RANKS];   // control words of every rank's window
    int n;                            // ranks (0 = no push: plain local store)
    int rank;
    long long dst_off;                // element offset of row 0 of this slice inside the data area
};

__device__ __forceinline__ int ld_acquire_sys(const int *p)
{
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int *p, int v)
{
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by ONE thread of a CTA after all of the CTA's remote stores were followed by
// __threadfence_system() and a CTA-level barrier.  The last CTA publishes the exchange.
__device__ __forceinline__ void push_publish(const PushArgs &p, int total_ctas)
{
    MgpuCtrl *mine = p.ctrl[p.rank];
    __threadfence();
    const int prev = atomicAdd(&mine->cta_counter, 1);
    if (prev == total_ctas - 1) {
        __threadfence_system();
        mine->cta_counter = 0;
        const int e = mine->pushes + 1;
        mine->pushes = e;
        for (int r = 0; r < p.n; r++) st_release_sys(&p.ctrl[r]->flags[p.rank], e);
    }
}

// Any-shape push: src is this rank's [M x n_local] block (row stride n_local); it lands in every
// window at dst_off + m * dst_ld + j.  Used for GEMM outputs and for GEMVs the fused epilogue
// does not cover.
__global__ void mgpu_push_rows_kernel(const float *__restrict__ src, int M, int n_local, long long dst_ld, PushArgs p)
{
    const long long total = (long long)M * n_local;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long m = i / n_local, j = i - m * n_local;
        const float v = src[i];
        for (int r = 0; r < p.n; r++) p.data[r][p.dst_off + m * dst_ld + j] = v;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) push_publish(p, gridDim.x);
}

// One CTA, one lane per rank.
__global__ void mgpu_wait_kernel(MgpuCtrl *mine, int n, int *status)
{
    __shared__ int expected;
    if (threadIdx.x == 0) {
        expected = mine->waits + 1;
        mine->waits = expected;
    }
    __syncthreads();
    if ((int)threadIdx.x < n) {
        const long long t0 = clock64();
        while (ld_acquire_sys(&mine->flags[threadIdx.x]) < expected) {
            if (clock64() - t0 > MGPU_WAIT_CYCLES) {
                atomicExch(status, QZ_ERR_TIMEOUT);
                break;
            }
            __nanosleep(100);
        }
    }
}

}  // namespace qz
