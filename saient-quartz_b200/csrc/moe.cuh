// Batched mixture-of-experts FFN: out[t] = sum over the token's experts e of w(t,e) *
// down_e(swiglu(gate_e x_t, up_e x_t)), the batched form of the reference's per-token MoE branch
// (src/main.rs:941-990 on the CPU, src/cuda.rs:673-800 on the GPU, where every expert GEMV of every
// token is a launch of its own).  Tokens are grouped by expert on the host (the reference routes on
// the host as well, src/cuda.rs:673-701); per expert the token rows are gathered, pushed through
// three tensor-core GEMMs and scattered back with their routing weight.
#pragma once

#include "common.cuh"

namespace qz {

// rows[i] = index of the source row of gathered row i; one thread per float4
__global__ void moe_gather_kernel(const float *__restrict__ x, float *__restrict__ xe, const int *__restrict__ rows, int n_rows,
                                  int K)
{
    const int k4 = K >> 2;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_rows * k4) return;
    const int r = (int)(i / k4), c = (int)(i - (long long)r * k4);
    ((float4 *)xe)[i] = ((const float4 *)(x + (size_t)rows[r] * K))[c];
}

// h = swiglu(g, u) in place of g (src/cuda_kernels.cu:683-698; oai = the clamped variant)
__global__ void moe_swiglu_kernel(float *__restrict__ g, const float *__restrict__ u, long long n, int oai)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float a = g[i], b = u[i];
    if (oai) {
        const float x = fminf(a, 7.f), y = fmaxf(-7.f, fminf(7.f, b));
        g[i] = (x / (1.f + expf(-1.702f * x))) * (y + 1.f);
    } else {
        g[i] = (a / (1.f + expf(-a))) * b;
    }
}

// out[rows[i]] += w[i] * y[i]; a token appears at most once per expert, and the experts' launches are
// ordered by the stream, so plain read-modify-write is race-free and the sum order is fixed
__global__ void moe_scatter_kernel(float *__restrict__ out, const float *__restrict__ y, const int *__restrict__ rows,
                                   const float *__restrict__ w, int n_rows, int K)
{
    const int k4 = K >> 2;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_rows * k4) return;
    const int r = (int)(i / k4), c = (int)(i - (long long)r * k4);
    const float s = w[r];
    float4 *dst = (float4 *)(out + (size_t)rows[r] * K) + c;
    const float4 v = ((const float4 *)y)[i];
    float4 o = *dst;
    o.x = fmaf(s, v.x, o.x);
    o.y = fmaf(s, v.y, o.y);
    o.z = fmaf(s, v.z, o.z);
    o.w = fmaf(s, v.w, o.w);
    *dst = o;
}

}  // namespace qz
