// The f32 helper ops of the per-token decode step (the non-GEMV entry points of
// src/cuda.rs:20-54): residual/bias adds, RMSNorm, RoPE (+YaRN), KV append,
// attention scores / sink-softmax / value sum, SwiGLU.  Semantics follow
// src/cuda_kernels.cu:545-698 and :1194-1265; launch shapes are this project's own.
#pragma once

#include "common.cuh"

namespace qz {

__global__ void vec_add_kernel(float *__restrict__ dst, const float *__restrict__ src, int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] += src[i];
}

__global__ void vec_scale_add_kernel(float *__restrict__ dst, const float *__restrict__ src, float scale, int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] += scale * src[i];
}

__global__ void vec_zero_kernel(float *__restrict__ dst, int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) dst[i] = 0.f;
}

// block-wide sum / max through warp shuffles and one shared-memory hop
template <bool IS_MAX>
__device__ __forceinline__ float block_reduce(float v, float *sm)
{
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        float o = __shfl_xor_sync(0xFFFFFFFFu, v, off);
        v = IS_MAX ? fmaxf(v, o) : v + o;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
    __syncthreads();   // sm may still be read from a previous call
    if (lane == 0) sm[warp] = v;
    __syncthreads();
    v = (lane < nw) ? sm[lane] : (IS_MAX ? -INFINITY : 0.f);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        float o = __shfl_xor_sync(0xFFFFFFFFu, v, off);
        v = IS_MAX ? fmaxf(v, o) : v + o;
    }
    return v;
}

// out[i] = x[i] * rsqrt(mean(x^2) + 1e-5) * w[i]; the epsilon is fixed at 1e-5 as
// in the reference kernel (src/cuda_kernels.cu:573).  out may alias x.
__global__ void rms_norm_kernel(float *out, const float *x, const float *__restrict__ w, int n)
{
    __shared__ float sm[32];
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = block_reduce<false>(ss, sm);
    const float r = rsqrtf(ss / (float)n + 1e-5f);
    for (int i = threadIdx.x; i < n; i += blockDim.x) out[i] = x[i] * r * w[i];
}

// RoPE with optional YaRN frequency blend, src/cuda_kernels.cu:579-608: thread i of
// head h rotates the pair (i, i+half) (NEOX) or (2i, 2i+1) (NORM) by pos * inv_freq_i.
__global__ void rope_yarn_kernel(float *x, int head_dim, int pos, float theta, float yarn_scale, int yarn_orig_ctx,
                                 int neox)
{
    const int i = threadIdx.x, half = head_dim >> 1;
    if (i >= half) return;
    float *xh = x + (size_t)blockIdx.x * head_dim;
    const float PI = 3.14159265358979f;
    float inv = 1.f / powf(theta, 2.f * (float)i / (float)head_dim);
    float eff = inv;
    if (yarn_scale > 1.f && yarn_orig_ctx > 0) {
        float hi_w = (float)yarn_orig_ctx / 32.f, lo_w = (float)yarn_orig_ctx / 1.f;
        float wavelen = 2.f * PI / inv;
        float ramp = fmaxf(0.f, fminf(1.f, (lo_w - wavelen) / (lo_w - hi_w)));
        eff = ramp * inv + (1.f - ramp) * (inv / yarn_scale);
    }
    float s, c;
    sincosf((float)pos * eff, &s, &c);
    const int i0 = neox ? i : 2 * i, i1 = neox ? i + half : 2 * i + 1;
    const float a = xh[i0], b = xh[i1];
    xh[i0] = a * c - b * s;
    xh[i1] = a * s + b * c;
}

__global__ void kv_append_kernel(float *__restrict__ k_cache, float *__restrict__ v_cache, const float *__restrict__ k,
                                 const float *__restrict__ v, int pos, int kv_dim)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kv_dim) {
        k_cache[(size_t)pos * kv_dim + i] = k[i];
        v_cache[(size_t)pos * kv_dim + i] = v[i];
    }
}

// scores[head*max_seq + t] = scale * <q[head], K[t, kv_head]>, kv_head = head*n_kv/n_heads
// (src/cuda_kernels.cu:1194-1209).  One warp per (head, t), 8 warps per CTA.
__global__ void attn_score_all_kernel(float *__restrict__ scores, const float *__restrict__ q,
                                      const float *__restrict__ k_cache, int n_heads, int n_kv_heads, int seq_len,
                                      int head_dim, int kv_dim, int max_seq, float scale)
{
    const int head = blockIdx.x;
    const int t = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= seq_len) return;
    const int kv_head = (head * n_kv_heads) / n_heads;
    const float *qh = q + (size_t)head * head_dim;
    const float *kt = k_cache + (size_t)t * kv_dim + (size_t)kv_head * head_dim;
    float acc = 0.f;
    for (int i = lane; i < head_dim; i += 32) acc = fmaf(qh[i], kt[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) scores[(size_t)head * max_seq + t] = acc * scale;
}

// In-place softmax of x[0..n) with an optional sink logit that joins only the
// partition function (src/cuda_kernels.cu:639-666, 1214-1247); sink <= -1e29 means none.
__device__ __forceinline__ void softmax_sink_row(float *x, int n, float sink, float *sm)
{
    const bool has_sink = sink > -1e29f;
    float mx = -1e30f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, x[i]);
    mx = block_reduce<true>(mx, sm);
    mx = fmaxf(mx, has_sink ? sink : -1e30f);
    float sum = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float e = expf(x[i] - mx);
        x[i] = e;
        sum += e;
    }
    sum = block_reduce<false>(sum, sm);
    const float total = sum + (has_sink ? expf(sink - mx) : 0.f);
    for (int i = threadIdx.x; i < n; i += blockDim.x) x[i] /= total;
}

__global__ void softmax_sink_all_kernel(float *scores, int seq_len, int max_seq, const float *__restrict__ sinks)
{
    __shared__ float sm[32];
    softmax_sink_row(scores + (size_t)blockIdx.x * max_seq, seq_len, sinks ? sinks[blockIdx.x] : -INFINITY, sm);
}

__global__ void softmax_sink_kernel(float *x, int n, float sink)
{
    __shared__ float sm[32];
    softmax_sink_row(x, n, sink, sm);
}

// out[head*head_dim + i] = sum_t scores[head, t] * V[t, kv_head, i]
// (src/cuda_kernels.cu:1251-1265).  One CTA per head, thread i owns output i and
// walks t, so V rows are read coalesced.
__global__ void attn_values_all_kernel(float *__restrict__ out, const float *__restrict__ scores,
                                       const float *__restrict__ v_cache, int n_heads, int n_kv_heads, int seq_len,
                                       int head_dim, int kv_dim, int max_seq)
{
    const int head = blockIdx.x;
    const int kv_head = (head * n_kv_heads) / n_heads;
    const float *s = scores + (size_t)head * max_seq;
    for (int i = threadIdx.x; i < head_dim; i += blockDim.x) {
        const float *v = v_cache + (size_t)kv_head * head_dim + i;
        float acc = 0.f;
        for (int t = 0; t < seq_len; t++) acc = fmaf(s[t], v[(size_t)t * kv_dim], acc);
        out[(size_t)head * head_dim + i] = acc;
    }
}

// silu(gate) * up, src/cuda_kernels.cu:693-698
__global__ void swiglu_kernel(float *__restrict__ out, const float *__restrict__ gate, const float *__restrict__ up,
                              int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float g = gate[i];
    out[i] = (g / (1.f + expf(-g))) * up[i];
}

// clamped variant, src/cuda_kernels.cu:683-690
__global__ void swiglu_oai_kernel(float *__restrict__ out, const float *__restrict__ gate,
                                  const float *__restrict__ up, int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float alpha = 1.702f, limit = 7.f;
    float g = fminf(gate[i], limit);
    float u = fmaxf(-limit, fminf(limit, up[i]));
    out[i] = (g / (1.f + expf(-alpha * g))) * (u + 1.f);
}

}  // namespace qz
