// Fused decode-step kernels (additions; the reference runs these as separate launches,
// src/cuda.rs:548-823): producers that emit the block-fixed-point activation form the
// streaming GEMVs consume, RoPE+KV-append in one launch, and split-KV decode attention.
#pragma once

#include "decode_ops.cuh"
#include "gemv_stream.cuh"

namespace qz {

// RMSNorm (src/cuda_kernels.cu:563-575) whose result goes straight into activation form;
// optionally also stored as f32.  One CTA; n is a multiple of 4.
__global__ void rms_norm_q_kernel(const float *__restrict__ x, const float *__restrict__ w, int n, XQOut o,
                                  float *__restrict__ out_f32)
{
    __shared__ float sm[32];
    pdl_wait();
    pdl_trigger();
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = block_reduce<false>(ss, sm);
    const float r = rsqrtf(ss / (float)n + 1e-5f);
    const int n4 = n >> 2;
    for (int t0 = 0; t0 < n4; t0 += blockDim.x) {
        const int t = t0 + threadIdx.x;
        const bool valid = t < n4;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (valid) {
            const float4 a = *(const float4 *)(x + 4 * t), b = *(const float4 *)(w + 4 * t);
            v[0] = a.x * r * b.x; v[1] = a.y * r * b.y; v[2] = a.z * r * b.z; v[3] = a.w * r * b.w;
            if (out_f32) *(float4 *)(out_f32 + 4 * t) = make_float4(v[0], v[1], v[2], v[3]);
        }
        quantize4_store(v, t, valid, o);
    }
}

// SwiGLU (src/cuda_kernels.cu:683-698) into activation form.
__global__ void swiglu_q_kernel(const float *__restrict__ gate, const float *__restrict__ up, int n, int oai, XQOut o)
{
    pdl_wait();
    pdl_trigger();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = 4 * t < n;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (valid) {
        const float4 g = *(const float4 *)(gate + 4 * t), u = *(const float4 *)(up + 4 * t);
        const float gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (oai) {
                const float a = fminf(gg[i], 7.f), b = fmaxf(-7.f, fminf(7.f, uu[i]));
                v[i] = (a / (1.f + expf(-1.702f * a))) * (b + 1.f);
            } else {
                v[i] = (gg[i] / (1.f + expf(-gg[i]))) * uu[i];
            }
        }
    }
    quantize4_store(v, t, valid, o);
}

// rotation (cos, sin) of pair i at one position, exactly as rope_kv_kernel / src/cuda_kernels.cu:588-620 compute it
struct RopeArgsLite {
    int pos;
    float theta, yarn_scale;
    int yarn_orig_ctx;
};
__device__ __forceinline__ void rope_cs_lite(const RopeArgsLite &r, int i, int head_dim, float &c, float &s)
{
    const float PI = 3.14159265358979f;
    float inv = 1.f / powf(r.theta, 2.f * (float)i / (float)head_dim);
    float eff = inv;
    if (r.yarn_scale > 1.f && r.yarn_orig_ctx > 0) {
        float hi_w = (float)r.yarn_orig_ctx / 32.f, lo_w = (float)r.yarn_orig_ctx / 1.f;
        float wavelen = 2.f * PI / inv;
        float ramp = fmaxf(0.f, fminf(1.f, (lo_w - wavelen) / (lo_w - hi_w)));
        eff = ramp * inv + (1.f - ramp) * (inv / r.yarn_scale);
    }
    sincosf((float)r.pos * eff, &s, &c);
}

// RoPE on q (n_heads) and k (n_kv_heads) in place, then append k, v to the caches at `pos`:
// cuda_rope_yarn x2 + cuda_kv_append (src/cuda.rs:601-613) as one launch.  grid = n_heads +
// n_kv_heads, block = head_dim/2 rounded up to a warp.
__global__ void rope_kv_kernel(float *q, float *k, const float *__restrict__ v, float *__restrict__ k_cache,
                               float *__restrict__ v_cache, int n_heads, int head_dim, int pos, float theta,
                               float yarn_scale, int yarn_orig_ctx, int neox, int kv_dim)
{
    pdl_wait();
    pdl_trigger();
    const int i = threadIdx.x, half = head_dim >> 1;
    const bool is_k = (int)blockIdx.x >= n_heads;
    const int head = is_k ? blockIdx.x - n_heads : blockIdx.x;
    float *xh = (is_k ? k : q) + (size_t)head * head_dim;
    if (i < half) {
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
        const float r0 = a * c - b * s, r1 = a * s + b * c;
        xh[i0] = r0;
        xh[i1] = r1;
        if (is_k) {
            float *kc = k_cache + (size_t)pos * kv_dim + (size_t)head * head_dim;
            kc[i0] = r0;
            kc[i1] = r1;
        }
    }
    if (is_k) {
        const float *vh = v + (size_t)head * head_dim;
        float *vc = v_cache + (size_t)pos * kv_dim + (size_t)head * head_dim;
        for (int j = i; j < head_dim; j += blockDim.x) vc[j] = vh[j];
    }
}

// ---- batched (prompt) forms: the same ops for n_tok tokens at consecutive positions ----
// RMSNorm of every row of x [n_rows, n] (src/cuda_kernels.cu:563-575 per row); one CTA per row.  out may alias x.
__global__ void rms_norm_rows_kernel(float *out, const float *x, const float *__restrict__ w, int n)
{
    __shared__ float sm[32];
    pdl_wait();
    pdl_trigger();
    const float *xr = x + (size_t)blockIdx.x * n;
    float *orow = out + (size_t)blockIdx.x * n;
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(xr[i], xr[i], ss);
    ss = block_reduce<false>(ss, sm);
    const float r = rsqrtf(ss / (float)n + 1e-5f);
    for (int i = threadIdx.x; i < n; i += blockDim.x) orow[i] = xr[i] * r * w[i];
}

// rope_kv_kernel for token t = blockIdx.y at position pos0 + t: q [n_tok, n_heads*head_dim] and
// k [n_tok, kv_dim] rotated in place, k and v [n_tok, kv_dim] appended to the caches.
__global__ void rope_kv_rows_kernel(float *q, float *k, const float *__restrict__ v, float *__restrict__ k_cache,
                                    float *__restrict__ v_cache, int n_heads, int head_dim, int pos0, float theta,
                                    float yarn_scale, int yarn_orig_ctx, int neox, int kv_dim)
{
    pdl_wait();
    pdl_trigger();
    const int i = threadIdx.x, half = head_dim >> 1, t = blockIdx.y, pos = pos0 + t;
    const bool is_k = (int)blockIdx.x >= n_heads;
    const int head = is_k ? blockIdx.x - n_heads : blockIdx.x;
    float *xh = is_k ? k + (size_t)t * kv_dim + (size_t)head * head_dim
                     : q + (size_t)t * n_heads * head_dim + (size_t)head * head_dim;
    if (i < half) {
        const RopeArgsLite r{pos, theta, yarn_scale, yarn_orig_ctx};
        float s, c;
        rope_cs_lite(r, i, head_dim, c, s);
        const int i0 = neox ? i : 2 * i, i1 = neox ? i + half : 2 * i + 1;
        const float a = xh[i0], b = xh[i1];
        const float r0 = a * c - b * s, r1 = a * s + b * c;
        xh[i0] = r0;
        xh[i1] = r1;
        if (is_k) {
            float *kc = k_cache + (size_t)pos * kv_dim + (size_t)head * head_dim;
            kc[i0] = r0;
            kc[i1] = r1;
        }
    }
    if (is_k) {
        const float *vh = v + (size_t)t * kv_dim + (size_t)head * head_dim;
        float *vc = v_cache + (size_t)pos * kv_dim + (size_t)head * head_dim;
        for (int j = i; j < head_dim; j += blockDim.x) vc[j] = vh[j];
    }
}

// ---- split-KV decode attention -------------------------------------------------------------
// softmax(q K^T * scale [+ sink]) V for one new token, all heads (the three launches of
// src/cuda.rs:627-645 as two).  grid = (n_kv_heads, n_splits): a CTA stages CHUNK key rows and
// value rows of its kv head in shared memory once and serves every query head that maps to
// that kv head (GQA: head*n_kv/n_heads), so K and V are read from HBM exactly once.  Warp w
// handles query heads w, w+4, ...  Each (head, split) leaves (max, sum, unnormalised out[hd])
// in a scratch buffer; attn_combine_kernel merges the splits.
constexpr int ATT_CHUNK = 32;
constexpr int ATT_MAX_HD = 128;

__global__ void __launch_bounds__(128) attn_partial_kernel(float *__restrict__ part, const float *__restrict__ q,
                                                           const float *__restrict__ k_cache,
                                                           const float *__restrict__ v_cache, int n_heads, int n_kv_heads,
                                                           int seq_len, int head_dim, int kv_dim, float scale)
{
    __shared__ float ks[ATT_CHUNK][ATT_MAX_HD + 1];
    __shared__ float vs[ATT_CHUNK][ATT_MAX_HD];
    __shared__ float qs[4][ATT_MAX_HD];
    __shared__ float ps[4][ATT_CHUNK];
    pdl_wait();
    pdl_trigger();
    const int kvh = blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    const int t0 = split * ATT_CHUNK;
    const int nt = min(ATT_CHUNK, seq_len - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // stage K and V rows [t0, t0+nt) of this kv head: all of a thread's loads are issued before
    // the first shared-memory store, so the CTA pays one DRAM round trip, not one per row
    const int hd4 = head_dim >> 2;
    constexpr int MAX_IT = ATT_CHUNK * (ATT_MAX_HD / 4) / 128;   // 8 float4 pairs per thread
    float4 kreg[MAX_IT], vreg[MAX_IT];
#pragma unroll
    for (int it = 0; it < MAX_IT; it++) {
        const int idx = threadIdx.x + it * 128;
        if (idx < nt * hd4) {
            const int t = idx / hd4, c = idx - t * hd4;
            const size_t g = (size_t)(t0 + t) * kv_dim + (size_t)kvh * head_dim + 4 * c;
            kreg[it] = __ldg((const float4 *)(k_cache + g));
            vreg[it] = __ldg((const float4 *)(v_cache + g));
        }
    }
#pragma unroll
    for (int it = 0; it < MAX_IT; it++) {
        const int idx = threadIdx.x + it * 128;
        if (idx < nt * hd4) {
            const int t = idx / hd4, c = idx - t * hd4;
            ks[t][4 * c] = kreg[it].x; ks[t][4 * c + 1] = kreg[it].y; ks[t][4 * c + 2] = kreg[it].z; ks[t][4 * c + 3] = kreg[it].w;
            *(float4 *)&vs[t][4 * c] = vreg[it];
        }
    }
    // query heads of this kv head: those with (head * n_kv_heads) / n_heads == kvh
    const int h_lo = (kvh * n_heads + n_kv_heads - 1) / n_kv_heads;
    const int h_hi = ((kvh + 1) * n_heads + n_kv_heads - 1) / n_kv_heads;
    for (int hb = h_lo; hb < h_hi; hb += 4) {
        const int head = hb + warp;
        const bool live = head < h_hi;
        __syncthreads();   // staging done / previous round's qs no longer read
        if (live)
            for (int i = lane; i < head_dim; i += 32) qs[warp][i] = q[(size_t)head * head_dim + i];
        __syncthreads();
        if (!live) continue;
        // one key position per lane
        float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
        for (int i = 0; i < head_dim; i += 4) {
            c0 = fmaf(qs[warp][i], ks[lane][i], c0);
            c1 = fmaf(qs[warp][i + 1], ks[lane][i + 1], c1);
            c2 = fmaf(qs[warp][i + 2], ks[lane][i + 2], c2);
            c3 = fmaf(qs[warp][i + 3], ks[lane][i + 3], c3);
        }
        float sc = (c0 + c1) + (c2 + c3);
        sc = lane < nt ? sc * scale : -INFINITY;
        float mx = sc;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
        const float p = lane < nt ? expf(sc - mx) : 0.f;
        float sum = p;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
        ps[warp][lane] = p;
        __syncwarp();
        float *dst = part + ((size_t)head * n_splits + split) * (head_dim + 2);
        // lane owns outputs lane, lane+32, lane+64, lane+96 (four independent chains)
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
        for (int t = 0; t < nt; t++) {
            const float pt = ps[warp][t];
            o0 = fmaf(pt, vs[t][lane], o0);
            if (head_dim > 32) o1 = fmaf(pt, vs[t][lane + 32], o1);
            if (head_dim > 64) o2 = fmaf(pt, vs[t][lane + 64], o2);
            if (head_dim > 96) o3 = fmaf(pt, vs[t][lane + 96], o3);
        }
        dst[2 + lane] = o0;
        if (head_dim > 32) dst[2 + lane + 32] = o1;
        if (head_dim > 64) dst[2 + lane + 64] = o2;
        if (head_dim > 96) dst[2 + lane + 96] = o3;
        if (lane == 0) {
            dst[0] = mx;
            dst[1] = sum;
        }
        __syncwarp();
    }
}

// Merge the splits of every head; optionally emit the activation form for the output
// projection.  grid = n_heads, block = head_dim (a multiple of 32, <= 128).
__global__ void attn_combine_kernel(float *__restrict__ out, const float *__restrict__ part, int n_splits, int head_dim,
                                    const float *__restrict__ sinks, XQOut o, int emit_q)
{
    __shared__ float sm[32];
    extern __shared__ float fs[];   // n_splits rescale factors
    pdl_wait();
    pdl_trigger();
    const int head = blockIdx.x, i = threadIdx.x;
    const int stride = head_dim + 2;
    const float *p = part + (size_t)head * n_splits * stride;
    const float sink = sinks ? sinks[head] : -INFINITY;
    const bool has_sink = sink > -1e29f;
    // every thread takes a strided share of the splits' (max, sum) pairs
    float mx = has_sink ? sink : -1e30f;
    for (int s = i; s < n_splits; s += blockDim.x) mx = fmaxf(mx, p[(size_t)s * stride]);
    mx = block_reduce<true>(mx, sm);
    float tot = 0.f;
    for (int s = i; s < n_splits; s += blockDim.x) {
        const float f = expf(p[(size_t)s * stride] - mx);
        fs[s] = f;
        tot = fmaf(f, p[(size_t)s * stride + 1], tot);
    }
    tot = block_reduce<false>(tot, sm);   // (its barriers also publish fs)
    const float total = tot + (has_sink ? expf(sink - mx) : 0.f);
    // sixteen independent loads in flight per thread: the splits' rows sit in L2, this loop is pure latency
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    int s = 0;
    for (; s + 16 <= n_splits; s += 16) {
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; j++) v[j] = p[(size_t)(s + j) * stride + 2 + i];
#pragma unroll
        for (int j = 0; j < 16; j++) a[j & 3] = fmaf(fs[s + j], v[j], a[j & 3]);
    }
    for (; s + 4 <= n_splits; s += 4) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = p[(size_t)(s + j) * stride + 2 + i];
#pragma unroll
        for (int j = 0; j < 4; j++) a[j] = fmaf(fs[s + j], v[j], a[j]);
    }
    for (; s < n_splits; s++) a[0] = fmaf(fs[s], p[(size_t)s * stride + 2 + i], a[0]);
    const float acc = (a[0] + a[1]) + (a[2] + a[3]);
    const float r = acc / total;
    out[(size_t)head * head_dim + i] = r;
    if (emit_q) {
        // four consecutive outputs per converting thread: gather through shuffles
        const int lane = i & 31;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = __shfl_sync(0xFFFFFFFFu, r, (4 * lane + j) & 31);
        // lanes 0..7 of each warp own the warp's 32 outputs as 8 groups of 4
        const int base = (head * head_dim + (i & ~31)) >> 2;
        quantize4_store(v, base + (lane & 7), lane < 8, o);
    }
}

// ---- the whole attention block of a decode step in ONE launch ---------------------------------
// RoPE on q and k, append of k and v at `pos`, split-KV attention over positions [k_start, pos] and
// the merge of the splits (cuda_rope_yarn x2, cuda_kv_append, cuda_attn_score_all,
// cuda_softmax_sink_all, cuda_attn_values_all: src/cuda.rs:601-645).  grid = (n_kv_heads,
// n_splits), 128 threads.  Every CTA rotates the query heads of its kv head itself (from the
// un-rotated q, into shared memory); the CTA of the last split rotates the new key, writes key and
// value into the caches and then stages them like any other row.  Partials as in
// attn_partial_kernel; the CTA that finishes last for a kv head (a counter per kv head) merges that
// head group's splits and emits the output projection's activation form.
struct RopeArgs {
    int pos;
    float theta, yarn_scale;
    int yarn_orig_ctx, neox;
};

// rotation (cos, sin) of pair i, exactly as rope_kv_kernel / src/cuda_kernels.cu:588-620 compute it
__device__ __forceinline__ void rope_cs(const RopeArgs &r, int i, int head_dim, float &c, float &s)
{
    const float PI = 3.14159265358979f;
    float inv = 1.f / powf(r.theta, 2.f * (float)i / (float)head_dim);
    float eff = inv;
    if (r.yarn_scale > 1.f && r.yarn_orig_ctx > 0) {
        float hi_w = (float)r.yarn_orig_ctx / 32.f, lo_w = (float)r.yarn_orig_ctx / 1.f;
        float wavelen = 2.f * PI / inv;
        float ramp = fmaxf(0.f, fminf(1.f, (lo_w - wavelen) / (lo_w - hi_w)));
        eff = ramp * inv + (1.f - ramp) * (inv / r.yarn_scale);
    }
    sincosf((float)r.pos * eff, &s, &c);
}

// (cos, sin) of every rotation pair at one position: the same for all layers and heads of a decode
// step, so it is computed once per step instead of in every attention CTA
__global__ void rope_table_kernel(float2 *__restrict__ tab, RopeArgs r, int head_dim)
{
    pdl_wait();
    pdl_trigger();
    const int i = threadIdx.x;
    if (i < (head_dim >> 1)) {
        float c, s;
        rope_cs(r, i, head_dim, c, s);
        tab[i] = make_float2(c, s);
    }
}

__global__ void __launch_bounds__(128) attn_fused_kernel(float *__restrict__ out, float *__restrict__ part,
                                                         int *__restrict__ counters, const float *__restrict__ q,
                                                         const float *__restrict__ k_new, const float *__restrict__ v_new,
                                                         float *k_cache, float *v_cache, int n_heads, int n_kv_heads,
                                                         int k_start, int head_dim, int kv_dim, float scale,
                                                         const float *__restrict__ sinks, RopeArgs rope,
                                                         const float2 *__restrict__ rope_tab, XQOut o, int emit_q,
                                                         int do_merge)
{
    __shared__ float ks[ATT_CHUNK][ATT_MAX_HD + 1];
    __shared__ float vs[ATT_CHUNK][ATT_MAX_HD];
    __shared__ float qs[4][ATT_MAX_HD];
    __shared__ float ps[4][ATT_CHUNK];
    __shared__ int is_last;
    pdl_wait();
    pdl_trigger();
    const int kvh = blockIdx.x, split = blockIdx.y, n_splits = gridDim.y;
    const int seq_len = rope.pos - k_start + 1;
    const int t0 = split * ATT_CHUNK;                 // relative to k_start
    const int nt = min(ATT_CHUNK, seq_len - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = head_dim >> 1;
    const float *kc = k_cache + (size_t)k_start * kv_dim, *vc = v_cache + (size_t)k_start * kv_dim;
    const bool has_new = split == n_splits - 1;       // the new position is this CTA's last row
    const int n_old = has_new ? nt - 1 : nt;          // rows that come from the caches
    // 1. issue the loads of the cached K and V rows (all of a thread's loads before any use)
    const int hd4 = head_dim >> 2;
    constexpr int MAX_IT = ATT_CHUNK * (ATT_MAX_HD / 4) / 128;
    float4 kreg[MAX_IT], vreg[MAX_IT];
#pragma unroll
    for (int it = 0; it < MAX_IT; it++) {
        const int idx = threadIdx.x + it * 128;
        if (idx < n_old * hd4) {
            const int t = idx / hd4, c = idx - t * hd4;
            const size_t g = (size_t)(t0 + t) * kv_dim + (size_t)kvh * head_dim + 4 * c;
            kreg[it] = __ldg((const float4 *)(kc + g));
            vreg[it] = __ldg((const float4 *)(vc + g));
        }
    }
    // 2. while they fly: the new key (rotated) and value go to shared memory and to the caches
    if (has_new) {
        const float *kh = k_new + (size_t)kvh * head_dim, *vh = v_new + (size_t)kvh * head_dim;
        float *kd = k_cache + (size_t)rope.pos * kv_dim + (size_t)kvh * head_dim;
        float *vd = v_cache + (size_t)rope.pos * kv_dim + (size_t)kvh * head_dim;
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float2 cs = rope_tab[i];
            const int i0 = rope.neox ? i : 2 * i, i1 = rope.neox ? i + half : 2 * i + 1;
            const float a = kh[i0], b = kh[i1];
            const float r0 = a * cs.x - b * cs.y, r1 = a * cs.y + b * cs.x;
            kd[i0] = r0;
            kd[i1] = r1;
            ks[nt - 1][i0] = r0;
            ks[nt - 1][i1] = r1;
        }
        for (int j = threadIdx.x; j < head_dim; j += blockDim.x) {
            const float v = vh[j];
            vd[j] = v;
            vs[nt - 1][j] = v;
        }
    }
#pragma unroll
    for (int it = 0; it < MAX_IT; it++) {
        const int idx = threadIdx.x + it * 128;
        if (idx < n_old * hd4) {
            const int t = idx / hd4, c = idx - t * hd4;
            ks[t][4 * c] = kreg[it].x; ks[t][4 * c + 1] = kreg[it].y; ks[t][4 * c + 2] = kreg[it].z; ks[t][4 * c + 3] = kreg[it].w;
            *(float4 *)&vs[t][4 * c] = vreg[it];
        }
    }
    const int h_lo = (kvh * n_heads + n_kv_heads - 1) / n_kv_heads;
    const int h_hi = ((kvh + 1) * n_heads + n_kv_heads - 1) / n_kv_heads;
    const int stride = head_dim + 2;
    for (int hb = h_lo; hb < h_hi; hb += 4) {
        const int head = hb + warp;
        const bool live = head < h_hi;
        __syncthreads();   // staging done / previous round's qs no longer read
        if (live) {
            const float *qh = q + (size_t)head * head_dim;
            for (int i = lane; i < half; i += 32) {
                const float2 cs = rope_tab[i];
                const int i0 = rope.neox ? i : 2 * i, i1 = rope.neox ? i + half : 2 * i + 1;
                const float a = qh[i0], b = qh[i1];
                qs[warp][i0] = a * cs.x - b * cs.y;
                qs[warp][i1] = a * cs.y + b * cs.x;
            }
        }
        __syncthreads();
        if (!live) continue;
        float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
        for (int i = 0; i < head_dim; i += 4) {
            c0 = fmaf(qs[warp][i], ks[lane][i], c0);
            c1 = fmaf(qs[warp][i + 1], ks[lane][i + 1], c1);
            c2 = fmaf(qs[warp][i + 2], ks[lane][i + 2], c2);
            c3 = fmaf(qs[warp][i + 3], ks[lane][i + 3], c3);
        }
        float sc = (c0 + c1) + (c2 + c3);
        sc = lane < nt ? sc * scale : -INFINITY;
        float mx = sc;
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
        const float p = lane < nt ? expf(sc - mx) : 0.f;
        float sum = p;
#pragma unroll
        for (int o2 = 16; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o2);
        ps[warp][lane] = p;
        __syncwarp();
        float *dst = part + ((size_t)head * n_splits + split) * stride;
        float o0 = 0.f, o1 = 0.f, o2v = 0.f, o3 = 0.f;
        for (int t = 0; t < nt; t++) {
            const float pt = ps[warp][t];
            o0 = fmaf(pt, vs[t][lane], o0);
            if (head_dim > 32) o1 = fmaf(pt, vs[t][lane + 32], o1);
            if (head_dim > 64) o2v = fmaf(pt, vs[t][lane + 64], o2v);
            if (head_dim > 96) o3 = fmaf(pt, vs[t][lane + 96], o3);
        }
        dst[2 + lane] = o0;
        if (head_dim > 32) dst[2 + lane + 32] = o1;
        if (head_dim > 64) dst[2 + lane + 64] = o2v;
        if (head_dim > 96) dst[2 + lane + 96] = o3;
        if (lane == 0) {
            dst[0] = mx;
            dst[1] = sum;
        }
        __syncwarp();
    }
    if (!do_merge) return;   // the splits are merged by attn_combine_kernel (many splits: more CTAs for the merge)
    // ---- the last CTA of this kv head merges the head group's splits ----
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(&counters[kvh], 1);
        is_last = prev == n_splits - 1;
        if (is_last) counters[kvh] = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // Up to four heads at a time: warp w reduces head hb+w's (max, sum) pairs and leaves the splits'
    // rescale factors in shared memory; then every thread owns output dimension i of all four heads,
    // so its loads of the four heads' partials are independent and overlap.
    float *fs = &ks[0][0];                  // [4][n_splits] rescale factors (ks is free now)
    float *tot_s = &vs[0][0];               // [4] softmax denominators
    const int i = threadIdx.x;
    for (int hb = h_lo; hb < h_hi; hb += 4) {
        const int head_w = hb + warp;
        __syncthreads();                    // previous round's fs / tot_s no longer read
        if (head_w < h_hi) {
            const float *pp = part + (size_t)head_w * n_splits * stride;
            const float sink = sinks ? sinks[head_w] : -INFINITY;
            const bool has_sink = sink > -1e29f;
            float mx = has_sink ? sink : -1e30f;
            for (int s = lane; s < n_splits; s += 32) mx = fmaxf(mx, __ldcg(pp + (size_t)s * stride));
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
            float tot = 0.f;
            for (int s = lane; s < n_splits; s += 32) {
                const float f = expf(__ldcg(pp + (size_t)s * stride) - mx);
                fs[warp * n_splits + s] = f;
                tot = fmaf(f, __ldcg(pp + (size_t)s * stride + 1), tot);
            }
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1) tot += __shfl_xor_sync(0xFFFFFFFFu, tot, o2);
            if (lane == 0) tot_s[warp] = tot + (has_sink ? expf(sink - mx) : 0.f);
        }
        __syncthreads();
        float r[4] = {0.f, 0.f, 0.f, 0.f};
        if (i < head_dim) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int s = 0; s < n_splits; s++) {
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (hb + j < h_hi)
                        acc[j] = fmaf(fs[j * n_splits + s],
                                      __ldcg(part + ((size_t)(hb + j) * n_splits + s) * stride + 2 + i), acc[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (hb + j < h_hi) {
                    r[j] = acc[j] / tot_s[j];
                    out[(size_t)(hb + j) * head_dim + i] = r[j];
                }
        }
        if (emit_q) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (hb + j >= h_hi) break;   // uniform over the block
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; e++) v[e] = __shfl_sync(0xFFFFFFFFu, r[j], (4 * lane + e) & 31);
                const int base = ((hb + j) * head_dim + (i & ~31)) >> 2;
                quantize4_store(v, base + (lane & 7), lane < 8 && (i & ~31) < head_dim, o);
            }
        }
    }
}

}  // namespace qz
