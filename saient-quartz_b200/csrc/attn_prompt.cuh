// Causal attention over a whole prompt (batched prefill): token t at position pos0 + t attends to the cache
// positions [k_start(t), pos0 + t].  The reference has no batched GPU attention (its GPU prefill is token by token,
// src/main.rs:1410-1416, each token through cuda_attn_score_all / cuda_softmax_sink_all / cuda_attn_values_all,
// src/cuda.rs:601-645); its CPU form is the per-token loop of prefill_batched (src/main.rs:1157-1341).
//
// One CTA per (kv head, tile of TQ consecutive tokens).  The tile's TQ * G query rows (G = query heads per kv head)
// sit in shared memory; the K and V rows of the kv head stream through a double-buffered shared-memory tile of 32
// positions (16-byte asynchronous copies), so a cached row is read once per TQ tokens and G heads instead of once
// per token.  A warp owns up to eight query rows: one lane per key position for the scores (the K row's
// coefficients are loaded once and used for all of the warp's rows), an online softmax per row, one lane per four
// output dimensions for the values (a V row is loaded once for all rows).  Token tiles are issued longest first
// (the last tokens of the prompt see the most positions).
#pragma once

#include "attn_step.cuh"

namespace qz {

constexpr int AP_THREADS = 256;
constexpr int AP_WARPS = AP_THREADS / 32;
constexpr int AP_KT = 32;        // key positions per staged tile
constexpr int AP_RW = 8;         // most query rows per warp
constexpr int AP_MAX_ROWS = AP_WARPS * AP_RW;   // query rows per CTA (TQ * G)

struct AttnPromptArgs {
    float *out;                     // [n_tok][n_heads * head_dim]
    const float *q;                 // [n_tok][n_heads * head_dim], already rotated
    const float *k_cache, *v_cache; // [max_seq][kv_dim], already holding the prompt's rows
    int n_tok, n_heads, n_kv_heads, head_dim, kv_dim;
    int pos0, window, tq;
    float scale;
    const float *sinks;             // per head, or NULL
};

__host__ __device__ inline size_t attn_prompt_smem(int rows, int head_dim)
{
    return sizeof(float) * ((size_t)rows * head_dim + 2 * (size_t)AP_KT * (head_dim + 4) + 2 * (size_t)AP_KT * head_dim +
                            (size_t)AP_WARPS * AP_RW * AP_KT);
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(AP_THREADS) attn_prompt_kernel(const AttnPromptArgs a)
{
    extern __shared__ __align__(16) float sm[];
    const int hd = a.head_dim, hd4 = hd >> 2, kst = hd + 4;
    const int G = a.n_heads / a.n_kv_heads;
    const int kvh = blockIdx.x;
    const int tile_idx = (int)gridDim.y - 1 - (int)blockIdx.y;   // longest tiles first
    const int t0 = tile_idx * a.tq, nt = min(a.tq, a.n_tok - t0);
    const int rows = nt * G;                     // query row r = token (r / G), head (r % G) of the group
    const int rows_cap = a.tq * G;
    float *qs = sm;
    float *ks = qs + (size_t)rows_cap * hd;
    float *vs = ks + 2 * AP_KT * kst;
    float *ps = vs + 2 * AP_KT * hd;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    pdl_wait();   // q and the cache rows of this prompt come from the kernels before this one
    pdl_trigger();
    for (int idx = threadIdx.x; idx < rows * hd4; idx += AP_THREADS) {
        const int r = idx / hd4, c = idx - r * hd4;
        const float *src = a.q + ((size_t)(t0 + r / G) * a.n_heads + (size_t)kvh * G + (r % G)) * hd + 4 * c;
        *(float4 *)(qs + (size_t)r * hd + 4 * c) = __ldcg((const float4 *)src);
    }
    // positions any token of the tile may see
    const int p_first = a.pos0 + t0, p_last = a.pos0 + t0 + nt - 1;
    const int k_lo = a.window > 0 ? max(0, p_first + 1 - a.window) : 0;
    const int n_tiles = (p_last - k_lo) / AP_KT + 1;
    const float *kc = a.k_cache + (size_t)kvh * hd, *vc = a.v_cache + (size_t)kvh * hd;
    auto stage = [&](int tile, int buf) {
        const int base = k_lo + tile * AP_KT, n = min(AP_KT, p_last - base + 1);
        float *kd = ks + buf * AP_KT * kst, *vd = vs + buf * AP_KT * hd;
        for (int idx = threadIdx.x; idx < n * hd4; idx += AP_THREADS) {
            const int t = idx / hd4, c = idx - t * hd4;
            const size_t g = (size_t)(base + t) * a.kv_dim + 4 * c;
            cp_async16(kd + t * kst + 4 * c, kc + g);
            cp_async16(vd + t * hd + 4 * c, vc + g);
        }
        cp_async_commit();
    };
    // this warp's rows
    const int rw = (rows + AP_WARPS - 1) / AP_WARPS;   // <= AP_RW
    const int r_lo = warp * rw;
    float m_run[AP_RW], l_run[AP_RW], o_run[AP_RW][4];
    int p_tok[AP_RW], ks_tok[AP_RW];   // last and first position each row may see
#pragma unroll
    for (int r = 0; r < AP_RW; r++) {
        m_run[r] = -1e30f;
        l_run[r] = 0.f;
        o_run[r][0] = o_run[r][1] = o_run[r][2] = o_run[r][3] = 0.f;
        const int row = r_lo + r;
        const int pt = a.pos0 + t0 + (row < rows ? row / G : 0);
        p_tok[r] = (r < rw && row < rows) ? pt : -1;   // -1: no such row, every position is masked
        ks_tok[r] = a.window > 0 ? max(0, pt + 1 - a.window) : 0;
    }
    float *pw = ps + (size_t)warp * AP_RW * AP_KT;

    stage(0, 0);
    for (int tile = 0; tile < n_tiles; tile++) {
        const int buf = tile & 1;
        if (tile + 1 < n_tiles) {
            stage(tile + 1, buf ^ 1);
            cp_async_wait_group<1>();
        } else {
            cp_async_wait_group<0>();
        }
        __syncthreads();   // the tile (and, first time round, the query rows) are visible to every warp
        const int base = k_lo + tile * AP_KT, npos = min(AP_KT, p_last - base + 1);
        const float *kt = ks + buf * AP_KT * kst, *vt = vs + buf * AP_KT * hd;
        // ---- scores: lane = key position; the K row's coefficients are loaded once for all rows ----
        float sc[AP_RW];
#pragma unroll
        for (int r = 0; r < AP_RW; r++) sc[r] = 0.f;
        const float4 *kv = (const float4 *)(kt + lane * kst);
        for (int c = 0; c < hd4; c += 4) {
            const float4 k0 = kv[c], k1 = kv[c + 1], k2 = kv[c + 2], k3 = kv[c + 3];
#pragma unroll
            for (int r = 0; r < AP_RW; r++) {
                if (r < rw) {
                    const float4 *qv = (const float4 *)(qs + (size_t)(r_lo + r < rows ? r_lo + r : 0) * hd) + c;
                    const float4 q0 = qv[0], q1 = qv[1], q2 = qv[2], q3 = qv[3];
                    float s = sc[r];
                    s = fmaf(q0.x, k0.x, s); s = fmaf(q0.y, k0.y, s); s = fmaf(q0.z, k0.z, s); s = fmaf(q0.w, k0.w, s);
                    s = fmaf(q1.x, k1.x, s); s = fmaf(q1.y, k1.y, s); s = fmaf(q1.z, k1.z, s); s = fmaf(q1.w, k1.w, s);
                    s = fmaf(q2.x, k2.x, s); s = fmaf(q2.y, k2.y, s); s = fmaf(q2.z, k2.z, s); s = fmaf(q2.w, k2.w, s);
                    s = fmaf(q3.x, k3.x, s); s = fmaf(q3.y, k3.y, s); s = fmaf(q3.z, k3.z, s); s = fmaf(q3.w, k3.w, s);
                    sc[r] = s;
                }
            }
        }
        // ---- online softmax per row ----
        const int pos = base + lane;
#pragma unroll
        for (int r = 0; r < AP_RW; r++) {
            if (r < rw) {
                const bool valid = lane < npos && pos <= p_tok[r] && pos >= ks_tok[r];
                const float s = valid ? sc[r] * a.scale : -INFINITY;
                float mx = s;
#pragma unroll
                for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
                const float m_new = fmaxf(m_run[r], mx);
                const float p = valid ? __expf(s - m_new) : 0.f;
                float sum = p;
#pragma unroll
                for (int o2 = 16; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o2);
                const float corr = __expf(m_run[r] - m_new);
                m_run[r] = m_new;
                l_run[r] = l_run[r] * corr + sum;
                o_run[r][0] *= corr; o_run[r][1] *= corr; o_run[r][2] *= corr; o_run[r][3] *= corr;
                pw[r * AP_KT + lane] = p;
            }
        }
        __syncwarp();
        // ---- values: lane = four output dimensions; a V row is loaded once for all rows ----
        if (4 * lane < hd) {
            for (int t = 0; t < npos; t++) {
                const float4 vv = *(const float4 *)(vt + t * hd + 4 * lane);
#pragma unroll
                for (int r = 0; r < AP_RW; r++) {
                    if (r < rw) {
                        const float pt = pw[r * AP_KT + t];
                        o_run[r][0] = fmaf(pt, vv.x, o_run[r][0]);
                        o_run[r][1] = fmaf(pt, vv.y, o_run[r][1]);
                        o_run[r][2] = fmaf(pt, vv.z, o_run[r][2]);
                        o_run[r][3] = fmaf(pt, vv.w, o_run[r][3]);
                    }
                }
            }
        }
        __syncthreads();   // the buffer is free for the tile after next; the warp's probabilities have been read
    }
    // ---- normalise (with the head's sink, if any) and store ----
#pragma unroll
    for (int r = 0; r < AP_RW; r++) {
        const int row = r_lo + r;
        if (r < rw && row < rows && 4 * lane < hd) {
            const int head = kvh * G + row % G;
            const float sink = a.sinks ? a.sinks[head] : -INFINITY;
            const bool has_sink = sink > -1e29f;
            const float M = fmaxf(has_sink ? sink : -1e30f, m_run[r]);
            const float f = __expf(m_run[r] - M);
            const float tot = fmaf(l_run[r], f, has_sink ? __expf(sink - M) : 0.f);
            const float inv = 1.f / tot;
            float *dst = a.out + ((size_t)(t0 + row / G) * a.n_heads + head) * hd + 4 * lane;
            *(float4 *)dst = make_float4(o_run[r][0] * f * inv, o_run[r][1] * f * inv, o_run[r][2] * f * inv, o_run[r][3] * f * inv);
        }
    }
}

}  // namespace qz
