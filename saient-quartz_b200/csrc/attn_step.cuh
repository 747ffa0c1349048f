// The attention block of one decode step as ONE launch whose shape does not depend on the
// position: RoPE on q and k, append of k and v at `pos`, attention of every head over cache
// positions [k_start, pos], merge, and (optionally) the activation form of the result for the
// output projection (cuda_rope_yarn x2 + cuda_kv_append + cuda_attn_score_all +
// cuda_softmax_sink_all + cuda_attn_values_all of the reference, src/cuda.rs:601-645).
//
// The position is read from a device word, so a recorded graph serves every step of a
// generation loop.  Grid = n_kv_heads clusters of CL CTAs (thread-block clusters, CL <= 16): the
// CL CTAs of a kv head split the context into 32-position blocks.  Order of events in a CTA:
//   1. BEFORE the programmatic-dependency wait (the kernel that produces q, k, v may still be
//      running): read the position, start the asynchronous copies of this CTA's cached K and V
//      rows into shared memory (they were written by earlier steps), build the rotation table;
//   2. after the wait: rotate the head group's queries, rotate and append the new key / value
//      (the CTA that owns the last block), finish the copies;
//   3. every warp runs an online softmax over its 32-row groups for its query head (K and V rows
//      are staged once per CTA and shared by the whole head group);
//   4. the CTA's partial (max, sum, out[head_dim]) per head is PUSHED into the shared memory of the
//      cluster's CTAs (each receives the slice of outputs it will finish), one cluster barrier,
//      then CTA r merges G*head_dim/CL outputs from what it received.
// No global scratch, no second launch, no atomics, one cluster barrier.
#pragma once

#include <cooperative_groups.h>

#include "fused_ops.cuh"

namespace qz {

constexpr int AS_THREADS = 256;
constexpr int AS_WARPS = AS_THREADS / 32;
constexpr int AS_ROWS = 96;              // most K / V rows staged per round (three 32-position blocks)
constexpr int AS_MAX_G = 16;             // query heads per kv head
constexpr int AS_MAX_CL = 16;
constexpr int AS_KS_STRIDE = ATT_MAX_HD + 4;   // floats; keeps float4 rows conflict-free across a quarter warp

struct AttnStepArgs {
    float *out;
    const float *q, *k_new, *v_new;      // projections before RoPE
    float *k_cache, *v_cache;            // [max_seq][kv_dim]
    const int *step;                     // device words {token, pos}; NULL: pos_host
    int pos_host;
    int n_heads, n_kv_heads, head_dim, kv_dim, max_seq;
    int window;                          // > 0: attend to the last `window` positions only
    float scale;
    const float *sinks;
    float theta, yarn_scale;
    int yarn_orig_ctx, neox;
    XQOut o;
    int emit_q;
    int rows_cap;                        // K / V rows staged per round: 64 or 96 (sizes the shared memory)
    // prompt mode (grid.y = n tokens): token t = blockIdx.y sits at position pos_host + t; q and out are
    // [n, n_heads*head_dim]; q is ALREADY rotated and every token's k, v are ALREADY in the caches (appended by
    // the kernel before this one, so nothing is read ahead of the dependency wait); causal: keys up to pos.
    int prompt;
    // (cos, sin) per rotation pair of the step's position, written together with the step words (or NULL):
    // entries [0, head_dim/2), and the position they were computed for, as an int, in entry [ATT_MAX_HD/2].x
    const float2 *rope_tab;
};

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// split cluster barrier (every thread of the CTA executes both halves)
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// dynamic shared memory (floats): ks [AS_ROWS][AS_KS_STRIDE], vs [AS_ROWS][ATT_MAX_HD], qs [G][ATT_MAX_HD],
// ps [AS_WARPS][32], wres [AS_WARPS][2][ATT_MAX_HD + 2] (per-warp partials), recv [CL][2 G + S] (what the cluster's
// CTAs push here: their (max, sum) of every head and their part of this CTA's S outputs), cs_tab [ATT_MAX_HD / 2] x 2
__host__ __device__ inline size_t attn_step_smem(int G, int CL, int head_dim, int rows_cap)
{
    const int S = (G * head_dim) / CL;
    return sizeof(float) * ((size_t)rows_cap * AS_KS_STRIDE + (size_t)rows_cap * ATT_MAX_HD + (size_t)G * ATT_MAX_HD +
                            AS_WARPS * 32 + (size_t)AS_WARPS * 2 * (ATT_MAX_HD + 2) + (size_t)CL * (2 * G + S) + ATT_MAX_HD);
}

__global__ void __launch_bounds__(AS_THREADS) attn_step_kernel(const AttnStepArgs a)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    extern __shared__ __align__(16) float smem[];
    const int hd = a.head_dim, half = hd >> 1, hd4 = hd >> 2;
    const int G = a.n_heads / a.n_kv_heads;
    const int S = (G * hd) / CL;          // outputs this CTA finishes: a multiple of 32 (host-checked)
    const int RW = 2 * G + S;             // floats one CTA pushes to one peer
    constexpr int RS = ATT_MAX_HD + 2;
    const int ROWS = a.rows_cap;
    float *ks = smem;
    float *vs = ks + ROWS * AS_KS_STRIDE;
    float *qs = vs + ROWS * ATT_MAX_HD;
    float *ps = qs + G * ATT_MAX_HD;
    float *wres = ps + AS_WARPS * 32;
    float *recv = wres + AS_WARPS * 2 * RS;
    float2 *cs_tab = (float2 *)(recv + CL * RW);   // (cos, sin) per rotation pair

    const int kvh = blockIdx.x / CL;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h_lo = kvh * G;
    // Shared memory of another CTA may be written only once that CTA runs: arrive now, wait just before the pushes.
    cluster_arrive();

    // ---- 1. everything that does not depend on the kernel before this one ----
    // (the position words are written by a launch that precedes the whole recorded step)
    if (a.prompt) pdl_wait();
    // the three small loads go out together, ahead of the burst of row copies (the load/store unit works in order)
    int pos = a.prompt ? a.pos_host + (int)blockIdx.y : (a.step ? __ldcg(a.step + 1) : a.pos_host);
    const bool tab_lane = a.rope_tab && (int)threadIdx.x < (a.head_dim >> 1);
    const int tab_pos = tab_lane ? __float_as_int(__ldcg(&a.rope_tab[ATT_MAX_HD / 2].x)) : -1;
    const float2 tab_cs = tab_lane ? __ldcg(&a.rope_tab[threadIdx.x]) : make_float2(1.f, 0.f);
    if (pos >= a.max_seq) pos = a.max_seq - 1;   // never write past the caches (src/cuda.rs:517-520)
    if (pos < 0) pos = 0;
    const int k_start = a.window > 0 ? max(0, pos + 1 - a.window) : 0;
    const int seq_len = pos - k_start + 1;
    // this CTA's share of the context, in 32-position blocks
    const int nblk = (seq_len + 31) >> 5;
    const int base = nblk / CL, rem = nblk % CL;
    const int b0 = rank * base + min(rank, rem), bcnt = base + (rank < rem ? 1 : 0);
    const int p_lo = 32 * b0, p_hi = min(32 * (b0 + bcnt), seq_len);   // relative to k_start
    const bool owns_new = !a.prompt && bcnt > 0 && p_hi == seq_len;
    const float *kc = a.k_cache + (size_t)k_start * a.kv_dim + (size_t)kvh * hd;
    const float *vc = a.v_cache + (size_t)k_start * a.kv_dim + (size_t)kvh * hd;
    // cached rows [c0, c0 + n_old) -> shared rows 0 ..: 16-byte asynchronous copies.  A thread keeps its column and
    // steps through the rows when the row length divides the block (head_dim 32, 64, 128): no division per copy.
    auto stage_rows = [&](int c0, int n_old) {
        if (AS_THREADS % hd4 == 0) {
            const int c = threadIdx.x % hd4, dt = AS_THREADS / hd4;
            const float *kp = kc + (size_t)c0 * a.kv_dim + 4 * c, *vp = vc + (size_t)c0 * a.kv_dim + 4 * c;
            for (int t = threadIdx.x / hd4; t < n_old; t += dt) {
                cp_async16(ks + t * AS_KS_STRIDE + 4 * c, kp + (size_t)t * a.kv_dim);
                cp_async16(vs + t * ATT_MAX_HD + 4 * c, vp + (size_t)t * a.kv_dim);
            }
        } else {
            for (int idx = threadIdx.x; idx < n_old * hd4; idx += AS_THREADS) {
                const int t = idx / hd4, c = idx - t * hd4;
                const size_t g = (size_t)(c0 + t) * a.kv_dim + 4 * c;
                cp_async16(ks + t * AS_KS_STRIDE + 4 * c, kc + g);
                cp_async16(vs + t * ATT_MAX_HD + 4 * c, vc + g);
            }
        }
    };
    {
        const int n = min(ROWS, p_hi - p_lo);
        const bool has_new = owns_new && p_lo + n == seq_len;
        stage_rows(p_lo, has_new ? n - 1 : n);
    }
    if (threadIdx.x < half) {
        // the table written with the step words, when it is for this very position; computed here otherwise
        if (tab_lane && tab_pos == pos) {
            cs_tab[threadIdx.x] = tab_cs;
        } else {
            const RopeArgs r{pos, a.theta, a.yarn_scale, a.yarn_orig_ctx, a.neox};
            float c, s;
            rope_cs(r, threadIdx.x, hd, c, s);
            cs_tab[threadIdx.x] = make_float2(c, s);
        }
    }
    pdl_trigger();
    __syncthreads();

    // ---- 2. the new token's q, k, v ----
    pdl_wait();
    const size_t tok_off = a.prompt ? (size_t)blockIdx.y * a.n_heads * hd : 0;
    for (int idx = threadIdx.x; idx < G * half; idx += AS_THREADS) {
        const int g = idx / half, i = idx - g * half;
        const float2 cs = a.prompt ? make_float2(1.f, 0.f) : cs_tab[i];   // prompt mode: q arrives rotated
        const int i0 = a.neox ? i : 2 * i, i1 = a.neox ? i + half : 2 * i + 1;
        const float *qh = a.q + tok_off + (size_t)(h_lo + g) * hd;
        const float x0 = __ldcg(qh + i0), x1 = __ldcg(qh + i1);
        qs[g * ATT_MAX_HD + i0] = x0 * cs.x - x1 * cs.y;
        qs[g * ATT_MAX_HD + i1] = x0 * cs.y + x1 * cs.x;
    }

    // which (head, 32-row group) this warp serves: head = warp % Gw (+ 8 for the second round when G > 8), groups
    // sub, sub + wph, ... of every staged round
    const int Gw = G < AS_WARPS ? G : AS_WARPS;
    const int wph = AS_WARPS / Gw;                        // warps per head
    const int n_rounds = (G + AS_WARPS - 1) / AS_WARPS;   // heads per warp (G > 8)
    const int sub = warp / Gw;
    const bool warp_active = sub < wph;
    float m_run[2] = {-1e30f, -1e30f}, l_run[2] = {0.f, 0.f};
    float o_run[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};

    for (int c0 = p_lo; c0 < p_hi; c0 += ROWS) {
        const int n = min(ROWS, p_hi - c0);
        const bool has_new = owns_new && c0 + n == seq_len;   // the new position is this round's last row
        if (c0 > p_lo) {
            __syncthreads();   // the previous round's rows are no longer read
            stage_rows(c0, has_new ? n - 1 : n);
        }
        if (has_new) {
            // the new key (rotated) and value: into the caches and into this round's last row
            const float *kh = a.k_new + (size_t)kvh * hd, *vh = a.v_new + (size_t)kvh * hd;
            float *kd = a.k_cache + (size_t)pos * a.kv_dim + (size_t)kvh * hd;
            float *vd = a.v_cache + (size_t)pos * a.kv_dim + (size_t)kvh * hd;
            for (int i = threadIdx.x; i < half; i += AS_THREADS) {
                const float2 cs = cs_tab[i];
                const int i0 = a.neox ? i : 2 * i, i1 = a.neox ? i + half : 2 * i + 1;
                const float x0 = __ldcg(kh + i0), x1 = __ldcg(kh + i1);
                const float r0 = x0 * cs.x - x1 * cs.y, r1 = x0 * cs.y + x1 * cs.x;
                kd[i0] = r0;
                kd[i1] = r1;
                ks[(n - 1) * AS_KS_STRIDE + i0] = r0;
                ks[(n - 1) * AS_KS_STRIDE + i1] = r1;
            }
            for (int j = threadIdx.x; j < hd; j += AS_THREADS) {
                const float v = __ldcg(vh + j);
                vd[j] = v;
                vs[(n - 1) * ATT_MAX_HD + j] = v;
            }
        }
        cp_async_wait_all();
        __syncthreads();
        if (!warp_active) continue;
        // ---- 3. online softmax over this warp's 32-row groups ----
        for (int t_lo = 32 * sub; t_lo < n; t_lo += 32 * wph) {
            const int nt = min(32, n - t_lo);
#pragma unroll
            for (int r = 0; r < 2; r++) {
                if (r >= n_rounds) break;
                const int g = (warp % Gw) + r * AS_WARPS;
                if (g >= G) break;
                // one key position per lane
                const float4 *qv = (const float4 *)(qs + g * ATT_MAX_HD);
                const float4 *kv = (const float4 *)(ks + (t_lo + lane) * AS_KS_STRIDE);
                float c0a = 0.f, c1a = 0.f, c2a = 0.f, c3a = 0.f;
#pragma unroll 8
                for (int i = 0; i < hd4; i++) {
                    const float4 qq = qv[i], kk = kv[i];
                    c0a = fmaf(qq.x, kk.x, c0a);
                    c1a = fmaf(qq.y, kk.y, c1a);
                    c2a = fmaf(qq.z, kk.z, c2a);
                    c3a = fmaf(qq.w, kk.w, c3a);
                }
                float sc = (c0a + c1a) + (c2a + c3a);
                sc = lane < nt ? sc * a.scale : -INFINITY;
                float mx = sc;
#pragma unroll
                for (int o2 = 16; o2 > 0; o2 >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o2));
                const float m_new = fmaxf(m_run[r], mx);
                const float p = lane < nt ? __expf(sc - m_new) : 0.f;
                float sum = p;
#pragma unroll
                for (int o2 = 16; o2 > 0; o2 >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o2);
                const float corr = __expf(m_run[r] - m_new);
                m_run[r] = m_new;
                l_run[r] = l_run[r] * corr + sum;
                __syncwarp();
                ps[warp * 32 + lane] = p;
                __syncwarp();
                // lane owns output dimensions 4*lane .. 4*lane+3 (head_dim <= 128)
                float4 acc = make_float4(o_run[r][0] * corr, o_run[r][1] * corr, o_run[r][2] * corr, o_run[r][3] * corr);
                if (4 * lane < hd) {
#pragma unroll 8
                    for (int t = 0; t < nt; t++) {
                        const float pt = ps[warp * 32 + t];
                        const float4 vv = *(const float4 *)(vs + (t_lo + t) * ATT_MAX_HD + 4 * lane);
                        acc.x = fmaf(pt, vv.x, acc.x);
                        acc.y = fmaf(pt, vv.y, acc.y);
                        acc.z = fmaf(pt, vv.z, acc.z);
                        acc.w = fmaf(pt, vv.w, acc.w);
                    }
                }
                o_run[r][0] = acc.x; o_run[r][1] = acc.y; o_run[r][2] = acc.z; o_run[r][3] = acc.w;
            }
        }
    }

    // ---- this CTA's partial per head: the warps that shared a head leave theirs in shared memory ----
    __syncthreads();
    if (warp_active) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            if (r >= n_rounds) break;
            float *w = wres + (warp * 2 + r) * RS;
            if (lane == 0) { w[0] = m_run[r]; w[1] = l_run[r]; }
            if (4 * lane < hd) {
                *(float2 *)(w + 2 + 4 * lane) = make_float2(o_run[r][0], o_run[r][1]);
                *(float2 *)(w + 4 + 4 * lane) = make_float2(o_run[r][2], o_run[r][3]);
            }
        }
    }
    __syncthreads();

    // ---- 4. push the partials to the CTAs that finish them: destination d gets, in its recv[rank], this CTA's
    //         (max, sum) of every head followed by its part of d's S outputs ----
    cluster_wait();   // (arrived at the top) every CTA of the cluster has started
    // four outputs (one float4) or one head's (max, sum) pair (one float2) per remote store
    const int n_out4 = (G * hd) >> 2;
    for (int it = threadIdx.x; it < n_out4 + G * CL; it += AS_THREADS) {
        if (it < n_out4) {
            const int idx = 4 * it;
            const int g = idx / hd, d = idx - g * hd;          // (hd is a multiple of 32: the four share a head)
            const int r = g / AS_WARPS, w0 = g % AS_WARPS;     // G <= 8: r = 0, w0 = g
            float m = -1e30f;
            for (int s = 0; s < wph; s++) m = fmaxf(m, wres[((w0 + s * Gw) * 2 + r) * RS]);
            float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < wph; s++) {
                const float *w = wres + ((w0 + s * Gw) * 2 + r) * RS;
                const float f = __expf(w[0] - m);
                const float2 lo = *(const float2 *)(w + 2 + d), hi = *(const float2 *)(w + 4 + d);
                o.x = fmaf(lo.x, f, o.x);
                o.y = fmaf(lo.y, f, o.y);
                o.z = fmaf(hi.x, f, o.z);
                o.w = fmaf(hi.y, f, o.w);
            }
            const int dst = idx / S;
            float *remote = cluster.map_shared_rank(recv, dst) + rank * RW + 2 * G + (idx - dst * S);
            if ((G & 1) == 0) {
                *(float4 *)remote = o;                          // 16-byte aligned: RW and 2 G are multiples of 4 floats
            } else {
                *(float2 *)remote = make_float2(o.x, o.y);
                *(float2 *)(remote + 2) = make_float2(o.z, o.w);
            }
        } else {
            const int j = it - n_out4;
            const int dst = j / G, g = j - dst * G;
            const int r = g / AS_WARPS, w0 = g % AS_WARPS;
            float m = -1e30f;
            for (int s = 0; s < wph; s++) m = fmaxf(m, wres[((w0 + s * Gw) * 2 + r) * RS]);
            float l = 0.f;
            for (int s = 0; s < wph; s++) {
                const float *w = wres + ((w0 + s * Gw) * 2 + r) * RS;
                l = fmaf(w[1], __expf(w[0] - m), l);
            }
            float *remote = cluster.map_shared_rank(recv, dst) + rank * RW + 2 * g;
            *(float2 *)remote = make_float2(m, l);
        }
    }
    cluster_arrive();
    cluster_wait();   // every push has landed; nobody touches another CTA's shared memory afterwards

    // ---- merge: this CTA's S outputs from the CL partials it received ----
    for (int j = threadIdx.x; j < S; j += AS_THREADS) {
        const int idx = rank * S + j;
        const int g = idx / hd, d = idx - g * hd;
        const int head = h_lo + g;
        const float sink = a.sinks ? a.sinks[head] : -INFINITY;
        const bool has_sink = sink > -1e29f;
        float M = has_sink ? sink : -1e30f;
        for (int c = 0; c < CL; c++) M = fmaxf(M, recv[c * RW + 2 * g]);
        float tot = has_sink ? __expf(sink - M) : 0.f, acc = 0.f;
        for (int c = 0; c < CL; c++) {
            const float f = __expf(recv[c * RW + 2 * g] - M);
            tot = fmaf(recv[c * RW + 2 * g + 1], f, tot);
            acc = fmaf(recv[c * RW + 2 * G + j], f, acc);
        }
        const float r = acc / tot;
        a.out[tok_off + (size_t)head * hd + d] = r;
        if (a.emit_q) {
            // lanes 0..7 of each warp own the warp's 32 outputs as 8 groups of 4
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] = __shfl_sync(0xFFFFFFFFu, r, (4 * lane + e) & 31);
            const int first = h_lo * hd + rank * S + (j & ~31);
            quantize4_store(v, (first >> 2) + (lane & 7), lane < 8, a.o);
        }
    }
}

}  // namespace qz
