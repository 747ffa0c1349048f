// Batched mixture-of-experts FFN: out[t] = sum over the token's experts e of w(t,e) *
// down_e(swiglu(gate_e x_t, up_e x_t)), the batched form of the reference's per-token MoE branch
// (src/main.rs:941-990 on the CPU, src/cuda.rs:673-800 on the GPU, where every expert GEMV of every
// token is a launch of its own and the router's top-k runs on the host after a device-to-host copy).
//
// Everything here runs on the device, so a step needs no host synchronisation:
//   router_topk_kernel      top-k experts and their softmax weights per token from the router logits
//   moe_route_kernel        groups the (token, expert) assignments by expert: slot ranges per expert,
//                           token tiles, the gather list and its inverse (stable: by token, then by k)
//   moe_tiles_kernel        builds the bf16 activation tiles the tensor-core kernel reads, either from the
//                           gathered token rows or from swiglu(gate, up) of the first two GEMMs' outputs
//   (gemm_tc_kernel, grouped: one launch for gate and up of all experts, one for down)
//   moe_combine_kernel      out[t] = sum_k w(t,k) * y[slot(t,k)], in the token's own top-k order
// The per-expert form (host-side grouping, three GEMMs per expert) is kept for shapes the grouped
// kernel does not take.
#pragma once

#include "gemm_tc.cuh"

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

// ---- router: top-k experts of every token and their weights (src/cuda.rs:673-701, src/main.rs:952-990) ----
// One warp per token.  Selection = the k largest logits (+ bias), ties to the lower expert index (what a stable
// descending sort gives).  renorm = 1: softmax over the selected logits; 0: softmax over all experts, the
// selected entries taken from it.
__global__ void router_topk_kernel(const float *__restrict__ logits, const float *__restrict__ bias, int m, int n_experts,
                                   int top_k, int renorm, int *__restrict__ ids, float *__restrict__ w)
{
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (t >= m) return;
    const float *lg = logits + (size_t)t * n_experts;
    constexpr int PER = QZ_MOE_MAX_E / 32;
    float v[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int e = lane + 32 * j;
        v[j] = e < n_experts ? lg[e] + (bias ? bias[e] : 0.f) : -INFINITY;
    }
    float all_max = -INFINITY, all_den = 0.f;
    if (!renorm) {
#pragma unroll
        for (int j = 0; j < PER; j++) all_max = fmaxf(all_max, v[j]);
        for (int o = 16; o > 0; o >>= 1) all_max = fmaxf(all_max, __shfl_xor_sync(0xFFFFFFFFu, all_max, o));
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (lane + 32 * j < n_experts) all_den += expf(v[j] - all_max);
        for (int o = 16; o > 0; o >>= 1) all_den += __shfl_xor_sync(0xFFFFFFFFu, all_den, o);
    }
    float sel_v[8];
    int sel_e[8];
    for (int k = 0; k < top_k; k++) {
        float best = -INFINITY;
        int best_e = 0x7FFFFFFF;
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int e = lane + 32 * j;
            if (e < n_experts && (v[j] > best || (v[j] == best && e < best_e))) {
                best = v[j];
                best_e = e;
            }
        }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oe = __shfl_xor_sync(0xFFFFFFFFu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        sel_v[k] = best;
        sel_e[k] = best_e;
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (lane + 32 * j == best_e) v[j] = -INFINITY;   // taken
    }
    if (lane == 0) {
        float mx = renorm ? sel_v[0] : all_max, den = all_den;   // the first selected logit is the largest
        float ex[8];
        if (renorm) den = 0.f;
        for (int k = 0; k < top_k; k++) {
            ex[k] = expf(sel_v[k] - mx);
            if (renorm) den += ex[k];
        }
        for (int k = 0; k < top_k; k++) {
            ids[(size_t)t * top_k + k] = sel_e[k];
            w[(size_t)t * top_k + k] = ex[k] / den;
        }
    }
}

// ---- grouping of the assignments by expert ----
// grid = n_experts CTAs of 256 threads.  Every CTA builds the whole histogram in shared memory (the lists are a
// few thousand entries), so it knows its expert's slot range without waiting for anybody; its first warp then
// places the expert's assignments in order of (token, k).  CTA 0 also writes the summary the GEMM reads.
// Assignments with an id outside [0, n_experts) get slot -1 and take no part.
__global__ void __launch_bounds__(256) moe_route_kernel(const int *__restrict__ ids, const float *__restrict__ w, int n_assign,
                                                        int top_k, int n_experts, int tok_tile, GemmGroup *__restrict__ grp,
                                                        int *__restrict__ rows, float *__restrict__ wts,
                                                        int *__restrict__ slot_of)
{
    __shared__ int hist[QZ_MOE_MAX_E];
    const int e = blockIdx.x;
    for (int i = threadIdx.x; i < n_experts; i += blockDim.x) hist[i] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_assign; i += blockDim.x) {
        const int id = ids[i];
        if (id >= 0 && id < n_experts) atomicAdd(&hist[id], 1);
        else if (e == 0) slot_of[i] = -1;
    }
    __syncthreads();
    int off = 0;
    for (int j = 0; j < e; j++) off += hist[j];
    if (e == 0 && threadIdx.x == 0) {
        int o = 0, tt = 0;
        grp->n_experts = n_experts;
        for (int j = 0; j < n_experts; j++) {
            grp->counts[j] = hist[j];
            grp->offsets[j] = o;
            grp->tt_prefix[j] = tt;
            o += hist[j];
            tt += (hist[j] + tok_tile - 1) / tok_tile;
        }
        grp->offsets[n_experts] = o;
        grp->tt_prefix[n_experts] = tt;
        grp->n_tt_total = tt;
    }
    if (threadIdx.x >= 32) return;
    const int lane = threadIdx.x;
    int run = off;
    for (int i0 = 0; i0 < n_assign; i0 += 32) {
        const int i = i0 + lane;
        const bool mine = i < n_assign && ids[i] == e;
        const unsigned b = __ballot_sync(0xFFFFFFFFu, mine);
        if (mine) {
            const int p = run + __popc(b & ((1u << lane) - 1u));
            rows[p] = i / top_k;
            wts[p] = w[i];
            slot_of[i] = p;
        }
        run += __popc(b);
    }
}

// ---- activation tiles of a grouped GEMM ----
// For every token tile (tok_tile slots of one expert) and 64-wide K step a [tok_tile x 128 B] block in the
// shared-memory image of gemm_tc_kernel's B operand (16-byte chunk c of row r at chunk c ^ (r & 7), k order
// (0,2,1,3) inside every four; perm = 1: the Q6_K producer's K order, see convert_x_bf16_kernel).  One thread per
// 16-byte chunk.  MODE 0: row = token rows[slot] of x [m, K] (the gather).  MODE 1: row = swiglu(g, u) of slot
// (g, u: [slots, K] f32, the outputs of the gate and up GEMMs).  Rows past the expert's last slot are zero.
template <int MODE>
__global__ void moe_tiles_kernel(const float *__restrict__ x, const float *__restrict__ u, const int *__restrict__ rows,
                                 const GemmGroup *__restrict__ grp, __nv_bfloat16 *__restrict__ out, int K, int tok_tile,
                                 int max_tiles, int perm, int oai)
{
    const int ksteps = K / 64;
    const int n_tt = min(grp->n_tt_total, max_tiles);
    const long long total = (long long)n_tt * tok_tile * ksteps * 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i & 7);
        long long rest = i >> 3;
        const int r = (int)(rest % tok_tile);
        rest /= tok_tile;
        const int ks = (int)(rest % ksteps);
        const int gtt = (int)(rest / ksteps);
        const int e = group_find(grp->tt_prefix, grp->n_experts, gtt);
        const int in_e = (gtt - grp->tt_prefix[e]) * tok_tile + r;
        uint4 o = make_uint4(0, 0, 0, 0);
        if (in_e < grp->counts[e]) {
            const int slot = grp->offsets[e] + in_e;
            const int p = 8 * c;
            const int koff = perm ? 256 * (ks >> 2) + 128 * ((ks >> 1) & 1) + 32 * (p >> 4) + 16 * (ks & 1) + (p & 15) : ks * 64 + p;
            float v[8];
            if (MODE == 0) {
                const float *src = x + (size_t)rows[slot] * K + koff;
                const float4 v0 = *(const float4 *)src, v1 = *(const float4 *)(src + 4);
                v[0] = v0.x; v[1] = v0.y; v[2] = v0.z; v[3] = v0.w; v[4] = v1.x; v[5] = v1.y; v[6] = v1.z; v[7] = v1.w;
            } else {
                const float *pg = x + (size_t)slot * K + koff, *pu = u + (size_t)slot * K + koff;
                const float4 g0 = *(const float4 *)pg, g1 = *(const float4 *)(pg + 4);
                const float4 u0 = *(const float4 *)pu, u1 = *(const float4 *)(pu + 4);
                const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                const float uu[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    if (oai) {
                        const float a = fminf(gg[j], 7.f), b = fmaxf(-7.f, fminf(7.f, uu[j]));
                        v[j] = (a / (1.f + expf(-1.702f * a))) * (b + 1.f);
                    } else {
                        v[j] = (gg[j] / (1.f + expf(-gg[j]))) * uu[j];
                    }
                }
            }
            const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[2]), b = __floats2bfloat162_rn(v[1], v[3]);
            const __nv_bfloat162 d = __floats2bfloat162_rn(v[4], v[6]), f = __floats2bfloat162_rn(v[5], v[7]);
            o = make_uint4(*(const uint32_t *)&a, *(const uint32_t *)&b, *(const uint32_t *)&d, *(const uint32_t *)&f);
        }
        uint8_t *tile_base = (uint8_t *)out + ((size_t)gtt * ksteps + ks) * ((size_t)tok_tile * 128);
        *(uint4 *)(tile_base + (size_t)r * 128 + ((c ^ (r & 7)) << 4)) = o;
    }
}

// ---- batch-1 (decode) MoE with the experts chosen on the device ----
// h[k] = swiglu(gate[k] + gate_bias[ids[k]], up[k] + up_bias[ids[k]]) for the n_act active experts
// (cuda_vec_add x2 + cuda_swiglu / cuda_swiglu_oai per expert, src/cuda.rs:730-745, 765-777); biases may be NULL.
__global__ void moe_decode_act_kernel(float *__restrict__ out, const float *__restrict__ gate, const float *__restrict__ up,
                                      const float *__restrict__ gate_bias, const float *__restrict__ up_bias,
                                      const int *__restrict__ ids, int n_act, int F, int oai)
{
    pdl_wait();
    pdl_trigger();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)n_act * F) return;
    const int k = (int)(i / F), j = (int)(i - (long long)k * F);
    const int e = ids[k];
    float g = gate[i], u = up[i];
    if (gate_bias) g += gate_bias[(size_t)e * F + j];
    if (up_bias) u += up_bias[(size_t)e * F + j];
    if (oai) {
        const float x = fminf(g, 7.f), y = fmaxf(-7.f, fminf(7.f, u));
        out[i] = (x / (1.f + expf(-1.702f * x))) * (y + 1.f);
    } else {
        out[i] = (g / (1.f + expf(-g))) * u;
    }
}

// acc[j] (+)= sum_k w[k] * (down[k][j] + down_bias[ids[k]][j]), in the order of k (cuda_vec_add +
// cuda_vec_scale_add per expert, src/cuda.rs:750-760, 788-794)
__global__ void moe_decode_combine_kernel(float *__restrict__ acc, const float *__restrict__ down,
                                          const float *__restrict__ down_bias, const int *__restrict__ ids,
                                          const float *__restrict__ w, int n_act, int D, int accumulate)
{
    pdl_wait();
    pdl_trigger();
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= D) return;
    float s = accumulate ? acc[j] : 0.f;
    for (int k = 0; k < n_act; k++) {
        float v = down[(size_t)k * D + j];
        if (down_bias) v += down_bias[(size_t)ids[k] * D + j];
        s += w[k] * v;
    }
    acc[j] = s;
}

// out[t, :] = sum_k w[t, k] * y[slot_of[t * top_k + k], :], summed in the order of k (the order in which the
// reference's per-token loop adds its experts, src/main.rs:979-990).  One thread per float4.
__global__ void moe_combine_kernel(float *__restrict__ out, const float *__restrict__ y, const int *__restrict__ slot_of,
                                   const float *__restrict__ w, int m, int top_k, int K)
{
    const int k4 = K >> 2;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)m * k4) return;
    const int t = (int)(i / k4), c = (int)(i - (long long)t * k4);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < top_k; k++) {
        const int slot = slot_of[(size_t)t * top_k + k];
        if (slot < 0) continue;
        const float s = w[(size_t)t * top_k + k];
        const float4 v = ((const float4 *)(y + (size_t)slot * K))[c];
        acc.x = fmaf(s, v.x, acc.x);
        acc.y = fmaf(s, v.y, acc.y);
        acc.z = fmaf(s, v.z, acc.z);
        acc.w = fmaf(s, v.w, acc.w);
    }
    ((float4 *)out)[i] = acc;
}

}  // namespace qz
