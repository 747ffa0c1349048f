// A chain of dependent GEMVs in ONE persistent kernel.
//
// In a decode step every GEMV depends on its predecessor (o-projection -> gate/up -> down -> next
// layer's q/k/v), and at batch 1 each of them streams for only 2-10 us.  As separate kernels they pay,
// per link, the latency from one grid's completion to the release of its dependents plus an empty
// weight pipeline.  Here one CTA per SM runs the whole chain:
//   * the producer lane streams the weight rows of op 0, op 1, ... back to back through the same
//     shared-memory ring (weights depend on nothing, so it never waits for a link);
//   * the consumers finish op k, meet at a grid-wide barrier (a self-resetting count + generation in
//     global memory, polled with a bound), convert op k+1's activation vector from the outputs that
//     are now complete (RMSNorm / SwiGLU / plain f32, as in gemv_tma_kernel's prologue) and go on;
//     the ring has been refilled meanwhile.
// The reference runs each of these GEMVs, and each norm / SwiGLU between them, as a launch of its
// own (src/cuda.rs:548-823).
//
// Every mbarrier wait and the grid barrier's poll are bounded; a timeout sets the status word, a CTA-wide
// flag (the CTA's other warps then skip their waits and arithmetic but keep arriving at every barrier of
// the op, and the whole CTA leaves together at the next op boundary) and an abort word that the other
// CTAs see at their next grid barrier.  Every thread runs to the kernel's end.
#pragma once

#include "gemv_tma.cuh"

namespace qz {

constexpr int CHAIN_MAX_OPS = 8;
constexpr long long CHAIN_BARRIER_CYCLES = 1000000000LL;   // ~0.5 s

struct ChainOp {
    const uint8_t *W[QZ_MAX_MATS];
    float *y[QZ_MAX_MATS];
    uint32_t type;
    int n_mats, K, N, accumulate;
    int U, Upad, RP;        // units per row, threads per row, rows per stage
    int n_cta;              // CTAs per matrix (grid / n_mats, at most the tile count)
    XSrc xsrc;              // mode 1 (RMSNorm), 2 (SwiGLU) or 3 (plain f32 vector a)
};

struct GridBarrier {
    int count, gen, abort;
};

struct ChainArgs {
    ChainOp op[CHAIN_MAX_OPS];
    int n_ops;
    int independent;           // 1: no op reads another op's output: no grid barrier between them
    int slot_bytes, n_slots;   // ring geometry: every op's stage fits a slot
    GridBarrier *gb;
    int *status;
};

// state of the weight ring as one role sees it; survives from op to op
struct RingPos {
    int s;
    uint32_t parity;
};

__device__ __forceinline__ int ld_acquire_gpu(const int *p)
{
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by ONE thread per CTA, between two CTA-level barriers.  Returns false on abort / timeout.
__device__ __forceinline__ bool grid_barrier(GridBarrier *gb, int n_ctas, int *status)
{
    const int g = ld_acquire_gpu(&gb->gen);
    int prev;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(&gb->count) : "memory");
    if (prev == n_ctas - 1) {
        gb->count = 0;
        asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(&gb->gen), "r"(g + 1) : "memory");
        return ld_acquire_gpu(&gb->abort) == 0;
    }
    const long long t0 = clock64();
    while (ld_acquire_gpu(&gb->gen) == g) {
        if (ld_acquire_gpu(&gb->abort) != 0) return false;
        if (clock64() - t0 > CHAIN_BARRIER_CYCLES) {
            atomicExch(status, QZ_ERR_TIMEOUT);
            atomicExch(&gb->abort, 1);
            return false;
        }
    }
    return ld_acquire_gpu(&gb->abort) == 0;
}

// The consumer side of one op for policy F.  All TMA_CONSUMERS threads call it; threads beyond the op's
// Upad * RP take part in the ring protocol (every warp releases every stage) but compute nothing.
template <class F, int MODE>
__device__ __forceinline__ bool chain_consume(const ChainOp &op, int m, int cta, uint8_t *ring, int slot_bytes, int n_slots,
                                              uint64_t *full_bar, uint64_t *empty_bar, float (*part)[4 * (TMA_CONSUMERS / 32)],
                                              const XQ &xq, RingPos &rp, int *status, volatile int *cta_dead)
{
    const FormatInfo fi = format_info(F::TYPE);
    const int nb = op.K / fi.block_elems;
    const int row_bytes = nb * fi.block_bytes;
    const int ntiles = (op.N + op.RP - 1) / op.RP;
    const int n_consumers = op.Upad * op.RP;
    const bool worker = (int)threadIdx.x < n_consumers;
    const int u = threadIdx.x % op.Upad, rl = threadIdx.x / op.Upad;
    const bool active = worker && u < op.U;
    const int lane = threadIdx.x & 31;
    const int wpr = op.Upad >> 5;
    const int wir = MODE == 2 ? (threadIdx.x >> 5) % wpr : 0;
    float *y = op.y[m];
    typename F::XRegs xr;
    F::load_x(xr, xq, active ? u : 0);
    const typename F::Off off = F::make_off(nb, active ? u : 0);
    const int my_tiles = cta < op.n_cta ? (ntiles - cta + op.n_cta - 1) / op.n_cta : 0;
    const uint32_t ring0 = smem_u32(ring), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    const uint32_t row_off = (uint32_t)((worker ? rl : 0) * row_bytes);
    bool ok = true;   // warp-uniform
    for (int t0 = 0; t0 < my_tiles; t0 += 4) {
        float acc[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc[j] = 0.f;
            if (t0 + j < my_tiles) {
                if (ok && !mbar_wait_warp(full0 + 8 * rp.s, rp.parity, cta_dead)) {
                    if (lane == 0) {
                        atomicExch(status, QZ_ERR_TIMEOUT);
                        *cta_dead = 1;
                    }
                    ok = false;   // the warp keeps walking the stages and the named barriers, computing nothing
                }
                if (ok) {
                    if (worker) {
                        typename F::WRegs w;
                        F::template load_w<LdSharedAddr>(w, ring0 + (uint32_t)rp.s * (uint32_t)slot_bytes + row_off, off);
                        acc[j] = F::dot(w, xr, off, nullptr);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive_addr(empty0 + 8 * rp.s);
                }
                if (++rp.s == n_slots) { rp.s = 0; rp.parity ^= 1; }
            }
        }
        if (!worker) continue;   // (whole warps: n_consumers is a multiple of 32)
        const int row_j0 = (cta + t0 * op.n_cta) * op.RP + rl, row_step = op.n_cta * op.RP;
        auto store_y = [&](int row, float v) {
            if (*cta_dead) return;   // a warp of this CTA gave up: its rows are incomplete
            y[row] = op.accumulate ? __ldcg(y + row) + v : v;
        };
        const float v = warp_sum4(active ? acc[0] : 0.f, active ? acc[1] : 0.f, active ? acc[2] : 0.f, active ? acc[3] : 0.f,
                                  lane);
        const int j = lane >> 3;
        if (MODE == 1) {
            const int row = row_j0 + j * row_step;
            if ((lane & 7) == 0 && t0 + j < my_tiles && row < op.N) store_y(row, v);
        } else {
            float *p = part[(t0 >> 2) & 1] + rl * wpr * 4;
            if ((lane & 7) == 0) p[j * wpr + wir] = v;
            named_bar_sync(1 + rl, wpr * 32);
            if (wir == 0 && lane < 4) {
                float t = 0.f;
                for (int k = 0; k < wpr; k++) t += p[lane * wpr + k];
                const int row = row_j0 + lane * row_step;
                if (t0 + lane < my_tiles && row < op.N) store_y(row, t);
            }
        }
    }
    return ok;
}

__global__ void __launch_bounds__(TMA_CONSUMERS + 32, 1) gemv_chain_kernel(const __grid_constant__ ChainArgs a)
{
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ uint64_t full_bar[TMA_MAX_STAGES], empty_bar[TMA_MAX_STAGES];
    __shared__ float part[2][4 * (TMA_CONSUMERS / 32)];
    __shared__ float xred[TMA_CONSUMERS / 32];
    __shared__ int cta_ok, cta_dead;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.n_slots; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], TMA_CONSUMERS / 32);   // every consumer warp releases every stage
        }
        cta_ok = 1;
        cta_dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();

    if (threadIdx.x >= TMA_CONSUMERS) {
        // ---------------- producer: the weight rows of every op, back to back ----------------
        if (threadIdx.x != TMA_CONSUMERS) return;
        int s = 0, issued = 0;
        uint32_t round = 0;
        bool ok = true;
        for (int k = 0; k < a.n_ops && ok; k++) {
            const ChainOp &op = a.op[k];
            const FormatInfo fi = format_info(op.type);
            const int row_bytes = (op.K / fi.block_elems) * fi.block_bytes;
            const int ntiles = (op.N + op.RP - 1) / op.RP;
            const int m = blockIdx.x % op.n_mats, cta = blockIdx.x / op.n_mats;
            if (cta >= op.n_cta) continue;
            const uint8_t *W = op.W[m];
            for (int tile = cta; tile < ntiles; tile += op.n_cta) {
                if (round > 0) ok = mbar_wait(&empty_bar[s], (round - 1) & 1);
                if (!ok) break;
                const int row0 = tile * op.RP;
                const int rows = min(op.RP, op.N - row0);
                const uint32_t bytes = (uint32_t)rows * (uint32_t)row_bytes;
                mbar_arrive_expect_tx(&full_bar[s], bytes);
                tma_load_1d(ring + (size_t)s * a.slot_bytes, W + (size_t)row0 * row_bytes, bytes, &full_bar[s]);
                issued++;
                if (++s == a.n_slots) { s = 0; round++; }
            }
        }
        if (!ok) {
            atomicExch(a.status, QZ_ERR_TIMEOUT);
            // drain: copies already issued must land before this CTA's shared memory goes away
            for (int k = 0; k < a.n_slots && k < issued; k++) {
                const int j = issued - 1 - k;
                mbar_wait(&full_bar[j % a.n_slots], (j / a.n_slots) & 1);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int lane = threadIdx.x & 31;
    uint8_t *xarea = ring + (size_t)a.n_slots * a.slot_bytes;
    RingPos rp{0, 0};
    pdl_wait();   // op 0's inputs come from the preceding kernels
    bool ok = true;
    volatile int *dead_flag = &cta_dead;
    for (int k = 0; k < a.n_ops; k++) {
        const ChainOp &op = a.op[k];
        if (k > 0) {
            // every consumer warp arrives here, whether or not a wait of op k-1 ran out on it; afterwards the
            // whole CTA takes the same decision.  (Also: every warp has taken its activation registers, the
            // area is free.)
            named_bar_sync(13, TMA_CONSUMERS);
            if (!a.independent) {
                // ---- grid-wide barrier: op k-1's outputs are complete and visible ----
                if (threadIdx.x == 0) cta_ok = (!*dead_flag && grid_barrier(a.gb, gridDim.x, a.status)) ? 1 : 0;
                named_bar_sync(13, TMA_CONSUMERS);
            }
            ok = *(volatile int *)&cta_ok != 0 && !*dead_flag;
        }
        if (!ok) break;   // uniform over the CTA's consumers
        // ---- op k's activation vector, converted by this CTA into shared memory ----
        int8_t *sxl = (int8_t *)xarea, *sxh = sxl + op.K;
        float *sxs = (float *)(sxh + op.K), *sxsum = sxs + (op.K >> 5);
        {
            const XQOut o{sxl, sxh, sxs, sxsum};
            const float *pa = op.xsrc.a, *pb = op.xsrc.b;
            const int n4 = op.K >> 2;
            float4 xa[XSRC_MAX_IT], xb[XSRC_MAX_IT];
#pragma unroll
            for (int it = 0; it < XSRC_MAX_IT; it++) {
                const int t = it * TMA_CONSUMERS + threadIdx.x;
                if (t < n4) {
                    xa[it] = __ldcg((const float4 *)(pa + 4 * t));
                    xb[it] = op.xsrc.mode == 3 ? xa[it] : __ldcg((const float4 *)(pb + 4 * t));
                } else {
                    xa[it] = xb[it] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            float r = 1.f;
            if (op.xsrc.mode == 1) {
                float ss = 0.f;
#pragma unroll
                for (int it = 0; it < XSRC_MAX_IT; it++)
                    ss = fmaf(xa[it].x, xa[it].x, fmaf(xa[it].y, xa[it].y, fmaf(xa[it].z, xa[it].z, fmaf(xa[it].w, xa[it].w, ss))));
                for (int o2 = 16; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o2);
                if (lane == 0) xred[threadIdx.x >> 5] = ss;
                named_bar_sync(14, TMA_CONSUMERS);
                ss = 0.f;
                for (int w = 0; w < TMA_CONSUMERS / 32; w++) ss += xred[w];
                r = rsqrtf(ss / (float)op.K + 1e-5f);
            }
#pragma unroll
            for (int it = 0; it < XSRC_MAX_IT; it++) {
                if (it * TMA_CONSUMERS >= n4) break;   // uniform over the CTA
                const int t = it * TMA_CONSUMERS + threadIdx.x;
                const bool valid = t < n4;
                const float xx[4] = {xa[it].x, xa[it].y, xa[it].z, xa[it].w}, yy[4] = {xb[it].x, xb[it].y, xb[it].z, xb[it].w};
                float v[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    if (op.xsrc.mode == 1) {
                        v[i] = xx[i] * r * yy[i];
                    } else if (op.xsrc.mode == 3) {
                        v[i] = xx[i];
                    } else if (op.xsrc.oai) {
                        const float g = fminf(xx[i], 7.f), up = fmaxf(-7.f, fminf(7.f, yy[i]));
                        v[i] = __fdividef(g, 1.f + __expf(-1.702f * g)) * (up + 1.f);
                    } else {
                        v[i] = __fdividef(xx[i], 1.f + __expf(-xx[i])) * yy[i];   // fast exp / divide: this runs redundantly in every CTA
                    }
                }
                quantize4_store(v, t, valid, o);
            }
            named_bar_sync(14, TMA_CONSUMERS);
        }
        const XQ xq{sxl, sxh, sxs, sxsum};
        const int m = blockIdx.x % op.n_mats, cta = blockIdx.x / op.n_mats;
#define QZ_CHAIN_CASE(TT, POL)                                                                                              \
    case TT:                                                                                                                \
        ok = op.Upad == 32 ? chain_consume<POL, 1>(op, m, cta, ring, a.slot_bytes, a.n_slots, full_bar, empty_bar, part, xq, rp,  \
                                                   a.status, dead_flag)                                                     \
                           : chain_consume<POL, 2>(op, m, cta, ring, a.slot_bytes, a.n_slots, full_bar, empty_bar, part, xq, rp,  \
                                                   a.status, dead_flag);                                                    \
        break;
        switch (op.type) {
            QZ_CHAIN_CASE(T_Q4_K, StreamQ4K)
            QZ_CHAIN_CASE(T_Q6_K, StreamQ6K)
            QZ_CHAIN_CASE(T_Q8_0, StreamQ8_0)
        default: ok = false; break;
        }
#undef QZ_CHAIN_CASE
        // a warp whose wait ran out tells the other CTAs (they leave at their next grid barrier) and goes on to
        // this CTA's next meeting point like every other warp
        if (!ok) atomicExch(&a.gb->abort, 1);
    }
}

}  // namespace qz
