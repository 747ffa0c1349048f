// A chain of dependent GEMVs in ONE persistent kernel.
//
// In a decode step every GEMV depends on its predecessor (o-projection -> gate/up -> down -> next
// layer's q/k/v), and at batch 1 each of them streams for only 2-10 us.  As separate kernels they pay,
// per link, the latency from one grid's completion to the release of its dependents plus an empty
// weight pipeline.  Here one CTA per SM runs the whole chain:
//   * the producer lane streams the weight rows of op 0, op 1, ... back to back through the same
//     shared-memory ring (weights depend on nothing, so it never waits for a link).  The ring is a
//     circular BYTE buffer: a stage takes exactly the bytes of its op's row tile, so an op with small
//     stages keeps as many bytes in flight as one with large stages (a ring of fixed-size slots would
//     be sized for the largest stage of any op and run the others half empty);
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
    int rot;                // the op's CTA numbering starts at this CTA (spreads the ops' odd tiles over the grid)
    int x_off;              // byte offset of the op's converted activation vector behind the ring; < 0: the vector
                            // was converted by a kernel before this one and is read from `xg` (global memory)
    XQ xg;
    long long push_off;     // >= 0: rows go to every rank's window instead of y: matrix m at push_off + m * push_stride
    long long push_stride;
    XSrc xsrc;              // mode 1 (RMSNorm), 2 (SwiGLU) or 3 (plain f32 vector a)
};


struct GridBarrier {
    int count, gen, abort;
};

struct ChainArgs {
    ChainOp op[CHAIN_MAX_OPS];
    int n_ops;
    int independent;           // 1: no op reads another op's output: no grid barrier between them
    int exchange;              // 1 (dependent ops that push): between two ops the ranks exchange instead of the grid
                               // barrier: every CTA counts in, the last one publishes, every CTA polls all ranks' flags
    int ring_bytes;            // the circular byte buffer (a multiple of 128; every stage fits at least three times)
    GridBarrier *gb;
    int *status;
    PushArgs push;             // the ranks' windows, when an op pushes
};

// State of the weight ring as one role sees it; survives from op to op.  Stage number `seq` uses barrier
// seq % TMA_MAX_STAGES in its (seq / TMA_MAX_STAGES)-th phase and the bytes [off, off + size): `off` follows the
// previous stage, or is 0 when the stage would run past the end of the buffer.  Producer and consumers apply the same
// rule to the same sequence of stage sizes, so they agree on every offset without exchanging it.
struct RingPos {
    uint32_t seq;
    uint32_t next_off;
};
__device__ __forceinline__ uint32_t ring_place(RingPos &rp, uint32_t size, uint32_t ring_bytes)
{
    uint32_t off = rp.next_off;
    if (off + size > ring_bytes) off = 0;
    rp.next_off = off + size;
    return off;
}
__device__ __forceinline__ uint32_t chain_stage_bytes(const ChainOp &op)
{
    const FormatInfo fi = format_info(op.type);
    return (uint32_t)((op.RP * (op.K / fi.block_elems) * fi.block_bytes + 127) & ~127);
}

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
__device__ __forceinline__ bool chain_consume(const ChainOp &op, int m, int cta, uint8_t *ring, int ring_bytes,
                                              uint64_t *full_bar, uint64_t *empty_bar, float (*part)[4 * (TMA_CONSUMERS / 32)],
                                              const XQ &xq, RingPos &rp, int *status, volatile int *cta_dead,
                                              const PushArgs &push)
{
    // the fields of the op that the loops below use, in registers (the op sits in the kernel's parameter space and
    // is picked with a run-time index)
    const int op_n_cta = op.n_cta, op_RP = op.RP, op_N = op.N, op_acc = op.accumulate;
    const long long op_push_off = op.push_off, op_push_stride = op.push_stride;
    const FormatInfo fi = format_info(F::TYPE);
    const int nb = op.K / fi.block_elems;
    const int row_bytes = nb * fi.block_bytes;
    const int ntiles = (op_N + op_RP - 1) / op_RP;
    const int n_consumers = op.Upad * op_RP;
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
    const int my_tiles = cta < op_n_cta ? (ntiles - cta + op_n_cta - 1) / op_n_cta : 0;
    const uint32_t ring0 = smem_u32(ring), full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    const uint32_t row_off = (uint32_t)((worker ? rl : 0) * row_bytes);
    const uint32_t stage = chain_stage_bytes(op);
    bool ok = true;   // warp-uniform
    for (int t0 = 0; t0 < my_tiles; t0 += 4) {
        float acc[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc[j] = 0.f;
            if (t0 + j < my_tiles) {
                const uint32_t bs = rp.seq % TMA_MAX_STAGES, parity = (rp.seq / TMA_MAX_STAGES) & 1;
                const uint32_t off_s = ring_place(rp, stage, (uint32_t)ring_bytes);
                rp.seq++;
                if (ok && !mbar_wait_warp(full0 + 8 * bs, parity, cta_dead)) {
                    if (lane == 0) {
                        atomicExch(status, QZ_ERR_TIMEOUT);
                        *cta_dead = 1;
                    }
                    ok = false;   // the warp keeps walking the stages and the named barriers, computing nothing
                }
                if (ok) {
                    if (worker) {
                        typename F::WRegs w;
                        F::template load_w<LdSharedAddr>(w, ring0 + off_s + row_off, off);
                        acc[j] = F::dot(w, xr, off, nullptr);
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive_addr(empty0 + 8 * bs);
                }
            }
        }
        if (!worker) continue;   // (whole warps: n_consumers is a multiple of 32)
        const int row_j0 = (cta + t0 * op_n_cta) * op_RP + rl, row_step = op_n_cta * op_RP;
        auto store_y = [&](int row, float v) {
            if (*cta_dead) return;   // a warp of this CTA gave up: its rows are incomplete
            if (op_push_off >= 0) {
                for (int rk = 0; rk < push.n; rk++) push.data[rk][op_push_off + m * op_push_stride + row] = v;
            } else {
                y[row] = op_acc ? __ldcg(y + row) + v : v;
            }
        };
        const float v = warp_sum4(active ? acc[0] : 0.f, active ? acc[1] : 0.f, active ? acc[2] : 0.f, active ? acc[3] : 0.f,
                                  lane);
        const int j = lane >> 3;
        if (MODE == 1) {
            const int row = row_j0 + j * row_step;
            if ((lane & 7) == 0 && t0 + j < my_tiles && row < op_N) store_y(row, v);
        } else {
            float *p = part[(t0 >> 2) & 1] + rl * wpr * 4;
            if ((lane & 7) == 0) p[j * wpr + wir] = v;
            named_bar_sync(1 + rl, wpr * 32);
            if (wir == 0 && lane < 4) {
                float t = 0.f;
                for (int k = 0; k < wpr; k++) t += p[lane * wpr + k];
                const int row = row_j0 + lane * row_step;
                if (t0 + lane < my_tiles && row < op_N) store_y(row, t);
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
        for (int s = 0; s < TMA_MAX_STAGES; s++) {
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
        // `head` walks this CTA's stages and issues their copies.  Every stage also gets a VIRTUAL byte position that
        // only grows: its start is the previous stage's end plus the bytes skipped at the end of the buffer when the
        // stage did not fit there.  Stages are released in issue order, so the bytes still owned by stages in flight
        // are exactly the virtual span from the oldest stage's start to the newest one's end; a new stage may be
        // issued once that span, extended to the new stage's end, is no longer than the buffer.
        struct Walk {
            int k, tile;         // current stage: op and tile (tile < 0: the op has not been entered yet)
            RingPos rp;
            uint32_t off, size;  // the current stage's bytes
            // constants of op k for this CTA (filled when the op is entered)
            int n_cta, ntiles, first;
        };
        auto enter_op = [&](Walk &w) {   // op w.k: this CTA's first tile (or none), tile stride, stage size
            const ChainOp &op = a.op[w.k];
            const int me = ((int)blockIdx.x + (int)gridDim.x - op.rot) % (int)gridDim.x;
            const int cta = me / op.n_mats;
            w.n_cta = op.n_cta;
            w.ntiles = (op.N + op.RP - 1) / op.RP;
            w.first = cta < op.n_cta ? cta : w.ntiles;   // no tile at all: start past the end
            w.size = chain_stage_bytes(op);
        };
        auto advance = [&](Walk &w) -> bool {   // moves to the CTA's next stage; false when there is none
            for (;;) {
                if (w.k >= a.n_ops) return false;
                if (w.tile < 0) enter_op(w);
                const int next = w.tile < 0 ? w.first : w.tile + w.n_cta;
                if (next < w.ntiles) {
                    w.tile = next;
                    w.off = ring_place(w.rp, w.size, (uint32_t)a.ring_bytes);
                    w.rp.seq++;
                    return true;
                }
                w.k++;
                w.tile = -1;
            }
        };
        Walk head{0, -1, {0, 0}, 0, 0, 0, 0, 0};
        int cur_k = -1, row_bytes = 0, RPk = 0, Nk = 0;
        const uint8_t *Wk = nullptr;
        uint32_t vstart[TMA_MAX_STAGES];       // virtual start of stage number n at slot n % TMA_MAX_STAGES
        uint32_t head_v = 0, prev_end = 0;     // virtual end of the newest stage; buffer offset where it ended
        uint32_t oldest = 0, in_flight = 0;    // stages [oldest, oldest + in_flight) are in flight
        bool ok = true;
        while (ok && advance(head)) {
            const uint32_t v0 = head_v + (head.off == 0 && prev_end != 0 ? (uint32_t)a.ring_bytes - prev_end : 0u);
            const uint32_t v1 = v0 + head.size;
            while (in_flight && (in_flight >= TMA_MAX_STAGES || v1 - vstart[oldest % TMA_MAX_STAGES] > (uint32_t)a.ring_bytes)) {
                ok = mbar_wait(&empty_bar[oldest % TMA_MAX_STAGES], (oldest / TMA_MAX_STAGES) & 1);
                if (!ok) break;
                oldest++;
                in_flight--;
            }
            if (!ok) break;
            if (head.k != cur_k) {   // first stage of an op: its weight matrix and row geometry
                cur_k = head.k;
                const ChainOp &op = a.op[cur_k];
                const FormatInfo fi = format_info(op.type);
                row_bytes = (op.K / fi.block_elems) * fi.block_bytes;
                const int me = ((int)blockIdx.x + (int)gridDim.x - op.rot) % (int)gridDim.x;
                Wk = op.W[me % op.n_mats];
                RPk = op.RP;
                Nk = op.N;
            }
            const int row0 = head.tile * RPk;
            const int rows = min(RPk, Nk - row0);
            const uint32_t bytes = (uint32_t)rows * (uint32_t)row_bytes;
            const uint32_t hs = head.rp.seq - 1;
            mbar_arrive_expect_tx(&full_bar[hs % TMA_MAX_STAGES], bytes);
            tma_load_1d(ring + head.off, Wk + (size_t)row0 * row_bytes, bytes, &full_bar[hs % TMA_MAX_STAGES]);
            vstart[hs % TMA_MAX_STAGES] = v0;
            head_v = v1;
            prev_end = head.off + head.size;
            in_flight++;
        }
        if (!ok) {
            atomicExch(a.status, QZ_ERR_TIMEOUT);
            // drain: copies already issued must land before this CTA's shared memory goes away
            const uint32_t issued = head.rp.seq - 1;   // (the stage whose room was not found has not been issued)
            for (uint32_t k = 0; k < TMA_MAX_STAGES && k < issued; k++) {
                const uint32_t j = issued - 1 - k;
                mbar_wait(&full_bar[j % TMA_MAX_STAGES], (j / TMA_MAX_STAGES) & 1);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    const int lane = threadIdx.x & 31;
    uint8_t *xarea = ring + (size_t)a.ring_bytes;
    RingPos rp{0, 0};
    pdl_wait();   // op 0's inputs come from the preceding kernels
    bool ok = true;
    volatile int *dead_flag = &cta_dead;
    // an op's activation vector, converted by this CTA into its area behind the ring
    auto convert = [&](const ChainOp &op) {
        int8_t *sxl = (int8_t *)(xarea + op.x_off), *sxh = sxl + op.K;
        float *sxs = (float *)(sxh + op.K), *sxsum = sxs + (op.K >> 5);
        const XQOut o{sxl, sxh, sxs, sxsum};
        const float *pa = op.xsrc.a, *pb = op.xsrc.b;
        const int n4 = op.K >> 2;
        // The vector is taken in pieces of XSRC_MAX_IT float4 per thread; all loads of a piece are issued before
        // anything is computed.  RMSNorm needs the whole vector's sum of squares first: the host only plans it for
        // vectors of one piece.
        for (int base = 0; base < n4; base += XSRC_MAX_IT * TMA_CONSUMERS) {
            float4 xa[XSRC_MAX_IT], xb[XSRC_MAX_IT];
#pragma unroll
            for (int it = 0; it < XSRC_MAX_IT; it++) {
                const int t = base + it * TMA_CONSUMERS + threadIdx.x;
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
                named_bar_sync(14, TMA_CONSUMERS);   // the previous conversion's partial sums have been read
                if (lane == 0) xred[threadIdx.x >> 5] = ss;
                named_bar_sync(14, TMA_CONSUMERS);
                ss = 0.f;
                for (int w = 0; w < TMA_CONSUMERS / 32; w++) ss += xred[w];
                r = rsqrtf(ss / (float)op.K + 1e-5f);
            }
#pragma unroll
            for (int it = 0; it < XSRC_MAX_IT; it++) {
                if (base + it * TMA_CONSUMERS >= n4) break;   // uniform over the CTA
                const int t = base + it * TMA_CONSUMERS + threadIdx.x;
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
        }
    };
    if (a.independent) {
        // no op reads what another writes: every activation vector is converted up front, each into an area of
        // its own, while the ring fills; afterwards the ops follow one another without a pause
        bool any = false;
        for (int k = 0; k < a.n_ops; k++)
            if (a.op[k].x_off >= 0) {
                convert(a.op[k]);
                any = true;
            }
        if (any) named_bar_sync(14, TMA_CONSUMERS);
    }
    bool unpublished = false;   // an op has pushed rows that no publish has covered yet
    // exchanges this rank had published when the kernel started (read after the wait above: the previous kernel's
    // publish is then complete; this kernel's first publish needs every CTA, this one included, to finish op 0)
    const int push_base = a.exchange ? *(volatile const int *)&a.push.ctrl[a.push.rank]->pushes : 0;
    for (int k = 0; k < a.n_ops; k++) {
        const ChainOp &op = a.op[k];
        if (k > 0 && !a.independent) {
            // every consumer warp arrives here, whether or not a wait of op k-1 ran out on it; afterwards the
            // whole CTA takes the same decision.  (Also: every warp has taken its activation registers, the
            // area is free.)
            named_bar_sync(13, TMA_CONSUMERS);
            if (!a.exchange) {
                // ---- grid-wide barrier: op k-1's outputs are complete and visible ----
                if (threadIdx.x == 0) cta_ok = (!*dead_flag && grid_barrier(a.gb, gridDim.x, a.status)) ? 1 : 0;
            } else {
                // ---- exchange: op k-1's rows sit in every rank's window once every rank has published ----
                // This CTA counts in (the last CTA of the rank publishes); then lanes 0..n-1 poll this rank's flag
                // words until every rank has published k exchanges more than it had when the kernel started.  The
                // poll doubles as the grid barrier (this rank's own flag is one of them).  Bounded like every wait.
                if (threadIdx.x == 0) {
                    cta_ok = 1;
                    if (!*dead_flag) push_publish(a.push, gridDim.x);
                }
                unpublished = false;
                if ((int)threadIdx.x < 32) {
                    bool fine = true;
                    if ((int)threadIdx.x < a.push.n) {
                        const MgpuCtrl *mine = a.push.ctrl[a.push.rank];
                        const int expected = push_base + k;
                        const long long t0 = clock64();
                        while (ld_acquire_sys(&mine->flags[threadIdx.x]) - expected < 0) {
                            if (clock64() - t0 > MGPU_WAIT_CYCLES) {
                                atomicExch(a.status, QZ_ERR_TIMEOUT);
                                fine = false;
                                break;
                            }
                            __nanosleep(32);
                        }
                    }
                    if (!__all_sync(0xFFFFFFFFu, fine) && lane == 0) cta_ok = 0;
                }
            }
            named_bar_sync(13, TMA_CONSUMERS);
            ok = *(volatile int *)&cta_ok != 0 && !*dead_flag;
        }
        // Independent ops need no grid barrier, but the CTA's consumer warps still meet between two ops: the named
        // barriers (ids 1 + row group, counted per op's row geometry) and the partial-sum buffer of the row
        // reduction are laid out per op, and a warp that ran ahead into op k would use them with op k's thread
        // counts while a slower warp is still inside op k-1.
        if (k > 0 && a.independent) named_bar_sync(13, TMA_CONSUMERS);
        if (!ok) break;   // uniform over the CTA's consumers (independent ops: a dead CTA just walks on, storing nothing)
        if (!a.independent) {
            convert(op);
            named_bar_sync(14, TMA_CONSUMERS);
        }
        int8_t *sxl = (int8_t *)(xarea + (op.x_off >= 0 ? op.x_off : 0)), *sxh = sxl + op.K;
        float *sxs = (float *)(sxh + op.K), *sxsum = sxs + (op.K >> 5);
        unpublished = unpublished || op.push_off >= 0;
        const XQ xq = op.x_off >= 0 ? XQ{sxl, sxh, sxs, sxsum} : op.xg;
        const int me = ((int)blockIdx.x + (int)gridDim.x - op.rot) % (int)gridDim.x;
        const int m = me % op.n_mats, cta = me / op.n_mats;
#define QZ_CHAIN_CASE(TT, POL)                                                                                              \
    case TT:                                                                                                                \
        ok = op.Upad == 32 ? chain_consume<POL, 1>(op, m, cta, ring, a.ring_bytes, full_bar, empty_bar, part, xq, rp,          \
                                                   a.status, dead_flag, a.push)                                             \
                           : chain_consume<POL, 2>(op, m, cta, ring, a.ring_bytes, full_bar, empty_bar, part, xq, rp,          \
                                                   a.status, dead_flag, a.push);                                            \
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
        if (a.independent) ok = true;   // (independent ops: walk on; a dead CTA stores nothing and does not publish)
    }
    if (unpublished) {
        // all of this CTA's remote stores are issued: meet, then one thread fences them and counts the CTA in
        named_bar_sync(13, TMA_CONSUMERS);
        if (threadIdx.x == 0 && !*dead_flag) push_publish(a.push, gridDim.x, a.status, true);
    }
}

}  // namespace qz
