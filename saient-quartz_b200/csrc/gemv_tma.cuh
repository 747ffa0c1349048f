// TMA-staged streaming GEMV: the production batch-1 kernel.
//
// One persistent CTA per SM.  A producer lane walks this CTA's row tiles and moves
// each tile (RT consecutive rows = one contiguous, 16-byte aligned byte range in
// either weight layout) from HBM into a shared-memory ring with one bulk async copy
// (cp.async.bulk ... mbarrier::complete_tx::bytes), as many stages ahead as the ring
// is deep (~200 KB per SM in flight).  Memory traffic therefore never waits on
// arithmetic, and a matrix of a few tens of MB has all of its bytes requested within
// the first microsecond.  Sixteen consumer warps unpack from shared memory with the
// same per-format integer dot products as gemv_stream.cuh (activation slice in
// registers, dp4a on two int8 limbs), reduce each row with shuffles and a
// row-group named barrier, and hand the stage back through an "empty" mbarrier.
//
// Every wait is bounded: a warp that polls an mbarrier for longer than ~1 s of SM
// clocks records QZ_ERR_TIMEOUT in a device status word and raises a CTA-wide flag.
// From then on every consumer warp of the CTA skips its waits and its arithmetic but
// still walks the remaining stages and arrives at every named barrier, so no warp is
// left behind at one; nothing more is stored.  The producer drains its own outstanding
// copies (bounded) before it exits.
#pragma once

#include "gemv_formats_iq.cuh"
#include "gemv_formats_k.cuh"
#include "mgpu.cuh"

namespace qz {

constexpr int TMA_MAX_STAGES = 16;
#ifndef QZ_TMA_CONSUMERS
#define QZ_TMA_CONSUMERS 512
#endif
constexpr int TMA_CONSUMERS = QZ_TMA_CONSUMERS;
constexpr int XSRC_MAX_IT = 4;             // float4 loads per consumer thread in the fused activation prologue
constexpr long long TMA_WAIT_CYCLES = 2000000000LL;   // ~1 s at 1.9 GHz

// Where the activation vector comes from.  mode 0: already converted (xq).  mode 1: RMSNorm of the
// f32 vector a with weights b (src/cuda_kernels.cu:563-575, eps 1e-5 as there), mode 2: SwiGLU of
// gate a and up b (src/cuda_kernels.cu:683-698; oai = the clamped variant), mode 3: the f32 vector a
// as it is (what cuda_gemv gets).  For modes 1 to 3 every
// CTA converts the vector itself, into shared memory, while its weight pipeline fills: the producer of
// the activations needs no kernel of its own.
struct XSrc {
    int mode;
    const float *a, *b;
    int oai;
};

// Byte ranges (the weights of the operations that FOLLOW this GEMV) that the producer lanes pull into L2 once
// their own weight stream has been issued: while this kernel drains its ring, reduces, exits and its successor
// starts up, HBM keeps working for the successor, whose first tiles then come from L2.
constexpr int QZ_MAX_PREFETCH = 4;
struct PrefetchHint {
    const uint8_t *ptr[QZ_MAX_PREFETCH];
    unsigned bytes[QZ_MAX_PREFETCH];   // per range, a multiple of 16
    int n;
};

__device__ __forceinline__ void l2_prefetch_bulk(const void *gmem, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gmem), "r"(bytes) : "memory");
}

// 16 KB pieces of every hinted range, piece j issued by CTA j % n_cta: the front of a range (what the successor
// reads first) is requested first by everybody
__device__ __forceinline__ void issue_prefetch(const PrefetchHint &h, int cta, int n_cta)
{
    for (int i = 0; i < h.n; i++) {
        for (unsigned o = (unsigned)cta * 16384u; o < h.bytes[i]; o += (unsigned)n_cta * 16384u)
            l2_prefetch_bulk(h.ptr[i] + o, min(16384u, h.bytes[i] - o));
    }
}

struct TmaArgs {
    const uint8_t *W[QZ_MAX_MATS];
    XQ xq[QZ_MAX_MATS];
    float *y[QZ_MAX_MATS];
    int K, N;
    int accumulate;          // 1: y += W x
    int U, Upad, RP;         // units per row, threads per row, rows per stage
    int n_mats;
    int stage_bytes;         // RP * row_bytes, a multiple of 16
    int n_stages;
    int *status;             // device status word (0 = ok)
    PushArgs push;           // push.n > 0: rows go to every rank's window instead of y (single matrix)
    XSrc xsrc;
    PrefetchHint pf;         // weights of the following operations, to be pulled into L2
    const int *sel;          // not NULL: matrix m really starts at W[m] + sel[m] * sel_stride (expert ids chosen on the device)
    size_t sel_stride;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait; false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > TMA_WAIT_CYCLES) return false;
    }
    return true;
}
__device__ __forceinline__ void tma_load_1d(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// loads through 32-bit shared-window addresses (no generic-address arithmetic in the hot loop)
struct LdSharedAddr {
    __device__ static uint4 v4(uint32_t a)
    {
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
        return v;
    }
    __device__ static uint2 v2(uint32_t a)
    {
        uint2 v;
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
        return v;
    }
    __device__ static uint32_t u32(uint32_t a)
    {
        uint32_t v;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
        return v;
    }
    __device__ static uint32_t u16(uint32_t a)
    {
        uint16_t v;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
        return v;
    }
};

__device__ __forceinline__ bool mbar_try_wait_addr(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity)
{
    const long long t0 = clock64();
    while (!mbar_try_wait_addr(bar, parity)) {
        if (clock64() - t0 > TMA_WAIT_CYCLES) return false;
    }
    return true;
}
__device__ __forceinline__ bool mbar_wait_addr(uint32_t bar, uint32_t parity)
{
    if (mbar_try_wait_addr(bar, parity)) return true;
    return mbar_wait_slow(bar, parity);
}
// The same wait for the consumer warps of the streaming GEMVs: it also ends (false) as soon as another
// warp of the CTA has raised `*dead_flag`, so that after one timeout nobody spends a second on each stage.
__device__ __noinline__ bool mbar_wait_slow_flag(uint32_t bar, uint32_t parity, const volatile int *dead_flag)
{
    const long long t0 = clock64();
    while (!mbar_try_wait_addr(bar, parity)) {
        if (*dead_flag) return false;
        if (clock64() - t0 > TMA_WAIT_CYCLES) return false;
    }
    return true;
}
// Warp-uniform result: all 32 lanes call it together; false for the whole warp if any lane gave up.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const volatile int *dead_flag)
{
    bool ok = mbar_try_wait_addr(bar, parity);
    if (!ok) ok = mbar_wait_slow_flag(bar, parity, dead_flag);
    return __all_sync(0xFFFFFFFFu, ok);
}
__device__ __forceinline__ void mbar_arrive_addr(uint32_t bar)
{
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(bar) : "memory");
}

// MODE 0: fewer than 32 threads per row (K < 2048); 1: one warp per row; 2: several warps per row.
// A stage holds RP consecutive rows (one per thread-row); partial sums are carried over
// GROUP = 4 stages and reduced together (6 shuffles for 4 rows instead of 20).
template <class F, int MODE>
__global__ void __launch_bounds__(TMA_CONSUMERS + 32, 1) gemv_tma_kernel(const TmaArgs a)
{
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ uint64_t full_bar[TMA_MAX_STAGES], empty_bar[TMA_MAX_STAGES];
    __shared__ float part[2][4 * (TMA_CONSUMERS / 32)];
    __shared__ float xred[TMA_CONSUMERS / 32];
    __shared__ int cta_dead;   // raised by the first consumer warp whose wait ran out

    const int m = blockIdx.x % a.n_mats;
    const int cta = blockIdx.x / a.n_mats, n_cta = gridDim.x / a.n_mats;
    const FormatInfo fi = format_info(F::TYPE);
    const int nb = a.K / fi.block_elems;
    const int row_bytes = nb * fi.block_bytes;
    const int ntiles = (a.N + a.RP - 1) / a.RP;
    const int n_consumers = a.Upad * a.RP;

    uint8_t *tbl = ring + (size_t)a.n_stages * a.stage_bytes;   // codebook copy, behind the ring
    F::load_table(tbl, threadIdx.x, blockDim.x);
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.n_stages; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], (n_consumers + 31) >> 5);
        }
        cta_dead = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    pdl_trigger();

    const int first_producer = (int)blockDim.x - 32;   // the last warp is the producer warp
    if ((int)threadIdx.x >= first_producer) {
        // ---------------- producer ----------------
        // Weights are written by no kernel, so streaming starts at once, even while the kernel
        // that produces this GEMV's activations is still running.
        if ((int)threadIdx.x != first_producer) return;
        const uint8_t *W = a.W[m];
        if (a.sel) {
            pdl_wait();   // the ids are written by the kernel before this one
            W += (size_t)a.sel[m] * a.sel_stride;
        }
        int it = 0, s = 0;
        uint32_t round = 0;
        bool ok = true;
        for (int tile = cta; tile < ntiles; tile += n_cta, it++) {
            if (round > 0) ok = mbar_wait(&empty_bar[s], (round - 1) & 1);
            if (!ok) break;
            const int row0 = tile * a.RP;
            const int rows = min(a.RP, a.N - row0);
            const uint32_t bytes = (uint32_t)rows * (uint32_t)row_bytes;
            mbar_arrive_expect_tx(&full_bar[s], bytes);
            tma_load_1d(ring + (size_t)s * a.stage_bytes, W + (size_t)row0 * row_bytes, bytes, &full_bar[s]);
            if (++s == a.n_stages) { s = 0; round++; }
        }
        if (ok && a.pf.n > 0) issue_prefetch(a.pf, blockIdx.x, gridDim.x);
        if (!ok) {
            atomicExch(a.status, QZ_ERR_TIMEOUT);
            // drain: copies already issued must land before this CTA's shared memory goes away
            for (int k = 0; k < a.n_stages && k < it; k++) {
                const int j = it - 1 - k;
                mbar_wait(&full_bar[j % a.n_stages], (j / a.n_stages) & 1);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    if ((int)threadIdx.x >= n_consumers) return;
    const int u = threadIdx.x % a.Upad;
    const int rl = threadIdx.x / a.Upad;
    const bool active = u < a.U;
    const int lane = threadIdx.x & 31;
    const int wpr = a.Upad >> 5;
    const int wir = MODE == 2 ? (threadIdx.x >> 5) % wpr : 0;
    float *__restrict__ y = a.y[m];
    // the row's result: a local store, or (row-sharded layers) a store into every rank's window
    auto store_y = [&](int row, float v) {
        if (*(const volatile int *)&cta_dead) return;   // a warp of this CTA gave up: its rows are incomplete
        if (a.push.n == 0) {
            y[row] = a.accumulate ? y[row] + v : v;
        } else {
            for (int r = 0; r < a.push.n; r++) a.push.data[r][a.push.dst_off + row] = v;
        }
    };
    bool dead = false;

    // Padding lanes (u >= U) run on unit 0's bytes and are masked out of the sums; rows past
    // N in the last tile are computed from stale shared memory and simply never stored.
    pdl_wait();   // activations (and, for the accumulate epilogue, y) come from the preceding kernels
    typename F::XRegs xr;
    XQ xq = a.xq[m];
    if (a.xsrc.mode) {
        // the activation form of the whole vector, built by this CTA's consumers behind ring and codebook
        int8_t *sxl = (int8_t *)(tbl + ((F::TABLE_BYTES + 15) & ~15));
        int8_t *sxh = sxl + a.K;
        float *sxs = (float *)(sxh + a.K), *sxsum = sxs + (a.K >> 5);
        const XQOut o{sxl, sxh, sxs, sxsum};
        const float *__restrict__ pa = a.xsrc.a, *__restrict__ pb = a.xsrc.b;
        const int n4 = a.K >> 2;
        // all of this thread's loads are issued before anything is computed: one L2 round trip, not one per
        // pass (the host only takes this path when XSRC_MAX_IT passes cover the vector)
        float4 xa[XSRC_MAX_IT], xb[XSRC_MAX_IT];
#pragma unroll
        for (int it = 0; it < XSRC_MAX_IT; it++) {
            const int t = it * n_consumers + threadIdx.x;
            if (t < n4) {
                xa[it] = __ldcg((const float4 *)(pa + 4 * t));
                xb[it] = a.xsrc.mode == 3 ? xa[it] : __ldcg((const float4 *)(pb + 4 * t));
            } else {
                xa[it] = xb[it] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        float r = 1.f;
        if (a.xsrc.mode == 1) {
            float ss = 0.f;
#pragma unroll
            for (int it = 0; it < XSRC_MAX_IT; it++)
                ss = fmaf(xa[it].x, xa[it].x, fmaf(xa[it].y, xa[it].y, fmaf(xa[it].z, xa[it].z, fmaf(xa[it].w, xa[it].w, ss))));
            for (int o2 = 16; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(0xFFFFFFFFu, ss, o2);
            if (lane == 0) xred[threadIdx.x >> 5] = ss;
            named_bar_sync(14, n_consumers);
            ss = 0.f;
            for (int w = 0; w < (n_consumers >> 5); w++) ss += xred[w];
            r = rsqrtf(ss / (float)a.K + 1e-5f);
        }
#pragma unroll
        for (int it = 0; it < XSRC_MAX_IT; it++) {
            if (it * n_consumers >= n4) break;   // uniform over the CTA
            const int t = it * n_consumers + threadIdx.x;
            const bool valid = t < n4;
            const float xx[4] = {xa[it].x, xa[it].y, xa[it].z, xa[it].w}, yy[4] = {xb[it].x, xb[it].y, xb[it].z, xb[it].w};
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                if (a.xsrc.mode == 1) {
                    v[i] = xx[i] * r * yy[i];
                } else if (a.xsrc.mode == 3) {
                    v[i] = xx[i];
                } else if (a.xsrc.oai) {
                    const float g = fminf(xx[i], 7.f), up = fmaxf(-7.f, fminf(7.f, yy[i]));
                    v[i] = __fdividef(g, 1.f + __expf(-1.702f * g)) * (up + 1.f);
                } else {
                    v[i] = __fdividef(xx[i], 1.f + __expf(-xx[i])) * yy[i];   // fast exp / divide: this runs redundantly in every CTA
                }
            }
            quantize4_store(v, t, valid, o);
        }
        named_bar_sync(14, n_consumers);
        xq = XQ{sxl, sxh, sxs, sxsum};
    }
    F::load_x(xr, xq, active ? u : 0);
    const typename F::Off off = F::make_off(nb, active ? u : 0);

    const int my_tiles = (ntiles - cta + n_cta - 1) / n_cta;
    const int n_stages = a.n_stages;
    const uint32_t stage_bytes = (uint32_t)a.stage_bytes;
    const uint32_t row_base = smem_u32(ring) + (uint32_t)(rl * row_bytes);   // my row inside stage 0
    const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    uint32_t sp = row_base, bar_off = 0, parity = 0;
    int s = 0;
    const volatile int *dead_flag = &cta_dead;
    for (int t0 = 0; t0 < my_tiles; t0 += 4) {
        float acc[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            acc[j] = 0.f;
            if (t0 + j < my_tiles) {
                if (!dead && !mbar_wait_warp(full0 + bar_off, parity, dead_flag)) {
                    if (lane == 0) {
                        atomicExch(a.status, QZ_ERR_TIMEOUT);
                        cta_dead = 1;
                    }
                    dead = true;   // warp-uniform; the warp keeps walking the stages and the named barriers
                }
                if (!dead) {
                    typename F::WRegs w;
                    F::template load_w<LdSharedAddr>(w, sp, off);
                    acc[j] = F::dot(w, xr, off, tbl);
                    __syncwarp();
                    if (lane == 0) mbar_arrive_addr(empty0 + bar_off);   // this warp no longer reads the stage
                }
                sp += stage_bytes;
                bar_off += 8;
                if (++s == n_stages) { s = 0; sp = row_base; bar_off = 0; parity ^= 1; }
            }
        }
        // ---- reduce the group's (up to) four rows ----
        // row of group member j: tile (cta + (t0 + j) * n_cta), thread-row rl
        const int row_j0 = (cta + t0 * n_cta) * a.RP + rl, row_step = n_cta * a.RP;
        if (MODE == 0) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float v = active ? acc[j] : 0.f;
                for (int o = a.Upad >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                const int row = row_j0 + j * row_step;
                if (u == 0 && t0 + j < my_tiles && row < a.N) store_y(row, v);
            }
        } else {
            const float v = warp_sum4(active ? acc[0] : 0.f, active ? acc[1] : 0.f, active ? acc[2] : 0.f,
                                      active ? acc[3] : 0.f, lane);
            const int j = lane >> 3;   // which of the four rows this lane's total belongs to
            if (MODE == 1) {
                const int row = row_j0 + j * row_step;
                if ((lane & 7) == 0 && t0 + j < my_tiles && row < a.N) store_y(row, v);
            } else {
                // the row's warps meet at their own named barrier; its first warp finishes the sums
                float *p = part[(t0 >> 2) & 1] + rl * wpr * 4;
                if ((lane & 7) == 0) p[j * wpr + wir] = v;
                named_bar_sync(1 + rl, wpr * 32);
                if (wir == 0 && lane < 4) {
                    float t = 0.f;
                    for (int k = 0; k < wpr; k++) t += p[lane * wpr + k];
                    const int row = row_j0 + lane * row_step;
                    if (t0 + lane < my_tiles && row < a.N) store_y(row, t);
                }
            }
        }
    }
    if (a.push.n > 0) {
        // all of this CTA's remote stores are issued: meet, then one thread fences them (the barrier
        // makes the fence cumulative over the other threads' stores) and counts the CTA in
        named_bar_sync(15, n_consumers);
        if (threadIdx.x == 0 && !*(const volatile int *)&cta_dead) push_publish(a.push, gridDim.x);
    }
}

}  // namespace qz
