// Streaming dequant-GEMV kernels (batch 1): the HBM-bound hot path.
//
// Design, in the order the data flows:
//
//  * Activations are converted ONCE per GEMV into a 16-bit block-fixed-point form
//    (quantize_x_kernel): per run of 32 values a scale s = max|x| / 32512 and two
//    int8 limbs per value, X = 256*h + l, x ~= s*X (relative step 3e-5 of the run
//    maximum).  Every integer format here is "int code x block scale", so a row
//    dot-product becomes exact int32 dp4a sums (two per four weights) finished in
//    f32 with the block scales; "min" terms use the exact f32 sums of x.  This is
//    what keeps the kernel on the memory roofline: a Q4_K weight has 0.56 bytes,
//    so at 6.5 TB/s an SM must retire ~44 weights per clock, which leaves under
//    three issue slots per weight -- nibble->float conversion plus an FMA per
//    weight does not fit, four weights per dp4a does.
//  * A thread owns one 64-weight slice of the K dimension for the whole kernel:
//    its activation limbs live in 32 registers and are reused for every row, so
//    shared memory and L1 carry no per-row activation traffic at all.
//  * Weights stream with 128-bit ld.global.nc.L1::no_allocate loads, R rows (so
//    3R..4R independent 16-byte loads) in flight per thread, from the raw GGUF
//    layout where blocks are 16-byte multiples (Q4_K, Q5_K) and from the plane
//    layout (see formats.cuh) otherwise.
//  * Threads of one row are lanes of the same warp(s); the row sum is a shuffle
//    butterfly plus, for K > 2048, one shared-memory hop across the row's warps.
//  * Persistent grid-stride CTAs over row tiles; blockIdx.y selects one of up to
//    four (weights, activation, output) triples, which is how fused q/k/v and
//    multi-expert launches are expressed.
#pragma once

#include "formats.cuh"
#include "mgpu.cuh"

namespace qz {

// Block-fixed-point activations.  xl/xh: low/high int8 limbs [K]; xs: f32 scale per
// 32-run [K/32]; xsum: exact f32 sum of x per 16-run [K/16].
struct XQ {
    const int8_t *xl;
    const int8_t *xh;
    const float *xs;
    const float *xsum;
};

constexpr float XQ_RANGE = 32512.0f;   // 127 * 256: h, l both fit int8
// Runs whose largest magnitude is below this (2^-110) are taken as zero: XQ_RANGE / amax would overflow and the
// scale amax / XQ_RANGE would be subnormal; products of such activations underflow in f32 anyway.
constexpr float XQ_TINY = 7.703719777548943e-34f;

// Scale handling shared by every conversion site.  amax: largest magnitude of the 32-run; sum32: the run's f32
// sum, used only to notice a NaN or an infinity anywhere in the run (fmaxf drops NaNs): such a run gets a NaN
// scale, so every output that touches it becomes NaN, as it would in f32 arithmetic.
__device__ __forceinline__ void xq_run_scale(float amax, float sum32, float &inv, float &scale)
{
    if (!(fabsf(sum32) <= 3.0e38f) || !(amax <= 3.0e38f)) {   // NaN or infinite
        inv = 0.f;
        scale = __int_as_float(0x7FC00000);
    } else if (amax > XQ_TINY) {
        inv = XQ_RANGE / amax;
        scale = amax / XQ_RANGE;
    } else {
        inv = 0.f;
        scale = 0.f;
    }
}

// one thread per 4 values; 8 threads share a 32-run
// With `ctrl` set, x is (part of) a row-sharded vector whose slices other ranks push into this
// rank's window: every CTA first waits for the exchange to complete.  The dependent GEMV has been
// released by then and streams its weights meanwhile.
__global__ void quantize_x_kernel(const float *x, int8_t *__restrict__ xl, int8_t *__restrict__ xh,
                                  float *__restrict__ xs, float *__restrict__ xsum, int K, const MgpuCtrl *ctrl,
                                  int n_ranks, int *status)
{
    pdl_wait();
    pdl_trigger();
    if (ctrl) {
        mgpu_poll(ctrl, n_ranks, status);
        __syncthreads();
    }
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    int k = 4 * t;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (k < K) {
#pragma unroll
        // L2-coherent loads: with `ctrl` set, x is window memory that peers wrote while this kernel was
        // already running, so the read-only (non-coherent) path must not serve it
        for (int i = 0; i < 4; i++) v[i] = __ldcg(x + k + i);
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    float sum = (v[0] + v[1]) + (v[2] + v[3]);
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    const float sum32 = sum + __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
    if (k >= K) return;
    float inv, scale;
    xq_run_scale(amax, sum32, inv, scale);
    uint32_t wl = 0, wh = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int X = __float2int_rn(v[i] * inv);
        int l = ((X + 128) & 0xFF) - 128;
        int h = (X - l) >> 8;
        wl |= (uint32_t)(l & 0xFF) << (8 * i);
        wh |= (uint32_t)(h & 0xFF) << (8 * i);
    }
    ((uint32_t *)xl)[t] = wl;
    ((uint32_t *)xh)[t] = wh;
    if ((t & 7) == 0) xs[t >> 3] = scale;
    if ((t & 3) == 0) xsum[t >> 2] = sum;
}

struct XQOut {
    int8_t *xl, *xh;
    float *xs, *xsum;
};

// Convert four consecutive values (elements 4t .. 4t+3, t = global thread-of-4 index) exactly
// as quantize_x_kernel does.  All 32 lanes of the warp must call it (shuffles inside); lanes
// past the end pass valid = false.
__device__ __forceinline__ void quantize4_store(const float v[4], int t, bool valid, const XQOut &o)
{
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    float sum = (v[0] + v[1]) + (v[2] + v[3]);
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 4));
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    const float sum32 = sum + __shfl_xor_sync(0xFFFFFFFFu, sum, 4);
    if (!valid) return;
    float inv, scale;
    xq_run_scale(amax, sum32, inv, scale);
    uint32_t wl = 0, wh = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int X = __float2int_rn(v[i] * inv);
        int l = ((X + 128) & 0xFF) - 128;
        int h = (X - l) >> 8;
        wl |= (uint32_t)(l & 0xFF) << (8 * i);
        wh |= (uint32_t)(h & 0xFF) << (8 * i);
    }
    ((uint32_t *)o.xl)[t] = wl;
    ((uint32_t *)o.xh)[t] = wh;
    if ((t & 7) == 0) o.xs[t >> 3] = scale;
    if ((t & 3) == 0) o.xsum[t >> 2] = sum;
}

// Several vectors in one launch (grid.y = vector): what quantize_x_kernel does for one.
constexpr int QZ_QUANT_MULTI = 8;
struct QuantMulti {
    const float *x[QZ_QUANT_MULTI];
    XQOut o[QZ_QUANT_MULTI];
    int K[QZ_QUANT_MULTI];
};
__global__ void quantize_x_multi_kernel(const QuantMulti q)
{
    pdl_wait();
    pdl_trigger();
    const int i = blockIdx.y, K = q.K[i];
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (4 * (int)(blockIdx.x * blockDim.x) >= K) return;   // whole block past the end of this vector
    const bool valid = 4 * t < K;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (valid) {
        const float4 f = __ldcg((const float4 *)(q.x[i] + 4 * t));
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    }
    quantize4_store(v, t, valid, q.o[i]);
}

// d = sum over 4 bytes a_i (unsigned) * b_i (signed) + c
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

struct LdGlobal {
    __device__ static uint4 v4(const uint8_t *p) { return ld_stream(p); }
    __device__ static uint2 v2(const uint8_t *p)
    {
        uint2 v;
        asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
        return v;
    }
    __device__ static uint32_t u32(const uint8_t *p) { return ld_stream_u32(p); }
    __device__ static uint32_t u16(const uint8_t *p) { return ld_stream_u16(p); }
};

constexpr int QZ_MAX_MATS = 8;   // (weights, activation, output) triples one launch can serve

struct GemvArgs {
    const uint8_t *W[QZ_MAX_MATS];
    XQ xq[QZ_MAX_MATS];
    float *y[QZ_MAX_MATS];
    int K, N;
    int accumulate;   // 1: y += W x (residual epilogue), 0: y = W x
    int U;       // 64-weight units per row
    int Upad;    // threads per row: U rounded up to a power of two (<32) or a multiple of 32
    int RP;      // rows per pass = blockDim.x / Upad
};

// ---- per-format policies ------------------------------------------------------
// Each policy owns: the thread's activation slice (XRegs), the thread's byte offsets
// inside a row (Off: they depend on the unit only, never on the row), one row's bytes
// for the slice (WRegs), the loads, and the integer dot product.

// policies without a codebook
struct NoTable {
    static constexpr int TABLE_BYTES = 0;
    __device__ static void load_table(uint8_t *, int, int) {}
};

__device__ __forceinline__ void load_x64(uint32_t *xl, uint32_t *xh, const XQ &q, int at)
{
    const uint4 *pl = (const uint4 *)(q.xl + at), *ph = (const uint4 *)(q.xh + at);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint4 a = pl[i], b = ph[i];
        xl[4 * i] = a.x; xl[4 * i + 1] = a.y; xl[4 * i + 2] = a.z; xl[4 * i + 3] = a.w;
        xh[4 * i] = b.x; xh[4 * i + 1] = b.y; xh[4 * i + 2] = b.z; xh[4 * i + 3] = b.w;
    }
}

// byte b of v, sign-extended to 32 bits, by one PRMT (selector nibble b|8 replicates the sign)
__device__ __forceinline__ uint32_t sext_selector(int b) { return (uint32_t)(b | ((b | 8) << 4) | ((b | 8) << 8) | ((b | 8) << 12)); }
__device__ __forceinline__ int sext_byte(uint32_t v, uint32_t selector)
{
    int d;   // the __byte_perm intrinsic ignores the sign-replication bit of the selector; raw PRMT honours it
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(v), "r"(0u), "r"(selector));
    return d;
}

struct StreamQ4K : NoTable {
    static constexpr uint32_t TYPE = T_Q4_K;
    static constexpr bool PLANES = false;
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1, sum0, sum1; };
    struct Off { int hdr, qs; int hi_pair; uint32_t sel_sc, sel_m; };
    struct WRegs { uint4 hdr, q0, q1; };

    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1] * 0.0625f;   // high nibbles are used unshifted (x16)
        r.sum0 = q.xsum[4 * u] + q.xsum[4 * u + 1];
        r.sum1 = q.xsum[4 * u + 2] + q.xsum[4 * u + 3];
    }
    __device__ static Off make_off(int nb, int u)
    {
        Off o;
        const int p = u & 3;
        o.hdr = (u >> 2) * 144;
        o.qs = o.hdr + 16 + 32 * p;
        o.hi_pair = p >> 1;   // sub-blocks 4..7 take their 6-bit codes from the packed upper part
        // bytes (2p & 3) and (2p & 3) + 1 of the 4-byte code word, zero-extended into bytes 0 and 2
        const int b = 2 * (p & 1);
        o.sel_sc = (uint32_t)(b | (4 << 4) | ((b + 1) << 8) | (4 << 12));
        o.sel_m = o.sel_sc;
        return o;
    }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.hdr = LD::v4(row + o.hdr);
        w.q0 = LD::v4(row + o.qs);
        w.q1 = LD::v4(row + o.qs + 16);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &o, const uint8_t *)
    {
        const uint32_t q[8] = {w.q0.x, w.q0.y, w.q0.z, w.q0.w, w.q1.x, w.q1.y, w.q1.z, w.q1.w};
        int a0h = 0, a0l = 0, a1h = 0, a1l = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t lo = q[i] & 0x0F0F0F0Fu, hi = q[i] & 0xF0F0F0F0u;
            a0h = dp4a_us(lo, x.xh[i], a0h);
            a0l = dp4a_us(lo, x.xl[i], a0l);
            a1h = dp4a_us(hi, x.xh[8 + i], a1h);
            a1l = dp4a_us(hi, x.xl[8 + i], a1l);
        }
        // 6-bit scale / min codes of sub-blocks 2p and 2p+1 (src/dequant.rs:1471-1480)
        const uint32_t s0 = w.hdr.y, s1 = w.hdr.z, s2 = w.hdr.w;
        const uint32_t scw = o.hi_pair ? ((s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u)) : (s0 & 0x3F3F3F3Fu);
        const uint32_t mw = o.hi_pair ? (((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u)) : (s1 & 0x3F3F3F3Fu);
        const uint32_t sc2 = __byte_perm(scw, 0, o.sel_sc), m2 = __byte_perm(mw, 0, o.sel_m);   // two codes in 16-bit lanes
        const float sc0 = (float)(sc2 & 0xFFFF), sc1 = (float)(sc2 >> 16);
        const float m0 = (float)(m2 & 0xFFFF), m1 = (float)(m2 >> 16);
        const float2 dm = __half22float2(*(const __half2 *)&w.hdr.x);
        const float t0 = (float)(a0h * 256 + a0l) * x.s0;
        const float t1 = (float)(a1h * 256 + a1l) * x.s1;
        return dm.x * (sc0 * t0 + sc1 * t1) - dm.y * (m0 * x.sum0 + m1 * x.sum1);
    }
};

struct StreamQ6K : NoTable {
    static constexpr uint32_t TYPE = T_Q6_K;
    static constexpr bool PLANES = true;
    // unit u -> block u/4, half n = (u>>1)&1, 16-lane group g = u&1; run k holds the
    // weights 128n + 32k + 16g + [0,16) of the block
    struct XRegs { uint32_t xl[16], xh[16]; float s[4]; int nsx[4]; };
    struct Off { int ql, qh, sc, d; uint32_t sel0, sel1; };
    struct WRegs { uint4 ql0, ql1, qh; uint2 sc; uint32_t d; };

    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        const int base = 256 * (u >> 2) + 128 * ((u >> 1) & 1) + 16 * (u & 1);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            uint4 a = *(const uint4 *)(q.xl + base + 32 * k), b = *(const uint4 *)(q.xh + base + 32 * k);
            r.xl[4 * k] = a.x; r.xl[4 * k + 1] = a.y; r.xl[4 * k + 2] = a.z; r.xl[4 * k + 3] = a.w;
            r.xh[4 * k] = b.x; r.xh[4 * k + 1] = b.y; r.xh[4 * k + 2] = b.z; r.xh[4 * k + 3] = b.w;
            r.s[k] = q.xs[(base >> 5) + k];
            int sl = 0, shh = 0;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                sl = dp4a_ss(0x01010101u, r.xl[4 * k + i], sl);
                shh = dp4a_ss(0x01010101u, r.xh[4 * k + i], shh);
            }
            r.nsx[k] = -32 * (256 * shh + sl);   // the -32 offset of every 6-bit code, pre-summed
        }
    }
    __device__ static Off make_off(int nb, int u)
    {
        const int b = u >> 2, n = (u >> 1) & 1, g = u & 1;
        Off o;
        o.ql = b * 128 + 64 * n + 16 * g;
        o.qh = nb * 128 + b * 64 + 32 * n + 16 * g;
        o.sc = nb * 192 + b * 16 + 8 * n;
        o.d = nb * 208 + b * 2;
        o.sel0 = sext_selector(g);       // scale bytes g and g+2 of each 4-byte word
        o.sel1 = sext_selector(g + 2);
        return o;
    }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.ql0 = LD::v4(row + o.ql);
        w.ql1 = LD::v4(row + o.ql + 32);
        w.qh = LD::v4(row + o.qh);
        w.sc = LD::v2(row + o.sc);
        w.d = LD::u16(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &o, const uint8_t *)
    {
        const uint32_t a0[4] = {w.ql0.x, w.ql0.y, w.ql0.z, w.ql0.w};
        const uint32_t a1[4] = {w.ql1.x, w.ql1.y, w.ql1.z, w.ql1.w};
        const uint32_t hh[4] = {w.qh.x, w.qh.y, w.qh.z, w.qh.w};
        int dh[4] = {0, 0, 0, 0};
        int dl[4] = {x.nsx[0], x.nsx[1], x.nsx[2], x.nsx[3]};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t h = hh[i];
            uint32_t q0 = (a0[i] & 0x0F0F0F0Fu) | ((h << 4) & 0x30303030u);
            uint32_t q1 = (a1[i] & 0x0F0F0F0Fu) | ((h << 2) & 0x30303030u);
            uint32_t q2 = ((a0[i] >> 4) & 0x0F0F0F0Fu) | (h & 0x30303030u);
            uint32_t q3 = ((a1[i] >> 4) & 0x0F0F0F0Fu) | ((h >> 2) & 0x30303030u);
            dh[0] = dp4a_us(q0, x.xh[i], dh[0]);       dl[0] = dp4a_us(q0, x.xl[i], dl[0]);
            dh[1] = dp4a_us(q1, x.xh[4 + i], dh[1]);   dl[1] = dp4a_us(q1, x.xl[4 + i], dl[1]);
            dh[2] = dp4a_us(q2, x.xh[8 + i], dh[2]);   dl[2] = dp4a_us(q2, x.xl[8 + i], dl[2]);
            dh[3] = dp4a_us(q3, x.xh[12 + i], dh[3]);  dl[3] = dp4a_us(q3, x.xl[12 + i], dl[3]);
        }
        // scale bytes g, g+2, g+4, g+6 of the half's eight int8 scales
        const int sc[4] = {sext_byte(w.sc.x, o.sel0), sext_byte(w.sc.x, o.sel1), sext_byte(w.sc.y, o.sel0),
                           sext_byte(w.sc.y, o.sel1)};
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 4; k++) acc = fmaf((float)(sc[k] * (256 * dh[k] + dl[k])), x.s[k], acc);
        return acc * h2f((uint16_t)w.d);
    }
};

struct StreamQ8_0 : NoTable {
    static constexpr uint32_t TYPE = T_Q8_0;
    static constexpr bool PLANES = true;
    // unit u -> blocks 2u and 2u+1
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1; };
    struct Off { int qs, d; };
    struct WRegs { uint4 q[4]; uint32_t d2; };

    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1];
    }
    __device__ static Off make_off(int nb, int u) { return Off{nb * 2 + u * 64, u * 4}; }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
#pragma unroll
        for (int i = 0; i < 4; i++) w.q[i] = LD::v4(row + o.qs + 16 * i);
        w.d2 = LD::u32(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *)
    {
        int h0 = 0, l0 = 0, h1 = 0, l1 = 0;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const uint32_t a[4] = {w.q[i].x, w.q[i].y, w.q[i].z, w.q[i].w};
            const uint32_t b[4] = {w.q[2 + i].x, w.q[2 + i].y, w.q[2 + i].z, w.q[2 + i].w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                h0 = dp4a_ss(a[j], x.xh[4 * i + j], h0);      l0 = dp4a_ss(a[j], x.xl[4 * i + j], l0);
                h1 = dp4a_ss(b[j], x.xh[8 + 4 * i + j], h1);  l1 = dp4a_ss(b[j], x.xl[8 + 4 * i + j], l1);
            }
        }
        float2 d = __half22float2(*(const __half2 *)&w.d2);
        return d.x * ((float)(256 * h0 + l0) * x.s0) + d.y * ((float)(256 * h1 + l1) * x.s1);
    }
};

// Sum four per-lane values over the warp with 6 shuffles: afterwards every lane holds
// the warp total of value number (lane >> 3) (all 8 lanes of an octet hold the same).
__device__ __forceinline__ float warp_sum4(float a0, float a1, float a2, float a3, int lane)
{
    const bool up16 = lane & 16, up8 = lane & 8;
    float k0 = up16 ? a2 : a0, k1 = up16 ? a3 : a1;
    k0 += __shfl_xor_sync(0xFFFFFFFFu, up16 ? a0 : a2, 16);
    k1 += __shfl_xor_sync(0xFFFFFFFFu, up16 ? a1 : a3, 16);
    float k = up8 ? k1 : k0;
    k += __shfl_xor_sync(0xFFFFFFFFu, up8 ? k0 : k1, 8);
    k += __shfl_xor_sync(0xFFFFFFFFu, k, 4);
    k += __shfl_xor_sync(0xFFFFFFFFu, k, 2);
    k += __shfl_xor_sync(0xFFFFFFFFu, k, 1);
    return k;
}

// ---- the kernel ---------------------------------------------------------------
template <class F, int R>
__global__ void __launch_bounds__(512) gemv_stream_kernel(const GemvArgs a)
{
    __shared__ float part_w[2][4 * R * 16];   // [parity][(row-in-pass * R + i) * 16 + warp of the row]
    __shared__ __align__(16) uint8_t tbl[F::TABLE_BYTES > 0 ? F::TABLE_BYTES : 16];
    F::load_table(tbl, threadIdx.x, blockDim.x);   // codebooks are written by no kernel: before pdl_wait
    if (F::TABLE_BYTES > 0) __syncthreads();

    const int m = blockIdx.y;
    const uint8_t *__restrict__ W = a.W[m];
    float *__restrict__ y = a.y[m];
    const FormatInfo fi = format_info(F::TYPE);
    const int nb = a.K / fi.block_elems;
    const size_t row_bytes = (size_t)nb * fi.block_bytes;

    const int u = threadIdx.x % a.Upad;
    const int rl = threadIdx.x / a.Upad;
    const bool active = u < a.U;
    const int lane = threadIdx.x & 31;
    const int wpr = a.Upad >> 5;                 // warps per row (0 when Upad < 32)
    const int wir = (threadIdx.x >> 5) % (wpr > 0 ? wpr : 1);   // warp index inside the row

    pdl_wait();
    pdl_trigger();
    typename F::XRegs xr;
    if (active) F::load_x(xr, a.xq[m], u);
    const typename F::Off off = F::make_off(nb, u);

    const int rows_per_tile = a.RP * R;
    const int ntiles = (a.N + rows_per_tile - 1) / rows_per_tile;
    int parity = 0;
    for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, parity ^= 1) {
        const int row0 = tile * rows_per_tile + rl;
        typename F::WRegs w[R];
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int row = row0 + i * a.RP;
            if (active && row < a.N) F::template load_w<LdGlobal>(w[i], W + (size_t)row * row_bytes, off);
        }
        float acc[R];
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int row = row0 + i * a.RP;
            acc[i] = (active && row < a.N) ? F::dot(w[i], xr, off, tbl) : 0.f;
        }
        if (wpr == 0) {
            // several rows per warp: butterfly inside the row's Upad lanes
#pragma unroll
            for (int i = 0; i < R; i++) {
                float v = acc[i];
                for (int off = a.Upad >> 1; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
                const int row = row0 + i * a.RP;
                if (u == 0 && row < a.N) y[row] = a.accumulate ? y[row] + v : v;
            }
        } else {
#pragma unroll
            for (int i = 0; i < R; i++) acc[i] = warp_sum(acc[i]);
            if (wpr == 1) {
                if (lane == 0) {
#pragma unroll
                    for (int i = 0; i < R; i++) {
                        const int row = row0 + i * a.RP;
                        if (row < a.N) y[row] = a.accumulate ? y[row] + acc[i] : acc[i];
                    }
                }
            } else {
                if (lane == 0) {
#pragma unroll
                    for (int i = 0; i < R; i++) part_w[parity][(rl * R + i) * 16 + wir] = acc[i];
                }
                __syncthreads();
                if (threadIdx.x < rows_per_tile) {
                    const int rl2 = threadIdx.x / R, i2 = threadIdx.x % R;
                    float v = 0.f;
                    for (int k = 0; k < wpr; k++) v += part_w[parity][(rl2 * R + i2) * 16 + k];
                    const int row = tile * rows_per_tile + i2 * a.RP + rl2;
                    if (row < a.N) y[row] = a.accumulate ? y[row] + v : v;
                }
            }
        }
    }
}

}  // namespace qz
