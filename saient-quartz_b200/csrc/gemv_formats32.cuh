// Streaming-GEMV policies of the 32-weight block formats Q4_0, Q4_1, Q5_0, Q5_1
// (plane layout; a thread's 64-weight unit is two consecutive blocks).
//
// Common arithmetic: byte j of a block's 16 quant bytes holds weight j (low nibble) and
// weight j+16 (high nibble).  High nibbles are used unshifted (x16) in dp4a and the exact
// factor 16 is shifted out of the int32 sum afterwards.  Offsets (-8, -16) and additive
// minima go through precomputed sums of the activation slice.
#pragma once

#include "gemv_stream.cuh"

namespace qz {

// integer sum of the 32 block-fixed-point activations X = 256h + l held in 8+8 limb words
__device__ __forceinline__ int sum_x32(const uint32_t *xl, const uint32_t *xh)
{
    int sl = 0, sh = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        sl = dp4a_ss(0x01010101u, xl[i], sl);
        sh = dp4a_ss(0x01010101u, xh[i], sh);
    }
    return 256 * sh + sl;
}

// sum over one block of nibble(j) * X(j) + nibble(j+16) * X(j+16): q = 4 words of quant bytes,
// xl/xh = the block's 8 limb words each (words 0-3: weights 0-15, words 4-7: weights 16-31)
__device__ __forceinline__ int dot_nibbles32(const uint4 &qv, const uint32_t *xl, const uint32_t *xh)
{
    const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
    int lo_h = 0, lo_l = 0, hi_h = 0, hi_l = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t lo = q[i] & 0x0F0F0F0Fu, hi = q[i] & 0xF0F0F0F0u;
        lo_h = dp4a_us(lo, xh[i], lo_h);
        lo_l = dp4a_us(lo, xl[i], lo_l);
        hi_h = dp4a_us(hi, xh[4 + i], hi_h);
        hi_l = dp4a_us(hi, xl[4 + i], hi_l);
    }
    return 256 * (lo_h + (hi_h >> 4)) + lo_l + (hi_l >> 4);   // the x16 sums are exact multiples of 16
}

// fifth bits of four consecutive weights (bits b0..b3 of `bits`) moved to bit 4 of bytes 0..3.
// The multiplier places bit i at 4+8i; the 16 partial products land on distinct bit positions,
// so nothing carries into the masked bits.
__device__ __forceinline__ uint32_t spread4_to_bit4(uint32_t bits)
{
    return ((bits & 0xFu) * 0x02040810u) & 0x10101010u;
}

__device__ __forceinline__ int dot_q5_32(const uint4 &qv, uint32_t qh, const uint32_t *xl, const uint32_t *xh)
{
    const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
    int h = 0, l = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t lo = (q[i] & 0x0F0F0F0Fu) | spread4_to_bit4(qh >> (4 * i));
        const uint32_t hi = ((q[i] >> 4) & 0x0F0F0F0Fu) | spread4_to_bit4(qh >> (16 + 4 * i));
        h = dp4a_us(lo, xh[i], h);
        l = dp4a_us(lo, xl[i], l);
        h = dp4a_us(hi, xh[4 + i], h);
        l = dp4a_us(hi, xl[4 + i], l);
    }
    return 256 * h + l;
}

// ---- Q4_0: planes d[nb x 2] | qs[nb x 16]; w = d * (q - 8) ----
struct StreamQ4_0 : NoTable {
    static constexpr uint32_t TYPE = T_Q4_0;
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1; int off0, off1; };
    struct Off { int qs, d; };
    struct WRegs { uint4 q0, q1; uint32_t d2; };
    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1];
        r.off0 = -8 * sum_x32(r.xl, r.xh);
        r.off1 = -8 * sum_x32(r.xl + 8, r.xh + 8);
    }
    __device__ static Off make_off(int nb, int u) { return Off{nb * 2 + u * 32, u * 4}; }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q0 = LD::v4(row + o.qs);
        w.q1 = LD::v4(row + o.qs + 16);
        w.d2 = LD::u32(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *)
    {
        const int d0 = dot_nibbles32(w.q0, x.xl, x.xh) + x.off0;
        const int d1 = dot_nibbles32(w.q1, x.xl + 8, x.xh + 8) + x.off1;
        const float2 d = __half22float2(*(const __half2 *)&w.d2);
        return d.x * ((float)d0 * x.s0) + d.y * ((float)d1 * x.s1);
    }
};

// ---- Q4_1: planes (d,m)[nb x 4] | qs[nb x 16]; w = d * q + m ----
struct StreamQ4_1 : NoTable {
    static constexpr uint32_t TYPE = T_Q4_1;
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1, sum0, sum1; };
    struct Off { int qs, dm; };
    struct WRegs { uint4 q0, q1; uint2 dm; };
    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1];
        r.sum0 = q.xsum[4 * u] + q.xsum[4 * u + 1];
        r.sum1 = q.xsum[4 * u + 2] + q.xsum[4 * u + 3];
    }
    __device__ static Off make_off(int nb, int u) { return Off{nb * 4 + u * 32, u * 8}; }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q0 = LD::v4(row + o.qs);
        w.q1 = LD::v4(row + o.qs + 16);
        w.dm = LD::v2(row + o.dm);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *)
    {
        const int d0 = dot_nibbles32(w.q0, x.xl, x.xh);
        const int d1 = dot_nibbles32(w.q1, x.xl + 8, x.xh + 8);
        const float2 a = __half22float2(*(const __half2 *)&w.dm.x), b = __half22float2(*(const __half2 *)&w.dm.y);
        return a.x * ((float)d0 * x.s0) + a.y * x.sum0 + b.x * ((float)d1 * x.s1) + b.y * x.sum1;
    }
};

// ---- Q5_0: planes d[nb x 2] | qh[nb x 4] | qs[nb x 16]; w = (q5 - 16) * d ----
struct StreamQ5_0 : NoTable {
    static constexpr uint32_t TYPE = T_Q5_0;
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1; int off0, off1; };
    struct Off { int qs, qh, d; };
    struct WRegs { uint4 q0, q1; uint2 qh; uint32_t d2; };
    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1];
        r.off0 = -16 * sum_x32(r.xl, r.xh);
        r.off1 = -16 * sum_x32(r.xl + 8, r.xh + 8);
    }
    __device__ static Off make_off(int nb, int u) { return Off{nb * 6 + u * 32, nb * 2 + u * 8, u * 4}; }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q0 = LD::v4(row + o.qs);
        w.q1 = LD::v4(row + o.qs + 16);
        w.qh = LD::v2(row + o.qh);
        w.d2 = LD::u32(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *)
    {
        const int d0 = dot_q5_32(w.q0, w.qh.x, x.xl, x.xh) + x.off0;
        const int d1 = dot_q5_32(w.q1, w.qh.y, x.xl + 8, x.xh + 8) + x.off1;
        const float2 d = __half22float2(*(const __half2 *)&w.d2);
        return d.x * ((float)d0 * x.s0) + d.y * ((float)d1 * x.s1);
    }
};

// ---- Q5_1: planes (d,m)[nb x 4] | qh[nb x 4] | qs[nb x 16]; w = q5 * d + m ----
struct StreamQ5_1 : NoTable {
    static constexpr uint32_t TYPE = T_Q5_1;
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1, sum0, sum1; };
    struct Off { int qs, qh, dm; };
    struct WRegs { uint4 q0, q1; uint2 qh, dm; };
    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1];
        r.sum0 = q.xsum[4 * u] + q.xsum[4 * u + 1];
        r.sum1 = q.xsum[4 * u + 2] + q.xsum[4 * u + 3];
    }
    __device__ static Off make_off(int nb, int u) { return Off{nb * 8 + u * 32, nb * 4 + u * 8, u * 8}; }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q0 = LD::v4(row + o.qs);
        w.q1 = LD::v4(row + o.qs + 16);
        w.qh = LD::v2(row + o.qh);
        w.dm = LD::v2(row + o.dm);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *)
    {
        const int d0 = dot_q5_32(w.q0, w.qh.x, x.xl, x.xh);
        const int d1 = dot_q5_32(w.q1, w.qh.y, x.xl + 8, x.xh + 8);
        const float2 a = __half22float2(*(const __half2 *)&w.dm.x), b = __half22float2(*(const __half2 *)&w.dm.y);
        return a.x * ((float)d0 * x.s0) + a.y * x.sum0 + b.x * ((float)d1 * x.s1) + b.y * x.sum1;
    }
};

}  // namespace qz
