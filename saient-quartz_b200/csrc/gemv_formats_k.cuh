// Streaming-GEMV policies of Q5_K (raw layout: 176-byte blocks are 16-byte multiples),
// Q2_K and IQ4_NL (plane layout).
#pragma once

#include "gemv_formats32.cuh"

namespace qz {

// ---- Q5_K: [d f16][dmin f16][scales 12][qh 32][qs 128]; Q4_K plus bit `sub` of qh[l] as the
//      fifth bit of weight 32*sub + l (src/dequant.rs:1146-1181).  Unit = sub-block pair p. ----
struct StreamQ5K : NoTable {
    static constexpr uint32_t TYPE = T_Q5_K;
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1, sum0, sum1; };
    struct Off { int hdr, qs; int hi_pair, shift; uint32_t sel; };
    struct WRegs { uint4 hdr, h0, h1, q0, q1; };
    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1];
        r.sum0 = q.xsum[4 * u] + q.xsum[4 * u + 1];
        r.sum1 = q.xsum[4 * u + 2] + q.xsum[4 * u + 3];
    }
    __device__ static Off make_off(int nb, int u)
    {
        Off o;
        const int p = u & 3;
        o.hdr = (u >> 2) * 176;
        o.qs = o.hdr + 48 + 32 * p;
        o.hi_pair = p >> 1;
        o.shift = 2 * p;
        const int b = 2 * (p & 1);
        o.sel = (uint32_t)(b | (4 << 4) | ((b + 1) << 8) | (4 << 12));
        return o;
    }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.hdr = LD::v4(row + o.hdr);
        w.h0 = LD::v4(row + o.hdr + 16);
        w.h1 = LD::v4(row + o.hdr + 32);
        w.q0 = LD::v4(row + o.qs);
        w.q1 = LD::v4(row + o.qs + 16);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &o, const uint8_t *)
    {
        const uint32_t q[8] = {w.q0.x, w.q0.y, w.q0.z, w.q0.w, w.q1.x, w.q1.y, w.q1.z, w.q1.w};
        const uint32_t hb[8] = {w.h0.x, w.h0.y, w.h0.z, w.h0.w, w.h1.x, w.h1.y, w.h1.z, w.h1.w};
        int a0h = 0, a0l = 0, a1h = 0, a1l = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t t = hb[i] >> o.shift;   // bit 0 of each byte: sub-block 2p, bit 1: sub-block 2p+1
            const uint32_t lo = (q[i] & 0x0F0F0F0Fu) | ((t << 4) & 0x10101010u);
            const uint32_t hi = ((q[i] >> 4) & 0x0F0F0F0Fu) | ((t << 3) & 0x10101010u);
            a0h = dp4a_us(lo, x.xh[i], a0h);
            a0l = dp4a_us(lo, x.xl[i], a0l);
            a1h = dp4a_us(hi, x.xh[8 + i], a1h);
            a1l = dp4a_us(hi, x.xl[8 + i], a1l);
        }
        const uint32_t s0 = w.hdr.y, s1 = w.hdr.z, s2 = w.hdr.w;
        const uint32_t scw = o.hi_pair ? ((s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u)) : (s0 & 0x3F3F3F3Fu);
        const uint32_t mw = o.hi_pair ? (((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u)) : (s1 & 0x3F3F3F3Fu);
        const uint32_t sc2 = __byte_perm(scw, 0, o.sel), m2 = __byte_perm(mw, 0, o.sel);
        const float sc0 = (float)(sc2 & 0xFFFF), sc1 = (float)(sc2 >> 16);
        const float m0 = (float)(m2 & 0xFFFF), m1 = (float)(m2 >> 16);
        const float2 dm = __half22float2(*(const __half2 *)&w.hdr.x);
        const float t0 = (float)(a0h * 256 + a0l) * x.s0;
        const float t1 = (float)(a1h * 256 + a1l) * x.s1;
        return dm.x * (sc0 * t0 + sc1 * t1) - dm.y * (m0 * x.sum0 + m1 * x.sum1);
    }
};

// ---- Q2_K: planes scales[nb x 16] | qs[nb x 64] | (d,dmin)[nb x 4]; weight 128n + 32j + l takes
//      qs[32n + l] >> 2j and scale byte 8n + 2j + l/16 (low nibble scale, high nibble min),
//      src/dequant.rs:1113-1144.  Unit = (n, j in {2jp, 2jp+1}): 64 consecutive weights. ----
struct StreamQ2K : NoTable {
    static constexpr uint32_t TYPE = T_Q2_K;
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1, sum[4]; };
    struct Off { int sc, qs, dd, shift; };
    struct WRegs { uint4 q0, q1; uint32_t sc, dd; };
    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1];
#pragma unroll
        for (int g = 0; g < 4; g++) r.sum[g] = q.xsum[4 * u + g];
    }
    __device__ static Off make_off(int nb, int u)
    {
        const int b = u >> 2, n = (u >> 1) & 1, jp = u & 1;
        return Off{b * 16 + 8 * n + 4 * jp, nb * 16 + b * 64 + 32 * n, nb * 80 + b * 4, 4 * jp};
    }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q0 = LD::v4(row + o.qs);
        w.q1 = LD::v4(row + o.qs + 16);
        w.sc = LD::u32(row + o.sc);
        w.dd = LD::u32(row + o.dd);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &o, const uint8_t *)
    {
        const uint32_t q[8] = {w.q0.x, w.q0.y, w.q0.z, w.q0.w, w.q1.x, w.q1.y, w.q1.z, w.q1.w};
        // group g = 2*(j - 2jp) + (l / 16): 16 weights, limb words 4g .. 4g+3
        int H[4] = {0, 0, 0, 0}, L[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const uint32_t t = q[i] >> o.shift;
            const uint32_t c0 = t & 0x03030303u, c1 = (t >> 2) & 0x03030303u;   // j = 2jp, 2jp + 1
            const int g0 = i >> 2, g1 = 2 + (i >> 2);
            H[g0] = dp4a_us(c0, x.xh[4 * g0 + (i & 3)], H[g0]);
            L[g0] = dp4a_us(c0, x.xl[4 * g0 + (i & 3)], L[g0]);
            H[g1] = dp4a_us(c1, x.xh[4 * g1 + (i & 3)], H[g1]);
            L[g1] = dp4a_us(c1, x.xl[4 * g1 + (i & 3)], L[g1]);
        }
        float pos = 0.f, neg = 0.f;
#pragma unroll
        for (int g = 0; g < 4; g++) {
            const uint32_t scb = (w.sc >> (8 * g)) & 0xFF;
            pos = fmaf((float)(256 * H[g] + L[g]) * (g < 2 ? x.s0 : x.s1), (float)(scb & 0xF), pos);
            neg = fmaf((float)(scb >> 4), x.sum[g], neg);
        }
        const float2 dd = __half22float2(*(const __half2 *)&w.dd);
        return dd.x * pos - dd.y * neg;
    }
};

// ---- IQ4_NL: planes d[nb x 2] | qs[nb x 16]; w = d * table[nibble] (src/dequant.rs:1527-1574).
//      The 16-entry int8 table lives in four registers; four nibbles are looked up at once with
//      two PRMTs (entries 0-7 and 8-15) and a bytewise select on bit 3. ----
__device__ __forceinline__ uint32_t iq4nl_lookup4(uint32_t idx)   // idx: four 4-bit indices, one per byte
{
    const uint32_t x3 = idx & 0x07070707u;
    const uint32_t y = x3 | (x3 >> 4);                       // byte0 = i0 | i1<<4, byte2 = i2 | i3<<4
    const uint32_t sel = __byte_perm(y, 0, 0x4420);          // selector nibbles i0 i1 i2 i3
    const uint32_t lo = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, sel);   // -127 -104 -83 -65 | -49 -35 -22 -10
    const uint32_t hi = __byte_perm(0x26190D01u, 0x71594535u, sel);   //    1   13  25  38 |  53  69  89 113
    const uint32_t t = (idx << 4) & 0x80808080u;
    uint32_t m;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(m) : "r"(t), "r"(0u), "r"(0xBA98u));
    return (lo & ~m) | (hi & m);
}

struct StreamIQ4NL : NoTable {
    static constexpr uint32_t TYPE = T_IQ4_NL;
    struct XRegs { uint32_t xl[16], xh[16]; float s0, s1; };
    struct Off { int qs, d; };
    struct WRegs { uint4 q0, q1; uint32_t d2; };
    __device__ static void load_x(XRegs &r, const XQ &q, int u)
    {
        load_x64(r.xl, r.xh, q, 64 * u);
        r.s0 = q.xs[2 * u];
        r.s1 = q.xs[2 * u + 1];
    }
    __device__ static Off make_off(int nb, int u) { return Off{nb * 2 + u * 32, u * 4}; }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q0 = LD::v4(row + o.qs);
        w.q1 = LD::v4(row + o.qs + 16);
        w.d2 = LD::u32(row + o.d);
    }
    __device__ static int block_dot(const uint4 &qv, const uint32_t *xl, const uint32_t *xh)
    {
        const uint32_t q[4] = {qv.x, qv.y, qv.z, qv.w};
        int h = 0, l = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint32_t a = iq4nl_lookup4(q[i] & 0x0F0F0F0Fu), b = iq4nl_lookup4((q[i] >> 4) & 0x0F0F0F0Fu);
            h = dp4a_ss(a, xh[i], h);
            l = dp4a_ss(a, xl[i], l);
            h = dp4a_ss(b, xh[4 + i], h);
            l = dp4a_ss(b, xl[4 + i], l);
        }
        return 256 * h + l;
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *)
    {
        const int d0 = block_dot(w.q0, x.xl, x.xh), d1 = block_dot(w.q1, x.xl + 8, x.xh + 8);
        const float2 d = __half22float2(*(const __half2 *)&w.d2);
        return d.x * ((float)d0 * x.s0) + d.y * ((float)d1 * x.s1);
    }
};

}  // namespace qz
