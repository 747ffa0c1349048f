// Streaming-GEMV policies of the grid-codebook formats IQ2_XXS, IQ2_XS, IQ2_S, IQ3_XXS, IQ3_S
// (plane layout; a thread's 64-weight unit is two consecutive 32-weight groups of a block).
//
// The codebook (1-8 KB) is copied from the __device__ table the host uploaded into shared
// memory once per CTA; a lookup returns 4 or 8 small positive int8 magnitudes, the per-weight
// signs are applied bytewise in registers, and the result is a dp4a operand.  Everything
// up to the block scale is integer arithmetic on the two activation limbs.
#pragma once

#include "gemv_formats32.cuh"

namespace qz {

// Negate byte k of g when bit k of bits4 is set.  The multiplier moves bit k to the MSB of
// byte k (the 16 partial products fall on distinct bit positions); PRMT in sign-replicate
// mode widens each MSB to a byte mask; (g ^ mask) + lsb is the bytewise two's complement.
// Magnitudes are never zero in these codebooks, so no carry leaves a byte.
__device__ __forceinline__ uint32_t apply_signs4(uint32_t g, uint32_t bits4)
{
    const uint32_t t = ((bits4 & 0xFu) * 0x10204080u) & 0x80808080u;
    uint32_t mask;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(mask) : "r"(t), "r"(0u), "r"(0xBA98u));
    return (g ^ mask) + (t >> 7);
}

// KSIGNS_IQ2XS (src/iq2_tables.rs:9): the 7-bit index plus an eighth bit that makes the
// number of minus signs even
__device__ __forceinline__ uint32_t ksign8(uint32_t s7) { return s7 | ((__popc(s7) & 1u) << 7); }

template <int WORDS>
__device__ __forceinline__ void copy_table(uint8_t *dst, const void *src, int tid, int nthreads)
{
    for (int i = tid; i < WORDS; i += nthreads) ((uint32_t *)dst)[i] = ((const uint32_t *)src)[i];
}

// eight signed weights (one u64 grid entry) against limb words xi, xi+1
__device__ __forceinline__ void dot8(const uint2 g, uint32_t sign8, const uint32_t *xl, const uint32_t *xh, int xi,
                                     int &H, int &L)
{
    const uint32_t a = apply_signs4(g.x, sign8), b = apply_signs4(g.y, sign8 >> 4);
    H = dp4a_ss(a, xh[xi], H);
    L = dp4a_ss(a, xl[xi], L);
    H = dp4a_ss(b, xh[xi + 1], H);
    L = dp4a_ss(b, xl[xi + 1], L);
}

struct IqXRegs { uint32_t xl[16], xh[16]; float s0, s1; };

__device__ __forceinline__ void iq_load_x(IqXRegs &r, const XQ &q, int u)
{
    load_x64(r.xl, r.xh, q, 64 * u);
    r.s0 = q.xs[2 * u];
    r.s1 = q.xs[2 * u + 1];
}

// ---- IQ2_XXS: planes d[nb x 2] | qs[nb x 64]; src/dequant.rs:1011-1041 ----
struct StreamIQ2XXS {
    static constexpr uint32_t TYPE = T_IQ2_XXS;
    static constexpr int TABLE_BYTES = 256 * 8;
    using XRegs = IqXRegs;
    struct Off { int qs, d; };
    struct WRegs { uint4 q; uint32_t d; };
    __device__ static void load_table(uint8_t *dst, int tid, int n) { copy_table<512>(dst, g_iq2xxs_grid, tid, n); }
    __device__ static void load_x(XRegs &r, const XQ &q, int u) { iq_load_x(r, q, u); }
    __device__ static Off make_off(int nb, int u) { return Off{nb * 2 + (u >> 2) * 64 + (u & 3) * 16, (u >> 2) * 2}; }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q = LD::v4(row + o.qs);
        w.d = LD::u16(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *tbl)
    {
        const uint2 *grid = (const uint2 *)tbl;
        const uint32_t aux[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
        float acc = 0.f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t a0 = aux[2 * h], a1 = aux[2 * h + 1];
            int H = 0, L = 0;
#pragma unroll
            for (int l = 0; l < 4; l++)
                dot8(grid[(a0 >> (8 * l)) & 0xFF], ksign8((a1 >> (7 * l)) & 127), x.xl, x.xh, 8 * h + 2 * l, H, L);
            acc = fmaf((float)(256 * H + L) * (h ? x.s1 : x.s0), 0.5f + (float)(a1 >> 28), acc);
        }
        return acc * (0.25f * h2f((uint16_t)w.d));
    }
};

// ---- IQ2_XS: planes d | qs[nb x 64] (u16: 9-bit index, 7-bit sign index) | scales[nb x 8];
//      src/dequant.rs:1043-1075 ----
struct StreamIQ2XS {
    static constexpr uint32_t TYPE = T_IQ2_XS;
    static constexpr int TABLE_BYTES = 512 * 8;
    using XRegs = IqXRegs;
    struct Off { int qs, sc, d; };
    struct WRegs { uint4 q; uint32_t sc, d; };
    __device__ static void load_table(uint8_t *dst, int tid, int n) { copy_table<1024>(dst, g_iq2xs_grid, tid, n); }
    __device__ static void load_x(XRegs &r, const XQ &q, int u) { iq_load_x(r, q, u); }
    __device__ static Off make_off(int nb, int u)
    {
        const int b = u >> 2, p = u & 3;
        return Off{nb * 2 + b * 64 + p * 16, nb * 66 + b * 8 + p * 2, b * 2};
    }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q = LD::v4(row + o.qs);
        w.sc = LD::u16(row + o.sc);
        w.d = LD::u16(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *tbl)
    {
        const uint2 *grid = (const uint2 *)tbl;
        const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
        float acc = 0.f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t scb = (w.sc >> (8 * h)) & 0xFF;
            int H0 = 0, L0 = 0, H1 = 0, L1 = 0;
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint32_t q = (qw[2 * h + (l >> 1)] >> (16 * (l & 1))) & 0xFFFF;
                if (l < 2) dot8(grid[q & 511], ksign8(q >> 9), x.xl, x.xh, 8 * h + 2 * l, H0, L0);
                else dot8(grid[q & 511], ksign8(q >> 9), x.xl, x.xh, 8 * h + 2 * l, H1, L1);
            }
            const float t = (float)(256 * H0 + L0) * (0.5f + (float)(scb & 0xF)) +
                            (float)(256 * H1 + L1) * (0.5f + (float)(scb >> 4));
            acc = fmaf(t, h ? x.s1 : x.s0, acc);
        }
        return acc * (0.25f * h2f((uint16_t)w.d));
    }
};

// ---- IQ2_S: planes d | qs[nb x 64] (32 index bytes, 32 sign bytes) | qh[nb x 8] | scales[nb x 8];
//      src/dequant.rs:1077-1110 ----
struct StreamIQ2S {
    static constexpr uint32_t TYPE = T_IQ2_S;
    static constexpr int TABLE_BYTES = 1024 * 8;
    using XRegs = IqXRegs;
    struct Off { int idx, qh, sc, d; };
    struct WRegs { uint2 idx, sg; uint32_t qh, sc, d; };
    __device__ static void load_table(uint8_t *dst, int tid, int n) { copy_table<2048>(dst, g_iq2s_grid, tid, n); }
    __device__ static void load_x(XRegs &r, const XQ &q, int u) { iq_load_x(r, q, u); }
    __device__ static Off make_off(int nb, int u)
    {
        const int b = u >> 2, p = u & 3;
        return Off{nb * 2 + b * 64 + p * 8, nb * 66 + b * 8 + p * 2, nb * 74 + b * 8 + p * 2, b * 2};
    }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.idx = LD::v2(row + o.idx);
        w.sg = LD::v2(row + o.idx + 32);
        w.qh = LD::u16(row + o.qh);
        w.sc = LD::u16(row + o.sc);
        w.d = LD::u16(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *tbl)
    {
        const uint2 *grid = (const uint2 *)tbl;
        float acc = 0.f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t iw = h ? w.idx.y : w.idx.x, sw = h ? w.sg.y : w.sg.x;
            const uint32_t qhb = (w.qh >> (8 * h)) & 0xFF, scb = (w.sc >> (8 * h)) & 0xFF;
            int H0 = 0, L0 = 0, H1 = 0, L1 = 0;
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint32_t idx = ((iw >> (8 * l)) & 0xFF) | ((qhb << (8 - 2 * l)) & 0x300);
                const uint32_t s8 = (sw >> (8 * l)) & 0xFF;
                if (l < 2) dot8(grid[idx], s8, x.xl, x.xh, 8 * h + 2 * l, H0, L0);
                else dot8(grid[idx], s8, x.xl, x.xh, 8 * h + 2 * l, H1, L1);
            }
            const float t = (float)(256 * H0 + L0) * (0.5f + (float)(scb & 0xF)) +
                            (float)(256 * H1 + L1) * (0.5f + (float)(scb >> 4));
            acc = fmaf(t, h ? x.s1 : x.s0, acc);
        }
        return acc * (0.25f * h2f((uint16_t)w.d));
    }
};

// ---- IQ3_XXS: planes d | qs[nb x 64] (index bytes, 4 weights each) | scales_and_signs[nb x 32];
//      db = d * (0.5 + s) * 0.5 (ggml block_iq3_xxs; absent from the reference) ----
struct StreamIQ3XXS {
    static constexpr uint32_t TYPE = T_IQ3_XXS;
    static constexpr int TABLE_BYTES = 256 * 4;
    using XRegs = IqXRegs;
    struct Off { int qs, sas, d; };
    struct WRegs { uint4 q; uint2 sas; uint32_t d; };
    __device__ static void load_table(uint8_t *dst, int tid, int n) { copy_table<256>(dst, g_iq3xxs_grid, tid, n); }
    __device__ static void load_x(XRegs &r, const XQ &q, int u) { iq_load_x(r, q, u); }
    __device__ static Off make_off(int nb, int u)
    {
        const int b = u >> 2, p = u & 3;
        return Off{nb * 2 + b * 64 + p * 16, nb * 66 + b * 32 + p * 8, b * 2};
    }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q = LD::v4(row + o.qs);
        w.sas = LD::v2(row + o.sas);
        w.d = LD::u16(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &, const uint8_t *tbl)
    {
        const uint32_t *grid = (const uint32_t *)tbl;
        const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
        float acc = 0.f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t a1 = h ? w.sas.y : w.sas.x;
            int H = 0, L = 0;
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint32_t two = (qw[2 * h + (l >> 1)] >> (16 * (l & 1))) & 0xFFFF;   // index bytes 2l, 2l+1
                const uint2 g = make_uint2(grid[two & 0xFF], grid[two >> 8]);
                dot8(g, ksign8((a1 >> (7 * l)) & 127), x.xl, x.xh, 8 * h + 2 * l, H, L);
            }
            acc = fmaf((float)(256 * H + L) * (h ? x.s1 : x.s0), 0.5f + (float)(a1 >> 28), acc);
        }
        return acc * (0.5f * h2f((uint16_t)w.d));
    }
};

// ---- IQ3_S: planes d | qs[nb x 64] | qh[nb x 8] | signs[nb x 32] | scales[nb x 4];
//      db = d * (1 + 2 s), src/dequant.rs:1184-1237 ----
struct StreamIQ3S {
    static constexpr uint32_t TYPE = T_IQ3_S;
    static constexpr int TABLE_BYTES = 512 * 4;
    using XRegs = IqXRegs;
    struct Off { int qs, qh, sg, sc, d, sc_shift; };
    struct WRegs { uint4 q; uint2 sg; uint32_t qh, sc, d; };
    __device__ static void load_table(uint8_t *dst, int tid, int n) { copy_table<512>(dst, g_iq3s_grid, tid, n); }
    __device__ static void load_x(XRegs &r, const XQ &q, int u) { iq_load_x(r, q, u); }
    __device__ static Off make_off(int nb, int u)
    {
        const int b = u >> 2, p = u & 3;
        return Off{nb * 2 + b * 64 + p * 16, nb * 66 + b * 8 + p * 2, nb * 74 + b * 32 + p * 8, nb * 106 + b * 4, b * 2,
                   8 * p};
    }
    template <class LD, class P>
    __device__ static void load_w(WRegs &w, P row, const Off &o)
    {
        w.q = LD::v4(row + o.qs);
        w.sg = LD::v2(row + o.sg);
        w.qh = LD::u16(row + o.qh);
        w.sc = LD::u32(row + o.sc);
        w.d = LD::u16(row + o.d);
    }
    __device__ static float dot(const WRegs &w, const XRegs &x, const Off &o, const uint8_t *tbl)
    {
        const uint32_t *grid = (const uint32_t *)tbl;
        const uint32_t qw[4] = {w.q.x, w.q.y, w.q.z, w.q.w};
        const uint32_t scb = (w.sc >> o.sc_shift) & 0xFF;   // one byte per pair of 32-weight groups
        float acc = 0.f;
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const uint32_t qhb = (w.qh >> (8 * h)) & 0xFF, sw = h ? w.sg.y : w.sg.x;
            int H = 0, L = 0;
#pragma unroll
            for (int l = 0; l < 4; l++) {
                const uint32_t two = (qw[2 * h + (l >> 1)] >> (16 * (l & 1))) & 0xFFFF;
                const uint32_t i0 = (two & 0xFF) | ((qhb << (8 - 2 * l)) & 256);
                const uint32_t i1 = (two >> 8) | ((qhb << (7 - 2 * l)) & 256);
                dot8(make_uint2(grid[i0], grid[i1]), (sw >> (8 * l)) & 0xFF, x.xl, x.xh, 8 * h + 2 * l, H, L);
            }
            const float s = (float)(h ? (scb >> 4) : (scb & 0xF));
            acc = fmaf((float)(256 * H + L) * (h ? x.s1 : x.s0), 1.0f + 2.0f * s, acc);
        }
        return acc * h2f((uint16_t)w.d);
    }
};

}  // namespace qz
