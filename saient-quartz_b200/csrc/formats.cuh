// GGUF block formats: geometry, the two device layouts, and bit-exact decoders.
//
// Raw layout   : what the reference uploads verbatim (src/gguf.rs:118-123):
//                rows of K/block_elems blocks, each block its fields back to back.
// Plane layout : the one-time, size-preserving repack.  Inside every row the
//                blocks' fields are regrouped into planes, plane i holding field
//                i of block 0, 1, ... nb-1.  Plane i starts at nb * off_i (off_i =
//                the field's offset inside a raw block), so a row keeps its size
//                and its start, and pointer arithmetic over rows and experts
//                (src/cuda.rs:250-257, 723-725) stays valid.  With nb % 8 == 0
//                every plane starts on a 16-byte boundary, which is what makes
//                128-bit streaming loads legal for the 210-, 34-, 22-... byte
//                block formats.
//
// The decoders reproduce src/dequant.rs operation for operation with explicit
// round-to-nearest intrinsics (never contracted into FMAs), so the f32 weights
// they emit are bit-identical to the reference's CPU dequant().
#pragma once

#include "common.cuh"

namespace qz {

struct FormatInfo {
    int block_elems;
    int block_bytes;
    int nfields;
    int off[5];
    int size[5];
};

__host__ __device__ inline FormatInfo format_info(uint32_t t)
{
    switch (t) {
    case T_Q4_0:    return {32, 18, 2, {0, 2}, {2, 16}};
    case T_Q4_1:    return {32, 20, 2, {0, 4}, {4, 16}};
    case T_Q5_0:    return {32, 22, 3, {0, 2, 6}, {2, 4, 16}};
    case T_Q5_1:    return {32, 24, 3, {0, 4, 8}, {4, 4, 16}};
    case T_Q8_0:    return {32, 34, 2, {0, 2}, {2, 32}};
    case T_IQ4_NL:  return {32, 18, 2, {0, 2}, {2, 16}};
    case T_Q2_K:    return {256, 84, 3, {0, 16, 80}, {16, 64, 4}};
    case T_Q4_K:    return {256, 144, 2, {0, 16}, {16, 128}};
    case T_Q5_K:    return {256, 176, 3, {0, 16, 48}, {16, 32, 128}};
    case T_Q6_K:    return {256, 210, 4, {0, 128, 192, 208}, {128, 64, 16, 2}};
    case T_IQ2_XXS: return {256, 66, 2, {0, 2}, {2, 64}};
    case T_IQ2_XS:  return {256, 74, 3, {0, 2, 66}, {2, 64, 8}};
    case T_IQ2_S:   return {256, 82, 4, {0, 2, 66, 74}, {2, 64, 8, 8}};
    case T_IQ3_S:   return {256, 110, 5, {0, 2, 66, 74, 106}, {2, 64, 8, 32, 4}};
    case T_IQ3_XXS: return {256, 98, 3, {0, 2, 66}, {2, 64, 32}};
    case T_F32:     return {1, 4, 1, {0}, {4}};
    case T_F16:     return {1, 2, 1, {0}, {2}};
    case T_BF16:    return {1, 2, 1, {0}, {2}};
    default:        return {0, 0, 0, {0}, {0}};
    }
}

// Pointers to the fields of one block, in either layout.
struct Fields {
    const uint8_t *f[5];
};

template <bool PLANES>
__device__ __forceinline__ Fields block_fields(const FormatInfo &fi, const uint8_t *row, int nb, int b)
{
    Fields r;
#pragma unroll
    for (int i = 0; i < 5; i++) {
        if (i < fi.nfields)
            r.f[i] = PLANES ? row + (size_t)nb * fi.off[i] + (size_t)b * fi.size[i]
                            : row + (size_t)b * fi.block_bytes + fi.off[i];
        else
            r.f[i] = nullptr;
    }
    return r;
}

// ---- codebooks, uploaded by the host (cuda_set_*_grid; src/cuda.rs:131-140) ----
__device__ uint64_t g_iq2xxs_grid[256];
__device__ uint64_t g_iq2xs_grid[512];
__device__ uint64_t g_iq2s_grid[1024];
__device__ uint32_t g_iq3s_grid[512];
__device__ uint32_t g_iq3xxs_grid[256];
__device__ uint8_t g_ksigns[128];

__device__ __constant__ float c_iq4nl[16] = {-127.f, -104.f, -83.f, -65.f, -49.f, -35.f, -22.f, -10.f,
                                             1.f,    13.f,   25.f,  38.f,  53.f,  69.f,  89.f,  113.f};

// src/dequant.rs:1471-1480
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *s, int &sc, int &m)
{
    if (j < 4) {
        sc = s[j] & 63;
        m = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// (db * g) * (+-1), src/dequant.rs:1029-1036
__device__ __forceinline__ float signed_grid(float db, int g, uint32_t signs, int bit)
{
    return __fmul_rn(__fmul_rn(db, (float)g), (signs >> bit) & 1u ? -1.0f : 1.0f);
}

// decode32<T>(fields, sub, w): the 32 consecutive weights [32*sub, 32*sub+32) of a
// block (sub is 0 for the 32-weight formats).
template <uint32_t T>
__device__ __forceinline__ void decode32(const Fields &F, int sub, float *w);

// ggml block_q4_0 (absent from the reference): w = d * (q - 8)
template <>
__device__ __forceinline__ void decode32<T_Q4_0>(const Fields &F, int, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    const uint8_t *qs = F.f[1];
#pragma unroll
    for (int j = 0; j < 16; j++) {
        w[j] = __fmul_rn(d, (float)((int)(qs[j] & 0x0F) - 8));
        w[j + 16] = __fmul_rn(d, (float)((int)(qs[j] >> 4) - 8));
    }
}

// ggml block_q4_1 (absent from the reference): w = d * q + m
template <>
__device__ __forceinline__ void decode32<T_Q4_1>(const Fields &F, int, float *w)
{
    float d = h2f(ld_u16(F.f[0])), m = h2f(ld_u16(F.f[0] + 2));
    const uint8_t *qs = F.f[1];
#pragma unroll
    for (int j = 0; j < 16; j++) {
        w[j] = __fadd_rn(__fmul_rn(d, (float)(qs[j] & 0x0F)), m);
        w[j + 16] = __fadd_rn(__fmul_rn(d, (float)(qs[j] >> 4)), m);
    }
}

// src/dequant.rs:1381-1409
template <>
__device__ __forceinline__ void decode32<T_Q5_0>(const Fields &F, int, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    uint32_t qh = ld_u32_bytes(F.f[1]);
    const uint8_t *qs = F.f[2];
#pragma unroll
    for (int j = 0; j < 16; j++) {
        uint32_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
        w[j] = __fmul_rn((float)((int)((qs[j] & 0x0Fu) | xh0) - 16), d);
        w[j + 16] = __fmul_rn((float)((int)((uint32_t)(qs[j] >> 4) | xh1) - 16), d);
    }
}

// src/dequant.rs:1419-1443
template <>
__device__ __forceinline__ void decode32<T_Q5_1>(const Fields &F, int, float *w)
{
    float d = h2f(ld_u16(F.f[0])), m = h2f(ld_u16(F.f[0] + 2));
    uint32_t qh = ld_u32_bytes(F.f[1]);
    const uint8_t *qs = F.f[2];
#pragma unroll
    for (int j = 0; j < 16; j++) {
        uint32_t xh0 = ((qh >> j) << 4) & 0x10, xh1 = (qh >> (j + 12)) & 0x10;
        w[j] = __fadd_rn(__fmul_rn((float)((qs[j] & 0x0Fu) | xh0), d), m);
        w[j + 16] = __fadd_rn(__fmul_rn((float)((uint32_t)(qs[j] >> 4) | xh1), d), m);
    }
}

// src/dequant.rs:1450-1463
template <>
__device__ __forceinline__ void decode32<T_Q8_0>(const Fields &F, int, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    const int8_t *qs = (const int8_t *)F.f[1];
#pragma unroll
    for (int i = 0; i < 32; i++) w[i] = __fmul_rn(d, (float)qs[i]);
}

// src/dequant.rs:1557-1574
template <>
__device__ __forceinline__ void decode32<T_IQ4_NL>(const Fields &F, int, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    const uint8_t *qs = F.f[1];
#pragma unroll
    for (int k = 0; k < 16; k++) {
        w[k] = __fmul_rn(d, c_iq4nl[qs[k] & 0x0F]);
        w[k + 16] = __fmul_rn(d, c_iq4nl[qs[k] >> 4]);
    }
}

// src/dequant.rs:1113-1144.  Weight i = 128n + 32j + l uses qs[32n + l] >> 2j and
// scale byte 8n + 2j + l/16.
template <>
__device__ __forceinline__ void decode32<T_Q2_K>(const Fields &F, int sub, float *w)
{
    const uint8_t *scales = F.f[0], *qs = F.f[1];
    float d = h2f(ld_u16(F.f[2])), dmin = h2f(ld_u16(F.f[2] + 2));
    int n = sub >> 2, j = sub & 3;
    const uint8_t *q = qs + 32 * n;
#pragma unroll
    for (int hf = 0; hf < 2; hf++) {
        uint8_t sc = scales[8 * n + 2 * j + hf];
        float dl = __fmul_rn(d, (float)(sc & 0xF)), ml = __fmul_rn(dmin, (float)(sc >> 4));
#pragma unroll
        for (int l = 0; l < 16; l++)
            w[16 * hf + l] = __fsub_rn(__fmul_rn(dl, (float)((q[16 * hf + l] >> (2 * j)) & 3)), ml);
    }
}

// src/dequant.rs:1482-1519
template <>
__device__ __forceinline__ void decode32<T_Q4_K>(const Fields &F, int sub, float *w)
{
    float d = h2f(ld_u16(F.f[0])), dmin = h2f(ld_u16(F.f[0] + 2));
    int sc, mn;
    scale_min_k4(sub, F.f[0] + 4, sc, mn);
    float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
    const uint8_t *qs = F.f[1] + 32 * (sub >> 1);
    int sh = (sub & 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; l++) w[l] = __fsub_rn(__fmul_rn(d1, (float)((qs[l] >> sh) & 0x0F)), m1);
}

// src/dequant.rs:1146-1181: bit `sub` of qh[l] is the fifth bit of weight 32*sub + l
template <>
__device__ __forceinline__ void decode32<T_Q5_K>(const Fields &F, int sub, float *w)
{
    float d = h2f(ld_u16(F.f[0])), dmin = h2f(ld_u16(F.f[0] + 2));
    int sc, mn;
    scale_min_k4(sub, F.f[0] + 4, sc, mn);
    float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
    const uint8_t *qh = F.f[1], *ql = F.f[2] + 32 * (sub >> 1);
    int sh = (sub & 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; l++) {
        float q = __fadd_rn((float)((ql[l] >> sh) & 0x0F), ((qh[l] >> sub) & 1) ? 16.0f : 0.0f);
        w[l] = __fsub_rn(__fmul_rn(d1, q), m1);
    }
}

// src/dequant.rs:1583-1631.  Weight i = 128n + 32k + l: low nibble source
// ql[64n + 32(k&1) + l] >> 4(k>>1), high bits qh[32n + l] >> 2k, scale sc[8n + 2k + l/16].
template <>
__device__ __forceinline__ void decode32<T_Q6_K>(const Fields &F, int sub, float *w)
{
    int n = sub >> 2, k = sub & 3;
    const uint8_t *ql = F.f[0] + 64 * n + 32 * (k & 1), *qh = F.f[1] + 32 * n;
    const int8_t *sc = (const int8_t *)F.f[2] + 8 * n + 2 * k;
    float d = h2f(ld_u16(F.f[3]));
    int sh = (k >> 1) * 4;
#pragma unroll
    for (int l = 0; l < 32; l++) {
        int q = (int)(((ql[l] >> sh) & 0x0F) | (((qh[l] >> (2 * k)) & 3) << 4)) - 32;
        w[l] = __fmul_rn(__fmul_rn(d, (float)sc[l >> 4]), (float)q);
    }
}

// src/dequant.rs:1011-1041
template <>
__device__ __forceinline__ void decode32<T_IQ2_XXS>(const Fields &F, int sub, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    const uint8_t *a0 = F.f[1] + 8 * sub;
    uint32_t a1 = ld_u32_bytes(a0 + 4);
    float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(a1 >> 28))), 0.25f);
#pragma unroll
    for (int l = 0; l < 4; l++) {
        uint64_t g = g_iq2xxs_grid[a0[l]];
        uint32_t s = g_ksigns[(a1 >> (7 * l)) & 127];
#pragma unroll
        for (int j = 0; j < 8; j++) w[8 * l + j] = signed_grid(db, (int)(int8_t)(g >> (8 * j)), s, j);
    }
}

// src/dequant.rs:1043-1075
template <>
__device__ __forceinline__ void decode32<T_IQ2_XS>(const Fields &F, int sub, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    const uint8_t *qs = F.f[1] + 8 * sub;
    uint8_t scb = F.f[2][sub];
    float db0 = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(scb & 0xf))), 0.25f);
    float db1 = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(scb >> 4))), 0.25f);
#pragma unroll
    for (int l = 0; l < 4; l++) {
        uint32_t q = ld_u16(qs + 2 * l);
        uint64_t g = g_iq2xs_grid[q & 511];
        uint32_t s = g_ksigns[q >> 9];
        float db = l < 2 ? db0 : db1;
#pragma unroll
        for (int j = 0; j < 8; j++) w[8 * l + j] = signed_grid(db, (int)(int8_t)(g >> (8 * j)), s, j);
    }
}

// src/dequant.rs:1077-1110
template <>
__device__ __forceinline__ void decode32<T_IQ2_S>(const Fields &F, int sub, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    const uint8_t *qs = F.f[1];
    uint32_t qh = F.f[2][sub];
    uint8_t scb = F.f[3][sub];
    float db0 = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(scb & 0xf))), 0.25f);
    float db1 = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(scb >> 4))), 0.25f);
#pragma unroll
    for (int l = 0; l < 4; l++) {
        uint32_t idx = (uint32_t)qs[4 * sub + l] | ((qh << (8 - 2 * l)) & 0x300);
        uint64_t g = g_iq2s_grid[idx];
        uint32_t s = qs[32 + 4 * sub + l];
        float db = l < 2 ? db0 : db1;
#pragma unroll
        for (int j = 0; j < 8; j++) w[8 * l + j] = signed_grid(db, (int)(int8_t)(g >> (8 * j)), s, j);
    }
}

// src/dequant.rs:1184-1237: sub-block `sub` takes qs[8 sub..], qh[sub], signs[4 sub..],
// and nibble (sub & 1) of scales[sub / 2]
template <>
__device__ __forceinline__ void decode32<T_IQ3_S>(const Fields &F, int sub, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    const uint8_t *qs = F.f[1] + 8 * sub, *sg = F.f[3] + 4 * sub;
    uint32_t qhb = F.f[2][sub];
    uint8_t scb = F.f[4][sub >> 1];
    int sc = (sub & 1) ? (scb >> 4) : (scb & 0xf);
    float db = __fmul_rn(d, __fadd_rn(1.0f, __fmul_rn(2.0f, (float)sc)));
#pragma unroll
    for (int l = 0; l < 4; l++) {
        uint32_t g1 = g_iq3s_grid[(uint32_t)qs[2 * l] | ((qhb << (8 - 2 * l)) & 256)];
        uint32_t g2 = g_iq3s_grid[(uint32_t)qs[2 * l + 1] | ((qhb << (7 - 2 * l)) & 256)];
        uint32_t s = sg[l];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            w[8 * l + j] = signed_grid(db, (int)(int8_t)(g1 >> (8 * j)), s, j);
            w[8 * l + 4 + j] = signed_grid(db, (int)(int8_t)(g2 >> (8 * j)), s, j + 4);
        }
    }
}

// ggml block_iq3_xxs (absent from the reference): db = d*(0.5+s)*0.5
template <>
__device__ __forceinline__ void decode32<T_IQ3_XXS>(const Fields &F, int sub, float *w)
{
    float d = h2f(ld_u16(F.f[0]));
    const uint8_t *qs = F.f[1] + 8 * sub;
    uint32_t a1 = ld_u32_bytes(F.f[2] + 4 * sub);
    float db = __fmul_rn(__fmul_rn(d, __fadd_rn(0.5f, (float)(a1 >> 28))), 0.5f);
#pragma unroll
    for (int l = 0; l < 4; l++) {
        uint32_t g1 = g_iq3xxs_grid[qs[2 * l]], g2 = g_iq3xxs_grid[qs[2 * l + 1]];
        uint32_t s = g_ksigns[(a1 >> (7 * l)) & 127];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            w[8 * l + j] = signed_grid(db, (int)(uint8_t)(g1 >> (8 * j)), s, j);
            w[8 * l + 4 + j] = signed_grid(db, (int)(uint8_t)(g2 >> (8 * j)), s, j + 4);
        }
    }
}

}  // namespace qz
