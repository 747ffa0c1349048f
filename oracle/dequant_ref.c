/*
 * CPU oracle -- TEST INFRASTRUCTURE ONLY (see dequant_ref.h for the parity
 * status).  Plain-C restatement of the reference's src/dequant.rs.
 *
 * Floating-point discipline: Rust/LLVM neither contracts a*b+c into an FMA
 * nor reassociates, so this file must be compiled with -ffp-contract=off and
 * without -ffast-math; every expression below keeps the reference's
 * association, and every reduction runs serially in index order.
 */
#include "dequant_ref.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- codebooks (caller-supplied data) ----------------------------------- */
static const uint64_t *g_iq2xxs, *g_iq2xs, *g_iq2s;
static const uint32_t *g_iq3s, *g_iq3xxs;
static uint8_t g_ksigns[128];
static int g_ksigns_ready;

void qz_set_iq2xxs_grid(const uint64_t *g) { g_iq2xxs = g; }
void qz_set_iq2xs_grid(const uint64_t *g) { g_iq2xs = g; }
void qz_set_iq2s_grid(const uint64_t *g) { g_iq2s = g; }
void qz_set_iq3s_grid(const uint32_t *g) { g_iq3s = g; }
void qz_set_iq3xxs_grid(const uint32_t *g) { g_iq3xxs = g; }

/* KSIGNS_IQ2XS (src/iq2_tables.rs:9): entry i is i with bit 7 set when i has
 * odd parity, so that each 8-bit sign pattern has an even number of minus
 * signs.  Computed, not tabulated. */
const uint8_t *qz_ksigns(void)
{
    if (!g_ksigns_ready) {
        for (int i = 0; i < 128; i++)
            g_ksigns[i] = (uint8_t)(i | ((__builtin_popcount(i) & 1) << 7));
        g_ksigns_ready = 1;
    }
    return g_ksigns;
}

int qz_max_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

static int pick_threads(int threads)
{
    int m = qz_max_threads();
    if (threads <= 0 || threads > m) return m;
    return threads;
}

/* ---- block geometry: src/gguf.rs:172-191 -------------------------------- */
int qz_block_elems(uint32_t t)
{
    switch (t) {
    case QZ_F32: case QZ_F16: case QZ_BF16: return 1;
    case QZ_Q4_0: case QZ_Q4_1: case QZ_Q5_0: case QZ_Q5_1: case QZ_Q8_0: case QZ_IQ4_NL: return 32;
    case QZ_Q2_K: case QZ_Q4_K: case QZ_Q5_K: case QZ_Q6_K: case QZ_IQ2_XXS: case QZ_IQ2_XS:
    case QZ_IQ3_XXS: case QZ_IQ3_S: case QZ_IQ2_S: return 256;
    default: return 0;
    }
}

int qz_block_bytes(uint32_t t)
{
    switch (t) {
    case QZ_F32: return 4;
    case QZ_F16: case QZ_BF16: return 2;
    case QZ_Q4_0: return 18;   /* not in the reference: ggml block_q4_0 */
    case QZ_Q4_1: return 20;   /* not in the reference: ggml block_q4_1 */
    case QZ_Q5_0: return 22;
    case QZ_Q5_1: return 24;
    case QZ_Q8_0: return 34;
    case QZ_Q2_K: return 84;
    case QZ_Q4_K: return 144;
    case QZ_Q5_K: return 176;
    case QZ_Q6_K: return 210;
    case QZ_IQ4_NL: return 18;
    case QZ_IQ2_XXS: return 66;
    case QZ_IQ2_XS: return 74;
    case QZ_IQ3_XXS: return 98; /* not in the reference: ggml block_iq3_xxs */
    case QZ_IQ2_S: return 82;
    case QZ_IQ3_S: return 110;
    default: return 0;
    }
}

size_t qz_type_size(uint32_t t, size_t n)
{
    int be = qz_block_elems(t);
    if (!be) return 0;
    return (n / (size_t)be) * (size_t)qz_block_bytes(t);
}

/* ---- f16 -> f32: src/dequant.rs:1329-1349 ------------------------------- */
static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }

float qz_f16_to_f32(uint16_t bits)
{
    uint32_t sign = (uint32_t)(bits >> 15);
    uint32_t exp = (bits >> 10) & 0x1F;
    uint32_t mant = bits & 0x3FF;
    if (exp == 0) {
        if (mant == 0) return bits_f32(sign << 31);
        uint32_t e = 0, m = mant;
        while ((m & 0x400) == 0) { m <<= 1; e++; }
        return bits_f32((sign << 31) | ((127 - 15 - e + 1) << 23) | ((m & 0x3FF) << 13));
    }
    if (exp == 31) return bits_f32((sign << 31) | 0x7F800000u | (mant << 13));
    return bits_f32((sign << 31) | ((exp + 127 - 15) << 23) | (mant << 13));
}

static inline float rd_f16(const uint8_t *p) { return qz_f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }
static inline uint32_t rd_u32(const uint8_t *p)
{
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

/* ---- per-format block decoders (one block -> block_elems floats) -------- */

/* src/dequant.rs:1321-1371 */
static void blk_f32(const uint8_t *b, float *o) { o[0] = bits_f32(rd_u32(b)); }
static void blk_f16(const uint8_t *b, float *o) { o[0] = rd_f16(b); }
static void blk_bf16(const uint8_t *b, float *o) { o[0] = bits_f32((uint32_t)(b[0] | (b[1] << 8)) << 16); }

/* ggml block_q4_0 {f16 d; u8 qs[16]}: w[j] = d*((qs[j]&15)-8), w[j+16] = d*((qs[j]>>4)-8).
 * Absent from the reference; operation order of gguf-py 0.19.0 Q4_0.dequantize_blocks. */
static void blk_q4_0(const uint8_t *b, float *o)
{
    float d = rd_f16(b);
    const uint8_t *qs = b + 2;
    for (int j = 0; j < 16; j++) {
        o[j] = d * (float)((int)(qs[j] & 0x0F) - 8);
        o[j + 16] = d * (float)((int)(qs[j] >> 4) - 8);
    }
}

/* ggml block_q4_1 {f16 d; f16 m; u8 qs[16]}: w = d*q + m.  Absent from the
 * reference; order of gguf-py 0.19.0 Q4_1.dequantize_blocks. */
static void blk_q4_1(const uint8_t *b, float *o)
{
    float d = rd_f16(b), m = rd_f16(b + 2);
    const uint8_t *qs = b + 4;
    for (int j = 0; j < 16; j++) {
        o[j] = d * (float)(qs[j] & 0x0F) + m;
        o[j + 16] = d * (float)(qs[j] >> 4) + m;
    }
}

/* src/dequant.rs:1381-1409 */
static void blk_q5_0(const uint8_t *b, float *o)
{
    float d = rd_f16(b);
    uint32_t qh = rd_u32(b + 2);
    const uint8_t *qs = b + 6;
    for (int j = 0; j < 16; j++) {
        uint32_t xh0 = ((qh >> j) << 4) & 0x10;
        uint32_t xh1 = (qh >> (j + 12)) & 0x10;
        int x0 = (int)((qs[j] & 0x0Fu) | xh0) - 16;
        int x1 = (int)((uint32_t)(qs[j] >> 4) | xh1) - 16;
        o[j] = (float)x0 * d;
        o[j + 16] = (float)x1 * d;
    }
}

/* src/dequant.rs:1419-1443 */
static void blk_q5_1(const uint8_t *b, float *o)
{
    float d = rd_f16(b), m = rd_f16(b + 2);
    uint32_t qh = rd_u32(b + 4);
    const uint8_t *qs = b + 8;
    for (int j = 0; j < 16; j++) {
        uint32_t xh0 = ((qh >> j) << 4) & 0x10;
        uint32_t xh1 = (qh >> (j + 12)) & 0x10;
        float x0 = (float)((qs[j] & 0x0Fu) | xh0);
        float x1 = (float)((uint32_t)(qs[j] >> 4) | xh1);
        o[j] = x0 * d + m;
        o[j + 16] = x1 * d + m;
    }
}

/* src/dequant.rs:1450-1463 */
static void blk_q8_0(const uint8_t *b, float *o)
{
    float d = rd_f16(b);
    for (int i = 0; i < 32; i++) o[i] = d * (float)(int8_t)b[2 + i];
}

/* src/dequant.rs:1113-1144 */
static void blk_q2_k(const uint8_t *b, float *o)
{
    const uint8_t *scales = b, *qs = b + 16;
    float d = rd_f16(b + 80), dmin = rd_f16(b + 82);
    int is = 0, k = 0;
    for (int n = 0; n < 256; n += 128) {
        const uint8_t *q = qs + (n / 128) * 32;
        for (int j = 0; j < 4; j++) {
            int shift = 2 * j;
            uint8_t sc = scales[is++];
            float dl = d * (float)(sc & 0xF), ml = dmin * (float)(sc >> 4);
            for (int l = 0; l < 16; l++) o[k++] = dl * (float)((q[l] >> shift) & 3) - ml;
            sc = scales[is++];
            dl = d * (float)(sc & 0xF); ml = dmin * (float)(sc >> 4);
            for (int l = 0; l < 16; l++) o[k++] = dl * (float)((q[l + 16] >> shift) & 3) - ml;
        }
    }
}

/* src/dequant.rs:1471-1480 */
static inline void scale_min_k4(int j, const uint8_t *s, uint8_t *sc, uint8_t *m)
{
    if (j < 4) {
        *sc = s[j] & 63;
        *m = s[j + 4] & 63;
    } else {
        *sc = (uint8_t)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
        *m = (uint8_t)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
    }
}

/* src/dequant.rs:1482-1519 (identical arithmetic to q4k_row_batched :38-66) */
static void blk_q4_k(const uint8_t *b, float *o)
{
    float d = rd_f16(b), dmin = rd_f16(b + 2);
    const uint8_t *scales = b + 4, *qs = b + 16;
    int q_off = 0, is = 0, k = 0;
    for (int it = 0; it < 4; it++) {
        uint8_t sc1, mn1, sc2, mn2;
        scale_min_k4(is, scales, &sc1, &mn1);
        scale_min_k4(is + 1, scales, &sc2, &mn2);
        float d1 = d * (float)sc1, m1 = dmin * (float)mn1;
        float d2 = d * (float)sc2, m2 = dmin * (float)mn2;
        for (int l = 0; l < 32; l++) o[k++] = d1 * (float)(qs[q_off + l] & 0x0F) - m1;
        for (int l = 0; l < 32; l++) o[k++] = d2 * (float)(qs[q_off + l] >> 4) - m2;
        q_off += 32;
        is += 2;
    }
}

/* src/dequant.rs:1146-1181 */
static void blk_q5_k(const uint8_t *b, float *o)
{
    float d = rd_f16(b), dmin = rd_f16(b + 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *qs = b + 48;
    int is = 0, k = 0;
    uint8_t u1 = 1, u2 = 2;
    for (int jb = 0; jb < 4; jb++) {
        const uint8_t *ql = qs + jb * 32;
        uint8_t sc1, mn1, sc2, mn2;
        scale_min_k4(is, scales, &sc1, &mn1);
        float d1 = d * (float)sc1, m1 = dmin * (float)mn1;
        scale_min_k4(is + 1, scales, &sc2, &mn2);
        float d2 = d * (float)sc2, m2 = dmin * (float)mn2;
        for (int l = 0; l < 32; l++)
            o[k++] = d1 * ((float)(ql[l] & 0xF) + ((qh[l] & u1) ? 16.0f : 0.0f)) - m1;
        for (int l = 0; l < 32; l++)
            o[k++] = d2 * ((float)(ql[l] >> 4) + ((qh[l] & u2) ? 16.0f : 0.0f)) - m2;
        is += 2;
        u1 <<= 2;
        u2 <<= 2;
    }
}

/* src/dequant.rs:1583-1631 (identical arithmetic to q6k_row :714-746) */
static void blk_q6_k(const uint8_t *b, float *o)
{
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    float d = rd_f16(b + 208);
    float *y = o;
    for (int half = 0; half < 2; half++) {
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int q1 = (int)((ql[l] & 0x0F) | (((qh[l] >> 0) & 3) << 4)) - 32;
            int q2 = (int)((ql[l + 32] & 0x0F) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            y[l + 0] = d * (float)sc[is + 0] * (float)q1;
            y[l + 32] = d * (float)sc[is + 2] * (float)q2;
            y[l + 64] = d * (float)sc[is + 4] * (float)q3;
            y[l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
        ql += 64; qh += 32; sc += 8; y += 128;
    }
}

/* 8 weights from a u64 grid entry (8 x int8) and a sign byte:
 * out = (db * g[j]) * (+-1), src/dequant.rs:1029-1036. */
static inline void grid8(float db, uint64_t g, uint8_t signs, float *o)
{
    for (int j = 0; j < 8; j++) {
        float s = (signs & (1u << j)) ? -1.0f : 1.0f;   /* KMASK_IQ2XS[j] = 1<<j */
        o[j] = db * (float)(int8_t)(g >> (8 * j)) * s;
    }
}

/* src/dequant.rs:1011-1041 */
static void blk_iq2_xxs(const uint8_t *b, float *o)
{
    const uint8_t *ks = qz_ksigns();
    float d = rd_f16(b);
    const uint8_t *qs = b + 2;
    for (int ib32 = 0; ib32 < 8; ib32++) {
        const uint8_t *a0 = qs + 8 * ib32;
        uint32_t a1 = rd_u32(qs + 8 * ib32 + 4);
        float db = d * (0.5f + (float)(a1 >> 28)) * 0.25f;
        for (int l = 0; l < 4; l++)
            grid8(db, g_iq2xxs[a0[l]], ks[(a1 >> (7 * l)) & 127], o + 32 * ib32 + 8 * l);
    }
}

/* src/dequant.rs:1043-1075 */
static void blk_iq2_xs(const uint8_t *b, float *o)
{
    const uint8_t *ks = qz_ksigns();
    float d = rd_f16(b);
    const uint8_t *qs = b + 2, *scales = b + 66;
    for (int ib32 = 0; ib32 < 8; ib32++) {
        float db0 = d * (0.5f + (float)(scales[ib32] & 0xf)) * 0.25f;
        float db1 = d * (0.5f + (float)(scales[ib32] >> 4)) * 0.25f;
        for (int l = 0; l < 4; l++) {
            int qi = 2 * (4 * ib32 + l);
            uint32_t q = (uint32_t)qs[qi] | ((uint32_t)qs[qi + 1] << 8);
            grid8(l < 2 ? db0 : db1, g_iq2xs[q & 511], ks[q >> 9], o + 32 * ib32 + 8 * l);
        }
    }
}

/* src/dequant.rs:1077-1110 */
static void blk_iq2_s(const uint8_t *b, float *o)
{
    float d = rd_f16(b);
    const uint8_t *qs = b + 2, *qh = b + 66, *scales = b + 74;
    for (int ib32 = 0; ib32 < 8; ib32++) {
        float db0 = d * (0.5f + (float)(scales[ib32] & 0xf)) * 0.25f;
        float db1 = d * (0.5f + (float)(scales[ib32] >> 4)) * 0.25f;
        for (int l = 0; l < 4; l++) {
            uint32_t idx = (uint32_t)qs[4 * ib32 + l] | ((((uint32_t)qh[ib32]) << (8 - 2 * l)) & 0x300);
            grid8(l < 2 ? db0 : db1, g_iq2s[idx], qs[32 + 4 * ib32 + l], o + 32 * ib32 + 8 * l);
        }
    }
}

/* src/dequant.rs:1184-1237 */
static void blk_iq3_s(const uint8_t *b, float *o)
{
    float d = rd_f16(b);
    const uint8_t *qs = b + 2, *qh = b + 66, *sg = b + 74, *scales = b + 106;
    int qo = 0, so = 0, ho = 0, k = 0;
    for (int ib32 = 0; ib32 < 8; ib32 += 2) {
        float db1 = d * (1.0f + 2.0f * (float)(scales[ib32 / 2] & 0xf));
        float db2 = d * (1.0f + 2.0f * (float)(scales[ib32 / 2] >> 4));
        for (int half = 0; half < 2; half++) {
            float db = half ? db2 : db1;
            uint32_t qhb = qh[ho + half];
            int qbase = qo + half * 8, sbase = so + half * 4;
            for (int l = 0; l < 4; l++) {
                uint32_t i0 = (uint32_t)qs[qbase + 2 * l] | ((qhb << (8 - 2 * l)) & 256);
                uint32_t i1 = (uint32_t)qs[qbase + 2 * l + 1] | ((qhb << (7 - 2 * l)) & 256);
                uint32_t g1 = g_iq3s[i0], g2 = g_iq3s[i1];
                uint8_t s = sg[sbase + l];
                for (int j = 0; j < 4; j++)
                    o[k++] = db * (float)(int8_t)(g1 >> (8 * j)) * ((s & (1u << j)) ? -1.0f : 1.0f);
                for (int j = 0; j < 4; j++)
                    o[k++] = db * (float)(int8_t)(g2 >> (8 * j)) * ((s & (1u << (j + 4))) ? -1.0f : 1.0f);
            }
        }
        qo += 16; so += 8; ho += 2;
    }
}

/* ggml block_iq3_xxs {f16 d; u8 qs[64]; u8 scales_and_signs[32]}: per 32 weights
 * eight grid bytes (4 values each) and one u32 = 4 x 7-bit sign index | 4-bit
 * scale << 28; db = d*(0.5+s)*0.5; w = (db*grid)*sign.  Absent from the
 * reference; order of gguf-py 0.19.0 IQ3_XXS.dequantize_blocks. */
static void blk_iq3_xxs(const uint8_t *b, float *o)
{
    const uint8_t *ks = qz_ksigns();
    float d = rd_f16(b);
    const uint8_t *qs = b + 2, *sas = b + 66;
    for (int ib32 = 0; ib32 < 8; ib32++) {
        uint32_t a1 = rd_u32(sas + 4 * ib32);
        float db = d * (0.5f + (float)(a1 >> 28)) * 0.5f;
        for (int l = 0; l < 4; l++) {
            uint8_t s = ks[(a1 >> (7 * l)) & 127];
            uint32_t g1 = g_iq3xxs[qs[8 * ib32 + 2 * l]], g2 = g_iq3xxs[qs[8 * ib32 + 2 * l + 1]];
            float *y = o + 32 * ib32 + 8 * l;
            for (int j = 0; j < 4; j++)
                y[j] = db * (float)(uint8_t)(g1 >> (8 * j)) * ((s & (1u << j)) ? -1.0f : 1.0f);
            for (int j = 0; j < 4; j++)
                y[4 + j] = db * (float)(uint8_t)(g2 >> (8 * j)) * ((s & (1u << (j + 4))) ? -1.0f : 1.0f);
        }
    }
}

/* src/dequant.rs:1527-1530 */
static const float IQ4NL_TABLE[16] = {-127.0f, -104.0f, -83.0f, -65.0f, -49.0f, -35.0f, -22.0f, -10.0f,
                                      1.0f,    13.0f,   25.0f,  38.0f,  53.0f,  69.0f,  89.0f,  113.0f};

/* src/dequant.rs:1557-1574 */
static void blk_iq4_nl(const uint8_t *b, float *o)
{
    float d = rd_f16(b);
    const uint8_t *qs = b + 2;
    for (int k = 0; k < 16; k++) {
        o[k] = d * IQ4NL_TABLE[qs[k] & 0x0F];
        o[k + 16] = d * IQ4NL_TABLE[qs[k] >> 4];
    }
}

typedef void (*blk_fn)(const uint8_t *, float *);

static blk_fn decoder(uint32_t t)
{
    switch (t) {
    case QZ_F32: return blk_f32;
    case QZ_F16: return blk_f16;
    case QZ_BF16: return blk_bf16;
    case QZ_Q4_0: return blk_q4_0;
    case QZ_Q4_1: return blk_q4_1;
    case QZ_Q5_0: return blk_q5_0;
    case QZ_Q5_1: return blk_q5_1;
    case QZ_Q8_0: return blk_q8_0;
    case QZ_Q2_K: return blk_q2_k;
    case QZ_Q4_K: return blk_q4_k;
    case QZ_Q5_K: return blk_q5_k;
    case QZ_Q6_K: return blk_q6_k;
    case QZ_IQ2_XXS: return g_iq2xxs ? blk_iq2_xxs : NULL;
    case QZ_IQ2_XS: return g_iq2xs ? blk_iq2_xs : NULL;
    case QZ_IQ2_S: return g_iq2s ? blk_iq2_s : NULL;
    case QZ_IQ3_S: return g_iq3s ? blk_iq3_s : NULL;
    case QZ_IQ3_XXS: return g_iq3xxs ? blk_iq3_xxs : NULL;
    case QZ_IQ4_NL: return blk_iq4_nl;
    default: return NULL;
    }
}

/* src/dequant.rs:1239-1258: blocks decoded one after another */
int qz_dequant(const uint8_t *data, uint32_t t, size_t n, float *out)
{
    blk_fn f = decoder(t);
    if (!f) return -1;
    size_t be = (size_t)qz_block_elems(t), bb = (size_t)qz_block_bytes(t);
    size_t nb = n / be;
    for (size_t b = 0; b < nb; b++) f(data + b * bb, out + b * be);
    return 0;
}

/* ---- fused rows --------------------------------------------------------- */

/* src/dequant.rs:659-706: per sub-block sq = sum x*q, sx = sum x (index
 * order), acc += d1*sq - m1*sx. */
static float q4k_row(const float *x, const uint8_t *row, size_t bpr)
{
    float acc = 0.0f;
    for (size_t b = 0; b < bpr; b++) {
        const uint8_t *blk = row + b * 144;
        float d = rd_f16(blk), dmin = rd_f16(blk + 2);
        const uint8_t *scales = blk + 4, *qs = blk + 16;
        const float *xb = x + b * 256;
        int q_off = 0, is = 0, o = 0;
        for (int it = 0; it < 4; it++) {
            uint8_t sc1, mn1, sc2, mn2;
            scale_min_k4(is, scales, &sc1, &mn1);
            scale_min_k4(is + 1, scales, &sc2, &mn2);
            float d1 = d * (float)sc1, m1 = dmin * (float)mn1;
            float d2 = d * (float)sc2, m2 = dmin * (float)mn2;
            float sq1 = 0.0f, sx1 = 0.0f;
            for (int l = 0; l < 32; l++) {
                float xv = xb[o + l];
                sq1 += xv * (float)(qs[q_off + l] & 0x0F);
                sx1 += xv;
            }
            acc += d1 * sq1 - m1 * sx1;
            o += 32;
            float sq2 = 0.0f, sx2 = 0.0f;
            for (int l = 0; l < 32; l++) {
                float xv = xb[o + l];
                sq2 += xv * (float)(qs[q_off + l] >> 4);
                sx2 += xv;
            }
            acc += d2 * sq2 - m2 * sx2;
            o += 32;
            q_off += 32;
            is += 2;
        }
    }
    return acc;
}

/* src/dequant.rs:710-752: decode the block, then acc += x[i]*y[i] in order */
static float q6k_row(const float *x, const uint8_t *row, size_t bpr)
{
    float acc = 0.0f, y[256];
    for (size_t b = 0; b < bpr; b++) {
        blk_q6_k(row + b * 210, y);
        const float *xb = x + b * 256;
        for (int i = 0; i < 256; i++) acc += xb[i] * y[i];
    }
    return acc;
}

/* src/dequant.rs:916-944 */
static float q5_1_row(const float *x, const uint8_t *row, size_t bpr)
{
    float acc = 0.0f;
    for (size_t b = 0; b < bpr; b++) {
        const uint8_t *blk = row + b * 24;
        float d = rd_f16(blk), m = rd_f16(blk + 2);
        uint32_t qh = rd_u32(blk + 4);
        const uint8_t *qs = blk + 8;
        const float *xi = x + b * 32;
        for (int k = 0; k < 16; k++) {
            uint32_t xh0 = ((qh >> k) << 4) & 0x10;
            uint32_t xh1 = (qh >> (k + 12)) & 0x10;
            float q0 = (float)((qs[k] & 0x0Fu) | xh0);
            float q1 = (float)((uint32_t)(qs[k] >> 4) | xh1);
            acc += xi[k] * (q0 * d + m) + xi[k + 16] * (q1 * d + m);
        }
    }
    return acc;
}

/* src/dequant.rs:1532-1555 */
static float iq4nl_row(const float *x, const uint8_t *row, size_t bpr)
{
    float acc = 0.0f;
    for (size_t b = 0; b < bpr; b++) {
        const uint8_t *blk = row + b * 18;
        float d = rd_f16(blk);
        const uint8_t *qs = blk + 2;
        const float *xi = x + b * 32;
        for (int k = 0; k < 16; k++) {
            acc += xi[k] * d * IQ4NL_TABLE[qs[k] & 0x0F];
            acc += xi[k + 16] * d * IQ4NL_TABLE[qs[k] >> 4];
        }
    }
    return acc;
}

/* src/dequant.rs:859-865 and src/main.rs:710-718: sum a[k]*b[k] in order */
static float dot_row(const float *a, const float *b, size_t n)
{
    float s = 0.0f;
    for (size_t k = 0; k < n; k++) s += a[k] * b[k];
    return s;
}

/* src/dequant.rs:18-31.  The reference's fallback arm dequantizes the whole
 * matrix and then calls matmul (per row: sum x*w in index order); decoding
 * row by row gives the same numbers without the N*K*4-byte temporary. */
int qz_gemv(const float *x, const uint8_t *data, uint32_t t, size_t K, size_t N, float *y, int threads)
{
    blk_fn f = decoder(t);
    if (!f) return -1;
    size_t be = (size_t)qz_block_elems(t), bb = (size_t)qz_block_bytes(t);
    size_t bpr = K / be, row_bytes = bpr * bb;
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel num_threads(nt)
    {
        float *w = NULL;
        if (!(t == QZ_Q4_K || t == QZ_Q6_K || t == QZ_Q5_1 || t == QZ_IQ4_NL))
            w = (float *)malloc(sizeof(float) * (K ? K : 1));
#pragma omp for schedule(static)
        for (long long j = 0; j < (long long)N; j++) {
            const uint8_t *row = data + (size_t)j * row_bytes;
            switch (t) {
            case QZ_Q4_K: y[j] = q4k_row(x, row, bpr); break;
            case QZ_Q6_K: y[j] = q6k_row(x, row, bpr); break;
            case QZ_Q5_1: y[j] = q5_1_row(x, row, bpr); break;
            case QZ_IQ4_NL: y[j] = iq4nl_row(x, row, bpr); break;
            default:
                /* F32 (:962-981) and BF16 (:946-960) are sum x[k]*w[k] as well */
                for (size_t b = 0; b < bpr; b++) f(row + b * bb, w + b * be);
                y[j] = dot_row(x, w, K);
            }
        }
        free(w);
    }
    return 0;
}

/* src/dequant.rs:143-200.  Q4_K/Q6_K (:38-122): decode one block to wv[256],
 * per token s = sum xt[i]*wv[i], acc[t] += s.  Others: decode the row, dot. */
int qz_gemm(const float *x, const uint8_t *data, uint32_t t, size_t K, size_t N, size_t n, float *out,
            int threads)
{
    if (n == 1) return qz_gemv(x, data, t, K, N, out, threads);
    blk_fn f = decoder(t);
    if (!f) return -1;
    size_t be = (size_t)qz_block_elems(t), bb = (size_t)qz_block_bytes(t);
    size_t bpr = K / be, row_bytes = bpr * bb;
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel num_threads(nt)
    {
        float *w = (float *)malloc(sizeof(float) * (K ? K : 1));
        float *acc = (float *)malloc(sizeof(float) * n);
#pragma omp for schedule(static)
        for (long long j = 0; j < (long long)N; j++) {
            const uint8_t *row = data + (size_t)j * row_bytes;
            for (size_t tt = 0; tt < n; tt++) acc[tt] = 0.0f;
            if (t == QZ_Q4_K || t == QZ_Q6_K) {
                float wv[256];
                for (size_t b = 0; b < bpr; b++) {
                    f(row + b * bb, wv);
                    for (size_t tt = 0; tt < n; tt++) {
                        const float *xt = x + tt * K + b * 256;
                        float s = 0.0f;
                        for (int i = 0; i < 256; i++) s += xt[i] * wv[i];
                        acc[tt] += s;
                    }
                }
            } else {
                for (size_t b = 0; b < bpr; b++) f(row + b * bb, w + b * be);
                for (size_t tt = 0; tt < n; tt++) acc[tt] = dot_row(x + tt * K, w, K);
            }
            for (size_t tt = 0; tt < n; tt++) out[tt * N + (size_t)j] = acc[tt];
        }
        free(w);
        free(acc);
    }
    return 0;
}

int qz_row_norms(const uint8_t *data, uint32_t t, size_t K, size_t N, double *norms, int threads)
{
    blk_fn f = decoder(t);
    if (!f) return -1;
    size_t be = (size_t)qz_block_elems(t), bb = (size_t)qz_block_bytes(t);
    size_t bpr = K / be, row_bytes = bpr * bb;
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel num_threads(nt)
    {
        float *w = (float *)malloc(sizeof(float) * (K ? K : 1));
#pragma omp for schedule(static)
        for (long long j = 0; j < (long long)N; j++) {
            const uint8_t *row = data + (size_t)j * row_bytes;
            for (size_t b = 0; b < bpr; b++) f(row + b * bb, w + b * be);
            double s = 0.0;
            for (size_t k = 0; k < K; k++) s += (double)w[k] * (double)w[k];
            norms[j] = sqrt(s);
        }
        free(w);
    }
    return 0;
}

int qz_gemv_f64(const float *x, const uint8_t *data, uint32_t t, size_t K, size_t N, double *y, int threads)
{
    blk_fn f = decoder(t);
    if (!f) return -1;
    size_t be = (size_t)qz_block_elems(t), bb = (size_t)qz_block_bytes(t);
    size_t bpr = K / be, row_bytes = bpr * bb;
    int nt = pick_threads(threads);
    (void)nt;
#pragma omp parallel num_threads(nt)
    {
        float *w = (float *)malloc(sizeof(float) * (K ? K : 1));
#pragma omp for schedule(static)
        for (long long j = 0; j < (long long)N; j++) {
            const uint8_t *row = data + (size_t)j * row_bytes;
            for (size_t b = 0; b < bpr; b++) f(row + b * bb, w + b * be);
            double s = 0.0;
            for (size_t k = 0; k < K; k++) s += (double)x[k] * (double)w[k];
            y[j] = s;
        }
        free(w);
    }
    return 0;
}
