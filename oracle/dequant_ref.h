/*
 * CPU oracle for the quantized-weight GEMV/GEMM path -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU path (src/dequant.rs in the
 * reference project): dequant(), gemv(), gemm().  Only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark may load this
 * library; the CUDA product never calls it.
 *
 * Parity status: the reference ships no golden vectors for this path and its
 * Rust sources cannot be compiled in this environment, so the restatement is
 * pinned (bit-exact, u32 compare) against the independent `gguf` 0.19.0
 * Python package's dequantize() for every block format, and (within the GEMV
 * tolerance) against the reference's own CUDA kernels built unmodified into
 * oracle/_ref.  Formats 2 (Q4_0), 3 (Q4_1) and 18 (IQ3_XXS) do not exist in
 * the reference at all: for those three, parity is unpinned by the reference
 * and rests on gguf-py alone.
 */
#ifndef QZ_ORACLE_DEQUANT_REF_H
#define QZ_ORACLE_DEQUANT_REF_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml type ids, as in src/gguf.rs:172-188 (plus the three extension ids). */
enum {
    QZ_F32 = 0, QZ_F16 = 1, QZ_Q4_0 = 2, QZ_Q4_1 = 3, QZ_Q5_0 = 6, QZ_Q5_1 = 7,
    QZ_Q8_0 = 8, QZ_Q2_K = 10, QZ_Q4_K = 12, QZ_Q5_K = 13, QZ_Q6_K = 14,
    QZ_IQ2_XXS = 16, QZ_IQ2_XS = 17, QZ_IQ3_XXS = 18, QZ_IQ4_NL = 20,
    QZ_IQ3_S = 21, QZ_IQ2_S = 22, QZ_BF16 = 30
};

/* src/gguf.rs:172-191.  Returns 0 for a type the oracle does not know
 * (the reference panics there). */
size_t qz_type_size(uint32_t ggml_type, size_t n_elems);
/* weights per block / bytes per block; 0 if unknown */
int qz_block_elems(uint32_t ggml_type);
int qz_block_bytes(uint32_t ggml_type);

/* src/dequant.rs:1329-1349 */
float qz_f16_to_f32(uint16_t bits);

/* Codebooks are data the caller supplies (the reference vendors them in
 * src/iq2_tables.rs / src/iq3_tables.rs; the tests take them from the gguf
 * package).  Layouts as the reference's tables: u64 = 8 int8 grid values
 * (little endian), u32 = 4 uint8 grid values. */
void qz_set_iq2xxs_grid(const uint64_t *g256);
void qz_set_iq2xs_grid(const uint64_t *g512);
void qz_set_iq2s_grid(const uint64_t *g1024);
void qz_set_iq3s_grid(const uint32_t *g512);
void qz_set_iq3xxs_grid(const uint32_t *g256);
/* KSIGNS_IQ2XS[128] is arithmetic (index | odd-parity bit); exposed for tests. */
const uint8_t *qz_ksigns(void);

/* src/dequant.rs:1239-1258.  0 = ok, -1 = unsupported type or missing grid. */
int qz_dequant(const uint8_t *data, uint32_t ggml_type, size_t n_elems, float *out);

/* src/dequant.rs:18-31: y[out_dim] = W[out_dim x in_dim] * x.  Rows are spread
 * over `threads` OpenMP threads (0 = all cores) the way rayon spreads them. */
int qz_gemv(const float *x, const uint8_t *data, uint32_t ggml_type,
            size_t in_dim, size_t out_dim, float *y, int threads);

/* src/dequant.rs:143-200: X[n, in_dim] * W^T -> out[n, out_dim], token-major. */
int qz_gemm(const float *x, const uint8_t *data, uint32_t ggml_type,
            size_t in_dim, size_t out_dim, size_t n, float *out, int threads);

/* sqrt(sum w^2) of every dequantized row (f64 accumulation), for the
 * tolerance 1e-3 * ||w_row|| * ||x||. */
int qz_row_norms(const uint8_t *data, uint32_t ggml_type,
                 size_t in_dim, size_t out_dim, double *norms, int threads);

/* y in f64 from the dequantized weights (information only). */
int qz_gemv_f64(const float *x, const uint8_t *data, uint32_t ggml_type,
                size_t in_dim, size_t out_dim, double *y, int threads);

int qz_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
