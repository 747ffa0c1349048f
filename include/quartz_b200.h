/*
 * quartz_b200 -- C ABI of the B200 (sm_100a) quantized-weight GEMV/GEMM kernels.
 *
 * Part 1 is, symbol for symbol, the extern "C" block the reference's Rust host
 * binds (src/cuda.rs:6-55 in the reference project; implemented there by
 * src/cuda_kernels.cu:1025-1293).  A build of the reference links against this
 * library instead of its own libkernels.a without touching a call site.
 * Part 2 is additive: entry points the reference does not have.
 *
 * Conventions (as in the reference): every pointer is a device pointer unless
 * the parameter is named `host` or it is the host side of cuda_h2d / cuda_d2h;
 * dims are int; all work is issued on one stream (the legacy default stream
 * unless quartz_set_stream changed it); no function returns an error -- failures
 * are recorded in a sticky status readable with quartz_last_error().  The
 * library is single-caller: calls must not overlap from several host threads.
 */
#ifndef QUARTZ_B200_H
#define QUARTZ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ======================= Part 1: the reference's call surface ======================= */

/* src/cuda.rs:7-8, src/cuda_kernels.cu:1046-1079.  y[out_dim] = W[out_dim x in_dim] * x.
 * ggml_type ids as in src/gguf.rs:172-188, plus 2 (Q4_0), 3 (Q4_1), 18 (IQ3_XXS).
 * Unknown type: y is zero-filled, a line goes to stderr (reference behaviour) and
 * the sticky status becomes QZ_ERR_UNSUPPORTED_TYPE. */
void cuda_gemv(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, float *d_y, int in_dim, int out_dim);

/* src/cuda.rs:9-13, src/cuda_kernels.cu:1027-1041: upload the IQ codebooks (host pointers). */
void cuda_set_iq3s_grid(const uint32_t *host);   /* 512 x u32 */
void cuda_set_iq2s_grid(const uint64_t *host);   /* 1024 x u64 */
void cuda_set_iq2xxs_grid(const uint64_t *host); /* 256 x u64 */
void cuda_set_iq2xs_grid(const uint64_t *host);  /* 512 x u64 */
void cuda_set_ksigns(const uint8_t *host);       /* 128 bytes */

/* src/cuda.rs:14-19, src/cuda_kernels.cu:1042-1044, 1109-1125 */
void cuda_mem_info(size_t *free_b, size_t *total_b);
void *cuda_alloc(size_t bytes);          /* NULL on failure */
void cuda_drop(void *ptr);
void cuda_h2d(void *dst, const void *src, size_t bytes);   /* synchronous */
void cuda_d2h(void *dst, const void *src, size_t bytes);   /* synchronous */
void cuda_sync(void);

/* src/cuda.rs:20-37, src/cuda_kernels.cu:1129-1186 */
void cuda_vec_add(float *dst, const float *src, int n);
void cuda_vec_scale_add(float *dst, const float *src, float scale, int n);
void cuda_vec_zero(float *dst, int n);
void cuda_rms_norm(float *out, const float *x, const float *w, int n);
void cuda_rope_yarn(float *x, int n_heads, int head_dim, int pos, float theta, float yarn_scale, int yarn_orig_ctx,
                    int neox);
void cuda_kv_append(float *k_cache, float *v_cache, const float *k, const float *v, int pos, int kv_dim);
void cuda_attn_score(float *scores, const float *q, const float *k_cache, int seq_len, int head_dim, int kv_dim,
                     int kv_head_off, float scale);
void cuda_softmax_sink(float *x, int n, float sink);
void cuda_attn_values(float *out, const float *scores, const float *v_cache, int seq_len, int head_dim, int kv_dim,
                      int kv_head_off);
void cuda_swiglu(float *out, const float *gate, const float *up, int n);
void cuda_swiglu_oai(float *out, const float *gate, const float *up, int n);
/* The reference handles types 7, 20, 30 only; here every supported type works. */
void cuda_embed_lookup(float *out, const uint8_t *data, uint32_t ggml_type, int token, int embed_dim);

/* src/cuda.rs:39-45, src/cuda_kernels.cu:1085-1107: up to four (weights, x, y) GEMVs of one
 * shape in one call; slots >= n_act are ignored.  One launch for every streaming format
 * (the reference batches Q5_1 only). */
void cuda_gemv_moe4(uint32_t ggml_type, const uint8_t *w0, const uint8_t *w1, const uint8_t *w2, const uint8_t *w3,
                    const float *xi0, const float *xi1, const float *xi2, const float *xi3, float *o0, float *o1,
                    float *o2, float *o3, int n_act, int in_dim, int out_dim);

/* src/cuda.rs:47-54, src/cuda_kernels.cu:1267-1291 */
void cuda_attn_score_all(float *scores, const float *q, const float *k_cache, int n_heads, int n_kv_heads,
                         int seq_len, int head_dim, int kv_dim, int max_seq, float scale);
void cuda_softmax_sink_all(float *scores, int n_heads, int seq_len, int max_seq, const float *sinks);
void cuda_attn_values_all(float *out, const float *scores, const float *v_cache, int n_heads, int n_kv_heads,
                          int seq_len, int head_dim, int kv_dim, int max_seq);

/* ======================= Part 2: additions ======================= */

/* Sticky status (0 = ok; codes below).  The reference reports nothing
 * (src/cuda_kernels.cu:1109-1125 checks no CUDA call). */
enum {
    QZ_OK = 0, QZ_ERR_UNSUPPORTED_TYPE = 1, QZ_ERR_BAD_SHAPE = 2, QZ_ERR_CUDA = 3, QZ_ERR_MISSING_TABLE = 4,
    QZ_ERR_TOO_LARGE = 5, QZ_ERR_NOT_REPACKED = 6, QZ_ERR_TIMEOUT = 7
};
int quartz_last_error(void);
const char *quartz_error_string(void);
void quartz_clear_error(void);

/* All later launches and copies go to this cudaStream_t (NULL = legacy default stream,
 * the reference's behaviour, src/cuda_kernels.cu launches with <<<g,b>>> only). */
void quartz_set_stream(void *cuda_stream);

/* Number of kernels this library has launched (or recorded into a graph) so far. */
long long quartz_launch_count(void);

/* Which streaming GEMV serves the formats that have one: 0 = TMA-staged shared-memory ring
 * (default), 1 = register-streaming 128-bit loads.  For A/B measurements; both run the same
 * per-format integer dot products on the same converted activations and differ only in the
 * order in which a row's partial sums are added.  The environment variable
 * QUARTZ_GEMV_IMPL=ldg selects 1 at start-up. */
void quartz_set_gemv_impl(int impl);

/* Hint for the NEXT streaming GEMV launch of this library (cuda_gemv, cuda_gemv_q, cuda_gemv_rmsnorm, ...): once
 * that kernel's producer lanes have issued their own weight stream they also pull [d_ptr, d_ptr + bytes) -- the
 * weights of the operation that will FOLLOW it -- into the L2 cache, so that HBM keeps working while the kernel
 * drains, exits and its successor starts, and the successor's first tiles come from L2.  Up to four ranges per
 * launch (call it once per range), each capped at 24 MB (environment variable QUARTZ_PREFETCH_MB; 0 = off).
 * Purely a performance hint: results are unaffected, a launch that is not the TMA-staged kernel ignores it. */
void quartz_prefetch_next(const void *d_ptr, size_t bytes);

/* The IQ3_XXS codebook (256 x u32); the reference has no IQ3_XXS. */
void cuda_set_iq3xxs_grid(const uint32_t *host);

/* One-time, in-place, size-preserving repack of n_mats consecutive [out_dim x in_dim]
 * matrices from the raw GGUF block layout (src/gguf.rs:118-123) into the plane layout
 * the streaming kernels read with aligned 128-bit loads.  To be called once after the
 * upload (src/cuda.rs:170-172, 202-204 are the places).  The byte range is remembered:
 * cuda_gemv / cuda_gemv_moe4 / cuda_gemm / cuda_dequant on any pointer inside it (e.g.
 * an expert slice, src/cuda.rs:250-257) then read the new layout.  Returns 1 if the
 * bytes were rearranged, 0 if this format/shape is served from the raw layout (nothing
 * changed; not an error).  Unregistered pointers always mean raw layout. */
int cuda_repack_weights(uint32_t ggml_type, void *d_data, int in_dim, int out_dim, int n_mats);
/* Inverse of the above on a registered range (restores the raw bytes); 1 if undone. */
int cuda_unpack_weights(void *d_data);

/* Dequantize n_rows rows of in_dim weights to f32, bit-identical to the reference's
 * CPU dequant() (src/dequant.rs:1239-1258), from either layout. */
void cuda_dequant(uint32_t ggml_type, const uint8_t *d_data, float *d_out, int in_dim, long long n_rows);

/* No counterpart in the reference.  cuda_gemv for callers that must not allocate device memory
 * when they call it -- code running inside a stream capture, hosts with a fixed memory plan, or
 * processes whose allocator owns the whole device.  Same arguments, same results as cuda_gemv,
 * but the converted-activation scratch is a 78,080-byte array built into the library (resident
 * on every GPU that loads it) instead of a buffer obtained with cudaMalloc at first use; the
 * call makes no cudaMalloc/cudaFree and uses no allocating library routine.
 *   - limit: in_dim <= 32768; larger sizes set QZ_ERR_TOO_LARGE and leave d_y untouched.
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress), and the
 *     first call with an IQ2_XXS / IQ2_XS / IQ3_XXS matrix uploads the default sign table when the
 *     host has not called cuda_set_ksigns (a synchronous copy into a library table, no allocation);
 *     make those first calls before starting any stream capture on that device.
 *   - it never carries a fused exchange wait: a pending quartz_mgpu_fuse_next_wait() runs as a wait
 *     kernel of its own if the library's status word exists already (any earlier quartz_mgpu_wait
 *     or streaming GEMV created it) and is refused with QZ_ERR_BAD_SHAPE otherwise, because
 *     creating that word takes a cudaMalloc.
 *   - every block format that has a streaming kernel uses the built-in scratch; shapes and
 *     pointers the streaming kernel does not take (in_dim not a multiple of 64, unaligned rows)
 *     run the any-shape kernel, which needs no scratch at all.
 *   - all calls share the one array: two calls whose kernels can overlap on the GPU (different
 *     streams) race on it; calls on one stream are safe.  Nothing in it needs clearing between
 *     calls -- each call rewrites what it reads. */
void cuda_gemv_noalloc(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, float *d_y, int in_dim,
                       int out_dim);

/* ---- fused decode-step entry points (no counterparts in the reference, which issues these
 * steps as separate launches, src/cuda.rs:548-823).  The streaming GEMVs consume activations
 * in a 16-bit block-fixed-point form held in library scratch "slots" 0..3; these producers
 * write a slot directly, so the separate conversion launch of cuda_gemv disappears. ---- */
/* convert d_x[0..n) into slot */
void cuda_quantize_x(const float *d_x, int n, int slot);
/* cuda_rms_norm whose result lands in `slot` (and in out_f32 when not NULL) */
void cuda_rms_norm_q(const float *x, const float *w, int n, int slot, float *out_f32);
/* cuda_swiglu (oai = 0) / cuda_swiglu_oai (oai = 1) whose result lands in `slot` */
void cuda_swiglu_q(const float *gate, const float *up, int n, int slot, int oai);
/* 1 if (type, in_dim, pointer/layout) is served by the streaming kernel, else 0 */
int cuda_gemv_q_supported(uint32_t ggml_type, const uint8_t *d_data, int in_dim);
/* n_mats <= 8 same-shape GEMVs in ONE launch: d_y[i] (+)= W[i] * slot[slots[i]].  d_w, slots, d_y
 * are HOST arrays (of device pointers / slot numbers).  accumulate = 1 adds into d_y (residual
 * epilogue).  Generalises cuda_gemv_moe4; fused q/k/v is six 1024-row slices of three tensors. */
void cuda_gemv_q(uint32_t ggml_type, int n_mats, const uint8_t *const *d_w, const int *slots, float *const *d_y,
                 int in_dim, int out_dim, int accumulate);
/* cuda_rope_yarn on q and k + cuda_kv_append (src/cuda.rs:601-613) in one launch */
void cuda_rope_kv(float *q, float *k, const float *v, float *k_cache, float *v_cache, int n_heads, int n_kv_heads,
                  int head_dim, int pos, float theta, float yarn_scale, int yarn_orig_ctx, int neox);
/* cuda_attn_score_all + cuda_softmax_sink_all + cuda_attn_values_all (src/cuda.rs:627-645) as a
 * split-KV decode attention (K and V read once for all query heads of a kv head); sinks may be
 * NULL; out_slot >= 0 also writes the result's activation form for the output projection. */
void cuda_attn_decode(float *out, const float *q, const float *k_cache, const float *v_cache, int n_heads,
                      int n_kv_heads, int seq_len, int head_dim, int kv_dim, float scale, const float *sinks,
                      int out_slot);

/* ---- A decode step whose position and token id live in DEVICE memory, so that ONE recorded graph serves
 * every step of a generation loop (the reference passes `token` and `pos` to forward_gpu_step per call,
 * src/cuda.rs:507-851, and bakes them into its launches).  d_step points at two ints on the device:
 * d_step[0] = token id, d_step[1] = position.
 *   cuda_step_set          enqueue the update of the two words (a one-thread kernel with the values as
 *                          arguments: the host may call it again at once, nothing is read from host memory
 *                          later).  It runs on the stream recorded graphs replay on, so "set, replay, set,
 *                          replay ..." needs no synchronisation.
 *   cuda_embed_lookup_dev  cuda_embed_lookup of row d_step[0]
 *   cuda_attn_step         the whole attention block of the step in ONE launch whose grid does not depend on
 *                          the position: RoPE on q and k, append of k and v at the position, attention of all
 *                          heads over cache positions [k_start, pos], merge, and with out_slot >= 0 the
 *                          activation form of the result (cuda_rope_yarn x2 + cuda_kv_append +
 *                          cuda_attn_score_all + cuda_softmax_sink_all + cuda_attn_values_all,
 *                          src/cuda.rs:601-645).  q / k_new / v_new are the projections BEFORE RoPE and are
 *                          left untouched; caches are [max_seq][n_kv_heads*head_dim].  The position comes from
 *                          d_step[1] when d_step is not NULL, else from `pos`; positions >= max_seq are
 *                          clamped to max_seq-1 (src/cuda.rs:517-520).  window > 0: k_start = max(0, pos+1-window)
 *                          (the sliding-window layers of src/main.rs:231-237), else 0.  sinks may be NULL.
 *                          One thread-block cluster per kv head; its CTAs split the context and merge their
 *                          partial results through distributed shared memory.  head_dim a multiple of 32 up to
 *                          128, at most 16 query heads per kv head (cuda_attn_step_supported tells). */
void cuda_step_set(int *d_step, int token, int pos);
/* Registers a RoPE parameter set for a pair of step words: from then on cuda_step_set(d_step, ...) also writes the
 * (cos, sin) of every rotation pair at the new position, in the same launch as the words, and cuda_attn_step calls
 * with this d_step and these parameters read that table (after checking that it was written for the position in
 * d_step[1]) instead of computing sin / cos in every CTA of every layer; the values are the same either way.  At
 * most 4 sets per d_step.  Allocates: call it when the model is built, outside a graph recording.  No counterpart
 * in the reference (cuda_rope_yarn computes sin / cos per call, src/cuda_kernels.cu:588-620). */
void cuda_step_rope_table(int *d_step, int head_dim, float theta, float yarn_scale, int yarn_orig_ctx);
void cuda_embed_lookup_dev(float *out, const uint8_t *data, uint32_t ggml_type, const int *d_step, int embed_dim);
int cuda_attn_step_supported(int n_heads, int n_kv_heads, int head_dim);
void cuda_attn_step(float *out, const float *q, const float *k_new, const float *v_new, float *k_cache, float *v_cache,
                    int n_heads, int n_kv_heads, int head_dim, int max_seq, const int *d_step, int pos, int window,
                    float scale, const float *sinks, float theta, float yarn_scale, int yarn_orig_ctx, int neox,
                    int out_slot);

/* ---- Batched (prompt) forms of the per-token helpers, for n tokens at consecutive positions pos0 .. pos0+n-1; with
 * cuda_gemm for the projections they make up a batched GPU prefill (the reference's GPU prefill runs the decode step
 * token by token, src/main.rs:1410-1416; its batched prefill is CPU-only, src/main.rs:1157-1341).
 *   cuda_embed_lookup_rows  out[r, :] = dequantized row d_tokens[r] of the embedding table, r < n
 *   cuda_rms_norm_rows      cuda_rms_norm of every row of x [n_rows, n]; out may alias x
 *   cuda_rope_kv_rows       cuda_rope_kv for token t at position pos0 + t: q [n, n_heads*head_dim] and k [n, kv_dim]
 *                           rotated in place, k / v rows appended to the caches
 *   cuda_attn_prompt        causal attention of the n tokens: token t attends to cache positions [k_start, pos0 + t]
 *                           (window as in cuda_attn_step); q is already rotated and the caches already hold the n
 *                           new rows (cuda_rope_kv_rows).  out [n, n_heads*head_dim].  Same head-geometry limits
 *                           as cuda_attn_step.  One CTA per (kv head, tile of up to 16 tokens): the tile's query
 *                           rows share every staged K / V row. */
void cuda_embed_lookup_rows(float *out, const uint8_t *data, uint32_t ggml_type, const int *d_tokens, int n, int embed_dim);
void cuda_rms_norm_rows(float *out, const float *x, const float *w, int n_rows, int n);
void cuda_rope_kv_rows(float *q, float *k, const float *v, float *k_cache, float *v_cache, int n_tok, int n_heads,
                       int n_kv_heads, int head_dim, int pos0, float theta, float yarn_scale, int yarn_orig_ctx, int neox);
void cuda_attn_prompt(float *out, const float *q, const float *k_cache, const float *v_cache, int n_tok, int n_heads,
                      int n_kv_heads, int head_dim, int max_seq, int pos0, int window, float scale, const float *sinks);

/* A chain of dependent GEMVs as ONE persistent kernel (one CTA per SM): op k+1's activation vector is
 * computed from op k's outputs after a grid-wide barrier inside the kernel, while the weight rows of
 * op k+1 are already streaming.  In the reference every link is a kernel boundary (src/cuda.rs:548-823:
 * cuda_gemv, cuda_vec_add, cuda_rms_norm, cuda_swiglu one after the other).  Each op is a cuda_gemv_q-style
 * multi-matrix GEMV  y_i (+)= W_i * f(a, b)  with f = RMSNorm of a with weights b (src_mode 1, eps 1e-5),
 * SwiGLU of gate a and up b (src_mode 2; oai = clamped variant) or a itself (src_mode 3).  Takes Q4_K,
 * Q6_K and Q8_0 matrices that cuda_gemv_q_supported accepts, 2048 <= in_dim <= 16384, up to 8 ops;
 * anything else runs the same GEMVs one launch at a time (cuda_gemv_chain_supported tells which).
 * The grid barrier's poll is bounded (~0.5 s, QZ_ERR_TIMEOUT).  First call allocates three control words:
 * make it outside a graph recording. */
typedef struct qz_chain_op {
    uint32_t ggml_type;
    int n_mats;
    const uint8_t *const *d_w;
    float *const *d_y;
    int in_dim, out_dim, accumulate;
    int src_mode;
    const float *d_a, *d_b;
    int oai;
} qz_chain_op;
int cuda_gemv_chain_supported(int n_ops, const qz_chain_op *ops);
void cuda_gemv_chain(int n_ops, const qz_chain_op *ops);
/* The same kernel for GEMVs that do NOT depend on one another (no op reads what another writes): no
 * barrier between them, the weight stream runs through all of them without a break.  The
 * generalisation of cuda_gemv_moe4 (src/cuda.rs:39-45) to matrices of different shapes and types.
 * Plain-f32 activation vectors (src_mode 3) are converted by ONE small kernel ahead of the persistent one, into a
 * library scratch that is allocated at the first call (make that call outside a graph recording); the ops may
 * be run in any order inside the kernel.  Ops the persistent kernel does not take (cuda_gemv_chain_supported
 * tells) make the call run GEMV by GEMV with the same results. */
void cuda_gemv_batch(int n_ops, const qz_chain_op *ops);

/* The whole attention block of one decode step as ONE launch (two when the context spans more than 8
 * splits of 32 positions: the merge then gets a launch of its own): RoPE on q and k, append of k and v to the
 * caches at `pos`, attention of all heads over cache positions [k_start, pos], merge of the splits
 * (cuda_rope_yarn x2 + cuda_kv_append + cuda_attn_score_all + cuda_softmax_sink_all +
 * cuda_attn_values_all, src/cuda.rs:601-645).  q [n_heads*head_dim], k_new / v_new
 * [n_kv_heads*head_dim] are the projections BEFORE RoPE and are left untouched; the caches are
 * [max_seq][n_kv_heads*head_dim].  sinks may be NULL; out_slot >= 0 also writes the result's activation
 * form for the output projection.  head_dim a multiple of 32 up to 128, at most 64 kv heads. */
void cuda_attn_block(float *out, const float *q, const float *k_new, const float *v_new, float *k_cache, float *v_cache,
                     int n_heads, int n_kv_heads, int head_dim, int pos, int k_start, float scale, const float *sinks,
                     float theta, float yarn_scale, int yarn_orig_ctx, int neox, int out_slot);

/* cuda_gemv_q whose activation vector is computed by the GEMV kernel itself, in its prologue, while its
 * weight pipeline fills: y_i (+)= W_i * rmsnorm(x, norm_w)  (cuda_rms_norm + cuda_gemv, src/cuda.rs:556-597
 * and :760-775) and y_i (+)= W_i * swiglu(gate, up)  (cuda_swiglu / cuda_swiglu_oai + cuda_gemv,
 * src/cuda.rs:777-800).  eps is 1e-5 as in the reference kernel.  Same type/shape/layout conditions as
 * cuda_gemv_q (cuda_gemv_q_supported); in_dim floats of d_x / d_norm_w / d_gate / d_up, 16-byte aligned
 * and in_dim <= 8192 for the fused form (otherwise the two-launch form runs and uses the caller's scratch
 * slot 3: converting a long vector once is cheaper than converting it in every CTA). */
void cuda_gemv_rmsnorm(uint32_t ggml_type, int n_mats, const uint8_t *const *d_w, float *const *d_y, const float *d_x,
                       const float *d_norm_w, int in_dim, int out_dim, int accumulate);
void cuda_gemv_swiglu(uint32_t ggml_type, int n_mats, const uint8_t *const *d_w, float *const *d_y, const float *d_gate,
                      const float *d_up, int oai, int in_dim, int out_dim, int accumulate);

/* Asynchronous copies between page-locked host memory and the device, on the library's stream (the
 * reference's cuda_h2d / cuda_d2h, src/cuda_kernels.cu:1117-1123, are synchronous cudaMemcpy).  They may
 * be recorded into a graph together with the kernels, so that a whole step (inputs in, kernels,
 * results out) is one graph launch; the host reads the results after cuda_sync().  cuda_host_alloc
 * returns page-locked memory (NULL on failure). */
void cuda_h2d_async(void *d_dst, const void *h_src_pinned, size_t bytes);
void cuda_d2h_async(void *h_dst_pinned, const void *d_src, size_t bytes);
void *cuda_host_alloc(size_t bytes);
void cuda_host_free(void *p);

/* CUDA-graph helpers (no counterpart in the reference, which launches ~670 kernels per token one
 * by one, src/cuda.rs:548-843).  Between begin and end every call of this library is recorded
 * instead of executed; cuda_h2d / cuda_d2h / cuda_sync must stay outside (cuda_h2d_async and
 * cuda_d2h_async may be recorded), and every scratch buffer must
 * already exist (run the sequence once eagerly first).  end returns an executable graph (NULL on
 * failure); launch replays it, ordered with the default stream. */
/* 1 (default): kernels recorded into a graph are launched as programmatic dependents, so each
 * may begin (and a GEMV may start streaming its weights) while its predecessor drains; 0: plain
 * serial edges.  Results are identical. */
void quartz_set_pdl(int on);
int quartz_graph_begin(void);
void *quartz_graph_end(void);
void quartz_graph_launch(void *graph_exec);
void quartz_graph_destroy(void *graph_exec);

/* Batched form: Y[m, out_dim] = X[m, in_dim] * W^T, token-major like the reference's CPU
 * gemm() (src/dequant.rs:143-200).  The reference has no GPU counterpart. */
void cuda_gemm(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, float *d_y, int m, int in_dim,
               int out_dim);
/* The same with bf16 activations (raw 16-bit patterns, [m, in_dim]); in_dim a multiple of 64, pointers
 * 16-byte aligned.  Equal to cuda_gemm on the same values widened to f32 (up to the summation order of
 * output tiles that two CTAs share). */
void cuda_gemm_bf16(uint32_t ggml_type, const uint8_t *d_data, const uint16_t *d_x_bf16, float *d_y, int m, int in_dim,
                    int out_dim);

/* Batched mixture-of-experts FFN for m tokens:
 *   out[t] = sum over the top_k experts e of token t of  w(t,e) * down_e( swiglu(gate_e x_t, up_e x_t) )
 * the batched form of the reference's per-token MoE branch (src/main.rs:941-990; on the GPU every
 * expert GEMV of every token is its own launch, src/cuda.rs:673-800).  d_gate / d_up / d_down point at
 * the stacked expert tensors ([in_dim, out_dim, n_experts]: expert e at byte offset e * size(one
 * matrix), src/main.rs:941-950, src/cuda.rs:250-257); raw or repacked (cuda_repack_weights with
 * n_mats = n_experts).  d_x is [m, embed_dim], d_out [m, embed_dim], both f32 on the device.  The routing
 * lists hold m * top_k entries, token-major, the weights already normalised.
 *   cuda_moe_ffn       routing lists in HOST memory (the reference routes on the host, src/cuda.rs:673-701)
 *   cuda_moe_ffn_dev   routing lists in DEVICE memory (e.g. written by cuda_router_topk): no host involvement
 * Both group the assignments by expert on the device and run ONE tensor-core launch for gate and up of all
 * experts and one for down (tiles of every expert in one persistent grid), the SwiGLU between them and the
 * weighted sum of a token's experts in the order of its list; nothing synchronises with the host.  Shapes the
 * grouped kernel does not take (in_dim not a multiple of 64, unaligned rows, more than 256 experts) run
 * expert by expert with the assignments grouped on the host.  oai = 1 selects the clamped SwiGLU
 * (cuda_swiglu_oai).  Output tiles that two CTAs share are summed atomically (summation order of those
 * elements is not fixed). */
void cuda_moe_ffn(uint32_t type_gate_up, uint32_t type_down, const uint8_t *d_gate, const uint8_t *d_up,
                  const uint8_t *d_down, const float *d_x, float *d_out, int m, int embed_dim, int ffn_dim, int n_experts,
                  int top_k, const int *h_expert_ids, const float *h_expert_w, int oai);
void cuda_moe_ffn_dev(uint32_t type_gate_up, uint32_t type_down, const uint8_t *d_gate, const uint8_t *d_up,
                      const uint8_t *d_down, const float *d_x, float *d_out, int m, int embed_dim, int ffn_dim, int n_experts,
                      int top_k, const int *d_expert_ids, const float *d_expert_w, int oai);
/* The router's top-k on the device (the reference copies the logits to the host, synchronises and sorts
 * there, src/cuda.rs:673-701): for each of m rows of d_logits [m, n_experts] (+ d_bias [n_experts] when not
 * NULL) the top_k largest entries, ties to the lower index, into d_ids [m, top_k], and their weights into
 * d_w: renorm = 1 softmax over the selected logits, 0 softmax over all experts (src/main.rs:979-986).
 * n_experts <= 256, top_k <= 8. */
void cuda_router_topk(const float *d_logits, const float *d_bias, int m, int n_experts, int top_k, int renorm, int *d_ids,
                      float *d_w);

/* Batch-1 (decode) MoE with the experts chosen on the DEVICE, so that a step needs no device-to-host copy and
 * no synchronisation per layer (the reference reads the router logits back and sorts on the host,
 * src/cuda.rs:673-701, then passes expert pointers computed on the host, :714-794):
 *   cuda_gemv_experts        n_act <= 4 GEMVs in one launch; matrix k is the expert slice d_base + d_ids[k] *
 *                            expert_bytes of a stacked expert tensor (cuda_gemv_moe4 with the pointer arithmetic of
 *                            gpu_expert_slice, src/cuda.rs:242-258, done by the kernel).  x_stride = 0: every expert
 *                            reads d_x; otherwise expert k reads d_x + k * x_stride floats.  Output k at d_y + k *
 *                            out_dim.  Streaming types / shapes only (cuda_gemv_q_supported on d_base).
 *   cuda_moe_decode_act      h[k] = swiglu(gate[k] + gate_bias[ids[k]], up[k] + up_bias[ids[k]]) (oai = clamped),
 *                            k < n_act, vectors of ffn_dim; biases [n_experts, ffn_dim] or NULL
 *   cuda_moe_decode_combine  acc (+)= sum_k d_w[k] * (down[k] + down_bias[ids[k]]), in the order of k */
void cuda_gemv_experts(uint32_t ggml_type, const uint8_t *d_base, size_t expert_bytes, const int *d_ids, int n_act,
                       const float *d_x, size_t x_stride, float *d_y, int in_dim, int out_dim);
void cuda_moe_decode_act(float *d_out, const float *d_gate, const float *d_up, const float *d_gate_bias,
                         const float *d_up_bias, const int *d_ids, int n_act, int ffn_dim, int oai);
void cuda_moe_decode_combine(float *d_acc, const float *d_down, const float *d_down_bias, const int *d_ids, const float *d_w,
                             int n_act, int embed_dim, int accumulate);

/* ---- Row-sharded layers over the GPUs of one box (one process per GPU).  No counterpart in the
 * reference, which drives a single device (src/cuda.rs:301-358).  A layer's weight rows are split
 * over the ranks (the loader uploads rows [n0, n1) of each matrix on rank r); every rank computes
 * its slice of y and stores it, from the GEMV's own epilogue, into the "window" of every rank over
 * NVLink peer mappings, so that after quartz_mgpu_wait() each rank holds the complete vector.
 *
 *   quartz_set_device       select the CUDA device of this process (before any other call)
 *   quartz_mgpu_init        allocate this rank's window (data_bytes of f32 payload) and write its
 *                           inter-process handle (quartz_mgpu_handle_bytes() bytes) to handle_out
 *   quartz_mgpu_attach      handles = the handles of all ranks, in rank order, concatenated (the
 *                           host exchanges them by whatever means it has); maps the peers' windows
 *   quartz_mgpu_data        device pointer to this rank's payload area (read complete vectors here)
 *   cuda_gemv_push          cuda_gemv whose out_dim rows land at payload[dst_off + j] of EVERY rank
 *   cuda_gemv_batch_push    several independent GEMVs and their exchange as one launch (below)
 *   cuda_push_rows          the same exchange for an [m x n_local] block already in device memory
 *                           (GEMM outputs): element (i, j) lands at payload[dst_off + i*dst_ld + j]
 *   quartz_mgpu_wait        enqueue the wait for ALL exchanges pushed so far: every rank's slices have
 *                           landed when it completes (bounded: QZ_ERR_TIMEOUT after ~0.5 s)
 *   quartz_mgpu_fuse_next_wait  the same wait, but carried out by the activation-conversion kernel of
 *                           the next cuda_gemv / cuda_gemv_push / cuda_quantize_x call instead of a
 *                           launch of its own; that GEMV's weight stream starts while it waits
 * Every rank must issue the same sequence of pushes.  A payload region may be overwritten only after a
 * wait that followed an exchange into another region.  The int functions return 0 on success, -1 on
 * failure (see quartz_last_error). */
/* The NCCL form of the exchange: an all-gather of every rank's f32 slice on a communicator the library creates.
 * NCCL is bound at run time (libnccl.so.2, or the file QUARTZ_NCCL_LIB names); without it these calls set
 * QZ_ERR_CUDA and the rest of the library is unaffected.
 *   quartz_nccl_unique_id   rank 0: write the communicator id (quartz_nccl_id_bytes() bytes) to id_out; the host
 *                           hands it to the other ranks by whatever means it has
 *   quartz_nccl_init        every rank, with rank 0's id (collective: returns when all ranks have joined)
 *   quartz_mgpu_allgather   d_recv[r * count_per_rank ..] = rank r's d_send[0 .. count_per_rank), on the library's
 *                           stream (ncclAllGather, in place when d_send == d_recv + rank * count_per_rank)
 *   quartz_nccl_shutdown    destroy the communicator */
size_t quartz_nccl_id_bytes(void);
int quartz_nccl_unique_id(void *id_out);
int quartz_nccl_init(int rank, int world, const void *id);
void quartz_mgpu_allgather(const float *d_send, float *d_recv, size_t count_per_rank);
void quartz_nccl_shutdown(void);
size_t quartz_mgpu_handle_bytes(void);
int quartz_set_device(int device);
int quartz_mgpu_init(int rank, int world, size_t data_bytes, void *handle_out);
int quartz_mgpu_attach(const void *handles);
float *quartz_mgpu_data(void);
void cuda_gemv_push(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, size_t dst_off, int in_dim,
                    int out_dim);
void cuda_push_rows(const float *d_src, int m, int n_local, size_t dst_off, size_t dst_ld);
/* cuda_gemv_batch (independent GEMVs of different shapes in ONE persistent launch) with the push epilogue: op k's
 * rows (one matrix per op, no accumulate) land at payload[dst_off[k] + j] of EVERY rank, and the whole launch
 * publishes ONE exchange -- a row-sharded step of several independent GEMVs costs one launch and one wait instead of
 * one launch, one conversion and one publish per GEMV.  Returns 1 if launched, 0 if the persistent kernel does not
 * take these ops (nothing was launched: use cuda_gemv_push per op). */
/* The batched (tensor-core) GEMM of a row shard with the exchange in its epilogue: this rank's [m x out_dim] block
 * (out_dim = the rows this rank owns) of Y = X W^T goes straight from the accumulators into EVERY rank's window,
 * token t / local row n at element dst_off + t * dst_ld + n, and the last CTA publishes the exchange; complete it
 * with quartz_mgpu_wait() like any other.  One kernel does the tensor-core tiles and the peer stores, so the
 * transfer of finished tiles overlaps the computation of the others.  d_x is [m, in_dim] f32, replicated on every
 * rank.  Returns 1 if launched, 0 if the tensor-core kernel does not take the shape (m = 1, in_dim not a multiple
 * of 64, misaligned pointers; nothing was launched: use cuda_gemm + cuda_push_rows).  No counterpart in the
 * reference (single GPU, no batched GPU path). */
int cuda_gemm_push(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, int m, int in_dim, int out_dim,
                   size_t dst_off, size_t dst_ld);
int cuda_gemv_batch_push(int n_ops, const qz_chain_op *ops, const size_t *dst_off);
/* A chain of DEPENDENT row-sharded GEMVs with the exchanges inside one persistent kernel per rank (a whole sharded
 * FFN: gate/up shards -> exchange -> SwiGLU -> down shard -> exchange, as one launch).  Op k's rows go to every
 * rank's window: matrix i of the op at element offset dst_off[k] + i * dst_stride[k] (+ row); dst_stride may be NULL
 * when every op has one matrix.  Between op k and op k+1 the kernel publishes the exchange and polls, bounded
 * (~0.5 s, QZ_ERR_TIMEOUT), until every rank has published as many exchanges; op k+1's activation source
 * (d_a / d_b, normally addresses inside quartz_mgpu_data()) is read after that.  The last op's exchange is published
 * at the kernel's end and completed by quartz_mgpu_wait() like any other.  Every rank must run the same chain; the
 * ranks must be on different GPUs (a kernel that waits for another rank's kernel never shares a GPU with it).
 * No counterpart in the reference (single GPU).  Returns 1 if launched, 0 if the persistent kernel does not take
 * these ops (nothing was launched: use cuda_gemv_push per op with a wait between them). */
int cuda_gemv_chain_push(int n_ops, const qz_chain_op *ops, const size_t *dst_off, const size_t *dst_stride);
void quartz_mgpu_wait(void);
void quartz_mgpu_fuse_next_wait(void);
/* The next cuda_gemv_batch_push / cuda_gemv_chain_push / cuda_gemm_push completes its own exchange: the thread that
 * publishes then waits (bounded, ~0.5 s, QZ_ERR_TIMEOUT) until every rank has published as many exchanges, so the
 * kernel's end is the exchange's end and no quartz_mgpu_wait() launch is needed after it.  Every rank must have
 * launched the same call (the ranks run on different GPUs). */
void quartz_mgpu_wait_in_next_push(void);
void quartz_mgpu_shutdown(void);

#ifdef __cplusplus
}
#endif
#endif
