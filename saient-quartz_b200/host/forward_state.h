/*
 * Host side of the decode step, above the C ABI: a C++ restatement of the reference's
 * GpuBuf / GpuWeights / GpuForwardState (src/cuda.rs:59-90, 154-236, 301-851), written in C++
 * because the reference's own host language (Rust) has no toolchain in this environment.  It calls
 * nothing but the extern "C" surface of include/quartz_b200.h -- the same calls, in the same
 * order, that forward_gpu_step makes -- so it is what the Rust host would do after relinking.
 *
 * Two step functions:
 *   qh_forward_step        the reference sequence, call for call (src/cuda.rs:507-851)
 *   qh_forward_step_fused  the same arithmetic through the fused entry points, recorded ONCE per model as
 *                          a CUDA graph and replayed for every step: token id and position are two
 *                          device words (cuda_step_set) that the recorded kernels read
 *
 * The C interface below exists so that tests and the benchmark can drive it through ctypes.
 */
#ifndef QUARTZ_HOST_FORWARD_STATE_H
#define QUARTZ_HOST_FORWARD_STATE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* the fields of the reference's Config (src/main.rs:75-95) that the GPU forward uses */
typedef struct qh_config {
    int vocab_size, embed_dim, n_heads, n_kv_heads, n_layers, ffn_dim, head_dim;
    int n_experts, n_experts_used, moe_renorm, clamped_swiglu, swa_window, rope_neox;
    int yarn_orig_ctx, max_seq;
    float rope_theta, yarn_scale;
} qh_config;

enum qh_role {
    QH_EMBED = 0, QH_LM_HEAD, QH_FINAL_NORM,
    QH_Q, QH_K, QH_V, QH_O, QH_GATE, QH_UP, QH_DOWN,           /* quantized, per layer */
    QH_ATTN_NORM, QH_FFN_NORM, QH_Q_NORM, QH_K_NORM,           /* f32, per layer */
    QH_Q_BIAS, QH_K_BIAS, QH_V_BIAS, QH_O_BIAS, QH_SINKS,      /* f32, per layer, optional */
    QH_MOE_GATE, QH_MOE_UP, QH_MOE_DOWN,                       /* quantized 3-D expert tensors */
    QH_ROUTER_W, QH_ROUTER_B,                                  /* f32 */
    QH_MOE_GATE_BIAS, QH_MOE_UP_BIAS, QH_MOE_DOWN_BIAS
};

typedef struct qh_model qh_model;

qh_model *qh_create(const qh_config *cfg);
/* Build a model from a GGUF file: configuration from the metadata as the reference derives it
 * (Config::from_gguf, src/main.rs:96-215: "<arch>." keys with their fallbacks and defaults), tensors by
 * the names of src/main.rs:357-414 ("token_embd.weight", "output.weight" or tied, "blk.N.attn_q.weight",
 * ..., expert tensors "blk.N.ffn_*_exps.weight").  max_seq <= 0 takes the file's context length (capped at
 * 8192).  Norms, biases, sinks and router weights must be F32 in the file.  NULL on failure
 * (qh_load_error says why); cfg_out (optional) receives the derived configuration. */
qh_model *qh_load_gguf(const char *path, int max_seq, int repack, qh_config *cfg_out);
const char *qh_load_error(void);
void qh_destroy(qh_model *m);
/* upload one tensor (raw GGUF bytes, or f32 for norms/biases/router); repack=1 calls the repack hook */
int qh_set_tensor(qh_model *m, int role, int layer, uint32_t ggml_type, const void *host, size_t bytes, int repack);
/* allocate scratch + KV cache, default zero biases / no sinks (src/cuda.rs:361-492) */
int qh_finalize(qh_model *m);
/* write n_pos rows of K and V (f32 [n_pos x kv_dim]) into layer's caches (benchmark pre-fill) */
int qh_set_kv(qh_model *m, int layer, const float *k, const float *v, int n_pos);
/* read n_pos rows of K and V of a layer's caches back, starting at row pos0 */
int qh_get_kv(qh_model *m, int layer, float *k, float *v, int pos0, int n_pos);
/* returns 0 on success; logits_host (vocab floats) filled when need_logits */
int qh_forward_step(qh_model *m, int token, int pos, int need_logits, float *logits_host);
int qh_forward_step_fused(qh_model *m, int token, int pos, int need_logits, float *logits_host);
/* as fused, with output projection -> gate/up -> down -> next q/k/v of every layer as one persistent kernel */
int qh_forward_step_chained(qh_model *m, int token, int pos, int need_logits, float *logits_host);
/* Batched prefill: the n tokens of a prompt at positions pos0 .. pos0+n-1 in one pass (tensor-core GEMMs over all
 * tokens, batched RoPE / KV append / causal attention) instead of n decode steps; the reference's GPU prefill is
 * token by token (src/main.rs:1410-1416), its batched prefill CPU-only (src/main.rs:1157-1341).  Fills the caches;
 * logits_host (may be NULL) receives the LAST token's logits.  Models with QK-norm or projection biases run token
 * by token through the decode step.  0 on success. */
int qh_prefill(qh_model *m, const int *tokens, int n, int pos0, float *logits_host);
/* device-only variants for timing: no copies, the result stays in the device logits buffer; fused: 0 reference
 * sequence, 1 fused, 2 chained */
int qh_step_device(qh_model *m, int token, int pos, int fused);
int qh_read_hidden(qh_model *m, float *host);   /* d_hidden, for layer-level tests */
long long qh_launches_last_step(qh_model *m);    /* kernel launches issued by the last step (graph nodes if fused) */
/* 1: MoE layers route on the host as the reference does (router logits copied back, top-k on the CPU, one
 * synchronisation per layer, src/cuda.rs:673-701); 0 (default): router top-k and expert selection stay on the
 * device wherever the expert tensors are served by the streaming GEMV.  Also: QUARTZ_HOST_ROUTER=1. */
void qh_force_host_router(int on);
int qh_graphs_recorded(qh_model *m);             /* graph recordings made for this model so far (one per sequence kind) */

#ifdef __cplusplus
}
#endif
#endif
