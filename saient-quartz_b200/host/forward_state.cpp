// Host side of the decode step over the C ABI (see forward_state.h).
#include "forward_state.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <utility>
#include <vector>

#include "../../include/quartz_b200.h"

extern "C" long long quartz_launch_count(void);

namespace {

// src/gguf.rs:172-191 (+ the three extension ids); 0 = unknown
size_t ggml_type_size(uint32_t t, size_t n)
{
    switch (t) {
    case 0: return n * 4;
    case 1: case 30: return n * 2;
    case 2: return n / 32 * 18;
    case 3: return n / 32 * 20;
    case 6: return n / 32 * 22;
    case 7: return n / 32 * 24;
    case 8: return n / 32 * 34;
    case 20: return n / 32 * 18;
    case 10: return n / 256 * 84;
    case 12: return n / 256 * 144;
    case 13: return n / 256 * 176;
    case 14: return n / 256 * 210;
    case 16: return n / 256 * 66;
    case 17: return n / 256 * 74;
    case 18: return n / 256 * 98;
    case 21: return n / 256 * 110;
    case 22: return n / 256 * 82;
    default: return 0;
    }
}

// src/cuda.rs:59-90: owns one device allocation
struct GpuBuf {
    void *ptr = nullptr;
    size_t bytes = 0;
    uint32_t ggml_type = 0;
    GpuBuf() = default;
    GpuBuf(const GpuBuf &) = delete;
    GpuBuf &operator=(const GpuBuf &) = delete;
    GpuBuf(GpuBuf &&o) noexcept { *this = std::move(o); }
    GpuBuf &operator=(GpuBuf &&o) noexcept
    {
        drop();
        ptr = o.ptr; bytes = o.bytes; ggml_type = o.ggml_type;
        o.ptr = nullptr;
        return *this;
    }
    ~GpuBuf() { drop(); }
    void drop()
    {
        if (ptr) cuda_drop(ptr);
        ptr = nullptr;
    }
    bool upload(const void *data, size_t n)
    {
        drop();
        ptr = cuda_alloc(n ? n : 1);
        if (!ptr) return false;
        bytes = n;
        if (n) cuda_h2d(ptr, data, n);
        return true;
    }
    bool alloc_f32(size_t n)
    {
        drop();
        ptr = cuda_alloc(n ? n * 4 : 4);
        bytes = n * 4;
        return ptr != nullptr;
    }
    bool empty() const { return ptr == nullptr; }
    float *f() const { return (float *)ptr; }
    const uint8_t *u8() const { return (const uint8_t *)ptr; }
};

struct Layer {
    GpuBuf q, k, v, o, gate, up, down;
    GpuBuf attn_norm, ffn_norm, q_norm, k_norm;
    size_t q_norm_len = 0, k_norm_len = 0;
    GpuBuf q_bias, k_bias, v_bias, o_bias, sinks;
    bool has_qkv_bias = false;
    GpuBuf moe_gate, moe_up, moe_down, router_w, router_b_dev;
    std::vector<float> router_b;
    GpuBuf moe_gate_bias, moe_up_bias, moe_down_bias;
};

}  // namespace

struct qh_model {
    qh_config c;
    std::vector<Layer> L;
    GpuBuf embed, lm_head, final_norm;
    // scratch (src/cuda.rs:312-354)
    GpuBuf d_hidden, d_norm_out, d_q, d_k, d_v, d_attn_out, d_scores, d_gate, d_up, d_expert_out, d_expert_acc;
    GpuBuf d_gate_all, d_up_all, d_expert_out_all, d_down_all, d_router_logits, d_logits;
    std::vector<GpuBuf> kv_k, kv_v;
    bool finalized = false;
    long long last_launches = 0;
    int n_recorded = 0;        // graph recordings made so far
    // batched prefill scratch (grown on demand): token ids, hidden rows, normalised rows, q, k, v, attention out, gate, up
    GpuBuf p_tok, p_x, p_xn, p_q, p_k, p_v, p_att, p_g, p_u, p_ids, p_w;
    int p_cap = 0;
    GpuBuf d_moe_ids, d_moe_w; // experts of the current token and their weights, chosen on the device
    GpuBuf d_step;             // two device words {token, pos}: what the recorded step reads instead of arguments
    void *graphs[3] = {nullptr, nullptr, nullptr};   // one recorded step per sequence kind (1 fused, 2 chained)
    int q_d() const { return c.n_heads * c.head_dim; }
    int kv_d() const { return c.n_kv_heads * c.head_dim; }
};

extern "C" {

qh_model *qh_create(const qh_config *cfg)
{
    if (!cfg || cfg->n_layers <= 0 || cfg->embed_dim <= 0) return nullptr;
    qh_model *m = new qh_model();
    m->c = *cfg;
    m->L.resize(cfg->n_layers);
    return m;
}

void qh_destroy(qh_model *m)
{
    if (!m) return;
    for (void *g : m->graphs)
        if (g) quartz_graph_destroy(g);
    delete m;
}

int qh_set_tensor(qh_model *m, int role, int layer, uint32_t t, const void *host, size_t bytes, int repack)
{
    if (!m) return -1;
    const qh_config &c = m->c;
    GpuBuf *dst = nullptr;
    int K = 0, N = 0, mats = 1;
    const int d = c.embed_dim, fd = c.ffn_dim;
    if (role == QH_EMBED) { dst = &m->embed; K = d; N = c.vocab_size; }
    else if (role == QH_LM_HEAD) { dst = &m->lm_head; K = d; N = c.vocab_size; }
    else if (role == QH_FINAL_NORM) dst = &m->final_norm;
    else {
        if (layer < 0 || layer >= c.n_layers) return -2;
        Layer &l = m->L[layer];
        switch (role) {
        case QH_Q: dst = &l.q; K = d; N = m->q_d(); break;
        case QH_K: dst = &l.k; K = d; N = m->kv_d(); break;
        case QH_V: dst = &l.v; K = d; N = m->kv_d(); break;
        case QH_O: dst = &l.o; K = m->q_d(); N = d; break;
        case QH_GATE: dst = &l.gate; K = d; N = fd; break;
        case QH_UP: dst = &l.up; K = d; N = fd; break;
        case QH_DOWN: dst = &l.down; K = fd; N = d; break;
        case QH_ATTN_NORM: dst = &l.attn_norm; break;
        case QH_FFN_NORM: dst = &l.ffn_norm; break;
        case QH_Q_NORM: dst = &l.q_norm; l.q_norm_len = bytes / 4; break;
        case QH_K_NORM: dst = &l.k_norm; l.k_norm_len = bytes / 4; break;
        case QH_Q_BIAS: dst = &l.q_bias; l.has_qkv_bias = true; break;
        case QH_K_BIAS: dst = &l.k_bias; l.has_qkv_bias = true; break;
        case QH_V_BIAS: dst = &l.v_bias; l.has_qkv_bias = true; break;
        case QH_O_BIAS: dst = &l.o_bias; break;
        case QH_SINKS: dst = &l.sinks; break;
        case QH_MOE_GATE: dst = &l.moe_gate; K = d; N = fd; mats = c.n_experts; break;
        case QH_MOE_UP: dst = &l.moe_up; K = d; N = fd; mats = c.n_experts; break;
        case QH_MOE_DOWN: dst = &l.moe_down; K = fd; N = d; mats = c.n_experts; break;
        case QH_ROUTER_W: dst = &l.router_w; break;
        case QH_ROUTER_B:
            l.router_b.assign((const float *)host, (const float *)host + bytes / 4);
            return l.router_b_dev.upload(host, bytes) ? 0 : -5;   // the device-side router adds it on the device
        case QH_MOE_GATE_BIAS: dst = &l.moe_gate_bias; break;
        case QH_MOE_UP_BIAS: dst = &l.moe_up_bias; break;
        case QH_MOE_DOWN_BIAS: dst = &l.moe_down_bias; break;
        default: return -3;
        }
    }
    if (K > 0) {   // a quantized matrix: size must match the GGUF blob size (src/gguf.rs:172-191)
        if (ggml_type_size(t, (size_t)K * N * mats) != bytes) return -4;
    }
    if (!dst->upload(host, bytes)) return -5;   // cudaMalloc failed (src/cuda.rs:79)
    dst->ggml_type = t;
    // the one-line addition to upload_ti (src/cuda.rs:170-172): the embedding table stays raw
    if (K > 0 && repack && role != QH_EMBED) cuda_repack_weights(t, dst->ptr, K, N, mats);
    return 0;
}

int qh_finalize(qh_model *m)
{
    if (!m) return -1;
    const qh_config &c = m->c;
    const int d = c.embed_dim, q_d = m->q_d(), kv_d = m->kv_d(), fd = c.ffn_dim, nh = c.n_heads;
    const size_t mseq = c.max_seq;
    const size_t n_slots = (size_t)std::max(4, std::min(c.n_experts_used, 8));   // expert outputs kept side by side
    bool ok = m->d_hidden.alloc_f32(d) && m->d_norm_out.alloc_f32(d) && m->d_q.alloc_f32(q_d) &&
              m->d_k.alloc_f32(kv_d) && m->d_v.alloc_f32(kv_d) && m->d_attn_out.alloc_f32(q_d) &&
              m->d_scores.alloc_f32(nh * mseq) && m->d_gate.alloc_f32(fd) && m->d_up.alloc_f32(fd) &&
              m->d_expert_out.alloc_f32(fd) && m->d_expert_acc.alloc_f32(d) && m->d_gate_all.alloc_f32(n_slots * (size_t)fd) &&
              m->d_up_all.alloc_f32(n_slots * (size_t)fd) && m->d_expert_out_all.alloc_f32(n_slots * (size_t)fd) &&
              m->d_down_all.alloc_f32(n_slots * (size_t)d) && m->d_router_logits.alloc_f32(std::max(c.n_experts, 1)) &&
              m->d_logits.alloc_f32(c.vocab_size) && m->d_step.alloc_f32(4) && m->d_moe_ids.alloc_f32(16) &&
              m->d_moe_w.alloc_f32(16);
    if (!ok) return -2;
    // the (cos, sin) table of a step's position is written together with the step words
    cuda_step_rope_table((int *)m->d_step.ptr, c.head_dim, c.rope_theta, c.yarn_scale, c.yarn_orig_ctx);
    m->kv_k.resize(c.n_layers);
    m->kv_v.resize(c.n_layers);
    std::vector<float> zeros(std::max(q_d, kv_d), 0.f), no_sink(nh, -INFINITY);
    for (int l = 0; l < c.n_layers; l++) {
        if (!m->kv_k[l].alloc_f32(mseq * kv_d) || !m->kv_v[l].alloc_f32(mseq * kv_d)) return -3;
        Layer &L = m->L[l];
        // absent q/k/v biases are uploaded as zero vectors and added anyway (src/main.rs:366-368)
        if (L.q_bias.empty()) L.q_bias.upload(zeros.data(), (size_t)q_d * 4);
        if (L.k_bias.empty()) L.k_bias.upload(zeros.data(), (size_t)kv_d * 4);
        if (L.v_bias.empty()) L.v_bias.upload(zeros.data(), (size_t)kv_d * 4);
        if (L.sinks.empty()) L.sinks.upload(no_sink.data(), (size_t)nh * 4);   // src/cuda.rs:456-464
    }
    cuda_sync();
    m->finalized = true;
    return quartz_last_error() == 0 ? 0 : -4;
}

int qh_set_kv(qh_model *m, int layer, const float *k, const float *v, int n_pos)
{
    if (!m || !m->finalized || layer < 0 || layer >= m->c.n_layers || n_pos > m->c.max_seq) return -1;
    cuda_h2d(m->kv_k[layer].ptr, k, (size_t)n_pos * m->kv_d() * 4);
    cuda_h2d(m->kv_v[layer].ptr, v, (size_t)n_pos * m->kv_d() * 4);
    return 0;
}

int qh_get_kv(qh_model *m, int layer, float *k, float *v, int pos0, int n_pos)
{
    if (!m || !m->finalized || layer < 0 || layer >= m->c.n_layers || pos0 < 0 || n_pos < 0 || pos0 + n_pos > m->c.max_seq) return -1;
    const size_t off = (size_t)pos0 * m->kv_d() * 4, bytes = (size_t)n_pos * m->kv_d() * 4;
    cuda_d2h(k, (const uint8_t *)m->kv_k[layer].ptr + off, bytes);
    cuda_d2h(v, (const uint8_t *)m->kv_v[layer].ptr + off, bytes);
    cuda_sync();
    return 0;
}

static int attn_start(const qh_config &c, int layer, int pos)   // src/main.rs:231-237
{
    if (c.swa_window > 0 && layer % 2 == 0) return std::max(0, pos + 1 - c.swa_window);
    return 0;
}

static float attn_scale(const qh_config &c)   // src/cuda.rs:532-536
{
    float mscale2 = 1.f;
    if (c.yarn_scale > 1.f && c.yarn_orig_ctx > 0) {
        float ms = 1.f + 0.1f * logf(c.yarn_scale);
        mscale2 = ms * ms;
    }
    return (1.f / sqrtf((float)c.head_dim)) * mscale2;
}

// Router: logits to host, top-k, softmax weights (src/cuda.rs:673-701)
static void route(qh_model *m, int l, std::vector<std::pair<int, float>> &top, std::vector<float> &rw)
{
    const qh_config &c = m->c;
    Layer &L = m->L[l];
    const int ne = c.n_experts, d = c.embed_dim;
    cuda_gemv(0, L.router_w.u8(), m->d_norm_out.f(), m->d_router_logits.f(), d, ne);
    std::vector<float> logits(ne);
    cuda_d2h(logits.data(), m->d_router_logits.ptr, (size_t)ne * 4);
    cuda_sync();
    for (size_t i = 0; i < L.router_b.size() && i < (size_t)ne; i++) logits[i] += L.router_b[i];
    std::vector<std::pair<int, float>> idx(ne);
    for (int i = 0; i < ne; i++) idx[i] = {i, logits[i]};
    std::stable_sort(idx.begin(), idx.end(), [](const std::pair<int, float> &a, const std::pair<int, float> &b) { return a.second > b.second; });
    top.assign(idx.begin(), idx.begin() + c.n_experts_used);
    std::vector<float> e(top.size());
    float denom = 0.f;
    if (c.moe_renorm) {
        float mx = -INFINITY;
        for (auto &p : top) mx = std::max(mx, p.second);
        for (size_t i = 0; i < top.size(); i++) { e[i] = expf(top[i].second - mx); denom += e[i]; }
    } else {
        float mx = -INFINITY;
        for (float v : logits) mx = std::max(mx, v);
        for (float v : logits) denom += expf(v - mx);
        for (size_t i = 0; i < top.size(); i++) e[i] = expf(top[i].second - mx);
    }
    rw.resize(top.size());
    for (size_t i = 0; i < top.size(); i++) rw[i] = e[i] / denom;
}

// Can the experts of this layer be chosen on the device?  Every expert tensor must be served by the streaming
// GEMV (the kernel that takes device-side expert ids); QUARTZ_HOST_ROUTER=1 keeps the reference's host routing.
static int g_forced_host_router = -1;
static bool device_routing(qh_model *m, int l)
{
    if (g_forced_host_router < 0) {
        const char *e = getenv("QUARTZ_HOST_ROUTER");
        g_forced_host_router = (e && e[0] == '1') ? 1 : 0;
    }
    const int forced_host = g_forced_host_router;
    const qh_config &c = m->c;
    Layer &L = m->L[l];
    return !forced_host && c.n_experts <= 256 && c.n_experts_used <= 8 &&
           cuda_gemv_q_supported(L.moe_gate.ggml_type, L.moe_gate.u8(), c.embed_dim) &&
           cuda_gemv_q_supported(L.moe_up.ggml_type, L.moe_up.u8(), c.embed_dim) &&
           cuda_gemv_q_supported(L.moe_down.ggml_type, L.moe_down.u8(), c.ffn_dim);
}

// MoE FFN of one layer with router, top-k, expert selection and the weighted sum all on the device: the same
// arithmetic as moe_ffn below without its device-to-host copy and synchronisation per layer
// (src/cuda.rs:673-701 is what it replaces).
static void moe_ffn_device(qh_model *m, int l)
{
    const qh_config &c = m->c;
    Layer &L = m->L[l];
    const int d = c.embed_dim, fd = c.ffn_dim, ne = c.n_experts, n_act = c.n_experts_used;
    const uint32_t tg = L.moe_gate.ggml_type, tu = L.moe_up.ggml_type, td = L.moe_down.ggml_type;
    const size_t sg = ggml_type_size(tg, (size_t)d * fd), su = ggml_type_size(tu, (size_t)d * fd),
                 sd = ggml_type_size(td, (size_t)fd * d);
    const float *xn = m->d_norm_out.f();
    const int *ids = (const int *)m->d_moe_ids.ptr;
    const float *w = m->d_moe_w.f();
    cuda_gemv(0, L.router_w.u8(), xn, m->d_router_logits.f(), d, ne);
    cuda_router_topk(m->d_router_logits.f(), L.router_b_dev.empty() ? nullptr : L.router_b_dev.f(), 1, ne, n_act, c.moe_renorm,
                     (int *)m->d_moe_ids.ptr, m->d_moe_w.f());
    float *go = m->d_gate_all.f(), *uo = m->d_up_all.f(), *eo = m->d_expert_out_all.f(), *doo = m->d_down_all.f();
    for (int k0 = 0; k0 < n_act; k0 += 4) {
        const int n = std::min(4, n_act - k0);
        cuda_gemv_experts(tg, L.moe_gate.u8(), sg, ids + k0, n, xn, 0, go + (size_t)k0 * fd, d, fd);
        cuda_gemv_experts(tu, L.moe_up.u8(), su, ids + k0, n, xn, 0, uo + (size_t)k0 * fd, d, fd);
    }
    cuda_moe_decode_act(eo, go, uo, L.moe_gate_bias.empty() ? nullptr : L.moe_gate_bias.f(),
                        L.moe_up_bias.empty() ? nullptr : L.moe_up_bias.f(), ids, n_act, fd, c.clamped_swiglu);
    for (int k0 = 0; k0 < n_act; k0 += 4) {
        const int n = std::min(4, n_act - k0);
        cuda_gemv_experts(td, L.moe_down.u8(), sd, ids + k0, n, eo + (size_t)k0 * fd, (size_t)fd, doo + (size_t)k0 * d, fd, d);
    }
    cuda_moe_decode_combine(m->d_expert_acc.f(), doo, L.moe_down_bias.empty() ? nullptr : L.moe_down_bias.f(), ids, w, n_act, d, 0);
}

// MoE FFN of one layer on d_norm_out -> d_expert_acc (src/cuda.rs:667-798)
static void moe_ffn(qh_model *m, int l)
{
    if (device_routing(m, l)) {
        moe_ffn_device(m, l);
        return;
    }
    const qh_config &c = m->c;
    Layer &L = m->L[l];
    const int d = c.embed_dim, fd = c.ffn_dim;
    std::vector<std::pair<int, float>> top;
    std::vector<float> rw;
    route(m, l, top, rw);
    cuda_vec_zero(m->d_expert_acc.f(), d);
    const uint32_t tg = L.moe_gate.ggml_type, tu = L.moe_up.ggml_type, td = L.moe_down.ggml_type;
    const size_t sg = ggml_type_size(tg, (size_t)d * fd), su = ggml_type_size(tu, (size_t)d * fd),
                 sd = ggml_type_size(td, (size_t)fd * d);
    const float *xn = m->d_norm_out.f();
    const int n_act = (int)top.size();
    if (n_act == 4) {
        // four experts per launch (src/cuda.rs:714-761)
        const uint8_t *gp[4], *up[4], *dp[4];
        for (int k = 0; k < 4; k++) {
            gp[k] = L.moe_gate.u8() + top[k].first * sg;
            up[k] = L.moe_up.u8() + top[k].first * su;
            dp[k] = L.moe_down.u8() + top[k].first * sd;
        }
        float *go = m->d_gate_all.f(), *uo = m->d_up_all.f(), *eo = m->d_expert_out_all.f(), *doo = m->d_down_all.f();
        cuda_gemv_moe4(tg, gp[0], gp[1], gp[2], gp[3], xn, xn, xn, xn, go, go + fd, go + 2 * fd, go + 3 * fd, 4, d, fd);
        cuda_gemv_moe4(tu, up[0], up[1], up[2], up[3], xn, xn, xn, xn, uo, uo + fd, uo + 2 * fd, uo + 3 * fd, 4, d, fd);
        for (int k = 0; k < 4; k++) {
            const int e = top[k].first;
            if (!L.moe_gate_bias.empty()) cuda_vec_add(go + (size_t)k * fd, L.moe_gate_bias.f() + (size_t)e * fd, fd);
            if (!L.moe_up_bias.empty()) cuda_vec_add(uo + (size_t)k * fd, L.moe_up_bias.f() + (size_t)e * fd, fd);
            if (c.clamped_swiglu) cuda_swiglu_oai(eo + (size_t)k * fd, go + (size_t)k * fd, uo + (size_t)k * fd, fd);
            else cuda_swiglu(eo + (size_t)k * fd, go + (size_t)k * fd, uo + (size_t)k * fd, fd);
        }
        cuda_gemv_moe4(td, dp[0], dp[1], dp[2], dp[3], eo, eo + fd, eo + 2 * fd, eo + 3 * fd, doo, doo + d, doo + 2 * d,
                       doo + 3 * d, 4, fd, d);
        for (int k = 0; k < 4; k++) {
            if (!L.moe_down_bias.empty()) cuda_vec_add(doo + (size_t)k * d, L.moe_down_bias.f() + (size_t)top[k].first * d, d);
            cuda_vec_scale_add(m->d_expert_acc.f(), doo + (size_t)k * d, rw[k], d);
        }
    } else {
        // any active-expert count, one expert at a time (src/cuda.rs:762-794)
        float *g1 = m->d_gate.f(), *u1 = m->d_up.f(), *e1 = m->d_expert_out.f(), *dn = m->d_down_all.f();
        for (int k = 0; k < n_act; k++) {
            const int e = top[k].first;
            cuda_gemv(tg, L.moe_gate.u8() + e * sg, xn, g1, d, fd);
            if (!L.moe_gate_bias.empty()) cuda_vec_add(g1, L.moe_gate_bias.f() + (size_t)e * fd, fd);
            cuda_gemv(tu, L.moe_up.u8() + e * su, xn, u1, d, fd);
            if (!L.moe_up_bias.empty()) cuda_vec_add(u1, L.moe_up_bias.f() + (size_t)e * fd, fd);
            if (c.clamped_swiglu) cuda_swiglu_oai(e1, g1, u1, fd);
            else cuda_swiglu(e1, g1, u1, fd);
            cuda_gemv(td, L.moe_down.u8() + e * sd, e1, dn, fd, d);
            if (!L.moe_down_bias.empty()) cuda_vec_add(dn, L.moe_down_bias.f() + (size_t)e * d, d);
            cuda_vec_scale_add(m->d_expert_acc.f(), dn, rw[k], d);
        }
    }
}

// The reference sequence (src/cuda.rs:538-843), on-device part.
static void step_reference(qh_model *m, int token, int pos, bool need_logits)
{
    const qh_config &c = m->c;
    const int d = c.embed_dim, h = c.n_heads, kv = c.n_kv_heads, hd = c.head_dim, q_d = m->q_d(), kv_d = m->kv_d(),
              fd = c.ffn_dim, seq = pos + 1;
    const float scale = attn_scale(c);
    // The reference dequantizes the embedding row on the CPU and uploads it (src/cuda.rs:538-545);
    // here the table is resident and cuda_embed_lookup produces the same f32 row bit for bit.
    cuda_embed_lookup(m->d_hidden.f(), m->embed.u8(), m->embed.ggml_type, token, d);
    for (int l = 0; l < c.n_layers; l++) {
        Layer &L = m->L[l];
        cuda_rms_norm(m->d_norm_out.f(), m->d_hidden.f(), L.attn_norm.f(), d);
        cuda_gemv(L.q.ggml_type, L.q.u8(), m->d_norm_out.f(), m->d_q.f(), d, q_d);
        cuda_gemv(L.k.ggml_type, L.k.u8(), m->d_norm_out.f(), m->d_k.f(), d, kv_d);
        cuda_gemv(L.v.ggml_type, L.v.u8(), m->d_norm_out.f(), m->d_v.f(), d, kv_d);
        cuda_vec_add(m->d_q.f(), L.q_bias.f(), q_d);
        cuda_vec_add(m->d_k.f(), L.k_bias.f(), kv_d);
        cuda_vec_add(m->d_v.f(), L.v_bias.f(), kv_d);
        if (!L.q_norm.empty()) {   // QK-norm before RoPE (src/cuda.rs:576-599)
            if ((int)L.q_norm_len == hd) for (int hh = 0; hh < h; hh++) cuda_rms_norm(m->d_q.f() + hh * hd, m->d_q.f() + hh * hd, L.q_norm.f(), hd);
            else cuda_rms_norm(m->d_q.f(), m->d_q.f(), L.q_norm.f(), q_d);
        }
        if (!L.k_norm.empty()) {
            if ((int)L.k_norm_len == hd) for (int hh = 0; hh < kv; hh++) cuda_rms_norm(m->d_k.f() + hh * hd, m->d_k.f() + hh * hd, L.k_norm.f(), hd);
            else cuda_rms_norm(m->d_k.f(), m->d_k.f(), L.k_norm.f(), kv_d);
        }
        cuda_rope_yarn(m->d_q.f(), h, hd, pos, c.rope_theta, c.yarn_scale, c.yarn_orig_ctx, c.rope_neox);
        cuda_rope_yarn(m->d_k.f(), kv, hd, pos, c.rope_theta, c.yarn_scale, c.yarn_orig_ctx, c.rope_neox);
        cuda_kv_append(m->kv_k[l].f(), m->kv_v[l].f(), m->d_k.f(), m->d_v.f(), pos, kv_d);
        const int k_start = attn_start(c, l, pos), seq_a = seq - k_start;
        const float *kc = m->kv_k[l].f() + (size_t)k_start * kv_d, *vc = m->kv_v[l].f() + (size_t)k_start * kv_d;
        cuda_attn_score_all(m->d_scores.f(), m->d_q.f(), kc, h, kv, seq_a, hd, kv_d, c.max_seq, scale);
        cuda_softmax_sink_all(m->d_scores.f(), h, seq_a, c.max_seq, L.sinks.f());
        cuda_attn_values_all(m->d_attn_out.f(), m->d_scores.f(), vc, h, kv, seq_a, hd, kv_d, c.max_seq);
        cuda_gemv(L.o.ggml_type, L.o.u8(), m->d_attn_out.f(), m->d_norm_out.f(), q_d, d);
        if (!L.o_bias.empty()) cuda_vec_add(m->d_norm_out.f(), L.o_bias.f(), d);
        cuda_vec_add(m->d_hidden.f(), m->d_norm_out.f(), d);
        cuda_rms_norm(m->d_norm_out.f(), m->d_hidden.f(), L.ffn_norm.f(), d);
        if (c.n_experts > 0) {
            moe_ffn(m, l);
            cuda_vec_add(m->d_hidden.f(), m->d_expert_acc.f(), d);
        } else {
            cuda_gemv(L.gate.ggml_type, L.gate.u8(), m->d_norm_out.f(), m->d_gate.f(), d, fd);
            cuda_gemv(L.up.ggml_type, L.up.u8(), m->d_norm_out.f(), m->d_up.f(), d, fd);
            cuda_swiglu(m->d_expert_out.f(), m->d_gate.f(), m->d_up.f(), fd);
            cuda_gemv(L.down.ggml_type, L.down.u8(), m->d_expert_out.f(), m->d_norm_out.f(), fd, d);
            cuda_vec_add(m->d_hidden.f(), m->d_norm_out.f(), d);
        }
    }
    if (!need_logits) return;
    cuda_rms_norm(m->d_norm_out.f(), m->d_hidden.f(), m->final_norm.f(), d);
    cuda_gemv(m->lm_head.ggml_type, m->lm_head.u8(), m->d_norm_out.f(), m->d_logits.f(), d, c.vocab_size);
}

// Can this model take the fused sequence?  Dense FFN, no QK-norm, no biases to add (absent
// biases are zero vectors in the reference, so skipping them changes nothing), every
// projection served by the streaming kernel, q rows splittable into kv-sized slices.
static bool fusable(qh_model *m)
{
    const qh_config &c = m->c;
    if (c.n_experts > 0 || c.head_dim > 128 || c.head_dim % 32 || c.embed_dim % 64 || c.ffn_dim % 64) return false;
    if (m->q_d() % m->kv_d() != 0 || m->q_d() / m->kv_d() + 2 > 8) return false;
    if (!cuda_attn_step_supported(c.n_heads, c.n_kv_heads, c.head_dim)) return false;
    for (auto &L : m->L) {
        if (!L.q_norm.empty() || !L.k_norm.empty() || L.has_qkv_bias || !L.o_bias.empty()) return false;
        if (L.q.ggml_type != L.k.ggml_type || L.q.ggml_type != L.v.ggml_type || L.gate.ggml_type != L.up.ggml_type) return false;
        if (!cuda_gemv_q_supported(L.q.ggml_type, L.q.u8(), c.embed_dim) || !cuda_gemv_q_supported(L.k.ggml_type, L.k.u8(), c.embed_dim) ||
            !cuda_gemv_q_supported(L.v.ggml_type, L.v.u8(), c.embed_dim) || !cuda_gemv_q_supported(L.o.ggml_type, L.o.u8(), m->q_d()) ||
            !cuda_gemv_q_supported(L.gate.ggml_type, L.gate.u8(), c.embed_dim) || !cuda_gemv_q_supported(L.up.ggml_type, L.up.u8(), c.embed_dim) ||
            !cuda_gemv_q_supported(L.down.ggml_type, L.down.u8(), c.ffn_dim))
            return false;
    }
    return cuda_gemv_q_supported(m->lm_head.ggml_type, m->lm_head.u8(), c.embed_dim) != 0;
}

// Sliding-window layers (src/main.rs:231-237): the window the attention kernel applies on the device.
static int attn_window(const qh_config &c, int layer) { return (c.swa_window > 0 && layer % 2 == 0) ? c.swa_window : 0; }

// The attention block of layer l as one launch; token position comes from the device step words.
static void attn_layer(qh_model *m, int l, int out_slot)
{
    const qh_config &c = m->c;
    Layer &L = m->L[l];
    cuda_attn_step(m->d_attn_out.f(), m->d_q.f(), m->d_k.f(), m->d_v.f(), m->kv_k[l].f(), m->kv_v[l].f(), c.n_heads,
                   c.n_kv_heads, c.head_dim, c.max_seq, (const int *)m->d_step.ptr, 0, attn_window(c, l), attn_scale(c),
                   L.sinks.f(), c.rope_theta, c.yarn_scale, c.yarn_orig_ctx, c.rope_neox, out_slot);
}

// q (as kv_d-row slices), k and v of layer L as the matrices of one multi-matrix GEMV
static int qkv_mats(qh_model *m, Layer &L, const uint8_t **W, float **Y)
{
    const int d = m->c.embed_dim, kv_d = m->kv_d(), q_slices = m->q_d() / kv_d;
    const size_t q_slice_bytes = ggml_type_size(L.q.ggml_type, (size_t)d * kv_d);   // per layer: types may differ between layers
    int n = 0;
    for (int s = 0; s < q_slices; s++) { W[n] = L.q.u8() + s * q_slice_bytes; Y[n] = m->d_q.f() + (size_t)s * kv_d; n++; }
    W[n] = L.k.u8(); Y[n] = m->d_k.f(); n++;
    W[n] = L.v.u8(); Y[n] = m->d_v.f(); n++;
    return n;
}

// Tell the next streaming GEMV which weights follow it (it pulls their first megabytes into L2 while it drains).
static void hint_next(const GpuBuf &w, size_t cap = (size_t)16 << 20)
{
    if (!w.empty()) quartz_prefetch_next(w.ptr, w.bytes < cap ? w.bytes : cap);
}

// The fused sequence: five or six launches per layer instead of twenty-one (+ seven conversions).  Token id and
// position are read from the device step words (cuda_step_set), so the recording serves every step.
static void step_fused(qh_model *m, bool need_logits)
{
    const qh_config &c = m->c;
    const int d = c.embed_dim, q_d = m->q_d(), kv_d = m->kv_d(), fd = c.ffn_dim;
    cuda_embed_lookup_dev(m->d_hidden.f(), m->embed.u8(), m->embed.ggml_type, (const int *)m->d_step.ptr, d);
    for (int l = 0; l < c.n_layers; l++) {
        Layer &L = m->L[l];
        // q, k and v in one launch that normalises the hidden state in its prologue
        const uint8_t *W[8];
        float *Y[8];
        const int n = qkv_mats(m, L, W, Y);
        hint_next(L.o);
        cuda_gemv_rmsnorm(L.q.ggml_type, n, W, Y, m->d_hidden.f(), L.attn_norm.f(), d, kv_d, 0);
        // RoPE, KV append, attention over the whole context and its merge: one launch, which also leaves the
        // output projection's activation form in slot 1
        attn_layer(m, l, 1);
        {   // output projection, residual added in the epilogue
            const uint8_t *w1[1] = {L.o.u8()};
            float *y1[1] = {m->d_hidden.f()};
            int s1[1] = {1};
            hint_next(L.gate, (size_t)12 << 20);
            hint_next(L.up, (size_t)12 << 20);
            cuda_gemv_q(L.o.ggml_type, 1, w1, s1, y1, q_d, d, 1);
        }
        {
            const uint8_t *w2[2] = {L.gate.u8(), L.up.u8()};
            float *y2[2] = {m->d_gate.f(), m->d_up.f()};
            hint_next(L.down);
            cuda_gemv_rmsnorm(L.gate.ggml_type, 2, w2, y2, m->d_hidden.f(), L.ffn_norm.f(), d, fd, 0);
        }
        {   // down projection of swiglu(gate, up), computed in its prologue; residual added in the epilogue
            const uint8_t *w1[1] = {L.down.u8()};
            float *y1[1] = {m->d_hidden.f()};
            if (l + 1 < c.n_layers) {
                hint_next(m->L[l + 1].q);
                hint_next(m->L[l + 1].k);
                hint_next(m->L[l + 1].v);
            } else if (need_logits) {
                hint_next(m->lm_head);
            }
            cuda_gemv_swiglu(L.down.ggml_type, 1, w1, y1, m->d_gate.f(), m->d_up.f(), 0, fd, d, 1);
        }
    }
    if (!need_logits) return;
    const uint8_t *w1[1] = {m->lm_head.u8()};
    float *y1[1] = {m->d_logits.f()};
    cuda_gemv_rmsnorm(m->lm_head.ggml_type, 1, w1, y1, m->d_hidden.f(), m->final_norm.f(), d, c.vocab_size, 0);
}

// The chained sequence: per layer the attention launch and ONE persistent kernel that runs output projection ->
// gate/up -> down -> the next layer's q/k/v (or the output head) with grid-wide barriers between the links: two
// launches per layer.
static int chain_ops(qh_model *m, int l, bool need_logits, qz_chain_op *ops, const uint8_t **w1, const uint8_t **w2,
                     const uint8_t **w3, float **y1, float **y2, const uint8_t **W4, float **Y4)
{
    const qh_config &c = m->c;
    const int d = c.embed_dim, kv_d = m->kv_d(), q_d = m->q_d(), fd = c.ffn_dim;
    Layer &L = m->L[l];
    w1[0] = L.o.u8();
    w2[0] = L.gate.u8(); w2[1] = L.up.u8();
    w3[0] = L.down.u8();
    y1[0] = m->d_hidden.f();
    y2[0] = m->d_gate.f(); y2[1] = m->d_up.f();
    ops[0] = {L.o.ggml_type, 1, w1, y1, q_d, d, 1, 3, m->d_attn_out.f(), nullptr, 0};
    ops[1] = {L.gate.ggml_type, 2, w2, y2, d, fd, 0, 1, m->d_hidden.f(), L.ffn_norm.f(), 0};
    ops[2] = {L.down.ggml_type, 1, w3, y1, fd, d, 1, 2, m->d_gate.f(), m->d_up.f(), 0};
    if (l + 1 < c.n_layers) {
        Layer &Nx = m->L[l + 1];
        const int n = qkv_mats(m, Nx, W4, Y4);
        ops[3] = {Nx.q.ggml_type, n, W4, Y4, d, kv_d, 0, 1, m->d_hidden.f(), Nx.attn_norm.f(), 0};
        return 4;
    }
    if (need_logits) {
        W4[0] = m->lm_head.u8();
        Y4[0] = m->d_logits.f();
        ops[3] = {m->lm_head.ggml_type, 1, W4, Y4, d, c.vocab_size, 0, 1, m->d_hidden.f(), m->final_norm.f(), 0};
        return 4;
    }
    return 3;
}

static bool chainable(qh_model *m)
{
    const qh_config &c = m->c;
    if (m->q_d() % m->kv_d() != 0 || m->q_d() / m->kv_d() + 2 > 8) return false;
    for (int l = 0; l < c.n_layers; l++) {   // every layer: quantization types may differ from layer to layer
        const uint8_t *w1[1], *w2[2], *w3[1], *W4[8];
        float *y1[1], *y2[2], *Y4[8];
        qz_chain_op ops[4];
        const int n_ops = chain_ops(m, l, true, ops, w1, w2, w3, y1, y2, W4, Y4);
        if (!cuda_gemv_chain_supported(n_ops, ops)) return false;
    }
    return true;
}

static void step_chained(qh_model *m, bool need_logits)
{
    const qh_config &c = m->c;
    const int d = c.embed_dim, kv_d = m->kv_d();
    cuda_embed_lookup_dev(m->d_hidden.f(), m->embed.u8(), m->embed.ggml_type, (const int *)m->d_step.ptr, d);
    {
        const uint8_t *W[8];
        float *Y[8];
        const int n = qkv_mats(m, m->L[0], W, Y);
        cuda_gemv_rmsnorm(m->L[0].q.ggml_type, n, W, Y, m->d_hidden.f(), m->L[0].attn_norm.f(), d, kv_d, 0);
    }
    for (int l = 0; l < c.n_layers; l++) {
        attn_layer(m, l, -1);
        const uint8_t *w1[1], *w2[2], *w3[1], *W4[8];
        float *y1[1], *y2[2], *Y4[8];
        qz_chain_op ops[4];
        const int n_ops = chain_ops(m, l, need_logits, ops, w1, w2, w3, y1, y2, W4, Y4);
        cuda_gemv_chain(n_ops, ops);
    }
}

int qh_step_device(qh_model *m, int token, int pos, int fused)
{
    if (!m || !m->finalized || token < 0 || token >= m->c.vocab_size) return -1;
    if (pos >= m->c.max_seq) {   // src/cuda.rs:517-520: clamp with a warning, never write out of bounds
        fprintf(stderr, "KV cache full at pos %d (max_seq=%d); clamping to avoid OOB\n", pos, m->c.max_seq);
        pos = m->c.max_seq - 1;
    }
    const long long before = quartz_launch_count();
    if (!fused || !fusable(m)) {
        step_reference(m, token, pos, true);
        m->last_launches = quartz_launch_count() - before;
        return 0;
    }
    // fused == 2 asks for the chained sequence (falls back to the fused one where the chain kernel does not apply)
    const bool chain = fused == 2 && chainable(m);
    auto step = [&](qh_model *mm, bool nl) { chain ? step_chained(mm, nl) : step_fused(mm, nl); };
    // Token id and position go to the device step words; the step itself is recorded once per model and
    // sequence kind and replayed for every (token, position).
    cuda_step_set((int *)m->d_step.ptr, token, pos);
    void *&g = m->graphs[chain ? 2 : 1];
    if (!g) {
        step(m, true);   // eager once: creates every scratch buffer, warms the kernels
        cuda_sync();
        const long long b2 = quartz_launch_count();
        if (!quartz_graph_begin()) return -2;
        step(m, true);
        g = quartz_graph_end();
        if (!g) return -3;
        m->n_recorded++;
        m->last_launches = quartz_launch_count() - b2;
    }
    quartz_graph_launch(g);
    return 0;
}

// Can a prompt go through the batched path?  Same conditions as the fused decode sequence for the attention
// block (no QK-norm, no biases); dense FFN, or MoE without expert biases (the grouped MoE kernel has none).
static bool prefill_batchable(qh_model *m)
{
    const qh_config &c = m->c;
    if (c.head_dim > 128 || c.head_dim % 32 || !cuda_attn_step_supported(c.n_heads, c.n_kv_heads, c.head_dim)) return false;
    for (auto &L : m->L) {
        if (!L.q_norm.empty() || !L.k_norm.empty() || L.has_qkv_bias || !L.o_bias.empty()) return false;
        if (c.n_experts > 0 && (!L.moe_gate_bias.empty() || !L.moe_up_bias.empty() || !L.moe_down_bias.empty() ||
                                L.moe_gate.ggml_type != L.moe_up.ggml_type))
            return false;
    }
    return c.n_experts == 0 || (c.n_experts <= 256 && c.n_experts_used <= 8);
}

static bool prefill_scratch(qh_model *m, int n)
{
    if (n <= m->p_cap) return true;
    const qh_config &c = m->c;
    const size_t N = (size_t)n, d = c.embed_dim, q_d = m->q_d(), kv_d = m->kv_d(), fd = c.ffn_dim;
    const size_t used = (size_t)std::max(c.n_experts_used, 1);
    const bool ok = m->p_tok.alloc_f32(N) && m->p_x.alloc_f32(N * d) && m->p_xn.alloc_f32(N * d) && m->p_q.alloc_f32(N * q_d) &&
                    m->p_k.alloc_f32(N * kv_d) && m->p_v.alloc_f32(N * kv_d) && m->p_att.alloc_f32(N * std::max(q_d, d)) &&
                    m->p_g.alloc_f32(c.n_experts > 0 ? N * (size_t)std::max(c.n_experts, 1) : N * fd) &&
                    m->p_u.alloc_f32(c.n_experts > 0 ? 4 : N * fd) && m->p_ids.alloc_f32(N * used) && m->p_w.alloc_f32(N * used);
    m->p_cap = ok ? n : 0;
    return ok;
}

// Batched prefill: the n tokens of a prompt at positions pos0 .. pos0+n-1 in one pass -- every projection a
// tensor-core GEMM over all tokens (cuda_gemm), RoPE + KV append and causal attention batched over the tokens --
// instead of n decode steps (what the reference's GPU prefill does, src/main.rs:1410-1416; its batched prefill,
// src/main.rs:1157-1341, is CPU-only).  Leaves the caches filled and, when logits_host is not NULL, the logits
// of the LAST token there.  Models the batched path does not take run token by token.
int qh_prefill(qh_model *m, const int *tokens, int n, int pos0, float *logits_host)
{
    if (!m || !m->finalized || !tokens || n <= 0 || pos0 < 0 || pos0 + n > m->c.max_seq) return -1;
    const qh_config &c = m->c;
    for (int i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= c.vocab_size) return -1;
    if (!prefill_batchable(m) || n == 1) {
        for (int i = 0; i < n; i++) {
            const int rc = qh_step_device(m, tokens[i], pos0 + i, 1);
            if (rc) return rc;
        }
        if (logits_host) cuda_d2h(logits_host, m->d_logits.ptr, (size_t)c.vocab_size * 4);
        cuda_sync();
        return quartz_last_error() == 0 ? 0 : -10;
    }
    if (!prefill_scratch(m, n)) return -2;
    const int d = c.embed_dim, h = c.n_heads, kv = c.n_kv_heads, hd = c.head_dim, q_d = m->q_d(), kv_d = m->kv_d(), fd = c.ffn_dim;
    const float scale = attn_scale(c);
    float *X = m->p_x.f(), *Xn = m->p_xn.f(), *Q = m->p_q.f(), *K = m->p_k.f(), *V = m->p_v.f(), *A = m->p_att.f();
    cuda_h2d(m->p_tok.ptr, tokens, (size_t)n * 4);
    cuda_embed_lookup_rows(X, m->embed.u8(), m->embed.ggml_type, (const int *)m->p_tok.ptr, n, d);
    for (int l = 0; l < c.n_layers; l++) {
        Layer &L = m->L[l];
        cuda_rms_norm_rows(Xn, X, L.attn_norm.f(), n, d);
        cuda_gemm(L.q.ggml_type, L.q.u8(), Xn, Q, n, d, q_d);
        cuda_gemm(L.k.ggml_type, L.k.u8(), Xn, K, n, d, kv_d);
        cuda_gemm(L.v.ggml_type, L.v.u8(), Xn, V, n, d, kv_d);
        cuda_rope_kv_rows(Q, K, V, m->kv_k[l].f(), m->kv_v[l].f(), n, h, kv, hd, pos0, c.rope_theta, c.yarn_scale, c.yarn_orig_ctx,
                          c.rope_neox);
        cuda_attn_prompt(A, Q, m->kv_k[l].f(), m->kv_v[l].f(), n, h, kv, hd, c.max_seq, pos0, attn_window(c, l), scale, L.sinks.f());
        cuda_gemm(L.o.ggml_type, L.o.u8(), A, Xn, n, q_d, d);
        cuda_vec_add(X, Xn, n * d);
        cuda_rms_norm_rows(Xn, X, L.ffn_norm.f(), n, d);
        if (c.n_experts > 0) {
            // router logits of all tokens, top-k and weights on the device, grouped expert FFN
            float *RL = m->p_g.f();
            cuda_gemm(L.router_w.ggml_type, L.router_w.u8(), Xn, RL, n, d, c.n_experts);
            cuda_router_topk(RL, L.router_b_dev.empty() ? nullptr : L.router_b_dev.f(), n, c.n_experts, c.n_experts_used, c.moe_renorm,
                             (int *)m->p_ids.ptr, m->p_w.f());
            cuda_moe_ffn_dev(L.moe_gate.ggml_type, L.moe_down.ggml_type, L.moe_gate.u8(), L.moe_up.u8(), L.moe_down.u8(), Xn, A, n, d,
                             fd, c.n_experts, c.n_experts_used, (const int *)m->p_ids.ptr, m->p_w.f(), c.clamped_swiglu);
            cuda_vec_add(X, A, n * d);   // (the attention-output rows are free again: they hold the experts' sum)
        } else {
            float *Gt = m->p_g.f(), *U = m->p_u.f();
            cuda_gemm(L.gate.ggml_type, L.gate.u8(), Xn, Gt, n, d, fd);
            cuda_gemm(L.up.ggml_type, L.up.u8(), Xn, U, n, d, fd);
            cuda_swiglu(Gt, Gt, U, n * fd);
            cuda_gemm(L.down.ggml_type, L.down.u8(), Gt, Xn, n, fd, d);
            cuda_vec_add(X, Xn, n * d);
        }
    }
    // the last token's hidden state -> logits (the only row the caller needs)
    cuda_rms_norm(m->d_norm_out.f(), X + (size_t)(n - 1) * d, m->final_norm.f(), d);
    cuda_gemv(m->lm_head.ggml_type, m->lm_head.u8(), m->d_norm_out.f(), m->d_logits.f(), d, c.vocab_size);
    if (logits_host) cuda_d2h(logits_host, m->d_logits.ptr, (size_t)c.vocab_size * 4);
    cuda_sync();
    return quartz_last_error() == 0 ? 0 : -10;
}

static int step_host(qh_model *m, int token, int pos, int need_logits, float *logits_host, int fused)
{
    int rc = qh_step_device(m, token, pos, fused);
    if (rc) return rc;
    if (need_logits && logits_host) cuda_d2h(logits_host, m->d_logits.ptr, (size_t)m->c.vocab_size * 4);
    cuda_sync();
    return quartz_last_error() == 0 ? 0 : -10;
}

int qh_forward_step(qh_model *m, int token, int pos, int need_logits, float *logits_host)
{
    return step_host(m, token, pos, need_logits, logits_host, 0);
}

int qh_forward_step_fused(qh_model *m, int token, int pos, int need_logits, float *logits_host)
{
    return step_host(m, token, pos, need_logits, logits_host, 1);
}

int qh_forward_step_chained(qh_model *m, int token, int pos, int need_logits, float *logits_host)
{
    return step_host(m, token, pos, need_logits, logits_host, 2);
}

int qh_read_hidden(qh_model *m, float *host)
{
    if (!m || !m->finalized) return -1;
    cuda_d2h(host, m->d_hidden.ptr, (size_t)m->c.embed_dim * 4);
    cuda_sync();
    return 0;
}

long long qh_launches_last_step(qh_model *m) { return m ? m->last_launches : 0; }
int qh_graphs_recorded(qh_model *m) { return m ? m->n_recorded : 0; }
void qh_force_host_router(int on) { g_forced_host_router = on ? 1 : 0; }

}  // extern "C"
