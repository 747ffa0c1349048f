// qh_load_gguf: a model straight from a GGUF file.  Configuration as Config::from_gguf derives it
// (src/main.rs:96-215), tensors by the names Weights::load uses (src/main.rs:357-414).
#include <string.h>

#include <string>
#include <vector>

#include "forward_state.h"
#include "gguf_loader.h"

namespace {

thread_local std::string g_load_err;

struct Meta {
    const qg_file *f;
    std::string arch;
    // "<arch>.<key>" for the first key of the list that exists (src/main.rs: arch_u32_any / arch_f32_any)
    bool u32(std::initializer_list<const char *> keys, uint32_t &out) const
    {
        for (const char *k : keys)
            if (qg_meta_u32(f, (arch + "." + k).c_str(), &out)) return true;
        return false;
    }
    bool f32(std::initializer_list<const char *> keys, float &out) const
    {
        for (const char *k : keys)
            if (qg_meta_f32(f, (arch + "." + k).c_str(), &out)) return true;
        return false;
    }
};

bool contains(const std::string &s, const char *needle) { return s.find(needle) != std::string::npos; }

// upload tensor `name` into (role, layer); optional tensors that are absent are skipped
bool put(qh_model *m, const qg_file *f, const std::string &name, int role, int layer, bool quantized, bool required, int repack)
{
    const int i = qg_find_tensor(f, name.c_str());
    if (i < 0) {
        if (required) g_load_err = "missing tensor " + name;
        return !required;
    }
    const uint32_t t = qg_tensor_type(f, i);
    const void *data = qg_tensor_data(f, i);
    const uint64_t bytes = qg_tensor_bytes(f, i);
    if (!data || !bytes) {
        g_load_err = "tensor " + name + " has an unknown type or lies outside the file";
        return false;
    }
    if (!quantized && t != 0) {
        g_load_err = "tensor " + name + " must be F32";
        return false;
    }
    const int rc = qh_set_tensor(m, role, layer, t, data, (size_t)bytes, quantized ? repack : 0);
    if (rc != 0) {
        g_load_err = "upload of " + name + " failed (" + std::to_string(rc) + ")";
        return false;
    }
    return true;
}

}  // namespace

extern "C" {

const char *qh_load_error(void) { return g_load_err.c_str(); }

qh_model *qh_load_gguf(const char *path, int max_seq, int repack, qh_config *cfg_out)
{
    g_load_err.clear();
    qg_file *f = qg_open(path);
    if (!f) {
        g_load_err = qg_last_error();
        return nullptr;
    }
    auto fail = [&](const std::string &why) -> qh_model * {
        if (!why.empty()) g_load_err = why;
        qg_close(f);
        return nullptr;
    };
    const char *a = qg_meta_str(f, "general.architecture");
    Meta md{f, a ? a : "llama"};
    const std::string &arch = md.arch;
    qh_config c;
    memset(&c, 0, sizeof(c));
    uint32_t v = 0;
    if (!md.u32({"embedding_length"}, v)) return fail("missing embedding_length");
    c.embed_dim = (int)v;
    if (!md.u32({"head_count", "attention.head_count"}, v)) return fail("missing head_count");
    c.n_heads = (int)v;
    c.n_kv_heads = md.u32({"head_count_kv", "attention.head_count_kv"}, v) ? (int)v : c.n_heads;
    if (!md.u32({"block_count"}, v)) return fail("missing block_count");
    c.n_layers = (int)v;
    if (!md.u32({"expert_feed_forward_length", "feed_forward_length", "attention.feed_forward_length"}, v))
        return fail("missing feed_forward_length");
    c.ffn_dim = (int)v;
    c.rope_theta = 10000.f;
    md.f32({"rope.freq_base", "attention.rope.freq_base"}, c.rope_theta);
    int context = 8192;
    if (md.u32({"context_length"}, v) && v > 0) context = (int)v;
    c.head_dim = md.u32({"attention.key_length"}, v) ? (int)v : c.embed_dim / (c.n_heads > 0 ? c.n_heads : 1);
    uint64_t n_tok = 0;
    if (md.u32({"vocab_size"}, v)) c.vocab_size = (int)v;
    else if (qg_meta_array_len(f, "tokenizer.ggml.tokens", &n_tok)) c.vocab_size = (int)n_tok;
    else return fail("cannot determine vocab_size");
    c.n_experts = md.u32({"expert_count", "experts_count", "num_experts"}, v) ? (int)v : 0;
    c.n_experts_used = md.u32({"expert_used_count", "experts_used"}, v) ? (int)v : (c.n_experts > 0 ? 2 : 0);
    int flag = 0;
    c.moe_renorm = qg_meta_bool(f, (arch + ".expert_weights_norm").c_str(), &flag) ? flag : (arch != "olmoe");
    c.yarn_scale = 1.f;
    md.f32({"rope.scaling.factor"}, c.yarn_scale);
    c.yarn_orig_ctx = md.u32({"rope.scaling.original_context_length"}, v) ? (int)v : 0;
    c.clamped_swiglu = contains(arch, "gpt-oss") ? 1 : 0;
    c.swa_window = (contains(arch, "gpt-oss") && md.u32({"attention.sliding_window"}, v)) ? (int)v : 0;
    static const char *norm_rope[] = {"llama", "baichuan", "starcoder", "minicpm", "internlm2", "orion", "plamo", "xverse"};
    c.rope_neox = 1;
    for (const char *n : norm_rope)
        if (arch == n) c.rope_neox = 0;
    c.max_seq = max_seq > 0 ? max_seq : (context < 8192 ? context : 8192);
    if (c.embed_dim <= 0 || c.n_heads <= 0 || c.n_layers <= 0 || c.vocab_size <= 0) return fail("implausible configuration");
    if (cfg_out) *cfg_out = c;

    qh_model *m = qh_create(&c);
    if (!m) return fail("qh_create failed");
    auto bail = [&]() -> qh_model * {
        qh_destroy(m);
        return fail("");
    };
    if (!put(m, f, "token_embd.weight", QH_EMBED, 0, true, true, repack)) return bail();
    // tied embeddings: no output.weight, the head reuses token_embd (src/main.rs:411-417)
    const char *head = qg_find_tensor(f, "output.weight") >= 0 ? "output.weight" : "token_embd.weight";
    if (!put(m, f, head, QH_LM_HEAD, 0, true, true, repack)) return bail();
    if (!put(m, f, "output_norm.weight", QH_FINAL_NORM, 0, false, true, 0)) return bail();
    for (int l = 0; l < c.n_layers; l++) {
        const std::string b = "blk." + std::to_string(l) + ".";
        struct Item { const char *name; int role; bool quant, required; };
        const Item common[] = {
            {"attn_norm.weight", QH_ATTN_NORM, false, true}, {"attn_q_norm.weight", QH_Q_NORM, false, false},
            {"attn_k_norm.weight", QH_K_NORM, false, false}, {"attn_q.weight", QH_Q, true, true},
            {"attn_k.weight", QH_K, true, true},             {"attn_v.weight", QH_V, true, true},
            {"attn_output.weight", QH_O, true, true},        {"attn_q.bias", QH_Q_BIAS, false, false},
            {"attn_k.bias", QH_K_BIAS, false, false},        {"attn_v.bias", QH_V_BIAS, false, false},
            {"attn_output.bias", QH_O_BIAS, false, false},   {"attn_sinks.weight", QH_SINKS, false, false}};
        for (const Item &it : common)
            if (!put(m, f, b + it.name, it.role, l, it.quant, it.required, repack)) return bail();
        // the FFN's norm is stored under either name (src/main.rs:372-379)
        const std::string post = b + "post_attention_norm.weight";
        const std::string ffn_norm = qg_find_tensor(f, post.c_str()) >= 0 ? post : b + "ffn_norm.weight";
        if (!put(m, f, ffn_norm, QH_FFN_NORM, l, false, true, 0)) return bail();
        if (c.n_experts > 0) {
            const Item moe[] = {{"ffn_gate_inp.weight", QH_ROUTER_W, false, true},     {"ffn_gate_inp.bias", QH_ROUTER_B, false, false},
                                {"ffn_gate_exps.weight", QH_MOE_GATE, true, true},     {"ffn_up_exps.weight", QH_MOE_UP, true, true},
                                {"ffn_down_exps.weight", QH_MOE_DOWN, true, true},     {"ffn_gate_exps.bias", QH_MOE_GATE_BIAS, false, false},
                                {"ffn_up_exps.bias", QH_MOE_UP_BIAS, false, false},    {"ffn_down_exps.bias", QH_MOE_DOWN_BIAS, false, false}};
            for (const Item &it : moe)
                if (!put(m, f, b + it.name, it.role, l, it.quant, it.required, repack)) return bail();
        } else {
            const Item dense[] = {{"ffn_gate.weight", QH_GATE, true, true}, {"ffn_up.weight", QH_UP, true, true},
                                  {"ffn_down.weight", QH_DOWN, true, true}};
            for (const Item &it : dense)
                if (!put(m, f, b + it.name, it.role, l, it.quant, it.required, repack)) return bail();
        }
    }
    qg_close(f);   // every tensor has been copied to the device
    if (qh_finalize(m) != 0) {
        g_load_err = "qh_finalize failed";
        qh_destroy(m);
        return nullptr;
    }
    return m;
}

}  // extern "C"
