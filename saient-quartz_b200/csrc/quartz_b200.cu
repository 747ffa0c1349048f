// quartz_b200: the extern "C" boundary (include/quartz_b200.h) and its host logic.
// One translation unit on purpose: the IQ codebooks are __device__ globals shared
// by every kernel, and the library is built without relocatable device code.

#include "../../include/quartz_b200.h"

#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "formats.cuh"
#include "generic.cuh"
#include "gemv_stream.cuh"
#include "gemv_tma.cuh"
#include "decode_ops.cuh"
#include "fused_ops.cuh"
#include "attn_step.cuh"
#include "attn_prompt.cuh"
#include "gemm_tc.cuh"
#include "moe.cuh"
#include "gemv_chain.cuh"

namespace qz {

// ---- process state --------------------------------------------------------------
static cudaStream_t g_stream = 0;
static int g_err = QZ_OK;
static std::string g_err_msg;
static int g_sm_count = 0;
long long g_launch_count = 0;

void set_error(int code, const char *what)
{
    if (g_err == QZ_OK) {   // sticky: keep the first failure
        g_err = code;
        g_err_msg = what ? what : "";
    }
}
cudaStream_t stream() { return g_stream; }
int sm_count()
{
    if (!g_sm_count) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || g_sm_count <= 0)
            g_sm_count = 148;
    }
    return g_sm_count;
}

// ---- launch helper: ordinary launch, or programmatic dependent launch when enabled ----------
static bool g_pdl = false;

template <class... KArgs, class... Args>
static void launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args)
{
    g_launch_count++;
    if (g_pdl) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = smem;
        cfg.stream = g_stream;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        QZ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
    } else {
        kernel<<<grid, block, smem, g_stream>>>(KArgs(args)...);
        QZ_CUDA_CHECK(cudaGetLastError());
    }
}

// ---- registry of repacked byte ranges ---------------------------------------------
struct Range {
    uintptr_t end;
    uint32_t type;
    int K;
    long long rows;
};
static std::map<uintptr_t, Range> g_ranges;   // start -> range

static const Range *find_range(const void *p, uintptr_t *start_out = nullptr)
{
    if (g_ranges.empty()) return nullptr;
    uintptr_t a = (uintptr_t)p;
    auto it = g_ranges.upper_bound(a);
    if (it == g_ranges.begin()) return nullptr;
    --it;
    if (a >= it->second.end) return nullptr;
    if (start_out) *start_out = it->first;
    return &it->second;
}

// ---- activation scratch (block-fixed-point x), owned by the library ------------------
struct XQScratch {
    uint8_t *base = nullptr;
    size_t cap_k = 0;
    size_t slot_bytes = 0;
};
static XQScratch g_xq;

static size_t xq_slot_bytes(size_t K) { return ((2 * K + K / 8 + K / 4 + 64) + 255) & ~(size_t)255; }

static bool ensure_xq(int K)
{
    if ((size_t)K <= g_xq.cap_k) return true;
    if (g_xq.base) {
        cudaStreamSynchronize(g_stream);
        cudaFree(g_xq.base);
        g_xq.base = nullptr;
        g_xq.cap_k = 0;
    }
    size_t cap = (size_t)K < 32768 ? 32768 : (size_t)K;
    size_t sb = xq_slot_bytes(cap);
    if (cudaMalloc(&g_xq.base, 8 * sb) != cudaSuccess) {   // slots 0-3: cuda_gemv & co; 4-7: the *_q entry points
        cudaGetLastError();
        set_error(QZ_ERR_CUDA, "cudaMalloc of the activation scratch failed");
        return false;
    }
    g_xq.cap_k = cap;
    g_xq.slot_bytes = sb;
    return true;
}

struct XQMut {
    int8_t *xl, *xh;
    float *xs, *xsum;
};
static XQMut xq_slot(uint8_t *base, size_t slot_bytes, int slot, size_t cap_k)
{
    uint8_t *p = base + (size_t)slot * slot_bytes;
    XQMut q;
    q.xl = (int8_t *)p;
    q.xh = (int8_t *)(p + cap_k);
    q.xs = (float *)(p + 2 * cap_k);
    q.xsum = (float *)(p + 2 * cap_k + cap_k / 8 + 32);
    return q;
}

// set by quartz_mgpu_fuse_next_wait: the next activation conversion first waits for the exchange
static const MgpuCtrl *g_wait_ctrl = nullptr;
static int g_wait_ranks = 0;
static int *status_word();

static void launch_quantize(const float *x, const XQMut &q, int K)
{
    int threads = K / 4;
    int bs = 256, gs = (threads + bs - 1) / bs;
    const MgpuCtrl *ctrl = g_wait_ctrl;
    int *st = ctrl ? status_word() : nullptr;
    if (ctrl && !st) ctrl = nullptr;
    g_wait_ctrl = nullptr;
    launch(quantize_x_kernel, dim3(gs), dim3(bs), 0, x, q.xl, q.xh, q.xs, q.xsum, K, ctrl, g_wait_ranks, st);
}

// ---- one-time init: default sign table ------------------------------------------------
static bool g_ksigns_set = false;
static bool g_have_iq2xxs, g_have_iq2xs, g_have_iq2s, g_have_iq3s, g_have_iq3xxs;

static void ensure_ksigns()
{
    if (g_ksigns_set) return;
    // entry i = i with bit 7 set when i has odd parity (even number of minus signs per byte)
    uint8_t t[128];
    for (int i = 0; i < 128; i++) t[i] = (uint8_t)(i | ((__builtin_popcount(i) & 1) << 7));
    QZ_CUDA_CHECK(cudaMemcpyToSymbol(g_ksigns, t, 128));
    g_ksigns_set = true;
}

static bool tables_ready(uint32_t t)
{
    switch (t) {
    case T_IQ2_XXS: ensure_ksigns(); return g_have_iq2xxs;
    case T_IQ2_XS: ensure_ksigns(); return g_have_iq2xs;
    case T_IQ2_S: return g_have_iq2s;
    case T_IQ3_S: return g_have_iq3s;
    case T_IQ3_XXS: ensure_ksigns(); return g_have_iq3xxs;
    default: return true;
    }
}

// ---- dispatch helpers ---------------------------------------------------------------------
#define QZ_FOR_BLOCK_TYPES(X) \
    X(T_Q4_0) X(T_Q4_1) X(T_Q5_0) X(T_Q5_1) X(T_Q8_0) X(T_IQ4_NL) X(T_Q2_K) X(T_Q4_K) X(T_Q5_K) X(T_Q6_K) \
    X(T_IQ2_XXS) X(T_IQ2_XS) X(T_IQ2_S) X(T_IQ3_S) X(T_IQ3_XXS)

static bool is_plain(uint32_t t) { return t == T_F32 || t == T_F16 || t == T_BF16; }

static void launch_generic(uint32_t t, bool planes, const uint8_t *W, const float *x, float *y, int K, int N)
{
    dim3 grid((N + 3) / 4), block(128);
    switch (t) {
#define X(TT)                                                                             \
    case TT:                                                                              \
        if (planes) gemv_generic_kernel<TT, true><<<grid, block, 0, g_stream>>>(W, x, y, K, N);  \
        else gemv_generic_kernel<TT, false><<<grid, block, 0, g_stream>>>(W, x, y, K, N);        \
        break;
        QZ_FOR_BLOCK_TYPES(X)
#undef X
    case T_F32: gemv_plain_kernel<T_F32><<<grid, block, 0, g_stream>>>(W, x, y, K, N); break;
    case T_F16: gemv_plain_kernel<T_F16><<<grid, block, 0, g_stream>>>(W, x, y, K, N); break;
    case T_BF16: gemv_plain_kernel<T_BF16><<<grid, block, 0, g_stream>>>(W, x, y, K, N); break;
    default: break;
    }
    QZ_LAUNCH_CHECK();
}

// Which layout the streaming kernel of a format reads: 0 = no streaming kernel,
// 1 = raw GGUF blocks, 2 = planes.
static int stream_layout(uint32_t t)
{
    switch (t) {
    case T_Q4_K: case T_Q5_K: return 1;
    case T_Q6_K: case T_Q8_0: case T_Q4_0: case T_Q4_1: case T_Q5_0: case T_Q5_1:
    case T_IQ2_XXS: case T_IQ2_XS: case T_IQ2_S: case T_IQ3_XXS: case T_IQ3_S: case T_Q2_K: case T_IQ4_NL: return 2;
    default: return 0;
    }
}

#define QZ_FOR_STREAM_TYPES(X)                                                                              \
    X(T_Q4_K, StreamQ4K) X(T_Q6_K, StreamQ6K) X(T_Q8_0, StreamQ8_0) X(T_Q4_0, StreamQ4_0) X(T_Q4_1, StreamQ4_1) \
    X(T_Q5_0, StreamQ5_0) X(T_Q5_1, StreamQ5_1) X(T_IQ2_XXS, StreamIQ2XXS) X(T_IQ2_XS, StreamIQ2XS)          \
    X(T_IQ2_S, StreamIQ2S) X(T_IQ3_XXS, StreamIQ3XXS) X(T_IQ3_S, StreamIQ3S) X(T_Q5_K, StreamQ5K)               \
    X(T_Q2_K, StreamQ2K) X(T_IQ4_NL, StreamIQ4NL)

// ---- device status word written by kernels whose bounded waits gave up ------------------
static int *g_status = nullptr;
static int *status_word()
{
    if (!g_status) {
        if (cudaMalloc(&g_status, sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            g_status = nullptr;
            set_error(QZ_ERR_CUDA, "cudaMalloc of the status word failed");
            return nullptr;
        }
        cudaMemset(g_status, 0, sizeof(int));
    }
    return g_status;
}
static GridBarrier *g_grid_barrier = nullptr;   // count / generation / abort words of the chained-GEMV kernel
static void poll_status()
{
    if (!g_status) return;
    int h = 0;
    if (cudaMemcpy(&h, g_status, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess && h != 0) {
        set_error(h, "a device-side bounded wait gave up");
        cudaMemset(g_status, 0, sizeof(int));
        if (g_grid_barrier) cudaMemset(g_grid_barrier, 0, sizeof(GridBarrier));
    }
}

static int g_use_tma = -1;
// set by cuda_gemv_push around its GEMV: the TMA kernel takes it as its epilogue and clears `pending`
static PushArgs g_push_args;
static bool g_push_pending = false;
// set by cuda_gemv_rmsnorm / cuda_gemv_swiglu around their GEMV: the TMA kernel converts the activations itself
static XSrc g_xsrc = {0, nullptr, nullptr, 0};
static bool g_xsrc_pending = false;
// set by quartz_prefetch_next: ranges the next streaming GEMV pulls into L2 behind its own weight stream
static PrefetchHint g_pf = {{nullptr, nullptr, nullptr, nullptr}, {0, 0, 0, 0}, 0};
// set by cuda_gemv_experts around its GEMV: the matrices are expert slices picked by device-side ids
static const int *g_sel = nullptr;
static size_t g_sel_stride = 0;
// longest activation vector the streaming GEMV converts in its own prologue (every CTA converts the whole
// vector while its weight ring fills); longer vectors are converted once, by a kernel of their own.
// QUARTZ_XSRC_MAX_K overrides the default.
static int xsrc_max_k()
{
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("QUARTZ_XSRC_MAX_K");
        v = e ? atoi(e) : 8192;
        if (v < 0) v = 0;
    }
    return v;
}
static bool use_tma()
{
    if (g_use_tma < 0) {
        const char *e = getenv("QUARTZ_GEMV_IMPL");   // "ldg" selects the register-streaming kernel
        g_use_tma = (e && std::string(e) == "ldg") ? 0 : 1;
    }
    return g_use_tma == 1;
}

template <class F>
static bool launch_tma(const GemvArgs &g, int n_mats)
{
    const FormatInfo fi = format_info(F::TYPE);
    const size_t row_bytes = (size_t)(g.K / fi.block_elems) * fi.block_bytes;
    TmaArgs a;
    for (int i = 0; i < QZ_MAX_MATS; i++) { a.W[i] = g.W[i]; a.xq[i] = g.xq[i]; a.y[i] = g.y[i]; }
    a.accumulate = g.accumulate;
    a.K = g.K; a.N = g.N; a.U = g.U; a.Upad = g.Upad; a.n_mats = n_mats;
    // consumer threads per CTA: 512 (one CTA per SM), or 256 with two CTAs per SM when the row fits
    // (QUARTZ_GEMV_CONSUMERS=256): the CTAs of the next kernel of a chain then become resident, and start
    // streaming, while this kernel's CTAs are still draining
    static int cons_pref = -1;
    if (cons_pref < 0) {
        const char *e = getenv("QUARTZ_GEMV_CONSUMERS");
        cons_pref = (e && atoi(e) == 256) ? 256 : TMA_CONSUMERS;
    }
    const int cons = (cons_pref == 256 && g.Upad <= 256) ? 256 : TMA_CONSUMERS;
    const int per_sm = cons == 256 ? 2 : 1;
    a.RP = g.Upad >= cons ? 1 : cons / g.Upad;
    const int sms = sm_count() * per_sm;
    const int ctas_per_mat = sms / n_mats > 0 ? sms / n_mats : 1;
    a.stage_bytes = (int)((size_t)a.RP * row_bytes);
    const int smem_budget = (per_sm == 2 ? 100 : 200) * 1024;   // + up to 8 KB of codebook behind it
    // a fused activation source keeps the converted vector (2 K + 3 K / 8 bytes) behind the codebook
    const int x_bytes = g_xsrc_pending ? (int)((2 * (size_t)g.K + g.K / 8 + g.K / 4 + 31) & ~(size_t)15) : 0;
    const int ring_budget = smem_budget - x_bytes;
    if (a.stage_bytes * 2 > ring_budget) return false;
    if (g_xsrc_pending && g.K / 4 > XSRC_MAX_IT * a.Upad * a.RP) return false;   // the prologue holds the vector in registers
    const int ntiles = (g.N + a.RP - 1) / a.RP;
    const int n_cta = ntiles < ctas_per_mat ? ntiles : ctas_per_mat;
    int stages = ring_budget / a.stage_bytes;
    if (stages > TMA_MAX_STAGES) stages = TMA_MAX_STAGES;
    const int need = (ntiles + n_cta - 1) / n_cta;
    if (stages > need) stages = need;
    if (stages < 1) stages = 1;
    a.n_stages = stages;
    a.status = status_word();
    if (!a.status) return false;
    a.push.n = 0;
    if (g_push_pending && n_mats == 1 && !g.accumulate) {
        a.push = g_push_args;
        g_push_pending = false;
    }
    a.xsrc.mode = 0;
    if (g_xsrc_pending) {
        a.xsrc = g_xsrc;
        g_xsrc_pending = false;
    }
    a.pf = g_pf;
    g_pf.n = 0;
    a.sel = g_sel;
    a.sel_stride = g_sel_stride;
    static bool attr_set = false;
    if (!attr_set) {
        QZ_CUDA_CHECK(cudaFuncSetAttribute(gemv_tma_kernel<F, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024 + 16 + F::TABLE_BYTES));
        QZ_CUDA_CHECK(cudaFuncSetAttribute(gemv_tma_kernel<F, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024 + 16 + F::TABLE_BYTES));
        QZ_CUDA_CHECK(cudaFuncSetAttribute(gemv_tma_kernel<F, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024 + 16 + F::TABLE_BYTES));
        attr_set = true;
    }
    const dim3 grid(n_cta * n_mats), block(cons + 32);
    const size_t smem = (size_t)stages * a.stage_bytes + ((F::TABLE_BYTES + 15) & ~15) + x_bytes;
    if (g.Upad < 32) launch(gemv_tma_kernel<F, 0>, grid, block, smem, a);
    else if (g.Upad == 32) launch(gemv_tma_kernel<F, 1>, grid, block, smem, a);
    else launch(gemv_tma_kernel<F, 2>, grid, block, smem, a);
    return true;
}

template <class F>
static void launch_stream_r(const GemvArgs &a, int n_mats, int T)
{
    const int sms = sm_count();
    // rows per thread: as many as keep at least ~2 tiles per SM
    int R = 4;
    while (R > 1 && (long long)(a.N + a.RP * R - 1) / (a.RP * R) * n_mats < 2LL * sms) R >>= 1;
    const int ntiles = (a.N + a.RP * R - 1) / (a.RP * R);
    int per_sm = (T <= 256) ? 3 : 1;
    int gx = ntiles < sms * per_sm ? ntiles : sms * per_sm;
    if (gx < 1) gx = 1;
    dim3 grid(gx, n_mats), block(T);
    if (R == 4) launch(gemv_stream_kernel<F, 4>, grid, block, 0, a);
    else if (R == 2) launch(gemv_stream_kernel<F, 2>, grid, block, 0, a);
    else launch(gemv_stream_kernel<F, 1>, grid, block, 0, a);
}

static bool stream_shape_ok(uint32_t t, int K)
{
    if (!stream_layout(t) || K % 64 != 0 || K / 64 > 512) return false;
    const FormatInfo fi = format_info(t);
    return ((size_t)(K / fi.block_elems) * fi.block_bytes) % 16 == 0;
}

// Launch the streaming GEMV for n same-shape matrices whose activations already sit in the
// scratch slots slot_of[i].
static bool stream_core(uint32_t t, int n, const uint8_t *const *W, const int *slot_of, float *const *y, int K, int N,
                        int accumulate)
{
    GemvArgs a;
    a.K = K;
    a.N = N;
    a.accumulate = accumulate;
    a.U = K / 64;
    if (a.U < 32) {
        int p = 1;
        while (p < a.U) p <<= 1;
        a.Upad = p;
    } else {
        a.Upad = (a.U + 31) & ~31;
    }
    a.RP = a.Upad >= 256 ? 1 : 256 / a.Upad;
    const int T = a.Upad * a.RP;
    for (int i = 0; i < QZ_MAX_MATS; i++) {
        int j = i < n ? i : 0;
        XQMut q = xq_slot(g_xq.base, g_xq.slot_bytes, slot_of[j], g_xq.cap_k);
        a.W[i] = W[j];
        a.y[i] = y[j];
        a.xq[i] = XQ{q.xl, q.xh, q.xs, q.xsum};
    }
    if (use_tma()) {
        bool done = false;
        switch (t) {
#define X(TT, POL) case TT: done = launch_tma<POL>(a, n); break;
            QZ_FOR_STREAM_TYPES(X)
#undef X
        default: break;
        }
        if (done) return true;
    }
    if (g_xsrc_pending) return false;   // only the TMA kernel converts activations itself: let the caller do it
    switch (t) {
#define X(TT, POL) case TT: launch_stream_r<POL>(a, n, T); break;
        QZ_FOR_STREAM_TYPES(X)
#undef X
    default: return false;
    }
    return true;
}

// Streaming path for up to four same-shape GEMVs.  Returns false when the shape or the
// pointers do not qualify (the caller then falls back to the any-shape kernels).
static bool try_stream(uint32_t t, int n, const uint8_t *const *W, const float *const *x, float *const *y, int K,
                       int N, const bool *planes)
{
    if (!stream_shape_ok(t, K)) return false;
    const int want = stream_layout(t);
    for (int i = 0; i < n; i++) {
        if (((uintptr_t)W[i] & 15) || ((uintptr_t)x[i] & 3)) return false;
        if ((want == 2) != planes[i]) return false;
    }
    if (!ensure_xq(K)) return false;
    int slot_of[4];
    int n_slots = 0;
    // one activation vector for all matrices: the TMA kernel converts it in its own prologue (no launch of its
    // own for the conversion), unless the conversion kernel is needed as the carrier of a fused exchange wait
    bool same_x = true;
    for (int i = 1; i < n; i++) same_x = same_x && x[i] == x[0];
    if (same_x && use_tma() && !g_wait_ctrl && K <= xsrc_max_k() && !((uintptr_t)x[0] & 15)) {
        for (int i = 0; i < n; i++) slot_of[i] = 0;
        g_xsrc = XSrc{3, x[0], x[0], 0};
        g_xsrc_pending = true;
        const bool ok = stream_core(t, n, W, slot_of, y, K, N, 0);
        const bool consumed = !g_xsrc_pending;
        g_xsrc_pending = false;
        if (ok && consumed) return true;
    }
    // otherwise: quantize each distinct activation vector once
    for (int i = 0; i < n; i++) {
        int s = -1;
        for (int j = 0; j < i; j++)
            if (x[j] == x[i]) { s = slot_of[j]; break; }
        if (s < 0) {
            s = n_slots++;
            launch_quantize(x[i], xq_slot(g_xq.base, g_xq.slot_bytes, s, g_xq.cap_k), K);
        }
        slot_of[i] = s;
    }
    return stream_core(t, n, W, slot_of, y, K, N, 0);
}

static bool check_shape(uint32_t t, int K, int N, const char *who)
{
    const FormatInfo fi = format_info(t);
    if (fi.block_elems == 0) return false;
    if (K <= 0 || N < 0 || K % fi.block_elems != 0) {
        set_error(QZ_ERR_BAD_SHAPE, who);
        return false;
    }
    return true;
}

static void gemv_n(uint32_t t, int n, const uint8_t *const *W, const float *const *x, float *const *y, int K, int N)
{
    const FormatInfo fi = format_info(t);
    if (fi.block_elems == 0) {
        // reference behaviour (src/cuda_kernels.cu:1073-1077): zero the output, complain on stderr
        for (int i = 0; i < n; i++)
            if (N > 0) QZ_CUDA_CHECK(cudaMemsetAsync(y[i], 0, (size_t)N * sizeof(float), g_stream));
        fprintf(stderr, "cuda_gemv: unsupported ggml_type %u\n", t);
        set_error(QZ_ERR_UNSUPPORTED_TYPE, "cuda_gemv: unsupported ggml_type");
        return;
    }
    if (!check_shape(t, K, N, "cuda_gemv: in_dim must be a positive multiple of the block size") || N == 0) return;
    if (!tables_ready(t)) {
        for (int i = 0; i < n; i++) QZ_CUDA_CHECK(cudaMemsetAsync(y[i], 0, (size_t)N * sizeof(float), g_stream));
        set_error(QZ_ERR_MISSING_TABLE, "IQ codebook not uploaded (cuda_set_*_grid)");
        return;
    }
    bool planes[4] = {false, false, false, false};
    for (int i = 0; i < n; i++) {
        const Range *r = find_range(W[i]);
        if (r) {
            if (r->type != t || r->K != K) {
                set_error(QZ_ERR_BAD_SHAPE, "cuda_gemv: pointer lies in a repacked range of another type/in_dim");
                return;
            }
            planes[i] = true;
        }
    }
    if (!is_plain(t) && try_stream(t, n, W, x, y, K, N, planes)) {
        g_pf.n = 0;
        return;
    }
    g_pf.n = 0;   // a prefetch hint applies to the streaming kernel only
    if (g_wait_ctrl) {   // a fused wait was asked for, but this path converts no activations: wait in a kernel of its own
        int *st = status_word();
        if (st) {
            mgpu_wait_kernel<<<1, 32, 0, g_stream>>>(g_wait_ctrl, g_wait_ranks, st);
            QZ_LAUNCH_CHECK();
        }
        g_wait_ctrl = nullptr;
    }
    for (int i = 0; i < n; i++) launch_generic(t, planes[i], W[i], x[i], y[i], K, N);
}

static void dequant_rows(uint32_t t, const uint8_t *data, float *out, int K, long long rows, const int *row_sel = nullptr)
{
    const FormatInfo fi = format_info(t);
    if (fi.block_elems == 0) {
        set_error(QZ_ERR_UNSUPPORTED_TYPE, "cuda_dequant: unsupported ggml_type");
        return;
    }
    if (!check_shape(t, K, 0, "cuda_dequant: in_dim must be a positive multiple of the block size") || rows <= 0) return;
    if (!tables_ready(t)) {
        set_error(QZ_ERR_MISSING_TABLE, "IQ codebook not uploaded (cuda_set_*_grid)");
        return;
    }
    if (is_plain(t)) {
        long long n = rows * K;
        launch(dequant_plain_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, data, out, t, n, row_sel, K);
        return;
    }
    const Range *r = find_range(data);
    bool planes = false;
    if (r) {
        if (r->type != t || r->K != K) {
            set_error(QZ_ERR_BAD_SHAPE, "cuda_dequant: pointer lies in a repacked range of another type/in_dim");
            return;
        }
        planes = true;
    }
    long long n_sub = rows * (K / 32);
    unsigned grid = (unsigned)((n_sub + 127) / 128);
    switch (t) {
#define X(TT)                                                                                                \
    case TT:                                                                                                 \
        if (planes) launch(dequant_kernel<TT, true>, dim3(grid), dim3(128), 0, data, out, K, n_sub, row_sel);  \
        else launch(dequant_kernel<TT, false>, dim3(grid), dim3(128), 0, data, out, K, n_sub, row_sel);        \
        break;
        QZ_FOR_BLOCK_TYPES(X)
#undef X
    default: break;
    }
}

// ---- allocation-free GEMV: scratch that lives in the library image -------------------------
// Some hosts may not call cudaMalloc at the moment they need a GEMV: a thread that is in the
// middle of a CUDA stream capture, a real-time or sandboxed caller whose memory is fixed up
// front, or a process that has handed the whole device pool to another allocator.  For them
// the converted activation vector (the only scratch the streaming GEMV needs) lives in this
// file-scope device array instead of a lazily cudaMalloc'ed buffer.  One slot: in_dim <=
// QZ_NOALLOC_MAX_K.  Every GPU that loads the library carries these 78,080 bytes until exit.
constexpr int QZ_NOALLOC_MAX_K = 32768;
constexpr size_t QZ_NOALLOC_BYTES = 2 * (size_t)QZ_NOALLOC_MAX_K + QZ_NOALLOC_MAX_K / 8 + QZ_NOALLOC_MAX_K / 4 + 256;
static __device__ __align__(256) unsigned char qz_noalloc_scratch[QZ_NOALLOC_BYTES];

// In host code `qz_noalloc_scratch` is only a handle for the runtime, not a device address;
// the address a kernel can use comes from cudaGetSymbolAddress, per device.
static unsigned char *g_noalloc_ptr[64];

static unsigned char *noalloc_scratch_ptr()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        set_error(QZ_ERR_CUDA, "cuda_gemv_noalloc: cudaGetDevice failed");
        return nullptr;
    }
    if (!g_noalloc_ptr[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, qz_noalloc_scratch);
        if (e != cudaSuccess || !p) {
            cudaGetLastError();
            set_error(QZ_ERR_CUDA, "cuda_gemv_noalloc: cudaGetSymbolAddress failed");
            return nullptr;
        }
        g_noalloc_ptr[dev] = (unsigned char *)p;
    }
    return g_noalloc_ptr[dev];
}

template <class F>
static void launch_noalloc(const GemvArgs &a, int T)
{
    const int sms = sm_count();
    int R = 4;
    while (R > 1 && (long long)(a.N + a.RP * R - 1) / (a.RP * R) < 2LL * sms) R >>= 1;
    const int ntiles = (a.N + a.RP * R - 1) / (a.RP * R);
    const int per_sm = (T <= 256) ? 2 : 1;
    int gx = ntiles < sms * per_sm ? ntiles : sms * per_sm;
    if (gx < 1) gx = 1;
    if (R == 4) gemv_stream_kernel<F, 4><<<gx, T, 0, g_stream>>>(a);
    else if (R == 2) gemv_stream_kernel<F, 2><<<gx, T, 0, g_stream>>>(a);
    else gemv_stream_kernel<F, 1><<<gx, T, 0, g_stream>>>(a);
    QZ_LAUNCH_CHECK();
}

static void gemv_noalloc(uint32_t t, const uint8_t *W, const float *x, float *y, int K, int N)
{
    const FormatInfo fi = format_info(t);
    if (fi.block_elems == 0) {
        set_error(QZ_ERR_UNSUPPORTED_TYPE, "cuda_gemv_noalloc: unsupported ggml_type");
        return;
    }
    if (!check_shape(t, K, N, "cuda_gemv_noalloc: in_dim must be a positive multiple of the block size")) return;
    if (K > QZ_NOALLOC_MAX_K) {
        set_error(QZ_ERR_TOO_LARGE, "cuda_gemv_noalloc: in_dim exceeds the 32768 the built-in scratch holds");
        return;
    }
    if (N == 0) return;
    if (!tables_ready(t)) {
        set_error(QZ_ERR_MISSING_TABLE, "IQ codebook not uploaded (cuda_set_*_grid)");
        return;
    }
    bool planes = false;
    if (const Range *r = find_range(W)) {
        if (r->type != t || r->K != K) {
            set_error(QZ_ERR_BAD_SHAPE, "cuda_gemv_noalloc: pointer lies in a repacked range of another type/in_dim");
            return;
        }
        planes = true;
    }
    if (g_wait_ctrl) {
        // This entry point never carries a fused exchange wait (that path would create the status word with
        // cudaMalloc): the pending wait runs as a kernel of its own when the status word exists already, and
        // is refused otherwise.
        if (g_status) {
            mgpu_wait_kernel<<<1, 32, 0, g_stream>>>(g_wait_ctrl, g_wait_ranks, g_status);
            QZ_LAUNCH_CHECK();
        } else {
            set_error(QZ_ERR_BAD_SHAPE, "cuda_gemv_noalloc: a fused exchange wait is pending but cannot be carried without allocating; call quartz_mgpu_wait instead");
        }
        g_wait_ctrl = nullptr;
    }
    const int want = stream_layout(t);
    const size_t row_bytes = (size_t)(K / fi.block_elems) * fi.block_bytes;
    const bool streamable = want && K % 64 == 0 && K / 64 <= 512 && row_bytes % 16 == 0 && !((uintptr_t)W & 15) &&
                            !((uintptr_t)x & 3) && ((want == 2) == planes);
    if (!streamable) {
        launch_generic(t, planes, W, x, y, K, N);   // needs no scratch at all
        return;
    }
    unsigned char *base = noalloc_scratch_ptr();
    if (!base) return;
    // nothing in the scratch has to start at zero: the conversion below rewrites every byte
    // of [0, K) that the GEMV kernel reads, whatever an earlier call left there
    XQMut q;
    q.xl = (int8_t *)base;
    q.xh = (int8_t *)(base + QZ_NOALLOC_MAX_K);
    q.xs = (float *)(base + 2 * (size_t)QZ_NOALLOC_MAX_K);
    q.xsum = (float *)(base + 2 * (size_t)QZ_NOALLOC_MAX_K + QZ_NOALLOC_MAX_K / 8);
    launch_quantize(x, q, K);
    GemvArgs a;
    a.K = K;
    a.N = N;
    a.U = K / 64;
    if (a.U < 32) {
        int p = 1;
        while (p < a.U) p <<= 1;
        a.Upad = p;
    } else {
        a.Upad = (a.U + 31) & ~31;
    }
    a.RP = a.Upad >= 256 ? 1 : 256 / a.Upad;
    a.accumulate = 0;
    for (int i = 0; i < QZ_MAX_MATS; i++) {
        a.W[i] = W;
        a.y[i] = y;
        a.xq[i] = XQ{q.xl, q.xh, q.xs, q.xsum};
    }
    const int T = a.Upad * a.RP;
    switch (t) {
#define X(TT, POL) case TT: launch_noalloc<POL>(a, T); break;
        QZ_FOR_STREAM_TYPES(X)
#undef X
    default: break;
    }
}

// ---- batched GEMM on tcgen05 ------------------------------------------------------------------
static __nv_bfloat16 *g_xb = nullptr;   // bf16 copy of the activation tile (library scratch, grows)
static size_t g_xb_elems = 0;
// row-sharded GEMM (cuda_gemm_push) when tiles are scarce: the block is computed into this scratch and copied out
static float *g_gemm_ys = nullptr;
static size_t g_gemm_ys_elems = 0;
static bool ensure_gemm_push_scratch(size_t y_elems)
{
    if (y_elems <= g_gemm_ys_elems) return true;
    if (g_gemm_ys) {
        cudaStreamSynchronize(g_stream);
        cudaFree(g_gemm_ys);
    }
    if (cudaMalloc(&g_gemm_ys, y_elems * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        g_gemm_ys = nullptr;
        g_gemm_ys_elems = 0;
        set_error(QZ_ERR_CUDA, "cuda_gemm_push: cudaMalloc of the local output scratch failed");
        return false;
    }
    g_gemm_ys_elems = y_elems;
    return true;
}

template <uint32_t T, bool PLANES, int HALVES>
static void launch_gemm(GemmArgs a)
{
    // shared-memory plan: as many ring stages as fit (at most GEMM_STAGES).  Small token tiles stay
    // under half an SM's shared memory so that two CTAs are resident (the unpack is ALU-heavy and
    // wants the warps); large tiles take the SM.
    const int stage_bytes = HALVES * GEMM_ROWS * 128 + ((a.tok_tile * 128 + 1023) & ~1023);
    const bool two = gemm_fast_type<T, PLANES>() && HALVES == 1 && a.tok_tile <= 64;
    constexpr int table_bytes = AProd<T, PLANES>::TABLE_BYTES;
    const int budget = (two ? 110 : 200) * 1024 - table_bytes;
    a.stages = budget / stage_bytes;
    if (a.stages > GEMM_STAGES) a.stages = GEMM_STAGES;
    const size_t smem = (size_t)a.stages * stage_bytes + table_bytes;
    static bool attr_set = false;
    if (!attr_set) {
        QZ_CUDA_CHECK(cudaFuncSetAttribute(gemm_tc_kernel<T, PLANES, HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           216 * 1024));
        attr_set = true;
    }
    // work split over the resident CTAs: first as many whole tiles as every CTA can get, then one equal
    // share of the remaining (tile, K step) units per CTA, at least 8 units each.  Only tiles of that
    // second part can be shared between CTAs (zeroed here, added atomically by the kernel).
    const int cta_rows = HALVES * GEMM_ROWS, ksteps = a.K / GEMM_KSTEP;
    const long long tiles = (long long)((a.N + cta_rows - 1) / cta_rows) * a.n_tok_tiles;
    a.units = tiles * ksteps;
    long long ctas = (long long)sm_count() * (two ? 2 : 1);
    const long long whole = tiles / ctas;
    if (whole == 0 && ctas > (a.units + 7) / 8) ctas = (a.units + 7) / 8;
    a.dp_units = whole * ksteps;
    a.rem_begin = ctas * a.dp_units;
    const long long rem = a.units - a.rem_begin;
    long long sharers = ctas;
    if (sharers > (rem + 7) / 8) sharers = (rem + 7) / 8;
    a.units_per_cta = sharers > 0 ? (rem + sharers - 1) / sharers : 0;
    bool zero_shared = rem > 0;
    PushArgs copy_out;
    copy_out.n = 0;
    if (a.push.n > 0 && (whole >= 1 || (tiles * 2 >= ctas && ksteps <= 64))) {
        // row-sharded with about one tile per CTA or more: whole tiles only (the tiles left over after the equal part
        // go one each to the first CTAs), so every tile goes to the peers straight from its accumulator
        if (whole == 0) {
            ctas = tiles;
            a.dp_units = 0;
            a.rem_begin = 0;
        }
        a.units_per_cta = ksteps;
        zero_shared = false;
    } else if (a.push.n > 0) {
        // tiles are scarce: sharing them between CTAs (K-wise) matters more than the fused epilogue.  The block is
        // summed in local scratch as usual and a copy kernel stores it into the windows (measured faster than
        // having the completing warp of every shared tile read its sums back and push them)
        copy_out = a.push;
        a.push.n = 0;
    }
    if (whole == 0 && a.push.n == 0) ctas = (a.units + a.units_per_cta - 1) / a.units_per_cta;
    if (zero_shared) {
        // narrow token tiles are a few KB per tile: one block each; wide ones are split over up to 8
        const unsigned zero_slices = (unsigned)std::max(1, std::min(8, a.tok_tile / 32));
        gemm_zero_split_tiles_kernel<<<dim3((unsigned)ctas, zero_slices), 256, 0, g_stream>>>(a.Y, a.M, a.N, ksteps, a.n_tok_tiles, a.tok_tile,
                                                                                 cta_rows, a.units, a.rem_begin, a.units_per_cta);
        QZ_LAUNCH_CHECK();
    }
    gemm_tc_kernel<T, PLANES, HALVES><<<(unsigned)ctas, gemm_threads<HALVES>(), smem, g_stream>>>(a);
    QZ_LAUNCH_CHECK();
    if (copy_out.n > 0) {
        const long long total = (long long)a.M * a.N;
        int blocks = (int)((total / 4 + 255) / 256);
        if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
        if (blocks < 1) blocks = 1;
        const bool wait_after = copy_out.wait_after != 0;
        copy_out.wait_after = 0;
        mgpu_push_rows_kernel<<<blocks, 256, 0, g_stream>>>(a.Y, a.M, a.N, a.push_ld, copy_out);
        QZ_LAUNCH_CHECK();
        if (wait_after) {   // (this form has no kernel that could carry the wait)
            mgpu_wait_kernel<<<1, 32, 0, g_stream>>>((const MgpuCtrl *)copy_out.ctrl[copy_out.rank], copy_out.n, a.status);
            QZ_LAUNCH_CHECK();
        }
    }
}

template <uint32_t T, bool PLANES>
static void launch_gemm_type(const GemmArgs &a, int halves)
{
    if constexpr (gemm_fast_type<T, PLANES>()) {
        if (halves == 2) {
            launch_gemm<T, PLANES, 2>(a);
            return;
        }
    }
    launch_gemm<T, PLANES, 1>(a);
}

// Grouped form (a.grp set): the tile count is known on the device only, so the grid is the resident CTA count
// and the kernel splits the work itself; outputs must be zero beforehand (shared tiles are added atomically).
template <uint32_t T, bool PLANES>
static void launch_gemm_grouped(GemmArgs a)
{
    const int stage_bytes = GEMM_ROWS * 128 + ((a.tok_tile * 128 + 1023) & ~1023);
    const bool two = gemm_fast_type<T, PLANES>();
    constexpr int table_bytes = AProd<T, PLANES>::TABLE_BYTES;
    const int budget = (two ? 110 : 200) * 1024 - table_bytes;
    a.stages = budget / stage_bytes;
    if (a.stages > GEMM_STAGES) a.stages = GEMM_STAGES;
    const size_t smem = (size_t)a.stages * stage_bytes + table_bytes;
    static bool attr_set = false;
    if (!attr_set) {
        QZ_CUDA_CHECK(cudaFuncSetAttribute(gemm_tc_kernel<T, PLANES, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 216 * 1024));
        attr_set = true;
    }
    const unsigned ctas = (unsigned)(sm_count() * (two ? 2 : 1));
    gemm_tc_kernel<T, PLANES, 1><<<ctas, gemm_threads<1>(), smem, g_stream>>>(a);
    QZ_LAUNCH_CHECK();
}

static void gemm_grouped_dispatch(uint32_t t, bool planes, const GemmArgs &a)
{
    switch (t) {
#define X(TT)                                               \
    case TT:                                                \
        if (planes) launch_gemm_grouped<TT, true>(a);       \
        else launch_gemm_grouped<TT, false>(a);             \
        break;
        QZ_FOR_BLOCK_TYPES(X)
#undef X
    default: break;
    }
}

// push != nullptr: row-sharded form (cuda_gemm_push): returns false, having launched nothing, when the tensor-core
// kernel does not take the shape
static bool gemm_dispatch(uint32_t t, const uint8_t *W, const void *xv, float *y, int M, int K, int N, bool x_bf16 = false,
                          const PushArgs *push = nullptr, long long push_off = 0, long long push_ld = 0)
{
    const float *x = (const float *)xv;   // (bf16 input: only the tensor-core path below reads it)
    if (M <= 0 || N <= 0) return false;
    const FormatInfo fi = format_info(t);
    // n == 1 is the GEMV (src/dequant.rs:151-153); shapes/types the tensor-core kernel does not take
    // run token by token (what the reference's GPU prefill does, src/main.rs:1410-1416)
    const bool tc_ok = fi.block_elems >= 32 && K > 0 && K % GEMM_KSTEP == 0 && !((uintptr_t)W & 15) &&
                       !((uintptr_t)x & 15) && (((size_t)(K / fi.block_elems) * fi.block_bytes) % 16 == 0);
    if (x_bf16 && !tc_ok) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_gemm_bf16: in_dim must be a multiple of 64 and the pointers 16-byte aligned");
        return false;
    }
    if (push && (M == 1 || !tc_ok)) return false;
    if (!x_bf16 && (M == 1 || !tc_ok)) {
        for (int tkn = 0; tkn < M; tkn++) {
            const uint8_t *Wp[1] = {W};
            const float *xp[1] = {x + (size_t)tkn * K};
            float *yp[1] = {y + (size_t)tkn * N};
            gemv_n(t, 1, Wp, xp, yp, K, N);
        }
        return true;
    }
    if (!tables_ready(t)) {
        if (!push) QZ_CUDA_CHECK(cudaMemsetAsync(y, 0, (size_t)M * N * sizeof(float), g_stream));
        set_error(QZ_ERR_MISSING_TABLE, "IQ codebook not uploaded (cuda_set_*_grid)");
        return false;
    }
    bool planes = false;
    if (const Range *r = find_range(W)) {
        if (r->type != t || r->K != K) {
            set_error(QZ_ERR_BAD_SHAPE, "cuda_gemm: pointer lies in a repacked range of another type/in_dim");
            return false;
        }
        planes = true;
    }
    GemmArgs a = {};
    a.grp = nullptr;
    a.W = W; a.Y = y; a.M = M; a.K = K; a.N = N; a.planes = planes;
    a.tok_tile = M >= GEMM_MAX_TOKENS ? GEMM_MAX_TOKENS : ((M + 15) & ~15);
    a.n_tok_tiles = (M + a.tok_tile - 1) / a.tok_tile;
    const int m_pad = a.n_tok_tiles * a.tok_tile;
    const size_t need = (size_t)m_pad * K;
    if (need > g_xb_elems) {
        if (g_xb) {
            cudaStreamSynchronize(g_stream);
            cudaFree(g_xb);
        }
        if (cudaMalloc(&g_xb, need * sizeof(__nv_bfloat16)) != cudaSuccess) {
            cudaGetLastError();
            g_xb = nullptr;
            g_xb_elems = 0;
            set_error(QZ_ERR_CUDA, "cudaMalloc of the bf16 activation scratch failed");
            return false;
        }
        g_xb_elems = need;
    }
    a.Xb = g_xb;
    const long long chunks = (long long)need / 8;   // one thread per 16-byte chunk
    // the Q6_K producer emits each block's weights in its own K order; the activation tiles follow it
    const int perm = (t == T_Q6_K && planes) ? 1 : 0;
    if (x_bf16)
        convert_x_bf16_kernel<true><<<(unsigned)((chunks + 255) / 256), 256, 0, g_stream>>>(xv, g_xb, M, K, a.tok_tile,
                                                                                            a.n_tok_tiles, perm);
    else
        convert_x_bf16_kernel<false><<<(unsigned)((chunks + 255) / 256), 256, 0, g_stream>>>(xv, g_xb, M, K, a.tok_tile,
                                                                                             a.n_tok_tiles, perm);
    QZ_LAUNCH_CHECK();
    // 256-row CTA tiles (two accumulators) halve the activation bytes each CTA pulls from L2 per
    // flop; they pay off once the token tile is wide enough for that traffic to matter
    const bool fast = (t == T_Q4_K && !planes) || (planes && (t == T_Q6_K || t == T_IQ2_XS || t == T_IQ3_XXS));
    const int halves = (fast && a.tok_tile >= 128) ? 2 : 1;
    a.status = status_word();
    if (!a.status) return false;
    a.push.n = 0;
    if (push) {
        if (!ensure_gemm_push_scratch((size_t)m_pad * N)) return false;
        a.push = *push;
        a.push_off = push_off;
        a.push_ld = push_ld;
        a.Y = g_gemm_ys;
    }
    switch (t) {
#define X(TT)                                              \
    case TT:                                               \
        if (planes) launch_gemm_type<TT, true>(a, halves); \
        else launch_gemm_type<TT, false>(a, halves);       \
        break;
        QZ_FOR_BLOCK_TYPES(X)
#undef X
    default: break;
    }
    return true;
}

}  // namespace qz

using namespace qz;

extern "C" {

// ======================= Part 1 =======================

void cuda_gemv(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, float *d_y, int in_dim, int out_dim)
{
    gemv_n(ggml_type, 1, &d_data, &d_x, &d_y, in_dim, out_dim);
}

void cuda_gemv_moe4(uint32_t ggml_type, const uint8_t *w0, const uint8_t *w1, const uint8_t *w2, const uint8_t *w3,
                    const float *xi0, const float *xi1, const float *xi2, const float *xi3, float *o0, float *o1,
                    float *o2, float *o3, int n_act, int in_dim, int out_dim)
{
    const uint8_t *W[4] = {w0, w1, w2, w3};
    const float *x[4] = {xi0, xi1, xi2, xi3};
    float *y[4] = {o0, o1, o2, o3};
    if (n_act <= 0) return;
    if (n_act > 4) n_act = 4;
    gemv_n(ggml_type, n_act, W, x, y, in_dim, out_dim);
}

void cuda_set_iq3s_grid(const uint32_t *host)
{
    QZ_CUDA_CHECK(cudaMemcpyToSymbol(g_iq3s_grid, host, 512 * sizeof(uint32_t)));
    g_have_iq3s = true;
}
void cuda_set_iq2s_grid(const uint64_t *host)
{
    QZ_CUDA_CHECK(cudaMemcpyToSymbol(g_iq2s_grid, host, 1024 * sizeof(uint64_t)));
    g_have_iq2s = true;
}
void cuda_set_iq2xxs_grid(const uint64_t *host)
{
    QZ_CUDA_CHECK(cudaMemcpyToSymbol(g_iq2xxs_grid, host, 256 * sizeof(uint64_t)));
    g_have_iq2xxs = true;
}
void cuda_set_iq2xs_grid(const uint64_t *host)
{
    QZ_CUDA_CHECK(cudaMemcpyToSymbol(g_iq2xs_grid, host, 512 * sizeof(uint64_t)));
    g_have_iq2xs = true;
}
void cuda_set_ksigns(const uint8_t *host)
{
    QZ_CUDA_CHECK(cudaMemcpyToSymbol(g_ksigns, host, 128));
    g_ksigns_set = true;
}
void cuda_set_iq3xxs_grid(const uint32_t *host)
{
    QZ_CUDA_CHECK(cudaMemcpyToSymbol(g_iq3xxs_grid, host, 256 * sizeof(uint32_t)));
    g_have_iq3xxs = true;
}

void cuda_mem_info(size_t *free_b, size_t *total_b) { QZ_CUDA_CHECK(cudaMemGetInfo(free_b, total_b)); }

void *cuda_alloc(size_t bytes)
{
    void *p = nullptr;
    if (cudaMalloc(&p, bytes) != cudaSuccess) {
        cudaGetLastError();   // the caller checks for NULL (src/cuda.rs:79, 224); not a sticky error
        return nullptr;
    }
    return p;
}

void cuda_drop(void *p)
{
    if (!p) return;
    // forget repacked ranges that start inside this allocation's base
    auto it = g_ranges.find((uintptr_t)p);
    if (it != g_ranges.end()) g_ranges.erase(it);
    QZ_CUDA_CHECK(cudaFree(p));
}

void cuda_h2d(void *dst, const void *src, size_t bytes)
{
    if (g_stream == 0) {
        QZ_CUDA_CHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice));
    } else {
        QZ_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, g_stream));
        QZ_CUDA_CHECK(cudaStreamSynchronize(g_stream));
    }
}

void cuda_d2h(void *dst, const void *src, size_t bytes)
{
    if (g_stream == 0) {
        QZ_CUDA_CHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost));
    } else {
        QZ_CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, g_stream));
        QZ_CUDA_CHECK(cudaStreamSynchronize(g_stream));
    }
}

void cuda_sync(void)
{
    QZ_CUDA_CHECK(cudaDeviceSynchronize());
    poll_status();
}

// Asynchronous forms of cuda_h2d / cuda_d2h for page-locked host buffers: enqueued on the library's stream, so
// they are ordered with the kernels and can be recorded into a graph (quartz_graph_begin/end).  The host must
// not touch the buffer before a later cuda_sync().
void cuda_h2d_async(void *dst, const void *src_pinned, size_t bytes)
{
    QZ_CUDA_CHECK(cudaMemcpyAsync(dst, src_pinned, bytes, cudaMemcpyHostToDevice, g_stream));
}
void cuda_d2h_async(void *dst_pinned, const void *src, size_t bytes)
{
    QZ_CUDA_CHECK(cudaMemcpyAsync(dst_pinned, src, bytes, cudaMemcpyDeviceToHost, g_stream));
}
void *cuda_host_alloc(size_t bytes)
{
    void *p = nullptr;
    if (cudaMallocHost(&p, bytes) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}
void cuda_host_free(void *p)
{
    if (p) QZ_CUDA_CHECK(cudaFreeHost(p));
}

void cuda_vec_add(float *dst, const float *src, int n)
{
    if (n <= 0) return;
    vec_add_kernel<<<(n + 255) / 256, 256, 0, g_stream>>>(dst, src, n);
    QZ_LAUNCH_CHECK();
}
void cuda_vec_scale_add(float *dst, const float *src, float scale, int n)
{
    if (n <= 0) return;
    vec_scale_add_kernel<<<(n + 255) / 256, 256, 0, g_stream>>>(dst, src, scale, n);
    QZ_LAUNCH_CHECK();
}
void cuda_vec_zero(float *dst, int n)
{
    if (n <= 0) return;
    vec_zero_kernel<<<(n + 255) / 256, 256, 0, g_stream>>>(dst, n);
    QZ_LAUNCH_CHECK();
}
void cuda_rms_norm(float *out, const float *x, const float *w, int n)
{
    if (n <= 0) return;
    int bs = n >= 4096 ? 1024 : (n >= 1024 ? 512 : (n >= 256 ? 128 : 32));
    rms_norm_kernel<<<1, bs, 0, g_stream>>>(out, x, w, n);
    QZ_LAUNCH_CHECK();
}
void cuda_rope_yarn(float *x, int n_heads, int head_dim, int pos, float theta, float yarn_scale, int yarn_orig_ctx,
                    int neox)
{
    if (n_heads <= 0 || head_dim < 2) return;
    int half = head_dim / 2;
    int bs = (half + 31) & ~31;
    rope_yarn_kernel<<<n_heads, bs, 0, g_stream>>>(x, head_dim, pos, theta, yarn_scale, yarn_orig_ctx, neox);
    QZ_LAUNCH_CHECK();
}
void cuda_kv_append(float *k_cache, float *v_cache, const float *k, const float *v, int pos, int kv_dim)
{
    if (kv_dim <= 0) return;
    kv_append_kernel<<<(kv_dim + 255) / 256, 256, 0, g_stream>>>(k_cache, v_cache, k, v, pos, kv_dim);
    QZ_LAUNCH_CHECK();
}
void cuda_attn_score_all(float *scores, const float *q, const float *k_cache, int n_heads, int n_kv_heads,
                         int seq_len, int head_dim, int kv_dim, int max_seq, float scale)
{
    if (n_heads <= 0 || seq_len <= 0) return;
    dim3 grid(n_heads, (seq_len + 7) / 8);
    attn_score_all_kernel<<<grid, 256, 0, g_stream>>>(scores, q, k_cache, n_heads, n_kv_heads, seq_len, head_dim,
                                                      kv_dim, max_seq, scale);
    QZ_LAUNCH_CHECK();
}
void cuda_softmax_sink_all(float *scores, int n_heads, int seq_len, int max_seq, const float *sinks)
{
    if (n_heads <= 0 || seq_len <= 0) return;
    int bs = seq_len <= 64 ? 64 : 256;
    softmax_sink_all_kernel<<<n_heads, bs, 0, g_stream>>>(scores, seq_len, max_seq, sinks);
    QZ_LAUNCH_CHECK();
}
void cuda_attn_values_all(float *out, const float *scores, const float *v_cache, int n_heads, int n_kv_heads,
                          int seq_len, int head_dim, int kv_dim, int max_seq)
{
    if (n_heads <= 0 || head_dim <= 0) return;
    int bs = head_dim >= 128 ? 128 : ((head_dim + 31) & ~31);
    attn_values_all_kernel<<<n_heads, bs, 0, g_stream>>>(out, scores, v_cache, n_heads, n_kv_heads, seq_len,
                                                         head_dim, kv_dim, max_seq);
    QZ_LAUNCH_CHECK();
}
// Per-head forms (declared by the reference's FFI, unused by its forward pass): the
// all-heads kernels with one head and the head's column offset folded into the pointer.
void cuda_attn_score(float *scores, const float *q, const float *k_cache, int seq_len, int head_dim, int kv_dim,
                     int kv_head_off, float scale)
{
    cuda_attn_score_all(scores, q, k_cache + kv_head_off, 1, 1, seq_len, head_dim, kv_dim, seq_len, scale);
}
void cuda_softmax_sink(float *x, int n, float sink)
{
    if (n <= 0) return;
    softmax_sink_kernel<<<1, n <= 64 ? 64 : 256, 0, g_stream>>>(x, n, sink);
    QZ_LAUNCH_CHECK();
}
void cuda_attn_values(float *out, const float *scores, const float *v_cache, int seq_len, int head_dim, int kv_dim,
                      int kv_head_off)
{
    cuda_attn_values_all(out, scores, v_cache + kv_head_off, 1, 1, seq_len, head_dim, kv_dim, seq_len);
}
void cuda_swiglu(float *out, const float *gate, const float *up, int n)
{
    if (n <= 0) return;
    swiglu_kernel<<<(n + 255) / 256, 256, 0, g_stream>>>(out, gate, up, n);
    QZ_LAUNCH_CHECK();
}
void cuda_swiglu_oai(float *out, const float *gate, const float *up, int n)
{
    if (n <= 0) return;
    swiglu_oai_kernel<<<(n + 255) / 256, 256, 0, g_stream>>>(out, gate, up, n);
    QZ_LAUNCH_CHECK();
}
void cuda_embed_lookup(float *out, const uint8_t *data, uint32_t ggml_type, int token, int embed_dim)
{
    const FormatInfo fi = format_info(ggml_type);
    if (fi.block_elems == 0 || embed_dim <= 0 || embed_dim % fi.block_elems) {
        set_error(fi.block_elems ? QZ_ERR_BAD_SHAPE : QZ_ERR_UNSUPPORTED_TYPE, "cuda_embed_lookup");
        return;
    }
    size_t row_bytes = (size_t)(embed_dim / fi.block_elems) * fi.block_bytes;
    dequant_rows(ggml_type, data + (size_t)token * row_bytes, out, embed_dim, 1);
}

// ======================= Part 2 =======================

int quartz_last_error(void)
{
    poll_status();
    return g_err;
}
const char *quartz_error_string(void) { return g_err_msg.c_str(); }
void quartz_clear_error(void)
{
    g_err = QZ_OK;
    g_err_msg.clear();
}
void quartz_set_stream(void *s) { g_stream = (cudaStream_t)s; }
long long quartz_launch_count(void) { return g_launch_count; }
void quartz_set_gemv_impl(int impl) { g_use_tma = impl == 1 ? 0 : 1; }

void quartz_prefetch_next(const void *d_ptr, size_t bytes)
{
    static long long cap = -1;
    if (cap < 0) {
        const char *e = getenv("QUARTZ_PREFETCH_MB");   // per hinted range; 0 switches the hints off
        cap = (e ? atoll(e) : 24) << 20;
    }
    if (!d_ptr || bytes < 16 || cap == 0 || ((uintptr_t)d_ptr & 15) || g_pf.n >= QZ_MAX_PREFETCH) return;
    if ((long long)bytes > cap) bytes = (size_t)cap;
    g_pf.ptr[g_pf.n] = (const uint8_t *)d_ptr;
    g_pf.bytes[g_pf.n] = (unsigned)(bytes & ~(size_t)15);
    g_pf.n++;
}

int cuda_repack_weights(uint32_t ggml_type, void *d_data, int in_dim, int out_dim, int n_mats)
{
    const FormatInfo fi = format_info(ggml_type);
    if (fi.block_elems == 0) {
        set_error(QZ_ERR_UNSUPPORTED_TYPE, "cuda_repack_weights: unsupported ggml_type");
        return 0;
    }
    if (!check_shape(ggml_type, in_dim, out_dim, "cuda_repack_weights: bad shape") || n_mats <= 0) return 0;
    if (stream_layout(ggml_type) != 2) return 0;            // served from the raw layout
    const int nb = in_dim / fi.block_elems;
    if (nb % 8 != 0 || ((uintptr_t)d_data & 15)) return 0;  // planes would not be 16-byte aligned
    const size_t row_bytes = (size_t)nb * fi.block_bytes;
    if (row_bytes > 200 * 1024) return 0;                   // a row must fit the staging shared memory
    if (find_range(d_data)) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_repack_weights: range already repacked");
        return 0;
    }
    const long long rows = (long long)out_dim * n_mats;
    if (rows == 0) return 0;
    static bool attr_set = false;
    if (!attr_set) {
        QZ_CUDA_CHECK(cudaFuncSetAttribute(repack_rows_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           200 * 1024));
        QZ_CUDA_CHECK(cudaFuncSetAttribute(repack_rows_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           200 * 1024));
        attr_set = true;
    }
    unsigned grid = (unsigned)(rows < 65535 ? rows : 65535);
    repack_rows_kernel<true><<<grid, 256, row_bytes, g_stream>>>((uint8_t *)d_data, fi, nb, rows);
    QZ_LAUNCH_CHECK();
    uintptr_t a = (uintptr_t)d_data;
    g_ranges[a] = Range{a + (size_t)rows * row_bytes, ggml_type, in_dim, rows};
    return 1;
}

int cuda_unpack_weights(void *d_data)
{
    auto it = g_ranges.find((uintptr_t)d_data);
    if (it == g_ranges.end()) return 0;
    const Range r = it->second;
    const FormatInfo fi = format_info(r.type);
    const int nb = r.K / fi.block_elems;
    const size_t row_bytes = (size_t)nb * fi.block_bytes;
    unsigned grid = (unsigned)(r.rows < 65535 ? r.rows : 65535);
    repack_rows_kernel<false><<<grid, 256, row_bytes, g_stream>>>((uint8_t *)d_data, fi, nb, r.rows);
    QZ_LAUNCH_CHECK();
    g_ranges.erase(it);
    return 1;
}

void cuda_dequant(uint32_t ggml_type, const uint8_t *d_data, float *d_out, int in_dim, long long n_rows)
{
    dequant_rows(ggml_type, d_data, d_out, in_dim, n_rows);
}

void cuda_gemv_noalloc(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, float *d_y, int in_dim,
                       int out_dim)
{
    gemv_noalloc(ggml_type, d_data, d_x, d_y, in_dim, out_dim);
}

// ---- fused decode-step entry points (activation slots 0..3 map to scratch slots 4..7) ----
static bool user_slot(int slot, int n, XQOut *o)
{
    if (slot < 0 || slot > 3 || n <= 0 || n % 4 != 0) {
        set_error(QZ_ERR_BAD_SHAPE, "activation slot must be 0..3 and n a positive multiple of 4");
        return false;
    }
    if (!ensure_xq(n)) return false;
    XQMut q = xq_slot(g_xq.base, g_xq.slot_bytes, 4 + slot, g_xq.cap_k);
    *o = XQOut{q.xl, q.xh, q.xs, q.xsum};
    return true;
}

void cuda_quantize_x(const float *d_x, int n, int slot)
{
    XQOut o;
    if (!user_slot(slot, n, &o)) return;
    launch_quantize(d_x, XQMut{o.xl, o.xh, o.xs, o.xsum}, n);
}

void cuda_rms_norm_q(const float *x, const float *w, int n, int slot, float *out_f32)
{
    XQOut o;
    if (!user_slot(slot, n, &o)) return;
    launch(rms_norm_q_kernel, dim3(1), dim3(1024), 0, x, w, n, o, out_f32);
}

void cuda_swiglu_q(const float *gate, const float *up, int n, int slot, int oai)
{
    XQOut o;
    if (!user_slot(slot, n, &o)) return;
    const int threads = n / 4;
    launch(swiglu_q_kernel, dim3((threads + 255) / 256), dim3(256), 0, gate, up, n, oai, o);
}

int cuda_gemv_q_supported(uint32_t ggml_type, const uint8_t *d_data, int in_dim)
{
    if (!stream_shape_ok(ggml_type, in_dim) || ((uintptr_t)d_data & 15)) return 0;
    const Range *r = find_range(d_data);
    const bool planes = r && r->type == ggml_type && r->K == in_dim;
    return ((stream_layout(ggml_type) == 2) == planes) ? 1 : 0;
}

void cuda_gemv_q(uint32_t ggml_type, int n_mats, const uint8_t *const *d_w, const int *slots, float *const *d_y,
                 int in_dim, int out_dim, int accumulate)
{
    if (n_mats <= 0 || out_dim <= 0) return;
    if (n_mats > QZ_MAX_MATS) {
        set_error(QZ_ERR_TOO_LARGE, "cuda_gemv_q: at most 8 matrices per call");
        return;
    }
    int slot_of[QZ_MAX_MATS];
    for (int i = 0; i < n_mats; i++) {
        if (slots[i] < 0 || slots[i] > 3 || !cuda_gemv_q_supported(ggml_type, d_w[i], in_dim)) {
            set_error(QZ_ERR_BAD_SHAPE, "cuda_gemv_q: type/shape/layout has no streaming kernel (ask cuda_gemv_q_supported)");
            return;
        }
        slot_of[i] = 4 + slots[i];
    }
    if (!ensure_xq(in_dim)) return;
    stream_core(ggml_type, n_mats, d_w, slot_of, d_y, in_dim, out_dim, accumulate ? 1 : 0);
    g_pf.n = 0;
}

// The GEMVs whose activation vector is the RMSNorm of x / the SwiGLU of (gate, up): the streaming kernel
// converts it in its own prologue; where that kernel does not apply, the two-launch form runs instead.
static void gemv_xsrc(uint32_t ggml_type, int n_mats, const uint8_t *const *d_w, float *const *d_y, XSrc src, int in_dim,
                      int out_dim, int accumulate, const char *who)
{
    if (n_mats <= 0 || out_dim <= 0) return;
    if (n_mats > QZ_MAX_MATS) {
        set_error(QZ_ERR_TOO_LARGE, "fused GEMV: at most 8 matrices per call");
        return;
    }
    int slot_of[QZ_MAX_MATS];
    for (int i = 0; i < n_mats; i++) {
        if (!cuda_gemv_q_supported(ggml_type, d_w[i], in_dim)) {
            set_error(QZ_ERR_BAD_SHAPE, who);
            return;
        }
        slot_of[i] = 7;   // the caller's slot 3: used only if the fused prologue is not taken
    }
    if (!ensure_xq(in_dim)) return;
    // the prologue converts the whole vector in every CTA: worth it for short vectors (one launch less), not for
    // long ones (14336: +4 us per CTA against a 2 us conversion kernel)
    if (use_tma() && in_dim <= xsrc_max_k() && ((uintptr_t)src.a & 15) == 0 && ((uintptr_t)src.b & 15) == 0) {
        g_xsrc = src;
        g_xsrc_pending = true;
        const bool ok = stream_core(ggml_type, n_mats, d_w, slot_of, d_y, in_dim, out_dim, accumulate ? 1 : 0);
        const bool consumed = !g_xsrc_pending;
        g_xsrc_pending = false;
        if (ok && consumed) {
            g_pf.n = 0;
            return;
        }
    }
    if (src.mode == 1) cuda_rms_norm_q(src.a, src.b, in_dim, 3, nullptr);
    else cuda_swiglu_q(src.a, src.b, in_dim, 3, src.oai);
    stream_core(ggml_type, n_mats, d_w, slot_of, d_y, in_dim, out_dim, accumulate ? 1 : 0);
    g_pf.n = 0;
}

void cuda_gemv_rmsnorm(uint32_t ggml_type, int n_mats, const uint8_t *const *d_w, float *const *d_y, const float *d_x,
                       const float *d_norm_w, int in_dim, int out_dim, int accumulate)
{
    gemv_xsrc(ggml_type, n_mats, d_w, d_y, XSrc{1, d_x, d_norm_w, 0}, in_dim, out_dim, accumulate,
              "cuda_gemv_rmsnorm: type/shape/layout has no streaming kernel (ask cuda_gemv_q_supported)");
}

void cuda_gemv_swiglu(uint32_t ggml_type, int n_mats, const uint8_t *const *d_w, float *const *d_y, const float *d_gate,
                      const float *d_up, int oai, int in_dim, int out_dim, int accumulate)
{
    gemv_xsrc(ggml_type, n_mats, d_w, d_y, XSrc{2, d_gate, d_up, oai}, in_dim, out_dim, accumulate,
              "cuda_gemv_swiglu: type/shape/layout has no streaming kernel (ask cuda_gemv_q_supported)");
}

// ---- a chain of dependent GEMVs as one persistent kernel ----
// Activation scratch of the batched form: the plain-f32 vectors of independent ops are converted by ONE small
// kernel ahead of the persistent one (every CTA then reads its slices from L2), so the persistent kernel keeps its
// whole shared memory for the weight ring.
static XQScratch g_bxq;
static bool ensure_bxq(int K)
{
    if ((size_t)K <= g_bxq.cap_k) return true;
    if (g_bxq.base) {
        cudaStreamSynchronize(g_stream);
        cudaFree(g_bxq.base);
        g_bxq.base = nullptr;
        g_bxq.cap_k = 0;
    }
    const size_t cap = (size_t)K < 32768 ? 32768 : (size_t)K;
    const size_t sb = xq_slot_bytes(cap);
    if (cudaMalloc(&g_bxq.base, CHAIN_MAX_OPS * sb) != cudaSuccess) {
        cudaGetLastError();
        set_error(QZ_ERR_CUDA, "cudaMalloc of the batch activation scratch failed");
        return false;
    }
    g_bxq.cap_k = cap;
    g_bxq.slot_bytes = sb;
    return true;
}

static bool chain_plan(int n_ops, const qz_chain_op *ops, ChainArgs &a, size_t &smem, int independent = 0,
                       const size_t *push_off = nullptr, const size_t *push_stride = nullptr)
{
    if (n_ops < 1 || n_ops > CHAIN_MAX_OPS || !use_tma()) return false;
    const int grid = sm_count();
    int slot = 0, x_bytes = 0, rot = 0;
    for (int k = 0; k < n_ops; k++) {
        const int src = k;
        const qz_chain_op &o = ops[src];
        ChainOp &c = a.op[k];
        if (o.ggml_type != T_Q4_K && o.ggml_type != T_Q6_K && o.ggml_type != T_Q8_0) return false;
        if (o.n_mats < 1 || o.n_mats > QZ_MAX_MATS || o.n_mats > grid || o.out_dim <= 0) return false;
        if (o.src_mode < 1 || o.src_mode > 3 || !o.d_a || (o.src_mode != 3 && !o.d_b)) return false;
        if (((uintptr_t)o.d_a & 15) || (o.src_mode != 3 && ((uintptr_t)o.d_b & 15))) return false;
        if (o.in_dim < 2048 || o.in_dim % 64) return false;
        if (o.src_mode == 1 && o.in_dim / 4 > XSRC_MAX_IT * TMA_CONSUMERS) return false;   // RMSNorm: one piece only
        if (push_off && ((o.n_mats != 1 && !push_stride) || o.accumulate)) return false;
        if (push_off && push_stride && o.n_mats > 1 && push_stride[src] < (size_t)o.out_dim) return false;
        for (int i = 0; i < o.n_mats; i++)
            if (!cuda_gemv_q_supported(o.ggml_type, o.d_w[i], o.in_dim)) return false;
        const FormatInfo fi = format_info(o.ggml_type);
        const int row_bytes = (o.in_dim / fi.block_elems) * fi.block_bytes;
        c.type = o.ggml_type;
        c.n_mats = o.n_mats;
        c.K = o.in_dim;
        c.N = o.out_dim;
        c.accumulate = o.accumulate ? 1 : 0;
        c.U = o.in_dim / 64;
        c.Upad = (c.U + 31) & ~31;
        if (c.Upad > TMA_CONSUMERS) return false;
        c.RP = TMA_CONSUMERS / c.Upad;
        const int ntiles = (o.out_dim + c.RP - 1) / c.RP;
        const int per_mat = grid / o.n_mats;
        c.n_cta = ntiles < per_mat ? ntiles : per_mat;
        // independent ops: op k's CTA numbering starts where op k-1's odd tiles ended, so that the CTAs that get one
        // tile more than the others are not the same in every op (dependent ops keep the plain numbering)
        c.rot = independent ? rot % grid : 0;
        rot += (ntiles % c.n_cta) * o.n_mats;
        c.push_off = push_off ? (long long)push_off[src] : -1;
        c.push_stride = push_off && push_stride ? (long long)push_stride[src] : 0;
        c.xsrc = XSrc{o.src_mode, o.d_a, o.src_mode == 3 ? o.d_a : o.d_b, o.oai};
        for (int i = 0; i < QZ_MAX_MATS; i++) {
            c.W[i] = o.d_w[i < o.n_mats ? i : 0];
            c.y[i] = o.d_y[i < o.n_mats ? i : 0];
        }
        const int stage = c.RP * row_bytes;
        if (stage > slot) slot = stage;
        const int xb = (int)((2 * (size_t)o.in_dim + o.in_dim / 8 + o.in_dim / 4 + 31) & ~(size_t)15);
        if (independent && o.src_mode == 3) {
            // a plain vector of an independent op: converted ahead of the persistent kernel, read from global memory
            if (!ensure_bxq(o.in_dim)) return false;
            const XQMut q = xq_slot(g_bxq.base, g_bxq.slot_bytes, k, g_bxq.cap_k);
            c.x_off = -1;
            c.xg = XQ{q.xl, q.xh, q.xs, q.xsum};
        } else if (independent) {   // an area of its own (all are converted before the first op runs)
            c.x_off = x_bytes;
            x_bytes += xb;
        } else {
            c.x_off = 0;
            if (xb > x_bytes) x_bytes = xb;
        }
    }
    slot = (slot + 127) & ~127;
    const int budget = (222 * 1024 - x_bytes) & ~127;
    if (budget < 3 * slot) return false;   // the largest stage must fit the ring at least three times
    a.n_ops = n_ops;
    a.ring_bytes = budget;
    a.independent = independent;
    a.exchange = (!independent && push_off) ? 1 : 0;
    a.push.n = 0;
    smem = (size_t)budget + x_bytes;
    return true;
}

int cuda_gemv_chain_supported(int n_ops, const qz_chain_op *ops)
{
    ChainArgs a;
    size_t smem;
    return ops && chain_plan(n_ops, ops, a, smem) ? 1 : 0;
}

static void gemv_chain_launch(int n_ops, const qz_chain_op *ops, int independent, const size_t *push_off,
                              const size_t *push_stride = nullptr);

void cuda_gemv_chain(int n_ops, const qz_chain_op *ops) { gemv_chain_launch(n_ops, ops, 0, nullptr); }
void cuda_gemv_batch(int n_ops, const qz_chain_op *ops) { gemv_chain_launch(n_ops, ops, 1, nullptr); }

static bool fill_push(PushArgs &p, size_t dst_off, size_t elems);
static bool mgpu_is_attached();
static bool push_wait_after_take();   // the pending quartz_mgpu_wait_in_next_push request, cleared

int cuda_gemv_batch_push(int n_ops, const qz_chain_op *ops, const size_t *dst_off)
{
    if (n_ops <= 0 || !ops || !dst_off) return 0;
    static ChainArgs probe;   // (large: kept off the stack)
    size_t smem = 0;
    if (!chain_plan(n_ops, ops, probe, smem, 1, dst_off)) {
        push_wait_after_take();   // (a pending request belongs to this call, launched or not)
        return 0;
    }
    gemv_chain_launch(n_ops, ops, 1, dst_off);
    return 1;
}

int cuda_gemv_chain_push(int n_ops, const qz_chain_op *ops, const size_t *dst_off, const size_t *dst_stride)
{
    if (n_ops <= 0 || !ops || !dst_off) return 0;
    if (!mgpu_is_attached()) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_gemv_chain_push: the windows are not attached (quartz_mgpu_init / quartz_mgpu_attach)");
        return 0;
    }
    static ChainArgs probe;   // (large: kept off the stack)
    size_t smem = 0;
    if (!chain_plan(n_ops, ops, probe, smem, 0, dst_off, dst_stride)) {
        push_wait_after_take();
        return 0;
    }
    gemv_chain_launch(n_ops, ops, 0, dst_off, dst_stride);
    return 1;
}

static void gemv_chain_launch(int n_ops, const qz_chain_op *ops, int independent, const size_t *push_off,
                              const size_t *push_stride)
{
    if (n_ops <= 0 || !ops) return;
    static ChainArgs a;   // (large: kept off the stack)
    size_t smem = 0;
    if (!chain_plan(n_ops, ops, a, smem, independent, push_off, push_stride)) {
        if (push_off) return;   // (the push entry points have checked the plan already)
        // not a chain the persistent kernel takes: the same GEMVs one launch at a time
        for (int k = 0; k < n_ops; k++) {
            const qz_chain_op &o = ops[k];
            if (o.src_mode == 1) cuda_gemv_rmsnorm(o.ggml_type, o.n_mats, o.d_w, o.d_y, o.d_a, o.d_b, o.in_dim, o.out_dim, o.accumulate);
            else if (o.src_mode == 2) cuda_gemv_swiglu(o.ggml_type, o.n_mats, o.d_w, o.d_y, o.d_a, o.d_b, o.oai, o.in_dim, o.out_dim, o.accumulate);
            else {
                int slots[QZ_MAX_MATS] = {3, 3, 3, 3, 3, 3, 3, 3};
                cuda_quantize_x(o.d_a, o.in_dim, 3);
                cuda_gemv_q(o.ggml_type, o.n_mats, o.d_w, slots, o.d_y, o.in_dim, o.out_dim, o.accumulate);
            }
        }
        return;
    }
    if (push_off) {
        // every op's rows go to all ranks' windows; one publish for the whole launch
        size_t hi = 0;
        for (int k = 0; k < n_ops; k++)
            hi = std::max(hi, push_off[k] + (push_stride ? push_stride[k] * (size_t)(ops[k].n_mats - 1) : 0) + (size_t)ops[k].out_dim);
        if (!fill_push(a.push, 0, hi)) return;
        a.push.wait_after = push_wait_after_take() ? 1 : 0;
    }
    if (!g_grid_barrier) {
        if (cudaMalloc(&g_grid_barrier, sizeof(GridBarrier)) != cudaSuccess) {
            cudaGetLastError();
            g_grid_barrier = nullptr;
            set_error(QZ_ERR_CUDA, "cudaMalloc of the grid barrier failed");
            return;
        }
        cudaMemset(g_grid_barrier, 0, sizeof(GridBarrier));
    }
    a.gb = g_grid_barrier;
    a.status = status_word();
    if (!a.status) return;
    {
        // the vectors that are converted ahead of the persistent kernel: one launch for all of them
        QuantMulti qm;
        int nq = 0, max_k = 0;
        for (int k = 0; k < n_ops; k++) {
            if (a.op[k].x_off >= 0) continue;
            const XQMut q = xq_slot(g_bxq.base, g_bxq.slot_bytes, k, g_bxq.cap_k);
            qm.x[nq] = a.op[k].xsrc.a;
            qm.o[nq] = XQOut{q.xl, q.xh, q.xs, q.xsum};
            qm.K[nq] = a.op[k].K;
            max_k = std::max(max_k, a.op[k].K);
            nq++;
        }
        for (int i = nq; i < QZ_QUANT_MULTI; i++) { qm.x[i] = nullptr; qm.K[i] = 0; qm.o[i] = XQOut{nullptr, nullptr, nullptr, nullptr}; }
        if (nq > 0) launch(quantize_x_multi_kernel, dim3((max_k / 4 + 255) / 256, nq), dim3(256), 0, qm);
    }
    static bool attr_set = false;
    if (!attr_set) {
        QZ_CUDA_CHECK(cudaFuncSetAttribute(gemv_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
        attr_set = true;
    }
    launch(gemv_chain_kernel, dim3(sm_count()), dim3(TMA_CONSUMERS + 32), smem, a);
}

void cuda_rope_kv(float *q, float *k, const float *v, float *k_cache, float *v_cache, int n_heads, int n_kv_heads,
                  int head_dim, int pos, float theta, float yarn_scale, int yarn_orig_ctx, int neox)
{
    if (n_heads <= 0 || n_kv_heads <= 0 || head_dim < 2) return;
    const int bs = ((head_dim / 2) + 31) & ~31;
    launch(rope_kv_kernel, dim3(n_heads + n_kv_heads), dim3(bs), 0, q, k, v, k_cache, v_cache, n_heads, head_dim, pos,
           theta, yarn_scale, yarn_orig_ctx, neox, n_kv_heads * head_dim);
}

static float *g_attn_part = nullptr;
static size_t g_attn_part_floats = 0;

// attention scratch: 64 counters (zero between launches) followed by the split partials
static bool ensure_attn_scratch(size_t need_floats)
{
    if (need_floats <= g_attn_part_floats) return true;
    if (g_attn_part) {
        cudaStreamSynchronize(g_stream);
        cudaFree(g_attn_part);
    }
    size_t cap = need_floats < (size_t)(1 << 20) ? (size_t)(1 << 20) : need_floats * 2;   // room for longer contexts
    if (cudaMalloc(&g_attn_part, (cap + 64) * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        g_attn_part = nullptr;
        g_attn_part_floats = 0;
        set_error(QZ_ERR_CUDA, "cudaMalloc of the attention scratch failed");
        return false;
    }
    cudaMemset(g_attn_part, 0, 64 * sizeof(float));
    g_attn_part_floats = cap;
    return true;
}

void cuda_attn_decode(float *out, const float *q, const float *k_cache, const float *v_cache, int n_heads,
                      int n_kv_heads, int seq_len, int head_dim, int kv_dim, float scale, const float *sinks,
                      int out_slot)
{
    if (n_heads <= 0 || seq_len <= 0) return;
    if (head_dim > ATT_MAX_HD || head_dim % 32 != 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_attn_decode: head_dim must be a multiple of 32 up to 128, n_heads a multiple of n_kv_heads");
        return;
    }
    const int n_splits = (seq_len + ATT_CHUNK - 1) / ATT_CHUNK;
    if (!ensure_attn_scratch((size_t)n_heads * n_splits * (head_dim + 2))) return;
    XQOut o{nullptr, nullptr, nullptr, nullptr};
    if (out_slot >= 0 && !user_slot(out_slot, n_heads * head_dim, &o)) return;
    float *part = g_attn_part + 64;
    launch(attn_partial_kernel, dim3(n_kv_heads, n_splits), dim3(128), 0, part, q, k_cache, v_cache, n_heads,
           n_kv_heads, seq_len, head_dim, kv_dim, scale);
    launch(attn_combine_kernel, dim3(n_heads), dim3(head_dim), (size_t)n_splits * sizeof(float), out,
           (const float *)part, n_splits, head_dim, sinks, o, out_slot >= 0 ? 1 : 0);
}

// (cos, sin) table of the current decode position, shared by all layers of a step
static float2 *g_rope_tab = nullptr;
static RopeArgs g_rope_key = {-1, 0.f, 0.f, 0, 0};
static int g_rope_key_hd = 0;
static bool g_rope_tab_valid = false;   // cleared when a graph recording starts or ends

void cuda_attn_block(float *out, const float *q, const float *k_new, const float *v_new, float *k_cache, float *v_cache,
                     int n_heads, int n_kv_heads, int head_dim, int pos, int k_start, float scale, const float *sinks,
                     float theta, float yarn_scale, int yarn_orig_ctx, int neox, int out_slot)
{
    if (n_heads <= 0) return;
    if (head_dim > ATT_MAX_HD || head_dim % 32 != 0 || n_kv_heads <= 0 || n_kv_heads > 64 || n_heads % n_kv_heads != 0 ||
        pos < 0 || k_start < 0 || k_start > pos) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_attn_block: head_dim must be a multiple of 32 up to 128, n_heads a multiple of n_kv_heads (<= 64 kv heads), 0 <= k_start <= pos");
        return;
    }
    const int seq_len = pos - k_start + 1;
    const int n_splits = (seq_len + ATT_CHUNK - 1) / ATT_CHUNK;
    if (n_splits > ATT_CHUNK * ATT_MAX_HD / 4) {
        set_error(QZ_ERR_TOO_LARGE, "cuda_attn_block: context too long for the single-launch merge");
        return;
    }
    if (!ensure_attn_scratch((size_t)n_heads * n_splits * (head_dim + 2))) return;
    XQOut o{nullptr, nullptr, nullptr, nullptr};
    if (out_slot >= 0 && !user_slot(out_slot, n_heads * head_dim, &o)) return;
    const RopeArgs r{pos, theta, yarn_scale, yarn_orig_ctx, neox};
    if (!g_rope_tab && cudaMalloc(&g_rope_tab, (ATT_MAX_HD / 2) * sizeof(float2)) != cudaSuccess) {
        cudaGetLastError();
        g_rope_tab = nullptr;
        set_error(QZ_ERR_CUDA, "cudaMalloc of the RoPE table failed");
        return;
    }
    if (!g_rope_tab_valid || g_rope_key.pos != pos || g_rope_key.theta != theta || g_rope_key.yarn_scale != yarn_scale ||
        g_rope_key.yarn_orig_ctx != yarn_orig_ctx || g_rope_key_hd != head_dim) {
        launch(rope_table_kernel, dim3(1), dim3(ATT_MAX_HD / 2), 0, g_rope_tab, r, head_dim);
        g_rope_key = r;
        g_rope_key_hd = head_dim;
        g_rope_tab_valid = true;
    }
    // few splits: the last CTA of each kv head merges them in the same launch; many: a second, wider launch
    const int do_merge = n_splits <= 8 ? 1 : 0;
    launch(attn_fused_kernel, dim3(n_kv_heads, n_splits), dim3(128), 0, out, g_attn_part + 64, (int *)g_attn_part, q, k_new,
           v_new, k_cache, v_cache, n_heads, n_kv_heads, k_start, head_dim, n_kv_heads * head_dim, scale, sinks, r,
           (const float2 *)g_rope_tab, o, out_slot >= 0 ? 1 : 0, do_merge);
    if (!do_merge)
        launch(attn_combine_kernel, dim3(n_heads), dim3(head_dim), (size_t)n_splits * sizeof(float), out,
               (const float *)(g_attn_part + 64), n_splits, head_dim, sinks, o, out_slot >= 0 ? 1 : 0);
}

// ---- decode step whose position and token live in device memory ----
// RoPE parameter sets registered for a pair of step words: cuda_step_set writes their (cos, sin) tables for the new
// position in the same launch as the words, and cuda_attn_step reads the table instead of computing sin / cos of
// position * frequency in every CTA of every layer.
constexpr int QZ_MAX_ROPE_SETS = 4;
struct RopeSetDev { float2 *tab; int head_dim; float theta, yarn_scale; int yarn_orig_ctx; };
struct RopeSets { int n; RopeSetDev s[QZ_MAX_ROPE_SETS]; };
struct RopeReg { const int *step; RopeSetDev d; };
static RopeReg g_rope_reg[16];
static int g_rope_regs = 0;

__global__ void step_set_kernel(int *step, int token, int pos, RopeSets sets)
{
    pdl_wait();
    pdl_trigger();
    if (blockIdx.x == 0) {
        if (threadIdx.x == 0) {
            step[0] = token;
            step[1] = pos;
        }
        return;
    }
    const RopeSetDev &e = sets.s[blockIdx.x - 1];
    const int i = threadIdx.x;
    if (i < e.head_dim / 2) {
        const RopeArgs r{pos, e.theta, e.yarn_scale, e.yarn_orig_ctx, 0};
        float c, s;
        rope_cs(r, i, e.head_dim, c, s);
        e.tab[i] = make_float2(c, s);
    }
    if (i == 0) e.tab[ATT_MAX_HD / 2] = make_float2(__int_as_float(pos), 0.f);
}

static cudaStream_t g_graph_stream = nullptr, g_saved_stream = nullptr;

void cuda_step_set(int *d_step, int token, int pos)
{
    if (!d_step) return;
    // on the stream the recorded graphs replay on (when there is one), so the words are ordered with the replays
    cudaStream_t s = (g_graph_stream && g_stream == 0) ? g_graph_stream : g_stream;
    RopeSets sets;
    sets.n = 0;
    for (int i = 0; i < g_rope_regs && sets.n < QZ_MAX_ROPE_SETS; i++)
        if (g_rope_reg[i].step == d_step) sets.s[sets.n++] = g_rope_reg[i].d;
    step_set_kernel<<<1 + sets.n, ATT_MAX_HD / 2, 0, s>>>(d_step, token, pos, sets);
    QZ_LAUNCH_CHECK();
}

void cuda_step_rope_table(int *d_step, int head_dim, float theta, float yarn_scale, int yarn_orig_ctx)
{
    if (!d_step || head_dim < 2 || head_dim > ATT_MAX_HD || head_dim % 2) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_step_rope_table: head_dim must be even and at most 128");
        return;
    }
    int same_step = 0;
    for (int i = 0; i < g_rope_regs; i++) {
        const RopeReg &e = g_rope_reg[i];
        if (e.step != d_step) continue;
        if (e.d.head_dim == head_dim && e.d.theta == theta && e.d.yarn_scale == yarn_scale && e.d.yarn_orig_ctx == yarn_orig_ctx) return;
        same_step++;
    }
    if (g_rope_regs >= 16 || same_step >= QZ_MAX_ROPE_SETS) return;   // no room: such calls keep computing in the kernel
    float2 *tab = nullptr;
    if (cudaMalloc(&tab, (ATT_MAX_HD / 2 + 1) * sizeof(float2)) != cudaSuccess) {
        cudaGetLastError();
        set_error(QZ_ERR_CUDA, "cuda_step_rope_table: cudaMalloc failed");
        return;
    }
    cudaMemset(tab, 0xFF, (ATT_MAX_HD / 2 + 1) * sizeof(float2));   // position -1: matches no step until cuda_step_set ran
    g_rope_reg[g_rope_regs++] = RopeReg{d_step, RopeSetDev{tab, head_dim, theta, yarn_scale, yarn_orig_ctx}};
}

// the registered table of (step words, parameters), or NULL
static const float2 *rope_table_of(const int *d_step, int head_dim, float theta, float yarn_scale, int yarn_orig_ctx)
{
    for (int i = 0; i < g_rope_regs; i++) {
        const RopeReg &e = g_rope_reg[i];
        if (e.step == d_step && e.d.head_dim == head_dim && e.d.theta == theta && e.d.yarn_scale == yarn_scale &&
            e.d.yarn_orig_ctx == yarn_orig_ctx)
            return e.d.tab;
    }
    return nullptr;
}

void cuda_embed_lookup_dev(float *out, const uint8_t *data, uint32_t ggml_type, const int *d_step, int embed_dim)
{
    const FormatInfo fi = format_info(ggml_type);
    if (fi.block_elems == 0 || embed_dim <= 0 || embed_dim % fi.block_elems || !d_step) {
        set_error(fi.block_elems ? QZ_ERR_BAD_SHAPE : QZ_ERR_UNSUPPORTED_TYPE, "cuda_embed_lookup_dev");
        return;
    }
    dequant_rows(ggml_type, data, out, embed_dim, 1, d_step);
}

// cluster width of the attention kernel for a head group of G heads: the widest power of two (<= 16, or the
// value of QUARTZ_ATTN_CLUSTER) that leaves every CTA a whole number of 32-output runs and that the device
// can schedule; 0 = this head geometry is not served
static int attn_step_rows()
{
    static int rows = -1;
    if (rows < 0) {
        const char *e = getenv("QUARTZ_ATTN_ROWS");   // 64: less shared memory per CTA (two staging rounds when a CTA owns three blocks)
        rows = (e && atoi(e) == 64) ? 64 : AS_ROWS;
    }
    return rows;
}

static int attn_step_cluster(int G, int head_dim)
{
    static int cached_G = -1, cached_hd = -1, cached_cl = 0;
    if (G == cached_G && head_dim == cached_hd) return cached_cl;
    int want = AS_MAX_CL;
    if (const char *e = getenv("QUARTZ_ATTN_CLUSTER")) {
        const int v = atoi(e);
        if (v == 1 || v == 2 || v == 4 || v == 8 || v == 16) want = v;
    }
    static bool attr_set = false;
    if (!attr_set) {
        QZ_CUDA_CHECK(cudaFuncSetAttribute(attn_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)attn_step_smem(AS_MAX_G, AS_MAX_CL, ATT_MAX_HD, AS_ROWS)));
        if (cudaFuncSetAttribute(attn_step_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)
            cudaGetLastError();
        attr_set = true;
    }
    int cl = 0;
    for (int c = want; c >= 1; c >>= 1) {
        if ((G * head_dim) % (32 * c) != 0) continue;
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(c);
        cfg.blockDim = dim3(AS_THREADS);
        cfg.dynamicSmemBytes = attn_step_smem(G, c, head_dim, attn_step_rows());
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = c;
        at[0].val.clusterDim.y = 1;
        at[0].val.clusterDim.z = 1;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, attn_step_kernel, &cfg) == cudaSuccess && n >= 1) {
            cl = c;
            break;
        }
        cudaGetLastError();
    }
    cached_G = G;
    cached_hd = head_dim;
    cached_cl = cl;
    return cl;
}

void cuda_embed_lookup_rows(float *out, const uint8_t *data, uint32_t ggml_type, const int *d_tokens, int n, int embed_dim)
{
    const FormatInfo fi = format_info(ggml_type);
    if (fi.block_elems == 0 || embed_dim <= 0 || embed_dim % fi.block_elems || !d_tokens || n < 0) {
        set_error(fi.block_elems ? QZ_ERR_BAD_SHAPE : QZ_ERR_UNSUPPORTED_TYPE, "cuda_embed_lookup_rows");
        return;
    }
    if (n > 0) dequant_rows(ggml_type, data, out, embed_dim, n, d_tokens);
}

void cuda_rms_norm_rows(float *out, const float *x, const float *w, int n_rows, int n)
{
    if (n_rows <= 0 || n <= 0) return;
    const int bs = n >= 4096 ? 1024 : (n >= 1024 ? 512 : (n >= 256 ? 128 : 32));
    launch(rms_norm_rows_kernel, dim3((unsigned)n_rows), dim3(bs), 0, out, x, w, n);
}

void cuda_rope_kv_rows(float *q, float *k, const float *v, float *k_cache, float *v_cache, int n_tok, int n_heads,
                       int n_kv_heads, int head_dim, int pos0, float theta, float yarn_scale, int yarn_orig_ctx, int neox)
{
    if (n_tok <= 0 || n_heads <= 0 || n_kv_heads <= 0 || head_dim < 2 || pos0 < 0) return;
    const int bs = ((head_dim / 2) + 31) & ~31;
    launch(rope_kv_rows_kernel, dim3(n_heads + n_kv_heads, n_tok), dim3(bs), 0, q, k, v, k_cache, v_cache, n_heads, head_dim, pos0,
           theta, yarn_scale, yarn_orig_ctx, neox, n_kv_heads * head_dim);
}

static int attn_step_rows();
static int attn_step_cluster(int G, int head_dim);

void cuda_attn_prompt(float *out, const float *q, const float *k_cache, const float *v_cache, int n_tok, int n_heads,
                      int n_kv_heads, int head_dim, int max_seq, int pos0, int window, float scale, const float *sinks)
{
    if (n_tok <= 0) return;
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_heads / n_kv_heads > AS_MAX_G || head_dim > ATT_MAX_HD ||
        head_dim % 32 != 0 || pos0 < 0 || pos0 + n_tok > max_seq || n_tok > 65535) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_attn_prompt: head_dim must be a multiple of 32 up to 128, at most 16 query heads per kv head, pos0 + n_tok <= max_seq, n_tok <= 65535");
        return;
    }
    const int G = n_heads / n_kv_heads;
    static int simple = -1;   // QUARTZ_ATTN_PROMPT=simple: one CTA per (kv head, token), the decode kernel's prompt mode
    if (simple < 0) {
        const char *e = getenv("QUARTZ_ATTN_PROMPT");
        simple = (e && std::string(e) == "simple") ? 1 : 0;
    }
    if (!simple) {
        // tiles of TQ tokens: TQ * G query rows per CTA share every staged K / V row
        AttnPromptArgs p;
        p.out = out; p.q = q; p.k_cache = k_cache; p.v_cache = v_cache;
        p.n_tok = n_tok; p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim; p.kv_dim = n_kv_heads * head_dim;
        p.pos0 = pos0; p.window = window; p.scale = scale; p.sinks = sinks;
        p.tq = std::max(1, std::min(16, AP_MAX_ROWS / G));
        const size_t smem = attn_prompt_smem(p.tq * G, head_dim);
        static bool attr_set = false;
        if (!attr_set) {
            QZ_CUDA_CHECK(cudaFuncSetAttribute(attn_prompt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)attn_prompt_smem(AP_MAX_ROWS, ATT_MAX_HD)));
            attr_set = true;
        }
        launch(attn_prompt_kernel, dim3((unsigned)n_kv_heads, (unsigned)((n_tok + p.tq - 1) / p.tq)), dim3(AP_THREADS), smem, p);
        return;
    }
    attn_step_cluster(G, head_dim);   // (sets the kernel's attributes)
    AttnStepArgs a = {};
    a.out = out; a.q = q; a.k_new = nullptr; a.v_new = nullptr;
    a.k_cache = (float *)k_cache; a.v_cache = (float *)v_cache;
    a.step = nullptr; a.pos_host = pos0;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.kv_dim = n_kv_heads * head_dim;
    a.max_seq = max_seq; a.window = window; a.scale = scale; a.sinks = sinks;
    a.theta = 1.f; a.yarn_scale = 1.f; a.yarn_orig_ctx = 0; a.neox = 0;
    a.o = XQOut{nullptr, nullptr, nullptr, nullptr};
    a.emit_q = 0;
    a.rows_cap = attn_step_rows();
    a.prompt = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)n_kv_heads, (unsigned)n_tok);   // one CTA per (kv head, token): clusters of one
    cfg.blockDim = dim3(AS_THREADS);
    cfg.dynamicSmemBytes = attn_step_smem(G, 1, head_dim, a.rows_cap);
    cfg.stream = g_stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 1;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
    if (g_pdl) {
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = at;
    g_launch_count++;
    QZ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, attn_step_kernel, a));
}

int cuda_attn_step_supported(int n_heads, int n_kv_heads, int head_dim)
{
    if (n_heads <= 0 || n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return 0;
    const int G = n_heads / n_kv_heads;
    if (G > AS_MAX_G || head_dim > ATT_MAX_HD || head_dim % 32 != 0) return 0;
    return attn_step_cluster(G, head_dim) > 0 ? 1 : 0;
}

void cuda_attn_step(float *out, const float *q, const float *k_new, const float *v_new, float *k_cache, float *v_cache,
                    int n_heads, int n_kv_heads, int head_dim, int max_seq, const int *d_step, int pos, int window,
                    float scale, const float *sinks, float theta, float yarn_scale, int yarn_orig_ctx, int neox,
                    int out_slot)
{
    if (!cuda_attn_step_supported(n_heads, n_kv_heads, head_dim) || max_seq <= 0 || (!d_step && (pos < 0 || pos >= max_seq))) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_attn_step: head_dim must be a multiple of 32 up to 128, at most 16 query heads per kv head, 0 <= pos < max_seq");
        return;
    }
    const int G = n_heads / n_kv_heads;
    const int cl = attn_step_cluster(G, head_dim);
    AttnStepArgs a;
    a.out = out; a.q = q; a.k_new = k_new; a.v_new = v_new; a.k_cache = k_cache; a.v_cache = v_cache;
    a.step = d_step; a.pos_host = pos;
    a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.head_dim = head_dim; a.kv_dim = n_kv_heads * head_dim;
    a.max_seq = max_seq; a.window = window; a.scale = scale; a.sinks = sinks;
    a.theta = theta; a.yarn_scale = yarn_scale; a.yarn_orig_ctx = yarn_orig_ctx; a.neox = neox;
    a.o = XQOut{nullptr, nullptr, nullptr, nullptr};
    a.emit_q = 0;
    a.prompt = 0;
    a.rope_tab = d_step ? rope_table_of(d_step, head_dim, theta, yarn_scale, yarn_orig_ctx) : nullptr;
    a.rows_cap = attn_step_rows();
    if (out_slot >= 0) {
        if (!user_slot(out_slot, n_heads * head_dim, &a.o)) return;
        a.emit_q = 1;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_kv_heads * cl));
    cfg.blockDim = dim3(AS_THREADS);
    cfg.dynamicSmemBytes = attn_step_smem(G, cl, head_dim, a.rows_cap);
    cfg.stream = g_stream;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)cl;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
    if (g_pdl) {
        at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = at;
    g_launch_count++;
    QZ_CUDA_CHECK(cudaLaunchKernelEx(&cfg, attn_step_kernel, a));
}

// ---- CUDA-graph helpers: record a sequence of this library's calls once, replay it per token ----
static bool g_pdl_in_graphs = true;
static bool g_capturing = false;

int quartz_graph_begin(void)
{
    if (g_capturing) {
        set_error(QZ_ERR_BAD_SHAPE, "quartz_graph_begin: a capture is already open");
        return 0;
    }
    if (!g_graph_stream) {
        // a blocking stream: it stays ordered with the legacy default stream the copies use
        if (cudaStreamCreate(&g_graph_stream) != cudaSuccess) {
            cudaGetLastError();
            set_error(QZ_ERR_CUDA, "quartz_graph_begin: cudaStreamCreate failed");
            return 0;
        }
    }
    if (cudaStreamBeginCapture(g_graph_stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
        cudaGetLastError();
        set_error(QZ_ERR_CUDA, "quartz_graph_begin: cudaStreamBeginCapture failed");
        return 0;
    }
    g_saved_stream = g_stream;
    g_stream = g_graph_stream;
    g_capturing = true;
    g_rope_tab_valid = false;   // the table launch must be part of the recording
    g_pdl = g_pdl_in_graphs;   // recorded kernels become programmatic dependents of one another
    return 1;
}

void *quartz_graph_end(void)
{
    if (!g_capturing) return nullptr;
    g_capturing = false;
    g_rope_tab_valid = false;   // a recorded launch has not run
    g_stream = g_saved_stream;
    g_pdl = false;
    cudaGraph_t graph = nullptr;
    if (cudaStreamEndCapture(g_graph_stream, &graph) != cudaSuccess || !graph) {
        cudaGetLastError();
        set_error(QZ_ERR_CUDA, "quartz_graph_end: capture failed (a captured call synchronised or allocated?)");
        return nullptr;
    }
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) {
        cudaGetLastError();
        set_error(QZ_ERR_CUDA, "quartz_graph_end: cudaGraphInstantiate failed");
        return nullptr;
    }
    return (void *)exec;
}

void quartz_set_pdl(int on) { g_pdl_in_graphs = on != 0; }

void quartz_graph_launch(void *graph_exec)
{
    if (!graph_exec) return;
    QZ_CUDA_CHECK(cudaGraphLaunch((cudaGraphExec_t)graph_exec, g_graph_stream));
}

void quartz_graph_destroy(void *graph_exec)
{
    if (graph_exec) QZ_CUDA_CHECK(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
}

void cuda_gemm(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, float *d_y, int m, int in_dim,
               int out_dim)
{
    gemm_dispatch(ggml_type, d_data, d_x, d_y, m, in_dim, out_dim);
}

void cuda_gemm_bf16(uint32_t ggml_type, const uint8_t *d_data, const uint16_t *d_x_bf16, float *d_y, int m, int in_dim,
                    int out_dim)
{
    gemm_dispatch(ggml_type, d_data, d_x_bf16, d_y, m, in_dim, out_dim, true);
}

// ======================= batched mixture-of-experts FFN =======================
static uint8_t *g_moe = nullptr;   // library scratch: routing lists, activation tiles, gate / up / down outputs
static size_t g_moe_bytes = 0;

static bool ensure_moe(size_t need)
{
    if (need <= g_moe_bytes) return true;
    if (g_moe) {
        cudaStreamSynchronize(g_stream);
        cudaFree(g_moe);
    }
    if (cudaMalloc(&g_moe, need) != cudaSuccess) {
        cudaGetLastError();
        g_moe = nullptr;
        g_moe_bytes = 0;
        set_error(QZ_ERR_CUDA, "cuda_moe_ffn: cudaMalloc of the scratch failed");
        return false;
    }
    g_moe_bytes = need;
    return true;
}

// layout of one matrix type for the grouped kernel: false if the tensor-core kernel does not take it
static bool moe_mat_ok(uint32_t t, const uint8_t *W, int K, bool *planes)
{
    const FormatInfo fi = format_info(t);
    if (fi.block_elems < 32 || K <= 0 || K % GEMM_KSTEP != 0 || ((uintptr_t)W & 15) ||
        (((size_t)(K / fi.block_elems) * fi.block_bytes) % 16) != 0 || !tables_ready(t))
        return false;
    *planes = false;
    if (const Range *r = find_range(W)) {
        if (r->type != t || r->K != K) return false;
        *planes = true;
    }
    return true;
}

// The per-expert form: assignments grouped on the host, three GEMMs per expert.  Takes every type and shape.
static void moe_ffn_per_expert(uint32_t type_gate_up, uint32_t type_down, const uint8_t *d_gate, const uint8_t *d_up,
                               const uint8_t *d_down, const float *d_x, float *d_out, int m, int embed_dim, int ffn_dim,
                               int n_experts, int top_k, const int *h_expert_ids, const float *h_expert_w, int oai)
{
    const FormatInfo fg = format_info(type_gate_up), fd = format_info(type_down);
    const int A = m * top_k;
    std::vector<int> count(n_experts, 0), start(n_experts + 1, 0), rows(A);
    std::vector<float> wts(A);
    for (int i = 0; i < A; i++) count[h_expert_ids[i]]++;
    for (int e = 0; e < n_experts; e++) start[e + 1] = start[e] + count[e];
    std::vector<int> fill(start.begin(), start.end() - 1);
    for (int i = 0; i < A; i++) {
        const int e = h_expert_ids[i], p = fill[e]++;
        rows[p] = i / top_k;
        wts[p] = h_expert_w[i];
    }
    const size_t K = (size_t)embed_dim, F = (size_t)ffn_dim;
    const size_t lists = (((size_t)A * 8) + 255) & ~(size_t)255;
    if (!ensure_moe(lists + (size_t)A * (2 * K + 2 * F) * sizeof(float))) return;
    int *d_rows = (int *)g_moe;
    float *d_wts = (float *)(g_moe + (size_t)A * 4);
    float *xe = (float *)(g_moe + lists), *g = xe + (size_t)A * K, *u = g + (size_t)A * F, *yd = u + (size_t)A * F;
    QZ_CUDA_CHECK(cudaMemcpyAsync(d_rows, rows.data(), (size_t)A * 4, cudaMemcpyHostToDevice, g_stream));
    QZ_CUDA_CHECK(cudaMemcpyAsync(d_wts, wts.data(), (size_t)A * 4, cudaMemcpyHostToDevice, g_stream));
    QZ_CUDA_CHECK(cudaStreamSynchronize(g_stream));   // the host vectors die with this call
    QZ_CUDA_CHECK(cudaMemsetAsync(d_out, 0, (size_t)m * K * sizeof(float), g_stream));
    {
        const long long n4 = (long long)A * (K / 4);
        moe_gather_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, g_stream>>>(d_x, xe, d_rows, A, embed_dim);
        QZ_LAUNCH_CHECK();
    }
    const size_t gu_bytes = (K * F / fg.block_elems) * fg.block_bytes, dn_bytes = (F * K / fd.block_elems) * fd.block_bytes;
    for (int e = 0; e < n_experts; e++) {
        const int c = count[e];
        if (!c) continue;
        const size_t o = (size_t)start[e];
        gemm_dispatch(type_gate_up, d_gate + e * gu_bytes, xe + o * K, g + o * F, c, embed_dim, ffn_dim);
        gemm_dispatch(type_gate_up, d_up + e * gu_bytes, xe + o * K, u + o * F, c, embed_dim, ffn_dim);
    }
    {
        const long long n = (long long)A * F;
        moe_swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, g_stream>>>(g, u, n, oai);
        QZ_LAUNCH_CHECK();
    }
    for (int e = 0; e < n_experts; e++) {
        const int c = count[e];
        if (!c) continue;
        const size_t o = (size_t)start[e];
        gemm_dispatch(type_down, d_down + e * dn_bytes, g + o * F, yd + o * K, c, ffn_dim, embed_dim);
        const long long n4 = (long long)c * (K / 4);
        moe_scatter_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, g_stream>>>(d_out, yd + o * K, d_rows + o, d_wts + o, c,
                                                                             embed_dim);
        QZ_LAUNCH_CHECK();
    }
}

static bool moe_check(uint32_t type_gate_up, uint32_t type_down, int m, int embed_dim, int ffn_dim, int n_experts, int top_k,
                      const void *ids, const void *w)
{
    const FormatInfo fg = format_info(type_gate_up), fd = format_info(type_down);
    if (fg.block_elems == 0 || fd.block_elems == 0) {
        set_error(QZ_ERR_UNSUPPORTED_TYPE, "cuda_moe_ffn: unsupported ggml_type");
        return false;
    }
    if (n_experts <= 0 || top_k <= 0 || top_k > n_experts || embed_dim <= 0 || ffn_dim <= 0 || embed_dim % fg.block_elems ||
        ffn_dim % fd.block_elems || (embed_dim & 3) || (ffn_dim & 3) || !ids || !w || m <= 0) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_moe_ffn: bad dimensions or routing lists");
        return false;
    }
    return true;
}

// The grouped form, all on the device.  ids / w are DEVICE arrays of m * top_k entries.  Returns false when the
// shapes or types are not served (nothing has been launched then).
static bool moe_ffn_grouped(uint32_t type_gate_up, uint32_t type_down, const uint8_t *d_gate, const uint8_t *d_up,
                            const uint8_t *d_down, const float *d_x, float *d_out, int m, int embed_dim, int ffn_dim,
                            int n_experts, int top_k, const int *d_ids, const float *d_w, int oai)
{
    bool pg = false, pu = false, pd = false;
    if (n_experts > QZ_MOE_MAX_E || ((uintptr_t)d_x & 15) || ((uintptr_t)d_out & 15)) return false;
    if (!moe_mat_ok(type_gate_up, d_gate, embed_dim, &pg) || !moe_mat_ok(type_gate_up, d_up, embed_dim, &pu) || pg != pu ||
        !moe_mat_ok(type_down, d_down, ffn_dim, &pd))
        return false;
    const FormatInfo fg = format_info(type_gate_up), fd = format_info(type_down);
    const int A = m * top_k;
    const size_t K = (size_t)embed_dim, F = (size_t)ffn_dim;
    // token tile: the narrowest of 32 / 64 / 128 slots that holds 1.5 x the mean load of an expert
    const int mean15 = (3 * A + 2 * n_experts - 1) / (2 * n_experts);
    const int tok_tile = mean15 <= 32 ? 32 : (mean15 <= 64 ? 64 : 128);
    const int max_tt = A / tok_tile + n_experts;      // token tiles of all experts together, at most
    auto up256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t o_grp = up256((size_t)A * 4 * 3), o_xt = o_grp + up256(sizeof(GemmGroup));
    const size_t xt_bytes = (size_t)max_tt * (K / 64) * tok_tile * 128, ht_bytes = (size_t)max_tt * (F / 64) * tok_tile * 128;
    const size_t o_g = o_xt + up256(xt_bytes), o_u = o_g + up256((size_t)A * F * 4), o_ht = o_u + up256((size_t)A * F * 4);
    const size_t o_yd = o_ht + up256(ht_bytes), need = o_yd + up256((size_t)A * K * 4);
    if (!ensure_moe(need)) return true;   // (error recorded)
    int *rows = (int *)g_moe, *slot_of = rows + A;
    float *wts = (float *)(slot_of + A);
    GemmGroup *grp = (GemmGroup *)(g_moe + o_grp);
    __nv_bfloat16 *xt = (__nv_bfloat16 *)(g_moe + o_xt), *ht = (__nv_bfloat16 *)(g_moe + o_ht);
    float *G = (float *)(g_moe + o_g), *U = (float *)(g_moe + o_u), *Yd = (float *)(g_moe + o_yd);
    int *status = status_word();
    if (!status) return true;

    moe_route_kernel<<<n_experts, 256, 0, g_stream>>>(d_ids, d_w, A, top_k, n_experts, tok_tile, grp, rows, wts, slot_of);
    QZ_LAUNCH_CHECK();
    const int conv_blocks = 4 * sm_count();
    moe_tiles_kernel<0><<<conv_blocks, 256, 0, g_stream>>>(d_x, nullptr, rows, grp, xt, embed_dim, tok_tile, max_tt,
                                                           (type_gate_up == T_Q6_K && pg) ? 1 : 0, 0);
    QZ_LAUNCH_CHECK();
    QZ_CUDA_CHECK(cudaMemsetAsync(G, 0, (size_t)((uint8_t *)ht - (uint8_t *)G), g_stream));   // G and U: shared tiles are added onto zeros
    GemmArgs a = {};
    a.grp = grp;
    a.Wm[0] = d_gate; a.Wm[1] = d_up;
    a.Ym[0] = G; a.Ym[1] = U;
    a.expert_stride = (K * F / fg.block_elems) * fg.block_bytes;
    a.n_mats = 2;
    a.Xb = xt;
    a.K = embed_dim; a.N = ffn_dim; a.M = A; a.planes = pg;
    a.tok_tile = tok_tile; a.n_tok_tiles = 1;
    a.status = status;
    gemm_grouped_dispatch(type_gate_up, pg, a);
    moe_tiles_kernel<1><<<conv_blocks, 256, 0, g_stream>>>(G, U, rows, grp, ht, ffn_dim, tok_tile, max_tt,
                                                           (type_down == T_Q6_K && pd) ? 1 : 0, oai);
    QZ_LAUNCH_CHECK();
    QZ_CUDA_CHECK(cudaMemsetAsync(Yd, 0, (size_t)A * K * 4, g_stream));
    a.Wm[0] = d_down; a.Wm[1] = d_down;
    a.Ym[0] = Yd; a.Ym[1] = Yd;
    a.expert_stride = (F * K / fd.block_elems) * fd.block_bytes;
    a.n_mats = 1;
    a.Xb = ht;
    a.K = ffn_dim; a.N = embed_dim; a.planes = pd;
    gemm_grouped_dispatch(type_down, pd, a);
    const long long n4 = (long long)m * (K / 4);
    moe_combine_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, g_stream>>>(d_out, Yd, slot_of, d_w, m, top_k, embed_dim);
    QZ_LAUNCH_CHECK();
    return true;
}

void cuda_moe_ffn_dev(uint32_t type_gate_up, uint32_t type_down, const uint8_t *d_gate, const uint8_t *d_up,
                      const uint8_t *d_down, const float *d_x, float *d_out, int m, int embed_dim, int ffn_dim, int n_experts,
                      int top_k, const int *d_expert_ids, const float *d_expert_w, int oai)
{
    if (!moe_check(type_gate_up, type_down, m, embed_dim, ffn_dim, n_experts, top_k, d_expert_ids, d_expert_w)) return;
    if (moe_ffn_grouped(type_gate_up, type_down, d_gate, d_up, d_down, d_x, d_out, m, embed_dim, ffn_dim, n_experts, top_k,
                        d_expert_ids, d_expert_w, oai))
        return;
    // not a shape the grouped kernel takes: bring the lists to the host (one synchronisation) and go expert by expert
    const int A = m * top_k;
    std::vector<int> ids(A);
    std::vector<float> w(A);
    QZ_CUDA_CHECK(cudaMemcpyAsync(ids.data(), d_expert_ids, (size_t)A * 4, cudaMemcpyDeviceToHost, g_stream));
    QZ_CUDA_CHECK(cudaMemcpyAsync(w.data(), d_expert_w, (size_t)A * 4, cudaMemcpyDeviceToHost, g_stream));
    QZ_CUDA_CHECK(cudaStreamSynchronize(g_stream));
    for (int i = 0; i < A; i++)
        if (ids[i] < 0 || ids[i] >= n_experts) {
            set_error(QZ_ERR_BAD_SHAPE, "cuda_moe_ffn_dev: expert id out of range");
            return;
        }
    moe_ffn_per_expert(type_gate_up, type_down, d_gate, d_up, d_down, d_x, d_out, m, embed_dim, ffn_dim, n_experts, top_k,
                       ids.data(), w.data(), oai);
}

void cuda_moe_ffn(uint32_t type_gate_up, uint32_t type_down, const uint8_t *d_gate, const uint8_t *d_up,
                  const uint8_t *d_down, const float *d_x, float *d_out, int m, int embed_dim, int ffn_dim, int n_experts,
                  int top_k, const int *h_expert_ids, const float *h_expert_w, int oai)
{
    if (!moe_check(type_gate_up, type_down, m, embed_dim, ffn_dim, n_experts, top_k, h_expert_ids, h_expert_w)) return;
    const int A = m * top_k;
    for (int i = 0; i < A; i++)
        if (h_expert_ids[i] < 0 || h_expert_ids[i] >= n_experts) {
            set_error(QZ_ERR_BAD_SHAPE, "cuda_moe_ffn: expert id out of range");
            return;
        }
    // the routing lists go to a library buffer of their own (copied from pageable memory: staged before the call returns)
    static int *d_lists = nullptr;
    static size_t d_lists_cap = 0;
    if ((size_t)A * 8 > d_lists_cap) {
        if (d_lists) {
            cudaStreamSynchronize(g_stream);
            cudaFree(d_lists);
        }
        d_lists_cap = (size_t)A * 8 < 65536 ? 65536 : (size_t)A * 16;
        if (cudaMalloc(&d_lists, d_lists_cap) != cudaSuccess) {
            cudaGetLastError();
            d_lists = nullptr;
            d_lists_cap = 0;
            set_error(QZ_ERR_CUDA, "cuda_moe_ffn: cudaMalloc of the routing lists failed");
            return;
        }
    }
    int *d_ids = d_lists;
    float *d_w = (float *)(d_lists + A);
    QZ_CUDA_CHECK(cudaMemcpyAsync(d_ids, h_expert_ids, (size_t)A * 4, cudaMemcpyHostToDevice, g_stream));
    QZ_CUDA_CHECK(cudaMemcpyAsync(d_w, h_expert_w, (size_t)A * 4, cudaMemcpyHostToDevice, g_stream));
    if (moe_ffn_grouped(type_gate_up, type_down, d_gate, d_up, d_down, d_x, d_out, m, embed_dim, ffn_dim, n_experts, top_k,
                        d_ids, d_w, oai))
        return;
    moe_ffn_per_expert(type_gate_up, type_down, d_gate, d_up, d_down, d_x, d_out, m, embed_dim, ffn_dim, n_experts, top_k,
                       h_expert_ids, h_expert_w, oai);
}

void cuda_gemv_experts(uint32_t ggml_type, const uint8_t *d_base, size_t expert_bytes, const int *d_ids, int n_act,
                       const float *d_x, size_t x_stride, float *d_y, int in_dim, int out_dim)
{
    if (n_act <= 0 || out_dim <= 0) return;
    if (n_act > 4 || !d_ids || !cuda_gemv_q_supported(ggml_type, d_base, in_dim) || (expert_bytes & 15) || !use_tma()) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_gemv_experts: at most 4 experts per call, of a type/shape/layout the streaming kernel takes (ask cuda_gemv_q_supported)");
        return;
    }
    if (!tables_ready(ggml_type)) {
        set_error(QZ_ERR_MISSING_TABLE, "IQ codebook not uploaded (cuda_set_*_grid)");
        return;
    }
    if (!ensure_xq(in_dim)) return;
    const uint8_t *W[4];
    float *Y[4];
    int slot_of[4];
    for (int i = 0; i < n_act; i++) {
        W[i] = d_base;
        Y[i] = d_y + (size_t)i * out_dim;
        slot_of[i] = x_stride ? i : 0;
    }
    g_sel = d_ids;
    g_sel_stride = expert_bytes;
    bool done = false;
    if (!x_stride && in_dim <= xsrc_max_k() && !((uintptr_t)d_x & 15)) {
        // one activation vector for all experts: converted in the GEMV's own prologue
        g_xsrc = XSrc{3, d_x, d_x, 0};
        g_xsrc_pending = true;
        const bool ok = stream_core(ggml_type, n_act, W, slot_of, Y, in_dim, out_dim, 0);
        done = ok && !g_xsrc_pending;
        g_xsrc_pending = false;
    }
    if (!done) {
        const int n_x = x_stride ? n_act : 1;
        for (int i = 0; i < n_x; i++)
            launch_quantize(d_x + (size_t)i * x_stride, xq_slot(g_xq.base, g_xq.slot_bytes, i, g_xq.cap_k), in_dim);
        if (!stream_core(ggml_type, n_act, W, slot_of, Y, in_dim, out_dim, 0))
            set_error(QZ_ERR_BAD_SHAPE, "cuda_gemv_experts: the streaming kernel did not take this shape");
    }
    g_sel = nullptr;
    g_pf.n = 0;
}

void cuda_moe_decode_act(float *d_out, const float *d_gate, const float *d_up, const float *d_gate_bias,
                         const float *d_up_bias, const int *d_ids, int n_act, int ffn_dim, int oai)
{
    if (n_act <= 0 || ffn_dim <= 0) return;
    const long long n = (long long)n_act * ffn_dim;
    launch(moe_decode_act_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, d_out, d_gate, d_up, d_gate_bias, d_up_bias,
           d_ids, n_act, ffn_dim, oai);
}

void cuda_moe_decode_combine(float *d_acc, const float *d_down, const float *d_down_bias, const int *d_ids, const float *d_w,
                             int n_act, int embed_dim, int accumulate)
{
    if (n_act <= 0 || embed_dim <= 0) return;
    launch(moe_decode_combine_kernel, dim3((unsigned)((embed_dim + 255) / 256)), dim3(256), 0, d_acc, d_down, d_down_bias, d_ids,
           d_w, n_act, embed_dim, accumulate);
}

void cuda_router_topk(const float *d_logits, const float *d_bias, int m, int n_experts, int top_k, int renorm, int *d_ids,
                      float *d_w)
{
    if (m <= 0) return;
    if (n_experts <= 0 || n_experts > QZ_MOE_MAX_E || top_k <= 0 || top_k > 8 || top_k > n_experts || !d_logits || !d_ids || !d_w) {
        set_error(QZ_ERR_BAD_SHAPE, "cuda_router_topk: 1 <= top_k <= min(8, n_experts), n_experts <= 256");
        return;
    }
    launch(router_topk_kernel, dim3((unsigned)((m + 7) / 8)), dim3(256), 0, d_logits, d_bias, m, n_experts, top_k, renorm, d_ids,
           d_w);
}

// ======================= row-sharded layers: peer windows =======================
static uint8_t *g_win = nullptr;          // this rank's window (control words + data)
static size_t g_win_data_bytes = 0;
static int g_mg_rank = 0, g_mg_world = 0;
static void *g_peer_base[MGPU_MAX_RANKS] = {};
static bool g_mg_attached = false;

size_t quartz_mgpu_handle_bytes(void) { return sizeof(cudaIpcMemHandle_t); }

int quartz_set_device(int device)
{
    if (cudaSetDevice(device) != cudaSuccess) {
        cudaGetLastError();
        set_error(QZ_ERR_CUDA, "quartz_set_device: cudaSetDevice failed");
        return -1;
    }
    g_sm_count = 0;
    return 0;
}

int quartz_mgpu_init(int rank, int world, size_t data_bytes, void *handle_out)
{
    if (g_win || rank < 0 || world < 1 || world > MGPU_MAX_RANKS || rank >= world || !handle_out) {
        set_error(QZ_ERR_BAD_SHAPE, "quartz_mgpu_init: bad rank/world, or already initialised");
        return -1;
    }
    data_bytes = (data_bytes + 255) & ~(size_t)255;
    if (cudaMalloc(&g_win, MGPU_CTRL_BYTES + data_bytes) != cudaSuccess) {
        cudaGetLastError();
        g_win = nullptr;
        set_error(QZ_ERR_CUDA, "quartz_mgpu_init: cudaMalloc of the window failed");
        return -1;
    }
    QZ_CUDA_CHECK(cudaMemset(g_win, 0, MGPU_CTRL_BYTES + data_bytes));
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, g_win) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(g_win);
        g_win = nullptr;
        set_error(QZ_ERR_CUDA, "quartz_mgpu_init: cudaIpcGetMemHandle failed");
        return -1;
    }
    memcpy(handle_out, &h, sizeof(h));
    g_win_data_bytes = data_bytes;
    g_mg_rank = rank;
    g_mg_world = world;
    g_mg_attached = false;
    return 0;
}

int quartz_mgpu_attach(const void *handles)
{
    if (!g_win || !handles) {
        set_error(QZ_ERR_BAD_SHAPE, "quartz_mgpu_attach: call quartz_mgpu_init first");
        return -1;
    }
    for (int r = 0; r < g_mg_world; r++) {
        if (r == g_mg_rank) {
            g_peer_base[r] = g_win;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + (size_t)r * sizeof(h), sizeof(h));
        void *p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess || !p) {
            cudaGetLastError();
            set_error(QZ_ERR_CUDA, "quartz_mgpu_attach: cudaIpcOpenMemHandle failed (no peer access between the GPUs?)");
            return -1;
        }
        g_peer_base[r] = p;
    }
    g_mg_attached = true;
    return 0;
}

float *quartz_mgpu_data(void) { return g_win ? (float *)(g_win + MGPU_CTRL_BYTES) : nullptr; }

static bool mgpu_is_attached() { return g_mg_attached; }

static bool fill_push(PushArgs &p, size_t dst_off, size_t elems)
{
    if (!g_mg_attached) {
        set_error(QZ_ERR_BAD_SHAPE, "push: the windows are not attached (quartz_mgpu_init / quartz_mgpu_attach)");
        return false;
    }
    if ((dst_off + elems) * sizeof(float) > g_win_data_bytes) {
        set_error(QZ_ERR_BAD_SHAPE, "push: the slice does not fit the window");
        return false;
    }
    for (int r = 0; r < MGPU_MAX_RANKS; r++) {
        uint8_t *b = (uint8_t *)g_peer_base[r < g_mg_world ? r : g_mg_rank];
        p.ctrl[r] = (MgpuCtrl *)b;
        p.data[r] = (float *)(b + MGPU_CTRL_BYTES);
    }
    p.n = g_mg_world;
    p.rank = g_mg_rank;
    p.dst_off = (long long)dst_off;
    p.wait_after = 0;
    return true;
}

// set by quartz_mgpu_wait_in_next_push: the next cuda_gemv_batch_push / cuda_gemv_chain_push / cuda_gemm_push kernel
// completes its own exchange before it ends
static bool g_push_wait_after = false;
static bool push_wait_after_take()
{
    const bool v = g_push_wait_after;
    g_push_wait_after = false;
    return v;
}
void quartz_mgpu_wait_in_next_push(void)
{
    if (!g_mg_attached) {
        set_error(QZ_ERR_BAD_SHAPE, "quartz_mgpu_wait_in_next_push: the windows are not attached");
        return;
    }
    g_push_wait_after = true;
}

void cuda_push_rows(const float *d_src, int m, int n_local, size_t dst_off, size_t dst_ld)
{
    // an empty slice (a rank that owns no rows) still takes part in the exchange: it only publishes
    if (m < 0) m = 0;
    if (n_local < 0) n_local = 0;
    PushArgs p;
    const long long total = (long long)m * n_local;
    if (!fill_push(p, dst_off, total ? (size_t)(m - 1) * dst_ld + n_local : 0)) return;
    int blocks = (int)((total / 4 + 255) / 256);   // (a thread moves up to four values per pass)
    if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
    if (blocks < 1) blocks = 1;
    mgpu_push_rows_kernel<<<blocks, 256, 0, g_stream>>>(d_src, m, n_local, (long long)dst_ld, p);
    QZ_LAUNCH_CHECK();
}

int cuda_gemm_push(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, int m, int in_dim, int out_dim,
                   size_t dst_off, size_t dst_ld)
{
    if (m <= 0 || out_dim <= 0 || dst_ld < (size_t)out_dim) return 0;
    PushArgs p;
    if (!fill_push(p, dst_off, (size_t)(m - 1) * dst_ld + (size_t)out_dim)) return 0;
    p.wait_after = push_wait_after_take() ? 1 : 0;
    return gemm_dispatch(ggml_type, d_data, d_x, nullptr, m, in_dim, out_dim, false, &p, (long long)dst_off, (long long)dst_ld) ? 1 : 0;
}

void cuda_gemv_push(uint32_t ggml_type, const uint8_t *d_data, const float *d_x, size_t dst_off, int in_dim, int out_dim)
{
    if (out_dim <= 0) {
        cuda_push_rows(nullptr, 0, 0, dst_off, 0);
        return;
    }
    if (!fill_push(g_push_args, dst_off, (size_t)out_dim)) return;
    // the streaming kernel stores into every window from its epilogue; any other kernel writes the
    // local window and the slice is pushed by a copy kernel
    float *local = quartz_mgpu_data() + dst_off;
    g_push_pending = true;
    gemv_n(ggml_type, 1, &d_data, &d_x, &local, in_dim, out_dim);
    if (g_push_pending) {
        g_push_pending = false;
        cuda_push_rows(local, 1, out_dim, dst_off, (size_t)out_dim);
    }
}

void quartz_mgpu_wait(void)
{
    if (!g_mg_attached) {
        set_error(QZ_ERR_BAD_SHAPE, "quartz_mgpu_wait: the windows are not attached");
        return;
    }
    int *st = status_word();
    if (!st) return;
    mgpu_wait_kernel<<<1, 32, 0, g_stream>>>((const MgpuCtrl *)g_win, g_mg_world, st);
    QZ_LAUNCH_CHECK();
}

void quartz_mgpu_fuse_next_wait(void)
{
    if (!g_mg_attached) {
        set_error(QZ_ERR_BAD_SHAPE, "quartz_mgpu_fuse_next_wait: the windows are not attached");
        return;
    }
    g_wait_ctrl = (const MgpuCtrl *)g_win;
    g_wait_ranks = g_mg_world;
}

// ---- NCCL all-gather of the f32 output slices (the exchange in library form) ----
// NCCL is bound at run time (dlopen of libnccl.so.2), so the library itself links against nothing but the CUDA
// runtime and still loads on machines without NCCL; the declarations below restate the five NCCL entry points
// used (nccl.h: ncclGetUniqueId, ncclCommInitRank, ncclAllGather, ncclCommDestroy, ncclGetErrorString).
struct QzNcclId { char internal[128]; };   // ncclUniqueId
static void *g_nccl_so = nullptr;
static void *g_nccl_comm = nullptr;
static int (*p_ncclGetUniqueId)(QzNcclId *) = nullptr;
static int (*p_ncclCommInitRank)(void **, int, QzNcclId, int) = nullptr;
static int (*p_ncclAllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
static int (*p_ncclCommDestroy)(void *) = nullptr;
static const char *(*p_ncclGetErrorString)(int) = nullptr;

static bool nccl_bind()
{
    if (g_nccl_so) return true;
    const char *names[] = {getenv("QUARTZ_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n) continue;
        g_nccl_so = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl_so) break;
    }
    if (!g_nccl_so) {
        set_error(QZ_ERR_CUDA, "quartz_nccl: libnccl.so.2 not found (set QUARTZ_NCCL_LIB)");
        return false;
    }
    p_ncclGetUniqueId = (int (*)(QzNcclId *))dlsym(g_nccl_so, "ncclGetUniqueId");
    p_ncclCommInitRank = (int (*)(void **, int, QzNcclId, int))dlsym(g_nccl_so, "ncclCommInitRank");
    p_ncclAllGather = (int (*)(const void *, void *, size_t, int, void *, cudaStream_t))dlsym(g_nccl_so, "ncclAllGather");
    p_ncclCommDestroy = (int (*)(void *))dlsym(g_nccl_so, "ncclCommDestroy");
    p_ncclGetErrorString = (const char *(*)(int))dlsym(g_nccl_so, "ncclGetErrorString");
    if (!p_ncclGetUniqueId || !p_ncclCommInitRank || !p_ncclAllGather || !p_ncclCommDestroy) {
        set_error(QZ_ERR_CUDA, "quartz_nccl: libnccl lacks an entry point");
        dlclose(g_nccl_so);
        g_nccl_so = nullptr;
        return false;
    }
    return true;
}

static bool nccl_ok(int rc, const char *what)
{
    if (rc == 0) return true;
    std::string msg = std::string(what) + ": " + (p_ncclGetErrorString ? p_ncclGetErrorString(rc) : "NCCL error");
    set_error(QZ_ERR_CUDA, msg.c_str());
    return false;
}

size_t quartz_nccl_id_bytes(void) { return sizeof(QzNcclId); }

int quartz_nccl_unique_id(void *id_out)
{
    if (!id_out || !nccl_bind()) return -1;
    QzNcclId id;
    if (!nccl_ok(p_ncclGetUniqueId(&id), "ncclGetUniqueId")) return -1;
    memcpy(id_out, &id, sizeof(id));
    return 0;
}

int quartz_nccl_init(int rank, int world, const void *id)
{
    if (g_nccl_comm || !id || rank < 0 || world < 1 || rank >= world) {
        set_error(QZ_ERR_BAD_SHAPE, "quartz_nccl_init: bad rank/world, or already initialised");
        return -1;
    }
    if (!nccl_bind()) return -1;
    QzNcclId uid;
    memcpy(&uid, id, sizeof(uid));
    void *comm = nullptr;
    if (!nccl_ok(p_ncclCommInitRank(&comm, world, uid, rank), "ncclCommInitRank")) return -1;
    g_nccl_comm = comm;
    g_mg_rank = rank;
    if (!g_mg_world) g_mg_world = world;
    return 0;
}

void quartz_mgpu_allgather(const float *d_send, float *d_recv, size_t count_per_rank)
{
    if (!g_nccl_comm) {
        set_error(QZ_ERR_BAD_SHAPE, "quartz_mgpu_allgather: call quartz_nccl_init first");
        return;
    }
    if (count_per_rank == 0) return;
    g_launch_count++;
    nccl_ok(p_ncclAllGather(d_send, d_recv, count_per_rank, 7 /* ncclFloat32 */, g_nccl_comm, g_stream), "ncclAllGather");
}

void quartz_nccl_shutdown(void)
{
    if (!g_nccl_comm) return;
    cudaDeviceSynchronize();
    p_ncclCommDestroy(g_nccl_comm);
    g_nccl_comm = nullptr;
}

void quartz_mgpu_shutdown(void)
{
    if (!g_win) return;
    cudaDeviceSynchronize();
    for (int r = 0; r < g_mg_world; r++)
        if (r != g_mg_rank && g_peer_base[r]) cudaIpcCloseMemHandle(g_peer_base[r]);
    cudaFree(g_win);
    cudaGetLastError();
    g_win = nullptr;
    g_mg_attached = false;
    g_mg_world = 0;
    for (int r = 0; r < MGPU_MAX_RANKS; r++) g_peer_base[r] = nullptr;
}

}  // extern "C"
