"""Batched mixture-of-experts FFN (cuda_moe_ffn / cuda_moe_ffn_dev, cuda_router_topk) against the CPU oracle: per expert, the oracle's gemm()
(src/dequant.rs:143-200) on the tokens routed to it, SwiGLU, gemm() again, weighted sum in expert order
(src/main.rs:941-990 per token).

Bar: the composite of two chained GEMMs.  Each GEMM is allowed 1e-3 * ||w_row|| * ||x|| (the GEMV/GEMM
bar); an error dh of the hidden vector reaches the output as at most ||w_down_row|| * ||dh||.  The test
bounds the output error of token t, feature j by
    sum_e w(t,e) * ||down_e[j]|| * (1e-3 * ||h_e|| + ||dh_e||_bound),
with ||dh_e||_bound from the gate/up tolerances through SwiGLU's derivative (|d silu| <= 1.1)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _route(rng, m, n_experts, top_k):
    logits = rng.standard_normal((m, n_experts)).astype(np.float32)
    ids = np.argsort(-logits, axis=1)[:, :top_k].astype(np.int32)
    sel = np.take_along_axis(logits, ids, axis=1)
    w = np.exp(sel - sel.max(axis=1, keepdims=True))
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)   # softmax over the selected logits (moe_renorm)
    return np.ascontiguousarray(ids), np.ascontiguousarray(w)


def _silu(x):
    return x / (1.0 + np.exp(-x))


def _check_tokens(oracle_mod, got, X, ids, w, gate, up, down, t_gu, t_dn, K, F, E, tokens):
    """Oracle value and error bound of out[t] for the given tokens (all experts of each)."""
    worst = 0.0
    want = {int(t): np.zeros(K, dtype=np.float64) for t in tokens}
    bound = {int(t): np.zeros(K, dtype=np.float64) for t in tokens}
    tokset = set(int(t) for t in tokens)
    for e in range(E):
        toks, slot = np.nonzero(ids == e)
        keep = [i for i, t in enumerate(toks) if int(t) in tokset]
        if not keep:
            continue
        toks, slot = toks[keep], slot[keep]
        xe = np.ascontiguousarray(X[toks])
        g = oracle_mod.gemm(xe, gate[e], t_gu, K, F, len(toks)).astype(np.float64)
        u = oracle_mod.gemm(xe, up[e], t_gu, K, F, len(toks)).astype(np.float64)
        h = (_silu(g) * u).astype(np.float32)
        y = oracle_mod.gemm(np.ascontiguousarray(h), down[e], t_dn, F, K, len(toks)).astype(np.float64)
        ng, nu = oracle_mod.row_norms(gate[e], t_gu, K, F), oracle_mod.row_norms(up[e], t_gu, K, F)
        nd = oracle_mod.row_norms(down[e], t_dn, F, K)
        for i, (tk, sl) in enumerate(zip(toks, slot)):
            xn = float(np.linalg.norm(xe[i].astype(np.float64)))
            dgate, dup = 1e-3 * ng * xn, 1e-3 * nu * xn
            dh = np.linalg.norm(1.1 * np.abs(u[i]) * dgate + np.abs(_silu(g[i])) * dup + dgate * dup)
            hn = float(np.linalg.norm(h[i].astype(np.float64)))
            want[int(tk)] += w[tk, sl] * y[i]
            bound[int(tk)] += w[tk, sl] * nd * (1e-3 * hn + dh)
    for t in tokset:
        err = np.abs(got[t] - want[t])
        assert np.all(err <= bound[t]), f"token {t}: max err/bound {np.max(err / np.maximum(bound[t], 1e-30)):.3g}"
        worst = max(worst, float(np.max(err / np.maximum(bound[t], 1e-30))))
    return worst


@pytest.mark.parametrize("t_gu,t_dn,repack", [(18, 18, True), (17, 17, True), (12, 14, True), (18, 17, False), (8, 13, True)])
def test_moe_ffn_against_oracle(gpu, oracle_mod, t_gu, t_dn, repack):
    from saient_quartz_b200 import synth
    L = gpu.lib()
    K, F, E, top_k, M = 1024, 2048, 8, 2, 48
    rng = np.random.Generator(np.random.PCG64([0x30E, t_gu, t_dn]))
    gate = [synth.make_weights(t_gu, K, F, tensor_id=800 + e) for e in range(E)]
    up = [synth.make_weights(t_gu, K, F, tensor_id=820 + e) for e in range(E)]
    down = [synth.make_weights(t_dn, F, K, tensor_id=840 + e) for e in range(E)]
    dg, du, dd = (gpu.GpuBuf.upload(np.concatenate(g)) for g in (gate, up, down))
    if repack:
        L.cuda_repack_weights(t_gu, dg.ptr, K, F, E)
        L.cuda_repack_weights(t_gu, du.ptr, K, F, E)
        L.cuda_repack_weights(t_dn, dd.ptr, F, K, E)
    X = synth.make_x(K, tensor_id=860, rows=M)
    ids, w = _route(rng, M, E, top_k)
    ids[0, :] = (3, 3 ^ 1)          # make sure expert order inside a token is not sorted
    ids[ids == 6] = 5               # expert 6 gets no token at all
    dx, dout = gpu.GpuBuf.upload(X), gpu.GpuBuf.alloc_f32(M * K)
    for rep in range(2):            # twice: the scratch and the device-side lists are reused
        L.cuda_vec_zero(dout.ptr, M * K)
        L.cuda_moe_ffn(t_gu, t_dn, dg.ptr, du.ptr, dd.ptr, dx.ptr, dout.ptr, M, K, F, E, top_k, ids.ctypes.data, w.ctypes.data, 0)
        got = dout.download().reshape(M, K).astype(np.float64)
        gpu.check_error("cuda_moe_ffn")
        worst = _check_tokens(oracle_mod, got, X, ids, w, gate, up, down, t_gu, t_dn, K, F, E, range(M))
    print(f"types {t_gu}/{t_dn}: max err/bound {worst:.3g}")


@pytest.mark.parametrize("t", [18, 17])
def test_moe_ffn_benchmark_size_and_device_routing(gpu, oracle_mod, t):
    """The benchmarked configuration (8 experts, top-2, 256 tokens, 4096 <-> 14336, IQ3_XXS / IQ2_XS) with the
    routing done on the device: cuda_router_topk from the router logits, cuda_moe_ffn_dev on its lists.  The router
    is compared with numpy exactly (ids) and to 1e-6 (weights); the FFN output of 20 tokens (first, last, random)
    against the oracle.  IQ3_XXS has no counterpart in the reference: its oracle is pinned to gguf-py only."""
    from saient_quartz_b200 import synth
    L = gpu.lib()
    K, F, E, top_k, M = 4096, 14336, 8, 2, 256
    rng = np.random.Generator(np.random.PCG64([0x30F, t]))
    gate = [synth.make_weights(t, K, F, tensor_id=900 + e) for e in range(E)]
    up = [synth.make_weights(t, K, F, tensor_id=920 + e) for e in range(E)]
    down = [synth.make_weights(t, F, K, tensor_id=940 + e) for e in range(E)]
    dg, du, dd = (gpu.GpuBuf.upload(np.concatenate(g)) for g in (gate, up, down))
    L.cuda_repack_weights(t, dg.ptr, K, F, E)
    L.cuda_repack_weights(t, du.ptr, K, F, E)
    L.cuda_repack_weights(t, dd.ptr, F, K, E)
    X = synth.make_x(K, tensor_id=960, rows=M)
    logits = rng.standard_normal((M, E)).astype(np.float32)
    logits[5, 2] = logits[5, 6] = logits[5].max() + 1.0     # a tie: the lower index comes first
    ids = np.argsort(-logits, axis=1, kind="stable")[:, :top_k].astype(np.int32)
    sel = np.take_along_axis(logits, ids, axis=1)
    w = np.exp(sel - sel.max(axis=1, keepdims=True))
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    dl = gpu.GpuBuf.upload(logits)
    d_ids, d_w = gpu.GpuBuf.alloc_f32(M * top_k), gpu.GpuBuf.alloc_f32(M * top_k)
    L.cuda_router_topk(dl.ptr, None, M, E, top_k, 1, d_ids.ptr, d_w.ptr)
    got_ids, got_w = d_ids.download(np.int32).reshape(M, top_k), d_w.download().reshape(M, top_k)
    assert np.array_equal(got_ids, ids)
    assert np.abs(got_w - w).max() < 1e-6
    # softmax over all experts (moe_renorm = 0), with a bias
    bias = rng.standard_normal(E).astype(np.float32)
    db = gpu.GpuBuf.upload(bias)
    lb = logits + bias
    ids3 = np.argsort(-lb, axis=1, kind="stable")[:, :top_k].astype(np.int32)
    p_all = np.exp(lb - lb.max(axis=1, keepdims=True))
    p_all = p_all / p_all.sum(axis=1, keepdims=True)
    d_ids3, d_w3 = gpu.GpuBuf.alloc_f32(M * top_k), gpu.GpuBuf.alloc_f32(M * top_k)
    L.cuda_router_topk(dl.ptr, db.ptr, M, E, top_k, 0, d_ids3.ptr, d_w3.ptr)
    assert np.array_equal(d_ids3.download(np.int32).reshape(M, top_k), ids3)
    assert np.abs(d_w3.download().reshape(M, top_k) - np.take_along_axis(p_all, ids3, axis=1)).max() < 1e-6
    # the FFN on the device-side lists
    dx, dout = gpu.GpuBuf.upload(X), gpu.GpuBuf.alloc_f32(M * K)
    L.cuda_moe_ffn_dev(t, t, dg.ptr, du.ptr, dd.ptr, dx.ptr, dout.ptr, M, K, F, E, top_k, d_ids.ptr, d_w.ptr, 0)
    got = dout.download().reshape(M, K).astype(np.float64)
    gpu.check_error("cuda_moe_ffn_dev")
    tokens = sorted(set([0, 1, 2, 3, 5, 252, 253, 254, 255] + [int(v) for v in rng.integers(0, M, size=11)]))
    worst = _check_tokens(oracle_mod, got, X, ids, w, gate, up, down, t, t, K, F, E, tokens)
    print(f"type {t} at benchmark size: max err/bound {worst:.3g} over {len(tokens)} tokens")


def test_moe_ffn_rejects_bad_routing(gpu):
    L = gpu.lib()
    ids = np.array([[0, 9]], dtype=np.int32)
    w = np.array([[0.5, 0.5]], dtype=np.float32)
    buf = gpu.GpuBuf.alloc_f32(4096)
    L.cuda_moe_ffn(12, 12, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 1, 256, 256, 8, 2, ids.ctypes.data, w.ctypes.data, 0)
    assert L.quartz_last_error() == 2      # QZ_ERR_BAD_SHAPE
    L.quartz_clear_error()
