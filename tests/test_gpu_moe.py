"""Batched mixture-of-experts FFN (cuda_moe_ffn) against the CPU oracle: per expert, the oracle's gemm()
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


@pytest.mark.parametrize("t_gu,t_dn,repack", [(18, 18, True), (17, 17, True), (12, 14, True), (18, 17, False)])
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
    dx, dout = gpu.GpuBuf.upload(X), gpu.GpuBuf.alloc_f32(M * K)
    L.cuda_moe_ffn(t_gu, t_dn, dg.ptr, du.ptr, dd.ptr, dx.ptr, dout.ptr, M, K, F, E, top_k, ids.ctypes.data, w.ctypes.data, 0)
    got = dout.download().reshape(M, K).astype(np.float64)
    gpu.check_error("cuda_moe_ffn")

    want = np.zeros((M, K), dtype=np.float64)
    bound = np.zeros((M, K), dtype=np.float64)
    for e in range(E):
        toks, slot = np.nonzero(ids == e)
        if len(toks) == 0:
            continue
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
            want[tk] += w[tk, sl] * y[i]
            bound[tk] += w[tk, sl] * nd * (1e-3 * hn + dh)
    err = np.abs(got - want)
    assert np.all(err <= bound), f"max err/bound {np.max(err / np.maximum(bound, 1e-30)):.3g}"
    print(f"types {t_gu}/{t_dn}: max err/bound {np.max(err / np.maximum(bound, 1e-30)):.3g}")


def test_moe_ffn_rejects_bad_routing(gpu):
    L = gpu.lib()
    ids = np.array([[0, 9]], dtype=np.int32)
    w = np.array([[0.5, 0.5]], dtype=np.float32)
    buf = gpu.GpuBuf.alloc_f32(4096)
    L.cuda_moe_ffn(12, 12, buf.ptr, buf.ptr, buf.ptr, buf.ptr, buf.ptr, 1, 256, 256, 8, 2, ids.ctypes.data, w.ctypes.data, 0)
    assert L.quartz_last_error() == 2      # QZ_ERR_BAD_SHAPE
    L.quartz_clear_error()
