"""GPU tests of the decode step: the C++ host mirror of GpuForwardState::forward_gpu_step
(src/cuda.rs:507-851) over the C ABI -- reference sequence and fused/graph sequence -- against the
numpy restatement of the reference's CPU forward (src/main.rs:1045-1120).

Bar: logits within 5e-3 of max|logit| (the end-to-end analogue of the reference's --verify-gemv
relative check, src/main.rs:2653-2659, with room for 2 x n_layers chained f32 GEMVs); the fused
sequence and the reference sequence agree to 1e-3 of max|logit|."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float(np.abs(a.astype(np.float64) - b).max() / max(np.abs(b).max(), 1e-30))


def _tiny_dense(gpu, repack=True, types=None, **over):
    """Llama-shaped miniature.  Q6_K planes need in_dim % 2048 == 0, hence 2048 / 4096."""
    from saient_quartz_b200.host_model import HostModel, Q4K_M_TYPES
    cfg = dict(vocab_size=320, embed_dim=2048, n_heads=16, n_kv_heads=4, n_layers=3, ffn_dim=4096, head_dim=128,
               rope_theta=500000.0, max_seq=96)
    cfg.update(over)
    m = HostModel(repack=repack, keep_host=True, types=types or Q4K_M_TYPES, **cfg)
    m.fill_synthetic()
    return m


def _ref_for(m, oracle_mod, kv):
    from oracle.forward_ref import RefModel
    r = RefModel(m.cfg, m.host)
    for l, (k, v) in enumerate(kv):
        r.set_kv(l, k, v)
    return r


@pytest.mark.parametrize("repack", [True, False])
def test_tiny_dense_model_both_sequences(gpu, oracle_mod, repack):
    m = _tiny_dense(gpu, repack=repack)
    kv = m.fill_kv(40, keep=True)
    ref = _ref_for(m, oracle_mod, kv)
    want = ref.forward(17, 40)
    got = m.step(17, 40, fused=False)
    assert _rel(got, want) < 5e-3
    n_ref = m.launches()
    got_f = m.step(17, 40, fused=True)
    assert _rel(got_f, want) < 5e-3
    assert _rel(got_f, got) < 1e-3
    if repack:
        assert m.launches() < n_ref          # the fused sequence needs fewer launches
    # the recorded graph replays to the same numbers
    again = m.step(17, 40, fused=True)
    assert np.array_equal(again, got_f)
    # the chained sequence (one persistent kernel per layer for the four dependent GEMVs)
    got_c = m.step(17, 40, fused=2)
    assert _rel(got_c, want) < 5e-3 and _rel(got_c, got_f) < 1e-3
    if repack:
        assert m.launches() < 5 * 3 + 4       # four launches per layer + embedding + first q/k/v
    assert np.array_equal(m.step(17, 40, fused=2), got_c)
    gpu.check_error()


def test_small_dims_q4k_q8_0(gpu, oracle_mod):
    """Rows narrower than a warp of 64-weight units (in_dim 512 / 1024): the sub-warp row mode."""
    types = dict(Q=12, K=12, V=12, O=12, GATE=12, UP=12, DOWN=8, LM_HEAD=8, EMBED=14)
    m = _tiny_dense(gpu, types=types, embed_dim=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn_dim=1024)
    kv = m.fill_kv(33, keep=True)
    want = _ref_for(m, oracle_mod, kv).forward(5, 33)
    got, n_ref = m.step(5, 33, fused=False), m.launches()
    got_f = m.step(5, 33, fused=True)
    assert _rel(got, want) < 5e-3 and _rel(got_f, want) < 5e-3
    assert m.launches() < n_ref
    gpu.check_error()


def test_decode_several_positions_and_neox(gpu, oracle_mod):
    m = _tiny_dense(gpu, rope_neox=1)
    kv = m.fill_kv(5, keep=True)
    ref = _ref_for(m, oracle_mod, kv)
    for pos, tok in ((5, 3), (6, 300), (7, 0)):
        want = ref.forward(tok, pos)
        got = m.step(tok, pos, fused=(pos % 2 == 0))
        assert _rel(got, want) < 5e-3, pos
    gpu.check_error()


def test_generation_loop_through_one_recorded_graph(gpu, oracle_mod):
    """Consecutive positions with different tokens through the fused and the chained sequence: token id and
    position are device words, so the step is recorded once per model and sequence kind and replayed for
    every step (src/cuda.rs:507-851 takes `token` and `pos` per call)."""
    for fused in (1, 2):
        m = _tiny_dense(gpu)
        kv = m.fill_kv(29, keep=True)
        ref = _ref_for(m, oracle_mod, kv)
        # 29 .. 34 crosses a 32-position block boundary of the attention kernel
        for pos, tok in ((29, 3), (30, 300), (31, 0), (32, 77), (33, 5), (34, 5)):
            want = ref.forward(tok, pos)
            got = m.step(tok, pos, fused=fused)
            assert _rel(got, want) < 5e-3, (fused, pos)
        assert m.graphs_recorded() == 1, fused
        m.close()
    gpu.check_error()


def test_layers_with_different_quantization_types(gpu, oracle_mod):
    """A *_K_M-style mix: q/k/v (and the other projections) use another block format in every layer, so the
    byte size of a q slice differs from layer to layer."""
    from saient_quartz_b200 import synth
    from saient_quartz_b200.host_model import HostModel
    cfg = dict(vocab_size=320, embed_dim=2048, n_heads=16, n_kv_heads=4, n_layers=3, ffn_dim=4096, head_dim=128,
               rope_theta=500000.0, max_seq=64)
    m = HostModel(keep_host=True, **cfg)
    rng = np.random.Generator(np.random.PCG64([0x717]))
    d, fd, q_d, kv_d = 2048, 4096, 2048, 512
    tid = [900]

    def w(role, l, t, K, N):
        tid[0] += 1
        m.set(role, l, t, synth.make_weights(t, K, N, tensor_id=tid[0]))

    def norm(role, l, n):
        m.set(role, l, 0, (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32))

    w("EMBED", 0, 12, d, 320)
    for l, (tq, to, tg, td) in enumerate(((12, 12, 12, 14), (8, 14, 8, 12), (14, 8, 13, 8))):
        w("Q", l, tq, d, q_d); w("K", l, tq, d, kv_d); w("V", l, tq, d, kv_d); w("O", l, to, q_d, d)
        w("GATE", l, tg, d, fd); w("UP", l, tg, d, fd); w("DOWN", l, td, fd, d)
        norm("ATTN_NORM", l, d); norm("FFN_NORM", l, d)
    norm("FINAL_NORM", 0, d)
    w("LM_HEAD", 0, 14, d, 320)
    m.finalize()
    kv = m.fill_kv(10, keep=True)
    ref = _ref_for(m, oracle_mod, kv)
    for pos, tok in ((10, 1), (11, 319)):
        want = ref.forward(tok, pos)
        got_f = m.step(tok, pos, fused=1)
        assert _rel(got_f, want) < 5e-3, pos
    assert m.launches() <= 6 * 3 + 2      # the fused sequence ran (not the reference sequence)
    kv2 = m.fill_kv(10)
    ref2 = _ref_for(m, oracle_mod, kv)
    for pos, tok in ((10, 1), (11, 319)):
        assert _rel(m.step(tok, pos, fused=2), ref2.forward(tok, pos)) < 5e-3, pos
    gpu.check_error()


def test_first_token_empty_cache(gpu, oracle_mod):
    m = _tiny_dense(gpu)
    ref = _ref_for(m, oracle_mod, [])
    assert _rel(m.step(9, 0, fused=False), ref.forward(9, 0)) < 5e-3
    m2 = _tiny_dense(gpu)
    assert _rel(m2.step(9, 0, fused=True), _ref_for(m2, oracle_mod, []).forward(9, 0)) < 5e-3


@pytest.mark.parametrize("n_used", [2, 4])
def test_tiny_moe_model(gpu, oracle_mod, n_used):
    """MoE branch (src/cuda.rs:667-798): general path (top-2) and the four-expert launch (top-4),
    biases, sinks, QK-norm, YaRN and a sliding window switched on together."""
    from saient_quartz_b200 import synth
    from saient_quartz_b200.host_model import HostModel
    cfg = dict(vocab_size=256, embed_dim=256, n_heads=4, n_kv_heads=2, n_layers=2, ffn_dim=512, head_dim=64,
               rope_theta=150000.0, max_seq=64, n_experts=6, n_experts_used=n_used, moe_renorm=int(n_used == 2),
               clamped_swiglu=int(n_used == 4), swa_window=8, rope_neox=1, yarn_scale=4.0, yarn_orig_ctx=32)
    m = HostModel(keep_host=True, **cfg)
    rng = np.random.Generator(np.random.PCG64([77, n_used]))
    d, fd, q_d, kv_d, ne = 256, 512, 256, 128, 6
    tid = [500]

    def w(role, l, t, K, N):
        tid[0] += 1
        m.set(role, l, t, synth.make_weights(t, K, N, tensor_id=tid[0]))

    def f(role, l, n, scale=1.0, base=0.0):
        m.set(role, l, 0, (base + scale * rng.standard_normal(n)).astype(np.float32))

    w("EMBED", 0, 7, d, 256)
    for l in range(2):
        w("Q", l, 12, d, q_d); w("K", l, 14, d, kv_d); w("V", l, 8, d, kv_d); w("O", l, 7, q_d, d)
        f("ATTN_NORM", l, d, 0.1, 1.0); f("FFN_NORM", l, d, 0.1, 1.0)
        f("Q_NORM", l, 64, 0.1, 1.0); f("K_NORM", l, kv_d, 0.1, 1.0)
        f("Q_BIAS", l, q_d, 0.01); f("K_BIAS", l, kv_d, 0.01); f("V_BIAS", l, kv_d, 0.01); f("O_BIAS", l, d, 0.01)
        f("SINKS", l, 4)
        w("MOE_GATE", l, 17 if l else 12, d, fd * ne); w("MOE_UP", l, 12, d, fd * ne); w("MOE_DOWN", l, 14, fd, d * ne)
        f("ROUTER_W", l, ne * d, 0.2); f("ROUTER_B", l, ne, 0.1)
        f("MOE_GATE_BIAS", l, ne * fd, 0.01); f("MOE_UP_BIAS", l, ne * fd, 0.01); f("MOE_DOWN_BIAS", l, ne * d, 0.01)
    f("FINAL_NORM", 0, d, 0.1, 1.0)
    w("LM_HEAD", 0, 30, d, 256)
    m.finalize()
    kv = m.fill_kv(20, keep=True)
    ref = _ref_for(m, oracle_mod, kv)
    for pos, tok in ((20, 11), (21, 200)):
        want = ref.forward(tok, pos)
        got = m.step(tok, pos, fused=True)   # not fusable: must fall back to the reference sequence
        assert _rel(got, want) < 5e-3, (n_used, pos)
    gpu.check_error()


@pytest.mark.parametrize("n_used", [2, 5])
def test_moe_model_routed_on_the_device(gpu, oracle_mod, n_used):
    """MoE layers whose expert tensors the streaming GEMV serves: router top-k, expert selection, bias + SwiGLU and
    the weighted sum stay on the device (no device-to-host copy per layer, unlike src/cuda.rs:673-701).  Against the
    CPU oracle, and against the same model routed on the host (same experts, same arithmetic: equal to 1e-5)."""
    from saient_quartz_b200 import synth
    from saient_quartz_b200.host_model import HostModel, host_lib
    cfg = dict(vocab_size=256, embed_dim=512, n_heads=8, n_kv_heads=2, n_layers=2, ffn_dim=1024, head_dim=64,
               rope_theta=10000.0, max_seq=48, n_experts=6, n_experts_used=n_used, moe_renorm=int(n_used == 2),
               clamped_swiglu=int(n_used == 5))
    d, fd, q_d, kv_d, ne = 512, 1024, 512, 128, 6
    H = host_lib()

    def build():
        m = HostModel(keep_host=True, **cfg)
        rng = np.random.Generator(np.random.PCG64([78, n_used]))
        tid = [700]

        def w(role, l, t, K, N):
            tid[0] += 1
            m.set(role, l, t, synth.make_weights(t, K, N, tensor_id=tid[0]))

        def f(role, l, n, scale=1.0, base=0.0):
            m.set(role, l, 0, (base + scale * rng.standard_normal(n)).astype(np.float32))

        w("EMBED", 0, 12, d, 256)
        for l in range(2):
            w("Q", l, 12, d, q_d); w("K", l, 12, d, kv_d); w("V", l, 12, d, kv_d); w("O", l, 12, q_d, d)
            f("ATTN_NORM", l, d, 0.1, 1.0); f("FFN_NORM", l, d, 0.1, 1.0)
            w("MOE_GATE", l, 12, d, fd * ne); w("MOE_UP", l, 12 if l else 13, d, fd * ne); w("MOE_DOWN", l, 12, fd, d * ne)
            f("ROUTER_W", l, ne * d, 0.2); f("ROUTER_B", l, ne, 0.1)
            f("MOE_GATE_BIAS", l, ne * fd, 0.01); f("MOE_UP_BIAS", l, ne * fd, 0.01); f("MOE_DOWN_BIAS", l, ne * d, 0.01)
        f("FINAL_NORM", 0, d, 0.1, 1.0)
        w("LM_HEAD", 0, 12, d, 256)
        m.finalize()
        return m

    m = build()
    kv = m.fill_kv(9, keep=True)
    ref = _ref_for(m, oracle_mod, kv)
    got = {}
    for pos, tok in ((9, 11), (10, 200)):
        want = ref.forward(tok, pos)
        got[pos] = m.step(tok, pos, fused=False)
        assert _rel(got[pos], want) < 5e-3, (n_used, pos)
    gpu.check_error()
    try:
        H.qh_force_host_router(1)
        m2 = build()
        m2.fill_kv(9)
        for pos, tok in ((9, 11), (10, 200)):
            assert _rel(m2.step(tok, pos, fused=False), got[pos].astype(np.float64)) < 1e-5, (n_used, pos)
    finally:
        H.qh_force_host_router(0)
    gpu.check_error()


def test_batched_prefill_matches_token_by_token(gpu, oracle_mod):
    """qh_prefill (tensor-core GEMMs over the whole prompt, batched RoPE / KV append / causal attention) followed by
    one decode step gives the logits of n + 1 decode steps (bar 5e-3 of max |logit|; the GEMM carries weights and
    activations as bf16) and leaves the same cache rows (to the same relative bar); continuing a context (pos0 > 0)
    and a prompt whose length is not a multiple of any tile; logits of the prompt's last token against the oracle."""
    for (n, pos0) in ((37, 0), (21, 12)):
        rng = np.random.Generator(np.random.PCG64([0x9F, n]))
        tokens = rng.integers(0, 320, size=n + 1)
        a, b = _tiny_dense(gpu), _tiny_dense(gpu)
        kv = a.fill_kv(pos0, keep=True) if pos0 else []
        if pos0:
            b.fill_kv(pos0)
        ref = _ref_for(a, oracle_mod, kv)
        for i in range(n):
            last_a = a.step(int(tokens[i]), pos0 + i, fused=True)
            want = ref.forward(int(tokens[i]), pos0 + i)
        last_b = b.prefill(tokens[:n], pos0)
        assert _rel(last_b, want) < 5e-3, (n, pos0)
        assert _rel(last_b, last_a.astype(np.float64)) < 5e-3, (n, pos0)
        for l in range(3):
            ka, va = a.read_kv(l, pos0, n)
            kb, vb = b.read_kv(l, pos0, n)
            assert np.abs(ka - kb).max() <= 5e-3 * np.abs(ka).max() and np.abs(va - vb).max() <= 5e-3 * np.abs(va).max(), l
        nxt_a = a.step(int(tokens[n]), pos0 + n, fused=True)
        nxt_b = b.step(int(tokens[n]), pos0 + n, fused=True)
        assert _rel(nxt_b, nxt_a.astype(np.float64)) < 5e-3, (n, pos0)
        a.close(); b.close()
    gpu.check_error()


def test_batched_prefill_llama8b_shape_512_tokens(gpu):
    """The Llama-3-8B-shaped model: a 512-token prompt through qh_prefill, then one decode step, against 513 decode
    steps (bar 5e-3 of max |logit|)."""
    from saient_quartz_b200.host_model import HostModel, LLAMA3_8B
    n = 512
    rng = np.random.Generator(np.random.PCG64([0x9E]))
    tokens = rng.integers(0, LLAMA3_8B["vocab_size"], size=n + 1)
    m = HostModel(**LLAMA3_8B)
    m.fill_synthetic()
    for i in range(n):
        m.step_device(int(tokens[i]), i, 1)
    want = m.step(int(tokens[n]), n, fused=True)
    ka, va = m.read_kv(31, 0, n)
    m.prefill(tokens[:n], 0, want_logits=False)
    kb, vb = m.read_kv(31, 0, n)
    got = m.step(int(tokens[n]), n, fused=True)
    rk, rv = np.abs(ka - kb).max() / np.abs(ka).max(), np.abs(va - vb).max() / np.abs(va).max()
    print(f"layer-31 cache rows: rel diff K {rk:.2e} V {rv:.2e}; logits rel diff {_rel(got, want.astype(np.float64)):.2e}")
    assert rk <= 2e-2 and rv <= 2e-2      # 32 layers of bf16-operand GEMMs against integer-dot GEMVs
    assert _rel(got, want.astype(np.float64)) < 5e-3
    m.close()
    gpu.check_error()


def test_fused_entry_points_match_unfused(gpu):
    """cuda_rms_norm_q / cuda_swiglu_q / cuda_quantize_x + cuda_gemv_q reproduce cuda_rms_norm /
    cuda_swiglu + cuda_gemv bit for bit (same conversion, same kernels); accumulate adds."""
    import ctypes as C
    from saient_quartz_b200 import synth
    L = gpu.lib()
    K, N = 4096, 1024
    w = synth.make_weights(12, K, 2 * N, tensor_id=601)
    dw = gpu.GpuBuf.upload(w)
    x, g = synth.make_x(K, tensor_id=602), synth.make_x(K, tensor_id=603)
    nw = (1.0 + 0.1 * synth.make_x(K, tensor_id=604)).astype(np.float32)
    dx, dg, dn = gpu.GpuBuf.upload(x), gpu.GpuBuf.upload(g), gpu.GpuBuf.upload(nw)
    dt, dy, dy2 = gpu.GpuBuf.alloc_f32(K), gpu.GpuBuf.alloc_f32(2 * N), gpu.GpuBuf.alloc_f32(2 * N)
    half = synth.type_size(12, K * N)

    def gemv_q(slot, acc):
        W = (C.c_void_p * 2)(dw.ptr, dw.ptr + half)
        Y = (C.c_void_p * 2)(dy2.ptr, dy2.ptr + 4 * N)
        S = (C.c_int * 2)(slot, slot)
        L.cuda_gemv_q(12, 2, W, S, Y, K, N, acc)

    for mode in ("norm", "swiglu", "plain"):
        if mode == "norm":
            L.cuda_rms_norm(dt.ptr, dx.ptr, dn.ptr, K)
            L.cuda_rms_norm_q(dx.ptr, dn.ptr, K, 1, None)
        elif mode == "swiglu":
            L.cuda_swiglu(dt.ptr, dg.ptr, dx.ptr, K)
            L.cuda_swiglu_q(dg.ptr, dx.ptr, K, 1, 0)
        else:
            L.cuda_vec_zero(dt.ptr, K)
            L.cuda_vec_add(dt.ptr, dx.ptr, K)
            L.cuda_quantize_x(dx.ptr, K, 1)
        L.cuda_gemv(12, dw.ptr, dt.ptr, dy.ptr, K, 2 * N)
        gemv_q(1, 0)
        a, b = dy.download(), dy2.download()
        assert np.array_equal(a, b), mode
        gemv_q(1, 1)
        assert np.array_equal(dy2.download(), b + b), mode
    gpu.check_error()


@pytest.mark.parametrize("t,K,N", [(12, 4096, 1024), (14, 14336, 512), (8, 2048, 300), (12, 512, 256)])
def test_gemv_with_fused_norm_and_swiglu(gpu, t, K, N):
    """cuda_gemv_rmsnorm / cuda_gemv_swiglu (activation computed in the GEMV's prologue) against the
    two-launch forms cuda_rms_norm_q / cuda_swiglu_q + cuda_gemv_q.  The norm's sum of squares is reduced in
    another order and the prologue's SwiGLU uses the fast exponential and divide (2e-5 relative)."""
    import ctypes as C
    from saient_quartz_b200 import synth
    L = gpu.lib()
    w = synth.make_weights(t, K, 2 * N, tensor_id=611)
    dw = gpu.GpuBuf.upload(w)
    L.cuda_repack_weights(t, dw.ptr, K, 2 * N, 1)
    assert L.cuda_gemv_q_supported(t, dw.ptr, K)
    x, g = synth.make_x(K, tensor_id=612), synth.make_x(K, tensor_id=613)
    nw = (1.0 + 0.1 * synth.make_x(K, tensor_id=614)).astype(np.float32)
    dx, dg, dn = gpu.GpuBuf.upload(x), gpu.GpuBuf.upload(g), gpu.GpuBuf.upload(nw)
    dy, dy2 = gpu.GpuBuf.alloc_f32(2 * N), gpu.GpuBuf.alloc_f32(2 * N)
    half = synth.type_size(t, K * N)
    W = (C.c_void_p * 2)(dw.ptr, dw.ptr + half)
    Y = (C.c_void_p * 2)(dy.ptr, dy.ptr + 4 * N)
    Y2 = (C.c_void_p * 2)(dy2.ptr, dy2.ptr + 4 * N)
    S = (C.c_int * 2)(1, 1)
    for acc in (0, 1):
        L.cuda_vec_zero(dy.ptr, 2 * N)
        L.cuda_vec_zero(dy2.ptr, 2 * N)
        L.cuda_rms_norm_q(dx.ptr, dn.ptr, K, 1, None)
        L.cuda_gemv_q(t, 2, W, S, Y, K, N, acc)
        L.cuda_gemv_rmsnorm(t, 2, W, Y2, dx.ptr, dn.ptr, K, N, acc)
        a, b = dy.download(), dy2.download()
        assert np.abs(a - b).max() <= 2e-5 * np.abs(a).max(), ("norm", acc)
        L.cuda_vec_zero(dy.ptr, 2 * N)
        L.cuda_vec_zero(dy2.ptr, 2 * N)
        L.cuda_swiglu_q(dg.ptr, dx.ptr, K, 1, 0)
        L.cuda_gemv_q(t, 2, W, S, Y, K, N, acc)
        L.cuda_gemv_swiglu(t, 2, W, Y2, dg.ptr, dx.ptr, 0, K, N, acc)
        a, b = dy.download(), dy2.download()
        assert np.abs(a - b).max() <= 2e-5 * np.abs(a).max(), ("swiglu", acc)
    gpu.check_error()


@pytest.mark.parametrize("d,fd", [(4096, 14336), (2048, 4096)])
def test_gemv_chain_matches_separate_launches(gpu, d, fd):
    """cuda_gemv_chain (o-projection -> gate/up -> down -> next q/k/v in one persistent kernel, grid-wide
    barriers between the links) against the same four GEMVs as separate launches.  Run three times: the
    barrier words must reset themselves."""
    import ctypes as C
    from saient_quartz_b200 import synth
    L = gpu.lib()
    kvd = d // 4

    def mat(t, K, N, tid):
        b = gpu.GpuBuf.upload(synth.make_weights(t, K, N, tensor_id=tid))
        L.cuda_repack_weights(t, b.ptr, K, N, 1)
        return b
    wo, wg, wu, wd = mat(12, d, d, 621), mat(12, d, fd, 622), mat(12, d, fd, 623), mat(14, fd, d, 624)
    wq, wk = mat(12, d, kvd, 625), mat(12, d, kvd, 626)
    attn = synth.make_x(d, tensor_id=631)
    hid0 = synth.make_x(d, tensor_id=632)
    n1 = (1.0 + 0.1 * synth.make_x(d, tensor_id=633)).astype(np.float32)
    n2 = (1.0 + 0.1 * synth.make_x(d, tensor_id=634)).astype(np.float32)
    d_attn, d_n1, d_n2 = gpu.GpuBuf.upload(attn), gpu.GpuBuf.upload(n1), gpu.GpuBuf.upload(n2)

    def run(chain):
        hid = gpu.GpuBuf.upload(hid0)
        g, u = gpu.GpuBuf.alloc_f32(fd), gpu.GpuBuf.alloc_f32(fd)
        qo, ko = gpu.GpuBuf.alloc_f32(kvd), gpu.GpuBuf.alloc_f32(kvd)
        ops = [gpu.chain_op(12, [wo.ptr], [hid.ptr], d, d, 1, 3, d_attn.ptr),
               gpu.chain_op(12, [wg.ptr, wu.ptr], [g.ptr, u.ptr], d, fd, 0, 1, hid.ptr, d_n1.ptr),
               gpu.chain_op(14, [wd.ptr], [hid.ptr], fd, d, 1, 2, g.ptr, u.ptr),
               gpu.chain_op(12, [wq.ptr, wk.ptr], [qo.ptr, ko.ptr], d, kvd, 0, 1, hid.ptr, d_n2.ptr)]
        arr = (gpu.ChainOp * 4)(*ops)
        if chain:
            assert L.cuda_gemv_chain_supported(4, arr) == 1
            L.cuda_gemv_chain(4, arr)
        else:
            for op in ops:
                one = (gpu.ChainOp * 1)(op)
                if op.src_mode == 1:
                    L.cuda_gemv_rmsnorm(op.ggml_type, op.n_mats, op.d_w, op.d_y, op.d_a, op.d_b, op.in_dim, op.out_dim, op.accumulate)
                elif op.src_mode == 2:
                    L.cuda_gemv_swiglu(op.ggml_type, op.n_mats, op.d_w, op.d_y, op.d_a, op.d_b, 0, op.in_dim, op.out_dim, op.accumulate)
                else:
                    S = (C.c_int * 1)(2)
                    L.cuda_quantize_x(op.d_a, op.in_dim, 2)
                    L.cuda_gemv_q(op.ggml_type, 1, op.d_w, S, op.d_y, op.in_dim, op.out_dim, op.accumulate)
        L.cuda_sync()
        gpu.check_error("chain" if chain else "separate")
        return [b.download() for b in (hid, g, u, qo, ko)]
    want = run(False)
    for rep in range(3):
        got = run(True)
        for name, a, b in zip(("hidden", "gate", "up", "q", "k"), want, got):
            assert np.abs(a - b).max() <= 5e-5 * max(np.abs(a).max(), 1e-30), (name, rep)


def test_attn_decode_matches_three_kernel_attention(gpu):
    L = gpu.lib()
    r = np.random.Generator(np.random.PCG64([0xA77]))
    for (nh, nkv, hd, seq, max_seq, sink) in [(32, 8, 128, 1025, 1100, False), (8, 8, 64, 33, 64, True),
                                              (12, 2, 96, 70, 128, True), (4, 1, 128, 1, 16, False)]:
        kv_dim = nkv * hd
        kc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
        vc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
        q = r.standard_normal(nh * hd, dtype=np.float32)
        sinks = r.standard_normal(nh, dtype=np.float32) if sink else np.full(nh, -np.inf, np.float32)
        dk, dv, dq, ds = gpu.GpuBuf.upload(kc), gpu.GpuBuf.upload(vc), gpu.GpuBuf.upload(q), gpu.GpuBuf.upload(sinks)
        dsc, d1, d2 = gpu.GpuBuf.alloc_f32(nh * max_seq), gpu.GpuBuf.alloc_f32(nh * hd), gpu.GpuBuf.alloc_f32(nh * hd)
        scale = np.float32(1.0 / np.sqrt(hd))
        L.cuda_attn_score_all(dsc.ptr, dq.ptr, dk.ptr, nh, nkv, seq, hd, kv_dim, max_seq, scale)
        L.cuda_softmax_sink_all(dsc.ptr, nh, seq, max_seq, ds.ptr)
        L.cuda_attn_values_all(d1.ptr, dsc.ptr, dv.ptr, nh, nkv, seq, hd, kv_dim, max_seq)
        L.cuda_attn_decode(d2.ptr, dq.ptr, dk.ptr, dv.ptr, nh, nkv, seq, hd, kv_dim, scale, ds.ptr, -1)
        a, b = d1.download(), d2.download()
        assert np.abs(a - b).max() <= 2e-5 * max(np.abs(a).max(), 1e-30)
    gpu.check_error()


@pytest.mark.parametrize("neox", [0, 1])
def test_attn_block_matches_separate_launches(gpu, neox):
    """cuda_attn_block (RoPE + KV append + attention + merge in one launch) against cuda_rope_kv +
    cuda_attn_decode: same output, same cache rows, q / k_new left un-rotated; called twice in a row
    (the per-kv-head counters must have reset themselves)."""
    L = gpu.lib()
    r = np.random.Generator(np.random.PCG64([0xA78, neox]))
    for (nh, nkv, hd, pos, k_start, max_seq, sink) in [(32, 8, 128, 1024, 0, 1100, False), (8, 8, 64, 32, 0, 64, True),
                                                       (12, 2, 96, 69, 5, 128, True), (4, 1, 128, 0, 0, 16, False),
                                                       (16, 4, 128, 31, 0, 40, False)]:
        kv_dim = nkv * hd
        kc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
        vc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
        q = r.standard_normal(nh * hd, dtype=np.float32)
        k = r.standard_normal(kv_dim, dtype=np.float32)
        v = r.standard_normal(kv_dim, dtype=np.float32)
        sinks = r.standard_normal(nh, dtype=np.float32) if sink else np.full(nh, -np.inf, np.float32)
        scale = np.float32(1.0 / np.sqrt(hd))
        theta, ys, yc = np.float32(500000.0), np.float32(1.0), 0
        seq = pos - k_start + 1
        # separate launches (they rotate q and k in place)
        dk1, dv1 = gpu.GpuBuf.upload(kc), gpu.GpuBuf.upload(vc)
        dq1, dkn1, dvn = gpu.GpuBuf.upload(q), gpu.GpuBuf.upload(k), gpu.GpuBuf.upload(v)
        ds, o1 = gpu.GpuBuf.upload(sinks), gpu.GpuBuf.alloc_f32(nh * hd)
        L.cuda_rope_kv(dq1.ptr, dkn1.ptr, dvn.ptr, dk1.ptr, dv1.ptr, nh, nkv, hd, pos, theta, ys, yc, neox)
        L.cuda_attn_decode(o1.ptr, dq1.ptr, dk1.ptr + 4 * k_start * kv_dim, dv1.ptr + 4 * k_start * kv_dim, nh, nkv, seq, hd,
                           kv_dim, scale, ds.ptr, -1)
        want, want_k, want_v = o1.download(), dk1.download(), dv1.download()
        # one launch
        dk2, dv2 = gpu.GpuBuf.upload(kc), gpu.GpuBuf.upload(vc)
        dq2, dkn2, o2 = gpu.GpuBuf.upload(q), gpu.GpuBuf.upload(k), gpu.GpuBuf.alloc_f32(nh * hd)
        for rep in range(2):
            L.cuda_attn_block(o2.ptr, dq2.ptr, dkn2.ptr, dvn.ptr, dk2.ptr, dv2.ptr, nh, nkv, hd, pos, k_start, scale, ds.ptr,
                              theta, ys, yc, neox, -1)
            got = o2.download()
            assert np.abs(got - want).max() <= 2e-5 * max(np.abs(want).max(), 1e-30), (nh, hd, pos, rep)
        assert np.array_equal(dk2.download(), want_k) and np.array_equal(dv2.download(), want_v)
        assert np.array_equal(dq2.download(), q) and np.array_equal(dkn2.download(), k)
    gpu.check_error()


@pytest.mark.parametrize("neox", [0, 1])
def test_attn_step_matches_separate_launches(gpu, neox):
    """cuda_attn_step (RoPE + KV append + attention + cluster merge in one launch, position from a device word
    or from the argument) against cuda_rope_kv + cuda_attn_decode: same output, same cache rows, q / k_new
    left un-rotated; head groups of 1, 2, 4, 6, 8 and 16 query heads per kv head, sliding windows, sinks,
    positions inside and across the 32-position blocks the CTAs of a cluster share out."""
    import ctypes as C
    L = gpu.lib()
    r = np.random.Generator(np.random.PCG64([0xA79, neox]))
    step_words = gpu.GpuBuf.alloc_f32(4)
    # head_dim 128 and 64 read the (cos, sin) table that cuda_step_set writes with the words; 96 computes it in the kernel
    L.cuda_step_rope_table(step_words.ptr, 128, np.float32(500000.0), np.float32(1.0), 0)
    L.cuda_step_rope_table(step_words.ptr, 64, np.float32(500000.0), np.float32(1.0), 0)
    cases = [(32, 8, 128, 1024, 0, 1100, False), (8, 8, 64, 32, 0, 64, True), (12, 2, 96, 69, 65, 128, True),
             (4, 1, 128, 0, 0, 16, False), (16, 4, 128, 31, 0, 40, False), (64, 8, 128, 600, 0, 640, False),
             (32, 2, 64, 257, 100, 300, True), (8, 4, 128, 2047, 0, 2048, False), (32, 8, 128, 95, 64, 128, False)]
    for ci, (nh, nkv, hd, pos, window, max_seq, sink) in enumerate(cases):
        assert L.cuda_attn_step_supported(nh, nkv, hd) == 1
        kv_dim = nkv * hd
        kc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
        vc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
        q = r.standard_normal(nh * hd, dtype=np.float32)
        k = r.standard_normal(kv_dim, dtype=np.float32)
        v = r.standard_normal(kv_dim, dtype=np.float32)
        sinks = r.standard_normal(nh, dtype=np.float32) if sink else np.full(nh, -np.inf, np.float32)
        scale = np.float32(1.0 / np.sqrt(hd))
        theta, ys, yc = np.float32(500000.0), np.float32(1.0), 0
        k_start = max(0, pos + 1 - window) if window > 0 else 0
        seq = pos - k_start + 1
        dk1, dv1 = gpu.GpuBuf.upload(kc), gpu.GpuBuf.upload(vc)
        dq1, dkn1, dvn = gpu.GpuBuf.upload(q), gpu.GpuBuf.upload(k), gpu.GpuBuf.upload(v)
        ds, o1 = gpu.GpuBuf.upload(sinks), gpu.GpuBuf.alloc_f32(nh * hd)
        L.cuda_rope_kv(dq1.ptr, dkn1.ptr, dvn.ptr, dk1.ptr, dv1.ptr, nh, nkv, hd, pos, theta, ys, yc, neox)
        L.cuda_attn_decode(o1.ptr, dq1.ptr, dk1.ptr + 4 * k_start * kv_dim, dv1.ptr + 4 * k_start * kv_dim, nh, nkv, seq, hd,
                           kv_dim, scale, ds.ptr, -1)
        want, want_k, want_v = o1.download(), dk1.download(), dv1.download()
        dk2, dv2 = gpu.GpuBuf.upload(kc), gpu.GpuBuf.upload(vc)
        dq2, dkn2, o2 = gpu.GpuBuf.upload(q), gpu.GpuBuf.upload(k), gpu.GpuBuf.alloc_f32(nh * hd)
        for rep in range(2):
            if (ci + rep) & 1:      # position from the device step words
                L.cuda_step_set(step_words.ptr, 7, pos)
                L.cuda_attn_step(o2.ptr, dq2.ptr, dkn2.ptr, dvn.ptr, dk2.ptr, dv2.ptr, nh, nkv, hd, max_seq, step_words.ptr, 0,
                                 window, scale, ds.ptr, theta, ys, yc, neox, -1)
            else:
                L.cuda_attn_step(o2.ptr, dq2.ptr, dkn2.ptr, dvn.ptr, dk2.ptr, dv2.ptr, nh, nkv, hd, max_seq, None, pos,
                                 window, scale, ds.ptr, theta, ys, yc, neox, -1)
            got = o2.download()
            assert np.abs(got - want).max() <= 2e-5 * max(np.abs(want).max(), 1e-30), (nh, nkv, hd, pos, rep)
        assert np.array_equal(dk2.download(), want_k) and np.array_equal(dv2.download(), want_v)
        assert np.array_equal(dq2.download(), q) and np.array_equal(dkn2.download(), k)
    # the (cos, sin) table belongs to the position cuda_step_set wrote: when the position word is changed behind its
    # back (a plain copy), the kernel notices that the table is for another position and computes the rotation itself
    nh, nkv, hd, max_seq = 32, 8, 128, 256
    kv_dim = nkv * hd
    kc, vc = r.standard_normal((max_seq, kv_dim), dtype=np.float32), r.standard_normal((max_seq, kv_dim), dtype=np.float32)
    q, k, v = (r.standard_normal(n, dtype=np.float32) for n in (nh * hd, kv_dim, kv_dim))
    theta, scale = np.float32(500000.0), np.float32(1.0 / np.sqrt(hd))
    outs = []
    for stale in (False, True):
        dk, dv, dq, dkn, dvn = (gpu.GpuBuf.upload(a) for a in (kc, vc, q, k, v))
        o = gpu.GpuBuf.alloc_f32(nh * hd)
        L.cuda_step_set(step_words.ptr, 3, 17 if stale else 200)
        if stale:
            words = np.array([3, 200], dtype=np.int32)
            L.cuda_h2d(step_words.ptr, words.ctypes.data, 8)
        L.cuda_attn_step(o.ptr, dq.ptr, dkn.ptr, dvn.ptr, dk.ptr, dv.ptr, nh, nkv, hd, max_seq, step_words.ptr, 0, 0, scale,
                         None, theta, np.float32(1.0), 0, neox, -1)
        outs.append((o.download(), dk.download()[200].copy()))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    # the activation form it leaves for the output projection equals the conversion of its f32 output
    nh, nkv, hd, pos, max_seq = 32, 8, 128, 70, 96
    kv_dim, K, N = nkv * hd, nh * hd, 256
    from saient_quartz_b200 import synth
    kc, vc = r.standard_normal((max_seq, kv_dim), dtype=np.float32), r.standard_normal((max_seq, kv_dim), dtype=np.float32)
    q, k, v = (r.standard_normal(n, dtype=np.float32) for n in (K, kv_dim, kv_dim))
    dk, dv, dq, dkn, dvn = (gpu.GpuBuf.upload(a) for a in (kc, vc, q, k, v))
    o = gpu.GpuBuf.alloc_f32(K)
    w = gpu.GpuBuf.upload(synth.make_weights(12, K, N, tensor_id=690))
    y1, y2 = gpu.GpuBuf.alloc_f32(N), gpu.GpuBuf.alloc_f32(N)
    L.cuda_attn_step(o.ptr, dq.ptr, dkn.ptr, dvn.ptr, dk.ptr, dv.ptr, nh, nkv, hd, max_seq, None, pos, 0,
                     np.float32(0.088), None, np.float32(1e4), np.float32(1.0), 0, neox, 2)
    W, Y, S = (C.c_void_p * 1)(w.ptr), (C.c_void_p * 1)(y1.ptr), (C.c_int * 1)(2)
    L.cuda_gemv_q(12, 1, W, S, Y, K, N, 0)
    L.cuda_gemv(12, w.ptr, o.ptr, y2.ptr, K, N)
    assert np.array_equal(y1.download(), y2.download())
    gpu.check_error()


def test_rope_kv_matches_separate_calls(gpu):
    L = gpu.lib()
    r = np.random.Generator(np.random.PCG64([0xB0B]))
    for (nh, nkv, hd, pos, neox, ys, yo) in [(32, 8, 128, 1024, 0, 1.0, 0), (8, 2, 64, 7, 1, 8.0, 64)]:
        kv_dim = nkv * hd
        q, k, v = (r.standard_normal(n, dtype=np.float32) for n in (nh * hd, kv_dim, kv_dim))
        dq1, dk1, dv1 = gpu.GpuBuf.upload(q), gpu.GpuBuf.upload(k), gpu.GpuBuf.upload(v)
        dq2, dk2 = gpu.GpuBuf.upload(q), gpu.GpuBuf.upload(k)
        kc1, vc1 = gpu.GpuBuf.alloc_f32((pos + 1) * kv_dim), gpu.GpuBuf.alloc_f32((pos + 1) * kv_dim)
        kc2, vc2 = gpu.GpuBuf.alloc_f32((pos + 1) * kv_dim), gpu.GpuBuf.alloc_f32((pos + 1) * kv_dim)
        for b in (kc1, vc1, kc2, vc2):
            L.cuda_vec_zero(b.ptr, (pos + 1) * kv_dim)
        L.cuda_rope_yarn(dq1.ptr, nh, hd, pos, np.float32(5e5), np.float32(ys), yo, neox)
        L.cuda_rope_yarn(dk1.ptr, nkv, hd, pos, np.float32(5e5), np.float32(ys), yo, neox)
        L.cuda_kv_append(kc1.ptr, vc1.ptr, dk1.ptr, dv1.ptr, pos, kv_dim)
        L.cuda_rope_kv(dq2.ptr, dk2.ptr, dv1.ptr, kc2.ptr, vc2.ptr, nh, nkv, hd, pos, np.float32(5e5), np.float32(ys),
                       yo, neox)
        assert np.array_equal(dq1.download(), dq2.download())
        assert np.array_equal(dk1.download(), dk2.download())
        assert np.array_equal(kc1.download(), kc2.download())
        assert np.array_equal(vc1.download(), vc2.download())
    gpu.check_error()


def test_gemv_batch_of_independent_shapes(gpu, oracle_mod):
    """cuda_gemv_batch: GEMVs of different types and shapes that do not depend on one another, in one
    persistent launch, against the oracle and against cuda_gemv (same conversion, same dot products: equal
    bit for bit)."""
    from saient_quartz_b200 import synth
    L = gpu.lib()
    cases = [(12, 4096, 1024), (14, 14336, 512), (8, 2048, 300), (12, 2048, 4096)]
    ops, keep = [], []
    for i, (t, K, N) in enumerate(cases):
        w = synth.make_weights(t, K, N, tensor_id=650 + i)
        x = synth.make_x(K, tensor_id=660 + i).reshape(-1)
        dw = gpu.GpuBuf.upload(w)
        L.cuda_repack_weights(t, dw.ptr, K, N, 1)
        dx, dy, dy2 = gpu.GpuBuf.upload(x), gpu.GpuBuf.alloc_f32(N), gpu.GpuBuf.alloc_f32(N)
        keep.append((t, K, N, w, x, dw, dx, dy, dy2))
        ops.append(gpu.chain_op(t, [dw.ptr], [dy.ptr], K, N, 0, 3, dx.ptr))
    arr = (gpu.ChainOp * len(ops))(*ops)
    assert L.cuda_gemv_chain_supported(len(ops), arr) == 1
    L.cuda_gemv_batch(len(ops), arr)
    for (t, K, N, w, x, dw, dx, dy, dy2) in keep:
        L.cuda_gemv(t, dw.ptr, dx.ptr, dy2.ptr, K, N)
        y, y2 = dy.download(), dy2.download()
        assert np.array_equal(y, y2), (t, K, N)
        ref = oracle_mod.gemv(x, w, t, K, N)
        assert np.all(np.abs(y - ref) <= oracle_mod.tolerance(w, t, K, N, x)), (t, K, N)
    gpu.check_error()
    # long ops whose rows are shared out differently (2 warps per row, then 7, then 2): the consumer warps of a CTA
    # meet between two ops, so a warp that runs ahead never uses the next op's barrier counts beside a slower one
    cases2 = [(14, 4096, 32064), (14, 14336, 4096), (12, 4096, 14336), (8, 4096, 4096), (14, 14336, 1000)]
    ops2, keep2 = [], []
    for i, (t, K, N) in enumerate(cases2):
        w = synth.make_weights(t, K, N, tensor_id=680 + i)
        x = synth.make_x(K, tensor_id=690 + i).reshape(-1)
        dw = gpu.GpuBuf.upload(w)
        L.cuda_repack_weights(t, dw.ptr, K, N, 1)
        dx, dy, dy2 = gpu.GpuBuf.upload(x), gpu.GpuBuf.alloc_f32(N), gpu.GpuBuf.alloc_f32(N)
        keep2.append((t, K, N, dw, dx, dy, dy2))
        ops2.append(gpu.chain_op(t, [dw.ptr], [dy.ptr], K, N, 0, 3, dx.ptr))
    arr2 = (gpu.ChainOp * len(ops2))(*ops2)
    assert L.cuda_gemv_chain_supported(len(ops2), arr2) == 1
    for rep in range(3):
        L.cuda_gemv_batch(len(ops2), arr2)
    L.cuda_sync()
    gpu.check_error("batch of long ops")
    for (t, K, N, dw, dx, dy, dy2) in keep2:
        L.cuda_gemv(t, dw.ptr, dx.ptr, dy2.ptr, K, N)
        assert np.array_equal(dy.download(), dy2.download()), (t, K, N)
    # an op the persistent kernel does not take (in_dim below 2048) makes the call run launch by launch
    t, K, N = 12, 1024, 64
    w = synth.make_weights(t, K, N, tensor_id=670)
    x = synth.make_x(K, tensor_id=671).reshape(-1)
    dw, dx, dy = gpu.GpuBuf.upload(w), gpu.GpuBuf.upload(x), gpu.GpuBuf.alloc_f32(N)
    one = (gpu.ChainOp * 1)(gpu.chain_op(t, [dw.ptr], [dy.ptr], K, N, 0, 3, dx.ptr))
    assert L.cuda_gemv_chain_supported(1, one) == 0
    L.cuda_gemv_batch(1, one)
    assert np.all(np.abs(dy.download() - oracle_mod.gemv(x, w, t, K, N)) <= oracle_mod.tolerance(w, t, K, N, x))
    gpu.check_error()


@pytest.mark.parametrize("nh,nkv,hd,n_tok,pos0,window,sink", [
    (32, 8, 128, 70, 0, 0, False),        # Llama-3 heads, several token tiles, ragged last tile
    (32, 8, 128, 33, 100, 0, True),       # a prompt continuing an existing context, sinks
    (12, 2, 96, 45, 7, 16, True),         # six heads per kv head, head_dim 96, sliding window
    (8, 8, 64, 17, 0, 0, False),          # one head per kv head
    (64, 4, 128, 9, 3, 5, False),         # sixteen heads per kv head, window shorter than the prompt
])
def test_attn_prompt_against_numpy(gpu, nh, nkv, hd, n_tok, pos0, window, sink):
    """cuda_attn_prompt (causal attention of a whole prompt over the caches, token tiles sharing the staged K / V
    rows) against a float64 numpy softmax(q K^T) V per token and head: token t at position pos0 + t sees positions
    [max(0, p + 1 - window), p] (all of [0, p] without a window); sinks add exp(sink) to the denominator
    (src/cuda_kernels.cu:640-672).  Bar: 2e-5 of the largest output."""
    L = gpu.lib()
    r = np.random.Generator(np.random.PCG64([0xA77, nh, nkv, hd, n_tok]))
    max_seq = pos0 + n_tok + 5
    kv_dim, G = nkv * hd, nh // nkv
    kc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
    vc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
    q = r.standard_normal((n_tok, nh * hd), dtype=np.float32)
    sinks = r.standard_normal(nh).astype(np.float32) if sink else None
    scale = np.float32(1.0 / np.sqrt(hd))
    dk, dv, dq = gpu.GpuBuf.upload(kc), gpu.GpuBuf.upload(vc), gpu.GpuBuf.upload(q)
    ds = gpu.GpuBuf.upload(sinks) if sink else None
    out = gpu.GpuBuf.alloc_f32(n_tok * nh * hd)
    L.cuda_attn_prompt(out.ptr, dq.ptr, dk.ptr, dv.ptr, n_tok, nh, nkv, hd, max_seq, pos0, window, scale, ds.ptr if sink else None)
    got = out.download().reshape(n_tok, nh, hd).astype(np.float64)
    gpu.check_error("cuda_attn_prompt")
    want = np.zeros_like(got)
    for t in range(n_tok):
        p = pos0 + t
        lo = max(0, p + 1 - window) if window > 0 else 0
        for h in range(nh):
            kvh = h // G
            K = kc[lo:p + 1, kvh * hd:(kvh + 1) * hd].astype(np.float64)
            V = vc[lo:p + 1, kvh * hd:(kvh + 1) * hd].astype(np.float64)
            s = K @ q[t, h * hd:(h + 1) * hd].astype(np.float64) * float(scale)
            mx = max(s.max(), float(sinks[h])) if sink else s.max()
            e = np.exp(s - mx)
            den = e.sum() + (np.exp(float(sinks[h]) - mx) if sink else 0.0)
            want[t, h] = (e[:, None] * V).sum(axis=0) / den
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max(), np.abs(got - want).max()
