"""GPU tests of the f32 helper entry points of the decode step (src/cuda.rs:20-54),
against numpy restatements of the reference kernels' formulas
(src/cuda_kernels.cu:545-698, 1194-1265).  f32 tolerance: 1e-5 relative to the
largest magnitude of the result (transcendentals differ in the last ulps)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def _close(got, want, rtol=RTOL):
    scale = max(float(np.abs(want).max()), 1e-30)
    assert np.abs(got.astype(np.float64) - want.astype(np.float64)).max() <= rtol * scale


def _rng(i):
    return np.random.Generator(np.random.PCG64([0xDEC0DE, i]))


def test_vec_ops(gpu):
    L = gpu.lib()
    r = _rng(1)
    for n in (1, 255, 4096, 14336):
        a, b = r.standard_normal(n, dtype=np.float32), r.standard_normal(n, dtype=np.float32)
        da, db = gpu.GpuBuf.upload(a), gpu.GpuBuf.upload(b)
        L.cuda_vec_add(da.ptr, db.ptr, n)
        assert np.array_equal(da.download(), a + b)
        L.cuda_vec_scale_add(da.ptr, db.ptr, np.float32(0.375), n)
        _close(da.download(), (a + b) + np.float32(0.375) * b, 1e-6)
        L.cuda_vec_zero(da.ptr, n)
        assert np.all(da.download() == 0)
    gpu.check_error()


def test_rms_norm(gpu):
    L = gpu.lib()
    r = _rng(2)
    for n in (128, 4096, 8192, 2880):
        x, w = r.standard_normal(n, dtype=np.float32), r.standard_normal(n, dtype=np.float32)
        dx, dw, do = gpu.GpuBuf.upload(x), gpu.GpuBuf.upload(w), gpu.GpuBuf.alloc_f32(n)
        L.cuda_rms_norm(do.ptr, dx.ptr, dw.ptr, n)
        want = x * (1.0 / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-5)) * w
        _close(do.download(), want)
        L.cuda_rms_norm(dx.ptr, dx.ptr, dw.ptr, n)   # in place, as the QK-norm call sites do
        _close(dx.download(), want)
    gpu.check_error()


def _rope_ref(x, n_heads, hd, pos, theta, ys, yctx, neox):
    x = x.astype(np.float64).reshape(n_heads, hd).copy()
    half = hd // 2
    i = np.arange(half)
    inv = 1.0 / np.power(np.float64(theta), 2.0 * i / hd)
    eff = inv.copy()
    if ys > 1.0 and yctx > 0:
        hi_w, lo_w = yctx / 32.0, yctx / 1.0
        wavelen = 2 * np.pi / inv
        ramp = np.clip((lo_w - wavelen) / (lo_w - hi_w), 0, 1)
        eff = ramp * inv + (1 - ramp) * (inv / ys)
    ang = pos * eff
    s, c = np.sin(ang), np.cos(ang)
    i0, i1 = (i, i + half) if neox else (2 * i, 2 * i + 1)
    a, b = x[:, i0].copy(), x[:, i1].copy()
    x[:, i0] = a * c - b * s
    x[:, i1] = a * s + b * c
    return x.reshape(-1)


def test_rope_yarn(gpu):
    L = gpu.lib()
    r = _rng(3)
    for (nh, hd, pos, theta, ys, yctx, neox) in [(32, 128, 1024, 500000.0, 1.0, 0, 0), (8, 128, 77, 500000.0, 1.0, 0, 0),
                                                  (64, 64, 300, 150000.0, 32.0, 4096, 1), (4, 96, 5, 10000.0, 1.0, 0, 1)]:
        x = r.standard_normal(nh * hd, dtype=np.float32)
        dx = gpu.GpuBuf.upload(x)
        L.cuda_rope_yarn(dx.ptr, nh, hd, pos, theta, ys, yctx, neox)
        # angles reach ~1e3 rad in f32: compare at f32-angle precision
        _close(dx.download(), _rope_ref(x, nh, hd, pos, np.float32(theta), ys, yctx, neox), 2e-4)
    gpu.check_error()


def test_kv_append_and_attention(gpu):
    """kv_append + score_all + softmax_sink_all + values_all = softmax(q K^T * scale) V with GQA."""
    L = gpu.lib()
    r = _rng(4)
    for (nh, nkv, hd, seq, max_seq, sink) in [(32, 8, 128, 1025, 2048, False), (8, 8, 64, 33, 64, True),
                                              (4, 1, 128, 1, 16, False)]:
        kv_dim = nkv * hd
        kc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
        vc = r.standard_normal((max_seq, kv_dim), dtype=np.float32)
        q = r.standard_normal(nh * hd, dtype=np.float32)
        k_new, v_new = r.standard_normal(kv_dim, dtype=np.float32), r.standard_normal(kv_dim, dtype=np.float32)
        dk, dv = gpu.GpuBuf.upload(kc), gpu.GpuBuf.upload(vc)
        dq, dkn, dvn = gpu.GpuBuf.upload(q), gpu.GpuBuf.upload(k_new), gpu.GpuBuf.upload(v_new)
        pos = seq - 1
        L.cuda_kv_append(dk.ptr, dv.ptr, dkn.ptr, dvn.ptr, pos, kv_dim)
        kc[pos], vc[pos] = k_new, v_new
        assert np.array_equal(dk.download().reshape(max_seq, kv_dim)[pos], k_new)
        sinks = (r.standard_normal(nh, dtype=np.float32) if sink else np.full(nh, -np.inf, np.float32))
        ds = gpu.GpuBuf.upload(sinks)
        dsc, dout = gpu.GpuBuf.alloc_f32(nh * max_seq), gpu.GpuBuf.alloc_f32(nh * hd)
        scale = np.float32(1.0 / np.sqrt(hd))
        L.cuda_attn_score_all(dsc.ptr, dq.ptr, dk.ptr, nh, nkv, seq, hd, kv_dim, max_seq, scale)
        L.cuda_softmax_sink_all(dsc.ptr, nh, seq, max_seq, ds.ptr)
        L.cuda_attn_values_all(dout.ptr, dsc.ptr, dv.ptr, nh, nkv, seq, hd, kv_dim, max_seq)
        want = np.zeros((nh, hd))
        for h in range(nh):
            g = (h * nkv) // nh
            K_ = kc[:seq, g * hd:(g + 1) * hd].astype(np.float64)
            V_ = vc[:seq, g * hd:(g + 1) * hd].astype(np.float64)
            s = K_ @ q[h * hd:(h + 1) * hd].astype(np.float64) * scale
            mx = max(s.max(), sinks[h]) if sink else s.max()
            e = np.exp(s - mx)
            tot = e.sum() + (np.exp(sinks[h] - mx) if sink else 0.0)
            want[h] = (e / tot) @ V_
        _close(dout.download(), want.reshape(-1), 2e-5)
    gpu.check_error()


def test_per_head_attention_entry_points(gpu):
    """cuda_attn_score / cuda_softmax_sink / cuda_attn_values (declared at src/cuda.rs:28-33)."""
    L = gpu.lib()
    r = _rng(5)
    hd, kv_dim, seq, off = 64, 256, 50, 128
    kc = r.standard_normal((seq, kv_dim), dtype=np.float32)
    q = r.standard_normal(hd, dtype=np.float32)
    dk, dq = gpu.GpuBuf.upload(kc), gpu.GpuBuf.upload(q)
    dsc, dout = gpu.GpuBuf.alloc_f32(seq), gpu.GpuBuf.alloc_f32(hd)
    L.cuda_attn_score(dsc.ptr, dq.ptr, dk.ptr, seq, hd, kv_dim, off, np.float32(0.125))
    s = (kc[:, off:off + hd].astype(np.float64) @ q.astype(np.float64)) * 0.125
    _close(dsc.download(), s)
    L.cuda_softmax_sink(dsc.ptr, seq, np.float32(0.5))
    mx = max(s.max(), 0.5)
    e = np.exp(s - mx)
    p = e / (e.sum() + np.exp(0.5 - mx))
    _close(dsc.download(), p)
    L.cuda_attn_values(dout.ptr, dsc.ptr, dk.ptr, seq, hd, kv_dim, off)
    _close(dout.download(), p @ kc[:, off:off + hd].astype(np.float64), 2e-5)
    gpu.check_error()


def test_swiglu_variants(gpu):
    L = gpu.lib()
    r = _rng(6)
    n = 14336
    g, u = 4 * r.standard_normal(n, dtype=np.float32), 4 * r.standard_normal(n, dtype=np.float32)
    dg, du, do = gpu.GpuBuf.upload(g), gpu.GpuBuf.upload(u), gpu.GpuBuf.alloc_f32(n)
    L.cuda_swiglu(do.ptr, dg.ptr, du.ptr, n)
    g64, u64 = g.astype(np.float64), u.astype(np.float64)
    _close(do.download(), g64 / (1 + np.exp(-g64)) * u64)
    L.cuda_swiglu_oai(do.ptr, dg.ptr, du.ptr, n)
    x = np.minimum(g64, 7.0)
    y = np.clip(u64, -7.0, 7.0)
    _close(do.download(), x / (1 + np.exp(-1.702 * x)) * (y + 1))
    gpu.check_error()
