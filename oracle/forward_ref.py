"""CPU oracle of the per-token forward pass -- TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference's CPU path (src/main.rs: rms_norm :683-686, rope_yarn
:721-759, attention :788-919, ffn_lazy :923-937, moe_ffn :952-1039, embed_and_layers :1045-1105,
forward :1107-1120) in f32, with every matrix-vector product done by the C oracle's gemv().
The tests feed it the same host tensors that were uploaded to the GPU model.
"""
import numpy as np

from . import dequant, gemv

f32 = np.float32


def rms_norm(x, w, eps):
    rms = np.sqrt(f32(np.sum(x * x, dtype=f32) / f32(x.size) + f32(eps)))
    return (x / rms * w).astype(f32)


def rope_yarn(x, pos, dim, theta, yarn_scale, yarn_orig_ctx, neox):
    half = dim // 2
    i = np.arange(half, dtype=f32)
    std_inv = (f32(1.0) / np.power(f32(theta), f32(2.0) * i / f32(dim))).astype(f32)
    if yarn_scale <= 1.0 or yarn_orig_ctx == 0:
        eff = std_inv
    else:
        hfw, lfw = f32(yarn_orig_ctx) / f32(32.0), f32(yarn_orig_ctx) / f32(1.0)
        wavelen = f32(2.0 * np.pi) / std_inv
        ramp = np.clip((lfw - wavelen) / (lfw - hfw), 0.0, 1.0).astype(f32)
        eff = (ramp * std_inv + (f32(1.0) - ramp) * (std_inv / f32(yarn_scale))).astype(f32)
    ang = (f32(pos) * eff).astype(f32)
    s, c = np.sin(ang).astype(f32), np.cos(ang).astype(f32)
    idx = np.arange(half)
    i0, i1 = (idx, idx + half) if neox else (2 * idx, 2 * idx + 1)
    x0, x1 = x[i0].copy(), x[i1].copy()
    x[i0] = x0 * c - x1 * s
    x[i1] = x0 * s + x1 * c


def silu(x):
    return (x / (f32(1.0) + np.exp(-x))).astype(f32)


def swiglu_oai(g, u):
    x = np.minimum(g, f32(7.0))
    y = np.clip(u, f32(-7.0), f32(7.0))
    return ((x / (f32(1.0) + np.exp(f32(-1.702) * x))) * (y + f32(1.0))).astype(f32)


class RefModel:
    """Host tensors: dict (role, layer) -> (ggml_type, ndarray), as HostModel(keep_host=True).host."""

    def __init__(self, cfg, tensors, norm_eps=1e-5):
        self.c = dict(cfg)
        self.t = tensors
        self.eps = norm_eps
        kv_d = cfg["n_kv_heads"] * cfg["head_dim"]
        self.kv = [(np.zeros((0, kv_d), f32), np.zeros((0, kv_d), f32)) for _ in range(cfg["n_layers"])]

    def set_kv(self, layer, k, v):
        self.kv[layer] = (k.astype(f32).copy(), v.astype(f32).copy())

    def _mv(self, role, layer, x, K, N, expert=None):
        t, a = self.t[(role, layer)]
        a = a.view(np.uint8).reshape(-1)
        if expert is not None:
            per = a.size // self.c["n_experts"]
            a = a[expert * per:(expert + 1) * per]
        return gemv(x, a, t, K, N)

    def _opt(self, role, layer):
        v = self.t.get((role, layer))
        return None if v is None else v[1].astype(f32)

    def attention(self, l, x, pos):
        c = self.c
        d, h, kvh, hd = c["embed_dim"], c["n_heads"], c["n_kv_heads"], c["head_dim"]
        q_d, kv_d = h * hd, kvh * hd
        q, k, v = self._mv("Q", l, x, d, q_d), self._mv("K", l, x, d, kv_d), self._mv("V", l, x, d, kv_d)
        for role, vec in (("Q_BIAS", q), ("K_BIAS", k), ("V_BIAS", v)):
            b = self._opt(role, l)
            if b is not None:
                vec += b
        for role, vec, nh in (("Q_NORM", q, h), ("K_NORM", k, kvh)):
            w = self._opt(role, l)
            if w is not None:
                if w.size == hd:
                    for hh in range(nh):
                        vec[hh * hd:(hh + 1) * hd] = rms_norm(vec[hh * hd:(hh + 1) * hd], w, self.eps)
                else:
                    vec[:] = rms_norm(vec, w, self.eps)
        ys, yo = c.get("yarn_scale", 1.0), c.get("yarn_orig_ctx", 0)
        for hh in range(h):
            rope_yarn(q[hh * hd:(hh + 1) * hd], pos, hd, c["rope_theta"], ys, yo, c.get("rope_neox", 0))
        for hh in range(kvh):
            rope_yarn(k[hh * hd:(hh + 1) * hd], pos, hd, c["rope_theta"], ys, yo, c.get("rope_neox", 0))
        K_, V_ = self.kv[l]
        K_ = np.concatenate([K_[:pos], k[None, :]], 0)
        V_ = np.concatenate([V_[:pos], v[None, :]], 0)
        self.kv[l] = (K_, V_)
        seq = pos + 1
        mscale2 = f32(1.0)
        if ys > 1.0 and yo > 0:
            ms = f32(1.0) + f32(0.1) * f32(np.log(f32(ys)))
            mscale2 = ms * ms
        scale = f32(1.0) / np.sqrt(f32(hd)) * mscale2
        sw = c.get("swa_window", 0)
        k_start = max(0, pos + 1 - sw) if (sw > 0 and l % 2 == 0) else 0
        sinks = self._opt("SINKS", l)
        out = np.zeros(q_d, f32)
        for hh in range(h):
            g = (hh * kvh) // h
            qh = q[hh * hd:(hh + 1) * hd]
            sc = (K_[k_start:seq, g * hd:(g + 1) * hd] @ qh).astype(f32) * scale
            sink = sinks[hh] if sinks is not None and sinks.size > hh else f32(-np.inf)
            mx = max(sc.max(), sink)
            e = np.exp(sc - mx).astype(f32)
            tot = e.sum(dtype=f32) + (np.exp(sink - mx) if sink > -np.inf else f32(0.0))
            p = (e / tot).astype(f32)
            out[hh * hd:(hh + 1) * hd] = (p @ V_[k_start:seq, g * hd:(g + 1) * hd]).astype(f32)
        a = self._mv("O", l, out, q_d, d)
        ob = self._opt("O_BIAS", l)
        if ob is not None:
            a += ob
        return a

    def ffn(self, l, x):
        c = self.c
        d, fd = c["embed_dim"], c["ffn_dim"]
        g, u = self._mv("GATE", l, x, d, fd), self._mv("UP", l, x, d, fd)
        return self._mv("DOWN", l, (silu(g) * u).astype(f32), fd, d)

    def moe_ffn(self, l, x):
        c = self.c
        d, fd, ne, k = c["embed_dim"], c["ffn_dim"], c["n_experts"], c["n_experts_used"]
        rw_ = self.t[("ROUTER_W", l)][1].astype(f32).reshape(ne, d)
        logits = np.array([np.sum(x * rw_[j], dtype=f32) for j in range(ne)], f32)
        rb = self._opt("ROUTER_B", l)
        if rb is not None:
            logits += rb
        order = np.argsort(-logits, kind="stable")[:k]
        if c.get("moe_renorm", 1):
            mx = logits[order].max()
            e = np.exp(logits[order] - mx).astype(f32)
            den = e.sum(dtype=f32)
        else:
            mx = logits.max()
            den = np.exp(logits - mx).astype(f32).sum(dtype=f32)
            e = np.exp(logits[order] - mx).astype(f32)
        out = np.zeros(d, f32)
        for i, eid in enumerate(order):
            eid = int(eid)
            g = self._mv("MOE_GATE", l, x, d, fd, eid)
            u = self._mv("MOE_UP", l, x, d, fd, eid)
            gb, ub, db = self._opt("MOE_GATE_BIAS", l), self._opt("MOE_UP_BIAS", l), self._opt("MOE_DOWN_BIAS", l)
            if gb is not None:
                g += gb[eid * fd:(eid + 1) * fd]
            if ub is not None:
                u += ub[eid * fd:(eid + 1) * fd]
            hcur = swiglu_oai(g, u) if c.get("clamped_swiglu", 0) else (silu(g) * u).astype(f32)
            o = self._mv("MOE_DOWN", l, hcur, fd, d, eid)
            if db is not None:
                o += db[eid * d:(eid + 1) * d]
            out += (e[i] / den) * o
        return out

    def forward(self, token, pos, return_hidden=False):
        c = self.c
        d = c["embed_dim"]
        t, emb = self.t[("EMBED", 0)]
        emb = emb.view(np.uint8).reshape(c["vocab_size"], -1)
        x = dequant(emb[token], t, d)
        for l in range(c["n_layers"]):
            n1 = rms_norm(x, self.t[("ATTN_NORM", l)][1].astype(f32), self.eps)
            x = (x + self.attention(l, n1, pos)).astype(f32)
            n2 = rms_norm(x, self.t[("FFN_NORM", l)][1].astype(f32), self.eps)
            f = self.moe_ffn(l, n2) if c.get("n_experts", 0) > 0 else self.ffn(l, n2)
            x = (x + f).astype(f32)
        if return_hidden:
            return x
        xn = rms_norm(x, self.t[("FINAL_NORM", 0)][1].astype(f32), self.eps)
        return self._mv("LM_HEAD", 0, xn, d, c["vocab_size"])
