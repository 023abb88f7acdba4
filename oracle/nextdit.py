"""CPU oracle for the NextDiT denoiser forward and the Euler flow-matching loop.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg
of the benchmark; never by the shipped package.

A numpy restatement of the reference's strict CPU path.  Each function cites the reference
source it follows (paths relative to the reference repository root).  Norm statistics and
RoPE run in float64 exactly where the reference's do; linears run either through the strict
scalar kernels of oracle/cmf_oracle.c (``exact=True``) or as an f32 matmul over the exactly
dequantized weights (same products, BLAS summation order; differs by f32 rounding only).

Parity status: pinned against the reference's own numpy forward (python/nextdit_ref.py,
imported in the build container) through tests/golden/nextdit_ref_*.npz.
"""
import math

import numpy as np

from . import codecs


class QWeight:
    """A quantized projection as stored in the container: dtype id, shape, payload bytes."""

    def __init__(self, dtype, rows, cols, payload, cache=True):
        self.dtype, self.rows, self.cols = dtype, rows, cols
        self.cache = cache
        self.payload = np.ascontiguousarray(np.frombuffer(bytes(payload), np.uint8)) \
            if not isinstance(payload, np.ndarray) else payload
        self._dense = None

    @classmethod
    def quantize(cls, dtype, w):
        w = np.ascontiguousarray(w, np.float32)
        return cls(dtype, w.shape[0], w.shape[1], codecs.encode(dtype, w))

    def dense(self):
        if self._dense is not None:
            return self._dense
        d = codecs.dequant(self.dtype, self.payload, self.rows, self.cols)
        if self.cache:
            self._dense = d
        return d


def matmat(w, x, exact=False):
    """Proj::matmat / QTensor::matmat, strict arm: Y[b, rows] = X . W^T
    (crates/cortiq-engine/src/qtensor.rs:1441, exact kernels :3533-3546, :4418-4432, :4647-4661)."""
    x = np.ascontiguousarray(x, np.float32)
    if isinstance(w, QWeight):
        if exact:
            return codecs.matmat_exact(w.dtype, w.payload, w.rows, w.cols, x)
        return x @ w.dense().T
    w = np.asarray(w, np.float32)
    if exact:
        return codecs.gemm_nt(x, w)
    return x @ w.T


def silu(v):
    """crates/cortiq-engine/src/dit.rs:290-292"""
    v = np.asarray(v, np.float32)
    return (v / (np.float32(1.0) + np.exp(-v))).astype(np.float32)


def rms_norm(x, w, eps):
    """crates/cortiq-engine/src/dit.rs:259-275: f64 mean of squares, scale in f64, round to
    f32, then multiply by the f32 weight."""
    x = np.asarray(x, np.float32)
    ss = (x.astype(np.float64) ** 2).sum(-1, keepdims=True) / x.shape[-1]
    inv = 1.0 / np.sqrt(ss + eps)
    return (x.astype(np.float64) * inv).astype(np.float32) * np.asarray(w, np.float32)


def rope_table(ids, axes_dim):
    """crates/cortiq-engine/src/dit.rs:366-381 -> (cos, sin) float64 [n, sum(axes)/2]."""
    ids = np.asarray(ids, np.int64).reshape(-1, 3)
    cols = []
    for a, d in enumerate(axes_dim):
        j = np.arange(d // 2, dtype=np.float64)
        freq = 1.0 / np.power(10000.0, 2.0 * j / d)
        cols.append(ids[:, a:a + 1].astype(np.float64) * freq[None, :])
    ang = np.concatenate(cols, 1)
    return np.cos(ang), np.sin(ang)


def qk_norm_rope(v, heads, hd, w, cos, sin):
    """crates/cortiq-engine/src/dit.rs:1078-1102: per (token, head) RMS norm with eps 1e-5, then
    interleaved-pair rotation in f64."""
    n = v.shape[0]
    v = rms_norm(v.reshape(n, heads, hd), w, 1e-5)
    a = v[..., 0::2].astype(np.float64)
    b = v[..., 1::2].astype(np.float64)
    c, s = cos[:, None, :], sin[:, None, :]
    out = np.empty_like(v)
    out[..., 0::2] = (a * c - b * s).astype(np.float32)
    out[..., 1::2] = (a * s + b * c).astype(np.float32)
    return out.reshape(n, heads * hd)


def attention_seq(q, k, v, nh, nkv, hd):
    """crates/cortiq-engine/src/dit.rs:846-922: per head S = (q/sqrt(hd)) k^T, max-subtracted
    f32 softmax (dit.rs:331-351), O = P v; GQA maps head h to kv head h // (nh // nkv)."""
    n = q.shape[0]
    scale = np.float32(1.0 / math.sqrt(hd))
    q = q.reshape(n, nh, hd)
    k = k.reshape(n, nkv, hd)
    v = v.reshape(n, nkv, hd)
    out = np.empty((n, nh, hd), np.float32)
    hpk = nh // nkv
    for h in range(nh):
        kv = h // hpk
        s = (q[:, h] * scale) @ k[:, kv].T
        s = np.exp(s - s.max(-1, keepdims=True))
        den = s.sum(-1, keepdims=True, dtype=np.float32)
        p = s * (np.float32(1.0) / den)
        out[:, h] = p @ v[:, kv]
    return out.reshape(n, nh * hd)


class NextDitOracle:
    """The denoiser over a dict of ``dit.*`` tensors (names as in
    crates/cortiq-engine/src/dit.rs:510-589): f32 arrays or QWeight."""

    def __init__(self, tensors, cfg, exact=False):
        self.t = tensors
        self.exact = exact
        self.hs = int(cfg["hidden_size"])
        self.nh = int(cfg["num_attention_heads"])
        self.nkv = int(cfg.get("num_kv_heads", self.nh))
        self.hd = self.hs // self.nh
        self.c = int(cfg["in_channels"])
        self.p = int(cfg.get("patch_size", 2))
        self.axes = [int(a) for a in cfg["axes_dim_rope"]]
        self.eps = float(cfg.get("norm_eps", 1e-5))
        self.nl = int(cfg["num_layers"])
        self.nr = int(cfg.get("num_refiner_layers", 2))
        self.block_taps = None  # list to collect per-block outputs when set

    def _mm(self, name, x):
        return matmat(self.t[name], x, self.exact)

    def time_embed(self, t):
        """crates/cortiq-engine/src/dit.rs:592-605"""
        half = 128
        i = np.arange(half, dtype=np.float64)
        ang = float(np.float32(t)) * np.exp(-math.log(10000.0) * i / half)
        f = np.concatenate([np.cos(ang), np.sin(ang)]).astype(np.float32)[None, :]
        pre = "dit.time_caption_embed.timestep_embedder."
        h = matmat(self.t[pre + "linear_1.weight"], f, True)[0] + self.t[pre + "linear_1.bias"]
        h = silu(h)[None, :]
        return matmat(self.t[pre + "linear_2.weight"], h, True)[0] + self.t[pre + "linear_2.bias"]

    def modulation(self, pfx, temb):
        """crates/cortiq-engine/src/dit.rs:956-967, :980-993 -> s_msa, tanh(g_msa), s_mlp, tanh(g_mlp)"""
        m = self._mm(pfx + ".norm1.linear.weight", silu(temb)[None, :])[0] + self.t[pfx + ".norm1.linear.bias"]
        hs = self.hs
        return m[:hs], np.tanh(m[hs:2 * hs]), m[2 * hs:3 * hs], np.tanh(m[3 * hs:])

    def block_forward_seg(self, pfx, x, rope, temb, segs):
        """crates/cortiq-engine/src/dit.rs:943-1177 (host arm)."""
        t, hs, nh, nkv, hd = self.t, self.hs, self.nh, self.nkv, self.hd
        cos, sin = rope
        if temb is not None:
            s_msa, g_msa, s_mlp, g_mlp = self.modulation(pfx, temb)
            n1 = t[pfx + ".norm1.norm.weight"]
        else:
            s_msa = g_msa = s_mlp = g_mlp = None
            n1 = t[pfx + ".norm1.weight"]
        xn = rms_norm(x, n1, self.eps)
        if s_msa is not None:
            xn = xn * (np.float32(1.0) + s_msa)
        q = self._mm(pfx + ".attn.to_q.weight", xn)
        k = self._mm(pfx + ".attn.to_k.weight", xn)
        v = self._mm(pfx + ".attn.to_v.weight", xn)
        q = qk_norm_rope(q, nh, hd, t[pfx + ".attn.norm_q.weight"], cos, sin)
        k = qk_norm_rope(k, nkv, hd, t[pfx + ".attn.norm_k.weight"], cos, sin)
        attn = np.empty((x.shape[0], nh * hd), np.float32)
        off = 0
        for ns in segs:
            sl = slice(off, off + ns)
            attn[sl] = attention_seq(q[sl], k[sl], v[sl], nh, nkv, hd)
            off += ns
        proj = self._mm(pfx + ".attn.to_out.0.weight", attn)
        r = rms_norm(proj, t[pfx + ".norm2.weight"], self.eps)
        x = x + (g_msa * r if g_msa is not None else r)
        y = rms_norm(x, t[pfx + ".ffn_norm1.weight"], self.eps)
        if s_mlp is not None:
            y = y * (np.float32(1.0) + s_mlp)
        g = self._mm(pfx + ".feed_forward.linear_1.weight", y)
        u = self._mm(pfx + ".feed_forward.linear_3.weight", y)
        d = self._mm(pfx + ".feed_forward.linear_2.weight", silu(g) * u)
        r = rms_norm(d, t[pfx + ".ffn_norm2.weight"], self.eps)
        x = (x + (g_mlp * r if g_mlp is not None else r)).astype(np.float32)
        if self.block_taps is not None:
            self.block_taps.append((pfx, x.copy()))
        return x

    def refine_caption(self, cap):
        """crates/cortiq-engine/src/dit.rs:1201-1226"""
        cap = np.asarray(cap, np.float32)
        pre = "dit.time_caption_embed.caption_embedder."
        e = self._mm(pre + "1.weight", rms_norm(cap, self.t[pre + "0.weight"], self.eps)) + self.t[pre + "1.bias"]
        n = cap.shape[0]
        ids = np.stack([np.arange(n), np.zeros(n, np.int64), np.zeros(n, np.int64)], 1)
        rope = rope_table(ids, self.axes)
        for l in range(self.nr):
            e = self.block_forward_seg(f"dit.context_refiner.{l}", e, rope, None, [n])
        return e

    def patchify(self, latent, h, w):
        """crates/cortiq-engine/src/dit.rs:1255-1268: (dy, dx, ch) inner order."""
        c, p = self.c, self.p
        hp, wp = h // p, w // p
        return latent.reshape(c, hp, p, wp, p).transpose(1, 3, 2, 4, 0).reshape(hp * wp, p * p * c)

    def unpatchify(self, tok, h, w):
        """crates/cortiq-engine/src/dit.rs:1369-1386"""
        c, p = self.c, self.p
        hp, wp = h // p, w // p
        return np.ascontiguousarray(tok.reshape(hp, wp, p, p, c).transpose(4, 0, 2, 1, 3).reshape(c, h, w))

    def _img_ids(self, a0, h, w):
        wp = w // self.p
        n = (h // self.p) * wp
        i = np.arange(n)
        return np.stack([np.full(n, a0), i // wp, i % wp], 1)

    def _head(self, latent, h, w, temb, refiner_axis0):
        tok = self.patchify(np.asarray(latent, np.float32).reshape(self.c, h, w), h, w)
        img = matmat(self.t["dit.x_embedder.weight"], tok, self.exact) + self.t["dit.x_embedder.bias"]
        n_img = img.shape[0]
        rope_r = rope_table(self._img_ids(refiner_axis0, h, w), self.axes)
        for l in range(self.nr):
            img = self.block_forward_seg(f"dit.noise_refiner.{l}", img, rope_r, temb, [n_img])
        return img

    def _tail(self, x, temb):
        """norm_out (crates/cortiq-engine/src/dit.rs:1346-1368): LayerNorm eps 1e-6 without
        affine, times (1 + scale), then linear_2 + bias."""
        scale = matmat(self.t["dit.norm_out.linear_1.weight"], silu(temb)[None, :], True)[0] \
            + self.t["dit.norm_out.linear_1.bias"]
        x64 = x.astype(np.float64)
        mean = x64.sum(-1, keepdims=True) / self.hs
        var = ((x64 - mean) ** 2).sum(-1, keepdims=True) / self.hs
        xn = ((x64 - mean) * (1.0 / np.sqrt(var + 1e-6))).astype(np.float32) * (np.float32(1.0) + scale)
        return matmat(self.t["dit.norm_out.linear_2.weight"], xn, self.exact) + self.t["dit.norm_out.linear_2.bias"]

    def forward_with_cap(self, latent, h, w, cap_e, t):
        """crates/cortiq-engine/src/dit.rs:1389-1507 (single sequence; refiner image ids carry
        axis-0 = cap_n)."""
        temb = self.time_embed(t)
        cap_n = cap_e.shape[0]
        img = self._head(latent, h, w, temb, cap_n)
        ids = np.concatenate([np.stack([np.arange(cap_n), np.zeros(cap_n, np.int64), np.zeros(cap_n, np.int64)], 1),
                              self._img_ids(cap_n, h, w)], 0)
        rope = rope_table(ids, self.axes)
        x = np.concatenate([cap_e, img], 0).astype(np.float32)
        for l in range(self.nl):
            x = self.block_forward_seg(f"dit.layers.{l}", x, rope, temb, [x.shape[0]])
        out = self._tail(x, temb)
        return self.unpatchify(out[cap_n:], h, w)

    def forward_cfg_pair(self, latent, h, w, cap_c, cap_u, t):
        """crates/cortiq-engine/src/dit.rs:1238-1387: [cap_c | img | cap_u | img] as two segments;
        patchify and the noise refiners run once (refiner image ids use axis-0 = 0)."""
        temb = self.time_embed(t)
        img = self._head(latent, h, w, temb, 0)
        n_img = img.shape[0]

        def ids_for(cap_n):
            return np.concatenate([np.stack([np.arange(cap_n), np.zeros(cap_n, np.int64), np.zeros(cap_n, np.int64)], 1),
                                   self._img_ids(cap_n, h, w)], 0)
        nc, nu = cap_c.shape[0], cap_u.shape[0]
        rope = rope_table(np.concatenate([ids_for(nc), ids_for(nu)], 0), self.axes)
        x = np.concatenate([cap_c, img, cap_u, img], 0).astype(np.float32)
        segs = [nc + n_img, nu + n_img]
        for l in range(self.nl):
            x = self.block_forward_seg(f"dit.layers.{l}", x, rope, temb, segs)
        out = self._tail(x, temb)
        return self.unpatchify(out[nc:nc + n_img], h, w), self.unpatchify(out[segs[0] + nu:], h, w)


# ---- the loop around the forward (crates/cortiq-engine/src/imagegen.rs) ----

def sigmas(steps, shift=6.0):
    """crates/cortiq-engine/src/imagegen.rs:59-73"""
    out = []
    for i in range(steps):
        s = 1.0 if steps == 1 else 1.0 - i * (1.0 - 1.0 / steps) / (steps - 1)
        out.append(shift * s / (1.0 + (shift - 1.0) * s))
    out.append(0.0)
    return out


def gauss_latent(n, seed):
    """crates/cortiq-engine/src/imagegen.rs:75-108: SplitMix64 (sampler.rs:70-77) uniforms through
    Box-Muller."""
    mask = (1 << 64) - 1
    state = seed & mask

    def u():
        nonlocal state
        state = (state + 0x9E3779B97F4A7C15) & mask
        z = state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
        z ^= z >> 31
        return (z >> 11) / float(1 << 53)
    out = []
    while len(out) < n:
        a, b = max(u(), 1e-300), u()
        r = math.sqrt(-2.0 * math.log(a))
        ang = 2.0 * math.pi * b
        out.append(r * math.cos(ang))
        if len(out) < n:
            out.append(r * math.sin(ang))
    return np.asarray(out, np.float64).astype(np.float32)


def cfg_combine(cond, uncond, gs, lw, normalize=True):
    """crates/cortiq-engine/src/imagegen.rs:186-205: u + gs (c - u), then per row of width lw the
    f32 norm ratio ||c|| / ||comb||."""
    cond = np.asarray(cond, np.float32)
    uncond = np.asarray(uncond, np.float32)
    comb = (uncond + np.float32(gs) * (cond - uncond)).astype(np.float32)
    if normalize:
        c2, g2 = cond.reshape(-1, lw), comb.reshape(-1, lw)
        cn = np.sqrt((c2 * c2).sum(-1, dtype=np.float32))
        gn = np.sqrt((g2 * g2).sum(-1, dtype=np.float32))
        f = np.where(gn > 0, cn / np.where(gn > 0, gn, 1), np.float32(1.0)).astype(np.float32)
        comb = (g2 * f[:, None]).reshape(cond.shape)
    return comb


def denoise(model, latents, h, w, cap, cap_u, steps=30, gs=4.0, on_step=None, cfg_trunc_ratio=1.0,
            cfg_normalization=True):
    """crates/cortiq-engine/src/imagegen.rs:143-217.  ``cap`` / ``cap_u`` are raw caption
    features; refined once.  Step i is guided while (i + 1) / steps <= cfg_trunc_ratio in f32
    (:164); past it only the cond branch runs, through the single-sequence forward."""
    x = np.asarray(latents, np.float32).copy()
    sg = sigmas(steps)
    cap_r = model.refine_caption(cap)
    cap_u_r = model.refine_caption(cap_u) if cap_u is not None else None
    for i in range(steps):
        t = np.float32(1.0 - sg[i])
        cfg_on = cap_u_r is not None and np.float32(i + 1) / np.float32(steps) <= np.float32(cfg_trunc_ratio)
        if cfg_on:
            pc, pu = model.forward_cfg_pair(x, h, w, cap_r, cap_u_r, t)
            pred = cfg_combine(pc, pu, gs, w, normalize=cfg_normalization)
        else:
            pred = model.forward_with_cap(x, h, w, cap_r, t)
        d = np.float32(sg[i + 1] - sg[i])
        x = (x.reshape(-1) - d * pred.reshape(-1)).astype(np.float32).reshape(x.shape)
        if on_step:
            on_step(i, x)
    return x
