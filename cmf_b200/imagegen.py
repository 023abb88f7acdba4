"""Host-side mirror of the engine's image generation entry (crates/cortiq-engine/src/imagegen.rs
``generate`` :225-297 for a packaged .cmf): prompt token ids -> Gemma-2 caption features ->
flow-matching Euler loop over the NextDiT -> VAE decode -> RGB in [0, 1].  Every stage runs in
libcmf_cuda.so; tokenization is the caller's (the engine's tokenizer is not part of this backend)."""
import time

import numpy as np

from .container import Model
from .dit import GenParams, NextDit, denoise
from .textenc import GemmaEncoder
from .vae import VaeDecoder

_GOLDEN = np.uint64(0x9E3779B97F4A7C15)


def gauss_latent(n, seed):
    """imagegen.rs:75-108: SplitMix64 uniforms (53 bits) through Box-Muller, f64, cast to f32."""
    pairs = (n + 1) // 2
    with np.errstate(over="ignore"):
        idx = np.arange(1, 2 * pairs + 1, dtype=np.uint64)
        z = np.uint64(seed) + idx * _GOLDEN
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        z = z ^ (z >> np.uint64(31))
    u = (z >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    a, b = np.maximum(u[0::2], 1e-300), u[1::2]
    r = np.sqrt(-2.0 * np.log(a))
    ang = 2.0 * np.pi * b
    out = np.empty(2 * pairs, np.float64)
    out[0::2] = r * np.cos(ang)
    out[1::2] = r * np.sin(ang)
    return out[:n].astype(np.float32)


def to_rgb01(img):
    """imagegen.rs:219-223"""
    return np.clip(np.asarray(img, np.float32) / np.float32(2.0) + np.float32(0.5), 0.0, 1.0)


class Pipeline:
    """The three components of a packaged ``lumina2-image`` container, weights resident."""

    def __init__(self, model: Model):
        self.model = model
        self.encoder = GemmaEncoder(model)
        self.dit = NextDit(model)
        self.vae = VaeDecoder(model)

    def close(self):
        for part in (self.encoder, self.dit, self.vae):
            part.close()

    def generate(self, ids, uncond_ids, p: GenParams, stages=None):
        """ids / uncond_ids: prompt tokens (with BOS) of the conditional and the "" prompt.
        Returns RGB [3, height, width] in [0, 1].  ``stages`` (a dict) receives wall seconds."""
        if p.height % 16 or p.width % 16:
            raise ValueError("height/width must be multiples of 16")
        lh, lw = p.height // 8, p.width // 8
        want_uncond = p.guidance_scale > 1.0
        t0 = time.time()
        ids = np.asarray(ids, np.uint32)[: p.max_tokens]
        cap = self.encoder.caption_features(ids)
        cap_u = self.encoder.caption_features(np.asarray(uncond_ids, np.uint32)) if want_uncond else None
        t1 = time.time()
        c = self.dit.in_channels
        lat = gauss_latent(c * lh * lw, p.seed).reshape(1, c, lh, lw)
        lat = denoise(self.dit, lat, cap[None], None if cap_u is None else cap_u[None], p)
        t2 = time.time()
        rgb = to_rgb01(self.vae.decode(lat[0], lh, lw))
        if stages is not None:
            stages.update({"text encode": t1 - t0, "denoise": t2 - t1, "vae decode": time.time() - t2})
        return rgb


def generate(path, ids, uncond_ids, p: GenParams):
    with Model(path) as m:
        pipe = Pipeline(m)
        try:
            return pipe.generate(ids, uncond_ids, p)
        finally:
            pipe.close()
