"""Host-side mirror of the engine's NextDiT object and denoise loop
(crates/cortiq-engine/src/dit.rs ``NextDit``; crates/cortiq-engine/src/imagegen.rs ``denoise``),
driving the device-resident implementation in libcmf_cuda.so."""
import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import check, lib
from .container import Model


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


@dataclass
class GenParams:
    """imagegen.rs:24-55 (the fields this backend uses), with the engine's defaults."""
    steps: int = 30
    guidance_scale: float = 4.0
    cfg_trunc_ratio: float = 1.0     # fraction of steps that run with CFG; past it only cond runs
    cfg_normalization: bool = True   # rescale the guided prediction to the cond-branch norm per row
    seed: int = 42
    height: int = 512
    width: int = 512
    max_tokens: int = 256


class _CGenParams(C.Structure):
    """``cmfc_gen_params`` of include/cmf_cuda.h."""
    _fields_ = [("steps", C.c_uint32), ("guidance_scale", C.c_float), ("cfg_trunc_ratio", C.c_float),
                ("cfg_normalization", C.c_int32)]

    @classmethod
    def of(cls, p, steps=None):
        return cls(int(p.steps if steps is None else steps), float(p.guidance_scale), float(p.cfg_trunc_ratio),
                   1 if p.cfg_normalization else 0)


class NextDit:
    """``NextDit::from_cmf`` (dit.rs:510-589): binds a model; weights become device resident."""

    def __init__(self, model: Model):
        self.model = model
        h = C.c_void_p()
        check(lib().cmfc_nextdit_create(model.handle, C.byref(h)))
        self.handle = h
        dims = (C.c_uint32 * 8)()
        check(lib().cmfc_nextdit_dims(h, dims))
        (self.hidden, self.cap_feat, self.in_channels, self.patch, self.num_layers, self.num_refiner_layers,
         self.nh, self.nkv) = [int(v) for v in dims]

    def close(self):
        if self.handle:
            lib().cmfc_nextdit_destroy(self.handle)
            self.handle = None

    def refine_caption(self, cap, cap_n=None):
        """dit.rs:1201-1226"""
        cap = _f32(cap).reshape(-1, self.cap_feat)
        out = np.empty((cap.shape[0], self.hidden), np.float32)
        check(lib().cmfc_nextdit_refine_caption(self.handle, cap.ctypes.data, cap.shape[0], out.ctypes.data))
        return out

    def forward_with_cap(self, latent, h, w, cap_e, cap_n, t):
        """dit.rs:1389-1507"""
        latent, cap_e = _f32(latent), _f32(cap_e)
        pred = np.empty((self.in_channels, h, w), np.float32)
        check(lib().cmfc_nextdit_forward(self.handle, latent.ctypes.data, h, w, cap_e.ctypes.data, cap_n,
                                         C.c_float(t), pred.ctypes.data))
        return pred

    def forward(self, latent, h, w, cap, cap_n, t):
        """dit.rs:1182-1192"""
        return self.forward_with_cap(latent, h, w, self.refine_caption(cap), cap_n, t)

    def forward_cfg_pair(self, latent, h, w, cap_c, cap_c_n, cap_u, cap_u_n, t, taps=False):
        """dit.rs:1238-1387.  With ``taps`` also returns x after every joint block."""
        latent, cap_c, cap_u = _f32(latent), _f32(cap_c), _f32(cap_u)
        pc = np.empty((self.in_channels, h, w), np.float32)
        pu = np.empty_like(pc)
        if not taps:
            check(lib().cmfc_nextdit_forward_pair(self.handle, latent.ctypes.data, h, w, cap_c.ctypes.data, cap_c_n,
                                                  cap_u.ctypes.data, cap_u_n, C.c_float(t), pc.ctypes.data,
                                                  pu.ctypes.data))
            return pc, pu
        n_img = (h // self.patch) * (w // self.patch)
        n = cap_c_n + cap_u_n + 2 * n_img
        tp = np.empty((self.num_layers, n, self.hidden), np.float32)
        check(lib().cmfc_nextdit_forward_pair_taps(self.handle, latent.ctypes.data, h, w, cap_c.ctypes.data, cap_c_n,
                                                   cap_u.ctypes.data, cap_u_n, C.c_float(t), pc.ctypes.data,
                                                   pu.ctypes.data, tp.ctypes.data))
        return pc, pu, tp

    # ---- batched loop, split form ----
    def denoise_begin(self, latents, cap, cap_u, steps, guidance_scale, params=None):
        """``params`` (a GenParams) carries cfg_trunc_ratio / cfg_normalization; its step count and
        guidance scale are overridden by the explicit arguments."""
        latents, cap = _f32(latents), _f32(cap)
        b, c, h, w = latents.shape
        cap_n = cap.shape[1]
        cu_p, cu_n = None, 0
        if cap_u is not None:
            cap_u = _f32(cap_u)
            cu_p, cu_n = cap_u.ctypes.data, cap_u.shape[1]
        self._shape = latents.shape
        gp = _CGenParams.of(params or GenParams(), steps)
        gp.guidance_scale = float(guidance_scale)
        check(lib().cmfc_denoise_begin_ex(self.handle, latents.ctypes.data, b, h, w, cap.ctypes.data, cap_n, cu_p, cu_n,
                                          C.byref(gp)))

    def denoise_step(self, i):
        check(lib().cmfc_denoise_step(self.handle, i))

    def denoise_end(self, out=None):
        if out is None:
            out = np.empty(self._shape, np.float32)
        check(lib().cmfc_denoise_end(self.handle, out.ctypes.data))
        return out


def denoise(dit: NextDit, latents, cap, cap_u, p: GenParams):
    """imagegen.rs:143-217 for a batch of prompts: ``latents`` [b, c, h, w] start noise,
    ``cap`` [b, cap_n, cap_feat], ``cap_u`` [b, cap_u_n, cap_feat] or None.  Returns the denoised
    latents.  Host buffers in, host buffers out; everything between stays on the device."""
    latents = _f32(latents).copy()
    cap = _f32(cap)
    b, c, h, w = latents.shape
    cu_p, cu_n = None, 0
    if cap_u is not None:
        cap_u = _f32(cap_u)
        cu_p, cu_n = cap_u.ctypes.data, cap_u.shape[1]
    gp = _CGenParams.of(p)
    check(lib().cmfc_denoise_ex(dit.handle, latents.ctypes.data, b, h, w, cap.ctypes.data, cap.shape[1], cu_p, cu_n,
                                C.byref(gp)))
    return latents
