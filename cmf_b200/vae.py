"""Host-side mirror of the engine's VAE decoder (crates/cortiq-engine/src/vae.rs ``VaeDecoder``) and
of the facade's stand-alone convolution entries (crates/cortiq-engine/src/gpu.rs:2002-2046),
driving the device implementation in libcmf_cuda.so."""
import ctypes as C

import numpy as np

from ._lib import check, lib
from .container import Model


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class VaeDecoder:
    """``VaeDecoder::from_cmf`` (vae.rs:524-548): binds a model's ``vae.*`` tensors."""

    def __init__(self, model: Model):
        self.model = model
        h = C.c_void_p()
        check(lib().cmfc_vae_create(model.handle, C.byref(h)))
        self.handle = h
        lc, up = C.c_uint32(), C.c_uint32()
        sf, sh = C.c_float(), C.c_float()
        check(lib().cmfc_vae_info(h, C.byref(lc), C.byref(up), C.byref(sf), C.byref(sh)))
        self.latent_channels, self.upscale = int(lc.value), int(up.value)
        self.scaling_factor, self.shift_factor = float(sf.value), float(sh.value)

    def close(self):
        if self.handle:
            lib().cmfc_vae_destroy(self.handle)
            self.handle = None

    def decode(self, z, h, w):
        """vae.rs:637-690: latents [latent_channels, h, w] -> RGB [3, s*h, s*w]."""
        z = _f32(z)
        assert z.size == self.latent_channels * h * w
        out = np.empty((3, self.upscale * h, self.upscale * w), np.float32)
        check(lib().cmfc_vae_decode(self.handle, z.ctypes.data, h, w, out.ctypes.data))
        return out

    def decode_device(self, d_z, h, w, d_out):
        """The same on raw device pointers (ints)."""
        check(lib().cmfc_vae_decode_device(self.handle, C.c_void_p(d_z), h, w, C.c_void_p(d_out)))


def conv2d(w, bias, x, ic, oc, h, w_img, k):
    """gpu::vae_conv2d (gpu.rs:2026-2046)."""
    w, bias, x = _f32(w), _f32(bias), _f32(x)
    assert w.size == oc * ic * k * k and bias.size == oc and x.size == ic * h * w_img
    out = np.empty((oc, h, w_img), np.float32)
    check(lib().cmfc_vae_conv2d(w.ctypes.data, bias.ctypes.data, x.ctypes.data, ic, oc, h, w_img, k, out.ctypes.data))
    return out


def upsample_conv(w, bias, x, ic, oc, h, w_img, k):
    """gpu::vae_upsample_conv (gpu.rs:2002-2022)."""
    w, bias, x = _f32(w), _f32(bias), _f32(x)
    assert w.size == oc * ic * k * k and bias.size == oc and x.size == ic * h * w_img
    out = np.empty((oc, 2 * h, 2 * w_img), np.float32)
    check(lib().cmfc_vae_upsample_conv(w.ctypes.data, bias.ctypes.data, x.ctypes.data, ic, oc, h, w_img, k,
                                       out.ctypes.data))
    return out
