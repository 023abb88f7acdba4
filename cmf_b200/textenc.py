"""Host-side mirror of the engine's Gemma-2 prompt encoder
(crates/cortiq-engine/src/textenc.rs ``GemmaEncoder``), driving libcmf_cuda.so."""
import ctypes as C

import numpy as np

from ._lib import check, lib
from .container import Model


class GemmaEncoder:
    """``GemmaEncoder::from_cmf`` (textenc.rs:172-216): binds a model's ``te.*`` tensors."""

    def __init__(self, model: Model):
        self.model = model
        h = C.c_void_p()
        check(lib().cmfc_gemma_create(model.handle, C.byref(h)))
        self.handle = h
        dims = (C.c_uint32 * 8)()
        check(lib().cmfc_gemma_dims(h, dims))
        (self.hidden, self.num_layers, self.nh, self.nkv, self.head_dim, self.inter, self.vocab,
         self.window) = [int(v) for v in dims]

    def close(self):
        if self.handle:
            lib().cmfc_gemma_destroy(self.handle)
            self.handle = None

    def encode(self, ids, keep_layer_inputs=False):
        """textenc.rs:222-336: (final-normed hidden [n, hidden], streams) where ``streams`` is the
        list of residual streams entering every layer plus the pre-final-norm stream, or []."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        n = int(ids.size)
        out = np.empty((n, self.hidden), np.float32)
        streams = np.empty((self.num_layers + 1, n, self.hidden), np.float32) if keep_layer_inputs else None
        check(lib().cmfc_gemma_encode(self.handle, ids.ctypes.data, n, out.ctypes.data,
                                      streams.ctypes.data if streams is not None else None))
        return out, ([streams[i] for i in range(self.num_layers + 1)] if streams is not None else [])

    def caption_features(self, ids):
        """The features the denoiser is conditioned on: hidden_states[-2], the stream entering the
        last layer (crates/cortiq-engine/src/imagegen.rs:127-131)."""
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        out = np.empty((int(ids.size), self.hidden), np.float32)
        check(lib().cmfc_gemma_caption_features(self.handle, ids.ctypes.data, int(ids.size), out.ctypes.data))
        return out
