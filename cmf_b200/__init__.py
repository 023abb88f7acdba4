"""B200-native compute backend for the NextDiT denoiser path of the CMF engine
(and the VAE decoder that follows it).

The product is ``libcmf_cuda.so`` (hand-written sm_100a kernels behind a C ABI, see
``include/cmf_cuda.h``).  This package is the host-side mirror of the engine's backend
facade for that path: it loads the library, marshals numpy buffers through ctypes and keeps
the engine's function names and argument meaning.  There is no CPU fallback: every call
either runs on the device or raises :class:`CmfCudaError`.
"""
from ._lib import CmfCudaError, lib, library_path  # noqa: F401
from . import gpu  # noqa: F401
from .container import CmfWriter, Model  # noqa: F401
from .dit import NextDit, GenParams, denoise  # noqa: F401
from .vae import VaeDecoder  # noqa: F401
from .textenc import GemmaEncoder  # noqa: F401
from .imagegen import Pipeline, generate  # noqa: F401
