"""ctypes binding of libcmf_cuda.so.  Loading fails loudly when the library is absent."""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class CmfCudaError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"libcmf_cuda status {code}: {message}")
        self.code = code


def library_path():
    return os.path.join(HERE, "libcmf_cuda.so")


SYMBOLS = {
    # name: (restype, argtypes)
    "cmfc_last_error": (C.c_char_p, []),
    "cmfc_device_count": (C.c_int, []),
    "cmfc_set_device": (C.c_int, [C.c_int]),
    "cmfc_synchronize": (C.c_int, []),
    "cmfc_model_open": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "cmfc_model_close": (None, [C.c_void_p]),
    "cmfc_model_tensor_count": (C.c_int64, [C.c_void_p]),
    "cmfc_model_find": (C.c_int64, [C.c_void_p, C.c_char_p]),
    "cmfc_model_tensor_info": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                         C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)]),
    "cmfc_model_tensor_name": (C.c_char_p, [C.c_void_p, C.c_int64]),
    "cmfc_model_tensor_bytes": (C.c_void_p, [C.c_void_p, C.c_int64]),
    "cmfc_weight_is_resident": (C.c_int, [C.c_void_p, C.c_int64]),
    "cmfc_weight_dequant": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t]),
    "cmfc_q8_matmat": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_q4t_matmat": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_q4tp_matmat": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_dit_qkv": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t, C.c_size_t,
                               C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]),
    "cmfc_ffn": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t, C.c_size_t,
                           C.c_size_t, C.c_void_p]),
    "cmfc_dit_attention": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                     C.c_size_t, C.c_float, C.c_void_p]),
    "cmfc_dit_block_seg": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cmfc_dit_chain_supported": (C.c_int, []),
    "cmfc_dit_state_fetch": (C.c_int, [C.c_void_p, C.c_size_t]),
    "cmfc_fused_dit_block_available": (C.c_int, []),
    "cmfc_nextdit_create": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "cmfc_nextdit_destroy": (None, [C.c_void_p]),
    "cmfc_nextdit_dims": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "cmfc_nextdit_refine_caption": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cmfc_nextdit_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                                       C.c_float, C.c_void_p]),
    "cmfc_nextdit_forward_pair": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                                            C.c_void_p, C.c_size_t, C.c_float, C.c_void_p, C.c_void_p]),
    "cmfc_nextdit_forward_pair_taps": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p,
                                                 C.c_size_t, C.c_void_p, C.c_size_t, C.c_float, C.c_void_p,
                                                 C.c_void_p, C.c_void_p]),
    "cmfc_vae_create": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "cmfc_vae_destroy": (None, [C.c_void_p]),
    "cmfc_vae_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.POINTER(C.c_float),
                                C.POINTER(C.c_float)]),
    "cmfc_vae_decode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_vae_decode_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_vae_conv2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                  C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_vae_upsample_conv": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t,
                                         C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_bench_vae_decode": (C.c_int, [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.POINTER(C.c_float)]),
    "cmfc_bench_conv": (C.c_int, [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_int,
                                  C.POINTER(C.c_float)]),
    "cmfc_gemma_create": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "cmfc_gemma_destroy": (None, [C.c_void_p]),
    "cmfc_gemma_dims": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "cmfc_gemma_caption_features": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cmfc_bench_gemma": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int, C.POINTER(C.c_float)]),
    "cmfc_gemma_encode": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "cmfc_denoise": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                               C.c_void_p, C.c_size_t, C.c_uint32, C.c_float]),
    "cmfc_denoise_begin": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p,
                                     C.c_size_t, C.c_void_p, C.c_size_t, C.c_uint32, C.c_float]),
    "cmfc_denoise_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_size_t,
                                  C.c_void_p, C.c_size_t, C.c_void_p]),
    "cmfc_denoise_begin_ex": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p,
                                        C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cmfc_denoise_step": (C.c_int, [C.c_void_p, C.c_uint32]),
    "cmfc_denoise_end": (C.c_int, [C.c_void_p, C.c_void_p]),
    "cmfc_payload_nbytes": (C.c_size_t, [C.c_int, C.c_size_t, C.c_size_t]),
    "cmfc_encode": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_encode_random": (C.c_int, [C.c_int, C.c_uint64, C.c_float, C.c_size_t, C.c_size_t, C.c_void_p]),
    "cmfc_noalloc_max_elements": (C.c_size_t, []),
    "cmfc_matmat_device_noalloc": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p]),
    "cmfc_selftest_wait_timeout": (C.c_int, [C.c_uint32]),
    "cmfc_launch_count": (C.c_uint64, [C.c_int]),
    "cmfc_bench_gemm": (C.c_int, [C.c_void_p, C.c_int64, C.c_size_t, C.c_int, C.c_int, C.POINTER(C.c_float)]),
    "cmfc_bench_attention": (C.c_int, [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.POINTER(C.c_float)]),
    "cmfc_bench_rowop": (C.c_int, [C.c_int, C.c_size_t, C.c_size_t, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_double)]),
    "cmfc_stream_handle": (C.c_void_p, []),
    "cmfc_profile_enable": (C.c_int, [C.c_int]),
    "cmfc_profile_read": (C.c_int, [C.c_char_p, C.c_size_t]),
}


def lib():
    """The loaded library.  Raises if it was not built: there is no other implementation."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not os.path.exists(path):
            raise CmfCudaError(-7, f"{path} is missing; build it with `python cmf_b200/build.py` "
                                   "(nvcc, sm_100a).  This package has no CPU fallback.")
        L = C.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def check(rc):
    if rc is not None and rc < 0:
        msg = lib().cmfc_last_error()
        raise CmfCudaError(rc, msg.decode("utf-8", "replace") if msg else "")
    return rc
