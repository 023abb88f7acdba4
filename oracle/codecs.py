"""ctypes face of the CPU oracle's C restatement (oracle/cmf_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg
of the benchmark; never by the shipped package.
"""
import ctypes as C

import numpy as np

from . import build as _build

_lib = None

# TensorDtype ids (crates/cortiq-core/src/types.rs:10-98)
F32, U8, Q8_ROW, Q4_TILED, Q4TP = 0, 6, 3, 11, 15


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(_build.build())
        sz, vp = C.c_size_t, C.c_void_p
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_scale.restype = C.c_float
        L.orc_f16_scale.argtypes = [C.c_float]
        L.orc_q4tp_nbytes.restype = sz
        L.orc_q4tp_nbytes.argtypes = [sz, sz]
        L.orc_q4tp_code_stride.restype = sz
        L.orc_q4tp_code_stride.argtypes = [sz]
        L.orc_q4tp_code.restype = C.c_uint
        L.orc_q4tp_code.argtypes = [vp, sz, sz]
        for name in ("orc_encode_q8_row", "orc_encode_q4_tiled", "orc_encode_q4tp",
                     "orc_dequant_q8_row", "orc_dequant_q4tp", "orc_q4tp_scales"):
            getattr(L, name).argtypes = [vp, sz, sz, vp]
            getattr(L, name).restype = None
        L.orc_encode_q4_block.argtypes = [vp, sz, vp]
        L.orc_dequant_q4_tiled.argtypes = [vp, sz, vp]
        for name in ("orc_matmat_q8", "orc_matmat_q4t", "orc_matmat_q4tp"):
            getattr(L, name).argtypes = [vp, sz, sz, vp, sz, vp]
            getattr(L, name).restype = None
        L.orc_gemm_nt.argtypes = [vp, vp, vp, sz, sz, sz]
        L.orc_q4tp_ladder.argtypes = [C.c_uint16, C.c_uint16, vp]
        L.orc_num_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _f32c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _u8c(a):
    if isinstance(a, (bytes, bytearray, memoryview)):
        a = np.frombuffer(a, dtype=np.uint8)
    return np.ascontiguousarray(a, dtype=np.uint8)


def nbytes(dtype, rows, cols):
    """Payload size (crates/cortiq-core/src/quant.rs:552-613, the three codecs on this path)."""
    if dtype == Q8_ROW:
        return rows * cols + 2 * rows
    if dtype == Q4_TILED:
        return rows * cols // 32 * 18
    if dtype == Q4TP:
        return int(lib().orc_q4tp_nbytes(rows, cols))
    if dtype == F32:
        return rows * cols * 4
    raise ValueError(dtype)


def f16_to_f32(h):
    return float(lib().orc_f16_to_f32(int(h)))


def f32_to_f16(x):
    return int(lib().orc_f32_to_f16(float(x)))


def encode(dtype, w):
    w = _f32c(w)
    rows, cols = w.shape
    out = np.zeros(nbytes(dtype, rows, cols), np.uint8)
    if dtype == F32:
        return w.view(np.uint8).reshape(-1).copy()
    fn = {Q8_ROW: "orc_encode_q8_row", Q4_TILED: "orc_encode_q4_tiled", Q4TP: "orc_encode_q4tp"}[dtype]
    getattr(lib(), fn)(_p(w), rows, cols, _p(out))
    return out


def encode_q4_block(w):
    w = _f32c(w).reshape(-1)
    g = (w.size + 31) // 32
    out = np.zeros(g * 18, np.uint8)
    lib().orc_encode_q4_block(_p(w), w.size, _p(out))
    return out


def dequant(dtype, payload, rows, cols):
    """Exact f32 weights [rows, cols] -- the bit-exact weight definition."""
    p = _u8c(payload)
    assert p.size == nbytes(dtype, rows, cols), (p.size, nbytes(dtype, rows, cols))
    if dtype == F32:
        return p.view(np.float32).reshape(rows, cols).copy()
    dst = np.empty((rows, cols), np.float32)
    if dtype == Q8_ROW:
        lib().orc_dequant_q8_row(_p(p), rows, cols, _p(dst))
    elif dtype == Q4_TILED:
        lib().orc_dequant_q4_tiled(_p(p), rows * cols, _p(dst))
    elif dtype == Q4TP:
        lib().orc_dequant_q4tp(_p(p), rows, cols, _p(dst))
    else:
        raise ValueError(dtype)
    return dst


def q4tp_scales(payload, rows, cols):
    p = _u8c(payload)
    s = np.empty((rows, cols // 32), np.float32)
    lib().orc_q4tp_scales(_p(p), rows, cols, _p(s))
    return s


def q4tp_ladder(lo_h, step_h):
    t = np.empty(32, np.float32)
    lib().orc_q4tp_ladder(int(lo_h), int(step_h), _p(t))
    return t


def matmat_exact(dtype, payload, rows, cols, x):
    """Y[b, rows] = X[b, cols] . W^T in the reference's strict scalar order."""
    p = _u8c(payload)
    x = _f32c(x)
    b = x.shape[0]
    y = np.empty((b, rows), np.float32)
    if dtype == F32:
        lib().orc_gemm_nt(_p(x), _p(p.view(np.float32)), _p(y), b, cols, rows)
        return y
    fn = {Q8_ROW: "orc_matmat_q8", Q4_TILED: "orc_matmat_q4t", Q4TP: "orc_matmat_q4tp"}[dtype]
    getattr(lib(), fn)(_p(p), rows, cols, _p(x), b, _p(y))
    return y


def gemm_nt(x, w):
    x, w = _f32c(x), _f32c(w)
    y = np.empty((x.shape[0], w.shape[0]), np.float32)
    lib().orc_gemm_nt(_p(x), _p(w), _p(y), x.shape[0], x.shape[1], w.shape[0])
    return y


def num_threads():
    return int(lib().orc_num_threads())


def bf16_round(a):
    """f32 -> nearest-even bf16 -> f32 (how the GPU path quantizes GEMM operands)."""
    u = _f32c(a).view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return r.astype(np.uint32).view(np.float32).reshape(np.shape(a))
