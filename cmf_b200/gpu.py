"""Host-side mirror of the engine's GPU backend facade for the NextDiT path
(crates/cortiq-engine/src/gpu.rs): same function names, argument order and meaning.

Difference by design: the reference returns ``bool`` and the caller falls back to the CPU on
``False``; this backend has no fallback, so every function returns ``True`` or raises
:class:`CmfCudaError` with the library's status and message.
"""
import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np

from ._lib import check, lib
from .container import Model


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def device_count():
    """gpu.rs:962 device_count"""
    return int(lib().cmfc_device_count())


def set_current_device(i):
    """gpu.rs:978-1000 set_current_device (per thread)"""
    check(lib().cmfc_set_device(int(i)))


def synchronize():
    check(lib().cmfc_synchronize())


def weight_is_resident(model: Model, idx: int) -> bool:
    """gpu.rs:507"""
    return bool(lib().cmfc_weight_is_resident(model.handle, idx))


def _matmat(fn, model, idx, xs, b, rows, cols, out):
    xs = _f32(xs)
    assert xs.size == b * cols and out.size == b * rows and out.dtype == np.float32 and out.flags.c_contiguous
    check(fn(model.handle, idx, xs.ctypes.data, b, rows, cols, out.ctypes.data))
    return True


def q8_matmat(model: Model, idx: int, row_scale, pre, b: int, rows: int, cols: int, out) -> bool:
    """gpu.rs:1155.  ``row_scale`` is accepted for signature parity; the library decodes the
    container's own f16 row scales (the same values)."""
    return _matmat(lib().cmfc_q8_matmat, model, idx, pre, b, rows, cols, out)


def q4t_matmat(model: Model, idx: int, xs, b: int, rows: int, cols: int, out) -> bool:
    """gpu.rs:2439"""
    return _matmat(lib().cmfc_q4t_matmat, model, idx, xs, b, rows, cols, out)


def q4tp_matmat(model: Model, idx: int, xs, b: int, rows: int, cols: int, out) -> bool:
    """gpu.rs:2358"""
    return _matmat(lib().cmfc_q4tp_matmat, model, idx, xs, b, rows, cols, out)


def dit_qkv(model: Model, wq, wk, wv, xs, b, hidden, qrows, kvrows, q_out, k_out, v_out) -> bool:
    """gpu.rs:1891"""
    xs = _f32(xs)
    check(lib().cmfc_dit_qkv(model.handle, wq, wk, wv, xs.ctypes.data, b, hidden, qrows, kvrows,
                             q_out.ctypes.data, k_out.ctypes.data, v_out.ctypes.data))
    return True


def q4t_ffn(model: Model, w1, w3, w2, xs, b, hidden, inter, out) -> bool:
    """gpu.rs:1797 (also serves q8 projections)"""
    xs = _f32(xs)
    check(lib().cmfc_ffn(model.handle, w1, w3, w2, xs.ctypes.data, b, hidden, inter, out.ctypes.data))
    return True


q4tp_ffn = q4t_ffn  # gpu.rs:1773: same entry, the library reads each projection's codec


def dit_attention(qh, kh, vh, nh, nkv, n, hd, scale, out) -> bool:
    """gpu.rs:2332: q [nh][n][hd], k / v [nkv][n][hd] head-major; out [n][nh*hd]."""
    qh, kh, vh = _f32(qh), _f32(kh), _f32(vh)
    check(lib().cmfc_dit_attention(qh.ctypes.data, kh.ctypes.data, vh.ctypes.data, nh, nkv, n, hd,
                                   C.c_float(scale), out.ctypes.data))
    return True


class _BlockArgsC(C.Structure):
    _fields_ = [("n", C.c_uint32), ("hidden", C.c_uint32), ("inter", C.c_uint32), ("nh", C.c_uint32),
                ("nkv", C.c_uint32), ("hd", C.c_uint32), ("eps", C.c_float),
                ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
                ("norm1", C.c_void_p), ("norm2", C.c_void_p), ("ffn_norm1", C.c_void_p), ("ffn_norm2", C.c_void_p),
                ("norm_q", C.c_void_p), ("norm_k", C.c_void_p),
                ("s_msa", C.c_void_p), ("gate_msa", C.c_void_p), ("s_mlp", C.c_void_p), ("gate_mlp", C.c_void_p),
                ("wq", C.c_int64), ("wk", C.c_int64), ("wv", C.c_int64), ("wo", C.c_int64),
                ("w1", C.c_int64), ("w3", C.c_int64), ("w2", C.c_int64),
                ("q4tp", C.c_int32), ("resident_in", C.c_int32), ("resident_out", C.c_int32)]


@dataclass
class DitBlockArgs:
    """gpu.rs:1819-1857, field for field."""
    n: int
    hidden: int
    inter: int
    nh: int
    nkv: int
    hd: int
    eps: float
    rope_cos: np.ndarray
    rope_sin: np.ndarray
    norm1: np.ndarray
    norm2: np.ndarray
    ffn_norm1: np.ndarray
    ffn_norm2: np.ndarray
    norm_q: np.ndarray
    norm_k: np.ndarray
    s_msa: Optional[np.ndarray]
    gate_msa: Optional[np.ndarray]
    s_mlp: Optional[np.ndarray]
    gate_mlp: Optional[np.ndarray]
    wq: int
    wk: int
    wv: int
    wo: int
    w1: int
    w3: int
    w2: int
    q4tp: bool = False
    resident_in: bool = False
    resident_out: bool = False


def dit_block_seg(model: Model, a: DitBlockArgs, segs, x) -> bool:
    """gpu.rs:1936: one adaLN block over concatenated segments; ``x`` [n, hidden] in-out."""
    keep = []

    def ptr(v):
        if v is None:
            return None
        v = _f32(v)
        keep.append(v)
        return v.ctypes.data
    ca = _BlockArgsC(a.n, a.hidden, a.inter, a.nh, a.nkv, a.hd, a.eps, ptr(a.rope_cos), ptr(a.rope_sin),
                     ptr(a.norm1), ptr(a.norm2), ptr(a.ffn_norm1), ptr(a.ffn_norm2), ptr(a.norm_q), ptr(a.norm_k),
                     ptr(a.s_msa), ptr(a.gate_msa), ptr(a.s_mlp), ptr(a.gate_mlp),
                     a.wq, a.wk, a.wv, a.wo, a.w1, a.w3, a.w2, int(a.q4tp), int(a.resident_in), int(a.resident_out))
    sg = np.ascontiguousarray(segs, dtype=np.uint32)
    xp = None
    if x is not None:
        assert x.dtype == np.float32 and x.flags.c_contiguous
        xp = x.ctypes.data
    check(lib().cmfc_dit_block_seg(model.handle, C.byref(ca), sg.ctypes.data, sg.size, xp))
    return True


def dit_block(model: Model, a: DitBlockArgs, x) -> bool:
    """gpu.rs:1932"""
    return dit_block_seg(model, a, [a.n], x)


def dit_chain_supported() -> bool:
    """gpu.rs:1862"""
    return bool(lib().cmfc_dit_chain_supported())


def dit_state_fetch(x) -> bool:
    """gpu.rs:1873"""
    check(lib().cmfc_dit_state_fetch(x.ctypes.data, x.size))
    return True


def fused_dit_block_available() -> bool:
    """gpu.rs:1918: False, so the caller prefers the batched CFG pair (imagegen.rs:170)."""
    return bool(lib().cmfc_fused_dit_block_available())


def payload_nbytes(dtype, rows, cols):
    return int(lib().cmfc_payload_nbytes(dtype, rows, cols))


def encode(dtype, w):
    """Device-side quantizer, byte-identical to the reference encoders
    (crates/cortiq-cli/src/convert.rs:551-613, :883-992)."""
    w = _f32(w)
    rows, cols = w.shape
    out = np.empty(payload_nbytes(dtype, rows, cols), np.uint8)
    check(lib().cmfc_encode(dtype, w.ctypes.data, rows, cols, out.ctypes.data))
    return out


def encode_random(dtype, seed, std, rows, cols, out=None):
    """Quantize w ~ N(0, std) generated on the device from ``seed``."""
    if out is None:
        out = np.empty(payload_nbytes(dtype, rows, cols), np.uint8)
    check(lib().cmfc_encode_random(dtype, seed, C.c_float(std), rows, cols, out.ctypes.data))
    return out


def noalloc_max_elements():
    return int(lib().cmfc_noalloc_max_elements())


def matmat_device_noalloc(model: Model, idx: int, d_x_ptr: int, b: int, d_y_ptr: int) -> bool:
    """Quantized linear on caller-owned DEVICE buffers (raw pointers) for hosts that cannot allocate
    device memory at call time; the tensor must already be resident and b * cols must fit the
    library's fixed scratch (``noalloc_max_elements``).  No counterpart in the reference."""
    check(lib().cmfc_matmat_device_noalloc(model.handle, idx, d_x_ptr, b, d_y_ptr))
    return True


def selftest_wait_timeout(polls=2048):
    """Let a bounded device wait run out on purpose (a barrier nobody arrives on): raises
    CmfCudaError with code -5 (CMFC_ERR_DEVICE_WAIT); the context stays usable."""
    check(lib().cmfc_selftest_wait_timeout(polls))


def launch_count(reset=False):
    return int(lib().cmfc_launch_count(int(reset)))


def bench_gemm(model: Model, idx, M, mode=0, iters=10):
    ms = C.c_float()
    check(lib().cmfc_bench_gemm(model.handle, idx, M, mode, iters, C.byref(ms)))
    return ms.value


def bench_attention(nh, nkv, hd, n, nseg=1, iters=5):
    ms = C.c_float()
    check(lib().cmfc_bench_attention(nh, nkv, hd, n, nseg, iters, C.byref(ms)))
    return ms.value


def bench_rowop(kind, rows, cols, iters=10):
    """-> (ms per launch, algorithmic bytes per launch)"""
    ms, nb = C.c_float(), C.c_double()
    check(lib().cmfc_bench_rowop(kind, rows, cols, iters, C.byref(ms), C.byref(nb)))
    return ms.value, nb.value


def bench_vae_decode(vae, h, w, iters=3):
    ms = C.c_float()
    check(lib().cmfc_bench_vae_decode(vae.handle, h, w, iters, C.byref(ms)))
    return float(ms.value)


def bench_gemma(enc, n, iters=5):
    ms = C.c_float()
    check(lib().cmfc_bench_gemma(enc.handle, n, iters, C.byref(ms)))
    return float(ms.value)


def bench_conv(ic, oc, h, w, k=3, a_planes=1, iters=5):
    ms = C.c_float()
    check(lib().cmfc_bench_conv(ic, oc, h, w, k, a_planes, iters, C.byref(ms)))
    return float(ms.value)


def profile_enable(on=True):
    check(lib().cmfc_profile_enable(int(on)))


def profile_read():
    import json
    buf = C.create_string_buffer(8192)
    check(lib().cmfc_profile_read(buf, len(buf)))
    return json.loads(buf.value.decode())


def stream_handle():
    """Raw cudaStream_t of the current device context (for external event timing)."""
    return int(lib().cmfc_stream_handle() or 0)
