"""Minimal CMF v2 container writer and the mmap-backed model handle.

Layout written (crates/cortiq-core/src/format.rs:5-12, :28-50, :653-791): 128-byte envelope,
JSON header, directory ([count][pool_off] + 56-byte records + name pool), 4096-aligned data
section with 64-byte-aligned tensors (4096 for tensors of 16 KiB and more).  Only what the
NextDiT path reads is produced: no masks, vocab or index sections.
"""
import ctypes as C
import json
import struct

import numpy as np

from ._lib import check, lib

DT_F32, DT_F16, DT_U8, DT_Q8_ROW, DT_Q4_TILED, DT_Q4TP = 0, 1, 6, 3, 11, 15
_MASK = (1 << 64) - 1


def _fmix64(x):
    x = x ^ (x >> np.uint64(33))
    x = x * np.uint64(0xFF51AFD7ED558CCD)
    x = x ^ (x >> np.uint64(33))
    x = x * np.uint64(0xC4CEB9FE1A85EC53)
    return x ^ (x >> np.uint64(33))


def hash64(buf):
    """Container content hash (crates/cortiq-core/src/hash.rs:8-36)."""
    a = np.frombuffer(buf, dtype=np.uint8)
    n = a.size
    pad = (-n) % 8
    if pad:
        a = np.concatenate([a, np.zeros(pad, np.uint8)])
    w = a.view(np.uint64)
    with np.errstate(over="ignore"):
        if w.size:
            m = _fmix64(w) ^ (np.arange(w.size, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15))
            h = np.bitwise_xor.reduce(m)
        else:
            h = np.uint64(0)
        h = _fmix64(np.array([h ^ np.uint64(n)], dtype=np.uint64))[0]
    return int(h)


def _align(x, a):
    return (x + a - 1) // a * a


class CmfWriter:
    """Collects tensors, then writes one .cmf file."""

    def __init__(self, arch=None, quant_type="mixed"):
        self.arch = arch or {}
        self.quant_type = quant_type
        self.tensors = []  # (name, dtype, shape, bytes-like)

    def add(self, name, dtype, shape, payload):
        payload = memoryview(payload).cast("B") if not isinstance(payload, np.ndarray) else payload
        self.tensors.append((name, int(dtype), tuple(int(s) for s in shape), payload))

    def add_f32(self, name, array):
        a = np.ascontiguousarray(array, np.float32)
        self.add(name, DT_F32, a.shape, a.view(np.uint8).reshape(-1))

    def add_json(self, name, obj):
        b = np.frombuffer(json.dumps(obj).encode(), np.uint8)
        self.add(name, DT_U8, (b.size,), b)

    def write(self, path, hash_tensors=True):
        header = json.dumps({"format": "cmf", "version": 2, "arch": self.arch, "quant_type": self.quant_type}).encode()
        pool = bytearray()
        recs = []
        off = 0
        for name, dt, shape, payload in self.tensors:
            nb = payload.nbytes if hasattr(payload, "nbytes") else len(payload)
            off = _align(off, 4096 if nb >= 16384 else 64)
            nm = name.encode()
            sh = list(shape) + [0] * (6 - len(shape))
            th = hash64(payload) if hash_tensors else 0
            recs.append(struct.pack("<IHBB6IQQQ", len(pool), len(nm), dt, len(shape), *sh, off, nb, th))
            pool += nm
            off += nb
        data_len = off
        directory = struct.pack("<QQ", len(recs), 16 + 56 * len(recs)) + b"".join(recs) + bytes(pool)
        header_off = 128
        dir_off = _align(header_off + len(header), 64)
        data_off = _align(dir_off + len(directory), 4096)
        env = bytearray(128)
        env[0:4] = b"CMF\x01"
        struct.pack_into("<III", env, 4, 2, 0, 1)  # version, flags, required_features (tensor directory)
        struct.pack_into("<12Q", env, 16, header_off, len(header), dir_off, len(directory), data_off, data_len,
                         0, 0, 0, 0, 0, 0)
        struct.pack_into("<QQ", env, 0x70, hash64(header), hash64(directory))
        with open(path, "wb") as f:
            f.write(env)
            f.write(header)
            f.write(b"\0" * (dir_off - header_off - len(header)))
            f.write(directory)
            f.write(b"\0" * (data_off - dir_off - len(directory)))
            pos = 0
            for (name, dt, shape, payload), rec in zip(self.tensors, recs):
                toff = struct.unpack_from("<Q", rec, 32)[0]
                if toff > pos:
                    f.write(b"\0" * (toff - pos))
                    pos = toff
                f.write(payload)
                pos += payload.nbytes if hasattr(payload, "nbytes") else len(payload)
        return path


class Model:
    """An opened container (the engine's ``Arc<CmfModel>``): mmap'ed by the library."""

    def __init__(self, path):
        h = C.c_void_p()
        check(lib().cmfc_model_open(str(path).encode(), C.byref(h)))
        self.handle = h
        self.path = str(path)

    def close(self):
        if self.handle:
            lib().cmfc_model_close(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __len__(self):
        return int(lib().cmfc_model_tensor_count(self.handle))

    def index(self, name):
        return int(check(lib().cmfc_model_find(self.handle, name.encode())))

    def name(self, idx):
        n = lib().cmfc_model_tensor_name(self.handle, idx)
        return n.decode() if n else None

    def info(self, idx):
        dt, nd, nb = C.c_int(), C.c_int(), C.c_uint64()
        shape = (C.c_uint32 * 6)()
        check(lib().cmfc_model_tensor_info(self.handle, idx, C.byref(dt), C.byref(nd), shape, C.byref(nb)))
        return dt.value, tuple(shape[:nd.value]), nb.value

    def tensor_bytes(self, idx):
        dt, shape, nb = self.info(idx)
        p = lib().cmfc_model_tensor_bytes(self.handle, idx)
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_uint8)), shape=(nb,))

    def dequant(self, idx):
        """Exact f32 weights of a quantized 2-D tensor, dequantized on the device."""
        dt, shape, nb = self.info(idx)
        out = np.empty(shape, np.float32)
        check(lib().cmfc_weight_dequant(self.handle, idx, out.ctypes.data, out.size))
        return out
