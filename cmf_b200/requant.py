"""Recoding of an existing .cmf between quantization layouts on the device: the lossless-in-the-grid
case of the reference's ``cortiq requant`` (crates/cortiq-cli/src/requant.rs:48-57, Mode::FullQ4tp):
every 2-D q4_tiled tensor is dequantized exactly and re-encoded as q4tp (same 4-bit grid, the
per-tile scale re-expressed as a rung on a per-row ladder); everything else is copied verbatim.

    python -m cmf_b200.requant in.cmf out.cmf
"""
import json
import struct
import sys

import numpy as np

from . import gpu
from .container import CmfWriter, DT_Q4TP, DT_Q4_TILED, Model


def read_header(path):
    """The header JSON of a container (envelope layout: crates/cortiq-core/src/format.rs:653-728)."""
    with open(path, "rb") as f:
        env = f.read(128)
        if env[:4] != b"CMF\x01":
            raise ValueError(f"{path}: not a CMF container")
        off, ln = struct.unpack_from("<QQ", env, 16)
        f.seek(off)
        return json.loads(f.read(ln).decode())


def requant_q4tp(src, dst):
    """Returns (tensors recoded, bytes before, bytes after)."""
    hdr = read_header(src)
    w = CmfWriter(arch=hdr.get("arch", {}), quant_type=hdr.get("quant_type", "mixed"))
    recoded = before = after = 0
    with Model(src) as m:
        for i in range(len(m)):
            dt, shape, nb = m.info(i)
            name = m.name(i)
            before += nb
            if dt == DT_Q4_TILED and len(shape) == 2 and shape[1] % 32 == 0:
                payload = gpu.encode(DT_Q4TP, m.dequant(i))
                w.add(name, DT_Q4TP, shape, payload)
                recoded += 1
                after += payload.nbytes
            else:
                w.add(name, dt, shape, np.array(m.tensor_bytes(i), copy=True))
                after += nb
    w.write(dst)
    return recoded, before, after


def main():
    if len(sys.argv) != 3:
        raise SystemExit(__doc__)
    n, b, a = requant_q4tp(sys.argv[1], sys.argv[2])
    print(f"recoded {n} tensors to q4tp: {b / 1e6:.1f} MB -> {a / 1e6:.1f} MB of tensor data")


if __name__ == "__main__":
    main()
