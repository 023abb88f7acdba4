"""Generate tests/golden/codecs_ref.npz from the reference's own numpy encoders and reader
(converter/convert_dtgma_to_cmf.py, python/cmf_reader.py).  Build container only:
    python tests/golden/make_codecs_ref.py /path/to/reference
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def inputs():
    rng = np.random.default_rng(11)
    cases = {}
    for i, (r, c, std) in enumerate([(7, 64, 0.02), (16, 96, 1.0), (5, 256, 0.3)]):
        w = (rng.standard_normal((r, c)) * std).astype(np.float32)
        w[1] = 0.0                 # an all-zero row
        w[2, :32] = 0.0            # an all-zero group
        w[3, 5] = 40.0 * std       # an outlier
        cases[f"w{i}"] = w
    return cases


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "converter"))
    sys.path.insert(0, os.path.join(ref, "python"))
    import cmf_reader
    import convert_dtgma_to_cmf as cv
    out = {}
    for k, w in inputs().items():
        q8 = np.frombuffer(cv.encode_q8_row(w), np.uint8)
        q4 = np.frombuffer(cv.encode_q4_block(w), np.uint8)
        out[k + "_q8"] = q8
        out[k + "_q4block"] = q4
        out[k + "_q8_deq"] = cmf_reader.dequant(q8.tobytes(), "q8_row", w.shape)
        # q4_tiled bytes = q4_block values with the scale moved in front of each 16-byte group
        g = w.size // 32
        tiled = np.concatenate([q4[g * 16:].reshape(g, 2), q4[:g * 16].reshape(g, 16)], 1).reshape(-1)
        out[k + "_q4t_deq"] = cmf_reader.dequant(tiled.tobytes(), "q4_tiled", w.shape)
        out[k + "_hash"] = np.array([cmf_reader.hash64(q8.tobytes())], np.uint64)
    np.savez_compressed(os.path.join(HERE, "codecs_ref.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
