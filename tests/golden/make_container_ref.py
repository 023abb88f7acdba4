"""Generate tests/golden/container_ref_q8.cmf with the reference's OWN container writer
(converter/convert_dtgma_to_cmf.py: _write_cmf -> encode_directory, envelope, per-tensor hashes)
plus container_ref_q8.npz, the f32 inputs it was given.  Build container only:
    python tests/golden/make_container_ref.py /path/to/reference
The library's reader (cmfc_model_open) must open that file unchanged.
"""
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def inputs():
    rng = np.random.default_rng(23)
    w = {"model.layers.0.self_attn.q_proj.weight": (rng.standard_normal((128, 64)) * 0.02).astype(np.float32),
         "model.layers.1.mlp.down_proj.weight": (rng.standard_normal((64, 256)) * 0.3).astype(np.float32),
         "model.norm.weight": (1.0 + 0.1 * rng.standard_normal(64)).astype(np.float32),
         "lm_head.weight": (rng.standard_normal((96, 64)) * 0.05).astype(np.float32)}
    w["model.layers.1.mlp.down_proj.weight"][3] = 0.0      # an all-zero row
    return w


def main():
    if len(sys.argv) < 2:
        raise SystemExit(__doc__)
    sys.path.insert(0, os.path.join(sys.argv[1], "converter"))
    import convert_dtgma_to_cmf as conv
    w = inputs()
    arch = {"arch_name": "container-fixture", "hidden_size": 64, "num_layers": 2, "vocab_size": 96}
    out = os.path.join(HERE, "container_ref_q8.cmf")
    with tempfile.TemporaryDirectory() as d:
        conv._write_cmf(conv.DictSource(w), arch, "Q8_ROW", out, Path(d), None, None, None, None, None, False)
    np.savez_compressed(os.path.join(HERE, "container_ref_q8.npz"), **w)
    print(out, os.path.getsize(out), "bytes")


if __name__ == "__main__":
    main()
