"""Build synthetic NextDiT containers for the tests: weights from tests/synth.py, quantized with
the CPU oracle's encoders, written with the package's container writer."""
import numpy as np

from cmf_b200.container import CmfWriter
from oracle import codecs as oc
from oracle.nextdit import QWeight
from tests import synth


def build(cfg, path, plan, seed=0, norm_jitter=0.0, std=0.02, mutate=None):
    """Returns (tensors_for_oracle, config_json).  ``plan`` maps tensor name -> dtype id; every
    other tensor stays f32.  ``mutate(tensors)`` may edit the f32 tensors before they are quantized."""
    t = synth.make_tensors(cfg, seed, norm_jitter, std)
    if mutate is not None:
        mutate(t)
    w = CmfWriter(arch={"arch_name": "nextdit-synth", "hidden_size": cfg["hidden_size"],
                        "num_layers": cfg["num_layers"], "vocab_size": 0})
    oracle_t = {}
    for name, arr in t.items():
        dt = plan.get(name)
        if dt is None or arr.ndim != 2:
            w.add_f32(name, arr)
            oracle_t[name] = arr
        else:
            q = QWeight.quantize(dt, arr)
            w.add(name, dt, arr.shape, q.payload)
            oracle_t[name] = q
    cj = {k: cfg[k] for k in ("hidden_size", "num_layers", "num_refiner_layers", "num_attention_heads",
                              "num_kv_heads", "in_channels", "patch_size", "axes_dim_rope", "norm_eps")}
    w.add_json("dit.config_json", cj)
    w.write(path)
    return oracle_t, cj


def single_weight_file(path, entries):
    """entries: list of (name, dtype, f32 matrix).  Returns {name: QWeight}."""
    w = CmfWriter(arch={"arch_name": "weights-only", "hidden_size": 0, "num_layers": 0, "vocab_size": 0})
    out = {}
    for name, dt, arr in entries:
        q = QWeight.quantize(dt, arr)
        w.add(name, dt, arr.shape, q.payload)
        out[name] = q
    # the reference's own one-tensor test files carry an f32 pad tensor as well
    w.add_f32("pad", np.zeros((4, 4), np.float32))
    w.write(path)
    return out


def rel_l2(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def load_for_oracle(path, cache=True):
    """Read a container back for the oracle: {name: f32 array | QWeight}, config dict.  Tensor
    bytes come straight from the file mapping (host only)."""
    import json

    from cmf_b200.container import Model
    out = {}
    cfg = None
    m = Model(path)
    try:
        for i in range(len(m)):
            dt, shape, nb = m.info(i)
            name = m.name(i)
            raw = np.array(m.tensor_bytes(i), copy=True)
            if name.endswith(".config_json"):
                if name == "dit.config_json" or cfg is None:
                    cfg = json.loads(raw.tobytes().decode())
            elif dt == 0:
                out[name] = raw.view(np.float32).reshape(shape)
            elif dt in (3, 11, 15):
                out[name] = QWeight(dt, shape[0], shape[1], raw, cache=cache)
    finally:
        m.close()
    return out, cfg
