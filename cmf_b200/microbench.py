"""Kernel micro-benchmarks on synthetic device-resident inputs (CUDA-event timing inside the
library).  Used for the per-kernel roofline tables and as the small cases for profiler captures.

    python -m cmf_b200.microbench gemm --codec q4t --N 2304 --K 2304 --M 8704
    python -m cmf_b200.microbench attention --n 4352 --nseg 2
    python -m cmf_b200.microbench rowops --rows 8704
    python -m cmf_b200.microbench sweep          # dequant GEMM over (K, N) x M x codec: 4 Lumina-2 projection shapes, M = 256 / 4352 / 17408
    python -m cmf_b200.microbench conv --ic 128 --oc 128 --h 1024 --w 1024
    python -m cmf_b200.microbench vae --latent 128   # whole FLUX-VAE decode with per-stage times
    python -m cmf_b200.microbench gemma --n 128 --codec q4t   # Gemma-2-2B prompt encode with per-stage times
"""
import argparse
import json
import os
import tempfile

import numpy as np

from . import gpu
from .container import CmfWriter, Model
from .synth import CODECS

ROWOPS = {0: "rms_mod", 1: "gated_residual", 2: "residual_then_norm", 3: "qk_rope_pack"}


def _weight_file(entries):
    path = os.path.join(tempfile.gettempdir(), f"cmf_microbench_{os.getpid()}.cmf")
    w = CmfWriter(arch={"arch_name": "microbench"})
    for name, dt, N, K, seed in entries:
        w.add(name, dt, (N, K), gpu.encode_random(dt, seed, 0.02, N, K))
    w.write(path, hash_tensors=False)
    return path


def gemm(codec, N, K, M, iters, mode=0):
    path = _weight_file([("w", CODECS[codec], N, K, 7)])
    try:
        with Model(path) as m:
            ms = gpu.bench_gemm(m, m.index("w"), M, mode=mode, iters=iters)
    finally:
        os.remove(path)
    bpw = {"q8": 1.0, "q4t": 0.5625, "q4tp": 0.5195}[codec]
    return {"kernel": "gemm_dequant", "codec": codec, "mode": mode, "M": M, "N": N, "K": K, "ms": ms,
            "tflops": 2.0 * M * N * K / (ms * 1e-3) / 1e12,
            "algorithmic_bytes": K * N * bpw + 2.0 * M * K + (4.0 if mode == 0 else 2.0) * M * N}


def conv(ic, oc, h, w, k, planes, iters):
    ms = gpu.bench_conv(ic, oc, h, w, k, planes, iters)
    fl = 2.0 * h * w * oc * ic * k * k
    return {"kernel": "conv_f16x2", "ic": ic, "oc": oc, "h": h, "w": w, "k": k, "weight_planes": planes, "ms": ms,
            "conv_tflops": fl / (ms * 1e-3) / 1e12, "mma_tflops": fl * (planes + 1) / (ms * 1e-3) / 1e12,
            "algorithmic_bytes": 4.0 * h * w * (ic + oc) + 2.0 * planes * oc * ic * k * k}


def vae_flops(cfg, lh, lw):
    """Multiply-add FLOPs (2 per MAC) of one decode, convolutions and attention products."""
    from .synth import vae_tensor_list
    rev = list(reversed(cfg["block_out_channels"]))
    ups = {f"decoder.up_blocks.{b}": 2 ** b for b in range(len(rev))}   # resolution factor inside up block b
    total = 0.0
    for name, shape, kind in vae_tensor_list(cfg):
        if kind not in ("k", "l"):
            continue
        scale = 1
        for pre, f in ups.items():
            if name.startswith(pre + "."):
                scale = f * (2 if ".upsamplers." in name else 1)
        if name.startswith("decoder.conv_norm_out") or name.startswith("decoder.conv_out"):
            scale = 2 ** (len(rev) - 1)
        pix = lh * lw * scale * scale
        total += 2.0 * pix * float(np.prod(shape))
    n = lh * lw
    total += 4.0 * n * n * rev[0]
    return total


def vae_decode(latent, iters):
    from .synth import FLUX_VAE, write_vae_model
    from .vae import VaeDecoder
    path = os.path.join(tempfile.gettempdir(), f"cmf_microbench_vae_{os.getpid()}.cmf")
    write_vae_model(path, FLUX_VAE, 0)
    try:
        with Model(path) as m:
            dec = VaeDecoder(m)
            ms = gpu.bench_vae_decode(dec, latent, latent, iters)
            gpu.profile_enable(True)
            gpu.bench_vae_decode(dec, latent, latent, 1)
            spans = gpu.profile_read()
            gpu.profile_enable(False)
            dec.close()
    finally:
        os.remove(path)
    fl = vae_flops(FLUX_VAE, latent, latent)
    return {"kernel": "vae_decode", "latent": latent, "image": latent * 8, "ms": ms, "flops": fl,
            "tflops": fl / (ms * 1e-3) / 1e12, "stages": spans}


def gemma_encode(n, codec, iters):
    from .synth import GEMMA2_2B, write_gemma_model
    from .textenc import GemmaEncoder
    cfg = dict(GEMMA2_2B, vocab_size=4096)   # the forward touches n rows of the table; 4096 keep the file small
    path = os.path.join(tempfile.gettempdir(), f"cmf_microbench_te_{os.getpid()}.cmf")
    write_gemma_model(path, cfg, codec, 0)
    try:
        with Model(path) as m:
            enc = GemmaEncoder(m)
            ms = gpu.bench_gemma(enc, n, iters)
            gpu.profile_enable(True)
            gpu.bench_gemma(enc, n, 1)
            spans = gpu.profile_read()
            gpu.profile_enable(False)
            enc.close()
    finally:
        os.remove(path)
    hs, inter, nh, nkv, hd, nl = 2304, 9216, 8, 4, 256, 26
    params = (nh + 2 * nkv) * hd * hs + hs * nh * hd + 3 * inter * hs
    fl = 2.0 * n * params * (nl - 1)
    return {"kernel": "gemma_caption_features", "tokens": n, "codec": codec, "ms": ms, "gemm_flops": fl,
            "weights_bytes": params * (nl - 1) * {"q8": 1.0, "q4t": 0.5625, "q4tp": 0.5195}[codec], "stages": spans}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("what", choices=["gemm", "attention", "rowops", "sweep", "conv", "vae", "gemma"])
    ap.add_argument("--codec", default="q4t", choices=["q8", "q4t", "q4tp"])
    ap.add_argument("--N", type=int, default=2304)
    ap.add_argument("--K", type=int, default=2304)
    ap.add_argument("--M", type=int, default=8704)
    ap.add_argument("--n", type=int, default=4352)
    ap.add_argument("--nseg", type=int, default=2)
    ap.add_argument("--rows", type=int, default=8704)
    ap.add_argument("--cols", type=int, default=2304)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--mode", type=int, default=0, help="GEMM output: 0 f32, 1 bf16, 2 fused SwiGLU pairs")
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--ic", type=int, default=128)
    ap.add_argument("--oc", type=int, default=128)
    ap.add_argument("--h", type=int, default=1024)
    ap.add_argument("--w", type=int, default=1024)
    ap.add_argument("--k", type=int, default=3)
    ap.add_argument("--planes", type=int, default=1, help="weight planes: 1 f16 kernels, 2 f32 kernels")
    ap.add_argument("--latent", type=int, default=128, help="latent height = width for the vae decode")
    a = ap.parse_args()
    gpu.set_current_device(a.device)
    if a.what == "gemm":
        print(json.dumps(gemm(a.codec, a.N, a.K, a.M, a.iters, a.mode)))
    elif a.what == "attention":
        ms = gpu.bench_attention(24, 8, 96, a.n, a.nseg, a.iters)
        fl = 4.0 * a.n * a.n * 24 * 96 * a.nseg
        print(json.dumps({"kernel": "attention", "nh": 24, "nkv": 8, "hd": 96, "n": a.n, "nseg": a.nseg, "ms": ms,
                          "tflops": fl / (ms * 1e-3) / 1e12}))
    elif a.what == "rowops":
        for kind, name in ROWOPS.items():
            ms, nb = gpu.bench_rowop(kind, a.rows, a.cols, a.iters)
            print(json.dumps({"kernel": name, "rows": a.rows, "cols": a.cols, "ms": ms, "algorithmic_bytes": nb,
                              "gbs": nb / (ms * 1e-3) / 1e9}))
    elif a.what == "conv":
        print(json.dumps(conv(a.ic, a.oc, a.h, a.w, a.k, a.planes, a.iters)))
    elif a.what == "vae":
        print(json.dumps(vae_decode(a.latent, a.iters)))
    elif a.what == "gemma":
        print(json.dumps(gemma_encode(a.n if a.n != 4352 else 128, a.codec, a.iters)))
    else:
        for codec in ("q8", "q4t", "q4tp"):
            for K, N in ((2304, 2304), (2304, 6912), (2304, 9216), (9216, 2304)):
                for M in (256, 4352, 17408):
                    print(json.dumps(gemm(codec, N, K, M, a.iters)), flush=True)


if __name__ == "__main__":
    main()
