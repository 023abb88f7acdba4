#!/usr/bin/env python
"""Benchmark of the NextDiT denoise step on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path (oracle port)

Metric (BASELINE.json): denoise steps/s at 1024x1024 on a Lumina-2-size (2.6 B) q4t NextDiT.
One *step* = one Euler flow-matching step for one prompt: the batched cond/uncond forward
(2 x 4352 tokens through 2 noise-refiner + 26 joint blocks), CFG combine with per-row norm
rescale, and the latent update.  Every GPU holds its own memory-mapped weight copy and runs
`--prompts-per-gpu` prompts (weak scaling, no data-path collective); `value` is steps/s summed
over all GPUs.  Inputs are synthetic (seeded N(0,1) latents and caption features, random-init
N(0, 0.02) weights quantized by the device-side encoder, which is byte-identical to the
reference quantizer).

Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "nextdit_denoise_steps_per_s_1024sq_q4t"
UNIT = "steps/s"
H = W = 128                  # latent of a 1024x1024 image
CAP_N = 256
STEP_TFLOP = 45.9            # algorithmic FLOPs of one CFG-pair step at 1024^2 (26 joint + 4 refiner blocks)


def env_int(name, default):
    try:
        return int(os.environ.get(name, default))
    except ValueError:
        return default


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"bf16_sustained": d.get("bf16_tflops_sustained"), "bf16_burst": d.get("bf16_tflops"),
                "hbm": d.get("hbm_gbs"), "source": "measured"}
    return {"bf16_sustained": 1400.0, "bf16_burst": 1590.0, "hbm": 6650.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.05 and len(r) >= 8] or \
               [r for _, r in self.rows if len(r) >= 8]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[1]) for r in rows)
        reasons = [n for i, n in ((4, "hw_slowdown"), (5, "hw_thermal_slowdown"), (6, "sw_thermal_slowdown"),
                                  (7, "sw_power_cap")) if any(r[i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "reasons": reasons, "samples": len(rows),
                "power_w_max": max(float(r[3]) for r in rows)}


def gemm_flops_per_step(cfg, n_joint, n_img):
    """FLOPs of the dequant-GEMM launches of one step (per prompt): per block 2*rows*(qkv+o+w13+w2)."""
    hs, inter = cfg["hidden_size"], cfg["inter"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_kv_heads"]
    hd = hs // nh
    per_tok = (nh + 2 * nkv) * hd * hs + hs * nh * hd + 3 * inter * hs
    return 2.0 * per_tok * (cfg["num_layers"] * n_joint + cfg["num_refiner_layers"] * n_img)


# ------------------------------------------------------------------ reference arm (CPU oracle)
def run_reference(args, rank, world):
    if rank != 0:
        return
    from oracle import codecs as oc
    from oracle import nextdit as nd
    from cmf_b200 import synth
    cfg = synth.LUMINA2
    hs = cfg["hidden_size"]
    n_img = (H // 2) * (W // 2)
    segs = [CAP_N + n_img, CAP_N + n_img]
    n = sum(segs)
    rng = np.random.default_rng(0)
    # one joint block, q4t, weights quantized by the oracle's own encoder
    t = {}
    pfx = "dit.layers.0"
    shapes = {".attn.to_q.weight": (hs, hs), ".attn.to_k.weight": (hs // 3, hs), ".attn.to_v.weight": (hs // 3, hs),
              ".attn.to_out.0.weight": (hs, hs), ".feed_forward.linear_1.weight": (cfg["inter"], hs),
              ".feed_forward.linear_3.weight": (cfg["inter"], hs), ".feed_forward.linear_2.weight": (hs, cfg["inter"])}
    for k, s in shapes.items():
        t[pfx + k] = nd.QWeight.quantize(oc.Q4_TILED, (rng.standard_normal(s) * 0.02).astype(np.float32))
    t[pfx + ".norm1.linear.weight"] = nd.QWeight.quantize(oc.Q8_ROW, (rng.standard_normal((4 * hs, 1024)) * 0.02).astype(np.float32))
    t[pfx + ".norm1.linear.bias"] = (rng.standard_normal(4 * hs) * 0.02).astype(np.float32)
    for k in (".norm1.norm.weight", ".norm2.weight", ".ffn_norm1.weight", ".ffn_norm2.weight"):
        t[pfx + k] = np.ones(hs, np.float32)
    for k in (".attn.norm_q.weight", ".attn.norm_k.weight"):
        t[pfx + k] = np.ones(hs // cfg["num_attention_heads"], np.float32)
    orc = nd.NextDitOracle(t, dict(cfg, num_layers=1, num_refiner_layers=0))
    x = rng.standard_normal((n, hs)).astype(np.float32)
    temb = rng.standard_normal(1024).astype(np.float32)
    ids = np.zeros((n, 3), np.int64)
    ids[:, 1] = np.arange(n) // 64
    ids[:, 2] = np.arange(n) % 64
    rope = nd.rope_table(ids, cfg["axes_dim_rope"])
    blocks_per_step = cfg["num_layers"] + cfg["num_refiner_layers"] * (n_img / n)
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.time()
        orc.block_forward_seg(pfx, x, rope, temb, segs)
        if i >= args.warmup:
            times.append(time.time() - t0)
    per_block = sum(times) / len(times)
    step_s = per_block * blocks_per_step
    cores = os.cpu_count() or 1
    value = 1.0 / step_s
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "lumina2-2.6B q4t 1024x1024 CFG pair, 1 prompt", "timed": "cpu"},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"one joint block over 2x{CAP_N + n_img} tokens per timed step "
                                       f"({per_block:.2f} s), extrapolated x{blocks_per_step:.1f} blocks per denoise step; "
                                       "numpy/BLAS f32 over exactly dequantized q4t weights"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ this library
def cpu_baseline_sample(cfg):
    """~10-30 s of CPU work: the oracle (numpy/BLAS over exactly dequantized weights) on one joint
    block at the full 2 x 4352 tokens, extrapolated to the blocks of one step."""
    import argparse as _a
    ns = _a.Namespace(gpus=1, steps=2, warmup=1)
    import io
    import contextlib
    buf = io.StringIO()
    with contextlib.redirect_stdout(buf):
        run_reference(ns, 0, 1)
    d = json.loads(buf.getvalue().strip().splitlines()[-1])
    return d["cpu_baseline"]


def vae_leg(args, lh, lw, peaks, cpu=True):
    """The stage after the denoiser: FLUX-class VAE decode of one latent [16, lh, lw] (synthetic
    weights of the real architecture).  Device-resident time, end-to-end time through the public
    API with host buffers, and the CPU oracle on a bounded sample."""
    from cmf_b200 import Model, VaeDecoder, gpu, synth
    from cmf_b200.microbench import vae_flops
    path = os.path.join(args.model_dir, "cmf_bench_flux_vae.cmf")
    if not os.path.exists(path):
        synth.write_vae_model(path, synth.FLUX_VAE, 0)
    z = np.random.default_rng(5).standard_normal((16, lh, lw)).astype(np.float32)
    with Model(path) as m:
        dec = VaeDecoder(m)
        dec.decode(z, lh, lw)                               # warm-up: buffers, first-use costs
        ms = gpu.bench_vae_decode(dec, lh, lw, iters=5)     # CUDA events around 5 decodes, latent resident
        t0 = time.time()
        for _ in range(3):
            img = dec.decode(z, lh, lw)
        e2e_ms = (time.time() - t0) / 3 * 1e3
        dec.close()
    fl = vae_flops(synth.FLUX_VAE, lh, lw)
    out = {"workload": f"FLUX-class VAE decoder, latent 16x{lh}x{lw} -> RGB {8 * lh}x{8 * lw}, f32 semantics "
                       "(split-f16 operands, two MMA passes per convolution)",
           "ms": ms, "images_per_s": 1e3 / ms, "conv_tflops": fl / (ms * 1e-3) / 1e12,
           "tensor_tflops": 2 * fl / (ms * 1e-3) / 1e12, "tensor_peak": peaks["bf16_sustained"],
           "e2e": {"ms": e2e_ms, "images_per_s": 1e3 / e2e_ms, "h2d_bytes": z.nbytes, "d2h_bytes": img.nbytes,
                   "call": "cmf_b200.VaeDecoder(model).decode(z, h, w) with host buffers"}}
    if cpu:
        from oracle import vae as ovae
        t = synth.vae_tensors(synth.FLUX_VAE, 0)
        sh = 16
        zs = z[:, :sh, :sh].copy()
        t0 = time.time()
        ovae.decode(t, synth.FLUX_VAE, zs)
        dt = time.time() - t0
        scale = (lh * lw) / float(sh * sh)
        out["cpu_baseline"] = {"images_per_s": 1.0 / (dt * scale), "kind": "port", "cores": os.cpu_count(),
                               "sample": f"oracle decode of a {sh}x{sh} latent crop ({dt:.2f} s, numpy f64 matmuls), "
                                         f"scaled by the pixel ratio {scale:.0f} (convolutions are linear in pixels; "
                                         "the attention block's quadratic term is left out, which favours the CPU)"}
    return out


def encoder_leg(args, cpu=True, n=128):
    """The stage before the denoiser: Gemma-2-2B prompt encoder, caption features of one prompt of
    ``n`` tokens (synthetic q4_tiled weights of the real architecture, vocabulary cut to 4096 rows)."""
    from cmf_b200 import GemmaEncoder, Model, gpu, synth
    cfg = dict(synth.GEMMA2_2B, vocab_size=4096)
    path = os.path.join(args.model_dir, "cmf_bench_gemma2_q4t.cmf")
    if not os.path.exists(path):
        synth.write_gemma_model(path, cfg, "q4t", 0)
    ids = np.random.default_rng(9).integers(0, cfg["vocab_size"], n).astype(np.uint32)
    with Model(path) as m:
        enc = GemmaEncoder(m)
        enc.caption_features(ids)
        ms = gpu.bench_gemma(enc, n, iters=5)
        t0 = time.time()
        for _ in range(5):
            feats = enc.caption_features(ids)
        e2e_ms = (time.time() - t0) / 5 * 1e3
        enc.close()
    out = {"workload": f"Gemma-2-2B encoder (25 of 26 layers: hidden_states[-2]), q4_tiled projections, {n} tokens",
           "ms": ms, "prompts_per_s": 1e3 / ms,
           "e2e": {"ms": e2e_ms, "prompts_per_s": 1e3 / e2e_ms, "h2d_bytes": int(ids.nbytes + n * 2304 + 4 * n),
                   "d2h_bytes": int(feats.nbytes), "call": "cmf_b200.GemmaEncoder(model).caption_features(ids)"}}
    if cpu:
        from oracle import gemma as og
        from tests.modelfile import load_for_oracle
        t, _ = load_for_oracle(path, cache=False)
        t0 = time.time()
        og.GemmaOracle(t, cfg).encode(ids, keep_layer_inputs=False)
        dt = time.time() - t0
        out["cpu_baseline"] = {"prompts_per_s": 1.0 / dt, "kind": "port", "cores": os.cpu_count(),
                               "sample": f"oracle encode of the same {n} tokens, all 26 layers, numpy f32 matmuls over "
                                         f"exactly dequantized weights ({dt:.2f} s)"}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--prompts-per-gpu", type=int, default=1)
    ap.add_argument("--codec", default="q4t", choices=["q4t", "q4tp", "q8", "q4tp_ffn_q8_attn"])
    ap.add_argument("--latent", type=int, default=H, help="latent side (128 = 1024x1024 image, 256 = 2048x2048)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-vae", action="store_true", help="skip the VAE-decode leg (the stage after the denoiser)")
    ap.add_argument("--model-dir", default=os.environ.get("CMF_BENCH_DIR", tempfile.gettempdir()))
    args = ap.parse_args()

    rank, world, local = env_int("RANK", 0), env_int("WORLD_SIZE", 1), env_int("LOCAL_RANK", 0)
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import cmf_b200
    from cmf_b200 import GenParams, Model, NextDit, denoise, gpu, synth

    if world > 1:
        # stdout carries exactly one JSON line: while NCCL sets itself up (its version banner goes to
        # file descriptor 1) stdout is pointed at stderr, then restored
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        torch.cuda.set_device(local)
        sys.stdout.flush()
        saved_fd = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
            dist.barrier()          # creates the communicator now
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved_fd, 1)
            os.close(saved_fd)
    gpu.set_current_device(local)
    cfg = synth.LUMINA2
    attn, ffn = {"q4t": ("q4t", "q4t"), "q4tp": ("q4tp", "q4tp"), "q8": ("q8", "q8"),
                 "q4tp_ffn_q8_attn": ("q8", "q4tp")}[args.codec]
    path = os.path.join(args.model_dir, f"cmf_bench_lumina2_{args.codec}.cmf")
    # rank 0 writes the container once; every rank memory-maps the same file and uploads its own copy
    if rank == 0 and not os.path.exists(path):
        synth.write_model(path, cfg, attn=attn, ffn=ffn, seed=0)
    if world > 1:
        dist.barrier()
    model = Model(path)
    dit = NextDit(model)

    P = args.prompts_per_gpu
    LH = LW = args.latent
    rng = np.random.default_rng(1000 + rank)
    pin = lambda a: torch.from_numpy(a).pin_memory().numpy()
    lat = pin(rng.standard_normal((P, 16, LH, LW)).astype(np.float32))
    cap = pin(rng.standard_normal((P, CAP_N, cfg["cap_feat"])).astype(np.float32))
    cap_u = pin(rng.standard_normal((P, CAP_N, cfg["cap_feat"])).astype(np.float32))
    total_steps = 30
    K, Wm = args.steps, args.warmup
    n_img = (LH // 2) * (LW // 2)
    n_joint = 2 * (CAP_N + n_img)
    step_tflop = (gemm_flops_per_step(cfg, n_joint, n_img) + 4.0 * 2304 * (26 * 2 * (CAP_N + n_img) ** 2 + 2 * n_img ** 2)) / 1e12

    stream = torch.cuda.ExternalStream(gpu.stream_handle(), device=torch.device("cuda", local))

    def sync_all():
        gpu.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    # ---- device-resident steps: inputs already in HBM when the timed region starts ----
    dit.denoise_begin(lat, cap, cap_u, max(total_steps, K + Wm), 4.0)
    for i in range(Wm):
        dit.denoise_step(i)
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.12)
    gpu.launch_count(reset=True)
    gpu.profile_enable(True)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_wall0 = time.time()
    e0.record(stream)
    for i in range(Wm, Wm + K):
        dit.denoise_step(i)
    e1.record(stream)
    sync_all()
    t_wall1 = time.time()
    launches = gpu.launch_count()
    prof = gpu.profile_read()
    gpu.profile_enable(False)
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1)], device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms_total = float(ms.item())
    final = dit.denoise_end()
    assert np.isfinite(final).all()

    # ---- end to end through the public API: host buffers in, host buffers out ----
    def e2e_call(steps):
        out_ = denoise(dit, lat, cap, cap_u, GenParams(steps=steps, guidance_scale=4.0))
        if world > 1:
            # the one collective of the path: gather the final latents on rank 0 over NCCL
            from cmf_b200.shard import gather_latents
            gathered = gather_latents(out_, world * P, device=f"cuda:{local}")
            torch.cuda.synchronize()
            assert rank != 0 or gathered.shape[0] == world * P
        return out_

    e2e_call(1)  # untimed: first-use costs of the gather (peer connections) stay out of the number
    sync_all()
    t0 = time.time()
    out = e2e_call(K)
    e2e_s = torch.tensor([time.time() - t0], device=f"cuda:{local}")
    if world > 1:
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_s = float(e2e_s.item())
    h2d = lat.nbytes + cap.nbytes + cap_u.nbytes
    d2h = out.nbytes

    if rank == 0:
        peaks = load_peaks()
        value = world * P * K / (ms_total * 1e-3)
        gemm_ms = sum(prof.get(k, {}).get("ms", 0.0) for k in ("qkv-proj", "o-proj", "ffn-mm"))
        gemm_launches = sum(prof.get(k, {}).get("spans", 0) for k in ("qkv-proj", "o-proj")) + 2 * prof.get("ffn-mm", {}).get("spans", 0)
        gemm_tflop = gemm_flops_per_step(cfg, n_joint, n_img) * P * K / 1e12
        achieved = gemm_tflop / (gemm_ms * 1e-3) if gemm_ms else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": ms_total / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"lumina2-2.6B {args.codec} NextDiT, {8 * LH}x{8 * LW} (latent {LH}x{LW}), CFG pair "
                                   f"(2 x {CAP_N + n_img} tokens), {P} prompt(s) per GPU, Euler step incl. CFG combine",
                       "prompts_per_gpu": P, "parallelism": f"replicas x{world}, prompts sharded, no per-step collective",
                       "l2": "per-step working set (activations > 300 MB plus 1.5 GB of weights) exceeds the 126 MB L2"},
            "tflops_per_gpu": step_tflop * P * K / (ms_total * 1e-3),
            "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": world * P * K / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d / K, "d2h_bytes_per_step": d2h / K,
                    "call": "cmf_b200.denoise(dit, latents, cap, cap_u, GenParams(steps=K)) with pinned host buffers"
                            + ("; + NCCL gather of final latents to rank 0" if world > 1 else "")},
            "roofline": {"kernel": "gemm_dequant_pair_kernel (q4 nibble planes -> bf16 in TMEM -> tcgen05.mma.cta_group::2)",
                         "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
                         "frac": (achieved / peaks["bf16_sustained"]) if achieved else None,
                         "peak_source": peaks["source"] + " (sustained cuBLAS bf16)",
                         "launches_timed": gemm_launches, "traffic": None},
            "stage_ms_per_step": {k: v["ms"] / K for k, v in prof.items()},
        }
        if world == 1 and not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = cpu_baseline_sample(cfg)
            except Exception as e:  # the baseline is a reported figure; its failure must not hide the GPU line
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                                        "sample": f"failed: {e!r}"}
        if world == 1 and not args.no_vae:
            try:
                line["vae_decode"] = vae_leg(args, LH, LW, peaks, cpu=not args.no_cpu_baseline)
            except Exception as e:  # a secondary figure: never hide the headline line
                line["vae_decode"] = {"failed": repr(e)}
        if world == 1 and not args.no_vae:
            try:
                line["prompt_encode"] = encoder_leg(args, cpu=not args.no_cpu_baseline)
            except Exception as e:
                line["prompt_encode"] = {"failed": repr(e)}
        if args.codec in ("q4t", "q4tp"):
            # dram__bytes_read.sum + dram__bytes_write.sum of one captured launch of this kernel, the
            # gate/up GEMM of a block (N=18432, K=2304, M=8704, SwiGLU epilogue; algorithmic 224 MB; pair kernel):
            # profiles/gemm_dequant_q4t_swiglu_N18432_K2304_M8704.md
            line["roofline"]["traffic"] = 195.5e6
            line["roofline"]["traffic_launch"] = "gate/up GEMM of one block, N=18432 K=2304 M=8704"
        print(json.dumps(line), flush=True)
    dit.close()
    model.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
