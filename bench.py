#!/usr/bin/env python
"""Benchmark of the NextDiT denoise step on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # the reference's CPU path (oracle port)

Metric: denoise steps/s at 1024x1024 on a Lumina-2-size (2.6 B) q4_tiled NextDiT.  One *step* = one
Euler flow-matching step for one prompt: the batched cond/uncond forward (2 x 4352 tokens through
2 noise-refiner + 26 joint blocks), CFG combine with per-row norm rescale, and the latent update.
Every GPU holds its own memory-mapped weight copy and runs `--prompts-per-gpu` prompts (weak
scaling, no data-path collective); `value` is steps/s summed over all GPUs.  Inputs are synthetic
(seeded N(0,1) latents and caption features, random-init N(0, 0.02) weights quantized by the
device-side encoder, which is byte-identical to the reference quantizer).

Beside the headline the line carries `fixed_batch`: a FIXED batch of 8 prompts (q4tp feed-forward +
q8 attention weights, seeds 0..7) split over the N GPUs with one gather of the final latents, so
that the ratio of its `value` between N = 1 and N = 8 is the strong-scaling factor of the batched
CFG workload; with two or more GPUs also `fixed_batch_2048` (16 prompts at 2048x2048, q4_tiled); on one
GPU also `q8_30_steps` (q8_row weights, one prompt, the whole 30-step loop through the public call).

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


def workload_name(codec, latent, prompts_per_gpu):
    """One string for both arms: the reference arm times the same workload on the host cores."""
    n_img = (latent // 2) ** 2
    return (f"lumina2-2.6B {codec} NextDiT, {8 * latent}x{8 * latent} (latent {latent}x{latent}), CFG pair "
            f"(2 x {CAP_N + n_img} tokens), {prompts_per_gpu} prompt(s) per GPU, Euler step incl. CFG combine")


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
def host_threads():
    """All host cores this process may use, whatever the launcher put into OMP_NUM_THREADS
    (torch.distributed.run exports OMP_NUM_THREADS=1, which would throttle BLAS and OpenMP)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference(args, rank, world, emit=True):
    """The reference's CPU implementation of the path, restated (oracle/): one joint block over the
    full token count per timed step, extrapolated to the blocks of a denoise step.  Linears run as
    numpy/BLAS f32 matmuls over exactly dequantized weights (faster than the reference's strict
    scalar kernels, which are timed beside it on one projection: this favours the CPU)."""
    if rank != 0:
        return None
    from threadpoolctl import threadpool_info, threadpool_limits
    from oracle import codecs as oc
    from oracle import nextdit as nd
    from cmf_b200 import synth
    cfg = synth.LUMINA2
    hs = cfg["hidden_size"]
    latent, P = args.latent, args.prompts_per_gpu
    n_img = (latent // 2) * (latent // 2)
    segs = [CAP_N + n_img, CAP_N + n_img]
    n = sum(segs)
    attn_dt, ffn_dt = {"q4t": (oc.Q4_TILED, oc.Q4_TILED), "q4tp": (oc.Q4TP, oc.Q4TP), "q8": (oc.Q8_ROW, oc.Q8_ROW),
                       "q4tp_ffn_q8_attn": (oc.Q8_ROW, oc.Q4TP)}[args.codec]
    threads = host_threads()
    oc.num_threads()                      # loads the oracle's library (and its OpenMP runtime) before the limits are set
    np.ones((2, 2), np.float32) @ np.ones((2, 2), np.float32)
    with threadpool_limits(limits=threads):
        used = sorted({(i.get("user_api"), i.get("num_threads")) for i in threadpool_info()})
        omp_threads = oc.num_threads()
        rng = np.random.default_rng(0)
        # one joint block, weights quantized by the oracle's own encoders
        t = {}
        pfx = "dit.layers.0"
        shapes = {".attn.to_q.weight": (hs, hs), ".attn.to_k.weight": (hs // 3, hs), ".attn.to_v.weight": (hs // 3, hs),
                  ".attn.to_out.0.weight": (hs, hs), ".feed_forward.linear_1.weight": (cfg["inter"], hs),
                  ".feed_forward.linear_3.weight": (cfg["inter"], hs), ".feed_forward.linear_2.weight": (hs, cfg["inter"])}
        for k, sh in shapes.items():
            t[pfx + k] = nd.QWeight.quantize(attn_dt if ".attn." in k else ffn_dt, (rng.standard_normal(sh) * 0.02).astype(np.float32))
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
        # the reference's strict scalar kernel (crates/cortiq-engine/src/qtensor.rs:4418-4432 and twins)
        # on one projection and a bounded row count, OpenMP over weight rows
        q = t[pfx + ".attn.to_q.weight"]
        rows_s = 512
        t0 = time.time()
        oc.matmat_exact(q.dtype, q.payload, q.rows, q.cols, x[:rows_s])
        strict_s = time.time() - t0
    per_block = sum(times) / len(times)
    step_s = per_block * blocks_per_step * P
    value = 1.0 / (per_block * blocks_per_step)          # prompt-steps per second
    strict_gflops = 2.0 * rows_s * q.rows * q.cols / strict_s / 1e9
    blas_gflops = gemm_flops_per_step(dict(cfg, num_layers=1, num_refiner_layers=0), n, 0) / per_block / 1e9
    baseline = {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                "threads": {"blas_openmp_pools": used, "oracle_openmp": omp_threads},
                "extrapolated": True, "blocks_timed": len(times), "blocks_per_step": blocks_per_step,
                "linears": "numpy/BLAS sgemm over exactly dequantized weights (the figure the ratio uses)",
                "strict_kernel": {"what": f"oracle strict scalar kernel, to_q {q.rows}x{q.cols}, {rows_s} token rows, OpenMP",
                                  "seconds": strict_s, "gflops": strict_gflops,
                                  "blas_block_gflops_incl_attention_and_norms": blas_gflops},
                "sample": f"one joint block over 2x{CAP_N + n_img} tokens per timed step ({per_block:.2f} s, "
                          f"{len(times)} timed), extrapolated x{blocks_per_step:.1f} blocks per denoise step; "
                          f"numpy/BLAS f32 over exactly dequantized {args.codec} weights, {threads} threads"}
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "extrapolated": True,
            "config": {"workload": workload_name(args.codec, latent, P), "prompts_per_gpu": P, "timed": "cpu"},
            "cpu_baseline": baseline,
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if emit:
        print(json.dumps(line), flush=True)
    return line


# ------------------------------------------------------------------ this library
def cpu_baseline_sample(args):
    """~10-30 s of CPU work: the oracle (numpy/BLAS over exactly dequantized weights) on one joint
    block at the full token count, extrapolated to the blocks of one step."""
    import argparse as _a
    ns = _a.Namespace(gpus=1, steps=2, warmup=1, latent=args.latent, prompts_per_gpu=args.prompts_per_gpu, codec=args.codec)
    return run_reference(ns, 0, 1, emit=False)["cpu_baseline"]


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


def prompt_inputs(indices, latent, cap_feat, seed_base):
    """Seeded synthetic inputs of prompts `indices` (same arrays on whichever rank builds them):
    start noise by the engine's generator (SplitMix64 + Box-Muller, imagegen.rs:75-108) from seed
    seed_base + j, caption features ~ N(0, 1)."""
    import torch
    from cmf_b200.imagegen import gauss_latent
    lat = np.stack([gauss_latent(16 * latent * latent, seed_base + j).reshape(16, latent, latent) for j in indices])
    cap, cap_u = [], []
    for j in indices:
        rng = np.random.default_rng(seed_base + j)
        cap.append(rng.standard_normal((CAP_N, cap_feat), dtype=np.float32))
        cap_u.append(rng.standard_normal((CAP_N, cap_feat), dtype=np.float32))
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a, np.float32)).pin_memory().numpy()
    return pin(lat), pin(np.stack(cap)), pin(np.stack(cap_u))


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
    ap.add_argument("--no-vae", action="store_true", help="skip the VAE-decode and prompt-encoder legs (the stages around the denoiser)")
    ap.add_argument("--no-fixed-batch", action="store_true", help="skip the fixed-batch (strong scaling) legs")
    ap.add_argument("--fixed-prompts", type=int, default=8, help="prompts of the fixed batch split over the GPUs")
    ap.add_argument("--fixed-steps", type=int, default=4, help="timed steps of the fixed-batch legs")
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
    from cmf_b200.shard import denoise_sharded, shard_range

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
    dev = f"cuda:{local}"
    cfg = synth.LUMINA2
    codec_pair = {"q4t": ("q4t", "q4t"), "q4tp": ("q4tp", "q4tp"), "q8": ("q8", "q8"), "q4tp_ffn_q8_attn": ("q8", "q4tp")}

    def open_model(codec):
        attn, ffn = codec_pair[codec]
        path = os.path.join(args.model_dir, f"cmf_bench_lumina2_{codec}.cmf")
        # rank 0 writes the container once; every rank memory-maps the same file and uploads its own copy
        if rank == 0 and not os.path.exists(path):
            synth.write_model(path, cfg, attn=attn, ffn=ffn, seed=0)
        if world > 1:
            dist.barrier()
        m = Model(path)
        return m, NextDit(m)

    model, dit = open_model(args.codec)
    stream = torch.cuda.ExternalStream(gpu.stream_handle(), device=torch.device("cuda", local))

    def sync_all():
        gpu.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    def max_over_ranks(v):
        t = torch.tensor([float(v)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ranks_ok(ok):
        t = torch.tensor([1.0 if ok else 0.0], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return float(t.item()) > 0.5

    def timed_steps(d, first, count):
        """`count` graph-replayed steps starting at index `first`: CUDA events on the library's stream
        between barriers, max over ranks (milliseconds)."""
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for i in range(first, first + count):
            d.denoise_step(i)
        e1.record(stream)
        sync_all()
        return max_over_ranks(e0.elapsed_time(e1))

    P = args.prompts_per_gpu
    LH = LW = args.latent
    total = world * P
    my = list(range(rank * P, rank * P + P))
    lat, cap, cap_u = prompt_inputs(my, LH, cfg["cap_feat"], 1000)
    K, Wm = args.steps, args.warmup
    n_img = (LH // 2) * (LW // 2)
    n_joint = 2 * (CAP_N + n_img)
    step_tflop = (gemm_flops_per_step(cfg, n_joint, n_img) + 4.0 * 2304 * (26 * 2 * (CAP_N + n_img) ** 2 + 2 * n_img ** 2)) / 1e12

    # ---- device-resident steps on the production path (CUDA-graph replay, stage profiler off):
    # inputs already in HBM when the timed region starts ----
    dit.denoise_begin(lat, cap, cap_u, max(30, 2 * K + Wm + 2), 4.0)
    for i in range(Wm):
        dit.denoise_step(i)          # step 0 runs launch by launch, step 1 captures the graph, later ones replay it
    sync_all()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.12)
    gpu.launch_count(reset=True)
    t_wall0 = time.time()
    ms_total = timed_steps(dit, Wm, K)
    t_wall1 = time.time()
    launches = gpu.launch_count()
    clocks = sampler.stop(t_wall0, t_wall1) if rank == 0 else None
    # ---- the same K steps once more, launch by launch with a CUDA-event span around every stage:
    # per-stage times and the dequant GEMM's achieved rate (this pass is not the reported `value`) ----
    gpu.profile_enable(True)
    ms_profiled = timed_steps(dit, Wm + K, K)
    prof = gpu.profile_read()
    gpu.profile_enable(False)
    final = dit.denoise_end()
    assert np.isfinite(final).all()

    # ---- end to end through the public API: pinned host buffers in, host buffers out; with several
    # GPUs every rank holds the full batch's inputs and denoise_sharded runs its shard and gathers ----
    if world > 1:
        f_lat, f_cap, f_cap_u = prompt_inputs(list(range(total)), LH, cfg["cap_feat"], 1000)
    else:
        f_lat, f_cap, f_cap_u = lat, cap, cap_u

    def e2e_call(steps):
        return denoise_sharded(dit, f_lat, f_cap, f_cap_u, GenParams(steps=steps, guidance_scale=4.0), device=dev)

    e2e_call(1)  # untimed: first-use costs of the gather (peer connections) stay out of the number
    sync_all()
    t0 = time.time()
    out = e2e_call(K)
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.time() - t0)
    h2d = world * (lat.nbytes + cap.nbytes + cap_u.nbytes)
    d2h = world * lat.nbytes
    gather_checked = None
    if rank == 0:
        # the gathered latents are, prompt for prompt, what one GPU computes alone: recompute the last
        # rank's first prompt here for the same K steps (a prompt's result does not depend on its batch)
        j = shard_range(total, world, world - 1)[0]
        alone = denoise(dit, f_lat[j:j + 1], f_cap[j:j + 1], f_cap_u[j:j + 1], GenParams(steps=K, guidance_scale=4.0))
        dev_ = float(np.linalg.norm(alone[0].astype(np.float64) - out[j]) / np.linalg.norm(alone[0].astype(np.float64)))
        assert dev_ < 1e-5, f"gathered latent of prompt {j} differs from the single-GPU result: {dev_}"
        gather_checked = {"prompt": j, "rel_l2": dev_, "steps": K}

    line = None
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
            "config": {"workload": workload_name(args.codec, LH, P),
                       "prompts_per_gpu": P, "parallelism": f"replicas x{world}, prompts sharded, no per-step collective",
                       "timed": "CUDA-graph replay of the step, stage profiler off",
                       "l2": "per-step working set (activations > 300 MB plus 1.5 GB of weights) exceeds the 126 MB L2"},
            "tflops_per_gpu": step_tflop * P * K / (ms_total * 1e-3),
            "clocks": clocks, "gpu_launches": launches,
            "e2e": {"value": world * P * K / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d / K, "d2h_bytes_per_step": d2h / K,
                    "call": "cmf_b200.shard.denoise_sharded(dit, latents, cap, cap_u, GenParams(steps=K)) with pinned host "
                            "buffers (= cmf_b200.denoise on one GPU)"
                            + ("; includes the NCCL gather of the final latents to rank 0" if world > 1 else ""),
                    "gather_checked": gather_checked is not None, "gather_check": gather_checked},
            "roofline": {"kernel": "gemm_dequant_pair_kernel (q4 nibble planes -> bf16 in TMEM -> tcgen05.mma.cta_group::2)",
                         "bound": "tensor", "achieved": achieved, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
                         "frac": (achieved / peaks["bf16_sustained"]) if achieved else None,
                         "peak_source": peaks["source"] + " (sustained cuBLAS bf16)",
                         "launches_timed": gemm_launches,
                         "timed": "CUDA-event spans around the GEMM launches in a second, launch-by-launch pass of K steps",
                         "traffic": None},
            "profiled_pass": {"ms_per_step": ms_profiled / K, "note": "launch by launch with event spans; not the reported value"},
            "stage_ms_per_step": {k: v["ms"] / K for k, v in prof.items()},
        }
        if args.codec in ("q4t", "q4tp"):
            # dram__bytes_read.sum + dram__bytes_write.sum of one captured launch of this kernel, the
            # gate/up GEMM of a block (N=18432, K=2304, M=8704, SwiGLU epilogue; algorithmic 224 MB; pair kernel)
            line["roofline"]["traffic"] = 199.1e6
            line["roofline"]["traffic_launch"] = "gate/up GEMM of one block, N=18432 K=2304 M=8704"
            line["roofline"]["traffic_source"] = ("ncu capture of one launch, profiles/gemm_dequant_q4t_swiglu_N18432_K2304_M8704.md; "
                                                  "a constant, not measured by this run")

    # ---- fixed batch split over the GPUs (strong scaling): 8 prompts, q4tp FFN + q8 attention ----
    def fixed_batch_leg(codec, latent, n_prompts, steps, d=None):
        """n_prompts prompts (seeds 0 .. n_prompts-1) split with shard_range over the ranks: device-timed
        prompt-steps/s of the whole job, then the end-to-end call with the gather, checked on rank 0."""
        res = {"workload": f"lumina2-2.6B {codec} NextDiT, {8 * latent}x{8 * latent}, {n_prompts} prompts x CFG pair split over "
                           f"{world} GPU(s), seeds 0..{n_prompts - 1}", "total_prompts": n_prompts, "steps": steps, "unit": "prompt-steps/s"}
        own_model = None
        ok, err = True, None
        try:
            if d is None:
                own_model, d = open_model(codec)
            lo, hi = shard_range(n_prompts, world, rank)
            f_l, f_c, f_u = prompt_inputs(list(range(n_prompts)), latent, cfg["cap_feat"], 0)
            if hi > lo:
                d.denoise_begin(f_l[lo:hi], f_c[lo:hi], f_u[lo:hi], max(30, steps + 3), 4.0)
                for i in range(3):
                    d.denoise_step(i)
        except Exception as e:  # noqa: BLE001
            ok, err = False, repr(e)
        if not all_ranks_ok(ok):            # every rank learns of a failure before any collective
            res["failed"] = err or "another rank failed"
            return res
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if hi > lo:
            for i in range(3, 3 + steps):
                d.denoise_step(i)
        e1.record(stream)
        sync_all()
        ms = max_over_ranks(e0.elapsed_time(e1))
        if hi > lo:
            d.denoise_end()
        gp = GenParams(steps=steps, guidance_scale=4.0)
        denoise_sharded(d, f_l, f_c, f_u, GenParams(steps=1, guidance_scale=4.0), device=dev)
        sync_all()
        t0 = time.time()
        full = denoise_sharded(d, f_l, f_c, f_u, gp, device=dev)
        torch.cuda.synchronize()
        e2e = max_over_ranks(time.time() - t0)
        res.update({"value": n_prompts * steps / (ms * 1e-3), "ms_per_step": ms / steps,
                    "prompts_per_gpu": [shard_range(n_prompts, world, r)[1] - shard_range(n_prompts, world, r)[0] for r in range(world)],
                    "e2e": {"value": n_prompts * steps / e2e, "unit": "prompt-steps/s",
                            "call": "cmf_b200.shard.denoise_sharded with pinned host buffers, gather of the final latents included"}})
        if rank == 0:
            j = shard_range(n_prompts, world, world - 1)[0]
            alone = denoise(d, f_l[j:j + 1], f_c[j:j + 1], f_u[j:j + 1], gp)
            dv = float(np.linalg.norm(alone[0].astype(np.float64) - full[j]) / np.linalg.norm(alone[0].astype(np.float64)))
            res["gather_checked"] = bool(dv < 1e-5)
            res["gather_check"] = {"prompt": j, "rel_l2": dv}
        if own_model is not None:
            d.close()
            own_model.close()
        return res

    def full_loop_leg(codec, steps):
        """One prompt, CFG pair, the whole Euler loop of `steps` steps through cmf_b200.denoise with pinned host
        buffers in and out (q8_row weights on every projection: the largest weight footprint of the three codecs)."""
        res = {"workload": f"lumina2-2.6B {codec} NextDiT, {8 * H}x{8 * H}, 1 prompt x CFG pair, {steps} Euler steps, 1 GPU",
               "steps": steps, "unit": UNIT}
        try:
            m8, d8 = open_model(codec)
            f_l, f_c, f_u = prompt_inputs([0], H, cfg["cap_feat"], 0)
            gp = GenParams(steps=steps, guidance_scale=4.0)
            denoise(d8, f_l, f_c, f_u, GenParams(steps=2, guidance_scale=4.0))   # warm-up: upload, workspaces, capture
            torch.cuda.synchronize()
            t0 = time.time()
            out = denoise(d8, f_l, f_c, f_u, gp)
            torch.cuda.synchronize()
            dt = time.time() - t0
            res.update({"value": steps / dt, "ms_per_step": dt / steps * 1e3, "loops_per_s": 1.0 / dt,
                        "finite": bool(np.isfinite(out).all()),
                        "timed": "wall clock around the public call, host buffers in and out, loop set-up (caption "
                                 "refiner, RoPE tables, graph capture) included"})
            d8.close()
            m8.close()
        except Exception as e:  # noqa: BLE001  (a secondary figure: never hide the headline line)
            res["failed"] = repr(e)
        return res

    if not args.no_fixed_batch:
        fb = fixed_batch_leg("q4tp_ffn_q8_attn", H, args.fixed_prompts, args.fixed_steps)
        if rank == 0:
            line["fixed_batch"] = fb
        if world == 1 and args.codec == "q4t":
            line["q8_30_steps"] = full_loop_leg("q8", 30)
        if world > 1 and args.codec == "q4t":
            fb2 = fixed_batch_leg("q4t", 256, 16, 2, d=dit)
            if rank == 0:
                line["fixed_batch_2048"] = fb2

    if rank == 0:
        peaks = load_peaks()
        if world == 1 and not args.no_cpu_baseline:
            try:
                line["cpu_baseline"] = cpu_baseline_sample(args)
            except Exception as e:  # the baseline is a reported figure; its failure must not hide the GPU line
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": host_threads(), "kind": "port",
                                        "sample": f"failed: {e!r}"}
        if world == 1 and not args.no_vae:
            try:
                line["vae_decode"] = vae_leg(args, LH, LW, peaks, cpu=not args.no_cpu_baseline)
            except Exception as e:  # a secondary figure: never hide the headline line
                line["vae_decode"] = {"failed": repr(e)}
            try:
                line["prompt_encode"] = encoder_leg(args, cpu=not args.no_cpu_baseline)
            except Exception as e:
                line["prompt_encode"] = {"failed": repr(e)}
        print(json.dumps(line), flush=True)
    dit.close()
    model.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
