/*
 * libcmf_cuda -- B200 (sm_100a) compute backend for the NextDiT denoiser path of the CMF
 * engine (and the prompt encoder and VAE decoder on either side of it).  Plain C ABI: pointers
 * and sizes only.  Every entry returns 0 on success or a negative status; cmfc_last_error()
 * gives the thread's last message.  Nothing throws or
 * aborts across this boundary, and nothing falls back to the CPU: an entry either ran on the
 * device or failed with a status.
 *
 * Each entry names the reference interface it replaces (paths relative to the reference
 * repository; `gpu.rs` is crates/cortiq-engine/src/gpu.rs, the engine's backend facade).
 *
 * Host pointers are borrowed for the duration of the call.  Weight bytes are copied to the
 * device once per (model, directory index) and owned by the library until cmfc_model_close;
 * a cmfc_nextdit / cmfc_gemma / cmfc_vae handle refers to those copies and must be destroyed
 * before its model is closed.
 * Calls on one device context are serialized by the caller (the engine drives a denoise from
 * one thread); the current device is selected per thread with cmfc_set_device.
 */
#ifndef CMF_CUDA_H
#define CMF_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
#define CMFC_OK 0
#define CMFC_ERR_BAD_ARG (-1)      /* null pointer, zero size, segs not summing to n ... */
#define CMFC_ERR_UNSUPPORTED (-2)  /* dtype or geometry this backend does not implement */
#define CMFC_ERR_SHAPE (-3)        /* shape disagrees with the tensor's directory record */
#define CMFC_ERR_OOM (-4)
#define CMFC_ERR_DEVICE_WAIT (-5)  /* a kernel ran out of its bounded wait budget */
#define CMFC_ERR_CUDA (-6)
#define CMFC_ERR_IO (-7)
#define CMFC_ERR_FORMAT (-8)       /* container validation failed */
#define CMFC_ERR_NOT_FOUND (-9)

/* TensorDtype ids of the container (crates/cortiq-core/src/types.rs:10-98) */
#define CMFC_DT_F32 0
#define CMFC_DT_F16 1
#define CMFC_DT_U8 6
#define CMFC_DT_Q8_ROW 3
#define CMFC_DT_Q4_TILED 11
#define CMFC_DT_Q4TP 15

typedef struct cmfc_model cmfc_model;     /* an opened, memory-mapped .cmf container */
typedef struct cmfc_nextdit cmfc_nextdit; /* a NextDiT bound to a model, weights resident */
typedef struct cmfc_vae cmfc_vae;         /* a VAE decoder bound to a model, weights resident */
typedef struct cmfc_gemma cmfc_gemma;     /* a Gemma-2 prompt encoder bound to a model, weights resident */

/* Thread-local message of the last failing call on this thread
 * (style of crates/cortiq-ffi/include/cortiq.h:5-7, cortiq_last_error). */
const char* cmfc_last_error(void);

/* ---- devices: gpu.rs:962-1013 device_count / set_current_device / with_device ---- */
int cmfc_device_count(void);
int cmfc_set_device(int device); /* creates the device context on first use */
int cmfc_synchronize(void);

/* ---- container: crates/cortiq-core/src/format.rs:390-584 CmfModel::open (envelope :653-728,
 * directory :730-791).  The file is mmap'ed; tensors are uploaded on first use. ---- */
int cmfc_model_open(const char* path, cmfc_model** out);
void cmfc_model_close(cmfc_model* m);
int64_t cmfc_model_tensor_count(const cmfc_model* m);
/* directory index of `name`, or CMFC_ERR_NOT_FOUND  (format.rs CmfModel::tensor) */
int64_t cmfc_model_find(const cmfc_model* m, const char* name);
/* directory record idx -> dtype id, ndim, shape[6], payload bytes */
int cmfc_model_tensor_info(const cmfc_model* m, int64_t idx, int* dtype, int* ndim, uint32_t shape[6],
                           uint64_t* nbytes);
/* name of directory record idx (valid until close), NULL when out of range */
const char* cmfc_model_tensor_name(const cmfc_model* m, int64_t idx);
/* pointer into the mapping (valid until close) */
const void* cmfc_model_tensor_bytes(const cmfc_model* m, int64_t idx);

/* gpu.rs:507 weight_is_resident */
int cmfc_weight_is_resident(const cmfc_model* m, int64_t idx);
/* Exact f32 dequantization of tensor idx ON THE DEVICE from the planes the GEMM reads,
 * copied to `out` [rows*cols] -- the bit-exactness check against
 * crates/cortiq-core/src/quant.rs:91-103 / :322-344 / :413-431. */
int cmfc_weight_dequant(cmfc_model* m, int64_t idx, float* out, size_t out_len);

/* ---- quantized linears: Y[b, rows] = X[b, cols] . W^T, host f32 in / out.
 * gpu.rs:1155 q8_matmat, :2358 q4t_matmat, :2439 q4tp_matmat (called from
 * crates/cortiq-engine/src/qtensor.rs:1483-1584, :1637-1710, :1806-1858). ---- */
int cmfc_q8_matmat(cmfc_model* m, int64_t idx, const float* xs, size_t b, size_t rows, size_t cols, float* out);
int cmfc_q4t_matmat(cmfc_model* m, int64_t idx, const float* xs, size_t b, size_t rows, size_t cols, float* out);
int cmfc_q4tp_matmat(cmfc_model* m, int64_t idx, const float* xs, size_t b, size_t rows, size_t cols, float* out);

/* gpu.rs:1891 dit_qkv: three projections of one input in one submission */
int cmfc_dit_qkv(cmfc_model* m, int64_t wq, int64_t wk, int64_t wv, const float* xs, size_t b, size_t hidden,
                 size_t qrows, size_t kvrows, float* q_out, float* k_out, float* v_out);

/* gpu.rs:1773-1813 q4t_ffn / q4tp_ffn: out = (silu(x W1^T) * (x W3^T)) W2^T; any of the three
 * codecs is accepted for each projection */
int cmfc_ffn(cmfc_model* m, int64_t w1, int64_t w3, int64_t w2, const float* xs, size_t b, size_t hidden,
             size_t inter, float* out);

/* gpu.rs:2332 dit_attention: q [nh][n][hd], k and v [nkv][n][hd] head-major f32 (q NOT yet
 * scaled), out [n][nh*hd]; bidirectional softmax attention, GQA.  hd <= 128 (a multiple of 32)
 * runs the flash kernel with bf16 operands; a single head wider than that (nh = nkv = 1, hd a
 * multiple of 32: the VAE's attention block, vae.rs:438) runs in f32 semantics through the
 * split-f16 GEMMs and a materialised score plane. */
int cmfc_dit_attention(const float* qh, const float* kh, const float* vh, size_t nh, size_t nkv, size_t n,
                       size_t hd, float scale, float* out);

/* gpu.rs:1819-1857 DitBlockArgs, field for field (slices become pointers; lengths are implied
 * by n / hidden / hd as documented there; gates already tanh'd).  `codec` is informational:
 * the library reads each projection's dtype from the directory and accepts q8 / q4t / q4tp in
 * any mix. */
typedef struct cmfc_dit_block_args {
    uint32_t n, hidden, inter, nh, nkv, hd;
    float eps;
    const float* rope_cos; /* [n * hd/2] */
    const float* rope_sin;
    const float *norm1, *norm2, *ffn_norm1, *ffn_norm2; /* [hidden] */
    const float *norm_q, *norm_k;                       /* [hd] */
    const float *s_msa, *gate_msa, *s_mlp, *gate_mlp;   /* [hidden]; all four NULL = unmodulated block */
    int64_t wq, wk, wv, wo, w1, w3, w2;                 /* directory indices */
    int32_t q4tp;
    int32_t resident_in;  /* hidden state is already on the device from the previous block */
    int32_t resident_out; /* leave the result on the device */
} cmfc_dit_block_args;

/* gpu.rs:1936 dit_block_seg: one adaLN block over concatenated segments; x [n, hidden] in-out
 * (ignored on the way in when resident_in, on the way out when resident_out) */
int cmfc_dit_block_seg(cmfc_model* m, const cmfc_dit_block_args* a, const uint32_t* segs, size_t nseg, float* x);
/* gpu.rs:1862 dit_chain_supported, :1873 dit_state_fetch, :1918 fused_dit_block_available */
int cmfc_dit_chain_supported(void);
int cmfc_dit_state_fetch(float* x, size_t len);
int cmfc_fused_dit_block_available(void); /* 0: the batched CFG pair is the preferred shape */

/* ---- whole forward / whole loop, device-resident (the graph of
 * crates/cortiq-engine/src/dit.rs:1201-1507 and crates/cortiq-engine/src/imagegen.rs:143-217) ---- */

/* NextDit::from_cmf (dit.rs:510-589): reads dit.config_json, resolves and uploads dit.* */
int cmfc_nextdit_create(cmfc_model* m, cmfc_nextdit** out);
void cmfc_nextdit_destroy(cmfc_nextdit* d);
/* hidden_size, cap_feat, in_channels, patch_size, num_layers, num_refiner_layers, nh, nkv */
int cmfc_nextdit_dims(const cmfc_nextdit* d, uint32_t dims[8]);

/* NextDit::refine_caption (dit.rs:1201-1226): cap [cap_n, cap_feat] -> out [cap_n, hidden] */
int cmfc_nextdit_refine_caption(cmfc_nextdit* d, const float* cap, size_t cap_n, float* out);
/* NextDit::forward_with_cap (dit.rs:1389-1507): latent [c,h,w], refined caption, t -> pred [c,h,w] */
int cmfc_nextdit_forward(cmfc_nextdit* d, const float* latent, size_t h, size_t w, const float* cap_e,
                         size_t cap_n, float t, float* pred);
/* NextDit::forward_cfg_pair (dit.rs:1238-1387) */
int cmfc_nextdit_forward_pair(cmfc_nextdit* d, const float* latent, size_t h, size_t w, const float* cap_c,
                              size_t cap_c_n, const float* cap_u, size_t cap_u_n, float t, float* pred_c,
                              float* pred_u);
/* Debug tap: copy the hidden state after joint block `layer` of the LAST forward call is not
 * kept; instead this runs forward_pair and writes x after every joint block to
 * taps [num_layers][n_c+n_u][hidden] (parity tests per block). */
int cmfc_nextdit_forward_pair_taps(cmfc_nextdit* d, const float* latent, size_t h, size_t w, const float* cap_c,
                                   size_t cap_c_n, const float* cap_u, size_t cap_u_n, float t, float* pred_c,
                                   float* pred_u, float* taps);

/* imagegen::denoise (imagegen.rs:143-217) for a BATCH of prompts on this device: every prompt's
 * cond/uncond pair rides in one tall batch with one segment per sequence.
 *   latents   [batch, c, h, w]  in: start noise, out: denoised latents
 *   cap       [batch, cap_n, cap_feat]   raw caption features (refined once inside)
 *   cap_u     [batch, cap_u_n, cap_feat] or NULL (no CFG)
 * steps / guidance_scale as GenParams (imagegen.rs:41-55); sigma shift 6.0; cfg_trunc_ratio 1 and
 * CFG normalisation on, the engine's defaults. */
int cmfc_denoise(cmfc_nextdit* d, float* latents, size_t batch, size_t h, size_t w, const float* cap, size_t cap_n,
                 const float* cap_u, size_t cap_u_n, uint32_t steps, float guidance_scale);

/* The loop's switches of GenParams (imagegen.rs:24-39).  Step i (0-based) is guided while
 * (i + 1) / steps <= cfg_trunc_ratio (f32, imagegen.rs:164); later steps run the cond branch alone
 * through the single-sequence forward (dit.rs:1389-1507), as the engine does.  With
 * cfg_normalization the guided prediction is rescaled per latent row to the cond branch's norm
 * (imagegen.rs:192-204); without it the plain u + gs (c - u) is used. */
typedef struct cmfc_gen_params {
    uint32_t steps;
    float guidance_scale;
    float cfg_trunc_ratio;     /* engine default 1.0 */
    int32_t cfg_normalization; /* engine default 1 */
} cmfc_gen_params;
int cmfc_denoise_ex(cmfc_nextdit* d, float* latents, size_t batch, size_t h, size_t w, const float* cap, size_t cap_n,
                    const float* cap_u, size_t cap_u_n, const cmfc_gen_params* params);

/* Split form of the loop for benchmarking one step with device-resident state:
 * begin uploads inputs and refines captions; step runs denoise step i (0-based) of `steps`;
 * end copies latents back.  cmfc_denoise == begin + steps x step + end. */
int cmfc_denoise_begin(cmfc_nextdit* d, const float* latents, size_t batch, size_t h, size_t w, const float* cap,
                       size_t cap_n, const float* cap_u, size_t cap_u_n, uint32_t steps, float guidance_scale);
int cmfc_denoise_begin_ex(cmfc_nextdit* d, const float* latents, size_t batch, size_t h, size_t w, const float* cap,
                          size_t cap_n, const float* cap_u, size_t cap_u_n, const cmfc_gen_params* params);
int cmfc_denoise_step(cmfc_nextdit* d, uint32_t i);
int cmfc_denoise_end(cmfc_nextdit* d, float* latents);

/* ---- Gemma-2 prompt encoder (crates/cortiq-engine/src/textenc.rs): token ids -> hidden states.
 * Projections are the container's quantized tensors (q8_row / q4_tiled / q4tp) through the dequant
 * GEMM with bf16 activations; norms in f64 statistics, RoPE, soft-capped causal attention and the
 * residual stream in f32. ---- */

/* GemmaEncoder::from_cmf (textenc.rs:172-216): reads te.config_json and the te.* tensors */
int cmfc_gemma_create(cmfc_model* m, cmfc_gemma** out);
void cmfc_gemma_destroy(cmfc_gemma* g);
/* hidden_size, num_hidden_layers, nh, nkv, head_dim, intermediate_size, vocab, sliding_window */
int cmfc_gemma_dims(const cmfc_gemma* g, uint32_t dims[8]);
/* GemmaEncoder::encode (textenc.rs:222-336).  final_out: null, or [n, hidden] final-normed states;
 * streams_out: null, or [(layers + 1), n, hidden], the residual stream entering every layer and,
 * last, the pre-final-norm stream (keep_layer_inputs).  n must be below the sliding window. */
int cmfc_gemma_encode(cmfc_gemma* g, const uint32_t* ids, size_t n, float* final_out, float* streams_out);
/* What encode_prompt hands to the denoiser (crates/cortiq-engine/src/imagegen.rs:116-139):
 * hidden_states[-2], the stream entering the last layer, [n, hidden].  The last layer is not run. */
int cmfc_gemma_caption_features(cmfc_gemma* g, const uint32_t* ids, size_t n, float* out);

/* ---- VAE decoder (crates/cortiq-engine/src/vae.rs): latents [latent_channels, h, w] at model
 * scale -> RGB [3, s*h, s*w] in [-1, 1], s = 2^(up blocks with an upsampler), 8 for FLUX.
 * f32 semantics: every GEMM operand is carried as two f16 planes (hi + lo), accumulation in f32;
 * GroupNorm statistics in f64 as in vae.rs:270-294. ---- */

/* VaeDecoder::from_cmf (vae.rs:524-548): reads vae.config_json (norm_num_groups, latent_channels,
 * scaling_factor, shift_factor) and the vae.decoder.* tensors (f16 conv kernels, f32 the rest) */
int cmfc_vae_create(cmfc_model* m, cmfc_vae** out);
void cmfc_vae_destroy(cmfc_vae* v);
/* any out pointer may be null */
int cmfc_vae_info(const cmfc_vae* v, uint32_t* latent_channels, uint32_t* upscale, float* scaling_factor,
                  float* shift_factor);
/* VaeDecoder::decode (vae.rs:637-690): host z [latent_channels, h, w] -> host out [3, s*h, s*w] */
int cmfc_vae_decode(cmfc_vae* v, const float* z, size_t h, size_t w, float* out);
/* the same on device pointers (both f32, caller-owned); returns after the stream has drained */
int cmfc_vae_decode_device(cmfc_vae* v, const float* d_z, size_t h, size_t w, float* d_out);
/* gpu::vae_conv2d (gpu.rs:2026-2046): w [oc, ic, k, k], bias [oc], x [ic, h, w_img] -> out
 * [oc, h, w_img]; k is 1 or 3, padding k/2.  Host pointers. */
int cmfc_vae_conv2d(const float* w, const float* bias, const float* x, size_t ic, size_t oc, size_t h, size_t w_img,
                    size_t k, float* out);
/* gpu::vae_upsample_conv (gpu.rs:2002-2022): nearest 2x upsampling of x [ic, h, w_img], then the
 * convolution -> out [oc, 2h, 2w_img].  ic must be a multiple of 32. */
int cmfc_vae_upsample_conv(const float* w, const float* bias, const float* x, size_t ic, size_t oc, size_t h,
                           size_t w_img, size_t k, float* out);

/* ---- quantizers on the device, byte-identical to the reference encoders
 * (crates/cortiq-cli/src/convert.rs:551-566 encode_q8_row, :597-613 encode_q4_tiled,
 * :883-992 encode_q4tp).  w [rows, cols] host f32 -> payload (host, caller-sized with
 * cmfc_payload_nbytes, crates/cortiq-core/src/quant.rs:552-613 expected_nbytes). ---- */
size_t cmfc_payload_nbytes(int dtype, size_t rows, size_t cols);
int cmfc_encode(int dtype, const float* w, size_t rows, size_t cols, uint8_t* payload);
/* same, generating w ~ N(0, std) on the device from `seed` (synthetic models for benchmarks) */
int cmfc_encode_random(int dtype, uint64_t seed, float std, size_t rows, size_t cols, uint8_t* payload);

/* ---- for callers that cannot allocate device memory ----
 * No counterpart in the reference (its backends allocate freely); added for hosts where
 * cudaMalloc is not an option at call time: code running inside another framework's memory pool,
 * latency paths that cannot afford an allocation or the device-wide synchronization of a free, or
 * deployments with a device-memory budget fixed at start-up.
 *
 * Y[b, rows] = X[b, cols] . W^T with DEVICE pointers: d_x f32 [b, cols] in, d_y f32 [b, rows]
 * out, both owned by the caller.  The bf16 staging copy of X that the tensor-core kernel needs
 * lives in a fixed 8 MiB array inside the library's device image, so b * cols must not exceed
 * cmfc_noalloc_max_elements() (4 Mi); larger calls are rejected with CMFC_ERR_SHAPE.  The entry
 * calls no cudaMalloc / cudaFree and no allocating library routine.  Preconditions: the thread
 * has a device context (cmfc_set_device) and the tensor is already resident on it (any other
 * entry uploads it; cmfc_weight_is_resident tells) -- otherwise CMFC_ERR_BAD_ARG /
 * CMFC_ERR_NOT_FOUND.  The first call on a device looks up the array's device address (and, with
 * lazy module loading, may make the driver load this library's device image, which takes device
 * memory once); make that call early, before any stream capture.  All calls on a device share the
 * array and it keeps the last call's contents; nothing in it needs clearing between calls, but two
 * calls overlapping on the GPU would race, so serialize them.
 * Ordering: the work runs on the library's own non-blocking stream (cmfc_stream_handle), which is
 * ordered after NO other stream, the legacy default stream included.  d_x must therefore be
 * complete before the call, or the caller records an event after the work that fills d_x and makes
 * the library's stream wait on it (cudaStreamWaitEvent on cmfc_stream_handle()).  The call returns
 * after the result is complete in d_y, so no ordering is needed on the way out. */
size_t cmfc_noalloc_max_elements(void);
int cmfc_matmat_device_noalloc(cmfc_model* m, int64_t idx, const float* d_x, size_t b, float* d_y);

/* ---- instrumentation ---- */
/* Exercises the failure path of the bounded device waits (no counterpart in the reference, whose
 * shaders have no waits): launches a one-block kernel that waits, with a budget of `polls` polls
 * (1 .. 65536; a poll parks for at most 8 us), on a barrier nobody arrives on.  The kernel gives
 * up, records the site and exits normally; the call returns CMFC_ERR_DEVICE_WAIT, and the context
 * remains usable for further calls.  Nothing faults or hangs. */
int cmfc_selftest_wait_timeout(uint32_t polls);
/* kernels launched by this library on the current device since the last reset */
uint64_t cmfc_launch_count(int reset);
/* Time `iters` back-to-back launches of the dequant GEMM for tensor idx at M tokens with
 * device-resident synthetic bf16 activations; mean milliseconds per launch (CUDA events on the
 * library's stream).  mode: 0 f32 out, 1 bf16 out. */
int cmfc_bench_gemm(cmfc_model* m, int64_t idx, size_t M, int mode, int iters, float* ms_per_launch);
/* Time the flash-attention kernel on synthetic bf16 inputs: nseg segments of n tokens each. */
int cmfc_bench_attention(size_t nh, size_t nkv, size_t hd, size_t n, size_t nseg, int iters, float* ms_per_launch);
/* Time a bandwidth-bound row kernel on synthetic inputs; also returns its algorithmic bytes per
 * launch.  kind: 0 modulated RMSNorm, 1 gated residual, 2 gated residual + next modulated norm
 * (one pass), 3 qk-norm + RoPE + head packing. */
int cmfc_bench_rowop(int kind, size_t rows, size_t cols, int iters, float* ms_per_launch, double* bytes_per_launch);
/* Time cmfc_gemma_caption_features on a synthetic prompt of n tokens (device work only). */
int cmfc_bench_gemma(cmfc_gemma* g, size_t n, int iters, float* ms_per_prompt);
/* Time whole VAE decodes of a synthetic latent [latent_channels, h, w] resident on the device. */
int cmfc_bench_vae_decode(cmfc_vae* v, size_t h, size_t w, int iters, float* ms_per_decode);
/* Time the implicit-GEMM convolution ic -> oc (k x k, k 1 or 3) over an h x w image of synthetic
 * split planes; a_planes 1 = f16 kernels (two MMA passes), 2 = f32 kernels (three). */
int cmfc_bench_conv(size_t ic, size_t oc, size_t h, size_t w, size_t k, int a_planes, int iters, float* ms_per_launch);
/* the cudaStream_t every kernel of the current device's context is launched on (so a caller can
 * record its own events around library work) */
void* cmfc_stream_handle(void);
/* per-stage CUDA-event times of the last cmfc_denoise_step when profiling is on
 * (categories of crates/cortiq-engine/src/dit.rs:192-217) */
int cmfc_profile_enable(int on);
int cmfc_profile_read(char* buf, size_t buflen);

#ifdef __cplusplus
}
#endif
#endif /* CMF_CUDA_H */
