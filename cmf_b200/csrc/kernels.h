// Launchers of the device kernels (device pointers, explicit stream).  Host-callable; the C ABI
// in api.cu composes them.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cmfc {

// ---------------- dequant GEMM (gemm_dequant.cu) ----------------
enum GemmMode : int { GEMM_OUT_F32 = 0, GEMM_OUT_BF16 = 1, GEMM_OUT_SWIGLU = 2, GEMM_OUT_GEGLU = 3 };

struct GemmParams {
    int M, N, K;             // tokens, weight rows, reduction
    void* out;               // [M, ldo] f32 or bf16; SWIGLU / GEGLU write [M, N/2] bf16
    int ldo;
    int mode;
    const float* row_scale;  // q8 only: [N]
    uint32_t* status;        // device word; a kernel that ran out of wait budget records the site
    // pair kernel, f32 output only: the tiles of a mostly empty last wave (of every prompt of the
    // batch, see gemm_dequant_pair.cu) are cut along K into slices that spread over all CTA pairs; the
    // slices' partial sums land here ([slot][256 tokens][256 rows] f32, gemm_pair_splitk_bytes() in all)
    // and a second kernel adds them in slice order.  split_period_tokens: tokens of one prompt when the
    // launch is a stack of equal prompts (each a multiple of 256 tokens), 0 = the launch is one period.
    float* splitk_ws = nullptr;
    int split_period_tokens = 0;
    // pair kernel, SwiGLU / GeGLU modes: the epilogue stages each chunk in shared memory and a TMA store
    // writes it out (tm_out of launch_gemm_dequant_pair: bf16 [M, N/2], boxes of 32 tokens x 16 channels)
    int tma_out = 0;
    // f32 output of a fused QKV projection: weight rows >= vt_row0 are V channels and are written
    // as bf16 rows of V^T [N - vt_row0, vt_pitch] instead (token m of segment z at column
    // seg_table[nseg + 1 + z] + m - seg_table[z]); the f32 columns of those rows are left untouched.
    // vt == nullptr: plain output.  vt_row0 must be a multiple of 32.
    __nv_bfloat16* vt = nullptr;
    int vt_row0 = 0, vt_pitch = 0, nseg = 0;
    const int* seg_table = nullptr;  // device: [nseg + 1] token offsets, then [nseg] first V^T columns
};
constexpr size_t GEMM_SPLITK_SLOT_BYTES = 256 * 256 * 4;

int gemm_smem_bytes();
int gemm_tile_tokens();  // rows of the activation TMA box
int launch_gemm_dequant(int wkind, const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_s,
                        const GemmParams& p, int num_sms, cudaStream_t stream);

// The same GEMM on CTA pairs (gemm_dequant_pair.cu): tiles of 256 weight rows x 256 tokens, each CTA
// staging half of the activation tile.  Needs N % 256 == 0; tm_x must have a box of
// gemm_pair_tile_tokens() rows.
bool gemm_pair_supported(const GemmParams& p);
int gemm_pair_tile_tokens();
// bytes of GemmParams::splitk_ws this launch would use (0: the launch is not split)
size_t gemm_pair_splitk_bytes(const GemmParams& p, int num_sms, int period_tokens);
int launch_gemm_dequant_pair(int wkind, const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_s,
                             const CUtensorMap& tm_out, const GemmParams& p, int num_sms, cudaStream_t stream);


// ---------------- flash attention (attention.cu) ----------------
struct AttnParams {
    int nh, nkv, hd;         // hd must be a multiple of 32, <= 128
    int n_total;             // rows of q/k (all segments)
    int vt_pitch;            // elements per row of V^T (>= n_total, multiple of 8)
    const int* seg_start;    // [nseg+1] device, token offsets
    int nseg;
    int max_seg;             // longest segment (grid sizing)
    float scale;             // 1/sqrt(hd)
    __nv_bfloat16* out;      // [n_total, nh*hd]
    uint32_t* status;
    // Prologue form (q_raw != nullptr): the query tiles are not fetched as finished bf16 rows by TMA;
    // the kernel reads the raw f32 projection rows q_raw [n_total, ld_q] (head h at column h*hd),
    // applies the per-head RMS norm (eps 1e-5, weight norm_q [hd]) and the interleaved-pair rotation
    // with cos / sin [n_total, hd/2] f32, and writes the bf16 tile into shared memory itself.
    const float* q_raw = nullptr;
    int ld_q = 0;
    const float* norm_q = nullptr;
    const float* cos_t = nullptr;
    const float* sin_t = nullptr;
    // Bounded form (score_ref > 0).  The caller guarantees two things: the query rows are already
    // multiplied by scale * log2(e) (`scale` is then ignored), and every score of the launch lies
    // within +-score_ref, max |q_i| * max |k_j| <= score_ref <= ATTN_MAX_SCORE_REF.  The kernel then
    // takes P = exp2(S) straight from the MMA result: between 2^-96 and 2^96 nothing overflows or
    // vanishes in f32 / bf16 (a row sum stays below 2^96 times the key count, O below that times
    // |v|), softmax does not depend on the reference, and P and the row sum are floating point, so no
    // row maximum, no subtraction and no rescaling of O are needed.
    // 0: unknown bound; the kernel scales the scores itself and tracks the running row maximum.
    float score_ref = 0.0f;
    // Decision on the device (norm2_max != nullptr): the caller could not bound the scores from the norm
    // gains alone, measured the largest squared norms of the finished (pre-scaled) query heads and of the
    // key heads of this launch's inputs into norm2_max[0] / [1] (float bits), and launches BOTH forms;
    // every CTA of the form that does not apply returns at once: the bounded form runs when
    // sqrt(norm2_max[0] * norm2_max[1]) <= ATTN_MAX_SCORE_REF, the tracking form otherwise.
    const unsigned* norm2_max = nullptr;
};
constexpr float ATTN_MAX_SCORE_REF = 96.0f;
int attn_smem_bytes(int hd);
int attn_key_tile(int hd);  // keys per K tile: the row count of the K tensor map's box
int launch_attention(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_vt,
                     const AttnParams& p, cudaStream_t stream);

// ---------------- codecs (codec_kernels.cu) ----------------
// raw container payloads -> GEMM planes
void launch_q4t_split(const uint8_t* raw, int rows, int cols, uint8_t* nib, float* scales_t, cudaStream_t s);
void launch_q4tp_scales(const uint8_t* codes, int code_stride, const float* ladders /*[rows,32]*/, int rows,
                        int gpr, float* scales_t, cudaStream_t s);
void launch_f16_to_f32(const uint16_t* h, float* out, int n, cudaStream_t s);
// planes -> exact f32 weights [rows, cols] (the bit-exactness check)
void launch_dequant_q8(const int8_t* q, const float* row_scale, int rows, int cols, float* out, cudaStream_t s);
void launch_dequant_q4(const uint8_t* nib, const float* scales_t, int rows, int cols, int split_scales, float* out,
                       cudaStream_t s);
// in place: container nibble order -> GEMM plane order (see permute_nibbles in codec_kernels.cu)
void launch_permute_plane(uint8_t* nib, size_t bytes, cudaStream_t s);
// device-side encoders (bit-exact with the reference quantizer; transcendental values come
// from host-built lookup tables indexed by f16 bit pattern)
void launch_encode_q8_row(const float* w, int rows, int cols, uint8_t* payload, cudaStream_t s);
void launch_encode_q4_tiled(const float* w, int rows, int cols, uint8_t* payload, cudaStream_t s);
void launch_encode_q4tp(const float* w, int rows, int cols, uint8_t* payload, const float* log2_lut,
                        const float* exp2_lut, cudaStream_t s);

// ---------------- element-wise / row kernels (rowops.cu) ----------------
void launch_f32_to_bf16(const float* in, __nv_bfloat16* out, size_t n, cudaStream_t s);
// atomicMax of the squared norms of the bf16 head rows x [heads_total][hd] into *out (float bits; zero it first)
void launch_head_norm2_max(const __nv_bfloat16* x, size_t heads_total, int hd, unsigned* out, cudaStream_t s);
void launch_bf16_to_f32(const __nv_bfloat16* in, float* out, size_t n, cudaStream_t s);
// out_bf16[r, :] = rms(x[r, :]; w, eps) * (1 + shift)   (shift may be null)
void launch_rms_mod(const float* x, const float* w, const float* shift, double eps, int rows, int cols,
                    __nv_bfloat16* out_bf16, float* out_f32, cudaStream_t s);
// x[r, :] += gate * rms(src[r, :]; w, eps)   (gate may be null -> 1)
void launch_gated_residual(float* x, const float* src, const float* w, const float* gate, double eps, int rows,
                           int cols, cudaStream_t s);
// fused: x += gate*rms(src; w_res); then out = rms(x; w_next)*(1+shift)  (one pass over x)
void launch_residual_then_norm(float* x, const float* src, const float* w_res, const float* gate,
                               const float* w_next, const float* shift, double eps, int rows, int cols,
                               __nv_bfloat16* out_bf16, cudaStream_t s);
// per (token, head): qk RMS norm (eps 1e-5) + interleaved-pair RoPE (cos / sin [n, hd/2] f32); writes Q, K bf16
// token-major (V never passes through here: the QKV GEMM's epilogue writes V^T itself)
// q == nullptr: only the K heads (the attention kernel then normalises and rotates Q in its prologue)
// q_scale multiplies the finished query rows (1, or scale * log2(e) for the bounded attention form)
// norm2_max (optional, two zeroed words): receives the largest squared norms of the finished heads
void launch_qk_rope_pack(const float* qkv, int n, int nh, int nkv, int hd, const float* norm_q,
                         const float* norm_k, const float* cos_t, const float* sin_t, float q_scale, unsigned* norm2_max,
                         __nv_bfloat16* q,
                         __nv_bfloat16* k, cudaStream_t s);
// y[r] = act_out( dot(W[r, :], act_in(x)) * scale[r] + b[r] ); W f32 or int8 (+row scales)
// act_in: 0 none, 1 silu.  tanh_lo..tanh_hi: rows in [lo0,hi0) or [lo1,hi1) get tanh.
struct GemvParams {
    const void* w; int w_is_q8; const float* row_scale; const float* bias; const float* x;
    float* y; int rows, cols; int act_in; int tanh_lo0, tanh_hi0, tanh_lo1, tanh_hi1;
};
void launch_gemv(const GemvParams& p, cudaStream_t s);
// small exact-f32 GEMM: Y[M,N] = A[M,K] . W[N,K]^T + b
void launch_sgemm_nt_bias(const float* a, const float* w, const float* bias, float* y, int M, int N, int K,
                          cudaStream_t s);
void launch_time_freqs(const float* sched, const int* counter, float* out256, cudaStream_t s);
void launch_advance_step(int* counter, cudaStream_t s);
void launch_patchify(const float* latent, int c, int h, int w, int p, float* tok, cudaStream_t s);
void launch_unpatchify(const float* tok, int c, int h, int w, int p, float* latent, cudaStream_t s);
// LayerNorm without affine (eps 1e-6), times (1 + scale), f32 out
void launch_layernorm_scale(const float* x, const float* scale, int rows, int cols, float* out, cudaStream_t s);
void launch_silu_mul(const __nv_bfloat16* gu, int rows, int inter, __nv_bfloat16* out, cudaStream_t s);
// CFG combine with per-row norm rescale, then Euler update: x -= d * pred
// schedule: sched[2*i] = timestep t_i, sched[2*i+1] = sigma_{i+1} - sigma_i; *counter = current step
// use_cfg: 0 x -= d * cond; 1 guided prediction rescaled per row to the cond norm; 2 guided, no rescale
void launch_cfg_euler(float* latents, const float* cond, const float* uncond, float gs, const float* sched,
                      const int* counter, int rows, int lw, int use_cfg, cudaStream_t s);
void launch_transpose_head_major(const float* src_head_major, int heads, int n, int hd, float scale,
                                 __nv_bfloat16* dst_token_major, cudaStream_t s);
void launch_v_head_major_to_vt(const float* v_head_major, int nkv, int n, int hd, __nv_bfloat16* vt, int vt_pitch,
                               cudaStream_t s);
void launch_add_bias_rows(float* y, const float* bias, size_t rows, int cols, cudaStream_t s);
void launch_fill_normal(float* out, size_t n, uint64_t seed, float std, cudaStream_t s);
void launch_interleave_f32(float* dst, int dst_stride, int dst_off, const float* src, size_t count, cudaStream_t s);

// ---------------- VAE decoder: split-f16 implicit-GEMM convolution (conv_f16x2.cu) ----------------
// A "split" tensor is an f32 tensor stored as two f16 planes, hi = f16(v) and lo = f16(v - hi).
struct ConvParams {
    int ic;                  // input channels as stored (padded to a multiple of 32)
    int taps;                // 9 (3x3, padding 1) or 1 (1x1 / linear)
    int w, h;                // output = input extent in pixels; a linear over n tokens has w = n, h = 1
    int bw, bh;              // pixel tile, bw * bh = 256, bw a power of two
    int oc;                  // output channels (rows of the weight planes)
    int a_planes, b_planes;  // 1: hi only, 2: hi + lo
    const float* bias;       // [oc] or null
    float out_scale;         // applied to (acc + bias)
    const float* residual;   // f32, same indexing as the output, or null
    float* out_f32;          // any of the two outputs may be null
    __half *out_hi, *out_lo;
    int out_pitch;           // elements between pixels (pixel-major) or between channels (channel-major)
    int channel_major;       // 0: out[pixel * pitch + oc] (NHWC); 1: out[oc * pitch + pixel] (NCHW / V^T)
    double* stats_partial;   // null, or [2 * tiles_x * tiles_y][oc][2]: per-slot sum and sum of squares of the
                             // stored values per channel (input of the next GroupNorm), see conv_stats_slots
    int tiles_oc, tiles_x, tiles_y;  // filled by the launcher
    uint32_t* status;
};
// pixel tile chosen for an h x w image, and the number of statistics slots a launch fills
void conv_tile_shape(int w, int h, int* bw, int* bh);
size_t conv_stats_slots(int w, int h);
int launch_conv_f16x2(const CUtensorMap& tm_a_hi, const CUtensorMap& tm_a_lo, const CUtensorMap& tm_b_hi,
                      const CUtensorMap& tm_b_lo, ConvParams p, int num_sms, cudaStream_t stream);

// ---------------- VAE decoder: memory-bound passes (vae_kernels.cu) ----------------
// GroupNorm (eps 1e-6, f64 statistics) over NHWC f32 x [pixels, c], c a power of two in [32, 1024].
// stats: gn_stats_bytes(c) bytes; the first [c][2] doubles receive (sum, sum of squares) per
// channel, the rest is scratch for per-block partials that are reduced in a fixed order.
size_t gn_stats_bytes(int c);
// partials [slots][c][2] -> stats [c][2], summed in slot order
void launch_gn_finalize(const double* partials, size_t slots, int c, double* stats, cudaStream_t s);
int launch_gn_stats(const float* x, size_t pixels, int c, double* stats, cudaStream_t s);
// y = ((x - mean_g) * inv_g) as f32 * w + b, optional SiLU, written as split planes; when raw_hi is
// given the unnormalized x is also written as split planes (the input of a shortcut convolution).
int launch_gn_apply(const float* x, size_t pixels, int c, int groups, const double* stats, const float* w,
                    const float* b, int silu, __half* y_hi, __half* y_lo, __half* raw_hi, __half* raw_lo,
                    cudaStream_t s);
// nearest 2x upsampling of NHWC f32 [h, w, c] into split planes [2h, 2w, c]
void launch_upsample2x_split(const float* x, int h, int w, int c, __half* hi, __half* lo, cudaStream_t s);
// NCHW f32 [c, h*w] -> split NHWC planes [h*w, c_pad] with v * mul + add (pad channels zero)
void launch_nchw_to_split(const float* x, int c, size_t pixels, int c_pad, float div, float add, int affine,
                          __half* hi, __half* lo, cudaStream_t s);
// NHWC f32 [pixels, c] <-> NCHW f32 [c, pixels]
void launch_nhwc_to_nchw(const float* x, size_t pixels, int c, float* out, cudaStream_t s);
void launch_nchw_to_nhwc(const float* x, size_t pixels, int c, float* out, cudaStream_t s);
// OIHW f32 [oc, ic, k, k] -> split planes [oc, k*k, ic_pad]
void launch_conv_weight_split(const float* w, int oc, int ic, int taps, int ic_pad, __half* hi, __half* lo,
                              cudaStream_t s);
// row softmax of f32 scores [rows, cols] (row pitch ld) into split planes with row pitch ldp
int launch_softmax_rows_split(const float* scores, size_t rows, int cols, size_t ld, __half* hi, __half* lo,
                              size_t ldp, cudaStream_t s);
// f32 -> split planes, element-wise
void launch_split_f32(const float* x, size_t n, __half* hi, __half* lo, cudaStream_t s);
// group-normalized f32 output (no split): y = ((x - mean) * inv) as f32 * w + b, optional SiLU
int launch_gn_apply_f32(const float* x, size_t pixels, int c, int groups, const double* stats, const float* w,
                        const float* b, int silu, float* y, cudaStream_t s);


// ---------------- Gemma-2 prompt encoder (gemma_kernels.cu) ----------------
// out[r, :] = (q8[r, :] * scale[r]) * emb_scale over gathered embedding rows
void launch_embed_q8(const int8_t* q, const float* scale, int rows, int cols, float emb_scale, float* out, cudaStream_t s);
void launch_scale_f32(float* x, size_t n, float sc, cudaStream_t s);
// Activations of the encoder's GEMMs are split rows: [2n, K] bf16 with hi = bf16(v) in rows [0, n) and
// lo = bf16(v - hi) in rows [n, 2n); a GEMM output [2n, N] f32 is consumed as the sum of its halves.
// qkv [2n, pitch]: halves summed into rows [0, n); the first heads_qk heads get half-split RoPE in f32
void launch_rope_half(float* qkv, int n, int heads_qk, int heads_all, int pitch, int hd, const float* cos_t,
                      const float* sin_t, cudaStream_t s);
// h[r] += rms(src[r] + src[n + r]) * w_res (src may be null), then, if w_next: rms(h) * w_next as split rows
// and / or f32.  w_res / w_next hold 1 + weight.
void launch_gemma_residual_norm(float* h, const float* src, int n, int cols, const float* w_res, const float* w_next,
                                double eps, __nv_bfloat16* out_split, float* out_f32, cudaStream_t s);
// gu [2n, 2 * inter] (gate / up interleaved by column) -> gelu_tanh(g) * u as split rows [2n, inter]
void launch_geglu_split(const float* gu, int n, int inter, __nv_bfloat16* act, cudaStream_t s);
// causal GQA attention with logit soft-capping over rows [0, n) of qkv [., (nh + 2 nkv) * hd] f32 -> split rows
// out [2n, nh * hd]
int launch_attn_causal_f32(const float* qkv, int n, int nh, int nkv, int hd, float scale, float softcap,
                           __nv_bfloat16* out, cudaStream_t s);

}  // namespace cmfc
