// Kernels of the Gemma-2 prompt encoder that the denoiser path does not already have
// (crates/cortiq-engine/src/textenc.rs): embedding rows scaled by sqrt(hidden) (:237-246),
// half-split RoPE in f32 (:271-286), causal soft-capped attention in f32 (:287-323).
// A prompt is at most a few hundred tokens: these are small exact-f32 kernels; the projections
// go through the dequant GEMM.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace cmfc {
namespace {

// out[r, :] = (q8[r, :] * scale[r]) * emb_scale   (QTensor::row_f32 of a q8_row tensor, then the scale)
__global__ void embed_q8_kernel(const int8_t* __restrict__ q, const float* __restrict__ scale, int cols, float emb_scale,
                                float* __restrict__ out) {
    const size_t r = blockIdx.x;
    const float s = scale[r];
    for (int c = threadIdx.x; c < cols; c += blockDim.x)
        out[r * cols + c] = __fmul_rn(__fmul_rn((float)q[r * cols + c], s), emb_scale);
}

__global__ void scale_rows_kernel(float* __restrict__ x, size_t n, float s) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = __fmul_rn(x[i], s);
}

// The projections run on activations split into two bf16 rows per token (hi = bf16(v), lo = bf16(v - hi),
// stacked as rows [0, n) and [n, 2n) of one GEMM), so that the bf16 operand carries 16 significant
// bits; the consumer of a GEMM output adds the two halves.

__device__ __forceinline__ double block_sum_256(double v, double* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    for (int i = 0; i < 8; ++i) t += red[i];
    return t;
}

__device__ __forceinline__ void store_split(__nv_bfloat16* hi, __nv_bfloat16* lo, size_t o, float v) {
    const __nv_bfloat16 h = __float2bfloat16_rn(v);
    hi[o] = h;
    lo[o] = __float2bfloat16_rn(v - __bfloat162float(h));
}

// optional residual: h[r] += f32(d * inv_d) * w_res with d = src[r] + src[n + r]   (textenc.rs:326-334)
// optional norm:     out = f32(h * inv_h) * w_next as split rows and / or f32           (textenc.rs:59-68)
// w_res / w_next already hold 1 + weight.  One block of 256 threads per token row.
__global__ void __launch_bounds__(256) gemma_residual_norm_kernel(float* __restrict__ h, const float* __restrict__ src,
                                                                  int n, int cols, const float* __restrict__ w_res,
                                                                  const float* __restrict__ w_next, double eps,
                                                                  __nv_bfloat16* __restrict__ out_split,
                                                                  float* __restrict__ out_f32) {
    __shared__ double red[8];
    const size_t r = blockIdx.x;
    float* hr = h + r * cols;
    if (src) {
        const float* a = src + r * cols;
        const float* b = src + ((size_t)n + r) * cols;
        double ss = 0.0;
        for (int c = threadIdx.x; c < cols; c += 256) {
            const float d = __fadd_rn(a[c], b[c]);
            ss += (double)d * d;
        }
        ss = block_sum_256(ss, red);
        const double inv = 1.0 / sqrt(ss / cols + eps);
        for (int c = threadIdx.x; c < cols; c += 256) {
            const float d = __fadd_rn(a[c], b[c]);
            hr[c] = __fadd_rn(hr[c], __fmul_rn((float)((double)d * inv), w_res[c]));
        }
    }
    if (w_next) {
        double ss = 0.0;
        for (int c = threadIdx.x; c < cols; c += 256) ss += (double)hr[c] * hr[c];  // own writes: same thread, same columns
        ss = block_sum_256(ss, red);
        const double inv = 1.0 / sqrt(ss / cols + eps);
        for (int c = threadIdx.x; c < cols; c += 256) {
            const float o = __fmul_rn((float)((double)hr[c] * inv), w_next[c]);
            if (out_split) store_split(out_split, out_split + (size_t)n * cols, r * cols + c, o);
            if (out_f32) out_f32[r * cols + c] = o;
        }
    }
}

// qkv [2n, pitch] f32 (two halves): sum the halves into rows [0, n), rotating the q and k heads,
// pairs (i, i + hd/2), f32 as the engine does; v heads are only summed.
__global__ void rope_half_kernel(float* __restrict__ qkv, int n, int heads_qk, int heads_all, int pitch, int hd,
                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t) {
    const int p = blockIdx.x, half = hd / 2;
    float* row = qkv + (size_t)p * pitch;
    const float* row2 = qkv + ((size_t)n + p) * pitch;
    for (int t = threadIdx.x; t < heads_all * half; t += blockDim.x) {
        const int h = t / half, i = t % half;
        float* v = row + h * hd;
        const float* v2 = row2 + h * hd;
        const float a = __fadd_rn(v[i], v2[i]), b = __fadd_rn(v[i + half], v2[i + half]);
        if (h < heads_qk) {
            const float c = cos_t[(size_t)p * half + i], s = sin_t[(size_t)p * half + i];
            v[i] = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
            v[i + half] = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
        } else {
            v[i] = a;
            v[i + half] = b;
        }
    }
}

// gu [2n, 2 * inter] f32 (two halves; gate and up of channel c in columns 2c, 2c + 1):
// act = gelu_tanh(g) * u as split rows [2n, inter]   (textenc.rs:70-73, :352-354)
__global__ void geglu_split_kernel(const float* __restrict__ gu, int n, int inter, __nv_bfloat16* __restrict__ act) {
    const size_t total = (size_t)n * inter;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / inter, c = i % inter;
        const float2 a = *reinterpret_cast<const float2*>(gu + r * 2 * inter + 2 * c);
        const float2 b = *reinterpret_cast<const float2*>(gu + (n + r) * 2 * inter + 2 * c);
        const float g = __fadd_rn(a.x, b.x), u = __fadd_rn(a.y, b.y);
        const float t = tanhf(__fmul_rn(0.7978846f, __fadd_rn(g, __fmul_rn(__fmul_rn(__fmul_rn(0.044715f, g), g), g))));
        const float ge = __fmul_rn(__fmul_rn(0.5f, g), __fadd_rn(1.0f, t));
        store_split(act, act + total, i, __fmul_rn(ge, u));
    }
}

// Causal attention with logit soft-capping, exact f32, one block per (16 queries, head).
// Scores of the query tile against keys 0..last live in shared memory; the dot products, the
// softmax weights and the weighted sum of V follow the reference's order of operations.
constexpr int GQ = 16;
__global__ void __launch_bounds__(256) attn_causal_f32_kernel(const float* __restrict__ qkv, int n, int nh, int nkv,
                                                              int hd, int pitch, float scale, float softcap,
                                                              int s_pitch, __nv_bfloat16* __restrict__ out) {
    // out: split rows [2n, nh * hd]
    extern __shared__ float sm[];
    float* Qs = sm;                         // [GQ][hd]
    float* Ks = Qs + GQ * hd;               // [GQ][hd + 1]
    float* S = Ks + GQ * (hd + 1);          // [GQ][s_pitch]
    const int q0 = blockIdx.x * GQ, h = blockIdx.y, kv = h / (nh / nkv);
    const int last = min(q0 + GQ, n) - 1;   // last key any query of the tile may see
    const float* qbase = qkv + (size_t)h * hd;
    const float* kbase = qkv + (size_t)(nh + kv) * hd;
    const float* vbase = qkv + (size_t)(nh + nkv + kv) * hd;
    for (int t = threadIdx.x; t < GQ * hd; t += 256) {
        const int i = t / hd, d = t % hd;
        Qs[t] = (q0 + i < n) ? qbase[(size_t)(q0 + i) * pitch + d] : 0.0f;
    }
    const int i = threadIdx.x >> 4, jj = threadIdx.x & 15;
    for (int k0 = 0; k0 <= last; k0 += GQ) {
        __syncthreads();
        for (int t = threadIdx.x; t < GQ * hd; t += 256) {
            const int r = t / hd, d = t % hd;
            Ks[r * (hd + 1) + d] = (k0 + r < n) ? kbase[(size_t)(k0 + r) * pitch + d] : 0.0f;
        }
        __syncthreads();
        const int j = k0 + jj, p = q0 + i;
        float acc = 0.0f;
        for (int d = 0; d < hd; ++d) acc = __fadd_rn(acc, __fmul_rn(Qs[i * hd + d], Ks[jj * (hd + 1) + d]));
        float s = __fmul_rn(acc, scale);
        if (softcap > 0.0f) s = __fmul_rn(softcap, tanhf(__fdiv_rn(s, softcap)));
        if (j <= last) S[i * s_pitch + j] = (j <= p && p < n) ? s : -INFINITY;
    }
    __syncthreads();
    // softmax weights e * (1 / sum) per query row: two rows per warp
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp * 2; r < warp * 2 + 2; ++r) {
        const int p = q0 + r;
        float* row = S + r * s_pitch;
        if (p >= n) {
            for (int j = lane; j <= last; j += 32) row[j] = 0.0f;
            continue;
        }
        float mx = -INFINITY;
        for (int j = lane; j <= p; j += 32) mx = fmaxf(mx, row[j]);
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float den = 0.0f;
        for (int j = lane; j <= p; j += 32) {
            const float e = expf(row[j] - mx);
            row[j] = e;
            den += e;
        }
        den = warp_sum(den);
        const float inv = 1.0f / den;
        for (int j = lane; j <= last; j += 32) row[j] = j <= p ? __fmul_rn(row[j], inv) : 0.0f;
    }
    __syncthreads();
    for (int d = threadIdx.x; d < hd; d += 256) {
        float acc[GQ];
#pragma unroll
        for (int r = 0; r < GQ; ++r) acc[r] = 0.0f;
        // keys in ascending order (the reference's summation order); eight V loads in flight
        int j = 0;
        for (; j + 8 <= last + 1; j += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = vbase[(size_t)(j + u) * pitch + d];
#pragma unroll
            for (int u = 0; u < 8; ++u)
#pragma unroll
                for (int r = 0; r < GQ; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(S[r * s_pitch + j + u], v[u]));
        }
        for (; j <= last; ++j) {
            const float v = vbase[(size_t)j * pitch + d];
#pragma unroll
            for (int r = 0; r < GQ; ++r) acc[r] = __fadd_rn(acc[r], __fmul_rn(S[r * s_pitch + j], v));
        }
#pragma unroll
        for (int r = 0; r < GQ; ++r)
            if (q0 + r < n)
                store_split(out, out + (size_t)n * (nh * hd), (size_t)(q0 + r) * (nh * hd) + h * hd + d, acc[r]);
    }
}

}  // namespace

void launch_embed_q8(const int8_t* q, const float* scale, int rows, int cols, float emb_scale, float* out, cudaStream_t s) {
    embed_q8_kernel<<<rows, 256, 0, s>>>(q, scale, cols, emb_scale, out);
}

void launch_scale_f32(float* x, size_t n, float sc, cudaStream_t s) {
    const size_t blocks = (n + 1023) / 1024;
    scale_rows_kernel<<<(unsigned)(blocks < 1184 ? (blocks ? blocks : 1) : 1184), 256, 0, s>>>(x, n, sc);
}

void launch_rope_half(float* qkv, int n, int heads_qk, int heads_all, int pitch, int hd, const float* cos_t,
                      const float* sin_t, cudaStream_t s) {
    rope_half_kernel<<<n, 256, 0, s>>>(qkv, n, heads_qk, heads_all, pitch, hd, cos_t, sin_t);
}

void launch_gemma_residual_norm(float* h, const float* src, int n, int cols, const float* w_res, const float* w_next,
                                double eps, __nv_bfloat16* out_split, float* out_f32, cudaStream_t s) {
    gemma_residual_norm_kernel<<<n, 256, 0, s>>>(h, src, n, cols, w_res, w_next, eps, out_split, out_f32);
}

void launch_geglu_split(const float* gu, int n, int inter, __nv_bfloat16* act, cudaStream_t s) {
    const size_t blocks = ((size_t)n * inter + 1023) / 1024;
    geglu_split_kernel<<<(unsigned)(blocks < 1184 ? (blocks ? blocks : 1) : 1184), 256, 0, s>>>(gu, n, inter, act);
}

int launch_attn_causal_f32(const float* qkv, int n, int nh, int nkv, int hd, float scale, float softcap,
                           __nv_bfloat16* out, cudaStream_t s) {
    if (n <= 0 || nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || hd > 512)
        return fail(ERR_SHAPE, "causal attention: bad head geometry");
    const int s_pitch = ((n + 31) / 32) * 32 + 1;
    const size_t smem = sizeof(float) * ((size_t)GQ * hd + (size_t)GQ * (hd + 1) + (size_t)GQ * s_pitch);
    if (smem > 200 * 1024) return fail(ERR_UNSUPPORTED, "causal attention: prompt too long for the score tile in shared memory");
    static std::atomic<bool> configured[64];
    int dev = 0;
    CMFC_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        CMFC_CUDA(cudaFuncSetAttribute(attn_causal_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured[dev & 63] = true;
    }
    const int pitch = (nh + 2 * nkv) * hd;
    attn_causal_f32_kernel<<<dim3((n + GQ - 1) / GQ, nh), 256, smem, s>>>(qkv, n, nh, nkv, hd, pitch, scale, softcap, s_pitch, out);
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace cmfc
