// Memory-bound passes of the VAE decoder (crates/cortiq-engine/src/vae.rs): GroupNorm with f64
// statistics (:254-294), SiLU (:297), nearest 2x upsampling (:314), the row softmax of the
// attention block (:449-460), and the layout changes between the reference's NCHW f32 tensors
// and the NHWC split-f16 planes the convolution kernel reads.
#include <cuda_fp16.h>

#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace cmfc {
namespace {

struct Half4 {
    __half2 a, b;
};

__device__ __forceinline__ void split4(const float4& v, Half4& hi, Half4& lo) {
    hi.a = __floats2half2_rn(v.x, v.y);
    hi.b = __floats2half2_rn(v.z, v.w);
    const float2 ha = __half22float2(hi.a), hb = __half22float2(hi.b);
    lo.a = __floats2half2_rn(v.x - ha.x, v.y - ha.y);
    lo.b = __floats2half2_rn(v.z - hb.x, v.w - hb.y);
}

__device__ __forceinline__ float silu_ref(float v) { return v / (1.0f + expf(-v)); }

constexpr int MAX_GRID = 148 * 8;
int grid_for(size_t work_items, int per_block) {
    const size_t want = (work_items + per_block - 1) / per_block;
    return (int)std::max<size_t>(1, std::min<size_t>(want, MAX_GRID));
}

// ---- GroupNorm statistics: per-channel sum and sum of squares in f64 ----
// 256 threads; a thread keeps one channel quad and strides over pixels.
__global__ void __launch_bounds__(256) gn_stats_kernel(const float4* __restrict__ x, size_t pixels, int c4,
                                                       double* __restrict__ stats) {
    __shared__ double red[256][8];
    const int quad = threadIdx.x % c4, prow = threadIdx.x / c4, ppb = 256 / c4;
    double s[4] = {0, 0, 0, 0}, q[4] = {0, 0, 0, 0};
    for (size_t pix = (size_t)blockIdx.x * ppb + prow; pix < pixels; pix += (size_t)gridDim.x * ppb) {
        const float4 v = x[pix * c4 + quad];
        const double a = v.x, b = v.y, c = v.z, d = v.w;
        s[0] += a; s[1] += b; s[2] += c; s[3] += d;
        q[0] += a * a; q[1] += b * b; q[2] += c * c; q[3] += d * d;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        red[threadIdx.x][i] = s[i];
        red[threadIdx.x][4 + i] = q[i];
    }
    __syncthreads();
    if (prow == 0) {
        for (int r = 1; r < ppb; ++r)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                s[i] += red[r * c4 + quad][i];
                q[i] += red[r * c4 + quad][4 + i];
            }
        // per-block partials, reduced in a fixed order by gn_finalize_kernel (bit-reproducible)
        double* mine = stats + (size_t)blockIdx.x * (c4 * 8);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            mine[(quad * 4 + i) * 2] = s[i];
            mine[(quad * 4 + i) * 2 + 1] = q[i];
        }
    }
}

// partials [blocks][2c] -> stats [2c].  One warp per output: lane l adds blocks l, l + 32, ... in
// order, then the lanes are combined by a fixed butterfly, so the result does not depend on timing.
__global__ void gn_finalize_kernel(const double* __restrict__ partials, int blocks, int c2, double* __restrict__ stats) {
    const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (i >= c2) return;
    double a = 0;
    for (int b = lane; b < blocks; b += 32) a += partials[(size_t)b * c2 + i];
    a = warp_sum(a);
    if (lane == 0) stats[i] = a;
}

// ---- GroupNorm apply (+ SiLU) ----
// mean / inverse deviation per channel are rebuilt from the channel sums by every block.
template <bool SPLIT_OUT>
__global__ void __launch_bounds__(256) gn_apply_kernel(const float4* __restrict__ x, size_t pixels, int c4, int per,
                                                       const double* __restrict__ stats, const float* __restrict__ w,
                                                       const float* __restrict__ b, int silu, Half4* __restrict__ y_hi,
                                                       Half4* __restrict__ y_lo, Half4* __restrict__ raw_hi,
                                                       Half4* __restrict__ raw_lo, float4* __restrict__ y_f32) {
    __shared__ double s_mean[1024], s_inv[1024];
    const int c = c4 * 4;
    for (int ch = threadIdx.x; ch < c; ch += 256) {
        const int g0 = (ch / per) * per;
        double s = 0, q = 0;
        for (int j = 0; j < per; ++j) {
            s += stats[(g0 + j) * 2];
            q += stats[(g0 + j) * 2 + 1];
        }
        const double n = (double)pixels * per;
        const double mean = s / n;
        double var = q / n - mean * mean;
        if (var < 0) var = 0;
        s_mean[ch] = mean;
        s_inv[ch] = 1.0 / sqrt(var + 1e-6);
    }
    __syncthreads();
    const int quad = threadIdx.x % c4, prow = threadIdx.x / c4, ppb = 256 / c4;
    const int ch = quad * 4;
    const double m0 = s_mean[ch], m1 = s_mean[ch + 1], m2 = s_mean[ch + 2], m3 = s_mean[ch + 3];
    const double i0 = s_inv[ch], i1 = s_inv[ch + 1], i2 = s_inv[ch + 2], i3 = s_inv[ch + 3];
    const float4 ww = reinterpret_cast<const float4*>(w)[quad], bb = reinterpret_cast<const float4*>(b)[quad];
    for (size_t pix = (size_t)blockIdx.x * ppb + prow; pix < pixels; pix += (size_t)gridDim.x * ppb) {
        const size_t o = pix * c4 + quad;
        const float4 v = x[o];
        float4 y;
        y.x = __fadd_rn(__fmul_rn((float)(((double)v.x - m0) * i0), ww.x), bb.x);
        y.y = __fadd_rn(__fmul_rn((float)(((double)v.y - m1) * i1), ww.y), bb.y);
        y.z = __fadd_rn(__fmul_rn((float)(((double)v.z - m2) * i2), ww.z), bb.z);
        y.w = __fadd_rn(__fmul_rn((float)(((double)v.w - m3) * i3), ww.w), bb.w);
        if (silu) {
            y.x = silu_ref(y.x); y.y = silu_ref(y.y); y.z = silu_ref(y.z); y.w = silu_ref(y.w);
        }
        if (SPLIT_OUT) {
            Half4 hi, lo;
            split4(y, hi, lo);
            y_hi[o] = hi;
            y_lo[o] = lo;
            if (raw_hi) {
                split4(v, hi, lo);
                raw_hi[o] = hi;
                raw_lo[o] = lo;
            }
        } else {
            y_f32[o] = y;
        }
    }
}

__global__ void upsample2x_split_kernel(const float4* __restrict__ x, int h, int w, int c4, Half4* __restrict__ hi,
                                        Half4* __restrict__ lo) {
    const size_t total = (size_t)4 * h * w * c4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int quad = (int)(i % c4);
        const size_t pix = i / c4;
        const int ox = (int)(pix % (2 * w)), oy = (int)(pix / (2 * w));
        const float4 v = x[((size_t)(oy >> 1) * w + (ox >> 1)) * c4 + quad];
        Half4 a, b;
        split4(v, a, b);
        hi[i] = a;
        lo[i] = b;
    }
}

// 32 x 32 tiled transposes between [c, pixels] and [pixels, c_pad]
__global__ void nchw_to_split_kernel(const float* __restrict__ x, int c, size_t pixels, int c_pad, float div, float add,
                                     int affine, __half* __restrict__ hi, __half* __restrict__ lo) {
    __shared__ float tile[32][33];
    const size_t p0 = (size_t)blockIdx.x * 32;
    const int c0 = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const int ch = c0 + r;
        const size_t pix = p0 + threadIdx.x;
        float v = 0.0f;
        if (ch < c && pix < pixels) {
            v = x[(size_t)ch * pixels + pix];
            if (affine) v = __fadd_rn(__fdiv_rn(v, div), add);
        }
        tile[r][threadIdx.x] = v;
    }
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y) {
        const size_t pix = p0 + r;
        const int ch = c0 + threadIdx.x;
        if (pix < pixels && ch < c_pad) {
            const float v = tile[threadIdx.x][r];
            const __half h = __float2half_rn(v);
            hi[pix * c_pad + ch] = h;
            lo[pix * c_pad + ch] = __float2half_rn(v - __half2float(h));
        }
    }
}

// in [rows_in, cols_in] -> out [cols_in, rows_in]
__global__ void transpose_f32_kernel(const float* __restrict__ in, size_t rows_in, size_t cols_in, float* __restrict__ out) {
    __shared__ float tile[32][33];
    const size_t c0 = (size_t)blockIdx.x * 32, r0 = (size_t)blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y)
        if (r0 + r < rows_in && c0 + threadIdx.x < cols_in) tile[r][threadIdx.x] = in[(r0 + r) * cols_in + c0 + threadIdx.x];
    __syncthreads();
    for (int r = threadIdx.y; r < 32; r += blockDim.y)
        if (c0 + r < cols_in && r0 + threadIdx.x < rows_in) out[(c0 + r) * rows_in + r0 + threadIdx.x] = tile[threadIdx.x][r];
}

__global__ void conv_weight_split_kernel(const float* __restrict__ w, int oc, int ic, int taps, int ic_pad,
                                         __half* __restrict__ hi, __half* __restrict__ lo) {
    const size_t total = (size_t)oc * taps * ic_pad;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % ic_pad);
        const int tap = (int)((i / ic_pad) % taps);
        const size_t o = i / ((size_t)ic_pad * taps);
        const float v = c < ic ? w[(o * ic + c) * taps + tap] : 0.0f;
        const __half h = __float2half_rn(v);
        hi[i] = h;
        lo[i] = __float2half_rn(v - __half2float(h));
    }
}

__global__ void split_f32_kernel(const float* __restrict__ x, size_t n, __half* __restrict__ hi, __half* __restrict__ lo) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = x[i];
        const __half h = __float2half_rn(v);
        hi[i] = h;
        lo[i] = __float2half_rn(v - __half2float(h));
    }
}

// One block per score row, the row staged in shared memory: max, exp and sum in f32, then
// p = e * (1 / sum) as split planes (the reference's order of operations, vae.rs:449-460).
__global__ void __launch_bounds__(256) softmax_rows_split_kernel(const float* __restrict__ scores, int cols, size_t ld,
                                                                 __half* __restrict__ hi, __half* __restrict__ lo,
                                                                 size_t ldp) {
    extern __shared__ float row[];
    __shared__ float red[8];
    const float* src = scores + (size_t)blockIdx.x * ld;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float mx = -3.4028234663852886e38f;
    for (int i = threadIdx.x; i < cols; i += 256) {
        const float v = src[i];
        row[i] = v;
        mx = fmaxf(mx, v);
    }
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float den = 0.0f;
    for (int i = threadIdx.x; i < cols; i += 256) {
        const float e = expf(row[i] - mx);
        row[i] = e;
        den += e;
    }
    den = warp_sum(den);
    if (lane == 0) red[warp] = den;
    __syncthreads();
    den = 0.0f;
    for (int i = 0; i < 8; ++i) den += red[i];
    const float inv = 1.0f / den;
    __half* dh = hi + (size_t)blockIdx.x * ldp;
    __half* dl = lo + (size_t)blockIdx.x * ldp;
    for (int i = threadIdx.x; i < cols; i += 256) {
        const float p = row[i] * inv;
        const __half h = __float2half_rn(p);
        dh[i] = h;
        dl[i] = __float2half_rn(p - __half2float(h));
    }
}

// The same for rows longer than shared memory holds: three passes over the row in global memory
// (the row stays in L2 between them).
__global__ void __launch_bounds__(256) softmax_rows_split_long_kernel(const float* __restrict__ scores, int cols, size_t ld,
                                                                      __half* __restrict__ hi, __half* __restrict__ lo,
                                                                      size_t ldp) {
    __shared__ float red[8];
    const float* src = scores + (size_t)blockIdx.x * ld;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float mx = -3.4028234663852886e38f;
    for (int i = threadIdx.x; i < cols; i += 256) mx = fmaxf(mx, src[i]);
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
    __syncthreads();
    float den = 0.0f;
    for (int i = threadIdx.x; i < cols; i += 256) den += expf(src[i] - mx);
    den = warp_sum(den);
    if (lane == 0) red[warp] = den;
    __syncthreads();
    den = 0.0f;
    for (int i = 0; i < 8; ++i) den += red[i];
    const float inv = 1.0f / den;
    __half* dh = hi + (size_t)blockIdx.x * ldp;
    __half* dl = lo + (size_t)blockIdx.x * ldp;
    for (int i = threadIdx.x; i < cols; i += 256) {
        const float p = expf(src[i] - mx) * inv;
        const __half h = __float2half_rn(p);
        dh[i] = h;
        dl[i] = __float2half_rn(p - __half2float(h));
    }
}

bool gn_channels_ok(int c) { return c >= 32 && c <= 1024 && (c & (c - 1)) == 0; }

}  // namespace

size_t gn_stats_bytes(int c) { return sizeof(double) * 2 * (size_t)c * (1 + MAX_GRID); }

void launch_gn_finalize(const double* partials, size_t slots, int c, double* stats, cudaStream_t s) {
    gn_finalize_kernel<<<(2 * c + 7) / 8, 256, 0, s>>>(partials, (int)slots, 2 * c, stats);
}

int launch_gn_stats(const float* x, size_t pixels, int c, double* stats, cudaStream_t s) {
    if (!gn_channels_ok(c)) return fail(ERR_UNSUPPORTED, "group norm: channels must be a power of two in [32, 1024]");
    const int ppb = 256 / (c / 4);
    const int blocks = grid_for(pixels, ppb * 8);
    double* partials = stats + 2 * c;
    gn_stats_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const float4*>(x), pixels, c / 4, partials);
    gn_finalize_kernel<<<(2 * c + 7) / 8, 256, 0, s>>>(partials, blocks, 2 * c, stats);
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

int launch_gn_apply(const float* x, size_t pixels, int c, int groups, const double* stats, const float* w,
                    const float* b, int silu, __half* y_hi, __half* y_lo, __half* raw_hi, __half* raw_lo,
                    cudaStream_t s) {
    if (!gn_channels_ok(c) || groups <= 0 || c % groups) return fail(ERR_UNSUPPORTED, "group norm: unsupported channels / groups");
    const int ppb = 256 / (c / 4);
    gn_apply_kernel<true><<<grid_for(pixels, ppb * 4), 256, 0, s>>>(
        reinterpret_cast<const float4*>(x), pixels, c / 4, c / groups, stats, w, b, silu, reinterpret_cast<Half4*>(y_hi),
        reinterpret_cast<Half4*>(y_lo), reinterpret_cast<Half4*>(raw_hi), reinterpret_cast<Half4*>(raw_lo), nullptr);
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

int launch_gn_apply_f32(const float* x, size_t pixels, int c, int groups, const double* stats, const float* w,
                        const float* b, int silu, float* y, cudaStream_t s) {
    if (!gn_channels_ok(c) || groups <= 0 || c % groups) return fail(ERR_UNSUPPORTED, "group norm: unsupported channels / groups");
    const int ppb = 256 / (c / 4);
    gn_apply_kernel<false><<<grid_for(pixels, ppb * 4), 256, 0, s>>>(reinterpret_cast<const float4*>(x), pixels, c / 4,
                                                                    c / groups, stats, w, b, silu, nullptr, nullptr,
                                                                    nullptr, nullptr, reinterpret_cast<float4*>(y));
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

void launch_upsample2x_split(const float* x, int h, int w, int c, __half* hi, __half* lo, cudaStream_t s) {
    const size_t total = (size_t)4 * h * w * (c / 4);
    upsample2x_split_kernel<<<grid_for(total, 256 * 4), 256, 0, s>>>(reinterpret_cast<const float4*>(x), h, w, c / 4,
                                                                    reinterpret_cast<Half4*>(hi), reinterpret_cast<Half4*>(lo));
}

void launch_nchw_to_split(const float* x, int c, size_t pixels, int c_pad, float div, float add, int affine, __half* hi,
                          __half* lo, cudaStream_t s) {
    dim3 grid((unsigned)((pixels + 31) / 32), (unsigned)((c_pad + 31) / 32));
    nchw_to_split_kernel<<<grid, dim3(32, 8), 0, s>>>(x, c, pixels, c_pad, div, add, affine, hi, lo);
}

void launch_nhwc_to_nchw(const float* x, size_t pixels, int c, float* out, cudaStream_t s) {
    dim3 grid((unsigned)((c + 31) / 32), (unsigned)((pixels + 31) / 32));
    transpose_f32_kernel<<<grid, dim3(32, 8), 0, s>>>(x, pixels, (size_t)c, out);
}

void launch_nchw_to_nhwc(const float* x, size_t pixels, int c, float* out, cudaStream_t s) {
    dim3 grid((unsigned)((pixels + 31) / 32), (unsigned)((c + 31) / 32));
    transpose_f32_kernel<<<grid, dim3(32, 8), 0, s>>>(x, (size_t)c, pixels, out);
}

void launch_conv_weight_split(const float* w, int oc, int ic, int taps, int ic_pad, __half* hi, __half* lo,
                              cudaStream_t s) {
    const size_t total = (size_t)oc * taps * ic_pad;
    conv_weight_split_kernel<<<grid_for(total, 256), 256, 0, s>>>(w, oc, ic, taps, ic_pad, hi, lo);
}

int launch_softmax_rows_split(const float* scores, size_t rows, int cols, size_t ld, __half* hi, __half* lo, size_t ldp,
                              cudaStream_t s) {
    const size_t smem = (size_t)cols * 4;
    if (rows > 0x7fffffffu) return fail(ERR_SHAPE, "softmax: too many rows");
    if (smem > 200 * 1024) {
        softmax_rows_split_long_kernel<<<(unsigned)rows, 256, 0, s>>>(scores, cols, ld, hi, lo, ldp);
        CMFC_CUDA(cudaGetLastError());
        return OK;
    }
    static std::atomic<bool> configured[64];
    int dev = 0;
    CMFC_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        CMFC_CUDA(cudaFuncSetAttribute(softmax_rows_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        configured[dev & 63] = true;
    }
    softmax_rows_split_kernel<<<(unsigned)rows, 256, smem, s>>>(scores, cols, ld, hi, lo, ldp);
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

void launch_split_f32(const float* x, size_t n, __half* hi, __half* lo, cudaStream_t s) {
    split_f32_kernel<<<grid_for(n, 256 * 4), 256, 0, s>>>(x, n, hi, lo);
}

}  // namespace cmfc
