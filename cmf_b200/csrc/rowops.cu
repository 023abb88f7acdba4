// Bandwidth-bound row kernels of the NextDiT block: modulated RMSNorm, gated sandwich-norm
// residual, qk-norm + RoPE + head packing (V is packed by the QKV GEMM's epilogue), adaLN / time-embedding matvecs, patchify,
// final LayerNorm, CFG combine + Euler step.  One warp owns one row and keeps it in
// registers, so every tensor is read once and written once with 16-byte accesses.
// Norm statistics are accumulated in f64 (the reference's CPU path keeps them and the RoPE rotation
// in f64, crates/cortiq-engine/src/dit.rs:259-284, :1078-1102; what runs in f32 here is stated at
// each kernel).
#include "common.cuh"
#include "kernels.h"

namespace cmfc {
namespace {

constexpr int ROW_WARPS = 2;  // warps (rows) per block for the row kernels: small blocks keep the tail of a launch short

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st_bf16x4(__nv_bfloat16* p, float a, float b, float c, float d) {
    uint2 v;
    v.x = pack_bf16(a, b);
    v.y = pack_bf16(c, d);
    *reinterpret_cast<uint2*>(p) = v;
}

template <int NV>  // float4 per lane; cols = 128 * NV
__global__ void __launch_bounds__(32 * ROW_WARPS)
rms_mod_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ shift,
               double eps, int rows, __nv_bfloat16* __restrict__ out_bf16, float* __restrict__ out_f32) {
    const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    constexpr int cols = 128 * NV;
    const float* xr = x + (size_t)row * cols;
    float4 v[NV];
    double ss = 0.0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        v[i] = ld4(xr + (i * 32 + lane) * 4);
        ss += sq4(v[i]);
    }
    ss = warp_sum(ss);
    const float inv = (float)(1.0 / sqrt(ss / cols + eps));
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        float4 g = ld4(w + c);
        float4 o;
        o.x = rms_elem(v[i].x, inv, g.x); o.y = rms_elem(v[i].y, inv, g.y);
        o.z = rms_elem(v[i].z, inv, g.z); o.w = rms_elem(v[i].w, inv, g.w);
        if (shift) {
            float4 s = ld4(shift + c);
            o.x *= 1.0f + s.x; o.y *= 1.0f + s.y; o.z *= 1.0f + s.z; o.w *= 1.0f + s.w;
        }
        if (out_bf16) st_bf16x4(out_bf16 + (size_t)row * cols + c, o.x, o.y, o.z, o.w);
        if (out_f32) st4(out_f32 + (size_t)row * cols + c, o);
    }
}

// x += gate * rms(src; w_res, eps); optionally followed (same pass, x still in registers) by
// out = rms(x; w_next, eps) * (1 + shift) for the next sub-layer.
template <int NV, bool THEN_NORM>
__global__ void __launch_bounds__(32 * ROW_WARPS)
residual_kernel(float* __restrict__ x, const float* __restrict__ src, const float* __restrict__ w_res,
                const float* __restrict__ gate, const float* __restrict__ w_next, const float* __restrict__ shift,
                double eps, int rows, __nv_bfloat16* __restrict__ out_bf16) {
    const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    constexpr int cols = 128 * NV;
    const float* sr = src + (size_t)row * cols;
    float* xr = x + (size_t)row * cols;
    // both rows (the GEMM output and the residual stream) are requested up front: the second does
    // not depend on the statistics of the first, and twice the bytes are in flight per warp
    float4 d[NV], xin[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) d[i] = ld4(sr + (i * 32 + lane) * 4);
#pragma unroll
    for (int i = 0; i < NV; ++i) xin[i] = ld4(xr + (i * 32 + lane) * 4);
    double ss = 0.0;
#pragma unroll
    for (int i = 0; i < NV; ++i) ss += sq4(d[i]);
    ss = warp_sum(ss);
    const float inv = (float)(1.0 / sqrt(ss / cols + eps));
    double ss2 = 0.0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        float4 g = ld4(w_res + c);
        float4 xv = xin[i];
        float4 r;
        r.x = rms_elem(d[i].x, inv, g.x); r.y = rms_elem(d[i].y, inv, g.y);
        r.z = rms_elem(d[i].z, inv, g.z); r.w = rms_elem(d[i].w, inv, g.w);
        if (gate) {
            float4 t = ld4(gate + c);
            xv.x += t.x * r.x; xv.y += t.y * r.y; xv.z += t.z * r.z; xv.w += t.w * r.w;
        } else {
            xv.x += r.x; xv.y += r.y; xv.z += r.z; xv.w += r.w;
        }
        st4(xr + c, xv);
        if (THEN_NORM) {
            d[i] = xv;
            ss2 += sq4(xv);
        }
    }
    if (THEN_NORM) {
        ss2 = warp_sum(ss2);
        const float inv2 = (float)(1.0 / sqrt(ss2 / cols + eps));
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int c = (i * 32 + lane) * 4;
            float4 g = ld4(w_next + c);
            float4 o;
            o.x = rms_elem(d[i].x, inv2, g.x); o.y = rms_elem(d[i].y, inv2, g.y);
            o.z = rms_elem(d[i].z, inv2, g.z); o.w = rms_elem(d[i].w, inv2, g.w);
            if (shift) {
                float4 s = ld4(shift + c);
                o.x *= 1.0f + s.x; o.y *= 1.0f + s.y; o.z *= 1.0f + s.z; o.w *= 1.0f + s.w;
            }
            st_bf16x4(out_bf16 + (size_t)row * cols + c, o.x, o.y, o.z, o.w);
        }
    }
}

// LayerNorm without affine (eps 1e-6), times (1 + scale)   (dit.rs:1346-1362)
template <int NV>
__global__ void __launch_bounds__(32 * ROW_WARPS)
layernorm_scale_kernel(const float* __restrict__ x, const float* __restrict__ scale, int rows,
                       float* __restrict__ out) {
    const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    constexpr int cols = 128 * NV;
    const float* xr = x + (size_t)row * cols;
    float4 v[NV];
    double sum = 0.0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        v[i] = ld4(xr + (i * 32 + lane) * 4);
        sum += (double)v[i].x + (double)v[i].y + (double)v[i].z + (double)v[i].w;
    }
    const double mean = warp_sum(sum) / cols;
    double var = 0.0;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        double a = v[i].x - mean, b = v[i].y - mean, c = v[i].z - mean, d = v[i].w - mean;
        var += a * a + b * b + c * c + d * d;
    }
    const double inv = 1.0 / sqrt(warp_sum(var) / cols + 1e-6);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int c = (i * 32 + lane) * 4;
        float4 s = ld4(scale + c);
        float4 o;
        o.x = (float)((v[i].x - mean) * inv) * (1.0f + s.x);
        o.y = (float)((v[i].y - mean) * inv) * (1.0f + s.y);
        o.z = (float)((v[i].z - mean) * inv) * (1.0f + s.z);
        o.w = (float)((v[i].w - mean) * inv) * (1.0f + s.w);
        st4(out + (size_t)row * cols + c, o);
    }
}

#define DISPATCH_NV(cols, CALL)                                                  \
    switch ((cols) / 128) {                                                      \
        case 1: { constexpr int NV = 1; CALL; } break;                           \
        case 2: { constexpr int NV = 2; CALL; } break;                           \
        case 4: { constexpr int NV = 4; CALL; } break;                           \
        case 8: { constexpr int NV = 8; CALL; } break;                           \
        case 12: { constexpr int NV = 12; CALL; } break;                         \
        case 16: { constexpr int NV = 16; CALL; } break;                         \
        case 18: { constexpr int NV = 18; CALL; } break;                         \
        case 24: { constexpr int NV = 24; CALL; } break;                         \
        case 32: { constexpr int NV = 32; CALL; } break;                         \
        default: break;                                                          \
    }

// qk-norm + RoPE: four lanes own one (token, head); of every 32 consecutive elements of the head a
// lane holds eight (four rotation pairs): two 16-byte loads, one 16-byte store.  The head statistic
// is accumulated in f64 (see sq4); normalisation and the rotation (a c - b s, a s + b c) run in f32
// with cos / sin tables that the host computed in f64 and rounded once (the reference rotates in
// f64, dit.rs:1078-1102; the results here are rounded to bf16 right after).
constexpr int ROPE_THREADS = 128;
// MEASURE: the launch also leaves the largest squared norm of a finished query head (scale included) and
// of a key head in norm2_max[0] / [1] (float bit patterns, atomicMax; zeroed by the caller), from which
// attention decides on the device whether every score stays inside its bounded form's range.
template <int PPL, bool MEASURE>  // PPL = hd / 32
__global__ void __launch_bounds__(ROPE_THREADS, PPL <= 3 ? 8 : 4)
qk_rope_kernel(const float* __restrict__ qkv, int n, int nh, int nkv, const float* __restrict__ norm_q,
               const float* __restrict__ norm_k, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
               float q_scale, __nv_bfloat16* __restrict__ q_out, __nv_bfloat16* __restrict__ k_out,
               unsigned* __restrict__ norm2_max) {
    constexpr int hd = 32 * PPL;
    const int h_first = q_out ? 0 : nh;  // without a Q output only the K heads are walked
    const int heads = nh + nkv - h_first;
    const long item = (long)blockIdx.x * (ROPE_THREADS / 4) + (threadIdx.x >> 2);
    const int l = threadIdx.x & 3;
    const bool active = item < (long)n * heads;
    const int tok = active ? (int)(item / heads) : 0;
    const int h = h_first + (active ? (int)(item % heads) : 0);
    const bool is_q = h < nh;
    const int ld_in = (nh + 2 * nkv) * hd;
    const float* src = qkv + (size_t)tok * ld_in + (size_t)h * hd + l * 8;  // q heads then k heads are contiguous
    const float* w = (is_q ? norm_q : norm_k) + l * 8;
    const float* ct = cos_t + (size_t)tok * (hd / 2) + l * 4;
    const float* st = sin_t + (size_t)tok * (hd / 2) + l * 4;
    float4 v[PPL][2];
#pragma unroll
    for (int g = 0; g < PPL; ++g) {
        v[g][0] = ld4(src + g * 32);
        v[g][1] = ld4(src + g * 32 + 4);
    }
    double ss = 0.0;
#pragma unroll
    for (int g = 0; g < PPL; ++g) ss += sq4(v[g][0]) + sq4(v[g][1]);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    const float inv = (float)(1.0 / sqrt(ss / hd + 1e-5));
    const float os = is_q ? q_scale : 1.0f;
    if constexpr (MEASURE) {
        // the rotation keeps a pair's norm, so the head's norm is that of the normalised, weighted row
        float n2 = 0.0f;
#pragma unroll
        for (int g = 0; g < PPL; ++g) {
            const float4 g0 = ld4(w + g * 32), g1 = ld4(w + g * 32 + 4);
            const float e[8] = {rms_elem(v[g][0].x, inv, g0.x), rms_elem(v[g][0].y, inv, g0.y), rms_elem(v[g][0].z, inv, g0.z),
                                rms_elem(v[g][0].w, inv, g0.w), rms_elem(v[g][1].x, inv, g1.x), rms_elem(v[g][1].y, inv, g1.y),
                                rms_elem(v[g][1].z, inv, g1.z), rms_elem(v[g][1].w, inv, g1.w)};
#pragma unroll
            for (int i = 0; i < 8; ++i) n2 = fmaf(e[i], e[i], n2);
        }
        n2 += __shfl_xor_sync(0xffffffffu, n2, 2);
        n2 += __shfl_xor_sync(0xffffffffu, n2, 1);
        n2 *= os * os;
        float qm = (active && is_q) ? n2 : 0.0f, km = (active && !is_q) ? n2 : 0.0f;
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            qm = fmaxf(qm, __shfl_xor_sync(0xffffffffu, qm, o));
            km = fmaxf(km, __shfl_xor_sync(0xffffffffu, km, o));
        }
        if ((threadIdx.x & 31) == 0) {
            if (__float_as_uint(qm) > norm2_max[0]) atomicMax(norm2_max, __float_as_uint(qm));
            if (__float_as_uint(km) > norm2_max[1]) atomicMax(norm2_max + 1, __float_as_uint(km));
        }
    }
    if (!active) return;
    __nv_bfloat16* dst = (is_q ? q_out + (size_t)tok * nh * hd + (size_t)h * hd
                               : k_out + (size_t)tok * nkv * hd + (size_t)(h - nh) * hd) + l * 8;
#pragma unroll
    for (int g = 0; g < PPL; ++g) {
        const float4 g0 = ld4(w + g * 32), g1 = ld4(w + g * 32 + 4);
        const float4 cs = ld4(ct + g * 16), sn = ld4(st + g * 16);
        auto rot = [&](float x, float y, float gx, float gy, float c, float s_) {
            const float a = rms_elem(x, inv, gx), b = rms_elem(y, inv, gy);
            return pack_bf16(fmaf(a, c, -(b * s_)) * os, fmaf(a, s_, b * c) * os);
        };
        uint4 o;
        o.x = rot(v[g][0].x, v[g][0].y, g0.x, g0.y, cs.x, sn.x);
        o.y = rot(v[g][0].z, v[g][0].w, g0.z, g0.w, cs.y, sn.y);
        o.z = rot(v[g][1].x, v[g][1].y, g1.x, g1.y, cs.z, sn.z);
        o.w = rot(v[g][1].z, v[g][1].w, g1.z, g1.w, cs.w, sn.w);
        *reinterpret_cast<uint4*>(dst + g * 32) = o;
    }
}

__global__ void interleave_f32_kernel(float* __restrict__ dst, int dst_stride, int dst_off, const float* __restrict__ src,
                                      size_t count) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < count; i += (size_t)gridDim.x * blockDim.x)
        dst[i * dst_stride + dst_off] = src[i];
}

// One warp per output row: y = dot(W[r], x) * scale[r] + b[r], optional tanh on two row ranges,
// optional second output silu(y).
__global__ void __launch_bounds__(256)
gemv_kernel(GemvParams p, float* __restrict__ y_silu) {
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= p.rows) return;
    float acc = 0.0f;
    if (p.w_is_q8) {
        const int8_t* wr = reinterpret_cast<const int8_t*>(p.w) + (size_t)row * p.cols;
        for (int c = lane * 16; c < p.cols; c += 512) {
            const int4 q = *reinterpret_cast<const int4*>(wr + c);
            const int words[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 xv = ld4(p.x + c + 4 * k);
                acc += (float)(int8_t)(words[k] & 0xff) * xv.x + (float)(int8_t)((words[k] >> 8) & 0xff) * xv.y +
                       (float)(int8_t)((words[k] >> 16) & 0xff) * xv.z + (float)(int8_t)(words[k] >> 24) * xv.w;
            }
        }
    } else {
        const float* wr = reinterpret_cast<const float*>(p.w) + (size_t)row * p.cols;
        for (int c = lane * 4; c < p.cols; c += 128) {
            const float4 a = ld4(wr + c), xv = ld4(p.x + c);
            acc += a.x * xv.x + a.y * xv.y + a.z * xv.z + a.w * xv.w;
        }
    }
    acc = warp_sum(acc);
    if (lane == 0) {
        if (p.row_scale) acc *= p.row_scale[row];
        if (p.bias) acc += p.bias[row];
        if ((row >= p.tanh_lo0 && row < p.tanh_hi0) || (row >= p.tanh_lo1 && row < p.tanh_hi1)) acc = tanhf(acc);
        p.y[row] = acc;
        if (y_silu) y_silu[row] = acc / (1.0f + expf(-acc));
    }
}

// Small exact-f32 GEMM, 64x64 tile, 4x4 per thread: Y = A . W^T + bias
__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ a, const float* __restrict__ w, const float* __restrict__ bias,
                float* __restrict__ y, int M, int N, int K) {
    __shared__ float as[16][65], ws[16][65];
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, c = i & 15;
            as[c][r] = (m0 + r < M && k0 + c < K) ? a[(size_t)(m0 + r) * K + k0 + c] : 0.0f;
            ws[c][r] = (n0 + r < N && k0 + c < K) ? w[(size_t)(n0 + r) * K + k0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = as[k][ty * 4 + i]; wv[i] = ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * wv[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
            if (m < M && n < N) y[(size_t)m * N + n] = acc[i][j] + (bias ? bias[n] : 0.0f);
        }
}

// sinusoidal timestep features, cos first (dit.rs:592-600): f64 angle, f32 result
// The timestep comes from the device-resident schedule (t at sched[2*step], sigma step at
// sched[2*step+1], step = *counter), so the same launch sequence can be replayed as a CUDA graph.
__global__ void time_freqs_kernel(const float* __restrict__ sched, const int* __restrict__ counter, float* out) {
    const float t = sched[2 * *counter];
    const int i = threadIdx.x;  // 128 threads
    const double ang = (double)t * exp(-log(10000.0) * (double)i / 128.0);
    out[i] = (float)cos(ang);
    out[128 + i] = (float)sin(ang);
}

// tok[(ph*wp+pw), (dy*p+dx)*c+ch] = latent[ch, ph*p+dy, pw*p+dx]   (dit.rs:1255-1268)
__global__ void patchify_kernel(const float* __restrict__ latent, int c, int h, int w, int p, float* __restrict__ tok,
                                int inverse, float* __restrict__ latent_out) {
    const int pv = p * p * c, wp = w / p;
    const size_t total = (size_t)(h / p) * wp * pv;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int e = (int)(i % pv);
        const size_t t = i / pv;
        const int ph = (int)(t / wp), pw = (int)(t % wp);
        const int ch = e % c, dx = (e / c) % p, dy = e / (c * p);
        const size_t li = (size_t)ch * h * w + (size_t)(ph * p + dy) * w + pw * p + dx;
        if (inverse) latent_out[li] = tok[i];
        else tok[i] = latent[li];
    }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n4) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = ld4(in + 4 * i);
        st_bf16x4(out + 4 * i, v.x, v.y, v.z, v.w);
    }
}
__global__ void f32_to_bf16_tail(const float* in, __nv_bfloat16* out, size_t from, size_t n) {
    const size_t i = from + threadIdx.x;
    if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __bfloat162float(in[i]);
}

// a = silu(g) * u over a [rows, 2*inter] bf16 buffer laid out as [g | u] per row
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, int rows, int inter,
                                __nv_bfloat16* __restrict__ out) {
    const size_t total = (size_t)rows * inter / 2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = (2 * i) / inter, c = (2 * i) % inter;
        const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * inter + c);
        const __nv_bfloat162 u = *reinterpret_cast<const __nv_bfloat162*>(gu + r * 2 * inter + inter + c);
        const float g0 = __low2float(g), g1 = __high2float(g);
        const float a0 = g0 / (1.0f + __expf(-g0)) * __low2float(u), a1 = g1 / (1.0f + __expf(-g1)) * __high2float(u);
        *reinterpret_cast<uint32_t*>(out + r * inter + c) = pack_bf16(a0, a1);
    }
}

// CFG combine + per-row norm rescale + Euler update (imagegen.rs:186-213); one warp per row of lw
__global__ void __launch_bounds__(256)
cfg_euler_kernel(float* __restrict__ latents, const float* __restrict__ cond, const float* __restrict__ uncond,
                 float gs, const float* __restrict__ sched, const int* __restrict__ counter, int rows, int lw, int use_cfg) {
    const float d = sched[2 * *counter + 1];
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const size_t base = (size_t)row * lw;
    if (!use_cfg) {
        for (int c = lane; c < lw; c += 32) latents[base + c] -= d * cond[base + c];
        return;
    }
    float cn = 0.0f, gn = 0.0f;
    for (int c = lane; c < lw; c += 32) {
        const float cv = cond[base + c], uv = uncond[base + c];
        const float g = uv + gs * (cv - uv);
        cn += cv * cv;
        gn += g * g;
    }
    cn = sqrtf(warp_sum(cn));
    gn = sqrtf(warp_sum(gn));
    // use_cfg 1: rescale the guided row to the cond row's norm; 2: guidance without the rescale
    const bool rescale = use_cfg == 1 && gn > 0.0f;
    const float f = rescale ? cn / gn : 1.0f;
    for (int c = lane; c < lw; c += 32) {
        const float cv = cond[base + c], uv = uncond[base + c];
        float g = uv + gs * (cv - uv);
        if (rescale) g *= f;
        latents[base + c] -= d * g;
    }
}

// head-major f32 [heads][n][hd] (the facade's dit_attention layout) -> token-major bf16
__global__ void head_major_to_token_kernel(const float* __restrict__ src, int heads, int n, int hd, float scale,
                                           __nv_bfloat16* __restrict__ dst) {
    const size_t total = (size_t)heads * n * hd;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(i % hd);
        const size_t t = i / hd;
        const int tok = (int)(t % n), h = (int)(t / n);
        dst[((size_t)tok * heads + h) * hd + d] = __float2bfloat16_rn(src[i] * scale);
    }
}

__global__ void add_bias_rows_kernel(float* __restrict__ y, const float* __restrict__ bias, size_t rows, int cols) {
    const size_t total = rows * cols;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        y[i] += bias[i % cols];
}

// Counter-based normal generator: element i of stream `seed` is a pure function of (seed, i),
// so a synthetic tensor is reproducible whatever the launch geometry.  SplitMix64 finalizer
// for the bits, Box-Muller for the transform.
__device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__global__ void fill_normal_kernel(float* __restrict__ out, size_t n, uint64_t seed, float std) {
    const size_t pairs = (n + 1) / 2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < pairs; i += (size_t)gridDim.x * blockDim.x) {
        const uint64_t a = mix64(seed * 0x9E3779B97F4A7C15ull + 2 * i + 1), b = mix64(seed * 0x9E3779B97F4A7C15ull + 2 * i + 2);
        const float u1 = ((float)(a >> 40) + 1.0f) * (1.0f / 16777216.0f);  // (0, 1]
        const float u2 = (float)(b >> 40) * (1.0f / 16777216.0f);
        const float r = sqrtf(-2.0f * logf(u1)) * std;
        float sn, cs;
        sincospif(2.0f * u2, &sn, &cs);
        out[2 * i] = r * cs;
        if (2 * i + 1 < n) out[2 * i + 1] = r * sn;
    }
}

// max over heads of the squared Euclidean norm of bf16 head rows [heads_total][hd] (hd % 8 == 0),
// as the bit pattern of a non-negative float (orders like an unsigned integer)
__global__ void head_norm2_max_kernel(const __nv_bfloat16* __restrict__ x, size_t heads_total, int hd, unsigned* __restrict__ out) {
    float best = 0.0f;
    for (size_t h = blockIdx.x * (size_t)blockDim.x + threadIdx.x; h < heads_total; h += (size_t)gridDim.x * blockDim.x) {
        const uint4* src = reinterpret_cast<const uint4*>(x + h * hd);
        float ss = 0.0f;
        for (int i = 0; i < hd / 8; ++i) {
            const uint4 w = src[i];
            const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float a = __uint_as_float(u[k] << 16), b = __uint_as_float(u[k] & 0xffff0000u);
                ss = fmaf(a, a, fmaf(b, b, ss));
            }
        }
        best = fmaxf(best, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0 && best > 0.0f) atomicMax(out, __float_as_uint(best));
}

}  // namespace

void launch_head_norm2_max(const __nv_bfloat16* x, size_t heads_total, int hd, unsigned* out, cudaStream_t s) {
    size_t g = (heads_total + 255) / 256;
    head_norm2_max_kernel<<<(int)(g > 148 * 8 ? 148 * 8 : (g == 0 ? 1 : g)), 256, 0, s>>>(x, heads_total, hd, out);
}

static inline int grid_for(size_t n, int block) {
    size_t g = (n + block - 1) / block;
    return (int)(g > 148 * 16 ? 148 * 16 : (g == 0 ? 1 : g));
}

void launch_f32_to_bf16(const float* in, __nv_bfloat16* out, size_t n, cudaStream_t s) {
    const size_t n4 = n / 4;
    if (n4) f32_to_bf16_kernel<<<grid_for(n4, 256), 256, 0, s>>>(in, out, n4);
    if (n % 4) f32_to_bf16_tail<<<1, 4, 0, s>>>(in, out, n4 * 4, n);
}
void launch_bf16_to_f32(const __nv_bfloat16* in, float* out, size_t n, cudaStream_t s) {
    bf16_to_f32_kernel<<<grid_for(n, 256), 256, 0, s>>>(in, out, n);
}

void launch_rms_mod(const float* x, const float* w, const float* shift, double eps, int rows, int cols,
                    __nv_bfloat16* out_bf16, float* out_f32, cudaStream_t s) {
    const int grid = (rows + ROW_WARPS - 1) / ROW_WARPS;
    DISPATCH_NV(cols, (rms_mod_kernel<NV><<<grid, 32 * ROW_WARPS, 0, s>>>(x, w, shift, eps, rows, out_bf16, out_f32)));
}
void launch_gated_residual(float* x, const float* src, const float* w, const float* gate, double eps, int rows,
                           int cols, cudaStream_t s) {
    const int grid = (rows + ROW_WARPS - 1) / ROW_WARPS;
    DISPATCH_NV(cols, (residual_kernel<NV, false><<<grid, 32 * ROW_WARPS, 0, s>>>(x, src, w, gate, nullptr, nullptr,
                                                                                  eps, rows, nullptr)));
}
void launch_residual_then_norm(float* x, const float* src, const float* w_res, const float* gate,
                               const float* w_next, const float* shift, double eps, int rows, int cols,
                               __nv_bfloat16* out_bf16, cudaStream_t s) {
    const int grid = (rows + ROW_WARPS - 1) / ROW_WARPS;
    DISPATCH_NV(cols, (residual_kernel<NV, true><<<grid, 32 * ROW_WARPS, 0, s>>>(x, src, w_res, gate, w_next, shift,
                                                                                 eps, rows, out_bf16)));
}
void launch_layernorm_scale(const float* x, const float* scale, int rows, int cols, float* out, cudaStream_t s) {
    const int grid = (rows + ROW_WARPS - 1) / ROW_WARPS;
    DISPATCH_NV(cols, (layernorm_scale_kernel<NV><<<grid, 32 * ROW_WARPS, 0, s>>>(x, scale, rows, out)));
}

bool row_cols_supported(int cols) {
    switch (cols / 128) {
        case 1: case 2: case 4: case 8: case 12: case 16: case 18: case 24: case 32: return cols % 128 == 0;
        default: return false;
    }
}

template <int PPL>
static void rope_launch(int grid, const float* qkv, int n, int nh, int nkv, const float* norm_q, const float* norm_k,
                        const float* cos_t, const float* sin_t, float q_scale, unsigned* norm2_max, __nv_bfloat16* q,
                        __nv_bfloat16* k, cudaStream_t s) {
    if (norm2_max)
        qk_rope_kernel<PPL, true><<<grid, ROPE_THREADS, 0, s>>>(qkv, n, nh, nkv, norm_q, norm_k, cos_t, sin_t, q_scale, q, k, norm2_max);
    else
        qk_rope_kernel<PPL, false><<<grid, ROPE_THREADS, 0, s>>>(qkv, n, nh, nkv, norm_q, norm_k, cos_t, sin_t, q_scale, q, k, nullptr);
}
void launch_qk_rope_pack(const float* qkv, int n, int nh, int nkv, int hd, const float* norm_q,
                         const float* norm_k, const float* cos_t, const float* sin_t, float q_scale, unsigned* norm2_max,
                         __nv_bfloat16* q, __nv_bfloat16* k, cudaStream_t s) {
    const long items = (long)n * ((q ? nh : 0) + nkv);
    const int grid = (int)((items + ROPE_THREADS / 4 - 1) / (ROPE_THREADS / 4));
    switch (hd / 32) {
        case 1: rope_launch<1>(grid, qkv, n, nh, nkv, norm_q, norm_k, cos_t, sin_t, q_scale, norm2_max, q, k, s); break;
        case 2: rope_launch<2>(grid, qkv, n, nh, nkv, norm_q, norm_k, cos_t, sin_t, q_scale, norm2_max, q, k, s); break;
        case 3: rope_launch<3>(grid, qkv, n, nh, nkv, norm_q, norm_k, cos_t, sin_t, q_scale, norm2_max, q, k, s); break;
        case 4: rope_launch<4>(grid, qkv, n, nh, nkv, norm_q, norm_k, cos_t, sin_t, q_scale, norm2_max, q, k, s); break;
        default: break;
    }
}
void launch_interleave_f32(float* dst, int dst_stride, int dst_off, const float* src, size_t count, cudaStream_t s) {
    interleave_f32_kernel<<<grid_for(count, 256), 256, 0, s>>>(dst, dst_stride, dst_off, src, count);
}

void launch_gemv(const GemvParams& p, cudaStream_t s) {
    gemv_kernel<<<(p.rows + 7) / 8, 256, 0, s>>>(p, nullptr);
}
void launch_gemv_silu2(const GemvParams& p, float* y_silu, cudaStream_t s) {
    gemv_kernel<<<(p.rows + 7) / 8, 256, 0, s>>>(p, y_silu);
}
void launch_sgemm_nt_bias(const float* a, const float* w, const float* bias, float* y, int M, int N, int K,
                          cudaStream_t s) {
    dim3 g((N + 63) / 64, (M + 63) / 64);
    sgemm_nt_kernel<<<g, 256, 0, s>>>(a, w, bias, y, M, N, K);
}
__global__ void advance_step_kernel(int* counter) { *counter += 1; }
void launch_time_freqs(const float* sched, const int* counter, float* out256, cudaStream_t s) {
    time_freqs_kernel<<<1, 128, 0, s>>>(sched, counter, out256);
}
void launch_advance_step(int* counter, cudaStream_t s) { advance_step_kernel<<<1, 1, 0, s>>>(counter); }
void launch_patchify(const float* latent, int c, int h, int w, int p, float* tok, cudaStream_t s) {
    patchify_kernel<<<grid_for((size_t)c * h * w, 256), 256, 0, s>>>(latent, c, h, w, p, tok, 0, nullptr);
}
void launch_unpatchify(const float* tok, int c, int h, int w, int p, float* latent, cudaStream_t s) {
    patchify_kernel<<<grid_for((size_t)c * h * w, 256), 256, 0, s>>>(nullptr, c, h, w, p, const_cast<float*>(tok), 1,
                                                                     latent);
}
void launch_silu_mul(const __nv_bfloat16* gu, int rows, int inter, __nv_bfloat16* out, cudaStream_t s) {
    silu_mul_kernel<<<grid_for((size_t)rows * inter / 2, 256), 256, 0, s>>>(gu, rows, inter, out);
}
void launch_cfg_euler(float* latents, const float* cond, const float* uncond, float gs, const float* sched,
                      const int* counter, int rows, int lw, int use_cfg, cudaStream_t s) {
    cfg_euler_kernel<<<(rows + 7) / 8, 256, 0, s>>>(latents, cond, uncond, gs, sched, counter, rows, lw, use_cfg);
}
void launch_add_bias_rows(float* y, const float* bias, size_t rows, int cols, cudaStream_t s) {
    add_bias_rows_kernel<<<grid_for(rows * cols, 256), 256, 0, s>>>(y, bias, rows, cols);
}
void launch_fill_normal(float* out, size_t n, uint64_t seed, float std, cudaStream_t s) {
    fill_normal_kernel<<<grid_for((n + 1) / 2, 256), 256, 0, s>>>(out, n, seed, std);
}
void launch_transpose_head_major(const float* src, int heads, int n, int hd, float scale, __nv_bfloat16* dst,
                                 cudaStream_t s) {
    head_major_to_token_kernel<<<grid_for((size_t)heads * n * hd, 256), 256, 0, s>>>(src, heads, n, hd, scale, dst);
}

}  // namespace cmfc
