// Codec kernels: container payloads -> GEMM planes, planes -> exact f32 weights (the
// bit-exactness check), and device-side quantizers that reproduce the reference encoders
// byte for byte (crates/cortiq-cli/src/convert.rs:36-47, :551-613, :883-992;
// dequantizers crates/cortiq-core/src/quant.rs:91-103, :322-344, :396-431).
//
// Everything here uses explicitly rounded IEEE operations (__fdiv_rn, __fmul_rn, ...) so the
// compiler cannot contract a*b+c, and takes log2f / exp2f values from host-built tables
// indexed by f16 bit pattern (the only arguments those functions ever see on this path).
#include "common.cuh"
#include "kernels.h"

namespace cmfc {
namespace {

__device__ __forceinline__ float half_bits_to_f32(uint16_t h) { return __half2float(__ushort_as_half(h)); }

// f32 -> f16 bits with the reference's rounding: nearest-even for normal results, half-up for
// subnormal results (crates/cortiq-core/src/quant.rs:50-82).
__device__ __forceinline__ uint16_t f32_to_half_bits(float x) {
    const uint32_t bits = __float_as_uint(x);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int e = (int)((bits >> 23) & 0xFFu);
    const uint32_t m = bits & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0u));
    e -= 112;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return sign;
        const uint32_t full = m | 0x800000u;
        const uint32_t sh = (uint32_t)(14 - e);
        return (uint16_t)(sign | (uint16_t)((full >> sh) + ((full >> (sh - 1)) & 1u)));
    }
    const uint32_t half = ((uint32_t)e << 10) | (m >> 13);
    const uint32_t bump = ((m >> 12) & 1u) & ((uint32_t)((m & 0xFFFu) != 0) | (half & 1u));
    return (uint16_t)(sign | (uint16_t)(half + bump));
}

__device__ __forceinline__ float f16_scale(float raw) {
    return fmaxf(half_bits_to_f32(f32_to_half_bits(raw)), 6.1035156e-5f);
}
__device__ __forceinline__ float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

// ---- payload -> planes ----

// Nibble order inside every 32-bit word of a GEMM nibble plane.  The container stores element e
// of a word at nibble position e.  The plane stores elements (0,1,2,...,7) at positions
// (0,4,1,5,2,6,3,7): then (w >> 4i) & 0x000f000f holds the ADJACENT elements 2i (low half) and
// 2i+1 (high half), which is what a packed bf16x2 operand register needs.
__host__ __device__ __forceinline__ uint32_t permute_nibbles(uint32_t w) {
    uint32_t o = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const int pos = (e >> 1) + ((e & 1) << 2);
        o |= ((w >> (4 * e)) & 0xFu) << (4 * pos);
    }
    return o;
}
__host__ __device__ __forceinline__ uint32_t plane_nibble(uint32_t word, int e) {
    return (word >> (4 * ((e >> 1) + ((e & 1) << 2)))) & 0xFu;
}

// q4_tiled 18-byte tiles -> permuted nibble plane [rows, cols/2] + transposed group scales
// [cols/32, rows].  The f16 scale s is stored as two bf16 halves of one 32-bit word:
// hi = s truncated to 8 significant bits (low half), lo = s - hi (high half), both exact, so
// fma.bf16x2(t, hi, t*lo) rounds the exact product t*s once.
__global__ void q4t_split_kernel(const uint8_t* __restrict__ raw, int rows, int gpr, uint8_t* __restrict__ nib,
                                 float* __restrict__ scales_t) {
    const size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (g >= (size_t)rows * gpr) return;
    const uint16_t* t = reinterpret_cast<const uint16_t*>(raw + g * 18);
    const int r = (int)(g / gpr), gi = (int)(g % gpr);
    const float s = half_bits_to_f32(t[0]);
    const uint32_t hi_bits = __float_as_uint(s) & 0xFFFF0000u;
    const float lo = __fsub_rn(s, __uint_as_float(hi_bits));
    const uint32_t packed = (hi_bits >> 16) | (__float_as_uint(lo) & 0xFFFF0000u);
    reinterpret_cast<uint32_t*>(scales_t)[(size_t)gi * rows + r] = packed;
    uint32_t* dst = reinterpret_cast<uint32_t*>(nib + g * 16);
#pragma unroll
    for (int k = 0; k < 4; ++k) dst[k] = permute_nibbles((uint32_t)t[1 + 2 * k] | ((uint32_t)t[2 + 2 * k] << 16));
}

__global__ void permute_plane_kernel(uint32_t* __restrict__ words, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        words[i] = permute_nibbles(words[i]);
}

// q4tp 5-bit codes (LSB-first per row) + per-row ladders -> transposed f32 scales
__global__ void q4tp_scales_kernel(const uint8_t* __restrict__ codes, int stride, const float* __restrict__ ladders,
                                   int rows, int gpr, float* __restrict__ scales_t) {
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * gpr) return;
    const int r = (int)(i % rows), g = (int)(i / rows);
    const uint8_t* c = codes + (size_t)r * stride;
    const int bit = g * 5, b = bit >> 3, sh = bit & 7;
    uint32_t v = c[b];
    if (sh > 3 && b + 1 < stride) v |= (uint32_t)c[b + 1] << 8;
    scales_t[(size_t)g * rows + r] = ladders[(size_t)r * 32 + ((v >> sh) & 0x1Fu)];
}

__global__ void f16_to_f32_kernel(const uint16_t* __restrict__ h, float* __restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = half_bits_to_f32(h[i]);
}

// ---- planes -> exact f32 weights ----
__global__ void dequant_q8_kernel(const int8_t* __restrict__ q, const float* __restrict__ row_scale, int rows,
                                  int cols, float* __restrict__ out) {
    const size_t total = (size_t)rows * cols;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        out[i] = __fmul_rn((float)q[i], row_scale[i / cols]);
}
// split_scales: 1 = q4t planes (bf16 hi/lo scale halves), 0 = q4tp planes (f32 ladder scales)
__global__ void dequant_q4_kernel(const uint8_t* __restrict__ nib, const float* __restrict__ scales_t, int rows,
                                  int cols, int split_scales, float* __restrict__ out) {
    const size_t total = (size_t)rows * cols / 8;  // one plane word -> eight weights
    const uint32_t* words = reinterpret_cast<const uint32_t*>(nib);
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = (8 * i) / cols, c = (8 * i) % cols;
        float s = scales_t[(c / 32) * rows + r];
        if (split_scales) {
            const uint32_t u = __float_as_uint(s);
            s = __fadd_rn(__uint_as_float(u << 16), __uint_as_float(u & 0xFFFF0000u));  // hi + lo, exact
        }
        const uint32_t w = words[i];
#pragma unroll
        for (int e = 0; e < 8; ++e) out[8 * i + e] = __fmul_rn((float)plane_nibble(w, e) - 8.0f, s);
    }
}

// ---- encoders ----
__global__ void __launch_bounds__(256)
encode_q8_row_kernel(const float* __restrict__ w, int rows, int cols, uint8_t* __restrict__ payload) {
    __shared__ float red[8];
    const int r = blockIdx.x;
    const float* row = w + (size_t)r * cols;
    float m = 0.0f;
    for (int c = threadIdx.x; c < cols; c += 256) m = fmaxf(m, fabsf(row[c]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
    const float s = f16_scale(__fdiv_rn(m, 127.0f));
    for (int c = threadIdx.x; c < cols; c += 256)
        payload[(size_t)r * cols + c] = (uint8_t)(int8_t)clampf(rintf(__fdiv_rn(row[c], s)), -128.0f, 127.0f);
    if (threadIdx.x == 0)
        reinterpret_cast<uint16_t*>(payload + (size_t)rows * cols)[r] = f32_to_half_bits(s);
}

// one 32-group -> 16 nibble bytes; DIVIDE: q = rint(v / s) else q = rint(v * s)
template <bool DIVIDE>
__device__ __forceinline__ void pack_group(const float* g, float s, uint8_t* dst) {
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const float a = DIVIDE ? __fdiv_rn(g[2 * k], s) : __fmul_rn(g[2 * k], s);
        const float b = DIVIDE ? __fdiv_rn(g[2 * k + 1], s) : __fmul_rn(g[2 * k + 1], s);
        const uint8_t q0 = (uint8_t)((int)clampf(rintf(a), -8.0f, 7.0f) + 8);
        const uint8_t q1 = (uint8_t)((int)clampf(rintf(b), -8.0f, 7.0f) + 8);
        dst[k] = (uint8_t)((q0 & 0x0F) | (q1 << 4));
    }
}

__global__ void encode_q4_tiled_kernel(const float* __restrict__ w, size_t groups, uint8_t* __restrict__ payload) {
    const size_t g = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (g >= groups) return;
    float v[32];
    float m = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float4 t = *reinterpret_cast<const float4*>(w + g * 32 + 4 * k);
        v[4 * k] = t.x; v[4 * k + 1] = t.y; v[4 * k + 2] = t.z; v[4 * k + 3] = t.w;
        m = fmaxf(m, fmaxf(fmaxf(fabsf(t.x), fabsf(t.y)), fmaxf(fabsf(t.z), fabsf(t.w))));
    }
    const float s = f16_scale(__fdiv_rn(m, 7.0f));
    uint8_t nib[16];
    pack_group<true>(v, s, nib);
    uint16_t* dst = reinterpret_cast<uint16_t*>(payload + g * 18);
    dst[0] = f32_to_half_bits(s);
#pragma unroll
    for (int k = 0; k < 8; ++k) dst[1 + k] = (uint16_t)(nib[2 * k] | (nib[2 * k + 1] << 8));
}

// q4tp: one block per row, one thread per 32-group (strided when gpr > blockDim).
__global__ void __launch_bounds__(128)
encode_q4tp_kernel(const float* __restrict__ w, int rows, int cols, uint8_t* __restrict__ payload,
                   const float* __restrict__ log2_lut, const float* __restrict__ exp2_lut) {
    extern __shared__ uint8_t sm[];
    const int gpr = cols / 32;
    float* lg = reinterpret_cast<float*>(sm);                 // [gpr]
    uint8_t* dead = sm + (size_t)gpr * 4;                     // [gpr]
    uint8_t* code = dead + gpr;                               // [gpr]
    __shared__ float red_lo[4], red_hi[4], tab[32];
    __shared__ float s_lo_r, s_st;
    const int r = blockIdx.x;
    const float* row = w + (size_t)r * cols;
    const int stride = (gpr * 5 + 7) / 8;
    uint8_t* nib_plane = payload;
    uint8_t* params = payload + (size_t)rows * gpr * 16;
    uint8_t* codes = params + (size_t)rows * 4;

    float lo = INFINITY, hi = -INFINITY;
    for (int g = threadIdx.x; g < gpr; g += blockDim.x) {
        float m = 0.0f;
        for (int k = 0; k < 32; ++k) m = fmaxf(m, fabsf(row[g * 32 + k]));
        dead[g] = (m == 0.0f);
        const float sc = f16_scale(__fdiv_rn(m, 7.0f));
        lg[g] = log2_lut[f32_to_half_bits(sc)];
        if (!dead[g]) { lo = fminf(lo, lg[g]); hi = fmaxf(hi, lg[g]); }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    if ((threadIdx.x & 31) == 0) { red_lo[threadIdx.x >> 5] = lo; red_hi[threadIdx.x >> 5] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) { lo = fminf(lo, red_lo[i]); hi = fmaxf(hi, red_hi[i]); }
        lo = fminf(lo, red_lo[0]); hi = fmaxf(hi, red_hi[0]);
        if (!isfinite(lo)) { lo = lg[0]; hi = lo; }
        const uint16_t lo_h = f32_to_half_bits(lo);
        const float lo_r = half_bits_to_f32(lo_h);
        float span = __fsub_rn(hi, lo_r);
        if (!(span > 0.0f)) span = 0.0f;
        uint16_t st_h = f32_to_half_bits(__fdiv_rn(span, 31.0f));
        for (int it = 0; it < 64; ++it) {
            const float st = half_bits_to_f32(st_h);
            if (st > 0.0f && __fadd_rn(lo_r, __fmul_rn(31.0f, st)) >= hi) break;
            st_h = (uint16_t)(st_h + 1);
        }
        reinterpret_cast<uint16_t*>(params)[2 * r] = lo_h;
        reinterpret_cast<uint16_t*>(params)[2 * r + 1] = st_h;
        s_lo_r = lo_r;
        s_st = half_bits_to_f32(st_h);
        const float ratio = exp2_lut[st_h];
        float t = exp2_lut[lo_h];
        tab[0] = t;
        for (int c = 1; c < 32; ++c) { t = __fmul_rn(t, ratio); tab[c] = t; }
    }
    __syncthreads();
    const float lo_r = s_lo_r, st = s_st;
    for (int g = threadIdx.x; g < gpr; g += blockDim.x) {
        float tile[32];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float4 t = *reinterpret_cast<const float4*>(row + g * 32 + 4 * k);
            tile[4 * k] = t.x; tile[4 * k + 1] = t.y; tile[4 * k + 2] = t.z; tile[4 * k + 3] = t.w;
        }
        const bool frozen = dead[g] || !(st > 0.0f);
        int nominal = 0;
        if (!frozen) nominal = (int)clampf(rintf(__fdiv_rn(__fsub_rn(lg[g], lo_r), st)), 0.0f, 31.0f);
        int pick = nominal;
        if (!frozen) {
            float best = INFINITY;
            const int from = nominal >= 2 ? nominal - 2 : 0, to = nominal + 1 < 31 ? nominal + 1 : 31;
            for (int cand = from; cand <= to; ++cand) {
                const float sc = tab[cand];
                if (!(sc > 0.0f)) continue;
                const float iv = __fdiv_rn(1.0f, sc);
                float err = 0.0f;
#pragma unroll
                for (int k = 0; k < 32; ++k) {
                    const float q = clampf(rintf(__fmul_rn(tile[k], iv)), -8.0f, 7.0f);
                    const float d = __fsub_rn(tile[k], __fmul_rn(q, sc));
                    err = __fadd_rn(err, __fmul_rn(d, d));
                }
                if (err < best) { best = err; pick = cand; }
            }
        }
        code[g] = (uint8_t)pick;
        const float inv = tab[pick] > 0.0f ? __fdiv_rn(1.0f, tab[pick]) : 0.0f;
        uint8_t nb[16];
        pack_group<false>(tile, inv, nb);
        uint4 o;
        o.x = nb[0] | (nb[1] << 8) | (nb[2] << 16) | ((uint32_t)nb[3] << 24);
        o.y = nb[4] | (nb[5] << 8) | (nb[6] << 16) | ((uint32_t)nb[7] << 24);
        o.z = nb[8] | (nb[9] << 8) | (nb[10] << 16) | ((uint32_t)nb[11] << 24);
        o.w = nb[12] | (nb[13] << 8) | (nb[14] << 16) | ((uint32_t)nb[15] << 24);
        *reinterpret_cast<uint4*>(nib_plane + ((size_t)r * gpr + g) * 16) = o;
    }
    __syncthreads();
    // pack the 5-bit codes LSB-first; each thread builds whole output bytes
    uint8_t* crow = codes + (size_t)r * stride;
    for (int b = threadIdx.x; b < stride; b += blockDim.x) {
        uint32_t v = 0;
        const int first = (b * 8) / 5;  // first code overlapping this byte
        for (int g = first; g < gpr && g * 5 < b * 8 + 8; ++g) {
            const int bit = g * 5 - b * 8;  // may be negative
            const uint32_t cv = code[g];
            v |= bit >= 0 ? (cv << bit) : (cv >> (-bit));
        }
        crow[b] = (uint8_t)v;
    }
}

__global__ void v_head_major_to_vt_kernel(const float* __restrict__ v, int nkv, int n, int hd,
                                          __nv_bfloat16* __restrict__ vt, int pitch) {
    // vt[(h*hd + d), tok] = v[h][tok][d]; 32x32 tiles through shared memory
    __shared__ float tile[32][33];
    const int t0 = blockIdx.x * 32, d0 = blockIdx.y * 32, h = blockIdx.z;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8) {
        const int tok = t0 + r;
        tile[r][tx] = (tok < n && d0 + tx < hd) ? v[((size_t)h * n + tok) * hd + d0 + tx] : 0.0f;
    }
    __syncthreads();
    for (int r = ty; r < 32; r += 8) {
        const int d = d0 + r, tok = t0 + tx;
        if (d < hd && tok < pitch) vt[((size_t)h * hd + d) * pitch + tok] = __float2bfloat16_rn(tile[tx][r]);
    }
}

}  // namespace

static inline int blocks_for(size_t n, int block) { return (int)((n + block - 1) / block); }
static inline int capped(size_t n, int block) {
    size_t g = (n + block - 1) / block;
    return (int)(g > 148 * 32 ? 148 * 32 : (g ? g : 1));
}

void launch_q4t_split(const uint8_t* raw, int rows, int cols, uint8_t* nib, float* scales_t, cudaStream_t s) {
    const int gpr = cols / 32;
    q4t_split_kernel<<<blocks_for((size_t)rows * gpr, 256), 256, 0, s>>>(raw, rows, gpr, nib, scales_t);
}
void launch_q4tp_scales(const uint8_t* codes, int code_stride, const float* ladders, int rows, int gpr,
                        float* scales_t, cudaStream_t s) {
    q4tp_scales_kernel<<<blocks_for((size_t)rows * gpr, 256), 256, 0, s>>>(codes, code_stride, ladders, rows, gpr,
                                                                          scales_t);
}
void launch_f16_to_f32(const uint16_t* h, float* out, int n, cudaStream_t s) {
    f16_to_f32_kernel<<<blocks_for(n, 256), 256, 0, s>>>(h, out, n);
}
void launch_dequant_q8(const int8_t* q, const float* row_scale, int rows, int cols, float* out, cudaStream_t s) {
    dequant_q8_kernel<<<capped((size_t)rows * cols, 256), 256, 0, s>>>(q, row_scale, rows, cols, out);
}
void launch_dequant_q4(const uint8_t* nib, const float* scales_t, int rows, int cols, int split_scales, float* out,
                       cudaStream_t s) {
    dequant_q4_kernel<<<capped((size_t)rows * cols / 8, 256), 256, 0, s>>>(nib, scales_t, rows, cols, split_scales, out);
}
void launch_permute_plane(uint8_t* nib, size_t bytes, cudaStream_t s) {
    permute_plane_kernel<<<capped(bytes / 4, 256), 256, 0, s>>>(reinterpret_cast<uint32_t*>(nib), bytes / 4);
}
void launch_encode_q8_row(const float* w, int rows, int cols, uint8_t* payload, cudaStream_t s) {
    encode_q8_row_kernel<<<rows, 256, 0, s>>>(w, rows, cols, payload);
}
void launch_encode_q4_tiled(const float* w, int rows, int cols, uint8_t* payload, cudaStream_t s) {
    const size_t groups = (size_t)rows * cols / 32;
    encode_q4_tiled_kernel<<<blocks_for(groups, 128), 128, 0, s>>>(w, groups, payload);
}
void launch_encode_q4tp(const float* w, int rows, int cols, uint8_t* payload, const float* log2_lut,
                        const float* exp2_lut, cudaStream_t s) {
    const int gpr = cols / 32;
    encode_q4tp_kernel<<<rows, 128, (size_t)gpr * 6, s>>>(w, rows, cols, payload, log2_lut, exp2_lut);
}
void launch_v_head_major_to_vt(const float* v, int nkv, int n, int hd, __nv_bfloat16* vt, int vt_pitch,
                               cudaStream_t s) {
    dim3 g((vt_pitch + 31) / 32, (hd + 31) / 32, nkv);
    v_head_major_to_vt_kernel<<<g, 256, 0, s>>>(v, nkv, n, hd, vt, vt_pitch);
}

}  // namespace cmfc
