// Register-level pieces shared by the dequant GEMM kernels: unpacking of packed weight words to
// bf16x2 operands (bit-exact RN_bf16 of the reference dequantization) and the fused activations.
#pragma once
#include "common.cuh"

namespace cmfc {
namespace gemm_detail {

// ---- register unpack: 32 consecutive k of one weight row -> 16 packed bf16x2 ----

// int8 -> bf16 without a conversion instruction: for byte b, 0x4300|(b&0x7f) is the bf16
// 128+(b&0x7f) and 0x4300|(b&0x80) is 128 or 256; their difference is the signed level.
__device__ __forceinline__ void unpack_q8_word(uint32_t w, uint32_t& o0, uint32_t& o1) {
    uint32_t t0 = __byte_perm(w, 0u, 0x4140);
    uint32_t t1 = __byte_perm(w, 0u, 0x4342);
    uint32_t v0 = (t0 & 0x007f007fu) | 0x43004300u, c0 = (t0 & 0x00800080u) | 0x43004300u;
    uint32_t v1 = (t1 & 0x007f007fu) | 0x43004300u, c1 = (t1 & 0x00800080u) | 0x43004300u;
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(o0) : "r"(v0), "r"(c0));
    asm("sub.bf16x2 %0, %1, %2;" : "=r"(o1) : "r"(v1), "r"(c1));
}

// Nibble at bit position P (a multiple of 4, at most 16) of a word -> the f32 value of the signed
// level t = nib - 8: the nibble is OR-ed into the mantissa of 2^(23-P), which makes the float
// 2^(23-P) + nib exactly, and 2^(23-P) + 8 is subtracted exactly.  The exponent constant depends on
// the position, so every position yields t itself and ONE multiply by the group's f32 scale is the
// reference's own product (nib - 8) * s with its single rounding (crates/cortiq-core/src/quant.rs:413-431).
// Subtract and multiply are packed f32x2 operations (IEEE round to nearest per lane, one issue slot
// for the pair).
template <int P>
__device__ __forceinline__ float nib_as_float(uint32_t w) {
    static_assert(P % 4 == 0 && P <= 16, "the nibble must stay inside the mantissa");
    return __uint_as_float((w & (0xFu << P)) | ((uint32_t)(150 - P) << 23));
}
template <int P>
__device__ __forceinline__ constexpr float nib_bias() { return -((float)(1u << (23 - P)) + 8.0f); }

template <int PA, int PB>
__device__ __forceinline__ uint32_t nib_pair_times(uint32_t wa, uint32_t wb, uint64_t s2) {
    const uint64_t f = pack_f32x2(nib_as_float<PA>(wa), nib_as_float<PB>(wb));
    const uint64_t t = add_f32x2(f, pack_f32x2(nib_bias<PA>(), nib_bias<PB>()));
    float lo, hi;
    unpack_f32x2(mul_f32x2(t, s2), lo, hi);
    return pack_bf16(lo, hi);
}

struct Q4Scales {
    uint64_t s2;  // (s, s)
    __device__ __forceinline__ explicit Q4Scales(float s) : s2(pack_f32x2(s, s)) {}
};

// One plane word (elements 0..7 at nibble positions 0,4,1,5,2,6,3,7) -> four bf16x2 registers.
// f32 route, any f32 scale (q4tp ladder scales): exact product, one rounding to bf16.
__device__ __forceinline__ void unpack_q4_word(uint32_t w, const Q4Scales& sc, uint32_t* o) {
    const uint32_t hi = w >> 12;  // positions 4..7 -> bits 4, 8, 12, 16
    o[0] = nib_pair_times<0, 4>(w, hi, sc.s2);
    o[1] = nib_pair_times<4, 8>(w, hi, sc.s2);
    o[2] = nib_pair_times<8, 12>(w, hi, sc.s2);
    o[3] = nib_pair_times<12, 16>(w, hi, sc.s2);
}

// bf16x2 route for q4_tiled, whose scale is an f16 value s = hi + lo with hi (8 significant bits)
// and lo (3 bits) both exact bf16: t = nib - 8 is exact, t*lo is exact (at most 7 bits), and
// fma.rn(t, hi, t*lo) rounds the exact product t*s once -- the same bits as the f32 route.
__device__ __forceinline__ void unpack_q4t_word(uint32_t w, uint32_t hi2, uint32_t lo2, uint32_t* o) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t m = ((w >> (4 * i)) & 0x000f000fu) | 0x43004300u;  // bf16 128 + nib, twice
        uint32_t t, c;
        asm("sub.bf16x2 %0, %1, %2;" : "=r"(t) : "r"(m), "r"(0x43084308u));  // - 136
        asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(c) : "r"(t), "r"(lo2));
        asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(o[i]) : "r"(t), "r"(hi2), "r"(c));
    }
}

__device__ __forceinline__ uint4 lds128(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }

// Epilogue of the fused QKV projection for a V channel: 32 consecutive tokens (mb .. mb+31) of one
// output channel go straight into that channel's row of V^T (bf16, [channels, vt_pitch]), the
// layout the attention kernel's P.V product reads, instead of an f32 matrix that a second pass
// would transpose.  seg_table: [nseg+1] token offsets of the segments, then [nseg] first V^T column
// of each segment (a multiple of 8).  A chunk that lies inside one segment at a 16-byte aligned
// column is four 16-byte stores; otherwise token by token.
__device__ __forceinline__ void emit_vt_chunk(const uint32_t (&v)[32], float rs, int mb, int M, __nv_bfloat16* vrow,
                                              const int* __restrict__ seg_table, int nseg) {
    int z = 0;
    while (z + 1 < nseg && seg_table[z + 1] <= mb) ++z;
    int seg1 = seg_table[z + 1];
    int shift = seg_table[nseg + 1 + z] - seg_table[z];  // column = token + shift inside segment z
    if (mb + 32 <= seg1 && ((mb + shift) & 7) == 0) {
        uint4* dst = reinterpret_cast<uint4*>(vrow + mb + shift);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 o;
            o.x = pack_bf16(__uint_as_float(v[8 * q + 0]) * rs, __uint_as_float(v[8 * q + 1]) * rs);
            o.y = pack_bf16(__uint_as_float(v[8 * q + 2]) * rs, __uint_as_float(v[8 * q + 3]) * rs);
            o.z = pack_bf16(__uint_as_float(v[8 * q + 4]) * rs, __uint_as_float(v[8 * q + 5]) * rs);
            o.w = pack_bf16(__uint_as_float(v[8 * q + 6]) * rs, __uint_as_float(v[8 * q + 7]) * rs);
            dst[q] = o;
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {  // unrolled: v[] stays in registers
        const int m = mb + j;
        if (m < M) {
            while (m >= seg1) {  // m < M = seg_table[nseg], so z stays in range
                ++z;
                seg1 = seg_table[z + 1];
                shift = seg_table[nseg + 1 + z] - seg_table[z];
            }
            vrow[m + shift] = __float2bfloat16_rn(__uint_as_float(v[j]) * rs);
        }
    }
}

// silu(v) = v * sigmoid(v) with sigmoid(v) = 0.5 * tanh(v / 2) + 0.5: one special-function op
// (tanh.approx, relative error about 2^-11) instead of an exp2 and a reciprocal; the product is
// rounded to bf16 (2^-9) right after.
__device__ __forceinline__ float silu_f(float v) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * v));
    return v * fmaf(t, 0.5f, 0.5f);
}
// crates/cortiq-engine/src/textenc.rs:70-73
__device__ __forceinline__ float gelu_tanh_f(float v) {
    return 0.5f * v * (1.0f + tanhf(0.7978846f * (v + 0.044715f * v * v * v)));
}

}  // namespace gemm_detail
}  // namespace cmfc
