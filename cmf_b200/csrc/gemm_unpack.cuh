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

// Nibbles at bit positions PA of ``wa`` and PB of ``wb`` -> the bf16 pair of the exact f32 products
// (nib-8)*s: each nibble is OR-ed into the mantissa of 2^23, the bias (2^23 + 8*2^P) is subtracted
// exactly, and the result is scaled by s*2^-P (a power-of-two rescale, so the single rounding
// equals that of (nib-8)*s).  Subtract and multiply are packed f32x2 operations (IEEE round to
// nearest per lane, one issue slot for the pair).
template <int PA, int PB>
__device__ __forceinline__ uint32_t nib_pair_times(uint32_t wa, uint32_t wb, uint64_t s_shifted) {
    const uint64_t f = pack_f32x2(__uint_as_float((wa & (0xFu << PA)) | 0x4B000000u),
                                  __uint_as_float((wb & (0xFu << PB)) | 0x4B000000u));
    const uint64_t d = add_f32x2(f, pack_f32x2(-(8388608.0f + 8.0f * (float)(1u << PA)),
                                               -(8388608.0f + 8.0f * (float)(1u << PB))));
    float lo, hi;
    unpack_f32x2(mul_f32x2(d, s_shifted), lo, hi);
    return pack_bf16(lo, hi);
}

struct Q4Scales {
    uint64_t s0_4, s4_8, s8_12, s12_16;  // (s * 2^-a, s * 2^-b) pairs
    __device__ __forceinline__ explicit Q4Scales(float s) {
        const float s4 = s * 0.0625f, s8 = s * 0.00390625f, s12 = s * 0.000244140625f, s16 = s * 1.52587890625e-05f;
        s0_4 = pack_f32x2(s, s4);
        s4_8 = pack_f32x2(s4, s8);
        s8_12 = pack_f32x2(s8, s12);
        s12_16 = pack_f32x2(s12, s16);
    }
};

// One plane word (elements 0..7 at nibble positions 0,4,1,5,2,6,3,7) -> four bf16x2 registers.
// f32 route, any f32 scale (q4tp ladder scales): exact product, one rounding to bf16.
__device__ __forceinline__ void unpack_q4_word(uint32_t w, const Q4Scales& sc, uint32_t* o) {
    const uint32_t hi = w >> 12;  // positions 4..7 -> bits 4, 8, 12, 16
    o[0] = nib_pair_times<0, 4>(w, hi, sc.s0_4);
    o[1] = nib_pair_times<4, 8>(w, hi, sc.s4_8);
    o[2] = nib_pair_times<8, 12>(w, hi, sc.s8_12);
    o[3] = nib_pair_times<12, 16>(w, hi, sc.s12_16);
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
