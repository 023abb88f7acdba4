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

// nibble at bit position p of ``w`` -> exact f32 (nib-8)*s: the nibble is OR-ed into the
// mantissa of 2^23, the bias (2^23 + 8*2^p) is subtracted exactly, and the result is scaled
// by s*2^-p (a power-of-two rescale, so the single rounding equals that of (nib-8)*s).
template <int P>
__device__ __forceinline__ float nib_times(uint32_t w, float s_shifted) {
    float f = __uint_as_float((w & (0xFu << P)) | 0x4B000000u);
    f = __fsub_rn(f, 8388608.0f + 8.0f * (float)(1u << P));
    return __fmul_rn(f, s_shifted);
}

struct Q4Scales {
    float s0, s4, s8, s12, s16;
    __device__ __forceinline__ explicit Q4Scales(float s)
        : s0(s), s4(s * 0.0625f), s8(s * 0.00390625f), s12(s * 0.000244140625f), s16(s * 1.52587890625e-05f) {}
};

// One plane word (elements 0..7 at nibble positions 0,4,1,5,2,6,3,7) -> four bf16x2 registers.
// f32 route, any f32 scale (q4tp ladder scales): exact product, one rounding to bf16.
__device__ __forceinline__ void unpack_q4_word(uint32_t w, const Q4Scales& sc, uint32_t* o) {
    uint32_t hi = w >> 12;  // positions 4..7 -> bits 4, 8, 12, 16
    o[0] = pack_bf16(nib_times<0>(w, sc.s0), nib_times<4>(hi, sc.s4));
    o[1] = pack_bf16(nib_times<4>(w, sc.s4), nib_times<8>(hi, sc.s8));
    o[2] = pack_bf16(nib_times<8>(w, sc.s8), nib_times<12>(hi, sc.s12));
    o[3] = pack_bf16(nib_times<12>(w, sc.s12), nib_times<16>(hi, sc.s16));
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
