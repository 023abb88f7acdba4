/*
 * CPU oracle for the CMF NextDiT hot path: codecs and strict-f32 linear kernels.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing that ships links or calls this file; it exists so the
 * CUDA library can be checked against an independent restatement of the reference's CPU
 * arithmetic.  Every function names the reference source it restates (paths are relative
 * to the reference repository root).
 *
 * Built with -ffp-contract=off: the reference (Rust) never contracts a*b+c into an FMA, and
 * byte-exact encoder output depends on that.
 *
 * Parity status: f16 conversion pinned by the reference's known-answer values
 * (crates/cortiq-core/src/quant.rs:871-891); encode_q8_row / encode_q4_block and the q8 /
 * q4_tiled dequantizers pinned byte-for-byte against the reference's own numpy encoders and
 * reader (converter/convert_dtgma_to_cmf.py:94-204, python/cmf_reader.py) through committed
 * golden fixtures; q4tp decode pinned by the reference's property tests
 * (crates/cortiq-cli/src/convert.rs:4413-4484).  encode_q4tp has no second implementation
 * in the reference, so its *encoded bytes* are "parity unpinned" (its decode is pinned).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define GROUP 32
#define Q4_TILE_BYTES 18
#define Q4TP_NIB_BYTES 16
#define Q4TP_TOP_RUNG 31

/* ---- half precision <-> single (crates/cortiq-core/src/quant.rs:18-82) ---- */

float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) << 31;
    uint32_t e = (h >> 10) & 0x1Fu;
    uint32_t m = h & 0x3FFu;
    uint32_t bits;
    if (e == 0) {
        if (m == 0) {
            bits = sign;
        } else {
            /* subnormal half = m * 2^-24: shift the top set bit up to bit 10 */
            uint32_t shifts = 0;
            while (!(m & 0x400u)) { m <<= 1; ++shifts; }
            bits = sign | ((113u - shifts) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 0x1Fu) {
        bits = sign | 0x7F800000u | (m << 13);
    } else {
        bits = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

uint16_t orc_f32_to_f16(float x) {
    uint32_t bits;
    memcpy(&bits, &x, 4);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    int32_t e = (int32_t)((bits >> 23) & 0xFFu);
    uint32_t m = bits & 0x7FFFFFu;
    if (e == 0xFF) return (uint16_t)(sign | 0x7C00u | (m ? 0x200u : 0u));
    e -= 112;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return sign;
        /* subnormal result: the reference rounds half-up here (not ties-even) */
        uint32_t full = m | 0x800000u;
        uint32_t sh = (uint32_t)(14 - e);
        uint32_t half = full >> sh;
        uint32_t rnd = (full >> (sh - 1)) & 1u;
        return (uint16_t)(sign | (uint16_t)(half + rnd));
    }
    uint32_t half = ((uint32_t)e << 10) | (m >> 13);
    uint32_t rnd = (m >> 12) & 1u;
    uint32_t sticky = (m & 0xFFFu) != 0;
    uint32_t bump = rnd & (sticky | (half & 1u));
    return (uint16_t)(sign | (uint16_t)(half + bump));
}

/* crates/cortiq-cli/src/convert.rs:36-47: scale rounded through f16, floored at the
 * smallest normal half. */
static const float F16_FLOOR = 6.1035156e-5f;

float orc_f16_scale(float raw) {
    float r = orc_f16_to_f32(orc_f32_to_f16(raw));
    return r > F16_FLOOR ? r : F16_FLOOR; /* f32::max semantics for non-NaN input */
}

static inline float absmax_of(const float *v, size_t n) {
    float m = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float a = fabsf(v[i]);
        if (a > m) m = a;
    }
    return m;
}

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

static inline void put_u16(uint8_t *p, uint16_t v) { p[0] = (uint8_t)v; p[1] = (uint8_t)(v >> 8); }
static inline uint16_t get_u16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* ---- encoders ---- */

/* q8_row: [int8 rows*cols][f16 rows]   (crates/cortiq-cli/src/convert.rs:551-566) */
void orc_encode_q8_row(const float *w, size_t rows, size_t cols, uint8_t *out) {
    uint8_t *scales = out + rows * cols;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        const float *row = w + r * cols;
        float s = orc_f16_scale(absmax_of(row, cols) / 127.0f);
        for (size_t c = 0; c < cols; ++c) {
            float q = clampf(rintf(row[c] / s), -128.0f, 127.0f);
            out[r * cols + c] = (uint8_t)(int8_t)q;
        }
        put_u16(scales + 2 * r, orc_f32_to_f16(s));
    }
}

/* One 32-group against scale s -> 16 nibble bytes, low nibble = even element.
 * divide=1: q = rint(v / s)  (q4_block, convert.rs:569-590)
 * divide=0: q = rint(v * s)  where s is already the reciprocal (q4tp, convert.rs:975-983) */
static inline void pack_group(const float *g, float s, int divide, uint8_t *dst) {
    for (int k = 0; k < 16; ++k) {
        float a = divide ? g[2 * k] / s : g[2 * k] * s;
        float b = divide ? g[2 * k + 1] / s : g[2 * k + 1] * s;
        uint8_t q0 = (uint8_t)((int8_t)clampf(rintf(a), -8.0f, 7.0f) + 8);
        uint8_t q1 = (uint8_t)((int8_t)clampf(rintf(b), -8.0f, 7.0f) + 8);
        dst[k] = (uint8_t)((q0 & 0x0F) | (q1 << 4));
    }
}

/* q4_block over the flattened tensor: [16 B * groups][f16 * groups]
 * (crates/cortiq-cli/src/convert.rs:569-590).  n need not be a multiple of 32. */
void orc_encode_q4_block(const float *w, size_t n, uint8_t *out) {
    size_t groups = (n + GROUP - 1) / GROUP;
    uint8_t *scales = out + groups * 16;
#pragma omp parallel for schedule(static)
    for (size_t g = 0; g < groups; ++g) {
        float tmp[GROUP];
        for (int k = 0; k < GROUP; ++k) {
            size_t i = g * GROUP + (size_t)k;
            tmp[k] = i < n ? w[i] : 0.0f;
        }
        float s = orc_f16_scale(absmax_of(tmp, GROUP) / 7.0f);
        pack_group(tmp, s, 1, out + g * 16);
        put_u16(scales + 2 * g, orc_f32_to_f16(s));
    }
}

/* q4_tiled: the q4_block values re-laid as 18-byte tiles [f16 scale][16 B nibbles]
 * (crates/cortiq-cli/src/convert.rs:597-613). */
void orc_encode_q4_tiled(const float *w, size_t rows, size_t cols, uint8_t *out) {
    size_t groups = rows * cols / GROUP;
#pragma omp parallel for schedule(static)
    for (size_t g = 0; g < groups; ++g) {
        const float *grp = w + g * GROUP;
        float s = orc_f16_scale(absmax_of(grp, GROUP) / 7.0f);
        uint8_t *tile = out + g * Q4_TILE_BYTES;
        put_u16(tile, orc_f32_to_f16(s));
        pack_group(grp, s, 1, tile + 2);
    }
}

size_t orc_q4tp_code_stride(size_t gpr) { return (gpr * 5 + 7) / 8; }

size_t orc_q4tp_nbytes(size_t rows, size_t cols) {
    size_t gpr = cols / GROUP;
    return rows * gpr * Q4TP_NIB_BYTES + rows * 4 + rows * orc_q4tp_code_stride(gpr);
}

/* 5-bit code g of a row's LSB-first code stream (crates/cortiq-core/src/quant.rs:369-394). */
unsigned orc_q4tp_code(const uint8_t *codes, size_t stride, size_t g) {
    size_t bit = g * 5, b = bit >> 3;
    unsigned sh = (unsigned)(bit & 7);
    unsigned lo = codes[b];
    unsigned hi = (sh > 3 && b + 1 < stride) ? codes[b + 1] : 0u;
    return ((lo | (hi << 8)) >> sh) & 0x1Fu;
}

static void q4tp_put_code(uint8_t *codes, size_t g, unsigned code) {
    size_t bit = g * 5, b = bit >> 3;
    unsigned sh = (unsigned)(bit & 7);
    unsigned v = code & 0x1Fu;
    codes[b] |= (uint8_t)(v << sh);
    if (sh > 3) codes[b + 1] |= (uint8_t)(v >> (8 - sh));
}

/* Row ladder: t[0] = exp2f(lo), t[c] = t[c-1] * exp2f(step) -- iterated, never closed
 * form (crates/cortiq-core/src/quant.rs:396-411). */
void orc_q4tp_ladder(uint16_t lo_h, uint16_t step_h, float t[32]) {
    float ratio = exp2f(orc_f16_to_f32(step_h));
    t[0] = exp2f(orc_f16_to_f32(lo_h));
    for (int c = 1; c < 32; ++c) t[c] = t[c - 1] * ratio;
}

/* q4tp: [nibbles rows*gpr*16][rows * (f16 lo, f16 step)][rows * ceil(5 gpr / 8) codes]
 * (crates/cortiq-cli/src/convert.rs:883-992, with the rung search enabled, its default). */
void orc_encode_q4tp(const float *w, size_t rows, size_t cols, uint8_t *out) {
    size_t gpr = cols / GROUP;
    size_t stride = orc_q4tp_code_stride(gpr);
    uint8_t *nib = out;
    uint8_t *params = out + rows * gpr * Q4TP_NIB_BYTES;
    uint8_t *codes = params + rows * 4;
    memset(codes, 0, rows * stride);
#pragma omp parallel
    {
        float *lg = (float *)malloc(gpr * sizeof(float));
        uint8_t *dead = (uint8_t *)malloc(gpr);
#pragma omp for schedule(static)
        for (size_t r = 0; r < rows; ++r) {
            const float *row = w + r * cols;
            float lo = INFINITY, hi = -INFINITY;
            for (size_t g = 0; g < gpr; ++g) {
                float am = absmax_of(row + g * GROUP, GROUP);
                dead[g] = (am == 0.0f);
                lg[g] = log2f(orc_f16_scale(am / 7.0f));
                if (!dead[g]) {
                    if (lg[g] < lo) lo = lg[g];
                    if (lg[g] > hi) hi = lg[g];
                }
            }
            if (!isfinite(lo)) { lo = lg[0]; hi = lo; }
            uint16_t lo_h = orc_f32_to_f16(lo);
            float lo_r = orc_f16_to_f32(lo_h);
            float span = hi - lo_r;
            if (!(span > 0.0f)) span = 0.0f;
            uint16_t st_h = orc_f32_to_f16(span / (float)Q4TP_TOP_RUNG);
            /* nudge the step up one half-ulp at a time until rung 31 reaches the top scale */
            for (int it = 0; it < 64; ++it) {
                float st = orc_f16_to_f32(st_h);
                if (st > 0.0f && lo_r + (float)Q4TP_TOP_RUNG * st >= hi) break;
                st_h = (uint16_t)(st_h + 1);
            }
            put_u16(params + 4 * r, lo_h);
            put_u16(params + 4 * r + 2, st_h);
            float st = orc_f16_to_f32(st_h);
            float tab[32];
            orc_q4tp_ladder(lo_h, st_h, tab);
            uint8_t *crow = codes + r * stride;
            for (size_t g = 0; g < gpr; ++g) {
                const float *tile = row + g * GROUP;
                unsigned nominal = 0;
                int frozen = dead[g] || !(st > 0.0f);
                if (!frozen)
                    nominal = (unsigned)clampf(rintf((lg[g] - lo_r) / st), 0.0f, (float)Q4TP_TOP_RUNG);
                unsigned pick = nominal;
                if (!frozen) {
                    float best = INFINITY;
                    unsigned from = nominal >= 2 ? nominal - 2 : 0;
                    unsigned to = nominal + 1 < Q4TP_TOP_RUNG ? nominal + 1 : Q4TP_TOP_RUNG;
                    for (unsigned cand = from; cand <= to; ++cand) {
                        float sc = tab[cand];
                        if (!(sc > 0.0f)) continue;
                        float iv = 1.0f / sc;
                        float err = 0.0f;
                        for (int k = 0; k < GROUP; ++k) {
                            float q = clampf(rintf(tile[k] * iv), -8.0f, 7.0f);
                            float d = tile[k] - q * sc;
                            err += d * d;
                        }
                        if (err < best) { best = err; pick = cand; }
                    }
                }
                q4tp_put_code(crow, g, pick);
                float inv = tab[pick] > 0.0f ? 1.0f / tab[pick] : 0.0f;
                pack_group(tile, inv, 0, nib + (r * gpr + g) * Q4TP_NIB_BYTES);
            }
        }
        free(lg);
        free(dead);
    }
}

/* ---- dequantizers (the bit-exact weight definition) ---- */

/* crates/cortiq-core/src/quant.rs:91-103 */
void orc_dequant_q8_row(const uint8_t *p, size_t rows, size_t cols, float *dst) {
    const uint8_t *scales = p + rows * cols;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        float s = orc_f16_to_f32(get_u16(scales + 2 * r));
        for (size_t c = 0; c < cols; ++c) dst[r * cols + c] = (float)(int8_t)p[r * cols + c] * s;
    }
}

static inline void unpack_group(const uint8_t *nib, float s, float *dst) {
    for (int k = 0; k < 16; ++k) {
        dst[2 * k] = ((float)(nib[k] & 0x0F) - 8.0f) * s;
        dst[2 * k + 1] = ((float)(nib[k] >> 4) - 8.0f) * s;
    }
}

/* crates/cortiq-core/src/quant.rs:322-344 (n a multiple of 32 here) */
void orc_dequant_q4_tiled(const uint8_t *p, size_t n, float *dst) {
    size_t groups = n / GROUP;
#pragma omp parallel for schedule(static)
    for (size_t g = 0; g < groups; ++g) {
        const uint8_t *tile = p + g * Q4_TILE_BYTES;
        unpack_group(tile + 2, orc_f16_to_f32(get_u16(tile)), dst + g * GROUP);
    }
}

/* crates/cortiq-core/src/quant.rs:413-431 */
void orc_dequant_q4tp(const uint8_t *p, size_t rows, size_t cols, float *dst) {
    size_t gpr = cols / GROUP, stride = orc_q4tp_code_stride(gpr);
    const uint8_t *params = p + rows * gpr * Q4TP_NIB_BYTES;
    const uint8_t *codes = params + rows * 4;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < rows; ++r) {
        float tab[32];
        orc_q4tp_ladder(get_u16(params + 4 * r), get_u16(params + 4 * r + 2), tab);
        for (size_t g = 0; g < gpr; ++g) {
            float s = tab[orc_q4tp_code(codes + r * stride, stride, g)];
            unpack_group(p + (r * gpr + g) * Q4TP_NIB_BYTES, s, dst + r * cols + g * GROUP);
        }
    }
}

/* Per-tile f32 scales of a q4tp tensor, [rows][gpr] -- what the exact row kernel consumes
 * (crates/cortiq-engine/src/qtensor.rs:4470-4513 expands them once per row). */
void orc_q4tp_scales(const uint8_t *p, size_t rows, size_t cols, float *scales) {
    size_t gpr = cols / GROUP, stride = orc_q4tp_code_stride(gpr);
    const uint8_t *params = p + rows * gpr * Q4TP_NIB_BYTES;
    const uint8_t *codes = params + rows * 4;
    for (size_t r = 0; r < rows; ++r) {
        float tab[32];
        orc_q4tp_ladder(get_u16(params + 4 * r), get_u16(params + 4 * r + 2), tab);
        for (size_t g = 0; g < gpr; ++g)
            scales[r * gpr + g] = tab[orc_q4tp_code(codes + r * stride, stride, g)];
    }
}

/* ---- strict-f32 linear kernels: Y[b, rows] = X[b, cols] . W^T ---- */

/* q8: sequential f32 accumulate of int8*x, row scale applied last
 * (crates/cortiq-engine/src/qtensor.rs:3533-3546). */
void orc_matmat_q8(const uint8_t *p, size_t rows, size_t cols, const float *x, size_t b, float *y) {
    const uint8_t *scales = p + rows * cols;
#pragma omp parallel for schedule(dynamic, 8)
    for (size_t o = 0; o < rows; ++o) {
        float s = orc_f16_to_f32(get_u16(scales + 2 * o));
        const int8_t *row = (const int8_t *)p + o * cols;
        for (size_t bi = 0; bi < b; ++bi) {
            const float *xr = x + bi * cols;
            float acc = 0.0f;
            for (size_t j = 0; j < cols; ++j) acc += (float)row[j] * xr[j];
            y[bi * rows + o] = acc * s;
        }
    }
}

/* per-group partial ga (pairwise: lo*x0 + hi*x1 added as one term), then acc += ga * s
 * (crates/cortiq-engine/src/qtensor.rs:4418-4432 and :4647-4661). */
static inline float q4_row_dot(const uint8_t *nib_base, size_t nib_stride, size_t nib_off,
                               const float *scales, const uint8_t *scale_tiles, size_t gpr,
                               const float *x) {
    float acc = 0.0f;
    for (size_t g = 0; g < gpr; ++g) {
        const uint8_t *nib = nib_base + g * nib_stride + nib_off;
        float s = scales ? scales[g] : orc_f16_to_f32(get_u16(scale_tiles + g * nib_stride));
        const float *xg = x + g * GROUP;
        float ga = 0.0f;
        for (int k = 0; k < 16; ++k)
            ga += ((float)(nib[k] & 0x0F) - 8.0f) * xg[2 * k] + ((float)(nib[k] >> 4) - 8.0f) * xg[2 * k + 1];
        acc += ga * s;
    }
    return acc;
}

void orc_matmat_q4t(const uint8_t *p, size_t rows, size_t cols, const float *x, size_t b, float *y) {
    size_t gpr = cols / GROUP;
#pragma omp parallel for schedule(dynamic, 8)
    for (size_t o = 0; o < rows; ++o) {
        const uint8_t *tiles = p + o * gpr * Q4_TILE_BYTES;
        for (size_t bi = 0; bi < b; ++bi)
            y[bi * rows + o] = q4_row_dot(tiles, Q4_TILE_BYTES, 2, NULL, tiles, gpr, x + bi * cols);
    }
}

void orc_matmat_q4tp(const uint8_t *p, size_t rows, size_t cols, const float *x, size_t b, float *y) {
    size_t gpr = cols / GROUP;
    float *scales = (float *)malloc(rows * gpr * sizeof(float));
    orc_q4tp_scales(p, rows, cols, scales);
#pragma omp parallel for schedule(dynamic, 8)
    for (size_t o = 0; o < rows; ++o) {
        const uint8_t *nib = p + o * gpr * Q4TP_NIB_BYTES;
        for (size_t bi = 0; bi < b; ++bi)
            y[bi * rows + o] = q4_row_dot(nib, Q4TP_NIB_BYTES, 0, scales + o * gpr, NULL, gpr, x + bi * cols);
    }
    free(scales);
}

/* Plain f32 y[n, m] = x[n, k] . w[m, k]^T with sequential accumulation: the arithmetic of
 * the attention GEMMs and the exact-f32 projections (crates/cortiq-engine/src/fcd_ops.rs:302-435
 * computes the same products; its blocked summation order differs by rounding only). */
void orc_gemm_nt(const float *x, const float *w, float *y, size_t n, size_t k, size_t m) {
#pragma omp parallel for schedule(dynamic, 4)
    for (size_t i = 0; i < n; ++i)
        for (size_t j = 0; j < m; ++j) {
            float acc = 0.0f;
            for (size_t t = 0; t < k; ++t) acc += x[i * k + t] * w[j * k + t];
            y[i * m + j] = acc;
        }
}

int orc_num_threads(void) {
    int n = 1;
#ifdef _OPENMP
#pragma omp parallel
    {
#pragma omp single
        n = omp_get_num_threads();
    }
#endif
    return n;
}
