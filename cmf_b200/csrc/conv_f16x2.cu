// Convolution / linear as an implicit GEMM on tcgen05 with split-f16 operands, for the FLUX-class
// VAE decoder that follows the denoiser (crates/cortiq-engine/src/vae.rs: Conv2d::apply :153,
// AttnBlock::apply :415; the facade's vae_conv2d / vae_upsample_conv,
// crates/cortiq-engine/src/gpu.rs:2002-2060).
//
//   D[oc, pixel] = sum over taps (ky, kx) and channels c of  W[oc, (ky, kx), c] * X[y+ky-p, x+kx-p, c]
//
// Precision.  The decoder is an f32 network (its parity bar is 2e-3 max-abs on the image), so
// every f32 operand travels as TWO f16 planes, hi = f16(v) and lo = f16(v - hi): hi + lo carries
// 22 significand bits.  The container stores conv kernels as f16, so a conv weight is its hi
// plane alone and a convolution costs two kind::f16 MMAs per k-step (W*X_hi + W*X_lo), both
// accumulating in f32 in TMEM.  Operands that are f32 on both sides (the attention block's
// linears and its QK^T / PV products) use three (hi*hi + hi*lo + lo*hi).
//
// Layout.  Activations are NHWC planes (channels padded to a multiple of 32); the B operand of a
// k-block is a 3-D TMA box (32 channels x bw x bh pixels, bw * bh = 256) fetched at the tap's
// shifted coordinates, so the zero padding of the convolution is the TMA out-of-bounds fill and
// no im2col buffer exists.  Weights are [oc, taps * ic] planes, the A operand (128 rows x 32 k).
// Persistent CTAs walk output tiles (128 channels x 256 pixels); two accumulators in TMEM let
// the epilogue of one tile overlap the MMAs of the next.  The epilogue adds bias, scales, adds
// an optional f32 residual and writes f32 and/or split planes, pixel-major (NHWC) or
// channel-major ([oc][pixel]: NCHW, also V^T of the attention block).  Every wait is bounded.
#include <cuda_fp16.h>

#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace cmfc {
namespace {

constexpr int CV_OC = 128, CV_PIX = 256, CV_K = 32, CV_MAX_STAGES = 8;
constexpr int CV_A_BYTES = CV_OC * CV_K * 2;    // 8 KiB per plane
constexpr int CV_B_BYTES = CV_PIX * CV_K * 2;   // 16 KiB per plane
constexpr int CV_RING_BYTES = 5 * (CV_A_BYTES + 2 * CV_B_BYTES);  // 200 KiB
constexpr int CV_SMEM = CV_RING_BYTES + 1024 + 256;
constexpr int CV_THREADS = 32 * 10;             // TMA, MMA, eight epilogue warps

struct ConvBars {
    uint64_t full[CV_MAX_STAGES], empty[CV_MAX_STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base, abort_flag;
};

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// kind::f16 instruction descriptor: f32 accumulator, f16 (format 0) A and B, both K-major
__host__ __device__ constexpr uint32_t idesc_f16_f32(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

__device__ __forceinline__ void split_store(__half* hi, __half* lo, size_t o, float v) {
    const __half h = __float2half_rn(v);
    hi[o] = h;
    lo[o] = __float2half_rn(v - __half2float(h));
}

// BW: the tile's width in pixels when it is 16 (images) or 256 (token rows); 0 = read it from p.bw
template <int BW>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv_f16x2_kernel(const __grid_constant__ CUtensorMap tm_a_hi, const __grid_constant__ CUtensorMap tm_a_lo,
                  const __grid_constant__ CUtensorMap tm_b_hi, const __grid_constant__ CUtensorMap tm_b_lo,
                  ConvParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    ConvBars* bars = reinterpret_cast<ConvBars*>(ring + CV_RING_BYTES);
    volatile uint32_t* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stage_bytes = p.a_planes * CV_A_BYTES + p.b_planes * CV_B_BYTES;
    const int stages = min(CV_MAX_STAGES, CV_RING_BYTES / stage_bytes);
    const int b_off = p.a_planes * CV_A_BYTES;
    const int cchunks = p.ic / CV_K;
    const int kblocks = p.taps * cchunks;
    const int ksz = p.taps == 9 ? 3 : 1, pad = ksz / 2;
    const int ntiles = p.tiles_oc * p.tiles_x * p.tiles_y;
    const int bw_shift = __ffs(p.bw) - 1, bw_mask = p.bw - 1;  // bw is a power of two

    if (threadIdx.x == 0) {
        for (int s = 0; s < CV_MAX_STAGES; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&bars->acc_full[a], 1);
            mbar_init(&bars->acc_empty[a], 8);
        }
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tm_a_hi);
        tma_prefetch_desc(&tm_b_hi);
    }
    if (warp == 1) {
        tmem_alloc(&bars->tmem_base, 2 * CV_PIX);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        if (elect_one()) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int oc0 = (tile % p.tiles_oc) * CV_OC;
                const int r = tile / p.tiles_oc;
                const int x0 = (r % p.tiles_x) * p.bw, y0 = (r / p.tiles_x) * p.bh;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1u;
                    if (!mbar_wait<100>(&bars->empty[s], ph ^ 1u, abort_flag, 31)) { ok = false; break; }
                    const int tap = kb / cchunks, c0 = (kb % cchunks) * CV_K;
                    const int xs = x0 + tap % ksz - pad, ys = y0 + tap / ksz - pad;
                    uint8_t* st = ring + s * stage_bytes;
                    mbar_expect_tx(&bars->full[s], stage_bytes);
                    tma_load_2d(st, &tm_a_hi, &bars->full[s], tap * p.ic + c0, oc0);
                    if (p.a_planes == 2) tma_load_2d(st + CV_A_BYTES, &tm_a_lo, &bars->full[s], tap * p.ic + c0, oc0);
                    tma_load_3d(st + b_off, &tm_b_hi, &bars->full[s], c0, xs, ys);
                    if (p.b_planes == 2) tma_load_3d(st + b_off + CV_B_BYTES, &tm_b_lo, &bars->full[s], c0, xs, ys);
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            constexpr uint32_t IDESC = idesc_f16_f32(CV_OC, CV_PIX);
            uint32_t it = 0, lt = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++lt) {
                const uint32_t acc = lt & 1u, aph = (lt >> 1) & 1u;
                if (!mbar_wait(&bars->acc_empty[acc], aph ^ 1u, abort_flag, 34)) break;
                tc_fence_after();
                const uint32_t d = tmem + acc * CV_PIX;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % stages;
                    const uint32_t ph = (it / stages) & 1u;
                    if (!mbar_wait(&bars->full[s], ph, abort_flag, 32)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_hi = smem_u32(ring + s * stage_bytes), a_lo = a_hi + CV_A_BYTES;
                    const uint32_t b_hi = a_hi + b_off, b_lo = b_hi + CV_B_BYTES;
#pragma unroll
                    for (int j = 0; j < CV_K / 16; ++j) {
                        const uint32_t o = j * 32;
                        const uint64_t da = smem_desc_kmajor(a_hi + o, 64), db = smem_desc_kmajor(b_hi + o, 64);
                        mma_ss(d, da, db, IDESC, (kb | j) != 0);
                        if (p.b_planes == 2) mma_ss(d, da, smem_desc_kmajor(b_lo + o, 64), IDESC, 1);
                        if (p.a_planes == 2) mma_ss(d, smem_desc_kmajor(a_lo + o, 64), db, IDESC, 1);
                    }
                    tc_commit(&bars->empty[s]);
                }
                if (ok) tc_commit(&bars->acc_full[acc]);
            }
        }
    } else {
        // epilogue, eight warps: warp w may touch TMEM lanes 32 * (w % 4); the two warps of a lane
        // quarter split the tile's 256 pixel columns.  A thread owns output channel oc0 + row.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = ((uint32_t)(quarter * 32) << 16) + half * (CV_PIX / 2);
        const size_t step_x = p.channel_major ? 1 : (size_t)p.out_pitch;
        const size_t step_y = (size_t)p.w * step_x;
        uint32_t lt = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++lt) {
            const uint32_t acc = lt & 1u, aph = (lt >> 1) & 1u;
            const int oc = (tile % p.tiles_oc) * CV_OC + row;
            const int r = tile / p.tiles_oc;
            const int x0 = (r % p.tiles_x) * p.bw, y0 = (r / p.tiles_x) * p.bh;
            const int xlim = p.w - x0, ylim = p.h - y0;  // tile-relative extent of the image
            const bool live = oc < p.oc;
            const float bias_s = (p.bias && live) ? p.bias[oc] * p.out_scale : 0.0f;
            const size_t base = p.channel_major ? (size_t)oc * p.out_pitch + (size_t)y0 * p.w + x0
                                                : ((size_t)y0 * p.w + x0) * p.out_pitch + oc;
            // visit the 32 pixels of chunk ``c``: f(j, inside, element offset)
            auto for_chunk = [&](int c, auto&& f) {
                if constexpr (BW == 0) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int pi = c * 32 + j, dx = pi & bw_mask, dy = pi >> bw_shift;
                        f(j, dx < xlim && dy < ylim, base + dy * step_y + dx * step_x);
                    }
                } else {
                    constexpr int SEG = BW < 32 ? BW : 32, ROWS = 32 / SEG;
                    const int dy0 = (c * 32) / BW, dx0 = (c * 32) % BW;
#pragma unroll
                    for (int rr = 0; rr < ROWS; ++rr) {
                        size_t o = base + (size_t)(dy0 + rr) * step_y + (size_t)dx0 * step_x;
                        const bool row_ok = dy0 + rr < ylim;
#pragma unroll
                        for (int xx = 0; xx < SEG; ++xx, o += step_x) f(rr * SEG + xx, row_ok && dx0 + xx < xlim, o);
                    }
                }
            };
            // The residual does not depend on the accumulator: a chunk's values are fetched while
            // the previous chunk is in flight.  (The output may alias the residual, so they are all
            // read before any element of the chunk is written.)
            float res_a[32], res_b[32];
            auto fetch = [&](int c, float* dst) {
                for_chunk(c, [&](int j, bool ok, size_t o) { dst[j] = (ok && live) ? p.residual[o] : 0.0f; });
            };
            double ssum = 0.0, ssq = 0.0;
            auto emit = [&](int c, const uint32_t* v, const float* res) {
                for_chunk(c, [&](int j, bool ok, size_t o) {
                    if (ok) {
                        float val = fmaf(__uint_as_float(v[j]), p.out_scale, bias_s);
                        if (p.residual) val += res[j];
                        if (p.out_f32) p.out_f32[o] = val;
                        if (p.out_hi) split_store(p.out_hi, p.out_lo, o, val);
                        if (p.stats_partial) {
                            const double d = (double)val;
                            ssum += d;
                            ssq += d * d;
                        }
                    }
                });
            };
            const int chunk0 = half * (CV_PIX / 64);
            if (p.residual) fetch(chunk0, res_a);
            if (!mbar_wait<200>(&bars->acc_full[acc], aph, abort_flag, 33)) break;
            tc_fence_after();
            const uint32_t t0 = tmem + acc * CV_PIX + lane_addr;
#pragma unroll 1
            for (int cc = 0; cc < CV_PIX / 64; cc += 2) {
                uint32_t v[32];
                tmem_ld_x32(t0 + cc * 32, v);
                if (p.residual) fetch(chunk0 + cc + 1, res_b);
                tc_wait_ld();
                if (live) emit(chunk0 + cc, v, res_a);
                tmem_ld_x32(t0 + (cc + 1) * 32, v);
                if (p.residual && cc + 2 < CV_PIX / 64) fetch(chunk0 + cc + 2, res_a);
                tc_wait_ld();
                if (live) emit(chunk0 + cc + 1, v, res_b);
            }
            if (p.stats_partial && live) {
                // slot = (pixel tile, column half); reduced in slot order by the GroupNorm finalize
                double* slot = p.stats_partial + ((size_t)r * 2 + half) * (2 * (size_t)p.oc) + 2 * (size_t)oc;
                slot[0] = ssum;
                slot[1] = ssq;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, 2 * CV_PIX);
    }
    if (threadIdx.x == 0 && bars->abort_flag) atomicCAS(p.status, 0u, 0x300u | bars->abort_flag);
}

}  // namespace

void conv_tile_shape(int w, int h, int* bw, int* bh) {
    if (h == 1) { *bw = CV_PIX; *bh = 1; return; }
    int b = 16;
    while (b > w) b >>= 1;
    *bw = b;
    *bh = CV_PIX / b;
}

size_t conv_stats_slots(int w, int h) {
    int bw, bh;
    conv_tile_shape(w, h, &bw, &bh);
    return 2 * (size_t)((w + bw - 1) / bw) * ((h + bh - 1) / bh);
}

int launch_conv_f16x2(const CUtensorMap& tm_a_hi, const CUtensorMap& tm_a_lo, const CUtensorMap& tm_b_hi,
                      const CUtensorMap& tm_b_lo, ConvParams p, int num_sms, cudaStream_t stream) {
    if (p.ic <= 0 || p.ic % CV_K || p.bw * p.bh != CV_PIX || (p.taps != 1 && p.taps != 9))
        return fail(ERR_SHAPE, "conv: input channels must be a multiple of 32, taps 1 or 9, tile 256 pixels");
    if (p.a_planes < 1 || p.a_planes > 2 || p.b_planes < 1 || p.b_planes > 2)
        return fail(ERR_BAD_ARG, "conv: operand planes must be 1 or 2");
    if (p.oc <= 0 || p.w <= 0 || p.h <= 0) return fail(ERR_SHAPE, "conv: empty output");
    static std::atomic<bool> configured[64];
    int dev = 0;
    CMFC_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        CMFC_CUDA(cudaFuncSetAttribute(conv_f16x2_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, CV_SMEM));
        CMFC_CUDA(cudaFuncSetAttribute(conv_f16x2_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, CV_SMEM));
        CMFC_CUDA(cudaFuncSetAttribute(conv_f16x2_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, CV_SMEM));
        configured[dev & 63] = true;
    }
    p.tiles_oc = (p.oc + CV_OC - 1) / CV_OC;
    p.tiles_x = (p.w + p.bw - 1) / p.bw;
    p.tiles_y = (p.h + p.bh - 1) / p.bh;
    const long long ntiles = (long long)p.tiles_oc * p.tiles_x * p.tiles_y;
    const int grid = (int)std::min<long long>(ntiles, num_sms);
    if (p.bw == 16)
        conv_f16x2_kernel<16><<<grid, CV_THREADS, CV_SMEM, stream>>>(tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo, p);
    else if (p.bw == 256)
        conv_f16x2_kernel<256><<<grid, CV_THREADS, CV_SMEM, stream>>>(tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo, p);
    else
        conv_f16x2_kernel<0><<<grid, CV_THREADS, CV_SMEM, stream>>>(tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo, p);
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace cmfc
