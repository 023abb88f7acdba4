// Dequant-fused GEMM for the quantized linears of the NextDiT block:
//     Y[M, N] = X[M, K] . dequant(W[N, K])^T
// (replaces QTensor::matmat's Q8Row / Q4Tiled / Q4TiledP arms,
//  crates/cortiq-engine/src/qtensor.rs:1441-1861).
//
// The product is computed transposed, D[n, m] = W[n, :] . X[m, :], so that the dequantized
// weights are the tcgen05 A operand (one weight row per TMEM lane) and the activations are
// the B operand:
//   * X (bf16, K-major) tiles of 256 tokens x 64 k arrive by TMA with the 128-byte swizzle
//     and are consumed by the tensor core straight from shared memory;
//   * the packed weight tile of 128 rows x 64 k (int8, or 4-bit nibbles plus a per-group f32
//     scale) arrives by TMA as raw bytes; eight dequant warps, one weight row per thread,
//     unpack it in registers to bf16 and write it to TENSOR MEMORY with tcgen05.st;
//   * one elected thread issues tcgen05.mma (A from TMEM, B from SMEM, 128 x 256 x 16) into a
//     256-column f32 accumulator in TMEM; the other 256 columns are an 8-deep ring of A tiles,
//     so the dequant warps run up to 8 k-blocks ahead of the tensor core;
//   * four epilogue warps drain the finished accumulator with tcgen05.ld and store Y (f32 or
//     bf16, or the fused SwiGLU product when the weight rows interleave W1 and W3) while the
//     dequant warps already fill the A ring for the next tile.
// Persistent: grid = min(#tiles, #SMs); each CTA walks tiles blockIdx.x, +gridDim.x, ...
//
// bf16 operand definition: RN_bf16(exact f32 dequantized weight).  For q8 the integer level
// itself is the operand (exact in bf16) and the f32 row scale is applied to the accumulator.
#include <atomic>

#include "common.cuh"
#include "gemm_unpack.cuh"
#include "kernels.h"

namespace cmfc {
namespace {

constexpr int TW = 128;     // weight rows per tile  (UMMA M, TMEM lanes)
constexpr int TT = 256;     // tokens per tile       (UMMA N, accumulator columns)
constexpr int BK = 64;      // k per pipeline stage  (one 128-byte swizzle atom of bf16)
constexpr int STAGES = 5;    // shared-memory ring (X tile + packed W tile + scales)
constexpr int ASTAGES = 8;   // tensor-memory ring of dequantized A tiles
constexpr int NACC = 1;      // accumulators in TMEM (NACC * TT + ASTAGES * 32 <= 512 columns)
constexpr int X_STAGE = TT * BK * 2;   // 32 KiB
constexpr int W_STAGE = TW * BK;       // 8 KiB (q8: 64 B/row; q4 uses the first 4 KiB)
constexpr int S_STAGE = 2 * TW * 4;    // 1 KiB (q4: two groups x 128 rows of f32 scales)
constexpr int A_COL = NACC * TT;       // after the accumulator(s): the A ring, 32 columns per stage
constexpr int TMEM_COLS = 512;
constexpr int NUM_DQ_WARPS = 8;
constexpr int NUM_EPI_WARPS = 8;
constexpr int THREADS = 32 * (2 + NUM_DQ_WARPS + NUM_EPI_WARPS);
static_assert(A_COL + ASTAGES * 32 <= TMEM_COLS, "TMEM budget");
constexpr int SMEM_BYTES = STAGES * (X_STAGE + W_STAGE + S_STAGE) + 1024 /*align*/ + 256 /*barriers*/;

struct Bars {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t a_full[ASTAGES];
    uint64_t a_empty[ASTAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

using namespace gemm_detail;

// WKIND: 0 = q8 (int8 plane); 1 = q4tp (nibble plane + transposed f32 scales);
//        2 = q4_tiled (nibble plane + transposed scales split into bf16 hi/lo halves)
template <int WKIND>
__global__ void __launch_bounds__(THREADS, 1)
gemm_dequant_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                    const __grid_constant__ CUtensorMap tm_s, GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* x_smem = smem;
    uint8_t* w_smem = smem + STAGES * X_STAGE;
    uint8_t* s_smem = w_smem + STAGES * W_STAGE;
    Bars* bars = reinterpret_cast<Bars*>(s_smem + STAGES * S_STAGE);
    volatile uint32_t* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.K / BK;
    const int tiles_m = (p.M + TT - 1) / TT;
    // Tile order: consecutive tiles share the token tile, so the CTAs running at one time read the
    // same X rows (served by L2 after the first) while the small packed weights stay L2 resident.
    const int tiles_n = p.N / TW;
    const int tiles = tiles_m * tiles_n;
    constexpr uint32_t W_BYTES = (WKIND == 0) ? TW * BK : TW * BK / 2;
    constexpr uint32_t TX_BYTES = X_STAGE + W_BYTES + (WKIND != 0 ? S_STAGE : 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bars->full[s], 1);
            mbar_init(&bars->empty[s], 1 + NUM_DQ_WARPS);
        }
        for (int a = 0; a < ASTAGES; ++a) {
            mbar_init(&bars->a_full[a], NUM_DQ_WARPS);
            mbar_init(&bars->a_empty[a], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bars->acc_full[b], 1);
            mbar_init(&bars->acc_empty[b], NUM_EPI_WARPS);
        }
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_w);
        if (WKIND != 0) tma_prefetch_desc(&tm_s);
    }
    if (warp == 1) {
        tmem_alloc(&bars->tmem_base, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < tiles && !*abort_flag; tile += gridDim.x) {
                const int n0 = (tile % tiles_n) * TW, m0 = (tile / tiles_n) * TT;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait<200>(&bars->empty[s], ph ^ 1u, abort_flag, 1)) break;
                    mbar_expect_tx(&bars->full[s], TX_BYTES);
                    tma_load_2d(x_smem + s * X_STAGE, &tm_x, &bars->full[s], kb * BK, m0);
                    if (WKIND == 0) {
                        tma_load_2d(w_smem + s * W_STAGE, &tm_w, &bars->full[s], kb * BK, n0);
                    } else {
                        tma_load_2d(w_smem + s * W_STAGE, &tm_w, &bars->full[s], kb * (BK / 2), n0);
                        tma_load_2d(s_smem + s * S_STAGE, &tm_s, &bars->full[s], n0, kb * 2);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (elect_one()) {
            constexpr uint32_t IDESC = idesc_bf16_f32(TW, TT);
            uint32_t it = 0, tile_i = 0;
            for (int tile = blockIdx.x; tile < tiles && !*abort_flag; tile += gridDim.x, ++tile_i) {
                const uint32_t buf = tile_i % NACC, acc = tmem + buf * TT;
                // the epilogue warps must have drained this accumulator's previous tile
                if (!mbar_wait(&bars->acc_empty[buf], ((tile_i / NACC) & 1u) ^ 1u, abort_flag, 2)) break;
                tc_fence_after();
                bool ok = true;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES, ai = it % ASTAGES;
                    const uint32_t ph = (it / STAGES) & 1u, aph = (it / ASTAGES) & 1u;
                    if (!mbar_wait(&bars->full[s], ph, abort_flag, 3) ||
                        !mbar_wait(&bars->a_full[ai], aph, abort_flag, 4)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t xs = smem_u32(x_smem + s * X_STAGE);
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j) {
                        mma_ts(acc, tmem + A_COL + ai * 32 + j * 8, smem_desc_kmajor(xs + j * 32, 128),
                               IDESC, (kb | j) != 0);
                    }
                    tc_commit(&bars->empty[s]);
                    tc_commit(&bars->a_empty[ai]);
                }
                if (!ok) break;
                tc_commit(&bars->acc_full[buf]);
            }
        }
    } else if (warp < 2 + NUM_DQ_WARPS) {
        // ---------------- dequant warps ----------------
        const int dq = warp - 2;                 // 0..7
        const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
        const int half = dq >> 2;                // which 32 k of the 64-k stage
        const int row = quarter * 32 + lane;     // weight row inside the tile
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        int pending = -1;  // A stage whose tcgen05.st is still in flight
        // Software pipeline: the TMEM store of k-block i is left in flight while k-block i+1 is
        // unpacked; a_full[i] is signalled once that store has completed.
        auto flush = [&]() {
            if (pending >= 0) {
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->a_full[pending]);
                pending = -1;
            }
        };
        for (int tile = blockIdx.x; tile < tiles && ok && !*abort_flag; tile += gridDim.x) {
            for (int kb = 0; kb < kblocks; ++kb, ++it) {
                const int s = it % STAGES, ai = it % ASTAGES;
                const uint32_t ph = (it / STAGES) & 1u, aph = (it / ASTAGES) & 1u;
                if (!mbar_wait<100>(&bars->full[s], ph, abort_flag, 5)) { ok = false; break; }
                uint32_t a[16];
                if (WKIND == 0) {
                    const uint8_t* wrow = w_smem + s * W_STAGE + row * 64;
                    const int sw = (row >> 1) & 3;  // 64-byte swizzle: chunk ^= address bits [7,9)
                    uint4 v0 = lds128(wrow + (((2 * half) ^ sw) << 4));
                    uint4 v1 = lds128(wrow + (((2 * half + 1) ^ sw) << 4));
                    unpack_q8_word(v0.x, a[0], a[1]);   unpack_q8_word(v0.y, a[2], a[3]);
                    unpack_q8_word(v0.z, a[4], a[5]);   unpack_q8_word(v0.w, a[6], a[7]);
                    unpack_q8_word(v1.x, a[8], a[9]);   unpack_q8_word(v1.y, a[10], a[11]);
                    unpack_q8_word(v1.z, a[12], a[13]); unpack_q8_word(v1.w, a[14], a[15]);
                } else {
                    const uint8_t* wrow = w_smem + s * W_STAGE + row * 32;
                    const int sw = (row >> 2) & 1;  // 32-byte swizzle: chunk ^= address bit 7
                    uint4 v = lds128(wrow + ((half ^ sw) << 4));
                    if (WKIND == 1) {
                        const float sc = reinterpret_cast<const float*>(s_smem + s * S_STAGE)[half * TW + row];
                        const Q4Scales q(sc);
                        unpack_q4_word(v.x, q, a + 0);
                        unpack_q4_word(v.y, q, a + 4);
                        unpack_q4_word(v.z, q, a + 8);
                        unpack_q4_word(v.w, q, a + 12);
                    } else {
                        const uint32_t sc = reinterpret_cast<const uint32_t*>(s_smem + s * S_STAGE)[half * TW + row];
                        const uint32_t hi2 = __byte_perm(sc, sc, 0x1010), lo2 = __byte_perm(sc, sc, 0x3232);
                        unpack_q4t_word(v.x, hi2, lo2, a + 0);
                        unpack_q4t_word(v.y, hi2, lo2, a + 4);
                        unpack_q4t_word(v.z, hi2, lo2, a + 8);
                        unpack_q4t_word(v.w, hi2, lo2, a + 12);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->empty[s]);  // the packed bytes are in registers
                flush();
                // A stage ai is free once the MMAs that read its previous tile have committed
                if (!mbar_wait<100>(&bars->a_empty[ai], aph ^ 1u, abort_flag, 7)) { ok = false; break; }
                tc_fence_after();
                tmem_st_x16(tmem + lane_addr + A_COL + ai * 32 + half * 16, a);
                pending = ai;
            }
        }
        flush();
    } else {
        // ---------------- epilogue warps ----------------
        // This thread owns output channel n0+row and half of the tile's tokens.
        const int quarter = warp & 3;
        const int ehalf = (warp - 2 - NUM_DQ_WARPS) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        uint32_t tile_i = 0;
        for (int tile = blockIdx.x; tile < tiles && !*abort_flag; tile += gridDim.x, ++tile_i) {
            const int n0 = (tile % tiles_n) * TW, m0 = (tile / tiles_n) * TT;
            const uint32_t buf = tile_i % NACC;
            if (!mbar_wait<(NACC > 1 ? 1000 : 80)>(&bars->acc_full[buf], (tile_i / NACC) & 1u, abort_flag, 6)) break;
            tc_fence_after();
            const int n = n0 + row;
            float rs = 1.0f;
            if (WKIND == 0) rs = p.row_scale[n];
            // one 32-token chunk of this thread's output channel
            auto emit = [&](const uint32_t (&v)[32], int c) {
                const int mb = m0 + c * 32;
                if (mb >= p.M) return;
                if (p.mode == GEMM_OUT_F32 && p.vt && n >= p.vt_row0) {
                    emit_vt_chunk(v, rs, mb, p.M, p.vt + (size_t)(n - p.vt_row0) * p.vt_pitch, p.seg_table, p.nseg);
                } else if (p.mode == GEMM_OUT_F32) {
                    float* out = reinterpret_cast<float*>(p.out) + (size_t)mb * p.ldo + n;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (mb + j < p.M) out[(size_t)j * p.ldo] = __uint_as_float(v[j]) * rs;
                } else if (p.mode == GEMM_OUT_BF16) {
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)mb * p.ldo + n;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (mb + j < p.M) out[(size_t)j * p.ldo] = __float2bfloat16_rn(__uint_as_float(v[j]) * rs);
                } else if (p.mode == GEMM_OUT_GEGLU) {
                    // as GEMM_OUT_SWIGLU below, with the tanh-form GELU on the gate
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)mb * p.ldo + (n >> 1);
                    const bool odd = lane & 1;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float mine_a = __uint_as_float(v[j]), mine_b = __uint_as_float(v[j + 1]);
                        if (WKIND == 0) { mine_a *= rs; mine_b *= rs; }
                        float got = __shfl_xor_sync(0xffffffffu, odd ? mine_a : mine_b, 1);
                        float g = odd ? got : mine_a;
                        float u = odd ? mine_b : got;
                        int m = mb + j + (odd ? 1 : 0);
                        if (m < p.M) out[(size_t)(j + (odd ? 1 : 0)) * p.ldo] = __float2bfloat16_rn(gelu_tanh_f(g) * u);
                    }
                } else {
                    // GEMM_OUT_SWIGLU: even rows hold W1 (gate), odd rows W3 (up) of channel n/2.
                    // Lanes 2i and 2i+1 swap one value per token pair; the even lane finishes
                    // token j, the odd lane token j+1.
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)mb * p.ldo + (n >> 1);
                    const bool odd = lane & 1;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float mine_a = __uint_as_float(v[j]), mine_b = __uint_as_float(v[j + 1]);
                        if (WKIND == 0) { mine_a *= rs; mine_b *= rs; }
                        float got = __shfl_xor_sync(0xffffffffu, odd ? mine_a : mine_b, 1);
                        float g = odd ? got : mine_a;
                        float u = odd ? mine_b : got;
                        int m = mb + j + (odd ? 1 : 0);
                        if (m < p.M) out[(size_t)(j + (odd ? 1 : 0)) * p.ldo] = __float2bfloat16_rn(silu_f(g) * u);
                    }
                }
            };
            // The TMEM load of a chunk is issued before the previous chunk is converted and stored,
            // and the accumulator is handed back to the MMA warp as soon as the last load has landed
            // (the stores of the last chunk overlap the next tile's first MMAs).
            const int c0 = ehalf * (TT / 64);
            const uint32_t t0 = tmem + lane_addr + buf * TT + c0 * 32;
            uint32_t va[32], vb[32];
            tmem_ld_x32(t0, va);
#pragma unroll 1
            for (int i = 0; i < TT / 64; i += 2) {
                tc_wait_ld();
                tmem_ld_x32(t0 + (i + 1) * 32, vb);
                emit(va, c0 + i);
                tc_wait_ld();
                if (i + 2 < TT / 64) {
                    tmem_ld_x32(t0 + (i + 2) * 32, va);
                } else {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->acc_empty[buf]);
                }
                emit(vb, c0 + i + 1);
            }
        }
    }

    // ---------------- common exit ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
    if (threadIdx.x == 0 && bars->abort_flag) atomicCAS(p.status, 0u, 0x100u | bars->abort_flag);
}

}  // namespace

int gemm_smem_bytes() { return SMEM_BYTES; }
int gemm_tile_tokens() { return TT; }

int launch_gemm_dequant(int wkind, const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_s,
                        const GemmParams& p, int num_sms, cudaStream_t stream) {
    if (p.K % BK != 0 || p.N % TW != 0 || p.M <= 0)
        return fail(ERR_SHAPE, "dequant GEMM needs K % 64 == 0 and N % 128 == 0");
    static std::atomic<bool> configured[3][64];  // per codec kernel and device
    auto kern = wkind == 0 ? gemm_dequant_kernel<0> : (wkind == 1 ? gemm_dequant_kernel<1> : gemm_dequant_kernel<2>);
    int dev = 0;
    CMFC_CUDA(cudaGetDevice(&dev));
    if (!configured[wkind][dev & 63]) {
        CMFC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[wkind][dev & 63] = true;
    }
    const int tiles = ((p.M + TT - 1) / TT) * (p.N / TW);
    const int grid = tiles < num_sms ? tiles : num_sms;
    kern<<<grid, THREADS, SMEM_BYTES, stream>>>(tm_x, tm_w, tm_s, p);
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace cmfc
