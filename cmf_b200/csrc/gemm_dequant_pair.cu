// Dequant-fused GEMM on CTA PAIRS (tcgen05 cta_group::2): the two CTAs of a cluster compute one
// tile of 256 weight rows x 256 tokens.  Same operand definition and data path as
// gemm_dequant.cu (dequantized weights are the A operand in tensor memory, activations the B
// operand in shared memory), with the work of a tile split as the 2-SM MMA wants it:
//   * each CTA owns 128 of the 256 weight rows: it fetches and unpacks its own packed weight
//     tile into its own tensor memory, and drains its own 128 x 256 accumulator;
//   * each CTA fetches only HALF of the activation tile (128 tokens x 64 k, 16 KiB); the MMA of
//     the pair reads both halves from the two CTAs' shared memory, so an activation byte crosses
//     L2 -> SM once per 256 weight rows instead of once per 128, and the ring is 8 stages deep;
//   * one thread of the even CTA issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16) and
//     releases stages in both CTAs with multicast commits; the odd CTA's warps signal the even
//     CTA's barriers (A tile ready, accumulator drained) with remote arrives.
// Every bulk tensor load here is a plain or cta_group::2 load of this GPU's own memory, one copy per CTA.
// Every wait is bounded; the pair leaves through a cluster barrier so that neither CTA exits
// while the other may still touch its shared or tensor memory.
#include <cooperative_groups.h>
#include <algorithm>

#include <atomic>

#include "common.cuh"
#include "gemm_unpack.cuh"
#include "kernels.h"

namespace cmfc {
namespace {

using namespace gemm_detail;
namespace cg = cooperative_groups;

constexpr int TW = 128;      // weight rows per CTA (the pair covers 256)
constexpr int TT = 256;      // tokens per pair tile (UMMA N)
constexpr int TH = TT / 2;   // tokens whose activations this CTA stages
constexpr int BK = 64;
constexpr int STAGES = 8;
constexpr int ASTAGES = 8;
static_assert(STAGES == ASTAGES, "one commit per k-block releases both rings");
constexpr int X_STAGE = TH * BK * 2;   // 16 KiB
constexpr int W_STAGE = TW * BK;       // 8 KiB
constexpr int S_STAGE = 2 * TW * 4;    // 1 KiB
constexpr int A_COL = TT;
constexpr int TMEM_COLS = 512;
constexpr int NUM_DQ_WARPS = 8;     // dequant warps per k-block
constexpr int DQ_GROUPS = 2;        // groups of dequant warps taking k-blocks in turn
constexpr int NUM_EPI_WARPS = 8;
constexpr int THREADS = 32 * (2 + DQ_GROUPS * NUM_DQ_WARPS + NUM_EPI_WARPS);
constexpr int GLU_STAGE = 32 * 16 * 2;  // one epilogue warp's staged chunk: 32 tokens x 16 channels bf16
constexpr int SMEM_BYTES = STAGES * (X_STAGE + W_STAGE + S_STAGE) + NUM_EPI_WARPS * GLU_STAGE + 1024 + 512;
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address: the even CTA

struct Bars {
    uint64_t x_full[STAGES];    // even CTA: both activation halves have landed
    uint64_t w_full[STAGES];    // own packed weight tile (and scales) has landed
    uint64_t empty[STAGES];     // own packed weight stage consumed by the 8 dequant warps
    uint64_t a_full[ASTAGES];   // even CTA: both CTAs' A tiles are in tensor memory (16 arrivals)
    uint64_t a_empty[ASTAGES];  // the pair's MMAs of this k-block are done: A stage and activation stage free
                                // (one multicast commit per k-block; STAGES == ASTAGES, same index)
    uint64_t acc_full;          // own accumulator complete (multicast commit)
    uint64_t acc_empty;         // even CTA: both accumulators drained (16 arrivals)
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ __forceinline__ void arrive_on_even_cta(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & PEER_MASK) : "memory");
}
// activation half of this CTA; the transaction bytes are counted on the EVEN CTA's barrier
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar) & PEER_MASK), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// the pair's MMA: A (this CTA's and the peer's 128 rows) from tensor memory, B halves from both
// CTAs' shared memory at the descriptor's offset
__device__ __forceinline__ void mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc), "r"(0u)
        : "memory");
}
// completion of the pair's MMAs issued so far -> the barrier at this offset in BOTH CTAs
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(smem_u32(bar)), "h"((uint16_t)3)
        : "memory");
}

// How a launch's tiles become work units of the CTA pairs.  Tiles are numbered token-tile major
// (tile = token_tile * tiles_n + row_tile).  Without a K split every tile is one unit, dealt round
// robin.  With one, the launch is a whole number of PERIODS of `period` tiles each (the tiles of one
// prompt; the batch is a stack of equal prompts): the first `whole` tiles of every period are whole
// units (whole is a multiple of the number of pairs, so they fill complete waves) and each of the
// remaining period - whole tiles of every period is cut along K into `splits` slices whose partial
// sums a second kernel adds in slice order.  Which tiles are cut, and where, depends only on the
// position of a tile inside its prompt and on (N, K): a prompt's bits do not depend on its batch.
struct SplitPlan {
    int splits;   // 1: no K split
    int period;   // tiles per period
    int whole;    // whole-tile units per period
    int periods;  // periods in the launch
};
struct Unit {
    int tile, kb0, kb1;
    int slot;  // < 0: whole tile, the epilogue writes the output; else the partial-sum slot
};
__device__ __forceinline__ bool unit_at(int i, int pair, int pairs, int tiles, int kblocks, const SplitPlan& sp, Unit& u) {
    if (sp.splits <= 1) {
        u.tile = pair + i * pairs;
        u.kb0 = 0;
        u.kb1 = kblocks;
        u.slot = -1;
        return u.tile < tiles;
    }
    const int n_whole = sp.periods * sp.whole;
    const int g = pair + i * pairs;
    if (g < n_whole) {
        u.tile = (g / sp.whole) * sp.period + g % sp.whole;
        u.kb0 = 0;
        u.kb1 = kblocks;
        u.slot = -1;
        return true;
    }
    const int rem = sp.period - sp.whole;
    const int q = g - n_whole;  // n_whole is a multiple of pairs: slices start on a fresh wave
    if (q >= sp.periods * rem * sp.splits) return false;
    const int sl = q % sp.splits, r = q / sp.splits;
    u.tile = (r / rem) * sp.period + sp.whole + r % rem;
    u.kb0 = (int)((long)sl * kblocks / sp.splits);
    u.kb1 = (int)((long)(sl + 1) * kblocks / sp.splits);
    u.slot = q;
    return true;
}

template <int WKIND>
__global__ void __launch_bounds__(THREADS, 1)
gemm_dequant_pair_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                         const __grid_constant__ CUtensorMap tm_s, const __grid_constant__ CUtensorMap tm_o, GemmParams p,
                         SplitPlan sp) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* x_smem = smem;
    uint8_t* w_smem = smem + STAGES * X_STAGE;
    uint8_t* s_smem = w_smem + STAGES * W_STAGE;
    uint8_t* glu_smem = s_smem + STAGES * S_STAGE;
    Bars* bars = reinterpret_cast<Bars*>(glu_smem + NUM_EPI_WARPS * GLU_STAGE);
    volatile uint32_t* abort_flag = &bars->abort_flag;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();   // 0: even CTA (issues the MMAs), 1: odd CTA
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int kblocks = p.K / BK;
    const int tiles_m = (p.M + TT - 1) / TT;
    const int tiles_n = p.N / (2 * TW);
    const int tiles = tiles_m * tiles_n;
    constexpr uint32_t W_BYTES = (WKIND == 0) ? TW * BK : TW * BK / 2;
    constexpr uint32_t WTX_BYTES = W_BYTES + (WKIND != 0 ? S_STAGE : 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&bars->x_full[s], 1);
            mbar_init(&bars->w_full[s], 1);
            mbar_init(&bars->empty[s], NUM_DQ_WARPS);
        }
        for (int a = 0; a < ASTAGES; ++a) {
            mbar_init(&bars->a_full[a], 2 * NUM_DQ_WARPS);
            mbar_init(&bars->a_empty[a], 1);
        }
        mbar_init(&bars->acc_full, 1);
        mbar_init(&bars->acc_empty, 2 * NUM_EPI_WARPS);
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tm_x);
        tma_prefetch_desc(&tm_w);
        if (WKIND != 0) tma_prefetch_desc(&tm_s);
        if (p.tma_out) tma_prefetch_desc(&tm_o);
    }
    if (warp == 1) {
        tmem_alloc_pair(&bars->tmem_base, TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster.sync();  // both CTAs' barriers are initialised before anyone signals across the pair
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (elect_one()) {
            uint32_t it = 0;
            Unit u;
            for (int ui = 0; unit_at(ui, pair, pairs, tiles, kblocks, sp, u) && !*abort_flag; ++ui) {
                const int tile = u.tile;
                const int n0 = (tile % tiles_n) * (2 * TW) + rank * TW, m0 = (tile / tiles_n) * TT + rank * TH;
                for (int kb = u.kb0; kb < u.kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!mbar_wait<200>(&bars->empty[s], ph ^ 1u, abort_flag, 1)) break;
                    if (!mbar_wait<200>(&bars->a_empty[s], ph ^ 1u, abort_flag, 8)) break;
                    if (rank == 0) mbar_expect_tx(&bars->x_full[s], 2 * X_STAGE);
                    tma_load_2d_pair(x_smem + s * X_STAGE, &tm_x, &bars->x_full[s], kb * BK, m0);
                    mbar_expect_tx(&bars->w_full[s], WTX_BYTES);
                    if (WKIND == 0) {
                        tma_load_2d(w_smem + s * W_STAGE, &tm_w, &bars->w_full[s], kb * BK, n0);
                    } else {
                        tma_load_2d(w_smem + s * W_STAGE, &tm_w, &bars->w_full[s], kb * (BK / 2), n0);
                        tma_load_2d(s_smem + s * S_STAGE, &tm_s, &bars->w_full[s], n0, kb * 2);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (even CTA only) ----------------
        if (rank == 0 && elect_one()) {
            constexpr uint32_t IDESC = idesc_bf16_f32(2 * TW, TT);
            uint32_t it = 0, tile_i = 0;
            Unit u;
            for (int ui = 0; unit_at(ui, pair, pairs, tiles, kblocks, sp, u) && !*abort_flag; ++ui, ++tile_i) {
                if (!mbar_wait(&bars->acc_empty, (tile_i & 1u) ^ 1u, abort_flag, 2)) break;
                tc_fence_after();
                bool ok = true;
                for (int kb = u.kb0; kb < u.kb1; ++kb, ++it) {
                    const int s = it % STAGES, ai = it % ASTAGES;
                    const uint32_t ph = (it / STAGES) & 1u, aph = (it / ASTAGES) & 1u;
                    if (!mbar_wait(&bars->x_full[s], ph, abort_flag, 3) ||
                        !mbar_wait(&bars->a_full[ai], aph, abort_flag, 4)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t xs = smem_u32(x_smem + s * X_STAGE);
#pragma unroll
                    for (int j = 0; j < BK / 16; ++j)
                        mma_ts_pair(tmem, tmem + A_COL + ai * 32 + j * 8, smem_desc_kmajor(xs + j * 32, 128), IDESC, kb != u.kb0 || j != 0);
                    tc_commit_pair(&bars->a_empty[ai]);
                }
                if (!ok) break;
                tc_commit_pair(&bars->acc_full);
            }
        }
    } else if (warp < 2 + DQ_GROUPS * NUM_DQ_WARPS) {
        // ---------------- dequant warps (both CTAs, own weight rows) ----------------
        const int grp = (warp - 2) / NUM_DQ_WARPS;   // this group unpacks k-blocks it % DQ_GROUPS == grp
        const int dq = (warp - 2) % NUM_DQ_WARPS;
        const int quarter = warp & 3;
        const int half = dq >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        int pending = -1;
        auto flush = [&]() {
            if (pending >= 0) {
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) arrive_on_even_cta(&bars->a_full[pending]);
                pending = -1;
            }
        };
        Unit u;
        for (int ui = 0; unit_at(ui, pair, pairs, tiles, kblocks, sp, u) && ok && !*abort_flag; ++ui) {
            for (int kb = u.kb0; kb < u.kb1; ++kb, ++it) {
                if ((int)(it % DQ_GROUPS) != grp) continue;
                const int s = it % STAGES, ai = it % ASTAGES;
                const uint32_t ph = (it / STAGES) & 1u, aph = (it / ASTAGES) & 1u;
                if (!mbar_wait<100>(&bars->w_full[s], ph, abort_flag, 5)) { ok = false; break; }
                uint32_t a[16];
                if (WKIND == 0) {
                    const uint8_t* wrow = w_smem + s * W_STAGE + row * 64;
                    const int sw = (row >> 1) & 3;
                    uint4 v0 = lds128(wrow + (((2 * half) ^ sw) << 4));
                    uint4 v1 = lds128(wrow + (((2 * half + 1) ^ sw) << 4));
                    unpack_q8_word(v0.x, a[0], a[1]);   unpack_q8_word(v0.y, a[2], a[3]);
                    unpack_q8_word(v0.z, a[4], a[5]);   unpack_q8_word(v0.w, a[6], a[7]);
                    unpack_q8_word(v1.x, a[8], a[9]);   unpack_q8_word(v1.y, a[10], a[11]);
                    unpack_q8_word(v1.z, a[12], a[13]); unpack_q8_word(v1.w, a[14], a[15]);
                } else {
                    const uint8_t* wrow = w_smem + s * W_STAGE + row * 32;
                    const int sw = (row >> 2) & 1;
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
                if (lane == 0) mbar_arrive(&bars->empty[s]);
                flush();
                if (!mbar_wait<100>(&bars->a_empty[ai], aph ^ 1u, abort_flag, 7)) { ok = false; break; }
                tc_fence_after();
                tmem_st_x16(tmem + lane_addr + A_COL + ai * 32 + half * 16, a);
                pending = ai;
            }
        }
        flush();
    } else {
        // ---------------- epilogue warps (both CTAs, own accumulator rows) ----------------
        const int quarter = warp & 3;
        const int ehalf = (warp - 2 - DQ_GROUPS * NUM_DQ_WARPS) >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        // Staged output of the fused SwiGLU / GeGLU modes: the 32 tokens x 16 channels (bf16) a chunk
        // yields go to this warp's 1 KiB of shared memory, one `st.shared` per value at a fixed offset,
        // and one lane hands the box to a TMA store, which also clips the rows past M.  The kernel is
        // bound by instruction issue (with the epilogue's work removed the K = 2304 GEMMs run at
        // 1590-1650 TFLOP/s): address arithmetic, predicates and scattered 2-byte global stores were a
        // third of this epilogue's instructions.  The f32 modes store directly: staging them was
        // measured and changes nothing (their cost is the 128 KB per tile that has to leave through the
        // load/store path either way).
        const int epi = warp - 2 - DQ_GROUPS * NUM_DQ_WARPS;
        __nv_bfloat16* stage_bf = reinterpret_cast<__nv_bfloat16*>(glu_smem + epi * GLU_STAGE);
        bool store_pending = false;  // lane 0: a bulk store of this warp may still be reading the stage
        uint32_t tile_i = 0;
        Unit u;
        for (int ui = 0; unit_at(ui, pair, pairs, tiles, kblocks, sp, u) && !*abort_flag; ++ui, ++tile_i) {
            const int tile = u.tile;
            const int n0 = (tile % tiles_n) * (2 * TW) + rank * TW, m0 = (tile / tiles_n) * TT;
            if (!mbar_wait<80>(&bars->acc_full, tile_i & 1u, abort_flag, 6)) break;
            tc_fence_after();
            const int n = n0 + row;
            float rs = 1.0f;
            if (WKIND == 0) rs = p.row_scale[n];
            auto emit = [&](const uint32_t (&v)[32], int c) {
                const int mb = m0 + c * 32;
                if (mb >= p.M) return;
                if (p.tma_out) {  // SwiGLU / GeGLU, staged (whole tiles only: these modes are never K-split)
                    if (store_pending) bulk_wait_group_read0();
                    __syncwarp();
                    // gate / up of a channel in adjacent lanes (W1 / W3 rows interleaved): the lanes swap one
                    // value per token pair; the even lane finishes token j, the odd lane token j + 1
                    const bool odd = lane & 1;
                    const bool gelu = p.mode == GEMM_OUT_GEGLU;
                    __nv_bfloat16* dst = stage_bf + (odd ? 16 : 0) + (lane >> 1);
                    if (gelu) {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) {
                            float mine_a = __uint_as_float(v[j]), mine_b = __uint_as_float(v[j + 1]);
                            if (WKIND == 0) { mine_a *= rs; mine_b *= rs; }
                            const float got = __shfl_xor_sync(0xffffffffu, odd ? mine_a : mine_b, 1);
                            const float g = odd ? got : mine_a;
                            const float u_ = odd ? mine_b : got;
                            dst[j * 16] = __float2bfloat16_rn(gelu_tanh_f(g) * u_);
                        }
                    } else {
                        // two token pairs per step, the arithmetic of silu(g) * u as packed f32x2 operations
                        const uint64_t half2 = pack_f32x2(0.5f, 0.5f);
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float a0 = __uint_as_float(v[j]), b0 = __uint_as_float(v[j + 1]);
                            float a1 = __uint_as_float(v[j + 2]), b1 = __uint_as_float(v[j + 3]);
                            if (WKIND == 0) { a0 *= rs; b0 *= rs; a1 *= rs; b1 *= rs; }
                            const float got0 = __shfl_xor_sync(0xffffffffu, odd ? a0 : b0, 1);
                            const float got1 = __shfl_xor_sync(0xffffffffu, odd ? a1 : b1, 1);
                            const uint64_t g2 = pack_f32x2(odd ? got0 : a0, odd ? got1 : a1);
                            const uint64_t u2 = pack_f32x2(odd ? b0 : got0, odd ? b1 : got1);
                            float h0, h1, t0, t1, r0, r1;
                            unpack_f32x2(mul_f32x2(g2, half2), h0, h1);
                            asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(h0));
                            asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(h1));
                            const uint64_t sg2 = fma_f32x2(pack_f32x2(t0, t1), half2, half2);  // sigmoid(g) = 0.5 tanh(g / 2) + 0.5
                            unpack_f32x2(mul_f32x2(mul_f32x2(g2, sg2), u2), r0, r1);
                            dst[j * 16] = __float2bfloat16_rn(r0);
                            dst[(j + 2) * 16] = __float2bfloat16_rn(r1);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tm_o, stage_bf, (n0 + quarter * 32) >> 1, mb);
                        bulk_commit_group();
                        store_pending = true;
                    }
                    return;
                }
                if (u.slot >= 0) {
                    // K slice of a tile: partial sums, [token in tile][row in tile]
                    float* out = p.splitk_ws + ((size_t)u.slot * TT + c * 32) * (2 * TW) + rank * TW + row;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (mb + j < p.M) out[(size_t)j * (2 * TW)] = __uint_as_float(v[j]) * rs;
                } else if (p.mode == GEMM_OUT_F32 && p.vt && n >= p.vt_row0) {
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
                } else {
                    // gate / up pairs in adjacent lanes (see gemm_dequant.cu); SiLU or tanh-GELU on the gate
                    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)mb * p.ldo + (n >> 1);
                    const bool odd = lane & 1;
                    const bool gelu = p.mode == GEMM_OUT_GEGLU;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        float mine_a = __uint_as_float(v[j]), mine_b = __uint_as_float(v[j + 1]);
                        if (WKIND == 0) { mine_a *= rs; mine_b *= rs; }
                        float got = __shfl_xor_sync(0xffffffffu, odd ? mine_a : mine_b, 1);
                        float g = odd ? got : mine_a;
                        float u = odd ? mine_b : got;
                        int m = mb + j + (odd ? 1 : 0);
                        const float act = gelu ? gelu_tanh_f(g) : silu_f(g);
                        if (m < p.M) out[(size_t)(j + (odd ? 1 : 0)) * p.ldo] = __float2bfloat16_rn(act * u);
                    }
                }
            };
            const int c0 = ehalf * (TT / 64);
            const uint32_t t0 = tmem + lane_addr + c0 * 32;
#pragma unroll 1
            for (int i = 0; i < TT / 64; ++i) {
                uint32_t va[32];
                tmem_ld_x32(t0 + i * 32, va);
                tc_wait_ld();
                if (i + 1 == TT / 64) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) arrive_on_even_cta(&bars->acc_empty);
                }
                emit(va, c0 + i);
            }
        }
        if (store_pending) bulk_wait_group0();  // the staged stores have left shared memory and completed
    }

    // ---------------- common exit ----------------
    tc_fence_before();
    __syncthreads();
    cluster.sync();  // the peer is done with this CTA's shared and tensor memory
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, TMEM_COLS);
    }
    if (threadIdx.x == 0 && bars->abort_flag) atomicCAS(p.status, 0u, 0x400u | bars->abort_flag);
}

// Adds the K slices of every split tile in slice order and writes the f32 output.
// grid (split tiles of the launch, 16): a block covers 16 of the tile's 256 tokens.
__global__ void __launch_bounds__(256)
gemm_splitk_reduce_kernel(const float* __restrict__ ws, SplitPlan sp, int tiles_n, int M, float* __restrict__ out, int ldo) {
    const int r = blockIdx.x, rem = sp.period - sp.whole, splits = sp.splits;
    const int tile = (r / rem) * sp.period + sp.whole + r % rem;
    const int n0 = (tile % tiles_n) * (2 * TW), m0 = (tile / tiles_n) * TT;
    const int col = (threadIdx.x & 63) * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int mi = blockIdx.y * 16 + i * 4 + (threadIdx.x >> 6);
        if (m0 + mi >= M) continue;
        float4 acc = *reinterpret_cast<const float4*>(ws + (((size_t)r * splits) * TT + mi) * (2 * TW) + col);
        for (int sl = 1; sl < splits; ++sl) {
            const float4 v = *reinterpret_cast<const float4*>(ws + (((size_t)r * splits + sl) * TT + mi) * (2 * TW) + col);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *reinterpret_cast<float4*>(out + (size_t)(m0 + mi) * ldo + n0 + col) = acc;
    }
}

}  // namespace

bool gemm_pair_supported(const GemmParams& p) { return p.K % BK == 0 && p.N % (2 * TW) == 0 && p.M > 0; }
int gemm_pair_tile_tokens() { return TH; }

// The K-split plan of a launch (splits == 1: none).  `period_tokens`: tokens of one prompt when the
// launch is a stack of equal prompts, 0 when the launch is to be treated as a single period.
static SplitPlan plan_split(const GemmParams& p, int pairs, int period_tokens) {
    SplitPlan sp = {1, 0, 0, 0};
    const int tiles_n = p.N / (2 * TW), tiles_m = (p.M + TT - 1) / TT, kblocks = p.K / BK;
    if (p.mode != GEMM_OUT_F32 || p.vt || p.ldo % 4 || (reinterpret_cast<uintptr_t>(p.out) & 15)) return sp;
    int period_m = tiles_m, periods = 1;
    if (period_tokens > 0) {
        if (period_tokens % TT || p.M % period_tokens) return sp;  // prompts must start on tile boundaries
        period_m = period_tokens / TT;
        periods = p.M / period_tokens;
    }
    const int period = period_m * tiles_n, rem = period % pairs;
    // A partial wave that fills less than half of the pairs is cut along K instead: its tiles become
    // `splits` slices each, one slice per pair at most.  A slice shorter than 16 k-blocks is mostly ring
    // fill and drain, and a short K gains less than the reduction launch costs (measured: K = 2304 no
    // gain, K = 9216 +6 %).
    if (period <= pairs || rem == 0 || 2 * rem > pairs || kblocks < 64) return sp;
    const int splits = std::min(pairs / rem, kblocks / 16);
    if (splits < 2) return sp;
    sp.splits = splits; sp.period = period; sp.whole = period - rem; sp.periods = periods;
    return sp;
}

size_t gemm_pair_splitk_bytes(const GemmParams& p, int num_sms, int period_tokens) {
    if (!gemm_pair_supported(p)) return 0;
    const int tiles = ((p.M + TT - 1) / TT) * (p.N / (2 * TW));
    const int pairs = std::min(num_sms / 2, tiles);
    const SplitPlan sp = plan_split(p, pairs, period_tokens);
    return sp.splits > 1 ? (size_t)sp.periods * (sp.period - sp.whole) * sp.splits * GEMM_SPLITK_SLOT_BYTES : 0;
}

int launch_gemm_dequant_pair(int wkind, const CUtensorMap& tm_x, const CUtensorMap& tm_w, const CUtensorMap& tm_s,
                             const CUtensorMap& tm_out, const GemmParams& p, int num_sms, cudaStream_t stream) {
    if (!gemm_pair_supported(p)) return fail(ERR_SHAPE, "pair GEMM needs K % 64 == 0 and N % 256 == 0");
    static std::atomic<bool> configured[3][64];
    auto kern = wkind == 0 ? gemm_dequant_pair_kernel<0> : (wkind == 1 ? gemm_dequant_pair_kernel<1> : gemm_dequant_pair_kernel<2>);
    int dev = 0;
    CMFC_CUDA(cudaGetDevice(&dev));
    if (!configured[wkind][dev & 63]) {
        CMFC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[wkind][dev & 63] = true;
    }
    const int tiles = ((p.M + TT - 1) / TT) * (p.N / (2 * TW));
    int pairs = num_sms / 2;
    if (tiles < pairs) pairs = tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    SplitPlan sp = {1, 0, 0, 0};
    if (p.splitk_ws) sp = plan_split(p, pairs, p.split_period_tokens);
    CMFC_CUDA(cudaLaunchKernelEx(&cfg, kern, tm_x, tm_w, tm_s, tm_out, p, sp));
    if (sp.splits > 1) {
        gemm_splitk_reduce_kernel<<<dim3(sp.periods * (sp.period - sp.whole), TT / 16), 256, 0, stream>>>(
            p.splitk_ws, sp, p.N / (2 * TW), p.M, reinterpret_cast<float*>(p.out), p.ldo);
        CMFC_CUDA(cudaGetLastError());
    }
    return OK;
}

}  // namespace cmfc
