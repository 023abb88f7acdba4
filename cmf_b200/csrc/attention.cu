// Bidirectional softmax attention over image + caption tokens, flash style on tcgen05
// (replaces NextDit::attention_seq, crates/cortiq-engine/src/dit.rs:846-922, and the facade's
// dit_attention, crates/cortiq-engine/src/gpu.rs:2332).  The n x n score matrix is never
// materialized; segments (independent sequences in one tall batch) never see each other.
//
// One CTA owns 256 queries of one (segment, head): two 128-row query tiles A and B that share
// every K / V^T tile brought in by TMA.  Per key tile (96 keys for head_dim <= 96, else 128):
//   S = Q K^T      tcgen05.mma, Q and K from shared memory (64-byte swizzle atoms of 32 dims,
//                  so head_dim 96 needs no padding), 128 queries x one key tile, f32, into TMEM.  Inside a NextDiT
//                  block the query tiles are built in the kernel's prologue from the raw f32
//                  projection (head RMS norm + 2-D RoPE, see the softmax warps); the facade entry
//                  passes finished bf16 rows, which arrive by TMA like K
//   softmax        four warps per query tile, one query row per thread: tcgen05.ld the row,
//                  running max / sum in the exp2 domain, P packed to bf16 and written back
//                  over the S columns with tcgen05.st
//   O += P V       tcgen05.mma with P as the TMEM A operand and V^T (keys contiguous, 128-byte
//                  swizzle) from shared memory, accumulating into the tile's O columns in TMEM
//   rescale        lazily: the reference maximum of a row moves only when the new maximum exceeds
//                  it by more than 8 (in log2 units), so P stays below 2^8 and the O row in TMEM
//                  is multiplied by exp2(m_old - m_new) on the few tiles where that happens
// While the softmax warps of tile A work, the tensor core runs tile B, and vice versa.
// The special-function unit (16 exp2 per clock per SM) is the busiest pipe of this kernel: the
// softmax arithmetic around it is packed (fma / add .f32x2, three-input max: one issue slot per
// two scores) and a quarter of the exponentials are computed on the FMA pipe instead (round to
// integer with the 1.5 * 2^23 trick, a cubic for the fraction, exponent inserted by an integer add).
//
// TMEM plan for head_dim <= 96 ("split" plan), key tiles of 96: S of tile A / B at columns 0 / 96, a P
// buffer for each tile at 192 / 256 (48 columns of packed bf16), O of tile A / B at 320 / 416.  P does
// not overwrite S, so S(j+1) of a tile is issued as soon as its softmax warps have pulled S(j) into
// registers and is ready long before they need it; and each tile has its own P buffer, so no tile ever
// waits for the other.  (With key tiles of 128 only one P buffer fits beside two S and two O tiles;
// cycle stamps of that version showed the two tiles taking turns on it -- P store, signal, P V issue,
// P V execution, signal, the other tile's P store -- a serial chain of about 2380 cycles per key tile
// that hid neither behind the 1540 cycles of exponentials nor behind the 1540 cycles of MMA.)
// head_dim 128 does not fit that plan (O needs 2 x 128 columns) and keeps P over S with key tiles of 128.
#include <atomic>

#include "common.cuh"
#include "kernels.h"

namespace cmfc {
namespace {

constexpr int QT = 128;   // query rows per tile (UMMA M)
// keys per tile (UMMA N for S, K extent for P V): 96 under the split plan, which is what lets every
// query tile own a P buffer (see the TMEM plan), else 128
template <int HD> __host__ __device__ constexpr int key_tile() { return HD <= 96 ? 96 : 128; }
constexpr int MAX_KV_STAGES = 3;
// K / V^T ring depth.  Three under the split plan: K(j+1) and V(j) are then requested two key tiles
// before they are used (with two, a load had about half a key tile of lead and its latency showed up
// as a late S(j+1)); head_dim 128 has room for two.
template <int HD> __host__ __device__ constexpr int kv_stages() { return HD <= 96 ? 3 : 2; }
// Softmax warps per query tile.  With the row maximum tracked in the kernel a thread owns a whole
// score row (4 warps per tile).  With the reference fixed before the launch nothing couples the
// parts of a row except the final row sum, so under the split plan two warps share the rows of a
// lane quarter (8 warps per tile, each thread half of a tile's scores): two warps per scheduler work
// on a tile's exponentials during its turn instead of one, which hides the dependent
// FMA -> exp2 -> pack chains of a single warp.
template <int HD, bool FIXED> __host__ __device__ constexpr int warps_per_tile() { return (FIXED && HD <= 96) ? 8 : 4; }
// warps: TMA, MMA (tile A), the softmax warps of tile A then B, MMA (tile B, split plan)
template <int HD, bool FIXED> __host__ __device__ constexpr int attn_threads() { return 32 * (3 + 2 * warps_per_tile<HD, FIXED>()); }

__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[32]) { tmem_ld_x32(taddr, r); }
__device__ __forceinline__ void tmem_ld_n(uint32_t taddr, uint32_t (&r)[16]) { tmem_ld_x16(taddr, r); }
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[16]) { tmem_st_x16(taddr, r); }
__device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&r)[8]) { tmem_st_x8(taddr, r); }
template <int HD> __host__ __device__ constexpr bool split_plan() { return HD <= 96; }
template <int HD> __host__ __device__ constexpr int s_col(int t) { return t * key_tile<HD>(); }
template <int HD> __host__ __device__ constexpr int p_col(int t) { return split_plan<HD>() ? 192 + t * 64 : s_col<HD>(t); }
template <int HD> __host__ __device__ constexpr int r_col(int t) { return split_plan<HD>() ? 320 + t * 96 : 256 + t * 128; }
constexpr int ATTN_TMEM_COLS = 512;


struct AttnBars {
    uint64_t q_full;
    uint64_t k_full[MAX_KV_STAGES], k_empty[MAX_KV_STAGES];
    uint64_t v_full[MAX_KV_STAGES], v_empty[MAX_KV_STAGES];
    uint64_t s_full[2], p_full[2], r_full[2];
    uint64_t stagger;  // tile A's softmax warps are half way through their first key tile
    uint64_t turn[2];  // split plan: tile t's softmax warps are TURN_CH chunks into the exponentials of a key tile
    uint64_t s_read[2];  // split plan: the tile's softmax warps hold S(j) in registers
    uint32_t tmem_base;
    uint32_t abort_flag;
};

template <int HD>
struct AttnSmem {
    static constexpr int ATOMS = HD / 32;
    static constexpr int Q_TILE = ATOMS * QT * 64;     // bytes of one query tile
    static constexpr int KT = key_tile<HD>();
    static constexpr int K_TILE = ATOMS * KT * 64;
    static constexpr int V_TILE = 2 * HD * 128;        // two boxes of HD rows x 64 keys
    static constexpr int KV_STAGES = kv_stages<HD>();
    static constexpr int LSUM = 2 * 2 * QT * 4;  // partial row sums of the two threads of a row (8 warps per tile)
    static constexpr int TOTAL = 2 * Q_TILE + KV_STAGES * (K_TILE + V_TILE) + 1024 + 256 + LSUM;
};

// POLY_OF_8: pairs out of every eight whose exp2 runs on the FMA pipe instead of the special-function unit.
// FIXED: the queries arrive multiplied by scale * log2(e) and every score of the launch is known to lie
// within +-p.score_ref <= 96 (see AttnParams): P = exp2(S) as it comes out of the MMA -- no scaling, no
// reference, no row maximum, no rescaling of O.
template <int HD, int POLY_OF_8, bool FIXED>
__global__ void __launch_bounds__((attn_threads<HD, FIXED>()), 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_vt, AttnParams p) {
    using L = AttnSmem<HD>;
    constexpr int KT = L::KT;
    constexpr int KV_STAGES = L::KV_STAGES;
    constexpr int WPT = warps_per_tile<HD, FIXED>();  // softmax warps per query tile
    constexpr int HALVES = WPT / 4;                    // threads sharing a score row
    constexpr int COLS = KT / HALVES;                  // scores per thread and key tile
    constexpr int CW = HALVES == 2 ? 16 : 32;          // scores per TMEM load
    constexpr int NCH = COLS / CW;                     // chunks of a thread's scores
    constexpr int MMA_B_WARP = 2 + 2 * WPT;
    static_assert(FIXED || HALVES == 1, "the running row maximum needs the whole row in one thread");
    const int seg = blockIdx.z, head = blockIdx.y;
    const int seg0 = p.seg_start[seg];
    const int seg_len = p.seg_start[seg + 1] - seg0;
    const int q0 = blockIdx.x * 2 * QT;
    if (q0 >= seg_len) return;  // uniform for the CTA, before any barrier or TMEM use
    if (p.norm2_max) {
        // both forms were launched; the measured norms decide which one runs (2 % covers the rounding of
        // the finished rows to bf16 and the f32 arithmetic of the measurement)
        const float bound = sqrtf(__uint_as_float(p.norm2_max[0])) * sqrtf(__uint_as_float(p.norm2_max[1])) * 1.02f;
        if ((bound <= ATTN_MAX_SCORE_REF) != FIXED) return;
    }
    const int vt0 = p.seg_start[p.nseg + 1 + seg];  // first V^T column of this segment (8-aligned)
    const int kvh = head / (p.nh / p.nkv);
    const int nk = (seg_len + KT - 1) / KT;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_smem = smem;
    uint8_t* k_smem = q_smem + 2 * L::Q_TILE;
    uint8_t* v_smem = k_smem + KV_STAGES * L::K_TILE;
    AttnBars* bars = reinterpret_cast<AttnBars*>(v_smem + KV_STAGES * L::V_TILE);
    float* lsum = reinterpret_cast<float*>(v_smem + KV_STAGES * L::V_TILE + 256);  // [tile][half][row]
    volatile uint32_t* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    const bool q_prologue = p.q_raw != nullptr;  // the softmax warps build the query tiles themselves
    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, q_prologue ? 8 : 1);
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(&bars->k_full[s], 1);
            // split plan: each tile has its own MMA warp, and both must be done with a stage
            mbar_init(&bars->k_empty[s], split_plan<HD>() ? 2 : 1);
            mbar_init(&bars->v_full[s], 1);
            mbar_init(&bars->v_empty[s], split_plan<HD>() ? 2 : 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&bars->s_full[t], 1);
            mbar_init(&bars->p_full[t], WPT);
            mbar_init(&bars->r_full[t], 1);
            if (t == 0) mbar_init(&bars->stagger, 4);
            mbar_init(&bars->turn[t], WPT);
            mbar_init(&bars->s_read[t], WPT);
        }
        bars->abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_vt);
    }
    if (warp == 1) {
        tmem_alloc(&bars->tmem_base, ATTN_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (elect_one()) {
            if (!q_prologue) {
                mbar_expect_tx(&bars->q_full, 2 * L::Q_TILE);
                for (int t = 0; t < 2; ++t)
                    for (int a = 0; a < L::ATOMS; ++a)
                        tma_load_2d(q_smem + t * L::Q_TILE + a * QT * 64, &tm_q, &bars->q_full, head * HD + 32 * a,
                                    seg0 + q0 + t * QT);
            }
            for (int j = 0; j < nk; ++j) {
                const int s = j % KV_STAGES;
                const uint32_t ph = (j / KV_STAGES) & 1u;
                if (!mbar_wait<200>(&bars->k_empty[s], ph ^ 1u, abort_flag, 11)) break;
                mbar_expect_tx(&bars->k_full[s], L::K_TILE);
                for (int a = 0; a < L::ATOMS; ++a)
                    tma_load_2d(k_smem + s * L::K_TILE + a * KT * 64, &tm_k, &bars->k_full[s], kvh * HD + 32 * a,
                                seg0 + j * KT);
                if (!mbar_wait<200>(&bars->v_empty[s], ph ^ 1u, abort_flag, 12)) break;
                mbar_expect_tx(&bars->v_full[s], L::V_TILE);
                for (int b = 0; b < 2; ++b)
                    tma_load_2d(v_smem + s * L::V_TILE + b * HD * 128, &tm_vt, &bars->v_full[s], vt0 + j * KT + 64 * b,
                                kvh * HD);
            }
        }
    } else if (warp == 1 || warp == MMA_B_WARP) {
        // ---------------- MMA issuer(s) ----------------
        // split plan: warp 1 issues for tile A, the last warp for tile B, each in its tile's own order
        // (a single thread walking a fixed order over both tiles stalls one tile on the other).
        if (warp == MMA_B_WARP && !split_plan<HD>()) {
            // nothing to do
        } else if (elect_one()) {
            constexpr uint32_t IDESC_S = idesc_bf16_f32(QT, KT);
            constexpr uint32_t IDESC_R = idesc_bf16_f32(QT, HD);
            auto issue_s = [&](int t, int s) {
                const uint32_t qa = smem_u32(q_smem + t * L::Q_TILE), ka = smem_u32(k_smem + s * L::K_TILE);
#pragma unroll
                for (int a = 0; a < L::ATOMS; ++a)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
                        mma_ss(tmem + s_col<HD>(t), smem_desc_kmajor(qa + a * QT * 64 + h * 32, 64),
                               smem_desc_kmajor(ka + a * KT * 64 + h * 32, 64), IDESC_S, (a | h) != 0);
            };
            auto issue_r = [&](int t, int s, bool first) {
                const uint32_t va = smem_u32(v_smem + s * L::V_TILE);
#pragma unroll
                for (int kk = 0; kk < KT / 16; ++kk)
                    mma_ts(tmem + r_col<HD>(t), tmem + p_col<HD>(t) + kk * 8,
                           smem_desc_kmajor(va + (kk >> 2) * HD * 128 + (kk & 3) * 32, 128), IDESC_R, !first || kk != 0);
            };
            bool ok = mbar_wait(&bars->q_full, 0, abort_flag, 13);
            if (ok) ok = mbar_wait(&bars->k_full[0], 0, abort_flag, 14);
            if constexpr (split_plan<HD>()) {
                const int t = warp == 1 ? 0 : 1;
                // The two query tiles share the special-function unit (softmax) and the tensor pipe.
                // Started together they stay in phase, each waiting on the unit the other one holds;
                // tile B starts once tile A is half way through its first softmax.
                if (ok) {
                    tc_fence_after();
                    issue_s(t, 0);
                    tc_commit(&bars->s_full[t]);
                    tc_commit(&bars->k_empty[0]);
                }
                for (int j = 0; ok && j < nk; ++j) {
                    const int s = j % KV_STAGES, s1 = (j + 1) % KV_STAGES;
                    const uint32_t jp = j & 1u;
                    if (j + 1 < nk) {
                        // S(j + 1) as soon as the tile's softmax warps hold S(j) in registers
                        if (!mbar_wait(&bars->k_full[s1], ((j + 1) / KV_STAGES) & 1u, abort_flag, 16)) { ok = false; break; }
                        if (!mbar_wait(&bars->s_read[t], jp, abort_flag, 22)) { ok = false; break; }
                        tc_fence_after();
                        issue_s(t, s1);
                        tc_commit(&bars->s_full[t]);
                        tc_commit(&bars->k_empty[s1]);
                    }
                    if (!mbar_wait(&bars->v_full[s], (j / KV_STAGES) & 1u, abort_flag, 15)) { ok = false; break; }
                    if (!mbar_wait(&bars->p_full[t], jp, abort_flag, 17)) { ok = false; break; }
                    tc_fence_after();
                    issue_r(t, s, j == 0);
                    tc_commit(&bars->r_full[t]);
                    tc_commit(&bars->v_empty[s]);
                }
            } else {
                if (ok) {
                    tc_fence_after();
                    issue_s(0, 0);
                    tc_commit(&bars->s_full[0]);
                    ok = mbar_wait(&bars->stagger, 0, abort_flag, 18);
                    if (ok) {
                        issue_s(1, 0);
                        tc_commit(&bars->s_full[1]);
                        tc_commit(&bars->k_empty[0]);
                    }
                }
                for (int j = 0; ok && j < nk; ++j) {
                    const int s = j % KV_STAGES;
                    const uint32_t ph = (j / KV_STAGES) & 1u, jp = j & 1u;
                    const bool more = j + 1 < nk;
                    const int s1 = (j + 1) % KV_STAGES;
                    const uint32_t ph1 = ((j + 1) / KV_STAGES) & 1u;
                    if (!mbar_wait(&bars->v_full[s], ph, abort_flag, 15)) { ok = false; break; }
                    if (more && !mbar_wait(&bars->k_full[s1], ph1, abort_flag, 16)) { ok = false; break; }
                    for (int t = 0; t < 2; ++t) {
                        // P_t(j) is in TMEM (and the O row was rescaled if its reference maximum moved)
                        if (!mbar_wait(&bars->p_full[t], jp, abort_flag, 17)) { ok = false; break; }
                        tc_fence_after();
                        issue_r(t, s, j == 0);
                        tc_commit(&bars->r_full[t]);
                        if (more) {
                            issue_s(t, s1);
                            tc_commit(&bars->s_full[t]);
                        }
                    }
                    if (!ok) break;
                    tc_commit(&bars->v_empty[s]);
                    if (more) tc_commit(&bars->k_empty[s1]);
                }
            }
        }
    } else {
        // ---------------- softmax warps ----------------
        // A warp reaches the 32 TMEM lanes of its index modulo 4; four consecutive warps cover a tile's rows.
        const int grp = (warp - 2) >> 2;
        const int t = grp / HALVES;             // query tile A / B
        const int half = grp % HALVES;          // which COLS scores of a row this thread owns
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;    // query row inside the tile
        const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
        const float c = p.scale * 1.4426950408889634f;  // softmax in the exp2 domain
        float m_ref = -INFINITY, l_run = 0.0f;
        bool ok = true;
        if (q_prologue && half == 0) {
            // Prologue: this thread's query row from the raw f32 projection -> per-head RMS norm
            // (eps 1e-5; crates/cortiq-engine/src/dit.rs:1078-1102) -> interleaved-pair rotation ->
            // bf16, written where the TMA load would have put it: atoms of 32 dims, 64 bytes per row,
            // 16-byte chunks XOR-ed with address bits [7, 9) (the 64-byte swizzle).  Same arithmetic
            // as qk_rope_kernel, which still prepares K (a K tile is read by every query tile of its
            // three query heads; rotating it here would repeat the work 51 times at 4352 tokens).
            const int q = q0 + t * QT + row;
            uint8_t* qrow = q_smem + t * L::Q_TILE + row * 64;
            const int swz = (row >> 1) & 3;
            if (q < seg_len) {
                const size_t tok = (size_t)(seg0 + q);
                const float4* src = reinterpret_cast<const float4*>(p.q_raw + tok * p.ld_q + (size_t)head * HD);
                const float4* ct = reinterpret_cast<const float4*>(p.cos_t + tok * (HD / 2));
                const float4* st = reinterpret_cast<const float4*>(p.sin_t + tok * (HD / 2));
                const float4* wq = reinterpret_cast<const float4*>(p.norm_q);
                float4 x[HD / 4];
#pragma unroll
                for (int i = 0; i < HD / 4; ++i) x[i] = src[i];
                double ss = 0.0;
#pragma unroll
                for (int i = 0; i < HD / 4; ++i) ss += sq4(x[i]);
                const float inv = (float)(1.0 / sqrt(ss / HD + 1e-5));
                const float qs = FIXED ? c : 1.0f;  // the fixed form takes its queries pre-scaled
                auto rot = [&](float a0, float a1, float g0, float g1, float cs, float sn) {
                    const float a = rms_elem(a0, inv, g0), b = rms_elem(a1, inv, g1);
                    return pack_bf16(fmaf(a, cs, -(b * sn)) * qs, fmaf(a, sn, b * cs) * qs);
                };
#pragma unroll
                for (int k = 0; k < HD / 8; ++k) {  // eight dims = four rotation pairs = one 16-byte chunk
                    const float4 g0 = __ldg(wq + 2 * k), g1 = __ldg(wq + 2 * k + 1);
                    const float4 cs = ct[k], sn = st[k];
                    uint4 o;
                    o.x = rot(x[2 * k].x, x[2 * k].y, g0.x, g0.y, cs.x, sn.x);
                    o.y = rot(x[2 * k].z, x[2 * k].w, g0.z, g0.w, cs.y, sn.y);
                    o.z = rot(x[2 * k + 1].x, x[2 * k + 1].y, g1.x, g1.y, cs.z, sn.z);
                    o.w = rot(x[2 * k + 1].z, x[2 * k + 1].w, g1.z, g1.w, cs.w, sn.w);
                    *reinterpret_cast<uint4*>(qrow + (k >> 2) * (QT * 64) + (((k & 3) ^ swz) << 4)) = o;
                }
            } else {
#pragma unroll
                for (int k = 0; k < HD / 8; ++k)
                    *reinterpret_cast<uint4*>(qrow + (k >> 2) * (QT * 64) + (((k & 3) ^ swz) << 4)) = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async_smem();  // generic-proxy writes, read by the tensor core through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->q_full);
        }
        for (int j = 0; j < nk; ++j) {
            if (!mbar_wait<60>(&bars->s_full[t], j & 1u, abort_flag, 19)) { ok = false; break; }
            tc_fence_after();
            // the whole score row of this thread: four loads in flight, one wait
            uint32_t v[NCH][CW];
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch) tmem_ld_n(tmem + lane_addr + s_col<HD>(t) + half * COLS + ch * CW, v[ch]);
            tc_wait_ld();
            if constexpr (split_plan<HD>()) {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->s_read[t]);
            }
            const int valid = seg_len - j * KT;  // keys of this tile inside the segment
            if constexpr (FIXED) {
                if (valid < KT) {
#pragma unroll
                    for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
                        for (int i = 0; i < CW; ++i)
                            if (half * COLS + ch * CW + i >= valid) v[ch][i] = 0xc2fc0000u;  // -126: 2^-126 beside P >= 2^-96
                }
            } else if constexpr (HALVES == 1) {
            // row maximum: eight independent chains (a single running maximum is a 128-deep
            // dependency chain on the critical path between S and P)
            float mxs[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) mxs[a] = -INFINITY;
            if (valid >= KT) {
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        mxs[(i >> 1) & 7] = max3_f32(mxs[(i >> 1) & 7], __uint_as_float(v[ch][i]), __uint_as_float(v[ch][i + 1]));
            } else {
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (ch * 32 + i >= valid) v[ch][i] = 0xff800000u;  // -inf: exp2 gives 0
                        mxs[i & 7] = fmaxf(mxs[i & 7], __uint_as_float(v[ch][i]));
                    }
            }
            const float mx = fmaxf(fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])),
                                   fmaxf(fmaxf(mxs[4], mxs[5]), fmaxf(mxs[6], mxs[7])));
            const float m_cand = mx * c;
            const bool moved = m_cand > m_ref + 8.0f;  // always true on the first tile
            if (__any_sync(0xffffffffu, moved)) {
                // s_full(j) is signalled after every earlier MMA of this tile finished, P V of tile
                // j-1 included, and P V of tile j is not issued before this thread arrives on
                // p_full: the O row can be rescaled in place.
                const float alpha = moved ? ex2_approx(m_ref - m_cand) : 1.0f;
                if (moved) m_ref = m_cand;
                l_run *= alpha;
                if (j > 0) {
                    if constexpr (split_plan<HD>()) {
                        // S(j) was issued before P V of tile j-1: wait for that MMA before touching O
                        if (!mbar_wait(&bars->r_full[t], (j - 1) & 1u, abort_flag, 23)) { ok = false; break; }
                        tc_fence_after();
                    }
                    // rare path, small chunks: the score row stays live in registers meanwhile
#pragma unroll 1
                    for (int ch = 0; ch < HD / 8; ++ch) {
                        uint32_t o[8];
                        tmem_ld_x8(tmem + lane_addr + r_col<HD>(t) + ch * 8, o);
                        tc_wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_x8(tmem + lane_addr + r_col<HD>(t) + ch * 8, o);
                    }
                }
            }
            }  // !FIXED
            // exp2(s * c - m) in pairs: packed FMA and packed sums (one issue slot per two elements);
            // POLY_OF_8 of every eight pairs take the polynomial route on the FMA pipe instead of the
            // special-function unit, which is the pipe that bounds this loop
            if constexpr (split_plan<HD>() && FIXED) {
                // The two tiles take turns on the special-function unit: A(j), B(j), A(j+1), ...  Left
                // alone they drift into phase, exponentiate at the same time at half speed each and
                // then both wait for the tensor pipe.  In turns, one tile's P store, its wait for the
                // next S and its TMEM load hide behind the other tile's exponentials.  (With the row
                // maximum tracked in the kernel the turns measured slower than running free.)
                if (t == 1 || j > 0) {
                    if (!mbar_wait(&bars->turn[t ^ 1], (t == 1 ? j : j - 1) & 1u, abort_flag, 25)) { ok = false; break; }
                }
            }
            uint64_t sums[4] = {0ull, 0ull, 0ull, 0ull};
            uint32_t pk[NCH][CW / 2];
            if constexpr (split_plan<HD>() && FIXED) {
                // Inside the turn only what needs the special-function unit (and the polynomial route
                // that relieves it): the exponentials replace the scores in place.  Packing to bf16 and
                // the row sum follow after the turn is handed over, beside the other tile's exponentials.
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
                    for (int i = 0; i < CW; i += 2) {
                        const float t0 = __uint_as_float(v[ch][i]), t1 = __uint_as_float(v[ch][i + 1]);
                        float e0, e1;
                        // the polynomial pairs spread among the others (pairs 0, 3, 6 of eight for POLY_OF_8 = 3)
                        if ((((i >> 1) & 7) * POLY_OF_8) % 8 < POLY_OF_8) {
                            ex2_poly_x2<false>(t0, t1, e0, e1);
                        } else {
                            e0 = ex2_approx(t0);
                            e1 = ex2_approx(t1);
                        }
                        v[ch][i] = __float_as_uint(e0);
                        v[ch][i + 1] = __float_as_uint(e1);
                    }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->turn[t]);
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
                    for (int i = 0; i < CW; i += 2) {
                        const float e0 = __uint_as_float(v[ch][i]), e1 = __uint_as_float(v[ch][i + 1]);
                        sums[(i >> 1) & 3] = add_f32x2(sums[(i >> 1) & 3], pack_f32x2(e0, e1));
                        pk[ch][i >> 1] = pack_bf16(e0, e1);
                    }
            } else {
            const uint64_t c2 = pack_f32x2(c, c), nm2 = pack_f32x2(-m_ref, -m_ref);
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch) {
#pragma unroll
                for (int i = 0; i < CW; i += 2) {
                    float t0, t1, e0, e1;
                    if constexpr (FIXED) {
                        t0 = __uint_as_float(v[ch][i]);
                        t1 = __uint_as_float(v[ch][i + 1]);
                    } else {
                        unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[ch][i]), __uint_as_float(v[ch][i + 1])), c2, nm2), t0, t1);
                    }
                    if (((i >> 1) & 7) < POLY_OF_8) {
                        ex2_poly_x2<!FIXED>(t0, t1, e0, e1);
                    } else {
                        e0 = ex2_approx(t0);
                        e1 = ex2_approx(t1);
                    }
                    sums[(i >> 1) & 3] = add_f32x2(sums[(i >> 1) & 3], pack_f32x2(e0, e1));
                    pk[ch][i >> 1] = pack_bf16(e0, e1);
                }
                if constexpr (!split_plan<HD>()) {
                    tmem_st_x16(tmem + lane_addr + p_col<HD>(t) + ch * 16, pk[ch]);
                    if (ch == 1 && t == 0 && j == 0) {
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bars->stagger);
                    }
                }
            }
            }
            if constexpr (split_plan<HD>()) {
                // The tile's own P buffer is free once P V of its previous key tile has run, which was
                // issued a whole softmax ago.
                if (j > 0) {
                    if (!mbar_wait<40>(&bars->r_full[t], (j - 1) & 1u, abort_flag, 24)) { ok = false; break; }
                    tc_fence_after();
                }
#pragma unroll
                for (int ch = 0; ch < NCH; ++ch)
                    tmem_st_n(tmem + lane_addr + p_col<HD>(t) + half * (COLS / 2) + ch * (CW / 2), pk[ch]);
            }
            tc_wait_st();
            {
                float s0, s1;
                unpack_f32x2(add_f32x2(add_f32x2(sums[0], sums[1]), add_f32x2(sums[2], sums[3])), s0, s1);
                l_run += s0 + s1;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->p_full[t]);
        }
        if constexpr (HALVES == 2) {
            // the two threads of a row add their partial sums; every softmax warp of the tile gets
            // here whether or not a wait gave up, so the named barrier cannot be left waiting
            lsum[(t * 2 + half) * QT + row] = l_run;
            if (t == 0) asm volatile("bar.sync 1, %0;" ::"n"(32 * WPT) : "memory");
            else asm volatile("bar.sync 2, %0;" ::"n"(32 * WPT) : "memory");
            l_run += lsum[(t * 2 + (half ^ 1)) * QT + row];
        }
        if (ok && mbar_wait(&bars->r_full[t], (nk - 1) & 1u, abort_flag, 21)) {
            tc_fence_after();
            const int qrow = q0 + t * QT + row;
            const float inv = 1.0f / l_run;
            constexpr int OC = HD / HALVES;  // output columns of this thread
            __nv_bfloat16* dst = p.out + ((size_t)(seg0 + qrow) * p.nh + head) * HD + half * OC;
#pragma unroll
            for (int ch = 0; ch < OC / 16; ++ch) {
                uint32_t o[16];
                tmem_ld_x16(tmem + lane_addr + r_col<HD>(t) + half * OC + ch * 16, o);
                tc_wait_ld();
                if (qrow < seg_len) {
#pragma unroll
                    for (int d = 0; d < 16; d += 8) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(o[d]) * inv, __uint_as_float(o[d + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(o[d + 2]) * inv, __uint_as_float(o[d + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(o[d + 4]) * inv, __uint_as_float(o[d + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(o[d + 6]) * inv, __uint_as_float(o[d + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + ch * 16 + d) = w;
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, ATTN_TMEM_COLS);
    }
    if (threadIdx.x == 0 && bars->abort_flag) atomicCAS(p.status, 0u, 0x200u | bars->abort_flag);
}

}  // namespace

int attn_key_tile(int hd) { return hd <= 96 ? key_tile<96>() : key_tile<128>(); }

int attn_smem_bytes(int hd) {
    switch (hd) {
        case 32: return AttnSmem<32>::TOTAL;
        case 64: return AttnSmem<64>::TOTAL;
        case 96: return AttnSmem<96>::TOTAL;
        case 128: return AttnSmem<128>::TOTAL;
        default: return 0;
    }
}

template <int HD, int POLY, bool FIXED>
static int launch_hd(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_vt, const AttnParams& p,
                     cudaStream_t stream) {
    static std::atomic<bool> configured[64];  // per instantiation and device; never repeated inside a stream capture
    int dev = 0;
    CMFC_CUDA(cudaGetDevice(&dev));
    if (!configured[dev & 63]) {
        CMFC_CUDA(cudaFuncSetAttribute(attention_kernel<HD, POLY, FIXED>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       AttnSmem<HD>::TOTAL));
        configured[dev & 63] = true;
    }
    dim3 grid((p.max_seg + 2 * QT - 1) / (2 * QT), p.nh, p.nseg);
    attention_kernel<HD, POLY, FIXED><<<grid, attn_threads<HD, FIXED>(), AttnSmem<HD>::TOTAL, stream>>>(tm_q, tm_k, tm_vt, p);
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

template <int HD, int POLY>
static int launch_ref(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_vt, const AttnParams& p,
                      cudaStream_t stream) {
    // the bounded form balances its exponentials at POLY of 8 on the FMA pipe; the tracking form, whose
    // polynomial route also clamps its argument, at two of eight
    return p.score_ref > 0.0f ? launch_hd<HD, POLY, true>(tm_q, tm_k, tm_vt, p, stream)
                              : launch_hd<HD, 2, false>(tm_q, tm_k, tm_vt, p, stream);
}

int launch_attention(const CUtensorMap& tm_q, const CUtensorMap& tm_k, const CUtensorMap& tm_vt, const AttnParams& p,
                     cudaStream_t stream) {
    if (p.score_ref < 0.0f || p.score_ref > ATTN_MAX_SCORE_REF)
        return fail(ERR_BAD_ARG, "attention: the score bound must lie in (0, 96] log2 units, or be 0");
    switch (p.hd) {
        case 32: return launch_ref<32, 3>(tm_q, tm_k, tm_vt, p, stream);
        case 64: return launch_ref<64, 3>(tm_q, tm_k, tm_vt, p, stream);
        case 96: return launch_ref<96, 3>(tm_q, tm_k, tm_vt, p, stream);
        case 128: return launch_ref<128, 2>(tm_q, tm_k, tm_vt, p, stream);
        default: return fail(ERR_UNSUPPORTED, "attention: head_dim must be 32, 64, 96 or 128");
    }
}

}  // namespace cmfc
