// Shared device/host helpers for the sm_100a kernels: status codes, mbarrier / TMA / tcgen05
// PTX wrappers with bounded waits, and small numeric utilities.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace cmfc {

// ---- status codes (mirrored in include/cmf_cuda.h) ----
enum : int {
    OK = 0,
    ERR_BAD_ARG = -1,
    ERR_UNSUPPORTED = -2,
    ERR_SHAPE = -3,
    ERR_OOM = -4,
    ERR_DEVICE_WAIT = -5,
    ERR_CUDA = -6,
    ERR_IO = -7,
    ERR_FORMAT = -8,
    ERR_NOT_FOUND = -9,
};

void set_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define CMFC_CUDA(expr)                                                                      \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess)                                                              \
            return ::cmfc::fail(::cmfc::ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(e__)); \
    } while (0)

#define CMFC_TRY(expr)              \
    do {                            \
        int rc__ = (expr);          \
        if (rc__ != 0) return rc__; \
    } while (0)

// Device-side wait budget: polls of mbarrier.try_wait before a kernel gives up, records the
// site in its status word and leaves through the normal exit path.
constexpr uint32_t WAIT_POLLS = 1u << 18;
constexpr uint32_t WAIT_PARK_NS = 8000;

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a phase.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Same, but the hardware may park the thread for up to ``hint_ns`` while the phase is pending,
// so a waiting warp does not compete for issue slots with the warps doing the work.
__device__ __forceinline__ bool mbar_try_parked(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the budget ran out or another thread already flagged an
// abort (``abort_flag`` lives in shared memory); the caller then unwinds to the common exit.
// ``nap_ns`` > 0 makes a waiter that is not on the critical path sleep between polls, so it
// leaves the issue slots of its scheduler to the warps doing the work.  The budget is about two
// seconds either way.
template <uint32_t NAP_NS = 0>
__device__ __forceinline__ bool mbar_wait_budget(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                                 uint32_t site, uint32_t polls) {
    if (mbar_try(bar, parity)) return true;
    for (uint32_t i = 0; i < polls; ++i) {
        if (NAP_NS) __nanosleep(NAP_NS);
        if (NAP_NS ? mbar_try(bar, parity) : mbar_try_parked(bar, parity, WAIT_PARK_NS)) return true;
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    atomicCAS(const_cast<uint32_t*>(abort_flag), 0u, site);
    return false;
}
template <uint32_t NAP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t site) {
    constexpr uint32_t polls = NAP_NS ? (2000000000u / (NAP_NS + 200u)) : WAIT_POLLS;
    return mbar_wait_budget<NAP_NS>(bar, parity, abort_flag, site, polls);
}

// ---- TMA (tiled, no multicast) ----
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
// Tiled store shared -> global (out-of-range rows / columns of the box are clipped by the tensor
// map), tracked by the issuing thread's bulk async-groups.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's bulk stores have finished READING their shared-memory source
__device__ __forceinline__ void bulk_wait_group_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... have completed
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- tcgen05 / tensor memory ----
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, f32 accumulate.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Instruction descriptor for kind::f16 with bf16 A/B (both K-major), f32 accumulator:
// c_format F32 at bits [4,6), a_format/b_format BF16 at [7,10)/[10,13), N>>3 at [17,23),
// M>>4 at [24,29).
__host__ __device__ constexpr uint32_t idesc_bf16_f32(uint32_t m, uint32_t n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Shared-memory matrix descriptor for a K-major operand whose rows are ``row_bytes`` long and
// stored with the matching TMA swizzle (row_bytes = 128 -> SWIZZLE_128B, 64 -> SWIZZLE_64B):
// start address >> 4 at [0,14), leading byte offset (unused for swizzled K-major, set to 1)
// at [16,30), stride byte offset = 8 rows * row_bytes >> 4 at [32,46), descriptor version 1
// at [46,48), layout type at [61,64) (2 = 128B swizzle, 4 = 64B swizzle).
__device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t smem_addr, uint32_t row_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8u * row_bytes) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(row_bytes == 128 ? 2 : (row_bytes == 64 ? 4 : 6)) << 61;
    return d;
}

// tcgen05.ld / st, shape 32x32b: thread t of warp w touches TMEM lane 32*(w%4)+t and N
// consecutive 32-bit columns starting at the address's column.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
          "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st_x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
        "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
        "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

// two f32 -> packed bf16x2 (lo in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// 2^x on the special-function unit (ex2.approx: relative error about 2^-22; -inf gives 0)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- packed f32x2 arithmetic: one issue slot for two lanes of the FMA pipe ----
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3_f32(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// 2^t for a pair without the special-function unit: n = round(t) through the 1.5 * 2^23 trick,
// a cubic for 2^(t - n) on [-0.5, 0.5] (relative error 7.5e-5, far below the bf16 rounding the
// result gets), n added into the exponent field.  t is clamped at -126.
// CLAMP = false: the caller guarantees t >= -126.
template <bool CLAMP = true>
__device__ __forceinline__ void ex2_poly_x2(float t0, float t1, float& e0, float& e1) {
    const float MAGIC = 12582912.0f;
    const uint64_t t = CLAMP ? pack_f32x2(fmaxf(t0, -126.0f), fmaxf(t1, -126.0f)) : pack_f32x2(t0, t1);
    const uint64_t r = add_f32x2(t, pack_f32x2(MAGIC, MAGIC));
    const uint64_t n = add_f32x2(r, pack_f32x2(-MAGIC, -MAGIC));
    const uint64_t f = fma_f32x2(n, pack_f32x2(-1.0f, -1.0f), t);
    uint64_t q = fma_f32x2(f, pack_f32x2(0.0551716648042202f, 0.0551716648042202f),
                           pack_f32x2(0.2426111251115799f, 0.2426111251115799f));
    q = fma_f32x2(q, f, pack_f32x2(0.6932609677314758f, 0.6932609677314758f));
    q = fma_f32x2(q, f, pack_f32x2(0.9999280571937561f, 0.9999280571937561f));
    float r0, r1, q0, q1;
    unpack_f32x2(r, r0, r1);
    unpack_f32x2(q, q0, q1);
    // exponent insertion as one integer multiply-add: q + (r << 23)
    e0 = __uint_as_float(__float_as_uint(r0) * 0x800000u + __float_as_uint(q0));
    e1 = __uint_as_float(__float_as_uint(r1) * 0x800000u + __float_as_uint(q1));
}

// Row statistics: the squares of four neighbouring values are summed in f32 (relative error
// below 2^-22) and those partial sums are accumulated in f64 across the row and the warp; the
// reciprocal root is taken in f64 and rounded once to f32.  The reference keeps every square and
// the scaling product in f64 (dit.rs:269-275); the difference, about 1e-7 relative per element, is
// far below the bf16 rounding of the GEMM operands that follows, and conversions between f32 and
// f64 (16 per clock per SM) no longer bound these kernels.
__device__ __forceinline__ double sq4(const float4& v) {
    return (double)fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
}
// rms(v; w, eps) element: (v * inv) * w
__device__ __forceinline__ float rms_elem(float v, float inv, float w) { return (v * inv) * w; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

#endif  // __CUDACC__

// Host: encode a 2-D tiled tensor map (row-major [rows, cols] of ``elem_bytes`` elements,
// row pitch ``pitch_bytes``; box = box_cols x box_rows).  swizzle: 0 none, 1 32B, 2 64B, 3 128B.
int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle);

int make_tensor_map_nhwc16(CUtensorMap* out, const void* base, uint64_t channels, uint64_t width, uint64_t height,
                           uint64_t pixel_pitch_bytes, uint32_t box_c, uint32_t box_w, uint32_t box_h, int swizzle);

}  // namespace cmfc
