// Host runtime behind the C ABI: per-device context (stream, workspaces, weight cache),
// the memory-mapped container, device weights and the device-level ops composed from kernels.
#pragma once
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace cmfc {

enum : int { DT_F32 = 0, DT_F16 = 1, DT_U8 = 6, DT_Q8 = 3, DT_Q4T = 11, DT_Q4TP = 15 };

// ---- growable device buffer (no allocation in steady state) ----
// Bumped whenever a device buffer is (re)allocated or freed: a captured CUDA graph holds raw
// pointers, so a graph captured under an older epoch must not be replayed.
uint64_t alloc_epoch();

struct DevBuf {
    void* p = nullptr;
    size_t cap = 0;
    int ensure(size_t bytes);
    void release();
    template <class T> T* as() const { return reinterpret_cast<T*>(p); }
};

// ---- container (crates/cortiq-core/src/format.rs: envelope, directory) ----
struct TensorRec {
    std::string name;
    int dtype = 0, ndim = 0;
    uint32_t shape[6] = {0, 0, 0, 0, 0, 0};
    uint64_t off = 0, nbytes = 0, hash = 0;
};
struct Model {
    uint64_t uid = 0;
    std::string path;
    const uint8_t* map = nullptr;
    size_t map_len = 0;
    uint64_t data_off = 0;
    std::vector<TensorRec> recs;
    std::map<std::string, int64_t> by_name;
    const uint8_t* bytes(int64_t idx) const { return map + data_off + recs[idx].off; }
};
int model_open(const char* path, Model** out);
void model_close(Model* m);
uint64_t hash64(const uint8_t* p, size_t n);
size_t payload_nbytes(int dtype, size_t rows, size_t cols);
float half_bits_to_float(uint16_t h);  // IEEE binary16 bit pattern -> f32 (host)

// ---- a weight resident on the device, in the planes the kernels read ----
struct DevWeight {
    int dtype = 0;         // DT_Q8 / DT_Q4T / DT_Q4TP / DT_F32
    int rows = 0, cols = 0;
    uint8_t* plane = nullptr;   // q8: int8 [rows, cols]; q4: nibbles [rows, cols/2]; f32: dense
    float* scales = nullptr;    // q8: row scales [rows]; q4: transposed group scales [cols/32, rows]
    CUtensorMap tm_w, tm_s;     // TMA descriptors of the planes (valid when gemm_ready)
    bool gemm_ready = false;
    bool owns = true;
    size_t bytes = 0;
    bool is_q4() const { return dtype == DT_Q4T || dtype == DT_Q4TP; }
    DevWeight() = default;
    DevWeight(const DevWeight&) = delete;
    DevWeight& operator=(const DevWeight&) = delete;
    ~DevWeight();  // frees plane and scales when `owns` (a failed upload must not leak them)
};

struct SegTable {
    std::vector<int> host;  // segment lengths
    const int* dev = nullptr;  // [nseg+1] token offsets, then [nseg] V^T column offsets
    int n_total = 0, vt_pitch = 0, max_seg = 0;
};

struct Profile {
    bool on = false;
    std::vector<std::pair<std::string, std::pair<cudaEvent_t, cudaEvent_t>>> spans;
};

struct Context {
    int device = -1;
    cudaStream_t stream = nullptr;     // every launch goes here ...
    // ... except while a forward runs two independent halves of its batch side by side: then the
    // second half's launches go to `side_stream` (Lane swaps it into `stream` while they are
    // enqueued) and use their own set of block workspaces (lane 1)
    cudaStream_t main_stream = nullptr, side_stream = nullptr;  // `stream` is one of the two
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    int lane = 0;
    int num_sms = 0;
    uint32_t* status = nullptr;       // device status word for bounded-wait kernels
    uint32_t* status_host = nullptr;  // pinned mirror
    // denoise schedule on the device: [2 * MAX_STEPS] floats (t_i, d_i) followed by the step counter
    static constexpr int MAX_STEPS = 1024;
    float* sched = nullptr;
    int* step_counter = nullptr;
    float* sched_host = nullptr;      // pinned staging, 2 * MAX_STEPS floats + 1 int
    std::map<std::tuple<uint64_t, int64_t, int64_t, int64_t, int>, std::unique_ptr<DevWeight>> weights;
    std::map<std::string, DevBuf> ws;  // named workspaces
    std::vector<std::pair<SegTable, DevBuf>> seg_cache;  // a few recent segmentations, each with its device table
    std::vector<float> facade_rope_host;  // the caller's f32 RoPE table that ws["facade_rope"] currently holds
    DevBuf resident_x;                 // hidden state kept between chained dit_block_seg calls
    size_t resident_len = 0;
    int gemm_period_tokens = 0;        // tokens per prompt while a forward runs a stack of equal prompts (else 0)
    float* log2_lut = nullptr;         // [65536] log2f of every f16 value (host libm)
    float* exp2_lut = nullptr;         // [65536] exp2f of every f16 value
    uint64_t launches = 0;
    Profile prof;
    DevBuf& buf(const std::string& name) { return ws[name]; }
    // a workspace of the current lane (block-level buffers that two concurrent halves must not share)
    DevBuf& lane_buf(const std::string& name) { return lane ? ws[name + "#1"] : ws[name]; }
};

// While alive, launches of the calling thread's context go to the side stream and use lane 1.
struct Lane {
    Context* c;
    cudaStream_t saved;
    explicit Lane(Context* c_) : c(c_), saved(c_->stream) { c->stream = c->side_stream; c->lane = 1; }
    ~Lane() { c->stream = saved; c->lane = 0; }
};

const std::string& last_error();
Context* ctx();  // context of the calling thread's current device (created on demand), or null
Context* ctx_existing();  // same, but never creates a context (and so never allocates)
int ctx_set_device(int device);
int check_status(Context* c, const char* what);  // reads the device status word (after a sync)

// weights
int get_weight(Context* c, Model* m, int64_t idx, DevWeight** out);
// concatenation along rows of up to three tensors (qkv), or row-interleave of two (w1/w3)
int get_weight_concat(Context* c, Model* m, int64_t a, int64_t b, int64_t cc, DevWeight** out);
int get_weight_interleaved(Context* c, Model* m, int64_t a, int64_t b, DevWeight** out);
int upload_f32(Context* c, Model* m, int64_t idx, DevWeight** out);  // any float tensor -> dense f32

// device-level ops (device pointers; async on c->stream)
// V^T destination of a fused QKV projection (see GemmParams::vt)
struct GemmVt {
    __nv_bfloat16* vt;
    int row0, pitch, nseg;
    const int* seg_table;
};
int dev_gemm(Context* c, DevWeight* w, const __nv_bfloat16* x, int M, void* out, int ldo, int mode,
             const GemmVt* vt = nullptr);
int prepare_segs(Context* c, const std::vector<int>& segs, SegTable* out);
// raw (optional): the queries come as the raw f32 projection and are normalised and rotated in the
// kernel's prologue (AttnParams::q_raw); q is then only a placeholder for the tensor map
struct AttnRawQ {
    const float* q_raw;
    int ld_q;
    const float *norm_q, *cos_t, *sin_t;
};
// score_ref: AttnParams::score_ref (0: the kernel tracks the row maximum)
int dev_attention(Context* c, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* vt,
                  const SegTable& st, int nh, int nkv, int hd, float scale, __nv_bfloat16* out,
                  const AttnRawQ* raw = nullptr, float score_ref = 0.0f, const unsigned* norm2_max = nullptr);
// Measures max |q_i| and max |k_j| over finished bf16 rows on the device (one small launch each and a
// synchronizing 8-byte read: not for a captured stream) and returns the fixed softmax reference they
// allow, or 0 when it would exceed ATTN_MAX_SCORE_REF or CMFC_ATTN_FIXED_REF=0 is set.
int attention_score_ref(Context* c, const __nv_bfloat16* q, const __nv_bfloat16* k, size_t n_total, int nh, int nkv,
                        int hd, float scale, float* score_ref);
// the same from the gains of the head norms: rows leave the norm with |q| <= sqrt(hd) * max |w_q|
float attention_score_ref_from_gain(float qk_gain, int hd);

struct BlockWeights {
    DevWeight *qkv = nullptr, *o = nullptr, *w13 = nullptr, *w2 = nullptr;
    const float *norm1 = nullptr, *norm2 = nullptr, *ffn_norm1 = nullptr, *ffn_norm2 = nullptr;
    const float *norm_q = nullptr, *norm_k = nullptr;
    float qk_gain = 0.0f;  // max |norm_q| * max |norm_k| (0: unknown, attention tracks the row maximum)
};
struct BlockMod {  // all null for an unmodulated block; gates already tanh'd
    const float *s_msa = nullptr, *gate_msa = nullptr, *s_mlp = nullptr, *gate_mlp = nullptr;
};
// One block over x [n, hidden] f32 in place (crates/cortiq-engine/src/dit.rs:943-1177).
// Chaining: when `next` is given, the block's last pass also writes the NEXT block's modulated
// input norm (bf16) so that block can skip its own first pass (`xn_ready`); this saves one read
// of x per block.
struct BlockChain {
    bool xn_ready = false;            // the shared bf16 norm buffer already holds this block's input norm
    const float* next_norm1 = nullptr;  // next block's norm1 weight, or null
    const float* next_s_msa = nullptr;  // next block's s_msa (null for an unmodulated block)
};
int dev_block(Context* c, const BlockWeights& bw, const BlockMod& mod, float* x, int n, const std::vector<int>& segs,
              int hidden, int inter, int nh, int nkv, int hd, double eps, const float* cos_t, const float* sin_t,
              const BlockChain* chain = nullptr);

bool row_cols_supported(int cols);
// single-head attention with a head wider than the flash kernel's 128 (host f32 in / out), vae.cu
int attention_single_head_wide(const float* q, const float* k, const float* v, size_t n, size_t c_dim, float scale,
                               float* out);
void launch_gemv_silu2(const GemvParams& p, float* y_silu, cudaStream_t s);

struct SpanGuard {
    Context* c;
    size_t idx = (size_t)-1;
    SpanGuard(Context* c, const char* name);
    ~SpanGuard();
};

}  // namespace cmfc

// The opaque handle of the C ABI wraps the container.
struct cmfc_model {
    cmfc::Model* m;
};
