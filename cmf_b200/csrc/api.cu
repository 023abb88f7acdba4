// The C ABI (include/cmf_cuda.h): argument checks, host<->device staging, and the device-resident
// NextDiT forward and Euler loop composed from the kernels.
#include <math.h>
#include <string.h>

#include <sstream>

#include "../../include/cmf_cuda.h"
#include "runtime.h"

using namespace cmfc;

namespace cmfc {
const std::string& last_error();
}

#define NEED_CTX()                                                         \
    Context* c = ctx();                                                    \
    if (!c) return last_error().empty() ? fail(ERR_CUDA, "no CUDA device") : ERR_CUDA;
#define NEED(cond, msg) \
    if (!(cond)) return fail(ERR_BAD_ARG, msg)

extern "C" const char* cmfc_last_error(void) { return last_error().c_str(); }

extern "C" int cmfc_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
    return n;
}
extern "C" int cmfc_set_device(int device) { return ctx_set_device(device); }
extern "C" int cmfc_synchronize(void) {
    NEED_CTX();
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    return check_status(c, "synchronize");
}

// ---------------- container ----------------
extern "C" int cmfc_model_open(const char* path, cmfc_model** out) {
    NEED(path && out, "cmfc_model_open: null argument");
    Model* m = nullptr;
    CMFC_TRY(model_open(path, &m));
    *out = new cmfc_model{m};
    return OK;
}
extern "C" void cmfc_model_close(cmfc_model* m) {
    if (!m) return;
    model_close(m->m);
    delete m;
}
extern "C" int64_t cmfc_model_tensor_count(const cmfc_model* m) { return m ? (int64_t)m->m->recs.size() : 0; }
extern "C" int64_t cmfc_model_find(const cmfc_model* m, const char* name) {
    if (!m || !name) return fail(ERR_BAD_ARG, "cmfc_model_find: null argument");
    auto it = m->m->by_name.find(name);
    if (it == m->m->by_name.end()) return fail(ERR_NOT_FOUND, std::string("no tensor named ") + name);
    return it->second;
}
extern "C" int cmfc_model_tensor_info(const cmfc_model* m, int64_t idx, int* dtype, int* ndim, uint32_t shape[6],
                                      uint64_t* nbytes) {
    NEED(m && idx >= 0 && idx < (int64_t)m->m->recs.size(), "tensor index out of range");
    const TensorRec& t = m->m->recs[idx];
    if (dtype) *dtype = t.dtype;
    if (ndim) *ndim = t.ndim;
    if (shape) memcpy(shape, t.shape, sizeof(t.shape));
    if (nbytes) *nbytes = t.nbytes;
    return OK;
}
extern "C" const char* cmfc_model_tensor_name(const cmfc_model* m, int64_t idx) {
    if (!m || idx < 0 || idx >= (int64_t)m->m->recs.size()) return nullptr;
    return m->m->recs[idx].name.c_str();
}
extern "C" const void* cmfc_model_tensor_bytes(const cmfc_model* m, int64_t idx) {
    if (!m || idx < 0 || idx >= (int64_t)m->m->recs.size()) return nullptr;
    return m->m->bytes(idx);
}
extern "C" int cmfc_weight_is_resident(const cmfc_model* m, int64_t idx) {
    Context* c = ctx();
    if (!c || !m) return 0;
    return c->weights.count(std::make_tuple(m->m->uid, idx, (int64_t)-1, (int64_t)-1, 0)) ? 1 : 0;
}

static int dequant_to(Context* c, DevWeight* w, float* d_out) {
    if (w->dtype == DT_Q8) launch_dequant_q8(reinterpret_cast<const int8_t*>(w->plane), w->scales, w->rows, w->cols, d_out, c->stream);
    else if (w->is_q4()) launch_dequant_q4(w->plane, w->scales, w->rows, w->cols, w->dtype == DT_Q4T ? 1 : 0, d_out, c->stream);
    else return fail(ERR_UNSUPPORTED, "dequant: not a quantized weight");
    c->launches++;
    return OK;
}

extern "C" int cmfc_weight_dequant(cmfc_model* m, int64_t idx, float* out, size_t out_len) {
    NEED(m && out, "cmfc_weight_dequant: null argument");
    NEED_CTX();
    DevWeight* w = nullptr;
    CMFC_TRY(get_weight(c, m->m, idx, &w));
    NEED(out_len == (size_t)w->rows * w->cols, "cmfc_weight_dequant: out_len must be rows*cols");
    DevBuf& d = c->buf("dequant_out");
    CMFC_TRY(d.ensure(out_len * 4));
    CMFC_TRY(dequant_to(c, w, d.as<float>()));
    CMFC_CUDA(cudaMemcpyAsync(out, d.p, out_len * 4, cudaMemcpyDeviceToHost, c->stream));
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    return OK;
}

// ---------------- quantized linears ----------------
static int matmat_any(cmfc_model* m, int64_t idx, int want_dtype, const float* xs, size_t b, size_t rows, size_t cols,
                      float* out) {
    NEED(m && xs && out && b > 0, "matmat: null argument or empty batch");
    NEED_CTX();
    DevWeight* w = nullptr;
    CMFC_TRY(get_weight(c, m->m, idx, &w));
    if (want_dtype >= 0 && m->m->recs[idx].dtype != want_dtype)
        return fail(ERR_UNSUPPORTED, "matmat: tensor " + m->m->recs[idx].name + " has dtype " +
                                         std::to_string(m->m->recs[idx].dtype) + ", this entry serves dtype " + std::to_string(want_dtype));
    if ((size_t)w->rows != rows || (size_t)w->cols != cols) return fail(ERR_SHAPE, "matmat: rows/cols disagree with the tensor's directory record");
    DevBuf &xf = c->buf("mm_xf"), &xb = c->buf("mm_xb"), &y = c->buf("mm_y");
    CMFC_TRY(xf.ensure(b * cols * 4));
    CMFC_TRY(xb.ensure(b * cols * 2));
    CMFC_TRY(y.ensure(b * rows * 4));
    CMFC_CUDA(cudaMemcpyAsync(xf.p, xs, b * cols * 4, cudaMemcpyHostToDevice, c->stream));
    launch_f32_to_bf16(xf.as<float>(), xb.as<__nv_bfloat16>(), b * cols, c->stream);
    c->launches++;
    CMFC_TRY(dev_gemm(c, w, xb.as<__nv_bfloat16>(), (int)b, y.p, (int)rows, GEMM_OUT_F32));
    CMFC_CUDA(cudaMemcpyAsync(out, y.p, b * rows * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "matmat");
}
extern "C" int cmfc_q8_matmat(cmfc_model* m, int64_t idx, const float* xs, size_t b, size_t rows, size_t cols, float* out) {
    return matmat_any(m, idx, DT_Q8, xs, b, rows, cols, out);
}
extern "C" int cmfc_q4t_matmat(cmfc_model* m, int64_t idx, const float* xs, size_t b, size_t rows, size_t cols, float* out) {
    return matmat_any(m, idx, DT_Q4T, xs, b, rows, cols, out);
}
extern "C" int cmfc_q4tp_matmat(cmfc_model* m, int64_t idx, const float* xs, size_t b, size_t rows, size_t cols, float* out) {
    return matmat_any(m, idx, DT_Q4TP, xs, b, rows, cols, out);
}

extern "C" int cmfc_dit_qkv(cmfc_model* m, int64_t wq, int64_t wk, int64_t wv, const float* xs, size_t b, size_t hidden,
                            size_t qrows, size_t kvrows, float* q_out, float* k_out, float* v_out) {
    NEED(m && xs && q_out && k_out && v_out && b > 0, "dit_qkv: null argument or empty batch");
    NEED_CTX();
    DevWeight* w = nullptr;
    CMFC_TRY(get_weight_concat(c, m->m, wq, wk, wv, &w));
    if ((size_t)w->cols != hidden || (size_t)w->rows != qrows + 2 * kvrows) return fail(ERR_SHAPE, "dit_qkv: shapes disagree with the tensors");
    const size_t wd = qrows + 2 * kvrows;
    DevBuf &xf = c->buf("mm_xf"), &xb = c->buf("mm_xb"), &y = c->buf("mm_y");
    CMFC_TRY(xf.ensure(b * hidden * 4));
    CMFC_TRY(xb.ensure(b * hidden * 2));
    CMFC_TRY(y.ensure(b * wd * 4));
    CMFC_CUDA(cudaMemcpyAsync(xf.p, xs, b * hidden * 4, cudaMemcpyHostToDevice, c->stream));
    launch_f32_to_bf16(xf.as<float>(), xb.as<__nv_bfloat16>(), b * hidden, c->stream);
    c->launches++;
    CMFC_TRY(dev_gemm(c, w, xb.as<__nv_bfloat16>(), (int)b, y.p, (int)wd, GEMM_OUT_F32));
    CMFC_CUDA(cudaMemcpy2DAsync(q_out, qrows * 4, y.as<float>(), wd * 4, qrows * 4, b, cudaMemcpyDeviceToHost, c->stream));
    CMFC_CUDA(cudaMemcpy2DAsync(k_out, kvrows * 4, y.as<float>() + qrows, wd * 4, kvrows * 4, b, cudaMemcpyDeviceToHost, c->stream));
    CMFC_CUDA(cudaMemcpy2DAsync(v_out, kvrows * 4, y.as<float>() + qrows + kvrows, wd * 4, kvrows * 4, b, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "dit_qkv");
}

extern "C" int cmfc_ffn(cmfc_model* m, int64_t w1, int64_t w3, int64_t w2, const float* xs, size_t b, size_t hidden,
                        size_t inter, float* out) {
    NEED(m && xs && out && b > 0, "ffn: null argument or empty batch");
    NEED_CTX();
    DevWeight *w13 = nullptr, *wd = nullptr;
    CMFC_TRY(get_weight_interleaved(c, m->m, w1, w3, &w13));
    CMFC_TRY(get_weight(c, m->m, w2, &wd));
    if ((size_t)w13->cols != hidden || (size_t)w13->rows != 2 * inter || (size_t)wd->rows != hidden || (size_t)wd->cols != inter)
        return fail(ERR_SHAPE, "ffn: shapes disagree with the tensors");
    DevBuf &xf = c->buf("mm_xf"), &xb = c->buf("mm_xb"), &act = c->buf("blk_act"), &y = c->buf("mm_y");
    CMFC_TRY(xf.ensure(b * hidden * 4));
    CMFC_TRY(xb.ensure(b * hidden * 2));
    CMFC_TRY(act.ensure(b * inter * 2));
    CMFC_TRY(y.ensure(b * hidden * 4));
    CMFC_CUDA(cudaMemcpyAsync(xf.p, xs, b * hidden * 4, cudaMemcpyHostToDevice, c->stream));
    launch_f32_to_bf16(xf.as<float>(), xb.as<__nv_bfloat16>(), b * hidden, c->stream);
    c->launches++;
    CMFC_TRY(dev_gemm(c, w13, xb.as<__nv_bfloat16>(), (int)b, act.p, (int)inter, GEMM_OUT_SWIGLU));
    CMFC_TRY(dev_gemm(c, wd, act.as<__nv_bfloat16>(), (int)b, y.p, (int)hidden, GEMM_OUT_F32));
    CMFC_CUDA(cudaMemcpyAsync(out, y.p, b * hidden * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "ffn");
}

extern "C" int cmfc_dit_attention(const float* qh, const float* kh, const float* vh, size_t nh, size_t nkv, size_t n,
                                  size_t hd, float scale, float* out) {
    NEED(qh && kh && vh && out && n > 0 && nh > 0 && nkv > 0, "dit_attention: null argument or empty input");
    // the VAE's attention block: one head as wide as the channel count (vae.rs:438)
    if (hd > 128 && nh == 1 && nkv == 1) return attention_single_head_wide(qh, kh, vh, n, hd, scale, out);
    NEED_CTX();
    std::vector<int> segs{(int)n};
    SegTable st;
    CMFC_TRY(prepare_segs(c, segs, &st));
    DevBuf &in = c->buf("att_in"), &qb = c->buf("blk_q"), &kb = c->buf("blk_k"), &vt = c->buf("blk_vt"), &ob = c->buf("blk_attn"),
           &of = c->buf("att_out");
    const size_t qn = nh * n * hd, kn = nkv * n * hd;
    CMFC_TRY(in.ensure((qn + 2 * kn) * 4));
    CMFC_TRY(qb.ensure(qn * 2));
    CMFC_TRY(kb.ensure(kn * 2));
    if (vt.cap < (size_t)nkv * hd * st.vt_pitch * 2) {
        CMFC_TRY(vt.ensure((size_t)nkv * hd * st.vt_pitch * 2));
        CMFC_CUDA(cudaMemsetAsync(vt.p, 0, vt.cap, c->stream));
    }
    CMFC_TRY(ob.ensure(qn * 2));
    CMFC_TRY(of.ensure(qn * 4));
    float* d_in = in.as<float>();
    CMFC_CUDA(cudaMemcpyAsync(d_in, qh, qn * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(d_in + qn, kh, kn * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(d_in + qn + kn, vh, kn * 4, cudaMemcpyHostToDevice, c->stream));
    launch_transpose_head_major(d_in, (int)nh, (int)n, (int)hd, 1.0f, qb.as<__nv_bfloat16>(), c->stream);
    launch_transpose_head_major(d_in + qn, (int)nkv, (int)n, (int)hd, 1.0f, kb.as<__nv_bfloat16>(), c->stream);
    launch_v_head_major_to_vt(d_in + qn + kn, (int)nkv, (int)n, (int)hd, vt.as<__nv_bfloat16>(), st.vt_pitch, c->stream);
    c->launches += 3;
    float score_ref = 0.0f;
    CMFC_TRY(attention_score_ref(c, qb.as<__nv_bfloat16>(), kb.as<__nv_bfloat16>(), n, (int)nh, (int)nkv, (int)hd, scale, &score_ref));
    if (score_ref > 0.0f) {  // the bounded form takes its queries multiplied by scale * log2(e)
        launch_transpose_head_major(d_in, (int)nh, (int)n, (int)hd, scale * 1.4426950408889634f, qb.as<__nv_bfloat16>(), c->stream);
        c->launches++;
    }
    CMFC_TRY(dev_attention(c, qb.as<__nv_bfloat16>(), kb.as<__nv_bfloat16>(), vt.as<__nv_bfloat16>(), st, (int)nh, (int)nkv,
                           (int)hd, scale, ob.as<__nv_bfloat16>(), nullptr, score_ref));
    launch_bf16_to_f32(ob.as<__nv_bfloat16>(), of.as<float>(), qn, c->stream);
    c->launches++;
    CMFC_CUDA(cudaMemcpyAsync(out, of.p, qn * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "dit_attention");
}

// ---------------- one block through the facade ----------------
namespace {

// small host vectors -> one device scratch area, sub-allocated at 256-byte steps
struct Staging {
    Context* c;
    DevBuf* buf;
    size_t off = 0;
    std::vector<uint8_t> host;
    Staging(Context* c_, const char* name, size_t reserve) : c(c_), buf(&c_->buf(name)) { host.reserve(reserve); }
    size_t add(const void* p, size_t bytes) {
        size_t at = host.size();
        host.resize(at + ((bytes + 255) & ~size_t(255)));
        if (p) memcpy(host.data() + at, p, bytes);
        return at;
    }
    int commit() {
        CMFC_TRY(buf->ensure(host.size()));
        CMFC_CUDA(cudaMemcpyAsync(buf->p, host.data(), host.size(), cudaMemcpyHostToDevice, c->stream));
        CMFC_CUDA(cudaStreamSynchronize(c->stream));
        return OK;
    }
    template <class T> const T* at(size_t o) const { return reinterpret_cast<const T*>(buf->as<uint8_t>() + o); }
};

}  // namespace

extern "C" int cmfc_dit_block_seg(cmfc_model* m, const cmfc_dit_block_args* a, const uint32_t* segs, size_t nseg, float* x) {
    NEED(m && a && segs && nseg > 0, "dit_block_seg: null argument");
    NEED(a->resident_in || x, "dit_block_seg: x is null and the state is not resident");
    NEED(a->rope_cos && a->rope_sin && a->norm1 && a->norm2 && a->ffn_norm1 && a->ffn_norm2 && a->norm_q && a->norm_k,
         "dit_block_seg: null norm or rope pointer");
    const bool modulated = a->s_msa || a->gate_msa || a->s_mlp || a->gate_mlp;
    NEED(!modulated || (a->s_msa && a->gate_msa && a->s_mlp && a->gate_mlp), "dit_block_seg: partial modulation");
    NEED(a->hd % 2 == 0 && a->hidden == a->nh * a->hd, "dit_block_seg: hidden must equal nh*hd with an even hd");
    NEED_CTX();
    std::vector<int> sv(nseg);
    size_t tot = 0;
    for (size_t i = 0; i < nseg; ++i) { sv[i] = (int)segs[i]; tot += segs[i]; }
    NEED(tot == a->n, "dit_block_seg: segments do not sum to n");
    const size_t n = a->n, hs = a->hidden, pairs = a->hd / 2;
    BlockWeights bw;
    CMFC_TRY(get_weight_concat(c, m->m, a->wq, a->wk, a->wv, &bw.qkv));
    CMFC_TRY(get_weight(c, m->m, a->wo, &bw.o));
    CMFC_TRY(get_weight_interleaved(c, m->m, a->w1, a->w3, &bw.w13));
    CMFC_TRY(get_weight(c, m->m, a->w2, &bw.w2));
    if ((size_t)bw.qkv->rows != (a->nh + 2 * a->nkv) * (size_t)a->hd || (size_t)bw.qkv->cols != hs || (size_t)bw.w13->rows != 2 * (size_t)a->inter ||
        (size_t)bw.w2->cols != a->inter || (size_t)bw.o->rows != hs)
        return fail(ERR_SHAPE, "dit_block_seg: projection shapes disagree with the block geometry");
    // rope: the caller's f32 cos / sin tables as they are; re-uploaded only when they change.  The
    // host copy they are compared with belongs to the context, like the device buffer it describes,
    // so a thread that moves between devices never matches another GPU's table.
    std::vector<float>& rope_cache = c->facade_rope_host;
    DevBuf& rope = c->buf("facade_rope");
    const size_t rn = n * pairs;
    bool same = rope_cache.size() == 2 * rn && rope.p && !memcmp(rope_cache.data(), a->rope_cos, rn * 4) &&
                !memcmp(rope_cache.data() + rn, a->rope_sin, rn * 4);
    if (!same) {
        rope_cache.clear();
        CMFC_CUDA(cudaStreamSynchronize(c->stream));  // an earlier block may still read the old table
        CMFC_TRY(rope.ensure(2 * rn * 4));
        // on the stream the readers run on (it is not ordered after the legacy default stream)
        CMFC_CUDA(cudaMemcpyAsync(rope.p, a->rope_cos, rn * 4, cudaMemcpyHostToDevice, c->stream));
        CMFC_CUDA(cudaMemcpyAsync(rope.as<float>() + rn, a->rope_sin, rn * 4, cudaMemcpyHostToDevice, c->stream));
        CMFC_CUDA(cudaStreamSynchronize(c->stream));  // the caller's buffers are borrowed for this call only
        rope_cache.assign(a->rope_cos, a->rope_cos + rn);
        rope_cache.insert(rope_cache.end(), a->rope_sin, a->rope_sin + rn);
    }
    Staging st(c, "facade_vecs", 16 * hs * 4);
    const size_t o_n1 = st.add(a->norm1, hs * 4), o_n2 = st.add(a->norm2, hs * 4), o_f1 = st.add(a->ffn_norm1, hs * 4),
                 o_f2 = st.add(a->ffn_norm2, hs * 4), o_nq = st.add(a->norm_q, a->hd * 4), o_nk = st.add(a->norm_k, a->hd * 4);
    size_t o_sm = 0, o_gm = 0, o_sl = 0, o_gl = 0;
    if (modulated) {
        o_sm = st.add(a->s_msa, hs * 4); o_gm = st.add(a->gate_msa, hs * 4);
        o_sl = st.add(a->s_mlp, hs * 4); o_gl = st.add(a->gate_mlp, hs * 4);
    }
    CMFC_TRY(st.commit());
    bw.norm1 = st.at<float>(o_n1); bw.norm2 = st.at<float>(o_n2); bw.ffn_norm1 = st.at<float>(o_f1); bw.ffn_norm2 = st.at<float>(o_f2);
    bw.norm_q = st.at<float>(o_nq); bw.norm_k = st.at<float>(o_nk);
    {
        float gq = 0.0f, gk = 0.0f;
        for (size_t i = 0; i < a->hd; ++i) { gq = fmaxf(gq, fabsf(a->norm_q[i])); gk = fmaxf(gk, fabsf(a->norm_k[i])); }
        bw.qk_gain = gq * gk;
    }
    BlockMod mod;
    if (modulated) { mod.s_msa = st.at<float>(o_sm); mod.gate_msa = st.at<float>(o_gm); mod.s_mlp = st.at<float>(o_sl); mod.gate_mlp = st.at<float>(o_gl); }
    if (!a->resident_in) {
        CMFC_TRY(c->resident_x.ensure(n * hs * 4));
        CMFC_CUDA(cudaMemcpyAsync(c->resident_x.p, x, n * hs * 4, cudaMemcpyHostToDevice, c->stream));
        c->resident_len = n * hs;
    } else if (c->resident_len != n * hs) {
        return fail(ERR_BAD_ARG, "dit_block_seg: resident_in set but no state of this size is on the device");
    }
    CMFC_TRY(dev_block(c, bw, mod, c->resident_x.as<float>(), (int)n, sv, (int)hs, (int)a->inter, (int)a->nh, (int)a->nkv, (int)a->hd,
                       (double)a->eps, rope.as<float>(), rope.as<float>() + rn));
    if (!a->resident_out) {
        NEED(x, "dit_block_seg: x is null but resident_out is not set");
        CMFC_CUDA(cudaMemcpyAsync(x, c->resident_x.p, n * hs * 4, cudaMemcpyDeviceToHost, c->stream));
    }
    return check_status(c, "dit_block_seg");
}
extern "C" int cmfc_dit_chain_supported(void) { return 1; }
extern "C" int cmfc_fused_dit_block_available(void) { return 0; }
extern "C" int cmfc_dit_state_fetch(float* x, size_t len) {
    NEED(x, "dit_state_fetch: null pointer");
    NEED_CTX();
    NEED(len == c->resident_len && c->resident_x.p, "dit_state_fetch: no resident state of that length");
    CMFC_CUDA(cudaMemcpyAsync(x, c->resident_x.p, len * 4, cudaMemcpyDeviceToHost, c->stream));
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    return OK;
}

// ---------------- NextDiT, device resident ----------------
struct DitBlock {
    BlockWeights bw;
    bool modulated = false;
    DevWeight* mod_w = nullptr;   // q8 plane + row scales, or dense f32
    const float* mod_b = nullptr;
};

struct cmfc_nextdit {
    Model* m = nullptr;
    int hidden = 0, cap_feat = 0, ch = 0, patch = 2, nl = 0, nr = 2, nh = 0, nkv = 0, hd = 0, inter = 0, temb = 0;
    int axes[3] = {0, 0, 0};
    double eps = 1e-5;
    std::vector<DitBlock> ctx_ref, noise_ref, layers;
    const float *x_emb_w = nullptr, *x_emb_b = nullptr, *t1w = nullptr, *t1b = nullptr, *t2w = nullptr, *t2b = nullptr;
    const float *cap_norm = nullptr, *cap_b = nullptr, *out1_w = nullptr, *out1_b = nullptr, *out2_w = nullptr, *out2_b = nullptr;
    DevWeight* cap_w = nullptr;  // quantized (tensor core path) or dense f32
    // rope tables cached by geometry, one set per forward shape (index 0: one sequence per prompt,
    // 1: the cond/uncond pair), so the two captured step graphs never share a table
    std::string rope_key[2];
    DevBuf rope_joint[2], rope_img[2], rope_cap;
    uint64_t rope_epoch = 0;           // bumped by every table upload: a captured graph reads the tables' contents
    // denoise state
    DevBuf latents, cap_c_r, cap_u_r, pred_c, pred_u;
    size_t batch = 0, lh = 0, lw = 0, cap_n = 0, cap_u_n = 0;
    uint32_t steps = 0;
    uint32_t cfg_steps = 0;            // steps [0, cfg_steps) run the guided pair, the rest cond only
    float gs = 4.0f;
    bool cfg = false;
    bool cfg_norm = true;
    std::vector<double> sig;
    uint32_t next_step = 0;            // value of the device step counter
    // captured denoise steps (all launches of forward + CFG/Euler), replayed by later steps of the
    // same kind: index 0 = cond-only step, 1 = guided (pair) step
    struct StepGraph {
        cudaGraphExec_t exec = nullptr;
        uint64_t alloc_epoch = 0;      // allocation epoch at capture time
        uint64_t rope_epoch = 0;       // rope-table epoch at capture time
        uint64_t launches = 0;         // kernel launches inside the graph
        int eager_steps = 0;           // steps of this kind run eagerly since the last begin (the first warms buffers)
        void drop() {
            if (exec) cudaGraphExecDestroy(exec);
            exec = nullptr;
        }
    } graphs[2];
    std::string graph_key;
};

namespace {

int dense_f32(Context* c, Model* m, const std::string& name, const float** out, int* rows = nullptr, int* cols = nullptr) {
    auto it = m->by_name.find(name);
    if (it == m->by_name.end()) return fail(ERR_NOT_FOUND, "missing tensor " + name);
    const TensorRec& t = m->recs[it->second];
    DevWeight* w = nullptr;
    if (t.dtype == DT_F32 || t.dtype == DT_F16) {
        CMFC_TRY(upload_f32(c, m, it->second, &w));
    } else {
        // quantized where the engine expects a small dense matrix: dequantize once on the device
        auto key = std::make_tuple(m->uid, it->second, (int64_t)-1, (int64_t)-1, 8);
        auto f = c->weights.find(key);
        if (f != c->weights.end()) w = f->second.get();
        else {
            DevWeight* q = nullptr;
            CMFC_TRY(get_weight(c, m, it->second, &q));
            std::unique_ptr<DevWeight> d(new DevWeight());
            d->dtype = DT_F32; d->rows = q->rows; d->cols = q->cols;
            if (cudaMalloc(&d->plane, (size_t)q->rows * q->cols * 4) != cudaSuccess) return fail(ERR_OOM, "out of device memory for " + name);
            CMFC_TRY(dequant_to(c, q, reinterpret_cast<float*>(d->plane)));
            CMFC_CUDA(cudaStreamSynchronize(c->stream));
            w = d.get();
            c->weights[key] = std::move(d);
        }
    }
    *out = reinterpret_cast<const float*>(w->plane);
    if (rows) *rows = w->rows;
    if (cols) *cols = w->cols;
    return OK;
}

int64_t find_idx(Model* m, const std::string& name) {
    auto it = m->by_name.find(name);
    return it == m->by_name.end() ? -1 : it->second;
}

// minimal JSON number / array lookup for dit.config_json
bool json_num(const std::string& js, const char* key, double* out) {
    std::string k = std::string("\"") + key + "\"";
    size_t p = js.find(k);
    if (p == std::string::npos) return false;
    p = js.find(':', p + k.size());
    if (p == std::string::npos) return false;
    ++p;
    while (p < js.size() && isspace((unsigned char)js[p])) ++p;
    char* end = nullptr;
    double v = strtod(js.c_str() + p, &end);
    if (end == js.c_str() + p) return false;
    *out = v;
    return true;
}
bool json_arr3(const std::string& js, const char* key, int out[3]) {
    std::string k = std::string("\"") + key + "\"";
    size_t p = js.find(k);
    if (p == std::string::npos) return false;
    p = js.find('[', p);
    if (p == std::string::npos) return false;
    ++p;
    for (int i = 0; i < 3; ++i) {
        char* end = nullptr;
        out[i] = (int)strtol(js.c_str() + p, &end, 10);
        if (end == js.c_str() + p) return false;
        p = end - js.c_str();
        while (p < js.size() && (js[p] == ',' || isspace((unsigned char)js[p]))) ++p;
    }
    return true;
}

int load_block(Context* c, cmfc_nextdit* d, const std::string& p, bool modulated, DitBlock* b) {
    Model* m = d->m;
    auto need = [&](const std::string& n) -> int64_t { return find_idx(m, n); };
    const int64_t iq = need(p + ".attn.to_q.weight"), ik = need(p + ".attn.to_k.weight"), iv = need(p + ".attn.to_v.weight"),
                  io = need(p + ".attn.to_out.0.weight"), i1 = need(p + ".feed_forward.linear_1.weight"),
                  i3 = need(p + ".feed_forward.linear_3.weight"), i2 = need(p + ".feed_forward.linear_2.weight");
    if (iq < 0 || ik < 0 || iv < 0 || io < 0 || i1 < 0 || i3 < 0 || i2 < 0) return fail(ERR_NOT_FOUND, "block " + p + " is missing a projection");
    CMFC_TRY(get_weight_concat(c, m, iq, ik, iv, &b->bw.qkv));
    CMFC_TRY(get_weight(c, m, io, &b->bw.o));
    CMFC_TRY(get_weight_interleaved(c, m, i1, i3, &b->bw.w13));
    CMFC_TRY(get_weight(c, m, i2, &b->bw.w2));
    b->modulated = modulated;
    CMFC_TRY(dense_f32(c, m, p + (modulated ? ".norm1.norm.weight" : ".norm1.weight"), &b->bw.norm1));
    CMFC_TRY(dense_f32(c, m, p + ".norm2.weight", &b->bw.norm2));
    CMFC_TRY(dense_f32(c, m, p + ".ffn_norm1.weight", &b->bw.ffn_norm1));
    CMFC_TRY(dense_f32(c, m, p + ".ffn_norm2.weight", &b->bw.ffn_norm2));
    CMFC_TRY(dense_f32(c, m, p + ".attn.norm_q.weight", &b->bw.norm_q));
    CMFC_TRY(dense_f32(c, m, p + ".attn.norm_k.weight", &b->bw.norm_k));
    {
        const int hd = d->hd;
        std::vector<float> g(2 * (size_t)hd);
        CMFC_CUDA(cudaMemcpy(g.data(), b->bw.norm_q, hd * sizeof(float), cudaMemcpyDeviceToHost));
        CMFC_CUDA(cudaMemcpy(g.data() + hd, b->bw.norm_k, hd * sizeof(float), cudaMemcpyDeviceToHost));
        float gq = 0.0f, gk = 0.0f;
        for (int i = 0; i < hd; ++i) { gq = fmaxf(gq, fabsf(g[i])); gk = fmaxf(gk, fabsf(g[hd + i])); }
        b->bw.qk_gain = gq * gk;
    }
    if (modulated) {
        const int64_t im = need(p + ".norm1.linear.weight");
        if (im < 0) return fail(ERR_NOT_FOUND, "block " + p + " is missing its modulation linear");
        if (m->recs[im].dtype == DT_Q8) CMFC_TRY(get_weight(c, m, im, &b->mod_w));
        else {
            const float* dummy;
            CMFC_TRY(dense_f32(c, m, p + ".norm1.linear.weight", &dummy));
            const int key_kind = (m->recs[im].dtype == DT_F32 || m->recs[im].dtype == DT_F16) ? 9 : 8;
            b->mod_w = c->weights[std::make_tuple(m->uid, im, (int64_t)-1, (int64_t)-1, key_kind)].get();
        }
        CMFC_TRY(dense_f32(c, m, p + ".norm1.linear.bias", &b->mod_b));
    }
    return OK;
}

// host RoPE table (crates/cortiq-engine/src/dit.rs:366-381) for a list of position ids: angles, cos
// and sin in f64, rounded once to the f32 the device kernel reads
void rope_rows(const std::vector<int>& ids3, const int axes[3], std::vector<float>* cs, std::vector<float>* sn) {
    const size_t n = ids3.size() / 3;
    const int pairs = (axes[0] + axes[1] + axes[2]) / 2;
    cs->resize(n * pairs);
    sn->resize(n * pairs);
    std::vector<double> freq;
    std::vector<int> axis_of;
    for (int a = 0; a < 3; ++a)
        for (int j = 0; j < axes[a] / 2; ++j) {
            freq.push_back(1.0 / pow(10000.0, 2.0 * j / (double)axes[a]));
            axis_of.push_back(a);
        }
    for (size_t i = 0; i < n; ++i)
        for (int j = 0; j < pairs; ++j) {
            const double ang = (double)ids3[3 * i + axis_of[j]] * freq[j];
            (*cs)[i * pairs + j] = (float)cos(ang);
            (*sn)[i * pairs + j] = (float)sin(ang);
        }
}
int upload_rope(Context* c, DevBuf* buf, const std::vector<int>& ids3, const int axes[3]) {
    std::vector<float> cs, sn;
    rope_rows(ids3, axes, &cs, &sn);
    // kernels already queued on the stream may still read the previous table
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    CMFC_TRY(buf->ensure(cs.size() * 8));
    // on the stream the readers run on (it is not ordered after the legacy default stream)
    CMFC_CUDA(cudaMemcpyAsync(buf->p, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(buf->as<float>() + cs.size(), sn.data(), sn.size() * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaStreamSynchronize(c->stream));  // cs / sn are locals
    return OK;
}
void push_ids(std::vector<int>* v, int a, int b, int cc) { v->push_back(a); v->push_back(b); v->push_back(cc); }

// `next` / `next_mods`: the block that follows on the SAME rows (or null); `xn_ready`: the previous
// call already produced this block's input norm.
// `rope` holds cos then sin for `rope_rows_n` rows; the block runs on rows [row0, row0 + n) of that table.
int run_block(Context* c, cmfc_nextdit* d, const DitBlock& b, float* x, int n, const std::vector<int>& segs, const float* mods,
              const DevBuf& rope, size_t rope_rows_n, const DitBlock* next = nullptr, const float* next_mods = nullptr,
              bool xn_ready = false, size_t row0 = 0) {
    BlockMod mod;
    if (b.modulated) {
        mod.s_msa = mods; mod.gate_msa = mods + d->hidden; mod.s_mlp = mods + 2 * d->hidden; mod.gate_mlp = mods + 3 * d->hidden;
    }
    const size_t half = rope_rows_n * (d->hd / 2);
    BlockChain ch;
    ch.xn_ready = xn_ready;
    if (next) {
        ch.next_norm1 = next->bw.norm1;
        ch.next_s_msa = next->modulated ? next_mods : nullptr;
    }
    const size_t at = row0 * (d->hd / 2);
    return dev_block(c, b.bw, mod, x, n, segs, d->hidden, d->inter, d->nh, d->nkv, d->hd, d->eps, rope.as<float>() + at,
                     rope.as<float>() + half + at, &ch);
}

// y = W x + b for a small dense or q8 weight
void gemv(Context* c, const DevWeight* w, const float* bias, const float* x, float* y, float* y_silu, int tanh_hidden) {
    GemvParams p;
    p.w = w->plane; p.w_is_q8 = w->dtype == DT_Q8; p.row_scale = w->dtype == DT_Q8 ? w->scales : nullptr;
    p.bias = bias; p.x = x; p.y = y; p.rows = w->rows; p.cols = w->cols; p.act_in = 0;
    p.tanh_lo0 = p.tanh_hi0 = p.tanh_lo1 = p.tanh_hi1 = -1;
    if (tanh_hidden > 0) { p.tanh_lo0 = tanh_hidden; p.tanh_hi0 = 2 * tanh_hidden; p.tanh_lo1 = 3 * tanh_hidden; p.tanh_hi1 = 4 * tanh_hidden; }
    launch_gemv_silu2(p, y_silu, c->stream);
    c->launches++;
}
void gemv_dense(Context* c, const float* w, int rows, int cols, const float* bias, const float* x, float* y, float* y_silu) {
    DevWeight tmp;
    tmp.dtype = DT_F32; tmp.rows = rows; tmp.cols = cols; tmp.plane = reinterpret_cast<uint8_t*>(const_cast<float*>(w)); tmp.owns = false;
    gemv(c, &tmp, bias, x, y, y_silu, 0);
}

// caption features [rows, cap_feat] (device f32) -> refined [rows, hidden] over `segs`
int refine_caps(Context* c, cmfc_nextdit* d, const float* cap, const std::vector<int>& segs, float* out) {
    int rows = 0;
    for (int s : segs) rows += s;
    if (!row_cols_supported(d->cap_feat)) return fail(ERR_UNSUPPORTED, "caption feature width is not supported by the row kernels");
    if (d->cap_w->dtype == DT_F32) {
        DevBuf& nf = c->buf("cap_norm_f32");
        CMFC_TRY(nf.ensure((size_t)rows * d->cap_feat * 4));
        launch_rms_mod(cap, d->cap_norm, nullptr, d->eps, rows, d->cap_feat, nullptr, nf.as<float>(), c->stream);
        launch_sgemm_nt_bias(nf.as<float>(), reinterpret_cast<const float*>(d->cap_w->plane), d->cap_b, out, rows, d->hidden, d->cap_feat, c->stream);
        c->launches += 2;
    } else {
        DevBuf& nb = c->buf("cap_norm_bf16");
        CMFC_TRY(nb.ensure((size_t)rows * d->cap_feat * 2));
        launch_rms_mod(cap, d->cap_norm, nullptr, d->eps, rows, d->cap_feat, nb.as<__nv_bfloat16>(), nullptr, c->stream);
        c->launches++;
        CMFC_TRY(dev_gemm(c, d->cap_w, nb.as<__nv_bfloat16>(), rows, out, d->hidden, GEMM_OUT_F32));
        launch_add_bias_rows(out, d->cap_b, rows, d->hidden, c->stream);
        c->launches++;
    }
    std::vector<int> ids;
    for (int s : segs)
        for (int i = 0; i < s; ++i) push_ids(&ids, i, 0, 0);
    CMFC_TRY(upload_rope(c, &d->rope_cap, ids, d->axes));
    for (size_t l = 0; l < d->ctx_ref.size(); ++l) {
        const DitBlock* nx = l + 1 < d->ctx_ref.size() ? &d->ctx_ref[l + 1] : nullptr;
        CMFC_TRY(run_block(c, d, d->ctx_ref[l], out, rows, segs, nullptr, d->rope_cap, rows, nx, nullptr, l > 0));
    }
    return OK;
}

// Upload (t_i, d_i) pairs and reset the device step counter.  The pinned staging area is reused,
// so wait for earlier work on the stream that may still read it.
int upload_schedule(Context* c, const std::vector<float>& td, int start_step) {
    if (td.size() > 2 * (size_t)Context::MAX_STEPS) return fail(ERR_BAD_ARG, "too many steps (limit 1024)");
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    memcpy(c->sched_host, td.data(), td.size() * 4);
    reinterpret_cast<int*>(c->sched_host)[2 * Context::MAX_STEPS] = start_step;
    CMFC_CUDA(cudaMemcpyAsync(c->sched, c->sched_host, td.size() * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(c->step_counter, c->sched_host + 2 * Context::MAX_STEPS, 4, cudaMemcpyHostToDevice, c->stream));
    return OK;
}

// One velocity prediction for `batch` prompts.  caps[q] (device, refined) for q in [0, nseq):
// nseq = 1 (no CFG) or 2 (cond, uncond); each is [batch, cap_ns[q], hidden].  preds[q] receive
// [batch, c, h, w].  taps (optional, device): x after each joint layer.
int forward_device(Context* c, cmfc_nextdit* d, const float* latents, int batch, int h, int w, int nseq, const float* const caps[2],
                   const int cap_ns[2], float t, float* const preds[2], float* taps) {
    const int hs = d->hidden, p = d->patch, pv = p * p * d->ch;
    if (h % p || w % p) return fail(ERR_BAD_ARG, "latent height and width must be multiples of the patch size");
    const int hp = h / p, wp = w / p, n_img = hp * wp;
    cudaStream_t s = c->stream;
    // ---- conditioning vectors ----
    DevBuf& cv = c->buf("cond_vecs");
    const size_t n_mod = d->noise_ref.size() + d->layers.size();
    CMFC_TRY(cv.ensure((256 + 3 * (size_t)d->temb + hs + n_mod * 4 * hs) * 4 + 4096));
    float* freqs = cv.as<float>();
    float* h1_silu = freqs + 256;
    float* temb = h1_silu + d->temb;
    float* temb_silu = temb + d->temb;
    float* out_scale = temb_silu + d->temb;
    float* mods = out_scale + hs;
    {
        SpanGuard g(c, "head-tail");
        launch_time_freqs(c->sched, c->step_counter, freqs, s);
        c->launches++;
        gemv_dense(c, d->t1w, d->temb, 256, d->t1b, freqs, temb /*scratch*/, h1_silu);
        gemv_dense(c, d->t2w, d->temb, d->temb, d->t2b, h1_silu, temb, temb_silu);
        gemv_dense(c, d->out1_w, hs, d->temb, d->out1_b, temb_silu, out_scale, nullptr);
    }
    {
        SpanGuard g(c, "mod-norm");
        size_t k = 0;
        for (auto* grp : {&d->noise_ref, &d->layers})
            for (auto& b : *grp) gemv(c, b.mod_w, b.mod_b, temb_silu, mods + (k++) * 4 * hs, nullptr, hs);
    }
    // ---- image branch: patchify, embed, noise refiners (once per prompt) ----
    DevBuf &tok = c->buf("fw_tok"), &img = c->buf("fw_img"), &xb = c->buf("fw_x"), &xn = c->buf("fw_xn"), &outb = c->buf("fw_out");
    CMFC_TRY(tok.ensure((size_t)batch * n_img * pv * 4));
    CMFC_TRY(img.ensure((size_t)batch * n_img * hs * 4));
    {
        SpanGuard g(c, "head-tail");
        for (int b = 0; b < batch; ++b)
            launch_patchify(latents + (size_t)b * d->ch * h * w, d->ch, h, w, p, tok.as<float>() + (size_t)b * n_img * pv, s);
        launch_sgemm_nt_bias(tok.as<float>(), d->x_emb_w, d->x_emb_b, img.as<float>(), batch * n_img, hs, pv, s);
        c->launches += batch + 1;
    }
    // rope tables for this geometry
    std::ostringstream key;
    key << batch << ":" << h << ":" << w << ":" << nseq << ":" << cap_ns[0] << ":" << (nseq > 1 ? cap_ns[1] : 0);
    std::vector<int> segs_img(batch, n_img), segs_joint;
    int n_joint = 0;
    for (int b = 0; b < batch; ++b)
        for (int q = 0; q < nseq; ++q) { segs_joint.push_back(cap_ns[q] + n_img); n_joint += cap_ns[q] + n_img; }
    const int rs = nseq > 1 ? 1 : 0;
    DevBuf &rope_img = d->rope_img[rs], &rope_joint = d->rope_joint[rs];
    if (d->rope_key[rs] != key.str()) {
        std::vector<int> ids_img, ids_joint;
        // refiner image ids: axis 0 is 0 in the pair path and cap_n in the single path
        // (crates/cortiq-engine/src/dit.rs:1287-1292 vs :1431-1435)
        const int a0 = nseq > 1 ? 0 : cap_ns[0];
        for (int b = 0; b < batch; ++b)
            for (int i = 0; i < n_img; ++i) push_ids(&ids_img, a0, i / wp, i % wp);
        for (int b = 0; b < batch; ++b)
            for (int q = 0; q < nseq; ++q) {
                for (int i = 0; i < cap_ns[q]; ++i) push_ids(&ids_joint, i, 0, 0);
                for (int i = 0; i < n_img; ++i) push_ids(&ids_joint, cap_ns[q], i / wp, i % wp);
            }
        d->rope_key[rs].clear();
        d->rope_epoch++;
        CMFC_TRY(upload_rope(c, &rope_img, ids_img, d->axes));
        CMFC_TRY(upload_rope(c, &rope_joint, ids_joint, d->axes));
        d->rope_key[rs] = key.str();
    }
    // When every sequence of the batch has the same token count the GEMMs see a stack of equal periods
    // and may plan their K split per sequence (a prompt's result must not depend on its batch).
    struct PeriodGuard {
        Context* c;
        PeriodGuard(Context* c_, int tokens) : c(c_) { c->gemm_period_tokens = tokens; }
        ~PeriodGuard() { c->gemm_period_tokens = 0; }
    };
    size_t mk = 0;
    PeriodGuard img_period(c, n_img);
    for (size_t l = 0; l < d->noise_ref.size(); ++l, ++mk) {
        const DitBlock* nx = l + 1 < d->noise_ref.size() ? &d->noise_ref[l + 1] : nullptr;
        CMFC_TRY(run_block(c, d, d->noise_ref[l], img.as<float>(), batch * n_img, segs_img, mods + mk * 4 * hs, rope_img,
                           (size_t)batch * n_img, nx, mods + (mk + 1) * 4 * hs, l > 0));
    }
    // ---- joint sequences: [cap | img] per (prompt, branch) ----
    CMFC_TRY(xb.ensure((size_t)n_joint * hs * 4));
    {
        size_t row = 0;
        for (int b = 0; b < batch; ++b)
            for (int q = 0; q < nseq; ++q) {
                CMFC_CUDA(cudaMemcpyAsync(xb.as<float>() + row * hs, caps[q] + (size_t)b * cap_ns[q] * hs, (size_t)cap_ns[q] * hs * 4,
                                          cudaMemcpyDeviceToDevice, s));
                row += cap_ns[q];
                CMFC_CUDA(cudaMemcpyAsync(xb.as<float>() + row * hs, img.as<float>() + (size_t)b * n_img * hs, (size_t)n_img * hs * 4,
                                          cudaMemcpyDeviceToDevice, s));
                row += n_img;
            }
    }
    // the period is one SEQUENCE when all sequences have the same length (any launch, whole batch or
    // half of it, is then a stack of whole periods); with cond and uncond captions of different
    // lengths there is no common period and the GEMMs are not split
    bool equal_seqs = true;
    for (int sl : segs_joint) equal_seqs = equal_seqs && sl == segs_joint[0];
    PeriodGuard joint_period(c, equal_seqs ? segs_joint[0] : 0);
    // Sequences never see each other (attention is per segment, everything else per token), so the
    // batch is cut into two halves that walk the joint layers side by side on two streams: while a
    // persistent GEMM of one half drains its last, partly empty wave of tiles, the other half's next
    // kernel takes the free SMs, and a launch gap of one chain is covered by the other.  Results do not
    // depend on the cut (every kernel's arithmetic is per token or per segment).  CMFC_STREAMS=1 keeps
    // one chain; the stage profiler (one span per launch group) and the per-layer taps need it too.
    const char* streams_env = getenv("CMFC_STREAMS");  // read per call
    const bool two_lanes = segs_joint.size() >= 2 && !c->prof.on && !taps && !(streams_env && atoi(streams_env) == 1);
    if (two_lanes) {
        size_t cut = 1;
        int rows0 = segs_joint[0];
        while (cut + 1 < segs_joint.size() && 2 * (rows0 + segs_joint[cut]) <= n_joint) rows0 += segs_joint[cut++];
        const std::vector<int> segs0(segs_joint.begin(), segs_joint.begin() + cut), segs1(segs_joint.begin() + cut, segs_joint.end());
        const int rows1 = n_joint - rows0;
        CMFC_CUDA(cudaEventRecord(c->ev_fork, s));
        CMFC_CUDA(cudaStreamWaitEvent(c->side_stream, c->ev_fork, 0));
        int rc = OK;
        for (size_t l = 0; l < d->layers.size() && rc == OK; ++l, ++mk) {
            const DitBlock* nx = l + 1 < d->layers.size() ? &d->layers[l + 1] : nullptr;
            rc = run_block(c, d, d->layers[l], xb.as<float>(), rows0, segs0, mods + mk * 4 * hs, rope_joint, (size_t)n_joint, nx,
                           mods + (mk + 1) * 4 * hs, l > 0, 0);
            if (rc != OK) break;
            Lane side(c);
            rc = run_block(c, d, d->layers[l], xb.as<float>() + (size_t)rows0 * hs, rows1, segs1, mods + mk * 4 * hs, rope_joint,
                           (size_t)n_joint, nx, mods + (mk + 1) * 4 * hs, l > 0, (size_t)rows0);
        }
        // the side chain always rejoins, also after an error: a capture must not end with a forked stream
        cudaEventRecord(c->ev_join, c->side_stream);
        cudaStreamWaitEvent(s, c->ev_join, 0);
        CMFC_TRY(rc);
    } else {
        for (size_t l = 0; l < d->layers.size(); ++l) {
            const DitBlock* nx = l + 1 < d->layers.size() ? &d->layers[l + 1] : nullptr;
            CMFC_TRY(run_block(c, d, d->layers[l], xb.as<float>(), n_joint, segs_joint, mods + mk * 4 * hs, rope_joint, (size_t)n_joint,
                               nx, mods + (mk + 1) * 4 * hs, l > 0));
            ++mk;
            if (taps) CMFC_CUDA(cudaMemcpyAsync(taps + l * (size_t)n_joint * hs, xb.p, (size_t)n_joint * hs * 4, cudaMemcpyDeviceToDevice, s));
        }
    }
    // ---- tail: LayerNorm * (1 + scale), project, unpatchify the image tokens ----
    {
        SpanGuard g(c, "head-tail");
        CMFC_TRY(xn.ensure((size_t)n_joint * hs * 4));
        CMFC_TRY(outb.ensure((size_t)n_joint * pv * 4));
        launch_layernorm_scale(xb.as<float>(), out_scale, n_joint, hs, xn.as<float>(), s);
        launch_sgemm_nt_bias(xn.as<float>(), d->out2_w, d->out2_b, outb.as<float>(), n_joint, pv, hs, s);
        c->launches += 2;
        size_t row = 0;
        for (int b = 0; b < batch; ++b)
            for (int q = 0; q < nseq; ++q) {
                row += cap_ns[q];
                launch_unpatchify(outb.as<float>() + row * pv, d->ch, h, w, p, preds[q] + (size_t)b * d->ch * h * w, s);
                c->launches++;
                row += n_img;
            }
    }
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace

extern "C" int cmfc_nextdit_create(cmfc_model* mm, cmfc_nextdit** out) {
    NEED(mm && out, "nextdit_create: null argument");
    NEED_CTX();
    Model* m = mm->m;
    const int64_t ci = find_idx(m, "dit.config_json");
    if (ci < 0) return fail(ERR_NOT_FOUND, "container has no dit.config_json");
    const std::string js(reinterpret_cast<const char*>(m->bytes(ci)), m->recs[ci].nbytes);
    std::unique_ptr<cmfc_nextdit> d(new cmfc_nextdit());
    d->m = m;
    double v;
    if (!json_num(js, "hidden_size", &v)) return fail(ERR_FORMAT, "dit.config_json: hidden_size missing");
    d->hidden = (int)v;
    if (!json_num(js, "num_layers", &v)) return fail(ERR_FORMAT, "dit.config_json: num_layers missing");
    d->nl = (int)v;
    d->nr = json_num(js, "num_refiner_layers", &v) ? (int)v : 2;
    if (!json_num(js, "num_attention_heads", &v)) return fail(ERR_FORMAT, "dit.config_json: num_attention_heads missing");
    d->nh = (int)v;
    d->nkv = json_num(js, "num_kv_heads", &v) ? (int)v : d->nh;
    if (!json_num(js, "in_channels", &v)) return fail(ERR_FORMAT, "dit.config_json: in_channels missing");
    d->ch = (int)v;
    d->patch = json_num(js, "patch_size", &v) ? (int)v : 2;
    d->eps = json_num(js, "norm_eps", &v) ? v : 1e-5;
    if (!json_arr3(js, "axes_dim_rope", d->axes)) return fail(ERR_FORMAT, "dit.config_json: axes_dim_rope missing");
    d->hd = d->hidden / d->nh;
    if (d->axes[0] + d->axes[1] + d->axes[2] != d->hd) return fail(ERR_UNSUPPORTED, "axes_dim_rope must sum to the head dimension");
    for (int l = 0; l < d->nr; ++l) {
        d->ctx_ref.emplace_back();
        CMFC_TRY(load_block(c, d.get(), "dit.context_refiner." + std::to_string(l), false, &d->ctx_ref.back()));
    }
    for (int l = 0; l < d->nr; ++l) {
        d->noise_ref.emplace_back();
        CMFC_TRY(load_block(c, d.get(), "dit.noise_refiner." + std::to_string(l), true, &d->noise_ref.back()));
    }
    for (int l = 0; l < d->nl; ++l) {
        d->layers.emplace_back();
        CMFC_TRY(load_block(c, d.get(), "dit.layers." + std::to_string(l), true, &d->layers.back()));
    }
    d->inter = d->layers.empty() ? 0 : d->layers[0].bw.w2->cols;
    int r = 0, cc = 0;
    const std::string tp = "dit.time_caption_embed.";
    CMFC_TRY(dense_f32(c, m, "dit.x_embedder.weight", &d->x_emb_w));
    CMFC_TRY(dense_f32(c, m, "dit.x_embedder.bias", &d->x_emb_b));
    CMFC_TRY(dense_f32(c, m, tp + "timestep_embedder.linear_1.weight", &d->t1w, &r, &cc));
    d->temb = r;
    if (cc != 256) return fail(ERR_SHAPE, "timestep embedder expects 256 sinusoidal features");
    CMFC_TRY(dense_f32(c, m, tp + "timestep_embedder.linear_1.bias", &d->t1b));
    CMFC_TRY(dense_f32(c, m, tp + "timestep_embedder.linear_2.weight", &d->t2w));
    CMFC_TRY(dense_f32(c, m, tp + "timestep_embedder.linear_2.bias", &d->t2b));
    CMFC_TRY(dense_f32(c, m, tp + "caption_embedder.0.weight", &d->cap_norm, &r, &cc));
    d->cap_feat = r * cc;
    CMFC_TRY(dense_f32(c, m, tp + "caption_embedder.1.bias", &d->cap_b));
    const int64_t cw = find_idx(m, tp + "caption_embedder.1.weight");
    if (cw < 0) return fail(ERR_NOT_FOUND, "missing caption embedder weight");
    if (m->recs[cw].dtype == DT_F32 || m->recs[cw].dtype == DT_F16) CMFC_TRY(upload_f32(c, m, cw, &d->cap_w));
    else CMFC_TRY(get_weight(c, m, cw, &d->cap_w));
    CMFC_TRY(dense_f32(c, m, "dit.norm_out.linear_1.weight", &d->out1_w));
    CMFC_TRY(dense_f32(c, m, "dit.norm_out.linear_1.bias", &d->out1_b));
    CMFC_TRY(dense_f32(c, m, "dit.norm_out.linear_2.weight", &d->out2_w));
    CMFC_TRY(dense_f32(c, m, "dit.norm_out.linear_2.bias", &d->out2_b));
    if (d->temb % 16) return fail(ERR_SHAPE, "time embedding width must be a multiple of 16");
    *out = d.release();
    return OK;
}

extern "C" void cmfc_nextdit_destroy(cmfc_nextdit* d) {
    if (!d) return;
    for (auto& g : d->graphs) g.drop();
    for (DevBuf* b : {&d->rope_joint[0], &d->rope_joint[1], &d->rope_img[0], &d->rope_img[1], &d->rope_cap, &d->latents, &d->cap_c_r,
                      &d->cap_u_r, &d->pred_c, &d->pred_u})
        b->release();
    delete d;
}

extern "C" int cmfc_nextdit_dims(const cmfc_nextdit* d, uint32_t dims[8]) {
    NEED(d && dims, "nextdit_dims: null argument");
    const uint32_t v[8] = {(uint32_t)d->hidden, (uint32_t)d->cap_feat, (uint32_t)d->ch, (uint32_t)d->patch,
                           (uint32_t)d->nl, (uint32_t)d->nr, (uint32_t)d->nh, (uint32_t)d->nkv};
    memcpy(dims, v, sizeof(v));
    return OK;
}

extern "C" int cmfc_nextdit_refine_caption(cmfc_nextdit* d, const float* cap, size_t cap_n, float* out) {
    NEED(d && cap && out && cap_n > 0, "refine_caption: null argument or empty caption");
    NEED_CTX();
    DevBuf &in = c->buf("rc_in"), &o = c->buf("rc_out");
    CMFC_TRY(in.ensure(cap_n * d->cap_feat * 4));
    CMFC_TRY(o.ensure(cap_n * d->hidden * 4));
    CMFC_CUDA(cudaMemcpyAsync(in.p, cap, cap_n * d->cap_feat * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_TRY(refine_caps(c, d, in.as<float>(), {(int)cap_n}, o.as<float>()));
    CMFC_CUDA(cudaMemcpyAsync(out, o.p, cap_n * d->hidden * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "refine_caption");
}

static int forward_host(cmfc_nextdit* d, const float* latent, size_t h, size_t w, const float* cap_c, size_t cap_c_n,
                        const float* cap_u, size_t cap_u_n, float t, float* pred_c, float* pred_u, float* taps) {
    NEED(d && latent && cap_c && pred_c && cap_c_n > 0 && h > 0 && w > 0, "forward: null argument or empty input");
    NEED_CTX();
    const int nseq = cap_u ? 2 : 1;
    NEED(nseq == 1 || (pred_u && cap_u_n > 0), "forward_pair: uncond outputs missing");
    const size_t lat_n = (size_t)d->ch * h * w, hs = d->hidden;
    const size_t n_img = (h / d->patch) * (w / d->patch);
    const size_t n_joint = cap_c_n + n_img + (nseq > 1 ? cap_u_n + n_img : 0);
    DevBuf &lat = c->buf("fh_lat"), &cc = c->buf("fh_capc"), &cu = c->buf("fh_capu"), &pc = c->buf("fh_pc"), &pu = c->buf("fh_pu"),
           &tp = c->buf("fh_taps");
    CMFC_TRY(lat.ensure(lat_n * 4));
    CMFC_TRY(cc.ensure(cap_c_n * hs * 4));
    CMFC_TRY(pc.ensure(lat_n * 4));
    CMFC_CUDA(cudaMemcpyAsync(lat.p, latent, lat_n * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(cc.p, cap_c, cap_c_n * hs * 4, cudaMemcpyHostToDevice, c->stream));
    if (nseq > 1) {
        CMFC_TRY(cu.ensure(cap_u_n * hs * 4));
        CMFC_TRY(pu.ensure(lat_n * 4));
        CMFC_CUDA(cudaMemcpyAsync(cu.p, cap_u, cap_u_n * hs * 4, cudaMemcpyHostToDevice, c->stream));
    }
    if (taps) CMFC_TRY(tp.ensure((size_t)d->nl * n_joint * hs * 4));
    const float* caps[2] = {cc.as<float>(), cu.as<float>()};
    const int cap_ns[2] = {(int)cap_c_n, (int)cap_u_n};
    float* preds[2] = {pc.as<float>(), pu.as<float>()};
    CMFC_TRY(upload_schedule(c, {t, 0.0f}, 0));
    CMFC_TRY(forward_device(c, d, lat.as<float>(), 1, (int)h, (int)w, nseq, caps, cap_ns, t, preds, taps ? tp.as<float>() : nullptr));
    CMFC_CUDA(cudaMemcpyAsync(pred_c, pc.p, lat_n * 4, cudaMemcpyDeviceToHost, c->stream));
    if (nseq > 1) CMFC_CUDA(cudaMemcpyAsync(pred_u, pu.p, lat_n * 4, cudaMemcpyDeviceToHost, c->stream));
    if (taps) CMFC_CUDA(cudaMemcpyAsync(taps, tp.p, (size_t)d->nl * n_joint * hs * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "forward");
}

extern "C" int cmfc_nextdit_forward(cmfc_nextdit* d, const float* latent, size_t h, size_t w, const float* cap_e, size_t cap_n,
                                    float t, float* pred) {
    return forward_host(d, latent, h, w, cap_e, cap_n, nullptr, 0, t, pred, nullptr, nullptr);
}
extern "C" int cmfc_nextdit_forward_pair(cmfc_nextdit* d, const float* latent, size_t h, size_t w, const float* cap_c,
                                         size_t cap_c_n, const float* cap_u, size_t cap_u_n, float t, float* pred_c, float* pred_u) {
    NEED(cap_u, "forward_pair: cap_u is null");
    return forward_host(d, latent, h, w, cap_c, cap_c_n, cap_u, cap_u_n, t, pred_c, pred_u, nullptr);
}
extern "C" int cmfc_nextdit_forward_pair_taps(cmfc_nextdit* d, const float* latent, size_t h, size_t w, const float* cap_c,
                                              size_t cap_c_n, const float* cap_u, size_t cap_u_n, float t, float* pred_c,
                                              float* pred_u, float* taps) {
    NEED(cap_u && taps, "forward_pair_taps: null argument");
    return forward_host(d, latent, h, w, cap_c, cap_c_n, cap_u, cap_u_n, t, pred_c, pred_u, taps);
}

// ---------------- Euler loop ----------------
extern "C" int cmfc_denoise_begin_ex(cmfc_nextdit* d, const float* latents, size_t batch, size_t h, size_t w, const float* cap,
                                     size_t cap_n, const float* cap_u, size_t cap_u_n, const cmfc_gen_params* gp) {
    NEED(d && latents && cap && gp && batch > 0 && cap_n > 0 && gp->steps > 0, "denoise: null argument or empty input");
    NEED(gp->cfg_trunc_ratio == gp->cfg_trunc_ratio, "denoise: cfg_trunc_ratio is NaN");
    NEED_CTX();
    const uint32_t steps = gp->steps;
    const float guidance_scale = gp->guidance_scale;
    const size_t lat_n = batch * d->ch * h * w, hs = d->hidden, cf = d->cap_feat;
    d->batch = batch; d->lh = h; d->lw = w; d->cap_n = cap_n; d->cap_u_n = cap_u ? cap_u_n : 0; d->steps = steps;
    d->gs = guidance_scale;
    d->cfg = cap_u != nullptr;
    d->cfg_norm = gp->cfg_normalization != 0;
    NEED(!d->cfg || cap_u_n > 0, "denoise: empty uncond caption");
    // CFG truncation (crates/cortiq-engine/src/imagegen.rs:164): step i is guided while
    // (i + 1) / steps <= cfg_trunc_ratio, evaluated in f32 like the engine; past it only cond runs
    d->cfg_steps = 0;
    if (d->cfg)
        for (uint32_t i = 0; i < steps; ++i)
            if ((float)(i + 1) / (float)steps <= gp->cfg_trunc_ratio) d->cfg_steps = i + 1;
    // sigma schedule (crates/cortiq-engine/src/imagegen.rs:59-73), shift 6
    d->sig.clear();
    for (uint32_t i = 0; i < steps; ++i) {
        const double sv = steps == 1 ? 1.0 : 1.0 - (double)i * (1.0 - 1.0 / (double)steps) / (double)(steps - 1);
        d->sig.push_back(6.0 * sv / (1.0 + 5.0 * sv));
    }
    d->sig.push_back(0.0);
    CMFC_TRY(d->latents.ensure(lat_n * 4));
    CMFC_TRY(d->pred_c.ensure(lat_n * 4));
    CMFC_TRY(d->cap_c_r.ensure(batch * cap_n * hs * 4));
    CMFC_CUDA(cudaMemcpyAsync(d->latents.p, latents, lat_n * 4, cudaMemcpyHostToDevice, c->stream));
    DevBuf& raw = c->buf("dn_cap_raw");
    CMFC_TRY(raw.ensure(batch * (cap_n + d->cap_u_n) * cf * 4));
    CMFC_CUDA(cudaMemcpyAsync(raw.p, cap, batch * cap_n * cf * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_TRY(refine_caps(c, d, raw.as<float>(), std::vector<int>(batch, (int)cap_n), d->cap_c_r.as<float>()));
    if (d->cfg) {
        CMFC_TRY(d->pred_u.ensure(lat_n * 4));
        CMFC_TRY(d->cap_u_r.ensure(batch * cap_u_n * hs * 4));
        float* raw_u = raw.as<float>() + batch * cap_n * cf;
        CMFC_CUDA(cudaMemcpyAsync(raw_u, cap_u, batch * cap_u_n * cf * 4, cudaMemcpyHostToDevice, c->stream));
        CMFC_TRY(refine_caps(c, d, raw_u, std::vector<int>(batch, (int)cap_u_n), d->cap_u_r.as<float>()));
    }
    // timesteps t_i = 1 - sigma_i and step sizes d_i = sigma_{i+1} - sigma_i live on the device
    std::vector<float> td(2 * steps);
    for (uint32_t i = 0; i < steps; ++i) {
        td[2 * i] = (float)(1.0 - d->sig[i]);
        td[2 * i + 1] = (float)(d->sig[i + 1] - d->sig[i]);
    }
    CMFC_TRY(upload_schedule(c, td, 0));
    d->next_step = 0;
    std::ostringstream key;
    key << batch << ":" << h << ":" << w << ":" << cap_n << ":" << d->cap_u_n << ":" << guidance_scale << ":" << (int)d->cfg_norm;
    for (auto& g : d->graphs) {
        g.eager_steps = 0;
        if (key.str() != d->graph_key) g.drop();
    }
    d->graph_key = key.str();
    return OK;
}

extern "C" int cmfc_denoise_begin(cmfc_nextdit* d, const float* latents, size_t batch, size_t h, size_t w, const float* cap,
                                  size_t cap_n, const float* cap_u, size_t cap_u_n, uint32_t steps, float guidance_scale) {
    const cmfc_gen_params gp = {steps, guidance_scale, 1.0f, 1};
    return cmfc_denoise_begin_ex(d, latents, batch, h, w, cap, cap_n, cap_u, cap_u_n, &gp);
}

namespace {
// every launch of one denoise step, in stream order
int enqueue_step(Context* c, cmfc_nextdit* d, bool guided) {
    const float* caps[2] = {d->cap_c_r.as<float>(), d->cap_u_r.as<float>()};
    const int cap_ns[2] = {(int)d->cap_n, (int)d->cap_u_n};
    float* preds[2] = {d->pred_c.as<float>(), d->pred_u.as<float>()};
    CMFC_TRY(forward_device(c, d, d->latents.as<float>(), (int)d->batch, (int)d->lh, (int)d->lw, guided ? 2 : 1, caps, cap_ns, 0.0f, preds, nullptr));
    launch_cfg_euler(d->latents.as<float>(), d->pred_c.as<float>(), d->pred_u.as<float>(), d->gs, c->sched, c->step_counter,
                     (int)(d->batch * d->ch * d->lh), (int)d->lw, guided ? (d->cfg_norm ? 1 : 2) : 0, c->stream);
    launch_advance_step(c->step_counter, c->stream);
    c->launches += 2;
    CMFC_CUDA(cudaGetLastError());
    return OK;
}
}  // namespace

extern "C" int cmfc_denoise_step(cmfc_nextdit* d, uint32_t i) {
    NEED(d && d->batch > 0 && i < d->steps, "denoise_step: no loop in progress or step out of range");
    NEED_CTX();
    if (i != d->next_step) {  // out-of-order step: move the device counter
        CMFC_CUDA(cudaStreamSynchronize(c->stream));
        reinterpret_cast<int*>(c->sched_host)[2 * Context::MAX_STEPS] = (int)i;
        CMFC_CUDA(cudaMemcpyAsync(c->step_counter, c->sched_host + 2 * Context::MAX_STEPS, 4, cudaMemcpyHostToDevice, c->stream));
    }
    d->next_step = i + 1;
    // The step's launches (about 470 for the 30-block pair forward) are captured once into a CUDA
    // graph and replayed: the timestep and step size come from the device-resident schedule, so
    // nothing in the graph depends on i.  Guided and cond-only steps (CFG truncation) are different
    // graphs.  The first step of a kind after begin runs eagerly (it may grow workspaces and upload
    // tables); profiling spans need eager launches too.
    const bool guided = d->cfg && i < d->cfg_steps;
    cmfc_nextdit::StepGraph& sg = d->graphs[guided ? 1 : 0];
    const char* graph_env = getenv("CMFC_GRAPH");  // read per call, like the other switches
    const bool graphs_on = !(graph_env && atoi(graph_env) == 0);
    if (sg.exec && (sg.alloc_epoch != alloc_epoch() || sg.rope_epoch != d->rope_epoch)) sg.drop();
    if (graphs_on && !c->prof.on && sg.exec) {
        CMFC_CUDA(cudaGraphLaunch(sg.exec, c->stream));
        c->launches += sg.launches;
        return OK;
    }
    if (graphs_on && !c->prof.on && sg.eager_steps >= 1) {
        const uint64_t before = c->launches, epoch = alloc_epoch(), repoch = d->rope_epoch;
        cudaGraph_t g = nullptr;
        CMFC_CUDA(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
        const int rc = enqueue_step(c, d, guided);
        const cudaError_t ce = cudaStreamEndCapture(c->stream, &g);
        if (rc == OK && ce == cudaSuccess && g && epoch == alloc_epoch() && repoch == d->rope_epoch &&
            cudaGraphInstantiate(&sg.exec, g, 0) == cudaSuccess) {
            sg.launches = c->launches - before;
            c->launches = before;
            sg.alloc_epoch = epoch;
            sg.rope_epoch = repoch;
            cudaGraphDestroy(g);
            CMFC_CUDA(cudaGraphLaunch(sg.exec, c->stream));
            c->launches += sg.launches;
            return OK;
        }
        // capture did not work out (e.g. a workspace had to grow): nothing ran; fall through to eager
        if (g) cudaGraphDestroy(g);
        sg.exec = nullptr;
        c->launches = before;
        cudaGetLastError();
        if (rc != OK) return rc;
    }
    sg.eager_steps++;
    return enqueue_step(c, d, guided);
}

extern "C" int cmfc_denoise_end(cmfc_nextdit* d, float* latents) {
    NEED(d && latents && d->batch > 0, "denoise_end: null argument or no loop in progress");
    NEED_CTX();
    CMFC_CUDA(cudaMemcpyAsync(latents, d->latents.p, d->batch * d->ch * d->lh * d->lw * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "denoise");
}

extern "C" int cmfc_denoise_ex(cmfc_nextdit* d, float* latents, size_t batch, size_t h, size_t w, const float* cap, size_t cap_n,
                               const float* cap_u, size_t cap_u_n, const cmfc_gen_params* gp) {
    CMFC_TRY(cmfc_denoise_begin_ex(d, latents, batch, h, w, cap, cap_n, cap_u, cap_u_n, gp));
    for (uint32_t i = 0; i < gp->steps; ++i) CMFC_TRY(cmfc_denoise_step(d, i));
    return cmfc_denoise_end(d, latents);
}

extern "C" int cmfc_denoise(cmfc_nextdit* d, float* latents, size_t batch, size_t h, size_t w, const float* cap, size_t cap_n,
                            const float* cap_u, size_t cap_u_n, uint32_t steps, float guidance_scale) {
    const cmfc_gen_params gp = {steps, guidance_scale, 1.0f, 1};
    return cmfc_denoise_ex(d, latents, batch, h, w, cap, cap_n, cap_u, cap_u_n, &gp);
}

// ---------------- quantizers ----------------
extern "C" size_t cmfc_payload_nbytes(int dtype, size_t rows, size_t cols) { return payload_nbytes(dtype, rows, cols); }

static int encode_device(Context* c, int dtype, const float* d_w, size_t rows, size_t cols, uint8_t* d_payload) {
    if (dtype == DT_Q8) launch_encode_q8_row(d_w, (int)rows, (int)cols, d_payload, c->stream);
    else if (dtype == DT_Q4T) launch_encode_q4_tiled(d_w, (int)rows, (int)cols, d_payload, c->stream);
    else if (dtype == DT_Q4TP) launch_encode_q4tp(d_w, (int)rows, (int)cols, d_payload, c->log2_lut, c->exp2_lut, c->stream);
    else return fail(ERR_UNSUPPORTED, "encode: dtype must be q8_row, q4_tiled or q4tp");
    c->launches++;
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

extern "C" int cmfc_encode(int dtype, const float* w, size_t rows, size_t cols, uint8_t* payload) {
    NEED(w && payload && rows > 0 && cols > 0, "encode: null argument or empty tensor");
    NEED(dtype == DT_Q8 || cols % 32 == 0, "encode: 4-bit codecs need cols % 32 == 0");
    NEED_CTX();
    const size_t nb = payload_nbytes(dtype, rows, cols);
    if (!nb) return fail(ERR_UNSUPPORTED, "encode: unsupported dtype");
    DevBuf &dw = c->buf("enc_w"), &dp = c->buf("enc_p");
    CMFC_TRY(dw.ensure(rows * cols * 4));
    CMFC_TRY(dp.ensure(nb));
    CMFC_CUDA(cudaMemcpyAsync(dw.p, w, rows * cols * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_TRY(encode_device(c, dtype, dw.as<float>(), rows, cols, dp.as<uint8_t>()));
    CMFC_CUDA(cudaMemcpyAsync(payload, dp.p, nb, cudaMemcpyDeviceToHost, c->stream));
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    return OK;
}

extern "C" int cmfc_encode_random(int dtype, uint64_t seed, float std, size_t rows, size_t cols, uint8_t* payload) {
    NEED(payload && rows > 0 && cols > 0, "encode_random: null argument or empty tensor");
    NEED(dtype == DT_Q8 || dtype == DT_F32 || cols % 32 == 0, "encode_random: 4-bit codecs need cols % 32 == 0");
    NEED_CTX();
    const size_t nb = payload_nbytes(dtype, rows, cols);
    if (!nb) return fail(ERR_UNSUPPORTED, "encode_random: unsupported dtype");
    DevBuf &dw = c->buf("enc_w"), &dp = c->buf("enc_p");
    CMFC_TRY(dw.ensure(rows * cols * 4));
    launch_fill_normal(dw.as<float>(), rows * cols, seed, std, c->stream);
    c->launches++;
    if (dtype == DT_F32) {
        CMFC_CUDA(cudaMemcpyAsync(payload, dw.p, nb, cudaMemcpyDeviceToHost, c->stream));
    } else {
        CMFC_TRY(dp.ensure(nb));
        CMFC_TRY(encode_device(c, dtype, dw.as<float>(), rows, cols, dp.as<uint8_t>()));
        CMFC_CUDA(cudaMemcpyAsync(payload, dp.p, nb, cudaMemcpyDeviceToHost, c->stream));
    }
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    return OK;
}

// ---------------- instrumentation ----------------
extern "C" uint64_t cmfc_launch_count(int reset) {
    Context* c = ctx();
    if (!c) return 0;
    uint64_t v = c->launches;
    if (reset) c->launches = 0;
    return v;
}

extern "C" int cmfc_bench_gemm(cmfc_model* m, int64_t idx, size_t M, int mode, int iters, float* ms_per_launch) {
    NEED(m && ms_per_launch && M > 0 && iters > 0, "bench_gemm: bad argument");
    NEED(mode >= GEMM_OUT_F32 && mode <= GEMM_OUT_SWIGLU, "bench_gemm: mode must be 0 (f32), 1 (bf16) or 2 (SwiGLU pairs)");
    NEED_CTX();
    DevWeight* w = nullptr;
    CMFC_TRY(get_weight(c, m->m, idx, &w));
    DevBuf &xf = c->buf("bg_xf"), &xb = c->buf("bg_xb"), &y = c->buf("bg_y");
    CMFC_TRY(xf.ensure(M * w->cols * 4));
    CMFC_TRY(xb.ensure(M * w->cols * 2));
    CMFC_TRY(y.ensure(M * w->rows * 4));
    launch_fill_normal(xf.as<float>(), M * w->cols, 1234, 1.0f, c->stream);
    launch_f32_to_bf16(xf.as<float>(), xb.as<__nv_bfloat16>(), M * w->cols, c->stream);
    c->launches += 2;
    const int ldo = mode == GEMM_OUT_SWIGLU ? w->rows / 2 : w->rows;
    for (int i = 0; i < 3; ++i) CMFC_TRY(dev_gemm(c, w, xb.as<__nv_bfloat16>(), (int)M, y.p, ldo, mode));
    cudaEvent_t e0, e1;
    CMFC_CUDA(cudaEventCreate(&e0));
    CMFC_CUDA(cudaEventCreate(&e1));
    CMFC_CUDA(cudaEventRecord(e0, c->stream));
    for (int i = 0; i < iters; ++i) CMFC_TRY(dev_gemm(c, w, xb.as<__nv_bfloat16>(), (int)M, y.p, ldo, mode));
    CMFC_CUDA(cudaEventRecord(e1, c->stream));
    CMFC_CUDA(cudaEventSynchronize(e1));
    float ms = 0;
    CMFC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms_per_launch = ms / iters;
    return check_status(c, "bench_gemm");
}

extern "C" int cmfc_bench_attention(size_t nh, size_t nkv, size_t hd, size_t n, size_t nseg, int iters, float* ms_per_launch) {
    NEED(ms_per_launch && nh && nkv && n && nseg && iters > 0, "bench_attention: bad argument");
    NEED_CTX();
    std::vector<int> segs(nseg, (int)n);
    SegTable st;
    CMFC_TRY(prepare_segs(c, segs, &st));
    const size_t tot = n * nseg, qn = tot * nh * hd, kn = tot * nkv * hd, vn = (size_t)nkv * hd * st.vt_pitch;
    DevBuf &f = c->buf("ba_f"), &q = c->buf("ba_q"), &k = c->buf("ba_k"), &v = c->buf("ba_v"), &o = c->buf("ba_o");
    CMFC_TRY(f.ensure((qn > vn ? qn : vn) * 4));
    CMFC_TRY(q.ensure(qn * 2));
    CMFC_TRY(k.ensure(kn * 2));
    CMFC_TRY(v.ensure(vn * 2));
    CMFC_TRY(o.ensure(qn * 2));
    launch_fill_normal(f.as<float>(), qn, 11, 1.0f, c->stream);
    launch_f32_to_bf16(f.as<float>(), q.as<__nv_bfloat16>(), qn, c->stream);
    launch_fill_normal(f.as<float>(), kn, 12, 1.0f, c->stream);
    launch_f32_to_bf16(f.as<float>(), k.as<__nv_bfloat16>(), kn, c->stream);
    launch_fill_normal(f.as<float>(), vn, 13, 1.0f, c->stream);
    launch_f32_to_bf16(f.as<float>(), v.as<__nv_bfloat16>(), vn, c->stream);
    c->launches += 6;
    const float scale = 1.0f / sqrtf((float)hd);
    float score_ref = 0.0f;  // the form a NextDiT block launches: the reference known in advance
    CMFC_TRY(attention_score_ref(c, q.as<__nv_bfloat16>(), k.as<__nv_bfloat16>(), tot, (int)nh, (int)nkv, (int)hd, scale, &score_ref));
    if (score_ref > 0.0f) {  // same queries, multiplied by scale * log2(e)
        launch_fill_normal(f.as<float>(), qn, 11, scale * 1.4426950408889634f, c->stream);
        launch_f32_to_bf16(f.as<float>(), q.as<__nv_bfloat16>(), qn, c->stream);
        c->launches += 2;
    }
    for (int i = 0; i < 3; ++i)
        CMFC_TRY(dev_attention(c, q.as<__nv_bfloat16>(), k.as<__nv_bfloat16>(), v.as<__nv_bfloat16>(), st, (int)nh, (int)nkv, (int)hd, scale, o.as<__nv_bfloat16>(), nullptr, score_ref));
    cudaEvent_t e0, e1;
    CMFC_CUDA(cudaEventCreate(&e0));
    CMFC_CUDA(cudaEventCreate(&e1));
    CMFC_CUDA(cudaEventRecord(e0, c->stream));
    for (int i = 0; i < iters; ++i)
        CMFC_TRY(dev_attention(c, q.as<__nv_bfloat16>(), k.as<__nv_bfloat16>(), v.as<__nv_bfloat16>(), st, (int)nh, (int)nkv, (int)hd, scale, o.as<__nv_bfloat16>(), nullptr, score_ref));
    CMFC_CUDA(cudaEventRecord(e1, c->stream));
    CMFC_CUDA(cudaEventSynchronize(e1));
    float ms = 0;
    CMFC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms_per_launch = ms / iters;
    return check_status(c, "bench_attention");
}

// kind: 0 modulated RMSNorm (f32 -> bf16), 1 gated residual, 2 gated residual fused with the next
// modulated norm, 3 qk-norm + RoPE + head packing of Q and K (cols = hidden; nh/nkv/hd as Lumina-2 when hidden = 2304)
extern "C" int cmfc_bench_rowop(int kind, size_t rows, size_t cols, int iters, float* ms_per_launch, double* bytes_per_launch) {
    NEED(ms_per_launch && bytes_per_launch && rows && cols && iters > 0 && kind >= 0 && kind <= 3, "bench_rowop: bad argument");
    NEED_CTX();
    if (!row_cols_supported((int)cols)) return fail(ERR_UNSUPPORTED, "bench_rowop: unsupported row width");
    DevBuf &x = c->buf("br_x"), &src = c->buf("br_src"), &vec = c->buf("br_vec"), &ob = c->buf("br_ob"), &tab = c->buf("br_tab"), &o2 = c->buf("br_o2");
    const int hd = cols % 96 == 0 ? 96 : 64, nh = (int)cols / hd, nkv = nh % 3 == 0 ? nh / 3 : nh;
    const size_t qkvw = (size_t)(nh + 2 * nkv) * hd;
    CMFC_TRY(x.ensure(rows * (kind == 3 ? qkvw : cols) * 4));
    CMFC_TRY(src.ensure(rows * cols * 4));
    CMFC_TRY(vec.ensure(4 * cols * 4));
    CMFC_TRY(ob.ensure(rows * cols * 2));
    launch_fill_normal(x.as<float>(), rows * (kind == 3 ? qkvw : cols), 21, 1.0f, c->stream);
    launch_fill_normal(src.as<float>(), rows * cols, 22, 1.0f, c->stream);
    launch_fill_normal(vec.as<float>(), 4 * cols, 23, 0.1f, c->stream);
    const float* v0 = vec.as<float>();
    if (kind == 3) {
        CMFC_TRY(tab.ensure(rows * hd * 4));
        CMFC_TRY(o2.ensure(rows * nkv * hd * 2));
        CMFC_CUDA(cudaMemsetAsync(tab.p, 0, rows * hd * 4, c->stream));
    }
    auto run = [&]() {
        if (kind == 0) launch_rms_mod(x.as<float>(), v0, v0 + cols, 1e-5, (int)rows, (int)cols, ob.as<__nv_bfloat16>(), nullptr, c->stream);
        else if (kind == 1) launch_gated_residual(x.as<float>(), src.as<float>(), v0, v0 + cols, 1e-5, (int)rows, (int)cols, c->stream);
        else if (kind == 2) launch_residual_then_norm(x.as<float>(), src.as<float>(), v0, v0 + cols, v0 + 2 * cols, v0 + 3 * cols, 1e-5, (int)rows, (int)cols, ob.as<__nv_bfloat16>(), c->stream);
        else launch_qk_rope_pack(x.as<float>(), (int)rows, nh, nkv, hd, v0, v0 + hd, tab.as<float>(), tab.as<float>() + rows * hd / 2, 1.0f, nullptr, ob.as<__nv_bfloat16>(), o2.as<__nv_bfloat16>(), c->stream);
        c->launches++;
    };
    for (int i = 0; i < 3; ++i) run();
    cudaEvent_t e0, e1;
    CMFC_CUDA(cudaEventCreate(&e0));
    CMFC_CUDA(cudaEventCreate(&e1));
    CMFC_CUDA(cudaEventRecord(e0, c->stream));
    for (int i = 0; i < iters; ++i) run();
    CMFC_CUDA(cudaEventRecord(e1, c->stream));
    CMFC_CUDA(cudaEventSynchronize(e1));
    float ms = 0;
    CMFC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms_per_launch = ms / iters;
    const double e = (double)rows * cols;
    // algorithmic bytes: f32 reads/writes 4 B, bf16 writes 2 B per element
    // kind 3: the Q and K columns of the QKV matrix in (f32), Q and K out (bf16), the f32 cos / sin row
    const double qkw = (double)(nh + nkv) * hd;
    *bytes_per_launch = kind == 0 ? e * 6 : kind == 1 ? e * 12 : kind == 2 ? e * 14
                                  : (double)rows * (qkw * 4 + qkw * 2 + (double)(hd / 2) * 8);
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

extern "C" void* cmfc_stream_handle(void) {
    Context* c = ctx();
    return c ? (void*)c->stream : nullptr;
}

extern "C" int cmfc_profile_enable(int on) {
    NEED_CTX();
    for (auto& sp : c->prof.spans) { cudaEventDestroy(sp.second.first); cudaEventDestroy(sp.second.second); }
    c->prof.spans.clear();
    c->prof.on = on != 0;
    return OK;
}
extern "C" int cmfc_profile_read(char* buf, size_t buflen) {
    NEED(buf && buflen > 0, "profile_read: null buffer");
    NEED_CTX();
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    std::map<std::string, std::pair<double, int>> agg;
    for (auto& sp : c->prof.spans) {
        float ms = 0;
        if (cudaEventElapsedTime(&ms, sp.second.first, sp.second.second) == cudaSuccess) {
            agg[sp.first].first += ms;
            agg[sp.first].second++;
        }
        cudaEventDestroy(sp.second.first);
        cudaEventDestroy(sp.second.second);
    }
    c->prof.spans.clear();
    std::ostringstream os;
    os << "{";
    bool first = true;
    for (auto& kv : agg) {
        os << (first ? "" : ", ") << "\"" << kv.first << "\": {\"ms\": " << kv.second.first << ", \"spans\": " << kv.second.second << "}";
        first = false;
    }
    os << "}";
    const std::string s = os.str();
    if (s.size() + 1 > buflen) return fail(ERR_BAD_ARG, "profile_read: buffer too small");
    memcpy(buf, s.c_str(), s.size() + 1);
    return OK;
}
