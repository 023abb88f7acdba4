// Gemma-2 prompt encoder on the device (crates/cortiq-engine/src/textenc.rs): token ids -> the
// residual stream entering every layer and the final-normed hidden states.  Full-sequence causal
// forward, no KV cache: embedding * sqrt(hidden), RMSNorm with (1 + w), sandwich norms around
// attention and the GeGLU MLP, GQA with query_pre_attn_scalar scaling, logit soft-capping, RoPE.
// Projections run through the dequant GEMM (gemm_dequant.cu); the small f32 pieces are in
// gemma_kernels.cu; norms and residuals are the denoiser's row kernels (rowops.cu).
#include <cmath>
#include <cstring>

#include "../../include/cmf_cuda.h"
#include "runtime.h"

using namespace cmfc;

namespace {

#define NEED_CTX()                                                         \
    Context* c = ctx();                                                    \
    if (!c) return last_error().empty() ? fail(ERR_CUDA, "no CUDA device") : ERR_CUDA;
#define NEED(cond, msg) \
    if (!(cond)) return fail(ERR_BAD_ARG, msg)

bool json_number(const std::string& js, const char* key, double* out) {
    const std::string k = std::string("\"") + key + "\"";
    size_t p = js.find(k);
    if (p == std::string::npos) return false;
    p = js.find(':', p + k.size());
    if (p == std::string::npos) return false;
    ++p;
    while (p < js.size() && isspace((unsigned char)js[p])) ++p;
    char* end = nullptr;
    const double v = strtod(js.c_str() + p, &end);
    if (end == js.c_str() + p) return false;
    *out = v;
    return true;
}

int64_t find(Model* m, const std::string& name) {
    auto it = m->by_name.find(name);
    return it == m->by_name.end() ? -1 : it->second;
}

struct GemmaLayer {
    DevWeight *qkv = nullptr, *o = nullptr, *gate_up = nullptr, *down = nullptr;
    float *input_norm = nullptr, *post_attn_norm = nullptr, *pre_ffn_norm = nullptr, *post_ffn_norm = nullptr;  // 1 + w
};

}  // namespace

struct cmfc_gemma {
    Model* m = nullptr;
    int hidden = 0, nl = 0, nh = 0, nkv = 0, hd = 0, inter = 0, vocab = 0, window = 4096;
    float scale = 1.0f, softcap = 0.0f, theta = 10000.0f;
    double eps = 1e-6;
    int64_t embed_idx = -1;
    std::vector<GemmaLayer> layers;
    float* final_norm = nullptr;
    std::vector<void*> owned;
    DevBuf rope;        // cos [n, hd/2] then sin [n, hd/2], f32
    int rope_n = 0;
};

namespace {

// a norm weight vector as the (1 + w) factor the encoder multiplies by (textenc.rs:59-68)
int load_norm_plus_one(Context* c, cmfc_gemma* g, const std::string& name, int expect, float** out) {
    Model* m = g->m;
    const int64_t idx = find(m, name);
    if (idx < 0) return fail(ERR_NOT_FOUND, "missing tensor " + name);
    const TensorRec& t = m->recs[idx];
    size_t n = 1;
    for (int k = 0; k < t.ndim; ++k) n *= t.shape[k];
    if ((int)n != expect) return fail(ERR_SHAPE, "tensor " + name + ": unexpected length");
    std::vector<float> v(n);
    const uint8_t* src = m->bytes(idx);
    if (t.dtype == DT_F32) {
        memcpy(v.data(), src, n * 4);
    } else if (t.dtype == DT_F16) {
        for (size_t i = 0; i < n; ++i) {
            uint16_t h;
            memcpy(&h, src + 2 * i, 2);
            v[i] = half_bits_to_float(h);
        }
    } else {
        return fail(ERR_UNSUPPORTED, "tensor " + name + ": expected f32 or f16");
    }
    for (size_t i = 0; i < n; ++i) {
        volatile float w = 1.0f + v[i];  // the reference's f32 add
        v[i] = w;
    }
    void* d = nullptr;
    if (cudaMalloc(&d, n * 4) != cudaSuccess) return fail(ERR_OOM, "out of device memory for a norm weight");
    g->owned.push_back(d);
    CMFC_CUDA(cudaMemcpy(d, v.data(), n * 4, cudaMemcpyHostToDevice));
    CMFC_CUDA(cudaStreamSynchronize(0));  // readers run on a stream that is not ordered after the legacy one
    *out = reinterpret_cast<float*>(d);
    return OK;
}

int need_idx(Model* m, const std::string& name, int64_t* out) {
    *out = find(m, name);
    if (*out < 0) return fail(ERR_NOT_FOUND, "missing tensor " + name);
    return OK;
}

// cos / sin of position * theta^(-2i/hd) in f32, as textenc.rs:276-277 computes them
int ensure_rope(Context* c, cmfc_gemma* g, int n) {
    if (n <= g->rope_n) return OK;
    const int half = g->hd / 2;
    std::vector<float> tab((size_t)2 * n * half);
    for (int p = 0; p < n; ++p)
        for (int i = 0; i < half; ++i) {
            const float freq = 1.0f / powf(g->theta, 2.0f * (float)i / (float)g->hd);
            const float a = (float)p * freq;
            tab[(size_t)p * half + i] = cosf(a);
            tab[(size_t)n * half + (size_t)p * half + i] = sinf(a);
        }
    CMFC_CUDA(cudaStreamSynchronize(c->stream));  // kernels of an earlier call may still read the old table
    CMFC_TRY(g->rope.ensure(tab.size() * 4));
    CMFC_CUDA(cudaMemcpy(g->rope.p, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice));
    CMFC_CUDA(cudaStreamSynchronize(0));
    g->rope_n = n;
    return OK;
}

// rows ``ids`` of the embedding table, times sqrt(hidden), into h [n, hidden]
int embed_rows(Context* c, cmfc_gemma* g, const uint32_t* ids, int n, float* h) {
    Model* m = g->m;
    const TensorRec& t = m->recs[g->embed_idx];
    const int hs = g->hidden;
    const float emb_scale = sqrtf((float)hs);
    const uint8_t* src = m->bytes(g->embed_idx);
    for (int i = 0; i < n; ++i)
        if (ids[i] >= (uint32_t)g->vocab) return fail(ERR_BAD_ARG, "token id " + std::to_string(ids[i]) + " is outside the vocabulary");
    if (t.dtype == DT_Q8) {
        // q8_row payload: [int8 rows * cols][f16 rows] (crates/cortiq-core/src/quant.rs:18-40)
        std::vector<int8_t> q((size_t)n * hs);
        std::vector<float> sc(n);
        for (int i = 0; i < n; ++i) {
            memcpy(q.data() + (size_t)i * hs, src + (size_t)ids[i] * hs, hs);
            uint16_t hb;
            memcpy(&hb, src + (size_t)g->vocab * hs + 2 * (size_t)ids[i], 2);
            sc[i] = half_bits_to_float(hb);
        }
        DevBuf &bq = c->buf("te.embq"), &bs = c->buf("te.embs");
        CMFC_TRY(bq.ensure(q.size()));
        CMFC_TRY(bs.ensure(sc.size() * 4));
        CMFC_CUDA(cudaMemcpyAsync(bq.p, q.data(), q.size(), cudaMemcpyHostToDevice, c->stream));
        CMFC_CUDA(cudaMemcpyAsync(bs.p, sc.data(), sc.size() * 4, cudaMemcpyHostToDevice, c->stream));
        launch_embed_q8(bq.as<int8_t>(), bs.as<float>(), n, hs, emb_scale, h, c->stream);
        c->launches++;
        CMFC_CUDA(cudaStreamSynchronize(c->stream));  // q and sc are stack-owned
        return OK;
    }
    if (t.dtype == DT_F32 || t.dtype == DT_F16) {
        std::vector<float> rows((size_t)n * hs);
        for (int i = 0; i < n; ++i)
            for (int k = 0; k < hs; ++k) {
                if (t.dtype == DT_F32) {
                    memcpy(&rows[(size_t)i * hs + k], src + ((size_t)ids[i] * hs + k) * 4, 4);
                } else {
                    uint16_t hb;
                    memcpy(&hb, src + ((size_t)ids[i] * hs + k) * 2, 2);
                    rows[(size_t)i * hs + k] = half_bits_to_float(hb);
                }
            }
        CMFC_CUDA(cudaMemcpyAsync(h, rows.data(), rows.size() * 4, cudaMemcpyHostToDevice, c->stream));
        launch_scale_f32(h, rows.size(), emb_scale, c->stream);
        c->launches++;
        CMFC_CUDA(cudaStreamSynchronize(c->stream));
        return OK;
    }
    return fail(ERR_UNSUPPORTED, "te.embed_tokens.weight: expected q8_row, f32 or f16");
}

// streams: null, or device [(nl + 1), n, hidden]; final_out: null, or device [n, hidden].
// d_penultimate: null, or device [n, hidden] receiving the stream that enters the last layer; when
// nothing else is asked for, the last layer is not run.
int encode_device(Context* c, cmfc_gemma* g, const uint32_t* ids, int n, float* d_streams, float* d_final,
                  float* d_penultimate) {
    const int run_layers = (d_streams || d_final) ? g->nl : g->nl - 1;
    const int hs = g->hidden, nh = g->nh, nkv = g->nkv, hd = g->hd;
    const int qkv_cols = (nh + 2 * nkv) * hd;
    CMFC_TRY(ensure_rope(c, g, n));
    DevBuf &bh = c->buf("te.h"), &bxn = c->buf("te.xn"), &bqkv = c->buf("te.qkv"), &battn = c->buf("te.attn"),
           &bproj = c->buf("te.proj"), &bgu = c->buf("te.gu"), &bact = c->buf("te.act");
    const size_t n2 = 2 * (size_t)n;   // split rows: hi halves then lo halves
    CMFC_TRY(bh.ensure((size_t)n * hs * 4));
    CMFC_TRY(bxn.ensure(n2 * hs * 2));
    CMFC_TRY(bqkv.ensure(n2 * qkv_cols * 4));
    CMFC_TRY(battn.ensure(n2 * nh * hd * 2));
    CMFC_TRY(bproj.ensure(n2 * hs * 4));
    CMFC_TRY(bgu.ensure(n2 * 2 * g->inter * 4));
    CMFC_TRY(bact.ensure(n2 * g->inter * 2));
    float* h = bh.as<float>();
    __nv_bfloat16* xn = bxn.as<__nv_bfloat16>();
    const float* cos_t = g->rope.as<float>();
    const float* sin_t = cos_t + (size_t)g->rope_n * (hd / 2);
    CMFC_TRY(embed_rows(c, g, ids, n, h));
    cudaStream_t s = c->stream;
    {
        SpanGuard sg(c, "te-norm");
        launch_gemma_residual_norm(h, nullptr, n, hs, nullptr, g->layers[0].input_norm, g->eps, xn, nullptr, s);
        c->launches++;
    }
    for (int l = 0; l < run_layers; ++l) {
        const GemmaLayer& L = g->layers[l];
        if (d_penultimate && l == g->nl - 1)
            CMFC_CUDA(cudaMemcpyAsync(d_penultimate, h, (size_t)n * hs * 4, cudaMemcpyDeviceToDevice, s));
        if (d_streams)
            CMFC_CUDA(cudaMemcpyAsync(d_streams + (size_t)l * n * hs, h, (size_t)n * hs * 4, cudaMemcpyDeviceToDevice, s));
        {
            SpanGuard sg(c, "te-qkv");
            CMFC_TRY(dev_gemm(c, L.qkv, xn, 2 * n, bqkv.p, qkv_cols, GEMM_OUT_F32));
        }
        {
            SpanGuard sg(c, "te-attn");
            launch_rope_half(bqkv.as<float>(), n, nh + nkv, nh + 2 * nkv, qkv_cols, hd, cos_t, sin_t, s);
            CMFC_TRY(launch_attn_causal_f32(bqkv.as<float>(), n, nh, nkv, hd, g->scale, g->softcap, battn.as<__nv_bfloat16>(), s));
            c->launches += 2;
        }
        {
            SpanGuard sg(c, "te-o");
            CMFC_TRY(dev_gemm(c, L.o, battn.as<__nv_bfloat16>(), 2 * n, bproj.p, hs, GEMM_OUT_F32));
        }
        {
            // h += rms(proj) * (1 + post_attn); xn = rms(h) * (1 + pre_ffn)   (textenc.rs:326-345)
            SpanGuard sg(c, "te-norm");
            launch_gemma_residual_norm(h, bproj.as<float>(), n, hs, L.post_attn_norm, L.pre_ffn_norm, g->eps, xn, nullptr, s);
            c->launches++;
        }
        {
            SpanGuard sg(c, "te-ffn");
            CMFC_TRY(dev_gemm(c, L.gate_up, xn, 2 * n, bgu.p, 2 * g->inter, GEMM_OUT_F32));
            launch_geglu_split(bgu.as<float>(), n, g->inter, bact.as<__nv_bfloat16>(), s);
            c->launches++;
            CMFC_TRY(dev_gemm(c, L.down, bact.as<__nv_bfloat16>(), 2 * n, bproj.p, hs, GEMM_OUT_F32));
        }
        {
            SpanGuard sg(c, "te-norm");
            launch_gemma_residual_norm(h, bproj.as<float>(), n, hs, L.post_ffn_norm,
                                       l + 1 < g->nl ? g->layers[l + 1].input_norm : nullptr, g->eps, xn, nullptr, s);
            c->launches++;
        }
    }
    if (d_penultimate && run_layers == g->nl - 1)
        CMFC_CUDA(cudaMemcpyAsync(d_penultimate, h, (size_t)n * hs * 4, cudaMemcpyDeviceToDevice, s));
    if (d_streams)
        CMFC_CUDA(cudaMemcpyAsync(d_streams + (size_t)g->nl * n * hs, h, (size_t)n * hs * 4, cudaMemcpyDeviceToDevice, s));
    if (d_final) {
        launch_gemma_residual_norm(h, nullptr, n, hs, nullptr, g->final_norm, g->eps, nullptr, d_final, s);
        c->launches++;
    }
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace

extern "C" int cmfc_gemma_create(cmfc_model* mm, cmfc_gemma** out) {
    NEED(mm && out, "gemma_create: null argument");
    NEED_CTX();
    Model* m = mm->m;
    const int64_t ci = find(m, "te.config_json");
    if (ci < 0) return fail(ERR_NOT_FOUND, "container has no te.config_json");
    const std::string js(reinterpret_cast<const char*>(m->bytes(ci)), m->recs[ci].nbytes);
    std::unique_ptr<cmfc_gemma> g(new cmfc_gemma());
    struct Cleanup {
        std::unique_ptr<cmfc_gemma>& g;
        bool armed = true;
        ~Cleanup() {
            if (armed && g) for (void* p : g->owned) cudaFree(p);
        }
    } cleanup{g};
    g->m = m;
    double d;
    auto need_num = [&](const char* key, int* dst) -> int {
        if (!json_number(js, key, &d)) return fail(ERR_FORMAT, std::string("te.config_json: ") + key + " missing");
        *dst = (int)d;
        return OK;
    };
    CMFC_TRY(need_num("num_hidden_layers", &g->nl));
    CMFC_TRY(need_num("hidden_size", &g->hidden));
    CMFC_TRY(need_num("num_attention_heads", &g->nh));
    CMFC_TRY(need_num("num_key_value_heads", &g->nkv));
    CMFC_TRY(need_num("head_dim", &g->hd));
    g->scale = 1.0f / sqrtf(json_number(js, "query_pre_attn_scalar", &d) ? (float)d : 256.0f);
    g->softcap = json_number(js, "attn_logit_softcapping", &d) ? (float)d : 0.0f;
    g->theta = json_number(js, "rope_theta", &d) ? (float)d : 10000.0f;
    g->eps = json_number(js, "rms_norm_eps", &d) ? d : 1e-6;
    g->window = json_number(js, "sliding_window", &d) ? (int)d : 4096;
    if (g->nl <= 0 || g->nh <= 0 || g->nkv <= 0 || g->nh % g->nkv || g->hd <= 0 || g->hd % 2)
        return fail(ERR_FORMAT, "te.config_json: bad head geometry");
    CMFC_TRY(need_idx(m, "te.embed_tokens.weight", &g->embed_idx));
    {
        const TensorRec& e = m->recs[g->embed_idx];
        if (e.ndim != 2 || (int)e.shape[1] != g->hidden) return fail(ERR_SHAPE, "te.embed_tokens.weight: expected [vocab, hidden]");
        g->vocab = (int)e.shape[0];
    }
    for (int l = 0; l < g->nl; ++l) {
        const std::string p = "te.layers." + std::to_string(l);
        GemmaLayer L;
        int64_t q, k, v, o, gate, up, down;
        CMFC_TRY(need_idx(m, p + ".self_attn.q_proj.weight", &q));
        CMFC_TRY(need_idx(m, p + ".self_attn.k_proj.weight", &k));
        CMFC_TRY(need_idx(m, p + ".self_attn.v_proj.weight", &v));
        CMFC_TRY(need_idx(m, p + ".self_attn.o_proj.weight", &o));
        CMFC_TRY(need_idx(m, p + ".mlp.gate_proj.weight", &gate));
        CMFC_TRY(need_idx(m, p + ".mlp.up_proj.weight", &up));
        CMFC_TRY(need_idx(m, p + ".mlp.down_proj.weight", &down));
        CMFC_TRY(get_weight_concat(c, m, q, k, v, &L.qkv));
        CMFC_TRY(get_weight(c, m, o, &L.o));
        CMFC_TRY(get_weight_interleaved(c, m, gate, up, &L.gate_up));
        CMFC_TRY(get_weight(c, m, down, &L.down));
        if (L.qkv->rows != (g->nh + 2 * g->nkv) * g->hd || L.qkv->cols != g->hidden || L.o->rows != g->hidden ||
            L.o->cols != g->nh * g->hd || L.gate_up->cols != g->hidden || L.down->rows != g->hidden ||
            L.down->cols * 2 != L.gate_up->rows)
            return fail(ERR_SHAPE, "gemma layer " + std::to_string(l) + ": projection shapes disagree with te.config_json");
        if (l == 0) g->inter = L.down->cols;
        if (L.down->cols != g->inter) return fail(ERR_SHAPE, "gemma: layers differ in intermediate size");
        CMFC_TRY(load_norm_plus_one(c, g.get(), p + ".input_layernorm.weight", g->hidden, &L.input_norm));
        CMFC_TRY(load_norm_plus_one(c, g.get(), p + ".post_attention_layernorm.weight", g->hidden, &L.post_attn_norm));
        CMFC_TRY(load_norm_plus_one(c, g.get(), p + ".pre_feedforward_layernorm.weight", g->hidden, &L.pre_ffn_norm));
        CMFC_TRY(load_norm_plus_one(c, g.get(), p + ".post_feedforward_layernorm.weight", g->hidden, &L.post_ffn_norm));
        g->layers.push_back(L);
    }
    CMFC_TRY(load_norm_plus_one(c, g.get(), "te.norm.weight", g->hidden, &g->final_norm));
    CMFC_CUDA(cudaStreamSynchronize(0));
    cleanup.armed = false;
    *out = g.release();
    return OK;
}

extern "C" void cmfc_gemma_destroy(cmfc_gemma* g) {
    if (!g) return;
    for (void* p : g->owned) cudaFree(p);
    g->rope.release();
    delete g;
}

extern "C" int cmfc_gemma_dims(const cmfc_gemma* g, uint32_t dims[8]) {
    NEED(g && dims, "gemma_dims: null argument");
    const uint32_t v[8] = {(uint32_t)g->hidden, (uint32_t)g->nl, (uint32_t)g->nh, (uint32_t)g->nkv,
                           (uint32_t)g->hd,     (uint32_t)g->inter, (uint32_t)g->vocab, (uint32_t)g->window};
    memcpy(dims, v, sizeof(v));
    return OK;
}

extern "C" int cmfc_gemma_encode(cmfc_gemma* g, const uint32_t* ids, size_t n, float* final_out, float* streams_out) {
    NEED(g && ids && n > 0, "gemma_encode: null argument or empty prompt");
    NEED(final_out || streams_out, "gemma_encode: no output requested");
    if ((int64_t)n >= (int64_t)g->window)
        return fail(ERR_SHAPE, "gemma_encode: prompt of " + std::to_string(n) + " tokens exceeds the sliding window " +
                                   std::to_string(g->window));
    NEED_CTX();
    const size_t per = n * (size_t)g->hidden;
    DevBuf &bs = c->buf("te.streams"), &bf = c->buf("te.final");
    if (streams_out) CMFC_TRY(bs.ensure((size_t)(g->nl + 1) * per * 4));
    if (final_out) CMFC_TRY(bf.ensure(per * 4));
    CMFC_TRY(encode_device(c, g, ids, (int)n, streams_out ? bs.as<float>() : nullptr, final_out ? bf.as<float>() : nullptr,
                           nullptr));
    if (streams_out)
        CMFC_CUDA(cudaMemcpyAsync(streams_out, bs.p, (size_t)(g->nl + 1) * per * 4, cudaMemcpyDeviceToHost, c->stream));
    if (final_out) CMFC_CUDA(cudaMemcpyAsync(final_out, bf.p, per * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "gemma_encode");
}

extern "C" int cmfc_gemma_caption_features(cmfc_gemma* g, const uint32_t* ids, size_t n, float* out) {
    NEED(g && ids && out && n > 0, "gemma_caption_features: null argument or empty prompt");
    if ((int64_t)n >= (int64_t)g->window)
        return fail(ERR_SHAPE, "gemma_caption_features: prompt of " + std::to_string(n) +
                                   " tokens exceeds the sliding window " + std::to_string(g->window));
    NEED_CTX();
    const size_t per = n * (size_t)g->hidden;
    DevBuf& bp = c->buf("te.penult");
    CMFC_TRY(bp.ensure(per * 4));
    CMFC_TRY(encode_device(c, g, ids, (int)n, nullptr, nullptr, bp.as<float>()));
    CMFC_CUDA(cudaMemcpyAsync(out, bp.p, per * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "gemma_caption_features");
}

// instrumentation: device time of caption_features for a synthetic prompt of n tokens (CUDA events)
extern "C" int cmfc_bench_gemma(cmfc_gemma* g, size_t n, int iters, float* ms_per_prompt) {
    NEED(g && ms_per_prompt && n > 0 && iters > 0 && (int64_t)n < (int64_t)g->window, "bench_gemma: bad argument");
    NEED_CTX();
    std::vector<uint32_t> ids(n);
    for (size_t i = 0; i < n; ++i) ids[i] = (uint32_t)((i * 2654435761u) % (uint32_t)g->vocab);
    DevBuf& bp = c->buf("te.penult");
    CMFC_TRY(bp.ensure(n * (size_t)g->hidden * 4));
    CMFC_TRY(encode_device(c, g, ids.data(), (int)n, nullptr, nullptr, bp.as<float>()));
    cudaEvent_t e0, e1;
    CMFC_CUDA(cudaEventCreate(&e0));
    CMFC_CUDA(cudaEventCreate(&e1));
    CMFC_CUDA(cudaEventRecord(e0, c->stream));
    for (int i = 0; i < iters; ++i) CMFC_TRY(encode_device(c, g, ids.data(), (int)n, nullptr, nullptr, bp.as<float>()));
    CMFC_CUDA(cudaEventRecord(e1, c->stream));
    CMFC_CUDA(cudaEventSynchronize(e1));
    float ms = 0;
    CMFC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms_per_prompt = ms / iters;
    return check_status(c, "bench_gemma");
}
