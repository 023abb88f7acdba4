// FLUX-class VAE decoder on the device (crates/cortiq-engine/src/vae.rs): conv_in -> mid
// (resnet, single-head attention, resnet) -> up blocks (resnets, nearest 2x + conv) -> GroupNorm +
// SiLU -> conv_out, with the latent de-normalization z / scaling_factor + shift_factor in front.
// Activations stay on the device as NHWC f32 (the residual stream) and NHWC split-f16 planes (the
// operand of the next convolution); all matrix work goes through the split-f16 implicit-GEMM
// kernel (conv_f16x2.cu).  Also the facade's stand-alone conv entries on host tensors.
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

int round_up(int v, int m) { return (v + m - 1) / m * m; }

struct Planes {
    __half* hi = nullptr;
    __half* lo = nullptr;
};

// A weight of the implicit GEMM: [oc_pad, taps * ic_pad] split planes (+ f32 bias)
struct ConvW {
    int oc = 0, ic = 0, ic_pad = 0, taps = 0, a_planes = 2;
    Planes w;
    float* bias = nullptr;
    CUtensorMap tm_hi, tm_lo;
};
struct NormW {
    float* w = nullptr;
    float* b = nullptr;
    int c = 0;
};
struct ResnetW {
    NormW n1, n2;
    ConvW c1, c2, sc;
    bool has_sc = false;
};
struct UpW {
    std::vector<ResnetW> res;
    bool has_up = false;
    ConvW up;
};

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

}  // namespace

struct cmfc_vae {
    Model* m = nullptr;
    int device = -1;
    int groups = 32, latent_channels = 16;
    float scaling = 1.0f, shift = 0.0f;
    ConvW conv_in, conv_out;
    ResnetW mid1, mid2;
    NormW attn_norm;
    ConvW attn_q, attn_k, attn_v, attn_o;
    int attn_c = 0;
    std::vector<UpW> ups;
    NormW norm_out;
    std::vector<void*> owned;  // device allocations of this decoder
    int upscale() const {
        int s = 1;
        for (auto& u : ups) s *= u.has_up ? 2 : 1;
        return s;
    }
};

namespace {

int dev_alloc(std::vector<void*>& owned, size_t bytes, void** out) {
    if (cudaMalloc(out, bytes ? bytes : 16) != cudaSuccess) return fail(ERR_OOM, "out of device memory for a VAE weight");
    owned.push_back(*out);
    return OK;
}

// dense f32 [oc, ic, k, k] on the device -> padded split planes + maps
int build_conv(Context* c, std::vector<void*>& owned, const float* d_w, const float* d_b, int oc, int ic, int taps, bool f16_exact,
               ConvW* out) {
    out->oc = oc; out->ic = ic; out->taps = taps;
    out->ic_pad = round_up(ic, 32);
    out->a_planes = f16_exact ? 1 : 2;
    const int oc_pad = round_up(oc, 128);
    const size_t cols = (size_t)taps * out->ic_pad, n = (size_t)oc_pad * cols;
    CMFC_TRY(dev_alloc(owned, n * 2, reinterpret_cast<void**>(&out->w.hi)));
    CMFC_TRY(dev_alloc(owned, n * 2, reinterpret_cast<void**>(&out->w.lo)));
    CMFC_CUDA(cudaMemsetAsync(out->w.hi, 0, n * 2, c->stream));
    CMFC_CUDA(cudaMemsetAsync(out->w.lo, 0, n * 2, c->stream));
    launch_conv_weight_split(d_w, oc, ic, taps, out->ic_pad, out->w.hi, out->w.lo, c->stream);
    CMFC_CUDA(cudaGetLastError());
    out->bias = nullptr;
    if (d_b) {
        CMFC_TRY(dev_alloc(owned, (size_t)oc * 4, reinterpret_cast<void**>(&out->bias)));
        CMFC_CUDA(cudaMemcpyAsync(out->bias, d_b, (size_t)oc * 4, cudaMemcpyDeviceToDevice, c->stream));
    }
    CMFC_TRY(make_tensor_map_2d(&out->tm_hi, out->w.hi, 2, oc_pad, cols, cols * 2, 128, 32, 2));
    CMFC_TRY(make_tensor_map_2d(&out->tm_lo, out->w.lo, 2, oc_pad, cols, cols * 2, 128, 32, 2));
    return OK;
}

int load_conv(Context* c, cmfc_vae* v, const std::string& name, ConvW* out) {
    Model* m = v->m;
    const int64_t wi = find(m, name + ".weight"), bi = find(m, name + ".bias");
    if (wi < 0 || bi < 0) return fail(ERR_NOT_FOUND, "missing tensor " + name + ".weight / .bias");
    const TensorRec& t = m->recs[wi];
    int oc, ic, taps;
    if (t.ndim == 4) {
        if (t.shape[2] != t.shape[3] || (t.shape[2] != 1 && t.shape[2] != 3))
            return fail(ERR_UNSUPPORTED, "tensor " + t.name + ": only 1x1 and 3x3 kernels are supported");
        oc = (int)t.shape[0]; ic = (int)t.shape[1]; taps = (int)(t.shape[2] * t.shape[3]);
    } else if (t.ndim == 2) {
        oc = (int)t.shape[0]; ic = (int)t.shape[1]; taps = 1;
    } else {
        return fail(ERR_SHAPE, "tensor " + t.name + ": expected a 4-D conv kernel or a 2-D linear");
    }
    DevWeight *dw = nullptr, *db = nullptr;
    CMFC_TRY(upload_f32(c, m, wi, &dw));
    CMFC_TRY(upload_f32(c, m, bi, &db));
    if ((size_t)db->rows * db->cols != (size_t)oc) return fail(ERR_SHAPE, "tensor " + name + ".bias: length disagrees with the kernel");
    return build_conv(c, v->owned, reinterpret_cast<const float*>(dw->plane), reinterpret_cast<const float*>(db->plane), oc, ic,
                      taps, t.dtype == DT_F16, out);
}

int load_norm(Context* c, cmfc_vae* v, const std::string& name, NormW* out) {
    Model* m = v->m;
    const int64_t wi = find(m, name + ".weight"), bi = find(m, name + ".bias");
    if (wi < 0 || bi < 0) return fail(ERR_NOT_FOUND, "missing tensor " + name + ".weight / .bias");
    DevWeight *dw = nullptr, *db = nullptr;
    CMFC_TRY(upload_f32(c, m, wi, &dw));
    CMFC_TRY(upload_f32(c, m, bi, &db));
    out->c = dw->rows * dw->cols;
    if (db->rows * db->cols != out->c) return fail(ERR_SHAPE, "tensor " + name + ": weight and bias lengths differ");
    if (out->c % v->groups) return fail(ERR_SHAPE, "tensor " + name + ": channels not divisible by norm_num_groups");
    out->w = reinterpret_cast<float*>(dw->plane);
    out->b = reinterpret_cast<float*>(db->plane);
    return OK;
}

int load_resnet(Context* c, cmfc_vae* v, const std::string& name, ResnetW* out) {
    CMFC_TRY(load_norm(c, v, name + ".norm1", &out->n1));
    CMFC_TRY(load_conv(c, v, name + ".conv1", &out->c1));
    CMFC_TRY(load_norm(c, v, name + ".norm2", &out->n2));
    CMFC_TRY(load_conv(c, v, name + ".conv2", &out->c2));
    out->has_sc = find(v->m, name + ".conv_shortcut.weight") >= 0;
    if (out->has_sc) CMFC_TRY(load_conv(c, v, name + ".conv_shortcut", &out->sc));
    if (out->c1.ic != out->n1.c || out->c2.ic != out->n2.c || out->c1.oc != out->c2.ic || out->c2.oc != out->c1.oc)
        return fail(ERR_SHAPE, "resnet " + name + ": channel counts of norms and convs disagree");
    if (out->has_sc ? (out->sc.ic != out->c1.ic || out->sc.oc != out->c2.oc) : (out->c1.ic != out->c2.oc))
        return fail(ERR_SHAPE, "resnet " + name + ": shortcut channels disagree");
    return OK;
}

// ---- one implicit-GEMM launch ----
struct ConvOut {
    float* f32 = nullptr;
    Planes split;
    const float* residual = nullptr;
    int pitch = 0;          // 0: oc (pixel-major) / pixels (channel-major)
    int channel_major = 0;
    float scale = 1.0f;
    bool stats = false;     // also leave the per-channel sum / sum of squares of the output in "vae.stats"
};

// a: weight-side planes as a [oc rows, taps * ic_pad] matrix (maps prebuilt); b: NHWC planes with
// ``b_pitch`` stored channels per pixel of which ``b_c`` are addressable (the rest reads as zero)
int run_gemm(Context* c, const CUtensorMap& tm_a_hi, const CUtensorMap& tm_a_lo, int a_planes, int oc, int ic_pad,
             int taps, const float* bias, const Planes& b, int b_planes, int b_c, int b_pitch, int w, int h,
             const ConvOut& o) {
    ConvParams p;
    memset(&p, 0, sizeof(p));
    p.ic = ic_pad; p.taps = taps; p.w = w; p.h = h;
    conv_tile_shape(w, h, &p.bw, &p.bh);
    p.oc = oc; p.a_planes = a_planes; p.b_planes = b_planes;
    p.bias = bias; p.out_scale = o.scale; p.residual = o.residual;
    p.out_f32 = o.f32; p.out_hi = o.split.hi; p.out_lo = o.split.lo;
    p.channel_major = o.channel_major;
    p.out_pitch = o.pitch ? o.pitch : (o.channel_major ? w * h : oc);
    p.status = c->status;
    double* stats = c->buf("vae.stats").as<double>();
    const size_t slots = conv_stats_slots(w, h);
    if (o.stats) {
        if (c->buf("vae.stats").cap < (2048 + slots * 2 * (size_t)oc) * sizeof(double))
            return fail(ERR_SHAPE, "conv: statistics scratch too small");
        p.stats_partial = stats + 2048;
    }
    CUtensorMap tm_b_hi, tm_b_lo;
    CMFC_TRY(make_tensor_map_nhwc16(&tm_b_hi, b.hi, b_c, w, h, (uint64_t)b_pitch * 2, 32, p.bw, p.bh, 2));
    tm_b_lo = tm_b_hi;
    if (b_planes == 2) CMFC_TRY(make_tensor_map_nhwc16(&tm_b_lo, b.lo, b_c, w, h, (uint64_t)b_pitch * 2, 32, p.bw, p.bh, 2));
    c->launches++;
    CMFC_TRY(launch_conv_f16x2(tm_a_hi, tm_a_lo, tm_b_hi, tm_b_lo, p, c->num_sms, c->stream));
    if (o.stats) {
        launch_gn_finalize(p.stats_partial, slots, oc, stats, c->stream);
        CMFC_CUDA(cudaGetLastError());
        c->launches++;
    }
    return OK;
}

int run_conv(Context* c, const ConvW& cw, const Planes& x, int x_c, int w, int h, const ConvOut& o) {
    if (x_c != cw.ic_pad) return fail(ERR_SHAPE, "conv: input planes have the wrong channel count");
    return run_gemm(c, cw.tm_hi, cw.tm_lo, cw.a_planes, cw.oc, cw.ic_pad, cw.taps, cw.bias, x, 2, x_c, x_c, w, h, o);
}

// ``have_stats``: the convolution that produced x already left its channel statistics in "vae.stats"
int group_norm(Context* c, const NormW& n, int groups, const float* x, size_t pixels, int silu, const Planes& y,
               const Planes* raw, bool have_stats) {
    double* stats = c->buf("vae.stats").as<double>();
    if (!have_stats) {
        CMFC_TRY(launch_gn_stats(x, pixels, n.c, stats, c->stream));
        c->launches += 2;
    }
    CMFC_TRY(launch_gn_apply(x, pixels, n.c, groups, stats, n.w, n.b, silu, y.hi, y.lo, raw ? raw->hi : nullptr,
                             raw ? raw->lo : nullptr, c->stream));
    c->launches++;
    return OK;
}

struct Work {
    float *x = nullptr, *t1 = nullptr, *t2 = nullptr;
    Planes s0, s1;
    bool stats_ready = false;  // "vae.stats" holds the channel statistics of x
};

// x [pix, cin] -> [pix, cout]; the result lands in wk.x (buffers rotate)
int run_resnet(Context* c, const cmfc_vae* v, const ResnetW& r, Work& wk, int w, int h) {
    const size_t pix = (size_t)w * h;
    CMFC_TRY(group_norm(c, r.n1, v->groups, wk.x, pix, 1, wk.s0, r.has_sc ? &wk.s1 : nullptr, wk.stats_ready));
    ConvOut o1;
    o1.f32 = wk.t1;
    o1.stats = true;
    CMFC_TRY(run_conv(c, r.c1, wk.s0, r.n1.c, w, h, o1));
    CMFC_TRY(group_norm(c, r.n2, v->groups, wk.t1, pix, 1, wk.s0, nullptr, true));
    if (r.has_sc) {
        ConvOut os;
        os.f32 = wk.t2;
        CMFC_TRY(run_conv(c, r.sc, wk.s1, r.n1.c, w, h, os));
        ConvOut o2;
        o2.f32 = wk.t2;
        o2.residual = wk.t2;
        o2.stats = true;
        CMFC_TRY(run_conv(c, r.c2, wk.s0, r.n2.c, w, h, o2));
        std::swap(wk.x, wk.t2);
    } else {
        ConvOut o2;
        o2.f32 = wk.x;
        o2.residual = wk.x;
        o2.stats = true;
        CMFC_TRY(run_conv(c, r.c2, wk.s0, r.n2.c, w, h, o2));
    }
    wk.stats_ready = true;
    return OK;
}

// single-head attention over the h*w tokens (vae.rs:415-489); wk.x updated in place
int run_attention(Context* c, const cmfc_vae* v, Work& wk, int w, int h) {
    const int n = w * h, ch = v->attn_c, n_pad = round_up(n, 32);
    DevBuf &bq = c->buf("vae.q"), &bk = c->buf("vae.k"), &bvt = c->buf("vae.vt"), &bs = c->buf("vae.scores"),
           &bp = c->buf("vae.probs"), &bo = c->buf("vae.attn_o");
    const size_t tok = (size_t)n * ch;
    CMFC_TRY(bq.ensure(tok * 4));
    CMFC_TRY(bk.ensure(tok * 4));
    CMFC_TRY(bo.ensure(tok * 4));
    CMFC_TRY(bvt.ensure((size_t)ch * n_pad * 4));
    CMFC_TRY(bs.ensure((size_t)n * n_pad * 4));
    CMFC_TRY(bp.ensure((size_t)n * n_pad * 4));
    const Planes q{bq.as<__half>(), bq.as<__half>() + tok}, k{bk.as<__half>(), bk.as<__half>() + tok};
    const Planes ot{bo.as<__half>(), bo.as<__half>() + tok};
    const Planes vt{bvt.as<__half>(), bvt.as<__half>() + (size_t)ch * n_pad};
    const Planes pr{bp.as<__half>(), bp.as<__half>() + (size_t)n * n_pad};
    CMFC_TRY(group_norm(c, v->attn_norm, v->groups, wk.x, (size_t)n, 0, wk.s0, nullptr, wk.stats_ready));
    ConvOut oq; oq.split = q;
    CMFC_TRY(run_conv(c, v->attn_q, wk.s0, ch, n, 1, oq));
    ConvOut ok; ok.split = k;
    CMFC_TRY(run_conv(c, v->attn_k, wk.s0, ch, n, 1, ok));
    ConvOut ov; ov.split = vt; ov.channel_major = 1; ov.pitch = n_pad;
    CMFC_TRY(run_conv(c, v->attn_v, wk.s0, ch, n, 1, ov));
    // scores[i, j] = (q_i . k_j) / sqrt(c): A = K as [n rows, c], B = Q
    CUtensorMap tk_hi, tk_lo;
    CMFC_TRY(make_tensor_map_2d(&tk_hi, k.hi, 2, n, ch, (uint64_t)ch * 2, 128, 32, 2));
    CMFC_TRY(make_tensor_map_2d(&tk_lo, k.lo, 2, n, ch, (uint64_t)ch * 2, 128, 32, 2));
    ConvOut os; os.f32 = bs.as<float>(); os.pitch = n_pad; os.scale = 1.0f / sqrtf((float)ch);
    CMFC_TRY(run_gemm(c, tk_hi, tk_lo, 2, n, ch, 1, nullptr, q, 2, ch, ch, n, 1, os));
    CMFC_TRY(launch_softmax_rows_split(bs.as<float>(), (size_t)n, n, (size_t)n_pad, pr.hi, pr.lo, (size_t)n_pad, c->stream));
    c->launches++;
    // out[i, :] = sum_j p[i, j] v[j, :]: A = V^T as [c rows, n], B = P with n "channels"
    CUtensorMap tv_hi, tv_lo;
    CMFC_TRY(make_tensor_map_2d(&tv_hi, vt.hi, 2, ch, n, (uint64_t)n_pad * 2, 128, 32, 2));
    CMFC_TRY(make_tensor_map_2d(&tv_lo, vt.lo, 2, ch, n, (uint64_t)n_pad * 2, 128, 32, 2));
    ConvOut oo; oo.split = ot;
    CMFC_TRY(run_gemm(c, tv_hi, tv_lo, 2, ch, n_pad, 1, nullptr, pr, 2, n, n_pad, n, 1, oo));
    ConvOut of; of.f32 = wk.x; of.residual = wk.x; of.stats = true;
    CMFC_TRY(run_conv(c, v->attn_o, ot, ch, n, 1, of));
    wk.stats_ready = true;
    return OK;
}

}  // namespace

namespace {

struct Sizes {
    size_t max_elems = 0;
    size_t stats_doubles = 0;  // scratch of the fused GroupNorm statistics: slots x channels x 2
    int out_h = 0, out_w = 0;
};

// the largest activation (pixels x channels) the schedule touches, and the image extent
Sizes plan(const cmfc_vae* v, int h, int w) {
    Sizes s;
    auto see = [&](size_t pix, int ch) {
        s.max_elems = std::max(s.max_elems, pix * (size_t)ch);
        s.stats_doubles = std::max(s.stats_doubles, conv_stats_slots(w, h) * 2 * (size_t)ch);
    };
    size_t pix = (size_t)h * w;
    see(pix, v->conv_in.ic_pad);
    see(pix, v->conv_in.oc);
    auto res = [&](const ResnetW& r) { see(pix, r.c1.ic); see(pix, r.c1.oc); };
    res(v->mid1);
    res(v->mid2);
    for (auto& u : v->ups) {
        for (auto& r : u.res) res(r);
        if (u.has_up) {
            pix *= 4; h *= 2; w *= 2;
            see(pix, u.up.ic);
            see(pix, u.up.oc);
        }
    }
    see(pix, v->conv_out.ic);
    s.out_h = h; s.out_w = w;
    return s;
}

// d_z: device f32 [latent_channels, h, w]; d_out: device f32 [3, H, W]
int decode_device(Context* c, cmfc_vae* v, const float* d_z, int h, int w, float* d_out) {
    const Sizes sz = plan(v, h, w);
    if (sz.max_elems > (size_t)1 << 33) return fail(ERR_SHAPE, "vae_decode: latent too large");
    const char* names[5] = {"vae.x", "vae.t1", "vae.t2", "vae.s0", "vae.s1"};
    for (const char* n : names) CMFC_TRY(c->buf(n).ensure(sz.max_elems * 4));
    CMFC_TRY(c->buf("vae.stats").ensure(std::max(gn_stats_bytes(1024), (2048 + sz.stats_doubles) * sizeof(double))));
    Work wk;
    wk.x = c->buf("vae.x").as<float>();
    wk.t1 = c->buf("vae.t1").as<float>();
    wk.t2 = c->buf("vae.t2").as<float>();
    wk.s0 = Planes{c->buf("vae.s0").as<__half>(), c->buf("vae.s0").as<__half>() + sz.max_elems};
    wk.s1 = Planes{c->buf("vae.s1").as<__half>(), c->buf("vae.s1").as<__half>() + sz.max_elems};
    size_t pix = (size_t)h * w;
    {
        SpanGuard g(c, "vae-in");
        launch_nchw_to_split(d_z, v->latent_channels, pix, v->conv_in.ic_pad, v->scaling, v->shift, 1, wk.s0.hi, wk.s0.lo,
                             c->stream);
        CMFC_CUDA(cudaGetLastError());
        c->launches++;
        ConvOut o;
        o.f32 = wk.x;
        o.stats = true;
        CMFC_TRY(run_conv(c, v->conv_in, wk.s0, v->conv_in.ic_pad, w, h, o));
        wk.stats_ready = true;
    }
    {
        SpanGuard g(c, "vae-mid");
        CMFC_TRY(run_resnet(c, v, v->mid1, wk, w, h));
        CMFC_TRY(run_attention(c, v, wk, w, h));
        CMFC_TRY(run_resnet(c, v, v->mid2, wk, w, h));
    }
    int ui = 0;
    for (auto& u : v->ups) {
        const std::string span = "vae-up" + std::to_string(ui++);
        SpanGuard g(c, span.c_str());
        for (auto& r : u.res) CMFC_TRY(run_resnet(c, v, r, wk, w, h));
        if (u.has_up) {
            launch_upsample2x_split(wk.x, h, w, u.up.ic, wk.s0.hi, wk.s0.lo, c->stream);
            CMFC_CUDA(cudaGetLastError());
            c->launches++;
            h *= 2; w *= 2;
            ConvOut o;
            o.f32 = wk.t1;
            o.stats = true;
            CMFC_TRY(run_conv(c, u.up, wk.s0, u.up.ic, w, h, o));
            std::swap(wk.x, wk.t1);
        }
    }
    {
        SpanGuard g(c, "vae-out");
        pix = (size_t)h * w;
        CMFC_TRY(group_norm(c, v->norm_out, v->groups, wk.x, pix, 1, wk.s0, nullptr, wk.stats_ready));
        ConvOut o;
        o.f32 = d_out;
        o.channel_major = 1;
        CMFC_TRY(run_conv(c, v->conv_out, wk.s0, v->norm_out.c, w, h, o));
    }
    return OK;
}

int check_decode_args(const cmfc_vae* v, const void* z, size_t h, size_t w, const void* out) {
    NEED(v && z && out, "vae_decode: null argument");
    NEED(h > 0 && w > 0 && h <= 4096 && w <= 4096, "vae_decode: latent extent out of range");
    return OK;
}

}  // namespace

extern "C" int cmfc_vae_create(cmfc_model* mm, cmfc_vae** out) {
    NEED(mm && out, "vae_create: null argument");
    NEED_CTX();
    Model* m = mm->m;
    const int64_t ci = find(m, "vae.config_json");
    if (ci < 0) return fail(ERR_NOT_FOUND, "container has no vae.config_json");
    const std::string js(reinterpret_cast<const char*>(m->bytes(ci)), m->recs[ci].nbytes);
    std::unique_ptr<cmfc_vae> v(new cmfc_vae());
    struct Cleanup {
        std::unique_ptr<cmfc_vae>& v;
        bool armed = true;
        ~Cleanup() {
            if (armed && v) for (void* p : v->owned) cudaFree(p);
        }
    } cleanup{v};
    v->m = m;
    v->device = c->device;
    double d;
    v->groups = json_number(js, "norm_num_groups", &d) ? (int)d : 32;
    v->latent_channels = json_number(js, "latent_channels", &d) ? (int)d : 16;
    v->scaling = json_number(js, "scaling_factor", &d) ? (float)d : 1.0f;
    v->shift = json_number(js, "shift_factor", &d) ? (float)d : 0.0f;
    if (v->groups <= 0 || v->latent_channels <= 0 || v->scaling == 0.0f) return fail(ERR_FORMAT, "vae.config_json: bad values");
    const std::string dec = "vae.decoder.";
    CMFC_TRY(load_conv(c, v.get(), dec + "conv_in", &v->conv_in));
    if (v->conv_in.ic != v->latent_channels) return fail(ERR_SHAPE, "vae: conv_in channels differ from latent_channels");
    CMFC_TRY(load_resnet(c, v.get(), dec + "mid_block.resnets.0", &v->mid1));
    const std::string at = dec + "mid_block.attentions.0.";
    CMFC_TRY(load_norm(c, v.get(), at + "group_norm", &v->attn_norm));
    CMFC_TRY(load_conv(c, v.get(), at + "to_q", &v->attn_q));
    CMFC_TRY(load_conv(c, v.get(), at + "to_k", &v->attn_k));
    CMFC_TRY(load_conv(c, v.get(), at + "to_v", &v->attn_v));
    CMFC_TRY(load_conv(c, v.get(), at + "to_out.0", &v->attn_o));
    v->attn_c = v->attn_q.oc;
    if (v->attn_q.taps != 1 || v->attn_q.ic != v->attn_c || v->attn_norm.c != v->attn_c || v->attn_c % 32)
        return fail(ERR_SHAPE, "vae: attention projections must be square linears over a multiple of 32 channels");
    CMFC_TRY(load_resnet(c, v.get(), dec + "mid_block.resnets.1", &v->mid2));
    for (int b = 0;; ++b) {
        const std::string ub = dec + "up_blocks." + std::to_string(b);
        if (find(m, ub + ".resnets.0.conv1.weight") < 0) break;
        v->ups.emplace_back();
        for (int r = 0;; ++r) {
            const std::string rn = ub + ".resnets." + std::to_string(r);
            if (find(m, rn + ".conv1.weight") < 0) break;
            v->ups.back().res.emplace_back();
            CMFC_TRY(load_resnet(c, v.get(), rn, &v->ups.back().res.back()));
        }
        const std::string un = ub + ".upsamplers.0.conv";
        v->ups.back().has_up = find(m, un + ".weight") >= 0;
        if (v->ups.back().has_up) CMFC_TRY(load_conv(c, v.get(), un, &v->ups.back().up));
    }
    CMFC_TRY(load_norm(c, v.get(), dec + "conv_norm_out", &v->norm_out));
    CMFC_TRY(load_conv(c, v.get(), dec + "conv_out", &v->conv_out));
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    cleanup.armed = false;
    *out = v.release();
    return OK;
}

extern "C" void cmfc_vae_destroy(cmfc_vae* v) {
    if (!v) return;
    for (void* p : v->owned) cudaFree(p);
    delete v;
}

extern "C" int cmfc_vae_info(const cmfc_vae* v, uint32_t* latent_channels, uint32_t* upscale, float* scaling_factor,
                             float* shift_factor) {
    NEED(v, "vae_info: null argument");
    if (latent_channels) *latent_channels = (uint32_t)v->latent_channels;
    if (upscale) *upscale = (uint32_t)v->upscale();
    if (scaling_factor) *scaling_factor = v->scaling;
    if (shift_factor) *shift_factor = v->shift;
    return OK;
}

extern "C" int cmfc_vae_decode(cmfc_vae* v, const float* z, size_t h, size_t w, float* out) {
    CMFC_TRY(check_decode_args(v, z, h, w, out));
    NEED_CTX();
    const Sizes sz = plan(v, (int)h, (int)w);
    const size_t zin = (size_t)v->latent_channels * h * w * 4, zout = (size_t)v->conv_out.oc * sz.out_h * sz.out_w * 4;
    DevBuf &bz = c->buf("vae.z"), &bo = c->buf("vae.out");
    CMFC_TRY(bz.ensure(zin));
    CMFC_TRY(bo.ensure(zout));
    CMFC_CUDA(cudaMemcpyAsync(bz.p, z, zin, cudaMemcpyHostToDevice, c->stream));
    CMFC_TRY(decode_device(c, v, bz.as<float>(), (int)h, (int)w, bo.as<float>()));
    CMFC_CUDA(cudaMemcpyAsync(out, bo.p, zout, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "vae_decode");
}

extern "C" int cmfc_vae_decode_device(cmfc_vae* v, const float* d_z, size_t h, size_t w, float* d_out) {
    CMFC_TRY(check_decode_args(v, d_z, h, w, d_out));
    NEED_CTX();
    CMFC_TRY(decode_device(c, v, d_z, (int)h, (int)w, d_out));
    return check_status(c, "vae_decode_device");
}

// conv2d (and nearest-2x upsample + conv2d) on host NCHW tensors: the facade's vae_conv2d /
// vae_upsample_conv (crates/cortiq-engine/src/gpu.rs:2002-2060)
static int host_conv(const float* w, const float* bias, const float* x, size_t ic, size_t oc, size_t h, size_t w_img,
                     size_t k, int upsample, float* out) {
    NEED(w && bias && x && out, "vae_conv2d: null argument");
    NEED(ic > 0 && oc > 0 && h > 0 && w_img > 0 && (k == 1 || k == 3), "vae_conv2d: empty input or unsupported kernel size");
    NEED(h <= 8192 && w_img <= 8192 && ic <= 65536 && oc <= 65536, "vae_conv2d: extent out of range");
    NEED_CTX();
    const int taps = (int)(k * k), ic_pad = round_up((int)ic, 32);
    const size_t pix_in = h * w_img, oh = upsample ? 2 * h : h, ow = upsample ? 2 * w_img : w_img, pix_out = oh * ow;
    DevBuf &bw = c->buf("vc.w"), &bb = c->buf("vc.b"), &bx = c->buf("vc.x"), &bs = c->buf("vc.s"), &bn = c->buf("vc.n"),
           &bo = c->buf("vc.o");
    CMFC_TRY(bw.ensure(oc * ic * taps * 4));
    CMFC_TRY(bb.ensure(oc * 4));
    CMFC_TRY(bx.ensure(ic * pix_in * 4));
    CMFC_TRY(bs.ensure(pix_out * ic_pad * 4));
    CMFC_TRY(bo.ensure(oc * pix_out * 4));
    CMFC_CUDA(cudaMemcpyAsync(bw.p, w, oc * ic * taps * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(bb.p, bias, oc * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(bx.p, x, ic * pix_in * 4, cudaMemcpyHostToDevice, c->stream));
    std::vector<void*> owned;
    struct Free {
        std::vector<void*>& o;
        cudaStream_t s;
        ~Free() {
            cudaStreamSynchronize(s);
            for (void* p : o) cudaFree(p);
        }
    } guard{owned, c->stream};
    ConvW cw;
    CMFC_TRY(build_conv(c, owned, bw.as<float>(), bb.as<float>(), (int)oc, (int)ic, taps, false, &cw));
    const Planes s{bs.as<__half>(), bs.as<__half>() + pix_out * ic_pad};
    if (upsample) {
        if (ic % 4) return fail(ERR_SHAPE, "vae_upsample_conv: input channels must be a multiple of 4");
        CMFC_TRY(bn.ensure(pix_in * ic_pad * 4));
        CMFC_CUDA(cudaMemsetAsync(bn.p, 0, pix_in * ic_pad * 4, c->stream));
        if ((int)ic == ic_pad) {
            launch_nchw_to_nhwc(bx.as<float>(), pix_in, (int)ic, bn.as<float>(), c->stream);
        } else {
            return fail(ERR_SHAPE, "vae_upsample_conv: input channels must be a multiple of 32");
        }
        launch_upsample2x_split(bn.as<float>(), (int)h, (int)w_img, ic_pad, s.hi, s.lo, c->stream);
        c->launches += 2;
    } else {
        launch_nchw_to_split(bx.as<float>(), (int)ic, pix_in, ic_pad, 1.0f, 0.0f, 0, s.hi, s.lo, c->stream);
        c->launches++;
    }
    CMFC_CUDA(cudaGetLastError());
    ConvOut o;
    o.f32 = bo.as<float>();
    o.channel_major = 1;
    CMFC_TRY(run_conv(c, cw, s, ic_pad, (int)ow, (int)oh, o));
    CMFC_CUDA(cudaMemcpyAsync(out, bo.p, oc * pix_out * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "vae_conv2d");
}

extern "C" int cmfc_vae_conv2d(const float* w, const float* bias, const float* x, size_t ic, size_t oc, size_t h,
                               size_t w_img, size_t k, float* out) {
    return host_conv(w, bias, x, ic, oc, h, w_img, k, 0, out);
}

extern "C" int cmfc_vae_upsample_conv(const float* w, const float* bias, const float* x, size_t ic, size_t oc, size_t h,
                                      size_t w_img, size_t k, float* out) {
    return host_conv(w, bias, x, ic, oc, h, w_img, k, 1, out);
}

// ---- instrumentation: device-resident timings on synthetic inputs (CUDA events on the stream) ----

extern "C" int cmfc_bench_vae_decode(cmfc_vae* v, size_t h, size_t w, int iters, float* ms_per_decode) {
    NEED(v && ms_per_decode && iters > 0 && h > 0 && w > 0 && h <= 4096 && w <= 4096, "bench_vae_decode: bad argument");
    NEED_CTX();
    const Sizes sz = plan(v, (int)h, (int)w);
    DevBuf &bz = c->buf("vae.z"), &bo = c->buf("vae.out");
    CMFC_TRY(bz.ensure((size_t)v->latent_channels * h * w * 4));
    CMFC_TRY(bo.ensure((size_t)v->conv_out.oc * sz.out_h * sz.out_w * 4));
    launch_fill_normal(bz.as<float>(), (size_t)v->latent_channels * h * w, 21, 1.0f, c->stream);
    c->launches++;
    CMFC_TRY(decode_device(c, v, bz.as<float>(), (int)h, (int)w, bo.as<float>()));
    cudaEvent_t e0, e1;
    CMFC_CUDA(cudaEventCreate(&e0));
    CMFC_CUDA(cudaEventCreate(&e1));
    CMFC_CUDA(cudaEventRecord(e0, c->stream));
    for (int i = 0; i < iters; ++i) CMFC_TRY(decode_device(c, v, bz.as<float>(), (int)h, (int)w, bo.as<float>()));
    CMFC_CUDA(cudaEventRecord(e1, c->stream));
    CMFC_CUDA(cudaEventSynchronize(e1));
    float ms = 0;
    CMFC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms_per_decode = ms / iters;
    return check_status(c, "bench_vae_decode");
}

// one convolution ic -> oc (k x k) over an h x w image of synthetic split planes; a_planes 1 (f16
// weights) or 2 (f32 weights)
extern "C" int cmfc_bench_conv(size_t ic, size_t oc, size_t h, size_t w, size_t k, int a_planes, int iters,
                               float* ms_per_launch) {
    NEED(ms_per_launch && iters > 0 && ic && oc && h && w && (k == 1 || k == 3) && (a_planes == 1 || a_planes == 2),
         "bench_conv: bad argument");
    NEED(ic % 32 == 0 && h <= 8192 && w <= 8192, "bench_conv: ic must be a multiple of 32");
    NEED_CTX();
    const size_t pix = h * w, taps = k * k;
    DevBuf &bw = c->buf("bc.w"), &bb = c->buf("bc.b"), &bx = c->buf("bc.x"), &bs = c->buf("bc.s"), &bo = c->buf("bc.o");
    CMFC_TRY(bw.ensure(oc * ic * taps * 4));
    CMFC_TRY(bb.ensure(oc * 4));
    CMFC_TRY(bx.ensure(pix * ic * 4));
    CMFC_TRY(bs.ensure(pix * ic * 4));
    CMFC_TRY(bo.ensure(pix * oc * 4));
    launch_fill_normal(bw.as<float>(), oc * ic * taps, 31, 1.0f / sqrtf((float)(ic * taps)), c->stream);
    launch_fill_normal(bb.as<float>(), oc, 32, 1.0f, c->stream);
    launch_fill_normal(bx.as<float>(), pix * ic, 33, 1.0f, c->stream);
    const Planes s{bs.as<__half>(), bs.as<__half>() + pix * ic};
    launch_split_f32(bx.as<float>(), pix * ic, s.hi, s.lo, c->stream);
    c->launches += 4;
    std::vector<void*> owned;
    struct Free {
        std::vector<void*>& o;
        cudaStream_t s;
        ~Free() {
            cudaStreamSynchronize(s);
            for (void* p : o) cudaFree(p);
        }
    } guard{owned, c->stream};
    ConvW cw;
    CMFC_TRY(build_conv(c, owned, bw.as<float>(), bb.as<float>(), (int)oc, (int)ic, (int)taps, a_planes == 1, &cw));
    ConvOut o;
    o.f32 = bo.as<float>();
    for (int i = 0; i < 3; ++i) CMFC_TRY(run_conv(c, cw, s, (int)ic, (int)w, (int)h, o));
    cudaEvent_t e0, e1;
    CMFC_CUDA(cudaEventCreate(&e0));
    CMFC_CUDA(cudaEventCreate(&e1));
    CMFC_CUDA(cudaEventRecord(e0, c->stream));
    for (int i = 0; i < iters; ++i) CMFC_TRY(run_conv(c, cw, s, (int)ic, (int)w, (int)h, o));
    CMFC_CUDA(cudaEventRecord(e1, c->stream));
    CMFC_CUDA(cudaEventSynchronize(e1));
    float ms = 0;
    CMFC_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    *ms_per_launch = ms / iters;
    return check_status(c, "bench_conv");
}

// gpu::dit_attention as the VAE's attention block calls it (crates/cortiq-engine/src/vae.rs:438:
// one head, head dimension = channels = 512): host q, k, v [n, c] f32 -> out [n, c] f32 through the
// split-f16 GEMMs and the materialised score plane.  Reached from cmfc_dit_attention when the head
// dimension exceeds the flash kernel's 128.
namespace cmfc {
int attention_single_head_wide(const float* q, const float* k, const float* v, size_t n, size_t c_dim, float scale,
                               float* out) {
    Context* c = ctx();
    if (!c) return last_error().empty() ? fail(ERR_CUDA, "no CUDA device") : ERR_CUDA;
    if (c_dim % 32 || c_dim > 4096) return fail(ERR_SHAPE, "dit_attention: a head wider than 128 must be a multiple of 32 (<= 4096)");
    if (n > 131072) return fail(ERR_SHAPE, "dit_attention: wide-head path materialises n x n scores (n <= 131072)");
    const int ch = (int)c_dim, nn = (int)n, n_pad = round_up(nn, 32);
    const size_t tok = n * c_dim;
    DevBuf &bin = c->buf("wa.in"), &bq = c->buf("wa.q"), &bk = c->buf("wa.k"), &bvt = c->buf("wa.vt"), &bs = c->buf("wa.s"),
           &bp = c->buf("wa.p"), &bo = c->buf("wa.o");
    CMFC_TRY(bin.ensure(3 * tok * 4));
    CMFC_TRY(bq.ensure(tok * 4));
    CMFC_TRY(bk.ensure(tok * 4));
    CMFC_TRY(bvt.ensure((size_t)ch * n_pad * 4));
    CMFC_TRY(bs.ensure(n * (size_t)n_pad * 4));
    CMFC_TRY(bp.ensure(n * (size_t)n_pad * 4));
    CMFC_TRY(bo.ensure(tok * 4));
    float* d_in = bin.as<float>();
    CMFC_CUDA(cudaMemcpyAsync(d_in, q, tok * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(d_in + tok, k, tok * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaMemcpyAsync(d_in + 2 * tok, v, tok * 4, cudaMemcpyHostToDevice, c->stream));
    const Planes qp{bq.as<__half>(), bq.as<__half>() + tok}, kp{bk.as<__half>(), bk.as<__half>() + tok};
    const Planes vt{bvt.as<__half>(), bvt.as<__half>() + (size_t)ch * n_pad};
    const Planes pr{bp.as<__half>(), bp.as<__half>() + n * (size_t)n_pad};
    launch_split_f32(d_in, tok, qp.hi, qp.lo, c->stream);
    launch_split_f32(d_in + tok, tok, kp.hi, kp.lo, c->stream);
    // V [n, c] -> V^T split planes [c, n_pad]: the transpose kernel reads "NCHW" = [rows, pixels]
    CMFC_CUDA(cudaMemsetAsync(bvt.p, 0, (size_t)ch * n_pad * 4, c->stream));
    {
        DevBuf& bt = c->buf("wa.t");
        CMFC_TRY(bt.ensure(tok * 4));
        launch_nhwc_to_nchw(d_in + 2 * tok, n, ch, bt.as<float>(), c->stream);   // [n, c] -> [c, n]
        if (n_pad == nn) {
            launch_split_f32(bt.as<float>(), tok, vt.hi, vt.lo, c->stream);
        } else {
            for (int r = 0; r < ch; ++r)  // ragged pitch: row by row (small c)
                launch_split_f32(bt.as<float>() + (size_t)r * n, n, vt.hi + (size_t)r * n_pad, vt.lo + (size_t)r * n_pad, c->stream);
        }
    }
    CMFC_CUDA(cudaGetLastError());
    c->launches += 4;
    CUtensorMap tk_hi, tk_lo, tv_hi, tv_lo;
    CMFC_TRY(make_tensor_map_2d(&tk_hi, kp.hi, 2, n, ch, (uint64_t)ch * 2, 128, 32, 2));
    CMFC_TRY(make_tensor_map_2d(&tk_lo, kp.lo, 2, n, ch, (uint64_t)ch * 2, 128, 32, 2));
    ConvOut os; os.f32 = bs.as<float>(); os.pitch = n_pad; os.scale = scale;
    CMFC_TRY(run_gemm(c, tk_hi, tk_lo, 2, nn, ch, 1, nullptr, qp, 2, ch, ch, nn, 1, os));
    CMFC_TRY(launch_softmax_rows_split(bs.as<float>(), n, nn, (size_t)n_pad, pr.hi, pr.lo, (size_t)n_pad, c->stream));
    c->launches++;
    CMFC_TRY(make_tensor_map_2d(&tv_hi, vt.hi, 2, ch, n, (uint64_t)n_pad * 2, 128, 32, 2));
    CMFC_TRY(make_tensor_map_2d(&tv_lo, vt.lo, 2, ch, n, (uint64_t)n_pad * 2, 128, 32, 2));
    ConvOut oo; oo.f32 = bo.as<float>();
    CMFC_TRY(run_gemm(c, tv_hi, tv_lo, 2, ch, n_pad, 1, nullptr, pr, 2, nn, n_pad, nn, 1, oo));
    CMFC_CUDA(cudaMemcpyAsync(out, bo.p, tok * 4, cudaMemcpyDeviceToHost, c->stream));
    return check_status(c, "dit_attention");
}
}  // namespace cmfc
