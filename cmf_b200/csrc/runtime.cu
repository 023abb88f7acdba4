// Host runtime: errors, device contexts, the memory-mapped container reader, weight upload
// into kernel planes, and the device-level block composed from the kernels.
#include <algorithm>

#include "runtime.h"

#include <fcntl.h>
#include <math.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>

namespace cmfc {

// ---------------- errors ----------------
static thread_local std::string g_last_error;
void set_error(const std::string& msg) { g_last_error = msg; }
const std::string& last_error() { return g_last_error; }
int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

// ---------------- tensor maps ----------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

int make_tensor_map_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                       uint64_t pitch_bytes, uint32_t box_rows, uint32_t box_cols, int swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                             : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapSwizzle sw = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B
                            : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                           : CU_TENSOR_MAP_SWIZZLE_NONE;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15))
        return fail(ERR_BAD_ARG, "tensor map base and pitch must be 16-byte aligned");
    CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
    return OK;
}

// 3-D tiled map over an NHWC plane of 2-byte elements: dims (channels, width, height), box
// (box_c, box_w, box_h); out-of-range coordinates read as zero.  swizzle as in make_tensor_map_2d.
int make_tensor_map_nhwc16(CUtensorMap* out, const void* base, uint64_t channels, uint64_t width, uint64_t height,
                           uint64_t pixel_pitch_bytes, uint32_t box_c, uint32_t box_w, uint32_t box_h, int swizzle) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {channels, width, height};
    cuuint64_t strides[2] = {pixel_pitch_bytes, pixel_pitch_bytes * width};
    cuuint32_t box[3] = {box_c, box_w, box_h};
    cuuint32_t estr[3] = {1, 1, 1};
    CUtensorMapSwizzle sw = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B
                            : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B
                                           : CU_TENSOR_MAP_SWIZZLE_NONE;
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pixel_pitch_bytes & 15))
        return fail(ERR_BAD_ARG, "tensor map base and pitch must be 16-byte aligned");
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(ERR_CUDA, "cuTensorMapEncodeTiled (3-D) failed with code " + std::to_string((int)r));
    return OK;
}

// ---------------- buffers ----------------
static std::atomic<uint64_t> g_alloc_epoch{1};
uint64_t alloc_epoch() { return g_alloc_epoch.load(); }

int DevBuf::ensure(size_t bytes) {
    if (bytes <= cap && p) return OK;
    g_alloc_epoch++;
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
    size_t want = (bytes + 255) & ~size_t(255);
    cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
        p = nullptr;
        return fail(ERR_OOM, std::string("cudaMalloc of ") + std::to_string(want) + " bytes: " + cudaGetErrorString(e));
    }
    cap = want;
    return OK;
}
void DevBuf::release() {
    if (p) g_alloc_epoch++;
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
}

// ---------------- contexts ----------------
static std::mutex g_ctx_mu;
// never destroyed: at process exit the CUDA runtime may already be gone, and the contexts' device
// memory goes with the process anyway
static std::map<int, std::unique_ptr<Context>>& g_ctxs = *new std::map<int, std::unique_ptr<Context>>();
static thread_local int g_cur_device = -1;

int ctx_set_device(int device) {
    int count = 0;
    CMFC_CUDA(cudaGetDeviceCount(&count));
    if (device < 0 || device >= count) return fail(ERR_BAD_ARG, "no such CUDA device " + std::to_string(device));
    CMFC_CUDA(cudaSetDevice(device));
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    if (!g_ctxs.count(device)) {
        cudaDeviceProp prop;
        CMFC_CUDA(cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10)
            return fail(ERR_UNSUPPORTED, std::string("this library is built for sm_100a only; device is ") + prop.name +
                                             " (sm_" + std::to_string(prop.major) + std::to_string(prop.minor) + ")");
        std::unique_ptr<Context> c(new Context());
        c->device = device;
        c->num_sms = prop.multiProcessorCount;
        CMFC_CUDA(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
        c->main_stream = c->stream;
        CMFC_CUDA(cudaStreamCreateWithFlags(&c->side_stream, cudaStreamNonBlocking));
        CMFC_CUDA(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
        CMFC_CUDA(cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
        CMFC_CUDA(cudaMalloc(&c->status, 4));
        CMFC_CUDA(cudaMemset(c->status, 0, 4));
        CMFC_CUDA(cudaMallocHost(&c->status_host, 4));
        CMFC_CUDA(cudaMalloc(&c->sched, (2 * Context::MAX_STEPS + 1) * 4));
        CMFC_CUDA(cudaMemset(c->sched, 0, (2 * Context::MAX_STEPS + 1) * 4));
        c->step_counter = reinterpret_cast<int*>(c->sched + 2 * Context::MAX_STEPS);
        CMFC_CUDA(cudaMallocHost(&c->sched_host, (2 * Context::MAX_STEPS + 1) * 4));
        // log2f / exp2f of every half-precision value, from the host's libm: the device
        // quantizer must land on the bits the CPU encoder computes.
        std::vector<float> l2(65536), e2(65536);
        for (uint32_t h = 0; h < 65536; ++h) {
            uint32_t s = (h >> 15) << 31, e = (h >> 10) & 0x1F, m = h & 0x3FF, bits;
            if (e == 0) {
                if (!m) bits = s;
                else {
                    uint32_t sh = 0;
                    while (!(m & 0x400)) { m <<= 1; ++sh; }
                    bits = s | ((113 - sh) << 23) | ((m & 0x3FF) << 13);
                }
            } else if (e == 0x1F) bits = s | 0x7F800000u | (m << 13);
            else bits = s | ((e + 112) << 23) | (m << 13);
            float f;
            memcpy(&f, &bits, 4);
            l2[h] = log2f(f);
            e2[h] = exp2f(f);
        }
        CMFC_CUDA(cudaMalloc(&c->log2_lut, 65536 * 4));
        CMFC_CUDA(cudaMalloc(&c->exp2_lut, 65536 * 4));
        CMFC_CUDA(cudaMemcpy(c->log2_lut, l2.data(), 65536 * 4, cudaMemcpyHostToDevice));
        CMFC_CUDA(cudaMemcpy(c->exp2_lut, e2.data(), 65536 * 4, cudaMemcpyHostToDevice));
        CMFC_CUDA(cudaStreamSynchronize(0));  // readers run on c->stream, not ordered after the legacy stream
        g_ctxs[device] = std::move(c);
    }
    g_cur_device = device;
    return OK;
}

Context* ctx() {
    if (g_cur_device < 0) {
        if (ctx_set_device(0) != OK) return nullptr;
    } else {
        cudaSetDevice(g_cur_device);
    }
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    auto it = g_ctxs.find(g_cur_device);
    return it == g_ctxs.end() ? nullptr : it->second.get();
}

Context* ctx_existing() {
    if (g_cur_device < 0) return nullptr;
    cudaSetDevice(g_cur_device);
    std::lock_guard<std::mutex> lk(g_ctx_mu);
    auto it = g_ctxs.find(g_cur_device);
    return it == g_ctxs.end() ? nullptr : it->second.get();
}

int check_status(Context* c, const char* what) {
    CMFC_CUDA(cudaMemcpyAsync(c->status_host, c->status, 4, cudaMemcpyDeviceToHost, c->stream));
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    if (*c->status_host) {
        uint32_t v = *c->status_host;
        cudaMemsetAsync(c->status, 0, 4, c->stream);
        return fail(ERR_DEVICE_WAIT, std::string(what) + ": a kernel gave up a bounded wait (site " + std::to_string(v) + ")");
    }
    return OK;
}

SpanGuard::SpanGuard(Context* c_, const char* name) : c(c_) {
    if (!c->prof.on) return;
    cudaEvent_t a, b;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    cudaEventRecord(a, c->stream);
    idx = c->prof.spans.size();
    c->prof.spans.push_back({name, {a, b}});
}
SpanGuard::~SpanGuard() {
    if (idx != (size_t)-1) cudaEventRecord(c->prof.spans[idx].second.second, c->stream);
}

// ---------------- container ----------------
// 64-bit content hash of the container format (crates/cortiq-core/src/hash.rs:8-36): every
// little-endian u64 word goes through the murmur3 finalizer, is XOR-ed with its index times the
// golden-ratio constant, all are XOR-reduced, the byte length is mixed in and finalized again.
static inline uint64_t fmix64(uint64_t x) {
    x ^= x >> 33;
    x *= 0xFF51AFD7ED558CCDull;
    x ^= x >> 33;
    x *= 0xC4CEB9FE1A85EC53ull;
    x ^= x >> 33;
    return x;
}
uint64_t hash64(const uint8_t* p, size_t n) {
    uint64_t h = 0;
    size_t words = (n + 7) / 8;
    for (size_t i = 0; i < words; ++i) {
        uint64_t w = 0;
        size_t take = (i * 8 + 8 <= n) ? 8 : n - i * 8;
        memcpy(&w, p + i * 8, take);
        h ^= fmix64(w) ^ (i * 0x9E3779B97F4A7C15ull);
    }
    h ^= (uint64_t)n;
    return fmix64(h);
}

size_t payload_nbytes(int dtype, size_t rows, size_t cols) {
    switch (dtype) {
        case DT_F32: return rows * cols * 4;
        case DT_F16: return rows * cols * 2;
        case DT_U8: return rows * cols;
        case DT_Q8: return rows * cols + rows * 2;
        case DT_Q4T: return ((rows * cols + 31) / 32) * 18;
        case DT_Q4TP: {
            size_t gpr = cols / 32;
            return rows * gpr * 16 + rows * 4 + rows * ((gpr * 5 + 7) / 8);
        }
        default: return 0;
    }
}

static std::atomic<uint64_t> g_next_uid{1};

template <class T> static T rd(const uint8_t* p) {
    T v;
    memcpy(&v, p, sizeof(T));
    return v;
}

int model_open(const char* path, Model** out) {
    if (!path || !out) return fail(ERR_BAD_ARG, "model_open: null argument");
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(ERR_IO, std::string("cannot open ") + path);
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 128) {
        close(fd);
        return fail(ERR_FORMAT, std::string(path) + ": shorter than the 128-byte envelope");
    }
    void* mp = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (mp == MAP_FAILED) return fail(ERR_IO, std::string("mmap failed for ") + path);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(mp);
    const size_t len = (size_t)st.st_size;
    auto bad = [&](const std::string& why) {
        munmap(mp, len);
        return fail(ERR_FORMAT, std::string(path) + ": " + why);
    };
    if (memcmp(b, "CMF\x01", 4) != 0) return bad("bad magic");
    if (rd<uint32_t>(b + 4) != 2) return bad("unsupported container version");
    // Only bit 0 (the tensor directory) is implemented here; a file that REQUIRES binary masks
    // (bit 1) or the two-factor quantization (bit 2) must be refused, not run with them ignored
    // (crates/cortiq-core/src/format.rs:700-712 refuses what it does not understand).
    const uint32_t required = rd<uint32_t>(b + 12);
    if (required & ~0x1u) return bad("required feature bits " + std::to_string(required) + " are not supported by this backend");
    const uint64_t hdr_off = rd<uint64_t>(b + 0x10), hdr_len = rd<uint64_t>(b + 0x18);
    const uint64_t dir_off = rd<uint64_t>(b + 0x20), dir_len = rd<uint64_t>(b + 0x28);
    const uint64_t data_off = rd<uint64_t>(b + 0x30), data_len = rd<uint64_t>(b + 0x38);
    // offsets and lengths come from an untrusted file: compare without forming off + len, which wraps
    auto inside = [](uint64_t off, uint64_t n, uint64_t total) { return n <= total && off <= total - n; };
    if (!inside(hdr_off, hdr_len, len) || !inside(dir_off, dir_len, len) || !inside(data_off, data_len, len) || dir_len < 16)
        return bad("section outside the file");
    if (data_off % 4096) return bad("data section is not 4096-aligned");
    if (rd<uint64_t>(b + 0x70) != hash64(b + hdr_off, hdr_len)) return bad("header hash mismatch");
    const uint64_t dir_hash = rd<uint64_t>(b + 0x78);
    if (dir_hash && dir_hash != hash64(b + dir_off, dir_len)) return bad("directory hash mismatch");
    const uint8_t* d = b + dir_off;
    const uint64_t count = rd<uint64_t>(d), pool_off = rd<uint64_t>(d + 8);
    if (count > (dir_len - 16) / 56 || pool_off > dir_len) return bad("directory records overrun the section");
    std::unique_ptr<Model> m(new Model());
    m->uid = g_next_uid++;
    m->path = path;
    m->map = b;
    m->map_len = len;
    m->data_off = data_off;
    m->recs.resize(count);
    for (uint64_t i = 0; i < count; ++i) {
        const uint8_t* r = d + 16 + i * 56;
        TensorRec& t = m->recs[i];
        const uint32_t noff = rd<uint32_t>(r);
        const uint16_t nlen = rd<uint16_t>(r + 4);
        t.dtype = r[6];
        t.ndim = r[7];
        if (t.ndim > 6) return bad("tensor rank above 6");
        for (int k = 0; k < 6; ++k) t.shape[k] = rd<uint32_t>(r + 8 + 4 * k);
        t.off = rd<uint64_t>(r + 32);
        t.nbytes = rd<uint64_t>(r + 40);
        t.hash = rd<uint64_t>(r + 48);
        if (!inside((uint64_t)noff, (uint64_t)nlen, dir_len - pool_off)) return bad("tensor name outside the name pool");
        t.name.assign(reinterpret_cast<const char*>(d + pool_off + noff), nlen);
        if (t.off % 64) return bad("tensor " + t.name + " is not 64-byte aligned");
        if (!inside(t.off, t.nbytes, data_len)) return bad("tensor " + t.name + " runs past the data section");
        if (t.ndim == 2) {
            size_t want = payload_nbytes(t.dtype, t.shape[0], t.shape[1]);
            if (want && want != t.nbytes) return bad("tensor " + t.name + ": byte count disagrees with dtype and shape");
        }
        m->by_name[t.name] = (int64_t)i;
    }
    *out = m.release();
    return OK;
}

void model_close(Model* m) {
    if (!m) return;
    {
        std::lock_guard<std::mutex> lk(g_ctx_mu);
        // the caller's current device (torch's, in a one-process multi-GPU host) is left as found
        int caller_dev = -1;
        const bool have_dev = cudaGetDevice(&caller_dev) == cudaSuccess;
        for (auto& kv : g_ctxs) {
            Context* c = kv.second.get();
            cudaSetDevice(c->device);
            cudaStreamSynchronize(c->stream);
            for (auto it = c->weights.begin(); it != c->weights.end();) {
                if (std::get<0>(it->first) == m->uid) it = c->weights.erase(it);  // ~DevWeight frees the planes
                else ++it;
            }
        }
        if (have_dev) cudaSetDevice(caller_dev);
    }
    munmap(const_cast<uint8_t*>(m->map), m->map_len);
    delete m;
}

// ---------------- weights ----------------
static uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
static float half_to_float_host(uint16_t h) {
    uint32_t s = (uint32_t)(h >> 15) << 31, e = (h >> 10) & 0x1F, m = h & 0x3FF, bits;
    if (e == 0) {
        if (!m) bits = s;
        else {
            uint32_t sh = 0;
            while (!(m & 0x400)) { m <<= 1; ++sh; }
            bits = s | ((113 - sh) << 23) | ((m & 0x3FF) << 13);
        }
    } else if (e == 0x1F) bits = s | 0x7F800000u | (m << 13);
    else bits = s | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
float half_bits_to_float(uint16_t h) { return half_to_float_host(h); }

static int finish_gemm_maps(DevWeight* w) {
    if (w->dtype == DT_F32) return OK;
    if (w->rows % 128 || w->cols % 64) return OK;  // usable by gemv / dequant only
    if (w->dtype == DT_Q8) {
        CMFC_TRY(make_tensor_map_2d(&w->tm_w, w->plane, 1, w->rows, w->cols, w->cols, 128, 64, 2));
        w->tm_s = w->tm_w;
    } else {
        CMFC_TRY(make_tensor_map_2d(&w->tm_w, w->plane, 1, w->rows, w->cols / 2, w->cols / 2, 128, 32, 1));
        CMFC_TRY(make_tensor_map_2d(&w->tm_s, w->scales, 4, w->cols / 32, w->rows, (uint64_t)w->rows * 4, 2, 128, 0));
    }
    w->gemm_ready = true;
    return OK;
}

// Planes are freed on the device that is current: weights live in a context's map and are dropped
// either by model_close (which selects the context's device first) or on a failed upload (the
// uploading thread's device).
DevWeight::~DevWeight() {
    if (!owns) return;
    if (plane) cudaFree(plane);
    if (scales) cudaFree(scales);
}

static int alloc_planes(DevWeight* w) {
    size_t plane_b, scale_b;
    if (w->dtype == DT_Q8) { plane_b = (size_t)w->rows * w->cols; scale_b = (size_t)w->rows * 4; }
    else if (w->is_q4()) { plane_b = (size_t)w->rows * w->cols / 2; scale_b = (size_t)w->rows * (w->cols / 32) * 4; }
    else { plane_b = (size_t)w->rows * w->cols * 4; scale_b = 0; }
    if (cudaMalloc(&w->plane, plane_b) != cudaSuccess) return fail(ERR_OOM, "out of device memory for a weight plane");
    if (scale_b && cudaMalloc(&w->scales, scale_b) != cudaSuccess) return fail(ERR_OOM, "out of device memory for weight scales");
    w->bytes = plane_b + scale_b;
    return OK;
}

int get_weight(Context* c, Model* m, int64_t idx, DevWeight** out) {
    if (!m || idx < 0 || idx >= (int64_t)m->recs.size()) return fail(ERR_BAD_ARG, "tensor index out of range");
    auto key = std::make_tuple(m->uid, idx, (int64_t)-1, (int64_t)-1, 0);
    auto it = c->weights.find(key);
    if (it != c->weights.end()) { *out = it->second.get(); return OK; }
    const TensorRec& t = m->recs[idx];
    if (t.ndim != 2) return fail(ERR_SHAPE, "tensor " + t.name + " is not 2-D");
    if (t.dtype != DT_Q8 && t.dtype != DT_Q4T && t.dtype != DT_Q4TP)
        return fail(ERR_UNSUPPORTED, "tensor " + t.name + ": dtype " + std::to_string(t.dtype) + " is not q8_row / q4_tiled / q4tp");
    const int rows = (int)t.shape[0], cols = (int)t.shape[1];
    if (t.dtype != DT_Q8 && cols % 32) return fail(ERR_SHAPE, "tensor " + t.name + ": 4-bit codecs need cols % 32 == 0");
    if (cols % 16) return fail(ERR_SHAPE, "tensor " + t.name + ": cols must be a multiple of 16");
    std::unique_ptr<DevWeight> w(new DevWeight());
    w->dtype = t.dtype; w->rows = rows; w->cols = cols;
    CMFC_TRY(alloc_planes(w.get()));
    const uint8_t* src = m->bytes(idx);
    cudaStream_t s = c->stream;
    if (t.dtype == DT_Q8) {
        CMFC_CUDA(cudaMemcpyAsync(w->plane, src, (size_t)rows * cols, cudaMemcpyHostToDevice, s));
        std::vector<float> sc(rows);
        for (int r = 0; r < rows; ++r) sc[r] = half_to_float_host(rd16(src + (size_t)rows * cols + 2 * r));
        CMFC_CUDA(cudaMemcpyAsync(w->scales, sc.data(), (size_t)rows * 4, cudaMemcpyHostToDevice, s));
        CMFC_CUDA(cudaStreamSynchronize(s));
    } else if (t.dtype == DT_Q4T) {
        DevBuf& raw = c->buf("upload_raw");
        CMFC_TRY(raw.ensure(t.nbytes));
        CMFC_CUDA(cudaMemcpyAsync(raw.p, src, t.nbytes, cudaMemcpyHostToDevice, s));
        launch_q4t_split(raw.as<uint8_t>(), rows, cols, w->plane, w->scales, s);
        c->launches++;
        CMFC_CUDA(cudaStreamSynchronize(s));
    } else {
        const int gpr = cols / 32, stride = (gpr * 5 + 7) / 8;
        const size_t nib_b = (size_t)rows * gpr * 16;
        CMFC_CUDA(cudaMemcpyAsync(w->plane, src, nib_b, cudaMemcpyHostToDevice, s));
        // Ladders on the host, with the host's exp2f, iterated exactly as the format defines
        // (crates/cortiq-core/src/quant.rs:396-411).
        std::vector<float> lad((size_t)rows * 32);
        const uint8_t* params = src + nib_b;
        for (int r = 0; r < rows; ++r) {
            const float lo = half_to_float_host(rd16(params + 4 * r)), st = half_to_float_host(rd16(params + 4 * r + 2));
            const float ratio = exp2f(st);
            float tv = exp2f(lo);
            lad[(size_t)r * 32] = tv;
            for (int k = 1; k < 32; ++k) {
                volatile float nx = tv * ratio;  // plain IEEE multiply, never contracted
                tv = nx;
                lad[(size_t)r * 32 + k] = tv;
            }
        }
        DevBuf& raw = c->buf("upload_raw");
        const size_t codes_b = (size_t)rows * stride, lad_b = lad.size() * 4;
        CMFC_TRY(raw.ensure(((codes_b + 255) & ~size_t(255)) + lad_b));
        uint8_t* d_codes = raw.as<uint8_t>();
        float* d_lad = reinterpret_cast<float*>(d_codes + ((codes_b + 255) & ~size_t(255)));
        CMFC_CUDA(cudaMemcpyAsync(d_codes, params + (size_t)rows * 4, codes_b, cudaMemcpyHostToDevice, s));
        CMFC_CUDA(cudaMemcpyAsync(d_lad, lad.data(), lad_b, cudaMemcpyHostToDevice, s));
        launch_q4tp_scales(d_codes, stride, d_lad, rows, gpr, w->scales, s);
        launch_permute_plane(w->plane, nib_b, s);
        c->launches += 2;
        CMFC_CUDA(cudaStreamSynchronize(s));
    }
    CMFC_CUDA(cudaGetLastError());
    CMFC_TRY(finish_gemm_maps(w.get()));
    *out = w.get();
    c->weights[key] = std::move(w);
    return OK;
}

int upload_f32(Context* c, Model* m, int64_t idx, DevWeight** out) {
    if (!m || idx < 0 || idx >= (int64_t)m->recs.size()) return fail(ERR_BAD_ARG, "tensor index out of range");
    auto key = std::make_tuple(m->uid, idx, (int64_t)-1, (int64_t)-1, 9);
    auto it = c->weights.find(key);
    if (it != c->weights.end()) { *out = it->second.get(); return OK; }
    const TensorRec& t = m->recs[idx];
    size_t n = 1;
    for (int k = 0; k < t.ndim; ++k) n *= t.shape[k];
    std::unique_ptr<DevWeight> w(new DevWeight());
    w->dtype = DT_F32;
    w->rows = t.ndim == 2 ? (int)t.shape[0] : 1;
    w->cols = (int)(n / w->rows);
    if (cudaMalloc(&w->plane, n * 4) != cudaSuccess) return fail(ERR_OOM, "out of device memory for tensor " + t.name);
    w->bytes = n * 4;
    const uint8_t* src = m->bytes(idx);
    if (t.dtype == DT_F32) {
        if (t.nbytes != n * 4) return fail(ERR_SHAPE, "tensor " + t.name + ": byte count disagrees with shape");
        CMFC_CUDA(cudaMemcpy(w->plane, src, n * 4, cudaMemcpyHostToDevice));
    } else if (t.dtype == DT_F16) {
        std::vector<float> tmp(n);
        for (size_t i = 0; i < n; ++i) tmp[i] = half_to_float_host(rd16(src + 2 * i));
        CMFC_CUDA(cudaMemcpy(w->plane, tmp.data(), n * 4, cudaMemcpyHostToDevice));
    } else {
        return fail(ERR_UNSUPPORTED, "tensor " + t.name + ": expected f32 or f16, found dtype " + std::to_string(t.dtype));
    }
    // a copy from pageable memory may return before its DMA lands; readers run on c->stream,
    // which is not ordered after the legacy default stream
    CMFC_CUDA(cudaStreamSynchronize(0));
    *out = w.get();
    c->weights[key] = std::move(w);
    return OK;
}

// rows of a | b | cc stacked (all same dtype family and cols)
int get_weight_concat(Context* c, Model* m, int64_t a, int64_t b, int64_t cc, DevWeight** out) {
    auto key = std::make_tuple(m->uid, a, b, cc, 1);
    auto it = c->weights.find(key);
    if (it != c->weights.end()) { *out = it->second.get(); return OK; }
    DevWeight* parts[3] = {nullptr, nullptr, nullptr};
    CMFC_TRY(get_weight(c, m, a, &parts[0]));
    CMFC_TRY(get_weight(c, m, b, &parts[1]));
    CMFC_TRY(get_weight(c, m, cc, &parts[2]));
    const bool q4 = parts[0]->is_q4();
    int rows = 0;
    for (auto* p : parts) {
        // q4t and q4tp keep different scale formats on the device, so a fused view needs one codec
        if (p->cols != parts[0]->cols || p->dtype != parts[0]->dtype)
            return fail(ERR_UNSUPPORTED, "fused projection needs one codec and one input width");
        rows += p->rows;
    }
    std::unique_ptr<DevWeight> w(new DevWeight());
    w->dtype = parts[0]->dtype;
    w->rows = rows; w->cols = parts[0]->cols;
    CMFC_TRY(alloc_planes(w.get()));
    const size_t row_b = q4 ? w->cols / 2 : w->cols;
    size_t r0 = 0;
    for (auto* p : parts) {
        CMFC_CUDA(cudaMemcpyAsync(w->plane + r0 * row_b, p->plane, (size_t)p->rows * row_b, cudaMemcpyDeviceToDevice, c->stream));
        if (q4) {  // transposed scales [gpr, rows]: a column block per part
            CMFC_CUDA(cudaMemcpy2DAsync(w->scales + r0, (size_t)rows * 4, p->scales, (size_t)p->rows * 4, (size_t)p->rows * 4,
                                        w->cols / 32, cudaMemcpyDeviceToDevice, c->stream));
        } else {
            CMFC_CUDA(cudaMemcpyAsync(w->scales + r0, p->scales, (size_t)p->rows * 4, cudaMemcpyDeviceToDevice, c->stream));
        }
        r0 += p->rows;
    }
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    CMFC_TRY(finish_gemm_maps(w.get()));
    *out = w.get();
    c->weights[key] = std::move(w);
    return OK;
}

// rows alternate a[0], b[0], a[1], b[1], ... (gate / up of SwiGLU side by side in one tile)
int get_weight_interleaved(Context* c, Model* m, int64_t a, int64_t b, DevWeight** out) {
    auto key = std::make_tuple(m->uid, a, b, (int64_t)-1, 2);
    auto it = c->weights.find(key);
    if (it != c->weights.end()) { *out = it->second.get(); return OK; }
    DevWeight *pa = nullptr, *pb = nullptr;
    CMFC_TRY(get_weight(c, m, a, &pa));
    CMFC_TRY(get_weight(c, m, b, &pb));
    if (pa->rows != pb->rows || pa->cols != pb->cols || pa->dtype != pb->dtype)
        return fail(ERR_UNSUPPORTED, "SwiGLU gate and up projections must share shape and codec");
    const bool q4 = pa->is_q4();
    std::unique_ptr<DevWeight> w(new DevWeight());
    w->dtype = pa->dtype;
    w->rows = 2 * pa->rows; w->cols = pa->cols;
    CMFC_TRY(alloc_planes(w.get()));
    const size_t row_b = q4 ? w->cols / 2 : w->cols;
    DevWeight* parts[2] = {pa, pb};
    for (int k = 0; k < 2; ++k) {
        CMFC_CUDA(cudaMemcpy2DAsync(w->plane + k * row_b, 2 * row_b, parts[k]->plane, row_b, row_b, pa->rows,
                                    cudaMemcpyDeviceToDevice, c->stream));
        // scales: q8 [rows] -> stride 2 floats; q4 transposed [gpr, rows] -> every row of the
        // plane is itself interleaved, which is the same 4-byte element copy with pitch 8.
        const size_t count = q4 ? (size_t)pa->rows * (w->cols / 32) : (size_t)pa->rows;
        launch_interleave_f32(w->scales, 2, k, parts[k]->scales, count, c->stream);
    }
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    CMFC_TRY(finish_gemm_maps(w.get()));
    *out = w.get();
    c->weights[key] = std::move(w);
    return OK;
}

// ---------------- device-level ops ----------------
int dev_gemm(Context* c, DevWeight* w, const __nv_bfloat16* x, int M, void* out, int ldo, int mode, const GemmVt* vt) {
    if (!w->gemm_ready)
        return fail(ERR_SHAPE, "dequant GEMM needs rows % 128 == 0 and cols % 64 == 0 (got " + std::to_string(w->rows) +
                                   " x " + std::to_string(w->cols) + ")");
    GemmParams p;
    p.M = M; p.N = w->rows; p.K = w->cols;
    p.out = out; p.ldo = ldo; p.mode = mode;
    p.row_scale = w->dtype == DT_Q8 ? w->scales : nullptr;
    p.status = c->status;
    if (vt) {
        if (mode != GEMM_OUT_F32 || vt->row0 % 32 || vt->row0 > w->rows) return fail(ERR_BAD_ARG, "dev_gemm: bad V^T split");
        p.vt = vt->vt; p.vt_row0 = vt->row0; p.vt_pitch = vt->pitch; p.nseg = vt->nseg; p.seg_table = vt->seg_table;
    }
    const int wkind = w->dtype == DT_Q8 ? 0 : (w->dtype == DT_Q4TP ? 1 : 2);
    // CTA-pair kernel (2-SM MMA) whenever the weight rows tile by 256 and there is at least one
    // tile per pair of SMs; otherwise the single-CTA kernel.  CMFC_GEMM_PAIR=0 forces the latter.
    const char* pair_env = getenv("CMFC_GEMM_PAIR");  // read per call: tests flip it between calls
    const bool use_pair = !(pair_env && pair_env[0] == '0');
    const long pair_tiles = (long)((M + 255) / 256) * (w->rows / 256);
    const bool pair = use_pair && gemm_pair_supported(p) && pair_tiles >= c->num_sms / 2;
    // K split of a mostly empty last wave (pair kernel, f32 output).  Inside a NextDiT forward the
    // batch is a stack of equal prompts and the split is planned per prompt (c->gemm_period_tokens),
    // so a prompt's bits do not depend on its batch.  A launch without that structure is split only
    // on request: CMFC_GEMM_SPLITK=1 treats the whole launch as one period (its result then depends
    // on the token count in the last f32 bits), a value of 256 or more is the period in tokens.
    // CMFC_GEMM_SPLITK=0 turns the split off everywhere.
    if (pair && mode == GEMM_OUT_F32 && !vt) {
        const char* split_env = getenv("CMFC_GEMM_SPLITK");  // read per call: tests flip it between calls
        const int asked = split_env ? atoi(split_env) : -1;
        const bool off = asked == 0, force = asked == 1;
        int period = c->gemm_period_tokens > 0 && M % c->gemm_period_tokens == 0 ? c->gemm_period_tokens : 0;
        if (!period && asked >= 256 && M % asked == 0) period = asked;
        if (!off && (period > 0 || force)) {
            const size_t need = gemm_pair_splitk_bytes(p, c->num_sms, period);
            if (need) {
                DevBuf& ws = c->lane_buf("gemm_splitk");
                CMFC_TRY(ws.ensure(need));
                p.splitk_ws = ws.as<float>();
                p.split_period_tokens = period;
                c->launches++;  // the kernel that adds the slices
            }
        }
    }
    CUtensorMap tm_x;
    CMFC_TRY(make_tensor_map_2d(&tm_x, x, 2, (uint64_t)M, (uint64_t)w->cols, (uint64_t)w->cols * 2,
                                pair ? gemm_pair_tile_tokens() : gemm_tile_tokens(), 64, 3));
    c->launches++;
    if (pair) {
        // the fused SwiGLU / GeGLU output leaves through staged TMA stores when the matrix can be
        // described by a tensor map (16-byte aligned base and pitch)
        CUtensorMap tm_o = tm_x;
        if ((mode == GEMM_OUT_SWIGLU || mode == GEMM_OUT_GEGLU) && !(reinterpret_cast<uintptr_t>(out) & 15) && ldo % 8 == 0) {
            CMFC_TRY(make_tensor_map_2d(&tm_o, out, 2, (uint64_t)M, (uint64_t)w->rows / 2, (uint64_t)ldo * 2, 32, 16, 0));
            p.tma_out = 1;
        }
        return launch_gemm_dequant_pair(wkind, tm_x, w->tm_w, w->tm_s, tm_o, p, c->num_sms, c->stream);
    }
    return launch_gemm_dequant(wkind, tm_x, w->tm_w, w->tm_s, p, c->num_sms, c->stream);
}

// Segment table on the device: [nseg+1] token offsets, then [nseg] first V^T column of each
// segment (8-aligned, so every TMA x coordinate is a multiple of 16 bytes).  Re-uploaded only
// when the segmentation changes.
int prepare_segs(Context* c, const std::vector<int>& segs, SegTable* out) {
    for (size_t i = 0; i < c->seg_cache.size(); ++i)
        if (c->seg_cache[i].first.host == segs) {
            // most recently used last: an entry a forward has just used is never the one a later miss
            // of the same forward evicts (a captured step must find every table its warm-up step made)
            if (i + 1 != c->seg_cache.size())
                std::rotate(c->seg_cache.begin() + i, c->seg_cache.begin() + i + 1, c->seg_cache.end());
            *out = c->seg_cache.back().first;
            return OK;
        }
    std::vector<int> tab(2 * segs.size() + 1, 0);
    int mx = 0, col = 0;
    for (size_t i = 0; i < segs.size(); ++i) {
        if (segs[i] <= 0) return fail(ERR_BAD_ARG, "empty segment");
        tab[i + 1] = tab[i] + segs[i];
        tab[segs.size() + 1 + i] = col;
        col += (segs[i] + 7) & ~7;
        mx = segs[i] > mx ? segs[i] : mx;
    }
    if (c->seg_cache.size() >= 32) {  // a forward alternates between a handful of segmentations; the least recently used goes
        CMFC_CUDA(cudaStreamSynchronize(c->main_stream));  // queued kernels of either chain may still read the table
        CMFC_CUDA(cudaStreamSynchronize(c->side_stream));
        c->seg_cache.front().second.release();
        c->seg_cache.erase(c->seg_cache.begin());
    }
    c->seg_cache.emplace_back();
    auto& e = c->seg_cache.back();
    CMFC_TRY(e.second.ensure(tab.size() * 4));
    CMFC_CUDA(cudaMemcpyAsync(e.second.p, tab.data(), tab.size() * 4, cudaMemcpyHostToDevice, c->stream));
    CMFC_CUDA(cudaStreamSynchronize(c->stream));  // tab is a stack temporary
    e.first.host = segs;
    e.first.dev = e.second.as<int>();
    e.first.n_total = tab[segs.size()];
    e.first.vt_pitch = col;
    e.first.max_seg = mx;
    *out = e.first;
    return OK;
}

static bool fixed_ref_enabled() {
    const char* e = getenv("CMFC_ATTN_FIXED_REF");  // read per call
    return !(e && e[0] == '0');
}

float attention_score_ref_from_gain(float qk_gain, int hd) {
    if (!(qk_gain > 0.0f) || !fixed_ref_enabled()) return 0.0f;
    // q . k / sqrt(hd) <= |q| |k| / sqrt(hd) <= sqrt(hd) * gain; 2 % covers the f32 arithmetic of the
    // norm and rotation and the bf16 rounding of both operands
    const float ref = sqrtf((float)hd) * qk_gain * 1.02f * 1.4426950408889634f;
    return ref <= ATTN_MAX_SCORE_REF ? ref : 0.0f;
}

int attention_score_ref(Context* c, const __nv_bfloat16* q, const __nv_bfloat16* k, size_t n_total, int nh, int nkv,
                        int hd, float scale, float* score_ref) {
    *score_ref = 0.0f;
    if (!fixed_ref_enabled() || !(scale > 0.0f)) return OK;
    DevBuf& b = c->lane_buf("attn_norm2");
    CMFC_TRY(b.ensure(8));
    CMFC_CUDA(cudaMemsetAsync(b.p, 0, 8, c->stream));
    launch_head_norm2_max(q, n_total * nh, hd, b.as<unsigned>(), c->stream);
    launch_head_norm2_max(k, n_total * nkv, hd, b.as<unsigned>() + 1, c->stream);
    c->launches += 2;
    float n2[2];
    CMFC_CUDA(cudaMemcpyAsync(n2, b.p, 8, cudaMemcpyDeviceToHost, c->stream));
    CMFC_CUDA(cudaStreamSynchronize(c->stream));
    const float ref = sqrtf(n2[0]) * sqrtf(n2[1]) * scale * 1.4426950408889634f * 1.001f;
    if (ref > 0.0f && ref <= ATTN_MAX_SCORE_REF) *score_ref = ref;
    return OK;
}

int dev_attention(Context* c, const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* vt,
                  const SegTable& st, int nh, int nkv, int hd, float scale, __nv_bfloat16* out, const AttnRawQ* raw,
                  float score_ref, const unsigned* norm2_max) {
    if (hd % 32 || hd > 128 || hd < 32) return fail(ERR_UNSUPPORTED, "attention needs head_dim in {32, 64, 96, 128}");
    if (nh % nkv) return fail(ERR_BAD_ARG, "query heads must be a multiple of kv heads");
    CUtensorMap tm_q, tm_k, tm_vt;
    // Q / K: [n_total, heads*hd] bf16, boxes of 128 queries / one key tile x 32 dims, 64-byte swizzle
    CMFC_TRY(make_tensor_map_2d(&tm_q, q, 2, st.n_total, (uint64_t)nh * hd, (uint64_t)nh * hd * 2, 128, 32, 2));
    CMFC_TRY(make_tensor_map_2d(&tm_k, k, 2, st.n_total, (uint64_t)nkv * hd, (uint64_t)nkv * hd * 2, attn_key_tile(hd), 32, 2));
    // V^T: [nkv*hd, vt_pitch] bf16, boxes of hd rows x 64 keys, 128-byte swizzle
    CMFC_TRY(make_tensor_map_2d(&tm_vt, vt, 2, (uint64_t)nkv * hd, (uint64_t)st.vt_pitch, (uint64_t)st.vt_pitch * 2, hd, 64, 3));
    AttnParams p;
    p.nh = nh; p.nkv = nkv; p.hd = hd; p.n_total = st.n_total; p.vt_pitch = st.vt_pitch;
    p.seg_start = st.dev; p.nseg = (int)st.host.size(); p.max_seg = st.max_seg; p.scale = scale;
    p.out = out; p.status = c->status; p.score_ref = score_ref; p.norm2_max = norm2_max;
    if (raw) {
        if ((reinterpret_cast<uintptr_t>(raw->q_raw) & 15) || raw->ld_q % 4)
            return fail(ERR_BAD_ARG, "attention: the raw query rows must be 16-byte aligned");
        p.q_raw = raw->q_raw; p.ld_q = raw->ld_q; p.norm_q = raw->norm_q; p.cos_t = raw->cos_t; p.sin_t = raw->sin_t;
    }
    c->launches++;
    return launch_attention(tm_q, tm_k, tm_vt, p, c->stream);
}

int dev_block(Context* c, const BlockWeights& bw, const BlockMod& mod, float* x, int n, const std::vector<int>& segs,
              int hidden, int inter, int nh, int nkv, int hd, double eps, const float* cos_t, const float* sin_t,
              const BlockChain* chain) {
    cudaStream_t s = c->stream;
    const int qkv_w = (nh + 2 * nkv) * hd;
    SegTable st;
    CMFC_TRY(prepare_segs(c, segs, &st));
    if (st.n_total != n) return fail(ERR_BAD_ARG, "segments do not sum to the token count");
    const int vt_pitch = st.vt_pitch;
    if (!row_cols_supported(hidden)) return fail(ERR_UNSUPPORTED, "hidden size " + std::to_string(hidden) + " is not supported by the row kernels");
    DevBuf &xn = c->lane_buf("blk_xn"), &qkv = c->lane_buf("blk_qkv"), &qb = c->lane_buf("blk_q"), &kb = c->lane_buf("blk_k"),
           &vt = c->lane_buf("blk_vt"), &att = c->lane_buf("blk_attn"), &proj = c->lane_buf("blk_proj"), &act = c->lane_buf("blk_act");
    CMFC_TRY(xn.ensure((size_t)n * hidden * 2));
    CMFC_TRY(qkv.ensure((size_t)n * qkv_w * 4));
    CMFC_TRY(qb.ensure((size_t)n * nh * hd * 2));
    CMFC_TRY(kb.ensure((size_t)n * nkv * hd * 2));
    if (vt.cap < (size_t)nkv * hd * vt_pitch * 2) {
        CMFC_TRY(vt.ensure((size_t)nkv * hd * vt_pitch * 2));
        CMFC_CUDA(cudaMemsetAsync(vt.p, 0, vt.cap, s));  // pad columns must hold finite values
    }
    CMFC_TRY(att.ensure((size_t)n * nh * hd * 2));
    CMFC_TRY(proj.ensure((size_t)n * hidden * 4));
    CMFC_TRY(act.ensure((size_t)n * inter * 2));
    if (!(chain && chain->xn_ready)) {
        SpanGuard g(c, "mod-norm");
        launch_rms_mod(x, bw.norm1, mod.s_msa, eps, n, hidden, xn.as<__nv_bfloat16>(), nullptr, s);
        c->launches++;
    }
    {
        // Q and K leave the GEMM as f32 (the head norm comes first); V goes straight to V^T in bf16
        SpanGuard g(c, "qkv-proj");
        const GemmVt gv = {vt.as<__nv_bfloat16>(), (nh + nkv) * hd, vt_pitch, (int)segs.size(), st.dev};
        CMFC_TRY(dev_gemm(c, bw.qkv, xn.as<__nv_bfloat16>(), n, qkv.p, qkv_w, GEMM_OUT_F32, &gv));
    }
    // qk-norm + RoPE: one pass over Q and K between the QKV GEMM and attention.  With
    // CMFC_ROPE_PROLOGUE=1 only K takes that pass (a K tile is shared by every query tile of its
    // heads) and Q is normalised and rotated in the attention kernel's prologue, each query row exactly
    // once.  Measured on the 1024x1024 step: the prologue form makes the pass 0.66 ms shorter and
    // attention 1.15 ms longer (the prologue is serial work in front of every CTA's first MMA), so the
    // separate pass is the default.
    const char* pro_env = getenv("CMFC_ROPE_PROLOGUE");  // read per call
    const bool q_prologue = pro_env && pro_env[0] == '1';
    // the head norm bounds every score, so attention can take the bounded form (AttnParams::score_ref),
    // whose queries come multiplied by scale * log2(e)
    const float attn_scale = 1.0f / sqrtf((float)hd), log2e = 1.4426950408889634f;
    const float score_ref = attention_score_ref_from_gain(bw.qk_gain, hd);
    // Norm gains too large for that bound say little about real rows (the worst case puts a whole row's
    // weight on the largest gain): then the pass measures the finished heads and attention decides on the
    // device, both forms launched, one of them returning at once.
    const bool measured = score_ref == 0.0f && bw.qk_gain > 0.0f && fixed_ref_enabled() && !q_prologue;
    unsigned* norm2 = nullptr;
    if (measured) {
        DevBuf& nb = c->lane_buf("attn_norm2");
        CMFC_TRY(nb.ensure(8));
        CMFC_CUDA(cudaMemsetAsync(nb.p, 0, 8, s));
        norm2 = nb.as<unsigned>();
    }
    {
        SpanGuard g(c, "rope");
        launch_qk_rope_pack(qkv.as<float>(), n, nh, nkv, hd, bw.norm_q, bw.norm_k, cos_t, sin_t,
                            (score_ref > 0.0f || measured) ? attn_scale * log2e : 1.0f, norm2,
                            q_prologue ? nullptr : qb.as<__nv_bfloat16>(), kb.as<__nv_bfloat16>(), s);
        c->launches++;
    }
    {
        SpanGuard g(c, "attention");
        const AttnRawQ raw = {qkv.as<float>(), qkv_w, bw.norm_q, cos_t, sin_t};
        if (measured) {
            // the queries are pre-scaled either way: the tracking form gets scale * log2(e) = 1
            CMFC_TRY(dev_attention(c, qb.as<__nv_bfloat16>(), kb.as<__nv_bfloat16>(), vt.as<__nv_bfloat16>(), st, nh, nkv, hd,
                                   attn_scale, att.as<__nv_bfloat16>(), nullptr, ATTN_MAX_SCORE_REF, norm2));
            CMFC_TRY(dev_attention(c, qb.as<__nv_bfloat16>(), kb.as<__nv_bfloat16>(), vt.as<__nv_bfloat16>(), st, nh, nkv, hd,
                                   1.0f / log2e, att.as<__nv_bfloat16>(), nullptr, 0.0f, norm2));
        } else {
            CMFC_TRY(dev_attention(c, qb.as<__nv_bfloat16>(), kb.as<__nv_bfloat16>(), vt.as<__nv_bfloat16>(), st, nh, nkv, hd,
                                   attn_scale, att.as<__nv_bfloat16>(), q_prologue ? &raw : nullptr, score_ref));
        }
    }
    {
        SpanGuard g(c, "o-proj");
        CMFC_TRY(dev_gemm(c, bw.o, att.as<__nv_bfloat16>(), n, proj.p, hidden, GEMM_OUT_F32));
    }
    {
        SpanGuard g(c, "mod-norm");
        // x += gate_msa * rms(proj; norm2); xn = rms(x; ffn_norm1) * (1 + s_mlp)
        launch_residual_then_norm(x, proj.as<float>(), bw.norm2, mod.gate_msa, bw.ffn_norm1, mod.s_mlp, eps, n, hidden,
                                  xn.as<__nv_bfloat16>(), s);
        c->launches++;
    }
    {
        SpanGuard g(c, "ffn-mm");
        CMFC_TRY(dev_gemm(c, bw.w13, xn.as<__nv_bfloat16>(), n, act.p, inter, GEMM_OUT_SWIGLU));
        CMFC_TRY(dev_gemm(c, bw.w2, act.as<__nv_bfloat16>(), n, proj.p, hidden, GEMM_OUT_F32));
    }
    {
        SpanGuard g(c, "mod-norm");
        if (chain && chain->next_norm1)
            launch_residual_then_norm(x, proj.as<float>(), bw.ffn_norm2, mod.gate_mlp, chain->next_norm1, chain->next_s_msa, eps,
                                      n, hidden, xn.as<__nv_bfloat16>(), s);
        else
            launch_gated_residual(x, proj.as<float>(), bw.ffn_norm2, mod.gate_mlp, eps, n, hidden, s);
        c->launches++;
    }
    CMFC_CUDA(cudaGetLastError());
    return OK;
}

}  // namespace cmfc
