// A quantized linear for callers that must not allocate device memory.
//
// Some hosts of this library run where cudaMalloc is off limits: inside a region that another
// framework's caching allocator owns entirely, on a latency path where an allocation (and the
// implicit device synchronization of a later cudaFree) is not acceptable, or under a memory
// budget fixed at start-up.  cmfc_matmat_device_noalloc serves them: inputs and outputs are the
// caller's own device buffers, and the one piece of scratch the path needs -- the bf16 copy of
// the activations that the tensor-core kernel reads through TMA -- lives in a fixed array inside
// this library's device image instead of a workspace allocated on demand.
#include "../../include/cmf_cuda.h"
#include "runtime.h"

using namespace cmfc;

namespace {

// 8 MiB of bf16 activations: b * cols <= 4 Mi elements (e.g. 1820 tokens of width 2304).  Every
// GPU that loads the library holds this array until the process exits.
constexpr size_t NOALLOC_SCRATCH_BYTES = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
void* g_scratch_addr[MAX_DEVICES] = {nullptr};

// The array's name is only a host-side stand-in; the device address is looked up once per
// device, with that device current, and that address is what kernels and the TMA descriptor get.
int scratch_for_current_device(int device, void** out) {
    if (device < 0 || device >= MAX_DEVICES) return fail(ERR_BAD_ARG, "device index out of range");
    if (!g_scratch_addr[device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || !p)
            return fail(ERR_CUDA, std::string("cudaGetSymbolAddress(scratch): ") + cudaGetErrorString(e));
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return OK;
}

}  // namespace

extern "C" size_t cmfc_noalloc_max_elements(void) { return NOALLOC_SCRATCH_BYTES / 2; }

extern "C" int cmfc_matmat_device_noalloc(cmfc_model* m, int64_t idx, const float* d_x, size_t b, float* d_y) {
    if (!m || !d_x || !d_y || b == 0) return fail(ERR_BAD_ARG, "matmat_device_noalloc: null pointer or empty batch");
    Context* c = ctx_existing();
    if (!c) return fail(ERR_BAD_ARG, "matmat_device_noalloc: no device context on this thread; call cmfc_set_device first");
    auto it = c->weights.find(std::make_tuple(m->m->uid, idx, (int64_t)-1, (int64_t)-1, 0));
    if (it == c->weights.end())
        return fail(ERR_NOT_FOUND, "matmat_device_noalloc: tensor is not resident on this device; run any other entry on it "
                                   "once first (uploading allocates, this entry never does)");
    DevWeight* w = it->second.get();
    const size_t elems = b * (size_t)w->cols;
    if (elems * 2 > NOALLOC_SCRATCH_BYTES)
        return fail(ERR_SHAPE, "matmat_device_noalloc: b * cols = " + std::to_string(elems) + " exceeds the fixed scratch of " +
                                   std::to_string(NOALLOC_SCRATCH_BYTES / 2) + " bf16 elements; split the batch");
    void* scratch = nullptr;
    CMFC_TRY(scratch_for_current_device(c->device, &scratch));
    // Nothing in the scratch has to start at zero: the conversion overwrites exactly the region
    // the GEMM reads.  Two calls in flight on one GPU would share it and race.
    launch_f32_to_bf16(d_x, reinterpret_cast<__nv_bfloat16*>(scratch), elems, c->stream);
    c->launches++;
    CMFC_TRY(dev_gemm(c, w, reinterpret_cast<const __nv_bfloat16*>(scratch), (int)b, d_y, w->rows, GEMM_OUT_F32));
    return check_status(c, "matmat_device_noalloc");
}
