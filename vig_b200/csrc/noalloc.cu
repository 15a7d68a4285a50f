// vig_bigla_fwd_noalloc: the bi-GLA forward for callers that cannot allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they run the operator: a plugin
// that is handed only its input and output buffers, a serving loop whose memory pool is frozen after
// start-up, code running between the begin and end of a region where the runtime forbids allocation.
// vig_bigla_fwd needs a caller-provided workspace for sequences longer than one segment; this entry point
// instead keeps that workspace in a fixed array that is part of the library image.  Every GPU that loads
// the library therefore holds VIG_NOALLOC_SCRATCH_BYTES of device memory until the process exits.
#include <mutex>
#include "common.cuh"

using namespace vig;

namespace vig {
int bigla_fwd_internal(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, void* o,
                       int B, int H, int L, int dk, int dv, int dtype,
                       const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                       const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_o,
                       float scale, float out_scale, float gate_logit_normalizer, float clamp_min,
                       const float* init_state_fwd, const float* init_state_bwd, float* final_state_fwd, float* final_state_bwd,
                       float* total_logdecay_fwd, float* total_logdecay_bwd, int dir_mask, int impl, bool no_single,
                       void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream);
}

// The per-segment states and summed log-gates of one call (what `workspace` holds in vig_bigla_fwd).
static __device__ __align__(256) unsigned char g_bigla_scratch[VIG_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
void* g_scratch_ptr[MAX_DEVICES] = {};

// In host code `g_bigla_scratch` only names the symbol; the address the kernels must get is looked up
// once per device, with that device current.
int scratch_for_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= MAX_DEVICES) return VIG_ERR_DEVICE;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_bigla_scratch);
        if (e != cudaSuccess) return (int)e;
        if (!ptr) return VIG_ERR_DEVICE;
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return VIG_OK;
}
}  // namespace

extern "C" size_t vig_bigla_noalloc_scratch_bytes(void) { return VIG_NOALLOC_SCRATCH_BYTES; }

extern "C" int vig_bigla_fwd_noalloc(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, void* o,
                                     int B, int H, int L, int dk, int dv, int dtype,
                                     const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                                     const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_o,
                                     float scale, float out_scale, float gate_logit_normalizer, float clamp_min,
                                     int impl, int32_t* status_dev, void* stream) {
    if (!o) return VIG_ERR_NULL;
    void* scratch = nullptr;
    if (int st = scratch_for_current_device(&scratch)) return st;
    // The launcher sizes the scratch for the kernel family that will really run with these pointers and this shape
    // (nothing for a single 256-token segment on the tensor-core path) and refuses before any launch when the array
    // is too small.  The single-launch and wavefront forms need more scratch than the array holds: ruled out here.
    // Every workspace slot a call reads is written earlier in the same call, so nothing needs clearing
    // between calls; what the previous call left behind is simply overwritten.
    const int st = bigla_fwd_internal(q, k, v, g_fwd, g_bwd, o, B, H, L, dk, dv, dtype, strides_q, strides_k, strides_v, strides_gf,
                                      strides_gb, strides_o, scale, out_scale, gate_logit_normalizer, clamp_min,
                                      nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 3, impl, true,
                                      scratch, VIG_NOALLOC_SCRATCH_BYTES, status_dev, stream);
    return st == VIG_ERR_WORKSPACE ? VIG_ERR_SCRATCH_LIMIT : st;
}
