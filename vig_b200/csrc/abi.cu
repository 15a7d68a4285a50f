// C ABI of the bi-GLA operator: argument validation and dispatch to the SIMT or tensor-core launcher.
#include <cmath>
#include "common.cuh"

using namespace vig;

extern "C" int vig_version(void) { return 100; }

extern "C" const char* vig_strerror(int status) {
    switch (status) {
        case VIG_OK: return "ok";
        case VIG_ERR_NULL: return "a required pointer is NULL";
        case VIG_ERR_SHAPE: return "unsupported shape";
        case VIG_ERR_DTYPE: return "unknown dtype code";
        case VIG_ERR_ALIGN: return "pointer or stride not aligned as the kernel needs";
        case VIG_ERR_WORKSPACE: return "workspace missing or too small";
        case VIG_ERR_ARG: return "invalid argument";
        case VIG_ERR_DEVICE: return "device or driver does not support this kernel";
        case VIG_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the fixed no-allocation array holds; use vig_bigla_fwd with a workspace";
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "unknown status";
}

static bool dims_ok(int dk, int dv) {
    return (dk == 16 || dk == 32 || dk == 64 || dk == 128) && (dv == 32 || dv == 64 || dv == 128);
}

namespace vig {
size_t bigla_workspace_internal(int B, int H, int L, int dk, int dv, int dtype, int impl, bool no_single);
int bigla_fwd_internal(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, void* o,
                       int B, int H, int L, int dk, int dv, int dtype,
                       const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                       const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_o,
                       float scale, float out_scale, float gate_logit_normalizer, float clamp_min,
                       const float* init_state_fwd, const float* init_state_bwd, float* final_state_fwd, float* final_state_bwd,
                       float* total_logdecay_fwd, float* total_logdecay_bwd, int dir_mask, int impl, bool no_single,
                       void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream);
}

extern "C" size_t vig_bigla_workspace_bytes(int B, int H, int L, int dk, int dv, int dtype, int impl) {
    return bigla_workspace_internal(B, H, L, dk, dv, dtype, impl, false);
}

size_t vig::bigla_workspace_internal(int B, int H, int L, int dk, int dv, int dtype, int impl, bool no_single) {
    if (B <= 0 || H <= 0 || L <= 0 || !dims_ok(dk, dv)) return 0;
    size_t simt = bigla_simt_workspace(B, H, L, dk, dv);
    size_t tc = (dtype != VIG_DTYPE_F32 && impl != VIG_IMPL_SIMT) ? bigla_tc_workspace(B, H, L, dk, dv, no_single || !(impl == VIG_IMPL_TC_SINGLE || (impl != VIG_IMPL_TC_SPLIT && bigla_tc_prefers_single(L)))) : 0;
    size_t wave = (dtype != VIG_DTYPE_F32 && (impl == VIG_IMPL_TC_WAVE || impl == VIG_IMPL_AUTO) && (dk == 64 || dk == 32) && dv == 64) ? bigla_wave_workspace(B, H, L, dk, dv) : 0;
    if (impl == VIG_IMPL_TC_WAVE) return wave;
    if (no_single) wave = 0;
    size_t m = simt > tc ? simt : tc;
    return m > wave ? m : wave;
}

static void fill_strides(int64_t* dst, const int64_t* src, int H, int L, int d) {
    if (src) { dst[0] = src[0]; dst[1] = src[1]; dst[2] = src[2]; }
    else { dst[0] = (int64_t)H * L * d; dst[1] = (int64_t)L * d; dst[2] = d; }
}

extern "C" int vig_bigla_fwd(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, void* o,
                             int B, int H, int L, int dk, int dv, int dtype,
                             const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                             const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_o,
                             float scale, float out_scale, float gate_logit_normalizer, float clamp_min,
                             const float* init_state_fwd, const float* init_state_bwd,
                             float* final_state_fwd, float* final_state_bwd,
                             float* total_logdecay_fwd, float* total_logdecay_bwd,
                             int dir_mask, int impl,
                             void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream) {
    return bigla_fwd_internal(q, k, v, g_fwd, g_bwd, o, B, H, L, dk, dv, dtype, strides_q, strides_k, strides_v, strides_gf,
                              strides_gb, strides_o, scale, out_scale, gate_logit_normalizer, clamp_min, init_state_fwd,
                              init_state_bwd, final_state_fwd, final_state_bwd, total_logdecay_fwd, total_logdecay_bwd,
                              dir_mask, impl, false, workspace, workspace_bytes, status_dev, stream);
}

int vig::bigla_fwd_internal(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, void* o,
                            int B, int H, int L, int dk, int dv, int dtype,
                            const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                            const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_o,
                            float scale, float out_scale, float gate_logit_normalizer, float clamp_min,
                            const float* init_state_fwd, const float* init_state_bwd, float* final_state_fwd, float* final_state_bwd,
                            float* total_logdecay_fwd, float* total_logdecay_bwd, int dir_mask, int impl, bool no_single,
                            void* workspace, size_t workspace_bytes, int32_t* status_dev, void* stream) {
    if (dtype < 0 || dtype > 2) return VIG_ERR_DTYPE;
    if (B < 0 || H <= 0 || L < 0 || !dims_ok(dk, dv)) return VIG_ERR_SHAPE;
    if (dir_mask < 1 || dir_mask > 3) return VIG_ERR_ARG;
    if (impl < VIG_IMPL_AUTO || impl > VIG_IMPL_TC_WAVE) return VIG_ERR_ARG;
    if (B == 0 || L == 0) return VIG_OK;
    if (!k || !v) return VIG_ERR_NULL;
    if (o && !q) return VIG_ERR_NULL;
    if ((dir_mask & 1) && !g_fwd) return VIG_ERR_NULL;
    if ((dir_mask & 2) && !g_bwd) return VIG_ERR_NULL;
    const bool need_states = final_state_fwd || final_state_bwd || total_logdecay_fwd || total_logdecay_bwd;
    if (!o && !need_states) return VIG_ERR_NULL;
    if (!(gate_logit_normalizer >= 0.f)) return VIG_ERR_ARG;

    BiglaParams p{};
    p.q = q; p.k = k; p.v = v; p.gf = g_fwd; p.gb = g_bwd; p.o = o;
    fill_strides(p.sq, strides_q, H, L, dk); fill_strides(p.sk, strides_k, H, L, dk);
    fill_strides(p.sgf, strides_gf, H, L, dk); fill_strides(p.sgb, strides_gb, H, L, dk);
    fill_strides(p.sv, strides_v, H, L, dv); fill_strides(p.so, strides_o, H, L, dv);
    p.B = B; p.H = H; p.L = L; p.dk = dk; p.dv = dv; p.dtype = dtype;
    if (scale < 0.f) scale = 1.0f / std::sqrt((float)dk);
    p.qscale = scale * out_scale;
    p.gate_norm = gate_logit_normalizer; p.clamp_min = clamp_min;
    p.init_f = init_state_fwd; p.init_b = init_state_bwd;
    p.final_f = final_state_fwd; p.final_b = final_state_bwd;
    p.logdecay_f = total_logdecay_fwd; p.logdecay_b = total_logdecay_bwd;
    p.dir_mask = dir_mask; p.status = status_dev;

    if (impl == VIG_IMPL_TC_WAVE) {
        if (!bigla_wave_supported(p)) return VIG_ERR_SHAPE;
        if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255)) return VIG_ERR_ALIGN;
        return bigla_wave_launch(p, workspace, workspace_bytes, (cudaStream_t)stream);
    }
    if (impl == VIG_IMPL_AUTO && !no_single && bigla_wave_supported(p) && bigla_wave_preferred(p) && workspace &&
        !(reinterpret_cast<uintptr_t>(workspace) & 255) && workspace_bytes >= bigla_wave_workspace(B, H, L, dk, dv))
        return bigla_wave_launch(p, workspace, workspace_bytes, (cudaStream_t)stream);
    bool use_tc = false;
    if (impl == VIG_IMPL_TC || impl == VIG_IMPL_TC_SINGLE || impl == VIG_IMPL_TC_SPLIT) {
        if (!bigla_tc_supported(p)) return VIG_ERR_SHAPE;
        use_tc = true;
    } else if (impl == VIG_IMPL_AUTO) {
        use_tc = bigla_tc_supported(p);
    }
    if (use_tc) {
        // the single-launch form (on request, or by default where it is the faster one) needs the larger workspace;
        // with only the states' worth of workspace the call runs as three launches
        const size_t need = bigla_tc_min_workspace(p);
        if (need && (!workspace || workspace_bytes < need)) return VIG_ERR_WORKSPACE;
        if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 255)) return VIG_ERR_ALIGN;
        return bigla_tc_launch(p, workspace, workspace_bytes, !no_single && (impl == VIG_IMPL_TC_SINGLE || (impl != VIG_IMPL_TC_SPLIT && bigla_tc_prefers_single(L))), (cudaStream_t)stream);
    }
    const size_t need = bigla_simt_workspace(B, H, L, dk, dv);
    const bool needs_ws = need_states || L > 64;
    if (needs_ws && (!workspace || workspace_bytes < need)) return VIG_ERR_WORKSPACE;
    if (needs_ws && (reinterpret_cast<uintptr_t>(workspace) & 15)) return VIG_ERR_ALIGN;
    const size_t nchunk = (L + 63) / 64;
    p.ws_state = reinterpret_cast<float*>(workspace);
    p.ws_decay = p.ws_state ? p.ws_state + (size_t)B * H * nchunk * 2 * dk * dv : nullptr;
    return bigla_simt_launch(p, (cudaStream_t)stream);
}
