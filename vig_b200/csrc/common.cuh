// Shared helpers for the vig_b200 kernels: dtype traits, 16-byte vector access, parameter block.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include "../../include/vig_b200.h"

namespace vig {

template <typename T> struct DType;
template <> struct DType<float> {
    static constexpr int VEC = 4;
    __device__ static float to_f(float x) { return x; }
    __device__ static float from_f(float x) { return x; }
};
template <> struct DType<__nv_bfloat16> {
    static constexpr int VEC = 8;
    __device__ static float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
    __device__ static __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct DType<__half> {
    static constexpr int VEC = 8;
    __device__ static float to_f(__half x) { return __half2float(x); }
    __device__ static __half from_f(float x) { return __float2half_rn(x); }
};

// 16-byte vector of T, loaded / stored with one instruction, unpacked to fp32.
template <typename T> struct alignas(16) Vec16 {
    static constexpr int N = DType<T>::VEC;
    T e[N];
    __device__ void load(const T* p) { *reinterpret_cast<uint4*>(e) = *reinterpret_cast<const uint4*>(p); }
    __device__ void load_nc(const T* p) { *reinterpret_cast<uint4*>(e) = __ldg(reinterpret_cast<const uint4*>(p)); }
    __device__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(e); }
    __device__ void to_float(float* f) const {
#pragma unroll
        for (int i = 0; i < N; ++i) f[i] = DType<T>::to_f(e[i]);
    }
    __device__ void from_float(const float* f) {
#pragma unroll
        for (int i = 0; i < N; ++i) e[i] = DType<T>::from_f(f[i]);
    }
};

__device__ __forceinline__ float log_sigmoid(float x) {
    // min(x,0) - log1p(exp(-|x|)), the numerically stable form torch uses
    return fminf(x, 0.f) - log1pf(__expf(-fabsf(x)));
}

__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
// Sigmoid for kernels whose result is rounded to a 16-bit type: one MUFU (tanh.approx, ~2^-11 relative) instead of two
// (exp + reciprocal) -- these kernels are bound by the quarter-rate MUFU pipe, not by DRAM.  fp32 keeps the exact form.
template <typename T> __device__ __forceinline__ float sigmoid_t(float x) {
    if (sizeof(T) == 4) return sigmoidf_(x);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(0.5f, t, 0.5f);
}

// Parameter block of the bi-GLA launchers (host fills it from the C ABI arguments).
struct BiglaParams {
    const void *q, *k, *v, *gf, *gb;
    void* o;
    int64_t sq[3], sk[3], sv[3], sgf[3], sgb[3], so[3];  // element strides of (b, h, l)
    int B, H, L, dk, dv, dtype;
    float qscale;       // scale * out_scale, folded into q
    float gate_norm;    // > 0: gates are raw logits, g = logsigmoid(x) / gate_norm
    float clamp_min;    // NaN = no clamp
    const float *init_f, *init_b;
    float *final_f, *final_b, *logdecay_f, *logdecay_b;
    int dir_mask;
    float* ws_state;    // [B*H][nchunk][2][dk*dv]
    float* ws_decay;    // [B*H][nchunk][2][dk]
    int nchunk;
    int32_t* status;
    // single-launch tensor-core path: work tickets, per-(b,h) arrival counters, per-CTA scratch for operand tiles
    uint32_t* ticket;
    uint32_t* group_cnt;
    uint8_t* qscratch;
    int nseg;
};

__device__ __forceinline__ float gate_transform(float x, float gate_norm, float clamp_min) {
    float g = gate_norm > 0.f ? log_sigmoid(x) / gate_norm : x;
    if (clamp_min == clamp_min) g = fmaxf(g, clamp_min);
    return g;
}

int bigla_simt_launch(const BiglaParams& p, cudaStream_t stream);
size_t bigla_simt_workspace(int B, int H, int L, int dk, int dv);
// scan over p.nchunk per-chunk (or per-segment) local states in the workspace, in place (phase B)
int bigla_scan_launch(const BiglaParams& p, cudaStream_t stream);
int bigla_tc_launch(const BiglaParams& p, void* ws, size_t ws_bytes, bool allow_fused, cudaStream_t stream);
size_t bigla_tc_workspace(int B, int H, int L, int dk, int dv, bool split_only);
size_t bigla_tc_min_workspace(const BiglaParams& p);   // what this very call uses (0 for one segment with an output)
bool bigla_tc_supported(const BiglaParams& p);
bool bigla_tc_prefers_single(int L);
// warp-specialised wavefront form (large batches): one persistent CTA per SM, state hand-off between segments
bool bigla_wave_supported(const BiglaParams& p);
bool bigla_wave_preferred(const BiglaParams& p);
size_t bigla_wave_workspace(int B, int H, int L, int dk, int dv);
int bigla_wave_launch(const BiglaParams& p, void* ws, size_t ws_bytes, cudaStream_t stream);
// TMA-fed depthwise conv: launches and returns a status, or VIG_DWCONV_NOT_TAKEN when the shape is left to the other forms
constexpr int VIG_DWCONV_NOT_TAKEN = -1000;
int dwconv_tma_try(const void* x, const void* wt, const void* bias, void* y, int B, int h, int w, int C, int act, int dtype,
                   int32_t* status, cudaStream_t stream);

}  // namespace vig
