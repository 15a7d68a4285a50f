// Backward of the bi-directional gated linear attention (gradients of q, k, v and of both log-gate tensors),
// SIMT fp32.  Replaces, for the merged operator, what the reference's training path does with
// FusedChunkGLAFunction.backward (flash-linear-attention/fla/ops/gla/chunk_fuse.py:413-518): a sweep that
// rebuilds the scan state for dq, a reverse sweep for dk / dv, and the gate gradient as a cumulative sum of
// dq*q - dk*k (chunk_fuse.py:506-516).
//
// For one scan direction, in scan order (a_t = exp(g_t), c = scale * out_scale):
//     S_t  = diag(a_t) S_{t-1} + k_t^T v_t                      o_t = c q_t S_t
//     dq_t = c S_t do_t
//     D_t  = c q_t^T do_t + Z_{t+1},  Z_t = diag(a_t) D_t        (reverse scan order)
//     dk_t = D_t v_t,  dv_t = k_t D_t
//     e_t  = dq_t * q_t - dk_t * k_t ;  dg_t = sum of e over the tokens scanned at or after t
// The kernels are chunk-parallel like the forward SIMT path: local S and Z per 64-token chunk, a scan over
// chunks in each direction, then one CTA per chunk that replays both recurrences from its entering states.
// This file writes e per direction; the host wrapper takes the cumulative sums.
#include "common.cuh"

namespace vig {
namespace {

constexpr int CH = 64;
constexpr int NT = 256;

struct BwdParams {
    const void *q, *k, *v, *gf, *gb, *dout;
    void *out_dq, *out_dk, *out_dv;  // [B,H,L,d] contiguous, input dtype
    float *ef, *eb;                  // [B,H,L,dk] contiguous fp32
    int64_t sq[3], sk[3], sv[3], sgf[3], sgb[3], sdo[3];
    int B, H, L, dk, dv, dtype;
    float c;
    int dir_mask;
    float *ws_S, *ws_Z, *ws_decay;   // [BH][nchunk][2][dk*dv] x2, [BH][nchunk][2][dk]
    int nchunk;
};

template <typename T>
__device__ __forceinline__ const T* rowp(const void* base, const int64_t* s, int b, int h, int l) {
    return reinterpret_cast<const T*>(base) + b * s[0] + h * s[1] + (int64_t)l * s[2];
}

template <int D, typename T>
__device__ __forceinline__ void load_tile(float* dst, const void* x, const int64_t* sx, int b, int h, int t0, int n) {
    for (int idx = threadIdx.x; idx < CH * D; idx += NT) {
        const int i = idx / D, d = idx % D;
        dst[idx] = i < n ? DType<T>::to_f(rowp<T>(x, sx, b, h, t0 + i)[d]) : 0.f;
    }
}

// gates of the chunk -> per-channel sum to `sum_out` (may be null) -> decay factors exp(g) in place
template <int DK, typename T>
__device__ __forceinline__ void load_gates_exp(float* g, const void* src, const int64_t* sg, int b, int h, int t0, int n, float* sum_out) {
    load_tile<DK, T>(g, src, sg, b, h, t0, n);           // rows past the end: log-gate 0, decay 1
    __syncthreads();
    if (threadIdx.x < DK && sum_out) {
        float s = 0.f;
        for (int i = 0; i < CH; ++i) s += g[i * DK + threadIdx.x];
        sum_out[threadIdx.x] = s;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < CH * DK; idx += NT) g[idx] = __expf(g[idx]);
    __syncthreads();
}

// Layout A: thread = (value column j, slice s of DK/TPC key channels).  Layout B: thread = (key channel d,
// slice s of DV/TPB value columns).  A reduces over key channels inside TPC neighbouring lanes, B over value
// columns inside TPB neighbouring lanes.
template <int DK, int DV> struct LayA { static constexpr int TPC = NT / DV, DPT = DK / TPC; };
template <int DK, int DV> struct LayB { static constexpr int TPB = NT / DK, JPT = DV / TPB; };

// ---- phase A: local S (scan order, from zero) and local Z (reverse scan order, from zero) per chunk ------------
template <int DK, int DV, typename T>
__global__ void __launch_bounds__(NT) bwd_chunk_states(BwdParams p) {
    using A = LayA<DK, DV>;
    extern __shared__ float smem[];
    float* sq = smem;
    float* sk = sq + CH * DK;
    float* sg = sk + CH * DK;
    float* sv = sg + CH * DK;
    float* sdo = sv + CH * DV;
    const int c = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
    const int t0 = c * CH, n = min(CH, p.L - t0);
    const int j = threadIdx.x / A::TPC, s = threadIdx.x % A::TPC;
    load_tile<DK, T>(sq, p.q, p.sq, b, h, t0, n);
    load_tile<DK, T>(sk, p.k, p.sk, b, h, t0, n);
    load_tile<DV, T>(sv, p.v, p.sv, b, h, t0, n);
    load_tile<DV, T>(sdo, p.dout, p.sdo, b, h, t0, n);
    for (int dir = 0; dir < 2; ++dir) {
        if (!(p.dir_mask & (1 << dir))) continue;
        const size_t slot = ((size_t)bh * p.nchunk + c) * 2 + dir;
        __syncthreads();
        load_gates_exp<DK, T>(sg, dir ? p.gb : p.gf, dir ? p.sgb : p.sgf, b, h, t0, n, p.ws_decay + slot * DK);
        float st[A::DPT];
#pragma unroll
        for (int dd = 0; dd < A::DPT; ++dd) st[dd] = 0.f;
        for (int ii = 0; ii < n; ++ii) {                              // S: scan order
            const int i = dir ? n - 1 - ii : ii;
            const float vj = sv[i * DV + j];
#pragma unroll
            for (int dd = 0; dd < A::DPT; ++dd) {
                const int d = s * A::DPT + dd;
                st[dd] = fmaf(st[dd], sg[i * DK + d], sk[i * DK + d] * vj);
            }
        }
#pragma unroll
        for (int dd = 0; dd < A::DPT; ++dd) p.ws_S[slot * DK * DV + (s * A::DPT + dd) * DV + j] = st[dd];
#pragma unroll
        for (int dd = 0; dd < A::DPT; ++dd) st[dd] = 0.f;
        for (int ii = n - 1; ii >= 0; --ii) {                         // Z: reverse scan order, add then decay
            const int i = dir ? n - 1 - ii : ii;
            const float dj = p.c * sdo[i * DV + j];
#pragma unroll
            for (int dd = 0; dd < A::DPT; ++dd) {
                const int d = s * A::DPT + dd;
                st[dd] = (st[dd] + sq[i * DK + d] * dj) * sg[i * DK + d];
            }
        }
#pragma unroll
        for (int dd = 0; dd < A::DPT; ++dd) p.ws_Z[slot * DK * DV + (s * A::DPT + dd) * DV + j] = st[dd];
    }
}

// ---- phase B: local states -> entering states, in place.  S is scanned in scan order, Z against it. -------------
__global__ void __launch_bounds__(NT) bwd_state_scan(BwdParams p) {
    const int DKDV = p.dk * p.dv;
    const int per = (DKDV + NT - 1) / NT;
    int blk = blockIdx.x;
    const int part = blk % per; blk /= per;
    const int dir = blk % 2; blk /= 2;
    const int which = blk % 2;                                        // 0: S, 1: Z
    const int bh = blk / 2;
    if (!(p.dir_mask & (1 << dir))) return;
    const int e = part * NT + threadIdx.x;
    if (e >= DKDV) return;
    const int d = e / p.dv;
    float* ws = which ? p.ws_Z : p.ws_S;
    const bool descending = (dir != 0) != (which != 0);               // chunk order of this scan
    float acc = 0.f;
    for (int cc = 0; cc < p.nchunk; ++cc) {
        const int c = descending ? p.nchunk - 1 - cc : cc;
        const size_t slot = ((size_t)bh * p.nchunk + c) * 2 + dir;
        float* u = ws + slot * DKDV + e;
        const float local = *u;
        *u = acc;                                                     // state entering chunk c
        acc = fmaf(acc, __expf(p.ws_decay[slot * p.dk + d]), local);
    }
}

// ---- phase C: gradients of one chunk -----------------------------------------------------------------------------
template <int DK, int DV, typename T>
__global__ void __launch_bounds__(NT) bwd_chunk_grads(BwdParams p) {
    using A = LayA<DK, DV>;
    using Bl = LayB<DK, DV>;
    extern __shared__ float smem[];
    float* sq = smem;
    float* sk = sq + CH * DK;
    float* sg = sk + CH * DK;
    float* se = sg + CH * DK;              // dq*q - dk*k of the current direction
    float* sdq = se + CH * DK;
    float* sdk = sdq + CH * DK;
    float* sv = sdk + CH * DK;
    float* sdo = sv + CH * DV;
    float* sdv = sdo + CH * DV;
    const int c = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
    const int t0 = c * CH, n = min(CH, p.L - t0);
    load_tile<DK, T>(sq, p.q, p.sq, b, h, t0, n);
    load_tile<DK, T>(sk, p.k, p.sk, b, h, t0, n);
    load_tile<DV, T>(sv, p.v, p.sv, b, h, t0, n);
    load_tile<DV, T>(sdo, p.dout, p.sdo, b, h, t0, n);
    for (int idx = threadIdx.x; idx < CH * DK; idx += NT) { sdq[idx] = 0.f; sdk[idx] = 0.f; }
    for (int idx = threadIdx.x; idx < CH * DV; idx += NT) sdv[idx] = 0.f;
    for (int dir = 0; dir < 2; ++dir) {
        if (!(p.dir_mask & (1 << dir))) continue;
        const size_t slot = ((size_t)bh * p.nchunk + c) * 2 + dir;
        __syncthreads();
        load_gates_exp<DK, T>(sg, dir ? p.gb : p.gf, dir ? p.sgb : p.sgf, b, h, t0, n, nullptr);
        {   // layout B: dq from the rebuilt state (scan order), then dk from Z (reverse scan order)
            const int d = threadIdx.x / Bl::TPB, s = threadIdx.x % Bl::TPB;
            float st[Bl::JPT];
            const float* Sin = p.ws_S + slot * DK * DV + d * DV + s * Bl::JPT;
#pragma unroll
            for (int jj = 0; jj < Bl::JPT; ++jj) st[jj] = Sin[jj];
            for (int ii = 0; ii < n; ++ii) {
                const int i = dir ? n - 1 - ii : ii;
                const float a = sg[i * DK + d], kd = sk[i * DK + d];
                float acc = 0.f;
#pragma unroll
                for (int jj = 0; jj < Bl::JPT; ++jj) {
                    const int j = s * Bl::JPT + jj;
                    st[jj] = fmaf(st[jj], a, kd * sv[i * DV + j]);
                    acc = fmaf(st[jj], sdo[i * DV + j], acc);
                }
#pragma unroll
                for (int m = 1; m < Bl::TPB; m <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
                if (s == 0) {
                    const float dqd = p.c * acc;
                    sdq[i * DK + d] += dqd;
                    se[i * DK + d] = dqd * sq[i * DK + d];
                }
            }
            const float* Zin = p.ws_Z + slot * DK * DV + d * DV + s * Bl::JPT;
#pragma unroll
            for (int jj = 0; jj < Bl::JPT; ++jj) st[jj] = Zin[jj];
            for (int ii = n - 1; ii >= 0; --ii) {
                const int i = dir ? n - 1 - ii : ii;
                const float a = sg[i * DK + d], cq = p.c * sq[i * DK + d];
                float acc = 0.f;
#pragma unroll
                for (int jj = 0; jj < Bl::JPT; ++jj) {
                    const int j = s * Bl::JPT + jj;
                    const float ds = fmaf(cq, sdo[i * DV + j], st[jj]);
                    acc = fmaf(ds, sv[i * DV + j], acc);
                    st[jj] = ds * a;
                }
#pragma unroll
                for (int m = 1; m < Bl::TPB; m <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
                if (s == 0) {
                    sdk[i * DK + d] += acc;
                    se[i * DK + d] -= acc * sk[i * DK + d];
                }
            }
        }
        {   // layout A: dv from Z (reverse scan order)
            const int j = threadIdx.x / A::TPC, s = threadIdx.x % A::TPC;
            float st[A::DPT];
            const float* Zin = p.ws_Z + slot * DK * DV;
#pragma unroll
            for (int dd = 0; dd < A::DPT; ++dd) st[dd] = Zin[(s * A::DPT + dd) * DV + j];
            for (int ii = n - 1; ii >= 0; --ii) {
                const int i = dir ? n - 1 - ii : ii;
                const float dj = p.c * sdo[i * DV + j];
                float acc = 0.f;
#pragma unroll
                for (int dd = 0; dd < A::DPT; ++dd) {
                    const int d = s * A::DPT + dd;
                    const float ds = fmaf(sq[i * DK + d], dj, st[dd]);
                    acc = fmaf(sk[i * DK + d], ds, acc);
                    st[dd] = ds * sg[i * DK + d];
                }
#pragma unroll
                for (int m = 1; m < A::TPC; m <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
                if (s == 0) sdv[i * DV + j] += acc;
            }
        }
        __syncthreads();
        float* e_out = (dir ? p.eb : p.ef) + ((size_t)bh * p.L + t0) * DK;
        for (int idx = threadIdx.x; idx < n * DK; idx += NT) e_out[idx] = se[idx];
    }
    __syncthreads();
    T* dq = reinterpret_cast<T*>(p.out_dq) + ((size_t)bh * p.L + t0) * DK;
    T* dk = reinterpret_cast<T*>(p.out_dk) + ((size_t)bh * p.L + t0) * DK;
    T* dv = reinterpret_cast<T*>(p.out_dv) + ((size_t)bh * p.L + t0) * DV;
    for (int idx = threadIdx.x; idx < n * DK; idx += NT) { dq[idx] = DType<T>::from_f(sdq[idx]); dk[idx] = DType<T>::from_f(sdk[idx]); }
    for (int idx = threadIdx.x; idx < n * DV; idx += NT) dv[idx] = DType<T>::from_f(sdv[idx]);
}

template <int DK, int DV, typename T>
int launch_typed(const BwdParams& p, cudaStream_t stream) {
    dim3 grid(p.nchunk, p.B * p.H);
    const size_t smA = (size_t)CH * (3 * DK + 2 * DV) * sizeof(float);
    const size_t smC = (size_t)CH * (6 * DK + 3 * DV) * sizeof(float);
    auto kA = bwd_chunk_states<DK, DV, T>;
    auto kC = bwd_chunk_grads<DK, DV, T>;
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(kA, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smA)) != cudaSuccess) return (int)e;
    if ((e = cudaFuncSetAttribute(kC, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smC)) != cudaSuccess) return (int)e;
    kA<<<grid, NT, smA, stream>>>(p);
    const int per = (DK * DV + NT - 1) / NT;
    bwd_state_scan<<<p.B * p.H * 2 * 2 * per, NT, 0, stream>>>(p);
    kC<<<grid, NT, smC, stream>>>(p);
    return (int)cudaGetLastError();
}

template <typename T>
int launch_dims(const BwdParams& p, cudaStream_t stream) {
#define VIG_CASE(DKV, DVV) if (p.dk == DKV && p.dv == DVV) return launch_typed<DKV, DVV, T>(p, stream);
    VIG_CASE(16, 32) VIG_CASE(32, 32) VIG_CASE(32, 64) VIG_CASE(64, 64) VIG_CASE(64, 128)   // larger heads exceed shared memory
#undef VIG_CASE
    return VIG_ERR_SHAPE;
}

void fill(int64_t* dst, const int64_t* src, int H, int L, int d) {
    if (src) { dst[0] = src[0]; dst[1] = src[1]; dst[2] = src[2]; }
    else { dst[0] = (int64_t)H * L * d; dst[1] = (int64_t)L * d; dst[2] = d; }
}

}  // namespace
}  // namespace vig

using namespace vig;

extern "C" size_t vig_bigla_bwd_workspace_bytes(int B, int H, int L, int dk, int dv) {
    if (B <= 0 || H <= 0 || L <= 0 || dk <= 0 || dv <= 0) return 0;
    const size_t nchunk = (L + CH - 1) / CH;
    return (size_t)B * H * nchunk * 2 * (2 * (size_t)dk * dv + dk) * sizeof(float);
}

extern "C" int vig_bigla_bwd(const void* q, const void* k, const void* v, const void* g_fwd, const void* g_bwd, const void* d_out,
                             void* dq, void* dk_out, void* dv_out, float* e_fwd, float* e_bwd,
                             int B, int H, int L, int dk, int dv, int dtype,
                             const int64_t* strides_q, const int64_t* strides_k, const int64_t* strides_v,
                             const int64_t* strides_gf, const int64_t* strides_gb, const int64_t* strides_do,
                             float scale, float out_scale, int dir_mask,
                             void* workspace, size_t workspace_bytes, void* stream) {
    if (dtype < 0 || dtype > 2) return VIG_ERR_DTYPE;
    if (B < 0 || H <= 0 || L < 0) return VIG_ERR_SHAPE;
    if (dir_mask < 1 || dir_mask > 3) return VIG_ERR_ARG;
    if (B == 0 || L == 0) return VIG_OK;
    if (!q || !k || !v || !d_out || !dq || !dk_out || !dv_out) return VIG_ERR_NULL;
    if ((dir_mask & 1) && (!g_fwd || !e_fwd)) return VIG_ERR_NULL;
    if ((dir_mask & 2) && (!g_bwd || !e_bwd)) return VIG_ERR_NULL;
    const size_t need = vig_bigla_bwd_workspace_bytes(B, H, L, dk, dv);
    if (!workspace || workspace_bytes < need) return VIG_ERR_WORKSPACE;
    BwdParams p{};
    p.q = q; p.k = k; p.v = v; p.gf = g_fwd; p.gb = g_bwd; p.dout = d_out;
    p.out_dq = dq; p.out_dk = dk_out; p.out_dv = dv_out; p.ef = e_fwd; p.eb = e_bwd;
    fill(p.sq, strides_q, H, L, dk); fill(p.sk, strides_k, H, L, dk); fill(p.sv, strides_v, H, L, dv);
    fill(p.sgf, strides_gf, H, L, dk); fill(p.sgb, strides_gb, H, L, dk); fill(p.sdo, strides_do, H, L, dv);
    p.B = B; p.H = H; p.L = L; p.dk = dk; p.dv = dv; p.dtype = dtype;
    if (scale < 0.f) scale = 1.0f / sqrtf((float)dk);
    p.c = scale * out_scale;
    p.dir_mask = dir_mask;
    p.nchunk = (L + CH - 1) / CH;
    const size_t states = (size_t)B * H * p.nchunk * 2 * dk * dv;
    p.ws_S = reinterpret_cast<float*>(workspace);
    p.ws_Z = p.ws_S + states;
    p.ws_decay = p.ws_Z + states;
    switch (dtype) {
        case VIG_DTYPE_F32: return launch_dims<float>(p, (cudaStream_t)stream);
        case VIG_DTYPE_BF16: return launch_dims<__nv_bfloat16>(p, (cudaStream_t)stream);
        case VIG_DTYPE_F16: return launch_dims<__half>(p, (cudaStream_t)stream);
    }
    return VIG_ERR_DTYPE;
}
