// Bi-directional gated linear attention, SIMT fp32 path.
//
// Exact for any gate values: it evaluates the recurrence token by token (like the reference's
// recurrent kernel, fla/ops/gla/recurrent_fuse.py:18-148) but parallel over 64-token chunks:
//   phase A  per chunk, from a zero state: local end state U = sum_j diag(prod of later gates) k_j^T v_j
//            and the chunk's summed log-gates, for both directions;
//   phase B  sequential scan over chunks turning U[c] into the state that ENTERS chunk c
//            (forward: from the left, backward: from the right); also final states / total decay;
//   phase C  per chunk: forward recurrence from its entering state, reverse recurrence from the other
//            one, both accumulated into one shared-memory output tile, written once.
// All arithmetic is fp32; inputs may be fp32 / bf16 / fp16 with arbitrary (b,h,l) strides.
#include "common.cuh"

namespace vig {
namespace {

constexpr int CH = 64;        // tokens per chunk
constexpr int NT = 256;       // threads per CTA

template <typename T>
__device__ __forceinline__ const T* row_ptr(const void* base, const int64_t* s, int b, int h, int l) {
    return reinterpret_cast<const T*>(base) + b * s[0] + h * s[1] + (int64_t)l * s[2];
}

// Thread layout of the recurrence: lane = j * TPC + s, j = value column, s = slice of DK/TPC key channels.
template <int DK, int DV> struct Lay {
    static constexpr int TPC = NT / DV;          // threads per value column
    static constexpr int DPT = DK / TPC;         // key channels per thread
    static_assert(NT % DV == 0 && DK % TPC == 0 && DPT >= 1, "bad head dims");
};

template <int DK, int DV, typename T>
__device__ __forceinline__ void load_gates(float* dst, const void* g, const int64_t* sg, int b, int h, int t0, int n,
                                           float gate_norm, float clamp_min) {
    for (int idx = threadIdx.x; idx < CH * DK; idx += NT) {
        int i = idx / DK, d = idx % DK;
        float x = 0.f;
        if (i < n) x = gate_transform(DType<T>::to_f(row_ptr<T>(g, sg, b, h, t0 + i)[d]), gate_norm, clamp_min);
        dst[idx] = x;   // rows past the end: log-gate 0 (decay 1), like the reference's zero padding
    }
}

template <int D, typename T>
__device__ __forceinline__ void load_tile(float* dst, const void* x, const int64_t* sx, int b, int h, int t0, int n, float mul) {
    for (int idx = threadIdx.x; idx < CH * D; idx += NT) {
        int i = idx / D, d = idx % D;
        dst[idx] = i < n ? DType<T>::to_f(row_ptr<T>(x, sx, b, h, t0 + i)[d]) * mul : 0.f;
    }
}

// Sum the log-gates of the chunk per channel (threads < DK), then exponentiate the tile in place.
template <int DK>
__device__ __forceinline__ void sum_and_exp(float* g, float* sum_out /* global, may be null */) {
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

template <int DK, int DV, typename T>
__global__ void __launch_bounds__(NT) bigla_simt_chunk_state(BiglaParams p) {
    using L_ = Lay<DK, DV>;
    extern __shared__ float smem[];
    float* sk = smem;
    float* sv = sk + CH * DK;
    float* sg = sv + CH * DV;
    const int c = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
    const int t0 = c * CH, n = min(CH, p.L - t0);
    const int j = threadIdx.x / L_::TPC, s = threadIdx.x % L_::TPC;
    load_tile<DK, T>(sk, p.k, p.sk, b, h, t0, n, 1.f);
    load_tile<DV, T>(sv, p.v, p.sv, b, h, t0, n, 1.f);
    for (int dir = 0; dir < 2; ++dir) {
        if (!(p.dir_mask & (1 << dir))) continue;
        __syncthreads();
        load_gates<DK, DV, T>(sg, dir ? p.gb : p.gf, dir ? p.sgb : p.sgf, b, h, t0, n, p.gate_norm, p.clamp_min);
        const size_t slot = ((size_t)bh * p.nchunk + c) * 2 + dir;
        sum_and_exp<DK>(sg, p.ws_decay + slot * DK);
        float st[L_::DPT];
#pragma unroll
        for (int dd = 0; dd < L_::DPT; ++dd) st[dd] = 0.f;
        for (int ii = 0; ii < n; ++ii) {
            const int i = dir ? n - 1 - ii : ii;
            const float vj = sv[i * DV + j];
#pragma unroll
            for (int dd = 0; dd < L_::DPT; ++dd) {
                const int d = s * L_::DPT + dd;
                st[dd] = fmaf(st[dd], sg[i * DK + d], sk[i * DK + d] * vj);
            }
        }
        float* U = p.ws_state + slot * DK * DV;
#pragma unroll
        for (int dd = 0; dd < L_::DPT; ++dd) U[(s * L_::DPT + dd) * DV + j] = st[dd];
    }
}

// Phase B: one thread per state element, sequential over chunks in scan order.
__global__ void __launch_bounds__(NT) bigla_simt_state_scan(BiglaParams p) {
    const int DKDV = p.dk * p.dv;
    const int per = (DKDV + NT - 1) / NT;              // CTAs per (bh, dir)
    const int blk = blockIdx.x;
    const int part = blk % per, dir = (blk / per) % 2, bh = blk / (per * 2);
    if (!(p.dir_mask & (1 << dir))) return;
    const int e = part * NT + threadIdx.x;
    if (e >= DKDV) return;
    const int d = e / p.dv;
    const float* init = dir ? p.init_b : p.init_f;
    float S = init ? init[(size_t)bh * DKDV + e] : 0.f;
    float gsum = 0.f;
    constexpr int PF = 4;                               // loads of PF chunks are in flight before the dependent chain runs
    for (int cc0 = 0; cc0 < p.nchunk; cc0 += PF) {
        float u[PF], g[PF];
        float* slotp[PF];
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            const int cc = cc0 + i;
            const int c = dir ? p.nchunk - 1 - cc : cc;
            const size_t slot = ((size_t)bh * p.nchunk + (cc < p.nchunk ? c : 0)) * 2 + dir;
            slotp[i] = p.ws_state + slot * DKDV + e;
            u[i] = cc < p.nchunk ? __ldcg(slotp[i]) : 0.f;
            g[i] = cc < p.nchunk ? __ldcg(p.ws_decay + slot * p.dk + d) : 0.f;
        }
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            if (cc0 + i < p.nchunk) {
                *slotp[i] = S;                          // state entering chunk c
                S = fmaf(S, __expf(g[i]), u[i]);
                gsum += g[i];
            }
        }
    }
    float* fin = dir ? p.final_b : p.final_f;
    if (fin) fin[(size_t)bh * DKDV + e] = S;
    float* ld = dir ? p.logdecay_b : p.logdecay_f;
    if (ld && (e % p.dv) == 0) ld[(size_t)bh * p.dk + d] = gsum;
}

template <int DK, int DV, typename T>
__global__ void __launch_bounds__(NT) bigla_simt_chunk_out(BiglaParams p, int use_ws) {
    using L_ = Lay<DK, DV>;
    extern __shared__ float smem[];
    float* sq = smem;
    float* sk = sq + CH * DK;
    float* sg = sk + CH * DK;
    float* sv = sg + CH * DK;
    float* so = sv + CH * DV;
    const int c = blockIdx.x, bh = blockIdx.y, b = bh / p.H, h = bh % p.H;
    const int t0 = c * CH, n = min(CH, p.L - t0);
    const int j = threadIdx.x / L_::TPC, s = threadIdx.x % L_::TPC;
    load_tile<DK, T>(sq, p.q, p.sq, b, h, t0, n, p.qscale);
    load_tile<DK, T>(sk, p.k, p.sk, b, h, t0, n, 1.f);
    load_tile<DV, T>(sv, p.v, p.sv, b, h, t0, n, 1.f);
    for (int idx = threadIdx.x; idx < CH * DV; idx += NT) so[idx] = 0.f;
    for (int dir = 0; dir < 2; ++dir) {
        if (!(p.dir_mask & (1 << dir))) continue;
        __syncthreads();
        load_gates<DK, DV, T>(sg, dir ? p.gb : p.gf, dir ? p.sgb : p.sgf, b, h, t0, n, p.gate_norm, p.clamp_min);
        sum_and_exp<DK>(sg, nullptr);
        float st[L_::DPT];
        const float* Sin = nullptr;
        if (use_ws) Sin = p.ws_state + (((size_t)bh * p.nchunk + c) * 2 + dir) * DK * DV;
        else if (dir ? p.init_b : p.init_f) Sin = (dir ? p.init_b : p.init_f) + (size_t)bh * DK * DV;
#pragma unroll
        for (int dd = 0; dd < L_::DPT; ++dd) st[dd] = Sin ? Sin[(s * L_::DPT + dd) * DV + j] : 0.f;
        for (int ii = 0; ii < n; ++ii) {
            const int i = dir ? n - 1 - ii : ii;
            const float vj = sv[i * DV + j];
            float acc = 0.f;
#pragma unroll
            for (int dd = 0; dd < L_::DPT; ++dd) {
                const int d = s * L_::DPT + dd;
                st[dd] = fmaf(st[dd], sg[i * DK + d], sk[i * DK + d] * vj);
                acc = fmaf(sq[i * DK + d], st[dd], acc);
            }
#pragma unroll
            for (int m = 1; m < L_::TPC; m <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
            if (s == 0) so[i * DV + j] += acc;          // one writer per (i, j); directions run one after the other
        }
    }
    __syncthreads();
    T* obase = reinterpret_cast<T*>(p.o);
    for (int idx = threadIdx.x; idx < n * DV; idx += NT) {
        int i = idx / DV, jj = idx % DV;
        obase[b * p.so[0] + h * p.so[1] + (int64_t)(t0 + i) * p.so[2] + jj] = DType<T>::from_f(so[idx]);
    }
}

template <int DK, int DV, typename T>
int launch_typed(const BiglaParams& p, cudaStream_t stream) {
    const int BH = p.B * p.H;
    const bool need_states = p.final_f || p.final_b || p.logdecay_f || p.logdecay_b;
    const bool use_ws = p.nchunk > 1 || need_states;
    dim3 grid(p.nchunk, BH);
    if (use_ws) {
        const size_t smA = (size_t)CH * (2 * DK + DV) * sizeof(float);
        auto kA = bigla_simt_chunk_state<DK, DV, T>;
        cudaError_t e = cudaFuncSetAttribute(kA, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smA);
        if (e != cudaSuccess) return (int)e;
        kA<<<grid, NT, smA, stream>>>(p);
        const int per = (DK * DV + NT - 1) / NT;
        bigla_simt_state_scan<<<BH * 2 * per, NT, 0, stream>>>(p);
    }
    if (p.o) {
        const size_t smC = (size_t)CH * (3 * DK + 2 * DV) * sizeof(float);
        auto kC = bigla_simt_chunk_out<DK, DV, T>;
        cudaError_t e = cudaFuncSetAttribute(kC, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smC);
        if (e != cudaSuccess) return (int)e;
        kC<<<grid, NT, smC, stream>>>(p, use_ws ? 1 : 0);
    }
    return (int)cudaGetLastError();
}

template <typename T>
int launch_dims(const BiglaParams& p, cudaStream_t stream) {
#define VIG_CASE(DKV, DVV) if (p.dk == DKV && p.dv == DVV) return launch_typed<DKV, DVV, T>(p, stream);
    VIG_CASE(16, 32) VIG_CASE(32, 32) VIG_CASE(16, 64) VIG_CASE(32, 64) VIG_CASE(64, 64) VIG_CASE(128, 64)
    VIG_CASE(32, 128) VIG_CASE(64, 128) VIG_CASE(128, 128) VIG_CASE(64, 32) VIG_CASE(128, 32) VIG_CASE(16, 128)
#undef VIG_CASE
    return VIG_ERR_SHAPE;
}

}  // namespace

size_t bigla_simt_workspace(int B, int H, int L, int dk, int dv) {
    const size_t nchunk = (L + CH - 1) / CH;
    return (size_t)B * H * nchunk * 2 * ((size_t)dk * dv + dk) * sizeof(float);
}

int bigla_scan_launch(const BiglaParams& p, cudaStream_t stream) {
    const int per = (p.dk * p.dv + NT - 1) / NT;
    bigla_simt_state_scan<<<p.B * p.H * 2 * per, NT, 0, stream>>>(p);
    return (int)cudaGetLastError();
}

int bigla_simt_launch(const BiglaParams& p_in, cudaStream_t stream) {
    BiglaParams p = p_in;
    p.nchunk = (p.L + CH - 1) / CH;
    switch (p.dtype) {
        case VIG_DTYPE_F32: return launch_dims<float>(p, stream);
        case VIG_DTYPE_BF16: return launch_dims<__nv_bfloat16>(p, stream);
        case VIG_DTYPE_F16: return launch_dims<__half>(p, stream);
    }
    return VIG_ERR_DTYPE;
}

}  // namespace vig
