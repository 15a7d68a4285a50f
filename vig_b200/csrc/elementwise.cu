// Bandwidth-bound kernels of the ViG block: depthwise 3x3 conv in token-major layout, the 2-D gating
// locality injection, residual-add + RMSNorm, SwiGLU.  Every global access is a 16-byte vector;
// arithmetic and statistics are fp32.
#include <type_traits>
#include "common.cuh"

namespace vig {
namespace {

constexpr int EW_THREADS = 256;

// packed pair of 16-bit values <-> two floats
template <typename T> struct DType2;
template <> struct DType2<__nv_bfloat16> {
    __device__ static float2 to_f2(uint32_t u) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u)); }
    __device__ static uint32_t from_f2(float a, float b) { const __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<const uint32_t*>(&t); }
};
template <> struct DType2<__half> {
    __device__ static float2 to_f2(uint32_t u) { return __half22float2(*reinterpret_cast<const __half2*>(&u)); }
    __device__ static uint32_t from_f2(float a, float b) { const __half2 t = __floats2half2_rn(a, b); return *reinterpret_cast<const uint32_t*>(&t); }
};
template <> struct DType2<float> {                            // never instantiated for work; keeps templates well-formed
    __device__ static float2 to_f2(uint32_t) { return make_float2(0.f, 0.f); }
    __device__ static uint32_t from_f2(float, float) { return 0u; }
};

// ---------------------------------------------------------------------------------------------------
// Depthwise 3x3 conv, x: [B, h*w, C] (C contiguous).  One thread per (token, 16-byte channel group); its nine
// independent 16-byte loads are in flight together.  The taps of a token sit in rows y-1..y+1 of the image:
// the re-reads hit L1 (same row) or L2 (neighbouring rows), so DRAM traffic stays at one read + one write
// of the tensor.  Index arithmetic is 32-bit (the host rejects tensors with 2^31 or more vectors).
template <typename T>
__global__ void __launch_bounds__(EW_THREADS) dwconv3x3_kernel(const T* __restrict__ x, const T* __restrict__ wt,
                                                               const T* __restrict__ bias, T* __restrict__ y,
                                                               int B, int h, int w, int C, int act) {
    constexpr int V = DType<T>::VEC;
    const uint32_t cv = C / V;
    const uint32_t total = (uint32_t)B * h * w * cv;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < total; it += gridDim.x * blockDim.x) {
        const uint32_t c0 = (it % cv) * V;
        const uint32_t tok = it / cv;
        const int xx = (int)(tok % (uint32_t)w);
        const int yy = (int)((tok / (uint32_t)w) % (uint32_t)h);
        Vec16<T> xv[9];
        bool ok[9];
#pragma unroll
        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
            for (int kx = 0; kx < 3; ++kx) {
                const int y2 = yy + ky - 1, x2 = xx + kx - 1;
                ok[ky * 3 + kx] = y2 >= 0 && y2 < h && x2 >= 0 && x2 < w;
                if (ok[ky * 3 + kx]) xv[ky * 3 + kx].load_nc(x + ((size_t)tok + (ky - 1) * w + (kx - 1)) * C + c0);
            }
        float acc[V];
        if (bias) {
            Vec16<T> bv; bv.load_nc(bias + c0); bv.to_float(acc);
        } else {
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = 0.f;
        }
#pragma unroll
        for (int t = 0; t < 9; ++t) {
            if (!ok[t]) continue;
            Vec16<T> wv; wv.load_nc(wt + t * C + c0);
            float xf[V], wf[V];
            xv[t].to_float(xf); wv.to_float(wf);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = fmaf(xf[i], wf[i], acc[i]);
        }
        if (act) {
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] *= sigmoid_t<T>(acc[i]);
        }
        Vec16<T> ov; ov.from_float(acc); ov.store(y + (size_t)tok * C + c0);
    }
}

// ---------------------------------------------------------------------------------------------------
// Depthwise 3x3 conv for 16-bit types, sliding-window form.  A thread owns 4 channels and a run of RUN consecutive
// tokens of one image row: its 36 taps live in registers as fp32 (unpacked once), and every step loads only the three
// new inputs of the window's right column (8-byte loads), so an output costs 3 loads + 12 unpacks + 36 FMAs instead
// of 9 loads + 9 tap loads + 144 unpacks.  (The 16-byte form above spends most of its time unpacking on the
// half-rate integer pipe.)  Consecutive threads own consecutive channel groups, so loads and stores are coalesced.
template <typename T, int RUN>
__global__ void __launch_bounds__(EW_THREADS, 2) dwconv3x3_rows_kernel(const T* __restrict__ x, const T* __restrict__ wt,
                                                                    const T* __restrict__ bias, T* __restrict__ y,
                                                                    int B, int h, int w, int C, int act,
                                                                    const T* __restrict__ top, const T* __restrict__ bottom) {
    using P2 = typename std::conditional<std::is_same<T, __half>::value, __half2, __nv_bfloat162>::type;
    const uint32_t cq = C / 4, nrun = (w + RUN - 1) / RUN;
    const uint32_t total = (uint32_t)B * h * nrun * cq;
    const uint32_t gid = blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= total) return;
    const uint32_t c0 = (gid % cq) * 4;
    uint32_t r = gid / cq;
    const int x0 = (int)(r % nrun) * RUN; r /= nrun;
    const int yy = (int)(r % (uint32_t)h);
    const uint32_t b = r / (uint32_t)h;
    auto unpack4 = [](uint2 v, float* f) {
        const float2 a = DType2<T>::to_f2(v.x), c = DType2<T>::to_f2(v.y);
        f[0] = a.x; f[1] = a.y; f[2] = c.x; f[3] = c.y;
    };
    float tap[9][4];
#pragma unroll
    for (int k = 0; k < 9; ++k) unpack4(__ldg(reinterpret_cast<const uint2*>(wt + (size_t)k * C + c0)), tap[k]);
    float bf[4] = {0.f, 0.f, 0.f, 0.f};
    if (bias) unpack4(__ldg(reinterpret_cast<const uint2*>(bias + c0)), bf);
    const T* rowp[3];
    bool rok[3];
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) {
        const int y2 = yy + ky - 1;
        rok[ky] = y2 >= 0 && y2 < h;
        rowp[ky] = x + (((size_t)b * h + (rok[ky] ? y2 : yy)) * w) * C + c0;
        // rows just outside the slab come from the halo rows ([B, w, C]) when the caller has them: the slab is then a
        // band of a taller image whose other rows live elsewhere (another GPU); without them the slab is the whole image
        if (y2 < 0 && top) { rok[ky] = true; rowp[ky] = top + ((size_t)b * w) * C + c0; }
        if (y2 >= h && bottom) { rok[ky] = true; rowp[ky] = bottom + ((size_t)b * w) * C + c0; }
    }
    auto load_col = [&](int xx, uint2* raw) {                 // the three inputs of image column xx (zeros outside the image)
#pragma unroll
        for (int ky = 0; ky < 3; ++ky)
            raw[ky] = (rok[ky] && xx >= 0 && xx < w) ? __ldg(reinterpret_cast<const uint2*>(rowp[ky] + (size_t)xx * C)) : make_uint2(0u, 0u);
    };
    float win[3][3][4];                                       // [column slot][row][channel]; slot of image column xx is (xx - x0 + 1) % 3
    constexpr int PF = 3;                                     // columns in flight
    uint2 raw[PF][3];
    load_col(x0 - 1, raw[0]);
    load_col(x0, raw[1]);
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) unpack4(raw[0][ky], win[0][ky]);
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) unpack4(raw[1][ky], win[1][ky]);
#pragma unroll
    for (int j = 0; j < PF; ++j) load_col(x0 + 1 + j, raw[j]);
    T* yp = y + (((size_t)b * h + yy) * w) * C + c0;
#pragma unroll
    for (int i = 0; i < RUN; ++i) {
        const int xx = x0 + i;
        if (xx >= w) break;
        const int sl = i % 3, sc = (i + 1) % 3, sr = (i + 2) % 3;     // slots of columns xx-1, xx, xx+1 (static: the loop is unrolled)
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) unpack4(raw[i % PF][ky], win[sr][ky]);
        if (i + PF < RUN) load_col(xx + 1 + PF, raw[i % PF]); // the right columns of the next PF steps are in flight during this step's math
        float acc[4] = {bf[0], bf[1], bf[2], bf[3]};
#pragma unroll
        for (int ky = 0; ky < 3; ++ky)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                acc[c] = fmaf(win[sl][ky][c], tap[ky * 3 + 0][c], acc[c]);
                acc[c] = fmaf(win[sc][ky][c], tap[ky * 3 + 1][c], acc[c]);
                acc[c] = fmaf(win[sr][ky][c], tap[ky * 3 + 2][c], acc[c]);
            }
        if (act) {
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[c] *= sigmoid_t<T>(acc[c]);
        }
        uint2 o;
        o.x = DType2<T>::from_f2(acc[0], acc[1]); o.y = DType2<T>::from_f2(acc[2], acc[3]);
        *reinterpret_cast<uint2*>(yp + (size_t)xx * C) = o;
    }
}

// ---------------------------------------------------------------------------------------------------
// Gating injection.  LPG lanes share one (token, head) group of dv = LPG * VEC values.
template <typename T, int LPG>
__global__ void __launch_bounds__(EW_THREADS) gate_inject_kernel(const T* __restrict__ o, int64_t so_b, int64_t so_h, int64_t so_l,
                                                                 const T* __restrict__ local, const T* __restrict__ gl,
                                                                 const T* __restrict__ wg, const T* __restrict__ wl,
                                                                 T* __restrict__ y, int64_t ld_local, int64_t ld_gate, int64_t ld_y,
                                                                 int B, int H, int L, float eps, int out_act) {
    constexpr int V = DType<T>::VEC;
    constexpr int DV = LPG * V;
    const uint32_t groups = (uint32_t)B * L * H;
    const int lane = threadIdx.x % LPG;
    float wgf[V], wlf[V];
    { Vec16<T> t; t.load_nc(wg + lane * V); t.to_float(wgf); t.load_nc(wl + lane * V); t.to_float(wlf); }
    for (uint32_t g = (blockIdx.x * blockDim.x + threadIdx.x) / LPG; g < groups; g += gridDim.x * blockDim.x / LPG) {
        const int hh = (int)(g % (uint32_t)H);
        const uint32_t bl32 = g / (uint32_t)H;
        const int l = (int)(bl32 % (uint32_t)L);
        const int b = (int)(bl32 / (uint32_t)L);
        const int64_t bl = bl32;
        const int64_t col = hh * DV + lane * V;          // column inside the [B*L, H*dv] operands
        Vec16<T> ov, lv, gv;
        ov.load_nc(o + b * so_b + hh * so_h + (int64_t)l * so_l + lane * V);
        lv.load_nc(local + bl * ld_local + col);
        gv.load_nc(gl + bl * ld_gate + col);
        float of[V], lf[V], gf[V];
        ov.to_float(of); lv.to_float(lf); gv.to_float(gf);
        float so2 = 0.f, sl2 = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) { so2 = fmaf(of[i], of[i], so2); sl2 = fmaf(lf[i], lf[i], sl2); }
#pragma unroll
        for (int m = 1; m < LPG; m <<= 1) {
            so2 += __shfl_xor_sync(0xffffffffu, so2, m);
            sl2 += __shfl_xor_sync(0xffffffffu, sl2, m);
        }
        const float ro = rsqrtf(so2 * (1.f / DV) + eps), rl = rsqrtf(sl2 * (1.f / DV) + eps);
        float out[V];
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const float gate = sigmoid_t<T>(gf[i]);
            float val = of[i] * ro * wgf[i] * gate + lf[i] * rl * wlf[i] * (1.f - gate);
            if (out_act) val = val * sigmoid_t<T>(val);
            out[i] = val;
        }
        Vec16<T> yv; yv.from_float(out); yv.store(y + bl * ld_y + col);
    }
}

// ---------------------------------------------------------------------------------------------------
// (x + residual) -> RMSNorm.  One warp per row, the row stays in registers (MAXV vectors per lane).
template <typename T, int MAXV>
__global__ void __launch_bounds__(EW_THREADS) add_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ res,
                                                                 const T* __restrict__ w, T* __restrict__ y,
                                                                 T* __restrict__ res_out, int64_t rows, int N, float eps) {
    constexpr int V = DType<T>::VEC;
    const int lane = threadIdx.x & 31;
    const int nv = N / V;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp0; r < rows; r += nwarps) {
        float val[MAXV][V];
        float ss = 0.f;
#pragma unroll
        for (int m = 0; m < MAXV; ++m) {
            const int vi = lane + m * 32;
            if (vi < nv) {
                Vec16<T> xv; xv.load_nc(x + r * N + vi * V); xv.to_float(val[m]);
                if (res) {
                    Vec16<T> rv; rv.load_nc(res + r * N + vi * V);
                    float rf[V]; rv.to_float(rf);
#pragma unroll
                    for (int i = 0; i < V; ++i) val[m][i] += rf[i];
                    // the reference rounds the sum to the tensor dtype before the norm (rms_norm_ref: (x + residual).to(x.dtype))
                    Vec16<T> sv; sv.from_float(val[m]); sv.to_float(val[m]);
                    if (res_out) sv.store(res_out + r * N + vi * V);
                } else if (res_out) {
                    xv.store(res_out + r * N + vi * V);
                }
#pragma unroll
                for (int i = 0; i < V; ++i) ss = fmaf(val[m][i], val[m][i], ss);
            }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        const float rstd = rsqrtf(ss / (float)N + eps);
#pragma unroll
        for (int m = 0; m < MAXV; ++m) {
            const int vi = lane + m * 32;
            if (vi < nv) {
                Vec16<T> wv; wv.load_nc(w + vi * V);
                float wf[V]; wv.to_float(wf);
#pragma unroll
                for (int i = 0; i < V; ++i) val[m][i] = val[m][i] * rstd * wf[i];
                Vec16<T> ov; ov.from_float(val[m]); ov.store(y + r * N + vi * V);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// LayerNorm over the last dimension with affine parameters and an optional swish: the two LayerNorm2d
// stages of the patch-embedding stem on channels-last activations.  One warp per row, row in registers.
// Rows of at most 16 vectors (N <= 128 for 2-byte types): LPR = 8 or 16 lanes per row, several rows per warp.
template <typename T, int LPR>
__global__ void __launch_bounds__(EW_THREADS) layernorm_act_short_kernel(const T* __restrict__ x, const T* __restrict__ pre_bias,
                                                                         const T* __restrict__ w, const T* __restrict__ bias,
                                                                         T* __restrict__ y, int64_t rows, int N, float eps, int act) {
    constexpr int V = DType<T>::VEC;
    const int sub = threadIdx.x % LPR;
    const int nv = N / V;
    const int64_t g0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / LPR;
    const int64_t ng = ((int64_t)gridDim.x * blockDim.x) / LPR;
    const bool active = sub < nv;
    float wf[V], bf[V], pf[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { wf[i] = 0.f; bf[i] = 0.f; pf[i] = 0.f; }
    if (active) {
        Vec16<T> t; t.load_nc(w + sub * V); t.to_float(wf); t.load_nc(bias + sub * V); t.to_float(bf);
        if (pre_bias) { t.load_nc(pre_bias + sub * V); t.to_float(pf); }
    }
    constexpr int U = 2;                                                   // rows in flight per lane group
    for (int64_t r0 = g0; r0 < rows; r0 += U * ng) {
        float val[U][V];
        Vec16<T> xv[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (active && r0 + u * ng < rows) xv[u].load_nc(x + (r0 + u * ng) * N + sub * V);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t r = r0 + u * ng;
            const bool on = active && r < rows;
            float sum = 0.f;
            if (on) {
                xv[u].to_float(val[u]);
                if (pre_bias) {
#pragma unroll
                    for (int i = 0; i < V; ++i) val[u][i] = DType<T>::to_f(DType<T>::from_f(val[u][i] + pf[i]));
                }
#pragma unroll
                for (int i = 0; i < V; ++i) sum += val[u][i];
            }
#pragma unroll
            for (int m = LPR / 2; m >= 1; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
            const float mean = sum / (float)N;
            float ss = 0.f;
            if (on) {
#pragma unroll
                for (int i = 0; i < V; ++i) { const float d = val[u][i] - mean; ss = fmaf(d, d, ss); }
            }
#pragma unroll
            for (int m = LPR / 2; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
            const float rstd = rsqrtf(ss / (float)N + eps);
            if (on) {
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    float t = (val[u][i] - mean) * rstd * wf[i] + bf[i];
                    if (act) t *= sigmoid_t<T>(t);
                    val[u][i] = t;
                }
                Vec16<T> ov; ov.from_float(val[u]); ov.store(y + r * N + sub * V);
            }
        }
    }
}

template <typename T, int MAXV>
__global__ void __launch_bounds__(EW_THREADS) layernorm_act_kernel(const T* __restrict__ x, const T* __restrict__ pre_bias,
                                                                   const T* __restrict__ w, const T* __restrict__ bias,
                                                                   const T* __restrict__ post_add, int64_t post_period,
                                                                   T* __restrict__ y, int64_t rows, int N, float eps, int act,
                                                                   const T* __restrict__ rms_w, float rms_eps, T* __restrict__ h_out) {
    constexpr int V = DType<T>::VEC;
    const int lane = threadIdx.x & 31;
    const int nv = N / V;
    const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp0; r < rows; r += nwarps) {
        float val[MAXV][V];
        float sum = 0.f;
#pragma unroll
        for (int m = 0; m < MAXV; ++m) {
            const int vi = lane + m * 32;
            if (vi < nv) {
                Vec16<T> xv; xv.load_nc(x + r * N + vi * V); xv.to_float(val[m]);
                if (pre_bias) {                          // per-channel bias of the producing convolution, folded in here
                    Vec16<T> pv; pv.load_nc(pre_bias + vi * V);
                    float pf[V]; pv.to_float(pf);
#pragma unroll
                    for (int i = 0; i < V; ++i) val[m][i] = DType<T>::to_f(DType<T>::from_f(val[m][i] + pf[i]));
                }
#pragma unroll
                for (int i = 0; i < V; ++i) sum += val[m][i];
            }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
        const float mean = sum / (float)N;
        float ss = 0.f;
#pragma unroll
        for (int m = 0; m < MAXV; ++m) {
            const int vi = lane + m * 32;
            if (vi < nv) {
#pragma unroll
                for (int i = 0; i < V; ++i) { const float d = val[m][i] - mean; ss = fmaf(d, d, ss); }
            }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        const float rstd = rsqrtf(ss / (float)N + eps);
        float ss2 = 0.f;                                 // sum of squares of the finished row, for the RMSNorm that may follow
#pragma unroll
        for (int m = 0; m < MAXV; ++m) {
            const int vi = lane + m * 32;
            if (vi < nv) {
                Vec16<T> wv, bv; wv.load_nc(w + vi * V); bv.load_nc(bias + vi * V);
                float wf[V], bf[V]; wv.to_float(wf); bv.to_float(bf);
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    float t = (val[m][i] - mean) * rstd * wf[i] + bf[i];
                    if (act) t *= sigmoid_t<T>(t);
                    val[m][i] = t;
                }
                Vec16<T> ov; ov.from_float(val[m]);
                if (post_add) {                          // e.g. the position embedding: added to the rounded result, like a separate add
                    Vec16<T> pv; pv.load_nc(post_add + (r % post_period) * N + vi * V);
                    float pf[V]; pv.to_float(pf); ov.to_float(val[m]);
#pragma unroll
                    for (int i = 0; i < V; ++i) val[m][i] += pf[i];
                    ov.from_float(val[m]);
                }
                ov.store(y + r * N + vi * V);
                if (h_out) {                             // the rounded row, as a separate norm kernel would read it
                    ov.to_float(val[m]);
#pragma unroll
                    for (int i = 0; i < V; ++i) ss2 = fmaf(val[m][i], val[m][i], ss2);
                }
            }
        }
        if (h_out) {                                     // h = RMSNorm(y) * rms_w: the arithmetic of add_rmsnorm_kernel
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1) ss2 += __shfl_xor_sync(0xffffffffu, ss2, m);
            const float rstd2 = rsqrtf(ss2 / (float)N + rms_eps);
#pragma unroll
            for (int m = 0; m < MAXV; ++m) {
                const int vi = lane + m * 32;
                if (vi < nv) {
                    Vec16<T> wv; wv.load_nc(rms_w + vi * V);
                    float wf[V]; wv.to_float(wf);
#pragma unroll
                    for (int i = 0; i < V; ++i) val[m][i] = val[m][i] * rstd2 * wf[i];
                    Vec16<T> hv; hv.from_float(val[m]); hv.store(h_out + r * N + vi * V);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(EW_THREADS) swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ yy,
                                                            T* __restrict__ out, int64_t rows, int I, int64_t ld_in, int64_t ld_out) {
    constexpr int V = DType<T>::VEC;
    const uint32_t iv = I / V;
    const uint32_t total = (uint32_t)rows * iv;
    for (uint32_t it = blockIdx.x * blockDim.x + threadIdx.x; it < total; it += gridDim.x * blockDim.x) {
        const int64_t r = it / iv;
        const int c0 = (int)(it % iv) * V;
        Vec16<T> gv, yv;
        gv.load_nc(gate + r * ld_in + c0);
        yv.load_nc(yy + r * ld_in + c0);
        float gf[V], yf[V];
        gv.to_float(gf); yv.to_float(yf);
#pragma unroll
        for (int i = 0; i < V; ++i) gf[i] = gf[i] * yf[i] * sigmoid_t<T>(gf[i]);
        Vec16<T> ov; ov.from_float(gf); ov.store(out + r * ld_out + c0);
    }
}

// ---------------------------------------------------------------------------------------------------
// Space-to-depth of the input image for the stem's first convolution (kernel s+1, stride s, padding 1, evaluated
// as a 2x2 convolution over s x s pixel blocks): x [B, Cin, H, W]  ->  cells [B, H/s + 1, W/s + 1, s*s*Cin] with
// cells[b, cy, cx, (dy*s + dx)*Cin + ic] = x[b, ic, s*cy + dy - 1, s*cx + dx - 1] (zero outside the image).
// A block owns up to UNFOLD_CELLS consecutive cells of one cell row: it stages the 8 image rows x Cin planes that
// those cells cover in shared memory with aligned 16-byte loads (each image byte is read once, apart from one
// 8-pixel overlap between neighbouring blocks), then writes the cells, which are contiguous in memory, as 16-byte
// vectors gathered from the staged tile.
constexpr int UNFOLD_S = 8, UNFOLD_CIN = 3, UNFOLD_CELLS = 32;
constexpr int UNFOLD_TW = UNFOLD_S * (UNFOLD_CELLS + 1);                 // staged pixels per row: 8 before the first cell

template <typename T>
__global__ void __launch_bounds__(EW_THREADS) stem_unfold_kernel(const T* __restrict__ x, T* __restrict__ cells,
                                                                 int H, int W, int nseg) {
    constexpr int V = DType<T>::VEC, S = UNFOLD_S, C = UNFOLD_CIN;
    constexpr int CELL = S * S * C;                                       // 192 values per cell
    __shared__ __align__(16) T tile[S][C][UNFOLD_TW];
    const int ch = H / S + 1, cw = W / S + 1;
    int blk = blockIdx.x;
    const int seg = blk % nseg; blk /= nseg;
    const int cy = blk % ch;
    const int b = blk / ch;
    const int cx0 = seg * UNFOLD_CELLS;
    const int ncell = min(UNFOLD_CELLS, cw - cx0);
    const int px0 = S * cx0 - S;                                          // image x of staged column 0
    constexpr int VPR = UNFOLD_TW / V;                                    // vectors per staged row
    for (int i = threadIdx.x; i < S * C * VPR; i += EW_THREADS) {
        const int j = i % VPR, ic = (i / VPR) % C, dy = i / (VPR * C);
        const int y = S * cy + dy - 1, xx = px0 + j * V;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (y >= 0 && y < H && xx >= 0 && xx < W)                         // W is a multiple of 8: a vector is all in or all out
            val = __ldg(reinterpret_cast<const uint4*>(x + (((size_t)b * C + ic) * H + y) * W + xx));
        *reinterpret_cast<uint4*>(&tile[dy][ic][j * V]) = val;
    }
    __syncthreads();
    T* dst = cells + (((size_t)b * ch + cy) * cw + cx0) * CELL;
    const T* flat = &tile[0][0][0];
    for (int vi = threadIdx.x; vi < ncell * CELL / V; vi += EW_THREADS) {
        alignas(16) T vals[V];
        // element e = vi*V + i of the cell row is (cell, dy, dx, ic); the indices are split once and then stepped
        const int e0 = vi * V;
        int cell = e0 / CELL, r = e0 % CELL;
        int dy = r / (S * C), dx = (r % (S * C)) / C, ic = r % C;
        int off = (dy * C + ic) * UNFOLD_TW + S * cell + dx + S - 1;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            vals[i] = flat[off];
            ++ic; off += UNFOLD_TW;
            if (ic == C) {
                ic = 0; off -= C * UNFOLD_TW - 1; ++dx;
                if (dx == S) {
                    dx = 0; off += C * UNFOLD_TW - S; ++dy;
                    if (dy == S) { dy = 0; off -= S * C * UNFOLD_TW - S; }
                }
            }
        }
        reinterpret_cast<uint4*>(dst)[vi] = *reinterpret_cast<const uint4*>(vals);
    }
}

inline int grid_for(int64_t items, int per_block) {
    int64_t g = (items + per_block - 1) / per_block;
    const int64_t cap = 148 * 16;       // 148 SMs x resident CTAs; the kernels are grid-stride
    return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
int dwconv_t(const void* x, const void* wt, const void* bias, void* y, int B, int h, int w, int C, int act, cudaStream_t s,
             const void* top = nullptr, const void* bottom = nullptr) {
    constexpr int V = DType<T>::VEC;
    if (C % V) return VIG_ERR_SHAPE;
    if ((top || bottom) && !(sizeof(T) == 2 && C % 4 == 0)) return VIG_ERR_SHAPE;   // halo rows: 16-bit sliding-window form only
    const int64_t items = (int64_t)B * h * w * (C / V);
    if (items >= (1ll << 31)) return VIG_ERR_SHAPE;                             // 32-bit index arithmetic in the kernel
    if (sizeof(T) == 2 && C % 4 == 0) {                     // sliding-window form: 4 channels x RUN tokens per thread
        constexpr int RUN = 16;
        const int64_t threads = (int64_t)B * h * ((w + RUN - 1) / RUN) * (C / 4);
        if (threads < (1ll << 31)) {
            dwconv3x3_rows_kernel<T, RUN><<<(unsigned)((threads + EW_THREADS - 1) / EW_THREADS), EW_THREADS, 0, s>>>(
                (const T*)x, (const T*)wt, (const T*)bias, (T*)y, B, h, w, C, act, (const T*)top, (const T*)bottom);
            return (int)cudaGetLastError();
        }
        if (top || bottom) return VIG_ERR_SHAPE;
    }
    dwconv3x3_kernel<T><<<grid_for(items, EW_THREADS), EW_THREADS, 0, s>>>((const T*)x, (const T*)wt, (const T*)bias, (T*)y, B, h, w, C, act);
    return (int)cudaGetLastError();
}

template <typename T>
int gate_inject_t(const void* o, const int64_t* so, const void* local, const void* gl, const void* wg, const void* wl, void* y,
                  int64_t ld_local, int64_t ld_gate, int64_t ld_y, int B, int H, int L, int dv, float eps, int out_act, cudaStream_t s) {
    constexpr int V = DType<T>::VEC;
    const int lpg = dv / V;
    if (dv % V || (so[0] % V) || (so[1] % V) || (so[2] % V) || (ld_local % V) || (ld_gate % V) || (ld_y % V)) return VIG_ERR_ALIGN;
    const int64_t threads = (int64_t)B * L * H * lpg;
    if (threads >= (1ll << 31)) return VIG_ERR_SHAPE;                           // 32-bit index arithmetic in the kernel
    const int grid = grid_for(threads, EW_THREADS);
#define VIG_GI(LPG) case LPG: gate_inject_kernel<T, LPG><<<grid, EW_THREADS, 0, s>>>((const T*)o, so[0], so[1], so[2], (const T*)local, \
        (const T*)gl, (const T*)wg, (const T*)wl, (T*)y, ld_local, ld_gate, ld_y, B, H, L, eps, out_act); break;
    switch (lpg) { VIG_GI(4) VIG_GI(8) VIG_GI(16) VIG_GI(32) default: return VIG_ERR_SHAPE; }
#undef VIG_GI
    return (int)cudaGetLastError();
}

template <typename T>
int add_rmsnorm_t(const void* x, const void* res, const void* w, void* y, void* res_out, int64_t rows, int N, float eps, cudaStream_t s) {
    constexpr int V = DType<T>::VEC;
    if (N % V) return VIG_ERR_SHAPE;
    const int nv = N / V;
    const int grid = grid_for(rows * 32, EW_THREADS);
#define VIG_RN(MV) add_rmsnorm_kernel<T, MV><<<grid, EW_THREADS, 0, s>>>((const T*)x, (const T*)res, (const T*)w, (T*)y, (T*)res_out, rows, N, eps)
    if (nv <= 32) VIG_RN(1); else if (nv <= 64) VIG_RN(2); else if (nv <= 128) VIG_RN(4);
    else if (nv <= 256) VIG_RN(8); else if (nv <= 512 && V == 4) VIG_RN(16); else return VIG_ERR_SHAPE;
#undef VIG_RN
    return (int)cudaGetLastError();
}

template <typename T>
int layernorm_act_t(const void* x, const void* pb, const void* w, const void* b, const void* pa, int64_t pa_period, void* y, int64_t rows, int N,
                    float eps, int act, cudaStream_t s, const void* rms_w = nullptr, float rms_eps = 0.f, void* h_out = nullptr) {
    constexpr int V = DType<T>::VEC;
    if (N % V) return VIG_ERR_SHAPE;
    const int nv = N / V;
    if (nv <= 16 && !pa && !h_out) {
        const int lpr = nv <= 8 ? 8 : 16;
        const int g = grid_for(rows * lpr, EW_THREADS);
        if (lpr == 8) layernorm_act_short_kernel<T, 8><<<g, EW_THREADS, 0, s>>>((const T*)x, (const T*)pb, (const T*)w, (const T*)b, (T*)y, rows, N, eps, act);
        else layernorm_act_short_kernel<T, 16><<<g, EW_THREADS, 0, s>>>((const T*)x, (const T*)pb, (const T*)w, (const T*)b, (T*)y, rows, N, eps, act);
        return (int)cudaGetLastError();
    }
    const int grid = grid_for(rows * 32, EW_THREADS);
#define VIG_LN(MV) layernorm_act_kernel<T, MV><<<grid, EW_THREADS, 0, s>>>((const T*)x, (const T*)pb, (const T*)w, (const T*)b, (const T*)pa, pa_period, (T*)y, rows, N, eps, act, (const T*)rms_w, rms_eps, (T*)h_out)
    if (nv <= 32) VIG_LN(1); else if (nv <= 64) VIG_LN(2); else if (nv <= 128) VIG_LN(4);
    else if (nv <= 256) VIG_LN(8); else return VIG_ERR_SHAPE;
#undef VIG_LN
    return (int)cudaGetLastError();
}

template <typename T>
int swiglu_t(const void* g, const void* yy, void* out, int64_t rows, int I, int64_t ld_in, int64_t ld_out, cudaStream_t s) {
    constexpr int V = DType<T>::VEC;
    if (I % V || ld_in % V || ld_out % V) return VIG_ERR_ALIGN;
    if (rows * (I / V) >= (1ll << 31)) return VIG_ERR_SHAPE;                     // 32-bit index arithmetic in the kernel
    swiglu_kernel<T><<<grid_for(rows * (I / V), EW_THREADS), EW_THREADS, 0, s>>>((const T*)g, (const T*)yy, (T*)out, rows, I, ld_in, ld_out);
    return (int)cudaGetLastError();
}

}  // namespace
}  // namespace vig

using namespace vig;

#define VIG_DISPATCH(dtype, CALL)                                   \
    switch (dtype) {                                                \
        case VIG_DTYPE_F32: { using T = float; return CALL; }        \
        case VIG_DTYPE_BF16: { using T = __nv_bfloat16; return CALL; } \
        case VIG_DTYPE_F16: { using T = __half; return CALL; }       \
        default: return VIG_ERR_DTYPE;                              \
    }

extern "C" int vig_dwconv3x3_fwd(const void* x, const void* wt, const void* bias, void* y, int B, int h, int w, int C,
                                 int act_silu, int dtype, int32_t* status_dev, void* stream) {
    if (!x || !wt || !y) return VIG_ERR_NULL;
    if (B < 0 || h <= 0 || w <= 0 || C <= 0) return VIG_ERR_SHAPE;
    if (B == 0) return VIG_OK;
    if (!aligned16(x) || !aligned16(wt) || !aligned16(y) || (bias && !aligned16(bias))) return VIG_ERR_ALIGN;
    // large 16-bit problems: the TMA-fed form (bit-identical results); everything else: the register sliding-window forms
    const int taken = dwconv_tma_try(x, wt, bias, y, B, h, w, C, act_silu, dtype, status_dev, (cudaStream_t)stream);
    if (taken != VIG_DWCONV_NOT_TAKEN) return taken;
    VIG_DISPATCH(dtype, dwconv_t<T>(x, wt, bias, y, B, h, w, C, act_silu, (cudaStream_t)stream))
}

extern "C" int vig_dwconv3x3_halo_fwd(const void* x, const void* top, const void* bottom, const void* wt, const void* bias, void* y,
                                      int B, int h, int w, int C, int act_silu, int dtype, void* stream) {
    if (!x || !wt || !y) return VIG_ERR_NULL;
    if (B < 0 || h <= 0 || w <= 0 || C <= 0) return VIG_ERR_SHAPE;
    if (dtype != VIG_DTYPE_BF16 && dtype != VIG_DTYPE_F16) return VIG_ERR_DTYPE;
    if (B == 0) return VIG_OK;
    if (!aligned16(x) || !aligned16(wt) || !aligned16(y) || (bias && !aligned16(bias)) || (top && !aligned16(top)) ||
        (bottom && !aligned16(bottom))) return VIG_ERR_ALIGN;
    VIG_DISPATCH(dtype, dwconv_t<T>(x, wt, bias, y, B, h, w, C, act_silu, (cudaStream_t)stream, top, bottom))
}

extern "C" int vig_gate_inject_fwd(const void* o, const int64_t* strides_o, const void* local, const void* gate_logits,
                                   const void* w_gnorm, const void* w_lnorm, void* y,
                                   int64_t ld_local, int64_t ld_gate, int64_t ld_y, int B, int H, int L, int dv,
                                   float eps, int out_act_swish, int dtype, void* stream) {
    if (!o || !local || !gate_logits || !w_gnorm || !w_lnorm || !y) return VIG_ERR_NULL;
    if (B < 0 || H <= 0 || L < 0 || dv <= 0) return VIG_ERR_SHAPE;
    if (ld_local < (int64_t)H * dv || ld_gate < (int64_t)H * dv || ld_y < (int64_t)H * dv) return VIG_ERR_ARG;
    if (B == 0 || L == 0) return VIG_OK;
    if (!aligned16(o) || !aligned16(local) || !aligned16(gate_logits) || !aligned16(y) || !aligned16(w_gnorm) || !aligned16(w_lnorm))
        return VIG_ERR_ALIGN;
    int64_t so[3] = {(int64_t)H * L * dv, (int64_t)L * dv, dv};
    if (strides_o) { so[0] = strides_o[0]; so[1] = strides_o[1]; so[2] = strides_o[2]; }
    VIG_DISPATCH(dtype, gate_inject_t<T>(o, so, local, gate_logits, w_gnorm, w_lnorm, y, ld_local, ld_gate, ld_y, B, H, L, dv, eps, out_act_swish, (cudaStream_t)stream))
}

extern "C" int vig_add_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* residual_out,
                                   int64_t rows, int N, float eps, int dtype, void* stream) {
    if (!x || !w || !y) return VIG_ERR_NULL;
    if (rows < 0 || N <= 0) return VIG_ERR_SHAPE;
    if (rows == 0) return VIG_OK;
    if (!aligned16(x) || !aligned16(w) || !aligned16(y) || (residual && !aligned16(residual)) || (residual_out && !aligned16(residual_out)))
        return VIG_ERR_ALIGN;
    VIG_DISPATCH(dtype, add_rmsnorm_t<T>(x, residual, w, y, residual_out, rows, N, eps, (cudaStream_t)stream))
}

extern "C" int vig_layernorm_act_fwd(const void* x, const void* pre_bias, const void* w, const void* bias, void* y, int64_t rows,
                                    int N, float eps, int act_swish, int dtype, void* stream) {
    if (!x || !w || !bias || !y) return VIG_ERR_NULL;
    if (pre_bias && !aligned16(pre_bias)) return VIG_ERR_ALIGN;
    if (rows < 0 || N <= 0) return VIG_ERR_SHAPE;
    if (rows == 0) return VIG_OK;
    if (!aligned16(x) || !aligned16(w) || !aligned16(bias) || !aligned16(y)) return VIG_ERR_ALIGN;
    VIG_DISPATCH(dtype, layernorm_act_t<T>(x, pre_bias, w, bias, nullptr, 1, y, rows, N, eps, act_swish, (cudaStream_t)stream))
}

extern "C" int vig_layernorm_act_add_fwd(const void* x, const void* pre_bias, const void* w, const void* bias, const void* post_add,
                                        int64_t post_period, void* y, int64_t rows, int N, float eps, int act_swish, int dtype, void* stream) {
    if (!x || !w || !bias || !y || !post_add) return VIG_ERR_NULL;
    if (pre_bias && !aligned16(pre_bias)) return VIG_ERR_ALIGN;
    if (rows < 0 || N <= 0 || post_period <= 0) return VIG_ERR_SHAPE;
    if (rows == 0) return VIG_OK;
    if (!aligned16(x) || !aligned16(w) || !aligned16(bias) || !aligned16(y) || !aligned16(post_add)) return VIG_ERR_ALIGN;
    VIG_DISPATCH(dtype, layernorm_act_t<T>(x, pre_bias, w, bias, post_add, post_period, y, rows, N, eps, act_swish, (cudaStream_t)stream))
}

extern "C" int vig_layernorm_act_add_rmsnorm_fwd(const void* x, const void* pre_bias, const void* w, const void* bias, const void* post_add,
                                                int64_t post_period, void* y, const void* rms_w, float rms_eps, void* h, int64_t rows, int N,
                                                float eps, int act_swish, int dtype, void* stream) {
    if (!x || !w || !bias || !y || !rms_w || !h) return VIG_ERR_NULL;
    if (pre_bias && !aligned16(pre_bias)) return VIG_ERR_ALIGN;
    if (rows < 0 || N <= 0 || (post_add && post_period <= 0)) return VIG_ERR_SHAPE;
    if (rows == 0) return VIG_OK;
    if (!aligned16(x) || !aligned16(w) || !aligned16(bias) || !aligned16(y) || !aligned16(rms_w) || !aligned16(h) || (post_add && !aligned16(post_add)))
        return VIG_ERR_ALIGN;
    VIG_DISPATCH(dtype, layernorm_act_t<T>(x, pre_bias, w, bias, post_add, post_add ? post_period : 1, y, rows, N, eps, act_swish, (cudaStream_t)stream,
                                           rms_w, rms_eps, h))
}

extern "C" int vig_stem_unfold_fwd(const void* x, void* cells, int B, int Cin, int H, int W, int s, int dtype, void* stream) {
    if (!x || !cells) return VIG_ERR_NULL;
    if (B < 0 || Cin <= 0 || H <= 0 || W <= 0 || s <= 0 || H % s || W % s) return VIG_ERR_SHAPE;
    if (s != UNFOLD_S || Cin != UNFOLD_CIN) return VIG_ERR_SHAPE;      // the ViG stem: 8 x 8 pixel blocks of RGB
    if (B == 0) return VIG_OK;
    if (!aligned16(cells) || !aligned16(x)) return VIG_ERR_ALIGN;
    const int ch = H / s + 1, cw = W / s + 1;
    const int nseg = (cw + UNFOLD_CELLS - 1) / UNFOLD_CELLS;
    const int64_t blocks = (int64_t)B * ch * nseg;
    if (blocks >= (1ll << 31)) return VIG_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    switch (dtype) {
        case VIG_DTYPE_F32: stem_unfold_kernel<float><<<(int)blocks, EW_THREADS, 0, st>>>((const float*)x, (float*)cells, H, W, nseg); break;
        case VIG_DTYPE_BF16: stem_unfold_kernel<__nv_bfloat16><<<(int)blocks, EW_THREADS, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)cells, H, W, nseg); break;
        case VIG_DTYPE_F16: stem_unfold_kernel<__half><<<(int)blocks, EW_THREADS, 0, st>>>((const __half*)x, (__half*)cells, H, W, nseg); break;
        default: return VIG_ERR_DTYPE;
    }
    return (int)cudaGetLastError();
}

extern "C" int vig_swiglu_fwd(const void* gate, const void* y, void* out, int64_t rows, int I, int64_t ld_in, int64_t ld_out,
                              int dtype, void* stream) {
    if (!gate || !y || !out) return VIG_ERR_NULL;
    if (rows < 0 || I <= 0) return VIG_ERR_SHAPE;
    if (rows == 0) return VIG_OK;
    if (!aligned16(gate) || !aligned16(y) || !aligned16(out)) return VIG_ERR_ALIGN;
    VIG_DISPATCH(dtype, swiglu_t<T>(gate, y, out, rows, I, ld_in, ld_out, (cudaStream_t)stream))
}
