// Depthwise 3x3 conv (+SiLU) for 16-bit types on [B, h*w, C] tokens, TMA-fed persistent form
// (GatedLinearAttention.in_proj of classification/models/vig.py:276-283: Conv2d(groups = d_model) -> SiLU).
//
// The sliding-window kernel in elementwise.cu keeps only ~36 KB of loads in flight per SM (8-byte loads, nine per thread),
// less than the ~44 KB the memory system needs to stream at full rate, and ran at a third of the copy bandwidth.  Here a
// CTA per SM walks tiles of 2 image rows x WB columns x CC channels.  One TMA load brings the tile with its one-pixel
// border -- 4 rows x (WB + 2) columns -- into a ring of two shared-memory stages (~100 KB each, so a whole tile is in
// flight while the previous one is computed); coordinates outside the image are filled with zeros by the TMA unit, which
// is exactly the conv's zero padding, so the kernel has no border cases.  A compute thread owns 4 channels and a run of
// 8 columns: 36 taps live in registers as fp32, the 4-row window slides along the run and yields the outputs of both
// image rows per step (4 shared-memory loads and 36 two-wide fp32 FMAs per 8 outputs).  Arithmetic (fp32, tap order, SiLU) is
// that of the sliding-window kernel, so the two forms agree bit for bit.
#include <type_traits>
#include "tc_common.cuh"

namespace vig {
namespace {

using namespace tc;

constexpr int DW_COMPUTE = 384;                // compute threads (12 warps)
constexpr int DW_THREADS = DW_COMPUTE + 32;    // + the producer warp
constexpr int DW_SEG = 8;                      // columns per thread
constexpr int DW_ROWS = 2;                     // image rows per tile
constexpr int DW_STAGES = 2;

// sigmoid of both lanes; 16-bit outputs take the one-MUFU form of sigmoid_t: 0.5 tanh(x / 2) + 0.5
template <typename T> __device__ __forceinline__ F2 f2_sigmoid(F2 x) {
    const F2 half = f2_make(0.5f, 0.5f);
    const F2 hx = f2_mul(x, half);
    float t0, t1;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(f2_lo(hx)));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(f2_hi(hx)));
    return f2_fma(half, f2_make(t0, t1), half);
}

struct DwParams {
    const void *wt, *bias;
    void* y;
    int B, h, w, C, act;
    int CC, WB, groups, nseg;                  // channels and columns per tile; channel groups of 4 and column runs per tile
    int ncb, nxb, nyb, ntiles;
    uint32_t stage_bytes, box_bytes;
    int32_t* status;
};

template <typename T>
__global__ void __launch_bounds__(DW_THREADS, 1) dwconv3x3_tma_kernel(const __grid_constant__ CUtensorMap map, const DwParams p) {
    extern __shared__ __align__(1024) uint8_t dw_smem[];
    const uint32_t sbase = smem_u32(dw_smem);
    const uint32_t bar_full = sbase + DW_STAGES * p.stage_bytes, bar_empty = bar_full + 8 * DW_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(dw_smem + DW_STAGES * p.stage_bytes + 16 * DW_STAGES);
    const Waiter waiter{abort_flag, p.status};
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < DW_STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, DW_COMPUTE / 32); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto decode = [&](int t, int& b, int& yb, int& xb, int& cb) {
        cb = 0; xb = 0;                          // one channel chunk and one column block are the common case: one division
        if (p.ncb > 1) { cb = t % p.ncb; t /= p.ncb; }
        if (p.nxb > 1) { xb = t % p.nxb; t /= p.nxb; }
        b = t / p.nyb; yb = t - b * p.nyb;
    };
    if (warp == DW_COMPUTE / 32) {
        if (lane == 0) {                        // ---- producer: one TMA load per tile, two tiles ahead at most ----
            uint32_t k = 0;
            for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++k) {
                const uint32_t s = k % DW_STAGES;
                if (k >= DW_STAGES) waiter.wait(bar_empty + 8 * s, ((k / DW_STAGES) - 1) & 1);
                if (*abort_flag) break;
                int b, yb, xb, cb;
                decode(tile, b, yb, xb, cb);
                mbar_expect_tx(bar_full + 8 * s, p.box_bytes);
                // the tile with its border: columns x0-1 .. x0+WB, rows y0-1 .. y0+2; what lies outside the image reads as zero
                tma_load_4d(sbase + s * p.stage_bytes, &map, cb * p.CC, xb * p.WB - 1, yb * DW_ROWS - 1, b, bar_full + 8 * s);
            }
        }
    } else {
        // ---- compute warps ----
        const int cg = tid % p.groups, seg = tid / p.groups;
        const bool active = seg < p.nseg;
        // Arithmetic runs on pairs of fp32 values held in 64-bit registers (fma / mul .f32x2: one instruction for two
        // channels, each lane an IEEE fma, so results equal the scalar form's): the kernel is bound by instruction issue.
        auto unpack4 = [](uint2 v, F2* f) {        // four packed 16-bit values -> two fp32 pairs
            const float2 a = Pack2<T>::unpack(v.x), c = Pack2<T>::unpack(v.y);
            f[0] = f2_make(a.x, a.y); f[1] = f2_make(c.x, c.y);
        };
        F2 tap[9][2], bf[2] = {f2_make(0.f, 0.f), f2_make(0.f, 0.f)};
        int cb_loaded = -1;
        const uint32_t row_pitch = (uint32_t)(p.WB + 2) * p.CC * 2, col_pitch = (uint32_t)p.CC * 2;
        uint32_t k = 0;
        for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++k) {
            const uint32_t s = k % DW_STAGES;
            int b, yb, xb, cb;
            decode(tile, b, yb, xb, cb);
            const int c0 = cb * p.CC + cg * 4;
            if (active && cb != cb_loaded) {   // this thread's 36 taps (and bias) of the tile's channel chunk
                const T* wt = static_cast<const T*>(p.wt);
#pragma unroll
                for (int t = 0; t < 9; ++t) unpack4(__ldg(reinterpret_cast<const uint2*>(wt + (size_t)t * p.C + c0)), tap[t]);
                if (p.bias) unpack4(__ldg(reinterpret_cast<const uint2*>(static_cast<const T*>(p.bias) + c0)), bf);
                cb_loaded = cb;
            }
            waiter.wait_lite(bar_full + 8 * s, (k / DW_STAGES) & 1);     // taken by the whole warp
            if (*abort_flag) break;
            if (active) {
                const int y0 = yb * DW_ROWS, x0 = xb * p.WB + seg * DW_SEG;
                // tile column of image column x is x - (xb * WB - 1); the window's left column of output x0 is tile column seg * SEG
                uint32_t rowp[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) rowp[r] = sbase + s * p.stage_bytes + (uint32_t)(seg * DW_SEG) * col_pitch + (uint32_t)cg * 8u + r * row_pitch;
                auto load_col = [&](F2 (*dst)[2]) {                        // the four rows of the next tile column
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        uint2 v;
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(rowp[r]));
                        unpack4(v, dst[r]);
                        rowp[r] += col_pitch;
                    }
                };
                F2 win[3][4][2];                                           // [column slot][row][channel pair]
                load_col(win[0]);
                load_col(win[1]);
                T* y = static_cast<T*>(p.y);
                T* yp = y + (((size_t)b * p.h + y0) * p.w + x0) * p.C + c0;
                const size_t row_step = (size_t)p.w * p.C;
                const bool row1 = y0 + 1 < p.h;
#pragma unroll
                for (int i = 0; i < DW_SEG; ++i) {
                    const int sl = i % 3, sc = (i + 1) % 3, sr = (i + 2) % 3;
                    load_col(win[sr]);
                    if (x0 + i < p.w) {
#pragma unroll
                        for (int r = 0; r < DW_ROWS; ++r) {
                            F2 acc[2] = {bf[0], bf[1]};
#pragma unroll
                            for (int ky = 0; ky < 3; ++ky)
#pragma unroll
                                for (int c = 0; c < 2; ++c) {
                                    acc[c] = f2_fma(win[sl][r + ky][c], tap[ky * 3 + 0][c], acc[c]);
                                    acc[c] = f2_fma(win[sc][r + ky][c], tap[ky * 3 + 1][c], acc[c]);
                                    acc[c] = f2_fma(win[sr][r + ky][c], tap[ky * 3 + 2][c], acc[c]);
                                }
                            if (p.act) {
#pragma unroll
                                for (int c = 0; c < 2; ++c) acc[c] = f2_mul(acc[c], f2_sigmoid<T>(acc[c]));
                            }
                            uint2 o;
                            o.x = Pack2<T>::pack(f2_lo(acc[0]), f2_hi(acc[0])); o.y = Pack2<T>::pack(f2_lo(acc[1]), f2_hi(acc[1]));
                            if (r == 0 || row1) *reinterpret_cast<uint2*>(yp + r * row_step) = o;
                        }
                    }
                    yp += p.C;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(bar_empty + 8 * s);          // this warp has read the stage
        }
    }
    __syncthreads();
    if (tid == 0 && *abort_flag && p.status) atomicOr(p.status, 1);
}

}  // namespace

// Launches the TMA form when the shape suits it; returns VIG_DWCONV_NOT_TAKEN otherwise (the caller then uses the
// sliding-window kernel).  x, y: [B, h*w, C] contiguous; wt: [9, C]; bias: [C] or null.
int dwconv_tma_try(const void* x, const void* wt, const void* bias, void* y, int B, int h, int w, int C, int act, int dtype,
                   int32_t* status, cudaStream_t stream) {
    if (dtype != VIG_DTYPE_BF16 && dtype != VIG_DTYPE_F16) return VIG_DWCONV_NOT_TAKEN;
    if (C % 8 || (int64_t)B * h * w * C < (1ll << 22)) return VIG_DWCONV_NOT_TAKEN;   // small problems: launch-bound either way
    if (!tc::encode_fn()) return VIG_DWCONV_NOT_TAKEN;
    int CC = 0;
    if (C <= 256) CC = C;
    else for (int cand : {256, 192, 128, 64}) if (C % cand == 0) { CC = cand; break; }
    if (!CC || (CC % 4)) return VIG_DWCONV_NOT_TAKEN;
    DwParams p{};
    p.groups = CC / 4;
    int nseg = DW_COMPUTE / p.groups;
    const int w_runs = (w + DW_SEG - 1) / DW_SEG;
    if (nseg > w_runs) nseg = w_runs;
    if (nseg * DW_SEG > 248) nseg = 248 / DW_SEG;
    if (nseg < 1) return VIG_DWCONV_NOT_TAKEN;
    p.nseg = nseg; p.WB = nseg * DW_SEG; p.CC = CC;
    p.box_bytes = 4u * (uint32_t)(p.WB + 2) * CC * 2u;
    p.stage_bytes = (p.box_bytes + 1023u) & ~1023u;
    const int smem = (int)(DW_STAGES * p.stage_bytes) + 16 * DW_STAGES + 16;
    if (smem > 227 * 1024) return VIG_DWCONV_NOT_TAKEN;
    p.ncb = C / CC; p.nxb = (w + p.WB - 1) / p.WB; p.nyb = (h + DW_ROWS - 1) / DW_ROWS;
    const int64_t ntiles = (int64_t)B * p.nyb * p.nxb * p.ncb;
    if (ntiles >= (1ll << 31)) return VIG_DWCONV_NOT_TAKEN;
    p.ntiles = (int)ntiles;
    p.wt = wt; p.bias = bias; p.y = y; p.B = B; p.h = h; p.w = w; p.C = C; p.act = act; p.status = status;
    tc::MapKey key{};
    key.base = x; key.rank = 4; key.dtype = dtype; key.swizzle = 0;
    key.dims[0] = (uint64_t)C; key.dims[1] = (uint64_t)w; key.dims[2] = (uint64_t)h; key.dims[3] = (uint64_t)B;
    key.strides[0] = (uint64_t)C * 2; key.strides[1] = (uint64_t)w * C * 2; key.strides[2] = (uint64_t)h * w * C * 2;
    key.box[0] = (uint32_t)CC; key.box[1] = (uint32_t)(p.WB + 2); key.box[2] = 4; key.box[3] = 1;
    CUtensorMap map;
    if (!tc::encode_cached(&map, key)) return VIG_DWCONV_NOT_TAKEN;
    int dev = 0, sms = 0;
    cudaError_t e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    const int grid = p.ntiles < sms ? p.ntiles : sms;
    if (dtype == VIG_DTYPE_BF16) {
        auto kfn = dwconv3x3_tma_kernel<__nv_bfloat16>;
        if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
        kfn<<<grid, DW_THREADS, smem, stream>>>(map, p);
    } else {
        auto kfn = dwconv3x3_tma_kernel<__half>;
        if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
        kfn<<<grid, DW_THREADS, smem, stream>>>(map, p);
    }
    return (int)cudaGetLastError();
}

}  // namespace vig
