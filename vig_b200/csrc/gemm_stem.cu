// First convolution of the patch-embedding stem with its bias, the LayerNorm2d that follows and the swish after it, as
// one tcgen05 GEMM kernel (bf16 / fp16): classification/models/vig.py:650-656 (`V2PatchEmbed.proj[0..2]`, kernel s+1,
// stride s, padding 1 with s = 8 and 3 input channels).
//
// The image has been folded into cells of 8 x 8 pixels on 8-pixel boundaries (`vig_stem_fold_fwd`, below: cells[b, cy, cx,
// (dy*3 + ic)*8 + dx] = x[b, ic, 8cy + dy, 8cx + dx]; every run of 8 pixels is one aligned 16-byte vector, so the fold is a
// permutation of vectors).  The 9 x 9 window of output pixel (oy, ox) starts one pixel up and left of cell (oy, ox): it is that
// cell, the last pixel column of cell (oy, ox-1), the last pixel row of cell (oy-1, ox) and the last pixel of cell (oy-1, ox-1).
// As a GEMM: row = output pixel, K = 512 = cells (oy, ox) and (oy, ox-1) in full (2 x 192) + the last 64 values of the two cells
// above (the taps the kernel has there are among their last 24 values; the weight matrix is zero elsewhere), N = 96.  Cells
// outside the image are read as zeros by the TMA unit, which is the convolution's padding.
//
// One persistent CTA per SM.  Its [96 x 512] weight matrix stays in shared memory for the whole launch (8 swizzled
// boxes, 96 KB); tiles of 128 output pixels (Wt columns x Rt rows of the output, Wt * Rt = 128) stream through a ring of
// [128 x 64] boxes that the TMA unit cuts straight out of the cell tensor (box rows = consecutive cells, so no gather and
// no im2col copy); 32 M128.N96.K16 MMAs per tile into one of two accumulators in tensor memory.  Epilogue: a thread owns
// an output pixel (its TMEM lane) with all 96 channels in registers -- the convolution's rounding to the tensor type, the
// bias add (rounded like a separate add), mean, centred variance, affine, swish, all without leaving the thread, on fp32
// pairs -- and the tile leaves through shared memory as one TMA store, which also clips the pixels past the image's edge.
// Two sets of four epilogue warps take alternate tiles (one accumulator and one staging tile each): a single set, one warp
// per scheduler, took longer over a tile than its MMAs.
// Roles: warp 0 TMA producer, warp 1 MMA issue, warps 2..5 and 6..9 epilogue.  Every wait is bounded.
#include "tc_common.cuh"

namespace vig {
namespace {

using namespace tc;

constexpr int SC_CELL = 192, SC_N = 96;
constexpr int SC_KB = 8;                              // k boxes of 64 values: 3 + 3 from the pixel's cell row, 1 + 1 from the row above
constexpr int SC_THREADS = 64 + 256;
constexpr int SC_W_BOX = SC_N * 128;                  // [96 rows x 64 k] = 12 KB
constexpr int SC_A_BOX = 128 * 128;                   // [128 pixels x 64 k] = 16 KB
constexpr int SC_STAGES = 5;
constexpr int SC_ACC_STRIDE = 128;                    // TMEM columns between the two accumulators
constexpr int SO_W = 0;
constexpr int SO_A = SO_W + SC_KB * SC_W_BOX;         // 98304: a multiple of 1024, like every box start
constexpr int SC_OUT_TILE = 128 * SC_N * 2;           // [128 pixels x 96 channels], dense rows of 192 bytes
constexpr int SO_OUT = SO_A + SC_STAGES * SC_A_BOX;   // one staging tile per epilogue set
constexpr int SO_PAR = SO_OUT + 2 * SC_OUT_TILE;      // fp32 [3][96]: conv bias, norm weight, norm bias
constexpr int SO_BAR = SO_PAR + 3 * SC_N * 4;
constexpr int SO_MISC = SO_BAR + 8 * (2 * SC_STAGES + 5);
constexpr int SC_SMEM_BYTES = SO_MISC + 16 + 1024;    // + slack to start on a 1024-byte boundary
static_assert(SO_A % 1024 == 0 && SC_W_BOX % 1024 == 0 && SO_BAR % 8 == 0, "box alignment");
static_assert(SC_SMEM_BYTES <= 227 * 1024, "shared memory budget");

struct ScMaps { CUtensorMap a, w, y; };

__device__ __forceinline__ void sc_epi_sync(int set) { asm volatile("bar.sync %0, 128;" ::"r"(1 + set) : "memory"); }
__device__ __forceinline__ float sc_tanh(float x) { float t; asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(x)); return t; }

template <typename T>
__global__ void __launch_bounds__(SC_THREADS, 1) stem_conv_ln_kernel(const __grid_constant__ ScMaps maps, const T* __restrict__ conv_bias,
                                                                     const T* __restrict__ ln_w, const T* __restrict__ ln_b,
                                                                     int ntiles, int tiles_x, int tiles_y, int Wt, int Rt,
                                                                     float eps, int act, int32_t* status) {
    extern __shared__ uint8_t sc_smem_raw[];
    uint8_t* smem = sc_smem_raw + ((1024u - (smem_u32(sc_smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bar_full = sbase + SO_BAR, bar_empty = bar_full + 8 * SC_STAGES;
    const uint32_t bar_w = bar_empty + 8 * SC_STAGES, bar_acc_full = bar_w + 8, bar_acc_empty = bar_acc_full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + SO_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* par = reinterpret_cast<float*>(smem + SO_PAR);
    const Waiter waiter{abort_flag, status};

    for (int i = tid; i < SC_N; i += SC_THREADS) {
        par[i] = conv_bias ? DType<T>::to_f(conv_bias[i]) : 0.f;
        par[SC_N + i] = DType<T>::to_f(ln_w[i]);
        par[2 * SC_N + i] = DType<T>::to_f(ln_b[i]);
    }
    if (tid == 0) {
        for (int s = 0; s < SC_STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        mbar_init(bar_w, 1);
        for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // tile -> image, first output row, first output column
    auto coords = [&](int tile, int& b, int& oy0, int& ox0) {
        const int tx = tile % tiles_x, r = tile / tiles_x;
        ox0 = tx * Wt; oy0 = (r % tiles_y) * Rt; b = r / tiles_y;
    };

    if (warp == 0) {
        if (lane == 0) {                          // ---- TMA producer -------------------------------------------
            mbar_expect_tx(bar_w, SC_KB * SC_W_BOX);
            for (int kb = 0; kb < SC_KB; ++kb) tma_load_2d(sbase + SO_W + kb * SC_W_BOX, &maps.w, kb * 64, 0, bar_w);
            uint32_t st = 0, phase = 0;
            bool live = true;
            for (int tile = blockIdx.x; tile < ntiles && live; tile += gridDim.x) {
                int b, oy0, ox0;
                coords(tile, b, oy0, ox0);
                for (int kb = 0; kb < SC_KB; ++kb) {
                    // k box -> (cell row offset, cell column offset, first value inside the cell)
                    const int cyo = kb >= 6 ? -1 : 0, cxo = kb < 6 ? (kb >= 3 ? -1 : 0) : 6 - kb, e0 = kb < 6 ? 64 * (kb % 3) : 128;
                    waiter.wait(bar_empty + 8 * st, phase ^ 1u);
                    if (*abort_flag) { live = false; break; }
                    mbar_expect_tx(bar_full + 8 * st, SC_A_BOX);
                    tma_load_4d(sbase + SO_A + st * SC_A_BOX, &maps.a, e0, ox0 + cxo, oy0 + cyo, b, bar_full + 8 * st);
                    if (++st == (uint32_t)SC_STAGES) { st = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {                       // ---- MMA issue: the whole warp walks the loops, lane 0 issues ----
        constexpr uint32_t IDESC = make_idesc(Pack2<T>::FMT, 0, 0, 128, SC_N);
        const bool issuer = lane == 0;
        waiter.wait(bar_w, 0u);
        tc_fence_after();
        uint32_t st = 0, phase = 0, acc_it = 0;
        bool live = !*abort_flag;
        // Even a test of a long-completed mbarrier takes a few hundred cycles here, and a k box is only four MMAs: the next
        // barrier this warp will need is asked about (without blocking) before the current MMAs are issued, and a wait loop is
        // entered only on "not yet".
        uint32_t pre_full = 0, pre_acc = 0;
        for (int tile = blockIdx.x; tile < ntiles && live; tile += gridDim.x, ++acc_it) {
            const uint32_t buf = acc_it & 1u, use = acc_it >> 1;
            if (!pre_acc) waiter.wait(bar_acc_empty + 8 * buf, (use & 1u) ^ 1u);      // the epilogue has read this accumulator
            if (*abort_flag) break;
            tc_fence_after();
            const uint32_t d = tmem + buf * SC_ACC_STRIDE;
            for (int kb = 0; kb < SC_KB; ++kb) {
                if (!pre_full) waiter.wait(bar_full + 8 * st, phase);
                if (*abort_flag) { live = false; break; }
                tc_fence_after();
                const uint32_t nst = st + 1 == (uint32_t)SC_STAGES ? 0u : st + 1, nphase = nst ? phase : phase ^ 1u;
                pre_full = mbar_test_wait(bar_full + 8 * nst, nphase);
                if (kb == SC_KB - 1) pre_acc = mbar_test_wait(bar_acc_empty + 8 * (buf ^ 1u), ((((acc_it + 1) >> 1) & 1u) ^ 1u));
                const uint32_t a_lo = make_desc(sbase + SO_A + st * SC_A_BOX), b_lo = make_desc(sbase + SO_W + kb * SC_W_BOX);
#pragma unroll
                for (uint32_t k4 = 0; k4 < 4; ++k4) { if (issuer) tc_mma(d, a_lo + 2 * k4, b_lo + 2 * k4, IDESC, (kb | k4) ? 1u : 0u); }
                if (issuer) tc_commit(bar_empty + 8 * st);              // the stage is free when these MMAs are done
                __syncwarp();
                st = nst; phase = nphase;
            }
            if (live && issuer) tc_commit(bar_acc_full + 8 * buf);
            __syncwarp();
        }
    } else {                                      // ---- epilogue: one thread per output pixel, two sets on alternate tiles ----
        // (no early exit on an abort: the four warps of a set meet at named barriers, and after an abort every wait returns at once)
        const int set = (warp - 2) >> 2;
        const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;
        const int row = 32 * (warp & 3) + lane;   // my pixel of the tile = my TMEM lane
        const bool leader = (warp & 3) == 2 && lane == 0;
        const bool has_bias = conv_bias != nullptr;
        const uint32_t buf = (uint32_t)set;       // my set's accumulator
        uint8_t* otile = smem + SO_OUT + set * SC_OUT_TILE;
        const F2* par2 = reinterpret_cast<const F2*>(par);
        for (uint32_t acc_it = (uint32_t)set;; acc_it += 2) {
            const int64_t tile64 = (int64_t)blockIdx.x + (int64_t)acc_it * gridDim.x;
            if (tile64 >= ntiles) break;
            const int tile = (int)tile64;
            const uint32_t use = acc_it >> 1;
            int b, oy0, ox0;
            coords(tile, b, oy0, ox0);
            waiter.wait(bar_acc_full + 8 * buf, use & 1u);
            __syncwarp();
            tc_fence_after();
            float v[SC_N];
            const uint32_t acc = tmem + lane_base + buf * SC_ACC_STRIDE;
            tc_ld32(acc, v); tc_ld32(acc + 32, v + 32); tc_ld32(acc + 64, v + 64);
            tc_wait_ld();
            tc_fence_before();
            mbar_arrive_plain(bar_acc_empty + 8 * buf);               // the accumulator is read
            // the unfused path rounds the convolution to T, then the sum with the bias to T; arithmetic on fp32 pairs, sums
            // in four chains
            F2 vv[SC_N / 2];
            F2 s0 = f2_make(0.f, 0.f), s1 = s0;
#pragma unroll
            for (int i = 0; i < SC_N / 2; ++i) {
                float2 y = Pack2<T>::unpack(Pack2<T>::pack(v[2 * i], v[2 * i + 1]));
                F2 yy = f2_make(y.x, y.y);
                if (has_bias) {
                    const F2 z = f2_add(yy, par2[i]);
                    y = Pack2<T>::unpack(Pack2<T>::pack(f2_lo(z), f2_hi(z)));
                    yy = f2_make(y.x, y.y);
                }
                vv[i] = yy;
                if (i & 1) s1 = f2_add(s1, yy); else s0 = f2_add(s0, yy);
            }
            s0 = f2_add(s0, s1);
            const float mean = (f2_lo(s0) + f2_hi(s0)) * (1.f / SC_N);
            const F2 nmean = f2_make(-mean, -mean);
            F2 q0 = f2_make(0.f, 0.f), q1 = q0;
#pragma unroll
            for (int i = 0; i < SC_N / 2; ++i) {
                vv[i] = f2_add(vv[i], nmean);
                if (i & 1) q1 = f2_fma(vv[i], vv[i], q1); else q0 = f2_fma(vv[i], vv[i], q0);
            }
            q0 = f2_add(q0, q1);
            const float rstd = rsqrtf((f2_lo(q0) + f2_hi(q0)) * (1.f / SC_N) + eps);
            const F2 rstd2 = f2_make(rstd, rstd), half2 = f2_make(0.5f, 0.5f);
            // the previous store of my set has read the staging tile
            if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            sc_epi_sync(set);
            uint8_t* orow = otile + row * (SC_N * 2);
#pragma unroll
            for (int j = 0; j < SC_N / 8; ++j) {
                uint32_t o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = 4 * j + e;      // pair index
                    F2 t = f2_fma(f2_mul(vv[i], rstd2), par2[SC_N / 2 + i], par2[SC_N + i]);
                    if (act) {                    // t * sigmoid(t), sigmoid through the one-instruction tanh
                        const F2 h = f2_mul(t, half2);
                        const F2 sg = f2_fma(f2_make(sc_tanh(f2_lo(h)), sc_tanh(f2_hi(h))), half2, half2);
                        t = f2_mul(t, sg);
                    }
                    o[e] = Pack2<T>::pack(f2_lo(t), f2_hi(t));
                }
                *reinterpret_cast<uint4*>(orow + 16 * j) = make_uint4(o[0], o[1], o[2], o[3]);
            }
            fence_proxy_async();
            sc_epi_sync(set);
            if (leader) {
                tma_store_4d(&maps.y, 0, ox0, oy0, b, smem_u32(otile));   // pixels past the image's edge are clipped by the map
                bulk_commit();
            }
        }
        if (leader) bulk_store_wait_all();        // all stores have landed before the CTA exits
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}

// image -> cells (16-bit types): cells[b, cy, cx, (dy*3 + ic)*8 + dx] = x[b, ic, 8cy + dy, 8cx + dx], as 16-byte vectors.
// A block owns up to SF_CELLS consecutive cells of one cell row: 24 coalesced runs of the image (8 rows x 3 planes) go
// into shared memory (rows padded by one vector: the transposed read below is then free of bank conflicts) and leave as
// one contiguous run of cells.
constexpr int SF_CELLS = 64, SF_THREADS = 256;

__global__ void __launch_bounds__(SF_THREADS) stem_fold_kernel(const uint4* __restrict__ x, uint4* __restrict__ cells, int H, int W, int nseg) {
    __shared__ uint4 tile[24][SF_CELLS + 1];
    const int ch = H / 8, cw = W / 8;
    int blk = blockIdx.x;
    const int seg = blk % nseg; blk /= nseg;
    const int cy = blk % ch, b = blk / ch;
    const int cx0 = seg * SF_CELLS, ncell = min(SF_CELLS, cw - cx0);
    for (int i = threadIdx.x; i < 24 * SF_CELLS; i += SF_THREADS) {
        const int c = i % SF_CELLS, j = i / SF_CELLS, dy = j / 3, ic = j % 3;
        if (c < ncell) tile[j][c] = __ldg(x + (((size_t)b * 3 + ic) * H + 8 * cy + dy) * cw + cx0 + c);
    }
    __syncthreads();
    uint4* dst = cells + (((size_t)b * ch + cy) * cw + cx0) * 24;
    for (int v = threadIdx.x; v < ncell * 24; v += SF_THREADS) dst[v] = tile[v % 24][v / 24];
}

// Output tile of 128 pixels as Wt columns x Rt rows: the split that covers the output with the fewest tiles (the widest on a tie).
void sc_tile_shape(int OW, int OH, int& Wt, int& Rt) {
    int64_t best = -1;
    for (int rt = 1; rt <= 8; rt *= 2) {
        const int wt = 128 / rt;
        const int64_t cost = (int64_t)((OW + wt - 1) / wt) * ((OH + rt - 1) / rt);
        if (best < 0 || cost < best) { best = cost; Wt = wt; Rt = rt; }
    }
}

}  // namespace
}  // namespace vig

using namespace vig;

extern "C" int vig_stem_conv_ln_supported(int B, int CH, int CW, int cell, int N, int dtype) {
    if (dtype != VIG_DTYPE_BF16 && dtype != VIG_DTYPE_F16) return 0;
    if (B <= 0 || CH < 1 || CW < 1 || cell != SC_CELL || N != SC_N) return 0;
    return tc::encode_fn() != nullptr;
}

extern "C" int vig_stem_conv_ln_fwd(const void* cells, const void* w2, const void* conv_bias, const void* ln_w, const void* ln_b, void* y,
                                    int B, int CH, int CW, int cell, int N, float eps, int act_swish, int dtype,
                                    int32_t* status_dev, void* stream) {
    if (!cells || !w2 || !ln_w || !ln_b || !y) return VIG_ERR_NULL;
    if (!vig_stem_conv_ln_supported(B, CH, CW, cell, N, dtype)) return VIG_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(cells) | reinterpret_cast<uintptr_t>(w2) | reinterpret_cast<uintptr_t>(y)) & 15) return VIG_ERR_ALIGN;
    const int OH = CH, OW = CW;
    int Wt = 128, Rt = 1;
    sc_tile_shape(OW, OH, Wt, Rt);
    const int tiles_x = (OW + Wt - 1) / Wt, tiles_y = (OH + Rt - 1) / Rt;
    const int64_t ntiles = (int64_t)B * tiles_x * tiles_y;
    if (ntiles >= (1ll << 31)) return VIG_ERR_SHAPE;
    ScMaps maps;
    {
        tc::MapKey key{};                         // cells [B, CH, CW, 192]: boxes of 64 values x Wt cells x Rt cell rows
        key.base = cells; key.rank = 4; key.dtype = dtype; key.swizzle = 1;
        key.dims[0] = SC_CELL; key.dims[1] = (uint64_t)CW; key.dims[2] = (uint64_t)CH; key.dims[3] = (uint64_t)B;
        key.strides[0] = (uint64_t)SC_CELL * 2; key.strides[1] = (uint64_t)CW * SC_CELL * 2; key.strides[2] = (uint64_t)CH * CW * SC_CELL * 2;
        key.box[0] = 64; key.box[1] = (uint32_t)Wt; key.box[2] = (uint32_t)Rt; key.box[3] = 1;
        if (!tc::encode_cached(&maps.a, key)) return VIG_ERR_DEVICE;
    }
    if (!tc::make_map_2d(&maps.w, w2, SC_N, SC_KB * 64, SC_KB * 64, SC_N, dtype)) return VIG_ERR_DEVICE;
    {
        tc::MapKey key{};                         // y [B, OH, OW, 96]: one dense box per tile
        key.base = y; key.rank = 4; key.dtype = dtype; key.swizzle = 0;
        key.dims[0] = SC_N; key.dims[1] = (uint64_t)OW; key.dims[2] = (uint64_t)OH; key.dims[3] = (uint64_t)B;
        key.strides[0] = (uint64_t)SC_N * 2; key.strides[1] = (uint64_t)OW * SC_N * 2; key.strides[2] = (uint64_t)OH * OW * SC_N * 2;
        key.box[0] = SC_N; key.box[1] = (uint32_t)Wt; key.box[2] = (uint32_t)Rt; key.box[3] = 1;
        if (!tc::encode_cached(&maps.y, key)) return VIG_ERR_DEVICE;
    }
    static int sm_count[64] = {};
    int dev = 0;
    cudaError_t e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return VIG_ERR_DEVICE;
    if (!sm_count[dev]) {
        int sms = 0;
        if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        sm_count[dev] = sms;
    }
    const int grid = (int)(ntiles < sm_count[dev] ? ntiles : sm_count[dev]);
#define VIG_SC_LAUNCH(TT)                                                                                                       \
    {                                                                                                                           \
        auto kfn = stem_conv_ln_kernel<TT>;                                                                                     \
        if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), SC_SMEM_BYTES)) != cudaSuccess) return (int)e;       \
        kfn<<<grid, SC_THREADS, SC_SMEM_BYTES, (cudaStream_t)stream>>>(maps, (const TT*)conv_bias, (const TT*)ln_w, (const TT*)ln_b, \
                                                                       (int)ntiles, tiles_x, tiles_y, Wt, Rt, eps, act_swish, status_dev); \
    }
    if (dtype == VIG_DTYPE_BF16) VIG_SC_LAUNCH(__nv_bfloat16) else VIG_SC_LAUNCH(__half)
#undef VIG_SC_LAUNCH
    return (int)cudaGetLastError();
}

extern "C" int vig_stem_fold_fwd(const void* x, void* cells, int B, int Cin, int H, int W, int dtype, void* stream) {
    if (!x || !cells) return VIG_ERR_NULL;
    if (dtype != VIG_DTYPE_BF16 && dtype != VIG_DTYPE_F16) return VIG_ERR_DTYPE;
    if (B < 0 || Cin != 3 || H <= 0 || W <= 0 || H % 8 || W % 8) return VIG_ERR_SHAPE;
    if (B == 0) return VIG_OK;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(cells)) & 15) return VIG_ERR_ALIGN;
    const int nseg = (W / 8 + SF_CELLS - 1) / SF_CELLS;
    const int64_t blocks = (int64_t)B * (H / 8) * nseg;
    if (blocks >= (1ll << 31)) return VIG_ERR_SHAPE;
    stem_fold_kernel<<<(int)blocks, SF_THREADS, 0, (cudaStream_t)stream>>>((const uint4*)x, (uint4*)cells, H, W, nseg);
    return (int)cudaGetLastError();
}
