// out[M, N] = x W^T + bias: the stacked input projection of the ViG block as one tcgen05 GEMM (bf16 / fp16, K <= 192).
// One GEMM produces [q | k | v | output-gate logits | gate logits] per token (qkv_proj, g_proj and the folded gk_proj of
// GatedLinearAttention, classification/models/vig.py:283-290 and 431-439), N = 1152 at width 192.
//
// The product is write-bound (x: 100 MB in, z: 604 MB out at the headline shape).  Weight-stationary organisation: a
// persistent CTA owns ONE block of 192 output columns for the whole launch -- its [192 x K] slice of W (72 KB at K = 192)
// is loaded once and stays in shared memory -- and walks tiles of 128 rows of x, which stream through a two-stage ring
// (48 KB each) and are multiplied with one M128 N192 MMA per k step into one of two accumulators in tensor memory (tile
// t+1 is multiplied while tile t is read out).  The CTAs that hold the different column blocks of the same row tile have
// consecutive block indices and run in step, so a tile of x comes from DRAM once and from L2 for the others.  No weight
// box is ever reloaded: an earlier organisation that kept 256 rows of x resident and streamed the weights through a
// ring of one column block's boxes waited for reloads at every block and took 199 us.
// Twelve epilogue warps share a tile: a warp owns the 32 rows of its TMEM lane quarter and 64 columns, adds the bias in
// fp32, rounds, packs its [32 rows x 64 columns] into a swizzled 4 KB box of shared memory and lane 0 sends the box with ONE
// TMA store (a thread owns a row, so direct stores touch 32 lines per request: 32-byte stores straight from registers
// were tried and took 207 us).  Columns past N in the last column block are zero rows of W (TMA fill) on the way in and
// are clipped by the tensor map on the way out.
// Measured at M = 262144, K = 192, N = 1152: 171 us against 160-165 us for the vendor GEMM (a 2-CTA kernel), so the block
// keeps the vendor GEMM by default.  Switching phases off (timing only): without the stores 132, without the MMAs 150,
// without the box round 118 -- the output path is the bound (604 MB in 171 us = 3.5 TB/s of writes); boxes with 96-byte
// rows (sixteen warps of 48 columns) and with 128-byte rows take the same time, so it is not the TMA unit's row rate.
// Roles: warp 0 TMA producer, warp 1 MMA issuer (the whole warp walks the loops, only the issue is predicated on lane
// 0; barriers are asked about ahead of use with the non-blocking test), warps 2..13 epilogue.  Every wait is bounded.
#include "tc_common.cuh"

namespace vig {
namespace {

using namespace tc;

constexpr int GB_BK = 64;                          // k elements per box row (128 bytes)
constexpr int GB_A_BOX = 128 * GB_BK * 2;          // one [128 rows x 64 k] box of x
constexpr int GB_COLS = 192;                       // output columns per block (1152 = 6 x 192 at width 192)
constexpr int GB_W_BOX = GB_COLS * GB_BK * 2;      // one k box of the CTA's weight slice, 24 KB
constexpr int GB_XSTAGES = 2;                      // x tiles in flight
constexpr int GB_EPI_WARPS = 12;                   // 4 TMEM lane quarters x 3 groups of 64 columns
constexpr int GB_THREADS = 64 + 32 * GB_EPI_WARPS;
constexpr int GB_WCOLS = 64;                       // columns per epilogue warp: 128-byte rows in its output box
constexpr int GB_OUT_BOX = 32 * GB_WCOLS * 2;      // one epilogue warp's [32 rows x 64 columns] box, 128-byte swizzle

template <typename T> struct GbPk;
template <> struct GbPk<__nv_bfloat16> { static constexpr uint32_t FMT = 1;
    __device__ static uint32_t pack(float a, float b) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); } };
template <> struct GbPk<__half> { static constexpr uint32_t FMT = 0;
    __device__ static uint32_t pack(float a, float b) { __half2 t = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); } };

struct GbMaps { CUtensorMap x, w, o; };

// grid = row_groups * nblocks CTAs; CTA i holds column block i % nblocks and walks row tiles i / nblocks, + row_groups, ...
template <typename T>
__global__ void __launch_bounds__(GB_THREADS, 1) linear_bias_kernel(const __grid_constant__ GbMaps maps, const T* __restrict__ bias,
                                                                    int M, int N, int KB, int nblocks, int row_groups, int32_t* status) {
    extern __shared__ uint8_t gb_smem_raw[];
    uint8_t* smem = gb_smem_raw + ((1024u - (smem_u32(gb_smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t off_x = (uint32_t)KB * GB_W_BOX;                         // after the weight slice
    const uint32_t x_stage = (uint32_t)KB * GB_A_BOX;
    const uint32_t off_out = off_x + GB_XSTAGES * x_stage;
    const uint32_t off_bar = off_out + GB_EPI_WARPS * GB_OUT_BOX;
    // barriers: weight slice full; x stages full / empty; accumulators full / empty
    const uint32_t bar_w = sbase + off_bar;
    const uint32_t bar_x_full = bar_w + 8, bar_x_empty = bar_x_full + 8 * GB_XSTAGES;
    const uint32_t bar_acc_full = bar_x_empty + 8 * GB_XSTAGES, bar_acc_empty = bar_acc_full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + off_bar + 8 * (1 + 2 * GB_XSTAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const Waiter waiter{abort_flag, status};

    if (tid == 0) {
        mbar_init(bar_w, 1);
        for (int i = 0; i < GB_XSTAGES; ++i) { mbar_init(bar_x_full + 8 * i, 1); mbar_init(bar_x_empty + 8 * i, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, GB_EPI_WARPS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int ntiles = (M + 127) / 128;
    const int nb = (int)blockIdx.x % nblocks, rg = (int)blockIdx.x / nblocks;
    constexpr uint32_t IDESC = make_idesc(GbPk<T>::FMT, 0, 0, 128, GB_COLS);

    if (warp == 0) {
        if (lane == 0) {                          // ---- TMA producer -------------------------------------------
            mbar_expect_tx(bar_w, (uint32_t)KB * GB_W_BOX);
            for (int kb = 0; kb < KB; ++kb)
                tma_load_2d(sbase + kb * GB_W_BOX, &maps.w, kb * GB_BK, nb * GB_COLS, bar_w);      // rows past N arrive as zeros
            uint32_t st = 0, phase = 0;
            for (int tile = rg; tile < ntiles; tile += row_groups) {
                waiter.wait(bar_x_empty + 8 * st, phase ^ 1u);            // the MMAs of the tile two back have read this stage
                if (*abort_flag) break;
                mbar_expect_tx(bar_x_full + 8 * st, x_stage);
                for (int kb = 0; kb < KB; ++kb)
                    tma_load_2d(sbase + off_x + st * x_stage + kb * GB_A_BOX, &maps.x, kb * GB_BK, tile * 128, bar_x_full + 8 * st);
                if (++st == GB_XSTAGES) { st = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {                       // ---- MMA issuer ---------------------------------------------
        const bool issuer = lane == 0;
        const uint32_t w_lo0 = make_desc(sbase), x_lo0 = make_desc(sbase + off_x);
        waiter.wait_lite(bar_w, 0);
        uint32_t st = 0, phase = 0, it = 0;
        uint32_t pre_x = 0, pre_acc = 0;
        for (int tile = rg; tile < ntiles; tile += row_groups, ++it) {
            const uint32_t buf = it & 1u;
            if (!pre_acc) waiter.wait_lite(bar_acc_empty + 8 * buf, ((it >> 1) & 1u) ^ 1u);   // the epilogue has read this accumulator out
            if (!pre_x) waiter.wait_lite(bar_x_full + 8 * st, phase);
            if (*abort_flag) break;
            tc_fence_after();
            // asked before this tile's MMAs, answered while they are issued: the next tile's stage and accumulator
            const uint32_t st_next = st + 1 == GB_XSTAGES ? 0u : st + 1, ph_next = st + 1 == GB_XSTAGES ? phase ^ 1u : phase;
            pre_x = mbar_test_wait(bar_x_full + 8 * st_next, ph_next);
            pre_acc = mbar_test_wait(bar_acc_empty + 8 * (buf ^ 1u), (((it + 1) >> 1) & 1u) ^ 1u);
            const uint32_t d = tmem + buf * 256u;
            for (int kb = 0; kb < KB; ++kb) {
                const uint32_t a_lo = x_lo0 + (st * x_stage >> 4) + (uint32_t)kb * (GB_A_BOX >> 4);
                const uint32_t b_lo = w_lo0 + (uint32_t)kb * (GB_W_BOX >> 4);
#pragma unroll
                for (uint32_t k4 = 0; k4 < 4; ++k4) { if (issuer) tc_mma(d, a_lo + 2 * k4, b_lo + 2 * k4, IDESC, (kb | k4) > 0 ? 1u : 0u); }
            }
            if (issuer) { tc_commit(bar_x_empty + 8 * st); tc_commit(bar_acc_full + 8 * buf); }
            st = st_next; phase = ph_next;
        }
    } else {                                      // ---- epilogue: + bias -> out ----------------------------------
        const int ew = warp - 2;                  // 0..11
        const int cq = ew >> 2;                   // which 64 of the block's 192 columns
        const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;   // a warp reads the TMEM lanes of its quarter
        uint8_t* my_row = smem + off_out + ew * GB_OUT_BOX + lane * 128;
        const uint32_t sw = (uint32_t)(lane & 7);
        const uint32_t box_u32 = sbase + off_out + ew * GB_OUT_BOX;
        const int col0 = nb * GB_COLS + GB_WCOLS * cq;
        uint32_t it = 0;
        for (int tile = rg; tile < ntiles; tile += row_groups, ++it) {
            const uint32_t buf = it & 1u;
            waiter.wait_lite(bar_acc_full + 8 * buf, (it >> 1) & 1u);   // by the whole warp
            if (*abort_flag) break;
            tc_fence_after();
            const uint32_t acc = tmem + lane_base + buf * 256u + (uint32_t)(GB_WCOLS * cq);
            const int row0 = tile * 128 + 32 * (warp & 3);
            float v[GB_WCOLS];
            tc_ld32(acc, v);
            tc_ld32(acc + 32, v + 32);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(bar_acc_empty + 8 * buf);   // the accumulator is in registers: the MMA warp may refill it
            uint32_t pk[GB_WCOLS / 2];
#pragma unroll
            for (int j = 0; j < GB_WCOLS / 8; ++j) {                  // 8 columns at a time; N is a multiple of 8
                uint4 t = make_uint4(0u, 0u, 0u, 0u);
                // bias values: the same addresses for all lanes (one broadcast transaction per load, L1-resident)
                if (bias && col0 + 8 * j < N) t = __ldg(reinterpret_cast<const uint4*>(bias + col0 + 8 * j));
                const uint32_t w4[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 bb = Pack2<T>::unpack(w4[i]);
                    pk[4 * j + i] = GbPk<T>::pack(v[8 * j + 2 * i] + bb.x, v[8 * j + 2 * i + 1] + bb.y);
                }
            }
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous store has read the box
            __syncwarp();
#pragma unroll
            for (int j = 0; j < GB_WCOLS / 8; ++j)
                *reinterpret_cast<uint4*>(my_row + (((uint32_t)j ^ sw) << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && row0 < M && col0 < N) {
                tma_store_2d(&maps.o, col0, row0, box_u32);      // rows past M / columns past N are clipped by the tensor map
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every store has landed before the CTA exits
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag && status) atomicOr(status, 1);
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

// [rows, cols] with leading dimension ld: boxes of `box_rows` x `box_cols`, 128-byte swizzle when the box row is 128 bytes
bool gb_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows, int box_cols, int dtype) {
    tc::MapKey key{};
    key.base = base; key.rank = 2; key.dtype = dtype; key.swizzle = box_cols == 64 ? 1 : 0;
    key.dims[0] = (uint64_t)cols; key.dims[1] = (uint64_t)rows;
    key.strides[0] = (uint64_t)ld * 2;
    key.box[0] = (uint32_t)box_cols; key.box[1] = (uint32_t)box_rows;
    return tc::encode_cached(m, key);
}

}  // namespace
}  // namespace vig

using namespace vig;

// Shapes the kernel takes: 16-bit types, K a multiple of 64 up to 192, N a multiple of 8, and enough rows to
// give every SM a 256-row tile (smaller problems are left to the library GEMM).
extern "C" int vig_linear_bias_supported(int64_t M, int K, int N, int dtype) {
    if (dtype != VIG_DTYPE_BF16 && dtype != VIG_DTYPE_F16) return 0;
    if (M <= 0 || K <= 0 || N <= 0 || K % GB_BK || K > 3 * GB_BK || N % 8 || M >= (1ll << 31)) return 0;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (M < 256 * (int64_t)sms) return 0;
    return tc::encode_fn() != nullptr;
}

extern "C" int vig_linear_bias_fwd(const void* x, int64_t ldx, const void* w, const void* bias, void* out, int64_t ldo,
                                   int64_t M, int K, int N, int dtype, int32_t* status_dev, void* stream) {
    if (!x || !w || !out) return VIG_ERR_NULL;
    if (M == 0) return VIG_OK;
    if (!vig_linear_bias_supported(M, K, N, dtype)) return VIG_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias)) & 15) return VIG_ERR_ALIGN;
    if (ldx < K || ldo < N || (ldx * 2) % 16 || (ldo * 2) % 16) return VIG_ERR_ARG;
    GbMaps maps;
    if (!gb_map(&maps.x, x, M, K, ldx, 128, 64, dtype) || !gb_map(&maps.w, w, N, K, K, GB_COLS, 64, dtype) ||
        !gb_map(&maps.o, out, M, N, ldo, 32, GB_WCOLS, dtype)) return VIG_ERR_DEVICE;
    const int KB = K / GB_BK;
    int dev = 0, sms = 0;
    cudaError_t e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    const int smem = KB * GB_W_BOX + GB_XSTAGES * KB * GB_A_BOX + GB_EPI_WARPS * GB_OUT_BOX + 8 * (1 + 2 * GB_XSTAGES + 4) + 16 + 1024;
    const int nblocks = (N + GB_COLS - 1) / GB_COLS;
    if (nblocks > sms) return VIG_ERR_SHAPE;
    const int ntiles = (int)((M + 127) / 128);
    int row_groups = sms / nblocks;                            // CTAs per column block
    if (row_groups > ntiles) row_groups = ntiles;
    const int grid = row_groups * nblocks;
    if (dtype == VIG_DTYPE_BF16) {
        auto kfn = linear_bias_kernel<__nv_bfloat16>;
        if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
        kfn<<<grid, GB_THREADS, smem, (cudaStream_t)stream>>>(maps, (const __nv_bfloat16*)bias, (int)M, N, KB, nblocks, row_groups, status_dev);
    } else {
        auto kfn = linear_bias_kernel<__half>;
        if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
        kfn<<<grid, GB_THREADS, smem, (cudaStream_t)stream>>>(maps, (const __half*)bias, (int)M, N, KB, nblocks, row_groups, status_dev);
    }
    return (int)cudaGetLastError();
}
