// out[M, I] = swiglu(x Wg^T, x Wy^T) = silu(x Wg^T) * (x Wy^T), with W = [Wg ; Wy] of shape [2I, K]:
// the gate projection of the SwiGLU MLP and its activation in one kernel, so the [M, 2I] intermediate
// (classification/models/vig.py:494-497: gate_proj -> chunk -> swiglu) never goes to HBM.
//
// tcgen05 GEMM.  A persistent CTA owns tiles of BM = 128*S rows of x; the tile's whole K extent stays resident
// in shared memory (TMA, 128-byte swizzle), the weights stream through a ring of 16 KB stages holding 64 gate
// rows and the 64 matching y rows, so one M128 N128 MMA per subtile fills an accumulator [128 x (64 gate | 64 y)]
// in tensor memory.  Accumulators are double buffered: while the MMA warp works on feature block n+1, the
// epilogue warps read block n with tcgen05.ld and apply silu(g)*y.  Each warp packs its [32 rows x 64 features] piece
// into a swizzled 4 KB box of shared memory and lane 0 sends it out with one TMA store: a thread owns a row, so direct
// 16-byte stores would touch 32 lines per request and fill only half of each 32-byte sector.
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2.. epilogue.  Every wait is bounded.
#include "tc_common.cuh"

namespace vig {
namespace {

using namespace tc;

constexpr int BK = 64;                         // k elements per stage row (128 bytes)
constexpr int BNF = 64;                        // features per block: 64 gate rows + 64 y rows -> MMA N = 128
constexpr int NSTAGE = 6;                      // weight stages in flight (16 KB each)
constexpr int MAX_KB = 6;                      // k boxes of an x tile (K <= 384)
constexpr int A_BOX_BYTES = 128 * BK * 2;      // one [128 rows x 64 k] box
constexpr int B_STAGE_BYTES = 2 * BNF * BK * 2;
constexpr int MAX_A_BYTES = 96 * 1024;
constexpr int GS_THREADS = 64 + 256;
constexpr int OUT_BOX_BYTES = 32 * BNF * 2;    // one epilogue warp's [32 rows x 64 features] box
constexpr int OUT_STAGE_BYTES = 8 * OUT_BOX_BYTES;

// sigmoid(x) = 0.5 tanh(x / 2) + 0.5 with the single-instruction tanh: one MUFU per element instead of two
// (exp + reciprocal), which is what bounds the epilogue; its error (~2^-11) is below the bf16 / fp16 output step.
__device__ __forceinline__ float sigmoid_tanh(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(t, 0.5f, 0.5f);
}

struct GsWaiter {
    volatile int* abort_flag;
    int32_t* status;
    __device__ __forceinline__ void wait(uint32_t bar, uint32_t parity) const {
        for (uint32_t i = 0; i < (1u << 22); ++i) {
            if (mbar_try_wait(bar, parity)) return;
            if (i > 64) { if (*abort_flag) return; __nanosleep(32); }
        }
        *abort_flag = 1;
        if (status) atomicOr(status, 1);
    }
};

template <typename T> struct Pk;
template <> struct Pk<__nv_bfloat16> { static constexpr uint32_t FMT = 1;
    __device__ static uint32_t pack(float a, float b) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); } };
template <> struct Pk<__half> { static constexpr uint32_t FMT = 0;
    __device__ static uint32_t pack(float a, float b) { __half2 t = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); } };

struct GsMaps { CUtensorMap x, w, o; };

// S = subtiles of 128 rows per CTA tile (1 or 2); KB = K / 64.
template <typename T>
__global__ void __launch_bounds__(GS_THREADS, 1) linear_swiglu_kernel(const __grid_constant__ GsMaps maps, int M, int I, int KB, int S, int nsplit, int32_t* status) {
    extern __shared__ uint8_t gs_smem_raw[];
    uint8_t* smem = gs_smem_raw + ((1024u - (smem_u32(gs_smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t a_bytes = (uint32_t)S * KB * A_BOX_BYTES;
    const uint32_t off_b = a_bytes;
    const uint32_t off_out = off_b + NSTAGE * B_STAGE_BYTES;
    const uint32_t off_bar = off_out + OUT_STAGE_BYTES;
    const uint32_t bar_a_full = sbase + off_bar, bar_a_empty = bar_a_full + 8 * MAX_KB;   // one pair per k box of the x tile
    const uint32_t bar_b_full = bar_a_empty + 8 * MAX_KB, bar_b_empty = bar_b_full + 8 * NSTAGE;
    const uint32_t bar_acc_full = bar_b_empty + 8 * NSTAGE, bar_acc_empty = bar_acc_full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + off_bar + 8 * (2 * MAX_KB + 2 * NSTAGE + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const GsWaiter waiter{abort_flag, status};

    if (tid == 0) {
        for (int kb = 0; kb < MAX_KB; ++kb) { mbar_init(bar_a_full + 8 * kb, 1); mbar_init(bar_a_empty + 8 * kb, 1); }
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_b_full + 8 * s, 1); mbar_init(bar_b_empty + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, 128 * S); }
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

    const int BM = 128 * S;
    const int ntiles = ((M + BM - 1) / BM) * nsplit;   // work items: (row tile, group of feature blocks)
    const int nblocks_all = I / BNF;
    auto nb_begin = [&](int item) { return (int)((int64_t)(item % nsplit) * nblocks_all / nsplit); };
    auto nb_end = [&](int item) { return (int)((int64_t)(item % nsplit + 1) * nblocks_all / nsplit); };
    constexpr uint32_t IDESC = (1u << 4) | (Pk<T>::FMT << 7) | (Pk<T>::FMT << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

    if (warp == 0) {
        if (lane == 0) {                          // ---- TMA producer -------------------------------------------
            // The x tile is handed over per k box: box kb of the next tile is requested as soon as the last feature
            // block of this tile has used box kb, just ahead of the weight stage that needs it.
            uint32_t a_phase = 0, st = 0, b_phase = 0;
            for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
                const int nb0 = nb_begin(tile), nb1 = nb_end(tile);
                for (int nb = nb0; nb < nb1; ++nb)
                    for (int kb = 0; kb < KB; ++kb) {
                        if (nb == nb0) {
                            waiter.wait(bar_a_empty + 8 * kb, a_phase ^ 1u);    // the previous tile's MMAs have read this box
                            mbar_expect_tx(bar_a_full + 8 * kb, (uint32_t)S * A_BOX_BYTES);
                            for (int s = 0; s < S; ++s)
                                tma_load_2d(sbase + (s * KB + kb) * A_BOX_BYTES, &maps.x, kb * BK, (tile / nsplit) * BM + s * 128, bar_a_full + 8 * kb);
                        }
                        waiter.wait(bar_b_empty + 8 * st, b_phase ^ 1u);
                        mbar_expect_tx(bar_b_full + 8 * st, B_STAGE_BYTES);
                        const uint32_t dst = sbase + off_b + st * B_STAGE_BYTES;
                        tma_load_2d(dst, &maps.w, kb * BK, nb * BNF, bar_b_full + 8 * st);                    // gate rows
                        tma_load_2d(dst + BNF * BK * 2, &maps.w, kb * BK, I + nb * BNF, bar_b_full + 8 * st); // matching y rows
                        if (++st == NSTAGE) { st = 0; b_phase ^= 1u; }
                    }
                a_phase ^= 1u;
            }
        }
    } else if (warp == 1) {                       // ---- MMA issuer ---------------------------------------------
        // The whole warp walks the loop (uniform control flow keeps the descriptor arithmetic off the issuing lane's
        // critical path); lane 0 issues.  Descriptors advance by adding to their 14-bit address field (16-byte units).
        uint32_t a_phase = 0, st = 0, b_phase = 0, acc_it = 0;
        const uint32_t a_lo0 = make_desc(sbase), b_lo0 = make_desc(sbase + off_b);
        const uint32_t a_sub = (uint32_t)KB * (A_BOX_BYTES >> 4);
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            const int nb0 = nb_begin(tile), nb1 = nb_end(tile);
            for (int nb = nb0; nb < nb1; ++nb, ++acc_it) {
                const uint32_t buf = acc_it & 1u;
                waiter.wait(bar_acc_empty + 8 * buf, ((acc_it >> 1) & 1u) ^ 1u);    // the epilogue has drained this buffer
                tc_fence_after();
                const uint32_t d0 = tmem + buf * (uint32_t)(S * 128);
                uint32_t a_lo = a_lo0;
                for (int kb = 0; kb < KB; ++kb) {
                    if (nb == nb0) waiter.wait(bar_a_full + 8 * kb, a_phase);
                    waiter.wait(bar_b_full + 8 * st, b_phase);
                    tc_fence_after();
                    const uint32_t b_lo = b_lo0 + st * (B_STAGE_BYTES >> 4);
                    if (lane == 0) {
                        for (int s = 0; s < S; ++s) {
                            const uint32_t a_s = a_lo + s * a_sub, d = d0 + (uint32_t)s * 128u;
                            tc_mma(d, a_s, b_lo, IDESC, kb > 0 ? 1u : 0u);
                            tc_mma(d, a_s + 2, b_lo + 2, IDESC, 1u);
                            tc_mma(d, a_s + 4, b_lo + 4, IDESC, 1u);
                            tc_mma(d, a_s + 6, b_lo + 6, IDESC, 1u);
                        }
                        tc_commit(bar_b_empty + 8 * st);                // the stage is free when these MMAs are done
                        if (nb == nb1 - 1) tc_commit(bar_a_empty + 8 * kb);   // and, in the tile's last block, so is the x box
                    }
                    __syncwarp();
                    a_lo += A_BOX_BYTES >> 4;
                    if (++st == NSTAGE) { st = 0; b_phase ^= 1u; }
                }
                if (lane == 0) tc_commit(bar_acc_full + 8 * buf);
                __syncwarp();
            }
            a_phase ^= 1u;
        }
    } else {                                      // ---- epilogue: silu(gate) * y -> out ----------------------------
        const int ew = warp - 2;                  // 0..7
        const int sub = ew >> 2;                  // subtile
        if (sub < S) {
            const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;
            const int r_in_tile = sub * 128 + 32 * (warp & 3);          // first of this warp's 32 rows within the tile
            uint8_t* box = smem + off_out + ew * OUT_BOX_BYTES;
            const uint32_t box_u32 = sbase + off_out + ew * OUT_BOX_BYTES;
            uint8_t* my_row = box + lane * 128;
            const uint32_t sw = (uint32_t)(lane & 7);
            uint32_t acc_it = 0;
            for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
                const int row0 = (tile / nsplit) * BM + r_in_tile;
                for (int nb = nb_begin(tile); nb < nb_end(tile); ++nb, ++acc_it) {
                    const uint32_t buf = acc_it & 1u;
                    waiter.wait(bar_acc_full + 8 * buf, (acc_it >> 1) & 1u);   // by the whole warp: a wait by one lane with the others parked at a warp barrier resumes microseconds late
                    __syncwarp();
                    tc_fence_after();
                    const uint32_t acc = tmem + lane_base + buf * (uint32_t)(S * 128) + (uint32_t)sub * 128u;
                    uint32_t pk[BNF / 2];
#pragma unroll
                    for (int c = 0; c < BNF; c += 32) {
                        float g[32], y[32];
                        tc_ld32(acc + c, g);
                        tc_ld32(acc + BNF + c, y);
                        tc_wait_ld();
#pragma unroll
                        for (int e = 0; e < 32; e += 2)
                            pk[(c + e) / 2] = Pk<T>::pack(g[e] * y[e] * sigmoid_tanh(g[e]), g[e + 1] * y[e + 1] * sigmoid_tanh(g[e + 1]));
                    }
                    tc_fence_before();
                    mbar_arrive_plain(bar_acc_empty + 8 * buf);               // the accumulator is in registers: the MMA warp may refill it
                    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous store has read the box
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < BNF / 8; ++j)
                        *reinterpret_cast<uint4*>(my_row + (((uint32_t)j ^ sw) << 4)) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0 && row0 < M) {
                        tma_store_2d(&maps.o, nb * BNF, row0, box_u32);  // rows past M are clipped by the tensor map
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
            if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every store has landed before the CTA exits
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace
}  // namespace vig

using namespace vig;

extern "C" int vig_linear_swiglu_supported(int64_t M, int K, int I, int dtype) {
    if (dtype != VIG_DTYPE_BF16 && dtype != VIG_DTYPE_F16) return 0;
    if (M <= 0 || K <= 0 || I <= 0 || K % BK || I % BNF) return 0;
    if ((int64_t)128 * K * 2 > MAX_A_BYTES) return 0;            // one 128-row subtile of x must fit its shared-memory budget
    return tc::encode_fn() != nullptr;
}

// Measured on B200 against cuBLAS + the SwiGLU kernel: 1.5-1.7x faster while two 128-row subtiles of x fit in shared
// memory (K <= 192: the weights are then streamed from L2 once per 256 rows), slower at K = 384.
extern "C" int vig_linear_swiglu_preferred(int64_t M, int K, int I, int dtype) {
    return vig_linear_swiglu_supported(M, K, I, dtype) && (int64_t)256 * K * 2 <= MAX_A_BYTES;
}

extern "C" int vig_linear_swiglu_fwd(const void* x, int64_t ldx, const void* w, void* out, int64_t ldo,
                                     int64_t M, int K, int I, int dtype, int32_t* status_dev, void* stream) {
    if (!x || !w || !out) return VIG_ERR_NULL;
    if (M == 0) return VIG_OK;
    if (!vig_linear_swiglu_supported(M, K, I, dtype)) return VIG_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) return VIG_ERR_ALIGN;
    if (ldx < K || ldo < I || (ldx * 2) % 16 || (ldo * 2) % 16 || M >= (1ll << 31)) return VIG_ERR_ARG;
    GsMaps maps;
    if (!tc::make_map_2d(&maps.x, x, M, K, ldx, 128, dtype) || !tc::make_map_2d(&maps.w, w, 2 * (int64_t)I, K, K, BNF, dtype) ||
        !tc::make_map_2d(&maps.o, out, M, I, ldo, 32, dtype)) return VIG_ERR_DEVICE;
    const int KB = K / BK;
    const int S = ((int64_t)256 * K * 2 <= MAX_A_BYTES && M > 128) ? 2 : 1;
    const int smem = S * KB * A_BOX_BYTES + NSTAGE * B_STAGE_BYTES + OUT_STAGE_BYTES + 8 * (2 * MAX_KB + 2 * NSTAGE + 4) + 16 + 1024;
    int dev = 0, sms = 0;
    cudaError_t e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    // few row tiles (small M): split the feature blocks of a tile over several work items so every SM has work
    const int mtiles = (int)((M + 128 * S - 1) / (128 * S));
    int nsplit = (3 * sms + mtiles - 1) / mtiles;
    if (nsplit < 1) nsplit = 1;
    if (nsplit > I / BNF) nsplit = I / BNF;
    const int ntiles = mtiles * nsplit;
    const int grid = ntiles < sms ? ntiles : sms;
    if (dtype == VIG_DTYPE_BF16) {
        auto kfn = linear_swiglu_kernel<__nv_bfloat16>;
        if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
        kfn<<<grid, GS_THREADS, smem, (cudaStream_t)stream>>>(maps, (int)M, I, KB, S, nsplit, status_dev);
    } else {
        auto kfn = linear_swiglu_kernel<__half>;
        if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
        kfn<<<grid, GS_THREADS, smem, (cudaStream_t)stream>>>(maps, (int)M, I, KB, S, nsplit, status_dev);
    }
    return (int)cudaGetLastError();
}
