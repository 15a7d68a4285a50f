// out[M, I] = swiglu(x Wg^T, x Wy^T) = silu(x Wg^T) * (x Wy^T), with W = [Wg ; Wy] of shape [2I, K]:
// the gate projection of the SwiGLU MLP and its activation in one kernel, so the [M, 2I] intermediate
// (classification/models/vig.py:494-497: gate_proj -> chunk -> swiglu) never goes to HBM.
//
// tcgen05 GEMM.  A persistent CTA owns tiles of BM = 128*S rows of x; the tile's whole K extent stays resident
// in shared memory (TMA, 128-byte swizzle), the weights stream through a 96 KB ring holding, per k box, 64 gate
// rows and the 64 matching y rows, so one M128 N128 MMA per subtile fills an accumulator [128 x (64 gate | 64 y)]
// in tensor memory.  Accumulators are double buffered: while the MMA warp works on feature block n+1, the
// epilogue warps read block n with tcgen05.ld and apply silu(g)*y.
//
// What the timeline of the MMA warp showed, and what the organisation answers:
//  * tcgen05.mma issue is synchronous with the tensor pipe (a 128x128x16 MMA costs ~80 cycles to issue back to back),
//    so every cycle the issuing warp spends elsewhere is a cycle the tensor pipe idles.  A wait on an already completed
//    mbarrier costs ~200 cycles and a lane-0 branch around the issue another ~200 to reconverge: the ring is therefore
//    handed over in groups of up to 3 k boxes (one wait and one commit per group instead of per box), and the loops
//    are walked by the whole warp with only the issuing instruction predicated on the lane.
//  * an epilogue warp works through its piece in one dependent chain (TMEM load -> 64 sigmoids -> pack -> store), so
//    eight warps took ~4000 cycles per feature block, longer than its MMAs.  Sixteen warps now share a block, each
//    with [32 rows x 32 features]; a warp packs its piece into a 2 KB box of shared memory and lane 0 sends it out
//    with one TMA store (a thread owns a row, so direct stores would touch 32 lines per request).
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2..17 epilogue.  Every wait is bounded.
#include "tc_common.cuh"

namespace vig {
namespace {

using namespace tc;

constexpr int BK = 64;                         // k elements per stage row (128 bytes)
constexpr int BNF = 64;                        // features per block: 64 gate rows + 64 y rows -> MMA N = 128
constexpr int NSTAGE = 6;                      // weight k boxes in flight (16 KB each)
constexpr int MAX_KB = 6;                      // k boxes of an x tile (K <= 384)
constexpr int A_BOX_BYTES = 128 * BK * 2;      // one [128 rows x 64 k] box
constexpr int B_STAGE_BYTES = 2 * BNF * BK * 2;
constexpr int MAX_A_BYTES = 96 * 1024;
constexpr int GS_EPI_WARPS = 16;
constexpr int GS_THREADS = 64 + 32 * GS_EPI_WARPS;
constexpr int OUT_BOX_BYTES = 32 * 32 * 2;     // one epilogue warp's [32 rows x 32 features] box
constexpr int OUT_STAGE_BYTES = GS_EPI_WARPS * OUT_BOX_BYTES;

// sigmoid(x) = 0.5 tanh(x / 2) + 0.5 with the single-instruction tanh: one MUFU per element instead of two
// (exp + reciprocal); its error (~2^-11) is below the bf16 / fp16 output step.
__device__ __forceinline__ float sigmoid_tanh(float x) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
    return fmaf(t, 0.5f, 0.5f);
}

template <typename T> struct Pk;
template <> struct Pk<__nv_bfloat16> { static constexpr uint32_t FMT = 1;
    __device__ static uint32_t pack(float a, float b) { __nv_bfloat162 t = __floats2bfloat162_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); } };
template <> struct Pk<__half> { static constexpr uint32_t FMT = 0;
    __device__ static uint32_t pack(float a, float b) { __half2 t = __floats2half2_rn(a, b); return *reinterpret_cast<uint32_t*>(&t); } };

struct GsMaps { CUtensorMap x, w, o; };

// silu(g) * y for 32 features of a row, packed to 16-bit pairs.  The arithmetic runs two-wide (mul / fma .f32x2 on register
// pairs: the epilogue warps are bound by instruction issue); each lane of those is the scalar IEEE operation.
template <typename T>
__device__ __forceinline__ void swiglu_pack(const float* g, const float* y, uint32_t* pk) {
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
        unsigned long long g2, y2, h2, half2, s2, r2;
        asm("mov.b64 %0, {%1, %2};" : "=l"(g2) : "f"(g[e]), "f"(g[e + 1]));
        asm("mov.b64 %0, {%1, %2};" : "=l"(y2) : "f"(y[e]), "f"(y[e + 1]));
        asm("mov.b64 %0, {%1, %1};" : "=l"(half2) : "f"(0.5f));
        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(h2) : "l"(g2), "l"(half2));
        float h0, h1, t0, t1;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(h0), "=f"(h1) : "l"(h2));
        asm("tanh.approx.f32 %0, %1;" : "=f"(t0) : "f"(h0));
        asm("tanh.approx.f32 %0, %1;" : "=f"(t1) : "f"(h1));
        asm("mov.b64 %0, {%1, %2};" : "=l"(s2) : "f"(t0), "f"(t1));
        asm("fma.rn.f32x2 %0, %1, %2, %2;" : "=l"(s2) : "l"(s2), "l"(half2));   // sigmoid = 0.5 tanh(g / 2) + 0.5
        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r2) : "l"(g2), "l"(y2));
        asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r2) : "l"(r2), "l"(s2));
        float r0, r1;
        asm("mov.b64 {%0, %1}, %2;" : "=f"(r0), "=f"(r1) : "l"(r2));
        pk[e / 2] = Pk<T>::pack(r0, r1);
    }
}

// A warp's [32 rows x 32 features] piece goes out through its 2 KB box of shared memory (64-byte rows) as one TMA store.
__device__ __forceinline__ void send_box(uint8_t* my_row, uint32_t box_u32, const uint32_t* pk, const CUtensorMap* map, int col, int row,
                                         bool in_range, int lane) {
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous store has read the box
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(my_row + 16 * j) = make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0 && in_range) {
        tma_store_2d(map, col, row, box_u32);      // rows past M are clipped by the tensor map
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}

// S = subtiles of 128 rows per CTA tile (1 or 2); KB = K / 64; G = k boxes handed over together (a divisor of KB, <= 3).
template <typename T>
__global__ void __launch_bounds__(GS_THREADS, 1) linear_swiglu_kernel(const __grid_constant__ GsMaps maps, int M, int I, int KB, int S, int G, int nsplit, int32_t* status) {
    extern __shared__ uint8_t gs_smem_raw[];
    uint8_t* smem = gs_smem_raw + ((1024u - (smem_u32(gs_smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t a_bytes = (uint32_t)S * KB * A_BOX_BYTES;
    const uint32_t off_b = a_bytes;
    const uint32_t off_out = off_b + NSTAGE * B_STAGE_BYTES;
    const uint32_t off_bar = off_out + OUT_STAGE_BYTES;
    const uint32_t bar_a_full = sbase + off_bar, bar_a_empty = bar_a_full + 8 * MAX_KB;   // one pair per k box of the x tile
    const uint32_t bar_b_full = bar_a_empty + 8 * MAX_KB, bar_b_empty = bar_b_full + 8 * NSTAGE;   // one pair per group stage
    const uint32_t bar_acc_full = bar_b_empty + 8 * NSTAGE, bar_acc_empty = bar_acc_full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + off_bar + 8 * (2 * MAX_KB + 2 * NSTAGE + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const Waiter waiter{abort_flag, status};
    const int NG = NSTAGE / G;                     // group stages in the ring
    const int groups = KB / G;                     // groups per feature block

    if (tid == 0) {
        for (int kb = 0; kb < MAX_KB; ++kb) { mbar_init(bar_a_full + 8 * kb, 1); mbar_init(bar_a_empty + 8 * kb, 1); }
        for (int s = 0; s < NSTAGE; ++s) { mbar_init(bar_b_full + 8 * s, 1); mbar_init(bar_b_empty + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, 8 * S); }
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
    constexpr uint32_t IDESC = make_idesc(Pk<T>::FMT, 0, 0, 128, 128);

    if (warp == 0) {
        if (lane == 0) {                          // ---- TMA producer -------------------------------------------
            // The x tile is handed over per k box: box kb of the next tile is requested as soon as the last feature
            // block of this tile has used box kb, just ahead of the weight group that needs it.
            uint32_t a_phase = 0, st = 0, b_phase = 0;
            for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
                const int nb0 = nb_begin(tile), nb1 = nb_end(tile);
                for (int nb = nb0; nb < nb1; ++nb)
                    for (int gi = 0; gi < groups; ++gi) {
                        if (nb == nb0) {
                            for (int kb = gi * G; kb < (gi + 1) * G; ++kb) {
                                waiter.wait(bar_a_empty + 8 * kb, a_phase ^ 1u);    // the previous tile's MMAs have read this box
                                mbar_expect_tx(bar_a_full + 8 * kb, (uint32_t)S * A_BOX_BYTES);
                                for (int s = 0; s < S; ++s)
                                    tma_load_2d(sbase + (s * KB + kb) * A_BOX_BYTES, &maps.x, kb * BK, (tile / nsplit) * BM + s * 128, bar_a_full + 8 * kb);
                            }
                        }
                        waiter.wait(bar_b_empty + 8 * st, b_phase ^ 1u);
                        mbar_expect_tx(bar_b_full + 8 * st, (uint32_t)G * B_STAGE_BYTES);
                        for (int g = 0; g < G; ++g) {
                            const int kb = gi * G + g;
                            const uint32_t dst = sbase + off_b + (st * G + g) * B_STAGE_BYTES;
                            tma_load_2d(dst, &maps.w, kb * BK, nb * BNF, bar_b_full + 8 * st);                    // gate rows
                            tma_load_2d(dst + BNF * BK * 2, &maps.w, kb * BK, I + nb * BNF, bar_b_full + 8 * st); // matching y rows
                        }
                        if ((int)++st == NG) { st = 0; b_phase ^= 1u; }
                    }
                a_phase ^= 1u;
            }
        }
    } else if (warp == 1) {                       // ---- MMA issuer ---------------------------------------------
        // Descriptors advance by adding to their 14-bit address field (16-byte units).
        // A test of an mbarrier costs a few hundred cycles here even when its phase completed long ago (it queues behind the
        // epilogue warps' shared-memory traffic), and while the warp waits for the answer nothing is issued to the tensor
        // pipe.  The barriers of the next group (and of the next accumulator buffer) are therefore tested BEFORE the current
        // group's last MMAs are issued (with the non-blocking test): the answer arrives while those are being issued, and the
        // wait loop is entered only if it was "not yet".
        const bool issuer = lane == 0;
        uint32_t a_phase = 0, st = 0, b_phase = 0, acc_it = 0;
        const uint32_t a_lo0 = make_desc(sbase), b_lo0 = make_desc(sbase + off_b);
        const uint32_t a_sub = (uint32_t)KB * (A_BOX_BYTES >> 4);
        uint32_t pre_b = 0, pre_acc = 0;              // early answers for the next group's stage / the next block's buffer
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            const int nb0 = nb_begin(tile), nb1 = nb_end(tile);
            for (int nb = nb0; nb < nb1; ++nb, ++acc_it) {
                const uint32_t buf = acc_it & 1u;
                if (!pre_acc) waiter.wait_lite(bar_acc_empty + 8 * buf, ((acc_it >> 1) & 1u) ^ 1u);    // the epilogue has drained this buffer
                pre_acc = 0;
                const uint32_t d0 = tmem + buf * (uint32_t)(S * 128);
                for (int gi = 0; gi < groups; ++gi) {
                    if (nb == nb0)
                        for (int kb = gi * G; kb < (gi + 1) * G; ++kb) waiter.wait_lite(bar_a_full + 8 * kb, a_phase);
                    if (!pre_b) waiter.wait_lite(bar_b_full + 8 * st, b_phase);
                    tc_fence_after();
                    const uint32_t st_next = (int)(st + 1) == NG ? 0u : st + 1, ph_next = (int)(st + 1) == NG ? b_phase ^ 1u : b_phase;
                    for (int g = 0; g < G; ++g) {
                        // early tests, put before the group's last k box (its MMAs give the answer time to arrive, and the
                        // stage asked about has had the longest time to fill): the next group's stage, and before a
                        // block's last group the next block's buffer
                        if (g == G - 1) {
                            pre_b = mbar_test_wait(bar_b_full + 8 * st_next, ph_next);
                            if (gi == groups - 1) pre_acc = mbar_test_wait(bar_acc_empty + 8 * (buf ^ 1u), (((acc_it + 1) >> 1) & 1u) ^ 1u);
                        }
                        const int kb = gi * G + g;
                        const uint32_t b_lo = b_lo0 + (st * G + g) * (B_STAGE_BYTES >> 4);
                        const uint32_t a_lo = a_lo0 + kb * (A_BOX_BYTES >> 4);
                        for (int s = 0; s < S; ++s) {
                            const uint32_t a_s = a_lo + s * a_sub, d = d0 + (uint32_t)s * 128u;
#pragma unroll
                            for (uint32_t k4 = 0; k4 < 4; ++k4) { if (issuer) tc_mma(d, a_s + 2 * k4, b_lo + 2 * k4, IDESC, (kb | k4) > 0 ? 1u : 0u); }
                        }
                    }
                    if (issuer) tc_commit(bar_b_empty + 8 * st);        // the group's stage is free when these MMAs are done
                    if (nb == nb1 - 1)                                  // and, in the tile's last block, so are its x boxes
                        for (int kb = gi * G; kb < (gi + 1) * G; ++kb) { if (issuer) tc_commit(bar_a_empty + 8 * kb); }
                    st = st_next; b_phase = ph_next;
                }
                if (issuer) tc_commit(bar_acc_full + 8 * buf);
                if (*abort_flag) break;
            }
            if (*abort_flag) break;
            a_phase ^= 1u;
        }
    } else {                                      // ---- epilogue: silu(gate) * y -> out ----------------------------
        const int ew = warp - 2;                  // 0..15
        const int sub = (ew >> 2) & 1;            // subtile
        const int fh = ew >> 3;                   // which 32 of the block's 64 features
        if (sub < S) {
            const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;   // a warp reads the TMEM lanes of its quarter
            const int r_in_tile = sub * 128 + 32 * (warp & 3);          // first of this warp's 32 rows within the tile
            uint8_t* my_row = smem + off_out + ew * OUT_BOX_BYTES + lane * 64;
            const uint32_t box_u32 = sbase + off_out + ew * OUT_BOX_BYTES;
            uint32_t acc_it = 0;
            for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
                const int row0 = (tile / nsplit) * BM + r_in_tile;
                for (int nb = nb_begin(tile); nb < nb_end(tile); ++nb, ++acc_it) {
                    const uint32_t buf = acc_it & 1u;
                    waiter.wait_lite(bar_acc_full + 8 * buf, (acc_it >> 1) & 1u);   // by the whole warp: a wait by one lane with the others parked at a warp barrier resumes microseconds late
                    if (*abort_flag) break;
                    tc_fence_after();
                    const uint32_t acc = tmem + lane_base + buf * (uint32_t)(S * 128) + (uint32_t)sub * 128u + 32u * fh;
                    float g[32], y[32];
                    tc_ld32(acc, g);
                    tc_ld32(acc + BNF, y);
                    tc_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_plain(bar_acc_empty + 8 * buf);   // the accumulator is in registers: the MMA warp may refill it
                    uint32_t pk[16];
                    swiglu_pack<T>(g, y, pk);
                    send_box(my_row, box_u32, pk, &maps.o, nb * BNF + 32 * fh, row0, row0 < M, lane);
                }
                if (*abort_flag) break;
            }
            if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every store has landed before the CTA exits
        }
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort_flag && status) atomicOr(status, 1);
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}


// ---------------------------------------------------------------------------------------------------
// Weight-stationary form, for K <= 192 and I % 128 == 0 (the shipped MLP shapes at widths up to 192) and many rows.
//
// A 128x128x16 MMA takes ~80-130 cycles here where a 128x256x16 one takes ~130: at N = 128 the tensor pipe runs at half its
// rate.  This form multiplies a 128-row tile of x by 128 gate rows and their 128 y rows at once (N = 256).  A persistent CTA
// owns ONE block of 128 features for the whole launch: its [256 x K] slice of W (96 KB at K = 192) is loaded once and stays
// in shared memory, the x tiles stream through a two-stage ring (48 KB each), the accumulator [128 x 256] takes half of
// tensor memory and the two halves double-buffer (tile t+1 is multiplied while tile t is read out).  The CTAs that hold
// the feature blocks of the same row tile have consecutive block indices and run in step, so a tile of x comes from DRAM
// once and from L2 for the others.  (An earlier N = 256 form kept 256 rows of x resident and streamed the weights through
// a ring that held exactly one block's boxes: every block began by waiting for reloads, 134 us; before that the N = 128
// form, 155-165 us.)
constexpr int WB_FEAT = 128;                         // features per block
constexpr int WB_BOX_BYTES = 2 * WB_FEAT * BK * 2;   // one k box of the CTA's weight slice: 128 gate rows + 128 y rows, 32 KB
constexpr int WB_XSTAGES = 2;

struct GsWideMaps { CUtensorMap x, w, o; };

// grid = row_groups * nblocks CTAs; CTA i holds feature block i % nblocks and walks row tiles i / nblocks, + row_groups, ...
template <typename T>
__global__ void __launch_bounds__(GS_THREADS, 1) linear_swiglu_wide_kernel(const __grid_constant__ GsWideMaps maps, int M, int I, int KB, int nblocks,
                                                                           int row_groups, int32_t* status) {
    extern __shared__ uint8_t gs_smem_raw[];
    uint8_t* smem = gs_smem_raw + ((1024u - (smem_u32(gs_smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t off_x = (uint32_t)KB * WB_BOX_BYTES;                     // after the weight slice
    const uint32_t x_stage = (uint32_t)KB * A_BOX_BYTES;
    const uint32_t off_out = off_x + WB_XSTAGES * x_stage;
    const uint32_t off_bar = off_out + OUT_STAGE_BYTES;
    // barriers: weight slice full; x stages full / empty; accumulator halves full / empty
    const uint32_t bar_w = sbase + off_bar;
    const uint32_t bar_x_full = bar_w + 8, bar_x_empty = bar_x_full + 8 * WB_XSTAGES;
    const uint32_t bar_acc_full = bar_x_empty + 8 * WB_XSTAGES, bar_acc_empty = bar_acc_full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + off_bar + 8 * (1 + 2 * WB_XSTAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const Waiter waiter{abort_flag, status};

    if (tid == 0) {
        mbar_init(bar_w, 1);
        for (int i = 0; i < WB_XSTAGES; ++i) { mbar_init(bar_x_full + 8 * i, 1); mbar_init(bar_x_empty + 8 * i, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar_acc_full + 8 * b, 1); mbar_init(bar_acc_empty + 8 * b, GS_EPI_WARPS / 2); }
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
    constexpr uint32_t IDESC = make_idesc(Pk<T>::FMT, 0, 0, 128, 256);

    if (warp == 0) {
        if (lane == 0) {                          // ---- TMA producer -------------------------------------------
            mbar_expect_tx(bar_w, (uint32_t)KB * WB_BOX_BYTES);
            for (int kb = 0; kb < KB; ++kb) {
                tma_load_2d(sbase + kb * WB_BOX_BYTES, &maps.w, kb * BK, nb * WB_FEAT, bar_w);                          // gate rows
                tma_load_2d(sbase + kb * WB_BOX_BYTES + WB_FEAT * BK * 2, &maps.w, kb * BK, I + nb * WB_FEAT, bar_w);   // matching y rows
            }
            uint32_t st = 0, phase = 0;
            for (int tile = rg; tile < ntiles; tile += row_groups) {
                waiter.wait(bar_x_empty + 8 * st, phase ^ 1u);            // the MMAs of the tile two back have read this stage
                if (*abort_flag) break;
                mbar_expect_tx(bar_x_full + 8 * st, x_stage);
                for (int kb = 0; kb < KB; ++kb)
                    tma_load_2d(sbase + off_x + st * x_stage + kb * A_BOX_BYTES, &maps.x, kb * BK, tile * 128, bar_x_full + 8 * st);
                if (++st == WB_XSTAGES) { st = 0; phase ^= 1u; }
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
            if (!pre_acc) waiter.wait_lite(bar_acc_empty + 8 * buf, ((it >> 1) & 1u) ^ 1u);   // the epilogue has read this half out
            if (!pre_x) waiter.wait_lite(bar_x_full + 8 * st, phase);
            if (*abort_flag) break;
            tc_fence_after();
            // asked before this tile's MMAs, answered while they are issued: the next tile's stage and accumulator half
            const uint32_t st_next = st + 1 == WB_XSTAGES ? 0u : st + 1, ph_next = st + 1 == WB_XSTAGES ? phase ^ 1u : phase;
            pre_x = mbar_test_wait(bar_x_full + 8 * st_next, ph_next);
            pre_acc = mbar_test_wait(bar_acc_empty + 8 * (buf ^ 1u), (((it + 1) >> 1) & 1u) ^ 1u);
            const uint32_t d = tmem + buf * 256u;
            for (int kb = 0; kb < KB; ++kb) {
                const uint32_t a_lo = x_lo0 + (st * x_stage >> 4) + (uint32_t)kb * (A_BOX_BYTES >> 4);
                const uint32_t b_lo = w_lo0 + (uint32_t)kb * (WB_BOX_BYTES >> 4);
#pragma unroll
                for (uint32_t k4 = 0; k4 < 4; ++k4) { if (issuer) tc_mma(d, a_lo + 2 * k4, b_lo + 2 * k4, IDESC, (kb | k4) > 0 ? 1u : 0u); }
            }
            if (issuer) { tc_commit(bar_x_empty + 8 * st); tc_commit(bar_acc_full + 8 * buf); }
            st = st_next; phase = ph_next;
        }
    } else {                                      // ---- epilogue: silu(gate) * y -> out ----------------------------
        // Two sets of eight warps take alternate tiles (set = accumulator half), so a warp has two tile periods for its
        // [32 rows x 64 features]: the epilogue of a tile is a chain of latencies (accumulator ready -> TMEM load -> 32 sigmoids
        // -> box -> store, ~3 k cycles) longer than the tile's MMAs, and with all sixteen warps on every tile it set the pace.
        const int ew = warp - 2;                  // 0..15
        const uint32_t set = (uint32_t)ew >> 3;   // tiles of which parity / which accumulator half
        const int fh = (ew >> 2) & 1;             // which 64 of the block's 128 features (taken as two halves of 32)
        const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;   // a warp reads the TMEM lanes of its quarter
        uint8_t* my_row = smem + off_out + ew * OUT_BOX_BYTES + lane * 64;
        const uint32_t box_u32 = sbase + off_out + ew * OUT_BOX_BYTES;
        const uint32_t acc = tmem + lane_base + set * 256u + 64u * fh;
        uint32_t it = 0, uses = 0;
        for (int tile = rg; tile < ntiles; tile += row_groups, ++it) {
            if ((it & 1u) != set) continue;
            waiter.wait_lite(bar_acc_full + 8 * set, uses & 1u);   // by the whole warp
            ++uses;
            if (*abort_flag) break;
            tc_fence_after();
            const int row0 = tile * 128 + 32 * (warp & 3);
            const int col0 = nb * WB_FEAT + 64 * fh;
            float g[32], y[32];
            uint32_t pk[16];
            tc_ld32(acc, g);
            tc_ld32(acc + WB_FEAT, y);
            tc_wait_ld();
            swiglu_pack<T>(g, y, pk);
            tc_ld32(acc + 32, g);
            tc_ld32(acc + WB_FEAT + 32, y);
            tc_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_plain(bar_acc_empty + 8 * set);   // the accumulator is in registers: the MMA warp may refill it
            send_box(my_row, box_u32, pk, &maps.o, col0, row0, row0 < M, lane);
            swiglu_pack<T>(g, y, pk);
            send_box(my_row, box_u32, pk, &maps.o, col0 + 32, row0, row0 < M, lane);
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

}  // namespace
}  // namespace vig

using namespace vig;

// [rows, cols] output with leading dimension ld: boxes of 32 rows x 32 columns (64-byte rows, no swizzle), one per epilogue warp
static bool make_out_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int dtype) {
    tc::MapKey key{};
    key.base = base; key.rank = 2; key.dtype = dtype; key.swizzle = 0;
    key.dims[0] = (uint64_t)cols; key.dims[1] = (uint64_t)rows;
    key.strides[0] = (uint64_t)ld * 2;
    key.box[0] = 32; key.box[1] = 32;
    return tc::encode_cached(m, key);
}

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
    const int KB = K / BK;
    int dev = 0, sms = 0;
    cudaError_t e;
    if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
    if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
    if (KB <= 3 && I % WB_FEAT == 0 && M >= 256 * (int64_t)sms && I / WB_FEAT <= sms) {
        // weight-stationary form: N = 256 MMAs, a CTA per feature block and row group, when there are enough rows to fill the machine
        GsWideMaps maps;
        if (!tc::make_map_2d(&maps.x, x, M, K, ldx, 128, dtype) || !tc::make_map_2d(&maps.w, w, 2 * (int64_t)I, K, K, WB_FEAT, dtype) ||
            !make_out_map(&maps.o, out, M, I, ldo, dtype)) return VIG_ERR_DEVICE;
        const int smem = KB * WB_BOX_BYTES + WB_XSTAGES * KB * A_BOX_BYTES + OUT_STAGE_BYTES + 8 * (1 + 2 * WB_XSTAGES + 4) + 16 + 1024;
        const int nblocks = I / WB_FEAT;
        const int ntiles = (int)((M + 127) / 128);
        int row_groups = sms / nblocks;                        // CTAs per feature block
        if (row_groups > ntiles) row_groups = ntiles;
        const int grid = row_groups * nblocks;
        if (dtype == VIG_DTYPE_BF16) {
            auto kfn = linear_swiglu_wide_kernel<__nv_bfloat16>;
            if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
            kfn<<<grid, GS_THREADS, smem, (cudaStream_t)stream>>>(maps, (int)M, I, KB, nblocks, row_groups, status_dev);
        } else {
            auto kfn = linear_swiglu_wide_kernel<__half>;
            if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
            kfn<<<grid, GS_THREADS, smem, (cudaStream_t)stream>>>(maps, (int)M, I, KB, nblocks, row_groups, status_dev);
        }
        return (int)cudaGetLastError();
    }
    GsMaps maps;
    if (!tc::make_map_2d(&maps.x, x, M, K, ldx, 128, dtype) || !tc::make_map_2d(&maps.w, w, 2 * (int64_t)I, K, K, BNF, dtype) ||
        !make_out_map(&maps.o, out, M, I, ldo, dtype)) return VIG_ERR_DEVICE;
    const int G = KB % 3 == 0 ? 3 : (KB % 2 == 0 ? 2 : 1);       // k boxes handed over together
    const int S = ((int64_t)256 * K * 2 <= MAX_A_BYTES && M > 128) ? 2 : 1;
    const int smem = S * KB * A_BOX_BYTES + NSTAGE * B_STAGE_BYTES + OUT_STAGE_BYTES + 8 * (2 * MAX_KB + 2 * NSTAGE + 4) + 16 + 1024;
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
        kfn<<<grid, GS_THREADS, smem, (cudaStream_t)stream>>>(maps, (int)M, I, KB, S, G, nsplit, status_dev);
    } else {
        auto kfn = linear_swiglu_kernel<__half>;
        if ((e = tc::ensure_smem_attr(reinterpret_cast<const void*>(kfn), smem)) != cudaSuccess) return (int)e;
        kfn<<<grid, GS_THREADS, smem, (cudaStream_t)stream>>>(maps, (int)M, I, KB, S, G, nsplit, status_dev);
    }
    return (int)cudaGetLastError();
}
