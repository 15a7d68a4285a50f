// Bi-directional gated linear attention on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 / fp16.
//
// One CTA owns one (segment, batch*head): up to SEG_CHUNKS chunks of 128 tokens (two CTAs share an SM, so
// one of them computes gates while the other waits for TMA or the tensor pipe).  It sweeps its chunks
// twice -- left to right with the forward gates, right to left with the backward gates -- and keeps the
// output accumulators of all its chunks in tensor memory between the sweeps, so q/k/v and both gate
// tensors are fetched by TMA once per sweep and the output is written once.  Per chunk and direction:
//
//   G_i      inclusive cumulative log-gate inside the chunk (prefix for forward, suffix for backward), fp32
//   Qt, Kt   q * scale * exp(G_i - G_ref),  k * exp(G_ref - G_j)     (G_ref = G at the chunk's middle)
//   P        = mask(Qt Kt^T)            128x128x dk   MMA, accumulator in TMEM, masked to j<=i (j>=i)
//   O_chunk += bf16(P) V                128x 64x128   MMA
//   O_chunk += Qt (exp(G_ref) * S_in)   128x 64x dk   MMA   (S_in = state entering the chunk)
//   U        = Kt^T V                    64x 64x128   MMA   (both operands MN-major views of the tiles)
//   S_out    = exp(G_last) * S_in + exp(G_last - G_ref) * U          (fp32, in registers)
//
// Sequences longer than one segment use the same kernel three times over: STATES_ONLY per segment from a
// zero state, the scan over segments (SIMT, tiny), then the full pass with each segment's entering states.
//
// Every wait on an mbarrier is bounded: when it runs out the CTA sets bit 0 of the status word, stops
// waiting on anything else, finishes its control flow and frees its tensor memory.
#include "tc_common.cuh"

namespace vig {
namespace {

using namespace tc;
constexpr int SEG_CHUNKS = 2;         // chunks per CTA: 2 x 64 TMEM columns of output accumulators
constexpr int SEG = CHUNK * SEG_CHUNKS;
constexpr int NTHREADS = 256;
constexpr int DV = 64;

// TMEM columns (fp32), 256 per CTA so that two CTAs fit in an SM's 512: scores for key columns 0..63,
// scores for key columns 64..127 (reused for the state update once the scores are read), outputs
constexpr uint32_t TM_P0 = 0, TM_P1 = 64, TM_U = 64, TM_O = 128, TM_COLS = 256;

// shared memory map (bytes from a 1024-aligned base); ~108 KB so that two CTAs fit in one SM
constexpr int TILE_B = CHUNK * 64 * 2;                       // 16 KB: 128 rows x 128 B
constexpr int OFF_RQ = 0;                                    // raw q tile; later the P tile of key columns 0..63
constexpr int OFF_RK = OFF_RQ + TILE_B;                      // raw k tile
constexpr int OFF_RG = OFF_RK + TILE_B;                      // raw gate tile
constexpr int OFF_V = OFF_RG + TILE_B;                       // v tile (128-byte swizzle, MMA operand as loaded)
constexpr int OFF_QT = OFF_V + TILE_B;                       // scaled q operand; later the P tile of key columns 64..127
constexpr int OFF_KT = OFF_QT + TILE_B;
constexpr int OFF_ST = OFF_KT + TILE_B;                      // bf16 state operand, 64 rows x 128 B
constexpr int OFF_PART = OFF_ST + 64 * 128;                  // fp32 [16][64] group sums of log-gates
constexpr int OFF_VEC = OFF_PART + 16 * 64 * 4;              // fp32 [2][64]: exp(G_last), exp(G_last - G_ref)
constexpr int OFF_GTOT = OFF_VEC + 2 * 64 * 4;               // fp32 [64] summed log-gates of the segment
constexpr int OFF_BAR = OFF_GTOT + 64 * 4;                   // mbarriers: gk, q, v, p, o, x
constexpr int OFF_MISC = OFF_BAR + 8 * 8;                    // tmem base, abort flag, current work item
constexpr int OFF_CVEC = OFF_PART + 2048;                    // fp32 [4][64]: log2 scale of the deferred cross-segment term
                                                             // (the group sums use only the first 2 KB of their 4 KB)
constexpr int SMEM_BYTES = OFF_MISC + 16 + 1024;             // + slack for the manual 1024-byte alignment             // + slack for the manual 1024-byte alignment

// 128-thread named barriers with immediate ids (a register id would make the compiler reserve all 16 barriers)
__device__ __forceinline__ void half_bar_sync(int half) {
    if (half) asm volatile("bar.sync 2, 128;" ::: "memory");
    else asm volatile("bar.sync 1, 128;" ::: "memory");
}



// MODE 0: one segment per CTA, entering states from the workspace (or the caller's initial states).
// MODE 1: states only -- local end states of every segment from a zero state, no q, no output.
// MODE 2: single launch for long sequences.  Persistent CTAs draw (b*h, segment) items from a ticket counter; an
//         item is swept from a ZERO state, which yields its local end states (published for the other segments
//         of the sequence) and the output without the term that comes from the state entering the segment:
//             o_i += (q_i * 2^{G_i}) . S_enter        (G_i = cumulative gate from the segment's edge to token i)
//         The scaled q operand tiles are parked in a per-CTA scratch (L2-resident); when all segments of the
//         sequence have published, the CTA folds the other segments' states into S_enter and adds the missing
//         term with four small MMAs on the parked tiles, while the output accumulators are still in tensor memory.
//         Tickets are handed out in order, so the oldest unfinished sequence always has all its segments in
//         flight provided the grid holds at least as many resident CTAs as a sequence has segments (host check).
template <int DK, typename T, int MODE>
__global__ void __launch_bounds__(NTHREADS, 2) bigla_tc_kernel(const __grid_constant__ TcMaps maps, BiglaParams p, int use_ws) {
    constexpr bool STATES_ONLY = MODE == 1;
    constexpr bool FUSED = MODE == 2;
    extern __shared__ uint8_t smem_raw[];
    // align by an integer offset (not by casting through an integer) so that accesses stay shared-space loads
    uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nseg = FUSED ? p.nseg : (int)gridDim.x;
    int seg = blockIdx.x, bh = blockIdx.y, b = 0, h = 0, seg_t0 = 0, nch = 0, n_iter = 0;   // the current work item

    const uint32_t bar_gk = sbase + OFF_BAR, bar_q = bar_gk + 8, bar_v = bar_gk + 16, bar_p0 = bar_gk + 24, bar_o = bar_gk + 32;
    const uint32_t bar_x = bar_gk + 40;
    float* cvec = reinterpret_cast<float*>(smem + OFF_CVEC);
    volatile int* item_slot = reinterpret_cast<volatile int*>(smem + OFF_MISC + 8);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + OFF_MISC + 4);
    float* part = reinterpret_cast<float*>(smem + OFF_PART);
    float* vec = reinterpret_cast<float*>(smem + OFF_VEC);
    float* gtot = reinterpret_cast<float*>(smem + OFF_GTOT);
    const Waiter waiter{abort_flag, p.status};

    if (tid == 0) {
        // the tensor-core barriers count two arrivals: the MMAs of a step are issued by two threads (see `issuer`)
        mbar_init(bar_gk, 1); mbar_init(bar_q, 1); mbar_init(bar_v, 1); mbar_init(bar_p0, 2); mbar_init(bar_o, 2); mbar_init(bar_x, 2);
        *abort_flag = 0;
        if (FUSED) *item_slot = (int)atomicAdd(p.ticket, 1u);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // ---- thread roles ---------------------------------------------------------------------------
    // gate preparation: CPW lanes cover the channel pairs of one token row; a warp covers 32/CPW rows at once
    constexpr int CPW = DK / 2;
    constexpr int RPW = 32 / CPW;                 // token groups per warp
    constexpr int NG = 8 * RPW;                   // token groups per chunk
    constexpr int TPG = CHUNK / NG;               // tokens per group (16 for dk=64, 8 for dk=32)
    const int cp = lane % CPW;
    const int grp = warp * RPW + lane / CPW;
    // state rows: an M=64 accumulator puts row r in TMEM lane (r % 16) + 32 * (r / 16)
    // (16 TMEM lanes of each warp's quadrant).  A warp reads 32 columns of its 16 rows; lanes 0-15 keep columns
    // 0-15 of them and hand columns 16-31 to lanes 16-31, so every thread carries 16 state values.
    const int st_row = 16 * (warp & 3) + (lane & 15);         // key channel
    const bool st_thread = st_row < DK;
    const int st_ld0 = 32 * (warp >> 2);                      // first of the 32 value columns my warp reads
    const int st_col0 = st_ld0 + 16 * (lane >> 4);            // first of my 16 value columns
    const uint32_t lane_base = (uint32_t)(32 * (warp & 3)) << 16;
    const bool raw_logits = p.gate_norm > 0.f;
    const float inv_norm = raw_logits ? 1.f / p.gate_norm : 1.f;
    const float clamp_lo = (p.clamp_min == p.clamp_min) ? p.clamp_min * LOG2E : -INFINITY;
    const float lq = __log2f(fabsf(p.qscale));   // |scale * out_scale| folded into the exponent of the q operand
    const float o_sign = p.qscale < 0.f ? -1.f : 1.f;

    constexpr uint32_t IDESC_QK = make_idesc(Pack2<T>::FMT, 0, 0, 128, 128);
    constexpr uint32_t IDESC_OV = make_idesc(Pack2<T>::FMT, 0, 1, 128, 64);
    constexpr uint32_t IDESC_U = make_idesc(Pack2<T>::FMT, 1, 1, 64, 64);

    const int dir_first = (p.dir_mask & 1) ? 0 : 1, dir_last = (p.dir_mask & 2) ? 1 : 0;

    // Tiles of iteration n (thread 0 only).  Three groups with their own barriers, because their buffers become
    // free at different times: k and the gates right after the operand tiles are written, q and v only when
    // the MMAs of the iteration are done (the q buffer is reused for scores, v is an MMA operand).
    auto chunk_t0 = [&](int n) {
        const int dir = dir_first + n / nch, ci = n % nch;
        return seg_t0 + (dir ? nch - 1 - ci : ci) * CHUNK;
    };
    auto issue_gk = [&](int n) {
        const int dir = dir_first + n / nch, t0 = chunk_t0(n);
        mbar_expect_tx(bar_gk, 2 * CHUNK * DK * 2);
        tma_load_4d(sbase + OFF_RK, &maps.k, 0, t0, h, b, bar_gk);
        tma_load_4d(sbase + OFF_RG, dir ? &maps.gb : &maps.gf, 0, t0, h, b, bar_gk);
    };
    auto issue_qv = [&](int n) {
        const int t0 = chunk_t0(n);
        if (!STATES_ONLY) {
            mbar_expect_tx(bar_q, CHUNK * DK * 2);
            tma_load_4d(sbase + OFF_RQ, &maps.q, 0, t0, h, b, bar_q);
        }
        mbar_expect_tx(bar_v, CHUNK * DV * 2);
        tma_load_4d(sbase + OFF_V, &maps.v, 0, t0, h, b, bar_v);
    };
    float S[16];                                  // my 16 columns of state row st_row
    const uint32_t* sq = reinterpret_cast<const uint32_t*>(smem + OFF_RQ);
    const uint32_t* sk = reinterpret_cast<const uint32_t*>(smem + OFF_RK);
    const uint32_t* sg = reinterpret_cast<const uint32_t*>(smem + OFF_RG);

    // The MMAs of a step go to two disjoint accumulators each; they are issued by two threads of different warps
    // (issuing costs ~100 cycles per instruction), each of which commits to the step's barrier.
    const int issuer = tid == 0 ? 0 : (tid == 128 ? 1 : -1);
    bool s_zero = true;                           // the state entering the current chunk is exactly zero
    uint32_t it_count = 0;                        // iterations done by this CTA: parity of the per-iteration barriers
    uint32_t item_count = 0;                      // items done by this CTA: parity of bar_x
    int next_item = 0;
    for (;;) {                                    // work items (exactly one unless FUSED)
    if (FUSED) {
        const int item = *item_slot;              // drawn during the previous item (or at kernel start); the slot is
                                                  // rewritten only after several CTA barriers
        if (item >= p.B * p.H * nseg) break;
        bh = item / nseg; seg = item % nseg;
    }
    b = bh / p.H; h = bh % p.H;
    seg_t0 = seg * SEG;
    nch = min(SEG_CHUNKS, (p.L - seg_t0 + CHUNK - 1) / CHUNK);
    n_iter = (dir_last - dir_first + 1) * nch;    // iterations: sweeps x chunks
    if (tid == 0) { issue_gk(0); issue_qv(0); }

    for (int n = 0; n < n_iter; ++n, ++it_count) {
        const int dir = dir_first + n / nch, ci = n % nch;
        const int c = dir ? nch - 1 - ci : ci;
        const int t0 = seg_t0 + c * CHUNK;
        const uint32_t par = it_count & 1u;

        if (ci == 0) {                            // a sweep starts: entering state of the segment, zeroed gate total
            const float* src = nullptr;
            if (FUSED) {                          // only the sequence's own initial state is known at this point
                const float* init = dir ? p.init_b : p.init_f;
                if (init && seg == (dir ? nseg - 1 : 0)) src = init + (size_t)bh * DK * DV;
            } else if (!STATES_ONLY) {
                if (use_ws) src = p.ws_state + (((size_t)bh * nseg + seg) * 2 + dir) * DK * DV;
                else if (dir ? p.init_b : p.init_f) src = (dir ? p.init_b : p.init_f) + (size_t)bh * DK * DV;
            }
            s_zero = src == nullptr;              // a zero state contributes nothing: its product is not issued
            if (st_thread) {
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 t4 = src ? __ldg(reinterpret_cast<const float4*>(src + st_row * DV + st_col0 + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    S[j] = t4.x; S[j + 1] = t4.y; S[j + 2] = t4.z; S[j + 3] = t4.w;
                }
            }
            if (tid < DK) gtot[tid] = 0.f;
        }
        if (warp == 0) waiter.wait(bar_gk, par);              // one warp polls; the others sleep in the barrier
        __syncthreads();

        // ---- phase 1: cumulative gates (log2 units) and the scaled operand tiles ------------------------
        // One code path for both directions and for clamped / padded chunks (runtime selects, not template variants),
        // token loops in halves of 8 with the cumulative gates rotating through two register arrays: the instruction
        // cache, not the arithmetic, bounds this kernel.
        float2 gref = make_float2(0.f, 0.f), glast = make_float2(0.f, 0.f);
        bool out_of_range = false;
        {
            const int n_valid = p.L - t0;                             // rows at or past it are padding: decay 1
            const int dmask = dir ? TPG - 1 : 0;                      // scan order inside the group: token grp*TPG + (u ^ dmask)
            constexpr int HT = TPG < 8 ? TPG : 8, NH = TPG / HT;
            float2 glA[HT], glB[HT];
            float2 run = make_float2(0.f, 0.f);
#pragma unroll 1
            for (int hh = 0; hh < NH; ++hh) {
#pragma unroll
                for (int i = 0; i < HT; ++i) glA[i] = glB[i];
#pragma unroll
                for (int i = 0; i < HT; ++i) {
                    const int tok = grp * TPG + ((hh * HT + i) ^ dmask);
                    float2 g = Pack2<T>::unpack(sg[tok * CPW + cp]);
                    g.x = fmaxf(gate2_short(g.x, raw_logits, -inv_norm), clamp_lo);
                    g.y = fmaxf(gate2_short(g.y, raw_logits, -inv_norm), clamp_lo);
                    if (tok >= n_valid) g = make_float2(0.f, 0.f);
                    run.x += g.x; run.y += g.y;
                    glB[i] = run;                                     // inclusive cumulative sum
                }
            }
            if (NH == 1) {
#pragma unroll
                for (int i = 0; i < HT; ++i) glA[i] = glB[i];
            }
            reinterpret_cast<float2*>(part)[grp * CPW + cp] = run;
            if (!STATES_ONLY && warp == 0) waiter.wait(bar_q, par);   // q is first read after the barrier below
            __syncthreads();                                          // publishes `part`
            float2 off = make_float2(0.f, 0.f);
#pragma unroll 2
            for (int g2 = 0; g2 < NG; ++g2) {
                const float2 s2 = reinterpret_cast<const float2*>(part)[g2 * CPW + cp];
                const bool before = dir ? g2 > grp : g2 < grp;        // scanned before my group
                const bool in_ref = dir ? g2 >= NG / 2 : g2 < NG / 2; // part of the cumulative gate at the middle token
                if (before) { off.x += s2.x; off.y += s2.y; }
                if (in_ref) { gref.x += s2.x; gref.y += s2.y; }
                glast.x += s2.x; glast.y += s2.y;
            }
            off.x -= gref.x; off.y -= gref.y;
            float worst = 0.f;                                        // largest |exponent| before clamping
#pragma unroll 1
            for (int hh = 0; hh < NH; ++hh) {
                uint32_t rk[HT], rq[HT], offs[HT];
#pragma unroll
                for (int i = 0; i < HT; ++i) {                        // all reads of the half before its writes
                    const uint32_t tok = (uint32_t)(grp * TPG + ((hh * HT + i) ^ dmask));
                    offs[i] = swz(tok, cp * 4);
                    rk[i] = sk[tok * CPW + cp];
                    if (!STATES_ONLY) rq[i] = sq[tok * CPW + cp];
                }
#pragma unroll
                for (int i = 0; i < HT; ++i) {
                    float ex = off.x + glA[i].x, ey = off.y + glA[i].y;
                    worst = fmaxf(worst, fmaxf(fabsf(ex), fabsf(ey)));
                    ex = fminf(fmaxf(ex, -MAX_EXPONENT2), MAX_EXPONENT2);
                    ey = fminf(fmaxf(ey, -MAX_EXPONENT2), MAX_EXPONENT2);
                    const float2 kk = Pack2<T>::unpack(rk[i]);
                    *reinterpret_cast<uint32_t*>(smem + OFF_KT + offs[i]) = Pack2<T>::pack(kk.x * ex2(-ex), kk.y * ex2(-ey));
                    if (!STATES_ONLY) {
                        const float2 qq = Pack2<T>::unpack(rq[i]);
                        *reinterpret_cast<uint32_t*>(smem + OFF_QT + offs[i]) = Pack2<T>::pack(qq.x * ex2(ex + lq), qq.y * ex2(ey + lq));
                    }
                }
#pragma unroll
                for (int i = 0; i < HT; ++i) glA[i] = glB[i];
            }
            out_of_range = worst > MAX_EXPONENT2;
        }
        if (out_of_range && p.status) atomicOr(p.status, 2);
        if (grp == 0) {
            vec[2 * cp] = ex2(glast.x); vec[2 * cp + 1] = ex2(glast.y);
            vec[64 + 2 * cp] = ex2(glast.x - gref.x); vec[64 + 2 * cp + 1] = ex2(glast.y - gref.y);
            if (FUSED) {                          // log2 of (decay from the segment's edge to this chunk's reference token)
                cvec[n * 64 + 2 * cp] = gtot[2 * cp] + gref.x; cvec[n * 64 + 2 * cp + 1] = gtot[2 * cp + 1] + gref.y;
            }
            gtot[2 * cp] += glast.x; gtot[2 * cp + 1] += glast.y;
        }
        // state operand for the inter-chunk product: bf16(exp(G_ref) * S_in), MN-major [channel][value]
        if (!STATES_ONLY && st_thread && !s_zero) {
            float gr = 0.f;
#pragma unroll
            for (int g2 = 0; g2 < NG / 2; ++g2) gr += part[(dir ? g2 + NG / 2 : g2) * DK + st_row];
            const float eg = ex2(gr);
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
                uint4 w;
                w.x = Pack2<T>::pack(S[j] * eg, S[j + 1] * eg); w.y = Pack2<T>::pack(S[j + 2] * eg, S[j + 3] * eg);
                w.z = Pack2<T>::pack(S[j + 4] * eg, S[j + 5] * eg); w.w = Pack2<T>::pack(S[j + 6] * eg, S[j + 7] * eg);
                *reinterpret_cast<uint4*>(smem + OFF_ST + swz(st_row, (st_col0 + j) * 2)) = w;
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();                          // raw q / k / gate tiles are dead from here on
        if (tid == 0 && n + 1 < n_iter) issue_gk(n + 1);

        const uint32_t kt = sbase + OFF_KT, v_addr = sbase + OFF_V;
        bool o_has = dir != dir_first;            // the chunk's output accumulator already has content (issuer 0's view)
        if (!STATES_ONLY) {
            // ---- MMA issue 1: inter-chunk product (issuer 0) and the 128x128 scores (issuer 1) ----------------
            const uint32_t qt = sbase + OFF_QT;
            if (issuer == 0) {
                tc_fence_after();
                if (FUSED)                                // park the operand tile (same swizzled image) for the deferred term
                    bulk_store(p.qscratch + ((size_t)blockIdx.x * 4 + n) * TILE_B, qt, TILE_B);
                if (!s_zero) {
                    const uint32_t st = sbase + OFF_ST;
#pragma unroll
                    for (int k4 = 0; k4 < DK / 16; ++k4)
                        tc_mma(tmem + TM_O + c * 64, make_desc(qt + k4 * 32), make_desc(st + k4 * 2048), IDESC_OV, o_has || k4 > 0);
                    o_has = true;
                }
                if (FUSED) bulk_store_wait_read();        // the scores overwrite the tile once bar_p0 completes
                tc_commit(bar_p0);
            } else if (issuer == 1) {
                tc_fence_after();
#pragma unroll
                for (int k4 = 0; k4 < DK / 16; ++k4)      // all 128 key columns at once: TM_P0 and TM_P1 are adjacent
                    tc_mma(tmem + TM_P0, make_desc(qt + k4 * 32), make_desc(kt + k4 * 32), IDESC_QK, k4 > 0);
                tc_commit(bar_p0);                        // with issuer 0's commit: both readers of the scaled q tile are done
            }
            __syncwarp();
            // ---- scores -> masked bf16 P tiles (warps 0-3: keys 0..63 over the dead raw q tile,
            //      warps 4-7: keys 64..127 over the dead scaled q tile) ---------------------------------
            const int half = warp >> 2;
            const int quad = warp & 3;                                // my 32 query rows: 32*quad .. 32*quad+31
            const int row = 32 * quad + lane;                         // query token inside the chunk
            uint8_t* ptile = smem + (half ? OFF_QT : OFF_RQ);         // both tiles are dead once the score MMA is done
            if ((warp & 3) == 0) waiter.wait(bar_p0, par);
            half_bar_sync(half);
            tc_fence_after();
            // A 32x32 block of scores is wholly kept, wholly masked, or on the diagonal (warp-uniform test); on the
            // diagonal, bit j of `dbits` says whether key j of the block is kept for my query row.
            {
                const uint32_t dbits = dir ? ~((1u << lane) - 1u) : (lane == 31 ? 0xffffffffu : (2u << lane) - 1u);
#pragma unroll 1
                for (int part32 = 0; part32 < 2; ++part32) {
                    const int cb = 2 * half + part32;                 // key block: keys 32*cb .. 32*cb+31
                    const bool all_zero = dir ? cb < quad : cb > quad;
                    const uint32_t keep = cb == quad ? dbits : 0xffffffffu;
                    uint8_t* prow = ptile + row * 128;
                    const uint32_t chunk0 = (uint32_t)part32 * 4;     // first 16-byte chunk of this block in the 128-byte row
                    if (all_zero) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(prow + (((chunk0 + j) ^ (row & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                    } else {
                        float a[32];
                        tc_ld32(tmem + lane_base + (half ? TM_P1 : TM_P0) + 32 * part32, a);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            float mk[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) mk[e] = (keep >> (8 * j + e)) & 1u ? a[8 * j + e] : 0.f;
                            uint4 w;
                            w.x = Pack2<T>::pack(mk[0], mk[1]); w.y = Pack2<T>::pack(mk[2], mk[3]);
                            w.z = Pack2<T>::pack(mk[4], mk[5]); w.w = Pack2<T>::pack(mk[6], mk[7]);
                            *reinterpret_cast<uint4*>(prow + (((chunk0 + j) ^ (row & 7)) << 4)) = w;
                        }
                    }
                }
            }
            fence_proxy_async();
            tc_fence_before();
            __syncthreads();
        }
        // ---- MMA issue 2: P V into the output accumulator (issuer 0), K^T V into the second score buffer (issuer 1)
        if (issuer == 0) {
            if (!STATES_ONLY) {
                waiter.wait(bar_v, par);          // only the tensor core reads v, so only the issuing threads wait for it
                tc_fence_after();
#pragma unroll
                for (int k8 = 0; k8 < CHUNK / 16; ++k8)
                    tc_mma(tmem + TM_O + c * 64, make_desc(sbase + (k8 < 4 ? OFF_RQ : OFF_QT) + (k8 & 3) * 32),
                           make_desc(v_addr + k8 * 2048), IDESC_OV, o_has || k8 > 0);
            }
            tc_commit(bar_o);
        } else if (issuer == 1) {
            waiter.wait(bar_v, par);
            tc_fence_after();
#pragma unroll
            for (int k8 = 0; k8 < CHUNK / 16; ++k8)
                tc_mma(tmem + TM_U, make_desc(kt + k8 * 2048), make_desc(v_addr + k8 * 2048), IDESC_U, k8 > 0);
            tc_commit(bar_o);
        }
        __syncwarp();

        // ---- state update in registers ---------------------------------------------------------------
        if (warp == 0) {
            waiter.wait(bar_o, par);              // all MMAs of the iteration are done: every tile is free again
            if (tid == 0 && n + 1 < n_iter) issue_qv(n + 1);
        }
        __syncthreads();
        tc_fence_after();
        {
            float u[32];
            tc_ld32(tmem + lane_base + TM_U + st_ld0, u);             // rows live in lanes 0-15 of the warp
            tc_wait_ld();
            const float e_last = vec[st_row & 63], e_rel = vec[64 + (st_row & 63)];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float hi = __shfl_sync(0xffffffffu, u[16 + j], lane & 15);   // columns 16-31 go to lanes 16-31
                const float mine = lane < 16 ? u[j] : hi;
                S[j] = fmaf(S[j], e_last, e_rel * mine);
            }
        }
        s_zero = false;
        tc_fence_before();                        // ordered before the next tensor-core write of this buffer by the
                                                  // CTA barriers of the next iteration

        if (ci == nch - 1) {                      // a sweep ends: hand the state out
            float* dst = nullptr;
            float* gdst = nullptr;
            if (STATES_ONLY || FUSED) {
                const size_t slot = ((size_t)bh * nseg + seg) * 2 + dir;
                dst = p.ws_state + slot * DK * DV;
                gdst = p.ws_decay + slot * DK;
            } else if (!use_ws) {                 // single segment: final state / total decay straight to the caller
                if (dir ? p.final_b : p.final_f) dst = (dir ? p.final_b : p.final_f) + (size_t)bh * DK * DV;
                if (dir ? p.logdecay_b : p.logdecay_f) gdst = (dir ? p.logdecay_b : p.logdecay_f) + (size_t)bh * DK;
            }
            if (dst && st_thread) {
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    *reinterpret_cast<float4*>(dst + st_row * DV + st_col0 + j) = make_float4(S[j], S[j + 1], S[j + 2], S[j + 3]);
            }
            if (gdst && tid < DK) gdst[tid] = gtot[tid] * LN2;          // back to natural-log units
        }
    }

    if (FUSED) {
        // ---- publish: my local end states are in the workspace; count me in for my sequence ------------------
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            atomicAdd(p.group_cnt + bh, 1u);
            bulk_store_wait_all();                // the parking copies have landed
        }
        __syncthreads();
        // bring my parked q operand tiles back meanwhile (plain loads that bypass L1; measured faster here than bulk
        // copies issued by one thread); every tile buffer is free at this point
        {
            const uint8_t* src = p.qscratch + (size_t)blockIdx.x * 4 * TILE_B;
            const uint32_t dst_off[4] = {(uint32_t)OFF_QT, (uint32_t)OFF_KT, (uint32_t)OFF_RQ, (uint32_t)OFF_RK};
#pragma unroll
            for (int n = 0; n < 4; ++n) {
                if (n < n_iter) {
#pragma unroll
                    for (int r = 0; r < TILE_B / (NTHREADS * 16); ++r) {
                        const int o16 = (r * NTHREADS + tid) * 16;
                        *reinterpret_cast<uint4*>(smem + dst_off[n] + o16) = __ldcg(reinterpret_cast<const uint4*>(src + n * TILE_B + o16));
                    }
                }
            }
        }
        // Bounded wait until `count` of the sequence's segments have passed a point (one warp polls).
        auto group_wait = [&](const uint32_t* counter) {
            if (warp == 0) {
                bool ok = false;
                for (uint32_t i = 0; i < (1u << 21); ++i) {
                    if (ld_acquire_u32(counter) >= (uint32_t)nseg) { ok = true; break; }
                    if (*abort_flag) break;
                    __nanosleep(32);
                }
                if (!ok) { *abort_flag = 1; if (p.status) atomicOr(p.status, 1); }
            }
            __threadfence();
            __syncthreads();
        };
        group_wait(p.group_cnt + bh);             // every segment's local end state is in the workspace
        // ---- scan over the segments, split by state element across the sequence's CTAs: each CTA turns, for its
        //      slice of the dk x dv elements, every segment's local end state into the state that ENTERS that
        //      segment (in place), and delivers the sequence's final state / total decay for that slice ----------
        {
            constexpr int NE = DK * DV;
            const int slice = (NE + nseg - 1) / nseg;
            const int e_end = min(NE, (seg + 1) * slice);
            const bool on[2] = {(p.dir_mask & 1) != 0, (p.dir_mask & 2) != 0};
            for (int e = seg * slice + tid; e < e_end; e += NTHREADS) {
                const int row = e / DV;
                float E[2] = {0.f, 0.f}, gsum[2] = {0.f, 0.f};
                constexpr int PF = 8;             // both directions' loads of PF segments are in flight before the chains run
                for (int i0 = 0; i0 < nseg; i0 += PF) {
                    float u[2][PF], a[2][PF];
#pragma unroll
                    for (int d = 0; d < 2; ++d) {
#pragma unroll
                        for (int i = 0; i < PF; ++i) {
                            const bool in = on[d] && i0 + i < nseg;
                            const int sg_i = in ? i0 + i : 0;
                            const size_t slot = ((size_t)bh * nseg + (d ? nseg - 1 - sg_i : sg_i)) * 2 + d;
                            u[d][i] = in ? __ldcg(p.ws_state + slot * NE + e) : 0.f;
                            a[d][i] = in ? __ldcg(p.ws_decay + slot * DK + row) : 0.f;
                        }
                    }
#pragma unroll
                    for (int d = 0; d < 2; ++d) {
#pragma unroll
                        for (int i = 0; i < PF; ++i) { gsum[d] += a[d][i]; a[d][i] = __expf(a[d][i]); }
                    }
#pragma unroll
                    for (int i = 0; i < PF; ++i) {
#pragma unroll
                        for (int d = 0; d < 2; ++d) {
                            if (on[d] && i0 + i < nseg) {
                                const size_t slot = ((size_t)bh * nseg + (d ? nseg - 1 - (i0 + i) : i0 + i)) * 2 + d;
                                p.ws_state[slot * NE + e] = E[d];
                                E[d] = fmaf(E[d], a[d][i], u[d][i]);
                            }
                        }
                    }
                }
#pragma unroll
                for (int d = 0; d < 2; ++d) {
                    float* fin = d ? p.final_b : p.final_f;
                    float* ld = d ? p.logdecay_b : p.logdecay_f;
                    if (on[d] && fin) fin[(size_t)bh * NE + e] = E[d];
                    if (on[d] && ld && (e % DV) == 0) ld[(size_t)bh * DK + row] = gsum[d];
                }
            }
        }
        __threadfence();
        __syncthreads();
        uint32_t* scanned = p.group_cnt + (size_t)p.B * p.H + bh;
        if (tid == 0) atomicAdd(scanned, 1u);
        group_wait(scanned);                      // every slice of the entering states is in place
        // Draw the next item and keep it in a register until the end of this one, so that the round trip of the
        // atomic costs no stall.  Not earlier: a CTA that holds a ticket of a sequence it is still waiting for
        // could never be released.
        if (tid == 0) next_item = (int)atomicAdd(p.ticket, 1u);
        // ---- state operand of every chunk: bf16(2^{cvec} * S_enter), MN-major [channel][value] -------------------
        const uint32_t st_off[4] = {(uint32_t)OFF_ST, (uint32_t)OFF_RG, (uint32_t)(OFF_RG + 64 * 128), (uint32_t)OFF_V};
        float4 enter[2][4];                       // both directions' entering states are requested before either is used
#pragma unroll
        for (int dir = 0; dir < 2; ++dir) {
            const float4* src = reinterpret_cast<const float4*>(p.ws_state + (((size_t)bh * nseg + seg) * 2 + dir) * DK * DV + (st_row & (DK - 1)) * DV + st_col0);
#pragma unroll
            for (int j = 0; j < 4; ++j) enter[dir][j] = (p.dir_mask & (1 << dir)) ? __ldcg(src + j) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int dir = 0; dir < 2; ++dir) {
            if (!(p.dir_mask & (1 << dir))) continue;
            for (int ci = 0; ci < nch; ++ci) {
                const int n = (dir - dir_first) * nch + ci;
                if (st_thread) {
                    const float eg = ex2(cvec[n * 64 + st_row]);
#pragma unroll
                    for (int j = 0; j < 4; j += 2) {
                        const float4 a = enter[dir][j], b2 = enter[dir][j + 1];
                        uint4 w;
                        w.x = Pack2<T>::pack(a.x * eg, a.y * eg); w.y = Pack2<T>::pack(a.z * eg, a.w * eg);
                        w.z = Pack2<T>::pack(b2.x * eg, b2.y * eg); w.w = Pack2<T>::pack(b2.z * eg, b2.w * eg);
                        *reinterpret_cast<uint4*>(smem + st_off[n] + swz(st_row, (st_col0 + 4 * j) * 2)) = w;
                    }
                }
            }
        }
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        // ---- the deferred term: O_chunk += (parked q operand) x (entering state operand); issuer i owns chunk i --
        if (issuer >= 0) {
            tc_fence_after();
            const uint32_t q_off[4] = {(uint32_t)OFF_QT, (uint32_t)OFF_KT, (uint32_t)OFF_RQ, (uint32_t)OFF_RK};
            for (int n = 0; n < n_iter; ++n) {
                const int dir = dir_first + n / nch, ci = n % nch;
                const int c = dir ? nch - 1 - ci : ci;
                if (c != issuer) continue;
#pragma unroll
                for (int k4 = 0; k4 < DK / 16; ++k4)
                    tc_mma(tmem + TM_O + c * 64, make_desc(sbase + q_off[n] + k4 * 32), make_desc(sbase + st_off[n] + k4 * 2048), IDESC_OV, 1);
            }
            tc_commit(bar_x);
        }
        __syncwarp();
        if (warp == 0) waiter.wait(bar_x, item_count & 1u);
        __syncthreads();
        ++item_count;
    }

    // ---- epilogue: output accumulators -> global -----------------------------------------------------
    if (!STATES_ONLY && p.o) {
        tc_fence_after();
        T* obase = reinterpret_cast<T*>(p.o) + b * p.so[0] + h * p.so[1];
        const int row = 32 * (warp & 3) + lane, col0 = 32 * (warp >> 2);
        for (int c = 0; c < nch; ++c) {
            float a[32];
            tc_ld32(tmem + lane_base + TM_O + c * 64 + col0, a);
            tc_wait_ld();
            const int tok = seg_t0 + c * CHUNK + row;
            if (tok < p.L) {
                uint4* dst = reinterpret_cast<uint4*>(obase + (int64_t)tok * p.so[2] + col0);
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                    uint4 w;
                    w.x = Pack2<T>::pack(o_sign * a[j], o_sign * a[j + 1]); w.y = Pack2<T>::pack(o_sign * a[j + 2], o_sign * a[j + 3]);
                    w.z = Pack2<T>::pack(o_sign * a[j + 4], o_sign * a[j + 5]); w.w = Pack2<T>::pack(o_sign * a[j + 6], o_sign * a[j + 7]);
                    dst[j / 8] = w;
                }
            }
        }
    }
    if (!FUSED) break;
    if (tid == 0) *item_slot = next_item;
    tc_fence_before();                            // the accumulators are read out before the next item overwrites them
    __syncthreads();
    }                                             // work items
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TM_COLS) : "memory");
    }
}

constexpr int MAX_SLOTS = 320;                 // scratch slots of the single-launch path (>= resident CTAs of a B200)

size_t states_bytes(int B, int H, int L, int dk, int dv) {
    const size_t nseg = (L + SEG - 1) / SEG;
    return (size_t)B * H * nseg * 2 * ((size_t)dk * dv + dk) * sizeof(float);
}
size_t counter_bytes(int B, int H) { return ((2 * (size_t)B * H + 1) * sizeof(uint32_t) + 255) & ~(size_t)255; }   // ticket, arrivals, ready flags

template <int DK, typename T>
int launch_tc(const BiglaParams& p_in, const TcMaps& maps, bool allow_fused, cudaStream_t stream) {
    BiglaParams p = p_in;
    const int nseg = (p.L + SEG - 1) / SEG;
    const int BH = p.B * p.H;
    const bool need_states = p.final_f || p.final_b || p.logdecay_f || p.logdecay_b;
    const int use_ws = nseg > 1;
    dim3 grid(nseg, BH);
    auto kA = bigla_tc_kernel<DK, T, 1>;
    auto kC = bigla_tc_kernel<DK, T, 0>;
    auto kF = bigla_tc_kernel<DK, T, 2>;
    cudaError_t e;
    if (use_ws && p.o && allow_fused) {
        // Single launch: persistent CTAs, as many as are resident at once.  A sequence's segments wait for one
        // another, so the grid must hold at least nseg CTAs that run concurrently; otherwise use three launches.
        static int resident[64] = {};             // per device; 0 = not queried yet
        static int sm_count[64] = {};
        int dev = 0;
        if ((e = cudaGetDevice(&dev)) != cudaSuccess) return (int)e;
        if (dev >= 0 && dev < 64) {
            if ((e = ensure_smem_attr(reinterpret_cast<const void*>(kF), SMEM_BYTES)) != cudaSuccess) return (int)e;
            if (!resident[dev]) {
                if ((e = cudaFuncSetAttribute(kF, cudaFuncAttributePreferredSharedMemoryCarveout, 100)) != cudaSuccess) return (int)e;
                int per_sm = 0, sms = 0;
                if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kF, NTHREADS, SMEM_BYTES)) != cudaSuccess) return (int)e;
                if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
                resident[dev] = per_sm * sms > 0 ? per_sm * sms : -1;
                sm_count[dev] = sms;
            }
            // The occupancy query is conservative about the shared-memory carve-out (it reports one CTA per SM where
            // two run): it is used for the safety condition below, while the grid is sized for the two CTAs per SM
            // the kernel is built for.  CTAs that are not resident at first simply start later and find no work.
            const int items = BH * nseg;
            const int safe = resident[dev];
            int ctas = 2 * sm_count[dev] < MAX_SLOTS ? 2 * sm_count[dev] : MAX_SLOTS;
            if (ctas > items) ctas = items;
            if (ctas < safe) ctas = safe < MAX_SLOTS ? safe : MAX_SLOTS;
            const int running = ctas < safe ? ctas : safe;    // CTAs guaranteed to run concurrently
            if (running >= nseg) {
                if ((e = cudaMemsetAsync(p.ticket, 0, counter_bytes(p.B, p.H), stream)) != cudaSuccess) return (int)e;
                p.nseg = nseg;
                kF<<<ctas, NTHREADS, SMEM_BYTES, stream>>>(maps, p, 1);
                return (int)cudaGetLastError();
            }
        }
    }
    if (use_ws || (need_states && !p.o)) {
        if ((e = ensure_smem_attr(reinterpret_cast<const void*>(kA), SMEM_BYTES)) != cudaSuccess) return (int)e;
        kA<<<grid, NTHREADS, SMEM_BYTES, stream>>>(maps, p, 1);
        p.nchunk = nseg;
        if (int st = bigla_scan_launch(p, stream)) return st;
    }
    if (p.o) {
        if ((e = ensure_smem_attr(reinterpret_cast<const void*>(kC), SMEM_BYTES)) != cudaSuccess) return (int)e;
        kC<<<grid, NTHREADS, SMEM_BYTES, stream>>>(maps, p, use_ws);
    }
    return (int)cudaGetLastError();
}

}  // namespace


// Measured on B200: the single-launch form wins for sequences of 8..32 segments (2048..8192 tokens) and halves
// the DRAM traffic there; shorter sequences have too few segments to amortise the two group barriers, longer
// ones make every CTA wait for too many others.
bool bigla_tc_prefers_single(int L) {
    const int nseg = (L + SEG - 1) / SEG;
    return nseg >= 8 && nseg <= 32;
}

bool bigla_tc_supported(const BiglaParams& p) {
    if (p.dtype != VIG_DTYPE_BF16 && p.dtype != VIG_DTYPE_F16) return false;
    if (p.dv != DV || (p.dk != 32 && p.dk != 64)) return false;
    if (!tma_ok(p.q, p.sq, p.B, p.H) || !tma_ok(p.k, p.sk, p.B, p.H) || !tma_ok(p.v, p.sv, p.B, p.H) ||
        !tma_ok(p.gf, p.sgf, p.B, p.H) || !tma_ok(p.gb, p.sgb, p.B, p.H))
        return false;
    if (p.o && ((reinterpret_cast<uintptr_t>(p.o) & 15) || (p.so[0] * 2) % 16 || (p.so[1] * 2) % 16 || (p.so[2] * 2) % 16)) return false;
    return encode_fn() != nullptr;
}

// Workspace: [segment states | summed log-gates] for every path; the single-launch path adds
// [ticket + per-(b,h) counters | MAX_SLOTS x 4 parked operand tiles].
size_t bigla_tc_workspace(int B, int H, int L, int dk, int dv, bool split_only) {
    const size_t st = states_bytes(B, H, L, dk, dv);
    if (split_only || L <= SEG) return st;
    return ((st + 255) & ~(size_t)255) + counter_bytes(B, H) + (size_t)MAX_SLOTS * 4 * TILE_B;
}

// What this call really touches: nothing for a single segment with an output (its end states go straight to the caller).
size_t bigla_tc_min_workspace(const BiglaParams& p) {
    const bool need_states = p.final_f || p.final_b || p.logdecay_f || p.logdecay_b;
    if (p.L <= SEG && (p.o || !need_states)) return 0;
    return states_bytes(p.B, p.H, p.L, p.dk, p.dv);
}

int bigla_tc_launch(const BiglaParams& p_in, void* ws, size_t ws_bytes, bool allow_fused, cudaStream_t stream) {
    BiglaParams p = p_in;
    const size_t nseg = (p.L + SEG - 1) / SEG;
    const size_t st = states_bytes(p.B, p.H, p.L, p.dk, p.dv);
    const size_t min_ws = bigla_tc_min_workspace(p);
    if (min_ws && (!ws || ws_bytes < min_ws)) return VIG_ERR_WORKSPACE;
    if (!ws) ws_bytes = 0;
    if (ws_bytes < bigla_tc_workspace(p.B, p.H, p.L, p.dk, p.dv, false)) allow_fused = false;
    p.ws_state = reinterpret_cast<float*>(ws);
    p.ws_decay = p.ws_state + (size_t)p.B * p.H * nseg * 2 * p.dk * p.dv;
    if (allow_fused && nseg > 1) {
        uint8_t* extra = reinterpret_cast<uint8_t*>(ws) + ((st + 255) & ~(size_t)255);
        p.ticket = reinterpret_cast<uint32_t*>(extra);
        p.group_cnt = p.ticket + 1;
        p.qscratch = extra + counter_bytes(p.B, p.H);
    }
    TcMaps maps;
    const void* qsrc = p.q ? p.q : p.k;           // states-only calls pass no q; the map is then never used
    const int64_t* qs = p.q ? p.sq : p.sk;
    const void* gfs = p.gf ? p.gf : p.gb;
    const int64_t* gfst = p.gf ? p.sgf : p.sgb;
    const void* gbs = p.gb ? p.gb : p.gf;
    const int64_t* gbst = p.gb ? p.sgb : p.sgf;
    if (!make_map(&maps.q, qsrc, qs, p.B, p.H, p.L, p.dk, p.dtype, false) ||
        !make_map(&maps.k, p.k, p.sk, p.B, p.H, p.L, p.dk, p.dtype, false) ||
        !make_map(&maps.v, p.v, p.sv, p.B, p.H, p.L, p.dv, p.dtype, true) ||
        !make_map(&maps.gf, gfs, gfst, p.B, p.H, p.L, p.dk, p.dtype, false) ||
        !make_map(&maps.gb, gbs, gbst, p.B, p.H, p.L, p.dk, p.dtype, false))
        return VIG_ERR_DEVICE;
#define VIG_TC(DKV, TT) if (p.dk == DKV) return launch_tc<DKV, TT>(p, maps, allow_fused, stream);
    if (p.dtype == VIG_DTYPE_BF16) { VIG_TC(64, __nv_bfloat16) VIG_TC(32, __nv_bfloat16) }
    else { VIG_TC(64, __half) VIG_TC(32, __half) }
#undef VIG_TC
    return VIG_ERR_SHAPE;
}

}  // namespace vig
